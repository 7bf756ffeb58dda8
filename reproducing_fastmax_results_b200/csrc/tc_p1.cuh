// Order-1, non-causal forward (bf16, head dim 64) on tensor memory.  Included by tc_kernels.cu inside fm::tc.
//
//     S^T  = [V | 1]^T K            (80 x 64, float32 in TMEM; row 64 is sum_j k_j, the linear part of the denominator)
//     s0   = [V | 1]^T 1            (80 sums: sum_j v_j and the key count)
//     O'_c = Q_c (c1 S)  + a0 s0     per 128-query chunk;  o = O'[:, :64] / O'[:, 64],  g = O'[:, 64]
//
// 33 flop per byte: the call is bound by HBM (read q, k, v once, write o and g once).  One CTA per (batch, head)
// streams the head's K and V chunks through a two-deep TMA ring into the moment MMAs, rounds c1 S to bf16 into a
// K-major operand tile, then streams the Q chunks through the same ring; every epilogue warp stages its 32 output
// rows in shared memory and hands them to the copy engine (tiled bulk store: whole 128-byte lines, rows past the
// last query clipped by the tensor map).  Two CTAs fit on an SM, so one head's phase change hides behind the other's
// streaming.
// Warp roles (160 threads): 0-3 epilogue (TMEM lane = moment row, then = token), 4 TMA loads + MMA issue.
// TMEM columns (256 allocated): 0..63 S^T, 64..79 s0, 96..175 and 176..255 the two output accumulators.
#pragma once

namespace p1 {

constexpr int THREADS = 160;
constexpr int OFF_X = 0;                      // two 128 x 64 swizzled tiles: K chunks, later Q chunks
constexpr int OFF_V = 2 * REGION;             // two [V | 1] chunks of 10 column blocks; the moment MMA reads 16 blocks
constexpr int OFF_SB = OFF_V + 2 * 10 * BLK;  // 73728: c1 S as a K-major B operand, 80 rows x 128 B, 128-byte swizzle
constexpr int OFF_ONES = OFF_SB + 80 * 128;   // 83968: 1 KB of bf16 ones (B operand of the s0 MMA)
constexpr int OFF_T0 = OFF_ONES + 1024;       // 80 floats: a0 s0
constexpr int OFF_BAR = OFF_T0 + 512;
constexpr int OFF_OST = OFF_BAR + 512;        // 86016: output staging, one 32-row x 128-byte swizzled box per epilogue warp
constexpr int OFF_END = OFF_OST + 4 * 4096;
// rows 80..127 of the moment MMA's A operand read the 12 KB that follow a [V | 1] buffer (the other buffer, the
// S tile, the ones): finite or not, they only reach TMEM lanes 80..127, which nobody reads
static_assert(OFF_V + 10 * BLK + 16 * BLK <= OFF_END + 1024, "the moment MMA's A operand stays inside the allocation");
constexpr int SMEM_BYTES = OFF_END + 1024 + 1024;
static_assert(OFF_SB % 1024 == 0 && OFF_V % 1024 == 0 && OFF_OST % 1024 == 0, "swizzled tiles need 1024-byte alignment");
constexpr uint32_t COL_S = 0u, COL_S0 = 64u, COL_O = 96u;
constexpr int B_X_READY = 0, B_X_FREE = 2, B_S_DONE = 4, B_SB_READY = 5, B_O_DONE = 6, B_O_FREE = 8, B_COUNT = 10;

struct P1Params {
  View g;
  int heads, nq, nk;
  float c0, c1;   // a0, a1 / temperature
};

__global__ void __launch_bounds__(THREADS, 2)
p1_forward_kernel(const __grid_constant__ CUtensorMap tmq, const __grid_constant__ CUtensorMap tmk,
                  const __grid_constant__ CUtensorMap tmv, const __grid_constant__ CUtensorMap tmo, const P1Params P) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  uint8_t* sm = smem_raw + (((raw_addr + 1023u) & ~1023u) - raw_addr);
  uint8_t* xbuf = sm + OFF_X;
  uint8_t* vbuf = sm + OFF_V;
  uint8_t* sb = sm + OFF_SB;
  float* t0 = reinterpret_cast<float*>(sm + OFF_T0);
  uint64_t* bars = reinterpret_cast<uint64_t*>(sm + OFF_BAR);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(sm + OFF_BAR + 128);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(sm + OFF_BAR + 136);

  const int tid = threadIdx.x, w = tid >> 5, lane = tid & 31;
  const int head = blockIdx.x;
  const int b_idx = head / P.heads, h_idx = head - b_idx * P.heads;
  const int nkc = (P.nk + CH - 1) / CH, nqc = (P.nq + CH - 1) / CH;

  if (tid == 0) {
    for (int i = 0; i < 2; ++i) {
      mbar_init(&bars[B_X_READY + i], 1);
      mbar_init(&bars[B_X_FREE + i], 1);
      mbar_init(&bars[B_O_DONE + i], 1);
      mbar_init(&bars[B_O_FREE + i], 4);
    }
    mbar_init(&bars[B_S_DONE], 1);
    mbar_init(&bars[B_SB_READY], 4);
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (w == 0) tmem_alloc(tmem_slot, 256);
  // ones for the s0 MMA; zero pad blocks (column block 9 of both [V | 1] buffers; block 8 is rewritten per chunk)
  for (int i = tid; i < 1024 / 16; i += THREADS) reinterpret_cast<uint4*>(sm + OFF_ONES)[i] = make_uint4(0x3F803F80u, 0x3F803F80u, 0x3F803F80u, 0x3F803F80u);
  for (int i = tid; i < 2 * (2 * BLK / 16); i += THREADS) {
    const int b = i / (2 * BLK / 16), r = i - b * (2 * BLK / 16);
    reinterpret_cast<uint4*>(vbuf + b * 10 * BLK + 8 * BLK)[r] = make_uint4(0u, 0u, 0u, 0u);
  }
  fence_proxy_async_smem();
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  auto WAIT = [&](int bar, uint32_t n) -> bool { return mbar_wait_abortable(&bars[bar], n & 1u, WAIT_CYCLES, abort_flag); };
  auto FAIL = [&](int code) {
    if (*abort_flag == 0) atomicAdd(&g_tc_wait_hist[code & 255], 1);
    *abort_flag = 1;
    atomicExch(&g_tc_status, code);
  };

  if (w == 4) {
    // ================= TMA loads and MMA issue =================
    // The ring of two (X, [V | 1]) buffers carries the K / V chunks of the moment phase, then the Q chunks of the
    // apply phase (X only).  Load number n uses buffer n & 1; its `free` barrier counts the MMAs that read the buffer.
    bool ok = true;
    uint32_t loads = 0;   // loads issued so far (both phases)
    auto load = [&](int chunk, bool moment) -> bool {
      const uint32_t buf = loads & 1u;
      if (loads >= 2 && !WAIT(B_X_FREE + buf, (loads >> 1) - 1u)) { FAIL(400); return false; }
      const int pos0 = chunk * CH;
      uint8_t* vb = vbuf + buf * 10 * BLK;
      if (moment) {
        for (int r = lane; r < CH; r += 32)  // the ones column of [V | 1] (zero for rows past the last key)
          *reinterpret_cast<uint4*>(vb + 8 * BLK + r * 16) = make_uint4((pos0 + r < P.nk) ? 0x00003F80u : 0u, 0u, 0u, 0u);
        fence_proxy_async_smem();
      }
      __syncwarp();
      if (lane == 0) {
        mbar_arrive_expect_tx(&bars[B_X_READY + buf], moment ? REGION + 8 * BLK : REGION);
        tma_load_4d(xbuf + buf * REGION, moment ? &tmk : &tmq, &bars[B_X_READY + buf], 0, pos0, h_idx, b_idx);
        if (moment) {
#pragma unroll
          for (int j = 0; j < 8; ++j) tma_load_4d(vb + j * BLK, &tmv, &bars[B_X_READY + buf], 8 * j, pos0, h_idx, b_idx);
        }
      }
      __syncwarp();
      ++loads;
      return true;
    };
    uint32_t used = 0;    // loads consumed so far
    constexpr uint32_t IDESC_M = make_idesc_bf16(128, 64, 1, 1);    // A MN-major ([V | 1]), B MN-major (K tile)
    constexpr uint32_t IDESC_S0 = make_idesc_bf16(128, 16, 1, 0);   // A MN-major, B K-major (ones)
    constexpr uint32_t IDESC_A = make_idesc_bf16(128, 80, 0, 0);    // A K-major (Q tile), B K-major (c1 S)
    const uint64_t d_ones = make_smem_desc(smem_u32(sm + OFF_ONES), 128, 256, 0);
    // ---- moments ----
    if (nkc > 0) ok = load(0, true);
    for (int c = 0; c < nkc && ok; ++c) {
      if (c + 1 < nkc) ok = load(c + 1, true);
      if (!ok) break;
      const uint32_t buf = used & 1u;
      if (!WAIT(B_X_READY + buf, used >> 1)) { FAIL(401); ok = false; break; }
      __syncwarp();
      tc_fence_after_sync();
      if (elect_one()) {
        const uint64_t dV = make_smem_desc(smem_u32(vbuf + buf * 10 * BLK), 128, 2048, 0);
        const uint64_t dK = make_smem_desc(smem_u32(xbuf + buf * REGION), REGION, 1024, 2);
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
          mma_ss(tmem_base + COL_S, dV + (uint64_t)(16 * ks), dK + (uint64_t)(128 * ks), IDESC_M, (c > 0 || ks > 0) ? 1u : 0u);
          mma_ss(tmem_base + COL_S0, dV + (uint64_t)(16 * ks), d_ones, IDESC_S0, (c > 0 || ks > 0) ? 1u : 0u);
        }
        mma_commit(&bars[B_X_FREE + buf]);
        if (c == nkc - 1) mma_commit(&bars[B_S_DONE]);
      }
      __syncwarp();
      ++used;
    }
    // ---- apply ----
    if (ok && nqc > 0) ok = load(0, false);
    if (ok && nkc > 0 && !WAIT(B_SB_READY, 0)) { FAIL(402); ok = false; }
    for (int c = 0; c < nqc && ok; ++c) {
      if (c + 1 < nqc) ok = load(c + 1, false);
      if (!ok) break;
      const uint32_t buf = used & 1u, ob = (uint32_t)c & 1u;
      if (!WAIT(B_X_READY + buf, used >> 1)) { FAIL(403); ok = false; break; }
      if (c >= 2 && !WAIT(B_O_FREE + ob, (uint32_t)(c >> 1) - 1u)) { FAIL(404); ok = false; break; }
      __syncwarp();
      tc_fence_after_sync();
      if (elect_one()) {
        const uint64_t dQ = make_smem_desc(smem_u32(xbuf + buf * REGION), 16, 1024, 2);
        const uint64_t dS = make_smem_desc(smem_u32(sb), 16, 1024, 2);
#pragma unroll
        for (int ks = 0; ks < 4; ++ks)
          mma_ss(tmem_base + COL_O + 80u * ob, dQ + (uint64_t)(2 * ks), dS + (uint64_t)(2 * ks), IDESC_A, ks > 0 ? 1u : 0u);
        mma_commit(&bars[B_X_FREE + buf]);
        mma_commit(&bars[B_O_DONE + ob]);
      }
      __syncwarp();
      ++used;
    }
    // every MMA has completed before the CTA gives its tensor memory back
    if (ok && used > 0 && !WAIT(B_X_FREE + ((used - 1u) & 1u), (used - 1u) >> 1)) FAIL(405);
    tc_fence_after_sync();
  } else {
    // ================= epilogues: moment rows -> bf16 operand tile; output rows -> global memory =================
    const int l = w * 32 + lane;
    const uint32_t lane_addr = tmem_base + ((uint32_t)(w * 32) << 16);
    bool ok = true;
    if (nkc > 0) {
      if (!WAIT(B_S_DONE, 0)) { FAIL(410); ok = false; }
      if (ok) {
        __syncwarp();
        tc_fence_after_sync();
        uint32_t ra[32], rb[32], r8[8];
        tmem_ld32(lane_addr + COL_S, ra);
        tmem_ld32(lane_addr + COL_S + 32u, rb);
        tmem_ld8(lane_addr + COL_S0, r8);
        tmem_ld_wait();
        if (l < 80) {   // row l of c1 S^T: 64 bf16 = eight 16-byte pieces, 128-byte swizzle
          const int sw = l & 7;
#pragma unroll
          for (int c8 = 0; c8 < 8; ++c8) {
            const uint32_t* r = c8 < 4 ? &ra[8 * c8] : &rb[8 * (c8 - 4)];
            *reinterpret_cast<uint4*>(sb + l * 128 + ((c8 ^ sw) << 4)) =
                make_uint4(pack_bf16(__uint_as_float(r[0]) * P.c1, __uint_as_float(r[1]) * P.c1),
                           pack_bf16(__uint_as_float(r[2]) * P.c1, __uint_as_float(r[3]) * P.c1),
                           pack_bf16(__uint_as_float(r[4]) * P.c1, __uint_as_float(r[5]) * P.c1),
                           pack_bf16(__uint_as_float(r[6]) * P.c1, __uint_as_float(r[7]) * P.c1));
          }
          t0[l] = P.c0 * __uint_as_float(r8[0]);
        }
        fence_proxy_async_smem();
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(&bars[B_SB_READY]);
        // the other epilogue warps' t0 entries are needed below
        if (!WAIT(B_SB_READY, 0)) { FAIL(411); ok = false; }
      }
    } else {
      if (l < 80) t0[l] = 0.f;   // no keys: every output is 0 / 0 as the definition says
      __syncwarp();
    }
    float* gbase = P.g.ptr ? reinterpret_cast<float*>(const_cast<void*>(P.g.ptr)) + (long long)b_idx * P.g.sb + (long long)h_idx * P.g.sh : nullptr;
    uint8_t* ost = sm + OFF_OST + w * 4096;   // this warp's staging box: row = lane
    for (int c = 0; c < nqc && ok; ++c) {
      const uint32_t ob = (uint32_t)c & 1u;
      if (!WAIT(B_O_DONE + ob, (uint32_t)(c >> 1))) { FAIL(412); break; }
      __syncwarp();
      tc_fence_after_sync();
      uint32_t ra[32], rb[32], r8[8];
      tmem_ld32(lane_addr + COL_O + 80u * ob, ra);
      tmem_ld32(lane_addr + COL_O + 80u * ob + 32u, rb);
      tmem_ld8(lane_addr + COL_O + 80u * ob + 64u, r8);
      tmem_ld_wait();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(&bars[B_O_FREE + ob]);
        bulk_wait_read_all();   // the previous chunk's store has read the staging box
      }
      __syncwarp();
      const long long row = (long long)c * CH + l;
      const float gsum = __uint_as_float(r8[0]) + t0[64];
      const float inv = 1.f / gsum;
      const int sw = lane & 7;
#pragma unroll
      for (int c8 = 0; c8 < 8; ++c8) {
        const uint32_t* r = c8 < 4 ? &ra[8 * c8] : &rb[8 * (c8 - 4)];
        float x[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) x[e] = (__uint_as_float(r[e]) + t0[8 * c8 + e]) * inv;
        *reinterpret_cast<uint4*>(ost + lane * 128 + ((c8 ^ sw) << 4)) =
            make_uint4(pack_bf16(x[0], x[1]), pack_bf16(x[2], x[3]), pack_bf16(x[4], x[5]), pack_bf16(x[6], x[7]));
      }
      if (gbase && row < P.nq) gbase[row * P.g.sn] = gsum;
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0 && (long long)c * CH + w * 32 < P.nq) {
        tma_store_4d(&tmo, ost, 0, c * CH + w * 32, h_idx, b_idx);
        bulk_commit_group();
      }
    }
    if (lane == 0) bulk_wait_all();   // the last store has landed before the CTA retires
  }

  tc_fence_before_sync();
  __syncthreads();
  if (w == 0) tmem_dealloc(tmem_base, 256);
}

}  // namespace p1
