// Backward "chain-rule" scans with the state-update operands in tensor memory.  Included by tc_kernels.cu inside
// fm::tc, after tc_scan2.cuh (whose slab helpers and wait helpers it reuses).
//
// One kernel template serves the two scans that differentiate through Phi:
//   dq scan (DK = false), chunks ascending:   dq_c = chain(dO'_c  Sb_{<c}^T, Q_c)     S  += Phi(K_c)^T [V_c | 1]
//   dk scan (DK = true),  chunks descending:  dk_c = chain([V|1]_c dSb_{>c}^T, K_c)   dS += Phi(Q_c)^T dO'_c
// "G" is the 80-column tile that multiplies the state copy (dO' | [V|1]), "Y" the right-hand side of the state
// update ([V|1] | dO'), "X" the tile whose Phi^T builds the state (K | Q, from the transposed copies) and "Z" the
// rows the chain rule differentiates (Q | K, read straight from global memory by the chain-rule threads).
// Which chunks run the chain rule, which update the state and where its bf16 copy is refreshed comes from the
// call's schedule (Sched, tc_kernels.cu); the scan may start from a caller-provided state.
// Per 128-token chunk and 128-row feature tile t of the CTA's slice:
//   dphi    D_u (128 tok x 64 feat) = G_c (128 x 80, smem, K-major) * Sb_t[unit u]^T     per 64-feature unit u, SS MMA
//   update  S_t (128 feat x 80)    += Phi_t(X_c)^T (TMEM slabs, as in tc_scan2.cuh) * Y_c (128 tok x 80, smem)
//   chain   dz[8a+mi] += w D_u[mi][ri] z[8b+ri],  dz[8b+ri] += w D_u[mi][ri] z[8a+mi]    CUDA cores, out of TMEM
// The state copy Sb is a plain bf16 rounding of S; the polynomial weights (c2, 2 c2 for an off-diagonal unit, c1
// for the linear tile) are applied in float32 by the chain rule.
// TMEM columns: 0..319 four state accumulators, 320..447 two dphi buffers, 448..511 two update slabs.
// Warp roles (768 threads, six warp groups): 0-3 / 4-7 chain-rule groups (group g takes the units with sequence
// parity g and dphi buffer g), 8-11 / 12-15 update-slab producers (set s makes half s of every tile into ring slot
// s), 16-19 state conversion, 20 and 23 dphi issuers (one per chain-rule group), 21 update issuer, 22 TMA loader and
// dz drain.  The chain-rule groups raise their register allowance with setmaxnreg (block accumulators and half a
// dphi tile in registers), the others lower theirs.  The two groups add their dz blocks into a shared-memory
// staging tile; the loader warp adds it to the float32 accumulator in global memory with one bulk reduce per chunk
// and zeroes it again.  Every wait is bounded (abort flag + error code).
#pragma once

namespace s3 {

using s2::wait_fast;
using s2::fail_record;
using s2::KT_ROW;
using s2::KT_BOX;
using s2::KT_BUF;

constexpr int THREADS = 768;
constexpr int W_PROD = 8, W_CONS = 16, W_DPHI = 20, W_UPD = 21, W_TMA = 22, W_DPHI2 = 23;
// setmaxnreg moves registers inside the pool the CTA was LAUNCHED with (80 per thread x 768 threads, i.e. 6 x 80 = 480 per
// lane slot): an `inc` that the pool cannot satisfy blocks forever, so the four allowances below must add up to <= 480.
constexpr int REG_LAUNCH = 80;   // what ptxas gives a 768-thread kernel; the host checks it (cudaFuncGetAttributes) before launching
constexpr int REG_CHAIN = 136, REG_PROD = 56, REG_CONS = 56, REG_MISC = 40;
static_assert(2 * REG_CHAIN + 2 * REG_PROD + REG_CONS + REG_MISC <= 6 * REG_LAUNCH, "register pool of the CTA");
constexpr int TILE9 = 9 * BLK;                         // an 80-column tile stored as 9 column blocks (72 columns)
constexpr int OFF_SB = 0;                              // 4 x SB_TILE
constexpr int OFF_VP = OFF_SB + 4 * SB_TILE;           // 73728: [V|1], 2 buffers
constexpr int OFF_DO = OFF_VP + 2 * TILE9;             // 110592: dO', 2 buffers
constexpr int OFF_ZERO = OFF_DO + 2 * TILE9;           // 147456: one zero column block (column block 9 of G)
constexpr int OFF_XT = OFF_ZERO + BLK;                 // 149504: transposed X tile, 2 x KT_BUF
constexpr int OFF_STG = OFF_XT + 2 * KT_BUF;           // 186368: dz staging, 128 rows x ACC_LD floats
constexpr int STG_BYTES = CH * ACC_LD * 4;             // 34816
constexpr int OFF_BAR = OFF_STG + STG_BYTES;           // 221184
constexpr int SMEM_BYTES = OFF_BAR + 512 + 1024;
static_assert(OFF_XT % 128 == 0 && OFF_STG % 128 == 0 && OFF_BAR % 8 == 0, "tile alignment");
static_assert(SMEM_BYTES <= 232448, "shared memory budget");
constexpr uint32_t COL_DPHI = 320u, COL_A = 448u;
// barriers
constexpr int B_FULL = 0, B_EMPTY = 2, B_XT_READY = 4, B_XT_FREE = 6, B_VP_READY = 8, B_VP_FREE = 10, B_DO_READY = 12,
              B_DO_FREE = 14, B_SB_READY = 16, B_S_DONE = 20, B_A_DONE = 24, B_DPHI_DONE = 28, B_DPHI_FREE = 30,
              B_STG_FREE = 32, B_STG_HALF = 33, B_STG_FULL = 34, B_COUNT = 35;

struct ChainParams {
  float* out;          // dq accumulator [BH][nz][ACC_LD] | dk accumulator
  View z;              // rows the chain rule differentiates: q | k (bf16, strided)
  int heads;
  int nz;              // rows of Z and of the output (dq: nq; dk: nk)
  int nk;              // number of keys (rows of the ones column of [V|1] that are 1)
  int z_shift;         // Z row of chunk position p is p - z_shift (dq: nk - nq; dk: 0)
  int do_shift;        // dO' row of chunk position p is p - do_shift (nk - nq)
  int nchunks;
  float c1, c2;
  const float* state_in;   // optional: the state the scan starts from (dq: moments of earlier keys; dk: gradient moments of
                           // later queries), float32 [BH][state_rows][68]; sc.h = 1
  Sched sc;                // which chunks run the chain rule ("apply") / update the state
  int nslices, tps, tile_first, state_rows;   // as in s2::ApplyParams
};

template <int R> __device__ __forceinline__ void reg_inc() { asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(R)); }
template <int R> __device__ __forceinline__ void reg_dec() { asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(R)); }

__device__ __forceinline__ void unpack8(const uint4& x, float s, float (&out)[8]) {
  const uint32_t wv[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    out[2 * i] = __uint_as_float(wv[i] << 16) * s;
    out[2 * i + 1] = __uint_as_float(wv[i] & 0xffff0000u) * s;
  }
}

template <bool DK>
__global__ void __launch_bounds__(THREADS, 1)
scan_chain_kernel(const __grid_constant__ CUtensorMap tmxt, const __grid_constant__ CUtensorMap tmv,
                  const __grid_constant__ CUtensorMap tmdo, const ChainParams P) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  uint8_t* sm = smem_raw + (((raw_addr + 1023u) & ~1023u) - raw_addr);
  uint8_t* sb = sm + OFF_SB;
  uint8_t* vp = sm + OFF_VP;
  uint8_t* dop = sm + OFF_DO;
  uint8_t* xtile = sm + OFF_XT;
  float* stg = reinterpret_cast<float*>(sm + OFF_STG);
  uint64_t* bars = reinterpret_cast<uint64_t*>(sm + OFF_BAR);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(sm + OFF_BAR + 320);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(sm + OFF_BAR + 328);
  // roles of the two 80-column tiles
  uint8_t* gtile = DK ? vp : dop;     // A operand of dphi
  uint8_t* ytile = DK ? dop : vp;     // B operand of the state update
  constexpr int B_G_READY = DK ? B_VP_READY : B_DO_READY, B_G_FREE = DK ? B_VP_FREE : B_DO_FREE;
  constexpr int B_Y_READY = DK ? B_DO_READY : B_VP_READY, B_Y_FREE = DK ? B_DO_FREE : B_VP_FREE;

  const int tid = threadIdx.x, w = tid >> 5, lane = tid & 31;
  // The five slices of a head are neighbours in the grid, so they run at about the same time and share the head's
  // q / k / v tiles through L2.  gridDim.x = 5 * batch * heads.
  const int head = (int)blockIdx.x / P.nslices, slice = (int)blockIdx.x - P.nslices * head;
  const int b_idx = head / P.heads, h_idx = head - b_idx * P.heads;
  const int tile0 = P.tile_first + slice * P.tps;
  const int ntl = (NTILES - tile0) < P.tps ? (NTILES - tile0) : P.tps;
  const int nch = P.nchunks;
  const Sched sc = P.sc;
  auto chunk_of = [&](int i) -> int { return DK ? (nch - 1 - i) : i; };  // i-th chunk of the scan
  auto units_of = [&](int t) -> int { return (tile0 + t < NTILES - 1) ? 2 : 1; };  // the constant feature has no gradient

  if (tid == 0) {
    for (int i = 0; i < 2; ++i) {
      mbar_init(&bars[B_FULL + i], 4);     mbar_init(&bars[B_EMPTY + i], 1);
      mbar_init(&bars[B_XT_READY + i], 1); mbar_init(&bars[B_XT_FREE + i], 8);
      mbar_init(&bars[B_VP_READY + i], 1); mbar_init(&bars[B_VP_FREE + i], DK ? 2 : 1);   // G: one commit per dphi issuer
      mbar_init(&bars[B_DO_READY + i], 1); mbar_init(&bars[B_DO_FREE + i], DK ? 1 : 2);
      mbar_init(&bars[B_DPHI_DONE + i], 1); mbar_init(&bars[B_DPHI_FREE + i], 4);
    }
    for (int i = 0; i < 4; ++i) { mbar_init(&bars[B_SB_READY + i], 4); mbar_init(&bars[B_S_DONE + i], 1); mbar_init(&bars[B_A_DONE + i], 2); }
    mbar_init(&bars[B_STG_FREE], 1);
    mbar_init(&bars[B_STG_HALF], 4);   // group 0's warps
    mbar_init(&bars[B_STG_FULL], 4);   // group 1's warps
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (w == 0) tmem_alloc(tmem_slot, 512);
  // operands are read one column block past what is stored (times zeros): keep every byte of them finite
  for (int i = tid; i < OFF_XT / 16; i += THREADS) reinterpret_cast<uint4*>(sm)[i] = make_uint4(0u, 0u, 0u, 0u);
  for (int i = tid; i < STG_BYTES / 16; i += THREADS) reinterpret_cast<uint4*>(stg)[i] = make_uint4(0u, 0u, 0u, 0u);  // dz staging starts at zero
  fence_proxy_async_smem();
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  // (no out-of-line calls in this kernel: its warp groups run with different register allowances)
  auto WAIT = [&](int bar, uint32_t n) -> bool { return mbar_wait_abortable(&bars[bar], n & 1u, WAIT_CYCLES, abort_flag); };
  auto FAIL = [&](int code) {
    if (*abort_flag == 0) atomicAdd(&g_tc_wait_hist[code & 255], 1);
    *abort_flag = 1;
    atomicExch(&g_tc_status, code);
  };

  if (w < W_PROD) {
    // ================= chain rule: dphi (TMEM) -> dz rows =================
    // Group g takes the units with sequence parity g.  In any slice those touch at most five of the eight 8-column
    // blocks of dz, so a thread keeps five block accumulators (40 registers) instead of dz[64], which leaves room
    // to read half a dphi tile (32 values) per TMEM load.
    reg_inc<REG_CHAIN>();
    const int grp = w >> 2;
    const int l = (w & 3) * 32 + lane;
    const uint32_t dphi_addr = tmem_base + ((uint32_t)((w & 3) * 32) << 16) + COL_DPHI + 64u * grp;
    const __nv_bfloat16* zbase = reinterpret_cast<const __nv_bfloat16*>(P.z.ptr) + (long long)b_idx * P.z.sb + (long long)h_idx * P.z.sh;
    uint64_t pairs = 0;     // 16 bits per tile: block pairs (a0, b0, a1, b1) of its two 64-feature units
    uint32_t slot_of = 0xffffffffu;  // 4 bits per block: accumulator slot of the block in this group (15 = not used)
    uint32_t blk_of = 0;    // 4 bits per slot: the block it accumulates
    int nslots = 0;
    {
      int mm = 0;
      for (int t = 0; t < ntl; ++t) {
        if (tile0 + t == NTILES - 1) continue;
        int ab[4];
        pair_decode(2 * (tile0 + t), 8, ab[0], ab[1]);
        pair_decode(2 * (tile0 + t) + 1, 8, ab[2], ab[3]);
        pairs |= (uint64_t)(ab[0] | (ab[1] << 4) | (ab[2] << 8) | (ab[3] << 12)) << (16 * t);
        for (int u = 0; u < 2; ++u, ++mm) {
          if ((mm & 1) != grp) continue;
          for (int e = 0; e < 2; ++e) {
            const int blk = ab[2 * u + e];
            if (((slot_of >> (4 * blk)) & 15u) == 15u) {
              slot_of = (slot_of & ~(15u << (4 * blk))) | ((uint32_t)nslots << (4 * blk));
              blk_of |= (uint32_t)blk << (4 * nslots);
              ++nslots;
            }
          }
        }
      }
    }
    // this group's pair units of a chunk (the same in every chunk), 16 bits each: a | b << 4 | slot(a) << 8 | slot(b) << 12
    uint64_t my_units = 0;
    int n_mine = 0;
    bool lin_mine = false;   // the group also owns the linear tile's unit (the last unit of the chunk): added at the drain
    {
      int mm = 0;
      for (int t = 0; t < ntl; ++t) {
        const bool lin = (tile0 + t == NTILES - 1);
        const uint32_t pr = (uint32_t)(pairs >> (16 * t)) & 0xffffu;
        for (int u = 0; u < (lin ? 1 : 2); ++u, ++mm) {
          if ((mm & 1) != grp) continue;
          if (lin) { lin_mine = true; continue; }
          const uint32_t a = (u ? (pr >> 8) : pr) & 15u, b = (u ? (pr >> 12) : (pr >> 4)) & 15u;
          const uint32_t d16 = a | (b << 4) | (((slot_of >> (4 * a)) & 15u) << 8) | (((slot_of >> (4 * b)) & 15u) << 12);
          my_units |= (uint64_t)d16 << (16 * n_mine);
          ++n_mine;
        }
      }
    }
    float acc[5][8];
    uint32_t cnt = 0;     // units this group has taken = phase count of its dphi buffer
    bool ok = true;
    for (int ci = 0; ci < nch && ok; ++ci) {
      if (!sc.A(ci)) continue;
      const int c = chunk_of(ci);
      const long long row = (long long)c * CH + l - P.z_shift;
      const bool valid = row >= 0 && row < P.nz;
      const uint4* zrow = reinterpret_cast<const uint4*>(zbase + (valid ? row : 0) * P.z.sn);
#pragma unroll
      for (int sl = 0; sl < 5; ++sl)
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[sl][j] = 0.f;
      {
#pragma unroll 1
        for (int iu = 0; iu < n_mine; ++iu) {
          const uint32_t d16 = (uint32_t)(my_units >> (16 * iu)) & 0xffffu;
          const int a = (int)(d16 & 15u), b = (int)((d16 >> 4) & 15u), sa = (int)((d16 >> 8) & 15u), sbk = (int)(d16 >> 12);
          // the z blocks of this unit, before the wait so the loads fly meanwhile
          uint4 za4 = make_uint4(0u, 0u, 0u, 0u), zb4 = make_uint4(0u, 0u, 0u, 0u);
          if (valid) { za4 = zrow[a]; zb4 = zrow[b]; }
          if (!WAIT(B_DPHI_DONE + grp, cnt)) { FAIL(320); ok = false; break; }
          ++cnt;
          __syncwarp();
          tc_fence_after_sync();
          const float wgt = (a == b) ? P.c2 : 2.f * P.c2;
          // packed float32 FMAs (two per instruction): pairs run over ri
          float za[8], zb[8], dza[8];
          float2 dzb2[4];
          unpack8(za4, wgt, za);
          unpack8(zb4, wgt, zb);
#pragma unroll
          for (int j = 0; j < 8; ++j) dza[j] = 0.f;
#pragma unroll
          for (int j = 0; j < 4; ++j) dzb2[j] = make_float2(0.f, 0.f);
#pragma unroll
          for (int hf = 0; hf < 2; ++hf) {
            uint32_t r[32];
            tmem_ld32(dphi_addr + 32u * hf, r);
            tmem_ld_wait();
            if (hf == 1) {  // the whole unit has been read: the buffer can take the next one
              tc_fence_before_sync();
              __syncwarp();
              if (lane == 0) mbar_arrive(&bars[B_DPHI_FREE + grp]);
            }
#pragma unroll
            for (int mi = 0; mi < 4; ++mi) {
              float2 s2v = make_float2(0.f, 0.f);
              const float2 zam = make_float2(za[4 * hf + mi], za[4 * hf + mi]);
#pragma unroll
              for (int rp = 0; rp < 4; ++rp) {
                const float2 d = make_float2(__uint_as_float(r[mi * 8 + 2 * rp]), __uint_as_float(r[mi * 8 + 2 * rp + 1]));
                s2v = __ffma2_rn(d, make_float2(zb[2 * rp], zb[2 * rp + 1]), s2v);
                dzb2[rp] = __ffma2_rn(d, zam, dzb2[rp]);
              }
              dza[4 * hf + mi] += s2v.x + s2v.y;
            }
          }
          float dzb[8];
#pragma unroll
          for (int j = 0; j < 4; ++j) { dzb[2 * j] = dzb2[j].x; dzb[2 * j + 1] = dzb2[j].y; }
          // the slots are warp-uniform: selecting them with unrolled compares keeps the accumulators in registers
#pragma unroll
          for (int sl = 0; sl < 5; ++sl) {
            if (sa == sl) {
#pragma unroll
              for (int j = 0; j < 8; ++j) acc[sl][j] += dza[j];
            }
            if (sbk == sl) {
#pragma unroll
              for (int j = 0; j < 8; ++j) acc[sl][j] += dzb[j];
            }
          }
        }
      }
      if (!ok) break;
      // ---- the chunk's dz: both groups add their blocks into the (zeroed) staging rows, group 0 first; the drain
      //      warp then adds the rows to global memory with one bulk reduce and zeroes them again ----
      float* rowf = stg + l * ACC_LD;
      const uint32_t j = (uint32_t)sc.na_before(ci);  // drains so far
      if (grp == 0) {
        if (j > 0 && !WAIT(B_STG_FREE, j - 1)) { FAIL(321); break; }   // reduced, read and zeroed
      } else {
        if (!WAIT(B_STG_HALF, j)) { FAIL(322); break; }                // group 0's blocks are in
      }
#pragma unroll
      for (int sl = 0; sl < 5; ++sl) {
        if (sl < nslots) {
          float4* p4 = reinterpret_cast<float4*>(rowf + 8 * ((blk_of >> (4 * sl)) & 15u));
          float4 v0 = p4[0], v1 = p4[1];
          v0.x += acc[sl][0]; v0.y += acc[sl][1]; v0.z += acc[sl][2]; v0.w += acc[sl][3];
          v1.x += acc[sl][4]; v1.y += acc[sl][5]; v1.z += acc[sl][6]; v1.w += acc[sl][7];
          p4[0] = v0; p4[1] = v1;
        }
      }
      if (lin_mine) {  // linear tile: feature m = x[m], weight c1: dz[m] += c1 dphi[m]
        if (!WAIT(B_DPHI_DONE + grp, cnt)) { FAIL(324); break; }
        ++cnt;
        __syncwarp();
        tc_fence_after_sync();
        float4* p4 = reinterpret_cast<float4*>(rowf);
#pragma unroll
        for (int hf = 0; hf < 2; ++hf) {
          uint32_t r[32];
          tmem_ld32(dphi_addr + 32u * hf, r);
          tmem_ld_wait();
          if (hf == 1) {
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(&bars[B_DPHI_FREE + grp]);
          }
#pragma unroll
          for (int q = 0; q < 8; ++q) {
            float4 v = p4[8 * hf + q];
            v.x += P.c1 * __uint_as_float(r[4 * q]);     v.y += P.c1 * __uint_as_float(r[4 * q + 1]);
            v.z += P.c1 * __uint_as_float(r[4 * q + 2]); v.w += P.c1 * __uint_as_float(r[4 * q + 3]);
            p4[8 * hf + q] = v;
          }
        }
      }
      fence_proxy_async_smem();   // the copy engine reads these rows
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars[grp == 0 ? B_STG_HALF : B_STG_FULL]);
    }
  } else if (w < W_CONS) {
    // ================= producers: update slabs (Phi(X)^T, thread = feature) into the two TMEM slots =================
    reg_dec<REG_PROD>();
    const int set = (w - W_PROD) >> 2;    // = half of the tile's tokens = ring slot
    const int f = (w & 3) * 32 + lane;    // feature of the tile = TMEM lane
    const uint32_t slot_addr = tmem_base + ((uint32_t)((w & 3) * 32) << 16) + COL_A + 32u * set;
    uint64_t pairs = 0;
#pragma unroll
    for (int t = 0; t < 4; ++t) {
      int a0 = 0, b0 = 0, a1 = 0, b1 = 0;
      if (tile0 + t < NTILES - 1) { pair_decode(2 * (tile0 + t), 8, a0, b0); pair_decode(2 * (tile0 + t) + 1, 8, a1, b1); }
      pairs |= (uint64_t)(a0 | (b0 << 4) | (a1 << 8) | (b1 << 12)) << (16 * t);
    }
    uint32_t k = 0;   // slabs this set has produced = phase count of its slot
    bool ok = true;
    for (int ci = 0; ci < nch && ok; ++ci) {
      const int buf = ci & 1;
      if (!WAIT(B_XT_READY + buf, (uint32_t)(ci >> 1))) { FAIL(300); break; }
      const uint8_t* box = xtile + buf * KT_BUF + set * KT_BOX;
      for (int t = 0; t < ntl && ok && sc.U(ci); ++t, ++k) {
        const bool lin = (tile0 + t == NTILES - 1);
        const uint32_t pr = (uint32_t)(pairs >> (16 * t)) & 0xffffu;
        uint32_t r[32];
        if (!lin) {
          const uint32_t q = (f >> 6) ? (pr >> 8) : pr;
          s2::update_pair_slab(r, box, 8 * (int)(q & 15) + ((f >> 3) & 7), 8 * (int)((q >> 4) & 15) + (f & 7));
        } else if (f < 64) s2::copy_trow_slab(r, box, f);
        else s2::fill_slab(r, f == 64 ? 0x3F803F80u : 0u);
        if (k > 0 && !WAIT(B_EMPTY + set, k - 1)) { FAIL(301); ok = false; break; }
        __syncwarp();
        tc_fence_after_sync();
        tmem_st32(slot_addr, r);
        tmem_st_wait();
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(&bars[B_FULL + set]);
      }
      if (ok) {
        __syncwarp();
        if (lane == 0) mbar_arrive(&bars[B_XT_FREE + buf]);
      }
    }
  } else if (w < W_DPHI) {
    // ================= state conversion: S_t (TMEM, float32) -> Sb_t (shared memory, bf16) =================
    reg_dec<REG_CONS>();
    const int l = (w & 3) * 32 + lane;
    const uint32_t lane_addr = tmem_base + ((uint32_t)((w & 3) * 32) << 16);
    bool ok = true;
    auto convert_tile = [&](int t) {
      uint8_t* dst = sb + t * SB_TILE + l * 16;
#pragma unroll
      for (int part = 0; part < 2; ++part) {
        uint32_t r[32];
        tmem_ld32(lane_addr + 80u * t + 32u * part, r);
        tmem_ld_wait();
#pragma unroll
        for (int jb = 0; jb < 4; ++jb) store_block8_plain(dst + (4 * part + jb) * BLK, &r[8 * jb]);
      }
      uint32_t r8[8];
      tmem_ld8(lane_addr + 80u * t + 64u, r8);
      tmem_ld_wait();
      store_block8_plain(dst + 8 * BLK, r8);
      fence_proxy_async_smem();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars[B_SB_READY + t]);
    };
    if (sc.h) {
      // the scan starts from the caller's state: rows -> TMEM accumulators (80 columns: 64 values, the denominator
      // moment, zeros), then the first bf16 copy; the SB_READY arrival orders the stores before the first update MMA
      constexpr int ST_LD = 68;
      const float* sbase = P.state_in + (long long)head * P.state_rows * ST_LD;
      for (int t = 0; t < ntl; ++t) {
        const int srow = 128 * (tile0 + t - P.tile_first) + l;
        const bool have = srow < P.state_rows;
        const float4* src = reinterpret_cast<const float4*>(sbase + (long long)(have ? srow : 0) * ST_LD);
#pragma unroll
        for (int part = 0; part < 2; ++part) {
          uint32_t r[32];
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const float4 x = have ? src[8 * part + j] : make_float4(0.f, 0.f, 0.f, 0.f);
            r[4 * j] = __float_as_uint(x.x); r[4 * j + 1] = __float_as_uint(x.y); r[4 * j + 2] = __float_as_uint(x.z); r[4 * j + 3] = __float_as_uint(x.w);
          }
          tmem_st32(lane_addr + 80u * t + 32u * part, r);
        }
        uint32_t rc[16];
        rc[0] = have ? __float_as_uint(src[16].x) : 0u;
#pragma unroll
        for (int j = 1; j < 16; ++j) rc[j] = 0u;
        tmem_st16(lane_addr + 80u * t + 64u, rc);
        tmem_st_wait();
        convert_tile(t);
      }
    }
    for (int ci = 0; ci < nch && ok; ++ci) {
      if (!sc.C(ci)) continue;
      const int na_thr = sc.na_before(ci) + (sc.A(ci) ? 1 : 0);
      for (int t = 0; t < ntl && ok; ++t) {
        // S_t is final (this chunk's update) and Sb_t is no longer read (the dphi MMAs up to and including this chunk's)
        if (!WAIT(B_S_DONE + t, (uint32_t)(sc.nc_before(ci) - sc.h)) || (na_thr > 0 && !WAIT(B_A_DONE + t, (uint32_t)(na_thr - 1)))) { FAIL(310); ok = false; break; }
        __syncwarp();
        tc_fence_after_sync();
        convert_tile(t);
      }
    }
  } else {
    reg_dec<REG_MISC>();
    if (w == W_DPHI || w == W_DPHI2) {
      // ================= dphi issuers: D_u = G_c Sb_t[unit u]^T, five K = 16 steps over the 80 columns =================
      // One issuer per chain-rule group / dphi buffer: warp W_DPHI takes the units with an even index in the chunk,
      // warp W_DPHI2 the odd ones, so a group's next tile is issued while the group still works on the current one.
      constexpr uint32_t IDESC = make_idesc_bf16(128, 64, 0, 0);   // A K-major, B K-major
      const uint32_t db = (w == W_DPHI) ? 0u : 1u;
      uint32_t cnt = 0;   // units issued into this buffer
      bool ok = true;
      for (int ci = 0; ci < nch && ok; ++ci) {
        const int buf = ci & 1;
        int mu = 0;       // index of the unit within the chunk
        if (!WAIT(B_G_READY + buf, (uint32_t)(ci >> 1))) { FAIL(330); break; }
        const uint32_t g_addr = smem_u32(gtile + buf * TILE9);
        const uint64_t dA = make_smem_desc(g_addr, 2048, 128, 0);                       // column blocks 2 ks, 2 ks + 1
        const uint64_t dA_last = make_smem_desc(g_addr + 8 * BLK, smem_u32(sm + OFF_ZERO) - (g_addr + 8 * BLK), 128, 0);  // 8, zero
        const int nc = sc.nc_before(ci);
        for (int t = 0; t < ntl && ok && sc.A(ci); ++t) {
          if (nc > 0 && !WAIT(B_SB_READY + t, (uint32_t)(nc - 1))) { FAIL(331); ok = false; break; }
          const int nu = units_of(t);
          for (int u = 0; u < nu && ok; ++u, ++mu) {
            if ((uint32_t)(mu & 1) != db) continue;
            if (cnt > 0 && !WAIT(B_DPHI_FREE + db, cnt - 1u)) { FAIL(332); ok = false; break; }
            ++cnt;
            __syncwarp();
            tc_fence_after_sync();
            if (elect_one()) {
              const uint32_t d = tmem_base + COL_DPHI + 64u * db;
              const uint64_t b0 = make_smem_desc(smem_u32(sb + t * SB_TILE + u * 1024), 2048, 128, 0);
#pragma unroll
              for (int ks = 0; ks < 4; ++ks) mma_ss(d, dA + (uint64_t)(256 * ks), b0 + (uint64_t)(256 * ks), IDESC, ks > 0 ? 1u : 0u);
              mma_ss(d, dA_last, b0 + (uint64_t)(256 * 4), IDESC, 1u);
              mma_commit(&bars[B_DPHI_DONE + db]);
            }
            __syncwarp();
          }
          // this issuer's MMAs on Sb_t are all issued (possibly none): its half of the tile's "no longer read" signal
          if (ok && elect_one()) mma_commit(&bars[B_A_DONE + t]);
          __syncwarp();
        }
        if (ok && elect_one()) mma_commit(&bars[B_G_FREE + buf]);   // this issuer's dphi MMAs of the chunk have read G
        __syncwarp();
      }
      if (ok && nch > 0 && !WAIT(B_G_FREE + ((nch - 1) & 1), (uint32_t)((nch - 1) >> 1))) FAIL(333);
      tc_fence_after_sync();
    } else if (w == W_UPD) {
      // ================= update issuer: S_t += Phi_t(X_c)^T Y_c, two 64-token slabs per tile =================
      constexpr uint32_t IDESC = make_idesc_bf16(128, 80, 0, 1);   // A from TMEM (K-major), B MN-major
      uint32_t k = 0;   // tiles issued = phase count of both slots
      bool ok = true;
      for (int ci = 0; ci < nch && ok; ++ci) {
        const int buf = ci & 1;
        if (!WAIT(B_Y_READY + buf, (uint32_t)(ci >> 1))) { FAIL(340); break; }
        const uint64_t dB = make_smem_desc(smem_u32(ytile + buf * TILE9), 128, 2048, 0);
        const int nc = sc.nc_before(ci);
        const uint32_t acc0 = (sc.nu_before(ci) > 0 || sc.h) ? 1u : 0u;   // the first update starts the accumulators
        if (!sc.U(ci)) {   // nothing of this chunk reads the Y buffer: hand it back
          if (elect_one()) mma_commit(&bars[B_Y_FREE + buf]);
          __syncwarp();
          continue;
        }
        for (int t = 0; t < ntl && ok; ++t, ++k) {
          // S_t may be overwritten once the latest copy of it exists
          if (nc > 0 && !WAIT(B_SB_READY + t, (uint32_t)(nc - 1))) { FAIL(341); ok = false; break; }
          const uint32_t d = tmem_base + 80u * t;
#pragma unroll
          for (int hf = 0; hf < 2; ++hf) {
            if (!WAIT(B_FULL + hf, k)) { FAIL(342); ok = false; break; }
            __syncwarp();
            tc_fence_after_sync();
            if (elect_one()) {
              const uint32_t a0 = tmem_base + COL_A + 32u * hf;
              const uint64_t b0 = dB + (uint64_t)(64 * hf);
              mma_ts(d, a0, b0, IDESC, hf > 0 ? 1u : acc0);
              mma_ts(d, a0 + 8u, b0 + 16u, IDESC, 1u);
              mma_ts(d, a0 + 16u, b0 + 32u, IDESC, 1u);
              mma_ts(d, a0 + 24u, b0 + 48u, IDESC, 1u);
              mma_commit(&bars[B_EMPTY + hf]);
              if (hf == 1) {
                if (sc.SD(ci)) mma_commit(&bars[B_S_DONE + t]);
                if (t == ntl - 1) mma_commit(&bars[B_Y_FREE + buf]);
              }
            }
            __syncwarp();
          }
        }
      }
      if (ok && nch > 0 && !WAIT(B_Y_FREE + ((nch - 1) & 1), (uint32_t)((nch - 1) >> 1))) FAIL(343);
      tc_fence_after_sync();
    } else if (w == W_TMA) {
      // ================= TMA loader + dz drain =================
      // Besides streaming the tiles (two chunks ahead of the compute roles) this warp adds the staged dz rows of a
      // finished chunk to the accumulator in global memory: one bulk reduce-add, then the rows are zeroed again.
      float* obase = P.out + (long long)head * P.nz * ACC_LD;
      bool ok = true;
      uint32_t drained = 0;   // chain-rule chunks sc.a_first .. sc.a_first + drained - 1 have been drained
      const uint32_t na_total = (uint32_t)sc.na_total();
      auto drain_one = [&]() -> bool {
        const int ci = sc.a_first + (int)drained;
        if (!WAIT(B_STG_FULL, drained)) { FAIL(360); return false; }
        __syncwarp();
        if (lane == 0) {
          const long long q0 = (long long)chunk_of(ci) * CH - P.z_shift;  // output row of staging row 0
          const int r0 = q0 < 0 ? (int)(-q0 < CH ? -q0 : CH) : 0;
          const long long lim = (long long)P.nz - q0;
          const int r1 = lim < CH ? (lim < 0 ? 0 : (int)lim) : CH;
          if (r1 > r0) bulk_reduce_add_f32(obase + (q0 + r0) * ACC_LD, stg + r0 * ACC_LD, (uint32_t)(r1 - r0) * (uint32_t)(ACC_LD * 4));
          bulk_commit_group();
          bulk_wait_read_all();   // the copy engine has read the rows
        }
        __syncwarp();
        for (int i = lane; i < STG_BYTES / 16; i += 32) reinterpret_cast<uint4*>(stg)[i] = make_uint4(0u, 0u, 0u, 0u);
        __syncwarp();
        if (lane == 0) mbar_arrive(&bars[B_STG_FREE]);
        ++drained;
        return true;
      };
      for (int ci = 0; ci < nch && ok; ++ci) {
        const int pos0 = chunk_of(ci) * CH, buf = ci & 1;
        const uint32_t k = (uint32_t)(ci >> 1);
        if (k > 0 && !WAIT(B_XT_FREE + buf, k - 1)) { FAIL(350); break; }
        if (lane == 0) {
          mbar_arrive_expect_tx(&bars[B_XT_READY + buf], KT_BUF);
          tma_load_3d(xtile + buf * KT_BUF, &tmxt, &bars[B_XT_READY + buf], pos0, 0, head);
          tma_load_3d(xtile + buf * KT_BUF + KT_BOX, &tmxt, &bars[B_XT_READY + buf], pos0 + 64, 0, head);
        }
        if (k > 0 && !WAIT(B_VP_FREE + buf, k - 1)) { FAIL(351); break; }
        uint8_t* vbuf = vp + buf * TILE9;
        for (int r = lane; r < CH; r += 32)  // the ones column of [V | 1] (zero for rows past the last key)
          *reinterpret_cast<uint4*>(vbuf + 8 * BLK + r * 16) = make_uint4((pos0 + r < P.nk) ? 0x00003F80u : 0u, 0u, 0u, 0u);
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
          mbar_arrive_expect_tx(&bars[B_VP_READY + buf], 8 * BLK);
#pragma unroll
          for (int i = 0; i < 8; ++i) tma_load_4d(vbuf + i * BLK, &tmv, &bars[B_VP_READY + buf], 8 * i, pos0, h_idx, b_idx);
        }
        if (k > 0 && !WAIT(B_DO_FREE + buf, k - 1)) { FAIL(352); break; }
        if (lane == 0) {
          uint8_t* dbuf = dop + buf * TILE9;
          mbar_arrive_expect_tx(&bars[B_DO_READY + buf], 9 * BLK);
#pragma unroll
          for (int i = 0; i < 9; ++i) tma_load_4d(dbuf + i * BLK, &tmdo, &bars[B_DO_READY + buf], 8 * i, pos0 - P.do_shift, h_idx, b_idx);
        }
        __syncwarp();
        // the chunk two behind the one just loaded has left the chain-rule groups (or soon will): drain it
        if (drained < na_total && sc.a_first + (int)drained <= ci - 2) ok = drain_one();
      }
      while (ok && drained < na_total) ok = drain_one();
      if (lane == 0) bulk_wait_all();  // the last reduce has landed before the CTA retires
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (w == 0) tmem_dealloc(tmem_base, 512);
}

}  // namespace s3
