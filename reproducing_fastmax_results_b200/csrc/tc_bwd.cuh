// tcgen05 backward helpers (bf16, head dim 64, order 2, causal).  Included by tc_kernels.cu inside fm::tc.
//   intra_bwd_pipe_kernel     the masked, within-chunk part of dq, dk, dv (persistent, one CTA per SM)
//   bwd_prologue_bf16_kernel  dO' = [dO / g, -(dO . o) / g] rounded to bf16, the 80-column tile the scans read
// The inter-chunk parts are the scans of tc_scan2.cuh (dv) and tc_scan3.cuh (dq, dk).
#pragma once

constexpr int ACC_LD = 68;   // floats per row of the dq / dk / dv accumulators: 272-byte rows keep 128-bit per-thread row
                             // accesses to the shared-memory staging copies free of bank conflicts
// ------------------------------------------------------------------------------------------------------
// intra-chunk causal term of the backward pass, one work item per (chunk, batch*head):
//   P = tril f(Q K^T),  dSm = tril((dO' [V|1]^T) * f'(Q K^T))
//   dq_c += dSm K_c,   dk_c += dSm^T Q_c,   dv_c += P^T dO'_c[:, :64]
// ------------------------------------------------------------------------------------------------------
struct IntraBwdParams {
  float *dq_acc, *dk_acc, *dv_acc;
  int heads, nq, nk, off;
  float c0, c1, c2;
};

// ------------------------------------------------------------------------------------------------------
// A persistent kernel: one CTA per SM walks over (head, chunk) items; per item two MMA groups (scores and dP, then
// dq, dk, dv) with an element-wise pass between them.  A control warp prefetches the operands of the item after
// next (two operand sets in shared memory), issues the MMAs (the next item's scores right behind this item's second
// group) and hands the finished rows to the copy engine, so loads, stores and the first MMA group of neighbouring
// items overlap the compute of the current one.  Shared memory: operand set 0 | P and dS tiles | operand set 1; the output staging
// rows of an item reuse its own operand set and the part of the P / dS tiles next to it.
// Warps 0-7 compute (two 64-column halves x four TMEM lane quarters), warp 8 is the control warp.
// ------------------------------------------------------------------------------------------------------
constexpr int IP_THREADS = 288;
constexpr int IP_SET = 2 * REGION + 20 * BLK;            // 73728: q tile, k tile, [V|1] (10 blocks), dO' (10 blocks)
constexpr int IP_OFF_PD = IP_SET;                        // P (TILE) then dS (TILE)
constexpr int IP_OFF_SET1 = IP_OFF_PD + 2 * TILE;        // 139264
constexpr int IP_OFF_BAR = IP_OFF_SET1 + IP_SET;         // 212992
constexpr int IP_STAGE_BYTES = 3 * CH * ACC_LD * 4;      // 104448
constexpr int IP_SMEM_BYTES = IP_OFF_BAR + 256 + 1024;
static_assert(IP_OFF_PD % 1024 == 0 && IP_OFF_SET1 % 1024 == 0, "swizzled tiles need 1024-byte alignment");
static_assert(IP_STAGE_BYTES <= IP_SET + TILE, "staging = the item's operand set + at most one of the P / dS tiles");
static_assert(IP_SMEM_BYTES <= 232448, "shared memory budget");
constexpr int IPB_FULL = 0, IPB_MMA1 = 2, IPB_PD = 3, IPB_MMA2 = 4, IPB_STAGED = 5, IPB_STAGE_FREE = 6;

__global__ void __launch_bounds__(IP_THREADS, 1)
intra_bwd_pipe_kernel(const __grid_constant__ CUtensorMap tmq, const __grid_constant__ CUtensorMap tmk,
                      const __grid_constant__ CUtensorMap tmv, const __grid_constant__ CUtensorMap tmdo, const IntraBwdParams P,
                      int nch, int nitems) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  uint8_t* sm = smem_raw + (((raw_addr + 1023u) & ~1023u) - raw_addr);
  uint8_t* pt = sm + IP_OFF_PD;
  uint8_t* dt = sm + IP_OFF_PD + TILE;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sm + IP_OFF_BAR);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(sm + IP_OFF_BAR + 128);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(sm + IP_OFF_BAR + 136);
  const int tid = threadIdx.x, w = tid >> 5, lane = tid & 31;

  if (tid == 0) {
    mbar_init(&bars[IPB_FULL], 1);
    mbar_init(&bars[IPB_FULL + 1], 1);
    mbar_init(&bars[IPB_MMA1], 1);
    mbar_init(&bars[IPB_PD], 8);
    mbar_init(&bars[IPB_MMA2], 1);
    mbar_init(&bars[IPB_STAGED], 8);
    mbar_init(&bars[IPB_STAGE_FREE], 1);
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (w == 0) tmem_alloc(tmem_slot, 512);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  constexpr uint32_t COL_SC = 0u, COL_DP = 128u, COL_DQ = 256u, COL_DK = 320u, COL_DVV = 384u;
  auto WAIT = [&](int bar, uint32_t n) -> bool { return mbar_wait_abortable(&bars[bar], n & 1u, WAIT_CYCLES, abort_flag); };
  auto FAIL = [&](int code) {
    if (*abort_flag == 0) atomicAdd(&g_tc_wait_hist[code & 255], 1);
    *abort_flag = 1;
    atomicExch(&g_tc_status, code);
  };
  auto set_base = [&](uint32_t s) -> uint8_t* { return sm + (s ? IP_OFF_SET1 : 0); };
  // staging rows of an item in set s: set 0 -> [0, 104448); set 1 -> the 104448 bytes that end with set 1
  auto stage_base = [&](uint32_t s) -> float* {
    return reinterpret_cast<float*>(sm + (s ? IP_OFF_SET1 + IP_SET - IP_STAGE_BYTES : 0));
  };
  const int first = blockIdx.x, step = gridDim.x;
  const int my_items = first < nitems ? (nitems - first + step - 1) / step : 0;

  if (w == 8) {
    // ================= control warp: loads, MMA issue, stores =================
    auto prefetch = [&](int n) {   // n-th item of this CTA -> operand set n & 1
      const int item = first + n * step;
      const int head = item / nch, c = item - head * nch;
      const int b_idx = head / P.heads, h_idx = head - b_idx * P.heads;
      const int pos0 = c * CH;
      uint8_t* base = set_base((uint32_t)n & 1u);
      uint8_t* vp = base + 2 * REGION;
      uint8_t* dop = vp + 10 * BLK;
      for (int r = lane; r < CH; r += 32) {
        *reinterpret_cast<uint4*>(vp + 8 * BLK + r * 16) = make_uint4((pos0 + r < P.nk) ? 0x00003F80u : 0u, 0u, 0u, 0u);
        *reinterpret_cast<uint4*>(vp + 9 * BLK + r * 16) = make_uint4(0u, 0u, 0u, 0u);
      }
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) {
        uint64_t* full = &bars[IPB_FULL + (n & 1)];
        mbar_arrive_expect_tx(full, 2 * REGION + 18 * BLK);
        tma_load_4d(base, &tmq, full, 0, pos0 - P.off, h_idx, b_idx);
        tma_load_4d(base + REGION, &tmk, full, 0, pos0, h_idx, b_idx);
#pragma unroll
        for (int j = 0; j < 8; ++j) tma_load_4d(vp + j * BLK, &tmv, full, 8 * j, pos0, h_idx, b_idx);
#pragma unroll
        for (int j = 0; j < 10; ++j) tma_load_4d(dop + j * BLK, &tmdo, full, 8 * j, pos0 - P.off, h_idx, b_idx);
      }
      __syncwarp();
    };
    // scores and dP of the n-th item (its operands are loaded; the S / dP columns were read by the previous item's
    // element-wise pass): issued one item ahead, right behind the previous item's second MMA group
    auto issue_scores = [&](int n) -> bool {
      const uint32_t s = (uint32_t)n & 1u;
      uint8_t* base = set_base(s);
      uint8_t* vp = base + 2 * REGION;
      uint8_t* dop = vp + 10 * BLK;
      if (!WAIT(IPB_FULL + s, (uint32_t)(n >> 1))) { FAIL(61); return false; }
      __syncwarp();
      tc_fence_after_sync();
      if (elect_one()) {
        constexpr uint32_t IDESC_128 = make_idesc_bf16(128, 128, 0, 0);
        const uint64_t dq = make_smem_desc(smem_u32(base), 16, 1024, 2);
        const uint64_t dk = make_smem_desc(smem_u32(base + REGION), 16, 1024, 2);
#pragma unroll
        for (int ks = 0; ks < 4; ++ks) mma_ss(tmem_base + COL_SC, dq + (uint64_t)(2 * ks), dk + (uint64_t)(2 * ks), IDESC_128, ks > 0);
        const uint64_t dg = make_smem_desc(smem_u32(dop), 2048, 128, 0);
        const uint64_t dv = make_smem_desc(smem_u32(vp), 2048, 128, 0);
#pragma unroll
        for (int ks = 0; ks < 5; ++ks) mma_ss(tmem_base + COL_DP, dg + (uint64_t)(256 * ks), dv + (uint64_t)(256 * ks), IDESC_128, ks > 0);
        mma_commit(&bars[IPB_MMA1]);
      }
      __syncwarp();
      return true;
    };
    if (my_items > 0) prefetch(0);
    if (my_items > 1) prefetch(1);
    bool ok = my_items > 0 ? issue_scores(0) : true;
    for (int n = 0; n < my_items && ok; ++n) {
      const uint32_t s = (uint32_t)n & 1u;
      const int item = first + n * step;
      const int head = item / nch, c = item - head * nch;
      const int pos0 = c * CH;
      uint8_t* base = set_base(s);
      uint8_t* rawq = base;
      uint8_t* rawk = base + REGION;
      uint8_t* dop = base + 2 * REGION + 10 * BLK;
      if (!WAIT(IPB_PD, (uint32_t)n)) { FAIL(62); break; }
      __syncwarp();
      tc_fence_after_sync();
      if (elect_one()) {
        constexpr uint32_t IDESC_KMN = make_idesc_bf16(128, 64, 0, 1);   // A K-major,  B MN-major
        constexpr uint32_t IDESC_MNMN = make_idesc_bf16(128, 64, 1, 1);  // A MN-major, B MN-major
        const uint64_t dP_MN = make_smem_desc(smem_u32(pt), REGION, 1024, 2);
        const uint64_t dD_K = make_smem_desc(smem_u32(dt), 16, 1024, 2);
        const uint64_t dD_MN = make_smem_desc(smem_u32(dt), REGION, 1024, 2);
        const uint64_t dDo = make_smem_desc(smem_u32(dop), 128, 2048, 0);
        const uint64_t dKb = make_smem_desc(smem_u32(rawk), REGION, 1024, 2);
        const uint64_t dQb = make_smem_desc(smem_u32(rawq), REGION, 1024, 2);
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
          mma_ss(tmem_base + COL_DVV, dP_MN + (uint64_t)(128 * ks), dDo + (uint64_t)(16 * ks), IDESC_MNMN, ks > 0);
          mma_ss(tmem_base + COL_DQ, dD_K + (uint64_t)(((ks >> 2) * REGION + (ks & 3) * 32) >> 4), dKb + (uint64_t)(128 * ks),
                 IDESC_KMN, ks > 0);
          mma_ss(tmem_base + COL_DK, dD_MN + (uint64_t)(128 * ks), dQb + (uint64_t)(128 * ks), IDESC_MNMN, ks > 0);
        }
        mma_commit(&bars[IPB_MMA2]);
      }
      __syncwarp();
      if (n + 1 < my_items && !issue_scores(n + 1)) break;
      if (!WAIT(IPB_STAGED, (uint32_t)n)) { FAIL(63); break; }
      __syncwarp();
      if (lane == 0) {
        float* stage = stage_base(s);
        // valid row ranges: dq rows are query rows (chunk position - off), dk / dv rows are key positions
        const long long q0 = (long long)pos0 - P.off;
        const int qa = q0 < 0 ? (int)(-q0 < CH ? -q0 : CH) : 0;
        const long long qlim = (long long)P.nq - q0;
        const int qb = qlim < CH ? (qlim < 0 ? 0 : (int)qlim) : CH;
        const long long klim = (long long)P.nk - pos0;
        const int kb = klim < CH ? (klim < 0 ? 0 : (int)klim) : CH;
        // plain stores: this kernel runs before the scans of the call and covers every accumulator row exactly once
        if (qb > qa)
          bulk_store(P.dq_acc + ((long long)head * P.nq + q0 + qa) * ACC_LD, stage + qa * ACC_LD, (uint32_t)(qb - qa) * (uint32_t)(ACC_LD * 4));
        if (kb > 0) {
          bulk_store(P.dk_acc + ((long long)head * P.nk + pos0) * ACC_LD, stage + CH * ACC_LD, (uint32_t)kb * (uint32_t)(ACC_LD * 4));
          bulk_store(P.dv_acc + ((long long)head * P.nk + pos0) * ACC_LD, stage + 2 * CH * ACC_LD, (uint32_t)kb * (uint32_t)(ACC_LD * 4));
        }
        bulk_commit_group();
        bulk_wait_read_all();   // the copy engine has read the staging rows: the set and the P / dS tiles are free
        mbar_arrive(&bars[IPB_STAGE_FREE]);
      }
      __syncwarp();
      if (n + 2 < my_items) prefetch(n + 2);
    }
    if (lane == 0) bulk_wait_all();   // every row is in global memory before the CTA retires
  } else {
    // ================= compute warps =================
    const int h = w >> 2, quarter = w & 3, l = quarter * 32 + lane;
    const uint32_t lane_addr = tmem_base + ((uint32_t)(quarter * 32) << 16);
    const int sw = l & 7;
    for (int n = 0; n < my_items; ++n) {
      const uint32_t s = (uint32_t)n & 1u;
      if (!WAIT(IPB_MMA1, (uint32_t)n)) { FAIL(64); break; }
      // the P / dS tiles overlap the previous item's staging rows: wait until the copy engine has read those
      if (n > 0 && !WAIT(IPB_STAGE_FREE, (uint32_t)(n - 1))) { FAIL(65); break; }
      __syncwarp();
      tc_fence_after_sync();
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        uint32_t rs[32], rd[32];
        tmem_ld32(lane_addr + COL_SC + 64u * h + 32u * half, rs);
        tmem_ld32(lane_addr + COL_DP + 64u * h + 32u * half, rd);
        tmem_ld_wait();
#pragma unroll
        for (int jb = 0; jb < 4; ++jb) {
          float pv[8], dv8[8];
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            const int j = 64 * h + 32 * half + 8 * jb + e;
            const float sc = __uint_as_float(rs[8 * jb + e]);
            const float dp = __uint_as_float(rd[8 * jb + e]);
            const bool vis = (j <= l);
            pv[e] = vis ? (P.c0 + sc * (P.c1 + P.c2 * sc)) : 0.f;
            dv8[e] = vis ? dp * (P.c1 + 2.f * P.c2 * sc) : 0.f;
          }
          const int off = h * REGION + l * 128 + (((4 * half + jb) ^ sw) << 4);
          *reinterpret_cast<uint4*>(pt + off) =
              make_uint4(pack_bf16(pv[0], pv[1]), pack_bf16(pv[2], pv[3]), pack_bf16(pv[4], pv[5]), pack_bf16(pv[6], pv[7]));
          *reinterpret_cast<uint4*>(dt + off) = make_uint4(pack_bf16(dv8[0], dv8[1]), pack_bf16(dv8[2], dv8[3]),
                                                           pack_bf16(dv8[4], dv8[5]), pack_bf16(dv8[6], dv8[7]));
        }
      }
      fence_proxy_async_smem();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars[IPB_PD]);
      if (!WAIT(IPB_MMA2, (uint32_t)n)) { FAIL(66); break; }
      __syncwarp();
      tc_fence_after_sync();
      // dq_c, dk_c, dv_c -> three staging tiles of ACC_LD-float rows (this item's operands are dead by now)
      float* stage = stage_base(s);
      const uint32_t cols[3] = {COL_DQ, COL_DK, COL_DVV};
#pragma unroll
      for (int x = 0; x < 3; ++x) {
        uint32_t r[32];
        tmem_ld32(lane_addr + cols[x] + 32u * h, r);
        tmem_ld_wait();
        float4* rowp = reinterpret_cast<float4*>(stage + (x * CH + l) * ACC_LD + 32 * h);
#pragma unroll
        for (int j = 0; j < 8; ++j)
          rowp[j] = make_float4(__uint_as_float(r[4 * j]), __uint_as_float(r[4 * j + 1]), __uint_as_float(r[4 * j + 2]),
                                __uint_as_float(r[4 * j + 3]));
        if (h == 0) reinterpret_cast<float4*>(stage + (x * CH + l) * ACC_LD + 64)[0] = make_float4(0.f, 0.f, 0.f, 0.f);
      }
      fence_proxy_async_smem();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars[IPB_STAGED]);
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (w == 0) tmem_dealloc(tmem_base, 512);
}

// dO' = [dO / g, -(dO . o) / g, 0 x 15] as bf16, 80 columns per row; one warp per row.
__global__ void bwd_prologue_bf16_kernel(View dout, View o, View g, __nv_bfloat16* __restrict__ dop, int nq, int heads,
                                         long long nrows) {
  const long long row = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (row >= nrows) return;
  const int l = (int)(row % nq);
  const int head = (int)(row / nq);
  const int b = head / heads, hh = head - b * heads;
  const __nv_bfloat16* dp = reinterpret_cast<const __nv_bfloat16*>(dout.ptr) + (long long)b * dout.sb + (long long)hh * dout.sh + (long long)l * dout.sn;
  const __nv_bfloat16* op = reinterpret_cast<const __nv_bfloat16*>(o.ptr) + (long long)b * o.sb + (long long)hh * o.sh + (long long)l * o.sn;
  const float gv = *(reinterpret_cast<const float*>(g.ptr) + (long long)b * g.sb + (long long)hh * g.sh + (long long)l * g.sn);
  const float inv = 1.f / gv;
  // lane owns columns 2*lane, 2*lane+1 (rows of dO and o are 4-byte aligned: validated on the host)
  const float2 x = __bfloat1622float2(reinterpret_cast<const __nv_bfloat162*>(dp)[lane]);
  const float2 y = __bfloat1622float2(reinterpret_cast<const __nv_bfloat162*>(op)[lane]);
  float dot = x.x * y.x + x.y * y.y;
#pragma unroll
  for (int s = 16; s > 0; s >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, s);
  __nv_bfloat162* out = reinterpret_cast<__nv_bfloat162*>(dop + row * 80);
  out[lane] = __floats2bfloat162_rn(x.x * inv, x.y * inv);
  if (lane < 8) out[32 + lane] = __floats2bfloat162_rn(lane == 0 ? -dot * inv : 0.f, 0.f);
}

// Same, for 16-byte aligned rows of dO and o: eight threads per row, 128-bit loads and stores.
__global__ void bwd_prologue_bf16_vec_kernel(View dout, View o, View g, __nv_bfloat16* __restrict__ dop, int nq, int heads,
                                             long long nrows) {
  const long long row = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 3;
  const int sub = threadIdx.x & 7;
  const bool live = row < nrows;
  float dot = 0.f;
  float f[8];
  float inv = 0.f;
  if (live) {
    const int l = (int)(row % nq);
    const int head = (int)(row / nq);
    const int b = head / heads, hh = head - b * heads;
    const __nv_bfloat16* dp = reinterpret_cast<const __nv_bfloat16*>(dout.ptr) + (long long)b * dout.sb + (long long)hh * dout.sh + (long long)l * dout.sn;
    const __nv_bfloat16* op = reinterpret_cast<const __nv_bfloat16*>(o.ptr) + (long long)b * o.sb + (long long)hh * o.sh + (long long)l * o.sn;
    inv = 1.f / *(reinterpret_cast<const float*>(g.ptr) + (long long)b * g.sb + (long long)hh * g.sh + (long long)l * g.sn);
    const uint4 x = reinterpret_cast<const uint4*>(dp)[sub];
    const uint4 y = reinterpret_cast<const uint4*>(op)[sub];
    const uint32_t xs[4] = {x.x, x.y, x.z, x.w}, ys[4] = {y.x, y.y, y.z, y.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float x0 = __uint_as_float(xs[i] << 16), x1 = __uint_as_float(xs[i] & 0xffff0000u);
      const float y0 = __uint_as_float(ys[i] << 16), y1 = __uint_as_float(ys[i] & 0xffff0000u);
      f[2 * i] = x0; f[2 * i + 1] = x1;
      dot += x0 * y0 + x1 * y1;
    }
  }
#pragma unroll
  for (int s = 4; s > 0; s >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, s);
  if (!live) return;
  uint4* out = reinterpret_cast<uint4*>(dop + row * 80);
  out[sub] = make_uint4(pack_bf16(f[0] * inv, f[1] * inv), pack_bf16(f[2] * inv, f[3] * inv), pack_bf16(f[4] * inv, f[5] * inv),
                        pack_bf16(f[6] * inv, f[7] * inv));
  if (sub == 0) out[8] = make_uint4(pack_bf16(-dot * inv, 0.f), 0u, 0u, 0u);
  if (sub == 1) out[9] = make_uint4(0u, 0u, 0u, 0u);
}
