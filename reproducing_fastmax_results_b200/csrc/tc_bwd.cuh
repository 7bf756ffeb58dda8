// tcgen05 backward helpers (bf16, head dim 64, order 2, causal).  Included by tc_kernels.cu inside fm::tc.
//   intra_bwd_kernel          the masked, within-chunk part of dq, dk, dv (one CTA per chunk and head)
//   bwd_prologue_bf16_kernel  dO' = [dO / g, -(dO . o) / g] rounded to bf16, the 80-column tile the scans read
// The inter-chunk parts are the scans of tc_scan2.cuh (dv) and tc_scan3.cuh (dq, dk).
#pragma once

constexpr int ACC_LD = 68;   // floats per row of the dq / dk / dv accumulators: 272-byte rows keep 128-bit per-thread row
                             // accesses to the shared-memory staging copies free of bank conflicts
// ------------------------------------------------------------------------------------------------------
// intra-chunk causal term of the backward pass, one CTA per (chunk, batch*head):
//   P = tril f(Q K^T),  dSm = tril((dO' [V|1]^T) * f'(Q K^T))
//   dq_c += dSm K_c,   dk_c += dSm^T Q_c,   dv_c += P^T dO'_c[:, :64]
// ------------------------------------------------------------------------------------------------------
constexpr int IB_THREADS = 256;
constexpr int IB_OFF_Q = 0, IB_OFF_K = REGION, IB_OFF_P = 2 * REGION, IB_OFF_D = 2 * REGION + TILE,
              IB_OFF_VP = 2 * REGION + 2 * TILE, IB_OFF_DO = IB_OFF_VP + 10 * BLK, IB_OFF_BAR = IB_OFF_DO + 10 * BLK;
constexpr int IB_SMEM_BYTES = IB_OFF_BAR + 64 + 1024;
static_assert(3 * CH * ACC_LD * 4 <= IB_OFF_BAR, "the three output staging tiles reuse the operand tiles");

struct IntraBwdParams {
  float *dq_acc, *dk_acc, *dv_acc;
  int heads, nq, nk, off;
  float c0, c1, c2;
};

__global__ void __launch_bounds__(IB_THREADS, 1)
intra_bwd_kernel(const __grid_constant__ CUtensorMap tmq, const __grid_constant__ CUtensorMap tmk,
                 const __grid_constant__ CUtensorMap tmv, const __grid_constant__ CUtensorMap tmdo, const IntraBwdParams P) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  uint8_t* sm = smem_raw + (((raw_addr + 1023u) & ~1023u) - raw_addr);
  uint8_t* rawq = sm + IB_OFF_Q;
  uint8_t* rawk = sm + IB_OFF_K;
  uint8_t* pt = sm + IB_OFF_P;
  uint8_t* dt = sm + IB_OFF_D;
  uint8_t* vp = sm + IB_OFF_VP;
  uint8_t* dop = sm + IB_OFF_DO;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sm + IB_OFF_BAR);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(sm + IB_OFF_BAR + 32);

  const int tid = threadIdx.x, w = tid >> 5, lane = tid & 31;
  const int h = w >> 2, quarter = w & 3, l = quarter * 32 + lane;
  const int c = blockIdx.x, head = blockIdx.z;
  const int b_idx = head / P.heads, h_idx = head - b_idx * P.heads;
  const int pos0 = c * CH;

  if (tid == 0) {
    mbar_init(&bars[0], 1);
    mbar_init(&bars[1], 1);
    fence_mbar_init();
  }
  if (w == 0) tmem_alloc(tmem_slot, 512);
  if (tid < CH) {
    *reinterpret_cast<uint4*>(vp + 8 * BLK + tid * 16) = make_uint4((pos0 + tid < P.nk) ? 0x00003F80u : 0u, 0u, 0u, 0u);
    *reinterpret_cast<uint4*>(vp + 9 * BLK + tid * 16) = make_uint4(0u, 0u, 0u, 0u);
  }
  fence_proxy_async_smem();
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t lane_addr = tmem_base + ((uint32_t)(quarter * 32) << 16);
  constexpr uint32_t COL_SC = 0u, COL_DP = 128u, COL_DQ = 256u, COL_DK = 320u, COL_DVV = 384u;
  if (tid == 0) {
    mbar_arrive_expect_tx(&bars[0], 2 * REGION + 18 * BLK);
    tma_load_4d(rawq, &tmq, &bars[0], 0, pos0 - P.off, h_idx, b_idx);
    tma_load_4d(rawk, &tmk, &bars[0], 0, pos0, h_idx, b_idx);
#pragma unroll
    for (int j = 0; j < 8; ++j) tma_load_4d(vp + j * BLK, &tmv, &bars[0], 8 * j, pos0, h_idx, b_idx);
#pragma unroll
    for (int j = 0; j < 10; ++j) tma_load_4d(dop + j * BLK, &tmdo, &bars[0], 8 * j, pos0 - P.off, h_idx, b_idx);
  }
  bool ok = mbar_wait_bounded(&bars[0], 0, WAIT_CYCLES);
  ok = (__syncthreads_or(ok ? 0 : 1) == 0);
  if (ok) {
    if (tid == 0) {
      tc_fence_after_sync();
      constexpr uint32_t IDESC_128 = make_idesc_bf16(128, 128, 0, 0);
      const uint64_t dq = make_smem_desc(smem_u32(rawq), 16, 1024, 2);
      const uint64_t dk = make_smem_desc(smem_u32(rawk), 16, 1024, 2);
#pragma unroll
      for (int ks = 0; ks < 4; ++ks) mma_ss(tmem_base + COL_SC, dq + (uint64_t)(2 * ks), dk + (uint64_t)(2 * ks), IDESC_128, ks > 0);
      const uint64_t dg = make_smem_desc(smem_u32(dop), 2048, 128, 0);
      const uint64_t dv = make_smem_desc(smem_u32(vp), 2048, 128, 0);
#pragma unroll
      for (int ks = 0; ks < 5; ++ks) mma_ss(tmem_base + COL_DP, dg + (uint64_t)(256 * ks), dv + (uint64_t)(256 * ks), IDESC_128, ks > 0);
      mma_commit(&bars[1]);
    }
    ok = mbar_wait_bounded(&bars[1], 0, WAIT_CYCLES);
    ok = (__syncthreads_or(ok ? 0 : 1) == 0);
  }
  if (ok) {
    tc_fence_after_sync();
    const int sw = l & 7;
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
          const float s = __uint_as_float(rs[8 * jb + e]);
          const float dp = __uint_as_float(rd[8 * jb + e]);
          const bool vis = (j <= l);
          pv[e] = vis ? (P.c0 + s * (P.c1 + P.c2 * s)) : 0.f;
          dv8[e] = vis ? dp * (P.c1 + 2.f * P.c2 * s) : 0.f;
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
    __syncthreads();
    if (tid == 0) {
      tc_fence_after_sync();
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
      mma_commit(&bars[1]);
    }
    ok = mbar_wait_bounded(&bars[1], 1, WAIT_CYCLES);
    ok = (__syncthreads_or(ok ? 0 : 1) == 0);
  }
  if (ok) {
    // dq_c, dk_c, dv_c of this chunk -> three staging tiles of ACC_LD-float rows (the operand tiles are dead by
    // now) -> three bulk reduce-adds into the accumulators
    tc_fence_after_sync();
    float* stage = reinterpret_cast<float*>(sm);
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
    __syncthreads();
    if (tid == 0) {
      // valid row ranges: dq rows are query rows (chunk position - off), dk / dv rows are key positions
      const long long q0 = (long long)pos0 - P.off;
      const int qa = q0 < 0 ? (int)(-q0 < CH ? -q0 : CH) : 0;
      const long long qlim = (long long)P.nq - q0;
      const int qb = qlim < CH ? (qlim < 0 ? 0 : (int)qlim) : CH;
      const long long klim = (long long)P.nk - pos0;
      const int kb = klim < CH ? (klim < 0 ? 0 : (int)klim) : CH;
      // Plain stores, not reduce-adds: this kernel runs BEFORE the scans of the call (stream order) and its chunks
      // cover every row of the three accumulators exactly once, so it also initialises them; the scans add on top.
      if (qb > qa)
        bulk_store(P.dq_acc + ((long long)head * P.nq + q0 + qa) * ACC_LD, stage + qa * ACC_LD, (uint32_t)(qb - qa) * (uint32_t)(ACC_LD * 4));
      if (kb > 0) {
        bulk_store(P.dk_acc + ((long long)head * P.nk + pos0) * ACC_LD, stage + CH * ACC_LD, (uint32_t)kb * (uint32_t)(ACC_LD * 4));
        bulk_store(P.dv_acc + ((long long)head * P.nk + pos0) * ACC_LD, stage + 2 * CH * ACC_LD, (uint32_t)kb * (uint32_t)(ACC_LD * 4));
      }
      bulk_commit_group();
      bulk_wait_all();   // the rows are in global memory before the CTA retires (the scans' adds come later)
    }
  } else if (tid == 0) {
    atomicExch(&g_tc_status, 60);
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
