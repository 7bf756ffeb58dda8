// tcgen05 backward scans (bf16, head dim 64, order 2, causal).  Included by tc_kernels.cu inside fm::tc.
//
// Two launches of one kernel template:
//   KV = false  forward-direction scan carrying S = Phi(K)^T [V|1]:       dq_c = chain(dO'_c Sb^T, Q_c)
//   KV = true   reverse-direction scan carrying dS = Phi(Q)^T dO':        dk_c = chain([V|1]_c dSb^T, K_c)
//                                                                          dv_c = Phi(K_c) dSb[:, :64]
// Per 128-token chunk and 128-row feature tile t of the slice (Sb = weighted bf16 copy of the state):
//   dphi   D (128 x 64, per 64-feature unit) = G_c (128 x 80, K-major) * Sb_t[unit]^T      G = dO' | [V|1]
//   apply  dV (128 x 64) += Phi_t(K_c) (K-major) * Sb_t[:, :64]                             (KV only)
//   update S_t (128 x 80) += Phi_t(X_c)^T (MN-major) * Y_c (128 x 80)        (X, Y) = (K, [V|1]) | (Q, dO')
// The chain rule through Phi (dz[m] += dphi[m,r] z[r], dz[r] += dphi[m,r] z[m]) runs on CUDA cores straight
// out of TMEM; the weights of the polynomial are already inside Sb.
// Warp roles: 0-3 producers (Phi tiles), 4-7 chain rule + dq/dk drain, 8-11 state conversion + dV drain,
// 12 MMA issuer, 13 TMA loader (448 threads, so the chain-rule warps can keep dz[64] in registers).
// All waits are bounded (abort flag + error code, as in the forward scan).
#pragma once

constexpr int ACC_LD = 68;   // floats per row of the dq / dk / dv accumulators: 272-byte rows keep 128-bit per-thread row
                             // accesses to the shared-memory staging copies free of bank conflicts
constexpr int BW_THREADS = 448;
constexpr int BW_NPRODUCER = 128;
constexpr int BW_WARP_MMA = 12, BW_WARP_TMA = 13;
constexpr int BW_NSLOT = 2;
constexpr int BW_OFF_RING = 0;
constexpr int BW_OFF_SB = BW_OFF_RING + BW_NSLOT * TILE;      // 65536
constexpr int BW_OFF_VP = BW_OFF_SB + 4 * SB_TILE;            // 139264  [V|1]: 10 blocks, block 9 zero
constexpr int BW_OFF_DO = BW_OFF_VP + 10 * BLK;               // 159744  dO': 10 blocks
constexpr int BW_OFF_RAWQ = BW_OFF_DO + 10 * BLK;             // 180224
constexpr int BW_OFF_RAWK = BW_OFF_RAWQ + REGION;             // 196608
constexpr int BW_OFF_BAR = BW_OFF_RAWK + REGION;              // 212992
constexpr int BW_SMEM_BYTES = BW_OFF_BAR + 256 + 1024;
static_assert(BW_OFF_RAWQ % 1024 == 0 && BW_OFF_RAWK % 1024 == 0, "swizzled tiles need 1024-byte alignment");
// barrier indices
constexpr int C_FULL = 0, C_EMPTY = 2, C_SB_READY = 4, C_S_DONE = 8, C_RAW_READY = 12, C_RAW_FREE = 13,
              C_GY_READY = 14, C_GY_FREE = 15, C_DPHI_DONE = 16, C_DPHI_FREE = 18, C_DV_DONE = 20, C_DV_FREE = 21;

struct BwdParams {
  float* dz_acc;   // KV ? dk [BH][nk][64] : dq [BH][nq][64]
  float* dv_acc;   // KV only: [BH][nk][64]
  int heads, nq, nk, off, nchunks;
  float c0, c1, c2;
};

__device__ __forceinline__ void load_row_block(const uint8_t* raw, int l, int blk, float (&out)[8]) {
  const uint4 x = *reinterpret_cast<const uint4*>(raw + l * 128 + ((blk ^ (l & 7)) << 4));
  const uint32_t wv[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    out[2 * i] = __uint_as_float(wv[i] << 16);
    out[2 * i + 1] = __uint_as_float(wv[i] & 0xffff0000u);
  }
}

template <bool KV>
__global__ void __launch_bounds__(BW_THREADS, 1)
scan_bwd_kernel(const __grid_constant__ CUtensorMap tmq, const __grid_constant__ CUtensorMap tmk,
                const __grid_constant__ CUtensorMap tmv, const __grid_constant__ CUtensorMap tmdo, const BwdParams P) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  uint8_t* sm = smem_raw + (((raw_addr + 1023u) & ~1023u) - raw_addr);
  uint8_t* ring = sm + BW_OFF_RING;
  uint8_t* sb = sm + BW_OFF_SB;
  uint8_t* vp = sm + BW_OFF_VP;
  uint8_t* dop = sm + BW_OFF_DO;
  uint8_t* rawq = sm + BW_OFF_RAWQ;
  uint8_t* rawk = sm + BW_OFF_RAWK;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sm + BW_OFF_BAR);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(sm + BW_OFF_BAR + 192);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(sm + BW_OFF_BAR + 200);
  // roles of the four input tiles
  const uint8_t* ztile = KV ? rawk : rawq;   // rows the chain rule (and the dV apply) differentiates
  const uint8_t* xtile = KV ? rawq : rawk;   // rows whose Phi feeds the state update
  const uint8_t* gtile = KV ? vp : dop;      // A operand of dphi
  const uint8_t* ytile = KV ? dop : vp;      // B operand of the state update

  const int tid = threadIdx.x, w = tid >> 5, lane = tid & 31;
  const int slice = blockIdx.x, head = blockIdx.z;
  const int b_idx = head / P.heads, h_idx = head - b_idx * P.heads;
  const int tile0 = slice * 4;
  const int ntl = (NTILES - tile0) < 4 ? (NTILES - tile0) : 4;
  const int nch = P.nchunks;
  const bool do_dv = KV && P.dv_acc != nullptr;  // the dV apply can run in its own kernel instead

  if (tid == 0) {
    for (int i = 0; i < BW_NSLOT; ++i) { mbar_init(&bars[C_FULL + i], BW_NPRODUCER); mbar_init(&bars[C_EMPTY + i], 1); }
    for (int i = 0; i < 4; ++i) { mbar_init(&bars[C_SB_READY + i], 128); mbar_init(&bars[C_S_DONE + i], 1); }
    mbar_init(&bars[C_RAW_READY], 1);
    mbar_init(&bars[C_RAW_FREE], BW_NPRODUCER + 128);
    mbar_init(&bars[C_GY_READY], 1);
    mbar_init(&bars[C_GY_FREE], 1);
    for (int i = 0; i < 2; ++i) { mbar_init(&bars[C_DPHI_DONE + i], 1); mbar_init(&bars[C_DPHI_FREE + i], 128); }
    mbar_init(&bars[C_DV_DONE], 1);
    mbar_init(&bars[C_DV_FREE], 128);
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (w == 0) tmem_alloc(tmem_slot, 512);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  constexpr uint32_t COL_DPHI = 320u, COL_DV = 448u;

  auto WAIT = [&](int bar, uint32_t parity) -> bool {
    return mbar_wait_abortable(&bars[bar], parity & 1u, WAIT_CYCLES, abort_flag);
  };
  auto FAIL = [&](int code) {
    *abort_flag = 1;
    atomicExch(&g_tc_status, code);
  };
  // units of tile t that carry features: two, except the lin tile (x and the constant; the constant has no gradient)
  auto units_of = [&](int gt) -> int { return gt < NTILES - 1 ? 2 : 1; };

  // the bf16 state copy is read one column block past its 72 stored columns (times zeros): keep it finite
  for (int i = tid; i < (4 * SB_TILE) / 16; i += BW_THREADS) reinterpret_cast<uint4*>(sb)[i] = make_uint4(0u, 0u, 0u, 0u);
  for (int i = tid; i < BLK / 16; i += BW_THREADS) reinterpret_cast<uint4*>(vp + 9 * BLK)[i] = make_uint4(0u, 0u, 0u, 0u);
  fence_proxy_async_smem();
  __syncthreads();

  if (w < 4) {
    // ================= producers (each thread writes both 64-feature halves of its token row) =================
    const int l = w * 32 + lane;
    uint32_t n = 0;
    bool ok = true;
    for (int i = 0; i < nch && ok; ++i) {
      if (!WAIT(C_RAW_READY, i)) { FAIL(110); break; }
      for (int t = 0; t < ntl && ok; ++t) {
        const int gt = tile0 + t;
#pragma unroll 1
        for (int which = ((do_dv && i > 0) ? 0 : 1); which < 2; ++which) {  // 0: Phi(Z) for the dV apply, 1: Phi(X) for the update
          const uint32_t slot = n % BW_NSLOT, k = n / BW_NSLOT;
          if (k > 0 && !WAIT(C_EMPTY + slot, k - 1)) { FAIL(111); ok = false; break; }
          gen_tile(ring + slot * TILE, which == 0 ? ztile : xtile, gt, l, 0);
          gen_tile(ring + slot * TILE, which == 0 ? ztile : xtile, gt, l, 1);
          fence_proxy_async_smem();
          mbar_arrive(&bars[C_FULL + slot]);
          ++n;
        }
      }
      if (ok) mbar_arrive(&bars[C_RAW_FREE]);
    }
  } else if (w < 8) {
    // ================= chain rule: dphi (TMEM) -> dz rows =================
    const int l = (w & 3) * 32 + lane;
    const uint32_t lane_addr = tmem_base + ((uint32_t)((w & 3) * 32) << 16);
    float dz[64];
#pragma unroll
    for (int j = 0; j < 64; ++j) dz[j] = 0.f;
    uint32_t m = 0;
    bool ok = true;
    for (int i = 0; i < nch && ok; ++i) {
      const int c = KV ? (nch - 1 - i) : i;
      if (!WAIT(C_RAW_READY, i)) { FAIL(120); break; }
      if (i > 0) {
        for (int t = 0; t < ntl && ok; ++t) {
          const int gt = tile0 + t;
          const int nu = units_of(gt);
          for (int u = 0; u < nu; ++u) {
            const uint32_t buf = m & 1u;
            if (!WAIT(C_DPHI_DONE + buf, m >> 1)) { FAIL(121); ok = false; break; }
            tc_fence_after_sync();
            uint32_t r0[32], r1[32];
            tmem_ld32(lane_addr + COL_DPHI + 64u * buf, r0);
            tmem_ld32(lane_addr + COL_DPHI + 64u * buf + 32u, r1);
            tmem_ld_wait();
            tc_fence_before_sync();
            mbar_arrive(&bars[C_DPHI_FREE + buf]);
            ++m;
            if (gt < NTILES - 1) {
              int a, b;
              pair_decode(2 * gt + u, 8, a, b);
              float za[8], zb[8], dza[8], dzb[8];
              load_row_block(ztile, l, a, za);
              load_row_block(ztile, l, b, zb);
#pragma unroll
              for (int j = 0; j < 8; ++j) { dza[j] = 0.f; dzb[j] = 0.f; }
#pragma unroll
              for (int mi = 0; mi < 8; ++mi) {
#pragma unroll
                for (int ri = 0; ri < 8; ++ri) {
                  const float dphi = __uint_as_float(mi < 4 ? r0[mi * 8 + ri] : r1[(mi - 4) * 8 + ri]);
                  dza[mi] += dphi * zb[ri];
                  dzb[ri] += dphi * za[mi];
                }
              }
              // a, b are warp-uniform: selecting the block with an unrolled compare keeps dz in registers
#pragma unroll
              for (int blk = 0; blk < 8; ++blk) {
                if (a == blk) {
#pragma unroll
                  for (int j = 0; j < 8; ++j) dz[8 * blk + j] += dza[j];
                }
                if (b == blk) {
#pragma unroll
                  for (int j = 0; j < 8; ++j) dz[8 * blk + j] += dzb[j];
                }
              }
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j) {
                dz[j] += __uint_as_float(r0[j]);
                dz[32 + j] += __uint_as_float(r1[j]);
              }
            }
          }
        }
      }
      if (!ok) break;
      mbar_arrive(&bars[C_RAW_FREE]);
      if (i > 0) {
        const long long row = KV ? ((long long)c * CH + l) : ((long long)c * CH + l - P.off);
        const long long nrows = KV ? P.nk : P.nq;
        if (row >= 0 && row < nrows) {
          float* dst = P.dz_acc + ((long long)head * nrows + row) * ACC_LD;
#pragma unroll
          for (int j = 0; j < 16; ++j)
            atomicAdd(reinterpret_cast<float4*>(dst + 4 * j), make_float4(dz[4 * j], dz[4 * j + 1], dz[4 * j + 2], dz[4 * j + 3]));
        }
#pragma unroll
        for (int j = 0; j < 64; ++j) dz[j] = 0.f;
      }
    }
  } else if (w < 12) {
    // ================= state conversion (+ dV drain) =================
    const int l = (w & 3) * 32 + lane;
    const uint32_t lane_addr = tmem_base + ((uint32_t)((w & 3) * 32) << 16);
    bool ok = true;
    for (int i = 0; i < nch && ok; ++i) {
      const int c = KV ? (nch - 1 - i) : i;
      for (int t = 0; t < ntl && ok; ++t) {
        if (do_dv && i > 0 && t == ntl - 1) {
          if (!WAIT(C_DV_DONE, (uint32_t)(i - 1))) { FAIL(130); ok = false; break; }
          tc_fence_after_sync();
          uint32_t r0[32], r1[32];
          tmem_ld32(lane_addr + COL_DV, r0);
          tmem_ld32(lane_addr + COL_DV + 32u, r1);
          tmem_ld_wait();
          tc_fence_before_sync();
          mbar_arrive(&bars[C_DV_FREE]);
          const long long row = (long long)c * CH + l;
          if (row < P.nk) {
            float* dst = P.dv_acc + ((long long)head * P.nk + row) * ACC_LD;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              atomicAdd(reinterpret_cast<float4*>(dst + 4 * j),
                        make_float4(__uint_as_float(r0[4 * j]), __uint_as_float(r0[4 * j + 1]), __uint_as_float(r0[4 * j + 2]),
                                    __uint_as_float(r0[4 * j + 3])));
              atomicAdd(reinterpret_cast<float4*>(dst + 32 + 4 * j),
                        make_float4(__uint_as_float(r1[4 * j]), __uint_as_float(r1[4 * j + 1]), __uint_as_float(r1[4 * j + 2]),
                                    __uint_as_float(r1[4 * j + 3])));
            }
          }
        }
        if (i < nch - 1) {
          if (!WAIT(C_S_DONE + t, (uint32_t)i)) { FAIL(131); ok = false; break; }
          tc_fence_after_sync();
          const float wgt = tile_weight(tile0 + t, l, P.c0, P.c1, P.c2);
          uint8_t* dst = sb + t * SB_TILE + l * 16;
#pragma unroll
          for (int part = 0; part < 2; ++part) {
            uint32_t r[32];
            tmem_ld32(lane_addr + 80u * t + 32u * part, r);
            tmem_ld_wait();
#pragma unroll
            for (int jb = 0; jb < 4; ++jb) store_block8(dst + (4 * part + jb) * BLK, &r[8 * jb], wgt);
          }
          uint32_t r8[8];
          tmem_ld8(lane_addr + 80u * t + 64u, r8);
          tmem_ld_wait();
          store_block8(dst + 8 * BLK, r8, wgt);
          fence_proxy_async_smem();
          tc_fence_before_sync();
          mbar_arrive(&bars[C_SB_READY + t]);
        }
      }
    }
  }
  else if (w == BW_WARP_MMA) {
    // ================= MMA issuer =================
    constexpr uint32_t IDESC_DPHI = make_idesc_bf16(128, 64, 0, 0);   // A K-major,  B K-major
    constexpr uint32_t IDESC_DV = make_idesc_bf16(128, 64, 0, 1);     // A K-major,  B MN-major
    constexpr uint32_t IDESC_UPD = make_idesc_bf16(128, 80, 1, 1);    // A MN-major, B MN-major
    const uint64_t dA_K = make_smem_desc(smem_u32(ring), 16, 1024, 2);
    const uint64_t dA_MN = make_smem_desc(smem_u32(ring), REGION, 1024, 2);
    const uint64_t dA_G = make_smem_desc(smem_u32(gtile), 2048, 128, 0);     // rows x 80, K-major column blocks
    const uint64_t dB_Y = make_smem_desc(smem_u32(ytile), 128, 2048, 0);     // 80 columns, MN-major
    const uint64_t dB_S_K = make_smem_desc(smem_u32(sb), 2048, 128, 0);      // Sb as (features x 80), K-major
    const uint64_t dB_S_MN = make_smem_desc(smem_u32(sb), 128, 2048, 0);     // Sb as (128 features) x columns, MN-major
    uint32_t n = 0, m = 0;
    bool ok = true;
    for (int i = 0; i < nch && ok; ++i) {
      for (int t = 0; t < ntl && ok; ++t) {
        const int gt = tile0 + t;
        if (i > 0) {
          if (!WAIT(C_SB_READY + t, (uint32_t)(i - 1))) { FAIL(140); ok = false; break; }
          if (t == 0 && !WAIT(C_GY_READY, (uint32_t)i)) { FAIL(141); ok = false; break; }
          const int nu = units_of(gt);
          for (int u = 0; u < nu; ++u) {  // dphi of one 64-feature unit
            const uint32_t buf = m & 1u;
            if (m >= 2 && !WAIT(C_DPHI_FREE + buf, (m >> 1) - 1u)) { FAIL(142); ok = false; break; }
            tc_fence_after_sync();
            if (lane == 0) {
              const uint32_t d = tmem_base + COL_DPHI + 64u * buf;
              const uint64_t b0 = dB_S_K + (uint64_t)((t * SB_TILE + u * 1024) >> 4);
#pragma unroll
              for (int ks = 0; ks < 5; ++ks) mma_ss(d, dA_G + (uint64_t)(256 * ks), b0 + (uint64_t)(256 * ks), IDESC_DPHI, ks > 0);
              mma_commit(&bars[C_DPHI_DONE + buf]);
            }
            __syncwarp();
            ++m;
          }
          if (!ok) break;
          if (do_dv) {  // dV += Phi(K_c) Sb[:, :64]
            const uint32_t slot = n % BW_NSLOT, k = n / BW_NSLOT;
            if (!WAIT(C_FULL + slot, k)) { FAIL(143); ok = false; break; }
            if (t == 0 && i >= 2 && !WAIT(C_DV_FREE, (uint32_t)(i - 2))) { FAIL(144); ok = false; break; }
            tc_fence_after_sync();
            if (lane == 0) {
              const uint64_t a0 = dA_K + (uint64_t)((slot * TILE) >> 4);
              const uint64_t b0 = dB_S_MN + (uint64_t)((t * SB_TILE) >> 4);
#pragma unroll
              for (int ks = 0; ks < 8; ++ks)
                mma_ss(tmem_base + COL_DV, a0 + (uint64_t)(((ks >> 2) * REGION + (ks & 3) * 32) >> 4), b0 + (uint64_t)(16 * ks),
                       IDESC_DV, (t > 0 || ks > 0) ? 1u : 0u);
              mma_commit(&bars[C_EMPTY + slot]);
              if (t == ntl - 1) mma_commit(&bars[C_DV_DONE]);
            }
            __syncwarp();
            ++n;
          }
        }
        {  // state update
          const uint32_t slot = n % BW_NSLOT, k = n / BW_NSLOT;
          if (!WAIT(C_FULL + slot, k)) { FAIL(145); ok = false; break; }
          if (t == 0 && i == 0 && !WAIT(C_GY_READY, 0u)) { FAIL(146); ok = false; break; }
          tc_fence_after_sync();
          if (lane == 0) {
            const uint64_t a0 = dA_MN + (uint64_t)((slot * TILE) >> 4);
#pragma unroll
            for (int ks = 0; ks < 8; ++ks)
              mma_ss(tmem_base + 80u * t, a0 + (uint64_t)(128 * ks), dB_Y + (uint64_t)(16 * ks), IDESC_UPD, (i > 0 || ks > 0) ? 1u : 0u);
            mma_commit(&bars[C_EMPTY + slot]);
            mma_commit(&bars[C_S_DONE + t]);
            if (t == ntl - 1) mma_commit(&bars[C_GY_FREE]);
          }
          __syncwarp();
          ++n;
        }
      }
    }
    if (ok && nch > 0 && !WAIT(C_GY_FREE, (uint32_t)(nch - 1))) FAIL(147);  // every MMA has completed
    tc_fence_after_sync();
  } else if (w == BW_WARP_TMA) {
    // ================= TMA loader =================
    bool ok = true;
    for (int i = 0; i < nch && ok; ++i) {
      const int c = KV ? (nch - 1 - i) : i;
      const int pos0 = c * CH;
      if (i > 0 && !WAIT(C_RAW_FREE, (uint32_t)(i - 1))) { FAIL(150); break; }
      if (lane == 0) {
        mbar_arrive_expect_tx(&bars[C_RAW_READY], 2 * REGION);
        tma_load_4d(rawq, &tmq, &bars[C_RAW_READY], 0, pos0 - P.off, h_idx, b_idx);
        tma_load_4d(rawk, &tmk, &bars[C_RAW_READY], 0, pos0, h_idx, b_idx);
      }
      if (i > 0 && !WAIT(C_GY_FREE, (uint32_t)(i - 1))) { FAIL(151); break; }
      for (int r = lane; r < CH; r += 32)
        *reinterpret_cast<uint4*>(vp + 8 * BLK + r * 16) = make_uint4((pos0 + r < P.nk) ? 0x00003F80u : 0u, 0u, 0u, 0u);
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive_expect_tx(&bars[C_GY_READY], 18 * BLK);
#pragma unroll
        for (int j = 0; j < 8; ++j) tma_load_4d(vp + j * BLK, &tmv, &bars[C_GY_READY], 8 * j, pos0, h_idx, b_idx);
#pragma unroll
        for (int j = 0; j < 10; ++j) tma_load_4d(dop + j * BLK, &tmdo, &bars[C_GY_READY], 8 * j, pos0 - P.off, h_idx, b_idx);
      }
      __syncwarp();
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (w == 0) tmem_dealloc(tmem_base, 512);
}

// ------------------------------------------------------------------------------------------------------
// intra-chunk causal term of the backward pass, one CTA per (chunk, batch*head):
//   P = tril f(Q K^T),  dSm = tril((dO' [V|1]^T) * f'(Q K^T))
//   dq_c += dSm K_c,   dk_c += dSm^T Q_c,   dv_c += P^T dO'_c[:, :64]
// ------------------------------------------------------------------------------------------------------
constexpr int IB_THREADS = 256;
constexpr int IB_OFF_Q = 0, IB_OFF_K = REGION, IB_OFF_P = 2 * REGION, IB_OFF_D = 2 * REGION + TILE,
              IB_OFF_VP = 2 * REGION + 2 * TILE, IB_OFF_DO = IB_OFF_VP + 10 * BLK, IB_OFF_BAR = IB_OFF_DO + 10 * BLK;
constexpr int IB_SMEM_BYTES = IB_OFF_BAR + 64 + 1024;

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
    tc_fence_after_sync();
    const long long ql = (long long)pos0 + l - P.off;
    const long long kpos = (long long)pos0 + l;
    float* dsts[3] = {P.dq_acc + ((long long)head * P.nq + ql) * ACC_LD + 32 * h, P.dk_acc + ((long long)head * P.nk + kpos) * ACC_LD + 32 * h,
                      P.dv_acc + ((long long)head * P.nk + kpos) * ACC_LD + 32 * h};
    const bool valid[3] = {ql >= 0 && ql < P.nq, kpos < P.nk, kpos < P.nk};
    const uint32_t cols[3] = {COL_DQ, COL_DK, COL_DVV};
#pragma unroll
    for (int x = 0; x < 3; ++x) {
      uint32_t r[32];
      tmem_ld32(lane_addr + cols[x] + 32u * h, r);
      tmem_ld_wait();
      if (valid[x]) {
#pragma unroll
        for (int j = 0; j < 8; ++j)
          atomicAdd(reinterpret_cast<float4*>(dsts[x] + 4 * j),
                    make_float4(__uint_as_float(r[4 * j]), __uint_as_float(r[4 * j + 1]), __uint_as_float(r[4 * j + 2]),
                                __uint_as_float(r[4 * j + 3])));
      }
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
