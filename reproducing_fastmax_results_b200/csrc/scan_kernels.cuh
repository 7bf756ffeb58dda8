// CUDA-core (fp32 FFMA) Fastmax engine: moment build, chunked causal scan, state apply, and the two
// backward scans.  It covers every dtype / head dim / order / mask combination and is the exact-fp32
// path; the tcgen05 kernels take over the bf16 configurations they support.
//
// Work split: grid = (slice, segment, batch*head).
//   slice   : a group of <= UPS pair units of the feature axis (the state slice lives in shared memory);
//             the last slice owns the lin unit (x and the constant) and the intra-chunk causal term.
//   segment : a contiguous run of 64-token chunks; its initial state comes from the prefix kernel.
// Partial results of the slices are summed with float4 atomics into fp32 accumulators in the workspace.
//
// One chunk (C = 64 positions), roles by mode:
//   FWD     O'_c   = (Phi(Q_c) w) S          + tril(f(Q_c K_c^T)) V'_c       then S += Phi(K_c)^T V'_c
//   BWD_Q   dq_c   = chain(dO'_c S^T, Q_c)   + (tril(dO'_c V'_c^T) f') K_c   then S += Phi(K_c)^T V'_c
//   BWD_KV  dk_c   = chain(V'_c dS^T, K_c)   + (...)^T Q_c ;  dv_c = (Phi(K_c) w) dS + tril(f)^T dO'_c
//           (chunks in descending order)                                     then dS += Phi(Q_c)^T dO'_c
#pragma once
#include "common.cuh"

namespace fm {

template <int D>
struct Cfg {
  static constexpr int C = 64;            // positions per chunk
  static constexpr int NT = 256;          // threads per CTA
  static constexpr int NSUB = NT / C;     // threads per token in the apply phases
  static constexpr int MPS = 8 / NSUB;    // mi rows per sub-thread
  static constexpr int UPS = 4;           // max pair units per slice
  static constexpr int TR = (D >= 64) ? 8 : 4;  // feature rows per update tile
  static constexpr int SROWS = UPS * 64 + 8;
  static constexpr int LDA = C + 1;
};

// ------------------------------------------------------------------------------------------------
// state slice <-> global
// ------------------------------------------------------------------------------------------------
template <int D, int NT>
__device__ __forceinline__ void slice_rows(bool lin_slice, int u0, int nu, int order, int& grow0, int& nrows) {
  using G = Geo<D>;
  if (lin_slice) {
    grow0 = (order == 2) ? G::LIN_ROW0 : 0;
    nrows = D + 1;
  } else {
    grow0 = 64 * u0;
    nrows = 64 * nu;
  }
}

template <int D, int NT, int SROWS>
__device__ __forceinline__ void load_state_slice(float* Ss, const float* gstate, bool lin_slice, int u0, int nu,
                                                 int order, int tid) {
  using G = Geo<D>;
  int grow0, nrows;
  slice_rows<D, NT>(lin_slice, u0, nu, order, grow0, nrows);
  constexpr int VPR = G::LDS / 4;
  for (int idx = tid; idx < SROWS * VPR; idx += NT) {
    int r = idx / VPR;
    float4 val = make_float4(0.f, 0.f, 0.f, 0.f);
    if (gstate != nullptr && r < nrows)
      val = *reinterpret_cast<const float4*>(gstate + (long long)grow0 * G::LDS + idx * 4);
    *reinterpret_cast<float4*>(Ss + idx * 4) = val;
  }
}

template <int D, int NT>
__device__ __forceinline__ void store_state_slice(const float* Ss, float* gstate, bool lin_slice, int u0, int nu,
                                                  int order, int tid) {
  using G = Geo<D>;
  int grow0, nrows;
  slice_rows<D, NT>(lin_slice, u0, nu, order, grow0, nrows);
  constexpr int VPR = G::LDS / 4;
  for (int idx = tid; idx < nrows * VPR; idx += NT)
    *reinterpret_cast<float4*>(gstate + (long long)grow0 * G::LDS + idx * 4) =
        *reinterpret_cast<const float4*>(Ss + idx * 4);
}

// ------------------------------------------------------------------------------------------------
// update:  Ss[f][j] += sum_l Phi(x_l)_f * y_l[j]        thread tile = TR feature rows x 8 columns
// ------------------------------------------------------------------------------------------------
template <int D, int C, int NT, int TR>
__device__ __forceinline__ void update_phase(float* Ss, const float* __restrict__ Xs, const float* __restrict__ Ys,
                                             bool lin_slice, int u0, int nu, int tid) {
  using G = Geo<D>;
  constexpr int RH = 8 / TR;
  constexpr int NCGH = D / 8;
  const int nmi = lin_slice ? G::NLG : 8;
  const int units = lin_slice ? 1 : nu;
  const int heavy_per_unit = nmi * RH * NCGH;
  const int nheavy = units * heavy_per_unit;
  for (int t = tid; t < nheavy; t += NT) {
    int ul = t / heavy_per_unit;
    int rem = t - ul * heavy_per_unit;
    int cg = rem % NCGH;
    rem /= NCGH;
    int rh = rem % RH;
    int mi = rem / RH;
    int xa_col, xb_col, row0;
    if (lin_slice) {
      xa_col = D;  // the constant-1 column of the tile
      xb_col = 8 * mi + TR * rh;
      row0 = xb_col;
    } else {
      int a, b;
      pair_decode(u0 + ul, G::NB, a, b);
      xa_col = 8 * a + mi;
      xb_col = 8 * b + TR * rh;
      row0 = ul * 64 + mi * 8 + TR * rh;
    }
    const int col0 = 4 * cg, col1 = D / 2 + 4 * cg;
    float acc[TR][8];
#pragma unroll
    for (int i = 0; i < TR; ++i)
#pragma unroll
      for (int c = 0; c < 8; ++c) acc[i][c] = 0.f;
#pragma unroll 2
    for (int l = 0; l < C; ++l) {
      const float* xr = Xs + l * G::LDX;
      const float* yr = Ys + l * G::LDY;
      float xa = xr[xa_col];
      float xb[TR];
#pragma unroll
      for (int i4 = 0; i4 < TR / 4; ++i4) {
        float4 t4 = *reinterpret_cast<const float4*>(xr + xb_col + 4 * i4);
        xb[4 * i4 + 0] = t4.x; xb[4 * i4 + 1] = t4.y; xb[4 * i4 + 2] = t4.z; xb[4 * i4 + 3] = t4.w;
      }
      float4 y0 = *reinterpret_cast<const float4*>(yr + col0);
      float4 y1 = *reinterpret_cast<const float4*>(yr + col1);
#pragma unroll
      for (int i = 0; i < TR; ++i) {
        float p = xa * xb[i];
        acc[i][0] += p * y0.x; acc[i][1] += p * y0.y; acc[i][2] += p * y0.z; acc[i][3] += p * y0.w;
        acc[i][4] += p * y1.x; acc[i][5] += p * y1.y; acc[i][6] += p * y1.z; acc[i][7] += p * y1.w;
      }
    }
#pragma unroll
    for (int i = 0; i < TR; ++i) {
      float4* s0 = reinterpret_cast<float4*>(Ss + (row0 + i) * G::LDS + col0);
      float4* s1 = reinterpret_cast<float4*>(Ss + (row0 + i) * G::LDS + col1);
      float4 a0 = *s0, a1 = *s1;
      a0.x += acc[i][0]; a0.y += acc[i][1]; a0.z += acc[i][2]; a0.w += acc[i][3];
      a1.x += acc[i][4]; a1.y += acc[i][5]; a1.z += acc[i][6]; a1.w += acc[i][7];
      *s0 = a0;
      *s1 = a1;
    }
  }
  // column D (the ones column of [V|1] or the denominator part of dO')
  const int nlight = units * nmi * RH;
  for (int t = tid; t < nlight; t += NT) {
    int ul = t / (nmi * RH);
    int rem = t - ul * (nmi * RH);
    int rh = rem % RH;
    int mi = rem / RH;
    int xa_col, xb_col, row0;
    if (lin_slice) {
      xa_col = D;
      xb_col = 8 * mi + TR * rh;
      row0 = xb_col;
    } else {
      int a, b;
      pair_decode(u0 + ul, G::NB, a, b);
      xa_col = 8 * a + mi;
      xb_col = 8 * b + TR * rh;
      row0 = ul * 64 + mi * 8 + TR * rh;
    }
    float acc[TR];
#pragma unroll
    for (int i = 0; i < TR; ++i) acc[i] = 0.f;
    for (int l = 0; l < C; ++l) {
      const float* xr = Xs + l * G::LDX;
      float p = xr[xa_col] * Ys[l * G::LDY + D];
#pragma unroll
      for (int i = 0; i < TR; ++i) acc[i] += p * xr[xb_col + i];
    }
#pragma unroll
    for (int i = 0; i < TR; ++i) Ss[(row0 + i) * G::LDS + D] += acc[i];
  }
}

// ------------------------------------------------------------------------------------------------
// apply (forward form):  acc[j] += sum_f w_f Phi(z_l)_f Ss[f][j]      thread = (token l, sub)
// ------------------------------------------------------------------------------------------------
template <int D, int C, int NT>
__device__ __forceinline__ void apply_fwd_accum(float (&acc)[Geo<D>::LDS], const float* __restrict__ Ss,
                                                const float* __restrict__ Zs, bool lin_slice, int u0, int nu,
                                                float c0, float c1, float c2, int l, int sub) {
  using G = Geo<D>;
  constexpr int NSUB = NT / C;
  constexpr int MPS = 8 / NSUB;
  const float* zrow = Zs + l * G::LDX;
  if (!lin_slice) {
    for (int ul = 0; ul < nu; ++ul) {
      int a, b;
      pair_decode(u0 + ul, G::NB, a, b);
      const float w = (a == b) ? c2 : 2.f * c2;
      float zb[8];
      {
        float4 t0 = *reinterpret_cast<const float4*>(zrow + 8 * b);
        float4 t1 = *reinterpret_cast<const float4*>(zrow + 8 * b + 4);
        zb[0] = t0.x; zb[1] = t0.y; zb[2] = t0.z; zb[3] = t0.w;
        zb[4] = t1.x; zb[5] = t1.y; zb[6] = t1.z; zb[7] = t1.w;
      }
#pragma unroll
      for (int i = 0; i < MPS; ++i) {
        const float za = zrow[8 * a + sub * MPS + i] * w;
#pragma unroll
        for (int ri = 0; ri < 8; ++ri) {
          const float t = za * zb[ri];
          const float4* row = reinterpret_cast<const float4*>(Ss + (ul * 64 + (sub * MPS + i) * 8 + ri) * G::LDS);
#pragma unroll
          for (int j4 = 0; j4 < G::LDS / 4; ++j4) {
            float4 s = row[j4];
            acc[4 * j4 + 0] += t * s.x; acc[4 * j4 + 1] += t * s.y;
            acc[4 * j4 + 2] += t * s.z; acc[4 * j4 + 3] += t * s.w;
          }
        }
      }
    }
  } else {
    for (int g = sub; g < G::NLG; g += NSUB) {
#pragma unroll
      for (int ri = 0; ri < 8; ++ri) {
        const int m = 8 * g + ri;
        if (m <= D) {
          const float t = (m < D) ? c1 * zrow[m] : c0;
          const float4* row = reinterpret_cast<const float4*>(Ss + m * G::LDS);
#pragma unroll
          for (int j4 = 0; j4 < G::LDS / 4; ++j4) {
            float4 s = row[j4];
            acc[4 * j4 + 0] += t * s.x; acc[4 * j4 + 1] += t * s.y;
            acc[4 * j4 + 2] += t * s.z; acc[4 * j4 + 3] += t * s.w;
          }
        }
      }
    }
  }
}

// ------------------------------------------------------------------------------------------------
// apply (gradient form):  dphi_f = sum_j g_l[j] Ss[f][j];  dz_l = chain rule through Phi, summed into
// Dz[l][.] (shared, atomics: the sub-threads of a token overlap on the b-block columns).
// ------------------------------------------------------------------------------------------------
template <int D, int C, int NT>
__device__ __forceinline__ void apply_grad_phase(float* Dz, const float* __restrict__ Ss,
                                                 const float* __restrict__ Zs, const float* __restrict__ Gs,
                                                 bool lin_slice, int u0, int nu, float c1, float c2, int l,
                                                 int sub) {
  using G = Geo<D>;
  constexpr int NSUB = NT / C;
  constexpr int MPS = 8 / NSUB;
  const float* zrow = Zs + l * G::LDX;
  float gl[G::LDY];
#pragma unroll
  for (int j4 = 0; j4 < G::LDY / 4; ++j4) {
    float4 t = *reinterpret_cast<const float4*>(Gs + l * G::LDY + 4 * j4);
    gl[4 * j4 + 0] = t.x; gl[4 * j4 + 1] = t.y; gl[4 * j4 + 2] = t.z; gl[4 * j4 + 3] = t.w;
  }
  float* dzrow = Dz + l * G::LDY;
  if (!lin_slice) {
    for (int ul = 0; ul < nu; ++ul) {
      int a, b;
      pair_decode(u0 + ul, G::NB, a, b);
      const float w = (a == b) ? c2 : 2.f * c2;
      float zb[8], dzb[8];
      {
        float4 t0 = *reinterpret_cast<const float4*>(zrow + 8 * b);
        float4 t1 = *reinterpret_cast<const float4*>(zrow + 8 * b + 4);
        zb[0] = t0.x; zb[1] = t0.y; zb[2] = t0.z; zb[3] = t0.w;
        zb[4] = t1.x; zb[5] = t1.y; zb[6] = t1.z; zb[7] = t1.w;
      }
#pragma unroll
      for (int ri = 0; ri < 8; ++ri) dzb[ri] = 0.f;
#pragma unroll
      for (int i = 0; i < MPS; ++i) {
        const float za = zrow[8 * a + sub * MPS + i];
        float dza = 0.f;
#pragma unroll
        for (int ri = 0; ri < 8; ++ri) {
          const float4* row = reinterpret_cast<const float4*>(Ss + (ul * 64 + (sub * MPS + i) * 8 + ri) * G::LDS);
          float p0 = 0.f, p1 = 0.f, p2 = 0.f, p3 = 0.f;
#pragma unroll
          for (int j4 = 0; j4 < G::LDS / 4; ++j4) {
            float4 s = row[j4];
            p0 += gl[4 * j4 + 0] * s.x; p1 += gl[4 * j4 + 1] * s.y;
            p2 += gl[4 * j4 + 2] * s.z; p3 += gl[4 * j4 + 3] * s.w;
          }
          const float dphi = ((p0 + p1) + (p2 + p3)) * w;
          dza += dphi * zb[ri];
          dzb[ri] += dphi * za;
        }
        atomicAdd(dzrow + 8 * a + sub * MPS + i, dza);
      }
#pragma unroll
      for (int ri = 0; ri < 8; ++ri) atomicAdd(dzrow + 8 * b + ri, dzb[ri]);
    }
  } else {
    for (int g = sub; g < G::NLG; g += NSUB) {
#pragma unroll
      for (int ri = 0; ri < 8; ++ri) {
        const int m = 8 * g + ri;
        if (m < D) {
          const float4* row = reinterpret_cast<const float4*>(Ss + m * G::LDS);
          float p0 = 0.f, p1 = 0.f, p2 = 0.f, p3 = 0.f;
#pragma unroll
          for (int j4 = 0; j4 < G::LDS / 4; ++j4) {
            float4 s = row[j4];
            p0 += gl[4 * j4 + 0] * s.x; p1 += gl[4 * j4 + 1] * s.y;
            p2 += gl[4 * j4 + 2] * s.z; p3 += gl[4 * j4 + 3] * s.w;
          }
          atomicAdd(dzrow + m, ((p0 + p1) + (p2 + p3)) * c1);
        }
      }
    }
  }
}

// Adds per-thread partial rows into Red[l][0..NCOL) one sub-thread group at a time (deterministic).
template <int NCOL, int LD, int NSUB>
__device__ __forceinline__ void staged_add(float* Red, const float* acc, int l, int sub) {
  __syncthreads();
  for (int s = 0; s < NSUB; ++s) {
    if (sub == s) {
      float4* r = reinterpret_cast<float4*>(Red + l * LD);
#pragma unroll
      for (int j4 = 0; j4 < NCOL / 4; ++j4) {
        float4 t = r[j4];
        t.x += acc[4 * j4 + 0]; t.y += acc[4 * j4 + 1]; t.z += acc[4 * j4 + 2]; t.w += acc[4 * j4 + 3];
        r[j4] = t;
      }
    }
    __syncthreads();
  }
}

// Red[C][LD] (first NCOL columns) -> global fp32 accumulator rows (row stride GLD) with float4 atomics.
template <int C, int NT, int NCOL, int LD>
__device__ __forceinline__ void flush_rows(const float* Red, float* gout, int gld, long long row0, long long nrows,
                                           int tid) {
  constexpr int VPR = NCOL / 4;
  for (int idx = tid; idx < C * VPR; idx += NT) {
    int r = idx / VPR, cv = idx - r * VPR;
    long long row = row0 + r;
    if (row >= 0 && row < nrows) {
      float4 val = *reinterpret_cast<const float4*>(Red + r * LD + 4 * cv);
      atomicAdd(reinterpret_cast<float4*>(gout + row * gld + 4 * cv), val);
    }
  }
}

// ------------------------------------------------------------------------------------------------
// the scan kernel
// ------------------------------------------------------------------------------------------------
// Shared memory of one scan CTA, in floats: only the tiles the mode uses are laid out and the two intra-chunk
// matrices are stored as packed triangles, so that for head dims up to 32 two CTAs fit on an SM (93 / 94 / 111 KB for
// the forward / dq / dk-dv scans; their register need, capped at 128 by the launch bounds, allows it without spills).
template <int D, int MODE>
struct ScanSmem {
  using G = Geo<D>;
  using K = Cfg<D>;
  static constexpr int S = 0;
  static constexpr int Q = S + K::SROWS * G::LDS;                                   // q tile  [C][LDX]
  static constexpr int KK = Q + K::C * G::LDX;                                      // k tile  [C][LDX]
  static constexpr int V = KK + K::C * G::LDX;                                      // [V|1]   [C][LDY]
  static constexpr int O = V + K::C * G::LDY;                                       // dO'     [C][LDY]   (backward)
  static constexpr int RED = O + (MODE != MODE_FWD ? K::C * G::LDY : 0);            // output staging [C][LDY]
  static constexpr int RED2 = RED + K::C * G::LDY;                                  // second output (dv)   (dk/dv scan)
  static constexpr int TRI = K::C * (K::C + 1) / 2;    // a lower-triangular [C][C] matrix, packed: (l, j <= l) at l (l + 1) / 2 + j
  static constexpr int A = RED2 + (MODE == MODE_BWD_KV ? K::C * G::LDY : 0);        // tril f(QK^T)            (not dq)
  static constexpr int DM = A + (MODE != MODE_BWD_Q ? TRI : 0);                     // tril (dO' V'^T) f'      (backward)
  static constexpr int TOTAL = DM + (MODE != MODE_FWD ? TRI : 0);
};
template <int D, int MODE>
constexpr int scan_min_blocks() { return D <= 32 ? 2 : 1; }
__device__ __forceinline__ int tri_index(int l, int j) { return ((l * (l + 1)) >> 1) + j; }

template <typename T, int D, int MODE, bool CAUSAL>
__global__ void __launch_bounds__(Cfg<D>::NT, scan_min_blocks<D, MODE>()) scan_kernel(const ScanParams P) {
  using G = Geo<D>;
  using K = Cfg<D>;
  using L = ScanSmem<D, MODE>;
  constexpr int C = K::C, NT = K::NT, NSUB = K::NSUB;
  extern __shared__ __align__(16) float smem[];
  float* Ss = smem + L::S;
  float* Qs = smem + L::Q;
  float* Ks = smem + L::KK;
  float* Vs = smem + L::V;
  float* Os = smem + L::O;       // the pointers of tiles a mode does not have alias the next tile and are never used
  float* Red = smem + L::RED;
  float* Red2 = smem + L::RED2;
  float* Am = smem + L::A;
  float* Dm = smem + L::DM;

  const int tid = threadIdx.x;
  const int slice = blockIdx.x, seg = blockIdx.y, head = blockIdx.z;
  const bool lin_slice = (slice == P.npair_slices);
  int u0 = 0, nu = 0;
  if (!lin_slice) slice_units(slice, P.npair_slices, G::NPAIRS, u0, nu);

  const T* qb = head_base<T>(P.q, head, P.heads);
  const T* kb = head_base<T>(P.k, head, P.heads);
  const T* vb = head_base<T>(P.v, head, P.heads);
  const float* dopb = (MODE != MODE_FWD) ? P.dop + (long long)head * P.nq * G::LDY : nullptr;

  const float* gstate = nullptr;
  if (P.seg_state != nullptr)
    gstate = P.seg_state + (long long)head * P.seg_state_head_stride + (long long)seg * P.seg_state_seg_stride;
  load_state_slice<D, NT, K::SROWS>(Ss, gstate, lin_slice, u0, nu, P.order, tid);

  const int cbeg = seg * P.chunks_per_seg;
  const int cend = min(P.nchunks, cbeg + P.chunks_per_seg);
  const int l = tid % C, sub = tid / C;
  const bool do_intra = CAUSAL && lin_slice;

  for (int ci = cbeg; ci < cend; ++ci) {
    const int c = (MODE == MODE_BWD_KV && CAUSAL) ? (cend - 1 - (ci - cbeg)) : ci;
    const long long pos0 = (long long)c * C;  // causal: key position; non-causal: row of the Z tensor
    // ---- load ----
    if (CAUSAL) {
      load_tile<T, D, C, NT, G::LDX, false>(Qs, qb, P.q.sn, pos0 - P.off, P.nq, tid);
      load_tile<T, D, C, NT, G::LDX, false>(Ks, kb, P.k.sn, pos0, P.nk, tid);
      load_tile<T, D, C, NT, G::LDY, true>(Vs, vb, P.v.sn, pos0, P.nk, tid);
      if (MODE != MODE_FWD) load_dense_tile<C, NT, G::LDY>(Os, dopb, pos0 - P.off, P.nq, tid);
    } else {
      if (MODE == MODE_BWD_KV) {
        load_tile<T, D, C, NT, G::LDX, false>(Ks, kb, P.k.sn, pos0, P.nk, tid);
        load_tile<T, D, C, NT, G::LDY, true>(Vs, vb, P.v.sn, pos0, P.nk, tid);
      } else {
        load_tile<T, D, C, NT, G::LDX, false>(Qs, qb, P.q.sn, pos0, P.nq, tid);
        if (MODE == MODE_BWD_Q) load_dense_tile<C, NT, G::LDY>(Os, dopb, pos0, P.nq, tid);
      }
    }
    for (int idx = tid; idx < C * G::LDY; idx += NT) {
      Red[idx] = 0.f;
      if (MODE == MODE_BWD_KV) Red2[idx] = 0.f;
    }
    __syncthreads();

    // ---- intra-chunk score matrices (lin slice, causal) ----
    if (do_intra) {
      float qreg[D];
#pragma unroll
      for (int d4 = 0; d4 < D / 4; ++d4) {
        float4 t = *reinterpret_cast<const float4*>(Qs + l * G::LDX + 4 * d4);
        qreg[4 * d4 + 0] = t.x; qreg[4 * d4 + 1] = t.y; qreg[4 * d4 + 2] = t.z; qreg[4 * d4 + 3] = t.w;
      }
      for (int j = sub; j < C; j += NSUB) {
        float a = 0.f, ds = 0.f;
        if (j <= l) {
          const float* krow = Ks + j * G::LDX;
          float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
#pragma unroll
          for (int d4 = 0; d4 < D / 4; ++d4) {
            float4 kk = *reinterpret_cast<const float4*>(krow + 4 * d4);
            s0 += qreg[4 * d4 + 0] * kk.x; s1 += qreg[4 * d4 + 1] * kk.y;
            s2 += qreg[4 * d4 + 2] * kk.z; s3 += qreg[4 * d4 + 3] * kk.w;
          }
          const float s = (s0 + s1) + (s2 + s3);
          a = P.c0 + s * (P.c1 + P.c2 * s);
          if (MODE != MODE_FWD) {
            const float* orow = Os + l * G::LDY;
            const float* vrow = Vs + j * G::LDY;
            float p0 = 0.f, p1 = 0.f, p2 = 0.f, p3 = 0.f;
#pragma unroll
            for (int j4 = 0; j4 < G::LDY / 4; ++j4) {
              float4 oo = *reinterpret_cast<const float4*>(orow + 4 * j4);
              float4 vv = *reinterpret_cast<const float4*>(vrow + 4 * j4);
              p0 += oo.x * vv.x; p1 += oo.y * vv.y; p2 += oo.z * vv.z; p3 += oo.w * vv.w;
            }
            ds = ((p0 + p1) + (p2 + p3)) * (P.c1 + 2.f * P.c2 * s);
          }
        }
        if (j <= l) {   // entries above the diagonal are zero and not stored
          if (MODE != MODE_BWD_Q) Am[tri_index(l, j)] = a;
          if (MODE != MODE_FWD) Dm[tri_index(l, j)] = ds;
        }
      }
      __syncthreads();
    }

    // ---- apply + intra products ----
    if (MODE == MODE_FWD) {
      float acc[G::LDS];
#pragma unroll
      for (int j = 0; j < G::LDS; ++j) acc[j] = 0.f;
      apply_fwd_accum<D, C, NT>(acc, Ss, Qs, lin_slice, u0, nu, P.c0, P.c1, P.c2, l, sub);
      if (do_intra) {
        const int jmax = l | 31;
        for (int j = sub; j <= jmax; j += NSUB) {
          const float a = j <= l ? Am[tri_index(l, j)] : 0.f;   // the loop bound is warp-uniform: up to 31 zeros
          const float4* vrow = reinterpret_cast<const float4*>(Vs + j * G::LDY);
#pragma unroll
          for (int j4 = 0; j4 < G::LDY / 4; ++j4) {
            float4 vv = vrow[j4];
            acc[4 * j4 + 0] += a * vv.x; acc[4 * j4 + 1] += a * vv.y;
            acc[4 * j4 + 2] += a * vv.z; acc[4 * j4 + 3] += a * vv.w;
          }
        }
      }
      staged_add<G::LDY, G::LDY, NSUB>(Red, acc, l, sub);
    } else if (MODE == MODE_BWD_Q) {
      apply_grad_phase<D, C, NT>(Red, Ss, Qs, Os, lin_slice, u0, nu, P.c1, P.c2, l, sub);
      if (do_intra) {
        float acc[D];
#pragma unroll
        for (int d = 0; d < D; ++d) acc[d] = 0.f;
        const int jmax = l | 31;
        for (int j = sub; j <= jmax; j += NSUB) {
          const float ds = j <= l ? Dm[tri_index(l, j)] : 0.f;
          const float4* krow = reinterpret_cast<const float4*>(Ks + j * G::LDX);
#pragma unroll
          for (int d4 = 0; d4 < D / 4; ++d4) {
            float4 kk = krow[d4];
            acc[4 * d4 + 0] += ds * kk.x; acc[4 * d4 + 1] += ds * kk.y;
            acc[4 * d4 + 2] += ds * kk.z; acc[4 * d4 + 3] += ds * kk.w;
          }
        }
        staged_add<D, G::LDY, NSUB>(Red, acc, l, sub);
      } else {
        __syncthreads();
      }
    } else {  // MODE_BWD_KV
      apply_grad_phase<D, C, NT>(Red, Ss, Ks, Vs, lin_slice, u0, nu, P.c1, P.c2, l, sub);
      float acc[G::LDS];
#pragma unroll
      for (int j = 0; j < G::LDS; ++j) acc[j] = 0.f;
      apply_fwd_accum<D, C, NT>(acc, Ss, Ks, lin_slice, u0, nu, P.c0, P.c1, P.c2, l, sub);
      if (do_intra) {
        // thread = key j (= l here), queries ll >= j of the chunk
        float dkacc[D];
#pragma unroll
        for (int d = 0; d < D; ++d) dkacc[d] = 0.f;
        const int lmin = l & ~31;
        for (int ll = lmin + sub; ll < C; ll += NSUB) {
          const float ds = ll >= l ? Dm[tri_index(ll, l)] : 0.f;
          const float a = ll >= l ? Am[tri_index(ll, l)] : 0.f;
          const float4* qrow = reinterpret_cast<const float4*>(Qs + ll * G::LDX);
          const float4* orow = reinterpret_cast<const float4*>(Os + ll * G::LDY);
#pragma unroll
          for (int d4 = 0; d4 < D / 4; ++d4) {
            float4 qq = qrow[d4];
            float4 oo = orow[d4];
            dkacc[4 * d4 + 0] += ds * qq.x; dkacc[4 * d4 + 1] += ds * qq.y;
            dkacc[4 * d4 + 2] += ds * qq.z; dkacc[4 * d4 + 3] += ds * qq.w;
            acc[4 * d4 + 0] += a * oo.x; acc[4 * d4 + 1] += a * oo.y;
            acc[4 * d4 + 2] += a * oo.z; acc[4 * d4 + 3] += a * oo.w;
          }
        }
        staged_add<D, G::LDY, NSUB>(Red, dkacc, l, sub);
      }
      staged_add<D, G::LDY, NSUB>(Red2, acc, l, sub);
    }

    // ---- flush partial outputs, then advance the state ----
    if (MODE == MODE_FWD) {
      const long long r0 = CAUSAL ? pos0 - P.off : pos0;
      flush_rows<C, NT, G::LDY, G::LDY>(Red, P.out0 + (long long)head * P.nq * G::LDY, G::LDY, r0, P.nq, tid);
    } else if (MODE == MODE_BWD_Q) {
      const long long r0 = CAUSAL ? pos0 - P.off : pos0;
      flush_rows<C, NT, D, G::LDY>(Red, P.out0 + (long long)head * P.nq * D, D, r0, P.nq, tid);
    } else {
      flush_rows<C, NT, D, G::LDY>(Red, P.out0 + (long long)head * P.nk * D, D, pos0, P.nk, tid);
      flush_rows<C, NT, D, G::LDY>(Red2, P.out1 + (long long)head * P.nk * D, D, pos0, P.nk, tid);
    }
    if (CAUSAL) {
      if (MODE == MODE_BWD_KV)
        update_phase<D, C, NT, K::TR>(Ss, Qs, Os, lin_slice, u0, nu, tid);
      else
        update_phase<D, C, NT, K::TR>(Ss, Ks, Vs, lin_slice, u0, nu, tid);
    }
    __syncthreads();
  }
}

template <int D, int MODE>
constexpr size_t scan_smem_bytes() {
  return sizeof(float) * (size_t)ScanSmem<D, MODE>::TOTAL;
}

// ------------------------------------------------------------------------------------------------
// moments: total state of every segment,  T[head][seg] = sum_{t in seg} Phi(x_t)^T y_t
// ------------------------------------------------------------------------------------------------
template <typename T, int D, int SRC>
__global__ void __launch_bounds__(Cfg<D>::NT, 1) moments_kernel(const MomentParams P) {
  using G = Geo<D>;
  using K = Cfg<D>;
  constexpr int C = K::C, NT = K::NT;
  extern __shared__ __align__(16) float smem[];
  float* Ss = smem;
  float* Xs = Ss + K::SROWS * G::LDS;
  float* Ys = Xs + C * G::LDX;
  const int tid = threadIdx.x;
  const int slice = blockIdx.x, seg = blockIdx.y, head = blockIdx.z;
  const bool lin_slice = (slice == P.npair_slices);
  int u0 = 0, nu = 0;
  if (!lin_slice) slice_units(slice, P.npair_slices, G::NPAIRS, u0, nu);
  const T* xb = head_base<T>(P.x, head, P.heads);
  const T* vb = (SRC == MOM_KV) ? head_base<T>(P.v, head, P.heads) : nullptr;
  const float* dopb = (SRC == MOM_QG) ? P.dop + (long long)head * P.nrows_y * G::LDY : nullptr;
  load_state_slice<D, NT, K::SROWS>(Ss, nullptr, lin_slice, u0, nu, P.order, tid);
  const int cbeg = seg * P.chunks_per_seg;
  const int cend = min(P.nchunks, cbeg + P.chunks_per_seg);
  for (int c = cbeg; c < cend; ++c) {
    const long long pos0 = (long long)c * C;
    load_tile<T, D, C, NT, G::LDX, false>(Xs, xb, P.x.sn, pos0 - P.x_shift, P.nrows_x, tid);
    if (SRC == MOM_KV)
      load_tile<T, D, C, NT, G::LDY, true>(Ys, vb, P.v.sn, pos0, P.nrows_y, tid);
    else
      load_dense_tile<C, NT, G::LDY>(Ys, dopb, pos0 - P.x_shift, P.nrows_y, tid);
    __syncthreads();
    update_phase<D, C, NT, K::TR>(Ss, Xs, Ys, lin_slice, u0, nu, tid);
    __syncthreads();
  }
  const int rows = state_rows(D, P.order);
  float* gout = P.seg_total + ((long long)head * P.nseg + seg) * (long long)rows * G::LDS;
  store_state_slice<D, NT>(Ss, gout, lin_slice, u0, nu, P.order, tid);
}

template <int D>
constexpr size_t moments_smem_bytes() {
  using G = Geo<D>;
  using K = Cfg<D>;
  return sizeof(float) * (size_t)(K::SROWS * G::LDS + K::C * G::LDX + K::C * G::LDY);
}

}  // namespace fm
