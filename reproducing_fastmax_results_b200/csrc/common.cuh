// Shared definitions of the Fastmax engine: feature geometry, kernel parameter blocks, tile loaders.
//
// Feature map.  Phi(x) for head dim D is stored as "units":
//   pair unit u <-> (a, b), a <= b, 8-wide blocks of the head dim: 64 features x[8a+mi] * x[8b+ri]
//   (block-symmetric packing of x (x) x: an off-diagonal block stands for (a,b) and (b,a), weight 2)
//   the last unit ("lin") holds x[0..D-1] and the constant 1.
// State row of feature i of pair unit u: 64*u + i; lin rows: 64*NPAIRS + m (m < D), constant: 64*NPAIRS + D.
// For order 1 only the lin unit exists and its rows start at 0.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace fm {

template <int D>
struct Geo {
  static constexpr int NB = D / 8;
  static constexpr int NPAIRS = NB * (NB + 1) / 2;
  static constexpr int DV1 = D + 1;
  static constexpr int LDS = D + 4;    // state row stride (floats); columns D+1.. are padding
  static constexpr int LDX = D + 12;   // q/k tile row: [x(D), 1, 0 x 11]; LDX/4 odd -> conflict-free 128-bit rows
  static constexpr int LDY = D + 4;    // v/dO' tile row: [y(D), y_D, 0, 0, 0]; LDY/4 odd
  static constexpr int NLG = D / 8 + 1;  // 8-wide groups of the lin unit (x and the constant)
  static constexpr int LIN_ROW0 = 64 * NPAIRS;
  static constexpr int ROWS_P2 = 64 * NPAIRS + D + 1;
  static constexpr int ROWS_P1 = D + 1;
};

__host__ __device__ inline int state_rows(int d, int order) {
  int nb = d / 8;
  return order == 2 ? 64 * (nb * (nb + 1) / 2) + d + 1 : d + 1;
}
__host__ __device__ inline int state_ld(int d) { return d + 4; }

__host__ __device__ inline void pair_decode(int u, int nb, int& a, int& b) {
  a = 0;
  int len = nb;
  while (u >= len) {
    u -= len;
    ++a;
    --len;
  }
  b = a + u;
}

struct View {  // strided (batch, head, token, dim) view; strides in elements
  const void* ptr;
  long long sb, sh, sn;
};

enum Mode { MODE_FWD = 0, MODE_BWD_Q = 1, MODE_BWD_KV = 2 };
enum MomentSrc { MOM_KV = 0, MOM_QG = 1 };

struct ScanParams {
  View q, k, v;
  const float* dop;        // [BH][nq][LDY]      backward only
  float* out0;             // FWD: O' [BH][nq][LDY]; BWD_Q: dq [BH][nq][D]; BWD_KV: dk [BH][nk][D]
  float* out1;             // BWD_KV: dv [BH][nk][D]
  const float* seg_state;  // initial state of every segment, or NULL (zero)
  long long seg_state_head_stride;  // floats
  long long seg_state_seg_stride;   // floats (0 when every segment starts from the same state)
  int heads, nq, nk, off;  // off = nk - nq (causal alignment), 0 otherwise
  int order, causal;
  int nchunks, chunks_per_seg, nseg;
  int npair_slices;        // pair units are split evenly over this many slices; slice index npair_slices = lin slice
  float c0, c1, c2, inv_temp;  // a0, a1*inv_temp, a2*inv_temp^2
};

struct MomentParams {
  View x, v;               // MOM_KV: x = k, v = v.  MOM_QG: x = q
  const float* dop;        // MOM_QG
  float* seg_total;        // [BH][nseg][rows][LDS]
  int heads, nrows_x, nrows_y, x_shift;  // row index of x for position t is t - x_shift (MOM_QG causal: off)
  int order;
  int nchunks, chunks_per_seg, nseg;
  int npair_slices;
};

template <typename T>
__device__ __forceinline__ float4 load4(const T* p);
template <>
__device__ __forceinline__ float4 load4<float>(const float* p) {
  return *reinterpret_cast<const float4*>(p);
}
template <>
__device__ __forceinline__ float4 load4<__nv_bfloat16>(const __nv_bfloat16* p) {
  uint2 raw = *reinterpret_cast<const uint2*>(p);
  __nv_bfloat162 lo = *reinterpret_cast<__nv_bfloat162*>(&raw.x);
  __nv_bfloat162 hi = *reinterpret_cast<__nv_bfloat162*>(&raw.y);
  float2 a = __bfloat1622float2(lo), b = __bfloat1622float2(hi);
  return make_float4(a.x, a.y, b.x, b.y);
}

template <typename T>
__device__ __forceinline__ const T* head_base(const View& t, int head, int heads) {
  int b = head / heads, h = head - b * heads;
  return reinterpret_cast<const T*>(t.ptr) + (long long)b * t.sb + (long long)h * t.sh;
}

// Loads C rows (row0 + r) of a [nrows][D] strided source into dst[C][LD] as floats.  Rows outside
// [0, nrows) are zero.  Column D gets `tail` for valid rows when TAIL_VALID (the ones column of [V|1])
// or 1 always otherwise (the constant feature of a q/k tile); the remaining pad columns are zero.
template <typename T, int D, int C, int NT, int LD, bool TAIL_VALID>
__device__ __forceinline__ void load_tile(float* dst, const T* base, long long stride_n, long long row0,
                                          long long nrows, int tid) {
  constexpr int VPR = D / 4;
  for (int idx = tid; idx < C * VPR; idx += NT) {
    int r = idx / VPR, cv = idx - r * VPR;
    long long row = row0 + r;
    float4 val = make_float4(0.f, 0.f, 0.f, 0.f);
    if (row >= 0 && row < nrows) val = load4<T>(base + row * stride_n + cv * 4);
    *reinterpret_cast<float4*>(dst + r * LD + cv * 4) = val;
  }
  constexpr int TAIL = LD - D;
  for (int idx = tid; idx < C * TAIL; idx += NT) {
    int r = idx / TAIL, c = idx - r * TAIL;
    long long row = row0 + r;
    float t = 0.f;
    if (c == 0) t = TAIL_VALID ? ((row >= 0 && row < nrows) ? 1.f : 0.f) : 1.f;
    dst[r * LD + D + c] = t;
  }
}

// Dense float source with row stride LD (the dO' scratch): copies whole rows, zero outside [0, nrows).
template <int C, int NT, int LD>
__device__ __forceinline__ void load_dense_tile(float* dst, const float* base, long long row0, long long nrows,
                                                int tid) {
  constexpr int VPR = LD / 4;
  for (int idx = tid; idx < C * VPR; idx += NT) {
    int r = idx / VPR, cv = idx - r * VPR;
    long long row = row0 + r;
    float4 val = make_float4(0.f, 0.f, 0.f, 0.f);
    if (row >= 0 && row < nrows) val = *reinterpret_cast<const float4*>(base + row * LD + cv * 4);
    *reinterpret_cast<float4*>(dst + r * LD + cv * 4) = val;
  }
}

// first pair unit / number of pair units of pair slice s when `npairs` units are split evenly over ns slices
__host__ __device__ inline void slice_units(int s, int ns, int npairs, int& u0, int& nu) {
  u0 = (int)((long long)s * npairs / ns);
  int u1 = (int)((long long)(s + 1) * npairs / ns);
  nu = u1 - u0;
}

}  // namespace fm
