// Memory-bound helper kernels: segment-state scans, forward combine/divide, backward prologue, output casts
// and the q/k normalisation.
#pragma once
#include <cooperative_groups.h>
#include "common.cuh"

namespace fm {

template <typename T>
__device__ __forceinline__ float to_float(T v);
template <>
__device__ __forceinline__ float to_float<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_float<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T>
__device__ __forceinline__ T from_float(float v);
template <>
__device__ __forceinline__ float from_float<float>(float v) { return v; }
template <>
__device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

enum ScanOp { SCAN_PREFIX = 0, SCAN_SUFFIX = 1, SCAN_TOTAL = 2 };

// seg: [BH][nseg][n] segment totals.  PREFIX/SUFFIX: replaced in place by the exclusive running sum
// (starting from init[head] when given).  TOTAL: slot 0 of each head receives the sum of all segments.
// total_out[head] (optional) = init + all segments.
__global__ void state_scan_kernel(float* seg, int nseg, long long n, const float* init, float* total_out, int op,
                                  long long total_elems) {
  long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total_elems) return;
  long long head = idx / n, e = idx - head * n;
  float run = init ? init[idx] : 0.f;
  float* base = seg + head * nseg * n + e;
  if (op == SCAN_PREFIX) {
    for (int s = 0; s < nseg; ++s) {
      float t = base[(long long)s * n];
      base[(long long)s * n] = run;
      run += t;
    }
  } else if (op == SCAN_SUFFIX) {
    for (int s = nseg - 1; s >= 0; --s) {
      float t = base[(long long)s * n];
      base[(long long)s * n] = run;
      run += t;
    }
  } else {
    for (int s = 0; s < nseg; ++s) run += base[(long long)s * n];
    base[0] = run;
  }
  if (total_out) total_out[idx] = run;
}

// O' accumulator [BH][nq][ld] -> o = O'[:, :d] / O'[:, d] (dtype T, strided) and g = O'[:, d] (float, strided).
template <typename T>
__global__ void finalize_fwd_kernel(const float* __restrict__ acc, int ld, int d, int nq, int heads, View o, View g,
                                    long long total) {
  long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  int c = (int)(idx % d);
  long long row = idx / d;
  int l = (int)(row % nq);
  int head = (int)(row / nq);
  const float* r = acc + row * ld;
  float den = r[d];
  int b = head / heads, h = head - b * heads;
  T* op = reinterpret_cast<T*>(const_cast<void*>(o.ptr)) + (long long)b * o.sb + (long long)h * o.sh + (long long)l * o.sn;
  op[c] = from_float<T>(r[c] / den);
  if (c == 0 && g.ptr != nullptr) {
    float* gp = reinterpret_cast<float*>(const_cast<void*>(g.ptr)) + (long long)b * g.sb + (long long)h * g.sh +
                (long long)l * g.sn;
    *gp = den;
  }
}

// ---- 4-wide variants (grid.y = batch*head, 32-bit index math): used when the output view is 8/16-byte aligned ----
template <typename T>
__device__ __forceinline__ void store4(T* p, float a, float b, float c, float d);
template <>
__device__ __forceinline__ void store4<float>(float* p, float a, float b, float c, float d) {
  *reinterpret_cast<float4*>(p) = make_float4(a, b, c, d);
}
template <>
__device__ __forceinline__ void store4<__nv_bfloat16>(__nv_bfloat16* p, float a, float b, float c, float d) {
  __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
  uint2 v;
  v.x = *reinterpret_cast<uint32_t*>(&lo);
  v.y = *reinterpret_cast<uint32_t*>(&hi);
  *reinterpret_cast<uint2*>(p) = v;
}

template <typename T>
__global__ void finalize_fwd_vec_kernel(const float* __restrict__ acc, int ld, int d, int nq, int heads, View o, View g) {
  const int head = blockIdx.y;
  const int d4 = d >> 2;
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= nq * d4) return;
  const int l = t / d4, c = (t - l * d4) << 2;
  const float* r = acc + ((long long)head * nq + l) * ld;
  const float4 v = *reinterpret_cast<const float4*>(r + c);
  const float den = r[d];
  const float inv = 1.f / den;
  const int b = head / heads, h = head - b * heads;
  T* op = reinterpret_cast<T*>(const_cast<void*>(o.ptr)) + (long long)b * o.sb + (long long)h * o.sh + (long long)l * o.sn;
  store4<T>(op + c, v.x * inv, v.y * inv, v.z * inv, v.w * inv);
  if (c == 0 && g.ptr != nullptr)
    *(reinterpret_cast<float*>(const_cast<void*>(g.ptr)) + (long long)b * g.sb + (long long)h * g.sh + (long long)l * g.sn) = den;
}

// bf16 outputs, eight columns per thread: two 128-bit streaming loads of the float32 accumulator row, one 128-bit
// store (the accumulators are read exactly once, so they bypass L1 and are marked evict-first).
__device__ __forceinline__ uint32_t pack2_bf16(float lo, float hi) {
  __nv_bfloat162 r = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&r);
}
__global__ void finalize_fwd_bf16x8_kernel(const float* __restrict__ acc, int ld, int d, int nq, int heads, View o, View g) {
  const int head = blockIdx.y;
  const int d8 = d >> 3;
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= nq * d8) return;
  const int l = t / d8, c = (t - l * d8) << 3;
  const float* r = acc + ((long long)head * nq + l) * ld;
  const float4 v0 = __ldcs(reinterpret_cast<const float4*>(r + c));
  const float4 v1 = __ldcs(reinterpret_cast<const float4*>(r + c + 4));
  const float den = __ldcs(r + d);
  const float inv = 1.f / den;
  const int b = head / heads, h = head - b * heads;
  __nv_bfloat16* op = reinterpret_cast<__nv_bfloat16*>(const_cast<void*>(o.ptr)) + (long long)b * o.sb + (long long)h * o.sh + (long long)l * o.sn;
  *reinterpret_cast<uint4*>(op + c) = make_uint4(pack2_bf16(v0.x * inv, v0.y * inv), pack2_bf16(v0.z * inv, v0.w * inv),
                                                 pack2_bf16(v1.x * inv, v1.y * inv), pack2_bf16(v1.z * inv, v1.w * inv));
  if (c == 0 && g.ptr != nullptr)
    *(reinterpret_cast<float*>(const_cast<void*>(g.ptr)) + (long long)b * g.sb + (long long)h * g.sh + (long long)l * g.sn) = den;
}
__global__ void cast_out_bf16x8_kernel(const float* __restrict__ acc, int d, int n, int heads, View out, int acc_ld) {
  const int head = blockIdx.y;
  const int d8 = d >> 3;
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= n * d8) return;
  const int l = t / d8, c = (t - l * d8) << 3;
  const float* r = acc + ((long long)head * n + l) * acc_ld + c;
  const float4 v0 = __ldcs(reinterpret_cast<const float4*>(r));
  const float4 v1 = __ldcs(reinterpret_cast<const float4*>(r + 4));
  const int b = head / heads, h = head - b * heads;
  __nv_bfloat16* op = reinterpret_cast<__nv_bfloat16*>(const_cast<void*>(out.ptr)) + (long long)b * out.sb + (long long)h * out.sh + (long long)l * out.sn;
  *reinterpret_cast<uint4*>(op + c) = make_uint4(pack2_bf16(v0.x, v0.y), pack2_bf16(v0.z, v0.w), pack2_bf16(v1.x, v1.y), pack2_bf16(v1.z, v1.w));
}

template <typename T>
__global__ void cast_out_vec_kernel(const float* __restrict__ acc, int d, int n, int heads, View out, int acc_ld) {
  const int head = blockIdx.y;
  const int d4 = d >> 2;
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= n * d4) return;
  const int l = t / d4, c = (t - l * d4) << 2;
  const float4 v = *reinterpret_cast<const float4*>(acc + ((long long)head * n + l) * acc_ld + c);
  const int b = head / heads, h = head - b * heads;
  T* op = reinterpret_cast<T*>(const_cast<void*>(out.ptr)) + (long long)b * out.sb + (long long)h * out.sh + (long long)l * out.sn;
  store4<T>(op + c, v.x, v.y, v.z, v.w);
}

// dO'[row] = [dO/g, -(dO . o)/g, 0, 0, 0]  (float, row stride ld = d+4); one warp per row.
template <typename T>
__global__ void bwd_prologue_kernel(View dout, View o, View g, float* __restrict__ dop, int ld, int d, int nq,
                                    int heads, long long nrows) {
  long long row = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  int lane = threadIdx.x & 31;
  if (row >= nrows) return;
  int l = (int)(row % nq);
  int head = (int)(row / nq);
  int b = head / heads, h = head - b * heads;
  const T* dp = reinterpret_cast<const T*>(dout.ptr) + (long long)b * dout.sb + (long long)h * dout.sh + (long long)l * dout.sn;
  const T* op = reinterpret_cast<const T*>(o.ptr) + (long long)b * o.sb + (long long)h * o.sh + (long long)l * o.sn;
  const float gv = *(reinterpret_cast<const float*>(g.ptr) + (long long)b * g.sb + (long long)h * g.sh + (long long)l * g.sn);
  const float inv = 1.f / gv;
  float dot = 0.f;
  float* out = dop + row * ld;
  for (int c = lane; c < d; c += 32) {
    float x = to_float<T>(dp[c]);
    dot += x * to_float<T>(op[c]);
    out[c] = x * inv;
  }
#pragma unroll
  for (int s = 16; s > 0; s >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, s);
  if (lane == 0) out[d] = -dot * inv;
  if (lane >= 1 && lane < ld - d) out[d + lane] = 0.f;
}

// fp32 accumulator [BH][n][acc_ld] (first d columns) -> strided output of dtype T
template <typename T>
__global__ void cast_out_kernel(const float* __restrict__ acc, int d, int n, int heads, View out, long long total, int acc_ld) {
  long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  int c = (int)(idx % d);
  long long row = idx / d;
  int l = (int)(row % n);
  int head = (int)(row / n);
  int b = head / heads, h = head - b * heads;
  T* op = reinterpret_cast<T*>(const_cast<void*>(out.ptr)) + (long long)b * out.sb + (long long)h * out.sh + (long long)l * out.sn;
  op[c] = from_float<T>(acc[row * acc_ld + c]);
}

// ---------------------------------------------------------------------------------------------------
// q/k normalisation:  y = lim * (x - mean_d x) / max_l ||x_l - mean_d x_l||
// stats[head] is a packed 64-bit word: (bits of max squared norm) << 32 | (0xffffffff - argmax token),
// so an atomicMax picks the largest norm and, among equals, the first token (what argmax returns).
// ---------------------------------------------------------------------------------------------------
template <typename T>
__global__ void norm_stats_kernel(View x, int d, int n, int heads, unsigned long long* stats, long long nrows) {
  long long row = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  int lane = threadIdx.x & 31;
  if (row >= nrows) return;
  int l = (int)(row % n);
  int head = (int)(row / n);
  int b = head / heads, h = head - b * heads;
  const T* xp = reinterpret_cast<const T*>(x.ptr) + (long long)b * x.sb + (long long)h * x.sh + (long long)l * x.sn;
  float s = 0.f;
  for (int c = lane; c < d; c += 32) s += to_float<T>(xp[c]);
#pragma unroll
  for (int k = 16; k > 0; k >>= 1) s += __shfl_xor_sync(0xffffffffu, s, k);
  const float mean = s / (float)d;
  float q = 0.f;
  for (int c = lane; c < d; c += 32) {
    float t = to_float<T>(xp[c]) - mean;
    q += t * t;
  }
#pragma unroll
  for (int k = 16; k > 0; k >>= 1) q += __shfl_xor_sync(0xffffffffu, q, k);
  if (lane == 0) {
    unsigned long long packed = ((unsigned long long)__float_as_uint(q) << 32) | (unsigned long long)(0xffffffffu - (unsigned)l);
    atomicMax(stats + head, packed);
  }
}

template <typename T>
__global__ void norm_apply_kernel(View x, View y, int d, int n, int heads, const unsigned long long* stats, float lim,
                                  long long nrows) {
  long long row = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  int lane = threadIdx.x & 31;
  if (row >= nrows) return;
  int l = (int)(row % n);
  int head = (int)(row / n);
  int b = head / heads, h = head - b * heads;
  const T* xp = reinterpret_cast<const T*>(x.ptr) + (long long)b * x.sb + (long long)h * x.sh + (long long)l * x.sn;
  T* yp = reinterpret_cast<T*>(const_cast<void*>(y.ptr)) + (long long)b * y.sb + (long long)h * y.sh + (long long)l * y.sn;
  float s = 0.f;
  for (int c = lane; c < d; c += 32) s += to_float<T>(xp[c]);
#pragma unroll
  for (int k = 16; k > 0; k >>= 1) s += __shfl_xor_sync(0xffffffffu, s, k);
  const float mean = s / (float)d;
  const float m = sqrtf(__uint_as_float((unsigned)(stats[head] >> 32)));
  const float sc = lim / m;
  for (int c = lane; c < d; c += 32) yp[c] = from_float<T>((to_float<T>(xp[c]) - mean) * sc);
}

// ---- 128-bit variants of the four normalisation kernels (head dim a multiple of 8, 16-byte aligned rows) ----
// LPR = d / 8 lanes share a row, every lane moves eight elements per access, a warp covers 32 / LPR rows.  Row sums
// go over the LPR lanes with shuffles; when all rows of a warp belong to one head (the usual case) the warp issues
// ONE atomic for its rows instead of one per row.
template <typename T>
__device__ __forceinline__ void load8(const T* p, float (&v)[8]);
template <>
__device__ __forceinline__ void load8<float>(const float* p, float (&v)[8]) {
  const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
  v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
template <>
__device__ __forceinline__ void load8<__nv_bfloat16>(const __nv_bfloat16* p, float (&v)[8]) {
  const uint4 r = *reinterpret_cast<const uint4*>(p);
  const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    v[2 * i] = __uint_as_float(w[i] << 16);
    v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
  }
}
template <typename T>
__device__ __forceinline__ void store8(T* p, const float (&v)[8]);
template <>
__device__ __forceinline__ void store8<float>(float* p, const float (&v)[8]) {
  *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
  *reinterpret_cast<float4*>(p + 4) = make_float4(v[4], v[5], v[6], v[7]);
}
template <>
__device__ __forceinline__ void store8<__nv_bfloat16>(__nv_bfloat16* p, const float (&v)[8]) {
  *reinterpret_cast<uint4*>(p) = make_uint4(pack2_bf16(v[0], v[1]), pack2_bf16(v[2], v[3]), pack2_bf16(v[4], v[5]), pack2_bf16(v[6], v[7]));
}
template <int LPR>
__device__ __forceinline__ float row_sum(float x) {
#pragma unroll
  for (int k = LPR / 2; k > 0; k >>= 1) x += __shfl_xor_sync(0xffffffffu, x, k);
  return x;
}
// row of this thread: blockIdx.y is the (batch, head), blockIdx.x walks the head's tokens, so a warp never spans heads
// and no division is needed
struct RowOfLane {
  int l, head, b, h, c;
  bool valid, one_head;
};
constexpr int NORM_ITERS = 8;   // row tiles per block of the two reducing kernels: one atomic per 8 x 256 threads
template <int LPR>
__device__ __forceinline__ RowOfLane row_of_lane(int n, int heads, int it = 0, int iters = 1) {
  RowOfLane r;
  const int t = (blockIdx.x * iters + it) * blockDim.x + threadIdx.x;
  r.l = t / LPR;
  r.c = (t - r.l * LPR) * 8;
  r.valid = r.l < n;
  if (!r.valid) r.l = 0;
  r.head = blockIdx.y;
  r.b = r.head / heads;
  r.h = r.head - r.b * heads;
  r.one_head = true;
  return r;
}

template <typename T, int LPR>
__global__ void norm_stats_vec_kernel(View x, int n, int heads, unsigned long long* stats, long long nrows) {
  constexpr int D = 8 * LPR;
  __shared__ unsigned long long part[8];
  unsigned long long best = 0ull;
  int head = 0;
  for (int it = 0; it < NORM_ITERS; ++it) {
    const RowOfLane r = row_of_lane<LPR>(n, heads, it, NORM_ITERS);
    head = r.head;
    float v[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = 0.f;
    if (r.valid) load8<T>(reinterpret_cast<const T*>(x.ptr) + (long long)r.b * x.sb + (long long)r.h * x.sh + (long long)r.l * x.sn + r.c, v);
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) s += v[i];
    const float mean = row_sum<LPR>(s) / (float)D;
    float q = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) q += (v[i] - mean) * (v[i] - mean);
    q = row_sum<LPR>(q);
    if (r.valid && r.c == 0) {
      const unsigned long long packed = ((unsigned long long)__float_as_uint(q) << 32) | (unsigned long long)(0xffffffffu - (unsigned)r.l);
      best = packed > best ? packed : best;
    }
  }
#pragma unroll
  for (int k = 16; k > 0; k >>= 1) {
    const unsigned long long o = __shfl_xor_sync(0xffffffffu, best, k);
    best = o > best ? o : best;
  }
  if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = best;
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int i = 1; i < (int)(blockDim.x >> 5); ++i) best = part[i] > best ? part[i] : best;
    if (best != 0ull) atomicMax(stats + head, best);
  }
}

template <typename T, int LPR>
__global__ void norm_apply_vec_kernel(View x, View y, int n, int heads, const unsigned long long* stats, float lim, long long nrows) {
  constexpr int D = 8 * LPR;
  const RowOfLane r = row_of_lane<LPR>(n, heads);
  float v[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) v[i] = 0.f;
  if (r.valid) load8<T>(reinterpret_cast<const T*>(x.ptr) + (long long)r.b * x.sb + (long long)r.h * x.sh + (long long)r.l * x.sn + r.c, v);
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) s += v[i];
  const float mean = row_sum<LPR>(s) / (float)D;
  if (!r.valid) return;
  const float sc = lim / sqrtf(__uint_as_float((unsigned)(stats[r.head] >> 32)));
#pragma unroll
  for (int i = 0; i < 8; ++i) v[i] = (v[i] - mean) * sc;
  store8<T>(reinterpret_cast<T*>(const_cast<void*>(y.ptr)) + (long long)r.b * y.sb + (long long)r.h * y.sh + (long long)r.l * y.sn + r.c, v);
}

template <typename T, int LPR>
__global__ void norm_bwd_dot_vec_kernel(View y, View dy, int n, int heads, float* scratch, long long nrows) {
  __shared__ float part[8];
  float q = 0.f;
  int head = 0;
  for (int it = 0; it < NORM_ITERS; ++it) {
    const RowOfLane r = row_of_lane<LPR>(n, heads, it, NORM_ITERS);
    head = r.head;
    if (r.valid) {
      float a[8], g[8];
      load8<T>(reinterpret_cast<const T*>(y.ptr) + (long long)r.b * y.sb + (long long)r.h * y.sh + (long long)r.l * y.sn + r.c, a);
      load8<T>(reinterpret_cast<const T*>(dy.ptr) + (long long)r.b * dy.sb + (long long)r.h * dy.sh + (long long)r.l * dy.sn + r.c, g);
#pragma unroll
      for (int i = 0; i < 8; ++i) q += a[i] * g[i];
    }
  }
#pragma unroll
  for (int k = 16; k > 0; k >>= 1) q += __shfl_xor_sync(0xffffffffu, q, k);
  if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = q;
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int i = 1; i < (int)(blockDim.x >> 5); ++i) q += part[i];
    atomicAdd(scratch + head, q);
  }
}

template <typename T, int LPR>
__global__ void norm_bwd_apply_vec_kernel(View y, View dy, View dx, int n, int heads, const unsigned long long* stats,
                                          const float* scratch, float lim, long long nrows) {
  constexpr int D = 8 * LPR;
  const RowOfLane r = row_of_lane<LPR>(n, heads);
  float a[8], g[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) a[i] = g[i] = 0.f;
  if (r.valid) {
    load8<T>(reinterpret_cast<const T*>(y.ptr) + (long long)r.b * y.sb + (long long)r.h * y.sh + (long long)r.l * y.sn + r.c, a);
    load8<T>(reinterpret_cast<const T*>(dy.ptr) + (long long)r.b * dy.sb + (long long)r.h * dy.sh + (long long)r.l * dy.sn + r.c, g);
  }
  float sg = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) sg += g[i];
  const float gmean = row_sum<LPR>(sg) / (float)D;
  if (!r.valid) return;
  const unsigned long long st = stats[r.head];
  const float m = sqrtf(__uint_as_float((unsigned)(st >> 32)));
  const int am = (int)(0xffffffffu - (unsigned)(st & 0xffffffffu));
  const float sc = lim / m;
  const float extra = (r.l == am) ? -scratch[r.head] / (lim * m) : 0.f;
  float o[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) o[i] = sc * (g[i] - gmean) + extra * a[i];
  store8<T>(reinterpret_cast<T*>(const_cast<void*>(dx.ptr)) + (long long)r.b * dx.sb + (long long)r.h * dx.sh + (long long)r.l * dx.sn + r.c, o);
}

// ---- one-launch variants: a thread-block cluster per (batch, head) ---------------------------------------------
// gridDim = (CL, batch*heads) with CL blocks of 256 threads per cluster.  Pass 1: every block walks its share of the
// head's tokens and reduces (max squared norm / sum dy.y); the CL partial results meet through distributed shared
// memory (each block reads its peers' partial after a cluster barrier, in rank order, so the sum does not depend on
// timing).  Pass 2 walks the same tokens in the opposite order and writes the result; what it reads again comes from
// L2 as far as the tensors in flight fit there.  No atomics, no zeroed scratch, one launch per direction.
// (Measured against this form on B8 H16 N4096 D64 bf16, forward + backward, 0.113 ms: blocks of 1024 threads, one
// per SM, that keep their loads in registers between the passes took 0.156 ms, since with one block per SM nothing
// overlaps the barrier between the passes; fewer resident blocks of this form, for more L2 hits, took 0.119 ms.)
template <typename T, int LPR>
__global__ void __launch_bounds__(256) norm_fused_vec_kernel(View x, View y, int n, int heads, unsigned long long* stats, float lim) {
  constexpr int D = 8 * LPR, RPI = 256 / LPR;
  namespace cgx = cooperative_groups;
  cgx::cluster_group cluster = cgx::this_cluster();
  const int cl = (int)cluster.num_blocks(), rank = (int)cluster.block_rank();
  __shared__ unsigned long long part[8];
  __shared__ unsigned long long mine;     // this block's partial: read by the peers
  __shared__ unsigned long long total;
  const int head = blockIdx.y, b = head / heads, h = head - b * heads;
  const T* xb = reinterpret_cast<const T*>(x.ptr) + (long long)b * x.sb + (long long)h * x.sh;
  T* yb = reinterpret_cast<T*>(const_cast<void*>(y.ptr)) + (long long)b * y.sb + (long long)h * y.sh;
  const int iters = (n + RPI * cl - 1) / (RPI * cl);
  const int lrow = (int)threadIdx.x / LPR, c = ((int)threadIdx.x - lrow * LPR) * 8;
  unsigned long long best = 0ull;
#pragma unroll 4
  for (int it = 0; it < iters; ++it) {
    const int l = (it * cl + rank) * RPI + lrow;
    const bool valid = l < n;
    float v[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = 0.f;
    if (valid) load8<T>(xb + (long long)l * x.sn + c, v);
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) s += v[i];
    const float mean = row_sum<LPR>(s) / (float)D;
    float q = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) q += (v[i] - mean) * (v[i] - mean);
    q = row_sum<LPR>(q);
    if (valid && c == 0) {
      const unsigned long long packed = ((unsigned long long)__float_as_uint(q) << 32) | (unsigned long long)(0xffffffffu - (unsigned)l);
      best = packed > best ? packed : best;
    }
  }
#pragma unroll
  for (int k = 16; k > 0; k >>= 1) {
    const unsigned long long o = __shfl_xor_sync(0xffffffffu, best, k);
    best = o > best ? o : best;
  }
  if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = best;
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int i = 1; i < 8; ++i) best = part[i] > best ? part[i] : best;
    mine = best;
  }
  cluster.sync();                         // every block's partial is written and every block is known to run
  if (threadIdx.x == 0) {
    unsigned long long t = 0ull;
    for (int r = 0; r < cl; ++r) {
      const unsigned long long o = *cluster.map_shared_rank(&mine, r);
      t = o > t ? o : t;
    }
    total = t;
    if (rank == 0) stats[head] = t;
  }
  __syncthreads();
  const float sc = lim / sqrtf(__uint_as_float((unsigned)(total >> 32)));
#pragma unroll 4
  for (int it = iters - 1; it >= 0; --it) {
    const int l = (it * cl + rank) * RPI + lrow;
    const bool valid = l < n;
    float v[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = 0.f;
    if (valid) load8<T>(xb + (long long)l * x.sn + c, v);
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) s += v[i];
    const float mean = row_sum<LPR>(s) / (float)D;
    if (valid) {
#pragma unroll
      for (int i = 0; i < 8; ++i) v[i] = (v[i] - mean) * sc;
      store8<T>(yb + (long long)l * y.sn + c, v);
    }
  }
  cluster.sync();                         // no block leaves while a peer may still read its partial
}

template <typename T, int LPR>
__global__ void __launch_bounds__(256) norm_bwd_fused_vec_kernel(View y, View dy, View dx, int n, int heads,
                                                                  const unsigned long long* stats, float lim) {
  constexpr int D = 8 * LPR, RPI = 256 / LPR;
  namespace cgx = cooperative_groups;
  cgx::cluster_group cluster = cgx::this_cluster();
  const int cl = (int)cluster.num_blocks(), rank = (int)cluster.block_rank();
  __shared__ float part[8];
  __shared__ float mine;
  __shared__ float total;
  const int head = blockIdx.y, b = head / heads, h = head - b * heads;
  const T* yb = reinterpret_cast<const T*>(y.ptr) + (long long)b * y.sb + (long long)h * y.sh;
  const T* gb = reinterpret_cast<const T*>(dy.ptr) + (long long)b * dy.sb + (long long)h * dy.sh;
  T* ob = reinterpret_cast<T*>(const_cast<void*>(dx.ptr)) + (long long)b * dx.sb + (long long)h * dx.sh;
  const int iters = (n + RPI * cl - 1) / (RPI * cl);
  const int lrow = (int)threadIdx.x / LPR, c = ((int)threadIdx.x - lrow * LPR) * 8;
  float q = 0.f;
#pragma unroll 4
  for (int it = 0; it < iters; ++it) {
    const int l = (it * cl + rank) * RPI + lrow;
    if (l < n) {
      float a[8], g[8];
      load8<T>(yb + (long long)l * y.sn + c, a);
      load8<T>(gb + (long long)l * dy.sn + c, g);
#pragma unroll
      for (int i = 0; i < 8; ++i) q += a[i] * g[i];
    }
  }
#pragma unroll
  for (int k = 16; k > 0; k >>= 1) q += __shfl_xor_sync(0xffffffffu, q, k);
  if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = q;
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int i = 1; i < 8; ++i) q += part[i];
    mine = q;
  }
  cluster.sync();
  if (threadIdx.x == 0) {
    float t = 0.f;
    for (int r = 0; r < cl; ++r) t += *cluster.map_shared_rank(&mine, r);
    total = t;
  }
  __syncthreads();
  const unsigned long long st = stats[head];
  const float m = sqrtf(__uint_as_float((unsigned)(st >> 32)));
  const int am = (int)(0xffffffffu - (unsigned)(st & 0xffffffffu));
  const float sc = lim / m;
  const float extra_am = -total / (lim * m);
#pragma unroll 4
  for (int it = iters - 1; it >= 0; --it) {
    const int l = (it * cl + rank) * RPI + lrow;
    const bool valid = l < n;
    float a[8], g[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) a[i] = g[i] = 0.f;
    if (valid) {
      load8<T>(yb + (long long)l * y.sn + c, a);
      load8<T>(gb + (long long)l * dy.sn + c, g);
    }
    float sg = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) sg += g[i];
    const float gmean = row_sum<LPR>(sg) / (float)D;
    if (valid) {
      const float extra = (l == am) ? extra_am : 0.f;
      float o[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) o[i] = sc * (g[i] - gmean) + extra * a[i];
      store8<T>(ob + (long long)l * dx.sn + c, o);
    }
  }
  cluster.sync();
}

// per head: scratch[head] = sum_{l,c} dy * y      (y = normalised output; x - mean = y * m / lim)
template <typename T>
__global__ void norm_bwd_dot_kernel(View y, View dy, int d, int n, int heads, float* scratch, long long nrows) {
  long long row = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  int lane = threadIdx.x & 31;
  if (row >= nrows) return;
  int l = (int)(row % n);
  int head = (int)(row / n);
  int b = head / heads, h = head - b * heads;
  const T* yp = reinterpret_cast<const T*>(y.ptr) + (long long)b * y.sb + (long long)h * y.sh + (long long)l * y.sn;
  const T* gp = reinterpret_cast<const T*>(dy.ptr) + (long long)b * dy.sb + (long long)h * dy.sh + (long long)l * dy.sn;
  float q = 0.f;
  for (int c = lane; c < d; c += 32) q += to_float<T>(gp[c]) * to_float<T>(yp[c]);
#pragma unroll
  for (int k = 16; k > 0; k >>= 1) q += __shfl_xor_sync(0xffffffffu, q, k);
  if (lane == 0) atomicAdd(scratch + head, q);
}

// dx = (lim/m) * (dy - mean_d dy)  -  [l == argmax] * scratch[head] / (lim * m) * y
// (the max flows through its arg-max token only; y rows have zero mean, so centring leaves that term as is)
template <typename T>
__global__ void norm_bwd_apply_kernel(View y, View dy, View dx, int d, int n, int heads,
                                      const unsigned long long* stats, const float* scratch, float lim,
                                      long long nrows) {
  long long row = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  int lane = threadIdx.x & 31;
  if (row >= nrows) return;
  int l = (int)(row % n);
  int head = (int)(row / n);
  int b = head / heads, h = head - b * heads;
  const T* yp = reinterpret_cast<const T*>(y.ptr) + (long long)b * y.sb + (long long)h * y.sh + (long long)l * y.sn;
  const T* gp = reinterpret_cast<const T*>(dy.ptr) + (long long)b * dy.sb + (long long)h * dy.sh + (long long)l * dy.sn;
  T* op = reinterpret_cast<T*>(const_cast<void*>(dx.ptr)) + (long long)b * dx.sb + (long long)h * dx.sh + (long long)l * dx.sn;
  const unsigned long long st = stats[head];
  const float m = sqrtf(__uint_as_float((unsigned)(st >> 32)));
  const int am = (int)(0xffffffffu - (unsigned)(st & 0xffffffffu));
  const float sc = lim / m;
  float sg = 0.f;
  for (int c = lane; c < d; c += 32) sg += to_float<T>(gp[c]);
#pragma unroll
  for (int k = 16; k > 0; k >>= 1) sg += __shfl_xor_sync(0xffffffffu, sg, k);
  const float gmean = sg / (float)d;
  const float extra = (l == am) ? -scratch[head] / (lim * m) : 0.f;
  for (int c = lane; c < d; c += 32) {
    float v = sc * (to_float<T>(gp[c]) - gmean) + extra * to_float<T>(yp[c]);
    op[c] = from_float<T>(v);
  }
}

// ---- optional key prologue and output epilogue (dead code paths of the reference, offered as options) ----
// k <- k * inv_temp + rpe[(l + nk) mod (2 nk - 1)]   (rpe may be null: scale only).  Thread = four consecutive dims
// of one key row; grid.y = batch*head.  Needs 8-byte (bf16) / 16-byte (float) aligned rows.
template <typename T>
__global__ void key_prologue_kernel(View k, const float* __restrict__ rpe, float inv_temp, int d, int nk, int heads) {
  const int vpr = d / 4;
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (long long)nk * vpr) return;
  const int l = (int)(idx / vpr), c = (int)(idx - (long long)l * vpr) * 4;
  const int head = blockIdx.y, b = head / heads, h = head - b * heads;
  T* p = reinterpret_cast<T*>(const_cast<void*>(k.ptr)) + (long long)b * k.sb + (long long)h * k.sh + (long long)l * k.sn + c;
  float4 x = load4<T>(p);
  x.x *= inv_temp; x.y *= inv_temp; x.z *= inv_temp; x.w *= inv_temp;
  if (rpe != nullptr) {
    const float4 r = *reinterpret_cast<const float4*>(rpe + (long long)((l + nk) % (2 * nk - 1)) * d + c);
    x.x += r.x; x.y += r.y; x.z += r.z; x.w += r.w;
  }
  store4<T>(p, x.x, x.y, x.z, x.w);
}

// out <- x * (1 + scale * noise)   (out may alias x).  Same thread mapping.
template <typename T>
__global__ void output_noise_kernel(View x, View noise, View out, float scale, int d, int n, int heads) {
  const int vpr = d / 4;
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (long long)n * vpr) return;
  const int l = (int)(idx / vpr), c = (int)(idx - (long long)l * vpr) * 4;
  const int head = blockIdx.y, b = head / heads, h = head - b * heads;
  auto at = [&](const View& t) {
    return reinterpret_cast<T*>(const_cast<void*>(t.ptr)) + (long long)b * t.sb + (long long)h * t.sh + (long long)l * t.sn + c;
  };
  const float4 a = load4<T>(at(x)), z = load4<T>(at(noise));
  store4<T>(at(out), a.x * (1.f + scale * z.x), a.y * (1.f + scale * z.y), a.z * (1.f + scale * z.z), a.w * (1.f + scale * z.w));
}

}  // namespace fm
