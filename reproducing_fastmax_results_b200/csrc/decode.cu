// fastmax_decode_step: one new token per (batch, head) against the carried moment state.
//
//     S   <-  S + Phi(k)^T [v | 1]                (un-weighted sums, the exchange format of the forward call)
//     o'  =   sum_r  w_r Phi(q)_r S[r, :]          (w_r = a2/T^2 (x2 off the block diagonal), a1/T, a0)
//     o   =   o'[:D] / o'[D],   g = o'[D]
//
// The state of a head (D=64, order 2: 2369 rows x 68 floats = 644 KB) is read once and written once; nothing
// else moves, so the kernel is bound by HBM: 2 x state bytes per step.  A cluster of 1, 2, 4 or 8 thread blocks
// shares one head (the host picks the smallest cluster that still gives the GPU about a thousand blocks: few, long
// blocks stream best, but there must be enough of them to fill 148 SMs several times over), each block streams its
// share of the rows with 128-bit accesses (thread = one float4 column of a row, four rows in flight), the partial
// outputs meet in the first block's shared memory over the cluster's distributed shared memory, and that block
// divides and stores the token's output.
#include <cooperative_groups.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "../../include/fastmax_b200.h"
#include "common.cuh"
#include "launchers.cuh"

namespace cg = cooperative_groups;

namespace fm {

int report_cuda_error(cudaError_t e);

namespace dec {

constexpr int MAX_CL = 8;   // largest cluster: thread blocks that share one head
constexpr int RG = 16;      // rows a block works on at a time
constexpr int UNROLL = 4;   // rows a thread has in flight

struct DecodeParams {
  View q, k, v, o, g;
  float* state;
  int heads, rows;
  float c0, c1, c2;
};

template <typename T>
__device__ __forceinline__ float to_f(T x);
template <>
__device__ __forceinline__ float to_f<float>(float x) { return x; }
template <>
__device__ __forceinline__ float to_f<__nv_bfloat16>(__nv_bfloat16 x) { return __bfloat162float(x); }
template <typename T>
__device__ __forceinline__ T from_f(float x);
template <>
__device__ __forceinline__ float from_f<float>(float x) { return x; }
template <>
__device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float x) { return __float2bfloat16_rn(x); }

template <typename T, int D, int ORDER>
__global__ void __launch_bounds__(((D + 4) / 4) * RG)
decode_step_kernel(const DecodeParams P) {
  using G = Geo<D>;
  constexpr int C4 = (D + 4) / 4;          // float4 columns of a state row
  constexpr int NT = C4 * RG;
  constexpr int PAIR_ROWS = ORDER == 2 ? 64 * G::NPAIRS : 0;

  __shared__ float sq[D], sk[D];
  __shared__ float4 sv[C4];
  __shared__ float4 red[RG][C4];
  __shared__ float4 part[MAX_CL][C4];      // block 0 of the cluster: one row per block
  __shared__ unsigned char tab_a[G::NPAIRS], tab_b[G::NPAIRS];

  cg::cluster_group cluster = cg::this_cluster();
  const int tid = threadIdx.x;
  const int rank = (int)cluster.block_rank();
  const int CL = (int)gridDim.x;            // the cluster spans the grid's x extent
  const int head = blockIdx.y;
  const int bi = head / P.heads, hi = head - bi * P.heads;

  if (tid < D) {
    const long long off_q = (long long)bi * P.q.sb + (long long)hi * P.q.sh;
    const long long off_k = (long long)bi * P.k.sb + (long long)hi * P.k.sh;
    sq[tid] = to_f<T>(reinterpret_cast<const T*>(P.q.ptr)[off_q + tid]);
    sk[tid] = to_f<T>(reinterpret_cast<const T*>(P.k.ptr)[off_k + tid]);
  }
  if (tid < C4) {
    const T* vp = reinterpret_cast<const T*>(P.v.ptr) + (long long)bi * P.v.sb + (long long)hi * P.v.sh;
    float4 x = make_float4(1.f, 0.f, 0.f, 0.f);   // the ones column of [v | 1] and the padding
    if (tid < D / 4) x = make_float4(to_f<T>(vp[4 * tid]), to_f<T>(vp[4 * tid + 1]), to_f<T>(vp[4 * tid + 2]), to_f<T>(vp[4 * tid + 3]));
    sv[tid] = x;
  }
  if (ORDER == 2 && tid < G::NPAIRS) {
    int a, b;
    pair_decode(tid, G::NB, a, b);
    tab_a[tid] = (unsigned char)a;
    tab_b[tid] = (unsigned char)b;
  }
  __syncthreads();

  const int c4 = tid % C4, rg = tid / C4;
  const int rows_per = (P.rows + CL - 1) / CL;
  const int r0 = rank * rows_per;
  const int r1 = min(P.rows, r0 + rows_per);
  const float4 v4 = sv[c4];
  float4* base = reinterpret_cast<float4*>(P.state) + (long long)head * P.rows * C4 + c4;
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);

  // feature r of k (un-weighted) and of q (weighted)
  auto feature = [&](int r, float& pk, float& pq) {
    if (ORDER == 2 && r < PAIR_ROWS) {
      const int u = r >> 6, i = r & 63;
      const int a = tab_a[u], b = tab_b[u];
      const int m = 8 * a + (i >> 3), n = 8 * b + (i & 7);
      pk = sk[m] * sk[n];
      pq = sq[m] * sq[n] * (a == b ? P.c2 : 2.f * P.c2);
    } else {
      const int m = r - PAIR_ROWS;
      if (m < D) {
        pk = sk[m];
        pq = sq[m] * P.c1;
      } else {
        pk = 1.f;
        pq = P.c0;
      }
    }
  };

  for (int r = r0 + rg; r < r1; r += RG * UNROLL) {
    float4 s[UNROLL];
    float pk[UNROLL], pq[UNROLL];
#pragma unroll
    for (int j = 0; j < UNROLL; ++j) {
      const int rr = r + j * RG;
      if (rr < r1) {
        s[j] = __ldcs(base + (long long)rr * C4);
        feature(rr, pk[j], pq[j]);
      }
    }
#pragma unroll
    for (int j = 0; j < UNROLL; ++j) {
      const int rr = r + j * RG;
      if (rr < r1) {
        s[j].x = fmaf(pk[j], v4.x, s[j].x);
        s[j].y = fmaf(pk[j], v4.y, s[j].y);
        s[j].z = fmaf(pk[j], v4.z, s[j].z);
        s[j].w = fmaf(pk[j], v4.w, s[j].w);
        __stcs(base + (long long)rr * C4, s[j]);
        acc.x = fmaf(pq[j], s[j].x, acc.x);
        acc.y = fmaf(pq[j], s[j].y, acc.y);
        acc.z = fmaf(pq[j], s[j].z, acc.z);
        acc.w = fmaf(pq[j], s[j].w, acc.w);
      }
    }
  }

  red[rg][c4] = acc;
  // Every block of the cluster must be known to have started before another block writes into its shared memory;
  // this barrier also orders the `red` rows for the reduction below (it is a superset of __syncthreads).
  cluster.sync();
  if (tid < C4) {
    float4 t = red[0][tid];
#pragma unroll
    for (int j = 1; j < RG; ++j) {
      const float4 x = red[j][tid];
      t.x += x.x, t.y += x.y, t.z += x.z, t.w += x.w;
    }
    float4* dst = cluster.map_shared_rank(&part[rank][tid], 0);
    *dst = t;
  }
  cluster.sync();
  if (rank != 0) return;

  float* fin = reinterpret_cast<float*>(&red[0][0]);   // [C4 * 4]: o'[0..D-1], g, padding
  if (tid < C4) {
    float4 t = part[0][tid];
    for (int j = 1; j < CL; ++j) {
      const float4 x = part[j][tid];
      t.x += x.x, t.y += x.y, t.z += x.z, t.w += x.w;
    }
    reinterpret_cast<float4*>(fin)[tid] = t;
  }
  __syncthreads();
  const float gsum = fin[D];
  if (tid < D) {
    T* op = reinterpret_cast<T*>(const_cast<void*>(P.o.ptr)) + (long long)bi * P.o.sb + (long long)hi * P.o.sh;
    op[tid] = from_f<T>(fin[tid] / gsum);
  }
  if (tid == 0 && P.g.ptr != nullptr) {
    float* gp = reinterpret_cast<float*>(const_cast<void*>(P.g.ptr)) + (long long)bi * P.g.sb + (long long)hi * P.g.sh;
    *gp = gsum;
  }
}

template <typename T, int D>
static cudaError_t launch(int order, const DecodeParams& P, int bh, cudaStream_t st) {
  constexpr int NT = ((D + 4) / 4) * RG;
  int cl = 1;
  while (cl < MAX_CL && (long long)cl * bh < 1024) cl *= 2;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(cl, bh);
  cfg.blockDim = dim3(NT);
  cfg.dynamicSmemBytes = 0;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = cl;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (order == 2) return cudaLaunchKernelEx(&cfg, decode_step_kernel<T, D, 2>, P);
  return cudaLaunchKernelEx(&cfg, decode_step_kernel<T, D, 1>, P);
}

template <typename T>
static cudaError_t launch_d(int d, int order, const DecodeParams& P, int bh, cudaStream_t st) {
  switch (d) {
    case 16: return launch<T, 16>(order, P, bh, st);
    case 32: return launch<T, 32>(order, P, bh, st);
    default: return launch<T, 64>(order, P, bh, st);
  }
}

}  // namespace dec
}  // namespace fm

extern "C" int32_t fastmax_decode_step(const fastmax_problem* pb, const fastmax_decode_args* a, void* cuda_stream) {
  using namespace fm;
  if (!pb || !a) return FASTMAX_ERR_INVALID_ARGUMENT;
  if (pb->batch <= 0 || pb->heads <= 0) return FASTMAX_ERR_INVALID_ARGUMENT;
  if (pb->dtype != FASTMAX_F32 && pb->dtype != FASTMAX_BF16) return FASTMAX_ERR_INVALID_ARGUMENT;
  if (pb->d != 16 && pb->d != 32 && pb->d != 64) return FASTMAX_ERR_UNSUPPORTED;
  if (pb->order != 1 && pb->order != 2) return FASTMAX_ERR_UNSUPPORTED;
  if (pb->nq != 1 || pb->nk != 1) return FASTMAX_ERR_UNSUPPORTED;
  if ((long long)pb->batch * pb->heads > 65535) return FASTMAX_ERR_UNSUPPORTED;
  if (!a->q.ptr || !a->k.ptr || !a->v.ptr || !a->o.ptr || !a->state) return FASTMAX_ERR_INVALID_ARGUMENT;
  if (reinterpret_cast<uintptr_t>(a->state) % 16 != 0) return FASTMAX_ERR_MISALIGNED;
  dec::DecodeParams P;
  P.q = View{a->q.ptr, a->q.stride_b, a->q.stride_h, a->q.stride_n};
  P.k = View{a->k.ptr, a->k.stride_b, a->k.stride_h, a->k.stride_n};
  P.v = View{a->v.ptr, a->v.stride_b, a->v.stride_h, a->v.stride_n};
  P.o = View{a->o.ptr, a->o.stride_b, a->o.stride_h, a->o.stride_n};
  P.g = View{a->g.ptr, a->g.stride_b, a->g.stride_h, a->g.stride_n};
  P.state = a->state;
  P.heads = pb->heads;
  P.rows = state_rows(pb->d, pb->order);
  P.c0 = pb->a0;
  P.c1 = pb->a1 * pb->inv_temperature;
  P.c2 = pb->order == 2 ? pb->a2 * pb->inv_temperature * pb->inv_temperature : 0.f;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(cuda_stream);
  const int bh = pb->batch * pb->heads;
  cudaError_t e;
  {
    LaunchScope ls(KK_DECODE, st);
    e = pb->dtype == FASTMAX_BF16 ? dec::launch_d<__nv_bfloat16>(pb->d, pb->order, P, bh, st)
                                  : dec::launch_d<float>(pb->d, pb->order, P, bh, st);
  }
  return e == cudaSuccess ? FASTMAX_OK : report_cuda_error(e);
}
