// Definitions of the launch wrappers; included by scan_dXX.cu with the head dim to instantiate.
#pragma once
#include "launchers.cuh"
#include "scan_kernels.cuh"

namespace fm {

template <typename T, int D, int MODE, bool CAUSAL>
static cudaError_t launch_scan_one(const ScanParams& P, dim3 grid, cudaStream_t st) {
  auto kern = scan_kernel<T, D, MODE, CAUSAL>;
  constexpr size_t smem = scan_smem_bytes<D, MODE>();
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return e;
  {
    LaunchScope ls(MODE == MODE_FWD ? KK_SCAN_FWD : (MODE == MODE_BWD_Q ? KK_SCAN_BWD_Q : KK_SCAN_BWD_KV), st);
    kern<<<grid, Cfg<D>::NT, smem, st>>>(P);
  }
  return cudaGetLastError();
}

template <typename T, int D>
static cudaError_t launch_scan_t(int mode, bool causal, const ScanParams& P, dim3 grid, cudaStream_t st) {
  switch (mode) {
    case MODE_FWD:
      return causal ? launch_scan_one<T, D, MODE_FWD, true>(P, grid, st)
                    : launch_scan_one<T, D, MODE_FWD, false>(P, grid, st);
    case MODE_BWD_Q:
      return causal ? launch_scan_one<T, D, MODE_BWD_Q, true>(P, grid, st)
                    : launch_scan_one<T, D, MODE_BWD_Q, false>(P, grid, st);
    case MODE_BWD_KV:
      return causal ? launch_scan_one<T, D, MODE_BWD_KV, true>(P, grid, st)
                    : launch_scan_one<T, D, MODE_BWD_KV, false>(P, grid, st);
  }
  return cudaErrorInvalidValue;
}

template <int D>
cudaError_t launch_scan_d(int dtype, int mode, bool causal, const ScanParams& P, dim3 grid, cudaStream_t st) {
  return dtype == 0 ? launch_scan_t<float, D>(mode, causal, P, grid, st)
                    : launch_scan_t<__nv_bfloat16, D>(mode, causal, P, grid, st);
}

template <typename T, int D, int SRC>
static cudaError_t launch_moments_one(const MomentParams& P, dim3 grid, cudaStream_t st) {
  auto kern = moments_kernel<T, D, SRC>;
  constexpr size_t smem = moments_smem_bytes<D>();
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return e;
  {
    LaunchScope ls(SRC == MOM_KV ? KK_MOMENTS_KV : KK_MOMENTS_QG, st);
    kern<<<grid, Cfg<D>::NT, smem, st>>>(P);
  }
  return cudaGetLastError();
}

template <int D>
cudaError_t launch_moments_d(int dtype, int src, const MomentParams& P, dim3 grid, cudaStream_t st) {
  if (dtype == 0)
    return src == MOM_KV ? launch_moments_one<float, D, MOM_KV>(P, grid, st)
                         : launch_moments_one<float, D, MOM_QG>(P, grid, st);
  return src == MOM_KV ? launch_moments_one<__nv_bfloat16, D, MOM_KV>(P, grid, st)
                       : launch_moments_one<__nv_bfloat16, D, MOM_QG>(P, grid, st);
}

}  // namespace fm
