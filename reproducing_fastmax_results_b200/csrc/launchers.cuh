// Host-side launch wrappers of the templated kernels; each head dim is instantiated in its own
// translation unit (scan_d16.cu, scan_d32.cu, scan_d64.cu) so the files compile in parallel.
#pragma once
#include "common.cuh"

namespace fm {

template <int D>
cudaError_t launch_scan_d(int dtype, int mode, bool causal, const ScanParams& P, dim3 grid, cudaStream_t st);
template <int D>
cudaError_t launch_moments_d(int dtype, int src, const MomentParams& P, dim3 grid, cudaStream_t st);

extern template cudaError_t launch_scan_d<16>(int, int, bool, const ScanParams&, dim3, cudaStream_t);
extern template cudaError_t launch_scan_d<32>(int, int, bool, const ScanParams&, dim3, cudaStream_t);
extern template cudaError_t launch_scan_d<64>(int, int, bool, const ScanParams&, dim3, cudaStream_t);
extern template cudaError_t launch_moments_d<16>(int, int, const MomentParams&, dim3, cudaStream_t);
extern template cudaError_t launch_moments_d<32>(int, int, const MomentParams&, dim3, cudaStream_t);
extern template cudaError_t launch_moments_d<64>(int, int, const MomentParams&, dim3, cudaStream_t);

// Launch bookkeeping (defined with the C ABI): counts launches and, when profiling is enabled, brackets the
// launch with CUDA events on its stream so per-kernel device time can be read back.
enum KernelKind {
  KK_MOMENTS_KV = 0, KK_MOMENTS_QG, KK_STATE_SCAN, KK_SCAN_FWD, KK_SCAN_BWD_Q, KK_SCAN_BWD_KV, KK_FINALIZE,
  KK_PROLOGUE, KK_CAST, KK_NORMALIZE, KK_TC_FWD, KK_TC_BWD_Q, KK_TC_BWD_KV, KK_TC_MOMENTS, KK_P1_FWD, KK_TC_INTRA_FWD, KK_TC_INTRA_BWD, KK_TC_TRANSPOSE, KK_TC_BWD_DV, KK_DECODE, KK_KEY_PROLOGUE, KK_OUTPUT_NOISE, KK_TC_PAD, KK_COUNT
};
bool profiling_on();   // per-kernel timing is enabled: launch sequences then stay on one stream so the times do not overlap
void launch_begin(int kind, cudaStream_t st);
void launch_end(int kind, cudaStream_t st);
struct LaunchScope {
  int kind;
  cudaStream_t st;
  LaunchScope(int k, cudaStream_t s) : kind(k), st(s) { launch_begin(k, s); }
  ~LaunchScope() { launch_end(kind, st); }
};

}  // namespace fm
