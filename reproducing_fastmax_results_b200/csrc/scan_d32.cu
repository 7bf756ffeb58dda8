// Instantiates the CUDA-core Fastmax kernels for head dim 32.
#include "scan_inst.cuh"
namespace fm {
template cudaError_t launch_scan_d<32>(int, int, bool, const ScanParams&, dim3, cudaStream_t);
template cudaError_t launch_moments_d<32>(int, int, const MomentParams&, dim3, cudaStream_t);
}  // namespace fm
