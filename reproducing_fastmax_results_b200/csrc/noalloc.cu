// fastmax_forward_static_scratch: the forward pass for hosts that cannot hand the library a workspace.
//
// Some callers have no way to allocate device memory at the moment they need attention computed: a plugin
// running under a serving runtime that has already given every byte of HBM to its own pools, a host bound
// through an FFI that exposes no allocator, or code that runs after start-up under a rule of "no cudaMalloc
// on the request path".  For them the scratch the forward pass needs (the fp32 numerator/denominator
// accumulator and, for segmented scans, the per-segment states) lives in a fixed array inside this library's
// device image.  Every GPU that loads the library carries the array (FASTMAX_STATIC_SCRATCH_BYTES) until the
// process exits, which is why it is kept modest: problems that need more are refused.
#include <cuda_runtime.h>

#include <mutex>

#include "../../include/fastmax_b200.h"

namespace {

constexpr size_t kScratchBytes = FASTMAX_STATIC_SCRATCH_BYTES;
static __device__ __align__(256) unsigned char g_static_scratch[kScratchBytes];

// In host code `g_static_scratch` is only a handle for the runtime, not a device address.  The address a
// kernel can use comes from cudaGetSymbolAddress, asked once per device with that device current.
constexpr int kMaxDevices = 64;
void* g_scratch_addr[kMaxDevices] = {nullptr};
std::mutex g_mu;

int scratch_for_current_device(void** out) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return FASTMAX_ERR_CUDA;
  std::lock_guard<std::mutex> lk(g_mu);
  if (g_scratch_addr[dev] == nullptr) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_static_scratch) != cudaSuccess || p == nullptr) return FASTMAX_ERR_CUDA;
    g_scratch_addr[dev] = p;
  }
  *out = g_scratch_addr[dev];
  return FASTMAX_OK;
}

}  // namespace

extern "C" {

size_t fastmax_static_scratch_bytes(void) { return kScratchBytes; }

int32_t fastmax_forward_static_scratch(const fastmax_problem* pb, const fastmax_forward_args* args, void* cuda_stream) {
  if (!pb || !args) return FASTMAX_ERR_INVALID_ARGUMENT;
  fastmax_problem one = *pb;
  one.flags |= FASTMAX_FLAG_SINGLE_STREAM;
  size_t need = fastmax_forward_workspace(&one, args);
  if (need == 0) return fastmax_forward(pb, args, nullptr, 0, cuda_stream);  // reports what is wrong with the problem
  if (need > kScratchBytes) {
    // the tensor-memory kernels want more scratch than the CUDA-core engine (transposed and padded copies): a problem
    // that only fits without them runs there
    one.flags |= FASTMAX_FLAG_NO_TENSOR_CORES;
    need = fastmax_forward_workspace(&one, args);
    if (need == 0 || need > kScratchBytes) return FASTMAX_ERR_SCRATCH_LIMIT;
  }
  void* scratch = nullptr;
  const int rc = scratch_for_current_device(&scratch);
  if (rc != FASTMAX_OK) return rc;
  // The launch sequence zeroes the accumulators it sums into and overwrites the rest, so what the previous
  // call left in the array does not matter.  Everything stays on the caller's stream: this entry point creates
  // nothing, not even the internal side streams the ordinary call may set up on its first use.
  return fastmax_forward(&one, args, scratch, kScratchBytes, cuda_stream);
}

}  // extern "C"
