// Entry points of the tcgen05 / TMA kernels.  Each returns FASTMAX_TC_NOT_HANDLED when the problem is
// outside what the tensor-core kernels cover, and the caller then runs the CUDA-core engine.
#pragma once
#include <cuda_runtime.h>
#include <stddef.h>

#include "../../include/fastmax_b200.h"

namespace fm {
enum { FASTMAX_TC_NOT_HANDLED = -1 };
size_t tc_forward_workspace(const fastmax_problem* pb, const fastmax_forward_args* a);
size_t tc_backward_workspace(const fastmax_problem* pb, const fastmax_backward_args* a);
// Whether the tensor-memory kernels take the call (they may still hand it back at run time when the copy engine
// cannot describe a tensor's layout; the CUDA-core engine then runs it).
bool tc_takes_forward(const fastmax_problem* pb, const fastmax_forward_args* a);
bool tc_takes_backward(const fastmax_problem* pb, const fastmax_backward_args* a);
// Bytes of the per-segment moment arrays a segmented tensor-memory call reads or writes (0: the call is not segmented).
size_t tc_key_moments_bytes(const fastmax_problem* pb, const fastmax_forward_args* a);
size_t tc_grad_moments_bytes(const fastmax_problem* pb, const fastmax_backward_args* a);
int tc_forward(const fastmax_problem* pb, const fastmax_forward_args* a, void* ws, size_t ws_bytes, cudaStream_t st);
int tc_backward(const fastmax_problem* pb, const fastmax_backward_args* a, void* ws, size_t ws_bytes, cudaStream_t st);
// Reads (and clears) the device-side error word the bounded waits of the tensor-core kernels set.
int tc_device_status(int* out);
// Copies (and clears) the per-wait-site give-up counters (index = error code & 255).
int tc_wait_histogram(int* out, int n);
// Launches the test-only kernel that lets a bounded wait of `cycles` SM clocks run out and records wait site `code`.
int tc_wait_selftest(long long cycles, int code, cudaStream_t st);

// shared with the C-ABI translation unit
int report_cuda_error(cudaError_t e);  // remembers e for fastmax_last_cuda_error(), returns FASTMAX_ERR_CUDA
// acc: [batch*heads][n][acc_ld] float32 (acc_ld <= 0: dense, acc_ld = d)
int launch_cast_out(const fastmax_problem* pb, const float* acc, int n, const fastmax_tensor* out, cudaStream_t st, int acc_ld = 0);
int launch_finalize_fwd(const fastmax_problem* pb, const fastmax_forward_args* a, const float* oacc, cudaStream_t st);
}  // namespace fm
