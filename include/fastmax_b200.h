/*
 * fastmax_b200 -- C ABI of the B200 (sm_100a) Fastmax attention engine.
 *
 * Fastmax attention (per batch x head):
 *     s_lj = (q_l . k_j) * inv_temperature
 *     f(s) = a0 + a1 s + a2 s^2           (order 2)    or    a0 + a1 s      (order 1)
 *     A_lj = f(s_lj) for keys visible to query l, else 0
 *     g_l  = sum_j A_lj                   (denominator)
 *     o_l  = sum_j A_lj v_j / g_l
 * evaluated without the N x N matrix through running moments
 *     S = Phi(K)^T [V | 1],   Phi(x) = [x (x) x (8x8 block-symmetric packing), x, 1]
 * so cost and memory are linear in the sequence length.
 *
 * The entry points below are what a foreign-function binding of the reference's operator would bind.
 * Each one names the reference interface it replaces (paths are relative to the reference repository).
 * All pointers are DEVICE pointers unless stated otherwise; nothing here allocates device memory: the
 * caller passes a workspace whose size it asks for first.  All launches go to the given stream and
 * return without synchronising.  Every function returns a fastmax_status (0 = ok) and never throws.
 */
#ifndef FASTMAX_B200_H_
#define FASTMAX_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum {
  FASTMAX_OK = 0,
  FASTMAX_ERR_INVALID_ARGUMENT = 1,  /* null pointer, negative size, bad enum value                          */
  FASTMAX_ERR_UNSUPPORTED = 2,       /* head dim not in {16,32,64}, order not in {1,2}, nk < nq when causal   */
  FASTMAX_ERR_WORKSPACE = 3,         /* workspace missing, misaligned (256 B) or smaller than required         */
  FASTMAX_ERR_CUDA = 4,              /* a CUDA runtime call or launch failed; see fastmax_last_cuda_error()    */
  FASTMAX_ERR_DEVICE_TIMEOUT = 5,    /* a bounded device-side wait gave up (reported by fastmax_check_status)  */
  FASTMAX_ERR_MISALIGNED = 6,        /* a tensor base or stride breaks the 16-byte rule of the vector loads    */
  FASTMAX_ERR_SCRATCH_LIMIT = 7      /* fastmax_forward_static_scratch: the problem needs more than the built-in array */
} fastmax_status;

typedef enum { FASTMAX_F32 = 0, FASTMAX_BF16 = 1 } fastmax_dtype;

/* A 4-level strided view (batch, head, token, dim); the innermost dim is contiguous.
 * (n, b*h, d) tensors of the reference boundary:  batch=1, stride_h=d,   stride_n=b*h*d.
 * (b, h, n, d) tensors:                            stride_b=h*n*d, stride_h=n*d, stride_n=d.
 * (b, n, h, d) projections before the head split:  stride_b=n*h*d, stride_h=d,   stride_n=h*d.
 * Strides are in ELEMENTS. */
typedef struct {
  void* ptr;
  int64_t stride_b, stride_h, stride_n;
} fastmax_tensor;

/* Problem description shared by all entry points.  v has the same head dim as q and k
 * (the reference assumes it too: fastmax_cuda_forward.cu:385-409). */
typedef struct {
  int32_t batch, heads;    /* batch*heads independent attention problems                                */
  int32_t nq, nk;          /* query / key tokens; causal needs nk >= nq and aligns the queries to the    */
                           /* LAST nq keys (fastmax_cuda_forward.cu:161-172)                             */
  int32_t d;               /* head dim: 16, 32 or 64                                                     */
  int32_t order;           /* p of the reference: 1 or 2                                                 */
  int32_t causal;          /* `mask` of the reference                                                    */
  int32_t dtype;           /* fastmax_dtype of q, k, v, o, d_out, dq, dk, dv (accumulation is always f32) */
  float a0, a1, a2;        /* polynomial coefficients (fastmax_cuda_forward.cu:7-19)                      */
  float inv_temperature;   /* 1/temperature; the reference divides k by it in place (fwd.cu:282-292)      */
  int32_t flags;           /* FASTMAX_FLAG_*                                                              */
  int32_t reserved;
} fastmax_problem;

enum {
  FASTMAX_FLAG_NO_TENSOR_CORES = 1, /* force the CUDA-core kernels even where a tcgen05 kernel exists */
  FASTMAX_FLAG_SINGLE_STREAM = 2    /* keep every launch on the caller's stream.  By default the tensor-core path runs  */
                                    /* its independent scans side by side on up to three internal streams (created once */
                                    /* per device on first use, forked from and joined back into the caller's stream    */
                                    /* with events), which fills the partly empty last wave of each scan.               */
};

/* Moment state of one (batch, head): float32 [fastmax_state_rows][fastmax_state_ld], row-major, heads
 * contiguous.  Row r holds sum over keys of Phi(k)_r * [v | 1].  It is what a sequence-parallel caller
 * exchanges between ranks and what an incremental decoder carries between calls. */
int32_t fastmax_state_rows(int32_t d, int32_t order);
int32_t fastmax_state_ld(int32_t d);
size_t fastmax_state_bytes(const fastmax_problem* pb); /* all batch*heads states */

/* ---- forward --------------------------------------------------------------------------------------
 * Replaces forward_cuda / forwardpass (fastmax_cuda.cpp:17-24, fastmax_cuda_forward.cu:366-456) with
 * the kernels calc_unmasked / calc_masked (fwd.cu:23-280).
 *   o : same dtype as q, [.., nq, d] view; g : float32 view with stride_n in floats (dim stride unused).
 *       The reference packs both in one (nq, b*h, d+1) float tensor: pass o with stride_n=(d+1)*b*h and
 *       g.ptr = o.ptr + d with the same strides.
 *   state_in  (optional): moments of keys that precede this call's keys (same (b,h) order); causal only.
 *   state_out (optional): state_in + moments of this call's keys.
 *   If o.ptr is NULL only state_out is produced (the "chunk total" a sequence-parallel rank publishes).
 *   key_moments_out / key_moments_in (optional, both may be NULL): when the CUDA-core engine cuts the keys into
 *       segments it first sums Phi(K)^T [V | 1] per segment, one pass over k and v.  Those sums depend on k and v only
 *       (not on state_in), so a caller that comes back with the same k and v -- the forward after a state-only call
 *       of a sequence-parallel rank, the backward after the forward -- can hand them back and save that pass.
 *       key_moments_out receives them (fastmax_key_moments_bytes() bytes, float32); key_moments_in must hold what an
 *       earlier call with the same problem, k and v wrote.  No counterpart in the reference, which has no segments. */
typedef struct {
  fastmax_tensor q, k, v;
  fastmax_tensor o;
  fastmax_tensor g;
  const float* state_in;
  float* state_out;
  const float* key_moments_in;
  float* key_moments_out;
} fastmax_forward_args;

size_t fastmax_forward_workspace(const fastmax_problem* pb, const fastmax_forward_args* args);
/* Which engine takes this forward call: 1 = the tensor-memory (tcgen05) kernels, 0 = the CUDA-core engine.  A host
 * that holds float32 tensors and is allowed to compute in bfloat16 (PyTorch's float32 matmul precision "medium") asks
 * this for the bfloat16 form of its problem before it converts anything. */
int32_t fastmax_forward_engine(const fastmax_problem* pb, const fastmax_forward_args* args);
/* Size of the key_moments arrays for this problem and these arguments, or 0 when this call would neither write nor
 * read them (one segment per head, no keys, or a call the tensor-memory kernels take). */
size_t fastmax_key_moments_bytes(const fastmax_problem* pb, const fastmax_forward_args* args);
int32_t fastmax_forward(const fastmax_problem* pb, const fastmax_forward_args* args,
                        void* workspace, size_t workspace_bytes, void* cuda_stream);

/* Forward pass without a caller workspace.  No counterpart in the reference (its forward_cuda allocates with
 * torch::zeros on every call, fastmax_cuda_forward.cu:404-414).
 * For hosts that cannot allocate device memory when they call (a plugin inside a runtime that owns all of HBM,
 * an FFI binding without an allocator, a "no allocation after start-up" rule): the scratch is a fixed array of
 * FASTMAX_STATIC_SCRATCH_BYTES inside the library's device image, present on every GPU that loads the library
 * until the process exits.  Inputs and outputs are still the caller's.  Same arguments and results as
 * fastmax_forward.  A problem whose scratch exceeds the array is refused with FASTMAX_ERR_SCRATCH_LIMIT; when the
 * tensor-memory kernels' scratch (transposed and padded copies) does not fit but the CUDA-core engine's does, the call
 * runs on the latter.  The call itself performs no cudaMalloc / cudaFree.
 * The first call on each device looks the array's address up (cudaGetSymbolAddress): make that first call
 * before starting any stream capture.  All calls on a device share the one array: two calls whose kernels can
 * overlap on the GPU (different streams without an ordering between them) race; calls on one stream are safe. */
#define FASTMAX_STATIC_SCRATCH_BYTES (8u << 20)
size_t fastmax_static_scratch_bytes(void);
int32_t fastmax_forward_static_scratch(const fastmax_problem* pb, const fastmax_forward_args* args, void* cuda_stream);

/* ---- backward -------------------------------------------------------------------------------------
 * Replaces backward_cuda / backwardpass (fastmax_cuda.cpp:26-32, fastmax_cuda_backward.cu:518-613) with
 * div_grad_output, calc_gradq_*, calc_gradk_*, calc_gradv_* (bwd.cu:26-501).
 *   o, g: outputs of the forward call; d_out: upstream gradient (NOT modified, unlike bwd.cu:499).
 *   dq, dk, dv: gradients w.r.t. the q, k, v that were passed in (the temperature is inside).
 *   state_in     : same array the forward call received (moments of earlier keys), or NULL.
 *   dstate_in    : gradient moments sum Phi(q)^T dO' of LATER queries (sequence-parallel), or NULL.
 *   dstate_out   : dstate_in + this call's gradient moments, or NULL.
 *   If dq.ptr, dk.ptr and dv.ptr are all NULL only dstate_out is produced.
 *   key_moments_in (optional): what the forward call of the same problem, k and v wrote to key_moments_out.
 *   grad_moments_out / grad_moments_in (optional): the same for the per-segment sums Phi(Q)^T dO' of this call's
 *       q, o, g and d_out: the state-only call of a sequence-parallel rank writes them, its gradient call reads them
 *       (fastmax_grad_moments_bytes() bytes, float32). */
typedef struct {
  fastmax_tensor q, k, v, o, g, d_out;
  fastmax_tensor dq, dk, dv;
  const float* state_in;
  const float* dstate_in;
  float* dstate_out;
  const float* key_moments_in;
  const float* grad_moments_in;
  float* grad_moments_out;
} fastmax_backward_args;

size_t fastmax_backward_workspace(const fastmax_problem* pb, const fastmax_backward_args* args);
/* Size of the grad_moments arrays, or 0 when this call would neither write nor read them. */
size_t fastmax_grad_moments_bytes(const fastmax_problem* pb, const fastmax_backward_args* args);
int32_t fastmax_backward(const fastmax_problem* pb, const fastmax_backward_args* args,
                         void* workspace, size_t workspace_bytes, void* cuda_stream);

/* ---- incremental decoding --------------------------------------------------------------------------
 * One new token per (batch, head) against the carried moment state:
 *     state += Phi(k)^T [v | 1];   o' = Phi(q) . state (polynomial weights applied here);   o = o'[:d] / o'[d]
 * Replaces re-running the whole token window through forwardpass for every generated token, which is what the
 * reference's generation loop does (transformer/eval.py:8-32 calls the model on tokens[:, -max_tokens:] per new
 * token): the cost per token becomes one read and one write of the state, independent of the prefix length.
 *   pb: nq = nk = 1; batch, heads, d, order, dtype, a0..a2 and inv_temperature as in the forward call; `causal`
 *       is not used (the new query sees every earlier key and its own).
 *   q, k, v, o: one token per (batch, head): stride_b and stride_h are used, stride_n is not.
 *   g (optional, ptr may be NULL): float32, one value per (batch, head), strides in floats.
 *   state: float32 [batch*heads][fastmax_state_rows][fastmax_state_ld], 16-byte aligned, updated IN PLACE.  Start
 *       it from zeros, or from the state_out of a fastmax_forward call over the prompt.
 * Needs no workspace.  One launch (clusters of eight thread blocks per head). */
typedef struct {
  fastmax_tensor q, k, v;
  fastmax_tensor o;
  fastmax_tensor g;
  float* state;
} fastmax_decode_args;

int32_t fastmax_decode_step(const fastmax_problem* pb, const fastmax_decode_args* args, void* cuda_stream);

/* ---- optional key prologue and output epilogue -------------------------------------------------------
 * Two steps the reference's forward_cuda carries but never performs; offered so a caller can switch them on.
 *
 * fastmax_key_prologue replaces apply_rpe_and_temp (fastmax_cuda_forward.cu:282-292), including the line the
 * reference has commented out (:289):   k[l] <- k[l] * inv_temperature + rpe[(l + nk) mod (2 nk - 1)]   in place.
 * rpe: float32 (2 nk - 1, d) contiguous, 16-byte aligned, or NULL (scale only, which is all the reference does).
 * A caller that uses it passes inv_temperature = 1 to fastmax_forward afterwards.
 *
 * fastmax_output_noise replaces apply_dropout (fastmax_cuda_forward.cu:340-349):  out <- x * (1 + scale * noise),
 * element-wise on (batch, head, token, dim) views of the operator's dtype; out may alias x.  The reference
 * launches it with the literal scale 0.0 (:443), i.e. as a no-op. */
int32_t fastmax_key_prologue(int32_t batch, int32_t heads, int32_t nk, int32_t d, int32_t dtype, float inv_temperature,
                             const fastmax_tensor* k, const float* rpe, void* cuda_stream);
int32_t fastmax_output_noise(int32_t batch, int32_t heads, int32_t n, int32_t d, int32_t dtype, float scale,
                             const fastmax_tensor* x, const fastmax_tensor* noise, const fastmax_tensor* out,
                             void* cuda_stream);

/* ---- q/k normalisation ----------------------------------------------------------------------------
 * Replaces calc_norms / find_max / apply_norm (fastmax_cuda_forward.cu:294-338, 424-433) with the
 * normalisation the reference's oracle defines (attention_mechanisms/fastattention_einops.py:327-334):
 *     y = lim * (x - mean_d(x)) / max_tokens || x - mean_d(x) ||_2        per (batch, head), lim > 0
 * x and y may alias (in place, as the reference does).  stats: 8 bytes per (batch, head), opaque (largest
 * squared norm and its token); the backward needs it.
 * Backward: dx from dy and the normalised y (so the un-normalised x need not be kept); exact, the max
 * flowing through its arg-max token only.  dx and dy may alias.  scratch_bh: batch*heads floats. */
int32_t fastmax_normalize_forward(int32_t batch, int32_t heads, int32_t n, int32_t d, int32_t dtype,
                                  float lim, const fastmax_tensor* x, const fastmax_tensor* y,
                                  uint64_t* stats, void* cuda_stream);
int32_t fastmax_normalize_backward(int32_t batch, int32_t heads, int32_t n, int32_t d, int32_t dtype,
                                   float lim, const fastmax_tensor* y, const fastmax_tensor* dy,
                                   const fastmax_tensor* dx, const uint64_t* stats, float* scratch_bh,
                                   void* cuda_stream);

/* ---- diagnostics ---------------------------------------------------------------------------------- */
const char* fastmax_status_string(int32_t status);
int32_t fastmax_last_cuda_error(void);           /* cudaError_t of the calling thread's last failing runtime call */
const char* fastmax_last_cuda_error_string(void);
const char* fastmax_version(void);
/* Synchronous: copies back the device-side error word.  FASTMAX_ERR_DEVICE_TIMEOUT means a kernel of this
 * library gave up on a bounded wait (its outputs are then incomplete); the word is cleared by the call.
 * Call it after synchronising the stream.  No counterpart in the reference (it never checks its launches). */
int32_t fastmax_check_status(void);
/* Diagnostics for FASTMAX_ERR_DEVICE_TIMEOUT: out[i] = how many thread blocks gave up first at wait site i
 * (i = the site's code modulo 256; the codes are listed beside the waits in csrc/tc_*.cuh).  Synchronous; clears
 * the counters.  No counterpart in the reference. */
int32_t fastmax_debug_wait_histogram(int32_t* out, int32_t n);
/* Exercises the failure path of the bounded device-side waits without touching a production kernel: launches one
 * tiny thread block on `cuda_stream` that waits about a millisecond on a barrier nobody signals, gives up, and
 * reports it the way a production kernel would.  After synchronising, fastmax_check_status() returns
 * FASTMAX_ERR_DEVICE_TIMEOUT once (then FASTMAX_OK again) and fastmax_debug_wait_histogram() shows one block at
 * wait site 99.  The context stays usable; nothing faults, traps or hangs.  No counterpart in the reference. */
int32_t fastmax_debug_wait_selftest(void* cuda_stream);
/* Number of kernel launches issued by this library in this process (all entry points, all threads). */
uint64_t fastmax_launch_count(void);


/* Per-kernel device timing for benchmarks (off by default).  While enabled, every launch of the library is
 * bracketed by CUDA events on its stream.  fastmax_profile_collect waits for the recorded events, adds the
 * elapsed milliseconds and launch counts per kernel kind into ms[] / count[] (nkinds entries each) and clears
 * the records.  Kind names: fastmax_profile_kind_name(0 .. fastmax_profile_kinds()-1).  No counterpart in
 * the reference (it times with wall clocks around training, transformer/train.py:123-127). */
int32_t fastmax_profile_enable(int32_t on);
int32_t fastmax_profile_kinds(void);
const char* fastmax_profile_kind_name(int32_t kind);
int32_t fastmax_profile_collect(double* ms, uint64_t* count, int32_t nkinds);

#ifdef __cplusplus
}
#endif
#endif /* FASTMAX_B200_H_ */
