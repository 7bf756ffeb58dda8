// PyTorch extension `fastmax_cuda`: a thin shim over the C ABI of include/fastmax_b200.h.
//
// It exports the two functions of the reference's binding (fastmax_cuda.cpp:17-37)
//     forwardpass(q,k,v,drop_noise,rpe_matrix,mask,dropout,normalize,temperature,a0,a1,a2,lim,p) -> o
//     backwardpass(q,k,v,o,grad_output,mask,a0,a1,a2,p) -> [gradq, gradk, gradv]
// with the reference's tensor contract ((n, b*h, d) float32 contiguous CUDA tensors, o = (nq, b*h, d+1) with
// the denominator in the last column), plus strided/bf16 entry points used by the FastMax autograd Function.
// torch is used for memory (outputs, workspace from the caching allocator), the device guard and the
// current stream; all arithmetic happens in the library's own kernels.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include <vector>

#include "../../include/fastmax_b200.h"

namespace {

#define CHECK_CUDA(x) TORCH_CHECK(x.device().is_cuda(), #x " must be a CUDA tensor")
#define CHECK_CONTIGUOUS(x) TORCH_CHECK(x.is_contiguous(), #x " must be contiguous")
#define CHECK_INPUT(x) \
  CHECK_CUDA(x);       \
  CHECK_CONTIGUOUS(x)

void check_status(int rc, const char* what) {
  if (rc == FASTMAX_OK) return;
  if (rc == FASTMAX_ERR_CUDA)
    TORCH_CHECK(false, what, ": ", fastmax_status_string(rc), " (",
                fastmax_last_cuda_error_string(), ")");
  TORCH_CHECK(false, what, ": ", fastmax_status_string(rc));
}

int dtype_of(const torch::Tensor& t) {
  if (t.scalar_type() == torch::kFloat32) return FASTMAX_F32;
  if (t.scalar_type() == torch::kBFloat16) return FASTMAX_BF16;
  TORCH_CHECK(false, "fastmax: tensors must be float32 or bfloat16, got ", t.scalar_type());
}

// PyTorch's own switch for "float32 matmuls may run in bfloat16" (torch.set_float32_matmul_precision("medium")).
// float32 callers that set it get the tensor-memory kernels: q, k, v (and the upstream gradient) are converted to
// bfloat16 for the call and the results converted back; the default ("highest") keeps the exact float32 engine.
bool float32_may_use_bf16() { return at::globalContext().float32MatmulPrecision() == at::Float32MatmulPrecision::MEDIUM; }

// (n, bh, d) contiguous -> view with batch=1
fastmax_tensor view_nbd(const torch::Tensor& t) {
  return fastmax_tensor{t.data_ptr(), (int64_t)t.numel(), t.stride(1), t.stride(0)};   // one batch: its stride is never used as an offset
}
// (b, h, n, d) with unit innermost stride
fastmax_tensor view_bhnd(const torch::Tensor& t) {
  TORCH_CHECK(t.dim() == 4, "fastmax: expected a 4-D (b,h,n,d) tensor");
  TORCH_CHECK(t.size(3) == 1 || t.stride(3) == 1, "fastmax: the head dim must be contiguous");
  return fastmax_tensor{t.data_ptr(), t.stride(0), t.stride(1), t.stride(2)};
}
fastmax_tensor view_bhn(const torch::Tensor& t) {  // float (b,h,n)
  return fastmax_tensor{t.data_ptr(), t.stride(0), t.stride(1), t.stride(2)};
}

torch::Tensor workspace(size_t bytes, const torch::Tensor& like) {
  return torch::empty({(int64_t)(bytes + 256)}, like.options().dtype(torch::kUInt8));
}
void* aligned(const torch::Tensor& ws) {
  uintptr_t p = (uintptr_t)ws.data_ptr();
  return (void*)((p + 255) / 256 * 256);
}

// ---- the reference's binding -----------------------------------------------------------------------
torch::Tensor forwardpass(torch::Tensor q, torch::Tensor k, torch::Tensor v, torch::Tensor drop_noise,
                          torch::Tensor rpe_matrix, bool mask, float dropout, bool normalize, float temperature,
                          float a0, float a1, float a2, float lim, int p) {
  CHECK_INPUT(q);
  CHECK_INPUT(k);
  CHECK_INPUT(v);
  (void)drop_noise;  // dead inputs of the reference: its dropout kernel runs with scale 0 (fwd.cu:443)
  (void)rpe_matrix;  // and its RPE add is commented out (fwd.cu:289)
  (void)dropout;
  TORCH_CHECK(q.dim() == 3 && k.dim() == 3 && v.dim() == 3, "q, k, v must be (n, b*h, d)");
  TORCH_CHECK(q.scalar_type() == torch::kFloat32 && k.scalar_type() == torch::kFloat32 &&
                  v.scalar_type() == torch::kFloat32,
              "forwardpass takes float32 tensors");
  const c10::cuda::CUDAGuard guard(q.device());
  auto stream = at::cuda::getCurrentCUDAStream().stream();
  const int nq = q.size(0), nk = k.size(0), bh = q.size(1), d = q.size(2);
  // the reference scales k by 1/temperature in place (fwd.cu:282-292) and normalises q, k in place
  // (fwd.cu:424-433); callers keep the mutated tensors for backward (model.py:29-37).
  if (normalize) {
    auto stats = torch::empty({bh}, q.options().dtype(torch::kInt64));
    fastmax_tensor qv = view_nbd(q), kv = view_nbd(k);
    check_status(fastmax_normalize_forward(1, bh, nq, d, FASTMAX_F32, lim, &qv, &qv, (uint64_t*)stats.data_ptr(), stream),
                 "fastmax normalize(q)");
    check_status(fastmax_normalize_forward(1, bh, nk, d, FASTMAX_F32, lim, &kv, &kv, (uint64_t*)stats.data_ptr(), stream),
                 "fastmax normalize(k)");
  }
  if (temperature != 1.0f) {   // k <- k / temperature in place, as apply_rpe_and_temp does (fwd.cu:282-292)
    fastmax_tensor kv = view_nbd(k);
    check_status(fastmax_key_prologue(1, bh, nk, d, FASTMAX_F32, 1.0f / temperature, &kv, nullptr, stream), "fastmax key_prologue");
  }
  auto o = torch::empty({nq, bh, d + 1}, q.options());
  fastmax_problem pb{};
  pb.batch = 1; pb.heads = bh; pb.nq = nq; pb.nk = nk; pb.d = d; pb.order = p; pb.causal = mask ? 1 : 0;
  pb.dtype = FASTMAX_F32; pb.a0 = a0; pb.a1 = a1; pb.a2 = a2; pb.inv_temperature = 1.0f;
  fastmax_forward_args a{};
  a.q = view_nbd(q); a.k = view_nbd(k); a.v = view_nbd(v);
  a.o = fastmax_tensor{o.data_ptr(), 0, o.stride(1), o.stride(0)};
  a.g = fastmax_tensor{(float*)o.data_ptr() + d, 0, o.stride(1), o.stride(0)};
  if (float32_may_use_bf16()) {
    // the same call on bfloat16 copies, if the tensor-memory kernels take it: o' comes back in bfloat16 and is widened
    // into the first d columns of o; g goes straight into column d
    auto qb = q.to(torch::kBFloat16), kb = k.to(torch::kBFloat16), vb = v.to(torch::kBFloat16);
    auto ob = torch::empty({nq, bh, d}, qb.options());
    fastmax_problem pbb = pb;
    pbb.dtype = FASTMAX_BF16;
    fastmax_forward_args ab = a;
    ab.q = view_nbd(qb); ab.k = view_nbd(kb); ab.v = view_nbd(vb); ab.o = view_nbd(ob);
    if (fastmax_forward_engine(&pbb, &ab) == 1) {
      size_t need = fastmax_forward_workspace(&pbb, &ab);
      auto ws = workspace(need, q);
      check_status(fastmax_forward(&pbb, &ab, aligned(ws), need, stream), "fastmax forwardpass (bfloat16 compute)");
      o.narrow(2, 0, d).copy_(ob);
      return o;
    }
  }
  size_t need = fastmax_forward_workspace(&pb, &a);
  auto ws = workspace(need, q);
  check_status(fastmax_forward(&pb, &a, aligned(ws), need, stream), "fastmax forwardpass");
  return o;
}

std::vector<torch::Tensor> backwardpass(torch::Tensor q, torch::Tensor k, torch::Tensor v, torch::Tensor o,
                                        torch::Tensor grad_output, bool mask, float a0, float a1, float a2, int p) {
  CHECK_INPUT(q);
  CHECK_INPUT(k);
  CHECK_INPUT(v);
  CHECK_INPUT(o);
  CHECK_INPUT(grad_output);
  const c10::cuda::CUDAGuard guard(q.device());
  auto stream = at::cuda::getCurrentCUDAStream().stream();
  const int nq = q.size(0), nk = k.size(0), bh = q.size(1), d = q.size(2);
  TORCH_CHECK(o.size(2) == d + 1, "o must be the (nq, b*h, d+1) tensor returned by forwardpass");
  auto gradq = torch::empty_like(q), gradk = torch::empty_like(k), gradv = torch::empty_like(v);
  fastmax_problem pb{};
  pb.batch = 1; pb.heads = bh; pb.nq = nq; pb.nk = nk; pb.d = d; pb.order = p; pb.causal = mask ? 1 : 0;
  pb.dtype = FASTMAX_F32; pb.a0 = a0; pb.a1 = a1; pb.a2 = a2; pb.inv_temperature = 1.0f;
  fastmax_backward_args a{};
  a.q = view_nbd(q); a.k = view_nbd(k); a.v = view_nbd(v);
  a.o = fastmax_tensor{o.data_ptr(), 0, o.stride(1), o.stride(0)};
  a.g = fastmax_tensor{(float*)o.data_ptr() + d, 0, o.stride(1), o.stride(0)};
  a.d_out = view_nbd(grad_output);
  a.dq = view_nbd(gradq); a.dk = view_nbd(gradk); a.dv = view_nbd(gradv);
  if (float32_may_use_bf16()) {
    auto qb = q.to(torch::kBFloat16), kb = k.to(torch::kBFloat16), vb = v.to(torch::kBFloat16);
    auto ob = o.narrow(2, 0, d).to(torch::kBFloat16), gb = grad_output.to(torch::kBFloat16);   // contiguous (nq, bh, d) copies
    fastmax_problem pbb = pb;
    pbb.dtype = FASTMAX_BF16;
    fastmax_forward_args fb{};   // which engine the bfloat16 form of the forward call goes to decides for the pair
    fb.q = view_nbd(qb); fb.k = view_nbd(kb); fb.v = view_nbd(vb); fb.o = view_nbd(ob); fb.g = a.g;
    if (fastmax_forward_engine(&pbb, &fb) == 1) {
      auto dqb = torch::empty_like(qb), dkb = torch::empty_like(kb), dvb = torch::empty_like(vb);
      fastmax_backward_args ab = a;
      ab.q = fb.q; ab.k = fb.k; ab.v = fb.v; ab.o = fb.o; ab.d_out = view_nbd(gb);
      ab.dq = view_nbd(dqb); ab.dk = view_nbd(dkb); ab.dv = view_nbd(dvb);
      size_t need = fastmax_backward_workspace(&pbb, &ab);
      auto ws = workspace(need, q);
      check_status(fastmax_backward(&pbb, &ab, aligned(ws), need, stream), "fastmax backwardpass (bfloat16 compute)");
      gradq.copy_(dqb); gradk.copy_(dkb); gradv.copy_(dvb);
      return {gradq, gradk, gradv};
    }
  }
  size_t need = fastmax_backward_workspace(&pb, &a);
  auto ws = workspace(need, q);
  check_status(fastmax_backward(&pb, &a, aligned(ws), need, stream), "fastmax backwardpass");
  return {gradq, gradk, gradv};
}

// ---- strided / bf16 entry points ((b, h, n, d) views, no permute copies) ----------------------------
fastmax_problem make_problem(const torch::Tensor& q, const torch::Tensor& k, bool causal, double inv_temp, double a0,
                             double a1, double a2, int64_t p, int64_t flags) {
  fastmax_problem pb{};
  pb.batch = q.size(0); pb.heads = q.size(1); pb.nq = q.size(2); pb.nk = k.size(2); pb.d = q.size(3);
  pb.order = (int)p; pb.causal = causal ? 1 : 0; pb.dtype = dtype_of(q);
  pb.a0 = (float)a0; pb.a1 = (float)a1; pb.a2 = (float)a2; pb.inv_temperature = (float)inv_temp;
  pb.flags = (int)flags;
  return pb;
}

// returns (o, g, state_out or empty); with key_moments given or want_key_moments set a fourth entry follows: the
// per-segment key moments this call read or wrote (undefined when the call has none), to be handed to the next call
// with the same k and v (fastmax_forward_args.key_moments_in / _out)
std::vector<torch::Tensor> forward(torch::Tensor q, torch::Tensor k, torch::Tensor v, bool causal, double inv_temp,
                                   double a0, double a1, double a2, int64_t p, c10::optional<torch::Tensor> state_in,
                                   bool want_state, bool want_output, int64_t flags, c10::optional<torch::Tensor> out,
                                   c10::optional<torch::Tensor> key_moments, bool want_key_moments) {
  CHECK_CUDA(q); CHECK_CUDA(k); CHECK_CUDA(v);
  TORCH_CHECK(q.dim() == 4 && k.dim() == 4 && v.dim() == 4, "q, k, v must be (b, h, n, d)");
  TORCH_CHECK(k.scalar_type() == q.scalar_type() && v.scalar_type() == q.scalar_type(), "q, k, v dtypes differ");
  const c10::cuda::CUDAGuard guard(q.device());
  auto stream = at::cuda::getCurrentCUDAStream().stream();
  fastmax_problem pb = make_problem(q, k, causal, inv_temp, a0, a1, a2, p, flags);
  fastmax_forward_args a{};
  a.q = view_bhnd(q); a.k = view_bhnd(k); a.v = view_bhnd(v);
  torch::Tensor o, g, sout;
  if (want_output) {
    // The output takes q's memory layout (a head-split view (b,n,h,d)->(b,h,n,d) stays a view of a (b,n,h*d) buffer,
    // so the caller's merge `transpose(1,2).contiguous().view(b,n,h*d)` (model.py:335) copies nothing), or goes
    // straight into the caller's `out` tensor, whatever its strides.
    if (out.has_value() && out->defined()) {
      o = *out;
      CHECK_CUDA(o);
      TORCH_CHECK(o.sizes() == q.sizes() && o.scalar_type() == q.scalar_type(), "out must have q's shape and dtype");
    } else {
      o = torch::empty_like(q);
    }
    g = torch::empty({q.size(0), q.size(1), q.size(2)}, q.options().dtype(torch::kFloat32));
    a.o = view_bhnd(o);
    a.g = view_bhn(g);
  }
  if (state_in.has_value() && state_in->defined()) {
    TORCH_CHECK(state_in->is_contiguous() && state_in->scalar_type() == torch::kFloat32 &&
                    (size_t)state_in->numel() * 4 == fastmax_state_bytes(&pb),
                "state_in has the wrong size");
    a.state_in = (const float*)state_in->data_ptr();
  }
  if (want_state) {
    sout = torch::empty({q.size(0), q.size(1), fastmax_state_rows(pb.d, pb.order), fastmax_state_ld(pb.d)},
                        q.options().dtype(torch::kFloat32));
    a.state_out = (float*)sout.data_ptr();
  }
  torch::Tensor km;
  const bool km_given = key_moments.has_value() && key_moments->defined();
  if (km_given || want_key_moments) {
    const size_t nbytes = fastmax_key_moments_bytes(&pb, &a);
    if (nbytes != 0) {
      if (km_given && key_moments->is_contiguous() && key_moments->scalar_type() == torch::kFloat32 &&
          (size_t)key_moments->numel() * 4 == nbytes) {
        km = *key_moments;
        a.key_moments_in = (const float*)km.data_ptr();
      } else {
        km = torch::empty({(int64_t)(nbytes / 4)}, q.options().dtype(torch::kFloat32));
        a.key_moments_out = (float*)km.data_ptr();
      }
    }
  }
  size_t need = fastmax_forward_workspace(&pb, &a);
  auto ws = workspace(need, q);
  check_status(fastmax_forward(&pb, &a, aligned(ws), need, stream), "fastmax forward");
  if (km_given || want_key_moments) return {o, g, sout, km};
  return {o, g, sout};
}

// returns (dq, dk, dv, dstate_out or empty)
std::vector<torch::Tensor> backward(torch::Tensor q, torch::Tensor k, torch::Tensor v, torch::Tensor o, torch::Tensor g,
                                    torch::Tensor d_out, bool causal, double inv_temp, double a0, double a1, double a2,
                                    int64_t p, c10::optional<torch::Tensor> state_in,
                                    c10::optional<torch::Tensor> dstate_in, bool want_dstate, bool want_grads,
                                    int64_t flags, c10::optional<std::vector<torch::Tensor>> grads_out,
                                    c10::optional<torch::Tensor> key_moments, c10::optional<torch::Tensor> grad_moments,
                                    bool want_grad_moments) {
  CHECK_CUDA(q); CHECK_CUDA(k); CHECK_CUDA(v); CHECK_CUDA(o); CHECK_CUDA(g); CHECK_CUDA(d_out);
  TORCH_CHECK(g.scalar_type() == torch::kFloat32, "g must be float32");
  const c10::cuda::CUDAGuard guard(q.device());
  auto stream = at::cuda::getCurrentCUDAStream().stream();
  fastmax_problem pb = make_problem(q, k, causal, inv_temp, a0, a1, a2, p, flags);
  fastmax_backward_args a{};
  a.q = view_bhnd(q); a.k = view_bhnd(k); a.v = view_bhnd(v); a.o = view_bhnd(o); a.g = view_bhn(g);
  a.d_out = view_bhnd(d_out);
  torch::Tensor dq, dk, dv, dsout;
  if (want_grads) {
    // gradients take the layouts of q, k, v (see forward), or go into the caller's tensors
    if (grads_out.has_value()) {
      TORCH_CHECK(grads_out->size() == 3, "grads_out must be [dq, dk, dv]");
      dq = (*grads_out)[0]; dk = (*grads_out)[1]; dv = (*grads_out)[2];
      TORCH_CHECK(dq.sizes() == q.sizes() && dk.sizes() == k.sizes() && dv.sizes() == v.sizes() &&
                      dq.scalar_type() == q.scalar_type() && dk.scalar_type() == q.scalar_type() &&
                      dv.scalar_type() == q.scalar_type(),
                  "grads_out must have the shapes and dtype of q, k, v");
    } else {
      dq = torch::empty_like(q);
      dk = torch::empty_like(k);
      dv = torch::empty_like(v);
    }
    a.dq = view_bhnd(dq); a.dk = view_bhnd(dk); a.dv = view_bhnd(dv);
  }
  if (state_in.has_value() && state_in->defined()) a.state_in = (const float*)state_in->data_ptr();
  if (dstate_in.has_value() && dstate_in->defined()) a.dstate_in = (const float*)dstate_in->data_ptr();
  if (want_dstate) {
    dsout = torch::empty({q.size(0), q.size(1), fastmax_state_rows(pb.d, pb.order), fastmax_state_ld(pb.d)},
                         q.options().dtype(torch::kFloat32));
    a.dstate_out = (float*)dsout.data_ptr();
  }
  if (want_grads && key_moments.has_value() && key_moments->defined()) {
    // what the forward call of the same q, k, v wrote: valid when it has the size this problem's segments give
    fastmax_forward_args fa{};
    fa.q = a.q; fa.k = a.k; fa.v = a.v; fa.o = a.o; fa.g = a.g;
    const size_t nbytes = fastmax_key_moments_bytes(&pb, &fa);
    if (nbytes != 0 && key_moments->is_contiguous() && key_moments->scalar_type() == torch::kFloat32 &&
        (size_t)key_moments->numel() * 4 == nbytes)
      a.key_moments_in = (const float*)key_moments->data_ptr();
  }
  // the per-segment gradient moments this call reads or writes (fifth entry of the result when asked for)
  torch::Tensor gm;
  const bool gm_given = grad_moments.has_value() && grad_moments->defined();
  if (gm_given || want_grad_moments) {
    const size_t nbytes = fastmax_grad_moments_bytes(&pb, &a);
    if (nbytes != 0) {
      if (gm_given && grad_moments->is_contiguous() && grad_moments->scalar_type() == torch::kFloat32 &&
          (size_t)grad_moments->numel() * 4 == nbytes) {
        gm = *grad_moments;
        a.grad_moments_in = (const float*)gm.data_ptr();
      } else {
        gm = torch::empty({(int64_t)(nbytes / 4)}, q.options().dtype(torch::kFloat32));
        a.grad_moments_out = (float*)gm.data_ptr();
      }
    }
  }
  size_t need = fastmax_backward_workspace(&pb, &a);
  auto ws = workspace(need, q);
  check_status(fastmax_backward(&pb, &a, aligned(ws), need, stream), "fastmax backward");
  if (gm_given || want_grad_moments) return {dq, dk, dv, dsout, gm};
  return {dq, dk, dv, dsout};
}

// y = lim * normalise(x); returns (y, stats)
std::vector<torch::Tensor> normalize_forward(torch::Tensor x, double lim) {
  CHECK_CUDA(x);
  const c10::cuda::CUDAGuard guard(x.device());
  auto stream = at::cuda::getCurrentCUDAStream().stream();
  auto y = torch::empty_like(x);   // keeps x's layout (see forward)
  auto stats = torch::empty({x.size(0), x.size(1)}, x.options().dtype(torch::kInt64));
  fastmax_tensor xv = view_bhnd(x), yv = view_bhnd(y);
  check_status(fastmax_normalize_forward(x.size(0), x.size(1), x.size(2), x.size(3), dtype_of(x), (float)lim, &xv, &yv,
                                         (uint64_t*)stats.data_ptr(), stream),
               "fastmax normalize_forward");
  return {y, stats};
}

torch::Tensor normalize_backward(torch::Tensor y, torch::Tensor dy, torch::Tensor stats, double lim) {
  CHECK_CUDA(y); CHECK_CUDA(dy);
  const c10::cuda::CUDAGuard guard(y.device());
  auto stream = at::cuda::getCurrentCUDAStream().stream();
  auto dx = torch::empty_like(y);
  auto scratch = torch::empty({y.size(0) * y.size(1)}, y.options().dtype(torch::kFloat32));
  fastmax_tensor yv = view_bhnd(y), gv = view_bhnd(dy), dv = view_bhnd(dx);
  check_status(fastmax_normalize_backward(y.size(0), y.size(1), y.size(2), y.size(3), dtype_of(y), (float)lim, &yv, &gv,
                                          &dv, (const uint64_t*)stats.data_ptr(), (float*)scratch.data_ptr(), stream),
               "fastmax normalize_backward");
  return dx;
}

// k <- k * inv_temp (+ rpe rows) in place; returns k
torch::Tensor key_prologue(torch::Tensor k, double inv_temp, c10::optional<torch::Tensor> rpe) {
  CHECK_CUDA(k);
  const c10::cuda::CUDAGuard guard(k.device());
  auto stream = at::cuda::getCurrentCUDAStream().stream();
  const float* rp = nullptr;
  torch::Tensor r;
  if (rpe.has_value() && rpe->defined()) {
    r = rpe->to(torch::kFloat32).contiguous();
    TORCH_CHECK(r.dim() == 2 && r.size(0) == 2 * k.size(2) - 1 && r.size(1) == k.size(3), "rpe_matrix must be (2n-1, d)");
    rp = (const float*)r.data_ptr();
  }
  fastmax_tensor kv = view_bhnd(k);
  check_status(fastmax_key_prologue(k.size(0), k.size(1), k.size(2), k.size(3), dtype_of(k), (float)inv_temp, &kv, rp, stream),
               "fastmax key_prologue");
  return k;
}

// x * (1 + scale * noise)
torch::Tensor output_noise(torch::Tensor x, torch::Tensor noise, double scale) {
  CHECK_CUDA(x); CHECK_CUDA(noise);
  TORCH_CHECK(noise.sizes() == x.sizes() && noise.scalar_type() == x.scalar_type(), "drop_noise must look like the output");
  const c10::cuda::CUDAGuard guard(x.device());
  auto stream = at::cuda::getCurrentCUDAStream().stream();
  auto out = torch::empty_like(x);
  fastmax_tensor xv = view_bhnd(x), nv = view_bhnd(noise), ov = view_bhnd(out);
  check_status(fastmax_output_noise(x.size(0), x.size(1), x.size(2), x.size(3), dtype_of(x), (float)scale, &xv, &nv, &ov, stream),
               "fastmax output_noise");
  return out;
}

// 1 when the tensor-memory kernels take a forward call on these (b, h, n, d) tensors, 0 for the CUDA-core engine
int64_t forward_engine(torch::Tensor q, torch::Tensor k, torch::Tensor v, bool causal, int64_t p) {
  TORCH_CHECK(q.dim() == 4 && k.dim() == 4 && v.dim() == 4, "q, k, v must be (b, h, n, d)");
  fastmax_problem pb = make_problem(q, k, causal, 1.0, 1.0, 1.0, 0.5, p, 0);
  fastmax_forward_args a{};
  a.q = view_bhnd(q); a.k = view_bhnd(k); a.v = view_bhnd(v);
  a.o = view_bhnd(q);   // placeholders of the right shape: nothing is read or written
  a.g = fastmax_tensor{q.data_ptr(), q.size(1) * q.size(2), q.size(2), 1};
  return fastmax_forward_engine(&pb, &a);
}

int64_t launch_count() { return (int64_t)fastmax_launch_count(); }

}  // namespace

PYBIND11_MODULE(fastmax_cuda, m) {
  // The GIL is released for the duration of every call: the work is argument checks, allocation from torch's caching
  // allocator and asynchronous launches, none of which touches Python objects.
  using release = py::call_guard<py::gil_scoped_release>;
  m.def("forwardpass", &forwardpass, "forwardpass", release());
  m.def("backwardpass", &backwardpass, "backwardpass", release());
  m.def("forward", &forward, "strided (b,h,n,d) forward: returns [o, g, state_out]", py::arg("q"), py::arg("k"), py::arg("v"),
        py::arg("causal"), py::arg("inv_temp"), py::arg("a0"), py::arg("a1"), py::arg("a2"), py::arg("p"),
        py::arg("state_in") = py::none(), py::arg("want_state") = false, py::arg("want_output") = true,
        py::arg("flags") = 0, py::arg("out") = py::none(), py::arg("key_moments") = py::none(),
        py::arg("want_key_moments") = false, release());
  m.def("backward", &backward, "strided (b,h,n,d) backward: returns [dq, dk, dv, dstate_out]", py::arg("q"), py::arg("k"),
        py::arg("v"), py::arg("o"), py::arg("g"), py::arg("d_out"), py::arg("causal"), py::arg("inv_temp"), py::arg("a0"),
        py::arg("a1"), py::arg("a2"), py::arg("p"), py::arg("state_in") = py::none(), py::arg("dstate_in") = py::none(),
        py::arg("want_dstate") = false, py::arg("want_grads") = true, py::arg("flags") = 0,
        py::arg("grads_out") = py::none(), py::arg("key_moments") = py::none(), py::arg("grad_moments") = py::none(),
        py::arg("want_grad_moments") = false, release());
  m.def("normalize_forward", &normalize_forward, "q/k normalisation: returns [y, stats]", release());
  m.def("normalize_backward", &normalize_backward, "gradient of the q/k normalisation", release());
  m.def("key_prologue", &key_prologue, "k <- k * inv_temp + rpe rows, in place", py::arg("k"), py::arg("inv_temp"),
        py::arg("rpe") = py::none(), release());
  m.def("output_noise", &output_noise, "x * (1 + scale * noise)", release());
  m.def("forward_engine", &forward_engine, "1: tensor-memory kernels, 0: CUDA-core engine, for a forward call on these tensors");
  m.def("launch_count", &launch_count, "kernel launches issued by the library so far");
  m.def("version", []() { return std::string(fastmax_version()); });
}
