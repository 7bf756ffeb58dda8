"""Python side of the Fastmax operator, mirroring the reference's interface for this path.

  FASTMultiHeadAttention_Function   the reference's autograd.Function, line for line in behaviour
                                    (transformer/model.py:14-74): permutes to (n, b*h, d), calls
                                    fastmax_cuda.forwardpass / backwardpass, returns gradk / temperature.
  FastMax                           same signature, but works on the (b, h, n, d) tensors in place (no permute
                                    copies), accepts bfloat16, and differentiates through the q/k normalisation
                                    exactly (the reference's backward ignores it).
  FASTMultiHeadAttention, fastmax_custom, rpe_matrix_creator   as transformer/model.py:208-248.
"""
from __future__ import annotations

import math

import torch


def _ext():
    from . import load_extension

    return load_extension()


def _alert_not_deterministic(what):
    """PyTorch's convention for operators whose results can differ in the last bits from run to run: under
    torch.use_deterministic_algorithms(True) they raise, with warn_only=True they warn.  The scans sum the partial
    results of their feature slices with floating-point reduce-adds whose order depends on timing."""
    if not torch.are_deterministic_algorithms_enabled():
        return
    msg = (f"{what} does not have a deterministic implementation, but you set 'torch.use_deterministic_algorithms(True)'. "
           "Its feature slices add their partial sums in an order that depends on timing, so the low bits of the "
           "output and of the gradients can differ between runs. You can turn off determinism just for this operation, "
           "or use 'torch.use_deterministic_algorithms(True, warn_only=True)'.")
    if torch.is_deterministic_algorithms_warn_only_enabled():
        import warnings

        warnings.warn(msg, stacklevel=3)
    else:
        raise RuntimeError(msg)


class FASTMultiHeadAttention_Function(torch.autograd.Function):
    """Behavioural twin of transformer/model.py:14-74 on top of the new `fastmax_cuda` extension."""

    @staticmethod
    def forward(ctx, q, k, v, drop_noise, rpe_matrix=None, mask=False, dropout=0.0, normalize=False,
                temperature=1.0, a0=1.0, a1=1.0, a2=0.5, lim=1.0, p=2):
        _alert_not_deterministic("FASTMultiHeadAttention_Function")
        ext = _ext()
        b = 0
        if q.dim() == 4:
            b = q.shape[0]
            q = q.reshape(q.shape[0] * q.shape[1], q.shape[2], q.shape[3])
            k = k.reshape(k.shape[0] * k.shape[1], k.shape[2], k.shape[3])
            v = v.reshape(v.shape[0] * v.shape[1], v.shape[2], v.shape[3])
            drop_noise = drop_noise.reshape(-1, drop_noise.shape[2], drop_noise.shape[3])
        elif q.dim() != 3:
            print("q, k, and v should be either 3 or 4 dimensional tensors. If 3D: (b*h,n,d), if 4D: (b,h,n,d).")
        if rpe_matrix is None:
            print("Relative Positional Encoding must be given. Send a 2*n-1 by d matrix of all zeros if you don't want to use RPE.")
        # clone() guarantees private copies: forwardpass scales / normalises q and k in place (model.py:29-32)
        q = q.permute(1, 0, 2).contiguous().clone()
        k = k.permute(1, 0, 2).contiguous().clone()
        v = v.permute(1, 0, 2).contiguous()
        drop_noise = drop_noise.permute(1, 0, 2).contiguous()
        o = ext.forwardpass(q, k, v, drop_noise, rpe_matrix, mask, dropout, normalize, temperature, a0, a1, a2, lim, p)
        ctx.save_for_backward(q, k, v, o)
        ctx.mask, ctx.p, ctx.b, ctx.t = mask, p, b, temperature
        ctx.a0, ctx.a1, ctx.a2 = a0, a1, a2
        o = o[:, :, : q.shape[2]].permute(1, 0, 2).contiguous()
        if b != 0:
            o = o.reshape(b, o.shape[0] // b, o.shape[1], o.shape[2])
        return o

    @staticmethod
    def backward(ctx, grad_output):
        ext = _ext()
        q, k, v, o = ctx.saved_tensors
        b = ctx.b
        if b != 0:
            grad_output = grad_output.reshape(-1, grad_output.shape[2], grad_output.shape[3])
        grad_output = grad_output.permute(1, 0, 2).contiguous()
        gradq, gradk, gradv = ext.backwardpass(q, k, v, o, grad_output, ctx.mask, ctx.a0, ctx.a1, ctx.a2, ctx.p)
        gradq = gradq.permute(1, 0, 2).contiguous()
        gradk = gradk.permute(1, 0, 2).contiguous()
        gradv = gradv.permute(1, 0, 2).contiguous()
        if b != 0:
            gradq = gradq.reshape(b, gradq.shape[0] // b, gradq.shape[1], gradq.shape[2])
            gradk = gradk.reshape(b, gradk.shape[0] // b, gradk.shape[1], gradk.shape[2])
            gradv = gradv.reshape(b, gradv.shape[0] // b, gradv.shape[1], gradv.shape[2])
        return gradq, gradk / ctx.t, gradv, None, None, None, None, None, None, None, None, None, None, None


class FastMax(torch.autograd.Function):
    """Fastmax attention with the reference's operator signature, on (b, h, n, d) or (b*h, n, d) tensors.

    q, k, v may be float32 or bfloat16 and need not be contiguous (only the head dim must have stride 1), so
    the transposed views produced by a head split are consumed without a copy.  `drop_noise`, `rpe_matrix`
    and `dropout` are accepted and, by default, ignored, which is what the reference's kernels do with them
    (fastmax_cuda_forward.cu:289, 443).  Two trailing switches turn the dead code paths of the reference on:
    `apply_rpe` adds rpe_matrix[(l + n) mod (2n - 1)] to key l after the temperature scaling (the line commented out
    at fastmax_cuda_forward.cu:289) and `noise_dropout` multiplies the output by 1 + dropout * drop_noise (the
    reference's apply_dropout, :340-349, which it launches with scale 0).  With `normalize` the op computes
    lim * (x - mean_d x) / max_token ||x - mean_d x|| for q and k (fastattention_einops.py:327-334) and its
    exact gradient.  Scores are (q . k) / temperature.
    """

    @staticmethod
    def forward(ctx, q, k, v, drop_noise=None, rpe_matrix=None, mask=False, dropout=0.0, normalize=False,
                temperature=1.0, a0=1.0, a1=1.0, a2=0.5, lim=1.0, p=2, apply_rpe=False, noise_dropout=False):
        _alert_not_deterministic("FastMax (fastmax_custom)")
        ext = _ext()
        three_d = q.dim() == 3
        if three_d:
            q, k, v = q.unsqueeze(0), k.unsqueeze(0), v.unsqueeze(0)
            drop_noise = drop_noise.unsqueeze(0) if (noise_dropout and drop_noise is not None) else drop_noise
        elif q.dim() != 4:
            raise ValueError("q, k, v must be (b, h, n, d) or (b*h, n, d)")
        stats_q = stats_k = None
        if normalize:
            q, stats_q = ext.normalize_forward(q, float(lim))
            k, stats_k = ext.normalize_forward(k, float(lim))
        inv_t = 1.0 / float(temperature)
        k_scale = 1.0     # dk of the operator is w.r.t. the k it saw: times k_scale gives the gradient of the input k
        k_op = k
        if apply_rpe:
            if rpe_matrix is None:
                raise ValueError("apply_rpe needs rpe_matrix, a (2n-1, d) tensor")
            k_op = ext.key_prologue(k.clone(), inv_t, rpe_matrix)   # k / temperature + rpe rows, on a private copy
            k_scale, inv_t = inv_t, 1.0
        # float32 tensors under torch.set_float32_matmul_precision("medium") (PyTorch's switch for bfloat16 inside
        # float32 matmuls): the attention itself runs on bfloat16 copies when that puts it on the tensor-memory
        # kernels; the normalisation above, its gradient and everything the caller sees stay float32
        qc, kc, vc = q, k_op, v
        if q.dtype == torch.float32 and torch.get_float32_matmul_precision() == "medium":
            qb, kb, vb = q.bfloat16(), k_op.bfloat16(), v.bfloat16()
            if ext.forward_engine(qb, kb, vb, bool(mask), int(p)) == 1:
                qc, kc, vc = qb, kb, vb
        cast = qc is not q
        # the fourth entry: per-segment key moments when the call computed some (long sequences with few heads on the
        # CUDA-core engine); the backward reads them instead of passing over k and v again
        o, g, _, kmom = ext.forward(qc, kc, vc, bool(mask), inv_t, float(a0), float(a1), float(a2), int(p), None, False, True, 0,
                                    None, None, True)
        noise = None
        out = o
        if noise_dropout and float(dropout) != 0.0:
            if drop_noise is None:
                raise ValueError("noise_dropout needs drop_noise, a tensor shaped like q")
            noise = drop_noise.to(o.dtype)
            out = ext.output_noise(o, noise, float(dropout))
        if cast:
            out = out.float()
        extra = ([stats_q, stats_k] if normalize else []) + ([k] if (normalize and apply_rpe) else [])
        extra += [q, k] if (normalize and cast) else []   # the float32 normalised tensors, for the normalisation's gradient
        ctx.save_for_backward(qc, kc, vc, o, g, *extra, *([noise] if noise is not None else []))
        ctx.cast = cast
        ctx.cfg = (bool(mask), inv_t, float(a0), float(a1), float(a2), int(p), bool(normalize), float(lim), three_d,
                   k_scale, float(dropout) if noise is not None else 0.0, bool(apply_rpe))
        ctx.key_moments = kmom   # not an input or output of the function: kept on the context
        return out.squeeze(0) if three_d else out

    @staticmethod
    def backward(ctx, grad_output):
        ext = _ext()
        mask, inv_t, a0, a1, a2, p, normalize, lim, three_d, k_scale, noise_scale, apply_rpe = ctx.cfg
        q, k, v, o, g = ctx.saved_tensors[:5]
        if three_d:
            grad_output = grad_output.unsqueeze(0)
        if grad_output.stride(-1) != 1:
            grad_output = grad_output.contiguous()
        if ctx.cast:               # the attention ran on bfloat16 copies (float32 matmul precision "medium")
            grad_output = grad_output.to(o.dtype)
        if noise_scale != 0.0:     # out = o * (1 + s * noise)  ->  d o = d out * (1 + s * noise)
            grad_output = ext.output_noise(grad_output, ctx.saved_tensors[-1], noise_scale)
        dq, dk, dv, _ = ext.backward(q, k, v, o, g, grad_output, mask, inv_t, a0, a1, a2, p, None, None, False, True, 0,
                                     None, ctx.key_moments)
        if ctx.cast:
            dq, dk, dv = dq.float(), dk.float(), dv.float()
        if k_scale != 1.0:         # the operator saw k / temperature + rpe rows
            dk = ext.key_prologue(dk, k_scale, None)
        if normalize:
            stats_q, stats_k = ctx.saved_tensors[5:7]
            nxt = 8 if apply_rpe else 7
            yq, yk = (ctx.saved_tensors[nxt], ctx.saved_tensors[nxt + 1]) if ctx.cast else (q, ctx.saved_tensors[7] if apply_rpe else k)
            dq = ext.normalize_backward(yq, dq, stats_q, lim)
            dk = ext.normalize_backward(yk, dk, stats_k, lim)
        if three_d:
            dq, dk, dv = dq.squeeze(0), dk.squeeze(0), dv.squeeze(0)
        return dq, dk, dv, None, None, None, None, None, None, None, None, None, None, None, None, None


def fastmax(q, k, v, mask=False, normalize=False, temperature=None, a0=1.0, a1=1.0, a2=0.5, lim=1.0, p=2,
            normalize_term=8.0):
    """Functional form.  With temperature=None it follows the reference's CPU implementations
    (fastattention_einops.py:78-82, score_function.py:57): temperature = normalize_term * sqrt(d), or 1 when
    the tensors are normalised."""
    if temperature is None:
        temperature = 1.0 if normalize else normalize_term * math.sqrt(q.shape[-1])
    return FastMax.apply(q, k, v, None, None, mask, 0.0, normalize, temperature, a0, a1, a2, lim, p)


class FASTMultiHeadAttention(torch.nn.Module):
    """nn.Module shim of transformer/model.py:208-216."""

    def __init__(self, use_custom_gradient=True, zero_copy=True, apply_rpe=False, noise_dropout=False):
        super().__init__()
        self.use_custom_gradient = use_custom_gradient
        self.zero_copy = zero_copy
        self.apply_rpe = apply_rpe            # FastMax only: see its docstring
        self.noise_dropout = noise_dropout

    def forward(self, q, k, v, drop_noise=None, rpe_matrix=None, mask=False, dropout=0.0, normalize=False,
                temperature=1.0, a0=1.0, a1=1.0, a2=0.5, lim=1.0, p=2):
        if not self.use_custom_gradient:
            return 0  # what the reference returns (model.py:216)
        if self.zero_copy:
            return FastMax.apply(q, k, v, drop_noise, rpe_matrix, mask, dropout, normalize, temperature, a0, a1, a2, lim, p,
                                 self.apply_rpe, self.noise_dropout)
        return FASTMultiHeadAttention_Function.apply(q, k, v, drop_noise, rpe_matrix, mask, dropout, normalize, temperature,
                                                     a0, a1, a2, lim, p)


def rpe_matrix_creator(n, d, device, dtype, structured=False, is_zero=True):
    """Relative-positional-encoding table of transformer/model.py:218-247: a (2n-1, d) matrix.  The operator
    ignores it (as the reference's kernels do), it exists so call sites keep working unchanged."""
    if dtype != torch.float32:
        print("The data type must be float32 in order for Fastmax to work")
    if structured:
        pos = torch.arange(0, n, device=device, dtype=dtype).unsqueeze(1)
        div = torch.exp(torch.arange(0, d, 2, device=device, dtype=dtype) * -(math.log(10000.0) / d))
        pe_pos = torch.zeros(n, d, device=device, dtype=dtype)
        pe_neg = torch.zeros(n, d, device=device, dtype=dtype)
        pe_pos[:, 0::2], pe_pos[:, 1::2] = torch.sin(pos * div), torch.cos(pos * div)
        pe_neg[:, 0::2], pe_neg[:, 1::2] = torch.sin(-pos * div), torch.cos(-pos * div)
        return torch.cat([torch.flip(pe_pos, [0]), pe_neg[1:]], dim=0)
    if is_zero:
        return torch.zeros(size=(2 * n - 1, d), device=device, dtype=dtype)
    return torch.normal(0, 1, size=(2 * n - 1, d), device=device, dtype=dtype)


fastmax_custom = FASTMultiHeadAttention()
