"""Sequence-parallel causal Fastmax: each rank holds a contiguous piece of the sequence (all heads).

The reference has no multi-GPU path; this is the natural one for a linear-time attention: the only thing a rank
needs from the ranks before it is the SUM of their moment states (a fixed-size (rows x ld) float32 array per head,
independent of the sequence length), and the backward needs the sum of the gradient moments of the ranks after it.

    forward   T_r  = Phi(K_r)^T [V_r | 1]                      (local, state-only call)
              P_r  = sum_{r' < r} T_r'                          (all_gather + local exclusive prefix)
              o_r  = fastmax(q_r, k_r, v_r, state_in = P_r)
    backward  dT_r = Phi(Q_r)^T dO'_r                           (local, state-only call)
              R_r  = sum_{r' > r} dT_r'                         (all_gather + local exclusive suffix)
              dq_r, dk_r, dv_r = backward(..., state_in = P_r, dstate_in = R_r)

The exchange is one all_gather of world_size x state bytes per direction (config 3: 8 heads x 673 x 36 x 4 B =
775 KB per rank), latency-bound on NVLink.  The collective goes through torch.distributed (NCCL on GPUs; the same
code runs on gloo for the CPU tests, where the compute engine is replaced by the CPU oracle).
"""
from __future__ import annotations

import torch
import torch.distributed as dist


def _world(group=None):
    if not (dist.is_available() and dist.is_initialized()):
        return 1, 0
    return dist.get_world_size(group), dist.get_rank(group)


def _gather_all(local: torch.Tensor, world: int, group=None) -> torch.Tensor:
    """(world, *local.shape): every rank's `local`, one collective into one buffer."""
    local = local.contiguous()
    buf = torch.empty((world,) + tuple(local.shape), dtype=local.dtype, device=local.device)
    try:
        dist.all_gather_into_tensor(buf, local, group=group)
    except (RuntimeError, NotImplementedError):   # a backend without the single-buffer form
        dist.all_gather(list(buf.unbind(0)), local, group=group)
    return buf


def exclusive_prefix(local: torch.Tensor, group=None) -> torch.Tensor:
    """Sum of `local` over the ranks BEFORE this one (zeros on rank 0)."""
    world, rank = _world(group)
    if world == 1:
        return torch.zeros_like(local)
    buf = _gather_all(local, world, group)
    return buf[:rank].sum(0) if rank > 0 else torch.zeros_like(local)


def exclusive_suffix(local: torch.Tensor, group=None) -> torch.Tensor:
    """Sum of `local` over the ranks AFTER this one (zeros on the last rank)."""
    world, rank = _world(group)
    if world == 1:
        return torch.zeros_like(local)
    buf = _gather_all(local, world, group)
    return buf[rank + 1:].sum(0) if rank + 1 < world else torch.zeros_like(local)


class KeyMoments:
    """Per-segment key moments of one piece's k and v (see fastmax_forward_args.key_moments_out): written by the first
    call that gets the holder, read by the later calls on the same k and v, which then skip their pass over them."""

    def __init__(self):
        self.buf = None
        self.grad_buf = None   # the same for the gradient moments of the piece's q, o, g and upstream gradient


class CudaEngine:
    """The library's kernels through the `fastmax_cuda` extension ((b, h, n, d) CUDA tensors).  `moments`: a KeyMoments
    holder that belongs to the k and v of the call; sequence_parallel.forward / backward create one per piece."""

    reuses_key_moments = True

    def __init__(self, inv_temp, a0=1.0, a1=1.0, a2=0.5, p=2):
        from . import load_extension

        self.ext = load_extension()
        self.cfg = (float(inv_temp), float(a0), float(a1), float(a2), int(p))

    def _compute_dtype(self, k, v):
        """float32 pieces after torch.set_float32_matmul_precision("medium") (PyTorch's permission to compute float32
        matmuls in bfloat16) run on bfloat16 copies when that puts them on the tensor-memory kernels; the states that
        travel between the ranks, the outputs and the gradients stay float32."""
        if k.dtype != torch.float32 or torch.get_float32_matmul_precision() != "medium":
            return None
        kb, vb = k.bfloat16(), v.bfloat16()
        return torch.bfloat16 if self.ext.forward_engine(kb, kb, vb, True, self.cfg[4]) == 1 else None

    def key_state(self, k, v, moments=None):
        it, a0, a1, a2, p = self.cfg
        if self._compute_dtype(k, v) is not None:
            k, v = k.bfloat16(), v.bfloat16()
        if moments is None:
            return self.ext.forward(k, k, v, True, it, a0, a1, a2, p, None, True, False, 0)[2]
        res = self.ext.forward(k, k, v, True, it, a0, a1, a2, p, None, True, False, 0, None, moments.buf, True)
        moments.buf = res[3]
        return res[2]

    def forward(self, q, k, v, state_in, moments=None):
        it, a0, a1, a2, p = self.cfg
        cast = self._compute_dtype(k, v) is not None
        if cast:
            q, k, v = q.bfloat16(), k.bfloat16(), v.bfloat16()
        if moments is None:
            o, g, _ = self.ext.forward(q, k, v, True, it, a0, a1, a2, p, state_in, False, True, 0)
            return (o.float() if cast else o), g
        res = self.ext.forward(q, k, v, True, it, a0, a1, a2, p, state_in, False, True, 0, None, moments.buf, True)
        moments.buf = res[3]
        return (res[0].float() if cast else res[0]), res[1]

    def grad_state(self, q, k, v, o, g, do, state_in, moments=None):
        it, a0, a1, a2, p = self.cfg
        if self._compute_dtype(k, v) is not None:
            q, k, v, o, do = q.bfloat16(), k.bfloat16(), v.bfloat16(), o.bfloat16(), do.bfloat16()
        if moments is None:
            return self.ext.backward(q, k, v, o, g, do, True, it, a0, a1, a2, p, state_in, None, True, False, 0)[3]
        res = self.ext.backward(q, k, v, o, g, do, True, it, a0, a1, a2, p, state_in, None, True, False, 0, None, None,
                                moments.grad_buf, True)
        moments.grad_buf = res[4]
        return res[3]

    def backward(self, q, k, v, o, g, do, state_in, dstate_in, moments=None):
        it, a0, a1, a2, p = self.cfg
        cast = self._compute_dtype(k, v) is not None
        if cast:
            q, k, v, o, do = q.bfloat16(), k.bfloat16(), v.bfloat16(), o.bfloat16(), do.bfloat16()
        km, gm = (None, None) if moments is None else (moments.buf, moments.grad_buf)
        grads = self.ext.backward(q, k, v, o, g, do, True, it, a0, a1, a2, p, state_in, dstate_in, False, True, 0,
                                  None, km, gm, False)[:3]
        return tuple(t.float() for t in grads) if cast else tuple(grads)


def _moments_kw(engine, carry=None):
    if not getattr(engine, "reuses_key_moments", False):
        return {}
    return {"moments": KeyMoments() if carry is None else carry[1]}


def forward(engine, q, k, v, group=None):
    """Returns (o, g, carry) for this rank's piece; hand `carry` (the prefix state of the earlier ranks, None when there
    is one rank, and the piece's key moments) to backward()."""
    kw = _moments_kw(engine)
    if _world(group)[0] == 1:
        o, g = engine.forward(q, k, v, None, **kw)
        return o, g, (None, kw.get("moments"))
    prefix = exclusive_prefix(engine.key_state(k, v, **kw), group)
    o, g = engine.forward(q, k, v, prefix, **kw)
    return o, g, (prefix, kw.get("moments"))


def backward(engine, q, k, v, o, g, do, carry, group=None):
    """Returns (dq, dk, dv) for this rank's piece; `carry` is what forward() returned."""
    prefix = carry[0]
    kw = _moments_kw(engine, carry)
    if _world(group)[0] == 1:
        return engine.backward(q, k, v, o, g, do, prefix, None, **kw)
    suffix = exclusive_suffix(engine.grad_state(q, k, v, o, g, do, prefix, **kw), group)
    return engine.backward(q, k, v, o, g, do, prefix, suffix, **kw)


class SequenceParallelFastMax(torch.autograd.Function):
    """Causal Fastmax over a sequence that is split into contiguous pieces across the ranks of `group`."""

    @staticmethod
    def forward(ctx, q, k, v, temperature=1.0, a0=1.0, a1=1.0, a2=0.5, p=2, group=None):
        engine = CudaEngine(1.0 / float(temperature), a0, a1, a2, p)
        o, g, (prefix, moments) = forward(engine, q, k, v, group)
        ctx.save_for_backward(q, k, v, o, g, *([] if prefix is None else [prefix]))
        ctx.engine, ctx.group, ctx.moments = engine, group, moments
        return o

    @staticmethod
    def backward(ctx, grad_output):
        q, k, v, o, g = ctx.saved_tensors[:5]
        prefix = ctx.saved_tensors[5] if len(ctx.saved_tensors) > 5 else None
        if grad_output.stride(-1) != 1:
            grad_output = grad_output.contiguous()
        dq, dk, dv = backward(ctx.engine, q, k, v, o, g, grad_output, (prefix, ctx.moments), ctx.group)
        return dq, dk, dv, None, None, None, None, None, None
