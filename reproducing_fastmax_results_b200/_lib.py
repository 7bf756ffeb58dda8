"""ctypes binding of the C ABI (include/fastmax_b200.h).

This is the boundary the parity tests call through: plain device pointers, sizes and strides, no torch
types.  torch is only used by the helpers at the bottom to obtain device pointers and a workspace.
Loading fails loudly when the library has not been built: there is no CPU fallback.
"""
from __future__ import annotations

import ctypes as C
import os

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG, "libfastmax_b200.so")

FASTMAX_F32, FASTMAX_BF16 = 0, 1
FLAG_NO_TENSOR_CORES = 1
FLAG_SINGLE_STREAM = 2

EXPORTED_SYMBOLS = [
    "fastmax_state_rows", "fastmax_state_ld", "fastmax_state_bytes",
    "fastmax_forward_workspace", "fastmax_forward", "fastmax_key_moments_bytes", "fastmax_forward_engine",
    "fastmax_static_scratch_bytes", "fastmax_forward_static_scratch",
    "fastmax_backward_workspace", "fastmax_backward", "fastmax_grad_moments_bytes",
    "fastmax_decode_step",
    "fastmax_normalize_forward", "fastmax_normalize_backward",
    "fastmax_key_prologue", "fastmax_output_noise",
    "fastmax_status_string", "fastmax_last_cuda_error", "fastmax_last_cuda_error_string",
    "fastmax_version", "fastmax_launch_count", "fastmax_check_status", "fastmax_debug_wait_histogram",
    "fastmax_debug_wait_selftest",
    "fastmax_profile_enable", "fastmax_profile_kinds", "fastmax_profile_kind_name", "fastmax_profile_collect",
]


class Tensor(C.Structure):
    _fields_ = [("ptr", C.c_void_p), ("stride_b", C.c_int64), ("stride_h", C.c_int64), ("stride_n", C.c_int64)]


class Problem(C.Structure):
    _fields_ = [
        ("batch", C.c_int32), ("heads", C.c_int32), ("nq", C.c_int32), ("nk", C.c_int32), ("d", C.c_int32),
        ("order", C.c_int32), ("causal", C.c_int32), ("dtype", C.c_int32),
        ("a0", C.c_float), ("a1", C.c_float), ("a2", C.c_float), ("inv_temperature", C.c_float),
        ("flags", C.c_int32), ("reserved", C.c_int32),
    ]


class ForwardArgs(C.Structure):
    _fields_ = [("q", Tensor), ("k", Tensor), ("v", Tensor), ("o", Tensor), ("g", Tensor),
                ("state_in", C.c_void_p), ("state_out", C.c_void_p),
                ("key_moments_in", C.c_void_p), ("key_moments_out", C.c_void_p)]


class BackwardArgs(C.Structure):
    _fields_ = [("q", Tensor), ("k", Tensor), ("v", Tensor), ("o", Tensor), ("g", Tensor), ("d_out", Tensor),
                ("dq", Tensor), ("dk", Tensor), ("dv", Tensor),
                ("state_in", C.c_void_p), ("dstate_in", C.c_void_p), ("dstate_out", C.c_void_p),
                ("key_moments_in", C.c_void_p), ("grad_moments_in", C.c_void_p), ("grad_moments_out", C.c_void_p)]


class KeyMoments:
    """Holder of the per-segment key moments of one (k, v) pair (fastmax_forward_args.key_moments_out/in): the first
    call that is handed the holder fills it, later calls with the same problem, k and v (the forward after a
    state-only call, the backward after the forward) read it and skip their pass over k and v.  Stays empty for
    calls that have no such pass (one segment per head, tensor-memory kernels)."""

    def __init__(self):
        self.buf = None
        self.grad_buf = None   # the same for the gradient moments Phi(Q)^T dO' (fastmax_backward_args.grad_moments_*)


class DecodeArgs(C.Structure):
    _fields_ = [("q", Tensor), ("k", Tensor), ("v", Tensor), ("o", Tensor), ("g", Tensor), ("state", C.c_void_p)]


class FastmaxError(RuntimeError):
    def __init__(self, status, what, detail=""):
        self.status = status
        super().__init__(f"{what}: status {status} ({detail})")


_lib = None


def load():
    """Loads libfastmax_b200.so (once).  Raises if it is missing: build it with
    `python -m reproducing_fastmax_results_b200.build`."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing; the Fastmax engine has no CPU fallback. "
            "Build it: python -m reproducing_fastmax_results_b200.build")
    lib = C.CDLL(LIB_PATH)
    lib.fastmax_state_rows.restype = C.c_int32
    lib.fastmax_state_rows.argtypes = [C.c_int32, C.c_int32]
    lib.fastmax_state_ld.restype = C.c_int32
    lib.fastmax_state_ld.argtypes = [C.c_int32]
    lib.fastmax_state_bytes.restype = C.c_size_t
    lib.fastmax_state_bytes.argtypes = [C.POINTER(Problem)]
    lib.fastmax_forward_workspace.restype = C.c_size_t
    lib.fastmax_forward_workspace.argtypes = [C.POINTER(Problem), C.POINTER(ForwardArgs)]
    lib.fastmax_forward_engine.restype = C.c_int32
    lib.fastmax_forward_engine.argtypes = [C.POINTER(Problem), C.POINTER(ForwardArgs)]
    lib.fastmax_key_moments_bytes.restype = C.c_size_t
    lib.fastmax_key_moments_bytes.argtypes = [C.POINTER(Problem), C.POINTER(ForwardArgs)]
    lib.fastmax_forward.restype = C.c_int32
    lib.fastmax_forward.argtypes = [C.POINTER(Problem), C.POINTER(ForwardArgs), C.c_void_p, C.c_size_t, C.c_void_p]
    lib.fastmax_static_scratch_bytes.restype = C.c_size_t
    lib.fastmax_forward_static_scratch.restype = C.c_int32
    lib.fastmax_forward_static_scratch.argtypes = [C.POINTER(Problem), C.POINTER(ForwardArgs), C.c_void_p]
    lib.fastmax_backward_workspace.restype = C.c_size_t
    lib.fastmax_backward_workspace.argtypes = [C.POINTER(Problem), C.POINTER(BackwardArgs)]
    lib.fastmax_grad_moments_bytes.restype = C.c_size_t
    lib.fastmax_grad_moments_bytes.argtypes = [C.POINTER(Problem), C.POINTER(BackwardArgs)]
    lib.fastmax_backward.restype = C.c_int32
    lib.fastmax_backward.argtypes = [C.POINTER(Problem), C.POINTER(BackwardArgs), C.c_void_p, C.c_size_t, C.c_void_p]
    lib.fastmax_decode_step.restype = C.c_int32
    lib.fastmax_decode_step.argtypes = [C.POINTER(Problem), C.POINTER(DecodeArgs), C.c_void_p]
    lib.fastmax_normalize_forward.restype = C.c_int32
    lib.fastmax_normalize_forward.argtypes = [C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_float,
                                              C.POINTER(Tensor), C.POINTER(Tensor), C.c_void_p, C.c_void_p]
    lib.fastmax_normalize_backward.restype = C.c_int32
    lib.fastmax_normalize_backward.argtypes = [C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_float,
                                               C.POINTER(Tensor), C.POINTER(Tensor), C.POINTER(Tensor), C.c_void_p,
                                               C.c_void_p, C.c_void_p]
    lib.fastmax_key_prologue.restype = C.c_int32
    lib.fastmax_key_prologue.argtypes = [C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_float, C.POINTER(Tensor),
                                         C.c_void_p, C.c_void_p]
    lib.fastmax_output_noise.restype = C.c_int32
    lib.fastmax_output_noise.argtypes = [C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_float, C.POINTER(Tensor),
                                         C.POINTER(Tensor), C.POINTER(Tensor), C.c_void_p]
    lib.fastmax_status_string.restype = C.c_char_p
    lib.fastmax_status_string.argtypes = [C.c_int32]
    lib.fastmax_last_cuda_error.restype = C.c_int32
    lib.fastmax_last_cuda_error_string.restype = C.c_char_p
    lib.fastmax_version.restype = C.c_char_p
    lib.fastmax_launch_count.restype = C.c_uint64
    lib.fastmax_check_status.restype = C.c_int32
    lib.fastmax_debug_wait_histogram.restype = C.c_int32
    lib.fastmax_debug_wait_histogram.argtypes = [C.POINTER(C.c_int32), C.c_int32]
    lib.fastmax_debug_wait_selftest.restype = C.c_int32
    lib.fastmax_debug_wait_selftest.argtypes = [C.c_void_p]
    lib.fastmax_profile_enable.argtypes = [C.c_int32]
    lib.fastmax_profile_kind_name.restype = C.c_char_p
    lib.fastmax_profile_kind_name.argtypes = [C.c_int32]
    lib.fastmax_profile_collect.argtypes = [C.POINTER(C.c_double), C.POINTER(C.c_uint64), C.c_int32]
    _lib = lib
    return lib


def check(status, what):
    if status != 0:
        lib = load()
        detail = lib.fastmax_status_string(status).decode()
        if status == 4:
            detail += ": " + lib.fastmax_last_cuda_error_string().decode()
        raise FastmaxError(status, what, detail)


# ------------------------------------------------------------------------------------------------------
# helpers that turn torch CUDA tensors into ABI views (device pointer + element strides)
# ------------------------------------------------------------------------------------------------------
def view_bhnd(t):
    """(b, h, n, d) tensor (any strides, unit stride on d) -> Tensor view."""
    assert t.dim() == 4 and (t.shape[3] == 1 or t.stride(3) == 1)
    return Tensor(t.data_ptr(), t.stride(0), t.stride(1), t.stride(2))


def view_bhn(t):
    assert t.dim() == 3
    return Tensor(t.data_ptr(), t.stride(0), t.stride(1), t.stride(2))


def dtype_code(t):
    import torch

    if t.dtype == torch.float32:
        return FASTMAX_F32
    if t.dtype == torch.bfloat16:
        return FASTMAX_BF16
    raise TypeError(f"fastmax: float32 or bfloat16 expected, got {t.dtype}")


def problem_for(q, k, causal, inv_temp, a0=1.0, a1=1.0, a2=0.5, order=2, flags=0):
    return Problem(q.shape[0], q.shape[1], q.shape[2], k.shape[2], q.shape[3], order, int(bool(causal)),
                   dtype_code(q), a0, a1, a2, inv_temp, flags, 0)


def _stream():
    import torch

    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def _workspace(nbytes, device):
    import torch

    ws = torch.empty(nbytes + 256, dtype=torch.uint8, device=device)
    ptr = (ws.data_ptr() + 255) // 256 * 256
    return ws, C.c_void_p(ptr)


def _attach_key_moments(lib, pb, fargs, key_moments, device, sink, allow_fill):
    """Points sink.key_moments_in at the holder's buffer when it fits this call, or (allow_fill) gives the call a new
    buffer to fill.  `fargs`: the ForwardArgs that describe the call to fastmax_key_moments_bytes."""
    import torch

    nbytes = lib.fastmax_key_moments_bytes(C.byref(pb), C.byref(fargs))
    if nbytes == 0:
        return
    if key_moments.buf is not None and key_moments.buf.numel() * 4 == nbytes:
        sink.key_moments_in = key_moments.buf.data_ptr()
    elif allow_fill:
        key_moments.buf = torch.empty(nbytes // 4, dtype=torch.float32, device=device)
        sink.key_moments_out = key_moments.buf.data_ptr()


def forward(q, k, v, causal, inv_temp, a0=1.0, a1=1.0, a2=0.5, order=2, state_in=None, want_state=False,
            want_output=True, flags=0, out=None, key_moments=None):
    """Calls fastmax_forward on (b,h,n,d) CUDA tensors.  Returns (o, g, state_out).  `out`: optional (b,h,n,d) tensor
    of any strides (unit stride on d) that receives o, e.g. the transposed view of a (b, n, h*d) buffer.
    `key_moments`: optional KeyMoments holder for this (k, v)."""
    import torch

    lib = load()
    pb = problem_for(q, k, causal, inv_temp, a0, a1, a2, order, flags)
    args = ForwardArgs()
    args.q, args.k, args.v = view_bhnd(q), view_bhnd(k), view_bhnd(v)
    o = g = sout = None
    if want_output:
        o = torch.empty(q.shape, dtype=q.dtype, device=q.device) if out is None else out
        assert o.shape == q.shape and o.dtype == q.dtype
        g = torch.empty(q.shape[:3], dtype=torch.float32, device=q.device)
        args.o, args.g = view_bhnd(o), view_bhn(g)
    if state_in is not None:
        assert state_in.is_contiguous() and state_in.dtype == torch.float32
        args.state_in = state_in.data_ptr()
    if want_state:
        sout = torch.empty((q.shape[0], q.shape[1], lib.fastmax_state_rows(pb.d, pb.order), lib.fastmax_state_ld(pb.d)),
                           dtype=torch.float32, device=q.device)
        args.state_out = sout.data_ptr()
    if key_moments is not None:
        _attach_key_moments(lib, pb, args, key_moments, q.device, args, True)
    need = lib.fastmax_forward_workspace(C.byref(pb), C.byref(args))
    ws, wptr = _workspace(need, q.device)
    check(lib.fastmax_forward(C.byref(pb), C.byref(args), wptr, need, _stream()), "fastmax_forward")
    return o, g, sout


def forward_static_scratch(q, k, v, causal, inv_temp, a0=1.0, a1=1.0, a2=0.5, order=2, flags=0):
    """Calls fastmax_forward_static_scratch: same as forward(), but the library's built-in scratch array is used
    and no workspace is passed.  Returns (o, g)."""
    import torch

    lib = load()
    pb = problem_for(q, k, causal, inv_temp, a0, a1, a2, order, flags)
    args = ForwardArgs()
    args.q, args.k, args.v = view_bhnd(q), view_bhnd(k), view_bhnd(v)
    o = torch.empty(q.shape, dtype=q.dtype, device=q.device)
    g = torch.empty(q.shape[:3], dtype=torch.float32, device=q.device)
    args.o, args.g = view_bhnd(o), view_bhn(g)
    check(lib.fastmax_forward_static_scratch(C.byref(pb), C.byref(args), _stream()), "fastmax_forward_static_scratch")
    return o, g


def backward(q, k, v, o, g, d_out, causal, inv_temp, a0=1.0, a1=1.0, a2=0.5, order=2, state_in=None, dstate_in=None,
             want_dstate=False, want_grads=True, flags=0, grads_out=None, key_moments=None):
    """Calls fastmax_backward on (b,h,n,d) CUDA tensors.  Returns (dq, dk, dv, dstate_out).  `grads_out`: optional
    (dq, dk, dv) tensors of any strides (unit stride on d) that receive the gradients.  `key_moments`: the holder the
    forward call of the same q, k, v filled."""
    import torch

    lib = load()
    pb = problem_for(q, k, causal, inv_temp, a0, a1, a2, order, flags)
    args = BackwardArgs()
    args.q, args.k, args.v, args.o, args.g = view_bhnd(q), view_bhnd(k), view_bhnd(v), view_bhnd(o), view_bhn(g)
    args.d_out = view_bhnd(d_out)
    dq = dk = dv = dsout = None
    if want_grads:
        dq, dk, dv = (torch.empty(t.shape, dtype=t.dtype, device=t.device) for t in (q, k, v)) if grads_out is None \
            else grads_out
        args.dq, args.dk, args.dv = view_bhnd(dq), view_bhnd(dk), view_bhnd(dv)
    if state_in is not None:
        args.state_in = state_in.data_ptr()
    if dstate_in is not None:
        args.dstate_in = dstate_in.data_ptr()
    if want_dstate:
        dsout = torch.empty((q.shape[0], q.shape[1], lib.fastmax_state_rows(pb.d, pb.order), lib.fastmax_state_ld(pb.d)),
                            dtype=torch.float32, device=q.device)
        args.dstate_out = dsout.data_ptr()
    if key_moments is not None and key_moments.buf is not None and want_grads:
        fargs = ForwardArgs()
        fargs.q, fargs.k, fargs.v, fargs.o, fargs.g = args.q, args.k, args.v, args.o, args.g
        _attach_key_moments(lib, pb, fargs, key_moments, q.device, args, False)
    if key_moments is not None:
        nbytes = lib.fastmax_grad_moments_bytes(C.byref(pb), C.byref(args))
        if nbytes:
            if key_moments.grad_buf is not None and key_moments.grad_buf.numel() * 4 == nbytes:
                args.grad_moments_in = key_moments.grad_buf.data_ptr()
            else:
                key_moments.grad_buf = torch.empty(nbytes // 4, dtype=torch.float32, device=q.device)
                args.grad_moments_out = key_moments.grad_buf.data_ptr()
    need = lib.fastmax_backward_workspace(C.byref(pb), C.byref(args))
    ws, wptr = _workspace(need, q.device)
    check(lib.fastmax_backward(C.byref(pb), C.byref(args), wptr, need, _stream()), "fastmax_backward")
    return dq, dk, dv, dsout


def new_state(batch, heads, d, order=2, device="cuda"):
    """Zero moment state in the exchange layout: float32 (batch, heads, fastmax_state_rows, fastmax_state_ld)."""
    import torch

    lib = load()
    return torch.zeros((batch, heads, lib.fastmax_state_rows(d, order), lib.fastmax_state_ld(d)), dtype=torch.float32,
                       device=device)


def decode_step(q, k, v, state, inv_temp, a0=1.0, a1=1.0, a2=0.5, order=2, out=None):
    """Calls fastmax_decode_step: q, k, v are (b, h, d) or (b, h, 1, d) CUDA tensors holding ONE new token per
    head; `state` (from new_state() or forward(..., want_state=True)) is updated in place.  Returns (o, g) with
    o shaped like q and g float32 (b, h)."""
    import torch

    lib = load()
    q3, k3, v3 = (t.reshape(t.shape[0], t.shape[1], t.shape[-1]) if t.dim() == 4 else t for t in (q, k, v))
    for t in (q3, k3, v3):
        assert t.dim() == 3 and t.stride(2) == 1
    assert state.dtype == torch.float32 and state.is_contiguous()
    b, h, d = q3.shape
    assert tuple(state.shape) == (b, h, lib.fastmax_state_rows(d, order), lib.fastmax_state_ld(d)), state.shape
    o = torch.empty(q.shape, dtype=q.dtype, device=q.device) if out is None else out
    o3 = o.reshape(b, h, d) if o.dim() == 4 else o
    assert o3.data_ptr() == o.data_ptr() and o3.stride(2) == 1
    g = torch.empty((b, h), dtype=torch.float32, device=q.device)
    pb = Problem(b, h, 1, 1, d, order, 1, dtype_code(q), a0, a1, a2, inv_temp, 0, 0)
    args = DecodeArgs()
    args.q, args.k, args.v, args.o = (Tensor(t.data_ptr(), t.stride(0), t.stride(1), 0) for t in (q3, k3, v3, o3))
    args.g = Tensor(g.data_ptr(), g.stride(0), g.stride(1), 0)
    args.state = state.data_ptr()
    check(lib.fastmax_decode_step(C.byref(pb), C.byref(args), _stream()), "fastmax_decode_step")
    return o, g


def normalize_forward(x, lim=1.0):
    import torch

    lib = load()
    y = torch.empty_like(x)
    stats = torch.empty(x.shape[:2], dtype=torch.int64, device=x.device)
    xv, yv = view_bhnd(x), view_bhnd(y)
    check(lib.fastmax_normalize_forward(x.shape[0], x.shape[1], x.shape[2], x.shape[3], dtype_code(x), lim,
                                        C.byref(xv), C.byref(yv), stats.data_ptr(), _stream()), "fastmax_normalize_forward")
    return y, stats


def normalize_backward(y, dy, stats, lim=1.0):
    import torch

    lib = load()
    dx = torch.empty_like(y)
    scratch = torch.empty(y.shape[0] * y.shape[1], dtype=torch.float32, device=y.device)
    yv, gv, dv = view_bhnd(y), view_bhnd(dy), view_bhnd(dx)
    check(lib.fastmax_normalize_backward(y.shape[0], y.shape[1], y.shape[2], y.shape[3], dtype_code(y), lim,
                                         C.byref(yv), C.byref(gv), C.byref(dv), stats.data_ptr(), scratch.data_ptr(),
                                         _stream()), "fastmax_normalize_backward")
    return dx


def key_prologue(k, inv_temp, rpe=None):
    """Calls fastmax_key_prologue: k (b,h,n,d) is scaled by inv_temp in place and, with rpe (float32 (2n-1, d)), gets
    rpe[(l + n) mod (2n - 1)] added to key l."""
    lib = load()
    kv = view_bhnd(k)
    check(lib.fastmax_key_prologue(k.shape[0], k.shape[1], k.shape[2], k.shape[3], dtype_code(k), inv_temp, C.byref(kv),
                                   None if rpe is None else rpe.data_ptr(), _stream()), "fastmax_key_prologue")
    return k


def output_noise(x, noise, scale, out=None):
    """Calls fastmax_output_noise: returns x * (1 + scale * noise) (written into `out`, which may be x)."""
    import torch

    lib = load()
    out = torch.empty_like(x) if out is None else out
    xv, nv, ov = view_bhnd(x), view_bhnd(noise), view_bhnd(out)
    check(lib.fastmax_output_noise(x.shape[0], x.shape[1], x.shape[2], x.shape[3], dtype_code(x), scale, C.byref(xv),
                                   C.byref(nv), C.byref(ov), _stream()), "fastmax_output_noise")
    return out


def check_status():
    """Synchronises the device and raises if a kernel reported a bounded-wait timeout."""
    import torch

    torch.cuda.synchronize()
    check(load().fastmax_check_status(), "fastmax_check_status")


def wait_histogram():
    """Returns {wait-site code modulo 256: thread blocks that gave up there first} and clears the counters."""
    lib = load()
    h = (C.c_int32 * 256)()
    check(lib.fastmax_debug_wait_histogram(h, 256), "fastmax_debug_wait_histogram")
    return {i: int(c) for i, c in enumerate(h) if c}


def profile(enable):
    load().fastmax_profile_enable(1 if enable else 0)


def profile_collect():
    """Returns {kernel kind: (total ms, launches)} for the launches recorded since the last call."""
    lib = load()
    n = lib.fastmax_profile_kinds()
    ms = (C.c_double * n)()
    cnt = (C.c_uint64 * n)()
    check(lib.fastmax_profile_collect(ms, cnt, n), "fastmax_profile_collect")
    return {lib.fastmax_profile_kind_name(i).decode(): (ms[i], int(cnt[i])) for i in range(n) if cnt[i]}
