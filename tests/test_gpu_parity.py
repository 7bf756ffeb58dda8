"""Parity of the CUDA path (called through the C ABI) with the CPU oracle and the reference's golden vectors.

Tolerances (max |x - ref| / max |ref| per tensor): 1e-4 for float32, 2e-2 for bfloat16 inputs with float32
accumulation.  bfloat16 cases compare against the oracle evaluated on the bf16-rounded inputs.
"""
import os

import numpy as np
import pytest
import torch

from cases import CASES, make_inputs
from oracle import fastmax_oracle as orc

pytestmark = pytest.mark.gpu

TOL = {torch.float32: 1e-4, torch.bfloat16: 2e-2}
GOLD = np.load(os.path.join(os.path.dirname(__file__), "golden", "reference_vectors.npz"))


def lib():
    from reproducing_fastmax_results_b200 import _lib

    return _lib


def dev(x, dtype=torch.float32):
    return torch.from_numpy(np.ascontiguousarray(x)).to("cuda").to(dtype)


def host(t):
    return t.detach().float().cpu().numpy().astype(np.float64)


def run_fwd_bwd(q, k, v, do, causal, poly, dtype, flags=0):
    L = lib()
    qd, kd, vd, dod = (dev(x, dtype) for x in (q, k, v, do))
    o, g, _ = L.forward(qd, kd, vd, causal, poly.inv_temp, poly.a0, poly.a1, poly.a2, poly.p, flags=flags)
    dq, dk, dv, _ = L.backward(qd, kd, vd, o, g, dod, causal, poly.inv_temp, poly.a0, poly.a1, poly.a2, poly.p, flags=flags)
    torch.cuda.synchronize()
    rounded = tuple(host(t) for t in (qd, kd, vd, dod))
    return tuple(host(t) for t in (o, g, dq, dk, dv)), rounded


@pytest.mark.parametrize("name", sorted(CASES))
def test_golden_vectors_fp32(name):
    """The reference's own outputs and gradients (einops implementation) on its seeded inputs."""
    B, H, N, D, p, mask, nt, scale, upstream = CASES[name]
    q, k, v, do = make_inputs(name)
    poly = orc.poly_from_normalize_term(D, nt, False, p)
    (o, g, dq, dk, dv), _ = run_fwd_bwd(q, k, v, do, mask, poly, torch.float32)
    for got, key in ((o, "o"), (dq, "dq"), (dk, "dk"), (dv, "dv")):
        err = orc.max_norm_err(got, GOLD[f"{name}/einops/{key}"])
        assert err < 1e-4, f"{name} {key}: {err}"


SHAPES = [
    # B, H, nq, nk, D
    (1, 2, 64, 64, 16),
    (2, 3, 100, 100, 32),
    (1, 2, 200, 200, 64),
    (1, 1, 37, 90, 32),     # nk > nq: causal aligns the queries to the last nq keys
    (1, 2, 1, 1, 64),       # single token
]


@pytest.mark.parametrize("shape", SHAPES)
@pytest.mark.parametrize("order", [1, 2])
@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_forward_backward_vs_oracle(shape, order, causal, dtype):
    B, H, nq, nk, D = shape
    rng = np.random.default_rng(hash((shape, order, causal)) % (2 ** 31))
    q = rng.standard_normal((B, H, nq, D)).astype(np.float32)
    k = rng.standard_normal((B, H, nk, D)).astype(np.float32)
    v = rng.standard_normal((B, H, nk, D)).astype(np.float32)
    do = rng.standard_normal((B, H, nq, D)).astype(np.float32)
    poly = orc.Poly(1.0, 1.0, 0.5, 1.0 / (2.0 * np.sqrt(D)), order)
    (o, g, dq, dk, dv), (qr, kr, vr, dor) = run_fwd_bwd(q, k, v, do, causal, poly, dtype)
    o_ref, g_ref = orc.fastmax_naive(qr, kr, vr, causal, poly)
    tol = TOL[dtype]
    assert orc.max_norm_err(o, o_ref) < tol
    assert orc.max_norm_err(g, g_ref) < 1e-4
    # gradients: the kernel differentiates at its own (rounded) o, g; the oracle at the exact ones
    dq_ref, dk_ref, dv_ref = orc.fastmax_naive_grads(qr, kr, vr, dor, causal, poly)
    # with a single visible key o == v exactly and dq, dk vanish analytically: floor the normaliser there
    floor = 1e-2 if nk == 1 else 0.0
    for got, ref in ((dq, dq_ref), (dk, dk_ref), (dv, dv_ref)):
        assert np.abs(got - ref).max() / max(np.abs(ref).max(), floor) < tol


@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("D", [32, 64])
def test_long_sequence_uses_segments(causal, D):
    """Few heads and a long sequence: the launcher splits the sequence into segments with a prefix pass."""
    B, H, N = 1, 1, 4096
    rng = np.random.default_rng(11 + D)
    q, k, v, do = (rng.standard_normal((B, H, N, D)).astype(np.float32) for _ in range(4))
    poly = orc.Poly(1.0, 1.0, 0.5, 1.0 / (4.0 * np.sqrt(D)), 2)
    (o, g, dq, dk, dv), _ = run_fwd_bwd(q, k, v, do, causal, poly, torch.float32)
    o_ref, g_ref = orc.fastmax_naive(q, k, v, causal, poly)
    dq_ref, dk_ref, dv_ref = orc.fastmax_naive_grads(q, k, v, do, causal, poly)
    for got, ref in ((o, o_ref), (g, g_ref), (dq, dq_ref), (dk, dk_ref), (dv, dv_ref)):
        assert orc.max_norm_err(got, ref) < 1e-4


def test_general_coefficients_and_strided_views():
    """a0, a1, a2 other than the Taylor ones, and (b, n, h, d) storage read through strides (no copies)."""
    B, H, N, D = 2, 4, 96, 32
    rng = np.random.default_rng(3)
    poly = orc.Poly(0.9, 1.166666, 0.145833, 0.37, 2)  # the alternative fit listed in fastmax_cuda_forward.cu:7-12
    q, k, v, do = (rng.standard_normal((B, N, H, D)).astype(np.float32) for _ in range(4))
    L = lib()
    qd, kd, vd, dod = (dev(x).transpose(1, 2) for x in (q, k, v, do))  # (b,h,n,d) views of (b,n,h,d) storage
    assert not qd.is_contiguous()
    o, g, _ = L.forward(qd, kd, vd, True, poly.inv_temp, poly.a0, poly.a1, poly.a2, 2)
    dq, dk, dv, _ = L.backward(qd, kd, vd, o, g, dod, True, poly.inv_temp, poly.a0, poly.a1, poly.a2, 2)
    qt, kt, vt, dot = (x.transpose(0, 2, 1, 3) for x in (q, k, v, do))
    o_ref, _ = orc.fastmax_naive(qt, kt, vt, True, poly)
    dq_ref, dk_ref, dv_ref = orc.fastmax_naive_grads(qt, kt, vt, dot, True, poly)
    for got, ref in ((o, o_ref), (dq, dq_ref), (dk, dk_ref), (dv, dv_ref)):
        assert orc.max_norm_err(host(got), ref) < 1e-4


@pytest.mark.parametrize("dtype,D", [(torch.float32, 32), (torch.bfloat16, 64)])
def test_outputs_written_straight_into_merged_head_buffers(dtype, D):
    """o, dq, dk, dv go through strides into (b, n, h*d) buffers (the layout after the head merge of
    transformer/model.py:335), so no transpose copy is needed on either side of the operator."""
    B, H, N = 2, 16, 200
    tol = 1e-4 if dtype == torch.float32 else 2e-2
    rng = np.random.default_rng(9)
    poly = orc.Poly(1.0, 1.0, 0.5, 1.0 / (2.0 * np.sqrt(D)), 2)
    q, k, v, do = (rng.standard_normal((B, N, H * D)).astype(np.float32) for _ in range(4))
    L = lib()
    split = lambda t: t.view(B, N, H, D).transpose(1, 2)
    qd, kd, vd, dod = (split(dev(x).to(dtype)) for x in (q, k, v, do))
    bufs = [torch.full((B, N, H * D), float("nan"), device="cuda", dtype=dtype) for _ in range(4)]
    o, g, _ = L.forward(qd, kd, vd, True, poly.inv_temp, order=2, out=split(bufs[0]))
    L.backward(qd, kd, vd, o, g, dod, True, poly.inv_temp, order=2, grads_out=tuple(split(b) for b in bufs[1:]))
    torch.cuda.synchronize()
    ref_in = [host(t) for t in (qd, kd, vd, dod)]
    o_ref, _ = orc.fastmax_naive(ref_in[0], ref_in[1], ref_in[2], True, poly)
    refs = (o_ref,) + tuple(orc.fastmax_naive_grads(*ref_in, True, poly))
    for buf, ref in zip(bufs, refs):
        got = host(buf).reshape(B, N, H, D).transpose(0, 2, 1, 3)
        assert np.isfinite(got).all()
        assert orc.max_norm_err(got, ref) < tol


@pytest.mark.parametrize("D", [32, 64])
def test_state_carry_between_calls(D):
    """A causal sequence cut in two: the second call starts from the first call's state (what a
    sequence-parallel rank or an incremental decoder does), forward and backward."""
    B, H, N, cut = 1, 2, 300, 128
    rng = np.random.default_rng(5)
    q, k, v, do = (rng.standard_normal((B, H, N, D)).astype(np.float32) for _ in range(4))
    poly = orc.Poly(1.0, 1.0, 0.5, 1.0 / (2.0 * np.sqrt(D)), 2)
    L = lib()
    qd, kd, vd, dod = (dev(x) for x in (q, k, v, do))
    a = [t[:, :, :cut].contiguous() for t in (qd, kd, vd, dod)]
    b = [t[:, :, cut:].contiguous() for t in (qd, kd, vd, dod)]
    o1, g1, s1 = L.forward(a[0], a[1], a[2], True, poly.inv_temp, order=2, want_state=True)
    o2, g2, s2 = L.forward(b[0], b[1], b[2], True, poly.inv_temp, order=2, state_in=s1, want_state=True)
    # state-only call equals the state returned together with outputs
    _, _, s1b = L.forward(a[0], a[1], a[2], True, poly.inv_temp, order=2, want_state=True, want_output=False)
    assert torch.allclose(s1, s1b, rtol=1e-5, atol=1e-5)
    o_ref, g_ref = orc.fastmax_naive(q, k, v, True, poly)
    assert orc.max_norm_err(host(torch.cat([o1, o2], 2)), o_ref) < 1e-4
    # state layout: lin rows hold sum k (x) [v|1]; last row the plain sums
    rows = s2.shape[2]
    ks, vs = k[0, 0].astype(np.float64), v[0, 0].astype(np.float64)
    v1 = np.concatenate([vs, np.ones((N, 1))], 1)
    assert orc.max_norm_err(host(s2[0, 0, rows - 1, : D + 1]), v1.sum(0)) < 1e-5
    assert orc.max_norm_err(host(s2[0, 0, rows - 1 - D : rows - 1, : D + 1]), ks.T @ v1) < 1e-5
    # backward: later piece first (its gradient moments feed the earlier piece)
    dq2, dk2, dv2, ds2 = L.backward(b[0], b[1], b[2], o2, g2, b[3], True, poly.inv_temp, order=2, state_in=s1, want_dstate=True)
    dq1, dk1, dv1, _ = L.backward(a[0], a[1], a[2], o1, g1, a[3], True, poly.inv_temp, order=2, dstate_in=ds2)
    dq_ref, dk_ref, dv_ref = orc.fastmax_naive_grads(q, k, v, do, True, poly)
    assert orc.max_norm_err(host(torch.cat([dq1, dq2], 2)), dq_ref) < 1e-4
    assert orc.max_norm_err(host(torch.cat([dk1, dk2], 2)), dk_ref) < 1e-4
    assert orc.max_norm_err(host(torch.cat([dv1, dv2], 2)), dv_ref) < 1e-4


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_normalize_forward_backward(dtype):
    B, H, N, D = 2, 3, 77, 32
    rng = np.random.default_rng(9)
    x = rng.standard_normal((B, H, N, D)).astype(np.float32)
    dy = rng.standard_normal((B, H, N, D)).astype(np.float32)
    L = lib()
    xd, dyd = dev(x, dtype), dev(dy, dtype)
    y, stats = L.normalize_forward(xd, 1.5)
    dx = L.normalize_backward(y, dyd, stats, 1.5)
    tol = TOL[dtype]
    assert orc.max_norm_err(host(y), orc.normalize(host(xd), 1.5)) < tol
    assert orc.max_norm_err(host(dx), orc.normalize_grad(host(xd), host(dyd), 1.5)) < tol
    # in place
    x2 = xd.clone()
    xv = L.view_bhnd(x2)
    import ctypes as C
    L.check(L.load().fastmax_normalize_forward(B, H, N, D, L.dtype_code(x2), 1.5, C.byref(xv), C.byref(xv),
                                               stats.data_ptr(), None), "in place")
    torch.cuda.synchronize()
    assert torch.equal(x2, y)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("shape", [(8, 40, 333, 64), (4, 80, 333, 32), (8, 40, 1000, 16), (8, 16, 4096, 64)])
def test_normalize_one_launch_per_direction(shape, dtype):
    """Enough heads to fill the device: one launch per direction (a thread-block cluster per head), ragged token
    counts, every cluster size; the argmax token sits in the middle of the sequence."""
    B, H, N, D = shape
    rng = np.random.default_rng(N + D)
    x = rng.standard_normal((B, H, N, D)).astype(np.float32)
    x[:, :, N // 2] *= 3.0
    dy = rng.standard_normal((B, H, N, D)).astype(np.float32)
    L = lib()
    xd, dyd = dev(x, dtype), dev(dy, dtype)
    L.profile_collect()
    L.profile(True)
    y, stats = L.normalize_forward(xd, 1.5)
    dx = L.normalize_backward(y, dyd, stats, 1.5)
    torch.cuda.synchronize()
    L.profile(False)
    assert L.profile_collect()["normalize"][1] == 2
    tol = TOL[dtype]
    assert orc.max_norm_err(host(y), orc.normalize(host(xd), 1.5)) < tol
    assert orc.max_norm_err(host(dx), orc.normalize_grad(host(xd), host(dyd), 1.5)) < tol
    # the same call twice gives the same bits (no atomics in this form)
    y2, stats2 = L.normalize_forward(xd, 1.5)
    dx2 = L.normalize_backward(y2, dyd, stats2, 1.5)
    assert torch.equal(y, y2) and torch.equal(dx, dx2) and torch.equal(stats, stats2)


def test_normalize_golden_vectors():
    for name in ("small_p2_causal", "small_p2_noncausal"):
        q, k, v, do = make_inputs(name)
        L = lib()
        y, stats = L.normalize_forward(dev(q), 1.0)
        dx = L.normalize_backward(y, dev(do), stats, 1.0)
        assert orc.max_norm_err(host(y), GOLD[f"{name}/normalize/q"]) < 1e-5
        assert orc.max_norm_err(host(dx), GOLD[f"{name}/normalize/dq"]) < 1e-4


def test_empty_and_error_paths():
    L = lib()
    q = torch.zeros(1, 1, 0, 32, device="cuda")
    k = torch.randn(1, 1, 8, 32, device="cuda")
    o, g, _ = L.forward(q, k, k, False, 1.0)
    assert o.shape == (1, 1, 0, 32)
    with pytest.raises(L.FastmaxError) as e:  # nk < nq with the causal mask
        L.forward(k, q, q, True, 1.0)
    assert e.value.status == 2
    with pytest.raises(L.FastmaxError) as e:  # unsupported head dim
        L.forward(torch.randn(1, 1, 8, 24, device="cuda"), torch.randn(1, 1, 8, 24, device="cuda"),
                  torch.randn(1, 1, 8, 24, device="cuda"), False, 1.0)
    assert e.value.status == 2
    # the context is still usable
    x = torch.randn(1, 1, 8, 32, device="cuda")
    o, g, _ = L.forward(x, x, x, True, 0.1)
    assert torch.isfinite(o).all()


def test_no_queries_still_produce_the_key_state_and_zero_key_gradients():
    """nq = 0 with nk > 0: the forward writes state_out (= moments of the keys), the backward returns zero dk, dv."""
    B, H, N, D = 1, 2, 70, 32
    rng = np.random.default_rng(12)
    k, v = (dev(rng.standard_normal((B, H, N, D)).astype(np.float32)) for _ in range(2))
    q = torch.empty(B, H, 0, D, device="cuda")
    L = lib()
    poly = orc.Poly(1.0, 1.0, 0.5, 0.3, 2)
    o, g, s = L.forward(q, k, v, True, poly.inv_temp, order=2, want_state=True)
    _, _, s_ref = L.forward(k, k, v, True, poly.inv_temp, order=2, want_state=True, want_output=False)
    torch.cuda.synchronize()
    assert o.shape[2] == 0 and torch.equal(s, s_ref) and float(s.abs().max()) > 0
    do = torch.empty(B, H, 0, D, device="cuda")
    dq, dk, dv, _ = L.backward(q, k, v, o, g, do, True, poly.inv_temp, order=2)
    torch.cuda.synchronize()
    assert dq.shape[2] == 0 and float(dk.abs().max()) == 0.0 and float(dv.abs().max()) == 0.0


def _launches(L, fn):
    L.profile_collect()
    L.profile(True)
    out = fn()
    torch.cuda.synchronize()
    L.profile(False)
    return out, {k: v[1] for k, v in L.profile_collect().items()}


@pytest.mark.parametrize("causal,order,D", [(True, 2, 32), (True, 1, 64), (False, 2, 32)])
def test_key_moments_are_reused_by_later_calls(causal, order, D):
    """A long sequence with few heads is cut into segments; the per-segment key moments of the first call (a
    state-only call here, as a sequence-parallel rank makes) are handed to the forward and to the backward, which then
    skip their pass over k and v.  Same results as the calls that recompute them, one moment launch instead of three."""
    L = lib()
    B, H, N = 1, 2, 8192
    g = torch.Generator(device="cuda").manual_seed(17)
    q, k, v, do = (torch.randn(B, H, N, D, device="cuda", generator=g) * 0.8 for _ in range(4))
    it = 1.0 / (2.0 * D ** 0.5)
    state_in = None
    if causal:
        k0, v0 = (torch.randn(B, H, 256, D, device="cuda", generator=g) * 0.8 for _ in range(2))
        _, _, state_in = L.forward(k0, k0, v0, True, it, order=order, want_state=True, want_output=False)

    def plain():
        o, gg, _ = L.forward(q, k, v, causal, it, order=order, state_in=state_in)
        dtotal = L.backward(q, k, v, o, gg, do, causal, it, order=order, state_in=state_in, want_dstate=True, want_grads=False)[3]
        return (o, gg) + tuple(L.backward(q, k, v, o, gg, do, causal, it, order=order, state_in=state_in)[:3]) + (dtotal,)

    def reusing():
        km = L.KeyMoments()
        _, _, total = L.forward(k, k, v, causal, it, order=order, want_state=True, want_output=False, key_moments=km)
        assert km.buf is not None
        o, gg, _ = L.forward(q, k, v, causal, it, order=order, state_in=state_in, key_moments=km)
        dtotal = L.backward(q, k, v, o, gg, do, causal, it, order=order, state_in=state_in, want_dstate=True, want_grads=False,
                            key_moments=km)[3]
        assert km.grad_buf is not None
        grads = L.backward(q, k, v, o, gg, do, causal, it, order=order, state_in=state_in, key_moments=km)[:3]
        return (o, gg) + tuple(grads) + (dtotal, total)

    ref, n_plain = _launches(L, plain)
    got, n_reuse = _launches(L, reusing)
    assert n_plain["moments_kv"] == 2 and n_reuse["moments_kv"] == 1, (n_plain, n_reuse)
    assert n_plain["moments_qg"] == 2 and n_reuse["moments_qg"] == 1, (n_plain, n_reuse)
    for a, b in zip(got[:6], ref):
        assert orc.max_norm_err(host(a), host(b)) < 2e-6
    _, _, total_ref = L.forward(k, k, v, causal, it, order=order, want_state=True, want_output=False)
    assert orc.max_norm_err(host(got[6]), host(total_ref)) < 2e-6


def test_key_moments_holder_stays_empty_without_segments():
    """One segment per head (many heads) or a call the tensor-memory kernels take: nothing to reuse, nothing allocated."""
    L = lib()
    g = torch.Generator(device="cuda").manual_seed(3)
    for dtype, shape in ((torch.float32, (4, 40, 256, 32)), (torch.bfloat16, (2, 16, 512, 64))):
        q, k, v = (torch.randn(*shape, device="cuda", generator=g).to(dtype) for _ in range(3))
        km = L.KeyMoments()
        o, gg, _ = L.forward(q, k, v, True, 0.1, order=2, key_moments=km)
        assert km.buf is None
        L.backward(q, k, v, o, gg, q, True, 0.1, order=2, key_moments=km)
    torch.cuda.synchronize()
    assert L.load().fastmax_check_status() == 0
