"""The reference-facing operator: `fastmax_cuda.forwardpass/backwardpass`, the reference's autograd.Function
twin and the FastMax Function, checked against the oracle and the golden vectors."""
import math
import os

import numpy as np
import pytest
import torch

from cases import CASES, make_inputs
from oracle import fastmax_oracle as orc

pytestmark = pytest.mark.gpu
GOLD = np.load(os.path.join(os.path.dirname(__file__), "golden", "reference_vectors.npz"))


def host(t):
    return t.detach().float().cpu().numpy().astype(np.float64)


@pytest.mark.parametrize("mask", [False, True])
@pytest.mark.parametrize("p", [1, 2])
def test_forwardpass_backwardpass_contract(mask, p):
    """(n, b*h, d) float32 in, (nq, b*h, d+1) out with the denominator in the last column; k is scaled by
    1/temperature in place and the gradients are w.r.t. the scaled k (fastmax_cuda_forward.cu:282-292,
    transformer/model.py:74)."""
    import reproducing_fastmax_results_b200 as pkg

    ext = pkg.load_extension()
    n, bh, d, t = 50, 6, 32, 3.0
    rng = np.random.default_rng(1)
    q, k, v, do = (rng.standard_normal((n, bh, d)).astype(np.float32) for _ in range(4))
    qd, kd, vd, dod = (torch.from_numpy(x).cuda() for x in (q, k, v, do))
    noise = torch.zeros_like(qd)
    rpe = torch.zeros(2 * n - 1, d, device="cuda")
    o = ext.forwardpass(qd, kd, vd, noise, rpe, mask, 0.1, False, t, 1.0, 1.0, 0.5, 1.0, p)
    assert o.shape == (n, bh, d + 1)
    assert torch.allclose(kd, torch.from_numpy(k).cuda() / t)
    poly = orc.Poly(1.0, 1.0, 0.5, 1.0 / t, p)
    qh, kh, vh, doh = (np.transpose(x, (1, 0, 2)) for x in (q, k, v, do))
    o_ref, g_ref = orc.fastmax_naive(qh, kh, vh, mask, poly)
    assert orc.max_norm_err(host(o[:, :, :d]).transpose(1, 0, 2), o_ref) < 1e-4
    assert orc.max_norm_err(host(o[:, :, d]).T, g_ref) < 1e-4
    gq, gk, gv = ext.backwardpass(qd, kd, vd, o, dod, mask, 1.0, 1.0, 0.5, p)
    dq_ref, dk_ref, dv_ref = orc.fastmax_naive_grads(qh, kh, vh, doh, mask, poly)
    assert orc.max_norm_err(host(gq).transpose(1, 0, 2), dq_ref) < 1e-4
    assert orc.max_norm_err(host(gk).transpose(1, 0, 2) / t, dk_ref) < 1e-4
    assert orc.max_norm_err(host(gv).transpose(1, 0, 2), dv_ref) < 1e-4
    assert torch.equal(dod, torch.from_numpy(do).cuda())  # the upstream gradient is not modified


@pytest.mark.parametrize("fn_name", ["FastMax", "FASTMultiHeadAttention_Function"])
@pytest.mark.parametrize("name", ["small_p2_causal", "small_p1_noncausal", "cfg1_p2_noncausal"])
def test_autograd_functions_match_reference(fn_name, name):
    import reproducing_fastmax_results_b200 as pkg

    fn = getattr(pkg, fn_name)
    B, H, N, D, p, mask, nt, scale, upstream = CASES[name]
    q, k, v, do = (torch.from_numpy(x).cuda() for x in make_inputs(name))
    q.requires_grad_(True), k.requires_grad_(True), v.requires_grad_(True)
    noise = torch.zeros_like(q)
    rpe = pkg.rpe_matrix_creator(N, D, q.device, q.dtype)
    o = fn.apply(q, k, v, noise, rpe, mask, 0.0, False, nt * math.sqrt(D), 1.0, 1.0, 0.5, 1.0, p)
    o.backward(do)
    for got, key in ((o, "o"), (q.grad, "dq"), (k.grad, "dk"), (v.grad, "dv")):
        assert orc.max_norm_err(host(got), GOLD[f"{name}/einops/{key}"]) < 1e-4, key


@pytest.mark.parametrize("name", ["small_p2_causal", "small_p2_noncausal"])
def test_fastmax_normalized_attention_matches_reference(name):
    """normalize=True: q, k normalised as fastattention_einops.normalize does, gradient through it exact."""
    import reproducing_fastmax_results_b200 as pkg

    B, H, N, D, p, mask, nt, scale, upstream = CASES[name]
    q, k, v, do = (torch.from_numpy(x).cuda() for x in make_inputs(name))
    q.requires_grad_(True), k.requires_grad_(True), v.requires_grad_(True)
    o = pkg.fastmax(q, k, v, mask=mask, normalize=True, p=p)
    o.backward(do)
    for got, key in ((o, "o"), (q.grad, "dq"), (k.grad, "dk"), (v.grad, "dv")):
        assert orc.max_norm_err(host(got), GOLD[f"{name}/normalized_attention/{key}"]) < 1e-4, key


def test_fastmax_bf16_transposed_views_and_module():
    import reproducing_fastmax_results_b200 as pkg

    B, N, H, D = 2, 128, 4, 64
    torch.manual_seed(0)
    x = torch.randn(3, B, N, H, D, device="cuda", dtype=torch.bfloat16)
    q, k, v = (x[i].transpose(1, 2).detach().requires_grad_(True) for i in range(3))
    do = torch.randn(B, H, N, D, device="cuda", dtype=torch.bfloat16)
    o = pkg.fastmax_custom(q, k, v, None, None, True, 0.0, False, 8.0 * math.sqrt(D), 1.0, 1.0, 0.5, 1.0, 2)
    assert o.dtype == torch.bfloat16
    o.backward(do)
    poly = orc.Poly(1.0, 1.0, 0.5, 1.0 / (8.0 * math.sqrt(D)), 2)
    o_ref, _ = orc.fastmax_naive(host(q), host(k), host(v), True, poly)
    dq_ref, dk_ref, dv_ref = orc.fastmax_naive_grads(host(q), host(k), host(v), host(do), True, poly)
    assert orc.max_norm_err(host(o), o_ref) < 2e-2
    assert orc.max_norm_err(host(q.grad), dq_ref) < 2e-2
    assert orc.max_norm_err(host(k.grad), dk_ref) < 2e-2
    assert orc.max_norm_err(host(v.grad), dv_ref) < 2e-2
    assert pkg.FASTMultiHeadAttention(use_custom_gradient=False)(q, k, v) == 0


def test_host_pipeline_matches_the_single_call():
    """HostFastmax streams batch slices from pinned host memory through the GPU; every (batch, head) is
    independent, so the results equal one call over the whole batch (up to the order of float32 adds)."""
    from reproducing_fastmax_results_b200 import _lib as L
    from reproducing_fastmax_results_b200.host_pipeline import HostFastmax

    B, H, N, D = 5, 16, 260, 64
    g = torch.Generator().manual_seed(11)
    hq, hk, hv, hdo = (torch.randn(B, H, N, D, generator=g).bfloat16().pin_memory() for _ in range(4))
    outs = [torch.empty_like(hq).pin_memory() for _ in range(4)]
    temperature = 2.0 * math.sqrt(D)
    for pieces in (None, 2):
        op = HostFastmax(mask=True, temperature=temperature, p=2, pieces=pieces)
        for _ in range(2):   # the second call reuses the device buffers
            for t in outs:
                t.zero_()
            op.forward_backward(hq, hk, hv, hdo, *outs)
        q, k, v, do = (t.cuda() for t in (hq, hk, hv, hdo))
        o, gg, _ = L.forward(q, k, v, True, 1.0 / temperature, order=2)
        ref = (o,) + tuple(L.backward(q, k, v, o, gg, do, True, 1.0 / temperature, order=2)[:3])
        torch.cuda.synchronize()
        for got, want in zip(outs, ref):
            w = want.float().cpu()
            assert float((got.float() - w).abs().max()) <= 2e-2 * float(w.abs().max())


def test_forward_backward_replay_from_a_cuda_graph():
    """The launch sequences contain no synchronisation and no allocation of their own, so a caller can capture
    them (internal side streams included: they fork from and join back into the capturing stream) and replay."""
    from reproducing_fastmax_results_b200 import _lib as L

    B, H, N, D = 2, 16, 384, 64
    g = torch.Generator(device="cuda").manual_seed(5)
    q, k, v, do = (torch.randn(B, H, N, D, device="cuda", generator=g).bfloat16() for _ in range(4))
    it = 1.0 / (2.0 * math.sqrt(D))

    def run():
        o, gg, _ = L.forward(q, k, v, True, it, order=2)
        return (o,) + tuple(L.backward(q, k, v, o, gg, do, True, it, order=2)[:3])

    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):   # warm-up outside the capture: lazy initialisation (streams, tensor-map encoder)
        ref = [t.clone() for t in run()]
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        outs = run()
    for _ in range(2):
        q.copy_(torch.randn(B, H, N, D, device="cuda", generator=g).bfloat16())   # new inputs in the captured buffers
        graph.replay()
        torch.cuda.synchronize()
        L.check_status()
        want = run()
        torch.cuda.synchronize()
        for a, b in zip(outs, want):
            assert float((a.float() - b.float()).abs().max()) <= 5e-3 * float(b.float().abs().max()) + 1e-6
    assert float((ref[0].float() - outs[0].float()).abs().max()) > 0.0   # the replays really used the new q


def test_fastmax_keeps_the_head_split_layout_so_the_merge_is_free():
    """q, k, v as the (b,n,h,d)->(b,h,n,d) views of a projection (transformer/model.py:283-285): the output and the
    gradients come back in the same memory layout, so `transpose(1, 2).contiguous()` (model.py:335) copies nothing."""
    import reproducing_fastmax_results_b200 as pkg

    B, N, H, D = 2, 80, 4, 32
    torch.manual_seed(4)
    base = [torch.randn(B, N, H * D, device="cuda", requires_grad=True) for _ in range(3)]
    q, k, v = (t.view(B, N, H, D).transpose(1, 2) for t in base)
    o = pkg.fastmax_custom(q, k, v, None, None, True, 0.0, False, 4.0, 1.0, 1.0, 0.5, 1.0, 2)
    assert o.stride() == q.stride()
    merged = o.transpose(1, 2)
    assert merged.is_contiguous() and merged.contiguous().data_ptr() == o.data_ptr()
    merged.reshape(B, N, H * D).sum().backward()
    poly = orc.Poly(1.0, 1.0, 0.5, 0.25, 2)
    qh, kh, vh = (host(t) for t in (q, k, v))
    o_ref, _ = orc.fastmax_naive(qh, kh, vh, True, poly)
    assert orc.max_norm_err(host(o), o_ref) < 1e-4
    dq_ref, _, _ = orc.fastmax_naive_grads(qh, kh, vh, np.ones_like(qh), True, poly)
    assert orc.max_norm_err(host(base[0].grad).reshape(B, N, H, D).transpose(0, 2, 1, 3), dq_ref) < 1e-4


def test_extension_calls_release_the_gil():
    """A Python thread keeps running while another one is inside the extension (the reference's binding holds the GIL
    and synchronises the device, fastmax_cuda_forward.cu:423-444; this extension does neither)."""
    import threading
    import time

    import reproducing_fastmax_results_b200 as pkg

    ext = pkg.load_extension()
    x = torch.randn(4, 16, 2048, 64, device="cuda").bfloat16()
    ticks = []
    stop = threading.Event()

    def ticker():
        while not stop.is_set():
            ticks.append(time.perf_counter())
            time.sleep(0)

    th = threading.Thread(target=ticker)
    th.start()
    for _ in range(20):
        ext.forward(x, x, x, True, 0.1, 1.0, 1.0, 0.5, 2)
    torch.cuda.synchronize()
    stop.set()
    th.join()
    assert len(ticks) > 20


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_key_prologue_and_output_noise_kernels(dtype):
    """fastmax_key_prologue / fastmax_output_noise through the C ABI against the oracle's restatement of
    apply_rpe_and_temp (with its commented-out RPE line) and apply_dropout, on strided views."""
    from reproducing_fastmax_results_b200 import _lib as L

    B, H, N, D = 2, 3, 37, 32
    rng = np.random.default_rng(21)
    k, x, noise = (rng.standard_normal((B, N, H, D)).astype(np.float32) for _ in range(3))
    rpe = rng.standard_normal((2 * N - 1, D)).astype(np.float32)
    kd, xd, nd = (torch.from_numpy(a).cuda().to(dtype).transpose(1, 2) for a in (k, x, noise))
    tol = 1e-6 if dtype == torch.float32 else 1e-2
    k_ref = orc.key_prologue(host(kd), 0.3, rpe)
    L.key_prologue(kd, 0.3, torch.from_numpy(rpe).cuda())
    assert orc.max_norm_err(host(kd), k_ref) < tol
    k2 = torch.from_numpy(k).cuda().to(dtype).transpose(1, 2)
    L.key_prologue(k2, 0.5)
    assert orc.max_norm_err(host(k2), orc.key_prologue(host(torch.from_numpy(k).cuda().to(dtype).transpose(1, 2)), 0.5)) < tol
    out = L.output_noise(xd, nd, 0.1)
    assert orc.max_norm_err(host(out), orc.output_noise(host(xd), host(nd), 0.1)) < tol


def test_fastmax_with_rpe_and_noise_dropout_switched_on():
    """The two optional steps inside the operator, forward and gradients, against the oracle composed the same way."""
    import reproducing_fastmax_results_b200 as pkg

    B, H, N, D, t, rate = 2, 3, 40, 32, 3.0, 0.1
    rng = np.random.default_rng(23)
    q, k, v, do, noise = (rng.standard_normal((B, H, N, D)).astype(np.float32) for _ in range(5))
    rpe = 0.3 * rng.standard_normal((2 * N - 1, D)).astype(np.float32)
    qd, kd, vd = (torch.from_numpy(a).cuda().requires_grad_(True) for a in (q, k, v))
    dod, nd, rd = (torch.from_numpy(a).cuda() for a in (do, noise, rpe))
    op = pkg.FASTMultiHeadAttention(apply_rpe=True, noise_dropout=True)
    out = op(qd, kd, vd, nd, rd, True, rate, False, t, 1.0, 1.0, 0.5, 1.0, 2)
    out.backward(dod)
    poly = orc.Poly(1.0, 1.0, 0.5, 1.0, 2)
    k_op = orc.key_prologue(k, 1.0 / t, rpe)
    o_ref, _ = orc.fastmax_naive(q, k_op, v, True, poly)
    assert orc.max_norm_err(host(out), orc.output_noise(o_ref, noise, rate)) < 1e-4
    dq_ref, dk_ref, dv_ref = orc.fastmax_naive_grads(q, k_op, v, orc.output_noise(do, noise, rate), True, poly)
    assert orc.max_norm_err(host(qd.grad), dq_ref) < 1e-4
    assert orc.max_norm_err(host(kd.grad), dk_ref / t) < 1e-4
    assert orc.max_norm_err(host(vd.grad), dv_ref) < 1e-4
    # default switches: the arguments are ignored, as in the reference
    plain = pkg.fastmax_custom(qd, kd, vd, nd, rd, True, rate, False, t, 1.0, 1.0, 0.5, 1.0, 2)
    o_plain, _ = orc.fastmax_naive(q, k, v, True, orc.Poly(1.0, 1.0, 0.5, 1.0 / t, 2))
    assert orc.max_norm_err(host(plain), o_plain) < 1e-4


@pytest.mark.parametrize("which", ["FastMax", "FASTMultiHeadAttention_Function"])
@pytest.mark.parametrize("normalize", [False, True])
def test_float32_callers_reach_the_tensor_memory_kernels_under_medium_matmul_precision(which, normalize):
    """torch.set_float32_matmul_precision("medium") is PyTorch's permission to compute float32 matmuls in bfloat16.
    With it, float32 q, k, v of a shape the tensor-memory kernels take run there (on bfloat16 copies; inputs, outputs and
    gradients stay float32) and agree with the exact float32 engine to the bfloat16 tolerance; without it nothing changes."""
    import reproducing_fastmax_results_b200 as pkg
    from reproducing_fastmax_results_b200 import _lib
    from reproducing_fastmax_results_b200.attention import FASTMultiHeadAttention_Function, FastMax

    B, H, N, D = 2, 16, 384, 64
    g = torch.Generator(device="cuda").manual_seed(5)
    q0, k0, v0, do = (torch.randn(B, H, N, D, device="cuda", generator=g) * 0.6 for _ in range(4))
    noise, rpe = torch.zeros_like(q0), torch.zeros(2 * N - 1, D, device="cuda")
    temperature = 1.0 if normalize else 2.0 * math.sqrt(D)
    if which == "FASTMultiHeadAttention_Function" and normalize:
        pytest.skip("the reference's own Function ignores the normalisation in its backward")

    def run():
        q, k, v = (t.clone().requires_grad_(True) for t in (q0, k0, v0))
        _lib.profile_collect()
        _lib.profile(True)
        if which == "FastMax":
            o = FastMax.apply(q, k, v, noise, rpe, True, 0.0, normalize, temperature, 1.0, 1.0, 0.5, 1.0, 2)
        else:
            o = FASTMultiHeadAttention_Function.apply(q, k, v, noise, rpe, True, 0.0, normalize, temperature, 1.0, 1.0, 0.5, 1.0, 2)
        o.backward(do)
        torch.cuda.synchronize()
        _lib.profile(False)
        kinds = set(_lib.profile_collect())
        assert o.dtype == torch.float32 and q.grad.dtype == torch.float32
        return (o.detach(), q.grad, k.grad, v.grad), kinds

    pkg.load_extension()
    before = torch.get_float32_matmul_precision()
    try:
        torch.set_float32_matmul_precision("highest")
        exact, kinds_exact = run()
        assert "tc_scan_fwd" not in kinds_exact and "scan_fwd" in kinds_exact, kinds_exact
        torch.set_float32_matmul_precision("medium")
        fast, kinds_fast = run()
        assert {"tc_scan_fwd", "tc_scan_bwd_q", "tc_scan_bwd_kv", "tc_scan_bwd_dv"} <= kinds_fast, kinds_fast
        assert not ({"scan_fwd", "scan_bwd_q", "scan_bwd_kv"} & kinds_fast), kinds_fast
        for a, b in zip(fast, exact):
            assert orc.max_norm_err(host(a), host(b)) < 2e-2
        # a shape the tensor-memory kernels do not take (head dim 16) stays on the exact engine, in float32
        q, k, v = (torch.randn(2, 16, 128, 16, device="cuda", generator=g) for _ in range(3))
        _lib.profile_collect()
        _lib.profile(True)
        FastMax.apply(q, k, v, None, None, True, 0.0, False, 8.0, 1.0, 1.0, 0.5, 1.0, 2)
        torch.cuda.synchronize()
        _lib.profile(False)
        assert "scan_fwd" in set(_lib.profile_collect())
    finally:
        torch.set_float32_matmul_precision(before)


def test_medium_matmul_precision_with_every_option_of_the_operator_switched_on():
    """Normalisation, RPE add and noise dropout around the bfloat16 attention of a float32 caller under the "medium"
    float32 matmul precision: outputs and all three gradients agree with the exact float32 run to the bfloat16 tolerance."""
    import reproducing_fastmax_results_b200 as pkg
    from reproducing_fastmax_results_b200 import _lib

    B, H, N, D, rate = 2, 16, 256, 32, 0.1   # 32-wide heads: zero-padded on top
    g = torch.Generator(device="cuda").manual_seed(8)
    q0, k0, v0, do, noise = (torch.randn(B, H, N, D, device="cuda", generator=g) * 0.7 for _ in range(5))
    rpe = 0.05 * torch.randn(2 * N - 1, D, device="cuda", generator=g)
    op = pkg.FASTMultiHeadAttention(apply_rpe=True, noise_dropout=True)

    def run():
        q, k, v = (t.clone().requires_grad_(True) for t in (q0, k0, v0))
        _lib.profile_collect()
        _lib.profile(True)
        out = op(q, k, v, noise, rpe, True, rate, True, 1.0, 1.0, 1.0, 0.5, 1.0, 2)
        out.backward(do)
        torch.cuda.synchronize()
        _lib.profile(False)
        assert out.dtype == torch.float32
        return (out.detach(), q.grad, k.grad, v.grad), set(_lib.profile_collect())

    before = torch.get_float32_matmul_precision()
    try:
        torch.set_float32_matmul_precision("highest")
        exact, kinds_exact = run()
        torch.set_float32_matmul_precision("medium")
        fast, kinds_fast = run()
    finally:
        torch.set_float32_matmul_precision(before)
    assert "scan_fwd" in kinds_exact and "tc_scan_fwd" not in kinds_exact
    assert {"tc_pad", "tc_scan_fwd", "tc_scan_bwd_q"} <= kinds_fast and "scan_fwd" not in kinds_fast, kinds_fast
    for a, b, name in zip(fast, exact, ("out", "dq", "dk", "dv")):
        assert orc.max_norm_err(host(a), host(b)) < 2e-2, name
