"""BASELINE configurations at full size, checked through exact sampled rows / columns of the oracle
(O(N D) per sample in float64), since the N x N form does not fit at these sizes."""
import math

import numpy as np
import pytest
import torch

from oracle import fastmax_oracle as orc

pytestmark = pytest.mark.gpu


def host(t):
    return t.detach().float().cpu().numpy().astype(np.float64)


def _check_sampled(q, k, v, do, o, g, dq, dk, dv, causal, poly, heads, nrows, tol, rng, gtol=1e-4):
    B, H, N, D = q.shape
    for (b, h) in heads:
        qh, kh, vh = (host(t[b, h]) for t in (q, k, v))
        doh = host(do[b, h]) if do is not None else None
        oh, gh = host(o[b, h]), host(g[b, h])
        rows = sorted(set([0, 1, N // 2, N - 1] + list(rng.integers(0, N, nrows))))
        o_s, g_s = orc.sampled_forward_rows(qh, kh, vh, rows, causal, poly)
        scale_o = np.abs(oh).max()
        assert np.abs(oh[rows] - o_s).max() / scale_o < tol
        assert np.abs(gh[rows] - g_s).max() / np.abs(g_s).max() < gtol
        if dq is None:
            continue
        dq_s = orc.sampled_dq_rows(qh, kh, vh, oh, gh, doh, rows, causal, poly)
        dk_s, dv_s = orc.sampled_dkv_cols(qh, kh, vh, oh, gh, doh, rows, causal, poly)
        for got, ref in ((dq, dq_s), (dk, dk_s), (dv, dv_s)):
            full = host(got[b, h])
            assert np.abs(full[rows] - ref).max() / np.abs(full).max() < tol


def test_config2_bf16_causal_p2_full_size():
    """B=8, H=16, N=4096, D=64, bf16 inputs, fp32 accumulation, causal, order 2: forward + backward."""
    from reproducing_fastmax_results_b200 import _lib as L

    B, H, N, D = 8, 16, 4096, 64
    torch.manual_seed(0)
    q, k, v, do = (torch.randn(B, H, N, D, device="cuda").to(torch.bfloat16) for _ in range(4))
    poly = orc.Poly(1.0, 1.0, 0.5, 1.0 / (8.0 * math.sqrt(D)), 2)
    o, g, _ = L.forward(q, k, v, True, poly.inv_temp, order=2)
    dq, dk, dv, _ = L.backward(q, k, v, o, g, do, True, poly.inv_temp, order=2)
    rng = np.random.default_rng(0)
    _check_sampled(q, k, v, do, o, g, dq, dk, dv, True, poly, [(0, 0), (3, 7), (7, 15)], 12, 2e-2, rng)
    # causality at full size: perturbing the last key/value leaves every earlier output row unchanged
    k2, v2 = k.clone(), v.clone()
    k2[:, :, -1] += 1.0
    v2[:, :, -1] -= 1.0
    o2, _, _ = L.forward(q[:1], k2[:1], v2[:1], True, poly.inv_temp, order=2)
    assert torch.allclose(o2[:, :, :-1].float(), o[:1, :, :-1].float(), rtol=0, atol=2e-2 * float(o.float().abs().max()))


def test_config3_fp32_long_sequence_full_size():
    """B=1, H=8, N=131072, D=32, fp32, causal, order 2."""
    from reproducing_fastmax_results_b200 import _lib as L

    B, H, N, D = 1, 8, 131072, 32
    torch.manual_seed(0)
    q, k, v, do = (torch.randn(B, H, N, D, device="cuda") for _ in range(4))
    poly = orc.Poly(1.0, 1.0, 0.5, 1.0 / (8.0 * math.sqrt(D)), 2)
    o, g, _ = L.forward(q, k, v, True, poly.inv_temp, order=2)
    dq, dk, dv, _ = L.backward(q, k, v, o, g, do, True, poly.inv_temp, order=2)
    rng = np.random.default_rng(1)
    _check_sampled(q, k, v, do, o, g, dq, dk, dv, True, poly, [(0, 0), (0, 5)], 6, 1e-4, rng)


def test_config4_bf16_noncausal_p1_full_size():
    """B=64, H=12, N=1024, D=64, bf16, order 1, forward only; linearity in v as a size-independent check."""
    from reproducing_fastmax_results_b200 import _lib as L

    B, H, N, D = 64, 12, 1024, 64
    torch.manual_seed(0)
    q, k, v = ((torch.randn(B, H, N, D, device="cuda") * 0.5).to(torch.bfloat16) for _ in range(3))
    poly = orc.Poly(1.0, 1.0, 0.5, 1.0 / (8.0 * math.sqrt(D)), 1)
    o, g, _ = L.forward(q, k, v, False, poly.inv_temp, order=1)
    rng = np.random.default_rng(2)
    _check_sampled(q, k, v, None, o, g, None, None, None, False, poly, [(0, 0), (63, 11)], 8, 2e-2, rng)
    o2, g2, _ = L.forward(q, k, (v.float() * 2).to(torch.bfloat16), False, poly.inv_temp, order=1)
    assert torch.allclose(o2.float(), 2 * o.float(), rtol=2e-2, atol=1e-3)
    assert torch.allclose(g2, g)


def test_config2_shape_with_32_wide_bf16_heads_full_size():
    """B=8, H=16, N=4096, D=32, bf16, causal, order 2: the zero-padded form of the tensor-memory kernels at full size,
    forward + backward against exact sampled rows / columns; and the long float32 sequence of config 3 under the
    "medium" float32 matmul precision (bfloat16 copies, padded, cut into segments) at the bfloat16 tolerance."""
    from reproducing_fastmax_results_b200 import _lib as L
    from reproducing_fastmax_results_b200.attention import FastMax

    B, H, N, D = 8, 16, 4096, 32
    torch.manual_seed(2)
    q, k, v, do = (torch.randn(B, H, N, D, device="cuda").to(torch.bfloat16) for _ in range(4))
    poly = orc.Poly(1.0, 1.0, 0.5, 1.0 / (8.0 * math.sqrt(D)), 2)
    L.profile_collect()
    L.profile(True)
    o, g, _ = L.forward(q, k, v, True, poly.inv_temp, order=2)
    dq, dk, dv, _ = L.backward(q, k, v, o, g, do, True, poly.inv_temp, order=2)
    L.check_status()
    L.profile(False)
    kinds = set(L.profile_collect())
    assert "tc_pad" in kinds and "scan_fwd" not in kinds, kinds
    rng = np.random.default_rng(2)
    _check_sampled(q, k, v, do, o, g, dq, dk, dv, True, poly, [(0, 0), (5, 9)], 10, 2e-2, rng, gtol=2e-3)

    B, H, N = 1, 8, 131072
    q, k, v, do = (torch.randn(B, H, N, D, device="cuda") for _ in range(4))
    before = torch.get_float32_matmul_precision()
    try:
        torch.set_float32_matmul_precision("medium")
        qg, kg, vg = (t.clone().requires_grad_(True) for t in (q, k, v))
        L.profile_collect()
        L.profile(True)
        out = FastMax.apply(qg, kg, vg, None, None, True, 0.0, False, 8.0 * math.sqrt(D), 1.0, 1.0, 0.5, 1.0, 2)
        out.backward(do)
        L.check_status()
        L.profile(False)
    finally:
        torch.set_float32_matmul_precision(before)
    kinds = set(L.profile_collect())
    assert {"tc_pad", "tc_scan_fwd", "state_scan"} <= kinds and "scan_fwd" not in kinds, kinds
    assert out.dtype == torch.float32 and qg.grad.dtype == torch.float32
    # the denominators of the bfloat16 run, for the sampled-row check of the gradients
    qb, kb, vb = (t.bfloat16() for t in (q, k, v))
    _, gb, _ = L.forward(qb, kb, vb, True, poly.inv_temp, order=2)
    rng = np.random.default_rng(3)
    _check_sampled(qb, kb, vb, do.bfloat16(), out.detach(), gb, qg.grad, kg.grad, vg.grad, True, poly, [(0, 3)], 6, 2e-2, rng, gtol=2e-3)
