"""The tcgen05 / TMEM kernels (bf16, head dim 64, order 2, causal) against the CPU oracle and against the
CUDA-core engine on the same inputs."""
import math

import numpy as np
import pytest
import torch

from oracle import fastmax_oracle as orc

pytestmark = pytest.mark.gpu


def host(t):
    return t.detach().float().cpu().numpy().astype(np.float64)


SHAPES = [  # B, H, nq, nk
    (2, 8, 128, 128),
    (2, 8, 300, 300),      # ragged tail
    (1, 16, 1000, 1000),
    (2, 8, 200, 333),      # nk > nq: prefix keys without queries
    (1, 16, 64, 64),       # shorter than one chunk
]


@pytest.mark.parametrize("shape", SHAPES)
def test_tensorcore_forward_matches_oracle(shape):
    from reproducing_fastmax_results_b200 import _lib as L

    B, H, nq, nk = shape
    D = 64
    rng = np.random.default_rng(nq + nk)
    q = torch.from_numpy(rng.standard_normal((B, H, nq, D)).astype(np.float32)).cuda().bfloat16()
    k = torch.from_numpy(rng.standard_normal((B, H, nk, D)).astype(np.float32)).cuda().bfloat16()
    v = torch.from_numpy(rng.standard_normal((B, H, nk, D)).astype(np.float32)).cuda().bfloat16()
    poly = orc.Poly(1.0, 1.0, 0.5, 1.0 / (2.0 * math.sqrt(D)), 2)
    before = L.profile_collect()
    L.profile(True)
    o, g, _ = L.forward(q, k, v, True, poly.inv_temp, order=2)
    L.check_status()
    L.profile(False)
    kinds = L.profile_collect()
    assert "tc_scan_fwd" in kinds, f"tensor-core kernel did not run: {kinds}"
    o_ref, g_ref = orc.fastmax_naive(host(q), host(k), host(v), True, poly)
    assert orc.max_norm_err(host(g), g_ref) < 2e-2
    assert orc.max_norm_err(host(o), o_ref) < 2e-2
    o2, g2, _ = L.forward(q, k, v, True, poly.inv_temp, order=2, flags=L.FLAG_NO_TENSOR_CORES)
    assert orc.max_norm_err(host(o), host(o2)) < 2e-2


@pytest.mark.parametrize("shape", SHAPES)
def test_tensorcore_backward_matches_oracle(shape):
    from reproducing_fastmax_results_b200 import _lib as L

    B, H, nq, nk = shape
    D = 64
    rng = np.random.default_rng(7 * nq + nk)
    q = torch.from_numpy(rng.standard_normal((B, H, nq, D)).astype(np.float32)).cuda().bfloat16()
    k = torch.from_numpy(rng.standard_normal((B, H, nk, D)).astype(np.float32)).cuda().bfloat16()
    v = torch.from_numpy(rng.standard_normal((B, H, nk, D)).astype(np.float32)).cuda().bfloat16()
    do = torch.from_numpy(rng.standard_normal((B, H, nq, D)).astype(np.float32)).cuda().bfloat16()
    poly = orc.Poly(1.0, 1.0, 0.5, 1.0 / (2.0 * math.sqrt(D)), 2)
    o, g, _ = L.forward(q, k, v, True, poly.inv_temp, order=2)
    L.profile_collect()
    L.profile(True)
    dq, dk, dv, _ = L.backward(q, k, v, o, g, do, True, poly.inv_temp, order=2)
    L.check_status()
    L.profile(False)
    kinds = L.profile_collect()
    for name in ("tc_scan_bwd_q", "tc_scan_bwd_kv", "tc_intra_bwd"):
        assert name in kinds, f"{name} did not run: {kinds}"
    dq_ref, dk_ref, dv_ref = orc.fastmax_naive_grads(host(q), host(k), host(v), host(do), True, poly)
    errs = {n: orc.max_norm_err(host(a), b) for n, a, b in (("dq", dq, dq_ref), ("dk", dk, dk_ref), ("dv", dv, dv_ref))}
    assert max(errs.values()) < 2e-2, errs
