"""Pins the CPU oracle: golden vectors written by the reference + the reference's own property tests."""
import math
import os

import numpy as np
import pytest
import torch

from cases import CASES, make_inputs
from oracle import fastmax_oracle as orc

GOLD = np.load(os.path.join(os.path.dirname(__file__), "golden", "reference_vectors.npz"))


def _poly(name):
    B, H, N, D, p, mask, nt, scale, upstream = CASES[name]
    return orc.poly_from_normalize_term(D, nt, False, p), mask


@pytest.mark.parametrize("name", sorted(CASES))
def test_naive_matches_reference_outputs_and_grads(name):
    q, k, v, do = make_inputs(name)
    poly, mask = _poly(name)
    o, g = orc.fastmax_naive(q, k, v, mask, poly)
    dq, dk, dv = orc.fastmax_naive_grads(q, k, v, do, mask, poly)
    for impl in ("einops", "score"):
        assert orc.max_norm_err(o, GOLD[f"{name}/{impl}/o"]) < 2e-6
        assert orc.max_norm_err(dq, GOLD[f"{name}/{impl}/dq"]) < 2e-6
    assert orc.max_norm_err(dk, GOLD[f"{name}/einops/dk"]) < 2e-6
    assert orc.max_norm_err(dv, GOLD[f"{name}/einops/dv"]) < 2e-6


@pytest.mark.parametrize("name", sorted(CASES))
def test_factorized_restatement_matches_reference(name):
    q, k, v, do = (torch.from_numpy(x).double() for x in make_inputs(name))
    poly, mask = _poly(name)
    o, dq, dk, dv = orc.fastmax_factorized_fwd_bwd(q, k, v, do, mask, poly)
    assert orc.max_norm_err(o, GOLD[f"{name}/einops/o"]) < 2e-6
    assert orc.max_norm_err(dq, GOLD[f"{name}/einops/dq"]) < 2e-6
    assert orc.max_norm_err(dk, GOLD[f"{name}/einops/dk"]) < 2e-6
    assert orc.max_norm_err(dv, GOLD[f"{name}/einops/dv"]) < 2e-6


@pytest.mark.parametrize("name", sorted(CASES))
@pytest.mark.parametrize("chunk", [16, 64])
def test_streaming_matches_reference(name, chunk):
    q, k, v, do = make_inputs(name)
    poly, mask = _poly(name)
    B, H = q.shape[:2]
    for b in range(B):
        for h in range(H):
            o, g = orc.fastmax_streaming(q[b, h], k[b, h], v[b, h], mask, poly, chunk)
            dq, dk, dv = orc.fastmax_streaming_grads(q[b, h], k[b, h], v[b, h], do[b, h], mask, poly, chunk)
            assert orc.max_norm_err(o, GOLD[f"{name}/einops/o"][b, h]) < 2e-6
            assert orc.max_norm_err(dq, GOLD[f"{name}/einops/dq"][b, h]) < 2e-6
            assert orc.max_norm_err(dk, GOLD[f"{name}/einops/dk"][b, h]) < 2e-6
            assert orc.max_norm_err(dv, GOLD[f"{name}/einops/dv"][b, h]) < 2e-6


def test_streaming_state_carry_splits_a_sequence():
    q, k, v, do = make_inputs("ragged_p2_causal")
    poly, mask = _poly("ragged_p2_causal")
    q, k, v = q[0, 0], k[0, 0], v[0, 0]
    o_full, g_full = orc.fastmax_streaming(q, k, v, True, poly, 8)
    cut = 19
    o1, g1, S = orc.fastmax_streaming(q[:cut], k[:cut], v[:cut], True, poly, 8, return_state=True)
    assert np.allclose(S, orc.moment_state(k[:cut], v[:cut], poly))
    o2, g2 = orc.fastmax_streaming(q[cut:], k[cut:], v[cut:], True, poly, 8, state_in=S)
    assert np.allclose(np.concatenate([o1, o2]), o_full, atol=1e-12)
    # the same thing expressed as nk > nq (queries aligned to the last nq keys, fwd.cu:161-172)
    o3, g3 = orc.fastmax_streaming(q[cut:], k, v, True, poly, 8)
    assert np.allclose(o3, o_full[cut:], atol=1e-12)
    o4, g4 = orc.fastmax_naive(q[cut:], k, v, True, poly)
    assert np.allclose(o4, o_full[cut:], atol=1e-12)


@pytest.mark.parametrize("name", ["small_p2_causal", "small_p2_noncausal", "ragged_p2_causal"])
def test_sampled_rows_and_columns(name):
    q, k, v, do = make_inputs(name)
    poly, mask = _poly(name)
    q, k, v, do = q[0, 1], k[0, 1], v[0, 1], do[0, 1]
    o, g = orc.fastmax_naive(q, k, v, mask, poly)
    dq, dk, dv = orc.fastmax_naive_grads(q, k, v, do, mask, poly)
    rows = [0, 5, q.shape[0] - 1]
    o_s, g_s = orc.sampled_forward_rows(q, k, v, rows, mask, poly)
    assert np.allclose(o_s, o[rows], atol=1e-12) and np.allclose(g_s, g[rows], atol=1e-12)
    assert np.allclose(orc.sampled_dq_rows(q, k, v, o, g, do, rows, mask, poly), dq[rows], atol=1e-12)
    dk_s, dv_s = orc.sampled_dkv_cols(q, k, v, o, g, do, rows, mask, poly)
    assert np.allclose(dk_s, dk[rows], atol=1e-12) and np.allclose(dv_s, dv[rows], atol=1e-12)


@pytest.mark.parametrize("name", ["small_p2_causal", "small_p2_noncausal"])
def test_normalize_matches_reference(name):
    q, k, v, do = make_inputs(name)
    assert orc.max_norm_err(orc.normalize(q), GOLD[f"{name}/normalize/q"]) < 2e-6
    assert orc.max_norm_err(orc.normalize(k), GOLD[f"{name}/normalize/k"]) < 2e-6
    assert orc.max_norm_err(orc.normalize_grad(q, do), GOLD[f"{name}/normalize/dq"]) < 2e-6
    assert orc.max_norm_err(orc.normalize_grad(k, do), GOLD[f"{name}/normalize/dk"]) < 2e-6
    # normalised attention end to end (einops tensors_normalized=True: temperature 1)
    B, H, N, D, p, mask, nt, scale, upstream = CASES[name]
    poly = orc.Poly(1.0, 1.0, 0.5, 1.0, p)
    qn, kn = orc.normalize(q), orc.normalize(k)
    o, g = orc.fastmax_naive(qn, kn, v, mask, poly)
    dqn, dkn, dv = orc.fastmax_naive_grads(qn, kn, v, do, mask, poly)
    assert orc.max_norm_err(o, GOLD[f"{name}/normalized_attention/o"]) < 2e-6
    assert orc.max_norm_err(dv, GOLD[f"{name}/normalized_attention/dv"]) < 2e-6
    assert orc.max_norm_err(orc.normalize_grad(q, dqn), GOLD[f"{name}/normalized_attention/dq"]) < 2e-6
    assert orc.max_norm_err(orc.normalize_grad(k, dkn), GOLD[f"{name}/normalized_attention/dk"]) < 2e-6


# ---- the reference's own property tests (test/test_einops_fastmax.py), restated for the oracle ----
@pytest.fixture
def tiny():
    rng = np.random.default_rng(123)
    B, H, N, D = 5, 4, 3, 2          # test.py:17-23
    return (rng.standard_normal((B, H, N, D)) for _ in range(3))


@pytest.mark.parametrize("p", [1, 2])
@pytest.mark.parametrize("mask", [False, True])
def test_reference_property_forward(tiny, p, mask):
    """test.py:77-129: factorised output == row-normalised N x N attention with f = 1+x(+x^2/2), < 1e-7."""
    q, k, v = tiny
    D = q.shape[-1]
    poly = orc.poly_from_normalize_term(D, 1.0, False, p)
    s = np.einsum("bhid,bhjd->bhij", q, k) / math.sqrt(D)
    f = 1 + s + (s * s / 2 if p == 2 else 0)
    if mask:
        f = np.tril(f)
    expect = np.einsum("bhij,bhjd->bhid", f / f.sum(-1, keepdims=True), v)
    got = orc.fastmax_factorized(*(torch.from_numpy(x) for x in (q, k, v)), mask, poly).numpy()
    assert np.abs(got - expect).max() < 1e-7
    for b in range(q.shape[0]):
        for h in range(q.shape[1]):
            o, _ = orc.fastmax_streaming(q[b, h], k[b, h], v[b, h], mask, poly, chunk=2)
            assert np.abs(o - expect[b, h]).max() < 1e-7


@pytest.mark.parametrize("p", [1, 2])
@pytest.mark.parametrize("mask", [False, True])
@pytest.mark.parametrize("nt", [1.0, 42.0])
def test_reference_property_gradcheck(tiny, p, mask, nt):
    """test.py:131-225: finite-difference check (eps 1e-6, atol 1e-4) of the analytic gradients."""
    q, k, v = tiny
    q, k, v = q[0, 0], k[0, 0], v[0, 0]
    poly = orc.poly_from_normalize_term(q.shape[-1], nt, False, p)
    rng = np.random.default_rng(5)
    do = rng.standard_normal(v.shape)
    dq, dk, dv = orc.fastmax_naive_grads(q, k, v, do, mask, poly)
    sq, sk, sv = orc.fastmax_streaming_grads(q, k, v, do, mask, poly, chunk=2)
    eps = 1e-6
    for x, gx, sx in ((q, dq, sq), (k, dk, sk), (v, dv, sv)):
        num = np.zeros_like(x)
        for idx in np.ndindex(*x.shape):
            old = x[idx]
            x[idx] = old + eps
            fp = (orc.fastmax_naive(q, k, v, mask, poly)[0] * do).sum()
            x[idx] = old - eps
            fm = (orc.fastmax_naive(q, k, v, mask, poly)[0] * do).sum()
            x[idx] = old
            num[idx] = (fp - fm) / (2 * eps)
        assert np.abs(num - gx).max() < 1e-4
        assert np.abs(sx - gx).max() < 1e-9


def test_reference_property_causality(tiny):
    """test.py:257-274: with the mask, output row l must not depend on keys/values after l."""
    q, k, v = tiny
    q, k, v = q[0, 0], k[0, 0], v[0, 0]
    poly = orc.poly_from_normalize_term(2, 1.0, False, 2)
    o1, _ = orc.fastmax_streaming(q, k, v, True, poly, chunk=2)
    k2, v2 = k.copy(), v.copy()
    k2[-1] += 10.0
    v2[-1] -= 7.0
    o2, _ = orc.fastmax_streaming(q, k2, v2, True, poly, chunk=2)
    assert np.allclose(o1[:-1], o2[:-1]) and not np.allclose(o1[-1], o2[-1])


def test_key_prologue_and_output_noise_follow_the_reference_kernels():
    """apply_rpe_and_temp with its RPE line (fastmax_cuda_forward.cu:288-289) and apply_dropout (:346), as loops."""
    rng = np.random.default_rng(0)
    nk, d = 7, 4
    k = rng.standard_normal((3, nk, d))
    rpe = rng.standard_normal((2 * nk - 1, d))
    ref = k.copy()
    for l in range(nk):
        ref[:, l] = ref[:, l] / 2.5 + rpe[(l + nk) % (2 * nk - 1)]
    assert np.allclose(orc.key_prologue(k, 1 / 2.5, rpe), ref)
    assert np.allclose(orc.key_prologue(k, 1 / 2.5), k / 2.5)
    o, noise = rng.standard_normal((2, 5, d)), rng.standard_normal((2, 5, d))
    assert np.allclose(orc.output_noise(o, noise, 0.1), o * (1 + 0.1 * noise))
    assert np.allclose(orc.output_noise(o, noise, 0.0), o)   # what the reference actually runs (scale 0.0, :443)
