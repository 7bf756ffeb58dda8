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


def test_single_stream_flag_gives_the_same_results():
    """FASTMAX_FLAG_SINGLE_STREAM keeps every launch on the caller's stream; the default runs the independent
    scans side by side on internal streams.  Both orders of the float32 reduce-adds must agree to rounding."""
    from reproducing_fastmax_results_b200 import _lib as L

    B, H, N, D = 2, 8, 700, 64
    rng = np.random.default_rng(17)
    q, k, v, do = (torch.from_numpy(rng.standard_normal((B, H, N, D)).astype(np.float32)).cuda().bfloat16() for _ in range(4))
    it = 1.0 / (2.0 * math.sqrt(D))
    outs = []
    for flags in (0, L.FLAG_SINGLE_STREAM):
        o, g, _ = L.forward(q, k, v, True, it, order=2, flags=flags)
        dq, dk, dv, _ = L.backward(q, k, v, o, g, do, True, it, order=2, flags=flags)
        torch.cuda.synchronize()
        L.check_status()
        outs.append([host(t) for t in (o, dq, dk, dv)])
    for a, b in zip(*outs):
        assert orc.max_norm_err(a, b) < 5e-3


def test_wait_histogram_is_empty_after_clean_runs():
    from reproducing_fastmax_results_b200 import _lib as L

    lib = L.load()
    x = torch.randn(1, 16, 300, 64, device="cuda").bfloat16()
    o, g, _ = L.forward(x, x, x, True, 0.1, order=2)
    torch.cuda.synchronize()
    assert lib.fastmax_check_status() == 0
    assert L.wait_histogram() == {}
    assert lib.fastmax_debug_wait_histogram(None, 256) == 1  # FASTMAX_ERR_INVALID_ARGUMENT


def test_a_bounded_wait_that_runs_out_is_reported_and_the_context_stays_usable():
    """The failure path of the device-side waits (bounded wait -> wait-site record -> status word -> host): the
    test-only kernel waits ~1 ms on a barrier nobody signals and gives up; no production kernel is disturbed."""
    from reproducing_fastmax_results_b200 import _lib as L

    lib = L.load()
    torch.cuda.synchronize()
    assert lib.fastmax_check_status() == 0 and L.wait_histogram() == {}
    stream = torch.cuda.current_stream().cuda_stream
    assert lib.fastmax_debug_wait_selftest(stream) == 0
    torch.cuda.synchronize()
    assert lib.fastmax_check_status() == 5        # FASTMAX_ERR_DEVICE_TIMEOUT, reported once ...
    assert lib.fastmax_check_status() == 0        # ... and cleared by the read
    assert L.wait_histogram() == {99: 1}          # the wait site that gave up, one thread block
    assert L.wait_histogram() == {}
    # the next ordinary call works and is clean
    x = torch.randn(1, 16, 300, 64, device="cuda").bfloat16()
    o, g, _ = L.forward(x, x, x, True, 0.1, order=2)
    torch.cuda.synchronize()
    assert lib.fastmax_check_status() == 0 and torch.isfinite(o.float()).all()
    with pytest.raises(L.FastmaxError):           # the Python helper turns the status into an exception
        lib.fastmax_debug_wait_selftest(stream)
        L.check_status()
    assert L.wait_histogram() == {99: 1}


@pytest.mark.parametrize("shape", [(1, 13, 129, 129), (1, 16, 257, 385), (3, 5, 1024, 1024)])
def test_tensorcore_more_shapes_forward_backward(shape):
    """Chunk-boundary sizes, a key prefix that is not a multiple of the chunk, and head counts that are not a
    multiple of anything."""
    from reproducing_fastmax_results_b200 import _lib as L

    B, H, nq, nk = shape
    D = 64
    rng = np.random.default_rng(nq * 3 + nk)
    q, do = (torch.from_numpy(rng.standard_normal((B, H, nq, D)).astype(np.float32)).cuda().bfloat16() for _ in range(2))
    k, v = (torch.from_numpy(rng.standard_normal((B, H, nk, D)).astype(np.float32)).cuda().bfloat16() for _ in range(2))
    poly = orc.Poly(1.0, 1.0, 0.5, 1.0 / (2.0 * math.sqrt(D)), 2)
    L.profile_collect()
    L.profile(True)
    o, g, _ = L.forward(q, k, v, True, poly.inv_temp, order=2)
    dq, dk, dv, _ = L.backward(q, k, v, o, g, do, True, poly.inv_temp, order=2)
    L.check_status()
    L.profile(False)
    kinds = L.profile_collect()
    for name in ("tc_scan_fwd", "tc_scan_bwd_q", "tc_scan_bwd_kv", "tc_scan_bwd_dv"):
        assert name in kinds, f"{name} did not run: {kinds}"
    o_ref, _ = orc.fastmax_naive(host(q), host(k), host(v), True, poly)
    dq_ref, dk_ref, dv_ref = orc.fastmax_naive_grads(host(q), host(k), host(v), host(do), True, poly)
    errs = {n: orc.max_norm_err(host(a), b) for n, a, b in (("o", o, o_ref), ("dq", dq, dq_ref), ("dk", dk, dk_ref), ("dv", dv, dv_ref))}
    assert max(errs.values()) < 2e-2, errs


@pytest.mark.parametrize("shape", [(2, 8, 300, 300), (1, 16, 128, 200)])
def test_tensorcore_forward_writes_its_final_state(shape):
    """state_out without state_in stays on the tensor-memory path: the scan stores the moments of all keys."""
    from reproducing_fastmax_results_b200 import _lib as L

    B, H, nq, nk = shape
    D = 64
    rng = np.random.default_rng(nq + 7 * nk)
    q = torch.from_numpy(rng.standard_normal((B, H, nq, D)).astype(np.float32)).cuda().bfloat16()
    k, v = (torch.from_numpy(rng.standard_normal((B, H, nk, D)).astype(np.float32)).cuda().bfloat16() for _ in range(2))
    it = 1.0 / (2.0 * math.sqrt(D))
    L.profile_collect()
    L.profile(True)
    o, g, state = L.forward(q, k, v, True, it, order=2, want_state=True)
    L.check_status()
    L.profile(False)
    assert "tc_scan_fwd" in L.profile_collect()
    o_plain, g_plain, _ = L.forward(q, k, v, True, it, order=2)
    _, _, state_f32 = L.forward(q, k, v, True, it, order=2, want_state=True, flags=L.FLAG_NO_TENSOR_CORES)
    torch.cuda.synchronize()
    assert orc.max_norm_err(host(o), host(o_plain)) < 2e-3
    assert state.shape == state_f32.shape == (B, H, 64 * 36 + 65, 68)
    # against the exact float32 engine: only the bf16 rounding of the features separates the two
    for b in range(B):
        for h in range(0, H, 3):
            got, ref = host(state[b, h, :, :65]), host(state_f32[b, h, :, :65])
            assert orc.max_norm_err(got, ref) < 5e-3
            # linear rows and the constant row carry no product rounding at all
            assert orc.max_norm_err(got[-65:], ref[-65:]) < 1e-5
    assert float(state[..., 65:].abs().max()) == 0.0


@pytest.mark.parametrize("shape", [(4, 16, 300, 300), (2, 40, 128, 1024), (1, 64, 1000, 77), (64, 12, 1024, 1024)])
def test_order1_noncausal_forward_on_tensor_memory(shape):
    """Order 1 without a mask (BASELINE's wide-batch configuration): one streaming kernel per call."""
    from reproducing_fastmax_results_b200 import _lib as L

    B, H, nq, nk = shape
    D = 64
    g = torch.Generator(device="cuda").manual_seed(nq + nk)
    q = (torch.randn(B, H, nq, D, device="cuda", generator=g) * 0.5).bfloat16()
    k, v = ((torch.randn(B, H, nk, D, device="cuda", generator=g) * 0.5).bfloat16() for _ in range(2))
    poly = orc.Poly(1.0, 1.0, 0.5, 1.0 / (8.0 * math.sqrt(D)), 1)
    L.profile_collect()
    L.profile(True)
    o, gg, _ = L.forward(q, k, v, False, poly.inv_temp, order=1)
    L.check_status()
    L.profile(False)
    kinds = L.profile_collect()
    assert set(kinds) == {"p1_fwd"}, kinds
    o32, g32, _ = L.forward(q, k, v, False, poly.inv_temp, order=1, flags=L.FLAG_NO_TENSOR_CORES)
    torch.cuda.synchronize()
    assert orc.max_norm_err(host(o), host(o32)) < 2e-2
    assert orc.max_norm_err(host(gg), host(g32)) < 2e-3
    heads = [(0, 0), (B - 1, H - 1)]
    for b, h in heads:   # a few heads against the oracle itself
        o_ref, g_ref = orc.fastmax_naive(host(q[b, h]), host(k[b, h]), host(v[b, h]), False, poly)
        assert orc.max_norm_err(host(o[b, h]), o_ref) < 2e-2
        assert orc.max_norm_err(host(gg[b, h]), g_ref) < 2e-3


def test_order1_strided_views_and_other_coefficients():
    from reproducing_fastmax_results_b200 import _lib as L

    B, H, N, D = 2, 48, 200, 64
    g = torch.Generator(device="cuda").manual_seed(3)
    qkv = torch.randn(B, N, 3, H, D, device="cuda", generator=g).bfloat16()   # fused projection layout
    q, k, v = (qkv[:, :, i].permute(0, 2, 1, 3) for i in range(3))
    poly = orc.Poly(0.7, 1.3, 0.5, 0.11, 1)
    L.profile_collect()
    L.profile(True)
    o, gg, _ = L.forward(q, k, v, False, poly.inv_temp, poly.a0, poly.a1, poly.a2, order=1)
    L.check_status()
    L.profile(False)
    assert "p1_fwd" in L.profile_collect()
    for b, h in [(0, 5), (1, 47)]:
        o_ref, g_ref = orc.fastmax_naive(host(q[b, h]), host(k[b, h]), host(v[b, h]), False, poly)
        assert orc.max_norm_err(host(o[b, h]), o_ref) < 2e-2
        assert orc.max_norm_err(host(gg[b, h]), g_ref) < 2e-3


def test_two_host_threads_on_their_own_streams():
    """Two host threads issue calls on the same device at the same time, each on its own stream.  The library's
    internal side streams and events are shared per device; the calls must still be ordered correctly."""
    import threading

    from reproducing_fastmax_results_b200 import _lib as L

    B, H, N, D = 2, 16, 640, 64
    it = 1.0 / (2.0 * math.sqrt(D))
    gen = torch.Generator(device="cuda").manual_seed(9)
    sets = [[torch.randn(B, H, N, D, device="cuda", generator=gen).bfloat16() for _ in range(4)] for _ in range(2)]

    def run(x):
        q, k, v, do = x
        o, g, _ = L.forward(q, k, v, True, it, order=2)
        return (o,) + tuple(L.backward(q, k, v, o, g, do, True, it, order=2)[:3])

    refs = [[t.clone() for t in run(x)] for x in sets]
    torch.cuda.synchronize()
    errors = []

    def worker(i):
        try:
            stream = torch.cuda.Stream()
            with torch.cuda.stream(stream):
                for _ in range(8):
                    outs = run(sets[i])
                    stream.synchronize()
                    for a, b in zip(outs, refs[i]):
                        err = float((a.float() - b.float()).abs().max()) / float(b.float().abs().max())
                        if not err < 5e-3:
                            errors.append((i, err))
        except Exception as e:  # noqa: BLE001 - reported through the list
            errors.append((i, repr(e)))

    threads = [threading.Thread(target=worker, args=(i,)) for i in range(2)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    torch.cuda.synchronize()
    L.check_status()
    assert not errors, errors
