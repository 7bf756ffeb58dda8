"""fastmax_decode_step (one token per head against the carried moment state) against the CPU oracle: the
outputs of token-by-token decoding must equal the rows of the causal operator over the whole sequence, and
the state must equal the moments of all keys seen."""
import math

import numpy as np
import pytest
import torch

from oracle import fastmax_oracle as orc

pytestmark = pytest.mark.gpu


def host(t):
    return t.detach().float().cpu().numpy().astype(np.float64)


def exchange_state(k, v, order):
    """Moment state of one head in the library's layout: pair units (a <= b over 8-wide blocks of the head
    dim, 64 rows k[8a+mi] k[8b+ri] each), then the D linear rows, then the constant row; column D = sum of
    the feature alone."""
    k = np.asarray(k, np.float64)
    v1 = np.concatenate([np.asarray(v, np.float64), np.ones((v.shape[0], 1))], 1)
    D = k.shape[1]
    feats = []
    if order == 2:
        nb = D // 8
        for a in range(nb):
            for b in range(a, nb):
                ka, kb = k[:, 8 * a:8 * a + 8], k[:, 8 * b:8 * b + 8]
                feats.append((ka[:, :, None] * kb[:, None, :]).reshape(k.shape[0], 64))
    feats += [k, np.ones((k.shape[0], 1))]
    return np.concatenate(feats, 1).T @ v1


@pytest.mark.parametrize("D", [16, 32, 64])
@pytest.mark.parametrize("order", [1, 2])
def test_decode_from_empty_state_matches_causal_operator(D, order):
    from reproducing_fastmax_results_b200 import _lib as L

    B, H, T = 2, 3, 12
    rng = np.random.default_rng(100 * D + order)
    q, k, v = (rng.standard_normal((B, H, T, D)).astype(np.float32) for _ in range(3))
    poly = orc.Poly(0.9, 1.1, 0.45, 1.0 / (2.0 * math.sqrt(D)), order)
    qd, kd, vd = (torch.from_numpy(x).cuda() for x in (q, k, v))
    state = L.new_state(B, H, D, order)
    outs, gs = [], []
    for t in range(T):
        o, g = L.decode_step(qd[:, :, t], kd[:, :, t], vd[:, :, t], state, poly.inv_temp, poly.a0, poly.a1, poly.a2, order)
        outs.append(o)
        gs.append(g)
    torch.cuda.synchronize()
    o_ref, g_ref = orc.fastmax_naive(q, k, v, True, poly)
    assert orc.max_norm_err(host(torch.stack(outs, 2)), o_ref) < 1e-4   # float32 tolerance of the operator
    assert orc.max_norm_err(host(torch.stack(gs, 2)), g_ref) < 1e-4
    for b in range(B):
        for h in range(H):
            ref = exchange_state(k[b, h], v[b, h], order)
            assert orc.max_norm_err(host(state[b, h, :, : D + 1]), ref) < 1e-5


def test_decoder_prefill_then_steps_bf16():
    """The serving flow: causal operator over the prompt (tensor-memory kernels, which also write their final
    state out), then one launch per generated token; a second prompt block continues from the carried state
    (float32 engine)."""
    from reproducing_fastmax_results_b200.decoding import FastmaxDecoder

    B, H, N0, T, D = 2, 8, 200, 6, 64
    rng = np.random.default_rng(3)
    q, k, v = (torch.from_numpy(rng.standard_normal((B, H, N0 + T, D)).astype(np.float32)).cuda().bfloat16() for _ in range(3))
    temperature = 2.0 * math.sqrt(D)
    dec = FastmaxDecoder(B, H, D, p=2, temperature=temperature)
    o0 = dec.prefill(q[:, :, :N0], k[:, :, :N0], v[:, :, :N0])
    steps = [dec.step(q[:, :, N0 + t], k[:, :, N0 + t], v[:, :, N0 + t]) for t in range(T)]
    torch.cuda.synchronize()
    assert dec.tokens_seen == N0 + T
    poly = orc.Poly(1.0, 1.0, 0.5, 1.0 / temperature, 2)
    o_ref, _ = orc.fastmax_naive(host(q), host(k), host(v), True, poly)
    assert orc.max_norm_err(host(o0), o_ref[:, :, :N0]) < 2e-2          # bf16 tolerance of the operator
    assert orc.max_norm_err(host(torch.stack(steps, 2)), o_ref[:, :, N0:]) < 2e-2
    ref = exchange_state(host(k)[1, 5], host(v)[1, 5], 2)
    assert orc.max_norm_err(host(dec.state[1, 5, :, : D + 1]), ref) < 5e-3   # features rounded to bf16 in the prompt pass
    # a second block continues from the carried state
    dec2 = FastmaxDecoder(B, H, D, p=2, temperature=temperature)
    dec2.prefill(q[:, :, :100], k[:, :, :100], v[:, :, :100])
    o_b = dec2.prefill(q[:, :, 100:N0], k[:, :, 100:N0], v[:, :, 100:N0])
    assert orc.max_norm_err(host(o_b), o_ref[:, :, 100:N0]) < 2e-2
    dec2.reset()
    assert dec2.tokens_seen == 0 and float(dec2.state.abs().max()) == 0.0


def test_decode_reads_the_projection_layout_in_place():
    """q, k, v of one token straight out of a fused (b, 3, h, d) projection: strided views, no copies; the
    output goes into a caller tensor."""
    from reproducing_fastmax_results_b200 import _lib as L

    B, H, D = 3, 5, 32
    rng = np.random.default_rng(8)
    qkv = torch.from_numpy(rng.standard_normal((B, 3, H, D)).astype(np.float32)).cuda()
    state0 = torch.from_numpy(rng.standard_normal((B, H, 64 * 10 + D + 1, D + 4)).astype(np.float32)).cuda()
    state0[:, :, -1, D] = 50.0                       # keeps the denominator away from zero
    s_a, s_b = state0.clone(), state0.clone()
    it = 0.2
    out = torch.empty(B, H, D, device="cuda")
    o_a, g_a = L.decode_step(qkv[:, 0], qkv[:, 1], qkv[:, 2], s_a, it, out=out)
    assert o_a.data_ptr() == out.data_ptr()
    o_b, g_b = L.decode_step(qkv[:, 0].contiguous(), qkv[:, 1].contiguous(), qkv[:, 2].contiguous(), s_b, it)
    torch.cuda.synchronize()
    assert torch.equal(o_a, o_b) and torch.equal(g_a, g_b) and torch.equal(s_a, s_b)
    # against the definition, from the random starting state
    w = np.concatenate([np.repeat([0.5 * it * it * (1 if a == b else 2) for a in range(4) for b in range(a, 4)], 64),
                        np.full(D, it), [1.0]])
    for b in range(B):
        for h in range(H):
            qh, kh, vh = (host(qkv[b, j, h]) for j in range(3))
            s_new = host(state0[b, h, :, : D + 1]) + exchange_state(kh[None], vh[None], 2)
            op = (exchange_phi(qh) * w) @ s_new
            assert orc.max_norm_err(host(o_a[b, h]), op[:D] / op[D]) < 1e-4
            assert abs(float(g_a[b, h]) - op[D]) < 1e-4 * abs(op[D])


def exchange_phi(x):
    """Feature vector of one token in the state's row order."""
    D = x.shape[0]
    nb = D // 8
    f = [np.outer(x[8 * a:8 * a + 8], x[8 * b:8 * b + 8]).reshape(64) for a in range(nb) for b in range(a, nb)]
    return np.concatenate(f + [x, [1.0]])


def test_decode_rejects_bad_arguments():
    import ctypes as C

    from reproducing_fastmax_results_b200 import _lib as L

    lib = L.load()
    x = torch.zeros(1, 2, 64, device="cuda")
    state = L.new_state(1, 2, 64)
    args = L.DecodeArgs()
    args.q = args.k = args.v = args.o = L.Tensor(x.data_ptr(), 128, 64, 0)
    args.state = state.data_ptr()
    good = L.Problem(1, 2, 1, 1, 64, 2, 1, L.FASTMAX_F32, 1.0, 1.0, 0.5, 1.0, 0, 0)
    two_tokens = L.Problem(1, 2, 2, 2, 64, 2, 1, L.FASTMAX_F32, 1.0, 1.0, 0.5, 1.0, 0, 0)
    bad_dim = L.Problem(1, 2, 1, 1, 48, 2, 1, L.FASTMAX_F32, 1.0, 1.0, 0.5, 1.0, 0, 0)
    assert lib.fastmax_decode_step(C.byref(two_tokens), C.byref(args), None) == 2   # FASTMAX_ERR_UNSUPPORTED
    assert lib.fastmax_decode_step(C.byref(bad_dim), C.byref(args), None) == 2
    assert lib.fastmax_decode_step(None, C.byref(args), None) == 1                  # FASTMAX_ERR_INVALID_ARGUMENT
    args.state = state.data_ptr() + 4
    assert lib.fastmax_decode_step(C.byref(good), C.byref(args), None) == 6         # FASTMAX_ERR_MISALIGNED
    args.state = None
    assert lib.fastmax_decode_step(C.byref(good), C.byref(args), None) == 1
    torch.cuda.synchronize()


def test_decode_steps_replay_from_a_cuda_graph():
    """A generation loop captures one decode step and replays it per token (the launch is a few microseconds of
    host time against ~0.1 ms of kernel)."""
    from reproducing_fastmax_results_b200 import _lib as L

    B, H, D, T = 2, 4, 64, 5
    rng = np.random.default_rng(21)
    q, k, v = (torch.from_numpy(rng.standard_normal((B, H, T, D)).astype(np.float32)).cuda() for _ in range(3))
    poly = orc.Poly(1.0, 1.0, 0.5, 1.0 / (2.0 * math.sqrt(D)), 2)
    state = L.new_state(B, H, D, 2)
    qs, ks, vs = (torch.empty(B, H, D, device="cuda") for _ in range(3))
    out = torch.empty(B, H, D, device="cuda")
    scratch = L.new_state(B, H, D, 2)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        L.decode_step(qs, ks, vs, scratch, poly.inv_temp, out=out)   # warm-up on a throw-away state
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        L.decode_step(qs, ks, vs, state, poly.inv_temp, out=out)
    state.zero_()   # the capture itself does not run the kernel; start from an empty state anyway
    outs = []
    for t in range(T):
        qs.copy_(q[:, :, t]); ks.copy_(k[:, :, t]); vs.copy_(v[:, :, t])
        graph.replay()
        outs.append(out.clone())
    torch.cuda.synchronize()
    o_ref, _ = orc.fastmax_naive(host(q), host(k), host(v), True, poly)
    assert orc.max_norm_err(host(torch.stack(outs, 2)), o_ref) < 1e-4


def test_decoding_is_bit_for_bit_repeatable():
    """The decode step sums its partial results in a fixed order (rows of a block, then blocks of the cluster in rank
    order): two runs over the same tokens give the same bits in every output and in the state."""
    from reproducing_fastmax_results_b200 import _lib as L

    B, H, T, D, order = 3, 5, 24, 64, 2
    g = torch.Generator(device="cuda").manual_seed(4)
    q, k, v = (torch.randn(B, H, T, D, device="cuda", generator=g) for _ in range(3))
    runs = []
    for _ in range(2):
        state = L.new_state(B, H, D, order)
        outs = []
        for t in range(T):
            o, gg = L.decode_step(q[:, :, t], k[:, :, t], v[:, :, t], state, 0.0625, 1.0, 1.0, 0.5, order)
            outs += [o, gg]
        torch.cuda.synchronize()
        runs.append((outs, state))
    assert all(torch.equal(a, b) for a, b in zip(runs[0][0], runs[1][0]))
    assert torch.equal(runs[0][1], runs[1][1])
