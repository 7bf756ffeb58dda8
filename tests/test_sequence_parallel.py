"""Sequence-parallel causal Fastmax (a sequence cut into contiguous pieces, one per rank).

CPU: two gloo ranks run `sequence_parallel.forward/backward` with the CPU oracle as the compute engine and
must reproduce the unsplit result; the collectives (exclusive prefix / suffix over ranks) are checked on their
own too.  GPU: the same schedule with the CUDA engine, the ranks emulated one after another on one device.
"""
import math
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import fastmax_oracle as orc
from reproducing_fastmax_results_b200 import sequence_parallel as sp


class OracleEngine:
    """CPU stand-in for the CUDA engine: float64 numpy, states in the oracle's (M, Dv+1) layout."""

    def __init__(self, poly):
        self.poly = poly

    @staticmethod
    def _heads(t):
        a = t.numpy()
        return a.reshape(-1, a.shape[-2], a.shape[-1])

    def key_state(self, k, v):
        return torch.from_numpy(np.stack([orc.moment_state(kk, vv, self.poly) for kk, vv in zip(self._heads(k), self._heads(v))]))

    def forward(self, q, k, v, state_in):
        outs = [orc.fastmax_streaming(a, b, c, True, self.poly, chunk=32, state_in=s.numpy())
                for a, b, c, s in zip(self._heads(q), self._heads(k), self._heads(v), state_in)]
        o = torch.from_numpy(np.stack([x[0] for x in outs])).reshape(q.shape)
        g = torch.from_numpy(np.stack([x[1] for x in outs])).reshape(q.shape[:-1])
        return o, g

    def grad_state(self, q, k, v, o, g, do, state_in):
        gs = g.numpy().reshape(-1, g.shape[-1])
        return torch.from_numpy(np.stack([orc.grad_moment_state(a, d, oo, gg, self.poly)
                                          for a, d, oo, gg in zip(self._heads(q), self._heads(do), self._heads(o), gs)]))

    def backward(self, q, k, v, o, g, do, state_in, dstate_in):
        res = [orc.fastmax_streaming_grads(a, b, c, d, True, self.poly, chunk=32, state_in=s.numpy(), dstate_in=ds.numpy())
               for a, b, c, d, s, ds in zip(self._heads(q), self._heads(k), self._heads(v), self._heads(do), state_in, dstate_in)]
        return tuple(torch.from_numpy(np.stack([r[i] for r in res])).reshape(q.shape) for i in range(3))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _inputs(B, H, N, D, seed=3):
    rng = np.random.default_rng(seed)
    return [rng.standard_normal((B, H, N, D)) for _ in range(4)]


def _gloo_worker(rank, world, port, cuts, out_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        # collectives on their own
        x = torch.full((3, 2), float(rank + 1), dtype=torch.float64)
        assert torch.equal(sp.exclusive_prefix(x), torch.full((3, 2), float(sum(range(1, rank + 1))), dtype=torch.float64))
        assert torch.equal(sp.exclusive_suffix(x), torch.full((3, 2), float(sum(range(rank + 2, world + 1))), dtype=torch.float64))
        B, H, N, D = 1, 2, cuts[-1], 16
        q, k, v, do = (torch.from_numpy(a[:, :, cuts[rank]:cuts[rank + 1]].copy()) for a in _inputs(B, H, N, D))
        poly = orc.Poly(1.0, 1.0, 0.5, 1.0 / (2.0 * math.sqrt(D)), 2)
        eng = OracleEngine(poly)
        o, g, prefix = sp.forward(eng, q, k, v)
        dq, dk, dv = sp.backward(eng, q, k, v, o, g, do, prefix)
        np.savez(os.path.join(out_dir, f"rank{rank}.npz"), o=o.numpy(), dq=dq.numpy(), dk=dk.numpy(), dv=dv.numpy())
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("cuts", [(0, 96, 200), (0, 50, 51, 200)])
def test_gloo_ranks_reproduce_the_unsplit_sequence(tmp_path, cuts):
    """world_size 2 (and 3 with a one-token piece): pieces of uneven length, forward and backward."""
    world = len(cuts) - 1
    mp.spawn(_gloo_worker, args=(world, _free_port(), cuts, str(tmp_path)), nprocs=world, join=True)
    B, H, N, D = 1, 2, cuts[-1], 16
    q, k, v, do = _inputs(B, H, N, D)
    poly = orc.Poly(1.0, 1.0, 0.5, 1.0 / (2.0 * math.sqrt(D)), 2)
    parts = [np.load(os.path.join(str(tmp_path), f"rank{r}.npz")) for r in range(world)]
    for h in range(H):
        o_ref, _ = orc.fastmax_naive(q[0, h], k[0, h], v[0, h], True, poly)
        refs = dict(zip(("dq", "dk", "dv"), orc.fastmax_naive_grads(q[0, h], k[0, h], v[0, h], do[0, h], True, poly)))
        refs["o"] = o_ref
        for name, ref in refs.items():
            got = np.concatenate([p[name][0, h] for p in parts], 0)
            assert orc.max_norm_err(got, ref) < 1e-10, name


@pytest.mark.gpu
@pytest.mark.parametrize("D,dtype,pieces", [(32, torch.float32, 4), (64, torch.float32, 2), (64, torch.bfloat16, 2)])
def test_cuda_engine_pieces_match_whole_sequence(D, dtype, pieces):
    """The schedule of sequence_parallel.forward/backward with the CUDA engine; the exchange between ranks is
    done by hand (sum of the other pieces' states) because all pieces live on one device here."""
    B, H, N = 1, 3, 128 * pieces + 40
    tol = 1e-4 if dtype == torch.float32 else 2e-2
    q, k, v, do = (torch.from_numpy(a).to("cuda", dtype) for a in _inputs(B, H, N, D, seed=11))
    temperature = 2.0 * math.sqrt(D)
    eng = sp.CudaEngine(1.0 / temperature)
    bounds = [0] + [128 * (i + 1) - 17 * i for i in range(pieces - 1)] + [N]
    sl = [slice(bounds[i], bounds[i + 1]) for i in range(pieces)]
    cut = lambda t, s: t[:, :, s].contiguous()
    totals = [eng.key_state(cut(k, s), cut(v, s)) for s in sl]
    prefixes = [sum(totals[:i], torch.zeros_like(totals[0])) for i in range(pieces)]
    outs = [eng.forward(cut(q, s), cut(k, s), cut(v, s), prefixes[i]) for i, s in enumerate(sl)]
    gtot = [eng.grad_state(cut(q, s), cut(k, s), cut(v, s), outs[i][0], outs[i][1], cut(do, s), prefixes[i])
            for i, s in enumerate(sl)]
    suffixes = [sum(gtot[i + 1:], torch.zeros_like(gtot[0])) for i in range(pieces)]
    grads = [eng.backward(cut(q, s), cut(k, s), cut(v, s), outs[i][0], outs[i][1], cut(do, s), prefixes[i], suffixes[i])
             for i, s in enumerate(sl)]
    torch.cuda.synchronize()
    poly = orc.Poly(1.0, 1.0, 0.5, 1.0 / temperature, 2)
    host = lambda t: t.float().cpu().numpy().astype(np.float64)
    qh, kh, vh, doh = (host(t) for t in (q, k, v, do))
    for h in range(H):
        o_ref, _ = orc.fastmax_naive(qh[0, h], kh[0, h], vh[0, h], True, poly)
        dq_ref, dk_ref, dv_ref = orc.fastmax_naive_grads(qh[0, h], kh[0, h], vh[0, h], doh[0, h], True, poly)
        got_o = np.concatenate([host(o_[0])[0, h] for o_ in outs], 0)
        assert orc.max_norm_err(got_o, o_ref) < tol
        for j, ref in enumerate((dq_ref, dk_ref, dv_ref)):
            got = np.concatenate([host(gr[j])[0, h] for gr in grads], 0)
            assert orc.max_norm_err(got, ref) < tol, ("dq", "dk", "dv")[j]
