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
@pytest.mark.parametrize("D,dtype,pieces", [(32, torch.float32, 4), (64, torch.float32, 2), (64, torch.bfloat16, 2),
                                            (32, torch.bfloat16, 2)])
def test_cuda_engine_pieces_match_whole_sequence(D, dtype, pieces):
    """The schedule of sequence_parallel.forward/backward with the CUDA engine; the exchange between ranks is
    done by hand (sum of the other pieces' states) because all pieces live on one device here."""
    from reproducing_fastmax_results_b200 import _lib

    B, H, N = 1, (16 if dtype == torch.bfloat16 else 3), 128 * pieces + 40
    tol = 1e-4 if dtype == torch.float32 else 2e-2
    _lib.profile_collect()
    _lib.profile(True)
    q, k, v, do = (torch.from_numpy(a).to("cuda", dtype) for a in _inputs(B, H, N, D, seed=11))
    temperature = 2.0 * math.sqrt(D)
    eng = sp.CudaEngine(1.0 / temperature)
    bounds = [0] + [128 * (i + 1) - 17 * i for i in range(pieces - 1)] + [N]
    sl = [slice(bounds[i], bounds[i + 1]) for i in range(pieces)]
    cut = lambda t, s: t[:, :, s].contiguous()
    kms = [sp.KeyMoments() for _ in sl]   # one holder per piece: its key moments go from call to call
    totals = [eng.key_state(cut(k, s), cut(v, s), moments=kms[i]) for i, s in enumerate(sl)]
    prefixes = [sum(totals[:i], torch.zeros_like(totals[0])) for i in range(pieces)]
    outs = [eng.forward(cut(q, s), cut(k, s), cut(v, s), prefixes[i], moments=kms[i]) for i, s in enumerate(sl)]
    gtot = [eng.grad_state(cut(q, s), cut(k, s), cut(v, s), outs[i][0], outs[i][1], cut(do, s), prefixes[i], moments=kms[i])
            for i, s in enumerate(sl)]
    suffixes = [sum(gtot[i + 1:], torch.zeros_like(gtot[0])) for i in range(pieces)]
    grads = [eng.backward(cut(q, s), cut(k, s), cut(v, s), outs[i][0], outs[i][1], cut(do, s), prefixes[i], suffixes[i],
                          moments=kms[i]) for i, s in enumerate(sl)]
    torch.cuda.synchronize()
    _lib.profile(False)
    kinds = set(_lib.profile_collect())
    if dtype == torch.bfloat16:   # every piece, with or without a carried state, runs on the tensor-memory kernels
        assert {"tc_scan_fwd", "tc_scan_bwd_q", "tc_scan_bwd_kv", "tc_scan_bwd_dv"} <= kinds, kinds
        assert not ({"scan_fwd", "scan_bwd_q", "scan_bwd_kv", "moments_kv", "moments_qg"} & kinds), kinds
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


def _failing_peer_worker(rank, world, port, out_dir):
    """Rank 1 raises before the exchange; rank 0 must come back from the collective with an error, not hang."""
    import datetime
    import time

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=8))
    x = torch.ones(4, 3, dtype=torch.float64)
    assert torch.equal(sp.exclusive_prefix(x), torch.full((4, 3), float(rank), dtype=torch.float64))  # healthy exchange first
    if rank == 1:
        raise RuntimeError("injected failure before the exchange")
    t0 = time.monotonic()
    try:
        sp.exclusive_prefix(x)
        verdict = "no error"
    except Exception as e:  # the process group reports the lost peer (closed connection or its timeout)
        verdict = "error: " + type(e).__name__
    with open(os.path.join(out_dir, "rank0.txt"), "w") as f:
        f.write("%s\n%.3f\n" % (verdict, time.monotonic() - t0))
    os._exit(0)   # skip the group's teardown handshake with a peer that is gone


def test_a_rank_that_fails_before_the_exchange_gives_its_peer_an_error(tmp_path):
    """Failure made on the host: no GPU is involved, nothing hangs.  The surviving rank gets an exception from the
    collective within the process group's timeout and can report it."""
    ctx = mp.get_context("spawn")
    port = _free_port()
    procs = [ctx.Process(target=_failing_peer_worker, args=(r, 2, port, str(tmp_path))) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(60)
    assert all(not p.is_alive() for p in procs), "a rank hung"
    assert procs[1].exitcode != 0
    text = open(os.path.join(str(tmp_path), "rank0.txt")).read().splitlines()
    assert text[0].startswith("error"), text
    assert float(text[1]) < 30.0, text


def _nccl_worker(rank, world, port, out_dir, D, dtype_name):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        from reproducing_fastmax_results_b200 import _lib

        dtype = torch.float32 if dtype_name == "f32" else torch.bfloat16
        B, H, N = 1, 16, 2 * 300
        cuts = [0, 260, N]   # uneven pieces, neither a multiple of the chunk length
        q, k, v, do = (torch.from_numpy(a[:, :, cuts[rank]:cuts[rank + 1]].copy()).to(dev, dtype)
                       for a in _inputs(B, H, N, D, seed=21))
        q.requires_grad_(True), k.requires_grad_(True), v.requires_grad_(True)
        _lib.profile_collect()
        _lib.profile(True)
        o = sp.SequenceParallelFastMax.apply(q, k, v, 2.0 * math.sqrt(D), 1.0, 1.0, 0.5, 2, None)
        o.backward(do)
        torch.cuda.synchronize()
        _lib.profile(False)
        kinds = sorted(_lib.profile_collect())
        _lib.check_status()
        host = lambda t: t.detach().float().cpu().numpy()
        np.savez(os.path.join(out_dir, f"rank{rank}.npz"), o=host(o), dq=host(q.grad), dk=host(k.grad), dv=host(v.grad),
                 kinds=np.array(kinds))
    finally:
        dist.destroy_process_group()


@pytest.mark.gpu
@pytest.mark.parametrize("D,dtype_name", [(32, "f32"), (64, "bf16")])
def test_nccl_ranks_reproduce_the_unsplit_sequence(tmp_path, D, dtype_name):
    """The real composition: two processes, one GPU each, CudaEngine + all_gather over NCCL
    (SequenceParallelFastMax forward and backward), against the unsplit float64 result."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    world = 2
    mp.spawn(_nccl_worker, args=(world, _free_port(), str(tmp_path), D, dtype_name), nprocs=world, join=True)
    B, H, N = 1, 16, 600
    tol = 1e-4 if dtype_name == "f32" else 2e-2
    q, k, v, do = _inputs(B, H, N, D, seed=21)
    if dtype_name == "bf16":
        q, k, v, do = (torch.from_numpy(a).bfloat16().double().numpy() for a in (q, k, v, do))
    poly = orc.Poly(1.0, 1.0, 0.5, 1.0 / (2.0 * math.sqrt(D)), 2)
    parts = [np.load(os.path.join(str(tmp_path), f"rank{r}.npz")) for r in range(world)]
    for h in range(H):
        o_ref, _ = orc.fastmax_naive(q[0, h], k[0, h], v[0, h], True, poly)
        refs = dict(zip(("dq", "dk", "dv"), orc.fastmax_naive_grads(q[0, h], k[0, h], v[0, h], do[0, h], True, poly)))
        refs["o"] = o_ref
        for name, ref in refs.items():
            got = np.concatenate([p[name][0, h] for p in parts], 0)
            assert orc.max_norm_err(got, ref) < tol, (name, h)
