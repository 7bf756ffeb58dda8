"""CPU restatement of the reference's Fastmax attention path.  TEST INFRASTRUCTURE ONLY.

This module is the checker that the CUDA path is compared with.  It is never the thing
that is shipped or measured as the product: only the test-suite, the smoke check and the
benchmark's CPU-baseline leg may import it.

Parity status: PINNED.  Every function here is checked (tests/test_oracle.py) against
  * the reference's own property tests (test/test_einops_fastmax.py:25-129, 257-274:
    factorised result == row-normalised N x N polynomial attention), and
  * golden vectors produced by importing the reference's
    attention_mechanisms/fastattention_einops.py and attention_mechanisms/score_function.py
    (tests/golden/make_golden.py wrote tests/golden/*.npz).

What Fastmax computes, per (batch, head):
    s_lj = (q_l . k_j) * inv_temp                 (einops.py:78-82: inv_temp = 1/(normalize_term*sqrt(D)))
    f(s) = a0 + a1 s + a2 s^2   (p=2)   or   a0 + a1 s   (p=1)        (einops.py:204-214, fwd.cu:35-142)
    A_lj = f(s_lj) if key j is visible to query l else 0
    g_l  = sum_j A_lj,   o_l = sum_j A_lj v_j / g_l                    (einops.py:97)
Causal visibility with nk >= nq aligns the queries to the LAST nq keys: query l sees keys
0 .. nk-nq+l  (fastmax_cuda_forward.cu:161-172).

Three evaluations of the same function are kept, because each one is usable at a different size:
  fastmax_naive        N x N matrix            (test.py:25-75, einops.py:337-381)   small N, fp64 truth
  fastmax_factorized   moments + cumsum (torch) (einops.py:185-322, score.py:88-221) the reference's own
                       algorithm; O(N D^3) memory when causal; this is what the CPU baseline times
  fastmax_streaming    chunked running moments   any N, O(D^2 Dv) memory; same chunk/state algebra the
                       CUDA kernels use, written independently in fp64
plus exact per-row / per-column evaluation (sampled_*), O(N D) per sample, for full-size configs.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import numpy as np


@dataclass(frozen=True)
class Poly:
    """f(s) = a0 + a1 s + a2 s^2 evaluated on s = (q.k) * inv_temp."""

    a0: float = 1.0
    a1: float = 1.0
    a2: float = 0.5
    inv_temp: float = 1.0
    p: int = 2

    def f(self, s):
        out = self.a0 + self.a1 * s
        if self.p == 2:
            out = out + self.a2 * s * s
        return out

    def df(self, s):
        out = np.full_like(s, self.a1)
        if self.p == 2:
            out = out + 2.0 * self.a2 * s
        return out


def poly_from_normalize_term(D: int, normalize_term: float = 8.0, tensors_normalized: bool = False, p: int = 2) -> Poly:
    """Parameter map of einops.py:78-82 and score.py:57: temperature = normalize_term * sqrt(D)."""
    t = 1.0 if tensors_normalized else normalize_term * math.sqrt(D)
    return Poly(1.0, 1.0, 0.5, 1.0 / t, p)


def _visible(nq: int, nk: int, mask: bool) -> np.ndarray:
    if not mask:
        return np.ones((nq, nk), dtype=bool)
    off = nk - nq
    return np.arange(nk)[None, :] <= (np.arange(nq)[:, None] + off)


# --------------------------------------------------------------------------------------------
# 1. naive N x N evaluation (fp64 truth).  Shapes (..., n, d); leading dims are batch/head.
# --------------------------------------------------------------------------------------------
def fastmax_naive(q, k, v, mask: bool, poly: Poly):
    """Row-normalised polynomial attention (test.py:25-75; einops.py:337-381).  Returns (o, g)."""
    q = np.asarray(q, dtype=np.float64)
    k = np.asarray(k, dtype=np.float64)
    v = np.asarray(v, dtype=np.float64)
    s = np.einsum("...id,...jd->...ij", q, k) * poly.inv_temp
    A = poly.f(s) * _visible(q.shape[-2], k.shape[-2], mask)
    g = A.sum(-1)
    o = np.einsum("...ij,...jd->...id", A, v) / g[..., None]
    return o, g


def fastmax_naive_grads(q, k, v, do, mask: bool, poly: Poly):
    """Analytic gradients of sum(o * do) w.r.t. q, k, v through the N x N form.

    With dO' = [do/g, -(do.o)/g]:  dA = dO' [V|1]^T,  dS = dA * f'(s) * visible,
    dq = dS K inv_temp, dk = dS^T Q inv_temp, dv = A^T (do/g)   (same grouping as bwd.cu:38-97).
    """
    q = np.asarray(q, dtype=np.float64)
    k = np.asarray(k, dtype=np.float64)
    v = np.asarray(v, dtype=np.float64)
    do = np.asarray(do, dtype=np.float64)
    vis = _visible(q.shape[-2], k.shape[-2], mask)
    s = np.einsum("...id,...jd->...ij", q, k) * poly.inv_temp
    A = poly.f(s) * vis
    g = A.sum(-1)
    o = np.einsum("...ij,...jd->...id", A, v) / g[..., None]
    dog = do / g[..., None]
    dg = -(do * o).sum(-1) / g
    dA = np.einsum("...id,...jd->...ij", dog, v) + dg[..., None]
    dS = dA * poly.df(s) * vis
    dq = np.einsum("...ij,...jd->...id", dS, k) * poly.inv_temp
    dk = np.einsum("...ij,...id->...jd", dS, q) * poly.inv_temp
    dv = np.einsum("...ij,...id->...jd", A, dog)
    return dq, dk, dv


# --------------------------------------------------------------------------------------------
# 2. the reference's own factorised algorithm, restated with torch on the CPU.
#    Non-causal: moment sums (einops.py:185-216, 253-285).  Causal: cumsum over tokens of the
#    per-token outer products (einops.py:219-250, 288-322; score.py:126-162) -> O(N D^3) memory.
#    Gradients come from autograd of this forward, which is what score.py relies on too.
# --------------------------------------------------------------------------------------------
def fastmax_factorized(q, k, v, mask: bool, poly: Poly):
    """q,k,v: torch tensors (B,H,N,D) (any float dtype, CPU).  Returns o (B,H,N,Dv)."""
    import torch

    c1 = poly.a1 * poly.inv_temp
    c2 = poly.a2 * poly.inv_temp * poly.inv_temp
    B, H, N, D = q.shape
    if k.shape[2] != N:
        raise ValueError("the factorised restatement follows the reference and needs nk == nq")
    if not mask:
        F = poly.a0 * v.sum(2, keepdim=True)
        F = F + c1 * torch.matmul(q, torch.matmul(k.transpose(-1, -2), v))
        g = poly.a0 * N + c1 * torch.matmul(q, k.sum(2).unsqueeze(-1)).squeeze(-1)
        if poly.p == 2:
            k2 = (k.unsqueeze(-1) * k.unsqueeze(-2)).flatten(-2)
            q2 = (q.unsqueeze(-1) * q.unsqueeze(-2)).flatten(-2)
            F = F + c2 * torch.matmul(q2, torch.matmul(k2.transpose(-1, -2), v))
            g = g + c2 * torch.matmul(q2, k2.sum(2).unsqueeze(-1)).squeeze(-1)
    else:
        F = poly.a0 * torch.cumsum(v, 2)
        kv = torch.cumsum(k.unsqueeze(-1) * v.unsqueeze(-2), 2)
        F = F + c1 * torch.einsum("bhim,bhimj->bhij", q, kv)
        cnt = torch.arange(1, N + 1, dtype=q.dtype)
        g = poly.a0 * cnt + c1 * (q * torch.cumsum(k, 2)).sum(-1)
        if poly.p == 2:
            k2 = (k.unsqueeze(-1) * k.unsqueeze(-2)).flatten(-2)
            q2 = (q.unsqueeze(-1) * q.unsqueeze(-2)).flatten(-2)
            kkv = torch.cumsum(k2.unsqueeze(-1) * v.unsqueeze(-2), 2)
            F = F + c2 * torch.einsum("bhim,bhimj->bhij", q2, kkv)
            g = g + c2 * (q2 * torch.cumsum(k2, 2)).sum(-1)
    return F / g.unsqueeze(-1)


def fastmax_factorized_fwd_bwd(q, k, v, do, mask: bool, poly: Poly):
    """Forward + backward of the factorised restatement (torch autograd).  Returns o, dq, dk, dv."""
    import torch

    q = q.detach().clone().requires_grad_(True)
    k = k.detach().clone().requires_grad_(True)
    v = v.detach().clone().requires_grad_(True)
    o = fastmax_factorized(q, k, v, mask, poly)
    o.backward(do)
    return o.detach(), q.grad, k.grad, v.grad


# --------------------------------------------------------------------------------------------
# 3. streaming chunked-moment evaluation (fp64, memory O(M * (Dv+1))).
#    State S = Phi(K)^T [V|1] with Phi(x) = [1, x, x (x) x];  O' = Phi(Q) S;  o = O'[:, :Dv] / O'[:, Dv].
#    Causal chunk c:  O'_c = Phi(Q_c) S_{<c} + tril(f(Q_c K_c^T)) V'_c ;  S_{<=c} = S_{<c} + Phi(K_c)^T V'_c.
#    Backward: dS_{>=j} = sum_{l>=j} Phi(q_l)^T dO'_l (reverse scan), dPhi(Q)_l = dO'_l S_{<=l}^T,
#    dPhi(K)_j = V'_j dS_{>=j}^T, dV_j = Phi(k_j) dS_{>=j}; chain rule through Phi.
# --------------------------------------------------------------------------------------------
def _phi(x, p):
    parts = [np.ones(x.shape[:-1] + (1,)), x]
    if p == 2:
        parts.append((x[..., :, None] * x[..., None, :]).reshape(x.shape[:-1] + (-1,)))
    return np.concatenate(parts, -1)


def _weights(D, poly: Poly):
    w = [np.full(1, poly.a0), np.full(D, poly.a1 * poly.inv_temp)]
    if poly.p == 2:
        w.append(np.full(D * D, poly.a2 * poly.inv_temp ** 2))
    return np.concatenate(w)


def _dphi_to_dx(dphi, x, p):
    """Chain rule through Phi: dx = dPhi1 + (dPhi2 + dPhi2^T) x."""
    D = x.shape[-1]
    dx = dphi[..., 1:1 + D].copy()
    if p == 2:
        d2 = dphi[..., 1 + D:].reshape(x.shape[:-1] + (D, D))
        dx += np.einsum("...mr,...r->...m", d2 + np.swapaxes(d2, -1, -2), x)
    return dx


def moment_state(k, v, poly: Poly):
    """Total state of a block of keys: (M, Dv+1) per head (un-weighted sums of Phi(k)^T [v|1])."""
    k = np.asarray(k, np.float64)
    v1 = np.concatenate([np.asarray(v, np.float64), np.ones(v.shape[:-1] + (1,))], -1)
    return np.einsum("...nf,...nj->...fj", _phi(k, poly.p), v1)


def fastmax_streaming(q, k, v, mask: bool, poly: Poly, chunk: int = 64, state_in=None, return_state=False):
    """One head at a time: q (nq,D), k (nk,D), v (nk,Dv), optional carried state (M,Dv+1).

    With mask=True and nk > nq the first nk-nq keys are a prefix visible to every query.
    `state_in` lets a caller continue a sequence that was split into contiguous pieces.
    """
    q = np.asarray(q, np.float64)
    k = np.asarray(k, np.float64)
    v = np.asarray(v, np.float64)
    nq, D = q.shape
    nk, Dv = v.shape
    w = _weights(D, poly)
    v1 = np.concatenate([v, np.ones((nk, 1))], -1)
    M = w.shape[0]
    S = np.zeros((M, Dv + 1)) if state_in is None else np.array(state_in, np.float64)
    Op = np.zeros((nq, Dv + 1))
    if not mask:
        S = S + _phi(k, poly.p).T @ v1
        for c0 in range(0, nq, chunk):
            Op[c0:c0 + chunk] = (_phi(q[c0:c0 + chunk], poly.p) * w) @ S
    else:
        off = nk - nq
        if off:
            S = S + _phi(k[:off], poly.p).T @ v1[:off]
        for c0 in range(0, nq, chunk):
            qc = q[c0:c0 + chunk]
            kc = k[off + c0:off + c0 + chunk]
            vc = v1[off + c0:off + c0 + chunk]
            P = np.tril(poly.f(qc @ kc.T * poly.inv_temp))
            Op[c0:c0 + chunk] = (_phi(qc, poly.p) * w) @ S + P @ vc
            S = S + _phi(kc, poly.p).T @ vc
    o = Op[:, :Dv] / Op[:, Dv:]
    if return_state:
        return o, Op[:, Dv], S
    return o, Op[:, Dv]


def grad_moment_state(q, do, o, g, poly: Poly):
    """Gradient moments of a block of queries: sum_l Phi(q_l)^T dO'_l, (M, Dv+1), un-weighted."""
    q = np.asarray(q, np.float64)
    do = np.asarray(do, np.float64)
    dO = np.concatenate([do / g[:, None], (-(do * o).sum(-1) / g)[:, None]], -1)
    return _phi(q, poly.p).T @ dO


def fastmax_streaming_grads(q, k, v, do, mask: bool, poly: Poly, chunk: int = 64, state_in=None, dstate_in=None,
                            return_dstate=False):
    """Chunked two-scan backward for one head (nq == nk when causal).  Returns dq, dk, dv.

    state_in: moments of keys that precede this piece (as in the forward); dstate_in: gradient moments
    sum Phi(q)^T dO' of the queries that FOLLOW this piece.  With return_dstate the piece's own gradient
    moments added to dstate_in are returned too (what a sequence-parallel rank hands to the rank before it)."""
    q = np.asarray(q, np.float64)
    k = np.asarray(k, np.float64)
    v = np.asarray(v, np.float64)
    do = np.asarray(do, np.float64)
    nq, D = q.shape
    nk, Dv = v.shape
    o, g = fastmax_streaming(q, k, v, mask, poly, chunk, state_in=state_in)
    w = _weights(D, poly)
    v1 = np.concatenate([v, np.ones((nk, 1))], -1)
    dO = np.concatenate([do / g[:, None], (-(do * o).sum(-1) / g)[:, None]], -1)
    dq = np.zeros_like(q)
    dk = np.zeros_like(k)
    dv = np.zeros_like(v)
    M = w.shape[0]
    if not mask:
        S = _phi(k, poly.p).T @ v1
        dS = _phi(q, poly.p).T @ dO
        dq = _dphi_to_dx((dO @ S.T) * w, q, poly.p)
        dk = _dphi_to_dx((v1 @ dS.T) * w, k, poly.p)
        dv = ((_phi(k, poly.p) * w) @ dS)[:, :Dv]
        return dq, dk, dv
    assert nq == nk
    # forward-direction scan: dq
    S = np.zeros((M, Dv + 1)) if state_in is None else np.array(state_in, np.float64)
    for c0 in range(0, nq, chunk):
        sl = slice(c0, c0 + chunk)
        sc = q[sl] @ k[sl].T * poly.inv_temp
        dA = np.tril((dO[sl] @ v1[sl].T) * poly.df(sc))
        dq[sl] = _dphi_to_dx((dO[sl] @ S.T) * w, q[sl], poly.p) + dA @ k[sl] * poly.inv_temp
        S = S + _phi(k[sl], poly.p).T @ v1[sl]
    # reverse-direction scan: dk, dv
    dS = np.zeros((M, Dv + 1)) if dstate_in is None else np.array(dstate_in, np.float64)
    starts = list(range(0, nq, chunk))
    for c0 in reversed(starts):
        sl = slice(c0, c0 + chunk)
        sc = q[sl] @ k[sl].T * poly.inv_temp
        A = np.tril(poly.f(sc))
        dA = np.tril((dO[sl] @ v1[sl].T) * poly.df(sc))
        dk[sl] = _dphi_to_dx((v1[sl] @ dS.T) * w, k[sl], poly.p) + dA.T @ q[sl] * poly.inv_temp
        dv[sl] = ((_phi(k[sl], poly.p) * w) @ dS)[:, :Dv] + A.T @ dO[sl][:, :Dv]
        dS = dS + _phi(q[sl], poly.p).T @ dO[sl]
    if return_dstate:
        return dq, dk, dv, dS
    return dq, dk, dv


# --------------------------------------------------------------------------------------------
# 4. exact sampled rows / columns for full-size configs (O(N D) per sample, fp64).
# --------------------------------------------------------------------------------------------
def sampled_forward_rows(q, k, v, rows, mask: bool, poly: Poly):
    """o and g for the given query rows of ONE head.  q (nq,D), k (nk,D), v (nk,Dv)."""
    q = np.asarray(q, np.float64)
    k = np.asarray(k, np.float64)
    v = np.asarray(v, np.float64)
    off = k.shape[0] - q.shape[0]
    o = np.zeros((len(rows), v.shape[1]))
    g = np.zeros(len(rows))
    for i, l in enumerate(rows):
        hi = off + l + 1 if mask else k.shape[0]
        a = poly.f(k[:hi] @ q[l] * poly.inv_temp)
        g[i] = a.sum()
        o[i] = a @ v[:hi] / g[i]
    return o, g


def sampled_dq_rows(q, k, v, o, g, do, rows, mask: bool, poly: Poly):
    """dq for the given query rows of one head; o, g, do are the full (nq, .) arrays of that head."""
    q = np.asarray(q, np.float64)
    k = np.asarray(k, np.float64)
    v = np.asarray(v, np.float64)
    off = k.shape[0] - q.shape[0]
    out = np.zeros((len(rows), q.shape[1]))
    for i, l in enumerate(rows):
        hi = off + l + 1 if mask else k.shape[0]
        s = k[:hi] @ q[l] * poly.inv_temp
        dog = np.asarray(do[l], np.float64) / g[l]
        dgl = -(np.asarray(do[l], np.float64) * o[l]).sum() / g[l]
        dA = v[:hi] @ dog + dgl
        out[i] = (dA * poly.df(s)) @ k[:hi] * poly.inv_temp
    return out


def sampled_dkv_cols(q, k, v, o, g, do, cols, mask: bool, poly: Poly):
    """dk, dv for the given key positions of one head (needs the full o, g, do of that head)."""
    q = np.asarray(q, np.float64)
    k = np.asarray(k, np.float64)
    v = np.asarray(v, np.float64)
    o = np.asarray(o, np.float64)
    g = np.asarray(g, np.float64)
    do = np.asarray(do, np.float64)
    off = k.shape[0] - q.shape[0]
    dog = do / g[:, None]
    dg = -(do * o).sum(-1) / g
    dk = np.zeros((len(cols), k.shape[1]))
    dv = np.zeros((len(cols), v.shape[1]))
    for i, j in enumerate(cols):
        lo = max(j - off, 0) if mask else 0
        s = q[lo:] @ k[j] * poly.inv_temp
        dA = dog[lo:] @ v[j] + dg[lo:]
        dk[i] = (dA * poly.df(s)) @ q[lo:] * poly.inv_temp
        dv[i] = poly.f(s) @ dog[lo:]
    return dk, dv


# --------------------------------------------------------------------------------------------
# 5. q/k normalisation (einops.py:327-334): per-token mean-subtract over d, then divide the
#    whole head by its largest token L2 norm; the op multiplies by `lim`.
# --------------------------------------------------------------------------------------------
def normalize(x, lim: float = 1.0):
    x = np.asarray(x, np.float64)
    xc = x - x.mean(-1, keepdims=True)
    nrm = np.sqrt((xc * xc).sum(-1))
    return lim * xc / nrm.max(-1)[..., None, None]


def normalize_grad(x, dy, lim: float = 1.0):
    """Gradient of sum(normalize(x) * dy) w.r.t. x; the max flows only through its arg-max token."""
    x = np.asarray(x, np.float64)
    dy = np.asarray(dy, np.float64)
    xc = x - x.mean(-1, keepdims=True)
    nrm = np.sqrt((xc * xc).sum(-1))
    m = nrm.max(-1)
    am = nrm.argmax(-1)
    dxc = lim * dy / m[..., None, None]
    coef = -lim * (dy * xc).sum((-1, -2)) / (m * m)          # d/dm
    flat_xc = xc.reshape(-1, xc.shape[-2], xc.shape[-1])
    add = np.zeros_like(flat_xc)
    cf = coef.reshape(-1)
    amf = am.reshape(-1)
    mf = m.reshape(-1)
    for i in range(flat_xc.shape[0]):
        add[i, amf[i]] = cf[i] * flat_xc[i, amf[i]] / mf[i]
    dxc = dxc + add.reshape(xc.shape)
    return dxc - dxc.mean(-1, keepdims=True)


# --------------------------------------------------------------------------------------------
# 5b. the two steps of forward_cuda that the reference carries but never performs
#     (fastmax_cuda_forward.cu:282-292 with the commented-out line 289; :340-349 called with scale 0 at :443)
# --------------------------------------------------------------------------------------------
def key_prologue(k, inv_temp: float, rpe=None):
    """k[l] * inv_temp + rpe[(l + nk) mod (2 nk - 1)]   (apply_rpe_and_temp with its RPE line switched on)."""
    k = np.asarray(k, np.float64) * inv_temp
    if rpe is not None:
        nk = k.shape[-2]
        idx = (np.arange(nk) + nk) % (2 * nk - 1)
        k = k + np.asarray(rpe, np.float64)[idx]
    return k


def output_noise(o, noise, scale: float):
    """o * (1 + scale * noise)   (apply_dropout, fastmax_cuda_forward.cu:340-349)."""
    return np.asarray(o, np.float64) * (1.0 + scale * np.asarray(noise, np.float64))


# --------------------------------------------------------------------------------------------
# 6. error metric used by every parity test (outputs cross zero, so errors are normalised by the
#    tensor's largest magnitude, never element by element).
# --------------------------------------------------------------------------------------------
def max_norm_err(x, ref) -> float:
    x = np.asarray(x, np.float64)
    ref = np.asarray(ref, np.float64)
    return float(np.abs(x - ref).max() / max(np.abs(ref).max(), 1e-300))
