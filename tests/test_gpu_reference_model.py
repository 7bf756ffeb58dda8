"""The reference's own transformer code (transformer/model.py, vendored by baseline/vendor_reference.py) running on
this package's `fastmax_cuda` extension: its Attention block (model.py:252-340) forward + backward against the same
block evaluated on the CPU in float64 with the oracle as the attention operator, and one training step of the small
Transformer (model.py:370-465).  The second caller of the operator (the nanoGPT-style head of
`nano_gpt fastmax copy.py:330-378`) is restated at the end: same call, (batch, heads, block, head-dim) reshape."""
import numpy as np
import pytest
import torch

from baseline import reference_model
from oracle import fastmax_oracle as orc

pytestmark = [pytest.mark.gpu,
              pytest.mark.skipif(not reference_model.available(),
                                 reason="baseline/_ref is not populated (python baseline/vendor_reference.py <reference>)")]


class _OracleAttention(torch.autograd.Function):
    """Fastmax through the oracle with the reference Function's gradient convention (model.py:51-74): q and k are
    normalised inside the forward, the gradients are those w.r.t. the NORMALISED q, k (no Jacobian of the
    normalisation), and dk is divided by the temperature."""

    @staticmethod
    def forward(ctx, q, k, v, mask, normalize, temperature, lim, p):
        qn, kn, vn = (t.detach().numpy().astype(np.float64) for t in (q, k, v))
        if normalize:
            qn, kn = orc.normalize(qn, lim), orc.normalize(kn, lim)
        poly = orc.Poly(1.0, 1.0, 0.5, 1.0 / temperature, p)
        o, _ = orc.fastmax_naive(qn, kn, vn, mask, poly)
        ctx.saved = (qn, kn, vn, mask, poly)
        return torch.from_numpy(o)

    @staticmethod
    def backward(ctx, do):
        qn, kn, vn, mask, poly = ctx.saved
        dq, dk, dv = orc.fastmax_naive_grads(qn, kn, vn, do.numpy().astype(np.float64), mask, poly)
        return torch.from_numpy(dq), torch.from_numpy(dk), torch.from_numpy(dv), None, None, None, None, None


def _block_on_cpu(attn, x, mask, normalize, p):
    """Attention.forward (model.py:272-340) restated in float64 on the CPU around the oracle."""
    w = {n: t.detach().double().cpu().requires_grad_(True) for n, t in attn.named_parameters()}
    xc = x.detach().double().cpu().requires_grad_(True)
    b, n, _ = xc.shape
    h, dh = attn.h, attn.d_head
    split = lambda t: t.view(b, n, h, dh).transpose(1, 2)
    q = split(xc @ w["query_transform.weight"].T)
    k = split(xc @ w["key_transform.weight"].T)
    v = split(xc @ w["value_transform.weight"].T)
    vh = _OracleAttention.apply(q, k, v, mask, normalize, 1.0, 1.0, p)
    vh = vh.transpose(1, 2).contiguous().view(b, n, h * dh)
    out = vh @ w["linear.weight"].T + w["linear.bias"]
    return out, xc, w


@pytest.mark.parametrize("p", [1, 2])
@pytest.mark.parametrize("d_head", [32, 64])
def test_reference_attention_block_on_the_new_operator(p, d_head):
    """p = 1 with mask and normalisation is the block exactly as shipped (model.py:292-300); p = 2 is the benchmark's
    configuration."""
    model = reference_model.load()
    torch.manual_seed(0)
    h, n, b = 4, 96, 2
    d_model = h * d_head
    attn = model.Attention(d_model, d_head, h, dropout_rate=0.0, use_masking=True, fastmax=True, normalize=True, p=p).cuda()
    x = torch.randn(b, n, d_model, device="cuda", requires_grad=True)
    upstream = torch.randn(b, n, d_model, device="cuda")
    from reproducing_fastmax_results_b200 import _lib

    before = _lib.load().fastmax_launch_count()
    out, amap = attn(x)
    assert amap is None
    (out * upstream).sum().backward()
    torch.cuda.synchronize()
    assert _lib.load().fastmax_launch_count() > before, "the block did not reach this library's kernels"
    ref, xc, w = _block_on_cpu(attn, x, True, True, p)
    (ref * upstream.double().cpu()).sum().backward()
    tol = 1e-4
    assert orc.max_norm_err(out.detach().cpu().numpy(), ref.detach().numpy()) < tol
    assert orc.max_norm_err(x.grad.cpu().numpy(), xc.grad.numpy()) < tol
    for name, prm in attn.named_parameters():
        assert orc.max_norm_err(prm.grad.cpu().numpy(), w[name].grad.numpy()) < tol, name


def test_reference_transformer_training_step():
    """Transformer(..., fastmax=True, p=2) (model.py:370-465) takes optimiser steps on the new operator: finite loss
    that goes down on a repeated batch, every parameter receives a gradient."""
    model = reference_model.load()
    torch.manual_seed(0)
    vocab, n = 97, 64
    net = model.Transformer(out_dim=vocab, max_tokens=n, d_model=128, d_mlp=256, heads_per_block=4, num_blocks=2,
                            dropout_rate=0.0, use_masking=True, vocab_size=vocab, fastmax=True, p=2).cuda()
    opt = torch.optim.AdamW(net.parameters(), lr=3e-4)
    ids = torch.randint(0, vocab, (4, n + 1), device="cuda")
    losses = []
    for _ in range(8):
        logits = net(ids[:, :-1])
        loss = torch.nn.functional.cross_entropy(logits.reshape(-1, vocab), ids[:, 1:].reshape(-1))
        opt.zero_grad(set_to_none=True)
        loss.backward()
        if not losses:
            assert all(prm.grad is not None and torch.isfinite(prm.grad).all() for prm in net.parameters())
        opt.step()
        losses.append(float(loss))
    assert all(np.isfinite(losses)) and losses[-1] < losses[0], losses


def test_zero_copy_operator_in_the_reference_block_bf16():
    """The same block with the package's `fastmax_custom` (FastMax: strided views, bfloat16) in place of the module-level
    one, under bf16 autocast: the call site (model.py:303) is untouched, the tensor-memory kernels take the call."""
    import reproducing_fastmax_results_b200 as pkg
    from reproducing_fastmax_results_b200 import _lib

    model = reference_model.load()
    torch.manual_seed(1)
    h, d_head, n, b = 8, 64, 256, 4
    d_model = h * d_head
    attn = model.Attention(d_model, d_head, h, dropout_rate=0.0, use_masking=True, fastmax=True, normalize=True, p=2).cuda()
    x = torch.randn(b, n, d_model, device="cuda", requires_grad=True)
    upstream = torch.randn(b, n, d_model, device="cuda")
    saved = model.fastmax_custom
    model.fastmax_custom = pkg.fastmax_custom
    try:
        _lib.profile_collect()
        _lib.profile(True)
        with torch.autocast("cuda", dtype=torch.bfloat16):
            out, _ = attn(x)
        (out.float() * upstream).sum().backward()
        torch.cuda.synchronize()
    finally:
        _lib.profile(False)
        model.fastmax_custom = saved
    kinds = set(_lib.profile_collect())
    assert "tc_scan_fwd" in kinds and "tc_scan_bwd_q" in kinds, kinds
    # comparator: float64 block with the exact normalisation gradient (FastMax differentiates through it)
    w = {nm: t.detach().double().cpu() for nm, t in attn.named_parameters()}
    xc = x.detach().double().cpu()
    split = lambda t: t.view(b, n, h, d_head).transpose(1, 2).numpy()
    q, k, v = (split(xc @ w[nm + "_transform.weight"].T) for nm in ("query", "key", "value"))
    o, _ = orc.fastmax_naive(orc.normalize(q), orc.normalize(k), v, True, orc.Poly(1.0, 1.0, 0.5, 1.0, 2))
    ref = torch.from_numpy(o).transpose(1, 2).reshape(b, n, d_model) @ w["linear.weight"].T + w["linear.bias"]
    assert orc.max_norm_err(out.detach().float().cpu().numpy(), ref.numpy()) < 2e-2
    assert torch.isfinite(x.grad).all() and float(x.grad.abs().max()) > 0


def test_nanogpt_style_head_calls_the_operator():
    """`nano_gpt fastmax copy.py:358-377`: q, k, v projected per head, reshaped to (batch, heads, block, dim) and passed
    to fastmax_custom with mask, normalisation, temperature 1 and the script's p; checked against the oracle."""
    import reproducing_fastmax_results_b200 as pkg

    torch.manual_seed(2)
    batch, heads, block, dim, n_embd = 3, 2, 40, 16, 48
    x = torch.randn(batch * heads, block, n_embd, device="cuda")
    wq, wk, wv = (torch.randn(n_embd, dim, device="cuda") / n_embd ** 0.5 for _ in range(3))
    q, k, v = ((x @ w).reshape(batch, heads, block, dim).requires_grad_(True) for w in (wq, wk, wv))
    rpe = pkg.rpe_matrix_creator(block, dim, q.device, q.dtype, structured=False, is_zero=True).contiguous()
    noise = torch.normal(0, 1, size=q.shape, dtype=q.dtype, device=q.device).contiguous()
    for p in (1, 2):
        for fn in (pkg.FASTMultiHeadAttention(zero_copy=False), pkg.fastmax_custom):
            out = fn(q, k, v, noise, rpe, True, 0.1, True, 1.0, 1.0, 1.0, 0.5, 1.0, p)
            qn, kn = orc.normalize(q.detach().cpu().numpy()), orc.normalize(k.detach().cpu().numpy())
            ref, _ = orc.fastmax_naive(qn, kn, v.detach().double().cpu().numpy(), True, orc.Poly(1.0, 1.0, 0.5, 1.0, p))
            assert orc.max_norm_err(out.detach().cpu().numpy(), ref) < 1e-4
            out.sum().backward()
            assert torch.isfinite(q.grad).all()
