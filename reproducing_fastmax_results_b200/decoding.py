"""Token-by-token Fastmax attention with a carried moment state.

The reference generates text by running the whole model, and with it the attention operator, on the full token
window for every new token (transformer/eval.py:8-32: `logits = model(token_chunk)` inside the loop over
`max_new_tokens`).  Fastmax attention does not need that: everything a later query needs from the keys and
values seen so far is the fixed-size moment state S = sum_j Phi(k_j)^T [v_j | 1].  `FastmaxDecoder` keeps that
state on the device; `prefill` runs the causal operator over a prompt and leaves the state behind, `step`
feeds one token per (batch, head) through `fastmax_decode_step`, whose cost does not depend on how many tokens
came before.

The q/k normalisation of the operator (`normalize=True`) divides by the largest token norm of the whole
sequence and therefore cannot be evaluated incrementally; the decoder takes un-normalised q and k, as the
reference's CPU implementations do by default (fastattention_einops.py:78-82).
"""
from __future__ import annotations

from . import _lib


class FastmaxDecoder:
    """Causal Fastmax attention over a growing sequence.

    batch, heads, d, p: problem geometry (d in {16, 32, 64}; p = polynomial order 1 or 2).
    temperature, a0, a1, a2: as in `fastmax_custom` (scores are q.k / temperature).
    The state is float32 (batch, heads, rows, d + 4) in the layout of `fastmax_forward`'s state_out and is
    updated in place by every call.
    """

    def __init__(self, batch, heads, d, p=2, temperature=1.0, a0=1.0, a1=1.0, a2=0.5, device="cuda"):
        if d not in (16, 32, 64):
            raise ValueError("head dim must be 16, 32 or 64")
        if p not in (1, 2):
            raise ValueError("p must be 1 or 2")
        self.batch, self.heads, self.d, self.p = int(batch), int(heads), int(d), int(p)
        self.inv_temperature = 1.0 / float(temperature)
        self.a0, self.a1, self.a2 = float(a0), float(a1), float(a2)
        self.state = _lib.new_state(self.batch, self.heads, self.d, self.p, device)
        self.tokens_seen = 0

    def reset(self):
        self.state.zero_()
        self.tokens_seen = 0

    def _check(self, t, name):
        if t.shape[0] != self.batch or t.shape[1] != self.heads or t.shape[-1] != self.d:
            raise ValueError(f"{name}: expected ({self.batch}, {self.heads}, ..., {self.d}), got {tuple(t.shape)}")

    def prefill(self, q, k, v):
        """Causal attention of a (b, h, n, d) block that continues the sequence seen so far.  Returns o (b, h, n, d)
        and adds the block's keys and values to the state."""
        for t, name in ((q, "q"), (k, "k"), (v, "v")):
            self._check(t, name)
        if q.dim() != 4 or q.shape[2] != k.shape[2]:
            raise ValueError("prefill takes (b, h, n, d) tensors with as many queries as keys")
        o, _, state = _lib.forward(q, k, v, True, self.inv_temperature, self.a0, self.a1, self.a2, self.p,
                                   state_in=self.state if self.tokens_seen else None, want_state=True)
        self.state = state
        self.tokens_seen += q.shape[2]
        return o

    def step(self, q, k, v, out=None):
        """One new token per (batch, head): q, k, v are (b, h, d) or (b, h, 1, d).  Returns o shaped like q."""
        for t, name in ((q, "q"), (k, "k"), (v, "v")):
            self._check(t, name)
        o, _ = _lib.decode_step(q, k, v, self.state, self.inv_temperature, self.a0, self.a1, self.a2, self.p, out=out)
        self.tokens_seen += 1
        return o
