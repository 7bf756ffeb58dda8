"""Seeded inputs shared by the golden-vector generator and the parity tests.

Inputs come from numpy's PCG64 generator (bit-stable across numpy versions and machines), so the
fixtures only need to store the reference's OUTPUTS.
"""
import numpy as np

# name -> (B, H, N, D, p, mask, normalize_term, scale, upstream)
CASES = {
    # BASELINE config 1: the reference's own CPU-runnable case, ones-like upstream gradient.
    "cfg1_p2_noncausal": (2, 4, 256, 32, 2, False, 8.0, 1.0, "ones"),
    "small_p1_noncausal": (2, 2, 48, 16, 1, False, 8.0, 1.0, "randn"),
    "small_p2_noncausal": (2, 2, 48, 16, 2, False, 8.0, 1.0, "randn"),
    "small_p1_causal": (2, 2, 48, 16, 1, True, 8.0, 1.0, "randn"),
    "small_p2_causal": (2, 2, 48, 16, 2, True, 8.0, 1.0, "randn"),
    # sharper temperature so the quadratic term matters, ragged N (not a multiple of any chunk)
    "ragged_p2_causal": (1, 3, 37, 32, 2, True, 0.5, 1.0, "randn"),
    "ragged_p2_noncausal": (1, 3, 37, 32, 2, False, 0.5, 1.0, "randn"),
    "d64_p2_causal": (1, 2, 40, 64, 2, True, 1.0, 0.5, "randn"),
}


def make_inputs(name):
    B, H, N, D, p, mask, nt, scale, upstream = CASES[name]
    seed = sorted(CASES).index(name)
    rng = np.random.default_rng(seed)
    q = (rng.standard_normal((B, H, N, D)) * scale).astype(np.float32)
    k = (rng.standard_normal((B, H, N, D)) * scale).astype(np.float32)
    v = (rng.standard_normal((B, H, N, D)) * scale).astype(np.float32)
    if upstream == "ones":
        do = np.ones((B, H, N, D), dtype=np.float32)
    else:
        do = rng.standard_normal((B, H, N, D)).astype(np.float32)
    return q, k, v, do
