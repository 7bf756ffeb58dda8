"""Writes tests/golden/reference_vectors.npz by running the REFERENCE implementation.

Run in a checkout that has the reference repository next to it:
    python tests/golden/make_golden.py /path/to/reproducing_fastmax_results
It imports attention_mechanisms/fastattention_einops.py (forward + its hand-derived backward) and
attention_mechanisms/score_function.py (pure-torch twin, autograd backward) unmodified, feeds them the
seeded inputs of tests/golden/cases.py in float64 and stores outputs and gradients as float32.
The reference is not needed to run the tests; only this script reads it.
"""
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
from cases import CASES, make_inputs  # noqa: E402


def main(ref_root):
    sys.path.insert(0, os.path.join(ref_root, "attention_mechanisms"))
    import fastattention_einops as ein  # noqa
    import score_function as score  # noqa

    out = {}
    for name, (B, H, N, D, p, mask, nt, scale, upstream) in CASES.items():
        q, k, v, do = (torch.from_numpy(x).double() for x in make_inputs(name))
        # einops Function (factorised forward, hand-derived factorised backward)
        qe, ke, ve = (t.clone().requires_grad_(True) for t in (q, k, v))
        o = ein.fastmax(qe, ke, ve, mask=mask, normalize_term=nt, tensors_normalized=False, p=p)
        o.backward(do)
        out[f"{name}/einops/o"] = o.detach().numpy().astype(np.float32)
        out[f"{name}/einops/dq"] = qe.grad.numpy().astype(np.float32)
        out[f"{name}/einops/dk"] = ke.grad.numpy().astype(np.float32)
        out[f"{name}/einops/dv"] = ve.grad.numpy().astype(np.float32)
        # score_function.fastmax (autograd)
        qs, ks, vs = (t.clone().requires_grad_(True) for t in (q, k, v))
        o2 = score.fastmax(qs, ks, vs, mask=mask, denum_term=nt, normalize=0, p=p)
        o2.backward(do)
        out[f"{name}/score/o"] = o2.detach().numpy().astype(np.float32)
        out[f"{name}/score/dq"] = qs.grad.numpy().astype(np.float32)
        # q/k normalisation of einops.py:327-334 with autograd gradients
        if name.startswith("small_p2"):
            qn, kn = (t.clone().requires_grad_(True) for t in (q, k))
            a, b = ein.fastattention_einops.normalize(qn, kn)
            (a * do).sum().backward()
            (b * do).sum().backward()
            out[f"{name}/normalize/q"] = a.detach().numpy().astype(np.float32)
            out[f"{name}/normalize/k"] = b.detach().numpy().astype(np.float32)
            out[f"{name}/normalize/dq"] = qn.grad.numpy().astype(np.float32)
            out[f"{name}/normalize/dk"] = kn.grad.numpy().astype(np.float32)
            # normalised attention end to end (tensors_normalized=True -> temperature 1)
            qn2, kn2, vn2 = (t.clone().requires_grad_(True) for t in (q, k, v))
            a2, b2 = ein.fastattention_einops.normalize(qn2, kn2)
            on = ein.fastmax(a2, b2, vn2, mask=mask, normalize_term=nt, tensors_normalized=True, p=p)
            on.backward(do)
            out[f"{name}/normalized_attention/o"] = on.detach().numpy().astype(np.float32)
            out[f"{name}/normalized_attention/dq"] = qn2.grad.numpy().astype(np.float32)
            out[f"{name}/normalized_attention/dk"] = kn2.grad.numpy().astype(np.float32)
            out[f"{name}/normalized_attention/dv"] = vn2.grad.numpy().astype(np.float32)
    path = os.path.join(HERE, "reference_vectors.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes,", len(out), "arrays")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: python make_golden.py <checkout of armingerami/reproducing_fastmax_results>")
    main(sys.argv[1])
