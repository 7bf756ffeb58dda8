"""The workspace-free forward entry point (fastmax_forward_static_scratch).

It exists for callers that cannot allocate device memory at call time (a plugin inside a serving runtime
that owns all of HBM, an FFI host without an allocator, a no-allocation-after-start-up rule): the scratch is a
fixed array inside the library.  The test calls it through the C ABI twice in a row (the array is shared and
keeps the previous call's contents) and compares with the ordinary entry point on the same inputs.
This file sorts last on purpose, so a run that stops at the first failure has already run everything else.
"""
import ctypes as C
import math

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _inputs(B, H, N, D, dtype, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return tuple(torch.randn(B, H, N, D, device="cuda", generator=g).to(dtype) for _ in range(3))


@pytest.mark.parametrize("case", [
    (1, 4, 300, 32, torch.float32, 1e-4, 1e-4),    # CUDA-core engine, ragged length
    (2, 8, 512, 64, torch.bfloat16, 2e-2, 1e-4),   # tensor-core engine
    # the padded tensor-core form needs 16 MB of scratch, the CUDA-core engine 3 MB: it runs there, while the ordinary
    # call it is compared with takes the tensor-core form (two engines: the denominators agree to bf16 accuracy)
    (4, 20, 256, 32, torch.bfloat16, 2e-2, 5e-3),
])
def test_static_scratch_forward_matches_workspace_forward_twice(case):
    from reproducing_fastmax_results_b200 import _lib as L

    B, H, N, D, dtype, tol, gtol = case
    inv_temp = 1.0 / (4.0 * math.sqrt(D))
    for call in range(2):  # second call: different data over the scratch the first call left behind
        q, k, v = _inputs(B, H, N, D, dtype, seed=100 + call)
        o_ref, g_ref, _ = L.forward(q, k, v, True, inv_temp, order=2)
        o, g = L.forward_static_scratch(q, k, v, True, inv_temp, order=2)
        L.check_status()
        scale = float(o_ref.float().abs().max())
        assert float((o.float() - o_ref.float()).abs().max()) <= tol * scale
        assert torch.allclose(g, g_ref, rtol=gtol, atol=gtol * float(g_ref.abs().max()))


def test_static_scratch_rejects_problems_beyond_its_size():
    from reproducing_fastmax_results_b200 import _lib as L

    lib = L.load()
    assert lib.fastmax_static_scratch_bytes() == 8 << 20
    q, k, v = _inputs(2, 16, 4096, 64, torch.bfloat16, seed=3)   # needs ~36 MB of scratch
    with pytest.raises(L.FastmaxError) as e:
        L.forward_static_scratch(q, k, v, True, 0.05, order=2)
    assert e.value.status == 7
    # nothing was launched and the device is fine: the ordinary call still works
    o, g, _ = L.forward(q, k, v, True, 0.05, order=2)
    L.check_status()
    assert torch.isfinite(o.float()).all()
