"""B200-native Fastmax attention: a drop-in for the reference's `fastmax_cuda` operator path.

Importing this package makes the in-tree PyTorch extension importable under the reference's module
name, `fastmax_cuda` (the reference does `import fastmax_cuda`, transformer/model.py:5).
There is no CPU fallback: a missing native build raises ImportError.
"""
import os as _os
import sys as _sys

_PKG = _os.path.dirname(_os.path.abspath(__file__))
if _PKG not in _sys.path:
    _sys.path.insert(0, _PKG)


def load_extension():
    """Imports and returns the `fastmax_cuda` extension module (raises ImportError when it is not built)."""
    import torch  # noqa: F401  (the extension links against libtorch)

    try:
        import fastmax_cuda
    except ImportError as e:  # pragma: no cover - exercised only on an unbuilt tree
        raise ImportError(
            "the fastmax_cuda extension is not built (no CPU fallback exists); run "
            "`python -m reproducing_fastmax_results_b200.build`") from e
    return fastmax_cuda


from .attention import (  # noqa: E402
    FastMax,
    FASTMultiHeadAttention,
    FASTMultiHeadAttention_Function,
    fastmax,
    fastmax_custom,
    rpe_matrix_creator,
)

__all__ = [
    "FastMax", "FASTMultiHeadAttention", "FASTMultiHeadAttention_Function", "fastmax", "fastmax_custom",
    "rpe_matrix_creator", "load_extension",
]
