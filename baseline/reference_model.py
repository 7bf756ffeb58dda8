"""Loader for the reference's transformer (transformer/model.py) as vendored by baseline/vendor_reference.py.

The model is the REFERENCE's code (one documented edit, see vendor_reference.py); the operator underneath is this
package: model.py does `import fastmax_cuda` (model.py:5) and calls `fastmax_cuda.forwardpass / backwardpass` from its
own autograd Function (model.py:34, 63), so importing the package first (it puts the in-tree extension on the
import path under that name) is all the wiring there is.
"""
import importlib
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.path.join(HERE, "_ref")


def available():
    return os.path.exists(os.path.join(REF, "transformer", "model.py"))


def load():
    """Returns the vendored `transformer.model` module (classes Attention, TransformerBlock, Transformer and the
    module-level `fastmax_custom`).  Raises FileNotFoundError when vendor_reference.py has not been run."""
    if not available():
        raise FileNotFoundError(
            "baseline/_ref/transformer/model.py is missing: run "
            "`python baseline/vendor_reference.py <checkout of the reference>` first")
    import reproducing_fastmax_results_b200  # noqa: F401  makes `import fastmax_cuda` resolve to the in-tree extension

    try:
        import kornia  # noqa: F401
    except ImportError:
        pass
    if REF not in sys.path:
        # appended, not prepended: a real kornia (or a real `transformer` package) earlier on the path wins only for
        # kornia; the vendored package is imported under a private name below so it cannot be shadowed
        sys.path.append(REF)
    if "fastmax_reference_transformer" in sys.modules:
        return sys.modules["fastmax_reference_transformer"].model
    spec = importlib.util.spec_from_file_location(
        "fastmax_reference_transformer", os.path.join(REF, "transformer", "__init__.py"),
        submodule_search_locations=[os.path.join(REF, "transformer")])
    pkg = importlib.util.module_from_spec(spec)
    sys.modules["fastmax_reference_transformer"] = pkg
    spec.loader.exec_module(pkg)
    model = importlib.import_module("fastmax_reference_transformer.model")
    pkg.model = model
    return model
