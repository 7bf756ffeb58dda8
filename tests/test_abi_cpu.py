"""CPU-side checks of the C-ABI library: it loads, exports every declared symbol, and validates arguments
before touching the GPU (no kernel is launched here)."""
import ctypes as C
import os
import re

import pytest

from reproducing_fastmax_results_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_functions():
    text = open(os.path.join(ROOT, "include", "fastmax_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(fastmax_[a-z_0-9]+)\s*\(", text)))


def test_header_symbols_are_exported():
    lib = _lib.load()
    names = _declared_functions()
    assert len(names) >= 12
    for n in names:
        assert hasattr(lib, n), f"{n} is declared in include/fastmax_b200.h but not exported"
    assert set(_lib.EXPORTED_SYMBOLS) <= set(names)


def test_state_geometry():
    lib = _lib.load()
    assert lib.fastmax_state_rows(64, 2) == 36 * 64 + 65
    assert lib.fastmax_state_rows(32, 2) == 10 * 64 + 33
    assert lib.fastmax_state_rows(16, 2) == 3 * 64 + 17
    assert lib.fastmax_state_rows(64, 1) == 65
    assert lib.fastmax_state_ld(64) == 68
    pb = _lib.Problem(2, 3, 10, 10, 32, 2, 1, 0, 1, 1, 0.5, 1.0, 0, 0)
    assert lib.fastmax_state_bytes(C.byref(pb)) == 6 * 673 * 36 * 4


def _args(ptr=4096):
    a = _lib.ForwardArgs()
    for t in (a.q, a.k, a.v, a.o, a.g):
        t.ptr, t.stride_b, t.stride_h, t.stride_n = ptr, 64 * 32, 32 * 64, 32
    return a


@pytest.mark.parametrize("field,value,status", [
    ("d", 48, 2), ("order", 3, 2), ("dtype", 7, 1), ("batch", 0, 1), ("nq", 200, 2),
])
def test_forward_rejects_bad_problem(field, value, status):
    lib = _lib.load()
    pb = _lib.Problem(1, 2, 64, 64, 32, 2, 1, 0, 1, 1, 0.5, 1.0, 0, 0)
    setattr(pb, field, value)
    a = _args()
    assert lib.fastmax_forward(C.byref(pb), C.byref(a), None, 0, None) == status
    assert lib.fastmax_status_string(status)


def test_forward_rejects_misaligned_and_small_workspace():
    lib = _lib.load()
    pb = _lib.Problem(1, 2, 64, 64, 32, 2, 1, 0, 1, 1, 0.5, 1.0, 0, 0)
    a = _args(ptr=4100)
    assert lib.fastmax_forward(C.byref(pb), C.byref(a), None, 0, None) == 6
    a = _args()
    a.k.stride_n = 33
    assert lib.fastmax_forward(C.byref(pb), C.byref(a), None, 0, None) == 6
    a = _args()
    need = lib.fastmax_forward_workspace(C.byref(pb), C.byref(a))
    assert need > 2 * 64 * 36 * 4
    assert lib.fastmax_forward(C.byref(pb), C.byref(a), C.c_void_p(4096), need - 1, None) == 3
    assert lib.fastmax_forward(C.byref(pb), C.byref(a), C.c_void_p(4097), need, None) == 3
    a.q.ptr = None
    assert lib.fastmax_forward(C.byref(pb), C.byref(a), C.c_void_p(4096), need, None) == 1
    pb.nq = 0  # no queries and no state requested: nothing to validate, nothing to launch
    assert lib.fastmax_forward(C.byref(pb), C.byref(a), C.c_void_p(4096), need, None) == 0


def test_backward_rejects_bad_arguments():
    lib = _lib.load()
    pb = _lib.Problem(1, 2, 64, 64, 32, 2, 1, 0, 1, 1, 0.5, 1.0, 0, 0)
    b = _lib.BackwardArgs()
    assert lib.fastmax_backward(C.byref(pb), C.byref(b), None, 0, None) == 1  # nothing requested
    for t in (b.q, b.k, b.v, b.o, b.g, b.d_out, b.dq):
        t.ptr, t.stride_b, t.stride_h, t.stride_n = 4096, 4096, 2048, 32
    assert lib.fastmax_backward(C.byref(pb), C.byref(b), None, 0, None) == 1  # dq without dk, dv
    assert lib.fastmax_launch_count() == 0


def test_python_extension_module_is_importable_under_reference_name():
    import reproducing_fastmax_results_b200 as pkg

    ext = pkg.load_extension()
    import fastmax_cuda

    assert ext is fastmax_cuda
    assert hasattr(ext, "forwardpass") and hasattr(ext, "backwardpass")


def test_optional_steps_validate_before_launching():
    lib = _lib.load()
    t = _lib.Tensor(4096, 64 * 32, 32 * 64, 32)
    assert lib.fastmax_key_prologue(1, 2, 64, 48, 0, 1.0, C.byref(t), None, None) == 2      # head dim not supported
    assert lib.fastmax_key_prologue(1, 2, 64, 32, 9, 1.0, C.byref(t), None, None) == 1      # bad dtype
    assert lib.fastmax_key_prologue(1, 2, 64, 32, 0, 1.0, None, None, None) == 1            # no tensor
    assert lib.fastmax_key_prologue(1, 2, 0, 32, 0, 1.0, C.byref(t), None, None) == 0       # nothing to do
    bad = _lib.Tensor(4100, 64 * 32, 32 * 64, 32)
    assert lib.fastmax_key_prologue(1, 2, 64, 32, 0, 1.0, C.byref(bad), None, None) == 6    # misaligned base
    assert lib.fastmax_output_noise(1, 2, 64, 32, 0, 0.1, C.byref(t), None, C.byref(t), None) == 1
    assert lib.fastmax_output_noise(1, 2, 64, 16, 1, 0.1, C.byref(t), C.byref(bad), C.byref(t), None) == 6


def test_operators_follow_torch_deterministic_algorithms_setting():
    """Under torch.use_deterministic_algorithms(True) the operators say that their reductions are not run-to-run
    deterministic (PyTorch's convention: raise, or warn with warn_only=True) before anything is launched."""
    import torch

    from reproducing_fastmax_results_b200.attention import FASTMultiHeadAttention_Function, FastMax, _alert_not_deterministic

    q = torch.zeros(1, 1, 4, 16)
    was, warn_only = torch.are_deterministic_algorithms_enabled(), torch.is_deterministic_algorithms_warn_only_enabled()
    try:
        torch.use_deterministic_algorithms(True)
        with pytest.raises(RuntimeError, match="does not have a deterministic implementation"):
            FastMax.apply(q, q, q)
        with pytest.raises(RuntimeError, match="does not have a deterministic implementation"):
            FASTMultiHeadAttention_Function.apply(q, q, q, q, torch.zeros(7, 16))
        torch.use_deterministic_algorithms(True, warn_only=True)
        with pytest.warns(UserWarning, match="does not have a deterministic implementation"):
            _alert_not_deterministic("FastMax")
        torch.use_deterministic_algorithms(False)
        _alert_not_deterministic("FastMax")   # silent
    finally:
        torch.use_deterministic_algorithms(was, warn_only=warn_only)


def test_ctypes_structures_match_the_c_header(tmp_path):
    """The header compiles as plain C, and the ctypes mirrors in _lib.py have the sizes and field offsets the C
    compiler gives the structures (a field added on one side only would shift everything after it)."""
    import shutil
    import subprocess

    gcc = shutil.which("gcc")
    if gcc is None:
        pytest.skip("no C compiler")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    src = tmp_path / "abi.c"
    src.write_text(
        '#include <stdio.h>\n#include <stddef.h>\n#include "fastmax_b200.h"\n'
        "int main(void) {\n"
        '  printf("%zu %zu %zu %zu %zu ", sizeof(fastmax_tensor), sizeof(fastmax_problem), sizeof(fastmax_forward_args),\n'
        "         sizeof(fastmax_backward_args), sizeof(fastmax_decode_args));\n"
        '  printf("%zu %zu %zu %zu %zu %zu\\n", offsetof(fastmax_forward_args, state_in), offsetof(fastmax_forward_args, key_moments_out),\n'
        "         offsetof(fastmax_backward_args, dstate_out), offsetof(fastmax_backward_args, grad_moments_out),\n"
        "         offsetof(fastmax_problem, inv_temperature), offsetof(fastmax_decode_args, state));\n"
        "  return 0;\n}\n")
    exe = tmp_path / "abi"
    subprocess.run([gcc, "-std=c99", "-Wall", "-Werror", "-I", os.path.join(root, "include"), str(src), "-o", str(exe)], check=True)
    got = [int(x) for x in subprocess.run([str(exe)], check=True, capture_output=True, text=True).stdout.split()]
    want = [C.sizeof(_lib.Tensor), C.sizeof(_lib.Problem), C.sizeof(_lib.ForwardArgs), C.sizeof(_lib.BackwardArgs),
            C.sizeof(_lib.DecodeArgs), _lib.ForwardArgs.state_in.offset, _lib.ForwardArgs.key_moments_out.offset,
            _lib.BackwardArgs.dstate_out.offset, _lib.BackwardArgs.grad_moments_out.offset,
            _lib.Problem.inv_temperature.offset, _lib.DecodeArgs.state.offset]
    assert got == want
