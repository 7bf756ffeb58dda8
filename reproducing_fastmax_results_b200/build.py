"""Builds the native code of this package in-tree for sm_100a.

  libfastmax_b200.so                       C-ABI library (include/fastmax_b200.h): CUDA kernels + launch logic
  fastmax_cuda.cpython-*.so                PyTorch extension with the reference's `fastmax_cuda` interface

Usage:  python -m reproducing_fastmax_results_b200.build [--force] [--no-ext]
Objects go to build/ at the repository root; nothing is installed outside the tree.
"""
from __future__ import annotations

import concurrent.futures
import hashlib
import os
import subprocess
import sys
import sysconfig

PKG = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG)
CSRC = os.path.join(PKG, "csrc")
OBJ = os.path.join(ROOT, "build", "obj")
LIB = os.path.join(PKG, "libfastmax_b200.so")
EXT = os.path.join(PKG, "fastmax_cuda" + (sysconfig.get_config_var("EXT_SUFFIX") or ".so"))

NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-lineinfo", "-std=c++17",
    "-Xcompiler", "-fPIC", "-Xptxas", "-v",
]
CU_SOURCES = ["fastmax_abi.cu", "scan_d16.cu", "scan_d32.cu", "scan_d64.cu", "tc_kernels.cu", "noalloc.cu", "decode.cu"]


def _digest(paths):
    h = hashlib.sha256()
    for p in sorted(paths):
        with open(p, "rb") as f:
            h.update(p.encode())
            h.update(f.read())
    return h.hexdigest()


def _headers():
    out = [os.path.join(ROOT, "include", "fastmax_b200.h")]
    for n in os.listdir(CSRC):
        if n.endswith((".cuh", ".h")):
            out.append(os.path.join(CSRC, n))
    return out


def _run(cmd, log):
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    with open(log, "w") as f:
        f.write(" ".join(cmd) + "\n" + r.stdout)
    if r.returncode != 0:
        raise RuntimeError("build step failed: %s\n%s" % (" ".join(cmd), r.stdout[-4000:]))
    return r.stdout


def _compile_cu(src, force):
    os.makedirs(OBJ, exist_ok=True)
    path = os.path.join(CSRC, src)
    obj = os.path.join(OBJ, src + ".o")
    stamp = obj + ".sha"
    dig = _digest([path] + _headers()) + " ".join(NVCC_FLAGS)
    if not force and os.path.exists(obj) and os.path.exists(stamp) and open(stamp).read() == dig:
        return obj, False
    _run([NVCC] + NVCC_FLAGS + ["-c", path, "-o", obj], obj + ".log")
    with open(stamp, "w") as f:
        f.write(dig)
    return obj, True


def build_library(force=False):
    srcs = [s for s in CU_SOURCES if os.path.exists(os.path.join(CSRC, s))]
    with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, len(srcs))) as ex:
        res = list(ex.map(lambda s: _compile_cu(s, force), srcs))
    objs = [o for o, _ in res]
    if force or any(ch for _, ch in res) or not os.path.exists(LIB):
        _run([NVCC, "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", LIB] + objs, os.path.join(OBJ, "link.log"))
    return LIB


def build_extension(force=False):
    import torch
    from torch.utils import cpp_extension as ce

    src = os.path.join(CSRC, "fastmax_cuda_ext.cpp")
    stamp = os.path.join(OBJ, "ext.sha")
    dig = _digest([src, os.path.join(ROOT, "include", "fastmax_b200.h")]) + torch.__version__
    if not force and os.path.exists(EXT) and os.path.exists(stamp) and open(stamp).read() == dig:
        return EXT
    os.makedirs(OBJ, exist_ok=True)
    inc = []
    for p in ce.include_paths("cuda") + [sysconfig.get_paths()["include"]]:
        inc += ["-isystem", p]
    libdirs = ce.library_paths("cuda")
    cmd = ["g++", "-O2", "-std=c++17", "-fPIC", "-shared", "-DTORCH_EXTENSION_NAME=fastmax_cuda",
           "-DTORCH_API_INCLUDE_EXTENSION_H", "-D_GLIBCXX_USE_CXX11_ABI=%d" % int(torch._C._GLIBCXX_USE_CXX11_ABI),
           src, "-o", EXT] + inc
    for d in libdirs:
        cmd += ["-L" + d, "-Wl,-rpath," + d]
    cmd += ["-L" + PKG, "-lfastmax_b200", "-Wl,-rpath,$ORIGIN", "-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda",
            "-ltorch", "-ltorch_python"]
    _run(cmd, os.path.join(OBJ, "ext.log"))
    with open(stamp, "w") as f:
        f.write(dig)
    return EXT


def build_all(force=False, ext=True):
    lib = build_library(force)
    out = [lib]
    if ext:
        out.append(build_extension(force))
    return out


if __name__ == "__main__":
    force = "--force" in sys.argv
    for p in build_all(force, ext="--no-ext" not in sys.argv):
        print("built", p)
