"""Builds libvetr.so (the CUDA kernels + C ABI) in-tree with nvcc for sm_100a.

nvcc cross-compiles without a GPU.  The arithmetic that the bit-exact fragment order depends on is written with
non-contracting intrinsics (see csrc/vetr_math.cuh); -fmad=false additionally keeps the per-fragment gradient
arithmetic in the same rounding order as the CPU oracle, so that parity tests only have to allow for the order in
which fp32 atomics sum.
"""
from __future__ import annotations

import os
import subprocess
import sys

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libvetr.so")
SOURCES = [os.path.join(_HERE, "csrc", "vetr_kernels.cu")]
HEADERS = [os.path.join(_HERE, "csrc", "vetr_math.cuh"), os.path.join(_HERE, "csrc", "vetr_envmap.cuh"), os.path.join(_HERE, "csrc", "vetr_knn.cuh"), os.path.join(_HERE, "csrc", "vetr_points.cuh"), os.path.join(_HERE, "..", "include", "vetr.h")]
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-fmad=false",
         "-Xcompiler", "-fPIC", "-shared", "-ccbin", "/usr/bin/g++"]


def needs_build() -> bool:
    if not os.path.exists(LIB_PATH):
        return True
    t = os.path.getmtime(LIB_PATH)
    return any(os.path.getmtime(p) > t for p in SOURCES + HEADERS)


def build(force: bool = False, verbose: bool = False, defines=(), out: str = LIB_PATH) -> str:
    """`defines` (e.g. ["VETR_ITEM_THREADS=256"]) and `out` build tuning variants next to the default library."""
    if force or out != LIB_PATH or needs_build():
        cmd = [NVCC] + FLAGS + [f"-D{d}" for d in defines] + (["-Xptxas", "-v"] if verbose else []) + ["-o", out] + SOURCES
        subprocess.check_call(cmd)
    return out


SHIM_PATH = os.path.join(_HERE, "libvetr_torch.so")
SHIM_SOURCES = [os.path.join(_HERE, "torch_shim", "vetr_torch.cpp")]
SHIM_HEADERS = [os.path.join(_HERE, "torch_shim", "vetr_torch.h"), os.path.join(_HERE, "..", "include", "vetr.h")]


def build_torch_shim(force: bool = False) -> str:
    """Builds libvetr_torch.so: the C++/libtorch operator surface (host code only, g++) on top of libvetr.so."""
    import torch
    from torch.utils import cpp_extension as ce

    build()
    if not force and os.path.exists(SHIM_PATH):
        t = os.path.getmtime(SHIM_PATH)
        if all(os.path.getmtime(p) <= t for p in SHIM_SOURCES + SHIM_HEADERS + [LIB_PATH]):
            return SHIM_PATH
    torch_lib = os.path.join(os.path.dirname(torch.__file__), "lib")
    cmd = ["/usr/bin/g++", "-O2", "-std=c++17", "-fPIC", "-shared", "-D_GLIBCXX_USE_CXX11_ABI=" + str(int(torch._C._GLIBCXX_USE_CXX11_ABI))]
    for inc in ce.include_paths("cuda"):
        cmd += ["-isystem", inc]
    cmd += SHIM_SOURCES + ["-o", SHIM_PATH, "-L" + _HERE, "-lvetr", "-L" + torch_lib, "-ltorch", "-ltorch_cpu", "-lc10",
                           "-ltorch_cuda", "-lc10_cuda", "-Wl,-rpath,$ORIGIN", "-Wl,-rpath," + torch_lib]
    subprocess.check_call(cmd)
    return SHIM_PATH


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
    if "--shim" in sys.argv:
        print(build_torch_shim(force="--force" in sys.argv))
