"""In-tree build of the native parts for sm_100a.

  libfbw_b200.so        CUDA kernels + the C ABI of include/fbw_b200.h (nvcc, no torch)
  fbw/_build/fbw_core.so  torch extension `fbw_core` over that ABI (same module name and members
                        as the reference's, i6_native_ops/fbw/__init__.py:15, fbw_torch.cpp:31-40)

Both land inside the package directory so they travel with a source snapshot.
Usage:  python -m i6_native_ops_b200.build [--force] [--verbose]
"""
from __future__ import annotations

import os
import subprocess
import sys

PKG = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG)
INCLUDE = os.path.join(ROOT, "include")
LIB = os.path.join(PKG, "libfbw_b200.so")
EXT_DIR = os.path.join(PKG, "fbw", "_build")
EXT = os.path.join(EXT_DIR, "fbw_core.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-shared", "-Xcompiler", "-fPIC", "-Xlinker", "-soname=libfbw_b200.so",
]


def _newer(target: str, sources) -> bool:
    if not os.path.isfile(target):
        return False
    t = os.path.getmtime(target)
    return all(os.path.getmtime(s) <= t for s in sources)


def build_lib(force: bool = False, verbose: bool = False) -> str:
    src = os.path.join(PKG, "csrc", "fbw_b200.cu")
    hdr = os.path.join(INCLUDE, "fbw_b200.h")
    if not force and _newer(LIB, [src, hdr]):
        return LIB
    nvcc = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")
    cmd = [nvcc, *NVCC_FLAGS, "-I", INCLUDE, "-o", LIB, src]
    if verbose:
        cmd.insert(1, "-Xptxas=-v")
        print(" ".join(cmd))
    subprocess.run(cmd, check=True)
    return LIB


def build_ext(force: bool = False, verbose: bool = False) -> str:
    src = os.path.join(PKG, "csrc", "fbw_torch.cpp")
    hdr = os.path.join(INCLUDE, "fbw_b200.h")
    if not force and _newer(EXT, [src, hdr]):
        return EXT
    os.makedirs(EXT_DIR, exist_ok=True)
    os.environ.setdefault("TORCH_CUDA_ARCH_LIST", "10.0a")
    import ctypes

    from torch.utils.cpp_extension import load

    # the extension is linked against libfbw_b200.so by soname; have it loaded before torch
    # loads the freshly built module
    ctypes.CDLL(build_lib(), mode=ctypes.RTLD_GLOBAL)
    load(
        name="fbw_core",
        sources=[src],
        extra_include_paths=[INCLUDE],
        extra_ldflags=[f"-L{PKG}", "-lfbw_b200"],
        with_cuda=True,
        build_directory=EXT_DIR,
        is_python_module=False,
        verbose=verbose,
    )
    return EXT


def build_all(force: bool = False, verbose: bool = False):
    return build_lib(force, verbose), build_ext(force, verbose)


if __name__ == "__main__":
    print(build_all("--force" in sys.argv, "--verbose" in sys.argv))
