"""In-tree build of the native parts for sm_100a.

  libfbw_b200.so        CUDA kernels + the C ABI of include/fbw_b200.h (nvcc, no torch)
  fbw/_build/fbw_core.so  torch extension `fbw_core` over that ABI (same module name and members
                        as the reference's, i6_native_ops/fbw/__init__.py:15, fbw_torch.cpp:31-40)
  fast_viterbi/_build/fast_viterbi_core.so  torch extension `fast_viterbi_core` over the same ABI
                        (i6_native_ops/fast_viterbi/__init__.py:15, binding.cpp:27-29)

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
VIT_DIR = os.path.join(PKG, "fast_viterbi", "_build")
VIT_EXT = os.path.join(VIT_DIR, "fast_viterbi_core.so")

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
    csrc = os.path.join(PKG, "csrc")
    # the .inc files are included by fbw_b200.cu; host_fill.cpp is the library's one host-only source
    host_src = os.path.join(csrc, "host_fill.cpp")
    deps = [os.path.join(csrc, f) for f in os.listdir(csrc) if f.endswith((".cu", ".inc"))]
    deps += [host_src, os.path.join(csrc, "host_fill.h")]
    hdr = os.path.join(INCLUDE, "fbw_b200.h")
    if not force and _newer(LIB, deps + [hdr]):
        return LIB
    nvcc = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")
    cmd = [nvcc, *NVCC_FLAGS, "-Xcompiler", "-pthread", "-I", INCLUDE, "-o", LIB, src, host_src]
    if verbose:
        cmd.insert(1, "-Xptxas=-v")
        print(" ".join(cmd))
    subprocess.run(cmd, check=True)
    return LIB


def _build_torch_ext(name: str, source: str, out_dir: str, target: str, force: bool, verbose: bool) -> str:
    src = os.path.join(PKG, "csrc", source)
    deps = [src, os.path.join(PKG, "csrc", "torch_common.h"), os.path.join(INCLUDE, "fbw_b200.h")]
    build_lib(force, verbose)  # the extension links against the library: bring it up to date first
    if not force and _newer(target, deps):
        return target
    os.makedirs(out_dir, exist_ok=True)
    os.environ.setdefault("TORCH_CUDA_ARCH_LIST", "10.0a")
    import ctypes

    from torch.utils.cpp_extension import load

    # the extension is linked against libfbw_b200.so by soname; have it loaded before torch
    # loads the freshly built module
    ctypes.CDLL(build_lib(), mode=ctypes.RTLD_GLOBAL)
    load(
        name=name,
        sources=[src],
        extra_include_paths=[INCLUDE, os.path.join(PKG, "csrc")],
        extra_ldflags=[f"-L{PKG}", "-lfbw_b200"],
        with_cuda=True,
        build_directory=out_dir,
        is_python_module=False,
        verbose=verbose,
    )
    return target


def build_ext(force: bool = False, verbose: bool = False) -> str:
    return _build_torch_ext("fbw_core", "fbw_torch.cpp", EXT_DIR, EXT, force, verbose)


def build_viterbi_ext(force: bool = False, verbose: bool = False) -> str:
    return _build_torch_ext("fast_viterbi_core", "viterbi_torch.cpp", VIT_DIR, VIT_EXT, force, verbose)


def build_all(force: bool = False, verbose: bool = False):
    return build_lib(force, verbose), build_ext(force, verbose), build_viterbi_ext(force, verbose)


if __name__ == "__main__":
    print(build_all("--force" in sys.argv, "--verbose" in sys.argv))
