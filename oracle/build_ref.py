"""Build the UNMODIFIED reference fbw and fast_viterbi ops into oracle/_ref/ (test infrastructure only).

The reference's two fbw sources (i6_native_ops/fbw/fbw_torch.cpp and
i6_native_ops/fbw/fbw_op.cu) are compiled where they lie, read-only, as a torch
extension named ``fbw_core_ref`` for sm_100a.  Nothing is copied: only the built
shared object lands in ``oracle/_ref/``.  The op needs a CUDA device to run (it
rejects CPU tensors, fbw_torch.cpp:19-23), so the built module is only usable on
a GPU machine; there it serves as the bit-level parity target for the new kernels
and generates the golden fixtures under tests/golden/.

The reference's fast_viterbi op (i6_native_ops/fast_viterbi/binding.cpp and core.cu) is built the
same way as ``fast_viterbi_core_ref`` into ``oracle/_ref/viterbi/``.

Usage:  python oracle/build_ref.py [reference_root]
"""
import os
import sys


def default_reference_root() -> str:
    """Where the reference checkout lies: $I6_NATIVE_OPS_REFERENCE, else the default below."""
    return os.environ.get("I6_NATIVE_OPS_REFERENCE", "/root/reference")


def ref_dir() -> str:
    return os.path.join(os.path.dirname(os.path.abspath(__file__)), "_ref")


def built_path() -> str:
    return os.path.join(ref_dir(), "fbw_core_ref.so")


def build(reference_root: str = None, verbose: bool = False) -> str:
    """Compile the reference op; returns the path of the shared object."""
    reference_root = reference_root or default_reference_root()
    src = os.path.join(reference_root, "i6_native_ops", "fbw")
    if not os.path.isfile(os.path.join(src, "fbw_op.cu")):
        raise FileNotFoundError(f"reference sources not found under {reference_root}")
    os.makedirs(ref_dir(), exist_ok=True)
    os.environ.setdefault("TORCH_CUDA_ARCH_LIST", "10.0a")
    from torch.utils.cpp_extension import load

    load(
        name="fbw_core_ref",
        sources=[os.path.join(src, "fbw_torch.cpp"), os.path.join(src, "fbw_op.cu")],
        extra_include_paths=[src, os.path.join(reference_root, "i6_native_ops", "common")],
        build_directory=ref_dir(),
        verbose=verbose,
    )
    return built_path()


def viterbi_built_path() -> str:
    return os.path.join(ref_dir(), "viterbi", "fast_viterbi_core_ref.so")


def build_viterbi(reference_root: str = None, verbose: bool = False) -> str:
    """Compile the reference fast_viterbi op; returns the path of the shared object."""
    reference_root = reference_root or default_reference_root()
    src = os.path.join(reference_root, "i6_native_ops", "fast_viterbi")
    if not os.path.isfile(os.path.join(src, "core.cu")):
        raise FileNotFoundError(f"reference sources not found under {reference_root}")
    out = os.path.dirname(viterbi_built_path())
    os.makedirs(out, exist_ok=True)
    os.environ.setdefault("TORCH_CUDA_ARCH_LIST", "10.0a")
    from torch.utils.cpp_extension import load

    load(
        name="fast_viterbi_core_ref",
        sources=[os.path.join(src, "binding.cpp"), os.path.join(src, "core.cu")],
        extra_include_paths=[os.path.join(reference_root, "i6_native_ops", "common")],
        build_directory=out,
        verbose=verbose,
    )
    return viterbi_built_path()


def _load(name: str, path: str):
    if not os.path.isfile(path):
        return None
    import importlib.util

    import torch  # noqa: F401  (libtorch must be loaded first)

    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def load_ref():
    """Import the prebuilt reference fbw module (no compilation); None if it was never built."""
    return _load("fbw_core_ref", built_path())


def load_viterbi_ref():
    """Import the prebuilt reference fast_viterbi module; None if it was never built."""
    return _load("fast_viterbi_core_ref", viterbi_built_path())


if __name__ == "__main__":
    root = sys.argv[1] if len(sys.argv) > 1 else default_reference_root()
    print(build(root, verbose=True))
    print(build_viterbi(root, verbose=True))
