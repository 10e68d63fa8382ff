"""CPU checks of the drop-in boundary: the C-ABI library loads and exports every function the
public header declares, the status strings exist, and the Python surface mirrors the reference
package (i6_native_ops/fbw/__init__.py:27-68, fbw_torch.cpp:31-40).  No kernel is launched."""
import ctypes
import inspect
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "fbw_b200.h")
LIB = os.path.join(ROOT, "i6_native_ops_b200", "libfbw_b200.so")


def declared_functions():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(fbw_b200_[a-z_0-9]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    from i6_native_ops_b200 import build

    build.build_lib()
    lib = ctypes.CDLL(LIB)
    names = declared_functions()
    assert {"fbw_b200_prepare", "fbw_b200_run", "fbw_b200_plan_bytes", "fbw_b200_run_bytes",
            "fbw_b200_plan_summary", "fbw_b200_status_string", "fbw_b200_abi_version"} <= set(names)
    for n in names:
        assert hasattr(lib, n), f"{n} declared in include/fbw_b200.h but not exported"
    lib.fbw_b200_status_string.restype = ctypes.c_char_p
    assert lib.fbw_b200_status_string(0) == b"ok"
    for code in range(1, 6):
        assert lib.fbw_b200_status_string(code) not in (b"ok", b"unknown status")
    assert lib.fbw_b200_abi_version() >= 1


def test_argument_checks_without_a_device():
    """Bad arguments are rejected before any CUDA call."""
    lib = ctypes.CDLL(LIB)
    lib.fbw_b200_prepare.restype = ctypes.c_int
    i64 = ctypes.c_int64
    rc = lib.fbw_b200_prepare(None, None, None, None, i64(0), i64(1), i64(1), i64(0), i64(1), None,
                              ctypes.c_size_t(0), None)
    assert rc == 1
    lib.fbw_b200_run.restype = ctypes.c_int
    assert lib.fbw_b200_run(None, None, None, None, None, None, None, ctypes.c_size_t(0), None) == 1


def test_python_surface_mirrors_reference():
    import i6_native_ops_b200.fbw as m

    assert hasattr(m.core, "fbw") and hasattr(m.core, "DebugOptions")
    d = m.core.DebugOptions()
    assert (d.dump_alignment, d.dump_output, d.dump_every, d.pruning) == (False, False, 40, 10.0)
    assert list(inspect.signature(m.fbw_loss).parameters) == ["log_probs", "fsa", "seq_lens"]
    assert issubclass(m.FastBaumWelchLoss, __import__("torch").autograd.Function)


def test_reference_import_paths_resolve():
    """The shim package serves the reference's import paths (no kernel is launched)."""
    import i6_native_ops_b200.compat as compat

    compat.install()
    import i6_native_ops.fast_viterbi as v
    import i6_native_ops.fbw as f
    import i6_native_ops_b200.fast_viterbi as nv
    import i6_native_ops_b200.fbw as nf

    assert f.fbw_loss is nf.fbw_loss and f.FastBaumWelchLoss is nf.FastBaumWelchLoss and f.core is nf.core
    assert v.align_viterbi is nv.align_viterbi and v.core is nv.core
