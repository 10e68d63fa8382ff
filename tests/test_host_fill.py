"""CPU tests of the library's host threads (csrc/host_fill.cpp): the rows of a sparse (T,B,F) result
written from the class posteriors, and the scores the automata refer to picked out of a score tensor.
The source is compiled here with g++ together with a small C shim (tests/host_fill_shim.cpp) and called
through ctypes; the expected arrays are built with numpy."""
import ctypes
import os
import subprocess
import tempfile

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CSRC = os.path.join(ROOT, "i6_native_ops_b200", "csrc")


@pytest.fixture(scope="module")
def shim():
    out = os.path.join(tempfile.mkdtemp(), "libhost_fill_shim.so")
    subprocess.run(["g++", "-O2", "-std=c++17", "-shared", "-fPIC", "-pthread", "-I", CSRC, "-o", out,
                    os.path.join(ROOT, "tests", "host_fill_shim.cpp"), os.path.join(CSRC, "host_fill.cpp")],
                   check=True)
    lib = ctypes.CDLL(out)
    i32, i64, pi, pl, pf = (ctypes.c_int, ctypes.c_longlong, ctypes.POINTER(ctypes.c_int),
                            ctypes.POINTER(ctypes.c_longlong), ctypes.POINTER(ctypes.c_float))
    lib.shim_compose.argtypes = [i64, i64, i64, pi, pi, pi, pl, pi, i64, pf, i64, pf, i32, i32, i32, i32]
    lib.shim_gather.argtypes = [i64, i64, i64, pi, pi, pi, pl, pi, i64, pf, i32, pf, i64, i32]
    lib.shim_row_chunk.argtypes = [i32, i64, i32, i32]
    return lib


def ptr(a, t):
    return a.ctypes.data_as(ctypes.POINTER(t))


def make_case(rng, T, B, F, max_slots):
    """A plan as the host sees it: lengths (one sequence invalid), ascending classes per sequence at
    arbitrary offsets of the class list, posterior rows padded to four."""
    seq_T = rng.integers(1, T + 1, size=B).astype(np.int32)
    seq_T[0] = T
    if B > 2:
        seq_T[2] = 0
    nslot = rng.integers(1, max_slots + 1, size=B).astype(np.int32)
    slot_off = np.zeros(B, np.int32)
    gf_off = np.zeros(B, np.int64)
    emis = []
    p_floats = 0
    for b in range(B):
        emis += [0] * int(rng.integers(0, 5))  # unused entries between the sequences' lists
        slot_off[b] = len(emis)
        emis += sorted(rng.choice(F, size=int(nslot[b]), replace=False).tolist())
        gf_off[b] = p_floats
        p_floats += T * ((int(nslot[b]) + 3) & ~3)
    return seq_T, nslot, slot_off, gf_off, np.asarray(emis, np.int32), p_floats


@pytest.mark.parametrize("T,B,F,chunk_steps", [(70, 5, 1201, 32), (33, 3, 17, 1 << 30), (130, 4, 4099, 64)])
def test_rows_written_from_posteriors(shim, T, B, F, chunk_steps):
    rng = np.random.default_rng(T * 131 + F)
    seq_T, nslot, slot_off, gf_off, emis, p_floats = make_case(rng, T, B, F, min(40, F))
    P = rng.standard_normal(p_floats).astype(np.float32)
    raw = np.full(T * B * F + 16, -1.0, np.float32)
    out = raw[3:3 + T * B * F]  # rows at odd 4-byte offsets
    first_chunk = 1 if chunk_steps < T else 0
    chunks = {-1}
    for b in range(B):
        for t in range(T):
            chunks.add(shim.shim_row_chunk(int(seq_T[b]), t, chunk_steps, first_chunk))
    for c in sorted(chunks):
        rc = shim.shim_compose(T, B, F, ptr(seq_T, ctypes.c_int), ptr(nslot, ctypes.c_int),
                               ptr(slot_off, ctypes.c_int), ptr(gf_off, ctypes.c_longlong),
                               ptr(emis, ctypes.c_int), len(emis), ptr(P, ctypes.c_float), p_floats,
                               ptr(out, ctypes.c_float), chunk_steps, first_chunk, c, 3)
        assert rc == 0
    want = np.full((T, B, F), np.inf, np.float32)
    for b in range(B):
        Dp = (int(nslot[b]) + 3) & ~3
        cls = emis[slot_off[b]:slot_off[b] + nslot[b]]
        for t in range(int(seq_T[b])):
            want[t, b, cls] = P[gf_off[b] + t * Dp:gf_off[b] + t * Dp + nslot[b]]
    assert np.array_equal(out.reshape(T, B, F), want)
    assert raw[2] == -1.0 and raw[3 + T * B * F] == -1.0  # nothing written outside the tensor


def test_row_chunks_follow_the_sweeps(shim):
    """A frame's posteriors exist after the chunk in which both sweeps have passed its 32-frame tile."""
    Te, J = 200, 64
    for t in range(Te):
        k = t // 32
        last = min(k * 32 + 31, Te - 1)
        want = max(last // J, (Te - 1 - k * 32) // J)
        assert shim.shim_row_chunk(Te, t, J, 0) == want
        assert shim.shim_row_chunk(Te, t, J, 3) == max(want, 3)
    assert shim.shim_row_chunk(Te, Te, J, 0) == -1 and shim.shim_row_chunk(0, 0, J, 0) == -1


@pytest.mark.parametrize("batch_major", [0, 1])
def test_scores_picked_out_of_the_tensor(shim, batch_major):
    rng = np.random.default_rng(7 + batch_major)
    T, B, F = 50, 6, 2003
    seq_T, nslot, slot_off, gf_off, emis, g_floats = make_case(rng, T, B, F, 60)
    am = rng.standard_normal((B, T, F) if batch_major else (T, B, F)).astype(np.float32)
    G = np.full(g_floats, np.nan, np.float32)
    rc = shim.shim_gather(T, B, F, ptr(seq_T, ctypes.c_int), ptr(nslot, ctypes.c_int), ptr(slot_off, ctypes.c_int),
                          ptr(gf_off, ctypes.c_longlong), ptr(emis, ctypes.c_int), len(emis),
                          ptr(am, ctypes.c_float), batch_major, ptr(G, ctypes.c_float), g_floats, 4)
    assert rc == 0
    for b in range(B):
        Dp = (int(nslot[b]) + 3) & ~3
        cls = emis[slot_off[b]:slot_off[b] + nslot[b]]
        for t in range(T):
            row = G[gf_off[b] + t * Dp:gf_off[b] + (t + 1) * Dp]
            if t < seq_T[b]:
                src = am[b, t] if batch_major else am[t, b]
                assert np.array_equal(row[:nslot[b]], src[cls]) and np.all(row[nslot[b]:] == 0)
            else:
                assert np.all(np.isnan(row))  # frames past the sequence's end are not touched


def test_indices_outside_the_arrays_are_refused(shim):
    rng = np.random.default_rng(3)
    T, B, F = 20, 3, 101
    seq_T, nslot, slot_off, gf_off, emis, p_floats = make_case(rng, T, B, F, 10)
    P = np.zeros(p_floats, np.float32)
    out = np.zeros(T * B * F, np.float32)
    bad = emis.copy()
    bad[slot_off[1]] = F + 5  # a class outside the row
    rc = shim.shim_compose(T, B, F, ptr(seq_T, ctypes.c_int), ptr(nslot, ctypes.c_int), ptr(slot_off, ctypes.c_int),
                           ptr(gf_off, ctypes.c_longlong), ptr(bad, ctypes.c_int), len(bad), ptr(P, ctypes.c_float),
                           p_floats, ptr(out, ctypes.c_float), 1 << 30, 0, 0, 2)
    assert rc == 1
    assert 1 <= shim.shim_threads() <= 64


def test_threads_are_shared_out_over_the_processes_of_a_node(shim):
    """LOCAL_WORLD_SIZE (exported by torchrun) divides the CPUs the process may use; FBW_B200_HOST_THREADS
    overrides.  Read per call, so the environment can be changed in place."""
    allowed = len(os.sched_getaffinity(0))
    saved = {k: os.environ.pop(k, None) for k in ("LOCAL_WORLD_SIZE", "FBW_B200_HOST_THREADS")}
    try:
        assert shim.shim_threads() == min(allowed, 16)
        os.environ["LOCAL_WORLD_SIZE"] = "4"
        assert shim.shim_threads() == min(max(allowed // 4, 2), 16)
        os.environ["FBW_B200_HOST_THREADS"] = "3"
        assert shim.shim_threads() == 3
    finally:
        for k, v in saved.items():
            os.environ.pop(k, None)
            if v is not None:
                os.environ[k] = v
