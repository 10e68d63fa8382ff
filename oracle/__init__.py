"""TEST INFRASTRUCTURE ONLY -- CPU oracle for the fbw path and the Viterbi alignment.

Python face of ``oracle/fbw_oracle.c`` (a C restatement of the reference's
i6_native_ops/fbw/fbw_op.cu:226-393) and ``oracle/viterbi_oracle.c`` (the same for
i6_native_ops/fast_viterbi/core.cu:174-275) plus brute-force path enumerators for tiny
automata.  Only tests, the smoke check and the benchmark's CPU-baseline leg may import
this package; the shipped package never does.
"""
from __future__ import annotations

import ctypes
import os
import subprocess
from typing import Optional, Tuple

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "_build", "libfbw_oracle.so")
_VIT_PATH = os.path.join(_HERE, "_build", "libviterbi_oracle.so")
_SOURCES = ("fbw_oracle.c", "fbw_oracle_impl.inc", "viterbi_oracle.c", "Makefile")
_lib = None
_vit = None


def build(force: bool = False) -> str:
    """Compile the C oracle with the Makefile beside this file; returns the library path."""
    src_time = max(os.path.getmtime(os.path.join(_HERE, f)) for f in _SOURCES)
    stale = any(not os.path.isfile(p) or os.path.getmtime(p) < src_time for p in (_LIB_PATH, _VIT_PATH))
    if force or stale:
        subprocess.run(["make", "-B", "-C", _HERE, "all"], check=True, capture_output=True)
    return _LIB_PATH


def _load():
    global _lib
    if _lib is None:
        build()
        _lib = ctypes.CDLL(_LIB_PATH)
        i64, p = ctypes.c_int64, ctypes.c_void_p
        for name in ("fbw_oracle_f32", "fbw_oracle_f64"):
            fn = getattr(_lib, name)
            fn.restype = ctypes.c_int
            fn.argtypes = [p, i64, i64, i64, p, i64, p, p, p, i64, p, p, p, p, ctypes.c_int]
    return _lib


def fbw_oracle(
    am: np.ndarray,
    edges: np.ndarray,
    weights: np.ndarray,
    start_end: np.ndarray,
    seq_lens: np.ndarray,
    num_states: int,
    dtype: str = "f32",
    nthreads: Optional[int] = None,
    want_states: bool = False,
):
    """Run the oracle.  Returns (out (T,B,F), sums (T,B)) and, if ``want_states``, also
    (alpha, beta) of shape (T+1, S).  ``dtype`` 'f32' computes in the reference's fp32
    operation order, 'f64' in double precision."""
    lib = _load()
    am = np.ascontiguousarray(am, dtype=np.float32)
    edges = np.ascontiguousarray(edges, dtype=np.int32)
    weights = np.ascontiguousarray(weights, dtype=np.float32)
    start_end = np.ascontiguousarray(start_end, dtype=np.int32)
    seq_lens = np.ascontiguousarray(seq_lens, dtype=np.int32)
    T, B, F = am.shape
    assert edges.ndim == 2 and edges.shape[0] == 4
    E = edges.shape[1]
    assert weights.shape == (E,) and start_end.shape == (2, B) and seq_lens.shape == (B,)
    real = np.float32 if dtype == "f32" else np.float64
    out = np.empty((T, B, F), dtype=real)
    sums = np.empty((T, B), dtype=real)
    alpha = beta = None
    if want_states:
        alpha = np.empty((T + 1, num_states), dtype=real)
        beta = np.empty((T + 1, num_states), dtype=real)
    ptr = lambda a: a.ctypes.data_as(ctypes.c_void_p) if a is not None else None
    fn = lib.fbw_oracle_f32 if dtype == "f32" else lib.fbw_oracle_f64
    rc = fn(ptr(am), T, B, F, ptr(edges), E, ptr(weights), ptr(start_end), ptr(seq_lens),
            int(num_states), ptr(out), ptr(sums), ptr(alpha), ptr(beta),
            int(nthreads or os.cpu_count() or 1))
    if rc != 0:
        raise ValueError(f"fbw oracle rejected the input (code {rc})")
    if want_states:
        return out, sums, alpha, beta
    return out, sums


def brute_force(am: np.ndarray, edges: np.ndarray, weights: np.ndarray, start_end: np.ndarray,
                seq_lens: np.ndarray) -> Tuple[np.ndarray, np.ndarray]:
    """Enumerate every path of every sequence (tiny inputs only) in float64.

    A path for sequence b starts in start_end[0,b], takes exactly seq_lens[b] edges, one
    per frame, and must end in start_end[1,b]; its score is the sum of edge weights and of
    am[t,b,emission] along the way (the automaton semantics of fbw_op.cu:71-102 and 61-69).
    Returns (posterior (T,B,F) in the probability domain, nll (B,))."""
    T, B, F = am.shape
    E = edges.shape[1]
    post = np.zeros((T, B, F), dtype=np.float64)
    nll = np.full((B,), np.inf)
    for b in range(B):
        eb = [e for e in range(E) if edges[3, e] == b]
        n = int(seq_lens[b])
        if n < 1 or n > T:
            continue
        paths = []  # (score, [emissions])

        def walk(state, t, score, emis):
            if t == n:
                if state == start_end[1, b]:
                    paths.append((score, list(emis)))
                return
            for e in eb:
                if edges[0, e] == state:
                    emis.append(int(edges[2, e]))
                    walk(int(edges[1, e]), t + 1,
                         score + float(weights[e]) + float(am[t, b, edges[2, e]]), emis)
                    emis.pop()

        walk(int(start_end[0, b]), 0, 0.0, [])
        if not paths:
            continue
        scores = np.array([p[0] for p in paths])
        m = scores.min()
        total = m - np.log(np.exp(-(scores - m)).sum())
        nll[b] = total
        for sc, em in paths:
            p = np.exp(-(sc - total))
            for t, f in enumerate(em):
                post[t, b, f] += p
    return post, nll


def viterbi_oracle(am: np.ndarray, edges: np.ndarray, weights: np.ndarray, start_end: np.ndarray,
                   seq_lens: np.ndarray, num_states: int) -> Tuple[np.ndarray, np.ndarray]:
    """Best path per sequence.  ``am`` (T,B,F) holds POSITIVE log scores.  Returns
    (alignment (T,B) int32, scores (B,) float32) -- the two tensors of
    i6_native_ops/fast_viterbi/core.cu:274."""
    global _vit
    if _vit is None:
        build()
        _vit = ctypes.CDLL(_VIT_PATH)
        i64, p = ctypes.c_int64, ctypes.c_void_p
        _vit.viterbi_oracle_f32.restype = ctypes.c_int
        _vit.viterbi_oracle_f32.argtypes = [p, i64, i64, i64, p, i64, p, p, p, i64, p, p]
    am = np.ascontiguousarray(am, dtype=np.float32)
    edges = np.ascontiguousarray(edges, dtype=np.int32)
    weights = np.ascontiguousarray(weights, dtype=np.float32)
    start_end = np.ascontiguousarray(start_end, dtype=np.int32)
    seq_lens = np.ascontiguousarray(seq_lens, dtype=np.int32)
    T, B, F = am.shape
    E = edges.shape[1]
    assert edges.shape[0] == 4 and weights.shape == (E,) and start_end.shape == (2, B)
    alignment = np.zeros((T, B), dtype=np.int32)
    scores = np.zeros((B,), dtype=np.float32)
    ptr = lambda a: a.ctypes.data_as(ctypes.c_void_p)
    rc = _vit.viterbi_oracle_f32(ptr(am), T, B, F, ptr(edges), E, ptr(weights), ptr(start_end),
                                 ptr(seq_lens), int(num_states), ptr(alignment), ptr(scores))
    if rc != 0:
        raise ValueError(f"viterbi oracle rejected the input (code {rc})")
    return alignment, scores


def brute_force_best(am: np.ndarray, edges: np.ndarray, weights: np.ndarray, start_end: np.ndarray,
                     seq_lens: np.ndarray) -> np.ndarray:
    """Score of the best complete path of every sequence by enumeration (tiny inputs only),
    float64; -inf where no path exists.  Same path semantics as ``brute_force``, scores maximised."""
    T, B, F = am.shape
    E = edges.shape[1]
    best = np.full((B,), -np.inf)
    for b in range(B):
        eb = [e for e in range(E) if edges[3, e] == b]
        n = int(seq_lens[b])
        if n < 0 or n > T:
            continue

        def walk(state, t, score):
            if t == n:
                if state == start_end[1, b] and score > best[b]:
                    best[b] = score
                return
            for e in eb:
                if edges[0, e] == state:
                    walk(int(edges[1, e]), t + 1, score + float(weights[e]) + float(am[t, b, edges[2, e]]))

        walk(int(start_end[0, b]), 0, 0.0)
    return best
