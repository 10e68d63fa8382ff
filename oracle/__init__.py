"""TEST INFRASTRUCTURE ONLY -- CPU oracle for the fbw path.

Python face of ``oracle/fbw_oracle.c`` (a C restatement of the reference's
i6_native_ops/fbw/fbw_op.cu:226-393) plus a brute-force path enumerator for tiny
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
_lib = None


def build(force: bool = False) -> str:
    """Compile the C oracle with the Makefile beside this file; returns the library path."""
    src_time = max(
        os.path.getmtime(os.path.join(_HERE, f)) for f in ("fbw_oracle.c", "fbw_oracle_impl.inc", "Makefile")
    )
    if force or not os.path.isfile(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < src_time:
        subprocess.run(["make", "-B", "-C", _HERE], check=True, capture_output=True)
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
