"""CPU tests of the oracle (test infrastructure): the C restatement of the reference's fbw
arithmetic is checked against brute-force path enumeration, torch's CTC loss, the invariants
the reference's own test asserts (test/fbw.py:57-64) and the committed golden fixtures that
hold outputs of the reference op itself."""
import glob
import os

import numpy as np
import pytest
import torch

import oracle
from i6_native_ops_b200 import workloads as wl

GOLDEN = os.path.join(os.path.dirname(__file__), "golden")


def reference_unit_case():
    """The input of the reference's only fbw test (test/fbw.py:10-42)."""
    probs = np.array([[0.9, 0.1], [0.9, 0.1], [0.4, 0.6], [0.1, 0.9], [0.1, 0.9]], dtype=np.float32)
    am = -np.log(probs)[:, None, :]
    edges = np.array([[0, 0, 0, 0], [0, 1, 0, 0], [1, 1, 1, 0]], dtype=np.int32).T.copy()
    weights = np.ones(3, dtype=np.float32)
    start_end = np.array([[0], [1]], dtype=np.int32)
    seq_lens = np.array([5], dtype=np.int32)
    return am, edges, weights, start_end, seq_lens, 2


def random_small_fsa(rng, B=3, F=4, T=5, S_per=4, E_per=9):
    fr, to, em, sq, start, end = [], [], [], [], [], []
    for b in range(B):
        off = b * S_per
        for _ in range(E_per):
            fr.append(off + rng.integers(0, S_per))
            to.append(off + rng.integers(0, S_per))
            em.append(rng.integers(0, F))
            sq.append(b)
        start.append(off)
        end.append(off + S_per - 1)
    edges = np.array([fr, to, em, sq], dtype=np.int32)
    perm = rng.permutation(edges.shape[1])
    edges = np.ascontiguousarray(edges[:, perm])
    weights = rng.uniform(0, 2, size=edges.shape[1]).astype(np.float32)
    am = rng.uniform(0.1, 3, size=(T, B, F)).astype(np.float32)
    seq_lens = rng.integers(1, T + 1, size=B).astype(np.int32)
    return am, edges, weights, np.array([start, end], dtype=np.int32), seq_lens, B * S_per


def test_reference_unit_case_invariants():
    am, edges, w, se, sl, S = reference_unit_case()
    for dt, tol in (("f32", 1e-6), ("f64", 1e-12)):
        out, sums = oracle.fbw_oracle(am, edges, w, se, sl, S, dtype=dt)
        assert np.allclose(np.exp(-out).sum(-1), 1.0, atol=tol * 10)  # test/fbw.py:60-64
        assert np.allclose(sums, sums[0, 0], rtol=tol * 10)
    post, nll = oracle.brute_force(am, edges, w, se, sl)
    assert abs(nll[0] - sums[0, 0]) < 1e-12
    assert np.abs(post - np.exp(-out)).max() < 1e-12


@pytest.mark.parametrize("seed", range(6))
def test_oracle_vs_brute_force(seed):
    rng = np.random.default_rng(seed)
    am, edges, w, se, sl, S = random_small_fsa(rng)
    post, nll = oracle.brute_force(am, edges, w, se, sl)
    out, sums = oracle.fbw_oracle(am, edges, w, se, sl, S, dtype="f64")
    T, B, F = am.shape
    for b in range(B):
        n = int(sl[b])
        if np.isinf(nll[b]):  # no path: all frames empty
            assert np.all(sums[:, b] == 0) and np.all(np.isinf(out[:, b]))
            continue
        assert np.allclose(sums[:n, b], nll[b], rtol=1e-12)
        assert np.all(sums[n:, b] == 0)
        assert np.all(np.isinf(out[n:, b]))
        assert np.abs(np.exp(-out[:n, b]) - post[:n, b]).max() < 1e-12
    out32, sums32 = oracle.fbw_oracle(am, edges, w, se, sl, S, dtype="f32")
    assert np.abs(np.exp(-out32.astype(np.float64)) - np.exp(-out)).max() < 1e-5
    assert np.allclose(sums32, sums, rtol=1e-6, atol=0)


def test_oracle_vs_ctc_loss():
    b = wl.make_batch("ctc_tiny")
    am = wl.make_scores(b).numpy()
    out, sums = oracle.fbw_oracle(am, b.edges, b.weights, b.start_end, b.seq_lens, b.num_states, "f64")
    for i in range(b.B):
        rng = np.random.default_rng(i)
        L = int(rng.integers(5, 13))
        labels = rng.integers(1, b.F, size=L)
        n = int(b.seq_lens[i])
        lp = -torch.from_numpy(am[:n, i:i + 1, :]).double()
        ref = torch.nn.functional.ctc_loss(lp, torch.tensor(labels)[None], torch.tensor([n]),
                                           torch.tensor([L]), blank=0, reduction="sum")
        assert abs(float(ref) - sums[0, i]) < 1e-9
        assert np.allclose(np.exp(-out[:n, i]).sum(-1), 1.0, atol=1e-12)


@pytest.mark.parametrize("name,kw", [("monophone", dict(B=3, T=125, scale=0.25)),
                                     ("triphone", dict(B=2, T=150, F=501, scale=0.1)),
                                     ("bpe_ctc", dict(B=3, T=100, F=300, scale=0.25)),
                                     ("lattice", dict(B=3, F=50, T=200, scale=0.1))])
def test_oracle_f32_tracks_f64(name, kw):
    b = wl.make_batch(name, **kw)
    am = wl.make_scores(b).numpy()
    o64, s64 = oracle.fbw_oracle(am, b.edges, b.weights, b.start_end, b.seq_lens, b.num_states, "f64")
    o32, s32 = oracle.fbw_oracle(am, b.edges, b.weights, b.start_end, b.seq_lens, b.num_states, "f32")
    valid = s64 != 0
    assert valid.any()
    assert np.abs(s32[valid] - s64[valid]).max() / np.abs(s64[valid]).max() < 1e-5
    assert np.abs(np.exp(-o32.astype(np.float64)) - np.exp(-o64)).max() < 5e-3
    rows = np.exp(-o64).sum(-1)
    assert np.allclose(rows[valid], 1.0, atol=1e-9) and np.all(rows[~valid] == 0)


def test_oracle_rejects_bad_input():
    am, edges, w, se, sl, S = reference_unit_case()
    bad = edges.copy()
    bad[0, 0] = 7
    with pytest.raises(ValueError):
        oracle.fbw_oracle(am, bad, w, se, sl, S)


FBW_FIXTURES = sorted(p for p in glob.glob(os.path.join(GOLDEN, "*.npz"))
                      if not os.path.basename(p).startswith("viterbi_"))


@pytest.mark.parametrize("path", FBW_FIXTURES)
def test_oracle_matches_reference_golden(path):
    """Fixtures written by tests/golden/make_golden.py hold the outputs of the reference op
    itself (run on a GPU).  The fp32 oracle must agree within the libm-vs-libdevice rounding
    of the score magnitude; the fp64 oracle within the reference's own fp32 noise."""
    g = np.load(path)
    am, edges, w, se, sl = g["am"], g["edges"], g["weights"], g["start_end"], g["seq_lens"]
    S = int(g["num_states"])
    ref_out, ref_sums = g["ref_out"], g["ref_sums"]
    o32, s32 = oracle.fbw_oracle(am, edges, w, se, sl, S, "f32")
    o64, s64 = oracle.fbw_oracle(am, edges, w, se, sl, S, "f64")
    assert np.array_equal(ref_sums == 0, s32 == 0)
    assert np.array_equal(np.isinf(ref_out), np.isinf(o32))
    scale = max(1.0, float(np.abs(ref_sums).max()))
    tol_post = float(g["post_tol"]) if "post_tol" in g else max(1e-4, 4 * scale * 1.2e-7)
    assert np.abs(s32 - ref_sums).max() / scale < 1e-5
    assert np.abs(s64 - ref_sums).max() / scale < 1e-5
    p_ref = np.exp(-ref_out.astype(np.float64))
    assert np.abs(np.exp(-o32.astype(np.float64)) - p_ref).max() < tol_post
    assert np.abs(np.exp(-o64) - p_ref).max() < tol_post
