"""CPU tests of the Viterbi oracle (oracle/viterbi_oracle.c): the reference's own test case
(test/fast_viterbi.py:9-42, in the documented (B,T,F) layout), brute-force enumeration on tiny
automata, the tie rule of core.cu:37-40, the edge cases of the back-trace (core.cu:144-172) and the
golden fixtures produced by the reference op."""
import glob
import os

import numpy as np
import pytest

import oracle

GOLDEN = os.path.join(os.path.dirname(__file__), "golden")


def unit_case():
    probs = np.array([[0.9, 0.1], [0.9, 0.1], [0.4, 0.6], [0.1, 0.9], [0.1, 0.9]], dtype=np.float32)
    return dict(am=np.log(probs)[:, None, :],
                edges=np.array([[0, 0, 0, 0], [0, 1, 0, 0], [1, 1, 1, 0]], dtype=np.int32).T.copy(),
                weights=np.ones(3, dtype=np.float32), start_end=np.array([[0], [1]], dtype=np.int32),
                seq_lens=np.array([5], dtype=np.int32), num_states=2)


def run(c):
    return oracle.viterbi_oracle(c["am"], c["edges"], c["weights"], c["start_end"], c["seq_lens"],
                                 int(c["num_states"]))


def path_score(c, b, alignment):
    """Best score over all state paths that emit exactly `alignment[:, b]` (float64)."""
    E = c["edges"].shape[1]
    n = int(c["seq_lens"][b])
    cur = {int(c["start_end"][0, b]): 0.0}
    for t in range(n):
        nxt = {}
        for e in range(E):
            fr, to, em, sq = (int(x) for x in c["edges"][:, e])
            if sq == b and fr in cur and em == int(alignment[t, b]):
                v = cur[fr] + float(c["weights"][e]) + float(c["am"][t, b, em])
                if to not in nxt or v > nxt[to]:
                    nxt[to] = v
        cur = nxt
    return cur.get(int(c["start_end"][1, b]), -np.inf)


def test_reference_unit_case():
    alignment, scores = run(unit_case())
    assert alignment[:, 0].tolist() == [0, 0, 1, 1, 1]
    assert np.isclose(scores[0], 5.0 + np.log(0.9 * 0.9 * 0.6 * 0.9 * 0.9), rtol=1e-6)


def random_case(seed, B=3, T=6, F=5, S_per=4, E_per=9):
    rng = np.random.default_rng(seed)
    edges, weights = [], []
    for b in range(B):
        for _ in range(E_per):
            edges.append([b * S_per + rng.integers(S_per), b * S_per + rng.integers(S_per), rng.integers(F), b])
            weights.append(rng.normal())
    am = rng.normal(size=(T, B, F)).astype(np.float32)
    return dict(am=am, edges=np.array(edges, dtype=np.int32).T.copy(),
                weights=np.array(weights, dtype=np.float32),
                start_end=np.array([[b * S_per for b in range(B)], [b * S_per + S_per - 1 for b in range(B)]],
                                   dtype=np.int32),
                seq_lens=rng.integers(0, T + 1, size=B).astype(np.int32), num_states=B * S_per)


@pytest.mark.parametrize("seed", range(8))
def test_against_enumeration(seed):
    c = random_case(seed)
    alignment, scores = run(c)
    best = oracle.brute_force_best(c["am"], c["edges"], c["weights"], c["start_end"], c["seq_lens"])
    for b in range(len(best)):
        if np.isinf(best[b]):
            assert scores[b] == -np.inf
            continue
        assert np.isclose(scores[b], best[b], rtol=1e-5, atol=1e-5)
        # the alignment spells a path that reaches the best score
        assert np.isclose(path_score(c, b, alignment), best[b], rtol=1e-5, atol=1e-5)
        assert (alignment[int(c["seq_lens"][b]):, b] == 0).all()


def test_tie_takes_smaller_edge_index():
    # two parallel edges with equal value into the end state: edge 1 (emission 3) precedes edge 2 (emission 1)
    am = np.zeros((1, 1, 4), dtype=np.float32)
    edges = np.array([[0, 0, 2, 0], [0, 1, 3, 0], [0, 1, 1, 0]], dtype=np.int32).T.copy()
    c = dict(am=am, edges=edges, weights=np.zeros(3, np.float32), start_end=np.array([[0], [1]], np.int32),
             seq_lens=np.array([1], np.int32), num_states=2)
    alignment, scores = run(c)
    assert alignment[0, 0] == 3 and scores[0] == 0.0
    c["edges"] = edges[:, [0, 2, 1]].copy()
    alignment, _ = run(c)
    assert alignment[0, 0] == 1


def test_no_path_and_empty_sequences():
    c = unit_case()
    c["seq_lens"] = np.array([0], np.int32)  # no frames: the end state differs from the start state
    alignment, scores = run(c)
    assert scores[0] == -np.inf and (alignment == 0).all()
    c["seq_lens"] = np.array([9], np.int32)  # longer than T: treated as empty
    alignment, scores = run(c)
    assert scores[0] == -np.inf and (alignment == 0).all()
    # end state unreachable: the score is -inf, and the back-trace stays in the end state
    c = unit_case()
    c["edges"] = c["edges"][:, [0, 2]].copy()
    c["weights"] = c["weights"][:2]
    alignment, scores = run(c)
    assert scores[0] == -np.inf and (alignment == 0).all()


@pytest.mark.parametrize("path", sorted(glob.glob(os.path.join(GOLDEN, "viterbi_*.npz"))))
def test_golden(path):
    """Bit-exact against what the reference op returned on a B200."""
    g = np.load(path)
    c = np.load(os.path.join(GOLDEN, os.path.basename(path)[len("viterbi_"):]))
    alignment, scores = oracle.viterbi_oracle(-c["am"], c["edges"], c["weights"], c["start_end"], c["seq_lens"],
                                              int(c["num_states"]))
    assert np.array_equal(alignment, g["ref_alignment"])
    assert np.array_equal(scores, g["ref_scores"])
