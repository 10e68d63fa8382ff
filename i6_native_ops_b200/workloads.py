"""Seeded synthetic fbw workloads: automata in the reference's tuple format plus score tensors.

The automaton format is the one the reference documents at i6_native_ops/fbw/__init__.py:52-63:
``(num_states, edges (4,E) int32 rows from/to/emission/sequence, weights (E,) float32,
start_end_states (2,B) int32)``, with state ids global across the batch and every edge
consuming exactly one frame (i6_native_ops/fbw/fbw_op.cu:71-102).

Every sequence draws from its own generator seeded ``seed0 + global sequence id``, so a
sequence's automaton, length and scores do not depend on how a batch is sharded over ranks.
Five named workloads mirror the benchmark configurations: ``ctc_tiny``, ``monophone``,
``triphone``, ``bpe_ctc`` and ``lattice``.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np


@dataclass
class FbwBatch:
    """One batch of automata (host side, numpy) and the recipe for its scores."""

    name: str
    T: int
    B: int
    F: int
    num_states: int
    edges: np.ndarray  # (4,E) int32
    weights: np.ndarray  # (E,) float32
    start_end: np.ndarray  # (2,B) int32
    seq_lens: np.ndarray  # (B,) int32
    states_per_seq: np.ndarray  # (B,) int64
    edges_per_seq: np.ndarray  # (B,) int64
    seq_ids: np.ndarray  # (B,) global sequence ids (seeds)
    sigma: float = 1.0
    blank_bias: float = 0.0
    seed0: int = 0
    extra: Dict = field(default_factory=dict)

    @property
    def num_edges(self) -> int:
        return int(self.edges.shape[1])

    def fsa(self):
        return (self.num_states, self.edges, self.weights, self.start_end)

    def algorithmic_bytes(self) -> int:
        """Bytes one call must move: read scores, write the output, write and re-read the
        forward state scores of every valid frame, write the per-frame sums."""
        tbf = 4 * self.T * self.B * self.F
        ts = int((self.seq_lens.astype(np.int64).clip(0, self.T) * self.states_per_seq).sum())
        return 2 * tbf + 8 * ts + 4 * self.T * self.B

    def viterbi_algorithmic_bytes(self) -> int:
        """Bytes one best-path call must move: one 32-byte DRAM sector per score it needs (a
        distinct (frame, sequence, emission) triple; scores of one emission in adjacent frames lie
        B*F*4 bytes apart, so no two share a sector), the back-pointers of every valid frame written
        once and read once, and the (T,B) alignment plus the (B,) scores."""
        lens = self.seq_lens.astype(np.int64).clip(0, self.T)
        ts = int((lens * self.states_per_seq).sum())
        return self.score_sector_bytes() + 8 * ts + 4 * self.T * self.B + 4 * self.B

    def score_sector_bytes(self) -> int:
        """Bytes of the score tensor the ops actually read: one 32-byte sector per distinct
        (valid frame, sequence, emission) triple."""
        lens = self.seq_lens.astype(np.int64).clip(0, self.T)
        pairs = np.unique(self.edges[3].astype(np.int64) * self.F + self.edges[2].astype(np.int64))
        distinct = np.bincount(pairs // self.F, minlength=self.B)  # emissions per sequence
        return 32 * int((lens * distinct).sum())


# ----------------------------------------------------------------------------------------------
# per-sequence automaton builders; each returns (n_states, from, to, emission, weight, start, end)
# with local state ids 0..n_states-1
# ----------------------------------------------------------------------------------------------

def _ctc_fsa(labels: Sequence[int], blank: int = 0):
    """CTC topology with one separate final state.  States 0..2L alternate blank/label; the
    edge into state j emits that state's symbol; loop, advance, and skip between distinct
    labels.  Every edge entering one of the two last states gets a copy entering the final
    state 2L+1, which has no outgoing edge."""
    L = len(labels)
    n = 2 * L + 1
    sym = [blank if j % 2 == 0 else int(labels[(j - 1) // 2]) for j in range(n)]
    fr, to, em = [], [], []

    def add(a, b_):
        fr.append(a)
        to.append(b_)
        em.append(sym[b_])
        if b_ >= n - 2:  # copy into the final state
            fr.append(a)
            to.append(n)
            em.append(sym[b_])

    for j in range(n):
        add(j, j)
        if j + 1 < n:
            add(j, j + 1)
        if j % 2 == 1 and j + 2 < n and sym[j] != sym[j + 2]:
            add(j, j + 2)
    w = [0.0] * len(fr)
    return n + 1, fr, to, em, w, 0, n


def _chain_hmm(classes: Sequence[int], optional: Sequence[bool], loop_p: float, fwd_p: float,
               skip_p: Optional[float]):
    """Left-to-right HMM over ``classes`` with a virtual start state 0.  State i+1 carries
    classes[i]; the edge into a state emits its class.  ``optional[i]`` adds a bypass edge
    around state i+1; ``skip_p`` adds j -> j+2 edges everywhere."""
    n = len(classes) + 1
    fr, to, em, w = [], [], [], []
    wl, wf = -math.log(loop_p), -math.log(fwd_p)
    ws = -math.log(skip_p) if skip_p else None

    def add(a, b_, wt):
        fr.append(a)
        to.append(b_)
        em.append(int(classes[b_ - 1]))
        w.append(wt)

    add(0, 1, 0.0)
    for j in range(1, n):
        add(j, j, wl)
        if j + 1 < n:
            add(j, j + 1, wf)
        if j + 2 < n and (ws is not None or optional[j]):  # optional[j] belongs to state j+1
            add(j, j + 2, ws if ws is not None else wf)
    return n, fr, to, em, w, 0, n - 1


def _lattice(rng: np.random.Generator, S: int, F: int):
    fr, to, em, w = [], [], [], []
    for j in range(S):
        succ = [j]
        if j + 1 < S:
            deg = int(rng.integers(1, 5))
            hi = min(S - 1, j + 8)
            cand = np.arange(j + 1, hi + 1)
            pick = {j + 1}
            if deg > 1 and len(cand) > 1:
                pick.update(rng.choice(cand[1:], size=min(deg - 1, len(cand) - 1), replace=False).tolist())
            succ += sorted(pick)
        for s2 in succ:
            fr.append(j)
            to.append(int(s2))
    ne = len(fr)
    em = rng.integers(0, F, size=ne).tolist()
    w = (-np.log(rng.uniform(0.05, 1.0, size=ne))).tolist()
    return S, fr, to, em, w, 0, S - 1


# ----------------------------------------------------------------------------------------------

_SPECS = {
    #  name        B     T     F      sigma blank_bias
    "ctc_tiny": (4, 50, 41, 1.0, 0.0),
    "monophone": (32, 500, 121, 2.0, 0.0),
    "triphone": (64, 1500, 12001, 3.0, 0.0),
    "bpe_ctc": (256, 400, 10025, 2.0, 3.0),
    "lattice": (512, 2000, 5000, 2.0, 0.0),
}

WORKLOADS = tuple(_SPECS)


def _one_sequence(name: str, rng: np.random.Generator, T: int, F: int, scale: float = 1.0):
    """Returns (fsa tuple, T_b) for one sequence of workload ``name``.  ``scale`` < 1 shrinks the
    label/phoneme counts and the lower length bounds together (reduced test cases)."""

    def sc(x, lo=1):
        return max(lo, int(round(x * scale)))

    if name == "ctc_tiny":
        L = int(rng.integers(sc(5), sc(12) + 1))
        labels = rng.integers(1, F, size=L)
        return _ctc_fsa(labels), int(rng.integers(min(sc(40), T), T + 1))
    if name == "bpe_ctc":
        L = int(rng.integers(sc(20), sc(100) + 1))
        ranks = np.arange(1, F)
        p = ranks ** -1.1
        p /= p.sum()
        labels = rng.choice(ranks, size=L, p=p)
        return _ctc_fsa(labels), int(rng.integers(min(2 * L + 1, T), T + 1))
    if name == "monophone":
        L = int(rng.integers(sc(20), sc(60) + 1))
        phon = rng.integers(0, 40, size=L)
        classes: List[int] = [0]
        optional: List[bool] = [False]
        for ph in phon:
            for k in range(3):
                classes.append(1 + 3 * int(ph) + k)
                optional.append(False)
            if rng.random() < 0.2:
                classes.append(0)
                optional.append(True)
        if optional[-1]:  # the closing silence is mandatory
            optional[-1] = False
        else:
            classes.append(0)
            optional.append(False)
        return _chain_hmm(classes, optional, 0.3, 0.7, None), int(rng.integers(min(sc(350), T), T + 1))
    if name == "triphone":
        L = int(rng.integers(sc(50), sc(150) + 1))
        classes = [0] + rng.integers(1, F, size=3 * L).tolist() + [0]
        return _chain_hmm(classes, [False] * len(classes), 0.3, 0.7, 0.05), int(rng.integers(min(sc(1200), T), T + 1))
    if name == "lattice":
        S = int(rng.integers(sc(200, 2), sc(4000, 2) + 1))
        fsa = _lattice(rng, S, F)
        tb = int(round(float(rng.lognormal(6.5, 0.6)) * scale))
        tb = int(min(max(tb, max(S // 4, sc(100))), T))
        return fsa, tb
    raise ValueError(f"unknown workload {name!r}")


def make_batch(name: str, B: Optional[int] = None, seed0: int = 0,
               seq_ids: Optional[Sequence[int]] = None, T: Optional[int] = None,
               F: Optional[int] = None, shuffle_edges: bool = False,
               scale: float = 1.0) -> FbwBatch:
    """Build the automata of workload ``name``.  ``seq_ids`` selects global sequence ids (a
    shard); default is 0..B-1.  ``T``/``F`` override the workload's frame and class counts
    and ``scale`` shrinks automata and lengths (smaller test cases).  ``shuffle_edges`` permutes the edge columns (the op must not
    depend on edges being grouped by sequence)."""
    dB, dT, dF, sigma, bias = _SPECS[name]
    T = int(T or dT)
    F = int(F or dF)
    if seq_ids is None:
        seq_ids = np.arange(int(B or dB))
    seq_ids = np.asarray(seq_ids, dtype=np.int64)
    B = len(seq_ids)
    fr, to, em, sq, w = [], [], [], [], []
    start, end, lens, ns, ne = [], [], [], [], []
    off = 0
    for b, sid in enumerate(seq_ids):
        rng = np.random.default_rng(seed0 + int(sid))
        (n, f_, t_, e_, w_, s0, s1), tb = _one_sequence(name, rng, T, F, scale)
        fr.append(np.asarray(f_, dtype=np.int64) + off)
        to.append(np.asarray(t_, dtype=np.int64) + off)
        em.append(np.asarray(e_, dtype=np.int64))
        sq.append(np.full(len(f_), b, dtype=np.int64))
        w.append(np.asarray(w_, dtype=np.float32))
        start.append(off + s0)
        end.append(off + s1)
        lens.append(min(tb, T))
        ns.append(n)
        ne.append(len(f_))
        off += n
    edges = np.stack([np.concatenate(fr), np.concatenate(to), np.concatenate(em),
                      np.concatenate(sq)]).astype(np.int32)
    weights = np.concatenate(w).astype(np.float32)
    if shuffle_edges:
        perm = np.random.default_rng(seed0 + 7919).permutation(edges.shape[1])
        edges, weights = np.ascontiguousarray(edges[:, perm]), weights[perm]
    if name == "lattice":
        T = int(max(lens))
    return FbwBatch(name=name, T=T, B=B, F=F, num_states=off, edges=np.ascontiguousarray(edges),
                    weights=weights, start_end=np.array([start, end], dtype=np.int32),
                    seq_lens=np.array(lens, dtype=np.int32),
                    states_per_seq=np.array(ns, dtype=np.int64),
                    edges_per_seq=np.array(ne, dtype=np.int64), seq_ids=seq_ids, sigma=sigma,
                    blank_bias=bias, seed0=seed0)


def take_sequences(batch: FbwBatch, indices: Sequence[int]) -> FbwBatch:
    """The sequences ``indices`` of ``batch`` as a batch of their own (a rank's shard): sequence ids
    become 0..n-1 in the order given, state ids are renumbered densely, per-sequence seeds and the
    frame count T are kept, so scores and automata equal those of the full batch."""
    from .sharding import extract_shard

    idx = np.asarray(indices, dtype=np.int64)
    S, e, w, se, sl = extract_shard(batch.num_states, batch.edges, batch.weights, batch.start_end,
                                    batch.seq_lens, idx)
    return FbwBatch(name=batch.name, T=batch.T, B=len(idx), F=batch.F, num_states=S, edges=e, weights=w,
                    start_end=se, seq_lens=sl, states_per_seq=batch.states_per_seq[idx],
                    edges_per_seq=batch.edges_per_seq[idx], seq_ids=batch.seq_ids[idx], sigma=batch.sigma,
                    blank_bias=batch.blank_bias, seed0=batch.seed0)


def make_scores(batch: FbwBatch, device="cpu", out=None):
    """Scores of a batch as a (T,B,F) float32 torch tensor of negative log-probabilities:
    ``-log_softmax(N(0, sigma^2) logits)`` with the blank logit biased where the workload says
    so; sequence b is drawn from a generator seeded ``seed0 + seq_ids[b]`` on ``device``
    (frames past a sequence's length keep their random values; the op ignores them)."""
    import torch

    dev = torch.device(device)
    am = out if out is not None else torch.empty((batch.T, batch.B, batch.F), dtype=torch.float32, device=dev)
    for b, sid in enumerate(batch.seq_ids):
        g = torch.Generator(device=dev)
        g.manual_seed(int(batch.seed0 + int(sid)))
        logits = torch.randn((batch.T, batch.F), generator=g, device=dev, dtype=torch.float32)
        logits.mul_(batch.sigma)
        if batch.blank_bias:
            logits[:, 0] += batch.blank_bias
        am[:, b, :] = -torch.log_softmax(logits, dim=-1)
    return am


def to_torch(batch: FbwBatch, device="cpu"):
    """(fsa tuple, seq_lens) as torch tensors on ``device`` in the reference's format."""
    import torch

    dev = torch.device(device)
    fsa = (batch.num_states, torch.from_numpy(batch.edges).to(dev),
           torch.from_numpy(batch.weights).to(dev), torch.from_numpy(batch.start_end).to(dev))
    return fsa, torch.from_numpy(batch.seq_lens).to(dev)
