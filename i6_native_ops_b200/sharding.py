"""Shard a batch of automata by sequence over the GPUs of one node.

Sequences are independent in the reference op (no kernel of i6_native_ops/fbw/fbw_op.cu couples
two sequence indices), so every rank runs the op on its own sequences and the only exchange is
one all-reduce of two loss scalars.  This module holds the host logic: cost model, balanced
partition, extraction of a shard with sequence and state ids renumbered, and the reduced step.
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

import numpy as np


def sequence_costs(states_per_seq, edges_per_seq, seq_lens, T: int, F: int,
                   row_weight: float = 0.02) -> np.ndarray:
    """Relative cost of each sequence: sweep work (frames x edges) plus its share of the
    (T,F) row traffic; ``row_weight`` converts row floats into edge-relaxation units."""
    seq_lens = np.asarray(seq_lens, dtype=np.float64).clip(0, T)
    edges = np.asarray(edges_per_seq, dtype=np.float64)
    return 4.0 * seq_lens * edges + row_weight * float(T) * float(F) + 0.0 * np.asarray(states_per_seq)


def partition(costs: Sequence[float], world_size: int) -> List[np.ndarray]:
    """Longest-processing-time greedy partition.  Returns, per rank, the ascending indices of
    its sequences.  Every rank gets at least one sequence when there are enough; with fewer
    sequences than ranks some shards are empty (``sharded_fbw`` copes with that)."""
    costs = np.asarray(costs, dtype=np.float64)
    n = len(costs)
    if world_size < 1:
        raise ValueError("world_size must be >= 1")
    order = np.argsort(-costs, kind="stable")
    load = np.zeros(world_size)
    count = np.zeros(world_size, dtype=np.int64)
    cap = -(-n // world_size) if n else 0  # ceil: keeps shard sizes within one of each other
    parts: List[List[int]] = [[] for _ in range(world_size)]
    for i in order:
        open_ranks = np.flatnonzero(count < cap)
        r = open_ranks[np.argmin(load[open_ranks])]
        parts[r].append(int(i))
        load[r] += costs[i]
        count[r] += 1
    return [np.array(sorted(p), dtype=np.int64) for p in parts]


def extract_shard(num_states: int, edges: np.ndarray, weights: np.ndarray, start_end: np.ndarray,
                  seq_lens: np.ndarray, seq_indices: Sequence[int]):
    """Automata of the sequences ``seq_indices`` as a self-contained batch: sequence ids become
    0..n-1 (in the order given) and state ids are renumbered densely.  Edge order is kept.
    Returns (num_states, edges, weights, start_end, seq_lens)."""
    seq_indices = np.asarray(seq_indices, dtype=np.int64)
    B = start_end.shape[1]
    new_seq = np.full(B, -1, dtype=np.int64)
    new_seq[seq_indices] = np.arange(len(seq_indices))
    keep = new_seq[edges[3]] >= 0
    e = edges[:, keep].astype(np.int64)
    used = np.zeros(num_states, dtype=bool)
    used[e[0]] = True
    used[e[1]] = True
    used[start_end[:, seq_indices].ravel()] = True
    new_state = np.cumsum(used) - 1
    out_edges = np.stack([new_state[e[0]], new_state[e[1]], e[2], new_seq[e[3]]]).astype(np.int32)
    se = new_state[start_end[:, seq_indices]].astype(np.int32)
    return (int(used.sum()), np.ascontiguousarray(out_edges), np.ascontiguousarray(weights[keep]),
            np.ascontiguousarray(se), np.ascontiguousarray(seq_lens[seq_indices]))


def reduce_loss(loss2, group=None):
    """All-reduce (sum) of the two per-rank loss scalars; a no-op without an initialised
    process group.  ``loss2`` is a 2-element tensor on the rank's device (CUDA with NCCL, CPU
    with gloo)."""
    import torch.distributed as dist

    if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(loss2, op=dist.ReduceOp.SUM, group=group)
    return loss2


def _empty_step(am_scores, device):
    """Results of a rank whose shard has no sequence (fewer sequences than ranks): nothing to run,
    zero loss -- the rank still has to take part in the all-reduce or the others would wait for it."""
    import torch

    T = am_scores.shape[0]
    out = torch.empty(tuple(am_scores.shape), dtype=torch.float32, device=device)
    sums = torch.zeros((T, 0), dtype=torch.float32, device=device)
    return out, sums, torch.zeros(2, dtype=torch.float32, device=device)


def sharded_fbw(am_scores, fsa, seq_lens, plan=None, group=None):
    """One data-parallel step on this rank's shard: run the op on the local sequences and
    all-reduce the loss scalars on the same stream.  Returns (out, sums, loss2_global, plan);
    pass ``plan`` back in to reuse the prepared automata with new scores.  A rank with an empty
    shard (``am_scores.shape[1] == 0``) skips the op and contributes zeros to the reduction."""
    if am_scores.shape[1] == 0:
        out, sums, loss2 = _empty_step(am_scores, am_scores.device)
        reduce_loss(loss2, group)
        return out, sums, loss2, None
    from .fbw import core

    num_states, edges, weights, start_end = fsa
    if plan is None:
        plan = core.fbw_prepare(edges, weights, start_end, seq_lens, am_scores.shape[0],
                                am_scores.shape[2], int(num_states))
    out, sums, loss2 = core.fbw_run(plan, am_scores)
    reduce_loss(loss2, group)
    return out, sums, loss2, plan


def sharded_fbw_host_scores(am_scores_pinned, fsa, seq_lens, group=None, out=None, staged=True):
    """:func:`sharded_fbw` for scores that live in pinned host memory: the op reads the scores it needs
    in place (no copy of the whole tensor to the device); ``out``, if given, is a pinned host tensor
    that receives the (T,B,F) result (``staged``: sparse rows are written by the library's host threads
    from the posteriors the device sends, dense ones go through a device buffer that is copied out while
    the op runs; otherwise written in place by the output pass).  Returns (out, sums, loss2_global).  An empty
    shard is handled as in :func:`sharded_fbw`."""
    num_states, edges, weights, start_end = fsa
    if am_scores_pinned.shape[1] == 0:
        out, sums, loss2 = _empty_step(am_scores_pinned, edges.device)
        reduce_loss(loss2, group)
        return out, sums, loss2
    from .fbw import core

    out, sums, loss2 = core.fbw_host_scores(am_scores_pinned, edges, weights, start_end, seq_lens,
                                            int(num_states), out, bool(staged))
    reduce_loss(loss2, group)
    return out, sums, loss2
