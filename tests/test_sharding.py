"""CPU tests of the multi-GPU host logic: cost-balanced partition by sequence, shard extraction
with renumbered sequence/state ids, and the one collective of the path (an all-reduce of two
loss scalars), run as two gloo ranks.  The per-rank numbers come from the CPU oracle, used here
only as the checker; the GPU path itself is covered by the -m gpu tests."""
import os

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle
from i6_native_ops_b200 import sharding
from i6_native_ops_b200 import workloads as wl


def test_partition_is_balanced_and_complete():
    rng = np.random.default_rng(0)
    costs = rng.lognormal(0, 1, size=101)
    for world in (1, 2, 4, 8):
        parts = sharding.partition(costs, world)
        assert len(parts) == world
        allidx = np.sort(np.concatenate(parts))
        assert np.array_equal(allidx, np.arange(len(costs)))
        sizes = [len(p) for p in parts]
        assert max(sizes) - min(sizes) <= 1
        loads = np.array([costs[p].sum() for p in parts])
        assert loads.max() <= loads.mean() + costs.max()  # longest-processing-time bound
    assert [len(p) for p in sharding.partition([1.0, 2.0], 4)] .count(0) == 2


def test_extract_shard_matches_full_batch():
    b = wl.make_batch("lattice", B=7, F=40, T=120, scale=0.06, shuffle_edges=True)
    am = wl.make_scores(b).numpy()
    out, sums = oracle.fbw_oracle(am, b.edges, b.weights, b.start_end, b.seq_lens, b.num_states, "f64")
    costs = sharding.sequence_costs(b.states_per_seq, b.edges_per_seq, b.seq_lens, b.T, b.F)
    for idx in sharding.partition(costs, 3):
        S, e, w, se, sl = sharding.extract_shard(b.num_states, b.edges, b.weights, b.start_end,
                                                 b.seq_lens, idx)
        assert e[3].max() < len(idx) and e[:2].max() < S
        o, s = oracle.fbw_oracle(am[:, idx], e, w, se, sl, S, "f64")
        assert np.array_equal(s, sums[:, idx])
        assert np.array_equal(o, out[:, idx])


def test_extract_shard_matches_full_batch_viterbi():
    """The best-path alignment shards the same way and needs no collective at all."""
    b = wl.make_batch("lattice", B=7, F=40, T=120, scale=0.06, shuffle_edges=True)
    am = -wl.make_scores(b).numpy()
    alignment, scores = oracle.viterbi_oracle(am, b.edges, b.weights, b.start_end, b.seq_lens, b.num_states)
    costs = sharding.sequence_costs(b.states_per_seq, b.edges_per_seq, b.seq_lens, b.T, b.F)
    for idx in sharding.partition(costs, 2):
        S, e, w, se, sl = sharding.extract_shard(b.num_states, b.edges, b.weights, b.start_end,
                                                 b.seq_lens, idx)
        a, s_ = oracle.viterbi_oracle(am[:, idx], e, w, se, sl, S)
        assert np.array_equal(a, alignment[:, idx]) and np.array_equal(s_, scores[idx])


def test_shards_generated_independently_match_the_full_batch():
    """Per-sequence seeding: a rank that builds only its own sequences gets the same automata."""
    full = wl.make_batch("monophone", B=6, T=150, scale=0.3)
    part = wl.make_batch("monophone", seq_ids=[1, 4], T=150, scale=0.3)
    S, e, w, se, sl = sharding.extract_shard(full.num_states, full.edges, full.weights,
                                             full.start_end, full.seq_lens, [1, 4])
    assert S == part.num_states
    assert np.array_equal(e, part.edges) and np.array_equal(w, part.weights)
    assert np.array_equal(se, part.start_end) and np.array_equal(sl, part.seq_lens)
    assert torch.equal(wl.make_scores(full)[:, [1, 4]], wl.make_scores(part))


def _rank_main(rank, world, port, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        full = wl.make_batch("ctc_tiny", B=6)
        costs = sharding.sequence_costs(full.states_per_seq, full.edges_per_seq, full.seq_lens,
                                        full.T, full.F)
        mine = sharding.partition(costs, world)[rank]
        shard = wl.make_batch("ctc_tiny", seq_ids=mine)
        am = wl.make_scores(shard).numpy()
        _, sums = oracle.fbw_oracle(am, shard.edges, shard.weights, shard.start_end, shard.seq_lens,
                                    shard.num_states, "f64")
        loss2 = torch.tensor([sums.sum(), sums[0].sum()], dtype=torch.float64)
        sharding.reduce_loss(loss2)
        q.put((rank, loss2.tolist(), [int(i) for i in mine]))
    finally:
        dist.destroy_process_group()


def test_two_rank_loss_all_reduce_gloo():
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + (os.getpid() % 2000)
    procs = [ctx.Process(target=_rank_main, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = [q.get(timeout=120) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    full = wl.make_batch("ctc_tiny", B=6)
    am = wl.make_scores(full).numpy()
    _, sums = oracle.fbw_oracle(am, full.edges, full.weights, full.start_end, full.seq_lens,
                                full.num_states, "f64")
    want = [sums.sum(), sums[0].sum()]
    seen = sorted(i for r in res for i in r[2])
    assert seen == list(range(6))
    for _, loss2, _ in res:  # every rank holds the global sums
        assert np.allclose(loss2, want, rtol=1e-12)


def _rank_main_few_sequences(rank, world, port, q):
    """More ranks than sequences: the ranks without a sequence go through sharded_fbw itself (it
    must skip the op and still join the reduction); the others reduce their oracle numbers."""
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        full = wl.make_batch("ctc_tiny", B=2)
        costs = sharding.sequence_costs(full.states_per_seq, full.edges_per_seq, full.seq_lens,
                                        full.T, full.F)
        mine = sharding.partition(costs, world)[rank]
        if len(mine) == 0:
            am = torch.empty((full.T, 0, full.F))
            fsa = (1, torch.empty((4, 0), dtype=torch.int32), torch.empty(0), torch.empty((2, 0), dtype=torch.int32))
            out, sums, loss2, _ = sharding.sharded_fbw(am, fsa, torch.empty(0, dtype=torch.int32))
            assert out.shape == (full.T, 0, full.F) and sums.shape == (full.T, 0)
        else:
            shard = wl.make_batch("ctc_tiny", seq_ids=mine)
            _, sums = oracle.fbw_oracle(wl.make_scores(shard).numpy(), shard.edges, shard.weights,
                                        shard.start_end, shard.seq_lens, shard.num_states, "f64")
            loss2 = torch.tensor([sums.sum(), sums[0].sum()], dtype=torch.float32)
            sharding.reduce_loss(loss2)
        q.put((rank, loss2.tolist(), [int(i) for i in mine]))
    finally:
        dist.destroy_process_group()


def test_more_ranks_than_sequences_gloo():
    world = 3
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 31500 + (os.getpid() % 2000)
    procs = [ctx.Process(target=_rank_main_few_sequences, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = [q.get(timeout=120) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert sorted(len(r[2]) for r in res) == [0, 1, 1]
    full = wl.make_batch("ctc_tiny", B=2)
    _, sums = oracle.fbw_oracle(wl.make_scores(full).numpy(), full.edges, full.weights, full.start_end,
                                full.seq_lens, full.num_states, "f64")
    for _, loss2, _ in res:  # every rank, the idle one included, holds the global sums
        assert np.allclose(loss2, [sums.sum(), sums[0].sum()], rtol=1e-5)


def test_reduce_loss_is_a_noop_without_a_group():
    t = torch.tensor([1.0, 2.0])
    assert torch.equal(sharding.reduce_loss(t.clone()), t)
