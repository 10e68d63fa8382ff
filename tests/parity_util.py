"""Shared helpers of the GPU parity tests: running the new op and the reference op, the distance
measures of the task statement, and the per-sequence comparison against the fp64 CPU oracle.

Tolerances (task statement): |d loss| / loss <= 1e-5 and max-abs posterior difference <= 1e-4 against
the reference op in fp32.  The reference op accumulates with float atomics in no fixed order
(i6_native_ops/fbw/fbw_op.cu:50-59, 101, 152), so two runs of it on one input differ; where that
spread exceeds 5e-5 the 1e-4 bar against one particular run is not meaningful; on every case the test
demands that the new op is no farther from the fp64 truth than the reference is (bars below).
"""
import json
import os
import sys
import tempfile

import numpy as np
import torch

import oracle
from i6_native_ops_b200 import sharding
from i6_native_ops_b200 import workloads as wl

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LOSS_RTOL = 1e-5
POST_ATOL = 1e-4
REF_SPREAD_FOR_ATOL = 5e-5   # the 1e-4 bar applies where two reference runs agree to this
# "No farther from the fp64 truth than the reference op": the distance is measured as the root of the
# summed squared posterior error (a stable statistic) and as the largest single error (a noisy one:
# two runs of the reference differ by up to ~10 % in it on one and the same sequence).
RMS_FACTOR_CASE = 1.05       # whole case, root-sum-square error, against the farther reference run
RMS_FACTOR_SEQUENCE = 1.15   # the same per sequence
MAX_FACTOR_SEQUENCE = 1.25   # largest single error per sequence
TRUTH_SLACK = 2e-6           # absolute slack on the largest-error bars (tiny cases)


def report_path():
    """Where the parity records go: FBW_PARITY_REPORT if set, else a file in the temp directory."""
    return os.environ.get("FBW_PARITY_REPORT") or os.path.join(tempfile.gettempdir(), "fbw_parity.jsonl")


def report(name, **kv):
    try:
        with open(report_path(), "a") as f:
            f.write(json.dumps(dict(case=name, **kv)) + "\n")
    except OSError:
        pass


def load_ref_fbw():
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import build_ref

    return build_ref.load_ref()


def run_new(m, am, batch_or_tuple, dev):
    if isinstance(batch_or_tuple, wl.FbwBatch):
        fsa, sl = wl.to_torch(batch_or_tuple, dev)
    else:
        fsa, sl = batch_or_tuple
    out, sums = m.core.fbw(am, fsa[1], fsa[2], fsa[3], sl, int(fsa[0]), m.core.DebugOptions())
    return out, sums


def run_ref(ref, am, batch, dev):
    fsa, sl = wl.to_torch(batch, dev)
    torch.cuda.set_device(dev)  # the reference has no device guard
    out, sums = ref.fbw(am, fsa[1], fsa[2], fsa[3], sl, int(fsa[0]), ref.DebugOptions())
    torch.cuda.synchronize()
    return out, sums


def post_abs_diff(out_a, out_b, chunk=64):
    """max |exp(-a) - exp(-b)| over a (T,B,F) pair, chunked over T to bound memory."""
    worst = 0.0
    for t0 in range(0, out_a.shape[0], chunk):
        a = torch.exp(-out_a[t0:t0 + chunk].double())
        b = torch.exp(-out_b[t0:t0 + chunk].double())
        worst = max(worst, float((a - b).abs().max()))
    return worst


def loss_rel_diff(s_a, s_b):
    valid = s_b != 0
    if not bool(valid.any()):
        return 0.0
    return float(((s_a - s_b).abs()[valid] / s_b.abs()[valid]).max())


def check_padding(out, sums, seq_lens, T):
    """sums == 0 and out == +inf at and past seq_len (fbw_op.cu:120-124, 366-370)."""
    t = torch.arange(T, device=out.device)[:, None]
    pad = t >= seq_lens.to(out.device)[None, :].clamp(min=0)
    bad_len = (seq_lens < 1) | (seq_lens > T)
    pad = pad | bad_len.to(out.device)[None, :]
    assert bool((sums[pad] == 0).all())
    for t0 in range(0, T, 64):
        assert bool(torch.isinf(out[t0:t0 + 64][pad[t0:t0 + 64]]).all())


def merge_batches(first, second):
    """Two batches of one workload family (same T and F) as one: the sequences of ``second`` follow
    those of ``first``; state ids and sequence ids are offset, per-sequence seeds are kept."""
    assert first.T == second.T and first.F == second.F and first.sigma == second.sigma
    e2 = second.edges.copy()
    e2[0] += first.num_states
    e2[1] += first.num_states
    e2[3] += first.B
    return wl.FbwBatch(
        name=first.name, T=first.T, B=first.B + second.B, F=first.F,
        num_states=first.num_states + second.num_states,
        edges=np.ascontiguousarray(np.concatenate([first.edges, e2], axis=1)),
        weights=np.concatenate([first.weights, second.weights]),
        start_end=np.ascontiguousarray(np.concatenate([first.start_end, second.start_end + first.num_states], axis=1)),
        seq_lens=np.concatenate([first.seq_lens, second.seq_lens]),
        states_per_seq=np.concatenate([first.states_per_seq, second.states_per_seq]),
        edges_per_seq=np.concatenate([first.edges_per_seq, second.edges_per_seq]),
        seq_ids=np.concatenate([first.seq_ids, second.seq_ids]), sigma=first.sigma,
        blank_bias=first.blank_bias, seed0=first.seed0)


def sample_sequences(batch, n):
    """Indices of ``n`` sequences spread over the batch's cost order (most expensive and cheapest
    included); all sequences if the batch has no more than ``n``."""
    if batch.B <= n:
        return np.arange(batch.B)
    cost = batch.seq_lens.astype(np.int64) * batch.edges_per_seq
    order = np.argsort(-cost, kind="stable")
    pick = order[np.linspace(0, batch.B - 1, n).round().astype(int)]
    return np.sort(pick)


def truth_distances(batch, am, outs, sums_list, idx):
    """Per-sequence distances from the fp64 oracle for the sequences ``idx`` of ``batch``.

    ``outs`` / ``sums_list``: lists of (T,B,F) / (T,B) device tensors (new op, reference runs).
    Returns (post (len(outs), len(idx)) max-abs posterior distance, sq (same shape) summed squared
    posterior distance, loss (same shape) max relative distance of the per-frame sums, pattern_ok: the
    +inf / zero patterns equal the oracle's)."""
    dev = am.device
    idx = np.asarray(idx, dtype=np.int64)
    S, e, w, se, sl = sharding.extract_shard(batch.num_states, batch.edges, batch.weights, batch.start_end,
                                             batch.seq_lens, idx)
    sel = torch.from_numpy(idx).to(dev)
    am_h = am.index_select(1, sel).cpu().numpy()
    o64, s64 = oracle.fbw_oracle(am_h, e, w, se, sl, S, "f64")
    del am_h
    post = np.zeros((len(outs), len(idx)))
    sq = np.zeros((len(outs), len(idx)))
    loss = np.zeros((len(outs), len(idx)))
    pattern_ok = True
    for j, b in enumerate(idx):
        truth_out = torch.from_numpy(np.ascontiguousarray(o64[:, j, :])).to(dev)
        truth_post = torch.exp(-truth_out)
        truth_sum = torch.from_numpy(np.ascontiguousarray(s64[:, j])).to(dev)
        valid = truth_sum != 0
        for i, (out, sums) in enumerate(zip(outs, sums_list)):
            o = out[:, int(b), :]
            pattern_ok = pattern_ok and bool(torch.equal(torch.isinf(o), torch.isinf(truth_out)))
            pattern_ok = pattern_ok and bool(torch.equal(sums[:, int(b)] == 0, ~valid))
            err = torch.exp(-o.double()) - truth_post
            post[i, j] = float(err.abs().max())
            sq[i, j] = float((err * err).sum())
            if bool(valid.any()):
                s = sums[:, int(b)].double()
                loss[i, j] = float(((s - truth_sum).abs()[valid] / truth_sum.abs()[valid]).max())
        del truth_out, truth_post
    return post, sq, loss, pattern_ok


def full_parity(name, m, ref, batch, am, dev, sample=8, runs_of_reference=3, extra=None):
    """The complete comparison of one case: new op against the reference op (whole batch) and both
    against the fp64 oracle (per sequence on a sample).  Asserts the bars described at the top of
    this file and appends a record to the parity report.  Returns the record."""
    out, sums = run_new(m, am, batch, dev)
    torch.cuda.synchronize()
    fsa, sl = wl.to_torch(batch, dev)
    check_padding(out, sums, sl, batch.T)
    idx = sample_sequences(batch, sample)
    rec = dict(extra or {}, B=batch.B, T=batch.T, F=batch.F, E=batch.num_edges, S=batch.num_states,
               max_states=int(batch.states_per_seq.max()), max_edges=int(batch.edges_per_seq.max()),
               oracle_sequences=[int(i) for i in idx])
    outs, sums_list = [out], [sums]
    if ref is not None:
        for _ in range(runs_of_reference):
            r_out, r_sums = run_ref(ref, am, batch, dev)
            outs.append(r_out)
            sums_list.append(r_sums)
        rec["loss_vs_ref"] = loss_rel_diff(sums, sums_list[1])
        rec["post_vs_ref"] = min(post_abs_diff(out, r) for r in outs[1:])
        rec["ref_vs_ref_post"] = post_abs_diff(outs[1], outs[2]) if len(outs) > 2 else None
        assert bool(torch.equal(sums == 0, sums_list[1] == 0))
        for t0 in range(0, batch.T, 64):
            assert bool(torch.equal(torch.isinf(out[t0:t0 + 64]), torch.isinf(outs[1][t0:t0 + 64])))
    post, sq, loss, pattern_ok = truth_distances(batch, am, outs, sums_list, idx)
    rec["post_vs_f64"] = float(post[0].max())
    rec["loss_vs_f64"] = float(loss[0].max())
    # posteriors of a valid frame sum to one (the reference's own test, test/fbw.py:60-64), zero past
    # the length; fp32 scores of magnitude M carry rounding ~ M * 2^-23 into every posterior
    score_max = float(sums.abs().max())
    rec["score_max"] = score_max
    ulp_tol = max(1e-4, 64 * score_max * 2.0 ** -23)
    t = torch.arange(batch.T, device=dev)
    row_err = 0.0
    for b in idx:
        rows = torch.zeros(batch.T, dtype=torch.float64, device=dev)
        for t0 in range(0, batch.T, 256):
            rows[t0:t0 + 256] = torch.exp(-out[t0:t0 + 256, int(b), :].double()).sum(-1)
        valid = (t < int(batch.seq_lens[b])) & (sums[:, int(b)] != 0)
        assert bool((rows[~valid] == 0).all()), name
        if bool(valid.any()):
            row_err = max(row_err, float((rows[valid] - 1).abs().max()))
    rec["row_sum_err"] = row_err
    if ref is not None:
        ref_truth = post[1:].max(axis=0)   # per sequence, the farther of the reference runs
        rec["ref_post_vs_f64"] = float(post[1:].max())
        rec["max_ratio_worst_sequence"] = float((post[0] / np.maximum(ref_truth, 1e-12)).max())
        ref_sq = sq[1:].max(axis=0)
        rec["rms_ratio_case"] = float(np.sqrt(sq[0].sum() / max(sq[1:].sum(axis=1).max(), 1e-300)))
        rec["rms_ratio_worst_sequence"] = float(np.sqrt(sq[0] / np.maximum(ref_sq, 1e-300)).max())
        if len(outs) > 2:  # the same statistics between the reference's own runs, for the record
            rec["ref_max_ratio_between_runs"] = float((post[1:].max(axis=0) / np.maximum(post[1:].min(axis=0), 1e-12)).max())
            rec["ref_rms_ratio_between_runs"] = float(np.sqrt(sq[1:].max(axis=0) / np.maximum(sq[1:].min(axis=0), 1e-300)).max())
    report(name, **rec)
    assert pattern_ok, name
    assert rec["loss_vs_f64"] <= LOSS_RTOL, rec
    assert row_err <= ulp_tol, rec
    if ref is None:
        # without the reference build: the distance from the truth is bounded by fp32 rounding of the
        # score magnitude alone
        assert rec["post_vs_f64"] <= ulp_tol * 4, rec
    else:
        assert rec["loss_vs_ref"] <= LOSS_RTOL, rec
        # no farther from the truth than the incumbent: whole sample and every sequence of it
        floor = TRUTH_SLACK ** 2 * batch.T  # squared-error floor below which ratios mean nothing
        assert sq[0].sum() <= RMS_FACTOR_CASE ** 2 * sq[1:].sum(axis=1).max() + floor, rec
        assert bool((sq[0] <= RMS_FACTOR_SEQUENCE ** 2 * ref_sq + floor).all()), (rec, sq.tolist())
        assert bool((post[0] <= MAX_FACTOR_SEQUENCE * ref_truth + TRUTH_SLACK).all()), (rec, post.tolist())
        if rec["ref_vs_ref_post"] is not None and rec["ref_vs_ref_post"] <= REF_SPREAD_FOR_ATOL:
            assert rec["post_vs_ref"] <= POST_ATOL, rec
    return rec
