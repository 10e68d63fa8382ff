"""GPU tests of the DebugOptions text dumps (reference: write_alignment_to_file / write_output_to_file,
fbw_op.cu:155-224, triggered at fbw_op.cu:360-364, 380-382 every `dump_every`-th call).

The files are compared line by line with a restatement of the dump from the CPU oracle's forward state
scores and output, and with the files the reference op writes when its build is present.  Values are
printed with 6 significant digits, so they are compared within 2e-3; a line may be missing on one side
only if its value lies that close to the pruning threshold."""
import glob
import os
import sys

import numpy as np
import pytest
import torch

import oracle
from i6_native_ops_b200 import workloads as wl

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
TOL = 2e-3


@pytest.fixture(scope="module")
def fbw_mod(cuda):
    import i6_native_ops_b200.fbw as m

    return m


@pytest.fixture(scope="module")
def ref_core(cuda):
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import build_ref

    return build_ref.load_ref()


def read_dump(path):
    d = {}
    with open(path) as f:
        for line in f:
            t, i, v = line.split()
            d[(int(t), int(i))] = float(v)
    return d


def read_dumps(folder, kind, n_seqs):
    """{seq: {(t, index): value}} of the one call that wrote files into `folder`."""
    files = glob.glob(os.path.join(folder, f"{kind}.dump.*.*"))
    calls = {os.path.basename(p).split(".")[2] for p in files}
    assert len(calls) == 1, calls
    call = calls.pop()
    return {b: read_dump(os.path.join(folder, f"{kind}.dump.{call}.{b}")) for b in range(n_seqs)}


def same_dump(a, b, pruning):
    for key in set(a) | set(b):
        if key in a and key in b:
            assert abs(a[key] - b[key]) <= TOL + 1e-5 * abs(a[key]), (key, a[key], b[key])
        else:
            v = a.get(key, b.get(key))
            assert abs(v - pruning) <= TOL + 1e-5 * abs(v), (key, v, "present on one side only")


def expected_alignment(alpha, batch, pruning):
    """Restatement of the alignment dump from the oracle's (T+1, S) forward scores (float32 order)."""
    out = {}
    for b in range(batch.B):
        first, last = int(batch.start_end[0, b]), int(batch.start_end[1, b])
        d = {}
        for t in range(batch.T):
            if t > 0 and t >= int(batch.seq_lens[b]):
                break
            row = alpha[t, first:last + 1].astype(np.float64)
            finite = row[np.isfinite(row)]
            total = np.inf if finite.size == 0 else finite.min() - np.log(np.exp(-(finite - finite.min())).sum())
            for s, v in enumerate(row - total):
                if v <= pruning:
                    d[(t, s)] = float(v)
        out[b] = d
    return out


def expected_target(out_arr, batch, pruning):
    res = {}
    for b in range(batch.B):
        d = {}
        for t in range(batch.T):
            if t > 0 and t >= int(batch.seq_lens[b]):
                break
            for e in np.nonzero(out_arr[t, b] <= pruning)[0]:
                d[(t, int(e))] = float(out_arr[t, b, e])
        res[b] = d
    return res


@pytest.mark.parametrize("name,kw", [("ctc_tiny", dict()), ("monophone", dict(B=3, T=60, scale=0.12))])
def test_dumps_match_oracle_and_reference(fbw_mod, ref_core, cuda, tmp_path, monkeypatch, name, kw):
    batch = wl.make_batch(name, **kw)
    am = wl.make_scores(batch, cuda)
    fsa, sl = wl.to_torch(batch, cuda)
    pruning = 7.5
    new_dir = tmp_path / "new"
    new_dir.mkdir()
    monkeypatch.chdir(new_dir)
    opts = fbw_mod.core.DebugOptions()
    opts.dump_alignment, opts.dump_output, opts.dump_every, opts.pruning = True, True, 1, pruning
    out, sums = fbw_mod.core.fbw(am, fsa[1], fsa[2], fsa[3], sl, int(fsa[0]), opts)
    torch.cuda.synchronize()
    got_align = read_dumps(str(new_dir), "alignment", batch.B)
    got_target = read_dumps(str(new_dir), "target", batch.B)

    o_out, _, alpha, _ = oracle.fbw_oracle(am.cpu().numpy(), batch.edges, batch.weights, batch.start_end,
                                           batch.seq_lens, batch.num_states, "f32", want_states=True)
    want_align = expected_alignment(alpha, batch, pruning)
    want_target = expected_target(o_out, batch, pruning)
    for b in range(batch.B):
        assert len(got_align[b]) > 0 and len(got_target[b]) > 0
        same_dump(got_align[b], want_align[b], pruning)
        same_dump(got_target[b], want_target[b], pruning)

    if ref_core is not None:
        ref_dir = tmp_path / "ref"
        ref_dir.mkdir()
        monkeypatch.chdir(ref_dir)
        torch.cuda.set_device(0)
        ropts = ref_core.DebugOptions()
        ropts.dump_alignment, ropts.dump_output, ropts.dump_every, ropts.pruning = True, True, 1, pruning
        ref_core.fbw(am, fsa[1], fsa[2], fsa[3], sl, int(fsa[0]), ropts)
        torch.cuda.synchronize()
        ref_align = read_dumps(str(ref_dir), "alignment", batch.B)
        ref_target = read_dumps(str(ref_dir), "target", batch.B)
        for b in range(batch.B):
            same_dump(got_align[b], ref_align[b], pruning)
            same_dump(got_target[b], ref_target[b], pruning)


def test_dump_every_and_off_by_default(fbw_mod, cuda, tmp_path, monkeypatch):
    batch = wl.make_batch("ctc_tiny")
    am = wl.make_scores(batch, cuda)
    fsa, sl = wl.to_torch(batch, cuda)
    monkeypatch.chdir(tmp_path)
    fbw_mod.core.fbw(am, fsa[1], fsa[2], fsa[3], sl, int(fsa[0]), fbw_mod.core.DebugOptions())
    assert glob.glob(str(tmp_path / "*.dump.*")) == []  # both flags default to False
    opts = fbw_mod.core.DebugOptions()
    opts.dump_output, opts.dump_every = True, 2
    for _ in range(4):  # two of four consecutive calls fall on a multiple of dump_every
        fbw_mod.core.fbw(am, fsa[1], fsa[2], fsa[3], sl, int(fsa[0]), opts)
    files = glob.glob(str(tmp_path / "target.dump.*.0"))
    calls = sorted(int(os.path.basename(p).split(".")[2]) for p in files)
    assert len(calls) == 2 and all(c % 2 == 0 for c in calls)
    assert glob.glob(str(tmp_path / "alignment.dump.*")) == []
