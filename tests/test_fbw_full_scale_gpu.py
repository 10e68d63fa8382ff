"""GPU parity tests at the sizes of the benchmark configurations, and of the code paths that only
large or irregular automata reach:

  * lattice automata at full scale (up to 4000 states and ~14000 edges per sequence): the general
    plan builder (device-wide sorts), sweeps over more states than a CTA has threads, edge lists too
    large for shared memory;
  * a batch of small automata with one large one: the per-sequence plan builder gives up on that
    sequence and the plan is rebuilt by the general builder;
  * the large-vocabulary CTC batch at full size (B=256, T=400, F=10025);
  * a 64-sequence slice of the full-scale lattice batch (the largest piece of it one call of the
    reference op can take: its 32-bit sizes overflow beyond, i6_native_ops/fbw/fbw_op.cu:268-276);
  * 24 lattice sequences, as four size groups and as the pipeline over time chunks with the
    large-automaton sweeps;
  * a batch of more than 8192 sequences (grouping by sequence switches to a device-wide sort).

Targets: the fp64 CPU oracle on every sequence (or a sample of eight spread over the cost order) and
two runs of the reference op on the whole batch; bars in tests/parity_util.py.
"""
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

from i6_native_ops_b200 import workloads as wl
from parity_util import full_parity, load_ref_fbw, merge_batches

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def fbw_mod(cuda):
    import i6_native_ops_b200.fbw as m

    return m


@pytest.fixture(scope="module")
def ref_core(cuda):
    return load_ref_fbw()


def plan_info(m, batch, dev):
    fsa, sl = wl.to_torch(batch, dev)
    return m.core.fbw_prepare(fsa[1], fsa[2], fsa[3], sl, batch.T, batch.F, int(fsa[0])).info()


@pytest.mark.parametrize("shuffle", [False, True])
def test_lattice_full_scale(fbw_mod, ref_core, cuda, shuffle):
    """Eight full-scale lattice automata (F=5000, T up to 2000), edges grouped by sequence and shuffled."""
    b = wl.make_batch("lattice", B=8, shuffle_edges=shuffle)
    assert b.states_per_seq.max() > 1024 and b.edges_per_seq.max() > 4096
    am = wl.make_scores(b, cuda)
    full_parity(f"lattice_full_scale B=8 shuffle={shuffle}", fbw_mod, ref_core, b, am, cuda, sample=8)


def test_one_large_automaton_among_small_ones(fbw_mod, ref_core, cuda):
    """Average size small enough for the per-sequence plan builder, one sequence over its limit of 4096
    edges: the first plan reports that it must be rebuilt, the binding rebuilds it with the general
    builder."""
    small = wl.make_batch("lattice", B=11, F=257, T=600, scale=0.1)
    for sid in range(1000, 1040):  # the first generated automaton of 1300..3000 states
        large = wl.make_batch("lattice", seq_ids=[sid], F=257, T=600, scale=1.0)
        if 1300 <= large.num_states <= 3000:
            break
    small.T = large.T = 600
    large.seq_lens[:] = 600  # long enough for a path through 3000 states (a step advances 8 at most)
    b = merge_batches(small, large)
    assert b.edges_per_seq.max() > 4096 and b.num_edges / b.B <= 2048
    am = wl.make_scores(b, cuda)
    full_parity("one_large_among_small", fbw_mod, ref_core, b, am, cuda, sample=16)


def test_bpe_ctc_full_size(fbw_mod, ref_core, cuda):
    b = wl.make_batch("bpe_ctc")
    assert (b.B, b.T, b.F) == (256, 400, 10025)
    am = wl.make_scores(b, cuda)
    full_parity("bpe_ctc_full", fbw_mod, ref_core, b, am, cuda, sample=8)


def test_lattice_slice_of_64(fbw_mod, ref_core, cuda):
    """Sequences 0..63 of the B=512 lattice batch at full scale."""
    b = wl.make_batch("lattice", B=64)
    am = wl.make_scores(b, cuda)
    full_parity("lattice_full_scale B=64", fbw_mod, ref_core, b, am, cuda, sample=8)


def test_lattice_few_sequences(fbw_mod, ref_core, cuda):
    """24 full-scale lattice sequences: four size groups of six sequences, the two most expensive
    groups as clusters."""
    b = wl.make_batch("lattice", B=24)
    am = wl.make_scores(b, cuda)
    full_parity("lattice_full_scale B=24 (four groups)", fbw_mod, ref_core, b, am, cuda, sample=8)


def test_lattice_time_chunk_pipeline(cuda):
    """The same 24 sequences through the pipeline over time chunks, which the library no longer picks
    for large automata by itself (FBW_B200_NUM_GROUPS=1 switches the size groups off for a process): the
    sweeps (clusters, state scores stored four frames at a time) then run as several launches that hand
    their state vectors on.  Runs the test above in a child process."""
    env = dict(os.environ, FBW_B200_NUM_GROUPS="1")
    r = subprocess.run([sys.executable, "-m", "pytest", os.path.abspath(__file__), "-q", "-x", "-m", "gpu", "-k",
                        "test_lattice_few_sequences", "-p", "no:cacheprovider"],
                       env=env, capture_output=True, text=True, timeout=1200,
                       cwd=os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    assert r.returncode == 0 and "1 passed" in r.stdout, r.stdout[-2000:] + r.stderr[-2000:]


def test_more_than_8192_sequences(fbw_mod, cuda):
    """B = 8200 tiny CTC automata; the reference op cannot take more than 1024 sequences (it
    launches one block of B threads, fbw_op.cu:299, 344), so the target is the fp64 oracle alone."""
    b = wl.make_batch("ctc_tiny", B=8200, T=24, F=11, scale=0.4)
    am = wl.make_scores(b, cuda)
    full_parity("ctc_tiny B=8200", fbw_mod, None, b, am, cuda, sample=8200)
