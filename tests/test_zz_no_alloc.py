"""GPU test of fbw_b200_fbw_noalloc, the entry point for callers that may not allocate device
memory while they run (a server with a memory pool frozen at start-up, a plug-in that only gets
input and output buffers from its host).  Its plan and scratch live in a fixed array inside the
library.  The test calls it through the C ABI with ctypes, twice in a row on different inputs (the
array keeps the first call's contents, so the second call shows that stale contents do no harm),
and checks the results against the regular entry points on the same inputs and against the fp64 CPU
oracle.  A third call carries one automaton too large for the per-sequence plan builder, so the
entry's own rebuild of the plan with the general builder is exercised.  The file name makes pytest
collect it last."""
import ctypes
import os

import numpy as np
import pytest
import torch

from i6_native_ops_b200 import workloads as wl
from parity_util import merge_batches, truth_distances

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LIB = os.path.join(ROOT, "i6_native_ops_b200", "libfbw_b200.so")
LOSS_RTOL = 1e-5   # the tolerances of tests/test_fbw_gpu.py
POST_ATOL = 1e-4


def _outputs(am):
    T, B, _ = am.shape
    return (torch.empty_like(am), torch.empty((T, B), dtype=torch.float32, device=am.device),
            torch.empty(2, dtype=torch.float32, device=am.device))


def _noalloc(lib, am, fsa, sl, bufs=None):
    T, B, F = am.shape
    E = fsa[1].shape[1]
    out, sums, loss2 = bufs if bufs is not None else _outputs(am)
    i64, vp = ctypes.c_int64, ctypes.c_void_p
    stream = vp(torch.cuda.current_stream().cuda_stream)
    rc = lib.fbw_b200_fbw_noalloc(vp(am.data_ptr()), vp(fsa[1].data_ptr()), vp(fsa[2].data_ptr()),
                                  vp(fsa[3].data_ptr()), vp(sl.data_ptr()), i64(T), i64(B), i64(F),
                                  i64(E), i64(int(fsa[0])), vp(out.data_ptr()), vp(sums.data_ptr()),
                                  vp(loss2.data_ptr()), stream)
    return rc, out, sums, loss2


def test_noalloc_entry_matches_regular_entry_twice(cuda):
    import i6_native_ops_b200.fbw as m  # loads the library the extension is linked against

    lib = ctypes.CDLL(LIB)
    lib.fbw_b200_fbw_noalloc.restype = ctypes.c_int
    lib.fbw_b200_noalloc_capacity.restype = ctypes.c_size_t
    assert lib.fbw_b200_noalloc_capacity() == 64 << 20
    small = wl.make_batch("lattice", B=11, F=257, T=600, scale=0.1)
    large = wl.make_batch("lattice", seq_ids=[1002], F=257, T=600, scale=1.0)  # about 8700 edges
    small.T = large.T = 600
    large.seq_lens[:] = 600
    mixed = merge_batches(small, large)
    assert mixed.edges_per_seq.max() > 4096 and mixed.num_edges / mixed.B <= 2048
    cases = [wl.make_batch("monophone", B=8, T=200, scale=0.3), wl.make_batch("ctc_tiny"), mixed]
    # The first call on a device is the set-up call: the CUDA module with the fixed array gets
    # loaded and the array's address is looked up.  Device memory is compared around later calls.
    b0 = cases[1]
    fsa0, sl0 = wl.to_torch(b0, cuda)
    assert _noalloc(lib, wl.make_scores(b0, cuda), fsa0, sl0)[0] == 0
    torch.cuda.synchronize()
    for b in cases:  # calls in a row; each finds the previous call's data in the array
        am = wl.make_scores(b, cuda)
        fsa, sl = wl.to_torch(b, cuda)
        bufs = _outputs(am)  # the caller's output buffers exist before the call
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info()[0]
        rc, out, sums, loss2 = _noalloc(lib, am, fsa, sl, bufs)
        torch.cuda.synchronize()
        assert rc == 0
        # the call itself takes no device memory
        assert torch.cuda.mem_get_info()[0] == free_before
        ref_out, ref_sums = m.core.fbw(am, fsa[1], fsa[2], fsa[3], sl, int(fsa[0]), m.core.DebugOptions())
        assert torch.equal(sums == 0, ref_sums == 0)
        assert torch.equal(torch.isinf(out), torch.isinf(ref_out))
        valid = ref_sums != 0
        assert float(((sums - ref_sums).abs()[valid] / ref_sums.abs()[valid]).max()) <= LOSS_RTOL
        assert float((torch.exp(-out.double()) - torch.exp(-ref_out.double())).abs().max()) <= POST_ATOL
        assert abs(float(loss2[0]) - float(ref_sums.double().sum())) <= 1e-5 * float(ref_sums.double().sum())
        # and against the truth: per-frame sums to 1e-5, posteriors to the fp32 rounding of the scores
        post, _, loss, pattern_ok = truth_distances(b, am, [out], [sums], np.arange(b.B))
        assert pattern_ok and loss.max() <= LOSS_RTOL
        assert post.max() <= 4 * max(POST_ATOL, 64 * float(sums.abs().max()) * 2.0 ** -23)


def test_noalloc_entry_rejects_what_does_not_fit(cuda):
    lib = ctypes.CDLL(LIB)
    lib.fbw_b200_fbw_noalloc.restype = ctypes.c_int
    lib.fbw_b200_status_string.restype = ctypes.c_char_p
    # a call whose scratch cannot fit the 64 MiB array: many frames times many states
    b = wl.make_batch("triphone", B=16, T=1500, F=64)
    am = wl.make_scores(b, cuda)
    fsa, sl = wl.to_torch(b, cuda)
    rc, _, _, _ = _noalloc(lib, am, fsa, sl)
    assert rc == 5 and b"capacity" in lib.fbw_b200_status_string(rc)
    # a call above the size at which the op switches to its multi-stream pipeline
    big = torch.zeros((1000, 16, 7000), dtype=torch.float32, device=cuda)
    rc, _, _, _ = _noalloc(lib, big, fsa, sl)
    assert rc == 5
