"""GPU tests of the interface rows around the op: the (T,B) index-mask form of the lengths, the
reference-named import paths, and the ctypes recipe of INTEGRATION.md run as written there."""
import os
import re
import subprocess
import sys

import numpy as np
import pytest
import torch

from i6_native_ops_b200 import workloads as wl

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LIB = os.path.join(ROOT, "i6_native_ops_b200", "libfbw_b200.so")


def test_index_mask_gives_the_same_result_as_lengths(cuda):
    """`seq_lens` may be a (T,B) index mask (the calling convention of the older op this one
    descends from): lengths are the column sums."""
    import i6_native_ops_b200.fast_viterbi as v
    import i6_native_ops_b200.fbw as m

    b = wl.make_batch("monophone", B=6, T=180, scale=0.3)
    am = wl.make_scores(b, cuda)
    fsa, sl = wl.to_torch(b, cuda)
    mask = (torch.arange(b.T, device=cuda)[:, None] < sl[None, :]).to(torch.float32)  # (T,B)
    lp1 = (-am).transpose(0, 1).contiguous().requires_grad_(True)
    lp2 = lp1.detach().clone().requires_grad_(True)
    l1 = m.fbw_loss(lp1, fsa, sl)
    l2 = m.fbw_loss(lp2, fsa, mask)
    l1.sum().backward()
    l2.sum().backward()
    assert torch.equal(l1, l2) and torch.equal(lp1.grad, lp2.grad)
    l3 = m.fbw_loss_fused(lp1.detach(), fsa, mask.to(torch.int32))
    assert torch.equal(l1, l3)
    a1, s1 = v.align_viterbi(lp1.detach(), fsa, sl)
    a2, s2 = v.align_viterbi(lp1.detach(), fsa, mask)
    assert torch.equal(a1, a2) and torch.equal(s1, s2)
    with pytest.raises(RuntimeError):
        m.fbw_loss(lp1.detach(), fsa, mask[:-1])


def test_reference_import_paths(cuda):
    """`from i6_native_ops.fbw import fbw_loss` and `from i6_native_ops.fast_viterbi import
    align_viterbi` resolve to this library; the bodies of the reference's two unit tests
    (test/fbw.py:8-64, test/fast_viterbi.py:9-42) pass through those names."""
    import i6_native_ops_b200.compat as compat

    compat.install()
    from i6_native_ops.fast_viterbi import align_viterbi
    from i6_native_ops.fbw import fbw_loss

    probs = torch.tensor([[0.9, 0.1], [0.9, 0.1], [0.4, 0.6], [0.1, 0.9], [0.1, 0.9]], device=cuda)
    log_probs = probs.unsqueeze(0).log().requires_grad_(True)
    edges = torch.tensor([[0, 0, 0, 0], [0, 1, 0, 0], [1, 1, 1, 0]], device=cuda,
                         dtype=torch.int32).transpose(0, 1).contiguous()
    weights = torch.tensor([1, 1, 1], device=cuda, dtype=torch.float32)
    start_end = torch.tensor([[0], [1]], dtype=torch.int32, device=cuda)
    seq_lens = torch.tensor([5], dtype=torch.int32, device=cuda)
    fsa = (2, edges, weights, start_end)
    fbw_loss(log_probs, fsa, seq_lens).sum().backward()
    assert torch.isclose(log_probs.grad.sum(-1).neg(), torch.ones(1, 5, device=cuda)).all()
    output, scores = align_viterbi(log_probs.detach(), fsa, seq_lens)
    assert output[0].tolist() == [0, 0, 1, 1, 1]


@pytest.mark.parametrize("test_file", ["fbw.py", "fast_viterbi.py"])
def test_reference_test_files_run_unmodified(cuda, test_file):
    """Where a checkout of the reference is present ($I6_NATIVE_OPS_REFERENCE), its own test files
    run unmodified against this library through the import-path shim."""
    import i6_native_ops_b200.compat as compat

    ref = os.environ.get("I6_NATIVE_OPS_REFERENCE", "")
    path = os.path.join(ref, "test", test_file)
    if not ref or not os.path.isfile(path):
        pytest.skip("no reference checkout on this machine")
    env = dict(os.environ, PYTHONPATH=os.pathsep.join([compat.path(), ROOT, os.environ.get("PYTHONPATH", "")]))
    r = subprocess.run([sys.executable, "-m", "unittest", path], env=env, capture_output=True, text=True,
                       timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]


def test_ctypes_recipe_of_the_integration_notes(cuda):
    """The ctypes binding shown in INTEGRATION.md (section 3: prepare -> plan_summary -> run with
    caller-owned buffers) is executed as written and compared with the extension's result."""
    import i6_native_ops_b200.fbw as m

    text = open(os.path.join(ROOT, "INTEGRATION.md")).read()
    section = text[text.index("## 3."):]
    code = re.search(r"```python\n(.*?)```", section, flags=re.S).group(1)
    assert 'ctypes.CDLL("libfbw_b200.so")' in code
    scope = {}
    exec(code.replace('"libfbw_b200.so"', repr(LIB)), scope)  # only the library's location is filled in
    for name, kw in [("ctc_tiny", dict()), ("monophone", dict(B=8, T=200, scale=0.3))]:
        b = wl.make_batch(name, **kw)
        am = wl.make_scores(b, cuda)
        fsa, sl = wl.to_torch(b, cuda)
        out, sums = scope["fbw"](am, fsa[1], fsa[2], fsa[3], sl, int(fsa[0]))
        torch.cuda.synchronize()
        ref_out, ref_sums = m.core.fbw(am, fsa[1], fsa[2], fsa[3], sl, int(fsa[0]), m.core.DebugOptions())
        assert torch.equal(sums, ref_sums) and torch.equal(out, ref_out)
