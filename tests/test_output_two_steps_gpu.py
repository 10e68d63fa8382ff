"""The two ways the (T,B,F) output is written give the same bits.

Large calls with sparse rows write the +inf background while the sweeps run and put the posteriors
into it afterwards; the other calls compose every row once, after the posteriors.  The library picks
one per call; ``FBW_B200_OUTPUT=expand`` / ``patch`` fixes the choice for a process, which is what the
child processes here do.  Compared: the bit patterns of ``out`` and ``sums`` (as exact integer sums),
on calls large enough to run as groups of sequences: rows whose length is not a multiple of four words
(12001 classes), sequences shorter than T, an invalid length, and the BPE-CTC shape with several sweep
CTAs per SM; and the wrapper-fused form of the op on the same cases (gradient output).
"""
import json
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

CHILD = r"""
import json, sys
import numpy as np, torch
from i6_native_ops_b200 import workloads as wl
from i6_native_ops_b200.fbw import core
dev = torch.device("cuda:0")
res = []
for name, kw, bad in json.loads(sys.argv[1]):
    b = wl.make_batch(name, **kw)
    if bad:
        b.seq_lens[bad] = 0  # an invalid length: that sequence's rows are +inf, its sums 0
    am = wl.make_scores(b, dev)
    fsa, sl = wl.to_torch(b, dev)
    out, sums = core.fbw(am, fsa[1], fsa[2], fsa[3], sl, int(fsa[0]), core.DebugOptions())
    torch.cuda.synchronize()
    t = torch.arange(b.T, device=dev)[:, None]
    pad = t >= sl.to(dev)[None, :].clamp(min=0)
    # the wrapper-fused form of the op (gradient output: background 0, rows ordered (sequence, frame))
    lp = (-am).transpose(0, 1).contiguous()
    grad, _ = core.fbw_fused(lp, fsa[1], fsa[2], fsa[3], sl, int(fsa[0]))
    torch.cuda.synchronize()
    fused = int(grad.view(torch.int32).to(torch.int64).sum().item())
    del lp, grad
    res.append(dict(out=int(out.view(torch.int32).to(torch.int64).sum().item()), fused=fused,
                    sums=int(sums.view(torch.int32).to(torch.int64).sum().item()),
                    finite=int(torch.isfinite(out).sum().item()),
                    pad_ok=bool(torch.isinf(out[pad]).all().item()) and bool((sums[pad] == 0).all().item()),
                    launches=int(core.launch_count()) if hasattr(core, "launch_count") else -1))
    del out, sums, am
print("RESULT " + json.dumps(res))
"""

CASES = [["triphone", {}, 0], ["triphone", {"B": 66, "T": 333}, 5], ["bpe_ctc", {"B": 128}, 0],
         ["triphone", {"B": 9}, 3]]


def run_child(mode):
    env = dict(os.environ, FBW_B200_OUTPUT=mode, PYTHONPATH=ROOT + os.pathsep + os.environ.get("PYTHONPATH", ""))
    r = subprocess.run([sys.executable, "-c", CHILD, json.dumps(CASES)], env=env, capture_output=True, text=True,
                       timeout=900, cwd=ROOT)
    lines = [l for l in r.stdout.splitlines() if l.startswith("RESULT ")]
    assert r.returncode == 0 and lines, r.stderr[-2000:]
    return json.loads(lines[0][7:])


def test_background_then_posteriors_equals_one_pass(cuda):
    one_pass = run_child("expand")
    two_steps = run_child("patch")
    default = run_child("")
    for case, a, b, c in zip(CASES, one_pass, two_steps, default):
        assert a["pad_ok"] and b["pad_ok"] and c["pad_ok"], case
        assert a["finite"] > 0, case
        for key in ("out", "sums", "finite", "fused"):
            assert a[key] == b[key] == c[key], (case, key, a, b, c)
