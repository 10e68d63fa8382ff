"""Generate the golden fixtures of tests/golden/ by running the REFERENCE fbw op.

Needs a CUDA device and the reference op built into oracle/_ref/ (oracle/build_ref.py builds it
from the reference's own sources).  For each small seeded case it stores the inputs and the
reference's two outputs (fbw_op.cu:392) in one .npz.  The oracle and the CUDA path are both
tested against these files.

``--viterbi`` instead reads the inputs of the existing fixtures and stores, per case, what the
REFERENCE fast_viterbi op (core.cu:274) returns for the positive log scores ``-am`` in
``viterbi_<case>.npz`` (alignment (T,B) int32, scores (B,) float32); the fbw fixtures stay untouched.

Usage:  python tests/golden/make_golden.py [--viterbi] [output_dir]
"""
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "oracle"))

import build_ref  # noqa: E402
from i6_native_ops_b200 import workloads as wl  # noqa: E402

CASES = {
    "ctc_tiny": ("ctc_tiny", dict()),
    "monophone_small": ("monophone", dict(B=4, T=160, scale=0.3)),
    "triphone_small": ("triphone", dict(B=3, T=120, F=301, scale=0.08)),
    "lattice_small": ("lattice", dict(B=3, F=37, T=120, scale=0.05)),
}


def unit_case():
    probs = np.array([[0.9, 0.1], [0.9, 0.1], [0.4, 0.6], [0.1, 0.9], [0.1, 0.9]], dtype=np.float32)
    return dict(am=-np.log(probs)[:, None, :],
                edges=np.array([[0, 0, 0, 0], [0, 1, 0, 0], [1, 1, 1, 0]], dtype=np.int32).T.copy(),
                weights=np.ones(3, dtype=np.float32), start_end=np.array([[0], [1]], dtype=np.int32),
                seq_lens=np.array([5], dtype=np.int32), num_states=2)


def main(out_dir):
    ref = build_ref.load_ref()
    if ref is None:
        raise SystemExit("reference op not built: run oracle/build_ref.py where the reference is mounted")
    dev = torch.device("cuda:0")
    torch.cuda.set_device(0)  # the reference has no device guard
    os.makedirs(out_dir, exist_ok=True)
    cases = {"reference_unit_test": unit_case()}
    for key, (name, kw) in CASES.items():
        b = wl.make_batch(name, **kw)
        cases[key] = dict(am=wl.make_scores(b, dev).cpu().numpy(), edges=b.edges, weights=b.weights,
                          start_end=b.start_end, seq_lens=b.seq_lens, num_states=b.num_states)
    for key, c in cases.items():
        t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(dev)
        out, sums = ref.fbw(t(c["am"]), t(c["edges"]), t(c["weights"]), t(c["start_end"]),
                            t(c["seq_lens"]), int(c["num_states"]), ref.DebugOptions())
        torch.cuda.synchronize()
        np.savez_compressed(os.path.join(out_dir, key + ".npz"), ref_out=out.cpu().numpy(),
                            ref_sums=sums.cpu().numpy(), **c)
        print(key, c["am"].shape, float(sums.max()))


def main_viterbi(out_dir):
    ref = build_ref.load_viterbi_ref()
    if ref is None:
        raise SystemExit("reference fast_viterbi op not built: run oracle/build_ref.py where the reference is mounted")
    dev = torch.device("cuda:0")
    torch.cuda.set_device(0)
    os.makedirs(out_dir, exist_ok=True)
    for key in ["reference_unit_test"] + list(CASES):
        c = np.load(os.path.join(HERE, key + ".npz"))
        t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(dev)
        alignment, scores = ref.fast_viterbi(t(-c["am"]), t(c["edges"]), t(c["weights"]), t(c["start_end"]),
                                             t(c["seq_lens"]), int(c["num_states"]))
        torch.cuda.synchronize()
        np.savez_compressed(os.path.join(out_dir, "viterbi_" + key + ".npz"),
                            ref_alignment=alignment.cpu().numpy(), ref_scores=scores.cpu().numpy())
        print(key, alignment.shape, scores.cpu().numpy()[:4])


if __name__ == "__main__":
    args = [a for a in sys.argv[1:] if a != "--viterbi"]
    (main_viterbi if "--viterbi" in sys.argv else main)(args[0] if args else HERE)
