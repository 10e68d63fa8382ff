"""Run the op a few times on one synthetic workload: the command to put under a profiler.

    python -m i6_native_ops_b200.profile_call --workload lattice --seqs 8 --calls 2 [--op viterbi] [--timeline]

Builds the workload's automata and scores on cuda:0 (``workloads.make_batch`` / ``make_scores``), then
calls ``core.fbw`` (or ``core.fast_viterbi``) ``--calls`` times and synchronises.  Nothing is timed or
checked here; ``bench.py`` measures and the tests check.  ``--timeline`` records the last call with
torch's profiler (CUPTI) and prints every kernel's start, duration and stream in microseconds, which
shows how the stages of a call overlap.  Environment knobs of the library (``FBW_B200_*``) apply as usual.
"""
from __future__ import annotations

import argparse


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__.splitlines()[0])
    ap.add_argument("--workload", default="triphone")
    ap.add_argument("--seqs", type=int, default=None, help="sequences (default: the workload's batch size)")
    ap.add_argument("--calls", type=int, default=2)
    ap.add_argument("--scale", type=float, default=1.0, help="shrink automata and lengths")
    ap.add_argument("--op", default="fbw", choices=["fbw", "viterbi"])
    ap.add_argument("--timeline", action="store_true", help="print the kernel timeline of the last call")
    args = ap.parse_args()

    import torch

    from . import workloads as wl

    dev = torch.device("cuda:0")
    batch = wl.make_batch(args.workload, B=args.seqs, scale=args.scale)
    am = wl.make_scores(batch, dev)
    fsa, seq_lens = wl.to_torch(batch, dev)
    torch.cuda.synchronize()
    if args.op == "fbw":
        from .fbw import core

        opts = core.DebugOptions()

        def call():
            return core.fbw(am, fsa[1], fsa[2], fsa[3], seq_lens, int(fsa[0]), opts)
    else:
        from .fast_viterbi import core

        am.neg_()

        def call():
            return core.fast_viterbi(am, fsa[1], fsa[2], fsa[3], seq_lens, int(fsa[0]))

    for _ in range(args.calls - (1 if args.timeline else 0)):
        out = call()
    torch.cuda.synchronize()
    if args.timeline:
        import json
        import os
        import tempfile

        from torch.profiler import ProfilerActivity, profile

        with profile(activities=[ProfilerActivity.CUDA]) as prof:
            out = call()
            torch.cuda.synchronize()
        path = os.path.join(tempfile.mkdtemp(), "trace.json")
        prof.export_chrome_trace(path)
        events = [e for e in json.load(open(path))["traceEvents"]
                  if e.get("cat") in ("kernel", "gpu_memset", "gpu_memcpy")]
        os.remove(path)
        events.sort(key=lambda e: e["ts"])
        t0 = events[0]["ts"]
        print("start_us   dur_us  stream  kernel")
        for e in events:
            name = e["name"].replace("void ", "").replace("(anonymous namespace)::", "").split("(")[0][:48]
            print(f"{e['ts'] - t0:8.1f} {e['dur']:8.1f}  {str(e['args'].get('stream', '?')):>6}  {name}")
        print(f"call: {events[-1]['ts'] + events[-1]['dur'] - t0:.1f} us from the first kernel's start to the last one's end")
    print(f"{args.op} x{args.calls} on {args.workload}: T={batch.T} B={batch.B} F={batch.F} "
          f"E={batch.num_edges} S={batch.num_states}; out[0] finite entries {int(out[0].isfinite().sum())}")


if __name__ == "__main__":
    main()
