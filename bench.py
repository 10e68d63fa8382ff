#!/usr/bin/env python
"""Benchmark of the fbw (fast Baum-Welch) hot path.

  python bench.py --gpus N --steps K --warmup W [--impl reference] [--workload triphone]

One step = one op call (automaton preparation + gather + both sweeps + posteriors + output) on
one batch of synthetic input.  Default workload: the triphone configuration (B=64 sequences per
GPU, T=1500, F=12001, fp32), the one the headline target is quoted on.  With N GPUs every rank
owns 64 sequences of a 64*N batch (length-balanced partition by sequence, no data-path
collective; one all-reduce of two loss scalars per step), i.e. weak scaling.

Printed by rank 0: ONE JSON line.
  value      frames/s (T*B per call, summed over ranks) with inputs resident in HBM
  e2e        the same through the op with HOST buffers, inputs AND results in pinned host memory: the
             op's gather reads the score sectors it needs in place over the bus, the (T,B,F) result is
             copied device -> host, the automata host -> device and the (T,B) sums and the loss device
             -> host, all inside the timing.  Beside it: e2e_copy (whole tensors copied both ways around
             the op), e2e_in_place_out (the output pass writes the result straight into host memory)
             and e2e_out_on_device (result left on the device); each leg lists every rank's time and
             bus throughput
  roofline   whole-call algorithmic bytes / measured call time against the measured HBM peak
  strong     strong scaling of the two configurations that are sharded over GPUs: a fixed global batch
             (lattice B=512, bpe_ctc B=256) partitioned by sequence over the N ranks; step time is the
             slowest rank's, every rank's time and the partition's cost imbalance are listed
  reference_gpu_op  the reference's own CUDA op on the same tensors and GPU (N=1 only; never inside a
             timed region of this library)
  cpu_baseline  the CPU oracle (a C/OpenMP port of the reference's arithmetic; the reference has no
             CPU implementation of fbw) on a bounded sample of the same workload

--impl reference times that CPU port alone (the reference's op is CUDA-only and has no CPU path).

--op viterbi benchmarks the best-path alignment (fast_viterbi) on the same workloads instead: one
step = automaton preparation + gather + the per-sequence Viterbi kernel (all frames and the
back-trace); value = frames/s, e2e with host buffers, cpu_baseline = the sequential C oracle.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import numpy as np  # noqa: E402

SEQS_PER_GPU = {"triphone": 64, "bpe_ctc": 256, "monophone": 32, "ctc_tiny": 4, "lattice": 64}
CPU_SAMPLE_SEQS = None  # None: the full per-GPU batch of the workload

# dram__bytes_read.sum + dram__bytes_write.sum over all kernels of ONE op call, from an ncu capture
# of exactly that workload and per-GPU batch size; other sizes report no traffic figure.
MEASURED_TRAFFIC = {("triphone", 64): 9.106e9}  # (workload, sequences per GPU) -> bytes per call


def peaks():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons of one GPU with nvidia-smi.  start() launches the
    sampler and waits for its first line (nvidia-smi's start-up stalls CUDA calls for a while, so
    it has to be over before anything is timed); window() marks the timed region; summary()
    reports the samples that fell inside it (or the nearest ones if the region was shorter than
    one sampling period)."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int, period_ms: int = 25):
        self.index = index
        self.period_ms = period_ms
        self.proc = None
        self.lines = []  # (arrival time, text)
        self.t0 = self.t1 = None

    def start(self, timeout: float = 20.0):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}",
                 "--format=csv,noheader,nounits", "-lms", str(self.period_ms)],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return self
        threading.Thread(target=self._read, daemon=True).start()
        end = time.time() + timeout
        while not self.lines and time.time() < end:
            time.sleep(0.05)
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append((time.time(), line.strip()))

    def window(self, t0: float, t1: float):
        self.t0, self.t1 = t0, t1

    def stop(self):
        if self.proc is not None:
            time.sleep(2.5 * self.period_ms / 1000.0)
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self):
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        rows = []
        for ts, ln in self.lines:
            parts = [p.strip() for p in ln.split(",")]
            if len(parts) < 6:
                continue
            try:
                rows.append((ts, float(parts[0]), float(parts[1]),
                             [n for n, v in zip(names, parts[2:6]) if v.lower().startswith("active")]))
            except ValueError:
                continue
        if not rows:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        pad = self.period_ms / 1000.0
        inside = [r for r in rows if self.t0 is not None and self.t0 <= r[0] <= self.t1 + pad]
        if not inside and self.t0 is not None:  # region shorter than a period: nearest sample
            inside = [min(rows, key=lambda r: abs(r[0] - self.t1))]
        use = inside or rows
        reasons = sorted({n for r in use for n in r[3]})
        return {"sm_mhz": float(np.median([r[1] for r in use])), "sm_max_mhz": float(max(r[2] for r in use)),
                "reasons": reasons, "samples": len(use)}


def cpu_baseline_pass(workload: str, threads: int, passes: int, warm: int = 1, gpus: int = 1,
                      per_gpu: int = None):
    """Times the CPU oracle (test infrastructure) on a bounded sample: one per-GPU batch of the
    workload at full T and F -- with several GPUs the shard rank 0 gets -- a few passes."""
    import oracle
    from i6_native_ops_b200 import sharding
    from i6_native_ops_b200 import workloads as wl

    per_gpu = per_gpu or CPU_SAMPLE_SEQS or SEQS_PER_GPU[workload]
    if gpus > 1:
        full = wl.make_batch(workload, B=per_gpu * gpus)
        costs = sharding.sequence_costs(full.states_per_seq, full.edges_per_seq, full.seq_lens, full.T, full.F)
        batch = wl.make_batch(workload, seq_ids=sharding.partition(costs, gpus)[0], T=full.T)
    else:
        batch = wl.make_batch(workload, B=per_gpu)
    am = wl.make_scores(batch, "cpu").numpy()
    times = []
    for i in range(warm + passes):
        t0 = time.perf_counter()
        oracle.fbw_oracle(am, batch.edges, batch.weights, batch.start_end, batch.seq_lens,
                          batch.num_states, "f32", nthreads=threads)
        dt = time.perf_counter() - t0
        if i >= warm:
            times.append(dt)
    frames = batch.T * batch.B
    sample = (f"{batch.B} sequences of {workload} at full T={batch.T}, F={batch.F}; fp32 CPU port of the "
              f"reference arithmetic, OpenMP over sequences, {passes} passes")
    cpu_baseline_pass.last_batch = batch
    return frames, times, sample


def run_reference_arm(args):
    """The reference arm: the reference's fbw has no CPU implementation (its binding rejects CPU
    tensors), so this times the C/OpenMP port of its arithmetic on the host cores."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    frames, times, sample = cpu_baseline_pass(args.workload, threads, args.steps, max(1, min(args.warmup, 2)),
                                              gpus=max(1, args.gpus), per_gpu=args.seqs_per_gpu)
    total = float(sum(times))
    value = frames * len(times) / total
    line = {
        "impl": "reference", "metric": "fbw fwd+bwd frames/s", "value": value, "unit": "frames/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": 1e3 * total / len(times), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": config_of(args.workload, cpu_baseline_pass.last_batch,
                            (args.seqs_per_gpu or SEQS_PER_GPU[args.workload]) * max(1, args.gpus)),
        "cpu_baseline": {"value": value, "unit": "frames/s", "cores": threads, "kind": "port",
                         "sample": sample},
        "e2e": {"value": value, "unit": "frames/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def run_viterbi(args):
    """--op viterbi: the best-path alignment on the same synthetic workloads (positive log scores =
    minus the fbw scores).  Sequences are independent: with N GPUs every rank aligns its own
    sequences and nothing crosses GPUs."""
    import oracle  # noqa: F401  (only the cpu_baseline leg below calls it)
    from i6_native_ops_b200 import workloads as wl

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    per_gpu = args.seqs_per_gpu or SEQS_PER_GPU[args.workload]

    def cpu_pass(passes):
        batch = wl.make_batch(args.workload, B=per_gpu)
        am = -wl.make_scores(batch, "cpu").numpy()
        times = []
        for i in range(passes + 1):
            t0 = time.perf_counter()
            oracle.viterbi_oracle(am, batch.edges, batch.weights, batch.start_end, batch.seq_lens,
                                  batch.num_states)
            if i:
                times.append(time.perf_counter() - t0)
        sample = (f"{batch.B} sequences of {args.workload} at full T={batch.T}, F={batch.F}; sequential C "
                  f"port of the reference arithmetic, {passes} passes")
        return batch.T * batch.B * len(times) / float(sum(times)), sample

    if args.impl == "reference":  # the reference op is CUDA-only: its arithmetic on one host core
        if rank == 0:
            value, sample = cpu_pass(max(1, args.steps))
            print(json.dumps({
                "impl": "reference", "metric": "viterbi frames/s", "value": value, "unit": "frames/s",
                "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "higher_is_better": True,
                "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
                "config": {"workload": args.workload, "op": "viterbi", "sample": sample},
                "cpu_baseline": {"value": value, "unit": "frames/s", "cores": 1, "kind": "port", "sample": sample},
                "e2e": {"value": value, "unit": "frames/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
                "gpu_launches": 0}), flush=True)
        return

    import torch
    import torch.distributed as dist

    from i6_native_ops_b200 import sharding
    from i6_native_ops_b200.fast_viterbi import core

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback)")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
    global_b = per_gpu * world
    if world > 1:
        full = wl.make_batch(args.workload, B=global_b)
        costs = sharding.sequence_costs(full.states_per_seq, full.edges_per_seq, full.seq_lens, full.T, full.F)
        batch = wl.make_batch(args.workload, seq_ids=sharding.partition(costs, world)[rank], T=full.T)
    else:
        batch = wl.make_batch(args.workload, B=global_b)
    am = wl.make_scores(batch, dev).neg_()
    fsa, seq_lens = wl.to_torch(batch, dev)
    S = int(fsa[0])
    frames, alg_bytes = batch.T * batch.B, batch.viterbi_algorithmic_bytes()
    am_bytes = am.numel() * 4
    flush = torch.empty(64 * 1024 * 1024, dtype=torch.float32, device=dev) if am_bytes <= 2 * 126e6 else None

    def step():
        return core.fast_viterbi(am, fsa[1], fsa[2], fsa[3], seq_lens, S)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    clk = ClockSampler(local_rank).start()
    for _ in range(args.warmup):
        step()
    barrier()
    launches0 = core.launch_count()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    w0 = time.time()
    ms = 0.0
    if flush is None:
        ev0.record()
        for _ in range(args.steps):
            step()
        ev1.record()
        torch.cuda.synchronize()
        ms = ev0.elapsed_time(ev1)
    else:
        for _ in range(args.steps):
            flush.fill_(1.0)
            ev0.record()
            step()
            ev1.record()
            torch.cuda.synchronize()
            ms += ev0.elapsed_time(ev1)
    barrier()
    clk.window(w0, time.time())
    clk.stop()
    launches = core.launch_count() - launches0
    t_ms = torch.tensor([ms], device=dev, dtype=torch.float64)
    tot = torch.tensor([float(frames)], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t_ms, op=dist.ReduceOp.MAX)
        dist.all_reduce(tot, op=dist.ReduceOp.SUM)
    ms_per_step = float(t_ms.item()) / args.steps
    value = float(tot.item()) / (ms_per_step * 1e-3)

    e2e = None
    if not args.no_e2e:
        am_h = torch.empty(am.shape, dtype=am.dtype, pin_memory=True)
        am_h.copy_(am)
        host_fsa = [t.cpu().pin_memory() for t in (fsa[1], fsa[2], fsa[3], seq_lens)]
        align_h = torch.empty((batch.T, batch.B), dtype=torch.int32, pin_memory=True)
        del am
        am_d = torch.empty(am_h.shape, dtype=am_h.dtype, device=dev) if args.e2e_copy else None
        fsa_bytes = sum(t.numel() * t.element_size() for t in host_fsa)
        h2d = (am_h.numel() * 4 if args.e2e_copy else batch.score_sector_bytes()) + fsa_bytes
        d2h = align_h.numel() * 4 + 4 * batch.B

        def e2e_step():
            e_, w_, se_, sl_ = [t.to(dev, non_blocking=True) for t in host_fsa]
            if args.e2e_copy:
                am_d.copy_(am_h, non_blocking=True)
                alignment, scores = core.fast_viterbi(am_d, e_, w_, se_, sl_, S)
            else:  # the gather reads the scores it needs in place from pinned host memory
                alignment, scores = core.fast_viterbi_host_scores(am_h, e_, w_, se_, sl_, S)
            align_h.copy_(alignment, non_blocking=True)
            return scores.cpu()  # device -> host read of the scores; synchronises

        n_e2e = max(3, min(args.steps, 10))
        for _ in range(2):
            e2e_step()
        barrier()
        ev0.record()
        for _ in range(n_e2e):
            e2e_step()
        ev1.record()
        barrier()
        t_e = torch.tensor([ev0.elapsed_time(ev1) / n_e2e], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(t_e, op=dist.ReduceOp.MAX)
        e2e = {"value": float(tot.item()) / (float(t_e.item()) * 1e-3), "unit": "frames/s",
               "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(d2h),
               "ms_per_step": float(t_e.item()), "steps": n_e2e,
               "path": ("scores copied to the device, then the op" if args.e2e_copy else
                        "scores read in place from pinned host memory by the op's gather "
                        f"(32-byte sectors; the whole tensor is {am_h.numel() * 4} bytes)")}

    if rank == 0:
        peak, peak_kind = peaks()
        achieved = alg_bytes / (ms_per_step * 1e-3) / 1e9
        line = {
            "metric": "viterbi frames/s", "value": value, "unit": "frames/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
            "data": "synthetic",
            "config": {"workload": args.workload, "op": "viterbi", "T": batch.T, "B_per_gpu": batch.B,
                       "B_global": global_b, "F": batch.F, "edges_per_gpu": batch.num_edges,
                       "states_per_gpu": batch.num_states, "partition": "by sequence, length-balanced",
                       "l2": f"inputs ({am_bytes / 1e9:.2f} GB of scores per call) exceed the 126 MB L2; no flush"
                             if am_bytes > 2 * 126e6 else "an L2 flush (256 MB write) runs between timed steps",
                       "step": "prepare + gather + Viterbi kernel per call (automata re-sorted every step)"},
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                         "frac": achieved / peak, "traffic": None, "peak_kind": peak_kind,
                         "algorithmic_bytes_per_call": int(alg_bytes),
                         "scope": "whole op call (all kernels), per GPU; the frame recursion is a "
                                  "dependent chain, not a bandwidth-bound pass"},
            "gpu_launches": int(launches),
            "clocks": clk.summary(),
            "e2e": e2e,
        }
        if world == 1 and not args.no_cpu_baseline:
            cvalue, sample = cpu_pass(2)
            line["cpu_baseline"] = {"value": cvalue, "unit": "frames/s", "cores": 1, "kind": "port",
                                    "sample": sample}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def gpu_numa_cpus(index: int):
    """CPUs local to GPU `index` (its PCI device's local_cpulist in sysfs), or None if not exposed."""
    try:
        import torch

        pr = torch.cuda.get_device_properties(index)
        bus = f"{pr.pci_domain_id:04x}:{pr.pci_bus_id:02x}:{pr.pci_device_id:02x}.0"
        with open(f"/sys/bus/pci/devices/{bus}/local_cpulist") as f:
            text = f.read().strip()
        with open(f"/sys/bus/pci/devices/{bus}/numa_node") as f:
            node = int(f.read().strip())
        cpus = set()
        for part in text.split(","):
            lo, _, hi = part.partition("-")
            cpus.update(range(int(lo), int(hi or lo) + 1))
        return node, sorted(cpus)
    except Exception:
        return None


def config_of(workload, batch, global_b):
    """The `config` object of a bench line; the reference arm prints the same keys and values."""
    am_bytes = 4 * batch.T * batch.B * batch.F
    return {"workload": workload, "T": int(batch.T), "B_per_gpu": int(batch.B), "B_global": int(global_b),
            "F": int(batch.F), "edges_per_gpu": int(batch.num_edges), "states_per_gpu": int(batch.num_states),
            "partition": "by sequence, length-balanced",
            "l2": (f"inputs ({am_bytes / 1e9:.2f} GB of scores per call) exceed the 126 MB L2; no flush"
                   if am_bytes > 2 * 126e6 else "an L2 flush (256 MB write) runs between timed steps"),
            "step": "prepare + run per call (automata re-sorted every step)"}


STRONG = {"lattice": 512, "bpe_ctc": 256}  # workload -> fixed global batch of the strong-scaling legs


def strong_leg(name, global_b, world, rank, dev, steps, dist, torch, core, sharding, wl):
    """Strong scaling: a FIXED global batch of `global_b` sequences of workload `name` is partitioned
    by sequence over the ranks (length-balanced), every rank runs the op on its shard, and the step
    time is the slowest rank's.  Returns the report of the leg (identical on every rank)."""
    full = wl.make_batch(name, B=global_b)
    costs = sharding.sequence_costs(full.states_per_seq, full.edges_per_seq, full.seq_lens, full.T, full.F)
    parts = sharding.partition(costs, world)
    loads = np.array([costs[p].sum() for p in parts])
    batch = wl.take_sequences(full, parts[rank])
    am = wl.make_scores(batch, dev)
    fsa, seq_lens = wl.to_torch(batch, dev)
    def op_only():
        plan = core.fbw_prepare(fsa[1], fsa[2], fsa[3], seq_lens, batch.T, batch.F, int(fsa[0]))
        return core.fbw_run(plan, am)

    for _ in range(3):
        sharding.sharded_fbw(am, fsa, seq_lens)
    # this rank's own work, without the collective: shows how well the partition balances the ranks
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        op_only()
    e1.record()
    torch.cuda.synchronize()
    local_ms = e0.elapsed_time(e1) / steps
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(steps + 1)]
    ev[0].record()
    for i in range(steps):
        sharding.sharded_fbw(am, fsa, seq_lens)   # prepare + run + the all-reduce of the loss scalars
        ev[i + 1].record()
    torch.cuda.synchronize()
    mine = ev[0].elapsed_time(ev[steps]) / steps

    def gather(x):
        t = torch.tensor([x], device=dev, dtype=torch.float64)
        if world == 1:
            return [float(x)]
        got = [torch.zeros_like(t) for _ in range(world)]
        dist.all_gather(got, t)
        return [float(g.item()) for g in got]

    rank_ms = gather(mine)
    rank_local_ms = gather(local_ms)
    ms = max(rank_ms)
    alg = full.algorithmic_bytes()
    peak, _ = peaks()
    del am
    torch.cuda.empty_cache()
    return {"B_global": int(global_b), "B_per_rank": [int(len(p)) for p in parts], "T": int(full.T),
            "F": int(full.F), "steps": steps, "ms_per_step": ms, "frames_per_s": full.T * global_b / (ms * 1e-3),
            "rank_ms": rank_ms, "rank_op_ms": rank_local_ms,
            "rank_frames": [int(batch_frames) for batch_frames in
                            [full.seq_lens[p].astype(np.int64).sum() for p in parts]],
            "rank_max_states": [int(full.states_per_seq[p].max()) if len(p) else 0 for p in parts],
            "cost_imbalance": float(loads.max() / loads.mean()),
            "roofline_frac_per_gpu": alg / world / (ms * 1e-3) / 1e9 / peak,
            "scaling": "strong"}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="new", choices=["new", "reference"])
    ap.add_argument("--workload", default="triphone", choices=sorted(SEQS_PER_GPU))
    ap.add_argument("--seqs-per-gpu", type=int, default=None)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-strong", action="store_true", help="skip the strong-scaling legs (lattice, bpe_ctc)")
    ap.add_argument("--no-reference-gpu-op", action="store_true")
    ap.add_argument("--op", default="fbw", choices=["fbw", "viterbi"])
    ap.add_argument("--e2e-copy", action="store_true",
                    help="viterbi e2e leg: copy the whole score tensor to the device first (default: the op "
                         "reads the scores it needs from pinned host memory)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)

    if args.op == "viterbi":
        run_viterbi(args)
        return
    if args.impl == "reference":
        run_reference_arm(args)
        return

    import torch
    import torch.distributed as dist

    from i6_native_ops_b200 import sharding
    from i6_native_ops_b200 import workloads as wl
    from i6_native_ops_b200.fbw import core

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback)")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    # host threads and pinned buffers of a rank on the CPUs next to its GPU, where sysfs tells which
    numa = gpu_numa_cpus(local_rank)
    bound = False
    if numa is not None and numa[1]:
        try:
            allowed = sorted(set(numa[1]) & set(os.sched_getaffinity(0)))
            if allowed:
                os.sched_setaffinity(0, allowed)
                bound = True
        except OSError:
            pass
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)

    # ---- workload: 64*N sequences, partitioned by sequence, each rank builds its own shard ----
    per_gpu = args.seqs_per_gpu or SEQS_PER_GPU[args.workload]
    global_b = per_gpu * world
    if world > 1:
        full = wl.make_batch(args.workload, B=global_b)
        costs = sharding.sequence_costs(full.states_per_seq, full.edges_per_seq, full.seq_lens,
                                        full.T, full.F)
        mine = sharding.partition(costs, world)[rank]
        batch = wl.make_batch(args.workload, seq_ids=mine, T=full.T)
    else:
        batch = wl.make_batch(args.workload, B=global_b)
    am = wl.make_scores(batch, dev)
    fsa, seq_lens = wl.to_torch(batch, dev)
    frames = batch.T * batch.B
    alg_bytes = batch.algorithmic_bytes()
    am_bytes = am.numel() * 4
    flush = torch.empty(64 * 1024 * 1024, dtype=torch.float32, device=dev) if am_bytes <= 2 * 126e6 else None

    def step():
        out, sums, loss2, _ = sharding.sharded_fbw(am, fsa, seq_lens, plan=None)
        return sums, loss2

    def timed_steps(n):
        """n steps; returns device milliseconds.  Small workloads get an L2 flush before each step,
        timed separately per step so that the flush is outside the measured time."""
        if flush is None:
            ev0.record()
            for _ in range(n):
                step()
            ev1.record()
            torch.cuda.synchronize()
            return ev0.elapsed_time(ev1)
        total = 0.0
        for _ in range(n):
            flush.fill_(1.0)
            ev0.record()
            step()
            ev1.record()
            torch.cuda.synchronize()
            total += ev0.elapsed_time(ev1)
        return total

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def gather_ranks(x):
        """One float per rank -> list over ranks (on every rank)."""
        t = torch.tensor([float(x)], device=dev, dtype=torch.float64)
        if world == 1:
            return [float(x)]
        got = [torch.zeros_like(t) for _ in range(world)]
        dist.all_gather(got, t)
        return [float(g.item()) for g in got]

    clk = ClockSampler(local_rank).start()
    for _ in range(args.warmup):
        step()
    barrier()
    launches0 = core.launch_count()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    w0 = time.time()
    ms = timed_steps(args.steps)
    barrier()
    clk.window(w0, time.time())
    clk.stop()
    launches = core.launch_count() - launches0
    t_ms = torch.tensor([ms], device=dev, dtype=torch.float64)
    tot = torch.tensor([float(frames), float(alg_bytes)], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t_ms, op=dist.ReduceOp.MAX)
        dist.all_reduce(tot, op=dist.ReduceOp.SUM)
    ms = float(t_ms.item())
    ms_per_step = ms / args.steps
    total_frames, total_bytes = float(tot[0].item()), float(tot[1].item())
    value = total_frames / (ms_per_step * 1e-3)

    # ---- per-kernel device times of one call on this rank (outside the timed region) ----
    plan = core.fbw_prepare(fsa[1], fsa[2], fsa[3], seq_lens, batch.T, batch.F, fsa[0])
    phase = np.zeros(5)
    reps = 5
    for _ in range(reps):
        _, times = core.fbw_run_phases(plan, am)
        phase += np.array(times)
    phase /= reps
    pe0, pe1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    pe0.record()
    for _ in range(reps):
        core.fbw_prepare(fsa[1], fsa[2], fsa[3], seq_lens, batch.T, batch.F, fsa[0])
    pe1.record()
    torch.cuda.synchronize()
    prep_ms = pe0.elapsed_time(pe1) / reps
    del plan

    # ---- the reference's own GPU op on the same device and inputs (the incumbent; reported, never
    # ---- part of a timed region of this library; oracle/_ref is test infrastructure) ----
    reference_gpu_op = None
    if world == 1 and not args.no_reference_gpu_op:
        try:
            sys.path.insert(0, os.path.join(ROOT, "oracle"))
            import build_ref

            ref = build_ref.load_ref()
            if ref is None:
                reference_gpu_op = {"skipped": "oracle/_ref/fbw_core_ref.so is not built on this machine"}
            elif batch.T * batch.B * batch.F >= 2 ** 32 or batch.B > 1024:
                reference_gpu_op = {"skipped": "the reference op's 32-bit sizes / one-block launches cannot take this batch"}
            else:
                times = []
                for i in range(7):
                    pe0.record()
                    r = ref.fbw(am, fsa[1], fsa[2], fsa[3], seq_lens, int(fsa[0]), ref.DebugOptions())
                    pe1.record()
                    torch.cuda.synchronize()
                    del r
                    if i >= 2:
                        times.append(pe0.elapsed_time(pe1))
                med = float(np.median(times))
                reference_gpu_op = {"ms_per_call": med, "frames_per_s": frames / (med * 1e-3), "calls": len(times),
                                    "what": "median of the unmodified reference op (i6_native_ops/fbw, built "
                                            "from its own sources for sm_100a) on the same tensors, same GPU"}
        except Exception as e:  # a report line, not the product: never fail the bench over it
            reference_gpu_op = {"skipped": f"{type(e).__name__}: {e}"[:200]}

    # ---- end to end through the op with host buffers ----
    e2e = e2e_copy = e2e_dev_out = e2e_in_place = None
    if not args.no_e2e:
        am_h = torch.empty(am.shape, dtype=am.dtype, pin_memory=True)
        am_h.copy_(am)
        host_fsa = [t.cpu().pin_memory() for t in (fsa[1], fsa[2], fsa[3], seq_lens)]
        sums_h = torch.empty((batch.T, batch.B), dtype=torch.float32, pin_memory=True)
        out_h = torch.empty(am.shape, dtype=am.dtype, pin_memory=True)
        del am
        torch.cuda.empty_cache()
        fsa_bytes = sum(t.numel() * t.element_size() for t in host_fsa)
        out_bytes = out_h.numel() * 4
        small_d2h = sums_h.numel() * 4 + 8

        def finish(sums, loss2):
            sums_h.copy_(sums, non_blocking=True)
            return loss2.cpu()  # device -> host read of the reduced loss; synchronises

        def step_host_to_host():
            # scores read in place from pinned host memory by the gather (no copy of the tensor to the
            # device); of the (T,B,F) result only the class posteriors cross the bus, and the library's
            # host threads write the rows into pinned host memory while the device goes on (rows that
            # are not sparse would be produced on the device and copied out piece by piece instead)
            e_, w_, se_, sl_ = [t.to(dev, non_blocking=True) for t in host_fsa]
            _, sums, loss2 = sharding.sharded_fbw_host_scores(am_h, (fsa[0], e_, w_, se_), sl_, out=out_h)
            return finish(sums, loss2)

        def step_in_place():
            # as above, but the op's output pass writes the result straight into pinned host memory
            # (no device copy of the result exists; saves its HBM, costs bus efficiency)
            e_, w_, se_, sl_ = [t.to(dev, non_blocking=True) for t in host_fsa]
            _, sums, loss2 = sharding.sharded_fbw_host_scores(am_h, (fsa[0], e_, w_, se_), sl_, out=out_h,
                                                              staged=False)
            return finish(sums, loss2)

        def step_copy():
            # the classic route: whole score tensor host -> device, op, whole result device -> host
            e_, w_, se_, sl_ = [t.to(dev, non_blocking=True) for t in host_fsa]
            am_d = am_h.to(dev, non_blocking=True)
            out, sums, loss2, _ = sharding.sharded_fbw(am_d, (fsa[0], e_, w_, se_), sl_, plan=None)
            out_h.copy_(out, non_blocking=True)
            return finish(sums, loss2)

        def step_dev_out():
            # scores read in place, the (T,B,F) result left on the device (a trainer that consumes it there)
            e_, w_, se_, sl_ = [t.to(dev, non_blocking=True) for t in host_fsa]
            _, sums, loss2 = sharding.sharded_fbw_host_scores(am_h, (fsa[0], e_, w_, se_), sl_)
            return finish(sums, loss2)

        def time_leg(fn, h2d, d2h, path):
            n = max(3, min(args.steps, 6))
            for _ in range(2):
                fn()
            barrier()
            ev0.record()
            for _ in range(n):
                fn()
            ev1.record()
            barrier()
            mine = ev0.elapsed_time(ev1) / n
            rank_ms = gather_ranks(mine)
            t = max(rank_ms)
            return {"value": total_frames / (t * 1e-3), "unit": "frames/s", "h2d_bytes_per_step": int(h2d),
                    "d2h_bytes_per_step": int(d2h), "ms_per_step": t, "steps": n, "path": path,
                    "rank_ms": rank_ms,
                    "rank_bus_gbs": [(h2d + d2h) / (m * 1e-3) / 1e9 for m in rank_ms]}

        sectors = batch.score_sector_bytes()
        info = core.fbw_prepare(fsa[1], fsa[2], fsa[3], seq_lens, batch.T, batch.F, int(fsa[0])).info()
        sparse_rows = info["max_slots"] * 16 <= batch.F
        # what crosses the bus for the result: the posteriors and five small plan arrays where the host
        # writes the rows, else the whole tensor
        posterior_bytes = info["frame_floats"] * 4 + 20 * batch.B + 4 * (batch.num_edges + batch.B + 1)
        # what crosses the bus for the scores: the entries the automata refer to, picked out of the
        # pinned tensor by the library's host threads (one array, one copy), else 32-byte sectors read
        # in place by the device's gather
        host_helps = sparse_rows and am_h.numel() >= 1e7
        picked = info["frame_floats"] * 4 if host_helps else sectors
        e2e = time_leg(step_host_to_host, picked + fsa_bytes,
                       (posterior_bytes if sparse_rows else out_bytes) + small_d2h,
                       "inputs and results in pinned host memory: "
                       + (f"the scores the automata refer to are picked out of the {am_h.numel() * 4}-byte tensor by the "
                          "library's host threads and copied to the device as one array"
                          if host_helps else
                          f"scores read in place by the op's gather (32-byte sectors of a {am_h.numel() * 4}-byte tensor)")
                       + f"; the (T,B,F) result of {out_bytes} bytes "
                       + ("is written into pinned host memory by the library's host threads from the class posteriors, "
                          "which are all of it that crosses the bus (d2h_bytes_per_step), while the device goes on"
                          if sparse_rows else "is copied device -> host piece by piece while the op runs")
                       + "; sums and loss copied back")
        e2e["result_bytes_per_step"] = int(out_bytes)
        e2e_in_place = time_leg(step_in_place, sectors + fsa_bytes, out_bytes + small_d2h,
                                "as e2e, but the op's output pass writes the (T,B,F) result straight into "
                                "pinned host memory (no device copy of the result)")
        e2e_copy = time_leg(step_copy, am_h.numel() * 4 + fsa_bytes, out_bytes + small_d2h,
                            "whole score tensor copied host -> device, the op, whole result copied device -> host")
        e2e_dev_out = time_leg(step_dev_out, picked + fsa_bytes, small_d2h,
                               ("scores picked out of pinned host memory by the library's host threads"
                                if host_helps else "scores read in place from pinned host memory")
                               + ", the (T,B,F) result LEFT ON THE DEVICE, sums and loss copied back")
        del am_h, out_h
    else:
        del am
    torch.cuda.empty_cache()

    # ---- strong scaling on the configurations that are sharded over GPUs ----
    strong = None
    if not args.no_strong:
        strong = {}
        for name, gb in STRONG.items():
            strong[name] = strong_leg(name, gb, world, rank, dev, 5 if name == "lattice" else 10, dist, torch,
                                      core, sharding, wl)

    host = {"cpus_allowed": len(os.sched_getaffinity(0)), "bound_to_gpu_numa_node": bound,
            "gpu_numa_node": None if numa is None else numa[0]}
    if rank == 0:
        peak, peak_kind = peaks()
        achieved = alg_bytes / (ms_per_step * 1e-3) / 1e9  # this rank's call; ranks are symmetric
        traffic = MEASURED_TRAFFIC.get((args.workload, batch.B))
        line = {
            "metric": "fbw fwd+bwd frames/s", "value": value, "unit": "frames/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
            "data": "synthetic",
            "config": config_of(args.workload, batch, global_b),
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                         "frac": achieved / peak, "traffic": traffic, "peak_kind": peak_kind,
                         "traffic_note": ("dram__bytes_read.sum + dram__bytes_write.sum over the kernels of one "
                                          "call, ncu capture of this workload and batch size") if traffic else
                                         "no ncu capture of this workload at this batch size",
                         "algorithmic_bytes_per_call": int(alg_bytes),
                         "scope": "whole op call (all kernels), per GPU"},
            "kernels_ms": {"prepare": prep_ms, "gather": float(phase[0]), "sweep": float(phase[1]),
                           "posterior": float(phase[2]), "expand": float(phase[3]),
                           "loss": float(phase[4]),
                           "note": "every stage once over the whole batch on one stream (one-pass output); the timed "
                                   "step overlaps the stages and may write its output in two steps instead"},
            "gpu_launches": int(launches),
            "clocks": clk.summary(),
            "e2e": e2e,
            "e2e_copy": e2e_copy,
            "e2e_full": e2e_copy,  # the same leg under its other name: every input and result byte crosses the bus
            "e2e_in_place_out": e2e_in_place,
            "e2e_out_on_device": e2e_dev_out,
            "reference_gpu_op": reference_gpu_op,
            "strong": strong,
            "host": host,
        }
        if world == 1 and not args.no_cpu_baseline:
            threads = os.cpu_count() or 1
            cframes, ctimes, sample = cpu_baseline_pass(args.workload, threads, 5)
            line["cpu_baseline"] = {"value": cframes * len(ctimes) / float(sum(ctimes)),
                                    "unit": "frames/s", "cores": threads, "kind": "port",
                                    "sample": sample}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
