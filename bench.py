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
  e2e        the same through the op with HOST buffers: the scores stay in pinned host memory and the
             op's gather reads the sectors it needs from there over the bus (--e2e-copy: the whole
             tensor is copied to the device first), the automata are copied host -> device, the
             (T,B) result device -> host, all inside the timing
  roofline   whole-call algorithmic bytes / measured call time against the measured HBM peak
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

# dram__bytes_read.sum + dram__bytes_write.sum of all kernels of one triphone call divided by the
# call's algorithmic bytes, from the ncu capture summarised in profiles/
TRAFFIC_PER_ALGORITHMIC_BYTE = 0.89  # profiles/dram_traffic_triphone_b16.md (B=16 capture, scaled)


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


def cpu_baseline_pass(workload: str, threads: int, passes: int, warm: int = 1):
    """Times the CPU oracle (test infrastructure; the only use of oracle/ in this file) on a
    bounded sample: one per-GPU batch of the workload at full T and F, a few passes."""
    import oracle
    from i6_native_ops_b200 import workloads as wl

    batch = wl.make_batch(workload, B=CPU_SAMPLE_SEQS or SEQS_PER_GPU[workload])
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
    return frames, times, sample


def run_reference_arm(args):
    """The reference arm: the reference's fbw has no CPU implementation (its binding rejects CPU
    tensors), so this times the C/OpenMP port of its arithmetic on the host cores."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    frames, times, sample = cpu_baseline_pass(args.workload, threads, args.steps, max(1, min(args.warmup, 2)))
    total = float(sum(times))
    value = frames * len(times) / total
    line = {
        "impl": "reference", "metric": "fbw fwd+bwd frames/s", "value": value, "unit": "frames/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": 1e3 * total / len(times), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": args.workload, "sample": sample},
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
    ap.add_argument("--op", default="fbw", choices=["fbw", "viterbi"])
    ap.add_argument("--e2e-copy", action="store_true",
                    help="e2e leg: copy the whole score tensor to the device first (default: the op reads "
                         "the scores it needs from pinned host memory)")
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

    # ---- end to end through the op with host buffers ----
    e2e = None
    if not args.no_e2e:
        am_h = torch.empty(am.shape, dtype=am.dtype, pin_memory=True)
        am_h.copy_(am)
        host_fsa = [t.cpu().pin_memory() for t in (fsa[1], fsa[2], fsa[3], seq_lens)]
        sums_h = torch.empty((batch.T, batch.B), dtype=torch.float32, pin_memory=True)
        del am
        # The scores stay in pinned host memory: the op's gather reads the sectors it needs straight
        # from there (no copy of the whole tensor), so what crosses the bus per step is those
        # sectors plus the automata.  --e2e-copy takes the classic route instead (whole tensor copied
        # to the device first).
        am_d = torch.empty(am_h.shape, dtype=am_h.dtype, device=dev) if args.e2e_copy else None
        fsa_bytes = sum(t.numel() * t.element_size() for t in host_fsa)
        h2d = (am_h.numel() * 4 if args.e2e_copy else batch.score_sector_bytes()) + fsa_bytes
        d2h = sums_h.numel() * 4 + 8

        def e2e_step():
            e_, w_, se_, sl_ = [t.to(dev, non_blocking=True) for t in host_fsa]
            if args.e2e_copy:
                am_d.copy_(am_h, non_blocking=True)
                out, sums, loss2, _ = sharding.sharded_fbw(am_d, (fsa[0], e_, w_, se_), sl_, plan=None)
            else:
                out, sums, loss2 = sharding.sharded_fbw_host_scores(am_h, (fsa[0], e_, w_, se_), sl_)
            sums_h.copy_(sums, non_blocking=True)
            return loss2.cpu()  # device -> host read of the reduced loss; synchronises

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
        e2e = {"value": total_frames / (float(t_e.item()) * 1e-3), "unit": "frames/s",
               "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(d2h),
               "ms_per_step": float(t_e.item()), "steps": n_e2e,
               "path": ("scores copied to the device, then the op" if args.e2e_copy else
                        "scores read in place from pinned host memory by the op's gather "
                        f"(32-byte sectors; the whole tensor is {am_h.numel() * 4} bytes)")}

    if rank == 0:
        peak, peak_kind = peaks()
        achieved = alg_bytes / (ms_per_step * 1e-3) / 1e9  # this rank's call; ranks are symmetric
        traffic = (None if TRAFFIC_PER_ALGORITHMIC_BYTE is None
                   else float(TRAFFIC_PER_ALGORITHMIC_BYTE * alg_bytes))
        line = {
            "metric": "fbw fwd+bwd frames/s", "value": value, "unit": "frames/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
            "data": "synthetic",
            "config": {"workload": args.workload, "T": batch.T, "B_per_gpu": batch.B,
                       "B_global": global_b, "F": batch.F, "edges_per_gpu": batch.num_edges,
                       "states_per_gpu": batch.num_states, "partition": "by sequence, length-balanced",
                       "l2": f"inputs ({am_bytes / 1e9:.2f} GB of scores per call) exceed the 126 MB L2; no flush"
                             if am_bytes > 2 * 126e6 else "an L2 flush (256 MB write) runs between timed steps",
                       "step": "prepare + run per call (automata re-sorted every step)"},
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                         "frac": achieved / peak, "traffic": traffic, "peak_kind": peak_kind,
                         "algorithmic_bytes_per_call": int(alg_bytes),
                         "scope": "whole op call (all kernels), per GPU"},
            "kernels_ms": {"prepare": prep_ms, "gather": float(phase[0]), "sweep": float(phase[1]),
                           "posterior": float(phase[2]), "expand": float(phase[3]),
                           "loss": float(phase[4])},
            "gpu_launches": int(launches),
            "clocks": clk.summary(),
            "e2e": e2e,
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
