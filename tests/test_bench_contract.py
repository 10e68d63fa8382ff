"""CPU test of the benchmark's reference arm: `bench.py --impl reference` needs no GPU (it times the CPU
port of the reference arithmetic) and must print one JSON line with the agreed keys."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def run_bench(*extra):
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--steps", "1",
                          "--warmup", "3", "--workload", "monophone", *extra],
                         capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert out.returncode == 0, out.stderr[-2000:]
    lines = [l for l in out.stdout.splitlines() if l.strip()]
    assert len(lines) == 1
    return json.loads(lines[0])


def test_reference_arm_line():
    d = run_bench()
    assert d["impl"] == "reference" and d["metric"] == "fbw fwd+bwd frames/s" and d["unit"] == "frames/s"
    assert d["higher_is_better"] is True and d["value"] > 0 and d["n_gpus"] == 1 and d["steps"] == 1
    assert d["config"]["workload"] == "monophone"
    assert d["cpu_baseline"]["kind"] == "port" and d["cpu_baseline"]["cores"] >= 1
    assert d["cpu_baseline"]["value"] == d["value"]
    assert d["e2e"] == {"value": d["value"], "unit": "frames/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    assert d["gpu_launches"] == 0


def test_reference_arm_line_viterbi():
    d = run_bench("--op", "viterbi")
    assert d["impl"] == "reference" and d["metric"] == "viterbi frames/s" and d["value"] > 0
    assert d["config"]["op"] == "viterbi" and d["cpu_baseline"]["cores"] == 1
