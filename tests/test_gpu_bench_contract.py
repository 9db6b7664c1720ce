"""The benchmark's output contract: one JSON line on stdout with the keys the harness reads."""
import json
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(*args):
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), *args], cwd=ROOT, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    lines = [ln for ln in r.stdout.splitlines() if ln.strip()]
    assert len(lines) == 1, r.stdout[-2000:]
    return json.loads(lines[0])


def test_default_workload_line():
    d = _run("--steps", "3", "--warmup", "3", "--no-cpu-baseline")
    for key in ("metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling", "vs_baseline",
                "dtype", "data", "config", "clocks", "e2e", "gpu_launches", "roofline", "cpu_baseline"):
        assert key in d, key
    assert d["unit"] == "TFLOP/s" and d["n_gpus"] == 1 and d["steps"] == 3 and d["dtype"] == "bf16" and d["vs_baseline"] is None
    assert d["gpu_launches"] == 7 * 3 and d["value"] > 100.0
    assert abs(d["value"] - 7.559e11 / (d["ms_per_step"] * 1e-3) / 1e12) < 1e-2 * d["value"]
    rf = d["roofline"]
    assert rf["bound"] == "tensor" and rf["unit"] == "TFLOP/s" and abs(rf["frac"] - rf["achieved"] / rf["peak"]) < 1e-9 and rf["traffic"]
    e = d["e2e"]
    assert e["h2d_bytes_per_step"] == 8192 * 4096 * 2 and e["d2h_bytes_per_step"] == 4 and 0 < e["value"] < d["value"]
    assert "workload" in d["config"] and "l2" in d["config"]
    assert e["h2d_gbs"] > 1.0 and e["h2d_copy_ms"] > 0
    # the second scaling curve travels in the same line: the row-sharded 65536 x 16384 layer on the same GPUs
    sh = d["sharded"]
    assert sh["n_gpus"] == 1 and sh["scaling"] == "strong" and sh["unit"] == "TFLOP/s" and "65536x16384" in sh["workload"]
    assert sh["speedup_vs_single_gpu"] == 1.0 and sh["exchange"] == "single GPU" and sh["phases_ms"]
    assert abs(sh["value"] - 3.0236e12 / (sh["ms_per_step"] * 1e-3) / 1e12) < 1e-2 * sh["value"]


def test_gemv_workload_line():
    d = _run("--workload", "gemv", "--steps", "5", "--warmup", "3", "--no-cpu-baseline")
    assert d["unit"] == "GB/s" and d["roofline"]["bound"] == "hbm" and d["gpu_launches"] == 4 * 5 and d["dtype"] == "f32"
    assert d["eager_ms_per_step"] > 0 and d["value"] > 10.0
