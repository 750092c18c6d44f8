"""bench.py prints one JSON line with the keys the measurement contract names,
for this repository's arm and for the reference (CPU) arm."""
import json
import os
import subprocess
import sys

import pytest

from conftest import REPO

pytestmark = pytest.mark.gpu


def _run(args, timeout=900):
    r = subprocess.run([sys.executable, os.path.join(REPO, "bench.py")] + args, capture_output=True, text=True,
                       timeout=timeout, cwd=REPO)
    assert r.returncode == 0, r.stderr[-2000:]
    lines = [l for l in r.stdout.splitlines() if l.startswith("{")]
    assert len(lines) == 1, r.stdout[-2000:]
    return json.loads(lines[0])


def test_bench_line_of_this_arm():
    d = _run(["--steps", "2", "--warmup", "3", "--no-cpu-baseline", "--no-extras"])
    for k in ("metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better",
              "scaling", "vs_baseline", "dtype", "data", "config", "e2e", "gpu_launches", "clocks", "roofline"):
        assert k in d, k
    assert d["metric"].startswith("SD3.5-M DiT denoise steps/sec") and d["unit"] == "steps/s"
    assert d["n_gpus"] == 1 and d["steps"] == 2 and d["warmup"] >= 3 and d["higher_is_better"] is True
    assert d["dtype"] == "bf16" and d["data"] == "synthetic" and d["scaling"] == "strong"
    assert "workload" in d["config"] and "model" not in d["config"] and d["config"]["per_gpu_batch"] == 8
    assert abs(d["weak_value"] - d["value"]) < 1e-9  # one GPU: the two readings coincide
    assert abs(d["value"] * d["ms_per_step"] - 1000.0) < 1e-6 * 1000.0
    assert d["gpu_launches"] >= 2 * 250  # ~267 kernels per step
    e = d["e2e"]
    assert e["unit"] == "steps/s" and 0 < e["value"] <= 1.05 * d["value"]
    assert e["h2d_bytes_per_step"] == (8 * 16 * 128 * 128 + 8 * 333 * 4096 + 8 * 2048) * 2 + 8 * 4
    assert e["d2h_bytes_per_step"] == 8 * 16 * 128 * 128 * 2
    r = d["roofline"]
    assert r["bound"] in ("hbm", "tensor") and r["unit"] in ("GB/s", "TFLOP/s")
    assert abs(r["frac"] - r["achieved"] / r["peak"]) < 1e-3 and r["traffic"] > 0
    assert {"sm_mhz", "sm_max_mhz", "reasons"} <= set(d["clocks"])
    assert len(d["kernels"]) >= 8
    assert any(k["kernel"].startswith("[library, context only]") for k in d["kernels"])


def test_bench_line_of_the_reference_arm():
    d = _run(["--impl", "reference", "--steps", "1", "--warmup", "0"])
    assert d["impl"] == "reference" and d["unit"] == "steps/s" and d["value"] > 0
    assert d["metric"].startswith("SD3.5-M DiT denoise steps/sec")
    c = d["cpu_baseline"]
    assert c["kind"] in ("port", "reference") and c["cores"] >= 1 and c["value"] == d["value"] and c["sample"]
    e = d["e2e"]
    assert e["value"] == d["value"] and e["h2d_bytes_per_step"] == 0 and e["d2h_bytes_per_step"] == 0
    assert abs(d["value"] * d["full_batch_forward_s"] - 1.0) < 1e-6 and d["ms_per_step"] > 0
    assert d["config"]["workload"].startswith("SD3.5-medium DiT forward, 1024^2, batch 8")
