"""bench.py on a GPU, reduced size: the line carries every key the measurement contract names and
its parity record is inside the tolerance."""
import json
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_bench_line_keys_and_parity():
    res = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--scale", "0.05", "--steps", "5", "--warmup", "3",
                          "--cpu-seconds", "1", "--no-extras"], capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert res.returncode == 0, res.stderr[-2000:]
    d = json.loads(res.stdout.strip().splitlines()[-1])
    for k in ("metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling",
              "vs_baseline", "dtype", "data", "config", "roofline", "cpu_baseline", "cpu_baseline_sequential", "e2e",
              "gpu_launches", "clocks", "parity", "sustained", "build"):
        assert k in d, k
    assert d["n_gpus"] == 1 and d["steps"] == 5 and d["gpu_launches"] == 5 and d["dtype"] == "f32"
    assert d["config"]["workload"] == "c2" and d["config"]["n"] == 5000
    r = d["roofline"]
    for k in ("bound", "achieved", "peak", "unit", "frac", "traffic", "gather", "compulsory_bytes_per_launch"):
        assert k in r, k
    assert 0 < r["frac"] <= 1.2
    assert d["parity"]["rows"] == 1000 and d["parity"]["max_err_over_tol"] <= 1.0
    assert d["e2e"]["h2d_bytes_per_step"] == 5000 * 500 * 4 and d["e2e"]["value"] > 0
    assert d["cpu_baseline"]["cores"] >= 1 and d["cpu_baseline_sequential"]["cores"] == 1
