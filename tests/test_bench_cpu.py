"""The legs of bench.py that need no GPU keep working: the reference (CPU) arm and the creation
benchmark, each printing one JSON line with the agreed keys."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(*args):
    res = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), *args], capture_output=True, text=True,
                         timeout=600, cwd=ROOT)
    assert res.returncode == 0, res.stderr[-2000:]
    return json.loads(res.stdout.strip().splitlines()[-1])


def test_reference_arm_line():
    d = _run("--impl", "reference", "--steps", "2", "--warmup", "1", "--scale", "0.02")
    assert d["impl"] == "reference" and d["steps"] == 2 and d["unit"] == "GB/s" and d["value"] > 0
    assert d["metric"] == "cbm_spmm_algorithmic_GBps" and d["higher_is_better"] is True
    from oracle import reference
    assert d["cpu_baseline"]["kind"] == ("reference" if reference.ref_available() else "port")
    assert d["cpu_baseline"]["cores"] >= 1
    assert d["e2e"] == dict(value=d["value"], unit="GB/s", h2d_bytes_per_step=0, d2h_bytes_per_step=0)
    assert d["config"]["workload"] == "c2" and d["config"]["n"] == 2000
    # workload keys only: timings live outside config so that both arms print the same object
    assert set(d["config"]) == {"workload", "n", "nnz", "f", "alpha", "normalized", "n_delta", "n_root_children",
                                "depth", "l2"}
    assert "build_seconds" in d["build"]


def test_creation_benchmark_line():
    d = _run("--task", "build", "--workload", "c1", "--steps", "1", "--scale", "0.25")
    assert d["metric"] == "cbm_creation_seconds" and [r["alpha"] for r in d["per_alpha"]] == [0, 1, 2, 4, 8, 16, 32, 64]
    nd = [r["n_delta"] for r in d["per_alpha"]]
    assert nd == sorted(nd) and all(r["compression_ratio"] > 0.5 for r in d["per_alpha"])
