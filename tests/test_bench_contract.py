"""CPU: the benchmark's reference arm runs without a GPU and prints one JSON line with the agreed keys."""
import json
import os
import subprocess
import sys

from conftest import ROOT


def _run(*args):
    res = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", *args],
                         capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stderr[-2000:]
    lines = [l for l in res.stdout.splitlines() if l.startswith("{")]
    assert len(lines) == 1
    return json.loads(lines[0])


def test_reference_arm_line_default_workload_scaled():
    d = _run("--scale", "0.05", "--steps", "2", "--warmup", "1")
    for key in ("impl", "metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better",
                "scaling", "vs_baseline", "dtype", "data", "config", "cpu_baseline", "e2e"):
        assert key in d, key
    assert d["impl"] == "reference" and d["metric"] == "spmm_effective_hbm_gbs" and d["unit"] == "GB/s"
    assert d["config"]["workload"] == "cfg5_spmm" and d["data"] == "synthetic" and d["vs_baseline"] is None
    assert d["cpu_baseline"]["kind"] in ("reference", "port") and d["cpu_baseline"]["cores"] >= 1
    assert d["e2e"]["h2d_bytes_per_step"] == 0 and d["e2e"]["value"] == d["value"] > 0


def test_reference_arm_other_workloads():
    assert _run("--workload", "cfg1_spmv", "--scale", "0.1", "--steps", "2")["metric"] == "spmv_effective_hbm_gbs"
    d = _run("--workload", "cfg3_mlp", "--scale", "0.05", "--steps", "2")
    assert d["metric"] == "sparse_mlp_samples_per_s" and d["unit"] == "samples/s"
    assert _run("--workload", "cfg4_conv", "--scale", "0.1", "--steps", "1")["value"] > 0


def test_reference_arm_nonzero_ranks_stay_silent():
    env = dict(os.environ, RANK="1", WORLD_SIZE="2", LOCAL_RANK="1")
    res = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--scale", "0.05"],
                         capture_output=True, text=True, timeout=120, env=env)
    assert res.returncode == 0 and res.stdout.strip() == ""
