"""The CPU arm of bench.py (`--impl reference`): it needs no GPU, so its JSON contract is checked here."""
import json
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

REQUIRED = {"impl", "metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better",
            "scaling", "vs_baseline", "dtype", "data", "config", "cpu_baseline", "e2e", "gpu_launches"}


def _run(extra, env=None):
    cmd = [sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--steps", "2", "--warmup", "1"] + extra
    out = subprocess.run(cmd, cwd=ROOT, capture_output=True, text=True, timeout=300, env=env)
    assert out.returncode == 0, out.stderr[-2000:]
    return out.stdout.strip().splitlines()


@pytest.mark.parametrize("workload", ["cfg1_fp32_512_cube", "cfg4_batched_fp32_2048x64_cube"])
def test_reference_arm_line(workload):
    lines = _run(["--workload", workload])
    assert len(lines) == 1
    d = json.loads(lines[0])
    assert REQUIRED <= set(d)
    assert d["impl"] == "reference" and d["gpu_launches"] == 0
    assert d["metric"] == "gemm_tflops" and d["unit"] == "TFLOP/s" and d["higher_is_better"] is True
    assert d["config"]["workload"] == workload
    assert d["value"] > 0 and d["ms_per_step"] > 0
    cb = d["cpu_baseline"]
    assert cb["kind"] in ("reference", "port") and cb["cores"] >= 1 and cb["value"] == d["value"]
    assert d["e2e"] == {"value": d["value"], "unit": d["unit"], "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}


def test_reference_arm_other_ranks_print_nothing():
    env = dict(os.environ, RANK="1", LOCAL_RANK="1", WORLD_SIZE="2")
    assert _run(["--workload", "cfg1_fp32_512_cube", "--gpus", "2"], env=env) == []


def test_tiny_products_are_not_threaded():
    sys.path.insert(0, ROOT)
    import bench
    assert bench._parts(16, 64, 64, 64) == 1
    assert bench._parts(16, 512, 512, 512) == 13
    assert bench._parts(16, 4096, 8192, 8192) == 16
    assert bench._parts(16, 3, 8192, 8192) == 3
