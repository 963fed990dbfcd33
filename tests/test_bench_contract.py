"""bench.py's contract that can be checked without a GPU: the reference arm runs
the unmodified reference binary and prints one JSON line with the agreed keys;
our arm refuses to run (loudly) when there is no CUDA device."""
import json
import os
import subprocess
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.path.join(ROOT, "baseline", "_ref", "bin", "bench-all-reduce")


def run_bench(*args, timeout=600):
    env = dict(os.environ)
    for k in ("RANK", "WORLD_SIZE", "LOCAL_RANK", "KUNGFU_SELF_SPEC"):
        env.pop(k, None)
    return subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), *args], env=env,
                          stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True,
                          timeout=timeout, cwd=ROOT)


def test_reference_arm_prints_the_agreed_json_line():
    res = run_bench("--impl", "reference", "--gpus", "2", "--steps", "2", "--warmup", "1",
                    "--workload", "resnet50")
    assert res.returncode == 0, res.stderr[-2000:]
    line = json.loads(res.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference"
    if not os.path.exists(REF):
        assert "unavailable" in line
        return
    for key in ("metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step",
                "higher_is_better", "scaling", "dtype", "data", "config"):
        assert key in line, key
    assert line["n_gpus"] == 2 and line["steps"] == 2 and line["value"] > 0
    assert line["config"]["tensors"] == 161 and line["impl_detail"]["transport"] == "tcp-loopback"
    # end to end on host memory is what the reference measures: it says so itself
    assert line["e2e"]["value"] == line["value"] and line["e2e"]["unit"] == "GB/s"
    assert line["e2e"]["h2d_bytes_per_step"] == 0
    # both arms describe the workload with the same keys and values
    sys.path.insert(0, ROOT)
    import bench
    from stdml_collective_experimental_b200.models.gradsets import gradset_sizes
    assert line["config"] == bench.workload_config("resnet50", gradset_sizes("resnet50"), 2, "f32")


def test_reference_arm_reports_unsupported_dtype():
    res = run_bench("--impl", "reference", "--gpus", "1", "--dtype", "bf16")
    line = json.loads(res.stdout.strip().splitlines()[-1])
    assert res.returncode == 0 and line["impl"] == "reference" and "unavailable" in line


def test_our_arm_needs_a_gpu_and_says_so():
    if torch.cuda.is_available():
        pytest.skip("CPU-only behaviour")
    res = run_bench("--gpus", "1", "--steps", "1", "--warmup", "1")
    assert res.returncode != 0
    assert "CUDA" in res.stderr or "cuda" in res.stderr
