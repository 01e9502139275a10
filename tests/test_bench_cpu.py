"""bench.py on a machine without GPUs: the reference arm prints one well-formed line for any configuration, both
arms describe a configuration with the same dictionary, and the GPU arm refuses to run without a device."""
import json
import os
import subprocess
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent


def _run(*args, env=None):
    e = dict(os.environ)
    e.update(env or {})
    return subprocess.run([sys.executable, str(ROOT / "bench.py"), *args], capture_output=True, text=True, env=e, timeout=600)


@pytest.mark.parametrize("workload", ["softmax_f32", "gemm_f32_512", "attention_causal"])
def test_reference_arm_line(workload):
    r = _run("--impl", "reference", "--workload", workload, "--steps", "1", "--warmup", "3", "--no-extras",
             env={"OMP_NUM_THREADS": "1"})  # what a launcher exports; the arm must undo it
    assert r.returncode == 0, r.stderr
    line = json.loads(r.stdout.strip().splitlines()[-1])
    for key in ("impl", "metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling",
                "dtype", "data", "config", "cpu_baseline", "e2e"):
        assert key in line, key
    assert line["impl"] == "reference" and line["value"] > 0 and line["config"]["workload"] == workload
    assert line["cpu_baseline"]["kind"] == "port" and line["cpu_baseline"]["cores"] == len(os.sched_getaffinity(0))
    assert line["e2e"] == {"value": line["value"], "unit": line["unit"], "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}


def test_other_ranks_of_the_reference_arm_do_nothing():
    r = _run("--impl", "reference", "--steps", "1", "--no-extras", env={"RANK": "1", "WORLD_SIZE": "2"})
    assert r.returncode == 0 and r.stdout.strip() == ""


def test_both_arms_describe_a_configuration_identically():
    sys.path.insert(0, str(ROOT))
    import bench
    for name in bench.ORDER:
        assert bench.config_for(name) == bench.config_for(name)
        assert set(bench.SUMMARY) <= set(bench.ORDER)
    assert bench.config_for("gemm_bf16_8192")["m"] == 8192 and "l2" in bench.config_for("softmax_f32")


def test_gpu_arm_needs_a_gpu():
    import torch
    if torch.cuda.is_available():
        pytest.skip("this check is for machines without a GPU")
    r = _run("--steps", "1", "--no-extras")
    assert r.returncode != 0 and "no CPU fallback" in (r.stderr + r.stdout)
