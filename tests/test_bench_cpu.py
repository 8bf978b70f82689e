"""The benchmark's CPU arm (`bench.py --impl reference`): runs without a GPU, times the oracle on a
bounded sample and prints one JSON line with the keys of the GPU arm's line."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(*flags, env=None):
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), *flags], cwd=ROOT,
                         capture_output=True, text=True, timeout=600, env=env)
    assert out.returncode == 0, out.stderr[-2000:]
    return [json.loads(l) for l in out.stdout.splitlines() if l.startswith("{")]


def test_reference_arm_line():
    lines = _run("--impl", "reference", "--workload", "opt125m", "--steps", "1", "--warmup", "0")
    assert len(lines) == 1
    d = lines[0]
    assert d["impl"] == "reference" and d["metric"] == "gptq_wall_clock_s_per_model"
    assert d["unit"] == "s/model" and d["higher_is_better"] is False and d["gpu_launches"] == 0
    assert d["n_gpus"] == 1 and d["steps"] == 1 and d["warmup"] == 0
    assert d["value"] > 0 and abs(d["ms_per_step"] - 1e3 * d["value"]) < 1e-6 * d["ms_per_step"]
    cb = d["cpu_baseline"]
    assert cb["kind"] == "port" and cb["cores"] >= 1 and cb["value"] == d["value"]
    assert "oracle port" in cb["sample"] and "OPT-125m" in d["config"]["workload"]
    assert d["e2e"] == {"value": d["value"], "unit": "s/model", "h2d_bytes_per_step": 0,
                        "d2h_bytes_per_step": 0}


def test_reference_arm_other_ranks_print_nothing():
    env = dict(os.environ, RANK="1", WORLD_SIZE="2", LOCAL_RANK="1")
    assert _run("--impl", "reference", "--gpus", "2", "--workload", "opt125m", "--steps", "1",
                "--warmup", "0", env=env) == []
