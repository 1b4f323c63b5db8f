"""bench.py's reference arm runs on the host cores alone, so its JSON contract is
checked here without a GPU (the GPU arm is exercised by the round-end bench)."""

import json
import os
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent


def run_bench(*args, env=None):
    e = dict(os.environ)
    e.update(env or {})
    return subprocess.run([sys.executable, str(ROOT / "bench.py"), *args], cwd=ROOT, env=e,
                          capture_output=True, text=True, timeout=600)


def test_reference_arm_line():
    r = run_bench("--impl", "reference", "--workload", "c1", "--steps", "2", "--warmup", "1")
    assert r.returncode == 0, r.stderr
    line = json.loads(r.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and line["metric"] == "graph_throughput"
    assert line["unit"] == "TFLOP/s" and line["value"] > 0 and line["higher_is_better"] is True
    assert line["n_gpus"] == 1 and line["steps"] == 2 and line["ms_per_step"] > 0
    assert line["config"]["workload"].startswith("c1")
    base = line["cpu_baseline"]
    assert base["kind"] == "port" and base["cores"] >= 1 and base["value"] == line["value"]
    assert "sample" in base
    assert line["e2e"] == {"value": line["value"], "unit": "TFLOP/s", "h2d_bytes_per_step": 0,
                           "d2h_bytes_per_step": 0}


def test_reference_arm_for_a_data_movement_graph_reports_bandwidth():
    r = run_bench("--impl", "reference", "--workload", "c4a", "--steps", "1", "--warmup", "1")
    assert r.returncode == 0, r.stderr
    line = json.loads(r.stdout.strip().splitlines()[-1])
    assert line["unit"] == "GB/s" and line["cpu_baseline"]["unit"] == "GB/s" and line["value"] > 0


def test_reference_arm_other_ranks_print_nothing():
    r = run_bench("--impl", "reference", "--gpus", "2", "--workload", "c1", "--steps", "1",
                  env={"RANK": "1", "WORLD_SIZE": "2", "LOCAL_RANK": "1"})
    assert r.returncode == 0, r.stderr
    assert r.stdout.strip() == ""
