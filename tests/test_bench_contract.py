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
    assert "sample" in base and "random samples" in base["sample"]  # tuned before it is timed
    assert base["blas_ceiling"]["value"] > 0 and 0 < base["frac_of_host_fma_peak"] < 1.5
    assert line["mlir_toolchain_present"] is False and line["scaling"] == "weak"
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


def test_default_workload_is_one_curve_under_torchrun():
    """Launched by torch.distributed.run the arm benches c5 with fixed total work at every
    world size (1 included); a plain one-GPU run benches c2."""
    sys.path.insert(0, str(ROOT))
    import bench

    keep = {k: os.environ.pop(k, None) for k in ("TORCHELASTIC_RUN_ID", "LOCAL_RANK")}
    try:
        assert bench.default_workload() == "c2"
        os.environ["LOCAL_RANK"] = "0"
        assert bench.default_workload() == "c5"
    finally:
        os.environ.pop("LOCAL_RANK", None)
        for k, v in keep.items():
            if v is not None:
                os.environ[k] = v


def test_row_block_inputs_equal_slices_of_the_full_draw():
    """Each rank draws only its own rows of c5's A: the draw must equal the slice of the
    full seeded draw (checked on the generator arithmetic with a narrow stand-in)."""
    import numpy as np

    sys.path.insert(0, str(ROOT))
    from xtc_b200 import configs

    a, b = configs.input_rows("c5", 3, 5)
    rng = np.random.default_rng(4)
    rng.uniform(-1, 1, (3, 8192))  # the rows before
    assert np.array_equal(a, rng.uniform(-1, 1, (2, 8192)).astype(np.float32))
    a0, _ = configs.input_rows("c5", 0, 2)
    assert np.array_equal(a0, np.random.default_rng(4).uniform(-1, 1, (2, 8192)).astype(np.float32))
    assert b.shape == (8192, 8192) and abs(float(b.std()) * np.sqrt(8192) - 1) < 1e-2
