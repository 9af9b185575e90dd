"""CPU tests of bench.py's contract: the reference arm (MIGraphX's CPU ref target, a bounded sample)
prints exactly one JSON line with the agreed keys, only rank 0 of a multi-rank launch prints it,
and the product arm refuses to run without a CUDA device (there is no CPU path to fall back to)."""
import json
import os
import subprocess
import sys

import pytest

from oracle import ref_target as R

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
BENCH = os.path.join(ROOT, "bench.py")


@pytest.mark.skipif(not R.available(), reason="oracle/_ref is not built here")
def test_reference_arm_prints_one_json_line_with_the_contract_keys():
    r = subprocess.run([sys.executable, BENCH, "--impl", "reference", "--steps", "1", "--warmup", "1"],
                       capture_output=True, text=True, timeout=900, cwd=ROOT)
    assert r.returncode == 0, r.stderr[-2000:]
    lines = [l for l in r.stdout.splitlines() if l.strip()]
    assert len(lines) == 1, r.stdout
    d = json.loads(lines[0])
    assert d["impl"] == "reference" and d["metric"] == "int8_qdq_gemm_tops" and d["unit"] == "TOPS"
    assert d["higher_is_better"] is True and d["n_gpus"] == 1 and d["steps"] == 1 and d["value"] > 0
    assert d["cpu_baseline"]["kind"] == "reference" and d["cpu_baseline"]["cores"] >= 1
    assert d["cpu_baseline"]["value"] == d["value"] and "ref target" in d["cpu_baseline"]["sample"]
    assert d["e2e"] == {"value": d["value"], "unit": "TOPS", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    assert "workload" in d["config"] and "model" not in d["config"]


def test_reference_arm_is_silent_on_other_ranks():
    env = dict(os.environ, RANK="1", WORLD_SIZE="2", LOCAL_RANK="1")
    r = subprocess.run([sys.executable, BENCH, "--impl", "reference", "--gpus", "2", "--steps", "1", "--warmup", "1"],
                       capture_output=True, text=True, timeout=300, cwd=ROOT, env=env)
    assert r.returncode == 0 and r.stdout.strip() == "", r.stdout + r.stderr[-1000:]


def test_product_arm_needs_a_gpu():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a CUDA device is present")
    r = subprocess.run([sys.executable, BENCH, "--steps", "1", "--warmup", "1"], capture_output=True, text=True,
                       timeout=300, cwd=ROOT)
    assert r.returncode != 0 and r.stdout.strip() == ""
    assert "CUDA device" in r.stderr


def test_reference_linear_timing_script_runs():
    """oracle/time_ref_linears.py (the per-linear CPU baselines of the results table) prints one JSON
    object per line; --quick takes the smallest shape of each kind."""
    import json
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    out = subprocess.run([sys.executable, os.path.join(root, "oracle", "time_ref_linears.py"), "--quick"],
                         capture_output=True, text=True, timeout=300)
    lines = [json.loads(ln) for ln in out.stdout.splitlines() if ln.strip()]
    if "unavailable" in lines[0]:
        assert out.returncode == 1
        return
    assert out.returncode == 0 and lines[0]["threads"] >= 1
    assert lines[1]["op"].startswith("quant_dot") and lines[1]["seconds"] > 0
    assert lines[2]["weight_bytes"] == 4096 * 2048 + 2 * 4096 * 32 and lines[2]["seconds"] > 0
