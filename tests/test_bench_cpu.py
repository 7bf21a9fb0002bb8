"""bench.py's contract, as far as it can be checked without a GPU: the reference arm runs the CPU
kernel on the host and prints one JSON line with the agreed keys; our arm refuses to run without a
CUDA device instead of measuring a fallback."""
import json
import os
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent


def run(*args, env=None):
    e = dict(os.environ)
    e.update(env or {})
    return subprocess.run([sys.executable, str(ROOT / "bench.py"), *args], capture_output=True, text=True, cwd=ROOT,
                          env=e, timeout=600)


def test_reference_arm_prints_one_contract_line():
    p = run("--impl", "reference", "--steps", "1", "--warmup", "1")
    assert p.returncode == 0, p.stderr[-2000:]
    lines = [l for l in p.stdout.splitlines() if l.strip()]
    assert len(lines) == 1
    d = json.loads(lines[0])
    assert d["impl"] == "reference" and d["metric"] == "bf16_gemv_hbm_bandwidth" and d["unit"] == "GB/s"
    assert d["higher_is_better"] is True and d["n_gpus"] == 1 and d["steps"] == 1 and d["vs_baseline"] is None
    assert d["value"] > 0 and abs(d["cpu_baseline"]["value"] - d["value"]) < 1e-9
    assert d["cpu_baseline"]["kind"] == "port" and 1 <= d["cpu_baseline"]["cores"] <= 4     # the reference's thread policy
    assert d["e2e"] == {"value": d["value"], "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    assert "workload" in d["config"]


def test_reference_arm_under_torchrun_runs_on_rank_zero_only():
    env = {"RANK": "1", "WORLD_SIZE": "2", "LOCAL_RANK": "1"}
    p = run("--impl", "reference", "--gpus", "2", "--steps", "1", "--warmup", "1", env=env)
    assert p.returncode == 0 and p.stdout.strip() == ""


def test_our_arm_has_no_cpu_fallback():
    p = run("--steps", "1", env={"CUDA_VISIBLE_DEVICES": ""})
    assert p.returncode != 0
    assert "no CUDA device" in (p.stderr + p.stdout)
