"""bench.py's CPU-only leg: the reference arm must print one JSON line with the agreed keys, and
ranks other than 0 must stay silent.  (The GPU arm needs a device and is exercised on the GPU box.)"""
import json
import os
import subprocess
import sys
from pathlib import Path

REPO = Path(__file__).resolve().parent.parent


def run_bench(extra_env=None):
    env = dict(os.environ, **(extra_env or {}))
    proc = subprocess.run(
        [sys.executable, str(REPO / "bench.py"), "--impl", "reference", "--workload", "small_fp32",
         "--steps", "2", "--warmup", "1", "--cpu-sample-tokens", "32"],
        capture_output=True, text=True, env=env, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    return proc.stdout.strip()


def test_reference_arm_prints_one_json_line():
    out = run_bench()
    lines = [l for l in out.splitlines() if l.strip()]
    assert len(lines) == 1
    d = json.loads(lines[0])
    assert d["impl"] == "reference" and d["metric"] == "moe_layer_tokens_per_s" and d["unit"] == "tokens/s"
    assert d["higher_is_better"] is True and d["vs_baseline"] is None and d["data"] == "synthetic"
    assert d["value"] > 0 and d["steps"] == 2 and d["gpu_launches"] == 0
    assert d["config"]["workload"] == "small_fp32" and "model" not in d["config"]
    cb = d["cpu_baseline"]
    assert cb["kind"] == "port" and cb["cores"] >= 1 and cb["value"] == d["value"] and "32 of 64 tokens" in cb["sample"]
    assert d["e2e"] == {"value": d["value"], "unit": "tokens/s", "h2d_bytes_per_step": 0,
                        "d2h_bytes_per_step": 0}


def test_reference_arm_is_silent_on_other_ranks():
    assert run_bench({"RANK": "1", "LOCAL_RANK": "1", "WORLD_SIZE": "2"}) == ""
