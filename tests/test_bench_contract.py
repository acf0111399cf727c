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


def test_roofline_fraction_is_against_the_burst_peak():
    """``roofline.frac`` divides by the measured burst peak (the sustained figure is a named extra),
    the bound switches to HBM where streaming the weights takes longer than the FLOPs, and the
    traffic figures scale the algorithmic bytes by the per-kernel ncu ratios."""
    import importlib.util
    spec = importlib.util.spec_from_file_location("bench_module", REPO / "bench.py")
    bench = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(bench)
    peaks = {"hbm_gbs": 6453.1, "bf16_tflops": 1706.6, "bf16_tflops_sustained": 1411.1, "source": "measured"}
    wl = bench.WORKLOADS["mixtral_prefill_t8192_skew"]
    roof, extra = bench.gemm_roofline(wl, "single", 1, {"grouped_gemm_w13_swiglu": 2.8, "grouped_gemm_w2_scale": 1.4,
                                                        "moe_sum": 0.036}, peaks)
    flops = 4 * 4096 * 14336 * 2 * 8192
    assert roof["bound"] == "tensor" and roof["peak"] == 1706.6 and roof["unit"] == "TFLOP/s"
    assert abs(roof["achieved"] - flops / 2.8e-3 / 1e12) < 1e-6
    assert abs(roof["frac"] - roof["achieved"] / 1706.6) < 1e-12
    assert abs(roof["frac_of_sustained"] - roof["achieved"] / 1411.1) < 1e-12
    w13_bytes = 8 * 2 * 14336 * 4096 * 2 + 8192 * 2 * (4096 + 14336) * 2
    assert abs(roof["traffic"] - bench.NCU_TRAFFIC_RATIO["grouped_gemm_w13_swiglu"] * w13_bytes) < 1
    assert extra["moe_sum_frac_of_hbm"] == extra["moe_sum_gbs"] / 6453.1
    # Expert parallel over 8: an eighth of the tokens' pairs and one expert land on a rank.
    roof8, _ = bench.gemm_roofline(bench.WORKLOADS["mixtral_parallel_t16384"], "ep", 8,
                                   {"grouped_gemm_w13_swiglu": 0.66}, peaks)
    assert abs(roof8["achieved"] - 4 * 4096 * 14336 * 2 * 2048 / 0.66e-3 / 1e12) < 1e-6
    # Decode-sized batch: weight streaming is the longer floor.
    small, _ = bench.gemm_roofline(bench.WORKLOADS["mixtral_decode_t256"], "single", 1,
                                   {"grouped_gemm_w13_swiglu": 0.31}, peaks)
    assert small["bound"] == "hbm" and small["peak"] == 6453.1 and 0.9 < small["frac"] < 1.0
