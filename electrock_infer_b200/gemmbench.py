"""Interleaved A/B of the grouped-GEMM tilings at Mixtral-8x7B shape, and the cycle accounting of
the two-block kernel when the loaded library is a measurement build.

    python -m electrock_infer_b200.gemmbench [skew:8192 uni:16384 ...] [--tilings 1 2 3]
                                             [--steps 15] [--reps 3] [--lib PATH] [--cycles]

A case is ``routing:tokens``: ``skew`` is the routing of the benchmark workload
(mixtral_prefill_t8192_skew), ``uni`` the near-uniform routing of mixtral_parallel_t16384.
Tilings: 0 the library's own choice, 1 one M block per tile, 2 two M blocks per tile, 3 CTA pairs
(block_m 256); add 10 for the first GEMM's epilogue with per-lane stores instead of bulk tensor
stores.  Each variant runs ``--steps`` layer calls with a CUDA-event pair around every
launch; the variants are interleaved ``--reps`` times after one unmeasured round, and the median of
the per-repetition means is printed (under the board's power cap a kernel's time depends on what
ran before it, so only numbers of one run compare).  One JSON line per case and tiling.

``--cycles`` (needs a library built with ``-DB200MOE_MEASURE_CYCLES`` and passed with ``--lib``)
prints, per grouped GEMM and for each of the tilings 1 and 2 named in ``--tilings``, what
``b200moe_gemm_measured_cycles`` counted.
"""
from __future__ import annotations

import argparse
import ctypes
import json
import statistics
from dataclasses import replace
from pathlib import Path

import torch

from . import _lib
from .synthetic import WORKLOADS, make_inputs


def _base_inputs(kind: str, tokens: int, dev):
    wl = WORKLOADS["mixtral_prefill_t8192_skew" if kind == "skew" else "mixtral_parallel_t16384"]
    wl = replace(wl, num_tokens=tokens, dtype=torch.bfloat16)
    return wl, make_inputs(wl, device=dev, device_rng=True)


def run_tilings(cases, tilings, steps: int, reps: int, dev) -> None:
    from .layers.moe import fused_moe as fm
    lib = _lib.load()
    base = {}
    for kind in {k for k, _ in cases}:
        base[kind] = _base_inputs(kind, max(t for k, t in cases if k == kind), dev)
    for kind, tokens in cases:
        wl, inp = base[kind]
        x0, logits = inp["x"][:tokens].contiguous(), inp["logits"][:tokens].contiguous()
        x = torch.empty_like(x0)
        seen = {t: {"w13": [], "w2": []} for t in tilings}
        try:
            for rep in range(reps + 1):
                for tiling in tilings:
                    fm.FORCE_BLOCK_M = 256 if tiling % 10 == 3 else 128
                    _lib.check(lib.b200moe_gemm_set_tiling(tiling % 10 if tiling % 10 < 3 else 0), "set_tiling")
                    lib.b200moe_gemm_set_act_stores(0 if tiling >= 10 else 1)
                    fm.enable_kernel_timing(True)
                    for _ in range(steps):
                        x.copy_(x0)
                        fm.fused_experts(x, inp["w13"], inp["w2"], logits, 2, inplace=True)
                    ms = fm.collect_kernel_timings()
                    fm.enable_kernel_timing(False)
                    if rep > 0:
                        seen[tiling]["w13"].append(ms["grouped_gemm_w13_swiglu"])
                        seen[tiling]["w2"].append(ms["grouped_gemm_w2_scale"])
        finally:
            fm.FORCE_BLOCK_M = None
            lib.b200moe_gemm_set_tiling(0)
            lib.b200moe_gemm_set_act_stores(1)
        flops13 = 4 * wl.hidden * wl.inter * wl.top_k * tokens
        for tiling in tilings:
            k13 = statistics.median(seen[tiling]["w13"])
            k2 = statistics.median(seen[tiling]["w2"])
            print(json.dumps({"routing": kind, "tokens": tokens, "tiling": tiling,
                              "w13_ms": round(k13, 4), "w2_ms": round(k2, 4),
                              "w13_ms_reps": [round(v, 3) for v in seen[tiling]["w13"]],
                              "w2_ms_reps": [round(v, 3) for v in seen[tiling]["w2"]],
                              "w13_tflops": round(flops13 / k13 / 1e9, 1),
                              "w2_tflops": round(flops13 / 2 / k2 / 1e9, 1),
                              "gemm_status": lib.b200moe_gemm_device_status(1)}), flush=True)


def run_cycles(cases, steps: int, dev, tiling: int = 2) -> None:
    from .layers.moe import fused_moe as fm
    lib = _lib.load()
    out = (ctypes.c_uint64 * 8)()
    if lib.b200moe_gemm_measured_cycles(out, 1) != 1:
        raise SystemExit("--cycles needs a library built with -DB200MOE_MEASURE_CYCLES (pass it with --lib)")
    _lib.check(lib.b200moe_gemm_set_tiling(tiling), "set_tiling")
    for kind, tokens in cases:
        wl, inp = _base_inputs(kind, tokens, dev)
        x = torch.empty_like(inp["x"])
        acc = {"w13": [0] * 8, "w2": [0] * 8}
        real = {"w13": lib.b200moe_grouped_gemm_w13_swiglu, "w2": lib.b200moe_grouped_gemm_w2_scale}

        def counted(fn, key):
            def call(*args):
                torch.cuda.synchronize()
                lib.b200moe_gemm_measured_cycles(out, 1)
                rc = fn(*args)
                torch.cuda.synchronize()
                lib.b200moe_gemm_measured_cycles(out, 1)
                for i in range(8):
                    acc[key][i] += out[i]
                return rc
            return call

        fm.enable_kernel_timing(True)   # the step-by-step path, so that each GEMM is its own call
        lib.b200moe_grouped_gemm_w13_swiglu = counted(real["w13"], "w13")
        lib.b200moe_grouped_gemm_w2_scale = counted(real["w2"], "w2")
        try:
            for _ in range(steps):
                x.copy_(inp["x"])
                fm.fused_experts(x, inp["w13"], inp["w2"], inp["logits"], 2, inplace=True)
        finally:
            lib.b200moe_grouped_gemm_w13_swiglu, lib.b200moe_grouped_gemm_w2_scale = real["w13"], real["w2"]
            fm.collect_kernel_timings()
            fm.enable_kernel_timing(False)
        for key, a in acc.items():
            tiles = max(a[5], 1)
            print(json.dumps({"routing": kind, "tokens": tokens, "gemm": key, "tiling": tiling,
                              "cycles_per_tile": a[4] / tiles, "tiles_per_launch": a[5] / steps,
                              "wait_operands_cycles_per_tile": a[2] / tiles,
                              "of_which_first_k_steps": a[6] / tiles, "of_which_last_k_steps": a[7] / tiles,
                              "wait_accumulator_cycles_per_tile": a[3] / tiles,
                              "drain_cycles_per_accumulator": a[0] / max(a[1], 1)}), flush=True)
    lib.b200moe_gemm_set_tiling(0)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("cases", nargs="*", default=["skew:8192", "uni:16384"])
    ap.add_argument("--tilings", type=int, nargs="+", default=[1, 2], choices=[0, 1, 2, 3, 10, 11, 12, 13])
    ap.add_argument("--steps", type=int, default=15)
    ap.add_argument("--reps", type=int, default=3)
    ap.add_argument("--lib", default=None, help="another build of the library to load")
    ap.add_argument("--cycles", action="store_true")
    args = ap.parse_args()
    if not torch.cuda.is_available():
        raise SystemExit("gemmbench needs a CUDA device")
    if args.lib:
        _lib.LIB_PATH = Path(args.lib).resolve()
    cases = [(c.split(":")[0], int(c.split(":")[1])) for c in args.cases]
    dev = torch.device("cuda", 0)
    with torch.inference_mode():
        if args.cycles:
            for tiling in [t for t in args.tilings if t in (1, 2)] or [2]:
                run_cycles(cases, min(args.steps, 10), dev, tiling)
        else:
            run_tilings(cases, args.tilings, args.steps, args.reps, dev)


if __name__ == "__main__":
    main()
