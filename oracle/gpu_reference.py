"""The reference's own MoE pipeline on the GPU: ``fused_experts`` of the staged reference package
(its Triton ``fused_moe_kernel`` compiled by Triton for this GPU, layers/moe/fused_moe.py:15-125,
:170-293) with the reference's CUDA ops from ``oracle/_ref/ref_ops`` bound as its ``_C`` module.
TEST INFRASTRUCTURE / BASELINE ONLY: nothing here is part of the product path.

    python oracle/gpu_reference.py --workload mixtral_prefill_t8192_skew [--tokens T] [--steps K]

Prints one JSON object: tokens/s of the reference pipeline (CUDA events around K calls after
warm-up) and its error, on a fixed 64-token sample, against the fp32 oracle on the same
bf16-valued tensors: the yardstick for "this library's error is at most 1.5 times the reference
pipeline's own".  Needs ``oracle/stage_reference_python.py`` and ``oracle/build_ref_ops.py`` to
have been run where the reference tree is available; prints {"unavailable": ...} otherwise.
"""
from __future__ import annotations

import argparse
import importlib
import importlib.util
import json
import sys
import types
from pathlib import Path

HERE = Path(__file__).resolve().parent
REPO = HERE.parent
REF_DIR = HERE / "_ref"
SAMPLE_TOKENS = 64


def load_reference_fused_moe():
    """Imports the staged reference package with the compiled reference ops as its ``_C``."""
    staged = REF_DIR / "reference_python"
    ops = sorted(REF_DIR.glob("ref_ops*.so"))
    if not (staged / "electrock_infer").is_dir():
        raise FileNotFoundError("oracle/_ref/reference_python is not staged")
    if not ops:
        raise FileNotFoundError("oracle/_ref/ref_ops is not built")
    spec = importlib.util.spec_from_file_location("ref_ops", ops[0])
    ref_ops = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(ref_ops)
    # The package's __init__ pulls in the engine (tokenizer, attention libraries); only the MoE
    # modules are needed here, so the package is entered as a bare namespace.
    pkg = types.ModuleType("electrock_infer")
    pkg.__path__ = [str(staged / "electrock_infer")]
    pkg._C = ref_ops
    sys.modules["electrock_infer"] = pkg
    sys.modules["electrock_infer._C"] = ref_ops
    return importlib.import_module("electrock_infer.layers.moe.fused_moe")


def measure(workload: str, tokens, steps: int, warmup: int) -> dict:
    import torch
    sys.path.insert(0, str(REPO))
    from dataclasses import replace

    from electrock_infer_b200.synthetic import WORKLOADS, make_inputs
    from oracle import moe_oracle
    ref = load_reference_fused_moe()
    wl = replace(WORKLOADS[workload], dtype=torch.bfloat16)
    if tokens:
        wl = replace(wl, num_tokens=tokens)
    dev = torch.device("cuda", 0)
    inp = make_inputs(wl, device=dev, device_rng=True)
    x0, logits = inp["x"], inp["logits"]

    def step():
        return ref.fused_experts(x0.clone(), inp["w13"], inp["w2"], logits, wl.top_k,
                                 renormalize=True, inplace=True)

    with torch.inference_mode():
        for _ in range(warmup):
            out = step()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            out = step()
        e1.record()
        torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / steps
    n = min(SAMPLE_TOKENS, wl.num_tokens)
    sample = torch.randperm(wl.num_tokens, generator=torch.Generator().manual_seed(0))[:n].to(dev)
    want = moe_oracle.moe_block_ref(x0[sample], inp["w13"], inp["w2"], logits[sample], wl.top_k, True)
    st = moe_oracle.error_stats(out[sample].float().cpu(), want)
    import triton
    return {"pipeline": "reference fused_experts: Triton fused_moe_kernel + reference CUDA ops",
            "workload": wl.name, "num_tokens": wl.num_tokens, "tokens_per_s": wl.num_tokens / (ms * 1e-3),
            "ms_per_step": ms, "steps": steps, "max_abs": st["max_abs"], "rel_fro": st["rel_fro"],
            "sample_tokens": n, "triton": triton.__version__}


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--workload", default="mixtral_prefill_t8192_skew")
    ap.add_argument("--tokens", type=int, default=None)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    args = ap.parse_args()
    try:
        res = measure(args.workload, args.tokens, args.steps, args.warmup)
    except FileNotFoundError as e:
        res = {"unavailable": str(e)}
    except Exception as e:  # the reference's JIT path failing on this GPU is a result, not a crash
        res = {"unavailable": f"{type(e).__name__}: {str(e)[:300]}"}
    print(json.dumps(res), flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
