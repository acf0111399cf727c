"""Generates the golden fixtures in this directory by running the reference's own Python code.

Usage (only where the reference tree is available; the fixtures themselves are committed):

    python tests/golden/make_golden.py /path/to/electrock-infer
    ELECTROCK_REFERENCE=/path/to/electrock-infer python tests/golden/make_golden.py

What is run, unmodified, from the reference tree:
  * ``topk_softmax_torch`` and ``fused_topk``      layers/moe/softmax_topk.py, layers/moe/fused_moe.py
  * ``moe_align_block_size_torch``                 test/example/test_align_block.py:6-69
  * ``MixtralSparseMoeBlock``                      test/example/verify_hf_moe.py:43-86
  * ``fused_experts`` with its Triton kernel under ``TRITON_INTERPRET=1`` (fp32 tensors)
  * ``cpu_attention_golden``                       test/example/test_paged_attn.py:24-52
  * ``store_kvcache_naive_torch`` and the Triton ``store_kvcache_triton`` (interpreted)
                                                   test/example/test_store_kvcache.py:6-72
  * ``RMSNorm`` (with and without residual)       layers/layernorm.py:5-57
``--only kv`` / ``--only rmsnorm`` regenerate just that fixture.
The reference's compiled module ``electrock_infer._C`` cannot be built here (it targets another
vendor's compiler), so a stand-in module provides the three ops ``fused_experts`` calls, written
from the reference's documented formulas (the same functions the oracle exposes).

Inputs are the seeded tensors of ``electrock_infer_b200.synthetic``; each fixture stores a
digest of its inputs so that a change of the generator is noticed.
"""
from __future__ import annotations

import contextlib
import hashlib
import importlib.util
import io
import os
import sys
import types
from pathlib import Path

os.environ.setdefault("TRITON_INTERPRET", "1")
sys.dont_write_bytecode = True

import numpy as np  # noqa: E402
import torch  # noqa: E402

HERE = Path(__file__).resolve().parent
REPO = HERE.parent.parent
sys.path.insert(0, str(REPO))

from electrock_infer_b200.synthetic import MoEWorkload, WORKLOADS, make_inputs  # noqa: E402
from oracle import moe_oracle  # noqa: E402


def digest(*tensors) -> str:
    h = hashlib.sha256()
    for t in tensors:
        a = t.detach().cpu().contiguous()
        if a.dtype == torch.bfloat16:
            a = a.view(torch.int16)
        h.update(a.numpy().tobytes())
    return h.hexdigest()


def load_reference(ref_root: Path):
    """Imports the reference package with a stand-in ``_C`` and loads its two test goldens."""
    sys.path.insert(0, str(ref_root))
    stub = types.ModuleType("electrock_infer._C")

    def silu_and_mul(out, input):  # noqa: A002
        out.copy_(moe_oracle.silu_and_mul_ref(input).view_as(out))

    def moe_sum(input, output):  # noqa: A002
        output.copy_(moe_oracle.moe_sum_ref(input))

    def moe_align_block_size(topk_ids, num_experts, block_size, sorted_ids, expert_ids, npp):
        s, e, n, _ = moe_oracle.align_ref(topk_ids.numpy(), block_size, num_experts)
        used = int(n[0])
        sorted_ids[:used] = torch.from_numpy(s[:used])
        expert_ids[: used // block_size] = torch.from_numpy(e[: used // block_size])
        npp[0] = used

    stub.silu_and_mul = silu_and_mul
    stub.moe_sum = moe_sum
    stub.moe_align_block_size = moe_align_block_size
    sys.modules["electrock_infer._C"] = stub

    def load(name, rel):
        spec = importlib.util.spec_from_file_location(name, ref_root / rel)
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        return mod

    from electrock_infer.layers.moe import fused_moe  # noqa: E402
    from electrock_infer.layers.moe.softmax_topk import topk_softmax_torch  # noqa: E402
    hf = load("ref_verify_hf_moe", "test/example/verify_hf_moe.py")
    al = load("ref_test_align_block", "test/example/test_align_block.py")
    load_reference.load = load
    return fused_moe, topk_softmax_torch, hf, al


def make_kv() -> None:
    """Paged KV-cache fixtures: outputs of the reference tests' own CPU goldens on the seeded
    inputs of tests/kv_cases.py."""
    sys.path.insert(0, str(REPO / "tests"))
    import kv_cases
    pa = load_reference.load("ref_test_paged_attn", "test/example/test_paged_attn.py")
    sk = load_reference.load("ref_test_store_kvcache", "test/example/test_store_kvcache.py")
    kv = {}
    for name in kv_cases.ATTN_CASES:
        c = kv_cases.attn_case(name)
        out = pa.cpu_attention_golden(c["q"], c["k"], c["v"], c["context_lens"], c["scale"])
        mine = moe_oracle.paged_attn_varlen_ref(c["q"], c["k_cache"], c["v_cache"], c["context_lens"],
                                                c["block_table"], c["scale"])
        assert torch.equal(out, mine), f"{name}: oracle restatement differs from the reference golden"
        kv[f"attn_{name}_digest"] = np.array(kv_cases.digest(c["q"], c["k_cache"], c["v_cache"],
                                                             c["block_table"], c["context_lens"]))
        kv[f"attn_{name}_out_bits"] = out.view(torch.int16).numpy()
    c = kv_cases.store_case()
    k1, v1 = c["k_cache"].clone(), c["v_cache"].clone()
    sk.store_kvcache_naive_torch(c["key"], c["value"], k1, v1, c["slot_mapping"])
    k2, v2 = c["k_cache"].clone(), c["v_cache"].clone()
    sk.store_kvcache_triton(c["key"], c["value"], k2, v2, c["slot_mapping"])  # interpreted on CPU
    assert torch.equal(k1, k2) and torch.equal(v1, v2), "the reference's two store paths disagree"
    kv["store_digest"] = np.array(kv_cases.digest(c["key"], c["value"], c["k_cache"], c["v_cache"],
                                                  c["slot_mapping"]))
    kv["store_k_bits"] = k1.view(torch.int16).numpy()
    kv["store_v_bits"] = v1.view(torch.int16).numpy()
    np.savez_compressed(HERE / "kv.npz", **kv)


def make_rmsnorm() -> None:
    """Outputs of the reference's ``RMSNorm.forward`` (layers/layernorm.py:45-57), with and without
    a residual, on seeded inputs; the oracle restatement must reproduce them bit for bit."""
    from electrock_infer.layers.layernorm import RMSNorm
    sys.path.insert(0, str(REPO / "tests"))
    from rmsnorm_cases import RMSNORM_CASES, rmsnorm_inputs
    out = {}
    for name, (rows, hidden, dtype, eps) in RMSNORM_CASES.items():
        x, residual, weight, eps = rmsnorm_inputs(name)
        norm = RMSNorm(hidden, eps=eps).to(dtype)
        with torch.no_grad():
            norm.weight.copy_(weight)
            y = norm(x.clone())
            y_res, new_res = norm(x.clone(), residual.clone())
        mine = moe_oracle.rms_norm_ref(x, weight, eps)
        mine_res, mine_new = moe_oracle.rms_norm_ref(x, weight, eps, residual)
        assert torch.equal(y, mine) and torch.equal(y_res, mine_res), \
            f"{name}: oracle restatement differs from the reference RMSNorm"
        if dtype == torch.float32:
            # In fp32 the reference's casts are no-ops, so its in-place scaling also rewrites the
            # tensor it returns as the new residual (layers/layernorm.py:36-41): the residual it
            # hands back IS the normalised output.  The 16-bit dtypes (what the model runs in)
            # return the sum.  The fixture records what the reference returns; the oracle and the
            # kernels return the sum for every dtype.
            assert torch.equal(new_res, y_res)
            assert torch.equal(mine_new, x + residual)
        else:
            assert torch.equal(new_res, mine_new), f"{name}: residual differs from the reference"
        as_bits = (lambda t: t.view(torch.int16).numpy()) if dtype != torch.float32 else (lambda t: t.numpy())
        out[f"{name}_digest"] = np.array(digest(x, residual, weight))
        out[f"{name}_y"] = as_bits(y)
        out[f"{name}_y_with_residual"] = as_bits(y_res)
        out[f"{name}_new_residual"] = as_bits(new_res)
    np.savez_compressed(HERE / "rmsnorm.npz", **out)


def run_hf_block(hf, inputs, wl: MoEWorkload, dtype=torch.float32):
    cfg = {"hidden_size": wl.hidden, "intermediate_size": wl.inter, "num_experts": wl.num_experts,
           "top_k": wl.top_k, "hidden_act": "silu"}
    block = hf.MixtralSparseMoeBlock(cfg).to(dtype).eval()
    I = wl.inter
    with torch.no_grad():
        block.gate.weight.copy_(inputs["router_w"].to(dtype))
        for e in range(wl.num_experts):
            block.experts[e].w1.weight.copy_(inputs["w13"][e, :I].to(dtype))
            block.experts[e].w3.weight.copy_(inputs["w13"][e, I:].to(dtype))
            block.experts[e].w2.weight.copy_(inputs["w2"][e].to(dtype))
        with contextlib.redirect_stdout(io.StringIO()):
            out, logits = block(inputs["x"].to(dtype).view(1, wl.num_tokens, wl.hidden))
    return out.view(wl.num_tokens, wl.hidden), logits


def main() -> None:
    where = (sys.argv[1] if len(sys.argv) > 1 and not sys.argv[1].startswith("--")
             else os.environ.get("ELECTROCK_REFERENCE"))
    if not where or not (Path(where) / "electrock_infer").is_dir():
        raise SystemExit("give the path of the electrock-infer source tree as the first argument "
                         "or in ELECTROCK_REFERENCE")
    ref_root = Path(where)
    fused_moe, topk_softmax_torch, hf, al = load_reference(ref_root)
    if "--only" in sys.argv:
        which = sys.argv[sys.argv.index("--only") + 1]
        {"kv": make_kv, "rmsnorm": make_rmsnorm}[which]()
        print(f"{which}.npz", (HERE / f"{which}.npz").stat().st_size, "bytes")
        return

    # ------------------------------------------------------------------ router
    router = {}
    g = torch.Generator().manual_seed(11)
    cases = {
        "normal": torch.randn(1000, 8, generator=g),
        "skewed": torch.randn(777, 8, generator=g) + torch.tensor(
            [2.0, 1.0, 0.5, 0.0, 0.0, -0.5, -1.0, -2.0]),
        "wide": torch.randn(513, 8, generator=g) * 8.0,
    }
    for name, logits in cases.items():
        w_raw, ids = topk_softmax_torch(logits, 2)
        w_norm, ids2 = fused_moe.fused_topk(torch.empty(logits.shape[0], 1), logits, 2, True)
        assert torch.equal(ids, ids2)
        assert not moe_oracle.tie_rows(logits).any(), "fixture logits must be tie-free"
        router[f"{name}_logits"] = logits.numpy()
        router[f"{name}_weights_raw"] = w_raw.numpy()
        router[f"{name}_weights_renorm"] = w_norm.numpy()
        router[f"{name}_ids"] = ids.numpy()
    np.savez_compressed(HERE / "router.npz", **router)

    # ------------------------------------------------------------------ alignment
    align = {}
    g = torch.Generator().manual_seed(12)
    id_cases = {
        "uniform_t1000": torch.randint(0, 8, (2000,), generator=g),
        "skewed_t600": torch.multinomial(torch.tensor([8., 4, 2, 1, 1, .5, .25, .1]), 1200, True,
                                         generator=g),
        "empty_experts": torch.randint(0, 3, (300,), generator=g) * 3,  # experts 0, 3, 6 only
        "single_token": torch.tensor([5, 2]),
        "exact_blocks": torch.arange(8).repeat_interleave(64)[torch.randperm(512, generator=g)],
    }
    c0 = make_inputs(WORKLOADS["small_fp32"])
    _, c0_ids = fused_moe.fused_topk(c0["x"], c0["logits"], 2, True)
    id_cases["small_fp32_routing"] = c0_ids.reshape(-1).long()
    for name, ids in id_cases.items():
        for bs in (16, 64, 128):
            s, e, n = al.moe_align_block_size_torch(ids.long(), 8, bs)
            align[f"{name}_bs{bs}_sorted"] = s.numpy().astype(np.int32)
            align[f"{name}_bs{bs}_expert_ids"] = e.numpy().astype(np.int32)
            align[f"{name}_bs{bs}_npp"] = n.numpy().astype(np.int32)
        align[f"{name}_ids"] = ids.numpy().astype(np.int32)
    np.savez_compressed(HERE / "align.npz", **align)

    # ------------------------------------------------------------------ whole layer
    layer = {}
    wl0 = WORKLOADS["small_fp32"]
    out0, logits0 = run_hf_block(hf, c0, wl0)
    layer["small_fp32_inputs_sha256"] = np.array(digest(c0["x"], c0["router_w"], c0["w13"], c0["w2"]))
    layer["small_fp32_hf_block_out"] = out0.numpy()
    layer["small_fp32_hf_block_logits"] = logits0.detach().numpy()
    # The reference pipeline itself (Triton kernel interpreted on the CPU, fp32 tensors).
    fe = fused_moe.fused_experts(c0["x"].clone(), c0["w13"], c0["w2"], c0["logits"], 2,
                                 renormalize=True, inplace=False)
    layer["small_fp32_fused_experts_out"] = fe.numpy()

    wl1 = MoEWorkload("tiny_bf16", 96, 256, 512, seed=7)
    c1 = make_inputs(wl1)
    out1, _ = run_hf_block(hf, c1, wl1, torch.float32)  # fp32 math on bf16-valued tensors
    layer["tiny_bf16_inputs_sha256"] = np.array(digest(c1["x"], c1["router_w"], c1["w13"], c1["w2"]))
    layer["tiny_bf16_hf_block_out_fp32"] = out1.numpy()
    np.savez_compressed(HERE / "layer.npz", **layer)

    # ------------------------------------------------------------------ activation / sum formulas
    # The reference tests these two ops against torch expressions (test/example/test_silu.py:6-28,
    # test/example/test_moe_sum.py:8-11); evaluate exactly those expressions.
    ops = {}
    g = torch.Generator().manual_seed(13)
    xs = torch.randn(64, 2 * 224, generator=g).to(torch.bfloat16)
    d = xs.shape[-1] // 2
    ops["silu_in_bf16_bits"] = xs.view(torch.int16).numpy()
    ops["silu_out_bf16_bits"] = (torch.nn.functional.silu(xs[..., :d]) * xs[..., d:]).view(
        torch.int16).numpy()
    ms = torch.randn(48, 2, 320, generator=g).to(torch.float16)
    ops["moe_sum_in_f16"] = ms.numpy()
    ops["moe_sum_out_f16"] = torch.sum(ms, dim=1).numpy()
    np.savez_compressed(HERE / "ops.npz", **ops)
    make_kv()
    make_rmsnorm()

    for f in sorted(HERE.glob("*.npz")):
        print(f.name, f.stat().st_size, "bytes")


if __name__ == "__main__":
    main()
