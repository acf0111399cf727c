"""The CPU oracle against fixtures produced by the reference's own Python code
(tests/golden/make_golden.py).  This is what pins the oracle."""
import hashlib

import numpy as np
import pytest
import torch

from electrock_infer_b200.synthetic import MoEWorkload, WORKLOADS, make_inputs
from oracle import moe_oracle

ROUTER_CASES = ["normal", "skewed", "wide"]
ALIGN_CASES = ["uniform_t1000", "skewed_t600", "empty_experts", "single_token", "exact_blocks",
               "small_fp32_routing"]


def _digest(*tensors):
    h = hashlib.sha256()
    for t in tensors:
        a = t.detach().cpu().contiguous()
        if a.dtype == torch.bfloat16:
            a = a.view(torch.int16)
        h.update(a.numpy().tobytes())
    return h.hexdigest()


@pytest.mark.parametrize("case", ROUTER_CASES)
def test_router_matches_reference_torch_router(golden, case):
    g = golden["router"]
    logits = torch.from_numpy(g[f"{case}_logits"])
    w_raw, ids = moe_oracle.router_ref(logits, 2, renormalize=False)
    w_norm, ids2 = moe_oracle.router_ref(logits, 2, renormalize=True)
    assert np.array_equal(ids.numpy(), g[f"{case}_ids"])
    assert np.array_equal(ids2.numpy(), g[f"{case}_ids"])
    assert ids.dtype == torch.int32 and w_raw.dtype == torch.float32
    np.testing.assert_allclose(w_raw.numpy(), g[f"{case}_weights_raw"], rtol=0, atol=1e-7)
    np.testing.assert_allclose(w_norm.numpy(), g[f"{case}_weights_renorm"], rtol=0, atol=1e-7)


def test_router_tie_rule_is_lowest_index_first():
    logits = torch.tensor([[1.0, 1.0, 0.0, 0, 0, 0, 0, 0],
                           [0.0, 3.0, 3.0, 3.0, 0, 0, 0, 0],
                           [5.0, 0, 0, 0, 0, 0, 0, 5.0],
                           [0.0] * 8])
    _, ids = moe_oracle.router_ref(logits, 2, True)
    assert ids.tolist() == [[0, 1], [1, 2], [0, 7], [0, 1]]
    assert moe_oracle.tie_rows(logits).tolist() == [True, True, True, True]
    assert not moe_oracle.tie_rows(torch.arange(8.0).view(1, 8)).any()


@pytest.mark.parametrize("bs", [16, 64, 128])
@pytest.mark.parametrize("case", ALIGN_CASES)
def test_align_matches_reference_torch_golden(golden, case, bs):
    g = golden["align"]
    ids = g[f"{case}_ids"]
    want_sorted, want_eids, want_npp = (g[f"{case}_bs{bs}_sorted"], g[f"{case}_bs{bs}_expert_ids"],
                                        g[f"{case}_bs{bs}_npp"])
    for fn in (moe_oracle.align_ref, moe_oracle.align_ref_numpy):
        s, e, n, off = fn(ids, bs, 8)
        npp = int(n[0])
        assert npp == int(want_npp[0])
        assert off[-1] == npp and off[0] == 0
        # The reference golden returns exactly npp slots with -1 in the padding.
        assert np.array_equal(s[:npp], want_sorted)
        assert np.array_equal(e[: npp // bs], want_eids)
        assert (s[npp:] == -1).all() and (e[npp // bs:] == 0).all()
        cap, nblk = moe_oracle.align_sizes(ids.size, bs, 8)
        assert s.size == cap and e.size == nblk


def test_align_leaves_unwritten_slots_as_prefilled():
    ids = np.array([1, 1, 7], dtype=np.int32)
    s, e, n, _ = moe_oracle.align_ref(ids, 4, 8, prefill=-7)
    assert int(n[0]) == 8
    assert s[:8].tolist() == [0, 1, -7, -7, 2, -7, -7, -7]
    assert e[:2].tolist() == [1, 7]
    assert (s[8:] == -7).all()


def test_align_empty_input():
    for fn in (moe_oracle.align_ref, moe_oracle.align_ref_numpy):
        s, e, n, off = fn(np.zeros(0, dtype=np.int32), 64, 8)
        assert int(n[0]) == 0 and (s == -1).all() and (off == 0).all()


def test_layer_fp32_matches_reference_hf_block(golden):
    g = golden["layer"]
    wl = WORKLOADS["small_fp32"]
    inp = make_inputs(wl)
    assert _digest(inp["x"], inp["router_w"], inp["w13"], inp["w2"]) == str(g["small_fp32_inputs_sha256"])
    np.testing.assert_allclose(inp["logits"].numpy(), g["small_fp32_hf_block_logits"], atol=1e-5)
    out = moe_oracle.moe_block_ref(inp["x"], inp["w13"], inp["w2"], inp["logits"])
    np.testing.assert_allclose(out.numpy(), g["small_fp32_hf_block_out"], rtol=1e-4, atol=1e-5)


def test_layer_bf16_inputs_match_reference_hf_block(golden):
    g = golden["layer"]
    wl = MoEWorkload("tiny_bf16", 96, 256, 512, seed=7)
    inp = make_inputs(wl)
    assert _digest(inp["x"], inp["router_w"], inp["w13"], inp["w2"]) == str(g["tiny_bf16_inputs_sha256"])
    out = moe_oracle.moe_block_ref(inp["x"], inp["w13"], inp["w2"], inp["logits"])
    np.testing.assert_allclose(out.numpy(), g["tiny_bf16_hf_block_out_fp32"], rtol=1e-4, atol=1e-5)


def test_rounding_pipeline_matches_reference_fused_experts(golden):
    """fused_experts_ref restates every rounding point of the reference pipeline; the fixture is the
    reference pipeline itself with its Triton kernel interpreted on the CPU.  That interpreter
    truncates fp32 -> bf16 instead of rounding, so the comparison uses the same conversion; what is
    left is the accumulation order inside the dot products."""
    g = golden["layer"]
    inp = make_inputs(WORKLOADS["small_fp32"])
    want = torch.from_numpy(g["small_fp32_fused_experts_out"])
    out = moe_oracle.fused_experts_ref(inp["x"], inp["w13"], inp["w2"], inp["logits"],
                                       bf16_cast="truncate")
    st = moe_oracle.error_stats(out, want)
    assert st["rel_fro"] < 1e-3, st
    assert st["max_abs"] <= 2 ** -7, st  # one bf16 step at the output scale (|out| < 2)
    # With round-to-nearest (what a GPU does) the pipeline is about 3x closer to exact arithmetic
    # than with truncation; both stay within bf16 resolution of the exact block.
    exact = torch.from_numpy(g["small_fp32_hf_block_out"])
    rne = moe_oracle.fused_experts_ref(inp["x"], inp["w13"], inp["w2"], inp["logits"])
    assert moe_oracle.error_stats(rne, exact)["rel_fro"] < 5e-3
    assert moe_oracle.error_stats(want, exact)["rel_fro"] < 1.5e-2


def test_silu_and_moe_sum_formulas(golden):
    g = golden["ops"]
    x = torch.from_numpy(g["silu_in_bf16_bits"]).view(torch.bfloat16)
    want = torch.from_numpy(g["silu_out_bf16_bits"]).view(torch.bfloat16)
    got = moe_oracle.silu_and_mul_ref(x)
    # The reference's own test accepts atol = rtol = 1e-3 (test/example/test_silu.py:6-28).
    assert torch.allclose(got.float(), want.float(), atol=1e-3, rtol=1e-2)
    ms = torch.from_numpy(g["moe_sum_in_f16"])
    assert torch.equal(moe_oracle.moe_sum_ref(ms), torch.from_numpy(g["moe_sum_out_f16"]))
    inter = ms.permute(0, 2, 1).contiguous()
    assert torch.equal(moe_oracle.moe_sum_efficient_ref(inter), torch.from_numpy(g["moe_sum_out_f16"]))


# ------------------------------------------------------------------------- paged KV cache
def _kv_cases():
    import kv_cases  # tests/kv_cases.py (the tests directory is on sys.path under pytest)
    return kv_cases


@pytest.mark.parametrize("case", ["gqa4_bs32_bf16", "gqa8_bs16_f16", "mha_bs64_bf16", "gqa16_bs256_bf16"])
def test_paged_attention_oracle_matches_reference_cpu_golden(golden, case):
    """The fixture holds the output of the reference test's own CPU attention on contiguous K/V;
    the oracle reads the same K/V through the block table."""
    kc = _kv_cases()
    c = kc.attn_case(case)
    fx = golden["kv"]
    assert str(fx[f"attn_{case}_digest"]) == kc.digest(c["q"], c["k_cache"], c["v_cache"],
                                                        c["block_table"], c["context_lens"])
    out = moe_oracle.paged_attn_varlen_ref(c["q"], c["k_cache"], c["v_cache"], c["context_lens"],
                                           c["block_table"], c["scale"])
    assert np.array_equal(out.view(torch.int16).numpy(), fx[f"attn_{case}_out_bits"])


def test_paged_store_oracle_matches_reference_torch_and_triton_store(golden):
    kc = _kv_cases()
    c = kc.store_case()
    fx = golden["kv"]
    assert str(fx["store_digest"]) == kc.digest(c["key"], c["value"], c["k_cache"], c["v_cache"],
                                                c["slot_mapping"])
    k, v = moe_oracle.paged_store_kvcache_ref(c["key"], c["value"], c["k_cache"], c["v_cache"],
                                              c["slot_mapping"])
    assert np.array_equal(k.view(torch.int16).numpy(), fx["store_k_bits"])
    assert np.array_equal(v.view(torch.int16).numpy(), fx["store_v_bits"])
    # Negative slots are skipped (src/store_kv_cache.hip:28-31).
    slots = c["slot_mapping"].clone()
    slots[::3] = -1
    k2, v2 = moe_oracle.paged_store_kvcache_ref(c["key"], c["value"], c["k_cache"], c["v_cache"], slots)
    untouched = (k2 == 3.0).all(dim=-1).all(dim=-1).sum().item()
    assert untouched == c["k_cache"].shape[0] * c["k_cache"].shape[1] - int((slots >= 0).sum())


def _bits(t):
    return t.numpy() if t.dtype == torch.float32 else t.view(torch.int16).numpy()


@pytest.mark.parametrize("case", ["bf16_h4096", "bf16_h520", "f16_h1024", "f32_h768"])
def test_rms_norm_oracle_matches_reference_module(golden, case):
    """The fixture holds what the reference's ``RMSNorm.forward`` (layers/layernorm.py:45-57)
    returned, with and without a residual; the restatement must give the same bits."""
    from rmsnorm_cases import rmsnorm_inputs
    x, residual, weight, eps = rmsnorm_inputs(case)
    fx = golden["rmsnorm"]
    assert str(fx[f"{case}_digest"]) == _digest(x, residual, weight)
    y = moe_oracle.rms_norm_ref(x, weight, eps)
    y_res, new_res = moe_oracle.rms_norm_ref(x, weight, eps, residual)
    assert np.array_equal(_bits(y), fx[f"{case}_y"])
    assert np.array_equal(_bits(y_res), fx[f"{case}_y_with_residual"])
    if x.dtype == torch.float32:
        # fp32 only: the reference's no-op casts make its in-place scaling overwrite the tensor it
        # returns as the residual, which therefore equals its output.  The oracle (and the
        # kernels) return the sum for every dtype, as the 16-bit paths of the reference do.
        assert np.array_equal(fx[f"{case}_new_residual"], fx[f"{case}_y_with_residual"])
        assert torch.equal(new_res, x + residual)
    else:
        assert np.array_equal(_bits(new_res), fx[f"{case}_new_residual"])
