"""Paged KV-cache kernels on the GPU against the CPU oracle and the fixtures made by the
reference's own tests.

Store: bit-exact.  Decode attention: the reference test's bar is allclose(atol=1.6e-2, rtol=1e-2)
for bf16 and (1e-2, 1e-2) for fp16 against its fp32 CPU golden (test/example/test_paged_attn.py:78-82);
the bar here is tighter: |err| <= 4e-3 + 8e-3 * |ref| (bf16) and 1e-3 + 2e-3 * |ref| (fp16).
"""
import math

import numpy as np
import pytest
import torch

import kv_cases
from electrock_infer_b200 import _C, _lib
from oracle import moe_oracle

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
TOL = {torch.bfloat16: (4e-3, 8e-3), torch.float16: (1e-3, 2e-3)}


def close(got, want, dtype):
    atol, rtol = TOL[dtype]
    got, want = got.float().cpu(), want.float().cpu()
    bad = (got - want).abs() > atol + rtol * want.abs()
    return not bool(bad.any()), (got - want).abs().max().item()


def run_attn(c, num_splits=0):
    out = _C.paged_attn_varlen(c["q"].to(DEV), c["k_cache"].to(DEV), c["v_cache"].to(DEV), 0,
                               c["context_lens"].to(DEV), c["block_table"].to(DEV), c["scale"],
                               num_splits=num_splits)
    torch.cuda.synchronize()
    return out.cpu()


# ---------------------------------------------------------------------------------- store
def test_store_matches_reference_fixture(golden):
    c = kv_cases.store_case()
    k, v = c["k_cache"].to(DEV), c["v_cache"].to(DEV)
    _C.paged_store_kvcache(c["key"].to(DEV), c["value"].to(DEV), k, v, c["slot_mapping"].to(DEV))
    torch.cuda.synchronize()
    fx = golden["kv"]
    assert np.array_equal(k.cpu().view(torch.int16).numpy(), fx["store_k_bits"])
    assert np.array_equal(v.cpu().view(torch.int16).numpy(), fx["store_v_bits"])


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("tokens,kv_heads,head_dim,block_size,num_blocks",
                         [(1, 8, 128, 32, 4), (300, 8, 128, 256, 3), (1000, 2, 64, 16, 80),
                          (77, 1, 128, 32, 5), (513, 4, 256, 32, 20)])
def test_store_bit_exact_with_skips_and_strided_source(tokens, kv_heads, head_dim, block_size,
                                                       num_blocks, dtype):
    g = torch.Generator().manual_seed(tokens + kv_heads)
    row = kv_heads * head_dim
    # K and V as slices of one fused projection output: token stride 3 * row.
    qkv = torch.randn(tokens, 3 * row, generator=g).to(dtype)
    key = qkv[:, row:2 * row].view(tokens, kv_heads, head_dim)
    value = qkv[:, 2 * row:].view(tokens, kv_heads, head_dim)
    k_cache = torch.full((num_blocks, block_size, kv_heads, head_dim), 5.0, dtype=dtype)
    v_cache = torch.full((num_blocks, block_size, kv_heads, head_dim), -5.0, dtype=dtype)
    slots = torch.randperm(num_blocks * block_size, generator=g)[:tokens].to(torch.int32)
    slots[::7] = -1                                   # not cached
    want_k, want_v = moe_oracle.paged_store_kvcache_ref(key, value, k_cache, v_cache, slots)
    d_qkv = qkv.to(DEV)
    d_key = d_qkv[:, row:2 * row].view(tokens, kv_heads, head_dim)
    d_value = d_qkv[:, 2 * row:].view(tokens, kv_heads, head_dim)
    d_k, d_v = k_cache.to(DEV), v_cache.to(DEV)
    _C.paged_store_kvcache(d_key, d_value, d_k, d_v, slots.to(DEV))
    torch.cuda.synchronize()
    assert torch.equal(d_k.cpu(), want_k) and torch.equal(d_v.cpu(), want_v)


def test_store_skips_slots_beyond_the_cache():
    key = torch.ones(4, 2, 128, dtype=torch.bfloat16, device=DEV)
    k = torch.zeros(2, 16, 2, 128, dtype=torch.bfloat16, device=DEV)
    v = torch.zeros_like(k)
    slots = torch.tensor([0, 31, 32, 10 ** 6], dtype=torch.int32, device=DEV)
    _C.paged_store_kvcache(key, key, k, v, slots)
    torch.cuda.synchronize()
    assert k.view(32, -1).any(dim=1).sum().item() == 2 and v.view(32, -1).any(dim=1).sum().item() == 2


def test_store_argument_errors():
    k = torch.zeros(2, 16, 2, 128, dtype=torch.bfloat16, device=DEV)
    key = torch.zeros(4, 2, 128, dtype=torch.bfloat16, device=DEV)
    slots = torch.zeros(4, dtype=torch.int32, device=DEV)
    with pytest.raises(RuntimeError):
        _C.paged_store_kvcache(key, key, k, k.clone(), slots.long())
    with pytest.raises(RuntimeError):
        _C.paged_store_kvcache(key, key[:3], k, k.clone(), slots)
    with pytest.raises(RuntimeError):
        _C.paged_store_kvcache(key.cpu(), key.cpu(), k.cpu(), k.cpu(), slots.cpu())


# ------------------------------------------------------------------------ decode attention
@pytest.mark.parametrize("case", list(kv_cases.ATTN_CASES))
def test_attention_matches_reference_fixture(golden, case):
    c = kv_cases.attn_case(case)
    dtype = c["q"].dtype
    fx = golden["kv"]
    bits = torch.from_numpy(fx[f"attn_{case}_out_bits"].copy())
    want = bits.view(dtype)
    for splits in (1, 0, 3):
        ok, err = close(run_attn(c, splits), want, dtype)
        assert ok, (case, splits, err)


def make_case(batch, q_heads, kv_heads, block_size, lens, dtype, seed):
    g = torch.Generator().manual_seed(seed)
    max_blocks = max(1, max((n + block_size - 1) // block_size for n in lens))
    num_blocks = batch * max_blocks + 1
    q = torch.randn(batch, q_heads, 128, generator=g).to(dtype)
    k_cache = torch.randn(num_blocks, block_size, kv_heads, 128, generator=g).to(dtype)
    v_cache = torch.randn(num_blocks, block_size, kv_heads, 128, generator=g).to(dtype)
    table = torch.randperm(num_blocks, generator=g)[: batch * max_blocks].view(batch, max_blocks).to(torch.int32)
    return {"q": q, "k_cache": k_cache, "v_cache": v_cache, "block_table": table,
            "context_lens": torch.tensor(lens, dtype=torch.int32), "scale": 1.0 / math.sqrt(128)}


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("q_heads,kv_heads,block_size,lens,splits", [
    (32, 8, 256, [1, 15, 16, 17, 255, 256, 257, 1000], 0),     # Mixtral heads, engine block size
    (32, 8, 32, [700, 3, 64], 4),
    (8, 8, 16, [33, 200], 1),                                  # no grouping
    (12, 4, 48, [100, 47, 48, 49], 2),                         # group of 3, block size 48
    (16, 1, 64, [2048], 7),                                    # one long context, many splits
    (32, 8, 256, [0, 5, 0], 1),                                # empty contexts give zero rows
    (32, 8, 256, [0, 5, 0], 2),
])
def test_attention_against_oracle(q_heads, kv_heads, block_size, lens, splits, dtype):
    c = make_case(len(lens), q_heads, kv_heads, block_size, lens, dtype, seed=q_heads + len(lens))
    want = moe_oracle.paged_attn_varlen_ref(c["q"], c["k_cache"], c["v_cache"], c["context_lens"],
                                            c["block_table"], c["scale"])
    got = run_attn(c, splits)
    ok, err = close(got, want, dtype)
    assert ok, err
    for b, n in enumerate(lens):
        if n == 0:
            assert not got[b].any()


def test_attention_ignores_garbage_past_the_context():
    """Slots after the last token of a page may hold anything, NaN included."""
    c = make_case(3, 32, 8, 32, [40, 1, 31], torch.bfloat16, seed=9)
    want = moe_oracle.paged_attn_varlen_ref(c["q"], c["k_cache"], c["v_cache"], c["context_lens"],
                                            c["block_table"], c["scale"])
    for b, n in enumerate([40, 1, 31]):
        page = int(c["block_table"][b, n // 32]) if n % 32 else None
        if page is not None:
            c["k_cache"][page, n % 32:] = float("nan")
            c["v_cache"][page, n % 32:] = float("nan")
    got = run_attn(c, 1)
    ok, err = close(got, want, torch.bfloat16)
    assert ok and not torch.isnan(got.float()).any(), err


def test_attention_decode_batch_at_mixtral_shape():
    """128 sequences, 32 query / 8 KV heads, block size 256, contexts of 300-700 tokens; a
    sample of sequences is checked against the oracle."""
    g = torch.Generator().manual_seed(5)
    lens = torch.randint(300, 700, (128,), generator=g).tolist()
    c = make_case(128, 32, 8, 256, lens, torch.bfloat16, seed=6)
    got = run_attn(c, 0)
    pick = [0, 17, 101, 127]
    sub = {"q": c["q"][pick], "k_cache": c["k_cache"], "v_cache": c["v_cache"],
           "block_table": c["block_table"][pick], "context_lens": c["context_lens"][pick]}
    want = moe_oracle.paged_attn_varlen_ref(sub["q"], sub["k_cache"], sub["v_cache"],
                                            sub["context_lens"], sub["block_table"], c["scale"])
    ok, err = close(got[pick], want, torch.bfloat16)
    assert ok, err


def test_attention_argument_errors():
    c = make_case(2, 32, 8, 32, [10, 20], torch.bfloat16, seed=1)
    d = {k: (v.to(DEV) if torch.is_tensor(v) else v) for k, v in c.items()}
    with pytest.raises(RuntimeError):   # head_dim 64
        _C.paged_attn_varlen(d["q"][..., :64].contiguous(), d["k_cache"][..., :64].contiguous(),
                             d["v_cache"][..., :64].contiguous(), 0, d["context_lens"],
                             d["block_table"], 0.1)
    with pytest.raises(RuntimeError):   # fp32
        _C.paged_attn_varlen(d["q"].float(), d["k_cache"].float(), d["v_cache"].float(), 0,
                             d["context_lens"], d["block_table"], 0.1)
    with pytest.raises(RuntimeError):   # int64 lengths
        _C.paged_attn_varlen(d["q"], d["k_cache"], d["v_cache"], 0, d["context_lens"].long(),
                             d["block_table"], 0.1)
    lib = _lib.load()
    rc = lib.b200moe_paged_attn_varlen(d["q"].data_ptr(), d["k_cache"].data_ptr(), d["v_cache"].data_ptr(),
                                       d["q"].data_ptr(), d["block_table"].data_ptr(),
                                       d["context_lens"].data_ptr(), _lib.BF16, 2, 32, 8, 128,
                                       d["k_cache"].size(0), 32, 1, 0.1, 4, None, 0,
                                       torch.cuda.current_stream().cuda_stream)
    assert rc == -4  # workspace too small for num_splits = 4
