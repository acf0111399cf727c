"""Seeded inputs of the paged KV-cache tests, shared by the fixture generator
(``tests/golden/make_golden.py``) and the tests, so that the fixtures only need to hold the
reference's outputs and a digest of the inputs."""
from __future__ import annotations

import hashlib
import math

import torch

ATTN_CASES = {
    # name: (dtype, q_heads, kv_heads, block_size, context lengths, seed)
    # The reference's own test uses 16 query / 4 KV heads, block size 32 and context length 100
    # (test/example/test_paged_attn.py:88-94); contexts here also end mid-page, at a page edge
    # and after a single token.
    "gqa4_bs32_bf16": (torch.bfloat16, 16, 4, 32, [100, 1, 33, 64, 96, 17], 101),
    "gqa8_bs16_f16": (torch.float16, 8, 1, 16, [5, 48, 17, 1], 102),
    "mha_bs64_bf16": (torch.bfloat16, 2, 2, 64, [130, 64, 7], 103),
    "gqa16_bs256_bf16": (torch.bfloat16, 16, 1, 256, [300, 256, 11], 104),
}
HEAD_DIM = 128


def digest(*tensors) -> str:
    h = hashlib.sha256()
    for t in tensors:
        a = t.detach().cpu().contiguous()
        if a.dtype in (torch.bfloat16, torch.float16):
            a = a.view(torch.int16)
        h.update(a.numpy().tobytes())
    return h.hexdigest()


def attn_case(name: str) -> dict:
    """Query, contiguous K/V ``[batch, kv_heads, max_len, 128]`` (what the reference's CPU golden
    takes) and the same K/V laid out in pages that are dealt out in a shuffled physical order."""
    dtype, q_heads, kv_heads, block_size, lens, seed = ATTN_CASES[name]
    g = torch.Generator().manual_seed(seed)
    batch = len(lens)
    max_blocks = max((n + block_size - 1) // block_size for n in lens)
    max_len = max_blocks * block_size
    q = torch.randn(batch, q_heads, HEAD_DIM, generator=g).to(dtype)
    k = torch.randn(batch, kv_heads, max_len, HEAD_DIM, generator=g).to(dtype)
    v = torch.randn(batch, kv_heads, max_len, HEAD_DIM, generator=g).to(dtype)
    num_blocks = batch * max_blocks + 3
    order = torch.randperm(num_blocks, generator=g).tolist()
    # Unused slots of the caches hold large values: reading past a context would show.
    k_cache = torch.full((num_blocks, block_size, kv_heads, HEAD_DIM), 1000.0, dtype=dtype)
    v_cache = torch.full((num_blocks, block_size, kv_heads, HEAD_DIM), -1000.0, dtype=dtype)
    block_table = torch.full((batch, max_blocks), -1, dtype=torch.int32)
    nxt = 0
    for b, n in enumerate(lens):
        for i in range((n + block_size - 1) // block_size):
            phys = order[nxt]
            nxt += 1
            block_table[b, i] = phys
            lo, hi = i * block_size, min((i + 1) * block_size, n)
            k_cache[phys, : hi - lo] = k[b, :, lo:hi].transpose(0, 1)
            v_cache[phys, : hi - lo] = v[b, :, lo:hi].transpose(0, 1)
    return {"q": q, "k": k, "v": v, "k_cache": k_cache, "v_cache": v_cache,
            "block_table": block_table, "context_lens": torch.tensor(lens, dtype=torch.int32),
            "scale": 1.0 / math.sqrt(HEAD_DIM)}


def store_case() -> dict:
    """New key/value rows, caches with a recognisable fill and a slot mapping that visits the
    slots in a shuffled order."""
    g = torch.Generator().manual_seed(105)
    tokens, kv_heads, block_size, num_blocks = 37, 2, 16, 5
    key = torch.randn(tokens, kv_heads, HEAD_DIM, generator=g).to(torch.bfloat16)
    value = torch.randn(tokens, kv_heads, HEAD_DIM, generator=g).to(torch.bfloat16)
    k_cache = torch.full((num_blocks, block_size, kv_heads, HEAD_DIM), 3.0, dtype=torch.bfloat16)
    v_cache = torch.full((num_blocks, block_size, kv_heads, HEAD_DIM), -3.0, dtype=torch.bfloat16)
    slots = torch.randperm(num_blocks * block_size, generator=g)[:tokens].to(torch.int32)
    return {"key": key, "value": value, "k_cache": k_cache, "v_cache": v_cache, "slot_mapping": slots}
