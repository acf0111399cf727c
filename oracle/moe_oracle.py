"""CPU oracle of the Mixtral MoE hot path.  TEST INFRASTRUCTURE ONLY.

Nothing in the product package imports this module: it exists so that tests, the smoke check and
the CPU-baseline leg of the benchmark can compare the CUDA path with an independent restatement
of the reference's algorithm.  Every function names the electrock-infer source it follows.

Pinning: the functions here are checked against vectors produced by the reference's own Python
code (``tests/golden/make_golden.py`` imports it from the reference tree and writes
``tests/golden/*.npz``): the torch router, the pure-torch alignment golden of
test/example/test_align_block.py, the HF-style block of test/example/verify_hf_moe.py and the
reference ``fused_experts`` pipeline run through the Triton interpreter.  The reference's CUDA
``topk_softmax`` kernel and ``moe_sum_efficient`` have no test of their own in the reference
(parity for those two is pinned only against the torch formulas below).

Integer work is numpy / plain C (``align_oracle.c``); floating-point work uses torch on the CPU
because the reference's own CPU path is torch and its rounding rules for 16-bit types are the
ones to reproduce.
"""
from __future__ import annotations

import ctypes
import subprocess
from pathlib import Path
from typing import Optional, Tuple

import numpy as np
import torch

_HERE = Path(__file__).resolve().parent
_LIB = _HERE / "_build" / "liboracle.so"
_clib = None


def build_c_oracle(force: bool = False) -> Path:
    """Compiles ``align_oracle.c`` with gcc (see the Makefile beside it)."""
    src = _HERE / "align_oracle.c"
    if force or not _LIB.exists() or _LIB.stat().st_mtime < src.stat().st_mtime:
        _LIB.parent.mkdir(exist_ok=True)
        subprocess.run(["gcc", "-O2", "-Wall", "-shared", "-fPIC", "-o", str(_LIB), str(src)],
                       check=True)
    return _LIB


def _c() -> ctypes.CDLL:
    global _clib
    if _clib is None:
        _clib = ctypes.CDLL(str(build_c_oracle()))
        _clib.oracle_align_block_size.restype = ctypes.c_int
        _clib.oracle_align_block_size.argtypes = [
            ctypes.c_void_p, ctypes.c_int64, ctypes.c_int, ctypes.c_int, ctypes.c_void_p,
            ctypes.c_int64, ctypes.c_void_p, ctypes.c_int64, ctypes.c_void_p, ctypes.c_void_p]
    return _clib


# --------------------------------------------------------------------------------------- router
def router_ref(logits: torch.Tensor, topk: int = 2,
               renormalize: bool = True) -> Tuple[torch.Tensor, torch.Tensor]:
    """softmax in fp32 -> the ``topk`` largest, largest first -> optional renormalisation.

    Follows layers/moe/softmax_topk.py:23-29 and layers/moe/fused_moe.py:161-162.  Ties are
    broken towards the lower expert index, the rule of src/topk_softmax_kernels.cu:39,47
    (``torch.topk`` leaves the order of equal values unspecified).  Returns
    ``(weights f32 [T, topk], ids i32 [T, topk])``.
    """
    probs = torch.softmax(logits.detach().cpu().float(), dim=-1)
    # Stable descending sort == lowest index first among equals.
    order = torch.sort(probs, dim=-1, descending=True, stable=True).indices[:, :topk]
    weights = torch.gather(probs, 1, order)
    if renormalize:
        weights = weights / weights.sum(dim=-1, keepdim=True)
    return weights, order.to(torch.int32)


def gate_logits_ref(x: torch.Tensor, gate_w: torch.Tensor, round_bf16: bool = True) -> torch.Tensor:
    """Router logits of the reference block: ``gate(hidden_states)`` with a bias-free linear layer
    (models/mixtral.py:59; layers/linear.py:53-54).  Computed in fp32 from the stored values; the
    reference's bf16 layer returns them rounded to bf16 (``round_bf16``)."""
    logits = x.detach().cpu().float() @ gate_w.detach().cpu().float().T
    return logits.to(torch.bfloat16).float() if round_bf16 else logits


def tie_rows(logits: torch.Tensor, topk: int = 2) -> torch.Tensor:
    """Boolean mask of rows where the top-k *set or order* is decided by an exact tie, i.e. where
    two implementations with different tie rules may legitimately disagree."""
    vals = torch.sort(logits.detach().cpu().float(), dim=-1, descending=True).values
    return (vals[:, : topk] == vals[:, 1: topk + 1]).any(dim=-1)


# ------------------------------------------------------------------------------------ alignment
def align_sizes(numel: int, block_size: int, num_experts: int) -> Tuple[int, int]:
    """Buffer sizes of the reference wrapper (layers/moe/moe_align_block_size.py:32,41)."""
    cap = numel + num_experts * (block_size - 1)
    return cap, (cap + block_size - 1) // block_size


def align_ref(topk_ids, block_size: int, num_experts: int, prefill: int = -1):
    """Token alignment through the plain-C oracle, with the reference wrapper's allocation and
    prefill rules (sorted ids prefilled with ``-1``, expert ids zero-filled;
    layers/moe/moe_align_block_size.py:32-46).  Returns numpy arrays
    ``(sorted_token_ids, expert_ids, num_tokens_post_pad, expert_offsets)``."""
    ids = np.ascontiguousarray(np.asarray(topk_ids).reshape(-1).astype(np.int64))
    cap, nblk = align_sizes(ids.size, block_size, num_experts)
    sorted_ids = np.full(cap, prefill, dtype=np.int32)
    expert_ids = np.zeros(nblk, dtype=np.int32)
    npp = np.zeros(1, dtype=np.int32)
    offsets = np.zeros(num_experts + 1, dtype=np.int32)
    rc = _c().oracle_align_block_size(
        ids.ctypes.data, ids.size, num_experts, block_size, sorted_ids.ctypes.data, cap,
        expert_ids.ctypes.data, nblk, npp.ctypes.data, offsets.ctypes.data)
    if rc != 0:
        raise RuntimeError(f"oracle_align_block_size failed with {rc}")
    return sorted_ids, expert_ids, npp, offsets


def align_ref_numpy(topk_ids, block_size: int, num_experts: int, prefill: int = -1):
    """The same contract written with numpy primitives (stable argsort), independent of the C
    code; used to cross-check the two restatements against each other."""
    ids = np.asarray(topk_ids).reshape(-1).astype(np.int64)
    cap, nblk = align_sizes(ids.size, block_size, num_experts)
    valid = (ids >= 0) & (ids < num_experts)
    cnt = np.bincount(ids[valid], minlength=num_experts)
    padded = (cnt + block_size - 1) // block_size * block_size
    offsets = np.concatenate([[0], np.cumsum(padded)]).astype(np.int32)
    sorted_ids = np.full(cap, prefill, dtype=np.int32)
    expert_ids = np.zeros(nblk, dtype=np.int32)
    idx = np.nonzero(valid)[0]
    order = idx[np.argsort(ids[idx], kind="stable")]
    start = 0
    for e in range(num_experts):
        sorted_ids[offsets[e]: offsets[e] + cnt[e]] = order[start: start + cnt[e]]
        expert_ids[offsets[e] // block_size: offsets[e + 1] // block_size] = e
        start += cnt[e]
    return sorted_ids, expert_ids, np.array([offsets[-1]], dtype=np.int32), offsets


# ---------------------------------------------------------------------------- activation / sum
def silu_and_mul_ref(x: torch.Tensor) -> torch.Tensor:
    """``out[..., j] = cast(silu_f32(x[..., j])) * x[..., d + j]`` with the product taken in the
    element type (src/activation_kernels.cu:33-43; fp32: :74-92).  The CUDA kernels use the fast
    exponential for 16-bit types, so agreement with this function is to within one unit in the
    last place of the element type, not bit-exact."""
    x = x.detach().cpu()
    d = x.shape[-1] // 2
    gate, up = x[..., :d], x[..., d:]
    g32 = gate.float()
    silu = (g32 / (1.0 + torch.exp(-g32))).to(x.dtype)
    return silu * up  # torch multiplies 16-bit CPU tensors in fp32 and rounds once


def moe_sum_ref(x: torch.Tensor) -> torch.Tensor:
    """``[T, 2, H] -> [T, H]``: ``(0 + x[:, 0]) + x[:, 1]`` in the element type
    (src/moe_sum.cu:35-41)."""
    x = x.detach().cpu()
    acc = torch.zeros_like(x[:, 0])
    for k in range(x.shape[1]):
        acc = acc + x[:, k]
    return acc


def moe_sum_efficient_ref(x: torch.Tensor) -> torch.Tensor:
    """``[T, H, 2] -> [T, H]``: sum of the two adjacent values (src/moe_sum_efficient.cu:33-46)."""
    x = x.detach().cpu()
    return x[..., 0] + x[..., 1]


def moe_sum_ranks_ref(x: torch.Tensor) -> torch.Tensor:
    """``[R, T, 2, H] -> [T, H]``: the combine of the tensor-parallel layer when the ranks' partial
    rows meet in one buffer.  Each rank's two rows are summed and rounded to the element type as
    ``moe_sum`` does on that rank (the reference's ranks round their partial result before the
    all-reduce, layers/moe/fused_moe.py:291, layers/moe/mixtral_moe.py:114-116); the per-rank
    sums are then added in fp32 in rank order and rounded once.  For two ranks that is exactly the
    correctly rounded sum of the two partial results, i.e. what the all-reduce returns."""
    x = x.detach().cpu()
    acc = torch.zeros(x.shape[1], x.shape[3], dtype=torch.float32)
    for r in range(x.shape[0]):
        acc = acc + moe_sum_ref(x[r]).to(torch.float32)
    return acc.to(x.dtype)


def paged_store_kvcache_ref(key: torch.Tensor, value: torch.Tensor, k_cache: torch.Tensor,
                            v_cache: torch.Tensor, slot_mapping: torch.Tensor):
    """Returns copies of the caches ``[blocks, block_size, kv_heads, head_dim]`` with token ``i``'s
    key/value rows written to slot ``slot_mapping[i]`` (block ``slot // block_size``, offset
    ``slot % block_size``); negative slots are skipped (src/store_kv_cache.hip:26-31; the torch loop
    of test/example/test_store_kvcache.py:6-28 is the same copy)."""
    k_out, v_out = k_cache.detach().cpu().clone(), v_cache.detach().cpu().clone()
    block_size = k_out.shape[1]
    for i, slot in enumerate(slot_mapping.detach().cpu().tolist()):
        if slot < 0:
            continue
        k_out[slot // block_size, slot % block_size] = key[i].detach().cpu()
        v_out[slot // block_size, slot % block_size] = value[i].detach().cpu()
    return k_out, v_out


def paged_attn_varlen_ref(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                          context_lens: torch.Tensor, block_table: torch.Tensor,
                          softmax_scale: float) -> torch.Tensor:
    """Decode attention over the paged cache in fp32, result cast to the dtype of ``q``: per
    sequence and query head ``softmax(scale * q K^T) V`` over the first ``context_lens[b]`` tokens,
    query head ``h`` reading KV head ``h // (q_heads // kv_heads)`` — the arithmetic of the
    reference's CPU golden (test/example/test_paged_attn.py:24-52), with K and V collected from
    the pages the block table names instead of taken as contiguous tensors.  An empty context
    gives a zero row."""
    q, k_cache, v_cache = q.detach().cpu(), k_cache.detach().cpu(), v_cache.detach().cpu()
    batch, q_heads, _ = q.shape
    block_size, kv_heads = k_cache.shape[1], k_cache.shape[2]
    group = q_heads // kv_heads
    out = torch.zeros(q.shape, dtype=torch.float32)
    for b in range(batch):
        n = int(context_lens[b])
        if n <= 0:
            continue
        pages = block_table[b, : (n + block_size - 1) // block_size].long()
        k = k_cache[pages].reshape(-1, kv_heads, k_cache.shape[3])[:n].float()
        v = v_cache[pages].reshape(-1, kv_heads, v_cache.shape[3])[:n].float()
        for h in range(q_heads):
            s = (q[b, h].float() @ k[:, h // group].T) * softmax_scale
            out[b, h] = torch.softmax(s, dim=-1) @ v[:, h // group]
    return out.to(q.dtype)


def rms_norm_ref(x: torch.Tensor, weight: torch.Tensor, eps: float,
                 residual: Optional[torch.Tensor] = None):
    """RMSNorm, optionally after a residual add, as the reference runs it
    (layers/layernorm.py:17-43): sum and variance in fp32, normalised value cast to the element type,
    then multiplied by the weight in the element type.  Returns ``y`` or ``(y, new_residual)``."""
    orig = x.dtype
    xf = x.detach().cpu().to(torch.float32)
    new_res = None
    if residual is not None:
        xf = xf + residual.detach().cpu().to(torch.float32)
        new_res = xf.to(orig)
    var = xf.pow(2).mean(dim=-1, keepdim=True)
    y = (xf * torch.rsqrt(var + eps)).to(orig) * weight.detach().cpu().to(orig)
    return y if residual is None else (y, new_res)


# ------------------------------------------------------------------------------------ the layer
def moe_block_ref(x: torch.Tensor, w13: torch.Tensor, w2: torch.Tensor, logits: torch.Tensor,
                  topk: int = 2, renormalize: bool = True,
                  compute_dtype: torch.dtype = torch.float32) -> torch.Tensor:
    """Per-expert loop of the reference's torch golden (``MixtralSparseMoeBlock``,
    test/example/verify_hf_moe.py:59-86): route, then for every expert gather its tokens, apply
    ``w2(silu(w1 x) * w3 x)``, scale by the routing weight and ``index_add_`` into the output.

    ``w13 [E, 2I, H]`` holds w1 (gate) rows first, then w3 (up) rows; ``w2 [E, H, I]``.
    With ``compute_dtype=float32`` on bf16-valued inputs this is the fp32 reference the CUDA layer
    is judged against; with ``bfloat16`` it reproduces the reference's CPU timing path.
    """
    x = x.detach().cpu()
    weights, ids = router_ref(logits, topk, renormalize)
    num_experts, inter_x2, _ = w13.shape
    inter = inter_x2 // 2
    xc = x.to(compute_dtype)
    weights = weights.to(compute_dtype)
    out = torch.zeros_like(xc)
    ids64 = ids.long()
    for e in range(num_experts):
        tok, slot = torch.nonzero(ids64 == e, as_tuple=True)
        if tok.numel() == 0:
            continue
        we = w13[e].detach().cpu().to(compute_dtype)
        cur = xc[tok]
        h = torch.nn.functional.silu(cur @ we[:inter].T) * (cur @ we[inter:].T)
        y = h @ w2[e].detach().cpu().to(compute_dtype).T
        out.index_add_(0, tok, y * weights[tok, slot].unsqueeze(1))
    return out


def _to_bf16(t: torch.Tensor, mode: str) -> torch.Tensor:
    """fp32 -> bf16-valued fp32, rounding to nearest even (what a GPU cast does) or truncating
    (what the Triton 3.6 CPU interpreter does for ``.to(tl.bfloat16)``)."""
    t = t.float().contiguous()
    if mode == "rne":
        return t.to(torch.bfloat16).float()
    if mode == "truncate":
        return (t.view(torch.int32) & ~0xFFFF).view(torch.float32)
    raise ValueError(mode)


def fused_experts_ref(x: torch.Tensor, w13: torch.Tensor, w2: torch.Tensor, logits: torch.Tensor,
                      topk: int = 2, renormalize: bool = True,
                      bf16_cast: str = "rne") -> torch.Tensor:
    """The reference pipeline with every rounding point it has (layers/moe/fused_moe.py:250-291):
    GEMM1 fp32 accumulate -> bf16 (:120, compute_type is hard-coded bf16 at :254) -> stored in the
    tensor dtype; SiLU in fp32 -> element type -> product in the element type; GEMM2 fp32
    accumulate x fp32 routing weight -> bf16 (:116-120); sum of the two experts in the element
    type.  Used to measure how far the reference's own result is from exact arithmetic.
    ``bf16_cast="truncate"`` reproduces the reference run under the Triton CPU interpreter, whose
    bf16 conversion drops the low mantissa bits instead of rounding."""
    x = x.detach().cpu()
    dt = x.dtype
    weights, ids = router_ref(logits, topk, renormalize)
    num_tokens = x.shape[0]
    num_experts, inter_x2, _ = w13.shape
    cache3 = torch.zeros(num_tokens, topk, x.shape[1], dtype=dt)
    ids64 = ids.long()
    for e in range(num_experts):
        tok, slot = torch.nonzero(ids64 == e, as_tuple=True)
        if tok.numel() == 0:
            continue
        c1 = _to_bf16(x[tok].float() @ w13[e].detach().cpu().float().T, bf16_cast).to(dt)
        c2 = silu_and_mul_ref(c1)
        y = c2.float() @ w2[e].detach().cpu().float().T
        y = _to_bf16(y * weights[tok, slot].unsqueeze(1), bf16_cast).to(dt)
        cache3[tok, slot] = y
    return moe_sum_ref(cache3)


def error_stats(got: torch.Tensor, want: torch.Tensor) -> dict:
    """max-abs error, relative Frobenius error and the scale of ``want``."""
    g, w = got.detach().cpu().double(), want.detach().cpu().double()
    diff = (g - w).abs()
    return {
        "max_abs": float(diff.max()) if diff.numel() else 0.0,
        "rel_fro": float(torch.linalg.norm(g - w) / max(float(torch.linalg.norm(w)), 1e-30)),
        "ref_max_abs": float(w.abs().max()) if w.numel() else 0.0,
    }
