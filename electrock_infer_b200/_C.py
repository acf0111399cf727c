"""Drop-in for the reference's native module ``electrock_infer._C`` (pytorch_bind.cpp:11-50).

The ops keep the reference's names, keyword names, output convention (the MoE ops write into
caller-allocated tensors and return ``None``; ``paged_attn_varlen`` returns a new tensor, as in the
reference) and error type (``RuntimeError``, what a failed ``TORCH_CHECK`` surfaces as).  Each forwards raw device pointers to the C-ABI
library on the current CUDA stream of the tensor's device; nothing is computed in Python.
"""
from __future__ import annotations

import torch

from . import _lib

_FLOAT_TAGS = {torch.float32: _lib.F32, torch.float16: _lib.F16, torch.bfloat16: _lib.BF16}
_INT_TAGS = {torch.int32: _lib.I32, torch.int64: _lib.I64, torch.int16: _lib.I16,
             torch.int8: _lib.I8, torch.uint8: _lib.U8}


def _require_cuda(name: str, *tensors: torch.Tensor) -> torch.device:
    dev = tensors[0].device
    for t in tensors:
        if not t.is_cuda:
            raise RuntimeError(f"{name}: tensors must be on a CUDA device (got {t.device}); "
                               "there is no CPU implementation")
        if t.device != dev:
            raise RuntimeError(f"{name}: tensors are on different devices ({dev} vs {t.device})")
        if not t.is_contiguous():
            raise RuntimeError(f"{name}: tensors must be contiguous")
    return dev


def _stream(dev: torch.device) -> int:
    return torch.cuda.current_stream(dev).cuda_stream


def _float_tag(name: str, t: torch.Tensor) -> int:
    try:
        return _FLOAT_TAGS[t.dtype]
    except KeyError:
        raise RuntimeError(f"{name}: unsupported dtype {t.dtype}") from None


def topk_softmax(topk_weights: torch.Tensor, topk_indices: torch.Tensor,
                 gating_output: torch.Tensor, renormalize: bool = False) -> None:
    """softmax over 8 experts + top-2 (src/topk_softmax_kernels.cu:85-111).

    ``topk_weights`` f32 ``[T, 2]`` and ``topk_indices`` i32 ``[T, 2]`` are overwritten.  Like the
    reference the probabilities are not renormalised unless ``renormalize`` (an extension) is set.
    Unlike the reference, bf16/fp16 logits are accepted directly (no ``.float()`` copy needed).
    """
    name = "topk_softmax"
    dev = _require_cuda(name, topk_weights, topk_indices, gating_output)
    if topk_weights.dtype != torch.float32 or topk_indices.dtype != torch.int32:
        raise RuntimeError(f"{name}: topk_weights must be float32 and topk_indices int32")
    num_experts = gating_output.size(-1)
    num_tokens = gating_output.numel() // max(num_experts, 1)
    topk = topk_weights.size(-1)
    if topk_weights.numel() != num_tokens * topk or topk_indices.numel() != num_tokens * topk:
        raise RuntimeError(f"{name}: outputs must hold num_tokens * topk elements")
    with torch.cuda.device(dev):
        rc = _lib.load().b200moe_topk_softmax(
            topk_weights.data_ptr(), topk_indices.data_ptr(), gating_output.data_ptr(),
            _float_tag(name, gating_output), num_tokens, num_experts, topk, int(renormalize),
            _stream(dev))
    _lib.check(rc, name)
    _lib.count_launches(1 if num_tokens else 0)


def gate_topk_softmax(topk_weights: torch.Tensor, topk_indices: torch.Tensor,
                      hidden_states: torch.Tensor, gate_weight: torch.Tensor,
                      renormalize: bool = False, logits_out: torch.Tensor | None = None,
                      round_logits_bf16: bool = True) -> None:
    """Gate projection + softmax + top-2 in one kernel (no counterpart among the reference's ops:
    it replaces the gate ``F.linear`` of models/mixtral.py:59 followed by the router).

    ``hidden_states`` bf16 ``[T, H]``, ``gate_weight`` bf16 ``[8, H]``; ``topk_weights`` f32
    ``[T, 2]`` and ``topk_indices`` i32 ``[T, 2]`` are overwritten; ``logits_out`` (f32 ``[T, 8]``)
    optionally receives the logits.  ``round_logits_bf16`` rounds the fp32-accumulated logits to
    bf16 before routing, which is what the reference's bf16 gate layer produces.
    """
    name = "gate_topk_softmax"
    tensors = [topk_weights, topk_indices, hidden_states, gate_weight]
    if logits_out is not None:
        tensors.append(logits_out)
    dev = _require_cuda(name, *tensors)
    if hidden_states.dtype != torch.bfloat16 or gate_weight.dtype != torch.bfloat16:
        raise RuntimeError(f"{name}: hidden_states and gate_weight must be bfloat16")
    if topk_weights.dtype != torch.float32 or topk_indices.dtype != torch.int32:
        raise RuntimeError(f"{name}: topk_weights must be float32 and topk_indices int32")
    if hidden_states.dim() != 2 or gate_weight.dim() != 2 or gate_weight.size(1) != hidden_states.size(1):
        raise RuntimeError(f"{name}: expected hidden_states [T, H] and gate_weight [E, H]")
    num_tokens, hidden = hidden_states.shape
    num_experts, topk = gate_weight.size(0), topk_weights.size(-1)
    if topk_weights.numel() != num_tokens * topk or topk_indices.numel() != num_tokens * topk:
        raise RuntimeError(f"{name}: outputs must hold num_tokens * topk elements")
    if logits_out is not None and (logits_out.dtype != torch.float32
                                   or logits_out.numel() != num_tokens * num_experts):
        raise RuntimeError(f"{name}: logits_out must be float32 [num_tokens, num_experts]")
    with torch.cuda.device(dev):
        rc = _lib.load().b200moe_gate_topk_softmax(
            hidden_states.data_ptr(), gate_weight.data_ptr(), topk_weights.data_ptr(),
            topk_indices.data_ptr(), logits_out.data_ptr() if logits_out is not None else None,
            num_tokens, hidden, num_experts, topk, int(renormalize), int(round_logits_bf16),
            _stream(dev))
    _lib.check(rc, name)
    _lib.count_launches(1 if num_tokens else 0)


def moe_align_block_size(topk_ids: torch.Tensor, num_experts: int, block_size: int,
                         sorted_token_ids: torch.Tensor, expert_ids: torch.Tensor,
                         num_tokens_post_pad: torch.Tensor,
                         expert_offsets: torch.Tensor | None = None,
                         fill_pads: bool = False,
                         workspace: torch.Tensor | None = None) -> None:
    """Stable counting sort of pair indices by expert with per-expert padding
    (src/moe_align_block_size.cu:140-230).

    With the defaults the op writes exactly what the reference kernel writes (padding slots and
    the tail are left as the caller prefilled them).  ``fill_pads=True`` makes the kernel write the
    ``-1`` padding itself; ``expert_offsets`` (i32 ``[num_experts + 1]``) optionally receives the
    padded start offset of every expert.  Both are extensions.  Long inputs need a small scratch
    tensor (``align_workspace_numel`` int32 elements); it is allocated here unless ``workspace``
    is passed.
    """
    name = "moe_align_block_size"
    outs = [sorted_token_ids, expert_ids, num_tokens_post_pad]
    if expert_offsets is not None:
        outs.append(expert_offsets)
    dev = _require_cuda(name, topk_ids, *outs)
    for t in outs:
        if t.dtype != torch.int32:
            raise RuntimeError(f"{name}: outputs must be int32")
    if topk_ids.dtype not in _INT_TAGS:
        raise RuntimeError(f"{name}: topk_ids must be an integral tensor, got {topk_ids.dtype}")
    if expert_offsets is not None and expert_offsets.numel() < num_experts + 1:
        raise RuntimeError(f"{name}: expert_offsets needs num_experts + 1 elements")
    if num_tokens_post_pad.numel() < 1:
        raise RuntimeError(f"{name}: num_tokens_post_pad needs one element")
    lib = _lib.load()
    numel = topk_ids.numel()
    ws_bytes = lib.b200moe_align_workspace_bytes(numel, num_experts)
    ws = None
    own_ws = False
    if ws_bytes:
        if workspace is not None:
            if (workspace.dtype != torch.int32 or workspace.device != dev
                    or workspace.numel() * 4 < ws_bytes):
                raise RuntimeError(f"{name}: workspace must be an int32 tensor of at least "
                                   f"{ws_bytes // 4} elements on {dev}")
            ws = workspace
        else:
            ws = torch.empty(ws_bytes // 4, dtype=torch.int32, device=dev)
            own_ws = True
    with torch.cuda.device(dev):
        rc = lib.b200moe_align_block_size(
            topk_ids.data_ptr(), _INT_TAGS[topk_ids.dtype], numel, int(num_experts),
            int(block_size), sorted_token_ids.data_ptr(), sorted_token_ids.numel(),
            expert_ids.data_ptr(), expert_ids.numel(), num_tokens_post_pad.data_ptr(),
            expert_offsets.data_ptr() if expert_offsets is not None else None, int(fill_pads),
            ws.data_ptr() if ws is not None else None, ws_bytes, _stream(dev))
    _lib.check(rc, name)
    _lib.count_launches(3 if ws is not None else 1)
    if own_ws:
        ws.record_stream(torch.cuda.current_stream(dev))


def align_single_pass_max() -> int:
    """Longest input (pair indices) that ``moe_align_block_size`` handles in one launch."""
    return _lib.load().b200moe_align_single_pass_max()


def align_workspace_numel(numel: int, num_experts: int) -> int:
    """int32 elements of scratch that ``moe_align_block_size`` needs for ``numel`` pair indices
    (0 for short inputs)."""
    return _lib.load().b200moe_align_workspace_bytes(numel, num_experts) // 4


def silu_and_mul(out: torch.Tensor, input: torch.Tensor) -> None:  # noqa: A002 - reference name
    """``out[..., j] = silu(input[..., j]) * input[..., d + j]``
    (src/activation_kernels.cu:97-150)."""
    name = "silu_and_mul"
    dev = _require_cuda(name, out, input)
    if input.dim() < 2:
        raise RuntimeError(f"{name}: Input must have at least 2 dimensions!")
    d = input.size(-1) // 2
    if input.size(-1) != 2 * d:
        raise RuntimeError(f"{name}: Input last dimension must be 2*d!")
    if out.size(-1) != d:
        raise RuntimeError(f"{name}: Output last dimension must be d!")
    if out.dtype != input.dtype:
        raise RuntimeError(f"{name}: out and input must have the same dtype")
    rows = input.numel() // (2 * d) if d else 0
    if out.numel() != rows * d:
        raise RuntimeError(f"{name}: out holds {out.numel()} elements, expected {rows * d}")
    with torch.cuda.device(dev):
        rc = _lib.load().b200moe_silu_and_mul(out.data_ptr(), input.data_ptr(),
                                              _float_tag(name, input), rows, d, _stream(dev))
    _lib.check(rc, name)
    _lib.count_launches(1 if rows * d else 0)


def _moe_sum(name: str, input: torch.Tensor, output: torch.Tensor, layout: int) -> None:  # noqa: A002
    dev = _require_cuda(name, input, output)
    if input.dim() != 3:
        raise RuntimeError(f"{name}: input must be 3-dimensional")
    if input.dtype != output.dtype:
        raise RuntimeError(f"{name}: input and output must have the same dtype")
    if layout == 0:
        topk, hidden = input.size(1), input.size(2)
    else:
        hidden, topk = input.size(1), input.size(2)
    num_tokens = output.numel() // hidden if hidden else 0
    if input.numel() != num_tokens * topk * hidden:
        raise RuntimeError(f"{name}: input and output shapes do not match")
    with torch.cuda.device(dev):
        rc = _lib.load().b200moe_moe_sum(input.data_ptr(), output.data_ptr(),
                                         _float_tag(name, input), num_tokens, hidden, topk,
                                         layout, _stream(dev))
    _lib.check(rc, name)
    _lib.count_launches(1 if num_tokens * hidden else 0)


def moe_sum(input: torch.Tensor, output: torch.Tensor) -> None:  # noqa: A002
    """``output[t] = input[t, 0] + input[t, 1]`` for ``input [T, 2, H]`` (src/moe_sum.cu:50-74)."""
    _moe_sum("moe_sum", input, output, 0)


def moe_sum_efficient(input: torch.Tensor, output: torch.Tensor) -> None:  # noqa: A002
    """Same sum for the interleaved layout ``input [T, H, 2]``
    (src/moe_sum_efficient.cu:52-79); bf16 is accepted in addition to fp32/fp16."""
    _moe_sum("moe_sum_efficient", input, output, 1)


def _rms_norm(name: str, input: torch.Tensor, residual, epsilon: float,  # noqa: A002
              weight: torch.Tensor) -> None:
    tensors = [input, weight] + ([residual] if residual is not None else [])
    dev = _require_cuda(name, *tensors)
    if input.dim() != 2 or weight.dim() != 1 or weight.numel() != input.size(1):
        raise RuntimeError(f"{name}: expected input [num_tokens, hidden] and weight [hidden]")
    if weight.dtype != input.dtype or (residual is not None and (
            residual.dtype != input.dtype or residual.shape != input.shape)):
        raise RuntimeError(f"{name}: input, residual and weight must share dtype and shape")
    with torch.cuda.device(dev):
        rc = _lib.load().b200moe_add_rms_norm(
            input.data_ptr(), residual.data_ptr() if residual is not None else None,
            weight.data_ptr(), _float_tag(name, input), input.size(0), input.size(1),
            float(epsilon), _stream(dev))
    _lib.check(rc, name)
    _lib.count_launches(1 if input.numel() else 0)


def rms_norm(input: torch.Tensor, epsilon: float, weight: torch.Tensor) -> None:  # noqa: A002
    """In-place RMSNorm of every row (reference op: pytorch_bind.cpp:53-58)."""
    _rms_norm("rms_norm", input, None, epsilon, weight)


def add_rms_norm(input: torch.Tensor, residual: torch.Tensor, epsilon: float,  # noqa: A002
                 weight: torch.Tensor) -> None:
    """``residual <- input + residual`` then ``input <- RMSNorm(residual) * weight``, both in place
    (reference op: pytorch_bind.cpp:60-66; arithmetic of layers/layernorm.py:30-43)."""
    _rms_norm("add_rms_norm", input, residual, epsilon, weight)


def paged_store_kvcache(K: torch.Tensor, V: torch.Tensor, K_cache: torch.Tensor,  # noqa: N803
                        V_cache: torch.Tensor, slot_mapping: torch.Tensor) -> None:
    """Copies the new tokens' key/value rows into their cache slots
    (src/store_kv_cache.hip:65-110, pytorch_bind.cpp:92-99; the Triton ``store_kvcache`` of
    layers/attention_triton_kernel.py:96-106 has the same contract).

    ``K``, ``V`` ``[tokens, kv_heads, head_dim]`` (the token stride may exceed a row, as for
    slices of a fused QKV projection); caches ``[blocks, block_size, kv_heads, head_dim]``
    contiguous; ``slot_mapping`` int32 ``[tokens]``, negative entries are skipped.
    """
    name = "paged_store_kvcache"
    for t in (K, V, K_cache, V_cache, slot_mapping):
        if not t.is_cuda:
            raise RuntimeError(f"{name}: tensors must be on a CUDA device; there is no CPU implementation")
    dev = K.device
    if K.dim() != 3 or V.shape != K.shape:
        raise RuntimeError(f"{name}: K and V must both be [tokens, kv_heads, head_dim]")
    num_tokens, kv_heads, head_dim = K.shape
    if K_cache.dim() != 4 or V_cache.shape != K_cache.shape or tuple(K_cache.shape[2:]) != (kv_heads, head_dim):
        raise RuntimeError(f"{name}: caches must be [blocks, block_size, {kv_heads}, {head_dim}]")
    if not (K_cache.is_contiguous() and V_cache.is_contiguous() and slot_mapping.is_contiguous()):
        raise RuntimeError(f"{name}: caches and slot_mapping must be contiguous")
    for t in (K, V):
        if t.stride(2) != 1 or t.stride(1) != head_dim:
            raise RuntimeError(f"{name}: the heads of a token must be contiguous")
    if slot_mapping.dtype != torch.int32 or slot_mapping.numel() != num_tokens:
        raise RuntimeError(f"{name}: slot_mapping must be int32 with one entry per token")
    if not (K.dtype == V.dtype == K_cache.dtype == V_cache.dtype):
        raise RuntimeError(f"{name}: K, V and the caches must share a dtype")
    tag = _float_tag(name, K)
    with torch.cuda.device(dev):
        rc = _lib.load().b200moe_paged_store_kvcache(
            K.data_ptr(), V.data_ptr(), K_cache.data_ptr(), V_cache.data_ptr(),
            slot_mapping.data_ptr(), tag, num_tokens, kv_heads, head_dim,
            K.stride(0) if num_tokens > 1 else kv_heads * head_dim,
            V.stride(0) if num_tokens > 1 else kv_heads * head_dim,
            K_cache.size(0), K_cache.size(1), _stream(dev))
    _lib.check(rc, name)
    _lib.count_launches(1)


# Split-merge scratch of paged_attn_varlen, kept per (device, stream) so that steady-state calls
# allocate nothing and calls on different streams never share scratch.
_attn_workspaces: dict = {}


def paged_attn_varlen(Q: torch.Tensor, K_cache: torch.Tensor, V_cache: torch.Tensor,  # noqa: N803
                      max_seqlen_k: int, context_lens: torch.Tensor, block_table: torch.Tensor,
                      softmax_scale: float, num_splits: int = 0) -> torch.Tensor:
    """Decode attention of one query token per sequence over the paged cache, grouped-query heads
    (src/paged_attn_gqa_varlen.hip:216-268, pytorch_bind.cpp:68-77).  Returns a new ``O`` shaped
    like ``Q [batch, q_heads, 128]``, as the reference does.

    ``max_seqlen_k`` is accepted for signature parity (the reference ignores it; here a positive
    value only helps to choose ``num_splits``).  Extension: ``num_splits`` (0 = choose) cuts long
    contexts over several CTAs; block sizes other than 32 are accepted (any multiple of 16).
    """
    name = "paged_attn_varlen"
    dev = _require_cuda(name, Q, K_cache, V_cache, context_lens, block_table)
    if Q.dim() != 3 or K_cache.dim() != 4 or V_cache.shape != K_cache.shape:
        raise RuntimeError(f"{name}: Q must be [batch, heads, head_dim] and the caches "
                           "[blocks, block_size, kv_heads, head_dim]")
    batch, q_heads, head_dim = Q.shape
    num_blocks, block_size, kv_heads, cache_dim = K_cache.shape
    if cache_dim != head_dim:
        raise RuntimeError(f"{name}: head_dim of Q ({head_dim}) and of the caches ({cache_dim}) differ")
    if not (Q.dtype == K_cache.dtype == V_cache.dtype):
        raise RuntimeError(f"{name}: Q and the caches must share a dtype")
    if context_lens.dtype != torch.int32 or block_table.dtype != torch.int32:
        raise RuntimeError(f"{name}: context_lens and block_table must be int32")
    if block_table.dim() != 2 or block_table.size(0) != batch or context_lens.numel() != batch:
        raise RuntimeError(f"{name}: block_table must be [batch, max_blocks] and context_lens [batch]")
    tag = _float_tag(name, Q)
    lib = _lib.load()
    out = torch.empty_like(Q)
    max_blocks = block_table.size(1)
    if num_splits <= 0:
        longest = max_seqlen_k if max_seqlen_k > 0 else max_blocks * block_size
        with torch.cuda.device(dev):
            num_splits = lib.b200moe_paged_attn_num_splits(batch, kv_heads, longest)
    ws_ptr, ws_bytes = 0, 0
    if num_splits > 1:
        ws_bytes = lib.b200moe_paged_attn_workspace_bytes(batch, q_heads, num_splits)
        key = (dev, _stream(dev))
        ws = _attn_workspaces.get(key)
        if ws is None or ws.numel() < ws_bytes:
            if ws is None and len(_attn_workspaces) >= 8:  # bounded: drop the oldest entry
                _attn_workspaces.pop(next(iter(_attn_workspaces)))
            ws = torch.empty(ws_bytes, dtype=torch.uint8, device=dev)
            _attn_workspaces[key] = ws
        ws_ptr = ws.data_ptr()
    with torch.cuda.device(dev):
        rc = lib.b200moe_paged_attn_varlen(
            Q.data_ptr(), K_cache.data_ptr(), V_cache.data_ptr(), out.data_ptr(),
            block_table.data_ptr(), context_lens.data_ptr(), tag, batch, q_heads, kv_heads,
            head_dim, num_blocks, block_size, max_blocks, float(softmax_scale), num_splits,
            ws_ptr, ws_bytes, _stream(dev))
    _lib.check(rc, name)
    _lib.count_launches(2 if num_splits > 1 else 1)
    return out
