"""The MoE pipeline behind ``FusedMoE.forward``: router -> alignment -> grouped GEMM with SwiGLU
-> grouped GEMM with routing weight -> combine.

Function names, arguments and results follow the reference's layers/moe/fused_moe.py
(``fused_topk`` :130-164, ``fused_experts`` :170-293).  The reference runs about five torch
kernels for routing, four launches for alignment, two Triton GEMMs, ``silu_and_mul`` and
``moe_sum``; here one call is six C-ABI calls (alignment is one launch for decode-sized batches
and three for long ones):

    topk_softmax (renormalising) -> align_block_size (writes its own padding) -> gather_rows
    -> grouped_gemm_w13_swiglu -> grouped_gemm_w2_scale -> moe_sum
"""
from __future__ import annotations

from typing import Dict, Optional, Tuple

import torch

from ... import _C, _lib

# Rows per M tile of the tensor-core kernels; token alignment pads every expert to this.
# 128 rows: one CTA per 128 x 256 tile.  256 rows: a pair of CTAs (tcgen05 cta_group::2) per
# 256 x 256 tile, which moves a third less operand data per FLOP but pads every expert to 256 rows
# and issues slower M=256 MMAs; measured on B200 at Mixtral shape it is 3-6 % slower than the
# one-CTA tiling at T=8192, so it is available but not chosen by default.
BLOCK_SIZE_M = 128
PAIR_BLOCK_SIZE_M = 256
FORCE_BLOCK_M = None  # set to 128 or 256 to override the choice (benchmarks, tests)


def choose_block_m(num_tokens: int, topk: int, num_experts: int) -> int:
    """M tile (= alignment block) used for a batch of this size."""
    if FORCE_BLOCK_M is not None:
        return FORCE_BLOCK_M
    return BLOCK_SIZE_M


def fused_topk(hidden_states: torch.Tensor, gating_output: torch.Tensor, topk: int,
               renormalize: bool) -> Tuple[torch.Tensor, torch.Tensor]:
    """softmax(fp32) -> top-k -> optional renormalisation, in one kernel.

    Returns ``(topk_weights f32 [T, topk], topk_ids i32 [T, topk])`` like the reference
    (fused_moe.py:130-164).  On exactly equal logits the lower expert index is chosen, the rule of
    the reference's own kernel (src/topk_softmax_kernels.cu:39,47).
    """
    assert hidden_states.shape[0] == gating_output.shape[0], "Number of tokens mismatch"
    num_tokens = gating_output.shape[0]
    topk_weights = torch.empty(num_tokens, topk, dtype=torch.float32, device=gating_output.device)
    topk_ids = torch.empty(num_tokens, topk, dtype=torch.int32, device=gating_output.device)
    _C.topk_softmax(topk_weights, topk_ids, gating_output.contiguous(), renormalize=renormalize)
    return topk_weights, topk_ids


def capacity_bucket(num_tokens: int) -> int:
    """Token capacity scratch is sized for: the next power of two, at least 256.  A serving loop
    whose batch size changes every step therefore reallocates only when a batch exceeds every
    earlier one by a factor, and never in steady state."""
    return max(256, 1 << max(num_tokens - 1, 0).bit_length())


class _Workspace:
    """Scratch tensors of ``fused_experts``, kept per (device, stream, layer shape) and sized for a
    token capacity bucket; a call uses a prefix of them, so steady-state calls allocate nothing
    whatever their batch size, and calls on different streams never share scratch.  The reference
    allocates its three caches on every call (fused_moe.py:223-239).

    CUDA graphs: a captured call keeps raw pointers into these tensors.  An entry used during
    stream capture is therefore never freed (when a larger batch replaces it, it is retired, not
    released), and a call that would have to allocate during capture raises instead: run the
    layer once on the capture stream with the largest batch, or call ``reserve_workspace``,
    before capturing."""

    MAX_ENTRIES = 8
    MAX_VIEWS = 32

    def __init__(self) -> None:
        self._cache: Dict[tuple, dict] = {}
        self._retired: list = []

    def _allocate(self, device, max_tokens, topk, num_experts, hidden, inter, block_m) -> dict:
        pairs = max_tokens * topk
        capacity = pairs + num_experts * (block_m - 1)
        blocks = (capacity + block_m - 1) // block_m
        i32 = dict(dtype=torch.int32, device=device)
        bf16 = dict(dtype=torch.bfloat16, device=device)
        return {
            "max_tokens": max_tokens, "pinned": False, "views": {},
            "topk_weights": torch.empty(max_tokens, topk, dtype=torch.float32, device=device),
            "topk_ids": torch.empty(max_tokens, topk, **i32),
            "sorted_ids": torch.empty(capacity, **i32),
            "expert_ids": torch.zeros(blocks, **i32),
            "num_post_pad": torch.zeros(1, **i32),
            "align_ws": torch.empty(max(_C.align_workspace_numel(pairs, num_experts), 1), **i32),
            "a_sorted": torch.empty(capacity, hidden, **bf16),
            "act": torch.empty(capacity, inter, **bf16),
            "cache3": torch.empty(max_tokens, topk, hidden, **bf16),
        }

    def get(self, device: torch.device, num_tokens: int, topk: int, num_experts: int,
            hidden: int, inter: int, block_m: int, reserve_only: bool = False) -> Optional[dict]:
        stream = torch.cuda.current_stream(device).cuda_stream
        key = (device, stream, topk, num_experts, hidden, inter, block_m)
        entry = self._cache.get(key)
        capturing = torch.cuda.is_current_stream_capturing()
        if entry is None or entry["max_tokens"] < num_tokens:
            if capturing:
                raise RuntimeError(
                    "fused_experts: scratch for this batch size does not exist yet and cannot be "
                    "allocated during stream capture; run the layer once on this stream with a "
                    "batch at least this large (or call reserve_workspace) before capturing")
            if entry is not None and entry["pinned"]:
                self._retired.append(entry)  # a captured graph may still point into it
            if entry is None and len(self._cache) >= self.MAX_ENTRIES:
                for old_key, old in list(self._cache.items()):  # oldest entry no graph refers to
                    if not old["pinned"]:
                        del self._cache[old_key]
                        break
            entry = self._allocate(device, capacity_bucket(num_tokens), topk, num_experts, hidden,
                                   inter, block_m)
            self._cache[key] = entry
        if capturing:
            entry["pinned"] = True
        if reserve_only:
            return None
        ws = entry["views"].get(num_tokens)
        if ws is None:
            if len(entry["views"]) >= self.MAX_VIEWS:
                entry["views"].pop(next(iter(entry["views"])))
            capacity = num_tokens * topk + num_experts * (block_m - 1)
            blocks = (capacity + block_m - 1) // block_m
            ws = {
                "capacity": capacity,
                "topk_weights": entry["topk_weights"][:num_tokens],
                "topk_ids": entry["topk_ids"][:num_tokens],
                "sorted_ids": entry["sorted_ids"][:capacity],
                "expert_ids": entry["expert_ids"][:blocks],
                "num_post_pad": entry["num_post_pad"],
                "align_ws": entry["align_ws"],
                "a_sorted": entry["a_sorted"][:capacity],
                "act": entry["act"][:capacity],
                "cache3": entry["cache3"][:num_tokens],
            }
            entry["views"][num_tokens] = ws
        return ws


_workspace = _Workspace()
_LOGIT_TAGS = {torch.float32: _lib.F32, torch.float16: _lib.F16, torch.bfloat16: _lib.BF16}


def reserve_workspace(device, max_tokens: int, topk: int, num_experts: int, hidden: int,
                      inter: int) -> None:
    """Allocates the scratch of ``fused_experts`` on ``device``'s current stream for batches of up
    to ``max_tokens`` tokens, so that no later call (smaller or equal) allocates: for serving
    loops with a known maximum batch and before CUDA graph capture."""
    device = torch.device(device)
    _workspace.get(device, max_tokens, topk, num_experts, hidden, inter,
                   choose_block_m(max_tokens, topk, num_experts), reserve_only=True)

# Optional per-kernel timing for benchmarks: when enabled, every launch of fused_experts is
# bracketed by a pair of CUDA events on the launching stream.
_timing_enabled = False
_timing_events: list = []


def enable_kernel_timing(on: bool) -> None:
    global _timing_enabled
    _timing_enabled = bool(on)
    _timing_events.clear()


def collect_kernel_timings() -> Dict[str, float]:
    """Mean milliseconds per launch of every kernel timed since ``enable_kernel_timing(True)``.
    Synchronises with the device."""
    torch.cuda.synchronize()
    sums: Dict[str, list] = {}
    for name, e0, e1 in _timing_events:
        sums.setdefault(name, []).append(e0.elapsed_time(e1))
    _timing_events.clear()
    return {k: sum(v) / len(v) for k, v in sums.items()}


class _timed:
    def __init__(self, name: str):
        self.name = name

    def __enter__(self):
        if _timing_enabled:
            self.e0 = torch.cuda.Event(enable_timing=True)
            self.e0.record()

    def __exit__(self, *exc):
        if _timing_enabled:
            e1 = torch.cuda.Event(enable_timing=True)
            e1.record()
            _timing_events.append((self.name, self.e0, e1))
        return False


_bf16_weight_copies: Dict[tuple, torch.Tensor] = {}


def _bf16_weights(w: torch.Tensor) -> torch.Tensor:
    """bf16 copy of an fp16/fp32 weight tensor, made once per (storage, version): the grouped GEMMs
    read bf16 operands only."""
    if w.dtype == torch.bfloat16:
        return w
    key = (w.data_ptr(), w._version, tuple(w.shape), w.dtype)
    hit = _bf16_weight_copies.get(key)
    if hit is None:
        for old in [k for k in _bf16_weight_copies if k[0] == key[0]]:
            del _bf16_weight_copies[old]   # the parameter changed: drop the stale copy
        if len(_bf16_weight_copies) >= 64:
            _bf16_weight_copies.pop(next(iter(_bf16_weight_copies)))
        hit = w.detach().to(torch.bfloat16).contiguous()
        _bf16_weight_copies[key] = hit
    return hit


def fused_experts(hidden_states: torch.Tensor, w1: torch.Tensor, w2: torch.Tensor,
                  gating_output: Optional[torch.Tensor], topk: int, renormalize: bool = True,
                  inplace: bool = False, activation: str = "silu",
                  gate_weight: Optional[torch.Tensor] = None, tp_reduce=None) -> torch.Tensor:
    """Mixture-of-experts forward for ``hidden_states [T, H]`` (reference fused_moe.py:170-293).

    ``w1`` is the stacked gate/up weight ``[E, 2*I, H]`` (gate rows first), ``w2`` is
    ``[E, H, I]``, ``gating_output`` the router logits ``[T, E]`` in any float dtype.  With
    ``inplace`` the result overwrites and aliases ``hidden_states``, as the layer relies on.
    Tensors must be on a CUDA device: there is no other implementation behind this call.

    Element types: the reference takes any float dtype and computes in bf16 whatever it is given
    (``compute_type=tl.bfloat16``, fused_moe.py:254,286).  Here bf16 tensors are the native case.
    fp16 or fp32 ``hidden_states`` are converted to bf16 on entry and the result is converted back
    into a tensor of the caller's dtype (into ``hidden_states`` itself with ``inplace``); fp16 or
    fp32 weights are converted once and the bf16 copy is kept until the parameter changes
    (``_bf16_weights``), which doubles their memory: load bf16 weights where that matters.

    Extension: with ``gate_weight`` (bf16 ``[E, H]``) the gate projection is computed by the router
    kernel itself and ``gating_output`` may be ``None``.  With ``tp_reduce`` (a
    ``parallel.TensorParallelReduce`` whose ``usable(num_tokens)`` holds on every rank) the result
    is also summed over the tensor-parallel ranks: the second GEMM stores its rows into the owning
    ranks' buffers over NVLink and the combine kernel finishes the all-reduce.
    """
    if activation != "silu":
        raise NotImplementedError(f"Activation {activation} not supported.")
    if not hidden_states.is_cuda:
        raise RuntimeError("fused_experts: tensors must be on a CUDA device; no CPU path exists")
    floats = (torch.bfloat16, torch.float16, torch.float32)
    if hidden_states.dtype not in floats or w1.dtype not in floats or w2.dtype not in floats:
        raise RuntimeError("fused_experts: hidden_states, w1 and w2 must be bf16, fp16 or fp32 "
                           f"(got {hidden_states.dtype}, {w1.dtype}, {w2.dtype})")
    if w1.dtype != torch.bfloat16 or w2.dtype != torch.bfloat16:
        w1, w2 = _bf16_weights(w1), _bf16_weights(w2)
    if hidden_states.dtype != torch.bfloat16:
        # Compute in bf16 like the reference, hand the result back in the caller's dtype.
        result = fused_experts(hidden_states.to(torch.bfloat16), w1, w2, gating_output, topk,
                               renormalize, True, activation, gate_weight, tp_reduce)
        if inplace:
            return hidden_states.copy_(result)
        return result.to(hidden_states.dtype)
    num_tokens, hidden = hidden_states.shape
    num_experts, inter_x2, w1_k = w1.shape
    inter = inter_x2 // 2
    if w1_k != hidden or tuple(w2.shape) != (num_experts, hidden, inter):
        raise RuntimeError(f"fused_experts: weight shapes {tuple(w1.shape)} / {tuple(w2.shape)} "
                           f"do not match hidden={hidden}")
    if gate_weight is None:
        if gating_output is None or gating_output.shape != (num_tokens, num_experts):
            raise RuntimeError("fused_experts: gating_output must be [num_tokens, num_experts]")
    elif tuple(gate_weight.shape) != (num_experts, hidden) or not gate_weight.is_contiguous():
        raise RuntimeError("fused_experts: gate_weight must be a contiguous [num_experts, hidden] tensor")
    for t in (hidden_states, w1, w2):
        if not t.is_contiguous():
            raise RuntimeError("fused_experts: hidden_states, w1 and w2 must be contiguous")

    output = hidden_states if inplace else torch.empty_like(hidden_states)
    if num_tokens == 0:
        return output

    dev = hidden_states.device
    lib = _lib.load()
    block_m = choose_block_m(num_tokens, topk, num_experts)
    ws = _workspace.get(dev, num_tokens, topk, num_experts, hidden, inter, block_m)
    peer = None
    if tp_reduce is not None:
        if topk != 2 or not tp_reduce.usable(num_tokens):
            raise RuntimeError("fused_experts: tp_reduce needs top_k=2 and a token count divisible "
                               "by the tensor-parallel size")
        peer = tp_reduce.state(num_tokens, topk, hidden, dev)  # set-up on first use
    capacity = ws["capacity"]
    gating = None
    if gate_weight is None:
        gating = gating_output if gating_output.is_contiguous() else gating_output.contiguous()

    if (gate_weight is None and tp_reduce is None and not _timing_enabled and block_m == BLOCK_SIZE_M
            and topk == 2 and gating.dtype in _LOGIT_TAGS):
        # The common case in one C-ABI call: the library issues the six steps itself.
        ptrs = ws.get("ptrs")
        if ptrs is None:
            ptrs = ws["ptrs"] = (ws["topk_weights"].data_ptr(), ws["topk_ids"].data_ptr(),
                                 ws["sorted_ids"].data_ptr(), ws["expert_ids"].data_ptr(),
                                 ws["num_post_pad"].data_ptr(), ws["align_ws"].data_ptr(),
                                 ws["align_ws"].numel() * 4, ws["a_sorted"].data_ptr(),
                                 ws["act"].data_ptr(), ws["cache3"].data_ptr())
            ws["launches"] = 5 + (3 if num_tokens * topk > _C.align_single_pass_max() else 1)
        with torch.cuda.device(dev):
            _lib.check(lib.b200moe_fused_experts(
                hidden_states.data_ptr(), gating.data_ptr(), _LOGIT_TAGS[gating.dtype], w1.data_ptr(),
                w2.data_ptr(), output.data_ptr(), num_tokens, num_experts, topk, hidden, inter,
                int(renormalize), *ptrs, torch.cuda.current_stream(dev).cuda_stream), "fused_experts")
        _lib.count_launches(ws["launches"])
        return output

    with torch.cuda.device(dev):
        stream = torch.cuda.current_stream(dev).cuda_stream
        if gate_weight is None:
            with _timed("topk_softmax"):
                _C.topk_softmax(ws["topk_weights"], ws["topk_ids"], gating, renormalize=renormalize)
        else:
            with _timed("gate_topk_softmax"):
                _C.gate_topk_softmax(ws["topk_weights"], ws["topk_ids"], hidden_states, gate_weight,
                                     renormalize=renormalize)
        with _timed("moe_align_block_size"):
            _C.moe_align_block_size(ws["topk_ids"], num_experts, block_m, ws["sorted_ids"],
                                    ws["expert_ids"], ws["num_post_pad"], fill_pads=True,
                                    workspace=ws["align_ws"])
        # The A rows are gathered into expert-sorted order once, then read as dense TMA tiles.
        # (b200moe_grouped_gemm_w13_swiglu_gather folds the gather into the GEMM with TMA
        # tile::gather4, but 32 four-row gathers per K step run the kernel 2.6x slower than one
        # tiled box on B200, so the layer does not use it.)
        with _timed("gather_rows"):
            _lib.check(lib.b200moe_gather_rows(
                hidden_states.data_ptr(), ws["a_sorted"].data_ptr(), ws["sorted_ids"].data_ptr(),
                ws["num_post_pad"].data_ptr(), capacity, num_tokens, hidden, topk, stream),
                "gather_rows")
        with _timed("grouped_gemm_w13_swiglu"):
            _lib.check(lib.b200moe_grouped_gemm_w13_swiglu(
                ws["a_sorted"].data_ptr(), w1.data_ptr(), ws["act"].data_ptr(),
                ws["expert_ids"].data_ptr(), ws["num_post_pad"].data_ptr(), capacity, num_experts,
                hidden, inter, block_m, stream), "grouped_gemm_w13_swiglu")
        if tp_reduce is None:
            with _timed("grouped_gemm_w2_scale"):
                _lib.check(lib.b200moe_grouped_gemm_w2_scale(
                    ws["act"].data_ptr(), w2.data_ptr(), ws["cache3"].data_ptr(),
                    ws["topk_weights"].data_ptr(), ws["sorted_ids"].data_ptr(),
                    ws["expert_ids"].data_ptr(), ws["num_post_pad"].data_ptr(), capacity,
                    num_tokens * topk, num_experts, hidden, inter, block_m, stream),
                    "grouped_gemm_w2_scale")
            _lib.count_launches(3)
            with _timed("moe_sum"):
                _C.moe_sum(ws["cache3"], output)
        else:
            with _timed("grouped_gemm_w2_scale"):
                _lib.check(lib.b200moe_grouped_gemm_w2_scale_peer(
                    ws["act"].data_ptr(), w2.data_ptr(), peer["push_table"].data_ptr(),
                    tp_reduce.world, peer["tokens_per_rank"] * topk,
                    ws["topk_weights"].data_ptr(), ws["sorted_ids"].data_ptr(),
                    ws["expert_ids"].data_ptr(), ws["num_post_pad"].data_ptr(), capacity,
                    num_experts, hidden, inter, block_m, stream), "grouped_gemm_w2_scale_peer")
            _lib.count_launches(3)
            tp_reduce.finish(peer, output, topk)
    return output
