"""Sharding the MoE layer over the GPUs of one NVLink/NVSwitch box with ``torch.distributed``.

Tensor parallel is what the reference does: ``FusedMoE(tp_size=world, reduce_results=True)`` shards
the intermediate dimension and all-reduces the combined output (layers/moe/mixtral_moe.py:114-116).
The class in ``layers.moe`` does that with NCCL, or, through :class:`TensorParallelReduce` below,
inside the layer's own kernels over NVLink peer mappings.

Expert parallel has no counterpart in the reference (its docstring says EP was removed,
layers/moe/mixtral_moe.py:9-13).  ``ExpertParallelMoE`` keeps ``num_experts / world`` whole experts
on each rank and a slice of the tokens on each rank:

    route locally -> sort pairs by expert -> exchange per-expert counts (all-to-all)
    -> exchange rows and routing weights (all-to-all, variable splits)
    -> local alignment + grouped GEMMs over the rank's experts
    -> return rows (all-to-all) -> scatter to pair order -> combine

Rows always land in the receiving GPU's own memory (NCCL receive buffers) before any TMA load
touches them.  Every arithmetic step is the one the single-GPU layer performs on the same row, so
the result is bit-identical to the single-GPU result for the same tokens.

That exchange needs the split sizes on the host, i.e. one device synchronisation per call.  When
every rank holds the same number of tokens, or a bound on the tokens per rank is given,
``ExpertParallelMoE`` instead moves the rows inside its own kernels over NVLink peer mappings and
never synchronises with the host:

    route locally -> copy the tokens into a peer-visible staging buffer
    -> all-gather the (tiny) expert ids and routing weights
    -> align the global ids against the local experts (ids of other ranks' experts are skipped)
    -> gather_rows_peer: PULL the routed rows from their owners' staging buffers
    -> grouped GEMM 1 -> grouped GEMM 2 whose epilogue STORES every output row into the owner's
       [T_local, top_k, H] buffer -> one-word all-reduce (every rank's stores are done) -> combine

The exchange logic is written against a small ``ops`` object so that it can be exercised on CPU
ranks (gloo) in tests with a stand-in ``ops``; the product default is :class:`CudaOps` and nothing
in this package implements the arithmetic on the CPU.
"""
from __future__ import annotations

from typing import List, Optional, Tuple

import torch
import torch.distributed as dist
import torch.nn as nn

from . import _C, _lib
from .layers.moe.fused_moe import BLOCK_SIZE_M, _timed, capacity_bucket


class _RawDeviceMemory:
    """Adapter that lets torch view a raw device allocation."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False),
                                         "version": 3, "strides": None}


class PeerMemoryUnavailable(RuntimeError):
    """Raised on EVERY rank of the group when any rank could not allocate or map a peer-visible
    buffer (no peer access between the GPUs, CUDA IPC not permitted, out of memory)."""


class PeerBuffer:
    """A device buffer that every rank of ``group`` (all on one node) can address: a cudaMalloc
    allocation per rank, shared with CUDA IPC handles.  ``table`` is a device int64 tensor holding
    the address of every rank's buffer as seen from this process (own buffer: the local address);
    ``local`` is a uint8 torch view of the own buffer.  Creating one is a set-up step (it
    allocates, synchronises and exchanges handles through the process group).

    Construction is collective and fails collectively: the ranks compare notes before anyone uses
    the buffers, and if one of them failed, all of them release what they hold and raise
    :class:`PeerMemoryUnavailable`, so that callers can fall back to NCCL on every rank alike."""

    def __init__(self, nbytes: int, device: torch.device, group=None):
        import ctypes
        lib = _lib.load()
        self._lib = lib
        self.nbytes = nbytes
        self.group = group
        self.rank = dist.get_rank(group)
        world = dist.get_world_size(group)
        own = ctypes.c_void_p()
        handle = ctypes.create_string_buffer(64)
        error = None
        mapped_ptrs = {}
        with torch.cuda.device(device):
            if lib.b200moe_peer_alloc(nbytes, ctypes.byref(own), handle) != 0:
                error = "peer_alloc: " + lib.b200moe_last_error().decode(errors="replace")
            handles = [None] * world
            dist.all_gather_object(handles, None if error else handle.raw, group=group)
            if error is None and any(h is None for h in handles):
                error = "another rank could not allocate its buffer"
            if error is None:
                for r in range(world):
                    if r == self.rank:
                        continue
                    mapped = ctypes.c_void_p()
                    buf = ctypes.create_string_buffer(handles[r], 64)
                    if lib.b200moe_peer_open(buf, ctypes.byref(mapped)) != 0:
                        error = f"peer_open (rank {r}): " + lib.b200moe_last_error().decode(errors="replace")
                        break
                    mapped_ptrs[r] = mapped.value
            errors = [None] * world
            dist.all_gather_object(errors, error, group=group)
            if any(e is not None for e in errors):
                for ptr in mapped_ptrs.values():
                    lib.b200moe_peer_close(ptr)
                dist.barrier(group=group)  # nobody frees a buffer another rank still maps
                if own.value:
                    lib.b200moe_peer_free(own.value)
                self.ptrs = []
                raise PeerMemoryUnavailable("; ".join(
                    f"rank {r}: {e}" for r, e in enumerate(errors) if e is not None))
        self.ptrs = [own.value if r == self.rank else mapped_ptrs[r] for r in range(world)]
        self.table = torch.tensor(self.ptrs, dtype=torch.int64, device=device)
        self.local = torch.as_tensor(_RawDeviceMemory(own.value, nbytes), device=device)

    def close(self) -> None:
        """Collective over the group: every rank unmaps the other ranks' buffers, and only when
        all have done so does each rank free its own (an allocation must outlive its mappings in
        other processes).  Call it with no work on the buffers in flight."""
        if not self.ptrs:
            return
        torch.cuda.synchronize(self.local.device)
        for r, ptr in enumerate(self.ptrs):
            if r != self.rank:
                self._lib.b200moe_peer_close(ptr)
        dist.barrier(group=self.group)
        self._lib.b200moe_peer_free(self.ptrs[self.rank])
        self.ptrs = []
        self.local = None


class TensorParallelReduce:
    """The all-reduce of the tensor-parallel layer done by the layer's own kernels over NVLink
    peer mappings instead of an NCCL all-reduce of the ``[T, H]`` result.

    Rank ``j`` owns the token slice ``[j * T / tp, (j + 1) * T / tp)``:

        second grouped GEMM: the epilogue STORES the scaled rows of slice ``j`` into rank ``j``'s
        receive buffer, slot = source rank (``b200moe_grouped_gemm_w2_scale_peer``)
        -> one-word all-reduce (every rank's GEMM has finished)
        -> ``b200moe_moe_sum_ranks_push``: sums each own token's rows (per source rank like
           ``moe_sum``, then over the ranks in fp32 with one rounding) and stores the row into
           EVERY rank's output buffer
        -> one-word all-reduce (every rank's rows have landed) -> copy into ``hidden_states``

    No kernel waits on a flag: the ranks are ordered by the two tiny stream-ordered collectives.
    Rounding follows the reference (each rank's two-row sum is rounded to bf16 before the ranks
    are added, layers/moe/mixtral_moe.py:114-116): with two ranks the result has the same bits as
    the NCCL all-reduce; with more it is one fp32 sum in rank order, where an all-reduce rounds
    between its steps in an order of its own choosing.  Every rank receives the same bits.
    The peer buffers are sized for a token capacity (``capacity_for``) and reused for every
    smaller batch; ``state`` allocates and synchronises only when a batch exceeds it.
    """

    def __init__(self, group=None):
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self._buffers = {}   # (top_k, hidden, device) -> peer buffers sized for a token capacity

    def usable(self, num_tokens: int) -> bool:
        return num_tokens > 0 and num_tokens % self.world == 0 and self.world <= 8

    def capacity_for(self, num_tokens: int) -> int:
        """Token capacity the peer buffers are sized for: the power-of-two bucket of the batch,
        rounded up to a multiple of the group size.  Every rank sees the same batch size, so
        every rank computes the same capacity and grows its buffers in the same call."""
        cap = capacity_bucket(num_tokens)
        return (cap + self.world - 1) // self.world * self.world

    def reserve(self, max_tokens: int, top_k: int, hidden: int, device: torch.device) -> None:
        """Collective set-up for batches of up to ``max_tokens`` tokens: no later call within the
        bound allocates or synchronises."""
        self._buffers_for(max_tokens, top_k, hidden, device)

    def _buffers_for(self, num_tokens: int, top_k: int, hidden: int, device: torch.device) -> dict:
        key = (top_k, hidden, device)
        buf = self._buffers.get(key)
        if buf is None or buf["cap_tokens"] < num_tokens:
            if buf is not None:  # a larger batch than ever before: replace the buffers (collective)
                buf["recv"].close()
                buf["out"].close()
                del self._buffers[key]
            cap = self.capacity_for(num_tokens)
            recv = PeerBuffer(cap * top_k * hidden * 2, device, self.group)
            try:
                out = PeerBuffer(cap * hidden * 2, device, self.group)
            except PeerMemoryUnavailable:
                recv.close()
                raise
            buf = {"cap_tokens": cap, "recv": recv, "out": out, "per_batch": {},
                   "token": torch.zeros(1, dtype=torch.int32, device=device)}
            self._buffers[key] = buf
        return buf

    def state(self, num_tokens: int, top_k: int, hidden: int, device: torch.device) -> dict:
        """Buffers and tables for a batch of ``num_tokens`` tokens.  Allocates, maps and
        synchronises (collectively) only when the batch exceeds the capacity reserved so far; a
        smaller batch uses a prefix of the same buffers."""
        buf = self._buffers_for(num_tokens, top_k, hidden, device)
        st = buf["per_batch"].get(num_tokens)
        if st is None:
            if len(buf["per_batch"]) >= 64:
                buf["per_batch"].pop(next(iter(buf["per_batch"])))
            per = num_tokens // self.world
            slot_bytes = per * top_k * hidden * 2
            st = {
                "recv": buf["recv"], "out": buf["out"], "tokens_per_rank": per, "token": buf["token"],
                # Where this rank's rows go in every rank's receive buffer.
                "push_table": torch.tensor([p + self.rank * slot_bytes for p in buf["recv"].ptrs],
                                           dtype=torch.int64, device=device),
                "out_local": buf["out"].local.view(torch.bfloat16)[: num_tokens * hidden].view(
                    num_tokens, hidden),
            }
            buf["per_batch"][num_tokens] = st
        return st

    def close(self) -> None:
        """Unmaps and frees the peer-visible buffers (every rank, after the last step has
        finished on every rank)."""
        for buf in self._buffers.values():
            buf["recv"].close()
            buf["out"].close()
        self._buffers.clear()

    def finish(self, st: dict, output: torch.Tensor, top_k: int) -> None:
        """Everything after the second GEMM: barrier, combine + push, barrier, copy."""
        num_tokens, hidden = output.shape
        with _timed("barrier:gemm2_done"):
            dist.all_reduce(st["token"], group=self.group)
        with _timed("moe_sum_ranks_push"):
            _lib.check(_lib.load().b200moe_moe_sum_ranks_push(
                st["recv"].local.data_ptr(), st["out"].table.data_ptr(), self.world,
                self.rank * st["tokens_per_rank"], _lib.BF16,
                st["tokens_per_rank"], hidden, top_k,
                torch.cuda.current_stream(output.device).cuda_stream), "moe_sum_ranks_push")
        _lib.count_launches(1)
        with _timed("barrier:rows_landed"):
            dist.all_reduce(st["token"], group=self.group)
        with _timed("copy:result"):
            output.copy_(st["out_local"])


class CudaOps:
    """The arithmetic steps of the expert-parallel layer on the local GPU (C-ABI calls)."""

    def route(self, logits: torch.Tensor, top_k: int, renormalize: bool,
              out: Optional[Tuple[torch.Tensor, torch.Tensor]] = None
              ) -> Tuple[torch.Tensor, torch.Tensor]:
        """Routing weights (fp32) and expert ids (int32), ``[T, top_k]`` each; written into the
        tensors of ``out`` when given."""
        T = logits.shape[0]
        if out is not None:
            w, ids = out
        else:
            w = torch.empty(T, top_k, dtype=torch.float32, device=logits.device)
            ids = torch.empty(T, top_k, dtype=torch.int32, device=logits.device)
        with _timed("topk_softmax"):
            _C.topk_softmax(w, ids, logits.contiguous(), renormalize=renormalize)
        return w, ids

    def sort_pairs_by_expert(self, ids: torch.Tensor,
                             num_experts: int) -> Tuple[torch.Tensor, torch.Tensor]:
        """Stable order of the flat pair indices by expert, and the count per expert: token
        alignment with block size 1 (no padding)."""
        P = ids.numel()
        dev = ids.device
        order = torch.empty(max(P, 1), dtype=torch.int32, device=dev)
        blocks = torch.empty(max(P, 1), dtype=torch.int32, device=dev)
        npp = torch.empty(1, dtype=torch.int32, device=dev)
        offsets = torch.empty(num_experts + 1, dtype=torch.int32, device=dev)
        _C.moe_align_block_size(ids, num_experts, 1, order, blocks, npp, expert_offsets=offsets)
        return order[:P], offsets[1:] - offsets[:-1]

    def take_rows(self, src: torch.Tensor, index: torch.Tensor, top_k: int) -> torch.Tensor:
        """``dst[i] = src[index[i] // top_k]``."""
        n = index.numel()
        dst = torch.empty(n, src.shape[1], dtype=src.dtype, device=src.device)
        if n == 0:
            return dst
        count = torch.full((1,), n, dtype=torch.int32, device=src.device)
        rc = _lib.load().b200moe_gather_rows(
            src.data_ptr(), dst.data_ptr(), index.data_ptr(), count.data_ptr(), n, src.shape[0],
            src.shape[1], top_k, torch.cuda.current_stream(src.device).cuda_stream)
        _lib.check(rc, "gather_rows")
        _lib.count_launches(1)
        return dst

    def expert_ffn(self, rows: torch.Tensor, row_expert: torch.Tensor, row_weight: torch.Tensor,
                   w13: torch.Tensor, w2: torch.Tensor) -> torch.Tensor:
        """``y[i] = bf16(row_weight[i] * w2[e] (silu(w1[e] x) * (w3[e] x)))`` with ``e = row_expert[i]``
        over the local experts: alignment, gather, the two grouped GEMMs."""
        lib = _lib.load()
        R, H = rows.shape
        E, inter = w13.shape[0], w13.shape[1] // 2
        dev = rows.device
        out = torch.empty(R, H, dtype=rows.dtype, device=dev)
        if R == 0:
            return out
        cap = R + E * (BLOCK_SIZE_M - 1)
        nblk = (cap + BLOCK_SIZE_M - 1) // BLOCK_SIZE_M
        sorted_ids = torch.empty(cap, dtype=torch.int32, device=dev)
        expert_ids = torch.zeros(nblk, dtype=torch.int32, device=dev)
        npp = torch.empty(1, dtype=torch.int32, device=dev)
        a_sorted = torch.empty(cap, H, dtype=rows.dtype, device=dev)
        act = torch.empty(cap, inter, dtype=rows.dtype, device=dev)
        stream = torch.cuda.current_stream(dev).cuda_stream
        with _timed("moe_align_block_size"):
            _C.moe_align_block_size(row_expert, E, BLOCK_SIZE_M, sorted_ids, expert_ids, npp,
                                    fill_pads=True)
        with _timed("gather_rows"):
            _lib.check(lib.b200moe_gather_rows(rows.data_ptr(), a_sorted.data_ptr(),
                                               sorted_ids.data_ptr(), npp.data_ptr(), cap, R, H, 1,
                                               stream), "gather_rows")
        with _timed("grouped_gemm_w13_swiglu"):
            _lib.check(lib.b200moe_grouped_gemm_w13_swiglu(
                a_sorted.data_ptr(), w13.data_ptr(), act.data_ptr(), expert_ids.data_ptr(),
                npp.data_ptr(), cap, E, H, inter, BLOCK_SIZE_M, stream), "grouped_gemm_w13_swiglu")
        with _timed("grouped_gemm_w2_scale"):
            _lib.check(lib.b200moe_grouped_gemm_w2_scale(
                act.data_ptr(), w2.data_ptr(), out.data_ptr(), row_weight.data_ptr(),
                sorted_ids.data_ptr(), expert_ids.data_ptr(), npp.data_ptr(), cap, R, E, H, inter,
                BLOCK_SIZE_M, stream), "grouped_gemm_w2_scale")
        _lib.count_launches(3)
        return out

    def combine(self, y_back: torch.Tensor, order: torch.Tensor, out: torch.Tensor,
                top_k: int) -> None:
        """Puts returned rows back at their pair index and sums each token's ``top_k`` rows."""
        T, H = out.shape
        cache = torch.empty(T, top_k, H, dtype=out.dtype, device=out.device)
        rc = _lib.load().b200moe_scatter_rows(
            y_back.data_ptr(), cache.data_ptr(), order.data_ptr(), order.numel(), T * top_k, H,
            torch.cuda.current_stream(out.device).cuda_stream)
        _lib.check(rc, "scatter_rows")
        _lib.count_launches(1)
        with _timed("moe_sum"):
            _C.moe_sum(cache, out)


def split_sizes(counts_per_expert: List[int], ep_size: int) -> List[int]:
    """Rows this rank sends to every rank: experts are dealt out in contiguous groups."""
    per = len(counts_per_expert) // ep_size
    return [sum(counts_per_expert[r * per:(r + 1) * per]) for r in range(ep_size)]


def received_row_experts(recv_counts: torch.Tensor, total: int) -> torch.Tensor:
    """Local expert index (int32) of every received row.  ``recv_counts[s * per + j]`` rows come
    from source rank ``s`` for local expert ``j``; each source's rows arrive ordered by expert.
    ``total`` is the known row count, so no device synchronisation is needed."""
    ep_times_per = recv_counts.numel()
    return torch.repeat_interleave(
        torch.arange(ep_times_per, dtype=torch.int32, device=recv_counts.device),
        recv_counts.long(), output_size=total)


class ExpertParallelMoE(nn.Module):
    """Mixtral experts split across the ranks of ``group``; tokens are data-parallel.

    Parameters hold only the local experts: ``w13_weight [E/ep, 2I, H]``, ``w2_weight [E/ep, H, I]``
    with the same row layout and ``weight_loader(param, w, shard_id, expert_id)`` signature as
    ``FusedMoE`` (experts that live elsewhere are ignored by the loader).
    ``forward(hidden_states [T_local, H], router_logits [T_local, E])`` overwrites and returns
    ``hidden_states``.

    ``exchange``: with ``max_tokens_per_rank`` set, ``"auto"`` and ``"peer"`` use the peer-memory
    exchange for ANY token counts up to that bound (ragged batches, ranks with no tokens at all):
    buffers are sized for the bound once, shorter batches are padded with pair indices the
    alignment skips, and no step synchronises with the host; every rank must stay within the
    bound.  Without a bound, ``"auto"`` uses the NCCL all-to-alls (any token counts), and
    ``"peer"`` is a promise by the caller that every rank passes the same number of tokens in
    every call (buffers then grow with the largest batch seen).  The constructor arguments must be
    the same on every rank: they alone decide which collectives a call enters
    (``peer_capacity``).
    """

    def __init__(self, num_experts: int, top_k: int, hidden_size: int, intermediate_size: int,
                 params_dtype: Optional[torch.dtype] = None, renormalize: bool = True,
                 group: Optional[dist.ProcessGroup] = None, ops=None,
                 exchange: str = "auto", max_tokens_per_rank: Optional[int] = None):
        super().__init__()
        if exchange not in ("auto", "peer", "nccl"):
            raise ValueError("exchange must be 'auto', 'peer' or 'nccl'")
        if max_tokens_per_rank is not None and max_tokens_per_rank < 1:
            raise ValueError("max_tokens_per_rank must be positive")
        self.exchange = exchange
        self.max_tokens_per_rank = max_tokens_per_rank
        self._peer_states = {}
        self.group = group
        self.ep_size = dist.get_world_size(group)
        self.ep_rank = dist.get_rank(group)
        if num_experts % self.ep_size != 0:
            raise ValueError(f"num_experts ({num_experts}) must be divisible by the expert-parallel "
                             f"size ({self.ep_size})")
        self.num_experts = num_experts
        self.experts_per_rank = num_experts // self.ep_size
        self.first_expert = self.ep_rank * self.experts_per_rank
        self.top_k = top_k
        self.hidden_size = hidden_size
        self.intermediate_size = intermediate_size
        self.renormalize = renormalize
        self.params_dtype = params_dtype or torch.get_default_dtype()
        self.ops = ops if ops is not None else CudaOps()
        self.w13_weight = nn.Parameter(torch.empty(
            self.experts_per_rank, 2 * intermediate_size, hidden_size, dtype=self.params_dtype),
            requires_grad=False)
        self.w2_weight = nn.Parameter(torch.empty(
            self.experts_per_rank, hidden_size, intermediate_size, dtype=self.params_dtype),
            requires_grad=False)
        self.w13_weight.weight_loader = self.weight_loader
        self.w2_weight.weight_loader = self.weight_loader

    def weight_loader(self, param: nn.Parameter, loaded_weight: torch.Tensor, shard_id: str,
                      expert_id: int) -> None:
        local = expert_id - self.first_expert
        if not 0 <= local < self.experts_per_rank:
            return
        inter = self.intermediate_size
        if shard_id == "w1":
            param.data[local, :inter].copy_(loaded_weight)
        elif shard_id == "w3":
            param.data[local, inter:].copy_(loaded_weight)
        elif shard_id == "w2":
            param.data[local].copy_(loaded_weight)
        else:
            raise ValueError(f"unknown shard_id: {shard_id}")

    def _all_to_all(self, send: torch.Tensor, send_splits: List[int],
                    recv_splits: List[int]) -> torch.Tensor:
        recv = torch.empty((sum(recv_splits),) + tuple(send.shape[1:]), dtype=send.dtype,
                           device=send.device)
        dist.all_to_all_single(recv, send.contiguous(), recv_splits, send_splits, group=self.group)
        return recv

    # ------------------------------------------------------------------ peer-memory exchange
    def peer_capacity(self, num_tokens: int) -> Optional[int]:
        """Tokens per rank the peer-memory buffers must hold for this call, or None when the call
        takes the NCCL exchange.  The answer must be the same on every rank in every call, or the
        ranks would enter different collectives; so it depends only on the constructor arguments
        and, in forced ``"peer"`` mode without a bound, on a token count that the caller
        guarantees to be equal on all ranks:

        * ``max_tokens_per_rank`` given: always that bound (ragged batches are padded up to it);
        * ``exchange="peer"`` without a bound: the power-of-two bucket of ``num_tokens``;
        * ``exchange="auto"`` without a bound, or ``"nccl"``: None.  Token counts that differ
          between ranks, or change unevenly from call to call, are exactly what the NCCL exchange
          is for, and nothing that one rank alone can see tells it what the others hold.
        """
        if self.exchange == "nccl":
            return None
        if self.max_tokens_per_rank is not None:
            return self.max_tokens_per_rank
        if self.exchange == "peer":
            return capacity_bucket(num_tokens)
        return None

    def _peer_state(self, num_tokens: int, hidden: int, device: torch.device):
        """Buffers of the peer-memory path, or None when the call takes the NCCL exchange.
        Set-up (allocation, mapping, synchronisation) happens the first time and whenever the
        capacity grows, on every rank in the same call."""
        cap_tokens = self.peer_capacity(num_tokens)
        if cap_tokens is None:
            return None
        key = (hidden, device)
        state = self._peer_states.get(key)
        if state is not None and state["cap_tokens"] >= cap_tokens:
            return state
        if state is not None:  # the bucket grew: replace the buffers (collective)
            state["x_stage"].close()
            state["cache3"].close()
            del self._peer_states[key]
        ep, k, per = self.ep_size, self.top_k, self.experts_per_rank
        pairs_total = ep * cap_tokens * k
        cap = pairs_total + per * (BLOCK_SIZE_M - 1)
        i32 = dict(dtype=torch.int32, device=device)
        bf16 = dict(dtype=torch.bfloat16, device=device)
        try:
            x_stage = PeerBuffer(cap_tokens * hidden * 2, device, self.group)
            try:
                cache3 = PeerBuffer(cap_tokens * k * hidden * 2, device, self.group)
            except PeerMemoryUnavailable:
                x_stage.close()
                raise
        except PeerMemoryUnavailable as e:
            # Every rank lands here together.  Forced peer mode has no other way; otherwise
            # the NCCL exchange takes over for good.
            if self.exchange == "peer":
                raise
            import warnings
            warnings.warn(f"ExpertParallelMoE: peer-memory exchange unavailable ({e}); "
                          "using NCCL all-to-alls")
            self.exchange = "nccl"
            return None
        state = {
            "x_stage": x_stage, "cache3": cache3, "capacity": cap, "cap_tokens": cap_tokens,
            "x_local": x_stage.local.view(torch.bfloat16).view(cap_tokens, hidden),
            "c3_local": cache3.local.view(torch.bfloat16).view(cap_tokens, k, hidden),
            # Own routing result, padded to cap_tokens rows: row 0 the expert ids (-1 never matches
            # an expert), row 1 the bits of the fp32 routing weights.  One all-gather moves both.
            "own": torch.full((2, cap_tokens * k), -1, **i32),
            "all": torch.empty(ep, 2, cap_tokens * k, **i32),
            "w_all": torch.empty(pairs_total, dtype=torch.float32, device=device),
            "sorted_ids": torch.empty(cap, **i32),
            "expert_ids": torch.zeros((cap + BLOCK_SIZE_M - 1) // BLOCK_SIZE_M, **i32),
            "num_post_pad": torch.zeros(1, **i32),
            "align_ws": torch.empty(max(_C.align_workspace_numel(pairs_total, per), 1), **i32),
            "a_sorted": torch.empty(cap, hidden, **bf16),
            "act": torch.empty(cap, self.intermediate_size, **bf16),
            "token": torch.zeros(1, **i32),
        }
        self._peer_states[key] = state
        return state

    def close(self) -> None:
        """Unmaps and frees the peer-visible buffers of the peer-memory exchange (every rank,
        after the last step has finished on every rank)."""
        for st in self._peer_states.values():
            st["x_stage"].close()
            st["cache3"].close()
        self._peer_states.clear()

    def _forward_peer(self, st: dict, hidden_states: torch.Tensor,
                      router_logits: torch.Tensor) -> torch.Tensor:
        lib = _lib.load()
        ep, per, k = self.ep_size, self.experts_per_rank, self.top_k
        num_tokens, hidden = hidden_states.shape
        dev = hidden_states.device
        cap, cap_tokens = st["capacity"], st["cap_tokens"]
        if num_tokens > cap_tokens:
            raise RuntimeError(f"ExpertParallelMoE: {num_tokens} tokens exceed max_tokens_per_rank="
                               f"{cap_tokens}")
        own = st["own"]
        if num_tokens < cap_tokens:  # a short batch: rows past num_tokens carry ids the alignment skips
            own[0, num_tokens * k:].fill_(-1)
        if num_tokens > 0:  # the router writes straight into the buffer that is exchanged
            self.ops.route(router_logits, k, self.renormalize,
                           out=(own[1, : num_tokens * k].view(torch.float32).view(num_tokens, k),
                                own[0, : num_tokens * k].view(num_tokens, k)))
        with _timed("copy:stage_tokens"):
            st["x_local"][:num_tokens].copy_(hidden_states)
        # The all-gather also orders every rank's staging copy before any rank's gather.
        with _timed("all_gather:ids_weights"):
            dist.all_gather_into_tensor(st["all"], own, group=self.group)
        local_ids = st["all"][:, 0, :] - self.first_expert  # other ranks' experts fall outside [0, per)
        st["w_all"].view(ep, cap_tokens * k).copy_(st["all"][:, 1, :].view(torch.float32))
        stream = torch.cuda.current_stream(dev).cuda_stream
        with _timed("moe_align_block_size"):
            _C.moe_align_block_size(local_ids, per, BLOCK_SIZE_M, st["sorted_ids"], st["expert_ids"],
                                    st["num_post_pad"], fill_pads=True, workspace=st["align_ws"])
        with _timed("gather_rows"):
            _lib.check(lib.b200moe_gather_rows_peer(
                st["x_stage"].table.data_ptr(), ep, cap_tokens, st["a_sorted"].data_ptr(),
                st["sorted_ids"].data_ptr(), st["num_post_pad"].data_ptr(), cap, hidden, k, stream),
                "gather_rows_peer")
        with _timed("grouped_gemm_w13_swiglu"):
            _lib.check(lib.b200moe_grouped_gemm_w13_swiglu(
                st["a_sorted"].data_ptr(), self.w13_weight.data_ptr(), st["act"].data_ptr(),
                st["expert_ids"].data_ptr(), st["num_post_pad"].data_ptr(), cap, per, hidden,
                self.intermediate_size, BLOCK_SIZE_M, stream), "grouped_gemm_w13_swiglu")
        with _timed("grouped_gemm_w2_scale"):
            _lib.check(lib.b200moe_grouped_gemm_w2_scale_peer(
                st["act"].data_ptr(), self.w2_weight.data_ptr(), st["cache3"].table.data_ptr(), ep,
                cap_tokens * k, st["w_all"].data_ptr(), st["sorted_ids"].data_ptr(),
                st["expert_ids"].data_ptr(), st["num_post_pad"].data_ptr(), cap, per, hidden,
                self.intermediate_size, BLOCK_SIZE_M, stream), "grouped_gemm_w2_scale_peer")
        _lib.count_launches(3)
        # Every rank's second GEMM (whose epilogue wrote into this rank's buffer) has finished once
        # this one-word all-reduce completes.
        with _timed("barrier:gemm2_done"):
            dist.all_reduce(st["token"], group=self.group)
        with _timed("moe_sum"):
            _C.moe_sum(st["c3_local"][:num_tokens], hidden_states)
        return hidden_states

    def forward(self, hidden_states: torch.Tensor, router_logits: torch.Tensor) -> torch.Tensor:
        if self.exchange != "nccl" and isinstance(self.ops, CudaOps):
            st = self._peer_state(hidden_states.shape[0], hidden_states.shape[1],
                                  hidden_states.device)
            if st is not None:
                return self._forward_peer(st, hidden_states, router_logits)
        ops, ep, per = self.ops, self.ep_size, self.experts_per_rank
        dev = hidden_states.device
        weights, ids = ops.route(router_logits, self.top_k, self.renormalize)
        order, counts = ops.sort_pairs_by_expert(ids, self.num_experts)

        # Per-expert counts: rank r receives, from every source, the counts of its own experts.
        recv_counts = torch.empty(ep * per, dtype=counts.dtype, device=dev)
        dist.all_to_all_single(recv_counts, counts.contiguous(), group=self.group)
        both = torch.cat([counts, recv_counts]).cpu()  # the one host synchronisation of the layer
        send_counts = both[: self.num_experts].tolist()
        recv_counts_host = both[self.num_experts:].view(ep, per)
        send_splits = split_sizes(send_counts, ep)
        recv_splits = [int(recv_counts_host[s].sum()) for s in range(ep)]

        send_rows = ops.take_rows(hidden_states, order, self.top_k)
        send_w = weights.reshape(-1)[order.long()]
        recv_rows = self._all_to_all(send_rows, send_splits, recv_splits)
        recv_w = self._all_to_all(send_w, send_splits, recv_splits)
        row_expert = received_row_experts(recv_counts, sum(recv_splits)) % per

        y = ops.expert_ffn(recv_rows, row_expert, recv_w.contiguous(), self.w13_weight,
                           self.w2_weight)
        y_back = self._all_to_all(y, recv_splits, send_splits)
        ops.combine(y_back, order, hidden_states, self.top_k)
        return hidden_states
