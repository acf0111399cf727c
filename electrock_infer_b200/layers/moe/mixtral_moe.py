"""``FusedMoE``: the tensor-parallel Mixtral expert layer with the reference's constructor,
parameters, ``forward`` and ``weight_loader`` (layers/moe/mixtral_moe.py:8-152)."""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist
import torch.nn as nn

from .fused_moe import _timed, fused_experts


class FusedMoE(nn.Module):
    """Unquantised Mixtral experts, sharded over the intermediate dimension.

    Parameters (reference mixtral_moe.py:64-79):
      ``w13_weight [E, 2 * I / tp, H]``  gate rows ``[0, I/tp)`` then up rows ``[I/tp, 2I/tp)``
      ``w2_weight  [E, H, I / tp]``
    both ``requires_grad=False`` and carrying ``.weight_loader``.

    ``forward(hidden_states [T, H], router_logits [T, E])`` overwrites ``hidden_states`` with the
    layer output and returns it (same storage); with ``reduce_results`` and ``tp_size > 1`` the
    result is summed over the default process group first (:114-116).

    Extension: ``tp_exchange`` chooses how that sum is done.  ``"nccl"`` is the reference's
    all-reduce of the ``[T, H]`` result.  ``"peer"`` does it inside the layer's own kernels over
    NVLink peer mappings (``parallel.TensorParallelReduce``; needs ``T`` divisible by ``tp_size``
    and all ranks on one node).  ``"auto"`` (default) uses the peer path when it applies and the
    result is at least ``PEER_REDUCE_MIN_BYTES`` large, else NCCL.
    """

    PEER_REDUCE_MIN_BYTES = 4 << 20

    def __init__(self, num_experts: int, top_k: int, hidden_size: int, intermediate_size: int,
                 tp_size: Optional[int] = None, params_dtype: Optional[torch.dtype] = None,
                 renormalize: bool = True, reduce_results: bool = False,
                 tp_exchange: str = "auto"):
        super().__init__()
        if tp_exchange not in ("auto", "peer", "nccl"):
            raise ValueError("tp_exchange must be 'auto', 'peer' or 'nccl'")
        self.tp_exchange = tp_exchange
        self._tp_reduce = None
        initialised = dist.is_available() and dist.is_initialized()
        if tp_size is None:
            tp_size = dist.get_world_size() if initialised else 1
        self.tp_size = tp_size
        self.tp_rank = dist.get_rank() if initialised else 0

        self.num_experts = num_experts
        self.top_k = top_k
        self.hidden_size = hidden_size
        self.intermediate_size = intermediate_size
        self.renormalize = renormalize
        self.reduce_results = reduce_results
        self.params_dtype = params_dtype or torch.get_default_dtype()

        if self.intermediate_size % self.tp_size != 0:
            raise ValueError(f"intermediate_size ({self.intermediate_size}) must be divisible by "
                             f"tp_size ({self.tp_size})")
        self.intermediate_size_per_partition = self.intermediate_size // self.tp_size

        self.w13_weight = nn.Parameter(
            torch.empty(self.num_experts, 2 * self.intermediate_size_per_partition,
                        self.hidden_size, dtype=self.params_dtype), requires_grad=False)
        self.w2_weight = nn.Parameter(
            torch.empty(self.num_experts, self.hidden_size, self.intermediate_size_per_partition,
                        dtype=self.params_dtype), requires_grad=False)
        self.w13_weight.weight_loader = self.weight_loader
        self.w2_weight.weight_loader = self.weight_loader

    def peer_reduce_for(self, hidden_states: torch.Tensor):
        """The ``TensorParallelReduce`` to hand to ``fused_experts`` for this batch, or None when
        the sum (if any) is an NCCL all-reduce.  Every rank sees the same token count, so every
        rank decides the same way."""
        if not (self.reduce_results and self.tp_size > 1) or self.tp_exchange == "nccl":
            return None
        num_tokens, hidden = hidden_states.shape
        applies = (hidden_states.is_cuda and self.top_k == 2 and self.tp_size <= 8
                   and self.tp_size == dist.get_world_size() and dist.get_backend() == "nccl"
                   and num_tokens > 0 and num_tokens % self.tp_size == 0)
        if self.tp_exchange == "peer":
            if not applies:
                raise RuntimeError("tp_exchange='peer' needs CUDA tensors, NCCL, top_k=2, tp_size <= 8 "
                                   "and a token count divisible by tp_size")
        elif not applies or num_tokens * hidden * hidden_states.element_size() < self.PEER_REDUCE_MIN_BYTES:
            return None
        from ...parallel import PeerMemoryUnavailable, TensorParallelReduce
        if self._tp_reduce is None:
            self._tp_reduce = TensorParallelReduce()
        try:  # set-up on first use; fails on every rank alike when peer mappings are not possible
            self._tp_reduce.state(num_tokens, self.top_k, hidden, hidden_states.device)
        except PeerMemoryUnavailable as e:
            if self.tp_exchange == "peer":
                raise
            import warnings
            warnings.warn(f"FusedMoE: in-kernel tensor-parallel reduce unavailable ({e}); "
                          "using the NCCL all-reduce")
            self.tp_exchange = "nccl"
            return None
        return self._tp_reduce

    def forward(self, hidden_states: torch.Tensor, router_logits: torch.Tensor) -> torch.Tensor:
        tp_reduce = self.peer_reduce_for(hidden_states)
        final_hidden_states = fused_experts(
            hidden_states=hidden_states, w1=self.w13_weight, w2=self.w2_weight,
            gating_output=router_logits, topk=self.top_k, renormalize=self.renormalize,
            inplace=True, activation="silu", tp_reduce=tp_reduce)
        if self.reduce_results and self.tp_size > 1 and tp_reduce is None:
            with _timed("all_reduce:result"):
                dist.all_reduce(final_hidden_states)
        return final_hidden_states

    def weight_loader(self, param: nn.Parameter, loaded_weight: torch.Tensor, shard_id: str,
                      expert_id: int) -> None:
        """Copies this rank's slice of one checkpoint tensor into the stacked parameter
        (reference mixtral_moe.py:121-152): ``w1``/``w3`` are ``[I, H]`` and are sliced by rows
        into the gate/up halves of ``w13_weight[expert_id]``; ``w2`` is ``[H, I]`` and is sliced
        by columns."""
        shard = self.intermediate_size_per_partition
        param_data = param.data[expert_id]
        if shard_id in ("w1", "w3"):
            loaded = loaded_weight.narrow(0, shard * self.tp_rank, shard)
            if shard_id == "w1":
                param_data[:shard, :].copy_(loaded)
            else:
                param_data[shard:, :].copy_(loaded)
        elif shard_id == "w2":
            loaded = loaded_weight.narrow(1, shard * self.tp_rank, shard)
            param_data.copy_(loaded)
        else:
            raise ValueError(f"unknown shard_id: {shard_id}")


class MixtralMoE(nn.Module):
    """Gate + experts, the block the reference's decoder layer calls (models/mixtral.py:21-63):
    ``gate`` is a replicated bias-free linear layer ``[hidden -> num_experts]`` (its parameter is
    ``gate.weight`` with the loader signature of layers/linear.py:47-49) and ``experts`` is a
    ``FusedMoE`` with ``reduce_results=True, renormalize=True``.

    ``forward(hidden_states)`` accepts 1-D or 2-D token shapes, overwrites the tokens with the
    layer output and returns them in the original shape, like the reference.  Unlike the
    reference, the gate projection is not a separate GEMM: the router kernel computes it while it
    reads the tokens.  ``fuse_gate=False`` restores the separate ``F.linear``.
    """

    def __init__(self, num_experts: int, top_k: int, hidden_size: int, intermediate_size: int,
                 params_dtype: Optional[torch.dtype] = None, tp_size: Optional[int] = None,
                 prefix: str = "", fuse_gate: bool = True, tp_exchange: str = "auto"):
        super().__init__()
        self.hidden_size = hidden_size
        self.fuse_gate = fuse_gate
        self.gate = nn.Linear(hidden_size, num_experts, bias=False,
                              dtype=params_dtype or torch.get_default_dtype())
        self.gate.weight.requires_grad_(False)
        self.gate.weight.weight_loader = self._gate_weight_loader
        self.experts = FusedMoE(num_experts=num_experts, top_k=top_k, hidden_size=hidden_size,
                                intermediate_size=intermediate_size, params_dtype=params_dtype,
                                reduce_results=True, renormalize=True, tp_size=tp_size,
                                tp_exchange=tp_exchange)

    @staticmethod
    def _gate_weight_loader(param: nn.Parameter, loaded_weight: torch.Tensor) -> None:
        assert param.size() == loaded_weight.size()
        param.data.copy_(loaded_weight)

    def forward(self, hidden_states: torch.Tensor) -> torch.Tensor:
        orig_shape = hidden_states.shape
        hidden_states = hidden_states.view(-1, self.hidden_size)
        if self.fuse_gate:
            tp_reduce = self.experts.peer_reduce_for(hidden_states)
            out = fused_experts(hidden_states, self.experts.w13_weight, self.experts.w2_weight, None,
                                self.experts.top_k, renormalize=True, inplace=True,
                                gate_weight=self.gate.weight, tp_reduce=tp_reduce)
            if self.experts.tp_size > 1 and tp_reduce is None:
                with _timed("all_reduce:result"):
                    dist.all_reduce(out)
        else:
            out = self.experts(hidden_states, self.gate(hidden_states))
        return out.view(orig_shape)
