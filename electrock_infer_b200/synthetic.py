"""Seeded synthetic inputs of the MoE layer: the workload definitions used by tests and benchmarks.

Shapes and distributions: activations ``x ~ N(0, 1)``; router weight ``W[E, H] ~ N(0, 0.02^2)``;
expert weights ``w1, w3 [I, H] ~ N(0, 1/H)`` and ``w2 [H, I] ~ N(0, 1/I)`` (standard deviation
``1/sqrt(fan_in)``), drawn in fp32 and cast to the working dtype; ``w13 = cat(w1, w3)`` per
expert, the row layout the reference's weight loader produces (layers/moe/mixtral_moe.py:132-150).
Router logits are computed in fp32 from the cast activations, ``x.float() @ W.float().T``, plus an
optional per-expert bias that skews the expert load.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, replace
from typing import Dict, Optional, Sequence

import torch


@dataclass(frozen=True)
class MoEWorkload:
    name: str
    num_tokens: int
    hidden: int
    inter: int
    num_experts: int = 8
    top_k: int = 2
    dtype: torch.dtype = torch.bfloat16
    seed: int = 0
    logit_bias: Optional[Sequence[float]] = None

    @property
    def flops(self) -> int:
        """Algorithmic FLOPs of the two grouped GEMMs: 6 * H * I * top_k per token."""
        return 6 * self.hidden * self.inter * self.top_k * self.num_tokens

    def with_tokens(self, num_tokens: int) -> "MoEWorkload":
        return replace(self, num_tokens=num_tokens)


SKEW_BIAS = (2.0, 1.0, 0.5, 0.0, 0.0, -0.5, -1.0, -2.0)

WORKLOADS: Dict[str, MoEWorkload] = {
    # Small fp32 layer that the torch CPU path runs in a fraction of a second.
    "small_fp32": MoEWorkload("small_fp32", 64, 512, 1024, dtype=torch.float32, seed=0),
    # Mixtral-8x7B, decode-sized batch, near-uniform expert load.
    "mixtral_decode_t256": MoEWorkload("mixtral_decode_t256", 256, 4096, 14336, seed=1),
    # Mixtral-8x7B, prefill-sized batch, busiest expert about 4x the idlest.
    "mixtral_prefill_t8192_skew": MoEWorkload("mixtral_prefill_t8192_skew", 8192, 4096, 14336,
                                              seed=2, logit_bias=SKEW_BIAS),
    # Mixtral-8x7B, multi-GPU step (tensor- or expert-parallel).
    "mixtral_parallel_t16384": MoEWorkload("mixtral_parallel_t16384", 16384, 4096, 14336, seed=3),
}


def make_inputs(wl: MoEWorkload, device: str | torch.device = "cpu", device_rng: bool = False,
                inter_slice: Optional[slice] = None,
                expert_slice: Optional[slice] = None) -> Dict[str, torch.Tensor]:
    """Draws ``x``, ``router_w``, ``logits`` (fp32), ``w13`` and ``w2`` for a workload.

    Values come from a CPU generator seeded with ``wl.seed`` and are therefore identical wherever
    they are drawn; ``device_rng=True`` draws on ``device`` instead (same distributions, different
    values, much faster for the full-size benchmark weights).  ``inter_slice`` keeps only a range
    of the intermediate dimension (a tensor-parallel shard: rows of w1/w3, columns of w2) and
    ``expert_slice`` only a range of experts (an expert-parallel shard); routing inputs are never
    sliced.  Expert weights are produced one expert at a time to bound host memory.
    """
    device = torch.device(device)
    rng_device = device if device_rng else torch.device("cpu")
    gen = torch.Generator(device=rng_device).manual_seed(wl.seed)
    T, H, I, E = wl.num_tokens, wl.hidden, wl.inter, wl.num_experts

    def randn(*shape):
        return torch.randn(*shape, generator=gen, device=rng_device, dtype=torch.float32)

    x = randn(T, H).to(wl.dtype).to(device)
    router_w = (randn(E, H) * 0.02).to(wl.dtype).to(device)
    logits = x.float() @ router_w.float().T
    if wl.logit_bias is not None:
        logits = logits + torch.tensor(list(wl.logit_bias), dtype=torch.float32, device=device)

    isl = inter_slice or slice(0, I)
    experts = range(E)[expert_slice] if expert_slice is not None else range(E)
    i_len = len(range(I)[isl])
    w13 = torch.empty(len(experts), 2 * i_len, H, dtype=wl.dtype, device=device)
    w2 = torch.empty(len(experts), H, i_len, dtype=wl.dtype, device=device)
    for e in range(E):
        # Every expert is drawn even when it is not kept, so that a shard sees the same values
        # as the full layer.
        w1_e = randn(I, H) * (1.0 / math.sqrt(H))
        w3_e = randn(I, H) * (1.0 / math.sqrt(H))
        w2_e = randn(H, I) * (1.0 / math.sqrt(I))
        if e in experts:
            j = e - experts[0]
            w13[j, :i_len].copy_(w1_e[isl].to(wl.dtype))
            w13[j, i_len:].copy_(w3_e[isl].to(wl.dtype))
            w2[j].copy_(w2_e[:, isl].to(wl.dtype))
    return {"x": x, "router_w": router_w, "logits": logits.contiguous(), "w13": w13, "w2": w2}
