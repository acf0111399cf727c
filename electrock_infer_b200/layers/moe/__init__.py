"""MoE layer modules, laid out like the reference's ``electrock_infer/layers/moe`` package."""
from .fused_moe import fused_experts, fused_topk
from .mixtral_moe import FusedMoE, MixtralMoE
from .moe_align_block_size import moe_align_block_size

__all__ = ["FusedMoE", "MixtralMoE", "fused_experts", "fused_topk", "moe_align_block_size"]
