"""Python wrapper of token alignment, same signature and return values as the reference's
``moe_align_block_size`` (layers/moe/moe_align_block_size.py:6-62)."""
from __future__ import annotations

from typing import Tuple

import torch

from ... import _C


def moe_align_block_size(topk_ids: torch.Tensor, block_size: int,
                         num_experts: int) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Sorts the flat (token, slot) pairs by expert and pads every expert to ``block_size``.

    Returns ``(sorted_token_ids, expert_ids, num_tokens_post_pad)`` with the reference's sizes:
    ``sorted_token_ids`` holds ``numel + num_experts * (block_size - 1)`` int32 with ``-1`` in
    every slot that carries no pair, ``expert_ids`` holds one int32 per block (zero beyond the
    used blocks).  The reference needs four launches for this (fill, zeros, empty, kernel); here
    the ``-1`` padding is written by the alignment kernel itself.
    """
    max_num_tokens_padded = topk_ids.numel() + num_experts * (block_size - 1)
    sorted_ids = torch.empty((max_num_tokens_padded,), dtype=torch.int32, device=topk_ids.device)
    max_num_m_blocks = (max_num_tokens_padded + block_size - 1) // block_size
    expert_ids = torch.zeros((max_num_m_blocks,), dtype=torch.int32, device=topk_ids.device)
    num_tokens_post_pad = torch.empty((1,), dtype=torch.int32, device=topk_ids.device)
    _C.moe_align_block_size(topk_ids, num_experts, block_size, sorted_ids, expert_ids,
                            num_tokens_post_pad, fill_pads=True)
    return sorted_ids, expert_ids, num_tokens_post_pad
