"""``RMSNorm`` with the reference's interface (layers/layernorm.py:5-57): ``forward(x)`` returns the
normalised tensor, ``forward(x, residual)`` returns ``(normalised, x + residual)``.  One fused kernel
does the add, the reduction and the scaling; like the reference's native op it works in place, so
the returned tensors alias the arguments."""
from __future__ import annotations

import torch
from torch import nn

from .. import _C


class RMSNorm(nn.Module):
    def __init__(self, hidden_size: int, eps: float = 1e-5) -> None:
        super().__init__()
        self.hidden_size = hidden_size
        self.eps = eps
        self.weight = nn.Parameter(torch.ones(hidden_size))

    def forward(self, x: torch.Tensor, residual: torch.Tensor | None = None):
        flat = x.view(-1, self.hidden_size)
        if residual is None:
            _C.rms_norm(flat, self.eps, self.weight)
            return x
        _C.add_rms_norm(flat, residual.view(-1, self.hidden_size), self.eps, self.weight)
        return x, residual
