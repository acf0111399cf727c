"""Seeded inputs of the RMSNorm fixtures (tests/golden/rmsnorm.npz): shared by the generator that
runs the reference's ``RMSNorm`` and by the tests that check the oracle and the CUDA kernels."""
import torch

RMSNORM_CASES = {  # name: (rows, hidden, dtype, eps)
    "bf16_h4096": (24, 4096, torch.bfloat16, 1e-5),
    "bf16_h520": (7, 520, torch.bfloat16, 1e-6),
    "f16_h1024": (16, 1024, torch.float16, 1e-5),
    "f32_h768": (9, 768, torch.float32, 1e-5),
}


def rmsnorm_inputs(name: str):
    """``(x, residual, weight, eps)`` of one case."""
    rows, hidden, dtype, eps = RMSNORM_CASES[name]
    g = torch.Generator().manual_seed(sum(map(ord, name)))
    x = (torch.randn(rows, hidden, generator=g) * 3.0).to(dtype)
    residual = torch.randn(rows, hidden, generator=g).to(dtype)
    weight = (1.0 + 0.1 * torch.randn(hidden, generator=g)).to(dtype)
    return x, residual, weight, eps
