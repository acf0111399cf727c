"""libb200moe against the reference's own CUDA ops, compiled unmodified by oracle/build_ref_ops.py
(WARP_SIZE 32) and run on the same GPU with the same inputs.  Integer outputs and the two
element-wise ops must agree bit for bit.  Skipped when the oracle build is absent."""
import importlib.util
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

from electrock_infer_b200 import _C

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
REF_DIR = Path(__file__).resolve().parent.parent / "oracle" / "_ref"


@pytest.fixture(scope="module")
def ref_ops():
    hits = sorted(REF_DIR.glob("ref_ops*.so"))
    if not hits:
        pytest.skip("oracle/_ref/ref_ops is not built (needs the reference source tree)")
    spec = importlib.util.spec_from_file_location("ref_ops", hits[0])
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def bits(t):
    return t.view({2: torch.int16, 4: torch.int32}[t.element_size()])


@pytest.mark.parametrize("T", [4, 64, 1000, 8192, 100000])
def test_topk_softmax_matches_reference_kernel(ref_ops, T):
    # The reference kernel reads past its input unless T is a multiple of 4: only such T are run.
    assert T % 4 == 0
    g = torch.Generator().manual_seed(T)
    logits = (torch.randn(T, 8, generator=g) * 2).to(DEV)
    w0 = torch.empty(T, 2, device=DEV); i0 = torch.empty(T, 2, dtype=torch.int32, device=DEV)
    w1 = torch.empty(T, 2, device=DEV); i1 = torch.empty(T, 2, dtype=torch.int32, device=DEV)
    ref_ops.topk_softmax(w0, i0, logits)
    _C.topk_softmax(w1, i1, logits)
    assert torch.equal(i0, i1)                       # bit-exact expert choice
    assert (w0 - w1).abs().max().item() <= 1e-6      # different summation order of the softmax


def test_topk_softmax_tie_rule_matches_reference_kernel(ref_ops):
    logits = torch.tensor([[1.0, 1.0, 0, 0, 0, 0, 0, 0], [0, 3.0, 3.0, 3.0, 0, 0, 0, 0],
                           [5.0, 0, 0, 0, 0, 0, 0, 5.0], [0.0] * 8], device=DEV)
    w0 = torch.empty(4, 2, device=DEV); i0 = torch.empty(4, 2, dtype=torch.int32, device=DEV)
    w1 = torch.empty(4, 2, device=DEV); i1 = torch.empty(4, 2, dtype=torch.int32, device=DEV)
    ref_ops.topk_softmax(w0, i0, logits)
    _C.topk_softmax(w1, i1, logits)
    assert torch.equal(i0, i1) and i1.tolist() == [[0, 1], [1, 2], [0, 7], [0, 1]]


@pytest.mark.parametrize("numel,bs", [(2, 64), (128, 16), (1000, 64), (16384, 64), (16384, 128),
                                      (65536, 128), (200000, 64)])
@pytest.mark.parametrize("dtype", [torch.int32, torch.int64])
def test_align_matches_reference_kernel(ref_ops, numel, bs, dtype):
    g = torch.Generator().manual_seed(numel)
    ids = torch.randint(0, 8, (numel,), generator=g).to(dtype).to(DEV)
    cap = numel + 8 * (bs - 1)
    outs = []
    for fn in (ref_ops.moe_align_block_size, _C.moe_align_block_size):
        s = torch.full((cap,), -1, dtype=torch.int32, device=DEV)
        e = torch.zeros((cap + bs - 1) // bs, dtype=torch.int32, device=DEV)
        n = torch.zeros(1, dtype=torch.int32, device=DEV)
        fn(ids, 8, bs, s, e, n)
        outs.append((s, e, n))
    for a, b in zip(*outs):
        assert torch.equal(a, b)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("rows,d", [(1024, 7168), (33, 14336), (7, 224)])
def test_silu_and_mul_matches_reference_kernel(ref_ops, dtype, rows, d):
    g = torch.Generator().manual_seed(d)
    x = (torch.randn(rows, 2 * d, generator=g) * 3).to(dtype).to(DEV)
    a = torch.empty(rows, d, dtype=dtype, device=DEV)
    b = torch.empty(rows, d, dtype=dtype, device=DEV)
    ref_ops.silu_and_mul(a, x)
    _C.silu_and_mul(b, x)
    assert torch.equal(bits(a), bits(b))


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
def test_moe_sum_matches_reference_kernel(ref_ops, dtype):
    g = torch.Generator().manual_seed(3)
    x = (torch.randn(1024, 2, 4096, generator=g) * 4).to(dtype).to(DEV)
    x[0, :, :8] = -0.0
    a = torch.empty(1024, 4096, dtype=dtype, device=DEV)
    b = torch.empty(1024, 4096, dtype=dtype, device=DEV)
    ref_ops.moe_sum(x, a)
    _C.moe_sum(x, b)
    assert torch.equal(bits(a), bits(b))
    if dtype != torch.bfloat16:  # the reference's interleaved variant has no bf16 instantiation
        xi = x.permute(0, 2, 1).contiguous()
        ref_ops.moe_sum_efficient(xi, a)
        _C.moe_sum_efficient(xi, b)
        assert torch.equal(bits(a), bits(b))
