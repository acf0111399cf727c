"""Fused residual-add + RMSNorm against the reference's torch formulation (restated in the oracle)."""
import pytest
import torch

from electrock_infer_b200 import _C
from electrock_infer_b200.layers.layernorm import RMSNorm
from oracle import moe_oracle

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
ULP = {torch.bfloat16: 2.0 ** -7, torch.float16: 2.0 ** -10, torch.float32: 2.0 ** -22}


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("T,H", [(1, 8), (7, 4096), (300, 4096), (5, 1000), (33, 8192), (2, 16384)])
@pytest.mark.parametrize("with_residual", [False, True])
def test_rms_norm(dtype, T, H, with_residual):
    if dtype == torch.float32 and H > 8192:
        pytest.skip("fp32 rows are limited to 8192 elements")
    g = torch.Generator().manual_seed(T + H)
    x = (torch.randn(T, H, generator=g) * 2).to(dtype)
    res = (torch.randn(T, H, generator=g) * 2).to(dtype) if with_residual else None
    w = (1 + 0.1 * torch.randn(H, generator=g)).to(dtype)
    dx, dw = x.to(DEV), w.to(DEV)
    if with_residual:
        dres = res.to(DEV)
        _C.add_rms_norm(dx, dres, 1e-5, dw)
        want, want_res = moe_oracle.rms_norm_ref(x, w, 1e-5, res)
        as_int = torch.int32 if dtype == torch.float32 else torch.int16
        assert torch.equal(dres.cpu().view(as_int), want_res.view(as_int))   # exact: one fp32 add, one cast
    else:
        _C.rms_norm(dx, 1e-5, dw)
        want = moe_oracle.rms_norm_ref(x, w, 1e-5)
    got = dx.cpu().float()
    # The row sum of squares is accumulated in another order than torch's: the scale can differ in
    # its last fp32 bits, which may move a rounded output to the neighbouring value.
    if dtype == torch.float32:
        assert torch.allclose(got, want.float(), rtol=2e-6, atol=1e-6)
    else:
        assert ((got - want.float()).abs() <= 2 * ULP[dtype] * want.float().abs() + 1e-6).all()
        assert (got == want.float()).float().mean() > 0.97


@pytest.mark.parametrize("case", ["bf16_h4096", "bf16_h520", "f16_h1024", "f32_h768"])
def test_rms_norm_against_reference_fixture(golden, case):
    """The kernels against what the reference's own ``RMSNorm`` module returned on the same seeded
    inputs (tests/golden/rmsnorm.npz): the new residual bit for bit, the output to one rounding
    step of the element type (the kernel sums the squares in another order)."""
    from rmsnorm_cases import rmsnorm_inputs
    x, residual, weight, eps = rmsnorm_inputs(case)
    fx = golden["rmsnorm"]
    dtype = x.dtype

    def from_fixture(key):
        a = torch.from_numpy(fx[f"{case}_{key}"])
        return a if dtype == torch.float32 else a.view(dtype)

    def close(got, want):
        got, want = got.cpu().float(), want.float()
        if dtype == torch.float32:
            return torch.allclose(got, want, rtol=2e-6, atol=1e-6)
        return bool(((got - want).abs() <= 2 * ULP[dtype] * want.abs() + 1e-6).all())

    dx = x.to(DEV)
    _C.rms_norm(dx, eps, weight.to(DEV))
    assert close(dx, from_fixture("y"))
    dx, dres = x.to(DEV), residual.to(DEV)
    _C.add_rms_norm(dx, dres, eps, weight.to(DEV))
    assert close(dx, from_fixture("y_with_residual"))
    if dtype != torch.float32:  # fp32: the reference hands back its output as the residual (aliasing)
        assert torch.equal(dres.cpu(), from_fixture("new_residual"))
    else:
        assert torch.equal(dres.cpu(), x + residual)


def test_rms_norm_module_and_errors():
    norm = RMSNorm(512).to(DEV).to(torch.bfloat16)
    x = torch.randn(3, 40, 512, device=DEV).to(torch.bfloat16)
    r = torch.randn(3, 40, 512, device=DEV).to(torch.bfloat16)
    x0, r0 = x.clone(), r.clone()
    y, new_r = norm(x, r)
    assert y.data_ptr() == x.data_ptr() and new_r.data_ptr() == r.data_ptr()
    want, want_r = moe_oracle.rms_norm_ref(x0.view(-1, 512), norm.weight, 1e-5, r0.view(-1, 512))
    assert torch.equal(new_r.view(-1, 512).cpu(), want_r)
    assert torch.allclose(y.view(-1, 512).cpu().float(), want.float(), atol=2e-2, rtol=2e-2)
    with pytest.raises(RuntimeError, match="multiple of 8"):
        _C.rms_norm(torch.zeros(2, 12, dtype=torch.bfloat16, device=DEV), 1e-5,
                    torch.ones(12, dtype=torch.bfloat16, device=DEV))
