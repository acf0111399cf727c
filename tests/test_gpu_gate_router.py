"""The gate projection fused into the router (gate GEMM + softmax + top-2 in one kernel) and the
MixtralMoE block built on it, against the oracle."""
import pytest
import torch

from electrock_infer_b200 import _C
from electrock_infer_b200.layers.moe import MixtralMoE
from electrock_infer_b200.synthetic import MoEWorkload, make_inputs
from oracle import moe_oracle

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def run(x, w, renorm, rounded):
    T = x.shape[0]
    tw = torch.full((T, 2), -7.0, device=DEV)
    ids = torch.full((T, 2), -7, dtype=torch.int32, device=DEV)
    logits = torch.full((T, 8), -7.0, device=DEV)
    _C.gate_topk_softmax(tw, ids, x.to(DEV), w.to(DEV), renormalize=renorm, logits_out=logits,
                         round_logits_bf16=rounded)
    torch.cuda.synchronize()
    return tw.cpu(), ids.cpu(), logits.cpu()


@pytest.mark.parametrize("T", [1, 3, 4, 5, 257, 4099])
@pytest.mark.parametrize("H", [256, 4096])
@pytest.mark.parametrize("rounded", [False, True])
def test_gate_router(T, H, rounded):
    g = torch.Generator().manual_seed(T * 3 + H)
    x = torch.randn(T, H, generator=g).to(torch.bfloat16)
    w = (torch.randn(8, H, generator=g) * 0.02).to(torch.bfloat16)
    tw, ids, logits = run(x, w, True, rounded)
    exact = moe_oracle.gate_logits_ref(x, w, round_bf16=False)
    if rounded:
        # bf16-valued, and within one bf16 step of the rounded exact logits
        assert torch.equal(logits, logits.to(torch.bfloat16).float())
        assert ((logits - exact).abs() <= 2.0 ** -8 * exact.abs() + 1e-6).all()
    else:
        assert (logits - exact).abs().max() <= 2e-5 * max(1.0, float(exact.abs().max()))
    # The routing decision is exactly the router's decision on the logits the kernel reports.
    rw, rids = moe_oracle.router_ref(logits, 2, True)
    assert torch.equal(ids, rids)
    assert (tw - rw).abs().max() <= 1e-6
    # Against exact-arithmetic logits the chosen experts can only differ where the logits nearly tie.
    _, eids = moe_oracle.router_ref(moe_oracle.gate_logits_ref(x, w, round_bf16=rounded), 2, True)
    differ = (ids != eids).any(dim=1)
    if differ.any():
        top3 = torch.sort(exact[differ], dim=1, descending=True).values[:, :3]
        gap = torch.minimum(top3[:, 0] - top3[:, 1], top3[:, 1] - top3[:, 2])
        assert (gap <= (2.0 ** -7 if rounded else 1e-4) * top3.abs().max()).all()
        assert differ.float().mean() < 0.02


def test_gate_router_without_renormalisation_and_errors():
    g = torch.Generator().manual_seed(5)
    x = torch.randn(100, 512, generator=g).to(torch.bfloat16)
    w = (torch.randn(8, 512, generator=g) * 0.05).to(torch.bfloat16)
    tw, ids, logits = run(x, w, False, False)
    rw, rids = moe_oracle.router_ref(logits, 2, False)
    assert torch.equal(ids, rids) and (tw - rw).abs().max() <= 1e-6
    out_w = torch.empty(4, 2, device=DEV)
    out_i = torch.empty(4, 2, dtype=torch.int32, device=DEV)
    with pytest.raises(RuntimeError, match="multiple of 256"):
        _C.gate_topk_softmax(out_w, out_i, torch.zeros(4, 200, dtype=torch.bfloat16, device=DEV),
                             torch.zeros(8, 200, dtype=torch.bfloat16, device=DEV))
    with pytest.raises(RuntimeError, match="num_experts=8"):
        _C.gate_topk_softmax(out_w, out_i, torch.zeros(4, 256, dtype=torch.bfloat16, device=DEV),
                             torch.zeros(4, 256, dtype=torch.bfloat16, device=DEV))


@pytest.mark.parametrize("fuse_gate", [True, False])
def test_mixtral_moe_block(fuse_gate):
    wl = MoEWorkload("blk", 300, 512, 1024, seed=41)
    inp = make_inputs(wl)
    block = MixtralMoE(8, 2, wl.hidden, wl.inter, params_dtype=torch.bfloat16, tp_size=1,
                       fuse_gate=fuse_gate).to(DEV)
    block.gate.weight.weight_loader(block.gate.weight, inp["router_w"].to(DEV))
    for e in range(8):
        block.experts.weight_loader(block.experts.w13_weight, inp["w13"][e, : wl.inter].to(DEV), "w1", e)
        block.experts.weight_loader(block.experts.w13_weight, inp["w13"][e, wl.inter:].to(DEV), "w3", e)
        block.experts.weight_loader(block.experts.w2_weight, inp["w2"][e].to(DEV), "w2", e)
    x = inp["x"].to(DEV).clone().view(3, 100, wl.hidden)   # the block accepts any leading shape
    with torch.inference_mode():
        out = block(x)
    assert out.shape == x.shape and out.data_ptr() == x.data_ptr()
    # The reference routes on bf16 logits; a token whose 2nd and 3rd logits round to neighbouring
    # bf16 values may pick another expert, so compare through the logits the device used.
    logits = moe_oracle.gate_logits_ref(inp["x"], inp["router_w"], round_bf16=True)
    want = moe_oracle.moe_block_ref(inp["x"], inp["w13"], inp["w2"], logits)
    got = out.view(-1, wl.hidden).cpu().float()
    row_err = (got - want).abs().max(dim=1).values
    assert (row_err <= 3e-2).float().mean() >= 0.99   # at most a few near-tie rows routed differently
    st = moe_oracle.error_stats(got[row_err <= 3e-2], want[row_err <= 3e-2])
    assert st["rel_fro"] <= 1e-2, st
