"""Parity of the tensor-core grouped GEMMs and of the whole layer against the CPU oracle.

Tolerances (bf16 layer, judged against fp32 arithmetic on the same bf16-valued inputs):
  max-abs error <= 3e-2 and relative Frobenius error <= 1e-2.  The reference's own acceptance bar
  for this layer is allclose(atol=1e-1, rtol=1e-2) (test/example/verify_hf_moe.py:191).
Routing (expert ids, sorted ids, block experts, padded count) is compared bit-exactly.
"""
import numpy as np
import pytest
import torch

from electrock_infer_b200 import _C, _lib
from electrock_infer_b200.layers.moe import FusedMoE, fused_experts, fused_topk, moe_align_block_size
from electrock_infer_b200.layers.moe.fused_moe import BLOCK_SIZE_M
from electrock_infer_b200.synthetic import MoEWorkload, WORKLOADS, make_inputs
from oracle import moe_oracle

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
MAX_ABS, REL_FRO = 3e-2, 1e-2


def gemm_status():
    return _lib.load().b200moe_gemm_device_status(1)


@pytest.fixture(autouse=True)
def _automatic_tiling():
    """Tests that force a tiling of the grouped GEMMs leave the process-wide setting at automatic."""
    yield
    _lib.load().b200moe_gemm_set_tiling(0)


# (block_m, tiling): one 128-row block per tile, two blocks per tile, CTA pairs on 256-row tiles.
TILINGS = [(128, 1), (128, 2), (256, 0)]


def aligned(ids_flat, E, block_m=BLOCK_SIZE_M):
    s, e, n, _ = moe_oracle.align_ref(ids_flat, block_m, E)
    return s, e, n


# ------------------------------------------------------------------------------- grouped GEMMs
@pytest.mark.parametrize("block_m,tiling", TILINGS)
@pytest.mark.parametrize("T,H,I,E", [(100, 256, 128, 8), (300, 512, 1024, 8), (37, 64, 256, 3),
                                     (1000, 1024, 512, 8), (1, 256, 128, 8), (3000, 512, 256, 8),
                                     (2500, 128, 128, 2), (2100, 256, 128, 1), (700, 256, 384, 4)])
def test_grouped_gemm_w13_swiglu(T, H, I, E, block_m, tiling):
    _lib.check(_lib.load().b200moe_gemm_set_tiling(tiling), "set_tiling")
    got, want, used = run_w13(T, H, I, E, block_m)
    st = moe_oracle.error_stats(got[:used], want)
    assert st["rel_fro"] < 4e-3 and st["max_abs"] < 2e-2 * max(st["ref_max_abs"], 1.0), st
    assert (got[used:] == 9.0).all(), "rows beyond num_tokens_post_pad were written"


@pytest.mark.parametrize("tiling", [1, 2])
@pytest.mark.parametrize("T,H,I,E", [(300, 512, 1024, 8), (3000, 512, 256, 8), (700, 256, 384, 4)])
def test_w13_bulk_tensor_stores_and_per_lane_stores_agree_bit_for_bit(T, H, I, E, tiling):
    """The first GEMM's epilogue has two ways out of the SM (bulk tensor stores of 32 x 64 pieces where
    the tile's width is a multiple of 64 columns, 16-byte stores per lane otherwise): same bits."""
    lib = _lib.load()
    _lib.check(lib.b200moe_gemm_set_tiling(tiling), "set_tiling")
    try:
        lib.b200moe_gemm_set_act_stores(0)
        plain, want, used = run_w13(T, H, I, E, 128)
        lib.b200moe_gemm_set_act_stores(1)
        bulk, _, _ = run_w13(T, H, I, E, 128)
    finally:
        lib.b200moe_gemm_set_act_stores(1)
    assert torch.equal(plain, bulk)
    st = moe_oracle.error_stats(bulk[:used], want)
    assert st["rel_fro"] < 4e-3, st


def run_w13(T, H, I, E, block_m):
    lib = _lib.load()
    g = torch.Generator().manual_seed(T + H)
    x = torch.randn(T, H, generator=g).to(torch.bfloat16)
    w13 = (torch.randn(E, 2 * I, H, generator=g) / H ** 0.5).to(torch.bfloat16)
    ids = torch.randint(0, E, (T * 2,), generator=g, dtype=torch.int32)
    s, e, n = aligned(ids.numpy(), E, block_m)
    cap, used = s.size, int(n[0])
    rows = torch.from_numpy(s).long().clamp(min=0) // 2
    a_sorted = x[rows].contiguous()
    a_sorted[torch.from_numpy(s) < 0] = 0
    act = torch.full((cap, I), 9.0, dtype=torch.bfloat16, device=DEV)
    d_a, d_w, d_e, d_n = a_sorted.to(DEV), w13.to(DEV), torch.from_numpy(e).to(DEV), torch.from_numpy(n).to(DEV)
    rc = lib.b200moe_grouped_gemm_w13_swiglu(
        d_a.data_ptr(), d_w.data_ptr(), act.data_ptr(), d_e.data_ptr(), d_n.data_ptr(), cap, E, H, I,
        block_m, torch.cuda.current_stream().cuda_stream)
    _lib.check(rc, "w13")
    torch.cuda.synchronize()
    assert gemm_status() == 0
    got = act.cpu().float()
    slot_expert = torch.from_numpy(np.repeat(e[: used // block_m], block_m)).long()
    want = torch.zeros(used, I)
    for ex in range(E):
        m = slot_expert == ex
        if m.any():
            y = a_sorted[:used][m].float() @ w13[ex].float().T
            want[m] = torch.nn.functional.silu(y[:, :I]) * y[:, I:]
    return got, want, used


@pytest.mark.parametrize("block_m,tiling", TILINGS)
@pytest.mark.parametrize("T,H,I,E", [(100, 256, 128, 8), (300, 512, 1024, 8), (37, 256, 64, 3),
                                     (1000, 1024, 512, 8), (3000, 512, 256, 8), (2500, 256, 128, 2),
                                     (2100, 256, 128, 1)])
def test_grouped_gemm_w2_scale(T, H, I, E, block_m, tiling):
    lib = _lib.load()
    _lib.check(lib.b200moe_gemm_set_tiling(tiling), "set_tiling")
    g = torch.Generator().manual_seed(T + I)
    ids = torch.randint(0, E, (T * 2,), generator=g, dtype=torch.int32)
    s, e, n = aligned(ids.numpy(), E, block_m)
    cap, used = s.size, int(n[0])
    act = torch.randn(cap, I, generator=g).to(torch.bfloat16)
    w2 = (torch.randn(E, H, I, generator=g) / I ** 0.5).to(torch.bfloat16)
    tw = torch.rand(T * 2, generator=g)
    out = torch.full((T * 2, H), 9.0, dtype=torch.bfloat16, device=DEV)
    d_act, d_w, d_tw = act.to(DEV), w2.to(DEV), tw.to(DEV)
    d_s, d_e, d_n = torch.from_numpy(s).to(DEV), torch.from_numpy(e).to(DEV), torch.from_numpy(n).to(DEV)
    rc = lib.b200moe_grouped_gemm_w2_scale(
        d_act.data_ptr(), d_w.data_ptr(), out.data_ptr(), d_tw.data_ptr(), d_s.data_ptr(),
        d_e.data_ptr(), d_n.data_ptr(), cap, T * 2, E, H, I, block_m,
        torch.cuda.current_stream().cuda_stream)
    _lib.check(rc, "w2")
    torch.cuda.synchronize()
    assert gemm_status() == 0
    want = torch.zeros(T * 2, H)
    for slot in range(used):
        p = int(s[slot])
        if p >= 0:
            ex = int(e[slot // block_m])
            want[p] = (act[slot].float() @ w2[ex].float().T) * tw[p]
    st = moe_oracle.error_stats(out.cpu().float(), want)
    assert st["rel_fro"] < 4e-3 and st["max_abs"] < 2e-2 * max(st["ref_max_abs"], 1.0), st


@pytest.mark.parametrize("T,H,I,E,k", [(100, 256, 128, 8, 2), (1000, 1024, 512, 8, 2), (37, 64, 256, 3, 2),
                                       (513, 512, 256, 8, 1)])
def test_grouped_gemm_w13_gather_matches_pregathered_rows(T, H, I, E, k):
    """TMA row gathers inside the GEMM must give bit for bit what a separate gather pass gives."""
    lib = _lib.load()
    g = torch.Generator().manual_seed(T * 7 + H)
    x = torch.randn(T, H, generator=g).to(torch.bfloat16).to(DEV)
    w13 = (torch.randn(E, 2 * I, H, generator=g) / H ** 0.5).to(torch.bfloat16).to(DEV)
    ids = torch.randint(0, E, (T * k,), generator=g, dtype=torch.int32)
    s, e, n = aligned(ids.numpy(), E)
    cap, used = s.size, int(n[0])
    d_s, d_e, d_n = torch.from_numpy(s).to(DEV), torch.from_numpy(e).to(DEV), torch.from_numpy(n).to(DEV)
    stream = torch.cuda.current_stream().cuda_stream
    a_sorted = torch.empty(cap, H, dtype=torch.bfloat16, device=DEV)
    _lib.check(lib.b200moe_gather_rows(x.data_ptr(), a_sorted.data_ptr(), d_s.data_ptr(),
                                       d_n.data_ptr(), cap, T, H, k, stream), "gather_rows")
    act0 = torch.full((cap, I), 9.0, dtype=torch.bfloat16, device=DEV)
    act1 = torch.full((cap, I), 9.0, dtype=torch.bfloat16, device=DEV)
    _lib.check(lib.b200moe_grouped_gemm_w13_swiglu(a_sorted.data_ptr(), w13.data_ptr(), act0.data_ptr(),
                                                   d_e.data_ptr(), d_n.data_ptr(), cap, E, H, I, 128,
                                                   stream), "w13")
    _lib.check(lib.b200moe_grouped_gemm_w13_swiglu_gather(
        x.data_ptr(), T, k, d_s.data_ptr(), w13.data_ptr(), act1.data_ptr(), d_e.data_ptr(),
        d_n.data_ptr(), cap, E, H, I, 128, stream), "w13 gather")
    torch.cuda.synchronize()
    assert gemm_status() == 0
    live = torch.from_numpy(s[:used] >= 0).to(DEV)
    assert torch.equal(act0[:used][live], act1[:used][live])   # padding rows may differ: unused
    assert (act1[used:] == 9.0).all()


def test_peer_table_kernels_on_one_gpu():
    """The expert-parallel kernels address their source rows and output rows through a table of
    per-rank base pointers.  With two local buffers standing in for two ranks, the pull-gather and
    the table-driven epilogue must reproduce the single-buffer kernels bit for bit."""
    lib = _lib.load()
    ranks, T_loc, H, I, E, k = 2, 150, 512, 256, 4, 2
    T = ranks * T_loc
    g = torch.Generator().manual_seed(77)
    x = torch.randn(T, H, generator=g).to(torch.bfloat16).to(DEV)
    w13 = (torch.randn(E, 2 * I, H, generator=g) / H ** 0.5).to(torch.bfloat16).to(DEV)
    w2 = (torch.randn(E, H, I, generator=g) / I ** 0.5).to(torch.bfloat16).to(DEV)
    tw = torch.rand(T * k, generator=g).to(DEV)
    # Global expert ids over 8 experts; this "rank" owns experts 4..7, the others are skipped.
    ids = torch.randint(0, 8, (T * k,), generator=g, dtype=torch.int32) - 4
    s, e, n = aligned(ids.numpy(), E)
    cap = s.size
    d_s, d_e, d_n = torch.from_numpy(s).to(DEV), torch.from_numpy(e).to(DEV), torch.from_numpy(n).to(DEV)
    stream = torch.cuda.current_stream().cuda_stream
    halves = [x[:T_loc].clone(), x[T_loc:].clone()]
    src_table = torch.tensor([h.data_ptr() for h in halves], dtype=torch.int64, device=DEV)
    a0 = torch.empty(cap, H, dtype=torch.bfloat16, device=DEV)
    a1 = torch.empty(cap, H, dtype=torch.bfloat16, device=DEV)
    _lib.check(lib.b200moe_gather_rows(x.data_ptr(), a0.data_ptr(), d_s.data_ptr(), d_n.data_ptr(),
                                       cap, T, H, k, stream), "gather_rows")
    _lib.check(lib.b200moe_gather_rows_peer(src_table.data_ptr(), ranks, T_loc, a1.data_ptr(),
                                            d_s.data_ptr(), d_n.data_ptr(), cap, H, k, stream),
               "gather_rows_peer")
    used = int(n[0])
    assert torch.equal(a0[:used], a1[:used])
    act = torch.empty(cap, I, dtype=torch.bfloat16, device=DEV)
    _lib.check(lib.b200moe_grouped_gemm_w13_swiglu(a1.data_ptr(), w13.data_ptr(), act.data_ptr(),
                                                   d_e.data_ptr(), d_n.data_ptr(), cap, E, H, I, 128,
                                                   stream), "w13")
    out0 = torch.full((T * k, H), 5.0, dtype=torch.bfloat16, device=DEV)
    outs = [torch.full((T_loc * k, H), 5.0, dtype=torch.bfloat16, device=DEV) for _ in range(ranks)]
    out_table = torch.tensor([o.data_ptr() for o in outs], dtype=torch.int64, device=DEV)
    _lib.check(lib.b200moe_grouped_gemm_w2_scale(
        act.data_ptr(), w2.data_ptr(), out0.data_ptr(), tw.data_ptr(), d_s.data_ptr(), d_e.data_ptr(),
        d_n.data_ptr(), cap, T * k, E, H, I, 128, stream), "w2")
    _lib.check(lib.b200moe_grouped_gemm_w2_scale_peer(
        act.data_ptr(), w2.data_ptr(), out_table.data_ptr(), ranks, T_loc * k, tw.data_ptr(),
        d_s.data_ptr(), d_e.data_ptr(), d_n.data_ptr(), cap, E, H, I, 128, stream), "w2 peer")
    torch.cuda.synchronize()
    assert gemm_status() == 0
    assert torch.equal(out0, torch.cat(outs))   # rows of skipped pairs keep the 5.0 fill in both
    assert (out0 == 5.0).all(dim=1).sum().item() == int((ids < 0).sum() + (ids >= E).sum())


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("ranks,T_loc,H", [(2, 33, 256), (3, 7, 64), (8, 40, 512), (1, 5, 128)])
def test_moe_sum_ranks_push(ranks, T_loc, H, dtype):
    """fp32 sum over ranks * 2 rows in slot order, one rounding, the row stored to every rank's output."""
    g = torch.Generator().manual_seed(ranks * 100 + T_loc)
    recv = torch.randn(ranks, T_loc, 2, H, generator=g).to(dtype)
    d_recv = recv.to(DEV)
    row_offset = 3
    outs = [torch.full((row_offset + T_loc + 2, H), 7.0, dtype=dtype, device=DEV) for _ in range(ranks)]
    table = torch.tensor([o.data_ptr() for o in outs], dtype=torch.int64, device=DEV)
    _lib.check(_lib.load().b200moe_moe_sum_ranks_push(
        d_recv.data_ptr(), table.data_ptr(), ranks, row_offset, _C._FLOAT_TAGS[dtype], T_loc, H, 2,
        torch.cuda.current_stream().cuda_stream), "moe_sum_ranks_push")
    torch.cuda.synchronize()
    want = moe_oracle.moe_sum_ranks_ref(recv)
    for o in outs:
        assert torch.equal(o[row_offset:row_offset + T_loc].cpu(), want)
        assert (o[:row_offset] == 7.0).all() and (o[row_offset + T_loc:] == 7.0).all()


def test_tensor_parallel_peer_path_on_one_gpu():
    """The tensor-parallel layer with its all-reduce inside the kernels, both "ranks" played on one
    GPU one after the other: each rank's second GEMM stores the rows of token slice j into slot r
    of receive buffer j, then the combine of slice j adds all slots and stores to every output."""
    lib = _lib.load()
    ranks, T, H, I, E, k = 2, 384, 512, 1024, 8, 2
    T_loc, I_loc = T // ranks, I // ranks
    wl = MoEWorkload("tp1", T, H, I, seed=41, logit_bias=(1, 0, 0, 0, 0, 0, 0, -1))
    inp = make_inputs(wl)
    x = inp["x"].to(DEV)
    tw, ids = fused_topk(x, inp["logits"].to(DEV), k, True)
    s, e, n = aligned(ids.cpu().numpy().reshape(-1), E)
    cap = s.size
    d_s, d_e, d_n = torch.from_numpy(s).to(DEV), torch.from_numpy(e).to(DEV), torch.from_numpy(n).to(DEV)
    stream = torch.cuda.current_stream().cuda_stream
    a = torch.zeros(cap, H, dtype=torch.bfloat16, device=DEV)
    _lib.check(lib.b200moe_gather_rows(x.data_ptr(), a.data_ptr(), d_s.data_ptr(), d_n.data_ptr(), cap,
                                       T, H, k, stream), "gather_rows")
    slot = T_loc * k * H
    recv = [torch.full((ranks * slot,), 3.0, dtype=torch.bfloat16, device=DEV) for _ in range(ranks)]
    local = []
    keep = []
    for r in range(ranks):
        w1 = inp["w13"][:, r * I_loc:(r + 1) * I_loc]
        w3 = inp["w13"][:, I + r * I_loc:I + (r + 1) * I_loc]
        w13_r = torch.cat([w1, w3], dim=1).contiguous().to(DEV)
        w2_r = inp["w2"][:, :, r * I_loc:(r + 1) * I_loc].contiguous().to(DEV)
        act = torch.empty(cap, I_loc, dtype=torch.bfloat16, device=DEV)
        _lib.check(lib.b200moe_grouped_gemm_w13_swiglu(a.data_ptr(), w13_r.data_ptr(), act.data_ptr(),
                                                       d_e.data_ptr(), d_n.data_ptr(), cap, E, H, I_loc,
                                                       128, stream), "w13")
        out_r = torch.empty(T * k, H, dtype=torch.bfloat16, device=DEV)
        _lib.check(lib.b200moe_grouped_gemm_w2_scale(
            act.data_ptr(), w2_r.data_ptr(), out_r.data_ptr(), tw.data_ptr(), d_s.data_ptr(),
            d_e.data_ptr(), d_n.data_ptr(), cap, T * k, E, H, I_loc, 128, stream), "w2")
        push = torch.tensor([b.data_ptr() + r * slot * 2 for b in recv], dtype=torch.int64, device=DEV)
        _lib.check(lib.b200moe_grouped_gemm_w2_scale_peer(
            act.data_ptr(), w2_r.data_ptr(), push.data_ptr(), ranks, T_loc * k, tw.data_ptr(),
            d_s.data_ptr(), d_e.data_ptr(), d_n.data_ptr(), cap, E, H, I_loc, 128, stream), "w2 peer")
        local.append(out_r)
        keep += [w13_r, w2_r, act, push]
    outs = [torch.empty(T, H, dtype=torch.bfloat16, device=DEV) for _ in range(ranks)]
    table = torch.tensor([o.data_ptr() for o in outs], dtype=torch.int64, device=DEV)
    for j in range(ranks):
        _lib.check(lib.b200moe_moe_sum_ranks_push(recv[j].data_ptr(), table.data_ptr(), ranks, j * T_loc,
                                                  _lib.BF16, T_loc, H, k, stream), "moe_sum_ranks_push")
    torch.cuda.synchronize()
    assert gemm_status() == 0
    assert torch.equal(outs[0], outs[1])
    # Bit-exact against the restated combine over the ranks' locally computed rows ...
    stacked = torch.stack([o.view(T, k, H) for o in local]).cpu()
    assert torch.equal(outs[0].cpu(), moe_oracle.moe_sum_ranks_ref(stacked))
    # ... and within the layer tolerance of the fp32 block.
    want = moe_oracle.moe_block_ref(inp["x"], inp["w13"], inp["w2"], inp["logits"])
    st = moe_oracle.error_stats(outs[0].cpu().float(), want)
    assert st["max_abs"] <= MAX_ABS and st["rel_fro"] <= REL_FRO, st


# --------------------------------------------------------------------------------- whole layer
def run_layer(inp, wl, inplace=True):
    x = inp["x"].to(torch.bfloat16).to(DEV).clone()
    out = fused_experts(x, inp["w13"].to(torch.bfloat16).to(DEV), inp["w2"].to(torch.bfloat16).to(DEV),
                        inp["logits"].to(DEV), wl.top_k, renormalize=True, inplace=inplace)
    torch.cuda.synchronize()
    assert gemm_status() == 0
    return x, out


def check_layer(inp, wl, tokens=None):
    x, out = run_layer(inp, wl)
    assert out.data_ptr() == x.data_ptr(), "inplace result must alias hidden_states"
    sel = slice(None) if tokens is None else tokens
    bf = {k: inp[k].to(torch.bfloat16) for k in ("x", "w13", "w2")}
    want = moe_oracle.moe_block_ref(bf["x"][sel], bf["w13"], bf["w2"], inp["logits"][sel])
    st = moe_oracle.error_stats(out.cpu().float()[sel], want)
    assert st["max_abs"] <= MAX_ABS and st["rel_fro"] <= REL_FRO, st
    return st


def test_layer_tiny_bf16_against_reference_block(golden):
    wl = MoEWorkload("tiny_bf16", 96, 256, 512, seed=7)
    inp = make_inputs(wl)
    x, out = run_layer(inp, wl)
    want = torch.from_numpy(golden["layer"]["tiny_bf16_hf_block_out_fp32"])
    st = moe_oracle.error_stats(out.cpu().float(), want)
    assert st["max_abs"] <= MAX_ABS and st["rel_fro"] <= REL_FRO, st


def test_layer_small_config_in_bf16(golden):
    """The fp32 CPU configuration (T=64, H=512, I=1024) pushed through the bf16 GPU path: compared
    with fp32 arithmetic on the bf16-rounded tensors, and loosely with the fp32 fixture."""
    wl = WORKLOADS["small_fp32"]
    inp = make_inputs(wl)
    st = check_layer(inp, wl)
    x, out = run_layer(inp, wl)
    want32 = torch.from_numpy(golden["layer"]["small_fp32_hf_block_out"])
    agree = moe_oracle.router_ref(inp["logits"])[1] == moe_oracle.router_ref(
        inp["x"].to(torch.bfloat16).float() @ inp["router_w"].to(torch.bfloat16).float().T)[1]
    assert agree.all()  # logits are the fp32 ones in both runs, so routing is identical
    st32 = moe_oracle.error_stats(out.cpu().float(), want32)
    assert st32["rel_fro"] < 2e-2, st32  # inputs rounded to bf16: ~2^-9 relative per operand


@pytest.mark.parametrize("x_dtype,w_dtype", [(torch.float32, torch.float32),
                                             (torch.float16, torch.bfloat16),
                                             (torch.float32, torch.bfloat16)])
def test_layer_accepts_fp32_and_fp16_tensors(golden, x_dtype, w_dtype):
    """The fp32 CPU configuration (T=64, H=512, I=1024) handed over in its own dtype: like the
    reference, the layer computes in bf16 whatever it is given and returns the caller's dtype, in
    place.  Compared with the reference block's fp32 output (inputs rounded to bf16: about 2^-9
    relative per operand) and with the bf16 call bit for bit."""
    wl = WORKLOADS["small_fp32"]
    inp = make_inputs(wl)
    x = inp["x"].to(x_dtype).to(DEV)
    w13, w2 = inp["w13"].to(w_dtype).to(DEV), inp["w2"].to(w_dtype).to(DEV)
    out = fused_experts(x, w13, w2, inp["logits"].to(DEV), 2, renormalize=True, inplace=True)
    torch.cuda.synchronize()
    assert out.data_ptr() == x.data_ptr() and out.dtype == x_dtype and gemm_status() == 0
    want32 = torch.from_numpy(golden["layer"]["small_fp32_hf_block_out"])
    st = moe_oracle.error_stats(out.cpu().float(), want32)
    assert st["rel_fro"] < 2e-2, st
    xb = inp["x"].to(x_dtype).to(torch.bfloat16).to(DEV)
    ref = fused_experts(xb, w13.to(torch.bfloat16), w2.to(torch.bfloat16), inp["logits"].to(DEV), 2,
                        renormalize=True, inplace=False)
    assert torch.equal(out.cpu(), ref.to(x_dtype).cpu())
    # Not in place: a new tensor of the caller's dtype, the input untouched.
    x2 = inp["x"].to(x_dtype).to(DEV)
    keep = x2.clone()
    out2 = fused_experts(x2, w13, w2, inp["logits"].to(DEV), 2, renormalize=True, inplace=False)
    assert out2.dtype == x_dtype and torch.equal(x2, keep) and torch.equal(out2, out)


@pytest.mark.parametrize("T", [1, 2, 7, 8, 9, 130, 1000])
def test_layer_token_counts(T):
    wl = MoEWorkload("t", T, 512, 256, seed=T)
    check_layer(make_inputs(wl), wl)


@pytest.mark.parametrize("T", [5, 700, 4096, 20000])
def test_layer_block_sizes_agree_bit_for_bit(T):
    """One block per tile, two blocks per tile and the two-CTA (256-row) tiling run the same
    arithmetic per row.  T=20000 gives every expert many M blocks, an odd count for some, and a
    last round of tiles short enough to be dealt as one-block halves."""
    from electrock_infer_b200.layers.moe import fused_moe as fm
    wl = MoEWorkload("t", T, 512, 512, seed=100 + T, logit_bias=(1, 0, 0, 0, 0, 0, -1, -3))
    inp = make_inputs(wl)
    outs = []
    try:
        for bm, tiling in TILINGS:
            fm.FORCE_BLOCK_M = bm
            _lib.check(_lib.load().b200moe_gemm_set_tiling(tiling), "set_tiling")
            outs.append(run_layer(inp, wl)[1].clone())
    finally:
        fm.FORCE_BLOCK_M = None
    assert torch.equal(outs[0], outs[1])
    assert torch.equal(outs[0], outs[2])
    assert fm.choose_block_m(8192, 2, 8) == 128
    check_layer(inp, wl)


@pytest.mark.parametrize("T,logit_dtype", [(3, torch.float32), (700, torch.bfloat16), (40000, torch.float32)])
def test_one_call_entry_point_matches_the_step_by_step_path(T, logit_dtype):
    """``b200moe_fused_experts`` (the layer in one C-ABI call, what ``fused_experts`` uses by default)
    against the same six steps issued one by one from Python (the path taken while per-kernel
    timing is on): same bits.  T=40000 gives more pair indices than one alignment launch takes."""
    from electrock_infer_b200.layers.moe import fused_moe as fm
    wl = MoEWorkload("t", T, 256, 128, seed=7 + T, logit_bias=(1, 0, 0, 0, 0, 0, -1, -3))
    inp = make_inputs(wl)
    dev_in = [inp[k].to(torch.bfloat16).to(DEV) for k in ("x", "w13", "w2")]
    logits = inp["logits"].to(logit_dtype).to(DEV)
    before = _lib.launch_count()
    one_call = fused_experts(dev_in[0].clone(), dev_in[1], dev_in[2], logits, 2, inplace=True)
    launched = _lib.launch_count() - before  # 6 steps; 3 launches for long alignments; launch pairs of the GEMMs
    assert (8 if 2 * T > _C.align_single_pass_max() else 6) <= launched <= (10 if 2 * T > _C.align_single_pass_max() else 8)
    fm.enable_kernel_timing(True)
    try:
        stepwise = fused_experts(dev_in[0].clone(), dev_in[1], dev_in[2], logits, 2, inplace=True)
        assert set(fm.collect_kernel_timings()) >= {"topk_softmax", "grouped_gemm_w13_swiglu", "moe_sum"}
    finally:
        fm.enable_kernel_timing(False)
    torch.cuda.synchronize()
    assert gemm_status() == 0 and torch.equal(one_call, stepwise)
    want = moe_oracle.moe_block_ref(inp["x"].to(torch.bfloat16)[:512], inp["w13"].to(torch.bfloat16),
                                    inp["w2"].to(torch.bfloat16), logits[:512].float().cpu())
    st = moe_oracle.error_stats(one_call[:512].cpu().float(), want)
    assert st["max_abs"] <= MAX_ABS and st["rel_fro"] <= REL_FRO, st


def test_scratch_is_sized_by_capacity_bucket_and_reused():
    """A serving loop changes its batch size every step: after the largest batch has been seen (or
    reserved), smaller batches must run in a prefix of the same scratch without allocating, and
    give the results they give on their own."""
    from electrock_infer_b200.layers.moe import fused_moe as fm
    H, I = 768, 384   # a shape no other test uses, so the scratch entry is this test's own
    wl = MoEWorkload("bucket", 1000, H, I, seed=77, logit_bias=(1, 0, 0, 0, 0, 0, -1, -3))
    inp = make_inputs(wl)
    w13, w2 = inp["w13"].to(torch.bfloat16).to(DEV), inp["w2"].to(torch.bfloat16).to(DEV)
    x_all, logits_all = inp["x"].to(torch.bfloat16).to(DEV), inp["logits"].to(DEV)
    assert fm.capacity_bucket(700) == fm.capacity_bucket(1000) == 1024
    fm.reserve_workspace(DEV, 700, 2, 8, H, I)          # sizes the bucket of 1024 tokens
    want = moe_oracle.moe_block_ref(inp["x"].to(torch.bfloat16), inp["w13"].to(torch.bfloat16),
                                    inp["w2"].to(torch.bfloat16), inp["logits"])
    torch.cuda.synchronize()
    for T in (700, 300, 1000, 1, 513, 1024 - 24):
        x, lg = x_all[:T].clone(), logits_all[:T].contiguous()
        before = torch.cuda.memory_allocated()
        out = fused_experts(x, w13, w2, lg, 2, inplace=True)
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == before, f"T={T} allocated scratch"
        st = moe_oracle.error_stats(out.cpu().float(), want[:T])
        assert st["max_abs"] <= MAX_ABS and st["rel_fro"] <= REL_FRO, (T, st)
        del x, out   # the next step's measurement must not see this step's tensors being freed
    assert gemm_status() == 0
    # A batch beyond the bucket grows the scratch once; the next batches reuse the larger one.
    wl2 = MoEWorkload("bucket2", 1500, H, I, seed=78)
    inp2 = make_inputs(wl2)
    x2 = inp2["x"].to(torch.bfloat16).to(DEV)
    logits2 = inp2["logits"].to(DEV)
    grown = fused_experts(x2.clone(), w13, w2, logits2, 2, inplace=True)
    torch.cuda.synchronize()
    del grown
    x, lg = x_all[:900].clone(), logits_all[:900].contiguous()
    before = torch.cuda.memory_allocated()
    out = fused_experts(x, w13, w2, lg, 2, inplace=True)
    torch.cuda.synchronize()
    assert torch.cuda.memory_allocated() == before


def test_layer_skewed_and_empty_experts():
    wl = MoEWorkload("skew", 700, 256, 512, seed=3, logit_bias=(6, 5, 0, 0, -20, -20, -20, -20))
    inp = make_inputs(wl)
    ids = moe_oracle.router_ref(inp["logits"])[1]
    assert len(set(ids.reshape(-1).tolist())) <= 4  # several experts receive nothing
    check_layer(inp, wl)


def test_layer_routing_is_bit_exact():
    wl = WORKLOADS["mixtral_prefill_t8192_skew"]
    g = torch.Generator().manual_seed(wl.seed)
    logits = torch.randn(wl.num_tokens, 8, generator=g) + torch.tensor(wl.logit_bias)
    assert not moe_oracle.tie_rows(logits).any()
    w, ids = fused_topk(torch.empty(wl.num_tokens, 1, device=DEV), logits.to(DEV), 2, True)
    rw, rids = moe_oracle.router_ref(logits, 2, True)
    assert torch.equal(ids.cpu(), rids) and (w.cpu() - rw).abs().max() <= 1e-6
    load = torch.bincount(rids.reshape(-1).long(), minlength=8)
    assert load.max() >= 3 * load.min()  # the skewed workload really is skewed
    for bs in (16, 64, 128):
        s, e, n = moe_align_block_size(ids, bs, 8)
        rs, re_, rn, _ = moe_oracle.align_ref(rids.numpy(), bs, 8)
        assert int(n.item()) == int(rn[0])
        assert np.array_equal(s.cpu().numpy(), rs) and np.array_equal(e.cpu().numpy(), re_)


def test_layer_not_inplace_and_bf16_logits():
    wl = MoEWorkload("t", 257, 512, 512, seed=21)
    inp = make_inputs(wl)
    x, out = run_layer(inp, wl, inplace=False)
    assert out.data_ptr() != x.data_ptr() and torch.equal(x.cpu(), inp["x"])
    # bf16 logits, as the model's gate produces them: the router reads them directly.
    lb = inp["logits"].to(torch.bfloat16)
    out2 = fused_experts(x.clone(), inp["w13"].to(DEV), inp["w2"].to(DEV), lb.to(DEV), 2)
    want = moe_oracle.moe_block_ref(inp["x"], inp["w13"], inp["w2"], lb.float())
    st = moe_oracle.error_stats(out2.cpu().float(), want)
    assert st["max_abs"] <= MAX_ABS and st["rel_fro"] <= REL_FRO, st


def test_fused_moe_module_forward():
    wl = MoEWorkload("t", 200, 512, 1024, seed=33)
    inp = make_inputs(wl)
    layer = FusedMoE(8, 2, wl.hidden, wl.inter, tp_size=1, params_dtype=torch.bfloat16,
                     reduce_results=True).to(DEV)
    for e in range(8):
        layer.weight_loader(layer.w13_weight, inp["w13"][e, : wl.inter].to(DEV), "w1", e)
        layer.weight_loader(layer.w13_weight, inp["w13"][e, wl.inter:].to(DEV), "w3", e)
        layer.weight_loader(layer.w2_weight, inp["w2"][e].to(DEV), "w2", e)
    x = inp["x"].to(DEV).clone()
    with torch.inference_mode():
        out = layer(x, inp["logits"].to(DEV))
    assert out.data_ptr() == x.data_ptr()
    want = moe_oracle.moe_block_ref(inp["x"], inp["w13"], inp["w2"], inp["logits"])
    st = moe_oracle.error_stats(out.cpu().float(), want)
    assert st["max_abs"] <= MAX_ABS and st["rel_fro"] <= REL_FRO, st


@pytest.mark.parametrize("tp,T", [(2, 1024), (4, 300), (8, 4096), (8, 64)])
def test_layer_tensor_parallel_shard_shapes(tp, T):
    """One rank's share of the tensor-parallel layer (intermediate size 14336 / tp, hidden 4096) on
    a single GPU: the partial output must match the oracle's block evaluated on the same shard."""
    inter = 14336 // tp
    wl = MoEWorkload("shard", T, 4096, inter, seed=50 + tp)
    inp = make_inputs(wl)
    x, out = run_layer(inp, wl)
    sample = torch.randperm(T, generator=torch.Generator().manual_seed(1))[:64]
    want = moe_oracle.moe_block_ref(inp["x"][sample], inp["w13"], inp["w2"], inp["logits"][sample])
    st = moe_oracle.error_stats(out.cpu().float()[sample], want)
    assert st["max_abs"] <= MAX_ABS and st["rel_fro"] <= REL_FRO, st


def test_layer_replays_from_a_cuda_graph():
    """A warmed-up layer call allocates nothing and never synchronises, so it can be captured into
    a CUDA graph and replayed on new inputs written into the captured buffers."""
    wl = MoEWorkload("graph", 256, 512, 1024, seed=61)
    inp = make_inputs(wl)
    w13, w2 = inp["w13"].to(DEV), inp["w2"].to(DEV)
    x = inp["x"].to(DEV).clone()
    logits = inp["logits"].to(DEV).clone()
    stream = torch.cuda.Stream()
    stream.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(stream):
        for _ in range(2):  # warm-up on the capture stream: workspace allocation, attribute set-up
            fused_experts(x, w13, w2, logits, 2, inplace=True)
    torch.cuda.current_stream().wait_stream(stream)
    graph = torch.cuda.CUDAGraph()
    x.copy_(inp["x"])
    with torch.cuda.graph(graph, stream=stream):
        fused_experts(x, w13, w2, logits, 2, inplace=True)
    for seed in (62, 63):
        other = make_inputs(MoEWorkload("graph", 256, 512, 1024, seed=seed))
        x.copy_(other["x"])
        logits.copy_(other["logits"])
        graph.replay()
        torch.cuda.synchronize()
        assert gemm_status() == 0
        want = moe_oracle.moe_block_ref(other["x"], inp["w13"], inp["w2"], other["logits"])
        st = moe_oracle.error_stats(x.cpu().float(), want)
        assert st["max_abs"] <= MAX_ABS and st["rel_fro"] <= REL_FRO, st


@pytest.mark.parametrize("name", ["mid", "mixtral_decode_t256"])
def test_layer_error_is_within_the_reference_pipelines_own(name):
    """Error against fp32 arithmetic, side by side: this library, and the reference pipeline with
    every rounding point it has (GEMM1 -> bf16, SiLU -> bf16, product -> bf16, GEMM2 x weight ->
    bf16, sum -> bf16; restated in ``moe_oracle.fused_experts_ref`` and pinned by the reference's
    own interpreted run).  The fused epilogue rounds once where the reference rounds three times, so
    this library must not be further from fp32 than 1.5 times the reference's own distance."""
    wl = WORKLOADS[name] if name in WORKLOADS else MoEWorkload("mid", 300, 512, 1024, seed=31)
    inp = make_inputs(wl)
    x, out = run_layer(inp, wl)
    exact = moe_oracle.moe_block_ref(inp["x"], inp["w13"], inp["w2"], inp["logits"])
    ref_pipeline = moe_oracle.fused_experts_ref(inp["x"], inp["w13"], inp["w2"], inp["logits"])
    ours = moe_oracle.error_stats(out.cpu().float(), exact)
    theirs = moe_oracle.error_stats(ref_pipeline.float(), exact)
    print(name, "ours", ours, "reference pipeline", theirs)
    assert ours["rel_fro"] <= 1.5 * theirs["rel_fro"], (ours, theirs)
    assert ours["max_abs"] <= MAX_ABS and ours["rel_fro"] <= REL_FRO


def test_layer_mixtral_decode_shape():
    """Mixtral-8x7B shape, T=256 (the decode-sized configuration), full comparison."""
    wl = WORKLOADS["mixtral_decode_t256"]
    inp = make_inputs(wl)
    st = check_layer(inp, wl)
    print("mixtral_decode_t256", st)


def test_layer_mixtral_prefill_shape_sampled():
    """Mixtral-8x7B shape, T=8192 with skewed routing.  Every output row depends only on its own
    token, so the oracle is evaluated on a fixed sample of 192 tokens of the full-size run; the
    remaining rows are covered by a checksum property: running the layer on the first half of the
    tokens alone must reproduce the first half of the full result bit for bit."""
    wl = WORKLOADS["mixtral_prefill_t8192_skew"]
    inp = make_inputs(wl)
    sample = torch.randperm(wl.num_tokens, generator=torch.Generator().manual_seed(0))[:192]
    x, out = run_layer(inp, wl)
    full = out.clone()
    want = moe_oracle.moe_block_ref(inp["x"][sample], inp["w13"], inp["w2"], inp["logits"][sample])
    st = moe_oracle.error_stats(full.cpu().float()[sample], want)
    assert st["max_abs"] <= MAX_ABS and st["rel_fro"] <= REL_FRO, st
    print("mixtral_prefill_t8192_skew (192-token sample)", st)
    half = wl.num_tokens // 2
    xh = inp["x"][:half].to(DEV).clone()
    outh = fused_experts(xh, inp["w13"].to(DEV), inp["w2"].to(DEV), inp["logits"][:half].to(DEV), 2,
                         inplace=True)
    assert torch.equal(outh, full[:half])


def test_expert_parallel_peer_path_with_one_rank_and_ragged_batches():
    """The peer-memory exchange of ExpertParallelMoE in a process group of one rank: the same
    kernels and buffers as on several GPUs (the peer tables just hold one entry).  With a bound on
    the tokens per rank, batches shorter than the bound (and an empty one) are padded with pair
    indices the alignment skips; results must equal the plain layer bit for bit."""
    import socket

    import torch.distributed as dist

    from electrock_infer_b200.parallel import ExpertParallelMoE
    if dist.is_initialized():
        pytest.skip("a process group is already initialised in this process")
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    dev = torch.device(DEV)
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", init_method=f"tcp://127.0.0.1:{port}", rank=0, world_size=1,
                            device_id=dev)
    try:
        wl = MoEWorkload("ep1", 400, 512, 1024, seed=77, logit_bias=(1, 1, 0, 0, 0, 0, -1, -1))
        inp = make_inputs(wl)
        w13, w2 = inp["w13"].to(dev), inp["w2"].to(dev)
        single = fused_experts(inp["x"].to(dev), w13, w2, inp["logits"].to(dev), 2, inplace=False)
        layer = ExpertParallelMoE(8, 2, wl.hidden, wl.inter, params_dtype=torch.bfloat16,
                                  exchange="peer", max_tokens_per_rank=400).to(dev)
        layer.w13_weight.data.copy_(w13)
        layer.w2_weight.data.copy_(w2)
        for lo, hi in ((0, 400), (13, 350), (0, 0), (363, 400)):
            x = inp["x"][lo:hi].to(dev).clone()
            out = layer(x, inp["logits"][lo:hi].to(dev))
            torch.cuda.synchronize()
            assert out.data_ptr() == x.data_ptr() and out.shape[0] == hi - lo
            assert torch.equal(out, single[lo:hi]), (lo, hi)
        with pytest.raises(RuntimeError, match="max_tokens_per_rank"):
            layer(torch.zeros(401, wl.hidden, dtype=torch.bfloat16, device=dev),
                  torch.zeros(401, 8, device=dev))
        assert gemm_status() == 0
        layer.close()
    finally:
        dist.destroy_process_group()
