"""Parity of the small CUDA ops (router, alignment, activation, combine, gather) against the CPU
oracle and the committed golden fixtures.  Everything goes through the C-ABI library."""
import numpy as np
import pytest
import torch

from electrock_infer_b200 import _C, _lib
from oracle import moe_oracle

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def run_router(logits, renorm):
    T = logits.shape[0]
    w = torch.full((T, 2), -7.0, dtype=torch.float32, device=DEV)
    ids = torch.full((T, 2), -7, dtype=torch.int32, device=DEV)
    _C.topk_softmax(w, ids, logits.to(DEV).contiguous(), renormalize=renorm)
    torch.cuda.synchronize()
    return w.cpu(), ids.cpu()


# ------------------------------------------------------------------------------------- router
@pytest.mark.parametrize("case", ["normal", "skewed", "wide"])
def test_router_golden(golden, case):
    g = golden["router"]
    logits = torch.from_numpy(g[f"{case}_logits"])
    w, ids = run_router(logits, False)
    assert np.array_equal(ids.numpy(), g[f"{case}_ids"])           # bit-exact
    np.testing.assert_allclose(w.numpy(), g[f"{case}_weights_raw"], rtol=0, atol=1e-6)
    w, ids = run_router(logits, True)
    assert np.array_equal(ids.numpy(), g[f"{case}_ids"])
    np.testing.assert_allclose(w.numpy(), g[f"{case}_weights_renorm"], rtol=0, atol=1e-6)


@pytest.mark.parametrize("T", [1, 2, 3, 127, 128, 129, 511, 512, 513, 4099, 100003])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
def test_router_sizes_and_dtypes(T, dtype):
    g = torch.Generator().manual_seed(T)
    logits = (torch.randn(T, 8, generator=g) * 2).to(dtype)
    w, ids = run_router(logits, True)
    rw, rids = moe_oracle.router_ref(logits.float(), 2, True)
    ties = moe_oracle.tie_rows(logits.float())
    # 16-bit logits do tie; the kernel's rule (lowest index first) is the oracle's rule.
    assert torch.equal(ids, rids), f"{int(ties.sum())} tie rows"
    assert (w - rw).abs().max() <= 1e-6
    assert (w.sum(-1) - 1).abs().max() <= 1e-6


def test_router_ties_choose_lowest_index():
    logits = torch.tensor([[1.0, 1.0, 0, 0, 0, 0, 0, 0], [0, 3.0, 3.0, 3.0, 0, 0, 0, 0],
                           [5.0, 0, 0, 0, 0, 0, 0, 5.0], [0.0] * 8,
                           [0, 0, 0, 2.0, 2.0, 0, 0, 0], [0, 0, 0, 0, 0, 0, 4.0, 4.0],
                           [-1, -1, -1, -1, 9.0, -1, -1, -1]])
    w, ids = run_router(logits, True)
    assert ids.tolist() == [[0, 1], [1, 2], [0, 7], [0, 1], [3, 4], [6, 7], [4, 0]]
    rw, rids = moe_oracle.router_ref(logits, 2, True)
    assert torch.equal(ids, rids) and (w - rw).abs().max() <= 1e-6


def test_router_rejects_other_shapes():
    w = torch.empty(4, 2, device=DEV)
    ids = torch.empty(4, 2, dtype=torch.int32, device=DEV)
    with pytest.raises(RuntimeError, match="num_experts=8"):
        _C.topk_softmax(w, ids, torch.zeros(4, 16, device=DEV))
    with pytest.raises(RuntimeError, match="top_k=2"):
        _C.topk_softmax(torch.empty(4, 3, device=DEV), torch.empty(4, 3, dtype=torch.int32, device=DEV),
                        torch.zeros(4, 8, device=DEV))
    _C.topk_softmax(torch.empty(0, 2, device=DEV), torch.empty(0, 2, dtype=torch.int32, device=DEV),
                    torch.zeros(0, 8, device=DEV))  # empty input is fine


# ---------------------------------------------------------------------------------- alignment
def run_align(ids, bs, E=8, fill=False, prefill=-1, dtype=torch.int32, offsets=True):
    ids_t = torch.as_tensor(np.asarray(ids)).to(dtype).to(DEV)
    cap, nblk = moe_oracle.align_sizes(ids_t.numel(), bs, E)
    sorted_ids = torch.full((cap,), prefill, dtype=torch.int32, device=DEV)
    expert_ids = torch.zeros(nblk, dtype=torch.int32, device=DEV)
    npp = torch.full((1,), -5, dtype=torch.int32, device=DEV)
    off = torch.full((E + 1,), -5, dtype=torch.int32, device=DEV) if offsets else None
    _C.moe_align_block_size(ids_t, E, bs, sorted_ids, expert_ids, npp, expert_offsets=off,
                            fill_pads=fill)
    torch.cuda.synchronize()
    return (sorted_ids.cpu().numpy(), expert_ids.cpu().numpy(), npp.cpu().numpy(),
            off.cpu().numpy() if offsets else None)


def check_align(ids, bs, E=8, **kw):
    s, e, n, off = run_align(ids, bs, E, **kw)
    prefill = kw.get("prefill", -1)
    want_prefill = -1 if kw.get("fill") else prefill
    rs, re_, rn, roff = moe_oracle.align_ref(ids, bs, E, prefill=want_prefill)
    assert int(n[0]) == int(rn[0])
    assert np.array_equal(s, rs), "sorted_token_ids (pads and tail included) differ"
    assert np.array_equal(e, re_)
    if off is not None:
        assert np.array_equal(off, roff)


@pytest.mark.parametrize("bs", [16, 64, 128])
@pytest.mark.parametrize("case", ["uniform_t1000", "skewed_t600", "empty_experts", "single_token",
                                  "exact_blocks", "small_fp32_routing"])
def test_align_golden(golden, case, bs):
    g = golden["align"]
    ids = g[f"{case}_ids"]
    s, e, n, _ = run_align(ids, bs)
    npp = int(g[f"{case}_bs{bs}_npp"][0])
    assert int(n[0]) == npp
    assert np.array_equal(s[:npp], g[f"{case}_bs{bs}_sorted"])     # bit-exact, pads included
    assert np.array_equal(e[: npp // bs], g[f"{case}_bs{bs}_expert_ids"])
    assert (s[npp:] == -1).all()                                    # tail untouched (prefill)


@pytest.mark.parametrize("numel", [0, 1, 2, 127, 128, 129, 4097, 8191, 8192, 8193, 8300, 16384,
                                   16385, 32768, 32769, 65535, 65536, 65537, 70000, 131072, 131073,
                                   200000, 262143, 262144, 262145, 300000, 1000003])
@pytest.mark.parametrize("fill", [False, True])
def test_align_sizes(numel, fill):
    rng = np.random.default_rng(numel + 1)
    ids = rng.integers(0, 8, size=numel, dtype=np.int32)
    check_align(ids, 128 if numel % 2 else 64, fill=fill, prefill=-9)


@pytest.mark.parametrize("dtype", [torch.int64, torch.int16, torch.int8, torch.uint8])
@pytest.mark.parametrize("numel", [1000, 100000, 400000])
def test_align_id_dtypes(dtype, numel):
    rng = np.random.default_rng(3)
    check_align(rng.integers(0, 8, size=numel), 64, dtype=dtype)


def test_align_skew_empty_experts_and_fewer_experts():
    rng = np.random.default_rng(5)
    check_align(rng.choice(8, size=20000, p=[.5, .25, .1, .05, .05, .03, .01, .01]), 128, fill=True)
    check_align(np.full(5000, 6), 128, fill=True)                   # one expert takes everything
    check_align(rng.integers(0, 4, size=3000), 16, E=4)
    check_align(rng.integers(0, 5, size=200000), 32, E=5, fill=True)
    check_align(np.array([7, 0, 7, 0, 3]), 1)                       # block size 1: no padding


def test_align_ignores_out_of_range_experts():
    ids = np.array([0, 9, -1, 3, 3, 8, 1], dtype=np.int32)
    check_align(ids, 4, fill=True)


def test_align_is_a_stable_partition_at_full_size():
    """Size-independent properties at the largest configured token count (2^22 tokens, top-2)."""
    numel = 2 * (1 << 22)
    g = torch.Generator(device=DEV).manual_seed(9)
    ids = torch.randint(0, 8, (numel,), generator=g, device=DEV, dtype=torch.int32)
    bs = 128
    cap, nblk = moe_oracle.align_sizes(numel, bs, 8)
    s = torch.empty(cap, dtype=torch.int32, device=DEV)
    e = torch.zeros(nblk, dtype=torch.int32, device=DEV)
    n = torch.zeros(1, dtype=torch.int32, device=DEV)
    off = torch.zeros(9, dtype=torch.int32, device=DEV)
    _C.moe_align_block_size(ids, 8, bs, s, e, n, expert_offsets=off, fill_pads=True)
    npp = int(n.item())
    cnt = torch.bincount(ids.long(), minlength=8)
    padded = (cnt + bs - 1) // bs * bs
    assert npp == int(padded.sum()) and off.tolist() == [0] + torch.cumsum(padded, 0).tolist()
    live = s[:npp] >= 0
    assert int(live.sum()) == numel and (s[npp:] == -1).all()
    vals = s[:npp][live].long()
    assert torch.equal(torch.sort(vals).values, torch.arange(numel, device=DEV))  # a permutation
    slot_expert = torch.repeat_interleave(torch.arange(8, device=DEV), padded)
    assert torch.equal(ids[vals].long(), slot_expert[live])          # every index in its expert's run
    assert torch.equal(e[: npp // bs].long(), slot_expert[::bs])
    same = slot_expert[live][1:] == slot_expert[live][:-1]
    assert (vals[1:][same] > vals[:-1][same]).all()                  # stable: increasing within a run


# --------------------------------------------------------------------------- activation / combine
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("shape", [(1, 16), (7, 2 * 224), (64, 2 * 7168), (3, 5, 2 * 40), (5, 2 * 13),
                                   (33, 2 * 14336)])
def test_silu_and_mul(dtype, shape):
    g = torch.Generator().manual_seed(shape[-1])
    x = (torch.randn(*shape, generator=g) * 3).to(dtype)
    d = shape[-1] // 2
    out = torch.empty(*shape[:-1], d, dtype=dtype, device=DEV)
    _C.silu_and_mul(out, x.to(DEV))
    want = moe_oracle.silu_and_mul_ref(x)
    got = out.cpu()
    if dtype == torch.float32:
        assert torch.allclose(got, want, rtol=2e-6, atol=1e-7)
    else:
        # Fast exponential on the device: the rounded SiLU may differ by one unit in the last place,
        # which the rounded product can turn into two.
        ulp = 2.0 ** -7 if dtype == torch.bfloat16 else 2.0 ** -10
        assert ((got.float() - want.float()).abs() <= 3 * ulp * want.float().abs() + 1e-6).all()
        assert (got == want).float().mean() > 0.98


def test_silu_and_mul_golden(golden):
    g = golden["ops"]
    x = torch.from_numpy(g["silu_in_bf16_bits"]).view(torch.bfloat16)
    want = torch.from_numpy(g["silu_out_bf16_bits"]).view(torch.bfloat16)
    out = torch.empty(x.shape[0], x.shape[1] // 2, dtype=torch.bfloat16, device=DEV)
    _C.silu_and_mul(out, x.to(DEV))
    # Tolerance of the reference's own test (test/example/test_silu.py: atol = rtol = 1e-3 on bf16
    # values, which it passes because both sides round to bf16).
    assert torch.allclose(out.cpu().float(), want.float(), atol=1e-3, rtol=1e-2)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("T,H", [(1, 8), (5, 4096), (1024, 4096), (33, 1000), (7, 13), (257, 4104)])
def test_moe_sum_bit_exact(dtype, T, H):
    """Both layouts against the oracle's torch expressions, bit for bit.  For the interleaved layout
    (moe_sum_efficient) in bf16 this torch expression is the only yardstick there is: the reference
    instantiates that kernel for fp32 and fp16 only, so its bf16 parity is pinned against torch,
    not against the reference (the other dtypes also meet the reference's kernel in
    test_gpu_ref_ops.py)."""
    g = torch.Generator().manual_seed(T * H)
    x = (torch.randn(T, 2, H, generator=g) * 4).to(dtype)
    x[0, 0, 0], x[0, 1, 0] = -0.0, -0.0
    out = torch.empty(T, H, dtype=dtype, device=DEV)
    _C.moe_sum(x.to(DEV), out)
    want = moe_oracle.moe_sum_ref(x)
    as_int = {torch.bfloat16: torch.int16, torch.float16: torch.int16, torch.float32: torch.int32}[dtype]
    assert torch.equal(out.cpu().view(as_int), want.view(as_int))
    inter = x.permute(0, 2, 1).contiguous()
    out2 = torch.empty(T, H, dtype=dtype, device=DEV)
    _C.moe_sum_efficient(inter.to(DEV), out2)
    want2 = moe_oracle.moe_sum_efficient_ref(inter)
    assert torch.equal(out2.cpu().view(as_int), want2.view(as_int))


def test_moe_sum_golden_and_errors(golden):
    g = golden["ops"]
    x = torch.from_numpy(g["moe_sum_in_f16"])
    out = torch.empty(x.shape[0], x.shape[2], dtype=torch.float16, device=DEV)
    _C.moe_sum(x.to(DEV), out)
    assert torch.equal(out.cpu(), torch.from_numpy(g["moe_sum_out_f16"]))
    with pytest.raises(RuntimeError, match="top_k=2"):
        _C.moe_sum(torch.zeros(4, 3, 8, device=DEV), torch.zeros(4, 8, device=DEV))
    with pytest.raises(RuntimeError, match="top_k=2"):
        _C.moe_sum_efficient(torch.zeros(4, 8, 3, device=DEV), torch.zeros(4, 8, device=DEV))


def test_gather_rows():
    lib = _lib.load()
    T, H, k, bs = 300, 512, 2, 128
    g = torch.Generator().manual_seed(1)
    x = torch.randn(T, H, generator=g).to(torch.bfloat16).to(DEV)
    ids = torch.randint(0, 8, (T * k,), generator=g, dtype=torch.int32)
    s, e, n, _ = moe_oracle.align_ref(ids.numpy(), bs, 8)
    cap = s.size
    sorted_ids = torch.from_numpy(s).to(DEV)
    npp = torch.from_numpy(n).to(DEV)
    dst = torch.full((cap, H), 7.0, dtype=torch.bfloat16, device=DEV)
    rc = lib.b200moe_gather_rows(x.data_ptr(), dst.data_ptr(), sorted_ids.data_ptr(), npp.data_ptr(),
                                 cap, T, H, k, torch.cuda.current_stream().cuda_stream)
    _lib.check(rc, "gather_rows")
    want = torch.full((cap, H), 7.0, dtype=torch.bfloat16)
    used = int(n[0])
    live = torch.from_numpy(s[:used] >= 0)
    rows = torch.from_numpy(s[:used]).long().clamp(min=0) // k
    want[:used] = torch.where(live[:, None], x.cpu()[rows], torch.zeros((), dtype=torch.bfloat16))
    assert torch.equal(dst.cpu().view(torch.int16), want.view(torch.int16))
