"""Host-side checks that need no GPU: the library loads, exports what the header declares, rejects
bad arguments with the documented status codes, and the Python mirror of the reference interface
behaves like the reference's (constructor, weight loader, error types)."""
import ctypes
import re
from pathlib import Path

import pytest
import torch

import electrock_infer_b200 as pkg
from electrock_infer_b200 import _C, _lib
from electrock_infer_b200.layers.moe import FusedMoE, fused_experts
from electrock_infer_b200.synthetic import MoEWorkload, WORKLOADS, make_inputs

HEADER = Path(__file__).resolve().parent.parent / "include" / "b200moe.h"


def declared_symbols():
    text = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)
    return sorted(set(re.findall(r"\b(b200moe_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    lib = _lib.load()
    names = declared_symbols()
    assert len(names) >= 12
    for name in names:
        assert hasattr(lib, name), f"{name} is declared in b200moe.h but not exported"
    assert sorted(_lib.SIGNATURES) == names, "ctypes signatures and header are out of sync"
    assert lib.b200moe_abi_version() == 1


def test_argument_validation_without_a_device():
    lib = _lib.load()
    ptr = ctypes.c_void_p(256)  # never dereferenced: validation fails first
    assert lib.b200moe_topk_softmax(ptr, ptr, ptr, _lib.F32, 4, 7, 2, 0, None) == -1
    assert b"num_experts=8" in lib.b200moe_last_error()
    assert lib.b200moe_topk_softmax(ptr, ptr, ptr, _lib.F32, 4, 8, 3, 0, None) == -1
    assert lib.b200moe_topk_softmax(ptr, ptr, ptr, 9, 4, 8, 2, 0, None) == -2
    assert lib.b200moe_topk_softmax(None, ptr, ptr, _lib.F32, 4, 8, 2, 0, None) == -3
    assert lib.b200moe_topk_softmax(ptr, ptr, ctypes.c_void_p(260), _lib.F32, 4, 8, 2, 0, None) == -5
    assert lib.b200moe_topk_softmax(ptr, ptr, ptr, _lib.F32, 0, 8, 2, 0, None) == 0
    assert lib.b200moe_moe_sum(ptr, ptr, _lib.BF16, 4, 64, 3, 0, None) == -1
    assert b"top_k=2" in lib.b200moe_last_error()
    assert lib.b200moe_moe_sum(ptr, ptr, 7, 4, 64, 2, 0, None) == -2
    assert lib.b200moe_moe_sum(ptr, ptr, _lib.BF16, 0, 64, 2, 0, None) == 0
    assert lib.b200moe_silu_and_mul(None, ptr, _lib.BF16, 4, 64, None) == -3
    # sorted_token_ids too small for numel + E * (block - 1)
    assert lib.b200moe_align_block_size(ptr, _lib.I32, 100, 8, 64, ptr, 100, ptr, 10, ptr, None, 0,
                                        None, 0, None) == -1
    assert lib.b200moe_align_block_size(ptr, _lib.I32, 100, 9, 64, ptr, 1000, ptr, 100, ptr, None,
                                        0, None, 0, None) == -1
    # long input without a workspace
    n = lib.b200moe_align_single_pass_max() + 1
    assert lib.b200moe_align_workspace_bytes(n, 8) > 0
    assert lib.b200moe_align_workspace_bytes(n - 1, 8) == 0
    assert lib.b200moe_align_block_size(ptr, _lib.I32, n, 8, 64, ptr, n + 8 * 63, ptr, n, ptr, None,
                                        0, None, 0, None) == -4
    # grouped GEMM shape rules
    assert lib.b200moe_grouped_gemm_w13_swiglu(ptr, ptr, ptr, ptr, ptr, 1024, 8, 4096, 14336, 64,
                                               None) == -1
    assert b"block_m" in lib.b200moe_last_error()
    assert lib.b200moe_grouped_gemm_w13_swiglu(ptr, ptr, ptr, ptr, ptr, 1024, 8, 4100, 14336, 128,
                                               None) == -1
    assert lib.b200moe_grouped_gemm_w2_scale(ptr, ptr, ptr, ptr, ptr, ptr, ptr, 1024, 512, 8, 4096,
                                             14330, 128, None) == -1


def test_ops_refuse_cpu_tensors():
    w = torch.empty(4, 2)
    ids = torch.empty(4, 2, dtype=torch.int32)
    with pytest.raises(RuntimeError, match="CUDA"):
        _C.topk_softmax(w, ids, torch.zeros(4, 8))
    with pytest.raises(RuntimeError, match="CUDA"):
        _C.moe_sum(torch.zeros(4, 2, 8), torch.zeros(4, 8))
    with pytest.raises(RuntimeError, match="CUDA"):
        _C.silu_and_mul(torch.zeros(4, 8), torch.zeros(4, 16))
    with pytest.raises(RuntimeError, match="CUDA"):
        fused_experts(torch.zeros(4, 256, dtype=torch.bfloat16),
                      torch.zeros(8, 512, 256, dtype=torch.bfloat16),
                      torch.zeros(8, 256, 256, dtype=torch.bfloat16), torch.zeros(4, 8), 2)
    with pytest.raises(NotImplementedError):
        fused_experts(torch.zeros(4, 256), torch.zeros(8, 512, 256), torch.zeros(8, 256, 256),
                      torch.zeros(4, 8), 2, activation="gelu")


def test_fused_moe_constructor_and_weight_loader():
    with pytest.raises(ValueError):
        FusedMoE(8, 2, 256, 1000, tp_size=3)
    layer = FusedMoE(8, 2, 64, 256, tp_size=2, params_dtype=torch.bfloat16)
    assert layer.intermediate_size_per_partition == 128
    assert tuple(layer.w13_weight.shape) == (8, 256, 64)
    assert tuple(layer.w2_weight.shape) == (8, 64, 128)
    assert not layer.w13_weight.requires_grad and layer.w13_weight.dtype == torch.bfloat16
    assert layer.w13_weight.weight_loader == layer.weight_loader
    layer.tp_rank = 1
    g = torch.Generator().manual_seed(0)
    w1 = torch.randn(256, 64, generator=g).to(torch.bfloat16)
    w3 = torch.randn(256, 64, generator=g).to(torch.bfloat16)
    w2 = torch.randn(64, 256, generator=g).to(torch.bfloat16)
    layer.w13_weight.data.zero_()
    layer.w2_weight.data.zero_()
    layer.w13_weight.weight_loader(layer.w13_weight, w1, "w1", 3)
    layer.w13_weight.weight_loader(layer.w13_weight, w3, "w3", 3)
    layer.w2_weight.weight_loader(layer.w2_weight, w2, "w2", 3)
    assert torch.equal(layer.w13_weight[3, :128], w1[128:])
    assert torch.equal(layer.w13_weight[3, 128:], w3[128:])
    assert torch.equal(layer.w2_weight[3], w2[:, 128:])
    assert layer.w13_weight[2].abs().sum() == 0
    with pytest.raises(ValueError):
        layer.weight_loader(layer.w2_weight, w2, "w4", 0)


def test_synthetic_shards_are_slices_of_the_full_layer():
    wl = MoEWorkload("t", 8, 64, 256, seed=5)
    full = make_inputs(wl)
    tp = make_inputs(wl, inter_slice=slice(128, 256))
    assert torch.equal(tp["x"], full["x"]) and torch.equal(tp["logits"], full["logits"])
    assert torch.equal(tp["w13"][:, :128], full["w13"][:, 128:256])
    assert torch.equal(tp["w13"][:, 128:], full["w13"][:, 256 + 128:])
    assert torch.equal(tp["w2"], full["w2"][:, :, 128:])
    ep = make_inputs(wl, expert_slice=slice(4, 6))
    assert torch.equal(ep["w13"], full["w13"][4:6]) and torch.equal(ep["w2"], full["w2"][4:6])
    skew = make_inputs(MoEWorkload("s", 4000, 64, 128, seed=2, logit_bias=WORKLOADS[
        "mixtral_prefill_t8192_skew"].logit_bias))
    load = torch.bincount(skew["logits"].topk(2, dim=-1).indices.reshape(-1), minlength=8)
    assert load[0] > 2 * load[7]


def test_package_surface():
    assert set(pkg.__all__) >= {"_C", "layers", "install_into_reference"}
    for name in ("topk_softmax", "moe_align_block_size", "silu_and_mul", "moe_sum",
                 "moe_sum_efficient"):
        assert callable(getattr(_C, name))


def test_install_into_reference_replaces_the_layer_everywhere():
    """``install_into_reference()`` against the reference's real package (the copy staged by
    oracle/stage_reference_python.py, or the tree ELECTROCK_REFERENCE names): the model module,
    which binds ``FusedMoE`` by name when the package is imported, must end up holding this
    library's class, and the reference's ``_C`` must be this library's op module.  Runs in a child
    interpreter so that the reference package does not stay imported in the test process."""
    import os
    import subprocess
    import sys
    repo = Path(__file__).resolve().parent.parent
    staged = repo / "oracle" / "_ref" / "reference_python"
    where = staged if (staged / "electrock_infer").is_dir() else os.environ.get("ELECTROCK_REFERENCE")
    if not where or not (Path(where) / "electrock_infer").is_dir():
        pytest.skip("the reference's Python package is not available on this machine")
    code = (
        "import sys; sys.dont_write_bytecode = True\n"
        f"sys.path.insert(0, {str(repo)!r}); sys.path.insert(0, {str(where)!r})\n"
        "import electrock_infer_b200 as ours\n"
        "replaced = ours.install_into_reference()\n"
        "import electrock_infer, electrock_infer.models.mixtral as model\n"
        "import electrock_infer.layers.moe.mixtral_moe as layer, electrock_infer.layers.moe.fused_moe as fused\n"
        "from electrock_infer_b200.layers.moe import FusedMoE, fused_experts, fused_topk\n"
        "from electrock_infer_b200 import _C\n"
        "assert model.FusedMoE is FusedMoE and layer.FusedMoE is FusedMoE, replaced\n"
        "assert layer.fused_experts is fused_experts and fused.fused_experts is fused_experts\n"
        "assert fused.fused_topk is fused_topk and electrock_infer._C is _C and fused._C is _C\n"
        "assert 'electrock_infer.models.mixtral' in replaced\n"
        "print('ok')\n")
    proc = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0 and proc.stdout.strip().endswith("ok"), proc.stderr[-2000:]
