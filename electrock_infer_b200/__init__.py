"""B200-native Mixtral MoE layer behind electrock-infer's FusedMoE interface.

``electrock_infer_b200._C`` mirrors the reference's native op module, ``layers.moe`` mirrors its
Python layer package, and everything bottoms out in ``libb200moe.so`` (include/b200moe.h).
"""
from . import _lib  # noqa: F401  (no CUDA needed to import)

__all__ = ["_C", "_lib", "layers", "build", "install_into_reference"]
__version__ = "0.1.0"


def install_into_reference() -> None:
    """Makes an importable reference tree use this library: registers ``electrock_infer._C`` and
    replaces ``FusedMoE``/``fused_experts`` in the reference's MoE modules.  Call it before the
    reference's model modules are imported."""
    import importlib
    import sys

    from . import _C
    from .layers.moe import fused_moe, mixtral_moe

    sys.modules["electrock_infer._C"] = _C
    ref_pkg = importlib.import_module("electrock_infer")
    setattr(ref_pkg, "_C", _C)
    ref_fused = importlib.import_module("electrock_infer.layers.moe.fused_moe")
    ref_layer = importlib.import_module("electrock_infer.layers.moe.mixtral_moe")
    ref_fused.fused_experts = fused_moe.fused_experts
    ref_fused.fused_topk = fused_moe.fused_topk
    ref_layer.fused_experts = fused_moe.fused_experts
    ref_layer.FusedMoE = mixtral_moe.FusedMoE
