"""B200-native Mixtral MoE layer behind electrock-infer's FusedMoE interface.

``electrock_infer_b200._C`` mirrors the reference's native op module, ``layers.moe`` mirrors its
Python layer package, and everything bottoms out in ``libb200moe.so`` (include/b200moe.h).
"""
from . import _lib  # noqa: F401  (no CUDA needed to import)

__all__ = ["_C", "_lib", "layers", "build", "install_into_reference"]
__version__ = "0.1.0"


def install_into_reference() -> dict:
    """Makes an importable reference tree (``electrock_infer`` on ``sys.path``) use this library:
    registers this package's ``_C`` as ``electrock_infer._C`` and replaces ``FusedMoE``,
    ``fused_experts`` and ``fused_topk`` wherever the reference holds them.

    The reference's package ``__init__`` imports its engine, which imports the model, which binds
    ``FusedMoE`` by name (models/mixtral.py:13); importing any reference module therefore imports
    all of them.  So the replacement is done after the import, in every loaded
    ``electrock_infer.*`` module that holds one of the reference's objects under its own name.
    Call it before the model is constructed (``LLM(...)``), in every rank process.  Returns the
    names it replaced, per module."""
    import importlib
    import sys

    from . import _C
    from .layers.moe import fused_moe, mixtral_moe

    sys.modules["electrock_infer._C"] = _C
    ref_fused = importlib.import_module("electrock_infer.layers.moe.fused_moe")
    ref_layer = importlib.import_module("electrock_infer.layers.moe.mixtral_moe")
    sys.modules["electrock_infer"]._C = _C
    swaps = {}
    for name, ours in (("FusedMoE", mixtral_moe.FusedMoE), ("fused_experts", fused_moe.fused_experts),
                       ("fused_topk", fused_moe.fused_topk)):
        theirs = getattr(ref_layer, name, None) if name == "FusedMoE" else getattr(ref_fused, name, None)
        if theirs is not None and theirs is not ours:
            swaps[name] = (theirs, ours)
    replaced = {}
    for mod_name, mod in list(sys.modules.items()):
        if mod is None or not (mod_name == "electrock_infer" or mod_name.startswith("electrock_infer.")):
            continue
        if getattr(mod, "_C", _C) is not _C and mod_name != "electrock_infer._C":
            mod._C = _C
        for name, (theirs, ours) in swaps.items():
            if getattr(mod, name, None) is theirs:
                setattr(mod, name, ours)
                replaced.setdefault(mod_name, []).append(name)
    return replaced
