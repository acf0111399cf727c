"""ctypes binding of libb200moe.so: one Python callable per symbol declared in include/b200moe.h.

Nothing here computes anything: a missing library or a non-zero status raises, there is no
fallback path.
"""
from __future__ import annotations

import ctypes
from ctypes import c_char_p, c_float, c_int, c_int64, c_size_t, c_void_p
from pathlib import Path

LIB_PATH = Path(__file__).resolve().parent / "libb200moe.so"

# Element-type tags of include/b200moe.h.
F32, F16, BF16 = 0, 1, 2
I32, I64, I16, I8, U8 = 0, 1, 2, 3, 4

# (restype, argtypes) of every exported symbol, in header order.
SIGNATURES = {
    "b200moe_abi_version": (c_int, []),
    "b200moe_kernel_launch_count": (c_int64, []),
    "b200moe_last_error": (c_char_p, []),
    "b200moe_topk_softmax": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int64, c_int, c_int,
                                     c_int, c_void_p]),
    "b200moe_gate_topk_softmax": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64,
                                          c_int64, c_int, c_int, c_int, c_int, c_void_p]),
    "b200moe_align_block_size": (c_int, [c_void_p, c_int, c_int64, c_int, c_int, c_void_p, c_int64,
                                         c_void_p, c_int64, c_void_p, c_void_p, c_int, c_void_p,
                                         c_size_t, c_void_p]),
    "b200moe_align_workspace_bytes": (c_size_t, [c_int64, c_int]),
    "b200moe_align_single_pass_max": (c_int64, []),
    "b200moe_align_max_experts": (c_int, []),
    "b200moe_align_block_size_noalloc": (c_int, [c_void_p, c_int, c_int64, c_int, c_int, c_void_p,
                                                 c_int64, c_void_p, c_int64, c_void_p, c_void_p,
                                                 c_int, c_void_p]),
    "b200moe_align_noalloc_max_numel": (c_int64, []),
    "b200moe_silu_and_mul": (c_int, [c_void_p, c_void_p, c_int, c_int64, c_int64, c_void_p]),
    "b200moe_moe_sum": (c_int, [c_void_p, c_void_p, c_int, c_int64, c_int64, c_int, c_int,
                                c_void_p]),
    "b200moe_add_rms_norm": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int64, c_int64,
                                     ctypes.c_float, c_void_p]),
    "b200moe_gather_rows": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64,
                                    c_int64, c_int, c_void_p]),
    "b200moe_scatter_rows": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64,
                                     c_void_p]),
    "b200moe_grouped_gemm_w13_swiglu": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                                c_int64, c_int, c_int64, c_int64, c_int,
                                                c_void_p]),
    "b200moe_grouped_gemm_w13_swiglu_gather": (c_int, [c_void_p, c_int64, c_int, c_void_p, c_void_p,
                                                       c_void_p, c_void_p, c_void_p, c_int64, c_int,
                                                       c_int64, c_int64, c_int, c_void_p]),
    "b200moe_grouped_gemm_w2_scale": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                              c_void_p, c_void_p, c_int64, c_int64, c_int, c_int64,
                                              c_int64, c_int, c_void_p]),
    "b200moe_gather_rows_peer": (c_int, [c_void_p, c_int, c_int64, c_void_p, c_void_p, c_void_p,
                                         c_int64, c_int64, c_int, c_void_p]),
    "b200moe_grouped_gemm_w2_scale_peer": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int64,
                                                   c_void_p, c_void_p, c_void_p, c_void_p, c_int64,
                                                   c_int, c_int64, c_int64, c_int, c_void_p]),
    "b200moe_moe_sum_ranks_push": (c_int, [c_void_p, c_void_p, c_int, c_int64, c_int, c_int64,
                                           c_int64, c_int, c_void_p]),
    "b200moe_paged_store_kvcache": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                                            c_int64, c_int, c_int, c_int64, c_int64, c_int64, c_int,
                                            c_void_p]),
    "b200moe_paged_attn_num_splits": (c_int, [c_int, c_int, c_int64]),
    "b200moe_paged_attn_workspace_bytes": (c_size_t, [c_int, c_int, c_int]),
    "b200moe_paged_attn_varlen": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                          c_int, c_int, c_int, c_int, c_int, c_int64, c_int, c_int,
                                          c_float, c_int, c_void_p, c_size_t, c_void_p]),
    "b200moe_peer_alloc": (c_int, [c_size_t, ctypes.POINTER(c_void_p), c_void_p]),
    "b200moe_peer_open": (c_int, [c_void_p, ctypes.POINTER(c_void_p)]),
    "b200moe_peer_close": (c_int, [c_void_p]),
    "b200moe_peer_free": (c_int, [c_void_p]),
    "b200moe_fused_experts_rows": (c_size_t, [c_int64, c_int, c_int]),
    "b200moe_fused_experts": (c_int, [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int64,
                                      c_int, c_int, c_int64, c_int64, c_int, c_void_p, c_void_p,
                                      c_void_p, c_void_p, c_void_p, c_void_p, c_size_t, c_void_p,
                                      c_void_p, c_void_p, c_void_p]),
    "b200moe_gemm_device_status": (c_int, [c_int]),
    "b200moe_gemm_measured_cycles": (c_int, [c_void_p, c_int]),
    "b200moe_gemm_set_act_stores": (c_int, [c_int]),
    "b200moe_gemm_set_tiling": (c_int, [c_int]),
    "b200moe_gemm_two_block_choice": (c_int, [c_void_p, c_int, c_int, c_int64, c_int, c_int]),
    "b200moe_gemm_two_block_schedule": (c_int64, [c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
                                                  c_void_p, c_int64]),
}

_lib = None
_launches = 0


def count_launches(n: int = 1) -> None:
    """Kept for callers that announce their launches; the count that ``launch_count`` reports is
    the library's own (``b200moe_kernel_launch_count``), which needs no announcement."""
    global _launches
    _launches += n


def launch_count() -> int:
    """Kernels the library has launched in this process, counted by the library itself at every
    launch site (both kernels of a grouped-GEMM launch pair included)."""
    return int(load().b200moe_kernel_launch_count())


def load() -> ctypes.CDLL:
    """Loads the library once and types every entry point.  Raises if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `python -m electrock_infer_b200.build` "
            "(there is no fallback implementation)")
    lib = ctypes.CDLL(str(LIB_PATH))
    for name, (restype, argtypes) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError if the library is older than the header
        fn.restype = restype
        fn.argtypes = argtypes
    _lib = lib
    return lib


def check(status: int, what: str) -> None:
    """Turns a negative status into the RuntimeError the reference's TORCH_CHECKs raise."""
    if status != 0:
        msg = load().b200moe_last_error().decode("utf-8", "replace")
        raise RuntimeError(f"{what}: {msg} (status {status})")
