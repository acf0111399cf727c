"""The allocation-free alignment entry point, called through the C ABI.

Some hosts of this library cannot hand it a device workspace at call time: a server that gave the
whole GPU to a pre-sized pool when it started, a plain C / FFI host that owns no device allocator,
or a latency-critical loop in which a cudaMalloc would stall the device.  For them
``b200moe_align_block_size_noalloc`` keeps the segment counters of long inputs in an array built
into the library.  It must produce exactly what the workspace variant produces, also when called
twice in a row (the array keeps the previous call's contents), and must refuse inputs beyond its
stated limit.

This file is named so that pytest collects it last.
"""
import ctypes

import numpy as np
import pytest
import torch

from electrock_infer_b200 import _lib

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _outputs(numel, bs, E=8):
    cap = numel + E * (bs - 1)
    return (torch.full((cap,), -3, dtype=torch.int32, device=DEV),
            torch.full(((cap + bs - 1) // bs,), -3, dtype=torch.int32, device=DEV),
            torch.full((1,), -3, dtype=torch.int32, device=DEV),
            torch.full((E + 1,), -3, dtype=torch.int32, device=DEV))


def _tag(ids):
    return {torch.int32: _lib.I32, torch.int64: _lib.I64}[ids.dtype]


def _with_workspace(lib, ids, bs, fill, stream):
    s, e, n, off = _outputs(ids.numel(), bs)
    ws_bytes = lib.b200moe_align_workspace_bytes(ids.numel(), 8)
    ws = torch.empty(max(ws_bytes // 4, 1), dtype=torch.int32, device=DEV)
    rc = lib.b200moe_align_block_size(ids.data_ptr(), _tag(ids), ids.numel(), 8, bs, s.data_ptr(),
                                      s.numel(), e.data_ptr(), e.numel(), n.data_ptr(),
                                      off.data_ptr(), fill, ws.data_ptr(), ws_bytes, stream)
    _lib.check(rc, "align_block_size")
    torch.cuda.synchronize()
    return s, e, n, off


def _no_alloc(lib, ids, bs, fill, stream):
    s, e, n, off = _outputs(ids.numel(), bs)
    rc = lib.b200moe_align_block_size_noalloc(ids.data_ptr(), _tag(ids), ids.numel(), 8, bs,
                                              s.data_ptr(), s.numel(), e.data_ptr(), e.numel(),
                                              n.data_ptr(), off.data_ptr(), fill, stream)
    _lib.check(rc, "align_block_size_noalloc")
    torch.cuda.synchronize()
    return s, e, n, off


def test_no_alloc_alignment_matches_workspace_variant_twice_in_a_row():
    lib = _lib.load()
    stream = torch.cuda.current_stream().cuda_stream
    single_pass = lib.b200moe_align_single_pass_max()
    g = torch.Generator().manual_seed(2024)
    # Both inputs are long enough to need the segment counters; the second is shorter and has a
    # different expert mix, so stale counters from the first call would show.
    first = torch.randint(0, 8, (3 * single_pass + 777,), generator=g, dtype=torch.int32).to(DEV)
    second = torch.multinomial(torch.tensor([6., 3, 1, 1, 0.5, 0.2, 0.2, 0.1]), single_pass + 4099,
                               True, generator=g).to(torch.int32).to(DEV)
    assert first.numel() > single_pass and second.numel() > single_pass
    for ids, bs, fill in ((first, 128, 1), (second, 64, 0), (first, 64, 1)):
        want = _with_workspace(lib, ids, bs, fill, stream)
        got = _no_alloc(lib, ids, bs, fill, stream)
        for a, b in zip(got, want):
            assert torch.equal(a, b)  # integer outputs: bit-exact, untouched slots included
    # int64 expert ids (what torch.topk hands out) go through the same scratch.
    wide = second.to(torch.int64)
    for a, b in zip(_no_alloc(lib, wide, 128, 1, stream), _with_workspace(lib, wide, 128, 1, stream)):
        assert torch.equal(a, b)
    # Short inputs take the one-launch path and must agree as well.
    short = first[:5000].contiguous()
    for a, b in zip(_no_alloc(lib, short, 128, 1, stream), _with_workspace(lib, short, 128, 1, stream)):
        assert torch.equal(a, b)


def test_no_alloc_alignment_rejects_inputs_beyond_its_limit():
    lib = _lib.load()
    limit = lib.b200moe_align_noalloc_max_numel()
    assert limit == 1 << 24
    ptr = ctypes.c_void_p(256)  # never dereferenced: the size check comes first
    rc = lib.b200moe_align_block_size_noalloc(ptr, _lib.I32, limit + 1, 8, 128, ptr,
                                              limit + 1 + 8 * 127, ptr, limit, ptr, None, 0, None)
    assert rc == -1
    msg = lib.b200moe_last_error().decode()
    assert "exceeds the built-in scratch limit" in msg and "workspace" in msg
