"""Bandwidth sweep of the HBM-bound ops (router, alignment, combine, stand-alone SwiGLU, gate
router, RMSNorm, paged KV-cache store and decode attention).

    python -m electrock_infer_b200.opbench [--tokens 1048576 2097152 4194304] [--iters 20]

At the layer's own token counts the router and alignment move well under a megabyte, so a single
launch is latency-bound; this sweep runs them at 2^20..2^22 tokens, where their HBM rate is
meaningful.  Buffers are larger than L2 at these sizes except the router/alignment inputs, so an
L2-sized buffer is overwritten between timed launches.  Prints one JSON line per op and size with
the algorithmic bytes, the mean CUDA-event time and GB/s, and beside them the time a plain device
copy of the same number of bytes takes under the same timing (a launch of a few tens of megabytes
does not reach the large-copy rate whatever it does).
"""
from __future__ import annotations

import argparse
import json

import torch

from . import _C


def time_op(fn, iters: int, flush: torch.Tensor) -> float:
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    total = 0.0
    for _ in range(iters):
        flush.add_(1)  # evict L2 between timed launches
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        e1.synchronize()
        total += e0.elapsed_time(e1)
    return total / iters


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, nargs="+", default=[1 << 20, 1 << 21, 1 << 22])
    ap.add_argument("--combine-tokens", type=int, nargs="+", default=[2048, 8192, 16384, 65536])
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--hidden", type=int, default=4096)
    ap.add_argument("--skip-kv", action="store_true", help="leave out the paged KV-cache ops")
    ap.add_argument("--only-kv", action="store_true", help="run only the paged KV-cache ops")
    ap.add_argument("--kv-cases", nargs="+", default=["256:1024", "256:4096", "32:8192", "4:32768"],
                    help="decode attention cases as batch:max_context")
    args = ap.parse_args()
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    flush = torch.zeros(64 << 20, dtype=torch.int32, device=dev)  # 256 MiB > L2
    g = torch.Generator(device=dev).manual_seed(0)

    copy_ms = {}

    def same_bytes_copy_ms(nbytes):
        """A plain device copy that moves the same bytes (half read, half written): what a launch of
        this size can reach at all, ramp-up and tail included."""
        half = max(nbytes // 2 // 16 * 16, 16)
        if half not in copy_ms:
            src = torch.empty(half, dtype=torch.uint8, device=dev)
            dst = torch.empty_like(src)
            copy_ms[half] = time_op(lambda: dst.copy_(src), args.iters, flush)
            del src, dst
        return copy_ms[half]

    def report(op, tokens, nbytes, ms, **kw):
        cms = same_bytes_copy_ms(nbytes)
        print(json.dumps({"op": op, "tokens": tokens, "algorithmic_bytes": nbytes,
                          "ms": round(ms, 5), "gbs": round(nbytes / ms / 1e6, 1),
                          "same_bytes_copy_ms": round(cms, 5),
                          "time_vs_copy": round(ms / cms, 2), **kw}), flush=True)

    for T in ([] if args.only_kv else args.tokens):
        logits = torch.randn(T, 8, generator=g, device=dev)
        w = torch.empty(T, 2, device=dev)
        ids = torch.empty(T, 2, dtype=torch.int32, device=dev)
        ms = time_op(lambda: _C.topk_softmax(w, ids, logits, renormalize=True), args.iters, flush)
        report("topk_softmax", T, T * 48, ms)

        bs = 128
        cap = 2 * T + 8 * (bs - 1)
        s = torch.empty(cap, dtype=torch.int32, device=dev)
        e = torch.zeros((cap + bs - 1) // bs, dtype=torch.int32, device=dev)
        n = torch.zeros(1, dtype=torch.int32, device=dev)
        ms = time_op(lambda: _C.moe_align_block_size(ids, 8, bs, s, e, n, fill_pads=True),
                     args.iters, flush)
        npp = int(n.item())
        report("moe_align_block_size", T, 2 * T * 4 + npp * 4 + (npp // bs) * 4 + 4, ms, launches=3)

    H = args.hidden
    if args.only_kv:
        args.combine_tokens = []
    for T in args.combine_tokens:
        x = torch.randn(T, 2, H, generator=g, device=dev).to(torch.bfloat16)
        out = torch.empty(T, H, dtype=torch.bfloat16, device=dev)
        ms = time_op(lambda: _C.moe_sum(x, out), args.iters, flush)
        report("moe_sum", T, T * H * 2 * 3, ms)
        xi = x.view(T, H, 2)
        ms = time_op(lambda: _C.moe_sum_efficient(xi, out), args.iters, flush)
        report("moe_sum_efficient", T, T * H * 2 * 3, ms)
    for T in args.combine_tokens:
        x = torch.randn(T, H, generator=g, device=dev).to(torch.bfloat16)
        gw = (torch.randn(8, H, generator=g, device=dev) * 0.02).to(torch.bfloat16)
        w = torch.empty(T, 2, device=dev)
        ids = torch.empty(T, 2, dtype=torch.int32, device=dev)
        ms = time_op(lambda: _C.gate_topk_softmax(w, ids, x, gw, renormalize=True), args.iters, flush)
        report("gate_topk_softmax", T, T * (H * 2 + 16), ms)
        res = torch.randn(T, H, generator=g, device=dev).to(torch.bfloat16)
        nw = torch.ones(H, dtype=torch.bfloat16, device=dev)
        ms = time_op(lambda: _C.add_rms_norm(x, res, 1e-5, nw), args.iters, flush)
        report("add_rms_norm", T, T * H * 2 * 4, ms)
    for rows, d in (() if args.only_kv else ((16384, 14336), (4096, 14336))):
        x = torch.randn(rows, 2 * d, generator=g, device=dev).to(torch.bfloat16)
        out = torch.empty(rows, d, dtype=torch.bfloat16, device=dev)
        ms = time_op(lambda: _C.silu_and_mul(out, x), args.iters, flush)
        report("silu_and_mul", rows // 2, rows * d * 2 * 3, ms)

    if args.skip_kv:
        return
    # Paged KV cache at Mixtral's head shape (32 query / 8 KV heads of 128), engine block size 256.
    q_heads, kv_heads, hd, bs = 32, 8, 128, 256
    for tokens in (8192, 65536):
        nblk = tokens // bs + 1
        key = torch.randn(tokens, kv_heads, hd, generator=g, device=dev).to(torch.bfloat16)
        val = torch.randn(tokens, kv_heads, hd, generator=g, device=dev).to(torch.bfloat16)
        kc = torch.zeros(nblk, bs, kv_heads, hd, dtype=torch.bfloat16, device=dev)
        vc = torch.zeros_like(kc)
        slots = torch.randperm(nblk * bs, generator=g, device=dev)[:tokens].to(torch.int32)
        ms = time_op(lambda: _C.paged_store_kvcache(key, val, kc, vc, slots), args.iters, flush)
        report("paged_store_kvcache", tokens, tokens * kv_heads * hd * 2 * 4 + tokens * 4, ms)
    for batch, ctx in (tuple(int(v) for v in c.split(":")) for c in args.kv_cases):
        per_seq = (ctx + bs - 1) // bs
        nblk = batch * per_seq
        kc = torch.randn(nblk, bs, kv_heads, hd, generator=g, device=dev).to(torch.bfloat16)
        vc = torch.randn(nblk, bs, kv_heads, hd, generator=g, device=dev).to(torch.bfloat16)
        q = torch.randn(batch, q_heads, hd, generator=g, device=dev).to(torch.bfloat16)
        table = torch.randperm(nblk, generator=g, device=dev).view(batch, per_seq).to(torch.int32)
        # Context lengths spread over the upper half of the range, as in a running decode batch.
        lens = torch.randint(ctx // 2, ctx + 1, (batch,), generator=g, device=dev).to(torch.int32)
        total = int(lens.sum().item())
        ms = time_op(lambda: _C.paged_attn_varlen(q, kc, vc, ctx, lens, table, hd ** -0.5),
                     args.iters, flush)
        nbytes = total * kv_heads * hd * 2 * 2 + batch * q_heads * hd * 2 * 2
        report("paged_attn_varlen", total, nbytes, ms, batch=batch, max_context=ctx)


if __name__ == "__main__":
    main()
