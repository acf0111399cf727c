"""Tensor- and expert-parallel layer on 2 GPUs over NCCL, compared with the single-GPU layer and
the CPU oracle.  Skipped on a box with fewer than two GPUs."""
import os
import socket
import sys
from pathlib import Path

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

REPO = Path(__file__).resolve().parent.parent
if str(REPO) not in sys.path:
    sys.path.insert(0, str(REPO))

from electrock_infer_b200.synthetic import MoEWorkload, make_inputs  # noqa: E402

pytestmark = pytest.mark.gpu
WORLD = 2


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker_full_size(rank, port, mode, result_dir):
    """BASELINE config 3 at its own size: Mixtral-8x7B shape, T=16384 per step on two GPUs.  Weights
    and tokens are drawn on the device from the workload seed (both ranks draw the same values);
    the oracle runs on a fixed sample of tokens."""
    from electrock_infer_b200 import _lib
    from electrock_infer_b200.layers.moe import FusedMoE, fused_experts
    from electrock_infer_b200.parallel import ExpertParallelMoE
    from electrock_infer_b200.synthetic import WORKLOADS
    from oracle import moe_oracle
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    # Rendezvous through a file in the test's own directory: a TCP port found free by the parent can
    # be taken again before the workers bind it.
    dist.init_process_group("nccl", init_method=f"file://{result_dir}/rendezvous", rank=rank,
                            world_size=WORLD, device_id=dev)
    wl = WORKLOADS["mixtral_parallel_t16384"]
    T, I = wl.num_tokens, wl.inter
    full = make_inputs(wl, device=dev, device_rng=True)
    res = {}
    with torch.inference_mode():
        if mode == "ep_full_size":
            per = wl.num_experts // WORLD
            layer = ExpertParallelMoE(8, 2, wl.hidden, I, params_dtype=torch.bfloat16,
                                      max_tokens_per_rank=T // WORLD).to(dev)
            layer.w13_weight.data.copy_(full["w13"][rank * per:(rank + 1) * per])
            layer.w2_weight.data.copy_(full["w2"][rank * per:(rank + 1) * per])
            lo, hi = rank * T // WORLD, (rank + 1) * T // WORLD
        else:
            shard = I // WORLD
            layer = FusedMoE(8, 2, wl.hidden, I, tp_size=WORLD, params_dtype=torch.bfloat16,
                             reduce_results=True, tp_exchange="peer").to(dev)
            for e in range(8):
                layer.weight_loader(layer.w13_weight, full["w13"][e, :I], "w1", e)
                layer.weight_loader(layer.w13_weight, full["w13"][e, I:], "w3", e)
                layer.weight_loader(layer.w2_weight, full["w2"][e], "w2", e)
            assert layer.w13_weight.shape[1] == 2 * shard
            lo, hi = 0, T
        x = full["x"][lo:hi].clone()
        out = layer(x, full["logits"][lo:hi].contiguous())
        torch.cuda.synchronize()
        res["alias"] = out.data_ptr() == x.data_ptr()
        single = fused_experts(full["x"][lo:hi].clone(), full["w13"], full["w2"],
                               full["logits"][lo:hi].contiguous(), 2, inplace=True)
        torch.cuda.synchronize()
        res["bit_exact_vs_single"] = bool(torch.equal(out, single))
        res["vs_single"] = moe_oracle.error_stats(out.float().cpu(), single.float().cpu())
        sample = torch.randperm(hi - lo, generator=torch.Generator().manual_seed(rank))[:64].to(dev)
        want = moe_oracle.moe_block_ref(full["x"][lo:hi][sample].cpu(), full["w13"].cpu(),
                                        full["w2"].cpu(), full["logits"][lo:hi][sample].cpu())
        res["stats"] = moe_oracle.error_stats(out[sample].float().cpu(), want)
        if mode == "tp_full_size":
            both = [torch.empty_like(out) for _ in range(WORLD)]
            dist.all_gather(both, out)
            res["ranks_agree"] = bool(torch.equal(both[0], both[1]))
    res["gemm_status"] = _lib.load().b200moe_gemm_device_status(1)
    dist.barrier()
    if mode == "ep_full_size":
        layer.close()
    else:
        layer._tp_reduce.close()
    torch.save(res, os.path.join(result_dir, f"{mode}{rank}.pt"))
    dist.destroy_process_group()


@pytest.mark.parametrize("mode", ["ep_full_size", "tp_full_size"])
def test_two_gpu_layer_at_config_size(tmp_path, mode):
    """T=16384 at Mixtral shape, expert parallel over peer memory and tensor parallel with the
    in-kernel reduce: in-place result, oracle on a 64-token sample per rank, and against the
    single-GPU layer on the same rows (bit for bit for EP)."""
    if torch.cuda.device_count() < WORLD:
        pytest.skip("needs two GPUs")
    mp.spawn(_worker_full_size, args=(_free_port(), mode, str(tmp_path)), nprocs=WORLD, join=True)
    for rank in range(WORLD):
        r = torch.load(tmp_path / f"{mode}{rank}.pt")
        assert r["alias"] and r["gemm_status"] == 0, r
        assert r["stats"]["max_abs"] <= 3e-2 and r["stats"]["rel_fro"] <= 1e-2, r
        if mode == "ep_full_size":
            assert r["bit_exact_vs_single"], "expert-parallel rows must equal the single-GPU rows"
        else:
            assert r["vs_single"]["rel_fro"] <= 1e-2 and r["ranks_agree"], r


def _worker(rank, port, mode, result_dir):
    from electrock_infer_b200 import _lib
    from electrock_infer_b200.layers.moe import FusedMoE, fused_experts
    from electrock_infer_b200.parallel import ExpertParallelMoE
    from oracle import moe_oracle
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    # Rendezvous through a file in the test's own directory: a TCP port found free by the parent can
    # be taken again before the workers bind it.
    dist.init_process_group("nccl", init_method=f"file://{result_dir}/rendezvous", rank=rank,
                            world_size=WORLD, device_id=dev)
    tokens = 6 if mode == "ep_peer_tiny" else 600
    wl = MoEWorkload("par", tokens, 512, 1024, seed=23, logit_bias=(2, 1, 0.5, 0, 0, -0.5, -1, -2))
    full = make_inputs(wl)
    want = moe_oracle.moe_block_ref(full["x"], full["w13"], full["w2"], full["logits"])
    single = fused_experts(full["x"].to(dev), full["w13"].to(dev), full["w2"].to(dev),
                           full["logits"].to(dev), 2, inplace=False)
    res = {}
    if mode.endswith("_fallback") and rank == 1:
        # One rank cannot map its peers' buffers: every rank must notice and use NCCL instead.
        _lib.load().b200moe_peer_open = lambda *args: -6
    if mode.startswith("tp"):
        # "tp": the reference's NCCL all-reduce; "tp_peer": the all-reduce inside the layer's kernels.
        layer = FusedMoE(8, 2, wl.hidden, wl.inter, tp_size=WORLD, params_dtype=torch.bfloat16,
                         reduce_results=True,
                         tp_exchange={"tp_peer": "peer", "tp_auto_fallback": "auto"}.get(mode, "nccl")).to(dev)
        layer.PEER_REDUCE_MIN_BYTES = 0   # "auto" would otherwise keep NCCL for this small batch
        for e in range(8):
            layer.weight_loader(layer.w13_weight, full["w13"][e, : wl.inter].to(dev), "w1", e)
            layer.weight_loader(layer.w13_weight, full["w13"][e, wl.inter:].to(dev), "w3", e)
            layer.weight_loader(layer.w2_weight, full["w2"][e].to(dev), "w2", e)
        x = full["x"].to(dev).clone()
        out = layer(x, full["logits"].to(dev))
        torch.cuda.synchronize()
        res["alias"] = out.data_ptr() == x.data_ptr()
        res["stats"] = moe_oracle.error_stats(out.cpu().float(), want)
        res["vs_single"] = moe_oracle.error_stats(out.cpu().float(), single.cpu().float())
        if mode == "tp_auto_fallback":
            res["fell_back"] = layer.tp_exchange == "nccl"
        if mode == "tp_peer":
            # Every rank must hold the same bits, and a second call must reuse the buffers cleanly.
            both = [torch.empty_like(out) for _ in range(WORLD)]
            dist.all_gather(both, out)
            res["ranks_agree"] = bool(torch.equal(both[0], both[1]))
            x2 = full["x"].to(dev).flip(0).contiguous()
            out2 = layer(x2, full["logits"].to(dev).flip(0).contiguous())
            torch.cuda.synchronize()
            res["second_call"] = bool(torch.equal(out2, out.flip(0)))
            # With two ranks the in-kernel sum rounds where the reference does (each rank's partial
            # result to bf16, then one correctly rounded add): same bits as the NCCL all-reduce.
            layer.tp_exchange = "nccl"
            out3 = layer(full["x"].to(dev).clone(), full["logits"].to(dev))
            torch.cuda.synchronize()
            res["equals_nccl"] = bool(torch.equal(out3, out))
    elif mode == "ep_peer_ragged":
        # Peer-memory exchange with a per-rank bound: uneven token counts, then a rank with no
        # tokens at all, with no host synchronisation in either step.
        layer = ExpertParallelMoE(8, 2, wl.hidden, wl.inter, params_dtype=torch.bfloat16,
                                  exchange="peer", max_tokens_per_rank=400).to(dev)
        for e in range(8):
            layer.weight_loader(layer.w13_weight, full["w13"][e, : wl.inter].to(dev), "w1", e)
            layer.weight_loader(layer.w13_weight, full["w13"][e, wl.inter:].to(dev), "w3", e)
            layer.weight_loader(layer.w2_weight, full["w2"][e].to(dev), "w2", e)
        lo, hi = (0, 350) if rank == 0 else (350, 600)
        x = full["x"][lo:hi].to(dev).clone()
        out = layer(x, full["logits"][lo:hi].to(dev))
        torch.cuda.synchronize()
        res["alias"] = out.data_ptr() == x.data_ptr()
        res["stats"] = moe_oracle.error_stats(out.cpu().float(), want[lo:hi])
        res["bit_exact_vs_single"] = bool(torch.equal(out, single[lo:hi]))
        lo, hi = (0, 0) if rank == 0 else (563, 600)      # rank 0 sits this step out
        x2 = full["x"][lo:hi].to(dev).clone()
        out2 = layer(x2, full["logits"][lo:hi].to(dev))
        torch.cuda.synchronize()
        res["bit_exact_second_call"] = bool(torch.equal(out2, single[lo:hi])) and out2.shape[0] == hi - lo
    else:
        # "auto" takes the peer-memory exchange only with a bound on the tokens per rank.
        layer = ExpertParallelMoE(8, 2, wl.hidden, wl.inter, params_dtype=torch.bfloat16,
                                  exchange="peer" if mode.startswith("ep_peer") else
                                  ("auto" if mode == "ep_auto_fallback" else "nccl"),
                                  max_tokens_per_rank=tokens // 2 if mode == "ep_auto_fallback"
                                  else None).to(dev)
        for e in range(8):
            layer.weight_loader(layer.w13_weight, full["w13"][e, : wl.inter].to(dev), "w1", e)
            layer.weight_loader(layer.w13_weight, full["w13"][e, wl.inter:].to(dev), "w3", e)
            layer.weight_loader(layer.w2_weight, full["w2"][e].to(dev), "w2", e)
        if mode.startswith("ep_peer") or mode == "ep_auto_fallback":  # equal splits: "auto" tries peer memory
            lo, hi = (0, tokens // 2) if rank == 0 else (tokens // 2, tokens)
        else:
            lo, hi = (0, 350) if rank == 0 else (350, 600)  # uneven token split
        x = full["x"][lo:hi].to(dev).clone()
        out = layer(x, full["logits"][lo:hi].to(dev))
        torch.cuda.synchronize()
        res["alias"] = out.data_ptr() == x.data_ptr()
        res["stats"] = moe_oracle.error_stats(out.cpu().float(), want[lo:hi])
        res["bit_exact_vs_single"] = bool(torch.equal(out, single[lo:hi]))
        # Second call on the same buffers (staging and return buffers are reused every step).
        x2 = full["x"][lo:hi].to(dev).flip(0).contiguous()
        out2 = layer(x2, full["logits"][lo:hi].to(dev).flip(0).contiguous())
        torch.cuda.synchronize()
        res["bit_exact_second_call"] = bool(torch.equal(out2, single[lo:hi].flip(0)))
        if mode == "ep_auto_fallback":
            res["fell_back"] = layer.exchange == "nccl"
    res["gemm_status"] = _lib.load().b200moe_gemm_device_status(1)
    # Release the peer-visible buffers once every rank has finished with them.
    dist.barrier()
    if mode == "tp_peer":
        layer._tp_reduce.close()
    elif mode.startswith("ep_peer"):
        layer.close()
    torch.save(res, os.path.join(result_dir, f"{mode}{rank}.pt"))
    dist.destroy_process_group()


@pytest.mark.parametrize("mode", ["tp", "tp_peer", "tp_auto_fallback", "ep", "ep_peer", "ep_peer_tiny",
                                  "ep_peer_ragged", "ep_auto_fallback"])
def test_two_gpu_layer(tmp_path, mode):
    if torch.cuda.device_count() < WORLD:
        pytest.skip("needs two GPUs")
    mp.spawn(_worker, args=(_free_port(), mode, str(tmp_path)), nprocs=WORLD, join=True)
    for rank in range(WORLD):
        r = torch.load(tmp_path / f"{mode}{rank}.pt")
        assert r["alias"] and r["gemm_status"] == 0, r
        assert r["stats"]["max_abs"] <= 3e-2 and r["stats"]["rel_fro"] <= 1e-2, r
        if mode.endswith("_fallback"):
            assert r["fell_back"], "every rank must have switched to NCCL"
        if mode.startswith("ep"):
            assert r["bit_exact_vs_single"], "expert-parallel rows must equal the single-GPU rows"
            assert r["bit_exact_second_call"]
        else:
            # TP sums two bf16-rounded partial outputs: close to, not identical with, one GPU.
            assert r["vs_single"]["rel_fro"] <= 1e-2, r
            if mode == "tp_peer":
                assert r["ranks_agree"] and r["second_call"] and r["equals_nccl"], r
