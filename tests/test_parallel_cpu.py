"""Multi-rank host logic on CPU ranks (gloo, world size 2): the expert-parallel exchange (counts,
variable-split all-to-alls, return path, un-permutation) and the tensor-parallel all-reduce branch
of FusedMoE.forward.  The arithmetic is supplied by oracle-based stand-ins defined here; the
product's own arithmetic only exists on the GPU."""
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

WORLD = 2


class OracleOps:
    """CPU stand-in for parallel.CudaOps built from the oracle."""

    def route(self, logits, top_k, renormalize):
        from oracle import moe_oracle
        return moe_oracle.router_ref(logits, top_k, renormalize)

    def sort_pairs_by_expert(self, ids, num_experts):
        flat = ids.reshape(-1).long()
        order = torch.sort(flat, stable=True).indices.to(torch.int32)
        return order, torch.bincount(flat, minlength=num_experts).to(torch.int32)

    def take_rows(self, src, index, top_k):
        return src[index.long() // top_k].contiguous()

    def expert_ffn(self, rows, row_expert, row_weight, w13, w2):
        inter = w13.shape[1] // 2
        out = torch.zeros(rows.shape[0], rows.shape[1])
        for e in range(w13.shape[0]):
            m = row_expert == e
            if m.any():
                x = rows[m].float()
                h = torch.nn.functional.silu(x @ w13[e, :inter].float().T) * (x @ w13[e, inter:].float().T)
                out[m] = (h @ w2[e].float().T) * row_weight[m].unsqueeze(1)
        return out.to(rows.dtype)

    def combine(self, y_back, order, out, top_k):
        cache = torch.zeros(out.shape[0] * top_k, out.shape[1], dtype=y_back.dtype)
        cache[order.long()] = y_back
        out.copy_(cache.view(out.shape[0], top_k, out.shape[1]).float().sum(1).to(out.dtype))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _init(rank, port, result_dir):
    # MASTER_* stay set for code that reads them; the rendezvous itself goes through a file in the
    # test's own directory, because a TCP port found free by the parent can be taken again before
    # the workers bind it.
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", init_method=f"file://{result_dir}/rendezvous", rank=rank,
                            world_size=WORLD)


def _ep_worker(rank, port, skew, result_dir):
    from electrock_infer_b200.parallel import ExpertParallelMoE
    from oracle import moe_oracle
    _init(rank, port, result_dir)
    bias = (3, 2, 1, 0, 0, -1, -2, -9) if skew else None
    wl = MoEWorkload("ep", 70, 32, 64, dtype=torch.float32, seed=17, logit_bias=bias)
    full = make_inputs(wl)
    per = wl.num_experts // WORLD
    layer = ExpertParallelMoE(wl.num_experts, 2, wl.hidden, wl.inter, params_dtype=torch.float32,
                              ops=OracleOps())
    for e in range(wl.num_experts):  # the loader keeps only this rank's experts
        layer.weight_loader(layer.w13_weight, full["w13"][e, : wl.inter], "w1", e)
        layer.weight_loader(layer.w13_weight, full["w13"][e, wl.inter:], "w3", e)
        layer.weight_loader(layer.w2_weight, full["w2"][e], "w2", e)
    assert torch.equal(layer.w13_weight.data, full["w13"][rank * per:(rank + 1) * per])
    # Uneven token split: rank 0 gets 41 tokens, rank 1 gets 29.
    lo, hi = (0, 41) if rank == 0 else (41, 70)
    x = full["x"][lo:hi].clone()
    out = layer(x, full["logits"][lo:hi])
    assert out.data_ptr() == x.data_ptr()
    want = moe_oracle.moe_block_ref(full["x"], full["w13"], full["w2"], full["logits"])[lo:hi]
    err = (out - want).abs().max().item()
    torch.save({"err": err, "rows": out.shape[0]}, os.path.join(result_dir, f"ep{rank}.pt"))
    dist.destroy_process_group()


@pytest.mark.parametrize("skew", [False, True])
def test_expert_parallel_exchange_on_gloo(tmp_path, skew):
    mp.spawn(_ep_worker, args=(_free_port(), skew, str(tmp_path)), nprocs=WORLD, join=True)
    for rank, rows in ((0, 41), (1, 29)):
        r = torch.load(tmp_path / f"ep{rank}.pt")
        assert r["rows"] == rows and r["err"] < 1e-4, r


def _tp_worker(rank, port, result_dir):
    from electrock_infer_b200.layers.moe import FusedMoE, mixtral_moe
    from oracle import moe_oracle
    _init(rank, port, result_dir)
    wl = MoEWorkload("tp", 33, 32, 64, dtype=torch.float32, seed=19)
    full = make_inputs(wl)

    def cpu_fused_experts(hidden_states, w1, w2, gating_output, topk, renormalize, inplace,
                          activation, tp_reduce=None):
        assert tp_reduce is None  # CPU tensors / gloo: the sum stays a process-group all-reduce
        out = moe_oracle.moe_block_ref(hidden_states, w1, w2, gating_output, topk, renormalize)
        hidden_states.copy_(out)
        return hidden_states

    mixtral_moe.fused_experts = cpu_fused_experts  # this process only
    layer = FusedMoE(wl.num_experts, 2, wl.hidden, wl.inter, tp_size=WORLD,
                     params_dtype=torch.float32, reduce_results=True)
    assert layer.tp_rank == rank and layer.intermediate_size_per_partition == wl.inter // WORLD
    for e in range(wl.num_experts):
        layer.weight_loader(layer.w13_weight, full["w13"][e, : wl.inter], "w1", e)
        layer.weight_loader(layer.w13_weight, full["w13"][e, wl.inter:], "w3", e)
        layer.weight_loader(layer.w2_weight, full["w2"][e], "w2", e)
    shard = make_inputs(wl, inter_slice=slice(rank * 32, (rank + 1) * 32))
    assert torch.equal(layer.w13_weight.data, shard["w13"]) and torch.equal(layer.w2_weight.data, shard["w2"])
    x = full["x"].clone()
    out = layer(x, full["logits"])
    want = moe_oracle.moe_block_ref(full["x"], full["w13"], full["w2"], full["logits"])
    # The in-kernel all-reduce is refused, not silently replaced, where it cannot run.
    forced = FusedMoE(wl.num_experts, 2, wl.hidden, wl.inter, tp_size=WORLD,
                      params_dtype=torch.float32, reduce_results=True, tp_exchange="peer")
    try:
        forced.peer_reduce_for(torch.zeros(34, wl.hidden))
        refused = False
    except RuntimeError:
        refused = True
    # Token-slice ownership of the in-kernel reduce: only whole slices, never an empty batch.
    from electrock_infer_b200.parallel import TensorParallelReduce
    red = TensorParallelReduce()
    slices_ok = (red.world == WORLD and red.rank == rank and red.usable(600) and not red.usable(601)
                 and not red.usable(0))
    torch.save({"err": (out - want).abs().max().item(), "alias": out.data_ptr() == x.data_ptr(),
                "refused": refused and slices_ok},
               os.path.join(result_dir, f"tp{rank}.pt"))
    dist.destroy_process_group()


def test_tensor_parallel_all_reduce_on_gloo(tmp_path):
    mp.spawn(_tp_worker, args=(_free_port(), str(tmp_path)), nprocs=WORLD, join=True)
    for rank in range(WORLD):
        r = torch.load(tmp_path / f"tp{rank}.pt")
        assert r["alias"] and r["err"] < 1e-4 and r["refused"], r


def _decision_worker(rank, port, result_dir):
    """Which exchange a call takes must not depend on anything only one rank can see.  The ranks
    walk through batches whose sizes change unevenly between calls (the case in which a choice
    keyed on the local token count sent the ranks into different collectives) and record, call by
    call, what ``peer_capacity`` answers; with the oracle stand-in every call then runs the NCCL
    exchange to the end, which would hang if the ranks disagreed."""
    from electrock_infer_b200.parallel import ExpertParallelMoE, TensorParallelReduce
    _init(rank, port, result_dir)
    wl = MoEWorkload("ep", 100, 32, 64, dtype=torch.float32, seed=5)
    full = make_inputs(wl)
    counts = [(50, 50), (50, 45), (50, 50), (10, 0), (0, 30), (50, 50)]  # (rank 0, rank 1) per call
    seen = {}
    for name, kwargs in (("auto", {}), ("auto_bounded", {"max_tokens_per_rank": 64}),
                         ("nccl", {"exchange": "nccl"}),
                         ("peer_bounded", {"exchange": "peer", "max_tokens_per_rank": 64})):
        layer = ExpertParallelMoE(wl.num_experts, 2, wl.hidden, wl.inter, params_dtype=torch.float32,
                                  ops=OracleOps(), **kwargs)
        for e in range(wl.num_experts):
            layer.weight_loader(layer.w13_weight, full["w13"][e, : wl.inter], "w1", e)
            layer.weight_loader(layer.w13_weight, full["w13"][e, wl.inter:], "w3", e)
            layer.weight_loader(layer.w2_weight, full["w2"][e], "w2", e)
        answers = []
        for pair in counts:
            n = pair[rank]
            answers.append(layer.peer_capacity(n))
            lo = 0 if rank == 0 else 50
            out = layer(full["x"][lo:lo + n].clone(), full["logits"][lo:lo + n])
            assert out.shape[0] == n
        seen[name] = answers
    # Forced peer mode without a bound: the caller promises equal counts; the capacity is a bucket.
    forced = ExpertParallelMoE(wl.num_experts, 2, wl.hidden, wl.inter, params_dtype=torch.float32,
                               ops=OracleOps(), exchange="peer")
    seen["peer_unbounded"] = [forced.peer_capacity(n) for n in (1, 256, 257, 2048, 3000)]
    red = TensorParallelReduce()
    seen["tp_capacity"] = [red.capacity_for(n) for n in (2, 600, 8192, 8194)]
    torch.save(seen, os.path.join(result_dir, f"dec{rank}.pt"))
    dist.destroy_process_group()


def test_exchange_choice_is_the_same_on_every_rank(tmp_path):
    mp.spawn(_decision_worker, args=(_free_port(), str(tmp_path)), nprocs=WORLD, join=True)
    a, b = (torch.load(tmp_path / f"dec{r}.pt") for r in range(WORLD))
    assert a == b, (a, b)
    assert a["auto"] == [None] * 6 and a["nccl"] == [None] * 6
    assert a["auto_bounded"] == [64] * 6 and a["peer_bounded"] == [64] * 6
    assert a["peer_unbounded"] == [256, 256, 512, 2048, 4096]
    assert a["tp_capacity"] == [256, 1024, 8192, 16384]


def test_workspace_capacity_buckets():
    from electrock_infer_b200.layers.moe.fused_moe import capacity_bucket
    assert [capacity_bucket(n) for n in (0, 1, 255, 256, 257, 8191, 8192, 8193)] == \
        [256, 256, 256, 256, 512, 8192, 8192, 16384]


def test_split_sizes_and_row_experts():
    from electrock_infer_b200.parallel import received_row_experts, split_sizes
    assert split_sizes([3, 0, 2, 5, 1, 1, 0, 4], 2) == [10, 6]
    assert split_sizes([3, 0, 2, 5, 1, 1, 0, 4], 8) == [3, 0, 2, 5, 1, 1, 0, 4]
    counts = torch.tensor([2, 0, 1, 3], dtype=torch.int32)  # 2 sources x 2 local experts
    rows = received_row_experts(counts, 6) % 2
    assert rows.tolist() == [0, 0, 0, 1, 1, 1] and rows.dtype == torch.int32
