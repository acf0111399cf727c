"""MoE-layer throughput benchmark: tokens/s of ``FusedMoE.forward`` at Mixtral-8x7B shape.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--parallel ep|ep_nccl|tp|tp_nccl]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...
    python bench.py --impl reference ...      # the reference's torch CPU path on the host cores

One step is one pass of the layer over one batch of seeded synthetic tokens.  At one GPU the
workload is the prefill-sized, skew-routed Mixtral layer (T=8192); at N > 1 it is the T=16384 step
sharded expert-parallel (default) or tensor-parallel as the reference does (--parallel tp; tp_nccl
keeps the reference's NCCL all-reduce).  Rank 0 prints ONE JSON line:

  value         tokens/s with inputs resident in HBM (CUDA events around K steps, max over ranks)
  e2e           the same through host buffers: pinned H2D of activations and logits and D2H of the
                result inside the timed region, every step
  roofline      the dominant kernel (grouped GEMM w13 + SwiGLU): algorithmic FLOPs per launch over
                its mean launch time, measured with CUDA events inside the timed region
  cpu_baseline  the oracle's torch CPU block timed on this host on a bounded token sample
  clocks        SM clock and throttle reasons sampled with nvidia-smi during the timed region
"""
from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

from electrock_infer_b200.synthetic import WORKLOADS, MoEWorkload, make_inputs  # noqa: E402

METRIC = "moe_layer_tokens_per_s"
UNIT = "tokens/s"
# DRAM traffic of the w13 kernel measured with ncu (dram__bytes_read + dram__bytes_write) on the
# T=2048 case: 2.075 GB against 2.050 GB of algorithmic bytes (weights + A rows + output rows).
# Traffic is weights + rows x (H + I') x 2 bytes, so a full-size launch is scaled by the same ratio.
NCU_TRAFFIC_RATIO = 2.075 / 2.050
# Device buffers of the end-to-end pipeline: step i+3's upload waits for step i's download (the
# layer writes its result over its input), so three buffers let upload, kernels and download of
# neighbouring steps all overlap.
E2E_BUFFERS = 3
NCU_TRAFFIC_NOTE = ("algorithmic bytes x 1.012, the ncu DRAM read+write / algorithmic ratio of the "
                    "T=2048 capture (profiles/grouped_gemm_t2048_ncu_full.txt)")
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def load_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            d = json.loads(p.read_text())
            return {k: float(d[k]) for k in FALLBACK_PEAKS if k in d} | {"source": "measured"}
        except Exception:
            pass
    return dict(FALLBACK_PEAKS, source="fallback")


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu_index = gpu_index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                 "-i", str(self.gpu_index), "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._pump, daemon=True).start()
        except OSError:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append((time.time(), line.strip()))

    def stop(self, t0: float, t1: float) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        rows = [l.split(", ") for t, l in self.lines if t0 - 0.05 <= t <= t1 + 0.15]
        if not rows:
            rows = [l.split(", ") for _, l in self.lines[-3:]]
        sm, smax, power, reasons = [], [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in rows:
            try:
                sm.append(float(r[1])); smax.append(float(r[2])); power.append(float(r[3]))
            except (ValueError, IndexError):
                continue
            for name, v in zip(names, r[5:9]):
                if v.strip().lower() == "active":
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None,
                "sm_max_mhz": max(smax) if smax else None,
                "power_w": round(statistics.median(power), 1) if power else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def dist_env():
    return (int(os.environ.get("RANK", 0)), int(os.environ.get("LOCAL_RANK", 0)),
            int(os.environ.get("WORLD_SIZE", 1)))


# --------------------------------------------------------------------------------- reference arm
def cpu_block_tokens_per_s(wl: MoEWorkload, inp: dict, sample_tokens: int, steps: int, warmup: int,
                           dtype: torch.dtype):
    """Times the oracle's restatement of the reference torch block (MixtralSparseMoeBlock,
    test/example/verify_hf_moe.py:43-86) on the host cores for ``sample_tokens`` tokens."""
    from oracle import moe_oracle
    torch.set_num_threads(os.cpu_count() or 1)
    x = inp["x"][:sample_tokens].cpu()
    logits = inp["logits"][:sample_tokens].cpu()
    w13, w2 = inp["w13"].cpu(), inp["w2"].cpu()
    times = []
    for i in range(warmup + steps):
        t0 = time.perf_counter()
        moe_oracle.moe_block_ref(x, w13, w2, logits, wl.top_k, True, compute_dtype=dtype)
        if i >= warmup:
            times.append(time.perf_counter() - t0)
    mean = sum(times) / len(times)
    return sample_tokens / mean, mean


def run_reference(args, wl: MoEWorkload):
    rank, _, world = dist_env()
    if rank != 0:
        return
    cores = os.cpu_count() or 1
    sample = min(wl.num_tokens, args.cpu_sample_tokens)
    inp = make_inputs(wl.with_tokens(sample), device="cpu")
    tps, mean = cpu_block_tokens_per_s(wl, inp, sample, args.steps, max(args.warmup, 1),
                                       torch.bfloat16)
    sample_desc = (f"first {sample} of {wl.num_tokens} tokens of {wl.name}, bf16 torch CPU block, "
                   f"{cores} threads")
    line = {
        "impl": "reference", "metric": METRIC, "value": tps, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": max(args.warmup, 1), "ms_per_step": mean * 1e3,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic", "config": workload_config(wl, args, world),
        "cpu_baseline": {"value": tps, "unit": UNIT, "cores": cores, "cpu_model": cpu_model(),
                         "kind": "port", "sample": sample_desc},
        "e2e": {"value": tps, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def workload_config(wl: MoEWorkload, args, world: int) -> dict:
    par = "single" if world == 1 else f"{args.parallel}{world}"
    return {"workload": wl.name, "num_tokens": wl.num_tokens, "hidden": wl.hidden,
            "intermediate": wl.inter, "num_experts": wl.num_experts, "top_k": wl.top_k,
            "routing": "skewed ~4x" if wl.logit_bias else "near-uniform", "parallelism": par,
            "l2": "inputs larger than L2: every step streams the expert weights "
                  f"({(3 * wl.num_experts * wl.hidden * wl.inter * 2 / max(world, 1)) / 1e9:.2f} GB per GPU)"}


# --------------------------------------------------------------------------------------- our arm
def cpu_model() -> str:
    try:
        with open("/proc/cpuinfo") as f:
            for ln in f:
                if ln.lower().startswith("model name"):
                    return ln.split(":", 1)[1].strip()
    except OSError:
        pass
    return "unknown"


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", choices=["b200", "reference"], default="b200")
    ap.add_argument("--workload", default=None, choices=sorted(WORKLOADS))
    ap.add_argument("--parallel", choices=["tp", "tp_nccl", "ep", "ep_nccl"], default="ep",
                    help="N > 1: expert parallel over peer memory (ep) or NCCL all-to-alls "
                         "(ep_nccl), tensor parallel with the all-reduce inside the layer's "
                         "kernels (tp) or with NCCL's all-reduce (tp_nccl)")
    ap.add_argument("--cpu-sample-tokens", type=int, default=8192)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--graph", action="store_true",
                    help="replay each step of the device-resident measurement from a CUDA graph")
    ap.add_argument("--block-m", type=int, default=None, choices=[128, 256],
                    help="force the M tile of the grouped GEMMs (default: chosen by batch size)")
    ap.add_argument("--tokens", type=int, default=None,
                    help="override the workload's token count (profiling on a smaller case)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "b200" else args.warmup

    rank, local_rank, world = dist_env()
    name = args.workload or ("mixtral_prefill_t8192_skew" if max(world, args.gpus) == 1
                             else "mixtral_parallel_t16384")
    wl = WORKLOADS[name]
    if wl.dtype != torch.bfloat16:
        wl = MoEWorkload(wl.name, wl.num_tokens, wl.hidden, wl.inter, wl.num_experts, wl.top_k,
                         torch.bfloat16, wl.seed, wl.logit_bias)

    if args.tokens is not None:
        wl = MoEWorkload(f"{wl.name}@T={args.tokens}", args.tokens, wl.hidden, wl.inter,
                         wl.num_experts, wl.top_k, wl.dtype, wl.seed, wl.logit_bias)

    if args.impl == "reference":
        run_reference(args, wl)
        return

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU implementation to time; "
                         "use --impl reference for the CPU baseline)")
    import torch.distributed as dist
    from electrock_infer_b200 import _lib
    from electrock_infer_b200.layers.moe import FusedMoE
    from electrock_infer_b200.layers.moe import fused_moe as fm

    if args.block_m is not None:
        fm.FORCE_BLOCK_M = args.block_m
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        # NCCL prints its version banner on stdout when the communicator is created; send it to
        # stderr so that the JSON line is the only thing on stdout.
        sys.stdout.flush()
        saved_stdout = os.dup(1)
        os.dup2(2, 1)
        try:
            dist.init_process_group("nccl", device_id=dev)
            dist.barrier()
        finally:
            sys.stdout.flush()
            os.dup2(saved_stdout, 1)
            os.close(saved_stdout)
    if world > 1 and args.parallel in ("ep", "ep_nccl"):
        from electrock_infer_b200.parallel import ExpertParallelMoE
        layer_cls = ExpertParallelMoE
    else:
        layer_cls = None

    # ---- inputs (device generator: same distributions as the seeded CPU workload)
    T, H, I, E = wl.num_tokens, wl.hidden, wl.inter, wl.num_experts
    if layer_cls is None:
        shard = I // world
        inp = make_inputs(wl, device=dev, device_rng=True,
                          inter_slice=slice(rank * shard, (rank + 1) * shard) if world > 1 else None)
        layer = FusedMoE(E, wl.top_k, H, I, tp_size=world, params_dtype=torch.bfloat16,
                         reduce_results=True,
                         tp_exchange="nccl" if args.parallel == "tp_nccl" else "auto").to(dev)
        layer.w13_weight.data.copy_(inp["w13"])
        layer.w2_weight.data.copy_(inp["w2"])
        x0, logits = inp["x"], inp["logits"]
        step_tokens = T
    else:
        per = E // world
        inp = make_inputs(wl, device=dev, device_rng=True,
                          expert_slice=slice(rank * per, (rank + 1) * per))
        layer = layer_cls(E, wl.top_k, H, I, params_dtype=torch.bfloat16,
                          exchange="nccl" if args.parallel == "ep_nccl" else "auto").to(dev)
        layer.w13_weight.data.copy_(inp["w13"])
        layer.w2_weight.data.copy_(inp["w2"])
        t_loc = T // world
        x0 = inp["x"][rank * t_loc:(rank + 1) * t_loc].contiguous()
        logits = inp["logits"][rank * t_loc:(rank + 1) * t_loc].contiguous()
        step_tokens = T
    w13_cpu = w2_cpu = None
    x = torch.empty_like(x0)

    def eager_step():
        x.copy_(x0)  # the layer overwrites its input
        return layer(x, logits)

    step = eager_step

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(ms: float) -> float:
        if world == 1:
            return ms
        t = torch.tensor([ms], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    with torch.inference_mode():
        for _ in range(args.warmup):
            step()
        barrier()
        if args.graph and world == 1:
            cap = torch.cuda.Stream(dev)
            cap.wait_stream(torch.cuda.current_stream(dev))
            with torch.cuda.stream(cap):
                eager_step()  # the layer's scratch is kept per stream: create it before capturing
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=cap):
                eager_step()
            torch.cuda.current_stream(dev).wait_stream(cap)
            step = graph.replay
            for _ in range(3):
                step()
            barrier()
        status = _lib.load().b200moe_gemm_device_status(1)
        if status != 0:
            raise SystemExit(f"grouped GEMM reported device status {status:#x} during warm-up")

        # ---- device-resident throughput
        sampler = ClockSampler(local_rank)
        if rank == 0:
            sampler.start()
            time.sleep(0.3)
        launches0 = _lib.launch_count()
        barrier()
        wall0 = time.time()
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ev0.record()
        for _ in range(args.steps):
            step()
        ev1.record()
        barrier()
        wall1 = time.time()
        launches = _lib.launch_count() - launches0
        ms_total = max_over_ranks(ev0.elapsed_time(ev1))
        clocks = sampler.stop(wall0, wall1) if rank == 0 else None

        # ---- the same K steps again with a CUDA event pair around every kernel launch (on the
        # launching stream).  Kept out of the region above because an event between two launches
        # stops the second kernel's prologue from overlapping the first one's tail.
        fm.enable_kernel_timing(True)
        barrier()
        for _ in range(args.steps):
            eager_step()
        barrier()
        kernel_ms = fm.collect_kernel_timings()
        fm.enable_kernel_timing(False)

        # ---- end to end through host buffers: every step copies its inputs from pinned host
        # memory and copies its result back; copies and compute run on three streams with
        # E2E_BUFFERS device buffers, so step i+1's upload and step i-1's download overlap step i's
        # kernels.
        # Tensor parallel needs the same activations on every rank: each rank uploads 1/N of the
        # batch and the ranks all-gather over NVLink, and each rank downloads 1/N of the (replicated)
        # result.  Expert parallel is token-sharded to begin with.
        tp_split = layer_cls is None and world > 1
        t_loc = x0.shape[0] // world if tp_split else x0.shape[0]
        lo = rank * t_loc if tp_split else 0
        xh = x0[lo:lo + t_loc].cpu().pin_memory()
        lh = logits[lo:lo + t_loc].cpu().pin_memory()
        nbuf = E2E_BUFFERS
        oh = [torch.empty_like(xh).pin_memory() for _ in range(nbuf)]
        xd = [torch.empty_like(x0) for _ in range(nbuf)]
        ld = [torch.empty_like(logits) for _ in range(nbuf)]
        xs = [torch.empty_like(x0[:t_loc]) for _ in range(nbuf)] if tp_split else xd
        ls = [torch.empty_like(logits[:t_loc]) for _ in range(nbuf)] if tp_split else ld
        s_in, s_c, s_out = (torch.cuda.Stream(dev) for _ in range(3))
        ev_in = [torch.cuda.Event() for _ in range(nbuf)]
        ev_done = [torch.cuda.Event() for _ in range(nbuf)]
        ev_out = [torch.cuda.Event() for _ in range(nbuf)]

        def e2e_run(n):
            main = torch.cuda.current_stream(dev)
            for st in (s_in, s_c, s_out):
                st.wait_stream(main)
            for i in range(n):
                b = i % nbuf
                with torch.cuda.stream(s_in):
                    s_in.wait_event(ev_out[b])   # the result that aliases xd[b] has been downloaded
                    xs[b].copy_(xh, non_blocking=True)
                    ls[b].copy_(lh, non_blocking=True)
                    if tp_split:
                        dist.all_gather_into_tensor(xd[b], xs[b])
                        dist.all_gather_into_tensor(ld[b], ls[b])
                    ev_in[b].record(s_in)
                with torch.cuda.stream(s_c):
                    s_c.wait_event(ev_in[b])
                    out = layer(xd[b], ld[b])
                    ev_done[b].record(s_c)
                with torch.cuda.stream(s_out):
                    s_out.wait_event(ev_done[b])
                    oh[b].copy_(out[lo:lo + t_loc], non_blocking=True)
                    ev_out[b].record(s_out)
            for st in (s_in, s_c, s_out):
                main.wait_stream(st)

        e2e_run(3)
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        e2e_run(args.steps)
        e1.record()
        barrier()
        e2e_ms = max_over_ranks(e0.elapsed_time(e1))

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    peaks = load_peaks()
    ms_per_step = ms_total / args.steps
    value = step_tokens / (ms_per_step * 1e-3)
    e2e_value = step_tokens / (e2e_ms / args.steps * 1e-3)

    # Dominant kernel: grouped GEMM w13 + SwiGLU, 4*H*I'*top_k FLOP per token on this GPU.
    i_local = I // world if layer_cls is None else I
    tokens_local = T if layer_cls is None else T // world  # EP: pairs land where the experts are
    w13_flops = 4 * H * i_local * wl.top_k * tokens_local
    w2_flops = 2 * H * i_local * wl.top_k * tokens_local
    k13 = kernel_ms.get("grouped_gemm_w13_swiglu")
    k2 = kernel_ms.get("grouped_gemm_w2_scale")
    # The kernel is tensor-bound when its FLOPs take longer at the tensor peak than streaming its
    # weights once takes at the HBM peak, and HBM-bound (weight streaming) otherwise.
    experts_local = E if layer_cls is None else E // world
    w13_bytes = experts_local * 2 * i_local * H * 2 + tokens_local * wl.top_k * (H + i_local) * 2
    tensor_floor = w13_flops / (peaks["bf16_tflops_sustained"] * 1e12)
    hbm_floor = w13_bytes / (peaks["hbm_gbs"] * 1e9)
    if tensor_floor >= hbm_floor:
        peak = peaks["bf16_tflops_sustained"]
        roofline = {"bound": "tensor", "kernel": "grouped_gemm_w13_swiglu", "achieved": None,
                    "peak": peak, "unit": "TFLOP/s", "frac": None, "traffic": None,
                    "peak_source": f"{peaks['source']} sustained bf16 matmul (kernel timed inside "
                                   "a long step)"}
        if k13:
            ach = w13_flops / (k13 * 1e-3) / 1e12
            roofline.update(achieved=ach, frac=ach / peak, ms_per_launch=k13,
                            frac_of_burst=ach / peaks["bf16_tflops"])
        roofline.update(traffic=NCU_TRAFFIC_RATIO * w13_bytes, traffic_source=NCU_TRAFFIC_NOTE)
    else:
        peak = peaks["hbm_gbs"]
        roofline = {"bound": "hbm", "kernel": "grouped_gemm_w13_swiglu", "achieved": None,
                    "peak": peak, "unit": "GB/s", "frac": None, "traffic": None,
                    "peak_source": f"{peaks['source']} device copy bandwidth",
                    "algorithmic_bytes": w13_bytes}
        if k13:
            ach = w13_bytes / (k13 * 1e-3) / 1e9
            roofline.update(achieved=ach, frac=ach / peak, ms_per_launch=k13)
        roofline.update(traffic=NCU_TRAFFIC_RATIO * w13_bytes, traffic_source=NCU_TRAFFIC_NOTE)
    kernels = {k: round(v, 4) for k, v in kernel_ms.items()}
    extra = {}
    if k2:
        extra["grouped_gemm_w2_scale_tflops"] = w2_flops / (k2 * 1e-3) / 1e12
    if k13 and k2:
        extra["grouped_gemms_tflops"] = (w13_flops + w2_flops) / ((k13 + k2) * 1e-3) / 1e12
    comb = kernel_ms.get("moe_sum")
    if comb:
        extra["moe_sum_gbs"] = tokens_local * H * 2 * 3 / (comb * 1e-3) / 1e9
        extra["moe_sum_frac_of_hbm"] = extra["moe_sum_gbs"] / peaks["hbm_gbs"]

    cpu_baseline = None
    if world == 1 and not args.no_cpu_baseline:
        sample = min(T, args.cpu_sample_tokens)
        cores = os.cpu_count() or 1
        tps, mean = cpu_block_tokens_per_s(wl, inp, sample, 5, 1, torch.bfloat16)
        cpu_baseline = {"value": tps, "unit": UNIT, "cores": cores, "cpu_model": cpu_model(),
                        "kind": "port",
                        "sample": f"first {sample} of {T} tokens of {wl.name}, bf16 torch CPU block, "
                                  f"1 warm-up + 5 timed passes ({mean:.2f} s each)"}

    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": workload_config(wl, args, world),
        "e2e": {"value": e2e_value, "unit": UNIT,
                "h2d_bytes_per_step": (xh.numel() * 2 + lh.numel() * 4) * world,
                "d2h_bytes_per_step": oh[0].numel() * 2 * world,
                "overlap": f"3 streams, {E2E_BUFFERS} device buffers: uploads/downloads overlap the kernels"},
        "gpu_launches": launches,
        "roofline": roofline,
        "cpu_baseline": cpu_baseline,
        "clocks": clocks,
        "kernel_ms": kernels,
        "block_m": fm.choose_block_m(tokens_local, wl.top_k, E),
        "cuda_graph": bool(args.graph and world == 1),
        "layer_tflops": wl.flops / max(world, 1) / (ms_per_step * 1e-3) / 1e12 if layer_cls is None
        else wl.flops / world / (ms_per_step * 1e-3) / 1e12,
        **extra,
    }
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
