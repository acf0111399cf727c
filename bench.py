"""MoE-layer throughput benchmark: tokens/s of ``FusedMoE.forward`` at Mixtral-8x7B shape.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--parallel ep|ep_nccl|tp|tp_nccl]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...
    python bench.py --impl reference ...      # the reference's torch CPU path on the host cores

One step is one pass of the layer over one batch of seeded synthetic tokens.  At one GPU the
workload is the prefill-sized, skew-routed Mixtral layer (T=8192); at N > 1 it is the T=16384 step
sharded expert-parallel (the headline numbers) and, in the same run, tensor-parallel as the
reference does (reported under "tp"); --parallel picks one mode only (tp_nccl keeps the
reference's NCCL all-reduce, ep_nccl NCCL all-to-alls).  Rank 0 prints ONE JSON line:

  value         tokens/s with inputs resident in HBM (CUDA events around K steps, max over ranks)
  e2e           the same through host buffers: pinned H2D of activations and logits and D2H of the
                result inside the timed region, every step
  roofline      the dominant kernel (grouped GEMM w13 + SwiGLU): algorithmic FLOPs per launch over
                its mean launch time, measured with CUDA events inside the timed region
  cpu_baseline  the oracle's torch CPU block timed on this host on a bounded token sample
  clocks        SM clock and throttle reasons sampled with nvidia-smi during the timed region
  parity        outside every timed region: 64 sampled tokens of one more step's output on rank 0
                against the CPU oracle (fp32 arithmetic on the same bf16 tensors); the run exits
                non-zero when the layer tolerance (max-abs 3e-2, relative Frobenius 1e-2) fails
  gpu_reference (one GPU only) the reference's own Triton pipeline with its CUDA ops, JIT-compiled
                for this GPU and run in a child process on the same workload: tokens/s and error
                against the same oracle sample (absent where the reference was never staged)
  same_workload_n1  (one GPU only) the T=16384 workload of the N > 1 runs timed on this one GPU,
                so that the 1 -> N curve can be read on one workload
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
from dataclasses import replace
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

from electrock_infer_b200.synthetic import WORKLOADS, MoEWorkload, make_inputs  # noqa: E402

METRIC = "moe_layer_tokens_per_s"
UNIT = "tokens/s"
# DRAM traffic (ncu: dram__bytes_read.sum + dram__bytes_write.sum) over algorithmic bytes, per
# grouped-GEMM kernel, from one captured launch of each on the benchmark workload itself (T=8192,
# skewed routing, both GEMMs with two M blocks per tile): first GEMM 3.263 GB against 2.483 GB,
# second GEMM 3.232 GB against 1.544 GB.  The second GEMM streams an expert's weights once per
# L2-sized group of A rows by design (17 passes over 117 MB for this routing); the first GEMM
# re-reads weight tiles where CTAs working on one tile drift apart and for the second group of
# the 50-block expert.  Other token counts are scaled by the same ratio.
NCU_TRAFFIC_RATIO = {"grouped_gemm_w13_swiglu": 1.314, "grouped_gemm_w2_scale": 2.094}
NCU_TRAFFIC_NOTE = ("algorithmic bytes x the ncu DRAM read+write / algorithmic ratio of a captured "
                    "launch of the same kernel on mixtral_prefill_t8192_skew")
PARITY_TOKENS = 64
PARITY_MAX_ABS, PARITY_REL_FRO = 3e-2, 1e-2
# Device buffers of the end-to-end pipeline: step i+3's upload waits for step i's download (the
# layer writes its result over its input), so three buffers let upload, kernels and download of
# neighbouring steps all overlap.
E2E_BUFFERS = 3
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
                 "-i", str(self.gpu_index), "-lms", "25"],
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


class Bench:
    """One process of the GPU arm: the process group, the device and the helpers that every
    measured mode shares."""

    def __init__(self, args):
        import torch.distributed as dist
        self.args = args
        self.dist = dist
        self.rank, self.local_rank, self.world = dist_env()
        torch.cuda.set_device(self.local_rank)
        self.dev = torch.device("cuda", self.local_rank)
        if self.world > 1:
            # NCCL prints its version banner on stdout when the communicator is created; send it
            # to stderr so that the JSON line is the only thing on stdout.
            sys.stdout.flush()
            saved_stdout = os.dup(1)
            os.dup2(2, 1)
            try:
                dist.init_process_group("nccl", device_id=self.dev)
                dist.barrier()
            finally:
                sys.stdout.flush()
                os.dup2(saved_stdout, 1)
                os.close(saved_stdout)

    def barrier(self):
        if self.world > 1:
            self.dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(self, v: float) -> float:
        if self.world == 1:
            return v
        t = torch.tensor([v], dtype=torch.float64, device=self.dev)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return float(t.item())

    def close(self):
        if self.world > 1:
            self.dist.destroy_process_group()


def build_layer(b: Bench, mode: str, wl: MoEWorkload):
    """The layer of one parallel mode with this rank's shard of the seeded weights, and this
    rank's tokens.  Every rank draws the same values on its own device (same generator, same
    seed), so shards, tokens and the full weights used by the parity check all agree."""
    from electrock_infer_b200.layers.moe import FusedMoE
    rank, world, dev = b.rank, b.world, b.dev
    T, H, I, E = wl.num_tokens, wl.hidden, wl.inter, wl.num_experts
    if mode in ("ep", "ep_nccl"):
        from electrock_infer_b200.parallel import ExpertParallelMoE
        per = E // world
        inp = make_inputs(wl, device=dev, device_rng=True,
                          expert_slice=slice(rank * per, (rank + 1) * per))
        t_loc = T // world
        layer = ExpertParallelMoE(E, wl.top_k, H, I, params_dtype=torch.bfloat16,
                                  exchange="nccl" if mode == "ep_nccl" else "auto",
                                  max_tokens_per_rank=None if mode == "ep_nccl" else t_loc).to(dev)
        lo = rank * t_loc
        x0 = inp["x"][lo:lo + t_loc].contiguous()
        logits = inp["logits"][lo:lo + t_loc].contiguous()
    else:  # "single", "tp", "tp_nccl"
        shard = I // world
        inp = make_inputs(wl, device=dev, device_rng=True,
                          inter_slice=slice(rank * shard, (rank + 1) * shard) if world > 1 else None)
        layer = FusedMoE(E, wl.top_k, H, I, tp_size=world, params_dtype=torch.bfloat16,
                         reduce_results=True,
                         tp_exchange="nccl" if mode == "tp_nccl" else "auto").to(dev)
        lo = 0
        x0, logits = inp["x"], inp["logits"]
    layer.w13_weight.data.copy_(inp["w13"])
    layer.w2_weight.data.copy_(inp["w2"])
    full = inp if world == 1 else None
    del inp
    return layer, x0, logits, lo, full


def parity_check(b: Bench, mode: str, wl: MoEWorkload, layer, x0, logits, full) -> dict:
    """One more step, untimed, whose output rows for PARITY_TOKENS sampled tokens of rank 0 are
    compared with the CPU oracle (fp32 arithmetic on the same bf16-valued tensors)."""
    from oracle import moe_oracle
    x = x0.clone()
    out = layer(x, logits)
    b.barrier()
    if b.rank != 0:
        return {}
    if full is None:  # sharded run: draw the whole layer's weights again (same seed, same values)
        full = make_inputs(wl, device=b.dev, device_rng=True)
    n = min(PARITY_TOKENS, x0.shape[0])
    sample = torch.randperm(x0.shape[0], generator=torch.Generator().manual_seed(0))[:n].to(b.dev)
    want = moe_oracle.moe_block_ref(x0[sample], full["w13"], full["w2"], logits[sample], wl.top_k, True)
    st = moe_oracle.error_stats(out[sample].float().cpu(), want)
    ok = st["max_abs"] <= PARITY_MAX_ABS and st["rel_fro"] <= PARITY_REL_FRO
    return {"max_abs": st["max_abs"], "rel_fro": st["rel_fro"], "tokens": n, "ok": bool(ok),
            "against": "CPU oracle, fp32 arithmetic on the same bf16 tensors",
            "tolerance": {"max_abs": PARITY_MAX_ABS, "rel_fro": PARITY_REL_FRO}}


def run_mode(b: Bench, mode: str, wl: MoEWorkload, steps: int, warmup: int, e2e: bool = True,
             graph: bool = False) -> dict:
    """Warm-up, the device-resident timed region, the per-kernel timing pass, the end-to-end timed
    region through host buffers and the parity check of one parallel mode.  Collective: every
    rank calls it; the returned numbers are the maxima over the ranks."""
    from electrock_infer_b200 import _lib
    from electrock_infer_b200.layers.moe import fused_moe as fm
    dist, rank, world, dev = b.dist, b.rank, b.world, b.dev
    layer, x0, logits, lo, full = build_layer(b, mode, wl)
    x = torch.empty_like(x0)

    def eager_step():
        x.copy_(x0)  # the layer overwrites its input
        return layer(x, logits)

    step = eager_step
    res = {"mode": mode}
    with torch.inference_mode():
        for _ in range(warmup):
            step()
        b.barrier()
        if graph and world == 1:
            cap = torch.cuda.Stream(dev)
            cap.wait_stream(torch.cuda.current_stream(dev))
            with torch.cuda.stream(cap):
                eager_step()  # the layer's scratch is kept per stream: create it before capturing
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=cap):
                eager_step()
            torch.cuda.current_stream(dev).wait_stream(cap)
            step = g.replay
            for _ in range(3):
                step()
            b.barrier()
        status = _lib.load().b200moe_gemm_device_status(1)
        if status != 0:
            raise SystemExit(f"grouped GEMM reported device status {status:#x} during warm-up")

        # ---- device-resident throughput
        sampler = ClockSampler(b.local_rank)
        if rank == 0:
            sampler.start()
            time.sleep(0.3)
        launches0 = _lib.launch_count()
        b.barrier()
        wall0 = time.time()
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ev0.record()
        for _ in range(steps):
            step()
        ev1.record()
        b.barrier()
        wall1 = time.time()
        res["launches"] = _lib.launch_count() - launches0
        res["ms_per_step"] = b.max_over_ranks(ev0.elapsed_time(ev1)) / steps
        res["clocks"] = sampler.stop(wall0, wall1) if rank == 0 else None

        # ---- the same K steps again with a CUDA event pair around every kernel launch (on the
        # launching stream).  Kept out of the region above because an event between two launches
        # stops the second kernel's prologue from overlapping the first one's tail.
        fm.enable_kernel_timing(True)
        b.barrier()
        for _ in range(steps):
            eager_step()
        b.barrier()
        res["kernel_ms"] = fm.collect_kernel_timings()
        fm.enable_kernel_timing(False)

        if e2e:
            res["e2e"] = run_e2e(b, mode, layer, x0, logits, steps)
        res["parity"] = parity_check(b, mode, wl, layer, x0, logits, full)

    b.barrier()
    if hasattr(layer, "close"):
        layer.close()                      # expert parallel: peer-visible buffers
    elif getattr(layer, "_tp_reduce", None) is not None:
        layer._tp_reduce.close()           # tensor parallel with the in-kernel reduce
    del layer, x0, logits, x, full
    torch.cuda.empty_cache()
    return res


def run_e2e(b: Bench, mode: str, layer, x0, logits, steps: int) -> dict:
    """End to end through host buffers: every step copies its inputs from pinned host memory and
    copies its result back; copies and compute run on three streams with E2E_BUFFERS device
    buffers, so step i+1's upload and step i-1's download overlap step i's kernels.
    Tensor parallel needs the same activations on every rank: each rank uploads 1/N of the batch
    and the ranks all-gather over NVLink, and each rank downloads 1/N of the (replicated) result.
    Expert parallel is token-sharded to begin with."""
    dist, rank, world, dev = b.dist, b.rank, b.world, b.dev
    tp_split = mode in ("tp", "tp_nccl") and world > 1
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
    # Event pairs around the copies of one step in the middle of the run (bandwidth actually seen).
    probe = {"h2d": (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)),
             "d2h": (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))}

    def run(n, probe_at=-1):
        main = torch.cuda.current_stream(dev)
        for st in (s_in, s_c, s_out):
            st.wait_stream(main)
        for i in range(n):
            k = i % nbuf
            with torch.cuda.stream(s_in):
                s_in.wait_event(ev_out[k])   # the result that aliases xd[k] has been downloaded
                if i == probe_at:
                    probe["h2d"][0].record(s_in)
                xs[k].copy_(xh, non_blocking=True)
                ls[k].copy_(lh, non_blocking=True)
                if i == probe_at:
                    probe["h2d"][1].record(s_in)
                if tp_split:
                    dist.all_gather_into_tensor(xd[k], xs[k])
                    dist.all_gather_into_tensor(ld[k], ls[k])
                ev_in[k].record(s_in)
            with torch.cuda.stream(s_c):
                s_c.wait_event(ev_in[k])
                out = layer(xd[k], ld[k])
                ev_done[k].record(s_c)
            with torch.cuda.stream(s_out):
                s_out.wait_event(ev_done[k])
                if i == probe_at:
                    probe["d2h"][0].record(s_out)
                oh[k].copy_(out[lo:lo + t_loc], non_blocking=True)
                if i == probe_at:
                    probe["d2h"][1].record(s_out)
                ev_out[k].record(s_out)
        host_done = time.perf_counter()
        for st in (s_in, s_c, s_out):
            main.wait_stream(st)
        return host_done

    run(3)
    b.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    host0 = time.perf_counter()
    host1 = run(steps, probe_at=steps // 2)
    e1.record()
    b.barrier()
    ms = b.max_over_ranks(e0.elapsed_time(e1)) / steps
    host_ms = b.max_over_ranks((host1 - host0) * 1e3) / steps
    h2d_bytes = xh.numel() * 2 + lh.numel() * 4
    d2h_bytes = oh[0].numel() * 2
    h2d_ms = b.max_over_ranks(probe["h2d"][0].elapsed_time(probe["h2d"][1]))
    d2h_ms = b.max_over_ranks(probe["d2h"][0].elapsed_time(probe["d2h"][1]))
    return {"ms_per_step": ms, "h2d_bytes_per_step": h2d_bytes * world,
            "d2h_bytes_per_step": d2h_bytes * world,
            # Time the Python loop needs to issue one step (launches are asynchronous): when it is
            # close to ms_per_step the host, not the GPU or the copies, sets the pace.
            "host_issue_ms_per_step": host_ms,
            "h2d_gbs_per_rank": h2d_bytes / (h2d_ms * 1e-3) / 1e9 if h2d_ms > 0 else None,
            "d2h_gbs_per_rank": d2h_bytes / (d2h_ms * 1e-3) / 1e9 if d2h_ms > 0 else None,
            "overlap": f"3 streams, {E2E_BUFFERS} device buffers: uploads/downloads overlap the kernels"}


def gpu_reference(wl: MoEWorkload, steps: int) -> dict:
    """The reference's own GPU pipeline (its Triton grouped GEMM compiled for this GPU plus its CUDA
    ops, staged under oracle/_ref where the reference tree was available) timed on the same
    workload in a child process: a second baseline beside the CPU one, and the yardstick for the
    error of this library.  Never on the product path; absent or failing, it is reported as such."""
    script = ROOT / "oracle" / "gpu_reference.py"
    if not (ROOT / "oracle" / "_ref" / "reference_python").is_dir():
        return {"unavailable": "the reference's Python package is not staged under oracle/_ref"}
    try:
        proc = subprocess.run([sys.executable, str(script), "--workload", wl.name, "--steps",
                               str(steps)], capture_output=True, text=True, timeout=600)
        lines = [ln for ln in proc.stdout.splitlines() if ln.startswith("{")]
        return json.loads(lines[-1]) if lines else {
            "unavailable": f"exit {proc.returncode}: {proc.stderr.strip()[-300:]}"}
    except (subprocess.TimeoutExpired, ValueError, OSError) as e:
        return {"unavailable": f"{type(e).__name__}: {str(e)[:200]}"}


def gemm_roofline(wl: MoEWorkload, mode: str, world: int, kernel_ms: dict, peaks: dict):
    """Roofline of the dominant kernel (grouped GEMM w13 + SwiGLU: 4*H*I'*top_k FLOP per token on
    this GPU) from its mean event-timed launch, plus the figures of the second GEMM and of the
    combine kernel."""
    T, H, I, E = wl.num_tokens, wl.hidden, wl.inter, wl.num_experts
    tp_like = mode in ("single", "tp", "tp_nccl")
    i_local = I // world if tp_like else I
    tokens_local = T if tp_like else T // world  # EP: pairs land where the experts are
    experts_local = E if tp_like else E // world
    w13_flops = 4 * H * i_local * wl.top_k * tokens_local
    w2_flops = 2 * H * i_local * wl.top_k * tokens_local
    k13 = kernel_ms.get("grouped_gemm_w13_swiglu")
    k2 = kernel_ms.get("grouped_gemm_w2_scale")
    pairs = tokens_local * wl.top_k
    w13_bytes = experts_local * 2 * i_local * H * 2 + pairs * (H + i_local) * 2
    w2_bytes = experts_local * i_local * H * 2 + pairs * (H + i_local) * 2
    # Tensor-bound when the FLOPs take longer at the tensor peak than streaming the weights once
    # takes at the HBM peak, HBM-bound (weight streaming) otherwise.
    tensor_floor = w13_flops / (peaks["bf16_tflops"] * 1e12)
    hbm_floor = w13_bytes / (peaks["hbm_gbs"] * 1e9)
    traffic = NCU_TRAFFIC_RATIO["grouped_gemm_w13_swiglu"] * w13_bytes
    if tensor_floor >= hbm_floor:
        roof = {"bound": "tensor", "kernel": "grouped_gemm_w13_swiglu", "achieved": None,
                "peak": peaks["bf16_tflops"], "unit": "TFLOP/s", "frac": None, "traffic": traffic,
                "peak_source": f"{peaks['source']} burst bf16 matmul (cuBLAS, best of 10)"}
        if k13:
            ach = w13_flops / (k13 * 1e-3) / 1e12
            roof.update(achieved=ach, frac=ach / peaks["bf16_tflops"], ms_per_launch=k13,
                        frac_of_sustained=ach / peaks["bf16_tflops_sustained"],
                        sustained_peak=peaks["bf16_tflops_sustained"])
    else:
        roof = {"bound": "hbm", "kernel": "grouped_gemm_w13_swiglu", "achieved": None,
                "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": None, "traffic": traffic,
                "peak_source": f"{peaks['source']} device copy bandwidth",
                "algorithmic_bytes": w13_bytes}
        if k13:
            ach = w13_bytes / (k13 * 1e-3) / 1e9
            roof.update(achieved=ach, frac=ach / peaks["hbm_gbs"], ms_per_launch=k13)
    roof["traffic_source"] = NCU_TRAFFIC_NOTE
    roof["traffic_ratio"] = dict(NCU_TRAFFIC_RATIO)
    if roof["frac"] is not None and roof["frac"] > 1.0:
        roof["note"] = "fraction above 1: the peak was measured at another clock/power state"
    extra = {}
    if k2:
        extra["grouped_gemm_w2_scale_tflops"] = w2_flops / (k2 * 1e-3) / 1e12
        extra["grouped_gemm_w2_scale_frac_of_burst"] = extra["grouped_gemm_w2_scale_tflops"] / peaks["bf16_tflops"]
        extra["grouped_gemm_w2_scale_traffic"] = NCU_TRAFFIC_RATIO["grouped_gemm_w2_scale"] * w2_bytes
    if k13 and k2:
        extra["grouped_gemms_tflops"] = (w13_flops + w2_flops) / ((k13 + k2) * 1e-3) / 1e12
    comb = kernel_ms.get("moe_sum")
    if comb:
        sum_tokens = T if tp_like else T // world
        extra["moe_sum_gbs"] = sum_tokens * H * 2 * 3 / (comb * 1e-3) / 1e9
        extra["moe_sum_frac_of_hbm"] = extra["moe_sum_gbs"] / peaks["hbm_gbs"]
    return roof, extra


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", choices=["b200", "reference"], default="b200")
    ap.add_argument("--workload", default=None, choices=sorted(WORKLOADS))
    ap.add_argument("--parallel", choices=["tp", "tp_nccl", "ep", "ep_nccl"], default=None,
                    help="N > 1: measure only this mode: expert parallel over peer memory (ep) or "
                         "NCCL all-to-alls (ep_nccl), tensor parallel with the all-reduce inside the "
                         "layer's kernels (tp) or with NCCL's all-reduce (tp_nccl).  Default: ep as "
                         "the headline and tp beside it")
    ap.add_argument("--cpu-sample-tokens", type=int, default=8192)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extras", action="store_true",
                    help="skip the second measurements (tensor parallel beside expert parallel at "
                         "N > 1, the T=16384 workload at N = 1): profiling runs")
    ap.add_argument("--graph", action="store_true",
                    help="replay each step of the device-resident measurement from a CUDA graph")
    ap.add_argument("--block-m", type=int, default=None, choices=[128, 256],
                    help="force the M tile of the grouped GEMMs (default: chosen by batch size)")
    ap.add_argument("--tiling", type=int, default=0, choices=[0, 1, 2],
                    help="force one (1) or two (2) M blocks per tile of the one-CTA grouped GEMMs")
    ap.add_argument("--tokens", type=int, default=None,
                    help="override the workload's token count (profiling on a smaller case)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "b200" else args.warmup

    rank, local_rank, world = dist_env()
    name = args.workload or ("mixtral_prefill_t8192_skew" if max(world, args.gpus) == 1
                             else "mixtral_parallel_t16384")
    wl = replace(WORKLOADS[name], dtype=torch.bfloat16) if WORKLOADS[name].dtype != torch.bfloat16 \
        else WORKLOADS[name]
    if args.tokens is not None:
        wl = replace(wl, name=f"{wl.name}@T={args.tokens}", num_tokens=args.tokens)

    if args.impl == "reference":
        run_reference(args, wl)
        return

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU implementation to time; "
                         "use --impl reference for the CPU baseline)")
    from electrock_infer_b200 import _lib
    from electrock_infer_b200.layers.moe import fused_moe as fm

    if args.block_m is not None:
        fm.FORCE_BLOCK_M = args.block_m
    _lib.check(_lib.load().b200moe_gemm_set_tiling(args.tiling), "gemm_set_tiling")
    b = Bench(args)
    headline = "single" if world == 1 else (args.parallel or "ep")
    args.parallel = headline
    main_res = run_mode(b, headline, wl, args.steps, args.warmup, e2e=True, graph=args.graph)

    # ---- second measurements, outside the headline's timed regions
    tp_res = same_n1 = None
    extras = not args.no_extras and args.tokens is None and args.workload is None
    if extras and world > 1 and headline == "ep":
        tp_res = run_mode(b, "tp", wl, args.steps, args.warmup, e2e=True)
    if extras and world == 1:
        wl_par = WORKLOADS["mixtral_parallel_t16384"]
        r = run_mode(b, "single", wl_par, max(3, min(args.steps, 10)), 3, e2e=False)
        same_n1 = {"workload": wl_par.name, "value": wl_par.num_tokens / (r["ms_per_step"] * 1e-3),
                   "unit": UNIT, "ms_per_step": r["ms_per_step"],
                   "kernel_ms": {k: round(v, 4) for k, v in r["kernel_ms"].items()},
                   "parity": r["parity"]}

    if rank != 0:
        b.close()
        return

    gpu_ref = gpu_reference(wl, 5) if extras and world == 1 else None
    peaks = load_peaks()
    T = wl.num_tokens
    roofline, extra = gemm_roofline(wl, headline, world, main_res["kernel_ms"], peaks)
    e2e = main_res["e2e"]

    cpu_baseline = None
    if world == 1 and not args.no_cpu_baseline:
        sample = min(T, args.cpu_sample_tokens)
        cores = os.cpu_count() or 1
        inp = make_inputs(wl.with_tokens(sample), device=b.dev, device_rng=True)  # copied to the host below
        tps, mean = cpu_block_tokens_per_s(wl, inp, sample, 5, 1, torch.bfloat16)
        cpu_baseline = {"value": tps, "unit": UNIT, "cores": cores, "cpu_model": cpu_model(),
                        "kind": "port",
                        "sample": f"first {sample} of {T} tokens of {wl.name}, bf16 torch CPU block, "
                                  f"1 warm-up + 5 timed passes ({mean:.2f} s each)"}

    def e2e_block(r):
        e = dict(r["e2e"])
        e["value"] = T / (e["ms_per_step"] * 1e-3)
        e["unit"] = UNIT
        return e

    line = {
        "metric": METRIC, "value": T / (main_res["ms_per_step"] * 1e-3), "unit": UNIT,
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": main_res["ms_per_step"], "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": workload_config(wl, args, world),
        "e2e": e2e_block(main_res),
        "gpu_launches": main_res["launches"],
        "roofline": roofline,
        "cpu_baseline": cpu_baseline,
        "clocks": main_res["clocks"],
        "parity": main_res["parity"],
        "kernel_ms": {k: round(v, 4) for k, v in main_res["kernel_ms"].items()},
        "block_m": fm.choose_block_m(T, wl.top_k, wl.num_experts),
        "cuda_graph": bool(args.graph and world == 1),
        "layer_tflops": wl.flops / world / (main_res["ms_per_step"] * 1e-3) / 1e12,
        **extra,
    }
    if tp_res is not None:
        tp_roof, tp_extra = gemm_roofline(wl, "tp", world, tp_res["kernel_ms"], peaks)
        line["tp"] = {"parallelism": f"tp{world}, all-reduce inside the layer's kernels",
                      "value": T / (tp_res["ms_per_step"] * 1e-3), "unit": UNIT,
                      "ms_per_step": tp_res["ms_per_step"], "e2e": e2e_block(tp_res),
                      "kernel_ms": {k: round(v, 4) for k, v in tp_res["kernel_ms"].items()},
                      "gpu_launches": tp_res["launches"], "roofline": tp_roof,
                      "parity": tp_res["parity"], "clocks": tp_res["clocks"]}
    if same_n1 is not None:
        line["same_workload_n1"] = same_n1
    if gpu_ref is not None:
        if "rel_fro" in gpu_ref and main_res["parity"]:
            # Same sample, same oracle: this library's error relative to the reference pipeline's.
            gpu_ref["our_rel_fro_over_reference"] = main_res["parity"]["rel_fro"] / max(gpu_ref["rel_fro"], 1e-30)
        line["gpu_reference"] = gpu_ref
    print(json.dumps(line), flush=True)
    b.close()
    failed = [k for k, p in (("headline", main_res["parity"]),
                             ("tp", tp_res["parity"] if tp_res else None),
                             ("same_workload_n1", same_n1["parity"] if same_n1 else None))
              if p and not p.get("ok", False)]
    if failed:
        raise SystemExit(f"parity check failed for: {', '.join(failed)}")


if __name__ == "__main__":
    main()
