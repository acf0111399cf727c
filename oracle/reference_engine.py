"""End-to-end generation with the reference's own engine and this library's MoE layer: random-init
Mixtral-8x7B, tensor parallel, the workload of the reference's bench.py (:9-32).
TEST INFRASTRUCTURE / MEASUREMENT ONLY: nothing here is part of the product path.

    python oracle/reference_engine.py --tp 2 [--layers 32] [--requests 100] [--moe ours|reference]

The engine (scheduler, block manager, model runner, attention, sampler: electrock_infer/engine,
models/mixtral.py) is the staged, unmodified copy under ``oracle/_ref/reference_python``
(``oracle/stage_reference_python.py``); ``electrock_infer_b200.install_into_reference()`` puts this
library's ``FusedMoE`` and ``_C`` into it.  What has to be supplied around it, because the
reference expects a model directory with weights and a tokenizer:

  * a synthetic ``config.json`` (32 layers, hidden 4096, 32 query / 8 KV heads, vocab 32000,
    RMSNorm eps 1e-5; ``rope_theta`` 1e6 is set on the loaded config object because the installed
    transformers keeps it elsewhere and the reference reads ``hf_config.rope_theta``);
  * weights: the reference's ``load_model`` (utils/loader.py:20-58) finds no safetensors files, so
    it is replaced by a seeded normal initialisation of every parameter on the device;
  * the tokenizer: prompts are token ids already; a stand-in supplies ``eos_token_id``/``decode``;
  * the paged KV block size of 256: both ``Config.kvcache_block_size`` and the class constant
    ``Sequence.block_size`` (engine/sequence.py:15) are set.

The reference starts one process per extra rank with the ``spawn`` method; a spawned child runs
this file's top level (as ``__mp_main__``) before it unpickles its arguments, which is where
``prepare()`` installs all of the above in every rank.

Prints one JSON object: output tokens/s over the timed ``generate`` call, and the share of the
GPU time of rank 0 spent inside ``FusedMoE.forward`` (CUDA events around every call).
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import tempfile
import time
from pathlib import Path
from random import Random

HERE = Path(__file__).resolve().parent
REPO = HERE.parent
STAGED = HERE / "_ref" / "reference_python"
KV_BLOCK = 256
MODEL = {"architectures": ["MixtralForCausalLM"], "model_type": "mixtral", "hidden_size": 4096,
         "intermediate_size": 14336, "num_hidden_layers": 32, "num_attention_heads": 32,
         "num_key_value_heads": 8, "vocab_size": 32000, "rms_norm_eps": 1e-5,
         "num_local_experts": 8, "num_experts_per_tok": 2, "max_position_embeddings": 32768,
         "torch_dtype": "bfloat16", "tie_word_embeddings": False, "hidden_act": "silu"}
ROPE_THETA = 1e6
_moe_events: list = []


class _Tokenizer:
    eos_token_id = 2

    def encode(self, text):
        return [1] + [3 + (ord(c) % 1000) for c in text]

    def decode(self, token_ids):
        return " ".join(map(str, token_ids))


def prepare() -> bool:
    """Everything every rank process needs before the reference's engine runs.  False when the
    reference package has not been staged."""
    if not (STAGED / "electrock_infer").is_dir():
        return False
    sys.dont_write_bytecode = True
    for p in (str(REPO), str(STAGED)):
        if p not in sys.path:
            sys.path.insert(0, p)
    use_ours = os.environ.get("B200MOE_ENGINE_MOE", "ours") == "ours"
    import torch
    import torch.distributed as dist

    import electrock_infer_b200
    if use_ours:
        electrock_infer_b200.install_into_reference()
    else:  # the reference's own Triton layer with its CUDA ops, as a second arm
        import importlib.util
        ops = sorted((HERE / "_ref").glob("ref_ops*.so"))
        spec = importlib.util.spec_from_file_location("ref_ops", ops[0])
        ref_ops = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(ref_ops)
        sys.modules["electrock_infer._C"] = ref_ops
    import electrock_infer  # noqa: F401  (imports engine, model and layers)
    from electrock_infer import config as ref_config
    from electrock_infer.engine import llm_engine, model_runner, sequence

    sequence.Sequence.block_size = KV_BLOCK

    class _AutoConfig:
        @staticmethod
        def from_pretrained(path):
            from transformers import AutoConfig
            cfg = AutoConfig.from_pretrained(path)
            cfg.rope_theta = ROPE_THETA
            return cfg

    ref_config.AutoConfig = _AutoConfig

    class _AutoTokenizer:
        @staticmethod
        def from_pretrained(*args, **kwargs):
            return _Tokenizer()

    llm_engine.AutoTokenizer = _AutoTokenizer

    def random_init(model, path, rank, config):
        gen = torch.Generator(device="cuda").manual_seed(4 + rank)
        for name, param in model.named_parameters():
            if name.endswith("norm.weight") or name.endswith("layernorm.weight"):
                param.data.fill_(1.0)
            else:
                param.data.normal_(0.0, 0.02, generator=gen)

    model_runner.load_model = random_init

    # The reference names the rendezvous host "localhost", which need not resolve everywhere.
    real_init = dist.init_process_group

    def init_process_group(backend=None, init_method=None, **kwargs):
        if isinstance(init_method, str):
            init_method = init_method.replace("localhost", "127.0.0.1")
        return real_init(backend, init_method, **kwargs)

    dist.init_process_group = init_process_group

    # Time spent in the MoE layer on this rank: an event pair around every FusedMoE.forward.
    from electrock_infer.models import mixtral as ref_model
    moe_cls = ref_model.FusedMoE
    if not getattr(moe_cls, "_engine_timed", False):
        inner = moe_cls.forward

        def timed_forward(self, hidden_states, router_logits):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            out = inner(self, hidden_states, router_logits)
            e1.record()
            _moe_events.append((e0, e1, hidden_states.shape[0]))
            return out

        moe_cls.forward = timed_forward
        moe_cls._engine_timed = True
    return True


_READY = prepare()  # also runs in every spawned rank process, before it unpickles its arguments


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--tp", type=int, default=2)
    ap.add_argument("--layers", type=int, default=32)
    ap.add_argument("--requests", type=int, default=100)
    ap.add_argument("--max-input", type=int, default=1024)
    ap.add_argument("--max-output", type=int, default=256)
    ap.add_argument("--min-len", type=int, default=100)
    ap.add_argument("--gpu-memory-utilization", type=float, default=0.85)
    args = ap.parse_args()
    if not _READY:
        print(json.dumps({"unavailable": "the reference's Python package is not staged under oracle/_ref"}))
        return 0
    import torch
    from electrock_infer import LLM, SamplingParams

    moe = os.environ.get("B200MOE_ENGINE_MOE", "ours")
    model_dir = tempfile.mkdtemp(prefix="mixtral_random_")
    cfg = dict(MODEL, num_hidden_layers=args.layers)
    (Path(model_dir) / "config.json").write_text(json.dumps(cfg))
    rng = Random(4)
    prompts = [[rng.randrange(0, cfg["vocab_size"]) for _ in range(rng.randint(args.min_len, args.max_input))]
               for _ in range(args.requests)]
    params = [SamplingParams(temperature=0.6, ignore_eos=True,
                             max_tokens=rng.randint(min(args.min_len, args.max_output), args.max_output))
              for _ in range(args.requests)]
    res = {"moe_layer": "electrock_infer_b200.FusedMoE" if moe == "ours" else "reference FusedMoE (Triton)",
           "tensor_parallel": args.tp, "layers": args.layers, "requests": args.requests,
           "kv_block_size": KV_BLOCK}
    try:
        t0 = time.time()
        llm = LLM(model_dir, enforce_eager=True, max_model_len=4096, tensor_parallel_size=args.tp,
                  kvcache_block_size=KV_BLOCK, disable_tqdm=True,
                  gpu_memory_utilization=args.gpu_memory_utilization)
        res["init_s"] = round(time.time() - t0, 1)
        llm.generate([[1, 5, 9, 11]], SamplingParams(max_tokens=8))  # warm-up, as the reference does
        torch.cuda.synchronize()
        _moe_events.clear()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        t0 = time.time()
        outs = llm.generate(prompts, params, use_tqdm=False)
        e1.record()
        torch.cuda.synchronize()
        wall = time.time() - t0
        total_out = sum(p.max_tokens for p in params)
        assert all(len(o["token_ids"]) == p.max_tokens for o, p in zip(outs, params))
        moe_ms = sum(a.elapsed_time(b) for a, b, _ in _moe_events)
        res.update({"output_tokens": total_out, "input_tokens": sum(map(len, prompts)),
                    "seconds": wall, "output_tokens_per_s": total_out / wall,
                    "moe_forward_calls": len(_moe_events), "moe_forward_gpu_ms": moe_ms,
                    "moe_share_of_wall": moe_ms * 1e-3 / wall,
                    "gpu_elapsed_s": e0.elapsed_time(e1) * 1e-3})
    except Exception as e:
        import traceback
        res["failed"] = f"{type(e).__name__}: {str(e)[:500]}"
        res["traceback_tail"] = traceback.format_exc()[-1500:]
    print(json.dumps(res), flush=True)
    if "failed" in res:
        # The engine's own exit hook may never have been registered: do not leave rank processes
        # waiting for commands.
        import multiprocessing
        for child in multiprocessing.active_children():
            child.terminate()
        os._exit(1)
    return 0   # the reference's atexit hook tells the other ranks to leave


if __name__ == "__main__":
    sys.exit(main())
