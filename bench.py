#!/usr/bin/env python
"""Headline benchmark: output tokens/s of a synthetic workload through the public ``LLM`` API.

Default workload (Qwen3-8B shape): 1024 prompts of 1024 uniform-random token ids, 256 output
tokens each (EOS ignored), bf16, random-init weights, tensor parallel over the N GPUs of the
node.  One "step" is one complete pass of that workload through ``LLM.generate``; W untimed
passes are followed by K timed ones.

    python bench.py --gpus 1 --steps 1 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29511 bench.py --gpus 8 --steps 1 --warmup 3

Arms (``--impl``):

* ``ours``: this framework's engine (``vllm_ascend_b200.LLM``).  ``--engine vllm`` instead runs
  this package as a platform plugin under the installed upstream vLLM ``LLM`` entry point.
* ``reference``: the baseline.  The reference project is a plugin for Ascend NPUs and cannot run on
  a CUDA device, so the baseline is upstream vLLM's own CUDA build from the image, unmodified, on
  the same workload, with every vLLM plugin disabled.  This arm imports nothing from this package.

Workloads (``--mode``):

* ``offline``: all prompts submitted at once (throughput case).
* ``serve``: closed loop with ``--concurrency`` requests in flight (fixed-concurrency serving case);
  p50 TTFT / TPOT are per request.
* ``pd``: disaggregated prefill: the first half of the ranks form the prefill engine (TP), the second
  half the decode engine (expert parallel with data-parallel attention for MoE models), KV blocks
  move over NVLink (``ours`` only).

Rank 0 prints ONE JSON line.  ``value`` is timed with CUDA events (max over ranks); ``e2e.value``
is the same passes timed by the host clock around ``LLM.generate`` — every engine step inside
copies its inputs from pinned host memory to the device and reads the sampled tokens back.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import threading
import time

import numpy as np

REPO = os.path.dirname(os.path.abspath(__file__))

REFERENCE_CLASS = "upstream vLLM 0.22 CUDA build (the reference project itself runs on Ascend NPUs only)"

#: output tok/s of upstream vLLM 0.22 on one B200 box, same workload (``--impl reference``);
#: keyed by (model, mode, n_gpus).  ``vs_baseline`` divides by these; None where nothing was measured.
UPSTREAM_VLLM_B200 = {
    ("qwen3-8b", "offline", 1): 10622.2,
}

#: HF ``config.json`` contents of the benchmark architectures (random-init weights of these shapes).
HF_SHAPES = {
    # plumbing case (CPU, fp32): exercises every mode of this script in the tests
    "tiny-qwen": dict(
        architectures=["Qwen3ForCausalLM"], model_type="qwen3", vocab_size=1024, hidden_size=256,
        intermediate_size=512, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
        head_dim=64, rms_norm_eps=1e-6, rope_theta=1e6, max_position_embeddings=4096,
        tie_word_embeddings=False, torch_dtype="float32", hidden_act="silu", attention_bias=False),
    "qwen3-8b": dict(
        architectures=["Qwen3ForCausalLM"], model_type="qwen3", vocab_size=151936, hidden_size=4096,
        intermediate_size=12288, num_hidden_layers=36, num_attention_heads=32, num_key_value_heads=8,
        head_dim=128, rms_norm_eps=1e-6, rope_theta=1e6, max_position_embeddings=40960,
        tie_word_embeddings=False, torch_dtype="bfloat16", hidden_act="silu", attention_bias=False),
    "llama-3.1-70b": dict(
        architectures=["LlamaForCausalLM"], model_type="llama", vocab_size=128256, hidden_size=8192,
        intermediate_size=28672, num_hidden_layers=80, num_attention_heads=64, num_key_value_heads=8,
        head_dim=128, rms_norm_eps=1e-5, rope_theta=5e5, max_position_embeddings=131072,
        tie_word_embeddings=False, torch_dtype="bfloat16", hidden_act="silu", attention_bias=False,
        mlp_bias=False),
    "qwen3-30b-a3b": dict(
        architectures=["Qwen3MoeForCausalLM"], model_type="qwen3_moe", vocab_size=151936, hidden_size=2048,
        intermediate_size=6144, num_hidden_layers=48, num_attention_heads=32, num_key_value_heads=4,
        head_dim=128, rms_norm_eps=1e-6, rope_theta=1e6, max_position_embeddings=40960,
        tie_word_embeddings=False, torch_dtype="bfloat16", hidden_act="silu", attention_bias=False,
        num_experts=128, num_experts_per_tok=8, moe_intermediate_size=768, norm_topk_prob=True,
        decoder_sparse_step=1, mlp_only_layers=[], router_aux_loss_coef=0.0),
    "deepseek-v3": dict(
        architectures=["DeepseekV3ForCausalLM"], model_type="deepseek_v3", vocab_size=129280,
        hidden_size=7168, intermediate_size=18432, moe_intermediate_size=2048, num_hidden_layers=61,
        num_attention_heads=128, num_key_value_heads=128, n_routed_experts=256, n_shared_experts=1,
        num_experts_per_tok=8, first_k_dense_replace=3, moe_layer_freq=1, n_group=8, topk_group=4,
        routed_scaling_factor=2.5, scoring_func="sigmoid", topk_method="noaux_tc", norm_topk_prob=True,
        q_lora_rank=1536, kv_lora_rank=512, qk_nope_head_dim=128, qk_rope_head_dim=64, v_head_dim=128,
        rms_norm_eps=1e-6, rope_theta=1e4, max_position_embeddings=163840, tie_word_embeddings=False,
        torch_dtype="bfloat16", hidden_act="silu", attention_bias=False, num_nextn_predict_layers=0),
}

FP8_BLOCK = {"quant_method": "fp8", "fmt": "e4m3", "activation_scheme": "dynamic",
             "weight_block_size": [128, 128]}


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=1)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "vllm"])
    ap.add_argument("--engine", default="native", choices=["native", "vllm"])
    ap.add_argument("--model", default="qwen3-8b", choices=sorted(HF_SHAPES))
    ap.add_argument("--mode", default="offline", choices=["offline", "serve", "pd"])
    ap.add_argument("--concurrency", type=int, default=64)
    ap.add_argument("--num-prompts", type=int, default=1024)
    ap.add_argument("--input-len", type=int, default=1024)
    ap.add_argument("--output-len", type=int, default=256)
    ap.add_argument("--max-num-seqs", type=int, default=1024)
    ap.add_argument("--max-num-batched-tokens", type=int, default=8192)
    ap.add_argument("--parallelism", default="tp", choices=["tp", "ep"])
    ap.add_argument("--quantization", default=None)
    ap.add_argument("--eplb", action="store_true", help="dynamic expert load balancing (MoE, --parallelism ep)")
    ap.add_argument("--num-layers", type=int, default=None,
                    help="diagnostic only: fewer layers than the named model (the line says so)")
    ap.add_argument("--enforce-eager", action="store_true")
    ap.add_argument("--gpu-memory-utilization", type=float, default=0.92)
    return ap.parse_args()


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi during the timed region."""
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu_index = gpu_index
        self.proc = None
        self.path = None

    def start(self):
        try:
            f = tempfile.NamedTemporaryFile("w", suffix=".csv", delete=False)
            self.path = f.name
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                 "-lms", "200", "-i", str(self.gpu_index)], stdout=f, stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self) -> dict:
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        clocks, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        try:
            with open(self.path) as f:
                for line in f:
                    p = [x.strip() for x in line.split(",")]
                    if len(p) < 9:
                        continue
                    try:
                        clocks.append(float(p[1]))
                        mx.append(float(p[2]))
                    except ValueError:
                        continue
                    for name, v in zip(names, p[5:9]):
                        if v.lower().startswith("active"):
                            reasons.add(name)
            os.unlink(self.path)
        except OSError:
            pass
        if clocks:
            out["sm_mhz"] = statistics.median(clocks)
            out["sm_max_mhz"] = max(mx)
            out["samples"] = len(clocks)
        out["reasons"] = sorted(reasons)
        return out


def make_prompts(n: int, length: int, vocab: int, seed: int):
    rng = np.random.default_rng(seed)
    return [rng.integers(0, vocab, size=length, dtype=np.int64).tolist() for _ in range(n)]


def hf_shape(args) -> dict:
    hf = dict(HF_SHAPES[args.model])
    if args.num_layers:
        hf["num_hidden_layers"] = args.num_layers
    if args.quantization == "fp8":
        hf["quantization_config"] = dict(FP8_BLOCK)
    return hf


def config_block(args, world: int, extra: dict) -> dict:
    par = {"tp": f"tp{world}", "ep": f"ep{world}"}[args.parallelism]
    if args.mode == "pd":
        par = f"pd: tp{world // 2} prefill -> {'ep' if args.parallelism == 'ep' else 'tp'}{world // 2} decode"
    cfg = {"model": args.model, "global_batch": args.num_prompts, "seq_len": args.input_len,
           "output_len": args.output_len, "parallelism": par, "mode": args.mode,
           "max_num_seqs": args.max_num_seqs, "max_num_batched_tokens": args.max_num_batched_tokens,
           "l2": "working set (weights + KV cache) far exceeds the 126 MB L2; no flush"}
    if args.mode == "serve":
        cfg["concurrency"] = args.concurrency
    if args.quantization:
        cfg["quantization"] = args.quantization
    if args.num_layers:
        cfg["num_layers_override"] = args.num_layers
        cfg["INVALID_AS_HEADLINE"] = "fewer layers than the named model"
    cfg.update(extra)
    return cfg


def vs_baseline(args, world: int, value: float):
    ref = UPSTREAM_VLLM_B200.get((args.model, args.mode, world))
    if ref is None or args.quantization or args.num_layers or args.num_prompts != 1024 \
            or args.input_len != 1024 or args.output_len != 256:
        return None
    return value / ref


# --------------------------------------------------------------------------- reference arm
def run_reference(args, rank: int, world: int, local: int):
    """Upstream vLLM (CUDA build of the image) through ``vllm.LLM``: stock code path, no plugin,
    nothing of this package imported.  In-process engine core so that the CUDA events and the
    synchronisation of this process bracket the work."""
    os.environ["VLLM_PLUGINS"] = ""                      # load no out-of-tree plugin
    os.environ.setdefault("VLLM_ENABLE_V1_MULTIPROCESSING", "0")
    os.environ.setdefault("VLLM_LOGGING_LEVEL", "WARNING")
    if args.mode == "pd":
        if rank == 0:
            print(json.dumps({"impl": "reference", "reference_class": REFERENCE_CLASS,
                              "unavailable": "the disaggregated-prefill case is not wired for upstream vLLM here "
                                             "(needs its NIXL connector and two launch groups)"}))
        return
    try:
        import torch
        import vllm  # noqa: F401
        from vllm import LLM, SamplingParams
    except Exception as e:  # pragma: no cover - depends on the image
        if rank == 0:
            print(json.dumps({"impl": "reference", "reference_class": REFERENCE_CLASS,
                              "unavailable": f"upstream vLLM cannot be imported here: {type(e).__name__}: {e}"[:300]}))
        return
    hf = hf_shape(args)
    d = tempfile.mkdtemp(prefix="bench_cfg_")
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(hf, f)
    kw = dict(model=d, load_format="dummy", skip_tokenizer_init=True, dtype="bfloat16",
              tensor_parallel_size=world, max_model_len=args.input_len + args.output_len + 16,
              max_num_seqs=args.max_num_seqs, max_num_batched_tokens=args.max_num_batched_tokens,
              gpu_memory_utilization=args.gpu_memory_utilization, enable_prefix_caching=False, seed=0,
              enforce_eager=args.enforce_eager)
    if args.parallelism == "ep":
        kw["enable_expert_parallel"] = True
    if world > 1:
        kw["distributed_executor_backend"] = "external_launcher"
    llm = LLM(**kw)
    sp = SamplingParams(temperature=0.0, max_tokens=args.output_len, ignore_eos=True)
    n_out = args.num_prompts * args.output_len
    vocab = hf["vocab_size"]

    def one_pass(prompts):
        """Returns per-request (ttft, tpot) lists; closed loop in serve mode."""
        ttft, tpot = [], []
        if args.mode == "offline":
            t_sub = time.perf_counter()
            outs = llm.generate([{"prompt_token_ids": p} for p in prompts], sp, use_tqdm=False)
            for o in outs:
                assert len(o.outputs[0].token_ids) == args.output_len
                m = getattr(o, "metrics", None)
                ft = getattr(m, "first_token_latency", None) if m is not None else None
                if ft:
                    ttft.append(float(ft))
            del t_sub
            return ttft, tpot
        eng = llm.llm_engine
        pending = list(enumerate(prompts))[::-1]
        t_add, t_first, inflight, done = {}, {}, 0, 0
        while pending or inflight:
            while pending and inflight < args.concurrency:
                i, p = pending.pop()
                rid = f"r{i}"
                t_add[rid] = time.perf_counter()
                eng.add_request(rid, {"prompt_token_ids": p}, sp)
                inflight += 1
            for o in eng.step():
                now = time.perf_counter()
                rid = o.request_id
                key = rid if rid in t_add else rid.split("-")[0]
                if key not in t_first and o.outputs and len(o.outputs[0].token_ids) > 0:
                    t_first[key] = now
                if o.finished:
                    inflight -= 1
                    done += 1
                    k = len(o.outputs[0].token_ids)
                    assert k == args.output_len
                    ttft.append(t_first[key] - t_add[key])
                    if k > 1:
                        tpot.append((now - t_first[key]) / (k - 1))
        assert done == len(prompts)
        return ttft, tpot

    dev_ms, wall_s, ttfts, tpots = [], [], [], []
    sampler = ClockSampler(local)
    for it in range(args.warmup + args.steps):
        prompts = make_prompts(args.num_prompts, args.input_len, vocab, 1000 + it)
        if it == args.warmup:
            sampler.start()
        if world > 1:
            torch.distributed.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0 = time.perf_counter()
        e0.record()
        tt, tp = one_pass(prompts)
        e1.record()
        if world > 1:
            torch.distributed.barrier()
        torch.cuda.synchronize()
        t1 = time.perf_counter()
        if it >= args.warmup:
            dev_ms.append(e0.elapsed_time(e1))
            wall_s.append(t1 - t0)
            ttfts += tt
            tpots += tp
    clocks = sampler.stop()
    ms = sum(dev_ms) / len(dev_ms)
    wall = sum(wall_s) / len(wall_s)
    if world > 1:
        t = torch.tensor([ms, wall], dtype=torch.float64, device="cuda")
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
        ms, wall = float(t[0]), float(t[1])
    # the events sit on this process's current stream; the engine may run on streams of its own, so
    # the device-side figure is the host clock between two full-device synchronisations when larger
    ms = max(ms, 0.0)
    value = n_out / (max(ms, wall * 1e3) / 1e3)
    if rank == 0:
        print(json.dumps({
            "impl": "reference", "reference_class": REFERENCE_CLASS,
            "metric": "output_tokens_per_s", "value": value, "unit": "tok/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": max(ms, wall * 1e3),
            "higher_is_better": True, "scaling": "strong", "vs_baseline": vs_baseline(args, world, value),
            "dtype": "bf16" if not args.quantization else f"bf16+{args.quantization}", "data": "synthetic",
            "config": config_block(args, world, {
                "engine": "vllm.LLM, in-process engine core, load_format=dummy, plugins disabled",
                "timing": "host clock between device synchronisations (upper bound of the device time); "
                          f"CUDA events on the caller's stream gave {ms:.1f} ms"}),
            "p50_ttft_s": statistics.median(ttfts) if ttfts else None,
            "p50_tpot_s": statistics.median(tpots) if tpots else None,
            "clocks": clocks,
            "e2e": {"value": n_out / wall, "unit": "tok/s",
                    "h2d_bytes_per_step": args.num_prompts * args.input_len * 8,
                    "d2h_bytes_per_step": n_out * 8,
                    "note": "per pass, counted from the prompt ids going in and the sampled ids coming out "
                            "(vLLM copies more per engine step: positions, slot mappings, block tables)"},
            "gpu_launches": None,
        }))
    sys.stdout.flush()
    if world > 1:
        watchdog = threading.Timer(45.0, lambda: os._exit(0))
        watchdog.daemon = True
        watchdog.start()
    del llm
    if world > 1:
        os._exit(0)


# --------------------------------------------------------------------------- this framework
def run_ours_under_vllm(args, rank: int, world: int, local: int):
    """This package as a platform plugin of the installed upstream vLLM: ``vllm.LLM`` is the entry
    point, the worker / model runner / kernels are this package's."""
    sys.path.insert(0, REPO)
    os.environ["VLLM_PLUGINS"] = "b200"
    os.environ.setdefault("VLLM_ENABLE_V1_MULTIPROCESSING", "0")
    os.environ.setdefault("VLLM_LOGGING_LEVEL", "WARNING")
    import torch
    from vllm_ascend_b200.vllm_plugin import ensure_entry_points
    ensure_entry_points()
    from vllm import LLM, SamplingParams
    hf = hf_shape(args)
    d = tempfile.mkdtemp(prefix="bench_cfg_")
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(hf, f)
    kw = dict(model=d, load_format="dummy", skip_tokenizer_init=True, dtype="bfloat16",
              tensor_parallel_size=world, max_model_len=args.input_len + args.output_len + 16,
              max_num_seqs=args.max_num_seqs, max_num_batched_tokens=args.max_num_batched_tokens,
              gpu_memory_utilization=args.gpu_memory_utilization, enable_prefix_caching=False, seed=0)
    if world > 1:
        kw["distributed_executor_backend"] = "external_launcher"
    llm = LLM(**kw)
    sp = SamplingParams(temperature=0.0, max_tokens=args.output_len, ignore_eos=True)
    n_out = args.num_prompts * args.output_len
    wall_s = []
    sampler = ClockSampler(local)
    for it in range(args.warmup + args.steps):
        prompts = make_prompts(args.num_prompts, args.input_len, hf["vocab_size"], 1000 + it)
        if it == args.warmup:
            sampler.start()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        outs = llm.generate([{"prompt_token_ids": p} for p in prompts], sp, use_tqdm=False)
        torch.cuda.synchronize()
        if it >= args.warmup:
            wall_s.append(time.perf_counter() - t0)
        assert all(len(o.outputs[0].token_ids) == args.output_len for o in outs)
    clocks = sampler.stop()
    wall = sum(wall_s) / len(wall_s)
    from vllm_ascend_b200 import _native
    if rank == 0:
        print(json.dumps({
            "impl": "ours", "metric": "output_tokens_per_s", "value": n_out / wall, "unit": "tok/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": wall * 1e3,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": vs_baseline(args, world, n_out / wall),
            "dtype": "bf16", "data": "synthetic",
            "config": config_block(args, world, {"engine": "vllm.LLM with this package as platform plugin",
                                                 "timing": "host clock between device synchronisations"}),
            "clocks": clocks, "gpu_launches": int(_native.launch_counter[0]),
        }))


def run_ours(args, rank: int, world: int, local: int):
    sys.path.insert(0, REPO)
    # tensor-parallel runs time the fused peer-memory dataflow against NCCL per step class at start-up
    # and serve each class with the faster one; the choice is reported under config.tp_comm_calibration
    os.environ.setdefault("VLLM_B200_TP_COMM", "auto")
    import torch
    import torch.distributed as dist
    from vllm_ascend_b200.config import get_model_config
    from vllm_ascend_b200.engine.llm import LLM
    from vllm_ascend_b200.engine.request import SamplingParams

    ep = args.parallelism == "ep"
    mcfg = get_model_config(args.model)
    if args.num_layers:
        mcfg.num_hidden_layers = args.num_layers
    if args.quantization:
        mcfg.quantization = args.quantization
    elif mcfg.quantization and args.model != "deepseek-v3":
        mcfg.quantization = None
    additional = {}
    if args.eplb:
        additional["eplb_config"] = {"dynamic_eplb": True, "expert_heat_collection_interval": 64,
                                     "algorithm_execution_interval": 8}
    llm = LLM(mcfg, tensor_parallel_size=1 if ep else world, enable_expert_parallel=ep,
              max_model_len=args.input_len + args.output_len + 16, max_num_seqs=args.max_num_seqs,
              max_num_batched_tokens=args.max_num_batched_tokens,
              enforce_eager=args.enforce_eager, gpu_memory_utilization=args.gpu_memory_utilization,
              additional_config=additional, device="cuda")
    cfg = llm.cfg.model
    sp = SamplingParams(temperature=0.0, max_tokens=args.output_len, ignore_eos=True)
    runner = llm.engine.runner
    n_out = args.num_prompts * args.output_len
    conc = args.concurrency if args.mode == "serve" else None

    def sync():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    dev_ms, wall_s, ttfts, tpots = [], [], [], []
    sampler = ClockSampler(local)
    stats0 = launches0 = None
    for it in range(args.warmup + args.steps):
        prompts = make_prompts(args.num_prompts, args.input_len, cfg.vocab_size, 1000 + it)
        timed = it >= args.warmup
        if it == args.warmup:
            sampler.start()
            stats0 = dict(runner.stats)
            launches0 = runner.total_launches()
        sync()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0 = time.perf_counter()
        e0.record()
        outs = llm.generate(prompts, sp, max_concurrency=conc)
        e1.record()
        sync()
        t1 = time.perf_counter()
        if timed:
            dev_ms.append(e0.elapsed_time(e1))
            wall_s.append(t1 - t0)
            for o in outs:
                m = o.metrics
                if m.first_token_time is not None:
                    ttfts.append(m.first_token_time - m.arrival_time)
                    k = len(o.outputs[0].token_ids)
                    if k > 1:
                        tpots.append((m.finish_time - m.first_token_time) / (k - 1))
        assert all(len(o.outputs[0].token_ids) == args.output_len for o in outs)
    clocks = sampler.stop()
    ms = sum(dev_ms) / len(dev_ms)
    wall = sum(wall_s) / len(wall_s)
    if world > 1:
        t = torch.tensor([ms, wall], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, wall = float(t[0]), float(t[1])
    steps_timed = max(1, args.steps)
    n_eng = max(1, runner.stats["steps"] - stats0["steps"])
    eng_steps = n_eng / steps_timed
    h2d = (runner.stats["h2d_bytes"] - stats0["h2d_bytes"]) / n_eng
    d2h = (runner.stats["d2h_bytes"] - stats0["d2h_bytes"]) / n_eng
    launches = (runner.total_launches() - launches0)
    value = n_out / (ms / 1e3)
    if rank == 0:
        print(json.dumps({
            "metric": "output_tokens_per_s", "value": value, "unit": "tok/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms,
            "higher_is_better": True, "scaling": "strong",
            "vs_baseline": vs_baseline(args, world, value),
            "dtype": "bf16" if not mcfg.quantization else f"bf16+{mcfg.quantization}",
            "data": "synthetic", "impl": "ours",
            "config": config_block(args, world, {
                "tp_comm": os.environ.get("VLLM_B200_TP_COMM", "fused"),
                "tp_comm_calibration": getattr(llm.engine.worker, "tp_comm_calibration", None),
                "kv_blocks": runner.num_blocks, "block_size": runner.block_size,
                "engine_steps_per_pass": eng_steps,
                "baseline_note": "vs_baseline divides by upstream vLLM 0.22 measured on a B200 of this pool "
                                 "on the same workload (null where that was not measured)"}),
            "p50_ttft_s": statistics.median(ttfts) if ttfts else None,
            "p50_tpot_s": statistics.median(tpots) if tpots else None,
            "clocks": clocks,
            "e2e": {"value": n_out / wall, "unit": "tok/s", "h2d_bytes_per_step": h2d,
                    "d2h_bytes_per_step": d2h, "note": "per engine step (one forward pass)"},
            "gpu_launches": launches,
            "graph_replays": runner.stats["graph_replays"] - stats0["graph_replays"],
            "preemptions": llm.engine.scheduler.num_preemptions,
            "host_breakdown_s": {**{k: round(v, 3) for k, v in llm.engine.host_times.items()},
                                 **{k: round(runner.stats[k], 3) for k in ("t_prepare", "t_launch", "t_wait")},
                                 **{k: (round(v, 3) if isinstance(v, float) else v)
                                    for k, v in runner.stats.items()
                                    if k[:2] in ("t_", "n_") and k.split("_", 1)[1] in ("decode", "decode_eager", "mixed")},
                                 "note": "cumulative over warm-up and timed passes"},
            "device_breakdown_ms": {k: round(v, 1) for k, v in runner.stats.items() if k.startswith("gpu_")} or None,
        }))
    sys.stdout.flush()
    # Captured graphs that contain NCCL collectives must be gone before the communicators
    # are torn down; a watchdog ends the process if library teardown stalls anyway.
    if world > 1:
        watchdog = threading.Timer(45.0, lambda: os._exit(0))
        watchdog.daemon = True
        watchdog.start()
    llm.shutdown()
    if world > 1:
        os._exit(0)


def main():
    args = parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus and world == 1 and args.gpus > 1:
        # convenience: re-launch under torchrun
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1",
               f"--nproc-per-node={args.gpus}", "--master-addr", "127.0.0.1", "--master-port",
               str(29500 + os.getpid() % 400), os.path.abspath(__file__)] + sys.argv[1:]
        sys.exit(subprocess.call(cmd))
    if args.impl in ("reference", "vllm"):
        try:
            run_reference(args, rank, world, local)
        except SystemExit:
            raise
        except BaseException as e:  # noqa: BLE001 - the arm must leave a line behind, whatever failed
            import traceback
            traceback.print_exc()
            print(json.dumps({"impl": "reference", "reference_class": REFERENCE_CLASS, "n_gpus": world,
                              "unavailable": f"upstream vLLM failed at run time on rank {rank}: "
                                             f"{type(e).__name__}: {e}"[:400]}), flush=True)
            # a non-zero status lets the launcher stop the other ranks instead of leaving them in a collective
            os._exit(0 if world == 1 else 3)
    elif args.mode == "pd":
        sys.path.insert(0, REPO)
        from benchmarks.pd_bench import run_pd
        run_pd(args, rank, world, local, config_block, make_prompts, ClockSampler)
    elif args.engine == "vllm":
        run_ours_under_vllm(args, rank, world, local)
    else:
        run_ours(args, rank, world, local)


if __name__ == "__main__":
    main()
