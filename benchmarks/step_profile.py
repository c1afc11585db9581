"""Kernel time shares of engine steps (torch.profiler / CUPTI), split by step kind.

    python benchmarks/step_profile.py --model qwen3-8b --num-prompts 1024 --skip-steps 40 \
        --mixed-steps 3 --decode-steps 3 --out step_profile.txt
    (under torchrun with N ranks it profiles rank 0 of a TP=N engine)

Fills the engine with the benchmark workload, lets it reach steady state, then profiles a few
mixed (prefill chunk + decodes) steps and, once prefill is over, a few decode-only steps.
Numbers taken under the profiler are for shares only, never for throughput."""
from __future__ import annotations

import argparse
import os
import sys
from collections import defaultdict

import numpy as np
import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def _aggregate(prof, wall: float, title: str) -> str:
    agg = defaultdict(lambda: [0, 0.0])
    first, last = None, 0.0
    for ev in prof.events():
        if ev.device_type == torch.autograd.DeviceType.CUDA:
            a = agg[ev.name[:90]]
            a[0] += 1
            a[1] += ev.device_time
            tr = ev.time_range
            first = tr.start if first is None else min(first, tr.start)
            last = max(last, tr.end)
    total = sum(v[1] for v in agg.values())
    span = (last - first) if first is not None else 0.0
    out = [f"== {title}: wall {wall:.2f} s, device span {span / 1e6:.2f} s, "
           f"sum of kernel time {total / 1e6:.2f} s ({100 * total / max(span, 1):.1f}% of the span), "
           f"{sum(v[0] for v in agg.values())} launches"]
    for name, (cnt, us) in sorted(agg.items(), key=lambda kv: -kv[1][1])[:24]:
        out.append(f"  {us / total * 100:5.1f}%  {us / 1e6:8.3f} s  {cnt:7d}  {name}")
    return "\n".join(out)


def reference_whole_pass(args) -> None:
    """Kernel shares of one whole pass of the same workload through upstream vLLM (the benchmark's
    reference arm): in-process engine core so that CUPTI sees its kernels, no out-of-tree plugin."""
    import importlib.util
    import json
    import tempfile
    import time
    os.environ["VLLM_PLUGINS"] = ""
    os.environ["VLLM_ENABLE_V1_MULTIPROCESSING"] = "0"
    os.environ.setdefault("VLLM_LOGGING_LEVEL", "WARNING")
    spec = importlib.util.spec_from_file_location(
        "bench", os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "bench.py"))
    bench = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(bench)
    from vllm import LLM, SamplingParams
    hf = dict(bench.HF_SHAPES[args.model])
    d = tempfile.mkdtemp(prefix="profile_cfg_")
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(hf, f)
    llm = LLM(model=d, load_format="dummy", skip_tokenizer_init=True, dtype="bfloat16",
              max_model_len=args.input_len + args.output_len + 16, max_num_seqs=args.max_num_seqs,
              max_num_batched_tokens=args.max_num_batched_tokens, gpu_memory_utilization=0.92,
              enable_prefix_caching=False, seed=0)
    sp = SamplingParams(temperature=0.0, max_tokens=args.output_len, ignore_eos=True)
    mk = lambda seed: [{"prompt_token_ids": p} for p in
                       bench.make_prompts(args.num_prompts, args.input_len, hf["vocab_size"], seed)]
    llm.generate(mk(1), sp, use_tqdm=False)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    with torch.profiler.profile(activities=[torch.profiler.ProfilerActivity.CUDA]) as prof:
        llm.generate(mk(2), sp, use_tqdm=False)
        torch.cuda.synchronize()
    text = _aggregate(prof, time.perf_counter() - t0, "upstream vLLM, whole pass under the profiler")
    print(text)
    os.makedirs(os.path.dirname(os.path.abspath(args.out)), exist_ok=True)
    with open(args.out, "w") as f:
        f.write(text + "\n")
    sys.stdout.flush()
    os._exit(0)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="qwen3-8b")
    ap.add_argument("--num-prompts", type=int, default=1024)
    ap.add_argument("--input-len", type=int, default=1024)
    ap.add_argument("--output-len", type=int, default=256)
    ap.add_argument("--max-num-seqs", type=int, default=1024)
    ap.add_argument("--max-num-batched-tokens", type=int, default=8192)
    ap.add_argument("--skip-steps", type=int, default=40)
    ap.add_argument("--mixed-steps", type=int, default=3)
    ap.add_argument("--decode-steps", type=int, default=3)
    ap.add_argument("--out", default="step_profile.txt")
    ap.add_argument("--whole-pass", action="store_true",
                    help="profile one complete pass of the workload (device activity only) after a warm pass")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"],
                    help="reference: upstream vLLM (in-process, plugins off); whole-pass mode only")
    args = ap.parse_args()
    if args.impl == "reference":
        return reference_whole_pass(args)
    from vllm_ascend_b200.engine.llm import LLM
    from vllm_ascend_b200.engine.request import SamplingParams
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    llm = LLM(args.model, tensor_parallel_size=world, max_model_len=args.input_len + args.output_len + 16,
              max_num_seqs=args.max_num_seqs, max_num_batched_tokens=args.max_num_batched_tokens, device="cuda")
    eng = llm.engine
    rng = np.random.default_rng(0)
    sp = SamplingParams(temperature=0.0, max_tokens=args.output_len, ignore_eos=True)
    if args.whole_pass:
        import time
        mk = lambda: [rng.integers(0, llm.cfg.model.vocab_size, size=args.input_len).tolist()
                      for _ in range(args.num_prompts)]
        llm.generate(mk(), sp)
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        with torch.profiler.profile(activities=[torch.profiler.ProfilerActivity.CUDA]) as prof:
            llm.generate(mk(), sp)
            torch.cuda.synchronize()
        wall = time.perf_counter() - t0
        text = _aggregate(prof, wall, "whole pass under the profiler")
        if rank == 0:
            print(text)
            os.makedirs(os.path.dirname(os.path.abspath(args.out)), exist_ok=True)
            with open(args.out, "w") as f:
                f.write(text + "\n")
        sys.stdout.flush()
        llm.shutdown()
        os._exit(0)
    for _ in range(args.num_prompts):
        eng.add_request(rng.integers(0, llm.cfg.model.vocab_size, size=args.input_len).tolist(), sp)
    for _ in range(args.skip_steps):
        eng.step()
    acts = [torch.profiler.ProfilerActivity.CPU, torch.profiler.ProfilerActivity.CUDA]
    lines = []

    def profile(kind: str, n: int, want_decode: bool):
        # advance until the next step is of the wanted kind
        guard = 0
        while eng.has_unfinished() and guard < 100000:
            waiting_prefill = any(r.num_computed_tokens < r.num_prompt_tokens for r in eng.scheduler.running) \
                or len(eng.scheduler.waiting) > 0
            if want_decode != waiting_prefill:
                break
            eng.step()
            guard += 1
        if not eng.has_unfinished():
            lines.append(f"== {kind}: workload ended before such a step came up")
            return
        torch.cuda.synchronize()
        with torch.profiler.profile(activities=acts) as prof:
            for _ in range(n):
                eng.step()
            torch.cuda.synchronize()
        agg = defaultdict(lambda: [0, 0.0])
        for ev in prof.events():
            if ev.device_type == torch.autograd.DeviceType.CUDA:
                a = agg[ev.name[:90]]
                a[0] += 1
                a[1] += ev.device_time if hasattr(ev, "device_time") else ev.cuda_time
        total = sum(v[1] for v in agg.values())
        lines.append(f"== {kind}: {n} steps, {total / n / 1000:.2f} ms of kernel time per step, "
                     f"{sum(v[0] for v in agg.values()) // n} launches per step")
        for name, (cnt, us) in sorted(agg.items(), key=lambda kv: -kv[1][1])[:18]:
            lines.append(f"  {us / total * 100:5.1f}%  {us / n / 1000:8.3f} ms/step  {cnt // n:5d}/step  {name}")

    if args.mixed_steps > 0:
        profile("mixed (prefill chunk + decodes)", args.mixed_steps, want_decode=False)
    if args.decode_steps > 0:
        profile("decode only", args.decode_steps, want_decode=True)
    text = "\n".join(lines)
    if rank != 0:
        llm.shutdown()
        os._exit(0)
    print(text)
    os.makedirs(os.path.dirname(os.path.abspath(args.out)), exist_ok=True)
    with open(args.out, "w") as f:
        f.write(text + "\n")
    if world > 1:
        sys.stdout.flush()
        llm.shutdown()
        os._exit(0)


if __name__ == "__main__":
    main()
