"""Disaggregated-prefill arm of ``bench.py`` (``--mode pd``).

One launch of N ranks hosts two engines: ranks [0, N/2) form the prefill engine (tensor parallel
over N/2 GPUs, ``kv_role=kv_producer``), ranks [N/2, N) the decode engine (``kv_consumer``; tensor
parallel, or expert parallel with data-parallel attention under ``--parallelism ep``).  Each half
is its own ``torch.distributed`` world (own rendezvous port); a small TCP store that spans all N
ranks carries the hand-off: per wave of prompts the prefill engine publishes the
``kv_transfer_params`` it got back (block ids it keeps alive), the decode engine admits the wave
with those parameters, pulls the KV blocks over NVLink into its own block tables
(``NVLinkConnector``) and decodes.  The decode side keeps ``--concurrency`` requests in flight;
the prefill side runs at most two waves ahead of what the decode side has admitted.

Deployment shape of the reference's disaggregated cases
(tests/e2e/nightly/multi_node/internal_dp/config/Qwen3-235B-disagg-pd.yaml: prefill and decode
instances behind a proxy, KV over the Mooncake connector).
"""
from __future__ import annotations

import json
import os
import statistics
import sys
import time
from collections import deque
from datetime import timedelta


def run_pd(args, rank: int, world: int, local: int, config_block, make_prompts, ClockSampler) -> None:
    import torch
    import torch.distributed as dist
    if world < 2 or world % 2:
        raise SystemExit("--mode pd needs an even number of ranks (half prefill, half decode)")
    half = world // 2
    is_prefill = rank < half
    sub = rank % half
    port0 = int(os.environ.get("MASTER_PORT", "29500"))
    store = dist.TCPStore("127.0.0.1", port0 + 7, world_size=world, is_master=(rank == 0),
                          timeout=timedelta(seconds=1800))
    # each half is a world of its own
    os.environ["RANK"], os.environ["WORLD_SIZE"] = str(sub), str(half)
    os.environ["MASTER_PORT"] = str(port0 + (11 if is_prefill else 12))
    os.environ.setdefault("VLLM_B200_TP_COMM", "auto")
    repo = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    sys.path.insert(0, repo)
    from vllm_ascend_b200.config import get_model_config
    from vllm_ascend_b200.engine.llm import LLM
    from vllm_ascend_b200.engine.request import SamplingParams
    from vllm_ascend_b200.parallel import state as pstate

    on_gpu = torch.cuda.is_available()          # without a GPU the same flow runs on gloo ranks (tests)

    def dev_sync() -> None:
        if on_gpu:
            torch.cuda.synchronize()

    mcfg = get_model_config(args.model)
    if args.num_layers:
        mcfg.num_hidden_layers = args.num_layers
    if args.quantization:
        mcfg.quantization = args.quantization
    ep = args.parallelism == "ep" and not is_prefill
    kv_base = port0 + 40
    ktc = {"kv_connector": "NVLinkConnector", "kv_role": "kv_producer" if is_prefill else "kv_consumer",
           "engine_id": "P" if is_prefill else "D", "kv_port": kv_base + (0 if is_prefill else 16)}
    llm = LLM(mcfg, tensor_parallel_size=1 if ep else half, enable_expert_parallel=ep,
              max_model_len=args.input_len + args.output_len + 16, max_num_seqs=args.max_num_seqs,
              max_num_batched_tokens=args.max_num_batched_tokens, enforce_eager=args.enforce_eager,
              gpu_memory_utilization=args.gpu_memory_utilization, kv_transfer_config=ktc,
              device="cuda" if on_gpu else "cpu")
    eng = llm.engine
    cfg = llm.cfg.model
    n_out = args.num_prompts * args.output_len
    wave = max(1, min(args.concurrency, args.num_prompts))
    n_waves = (args.num_prompts + wave - 1) // wave
    sp1 = SamplingParams(temperature=0.0, max_tokens=1, ignore_eos=True)
    sp = SamplingParams(temperature=0.0, max_tokens=args.output_len, ignore_eos=True)
    grp = pstate.get_world_group()

    def world_barrier(tag: str) -> None:
        store.add(tag, 1)
        while int(store.add(tag, 0)) < world:
            time.sleep(0.002)

    def agree(v: int) -> int:
        """Value of sub-rank 0 on every rank of this half (the ranks must take the same decisions
        in the same engine iteration)."""
        if half == 1:
            return v
        t = torch.tensor([v], dtype=torch.int64)
        dist.broadcast(t, src=grp.ranks[0], group=grp.cpu_group)
        return int(t[0])

    def prefill_pass(it: int, prompts) -> None:
        c = eng.kv_connector
        for k in range(n_waves):
            if k >= 2:                       # stay at most two waves ahead of the decode engine
                while agree(int(store.check([f"d{it}w{k - 2}"]))) == 0:
                    c.reap(eng.scheduler)
                    time.sleep(0.001)
            batch = prompts[k * wave:(k + 1) * wave]
            t_send = time.time()
            outs = llm.generate([{"prompt_token_ids": p, "kv_transfer_params": {"do_remote_decode": True}}
                                 for p in batch], sp1)
            if sub == 0:
                store.set(f"p{it}w{k}", json.dumps({"t": t_send, "params": [o.kv_transfer_params for o in outs]}))
            c.reap(eng.scheduler)
        while agree(int(store.check([f"done{it}"]))) == 0:      # blocks stay alive until they were pulled
            c.reap(eng.scheduler)
            time.sleep(0.002)
        c.reap(eng.scheduler)

    def decode_pass(it: int, prompts):
        dp = eng.dp
        nd, me = max(1, dp.world_size), dp.rank_in_group
        limit = max(1, args.concurrency // nd)
        pending: deque = deque()
        mine: dict = {}
        t_sent: dict = {}
        fetched = 0
        ttft, tpot = [], []
        while True:
            avail = fetched
            if sub == 0:
                while avail < n_waves and store.check([f"p{it}w{avail}"]):
                    avail += 1
            avail = agree(avail)
            while fetched < avail:
                msg = json.loads(store.get(f"p{it}w{fetched}"))
                for j, ktp in enumerate(msg["params"]):
                    i = fetched * wave + j
                    if i % nd == me:
                        pending.append((i, ktp, msg["t"]))
                if sub == 0:
                    store.set(f"d{it}w{fetched}", "1")
                fetched += 1
            while pending and eng.scheduler.num_unfinished < limit:
                i, ktp, ts = pending.popleft()
                rid = eng.add_request(prompts[i], sp, kv_transfer_params=ktp)
                mine[rid] = eng.scheduler.requests[rid]
                t_sent[rid] = ts
            if nd > 1:
                busy = eng.step_dp()
            else:
                busy = eng.has_unfinished()
                if busy:
                    eng.step()
            if not busy:
                if fetched == n_waves and not pending:
                    break
                time.sleep(0.0005)
        for rid, r in mine.items():
            assert r.is_finished and len(r.output_token_ids) == args.output_len
            if r.first_token_time is not None:
                # time.monotonic() on this side vs time.time() at the sender: both taken on one host
                ttft.append(max(0.0, (time.time() - (time.monotonic() - r.first_token_time)) - t_sent[rid]))
                if r.finish_time and args.output_len > 1:
                    tpot.append((r.finish_time - r.first_token_time) / (args.output_len - 1))
            eng.scheduler.requests.pop(rid, None)
        return ttft, tpot

    dev_ms, wall_s, ttfts, tpots = [], [], [], []
    sampler = ClockSampler(local)
    for it in range(args.warmup + args.steps):
        prompts = make_prompts(args.num_prompts, args.input_len, cfg.vocab_size, 1000 + it)
        if it == args.warmup:
            sampler.start()
        dev_sync()
        world_barrier(f"start{it}")
        if on_gpu:
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0 = time.perf_counter()
        if on_gpu:
            e0.record()
        if is_prefill:
            prefill_pass(it, prompts)
            tt, tp = [], []
        else:
            tt, tp = decode_pass(it, prompts)
            dev_sync()
            store.add(f"dfin{it}", 1)
            if sub == 0:
                while int(store.add(f"dfin{it}", 0)) < half:
                    time.sleep(0.001)
                store.set(f"done{it}", "1")
        if on_gpu:
            e1.record()
        dev_sync()
        t_done = time.perf_counter()
        world_barrier(f"end{it}")
        t1 = time.perf_counter()
        if it >= args.warmup:
            dev_ms.append(e0.elapsed_time(e1) if on_gpu else (t_done - t0) * 1e3)
            wall_s.append(t1 - t0)
            ttfts += tt
            tpots += tp
    clocks = sampler.stop()
    ms = sum(dev_ms) / len(dev_ms)
    wall = sum(wall_s) / len(wall_s)
    store.set(f"res{rank}", json.dumps({"ms": ms, "wall": wall, "ttft": ttfts, "tpot": tpots,
                                        "pulled": (eng.kv_connector.stats if not is_prefill else None)}))
    world_barrier("results")
    if rank == 0:
        res = [json.loads(store.get(f"res{r}")) for r in range(world)]
        ms = max(r["ms"] for r in res)
        wall = max(r["wall"] for r in res)
        tt = [x for r in res for x in r["ttft"]]
        tp = [x for r in res for x in r["tpot"]]
        pulled = [r["pulled"] for r in res if r["pulled"]]
        value = n_out / (ms / 1e3)
        print(json.dumps({
            "metric": "output_tokens_per_s", "value": value, "unit": "tok/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None,
            "dtype": "bf16" if not mcfg.quantization else f"bf16+{mcfg.quantization}", "data": "synthetic",
            "impl": "ours",
            "config": config_block(args, world, {
                "decode_engine": f"{'ep' if ep or args.parallelism == 'ep' else 'tp'}{half}",
                "kv_transfer": "NVLinkConnector (CUDA IPC peer mapping, gather/scatter kernel over NVLink)",
                "wave": wave, "waves": n_waves,
                "kv_blocks_pulled": sum(p.get("pulled_blocks", 0) for p in pulled),
                "kv_pull_failures": sum(p.get("failed", 0) for p in pulled)}),
            "p50_ttft_s": statistics.median(tt) if tt else None,
            "p50_tpot_s": statistics.median(tp) if tp else None,
            "clocks": clocks,
            "e2e": {"value": n_out / wall, "unit": "tok/s",
                    "h2d_bytes_per_step": None, "d2h_bytes_per_step": None,
                    "note": "host clock around the pass incl. the hand-off between the two engines"},
            "gpu_launches": eng.runner.total_launches(),
        }), flush=True)
    # the store lives in rank 0: it leaves last
    store.add("leaving", 1)
    if rank == 0:
        while int(store.add("leaving", 0)) < world:
            time.sleep(0.002)
    sys.stdout.flush()
    os._exit(0)
