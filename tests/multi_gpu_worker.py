"""Worker for the multi-GPU tests; launched with torchrun, one rank per GPU.

    torchrun --nproc-per-node 2 tests/multi_gpu_worker.py tp_generate
Rank 0 prints one JSON line with the result."""
import json
import os
import sys

import numpy as np
import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def _cfg():
    from vllm_ascend_b200.config import ModelConfig
    # WIDE=1: enough heads for 8-way tensor parallelism
    wide = os.environ.get("WIDE", "0") == "1"
    if os.environ.get("MQA", "0") == "1":       # one KV head, replicated over the TP ranks
        return ModelConfig(name="t", architecture="Qwen3ForCausalLM", vocab_size=2048, hidden_size=512,
                           intermediate_size=1024, num_hidden_layers=3, num_attention_heads=8, num_key_value_heads=1,
                           head_dim=128, qk_norm=True, rope_theta=1e6, dtype="bfloat16", init_std=0.05)
    return ModelConfig(name="t", architecture="Qwen3ForCausalLM", vocab_size=2048, hidden_size=1024 if wide else 512,
                       intermediate_size=2048 if wide else 1024, num_hidden_layers=3,
                       num_attention_heads=16 if wide else 8, num_key_value_heads=8 if wide else 2, head_dim=128,
                       qk_norm=True, rope_theta=1e6, dtype="bfloat16", init_std=0.05)


def tp_generate():
    from vllm_ascend_b200.engine.llm import LLM
    from vllm_ascend_b200.engine.request import SamplingParams
    world = int(os.environ["WORLD_SIZE"])
    rng = np.random.default_rng(0)
    prompts = [rng.integers(0, 2048, size=n).tolist() for n in (150, 40, 333, 129, 7)]
    sp = SamplingParams(temperature=0.0, max_tokens=10, ignore_eos=True)
    pcp = int(os.environ.get("PCP", "1"))
    dcp = int(os.environ.get("DCP", "1"))
    llm = LLM(_cfg(), device="cuda", tensor_parallel_size=world // pcp, prefill_context_parallel_size=pcp,
              decode_context_parallel_size=dcp,
              max_model_len=512, max_num_seqs=8,
              max_num_batched_tokens=256, num_gpu_blocks_override=40,
              enforce_eager=os.environ.get("EAGER", "0") == "1", cudagraph_capture_sizes=[2, 4, 8])
    outs = llm.generate(prompts, sp)
    toks = [o.outputs[0].token_ids for o in outs]
    fused = llm.engine.runner.model.sp_ctx is not None
    if fused:
        llm.engine.runner.model.sp_ctx.check()
    nvls = bool(fused and llm.engine.runner.model.sp_ctx.nvls)
    # log-probabilities of the first generated token (top 8): compared across the communication paths
    lp = llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=1, ignore_eos=True, logprobs=8))
    first_lp = [{str(k): float(v) for k, v in o.outputs[0].logprobs[0].items()} for o in lp]
    if fused:
        llm.engine.runner.model.sp_ctx.check()
    return {"tokens": toks, "fused": fused, "nvls": nvls, "replays": llm.engine.runner.stats["graph_replays"],
            "first_logprobs": first_lp}


def fused_linear_ops():
    """AG->GEMM and GEMM->RS (+ reduce / norm / push) of the fused TP dataflow against fp32 math, at
    row counts that take the paired-CTA kernels (ragged last tile, columns not a multiple of 64)."""
    from vllm_ascend_b200 import _native
    from vllm_ascend_b200.parallel import state as pstate
    from vllm_ascend_b200.parallel.fused_linear import FusedTPContext
    rank, local, world = pstate.init_distributed()
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    st = pstate.initialize_model_parallel(tp=world)
    errs = []
    for T, H, K in ((1000, 1024, 512), (4096, 2048 + 32, 768), (300, 512, 256)):
        ctx = FusedTPContext(st.tp, dev, T + world, H)
        Tp, rl = ctx.begin(T)
        g = torch.Generator(device="cpu").manual_seed(7)
        x_full = (torch.randn(Tp, K * world, generator=g) * 0.5).bfloat16()      # [T, K_total], this rank holds a K slice
        w_full = (torch.randn(H, K * world, generator=g) * 0.05).bfloat16()
        res_full = (torch.randn(Tp, H, generator=g) * 0.5).bfloat16()
        norm_w = (torch.rand(H, generator=g) + 0.5).bfloat16()
        x = x_full[:, rank * K:(rank + 1) * K].contiguous().to(dev)
        w = w_full[:, rank * K:(rank + 1) * K].contiguous().to(dev)
        ctx.residual[:rl].copy_(res_full[rank * rl:(rank + 1) * rl].to(dev))
        for _ in range(2):                                   # epochs advance: run twice
            ctx.residual[:rl].copy_(res_full[rank * rl:(rank + 1) * rl].to(dev))
            ctx.gemm_rs(x, w)
            ctx.norm_push(norm_w.to(dev), 1e-6)
            got = ctx.gathered().float().cpu()
        ctx.check()
        y = (x_full.float() @ w_full.float().t()).bfloat16().float() + res_full.float()
        y = y.bfloat16().float()
        want = (y * torch.rsqrt((y * y).mean(-1, keepdim=True) + 1e-6) * norm_w.float()).bfloat16().float()
        errs.append(float((got[:T] - want[:T]).abs().max() / want[:T].abs().max()))
        # all-gather -> GEMM on the gathered rows
        w2 = (torch.randn(384, H, generator=g) * 0.05).bfloat16()
        out = ctx.ag_gemm(w2.to(dev)).float().cpu()
        ctx.check()
        want2 = got @ w2.float().t()
        errs.append(float((out[:T] - want2[:T]).abs().max() / want2[:T].abs().max()))
    torch.cuda.synchronize()
    all_errs = [None] * world
    torch.distributed.all_gather_object(all_errs, errs)        # every rank checked its own copy
    return {"max_rel_err": max(max(e) for e in all_errs), "errs": errs, "nvls": bool(ctx.nvls)}


def symm_allreduce():
    """One-shot all-reduce and barrier over peer memory vs NCCL."""
    import ctypes
    from vllm_ascend_b200 import _native
    from vllm_ascend_b200.parallel import state as pstate
    from vllm_ascend_b200.parallel.symm_mem import SymmetricMemory
    rank, local, world = pstate.init_distributed()
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    st = pstate.initialize_model_parallel(tp=world)
    n = 1 << 16
    sm = SymmetricMemory(st.tp, dev, n * 2)
    off = sm.region(n * 2)
    buf = sm.tensor(off, (n,), torch.bfloat16)
    errs = []
    for it in range(3):
        g = torch.Generator(device="cpu").manual_seed(100 * it + rank)
        x = torch.randn(n, generator=g).bfloat16().to(dev)
        buf.copy_(x)
        out = torch.empty_like(x)
        rc = _native.lib().b200_allreduce_oneshot(sm.ptr_array(off), sm.ctl_ptrs, out.data_ptr(), n,
                                                  sm.rank, world, _native.stream_ptr())
        assert rc == 0
        ref = x.float().clone()
        torch.distributed.all_reduce(ref)
        torch.cuda.synchronize()
        errs.append(float((out.float() - ref).abs().max()))
    sm.barrier()
    torch.cuda.synchronize()
    status = sm.read_status()
    return {"max_err": max(errs), "status": status}


def moe_fused():
    """Fused dispatch/GEMM/combine over peer memory vs a dense fp32 oracle that holds every
    expert; uneven token counts per rank, padded (-1) routes, eager and graph replay."""
    from types import SimpleNamespace
    from vllm_ascend_b200 import _native
    from vllm_ascend_b200.config import ModelConfig, EngineConfig
    from vllm_ascend_b200.ops.moe_fused import FusedMoEComm
    from vllm_ascend_b200.parallel import state as pstate
    rank, local, world = pstate.init_distributed()
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    _native.load(required=True)
    st = pstate.initialize_model_parallel(tp=1, dp=world)
    ep = pstate.get_ep_group() if pstate.get_ep_group().world_size == world else pstate.get_world_group()
    E, topk, H, I = 8 * world, 4, 512, 256
    mc = SimpleNamespace(hidden_size=H, moe_intermediate_size=I, num_experts=E, num_experts_per_tok=topk)
    comm = FusedMoEComm(SimpleNamespace(model=mc), dev, ep, capacity=64)
    g = torch.Generator(device="cpu").manual_seed(1)
    w13_full = (torch.randn(E, 2 * I, H, generator=g) * 0.05).bfloat16()
    w2_full = (torch.randn(E, H, I, generator=g) * 0.05).bfloat16()
    El = E // world
    block = SimpleNamespace(w13=w13_full[rank * El:(rank + 1) * El].contiguous().to(dev),
                            w2=w2_full[rank * El:(rank + 1) * El].contiguous().to(dev), quant=None)

    def oracle(x, w, ids):
        out = torch.zeros(x.shape[0], H)
        for t in range(x.shape[0]):
            for k in range(topk):
                e = int(ids[t, k])
                if e < 0:
                    continue
                h = w13_full[e].float() @ x[t].float()
                a = (torch.nn.functional.silu(h[:I]) * h[I:]).bfloat16().float()
                out[t] += float(w[t, k]) * (w2_full[e].float() @ a).bfloat16().float()
        return out

    errs = []
    token_counts = [[5, 64], [0, 17], [33, 1], [64, 64]]
    for it, cnt in enumerate(token_counts):
        T = cnt[rank % 2]
        gi = torch.Generator(device="cpu").manual_seed(10 * it + rank)
        x = (torch.randn(T, H, generator=gi) * 0.5).bfloat16()
        ids = torch.stack([torch.randperm(E, generator=gi)[:topk] for _ in range(T)]).int() if T else \
            torch.zeros(0, topk, dtype=torch.int32)
        if T > 2:
            ids[1, 2:] = -1            # padded routes
        w = torch.rand(T, topk, generator=gi)
        y = comm.forward(block, x.to(dev), w.to(dev), ids.to(dev))
        torch.cuda.synchronize()
        ref = oracle(x, w, ids)
        if T:
            errs.append(float((y.float().cpu() - ref).abs().max() / (ref.abs().max() + 1e-6)))
    # graph capture + replay of the four launches
    T = 16
    gi = torch.Generator(device="cpu").manual_seed(99 + rank)
    xs = (torch.randn(T, H, generator=gi) * 0.5).bfloat16().to(dev)
    ids = torch.stack([torch.randperm(E, generator=gi)[:topk] for _ in range(T)]).int().to(dev)
    w = torch.rand(T, topk, generator=gi).to(dev)
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        comm.forward(block, xs, w, ids)
    torch.cuda.current_stream().wait_stream(s)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        yg = comm.forward(block, xs, w, ids)
    for rep in range(2):
        xs.copy_((torch.randn(T, H, generator=gi) * 0.5).bfloat16())
        graph.replay()
        torch.cuda.synchronize()
        ref = oracle(xs.cpu(), w.cpu(), ids.cpu())
        errs.append(float((yg.float().cpu() - ref).abs().max() / (ref.abs().max() + 1e-6)))
    status = int(_native.status_word(dev).item())
    torch.distributed.barrier()
    graph = None
    all_errs = [None] * world
    torch.distributed.all_gather_object(all_errs, errs)
    return {"max_rel_err": max(max(e) for e in all_errs), "status": status, "calls": comm.calls}


def pp_generate():
    """Two pipeline stages on two GPUs (NCCL send / recv of hidden + residual, token broadcast)."""
    from vllm_ascend_b200.engine.llm import LLM
    from vllm_ascend_b200.engine.request import SamplingParams
    world = int(os.environ["WORLD_SIZE"])
    rng = np.random.default_rng(0)
    prompts = [rng.integers(0, 2048, size=n).tolist() for n in (150, 40, 333, 129, 7)]
    llm = LLM(_cfg(), device="cuda", tensor_parallel_size=1, pipeline_parallel_size=world, max_model_len=512,
              max_num_seqs=8, max_num_batched_tokens=256, num_gpu_blocks_override=40, enforce_eager=True)
    outs = llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=10, ignore_eos=True))
    lp = llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=1, ignore_eos=True, logprobs=8))
    return {"tokens": [o.outputs[0].token_ids for o in outs],
            "first_logprobs": [{str(k): float(v) for k, v in o.outputs[0].logprobs[0].items()} for o in lp]}


def weight_transfer():
    """RL weight update over NCCL: rank 0 is the trainer (holds other weights, serves no requests),
    rank 1 a live single-GPU engine that receives the buckets and applies them in place."""
    from vllm_ascend_b200.distributed.weight_transfer import NCCLWeightTransferEngine
    from vllm_ascend_b200.engine.llm import LLM
    from vllm_ascend_b200.engine.request import SamplingParams
    rank = int(os.environ["RANK"])
    port = int(os.environ["MASTER_PORT"]) + 17
    # each process is a world of its own for the engine; the transfer group spans both
    os.environ["WORLD_SIZE"], os.environ["RANK"] = "1", "0"
    os.environ["MASTER_PORT"] = str(int(os.environ["MASTER_PORT"]) + 31 + rank)
    torch.cuda.set_device(rank)
    cfg = _cfg()
    sp = SamplingParams(temperature=0.0, max_tokens=8, ignore_eos=True)
    prompts = [list(range(10, 90)), list(range(300, 340))]
    llm = LLM(cfg, device=f"cuda:{rank}", seed=42 if rank == 0 else 1, max_model_len=256, max_num_seqs=4, max_num_batched_tokens=128,
              num_gpu_blocks_override=16, enforce_eager=True)
    mine = [o.outputs[0].token_ids for o in llm.generate(prompts, sp)]
    eng = NCCLWeightTransferEngine("127.0.0.1", port, rank, 2, backend="nccl", bucket_bytes=4 << 20)
    if rank == 0:
        eng.send_weights(llm.engine.runner.model.named_parameters())
        out = {"trainer": mine, "buckets": eng.stats["buckets"]}
    else:
        w = llm.engine.worker
        w.start_weight_update()
        params = dict(w.runner.model.named_parameters())

        def apply(pairs):
            n = 0
            for name, tensor in pairs:
                params[name].copy_(tensor)
                n += 1
            return n
        n = eng.receive_weights(apply)
        w.finish_weight_update()
        llm.reset_prefix_cache()
        out = {"before": mine, "after": [o.outputs[0].token_ids for o in llm.generate(prompts, sp)], "applied": n,
               "params": len(params)}
    torch.cuda.synchronize()
    eng.close()
    # both sides report through files-free stdout lines; the test reads them per rank
    print("PART%d " % rank + json.dumps(out), flush=True)
    return out


if __name__ == "__main__":
    res = {"pp_generate": pp_generate, "weight_transfer": weight_transfer,
           "tp_generate": tp_generate, "symm_allreduce": symm_allreduce, "fused_linear_ops": fused_linear_ops, "moe_fused": moe_fused}[sys.argv[1]]()
    if int(os.environ.get("RANK", "0")) == 0:
        print("RESULT " + json.dumps(res), flush=True)
    if torch.distributed.is_initialized():
        torch.distributed.barrier()
        torch.distributed.destroy_process_group()
