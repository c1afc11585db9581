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
    return ModelConfig(name="t", architecture="Qwen3ForCausalLM", vocab_size=2048, hidden_size=512,
                       intermediate_size=1024, num_hidden_layers=3, num_attention_heads=8,
                       num_key_value_heads=2, head_dim=128, qk_norm=True, rope_theta=1e6,
                       dtype="bfloat16", init_std=0.05)


def tp_generate():
    from vllm_ascend_b200.engine.llm import LLM
    from vllm_ascend_b200.engine.request import SamplingParams
    world = int(os.environ["WORLD_SIZE"])
    rng = np.random.default_rng(0)
    prompts = [rng.integers(0, 2048, size=n).tolist() for n in (150, 40, 333, 129, 7)]
    sp = SamplingParams(temperature=0.0, max_tokens=10, ignore_eos=True)
    llm = LLM(_cfg(), device="cuda", tensor_parallel_size=world, max_model_len=512, max_num_seqs=8,
              max_num_batched_tokens=256, num_gpu_blocks_override=40,
              enforce_eager=os.environ.get("EAGER", "0") == "1", cudagraph_capture_sizes=[2, 4, 8])
    outs = llm.generate(prompts, sp)
    toks = [o.outputs[0].token_ids for o in outs]
    fused = llm.engine.runner.model.sp_ctx is not None
    if fused:
        llm.engine.runner.model.sp_ctx.check()
    return {"tokens": toks, "fused": fused, "replays": llm.engine.runner.stats["graph_replays"]}


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


if __name__ == "__main__":
    res = {"tp_generate": tp_generate, "symm_allreduce": symm_allreduce}[sys.argv[1]]()
    if int(os.environ.get("RANK", "0")) == 0:
        print("RESULT " + json.dumps(res), flush=True)
    if torch.distributed.is_initialized():
        torch.distributed.barrier()
        torch.distributed.destroy_process_group()
