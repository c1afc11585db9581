"""LoRA: gather-matvec ops against dense math, and engine generation with adapters against
the same model with the adapter merged into its weights (CPU fp32)."""
import numpy as np
import pytest
import torch

from vllm_ascend_b200 import LLM, SamplingParams
from vllm_ascend_b200.lora import ops as lops
from vllm_ascend_b200.lora.manager import LoRARequest
from vllm_ascend_b200.lora.punica import PunicaWrapperB200


def test_bgmv_and_sgmv_match_dense():
    g = torch.Generator().manual_seed(0)
    T, K, N, S, r = 21, 64, 48, 3, 8
    x = torch.randn(T, K, generator=g)
    A = torch.randn(S, 2 * r, K, generator=g) * 0.1
    B0 = torch.randn(S, N, r, generator=g) * 0.1
    B1 = torch.randn(S, N // 2, r, generator=g) * 0.1
    lens, slots = [5, 9, 7], [1, -1, 2]
    tok_slots = torch.tensor(np.repeat(slots, lens), dtype=torch.int32)
    y0 = torch.randn(T, N + N // 2, generator=g)
    want = y0.clone()
    for t in range(T):
        s = int(tok_slots[t])
        if s < 0:
            continue
        v = 0.5 * (A[s] @ x[t])
        want[t, :N] += B0[s] @ v[:r]
        want[t, N:] += B1[s] @ v[r:]
    v = lops.bgmv_shrink(x, A, tok_slots, 0.5)
    y = y0.clone()
    lops.bgmv_expand(v, B0, tok_slots, y, 0, 0)
    lops.bgmv_expand(v, B1, tok_slots, y, N, r)
    assert torch.allclose(y, want, atol=1e-5)
    seg = lops.Segments([0, 5, 14], lens, slots, torch.device("cpu"))
    assert seg.num_tiles == 1 + 2 + 1 and seg.num_tokens == T
    v2 = lops.sgmv_shrink(x, A, seg, 0.5)
    y2 = y0.clone()
    lops.sgmv_expand(v2, B0, seg, y2, 0, 0)
    lops.sgmv_expand(v2, B1, seg, y2, N, r)
    assert torch.allclose(y2, want, atol=1e-5)
    # the wrapper picks segments for prefill-shaped steps and per-token slots for decode
    pw = PunicaWrapperB200(64, 8, "cpu")
    pw.update_metadata(slots, lens)
    y3 = y0.clone()
    pw.add_lora_linear(y3, x, A, [B0, B1], 0.5, [N, N // 2], r)
    assert torch.allclose(y3, want, atol=1e-5)
    pw.update_metadata([-1, -1], [1, 1])
    assert not pw.any_active


def _adapter(cfg, rank, seed, targets=("q_proj", "k_proj", "v_proj", "o_proj", "gate_proj", "up_proj", "down_proj")):
    g = torch.Generator().manual_seed(seed)
    H, I = cfg.hidden_size, cfg.intermediate_size
    q, kv = cfg.num_attention_heads * cfg.head_dim, cfg.num_key_value_heads * cfg.head_dim
    dims = {"q_proj": (H, q), "k_proj": (H, kv), "v_proj": (H, kv), "o_proj": (q, H),
            "gate_proj": (H, I), "up_proj": (H, I), "down_proj": (I, H)}
    t = {}
    for li in range(cfg.num_hidden_layers):
        for name in targets:
            k, n = dims[name]
            mod = "self_attn" if name in ("q_proj", "k_proj", "v_proj", "o_proj") else "mlp"
            base = f"base_model.model.model.layers.{li}.{mod}.{name}"
            t[f"{base}.lora_A.weight"] = torch.randn(rank, k, generator=g) * 0.2
            t[f"{base}.lora_B.weight"] = torch.randn(n, rank, generator=g) * 0.2
    return t


def _merged_state(llm, adapter, rank, alpha):
    from vllm_ascend_b200.models.transformer import export_hf_state_dict
    sd = export_hf_state_dict(llm.engine.runner.model)
    for name, a in adapter.items():
        if "lora_A" not in name:
            continue
        b = adapter[name.replace("lora_A", "lora_B")]
        key = name.replace("base_model.model.", "").replace(".lora_A.weight", ".weight")
        sd[key] = sd[key].float() + (alpha / rank) * (b @ a)
    return sd


def test_engine_lora_matches_merged_weights_and_mixed_batches():
    kw = dict(device="cpu", seed=0, block_size=16, max_model_len=128, max_num_seqs=8)
    llm = LLM("tiny-qwen", enable_lora=True, max_loras=2, max_lora_rank=8, **kw)
    cfg = llm.cfg.model
    ad1, ad2 = _adapter(cfg, 8, 1), _adapter(cfg, 4, 2, targets=("q_proj", "v_proj", "down_proj"))
    r1 = LoRARequest("a1", 1, tensors=ad1, rank=8, alpha=16.0)
    r2 = LoRARequest("a2", 2, tensors=ad2, rank=4, alpha=4.0)
    rng = np.random.default_rng(0)
    prompts = [rng.integers(1, 500, size=n).tolist() for n in (19, 33, 7, 26)]
    sp = SamplingParams(max_tokens=6, temperature=0.0, ignore_eos=True)
    got = llm.generate(prompts, sp, lora_request=[r1, None, r2, r1])
    toks = [o.outputs[0].token_ids for o in got]
    assert llm.engine.runner.lora_manager.list() == {1, 2}

    def oracle(adapter, rank, alpha, idx):
        ref = LLM("tiny-qwen", **kw)
        if adapter is not None:
            ref.engine.runner.model.load_weights(_merged_state(ref, adapter, rank, alpha).items())
        return [o.outputs[0].token_ids for o in ref.generate([prompts[i] for i in idx], sp)]
    assert [toks[0], toks[3]] == oracle(ad1, 8, 16.0, [0, 3])
    assert [toks[1]] == oracle(None, 0, 0, [1])
    assert [toks[2]] == oracle(ad2, 4, 4.0, [2])
    # the adapters really change the output
    assert toks[0] != oracle(None, 0, 0, [0])[0]


def test_lora_slot_eviction_and_pinning():
    llm = LLM("tiny-qwen", device="cpu", seed=0, block_size=16, max_model_len=64, max_num_seqs=4,
              enable_lora=True, max_loras=2, max_lora_rank=8)
    mgr = llm.engine.runner.lora_manager
    cfg = llm.cfg.model
    reqs = [LoRARequest(f"a{i}", i, tensors=_adapter(cfg, 4, i, targets=("q_proj",)), rank=4, alpha=4.0)
            for i in (1, 2, 3)]
    assert mgr.add(reqs[0]) and mgr.add(reqs[1])
    assert mgr.pin(1)
    assert mgr.add(reqs[2])                      # evicts adapter 2 (1 is pinned)
    assert mgr.list() == {1, 3}
    assert not mgr.add(reqs[1], in_use={3})      # 1 pinned, 3 in use: nowhere to go
    assert mgr.remove(3) and mgr.add(reqs[1]) and mgr.list() == {1, 2}
    with pytest.raises(ValueError):
        mgr.add(LoRARequest("big", 9, tensors=_adapter(cfg, 16, 9, targets=("q_proj",)), rank=16, alpha=16.0),
                in_use=set()) if mgr.remove(2) else None
    with pytest.raises(ValueError):
        LLM("tiny-qwen", device="cpu", seed=0, block_size=16, max_model_len=64, max_num_seqs=4) \
            .engine.add_request([1, 2, 3], SamplingParams(max_tokens=1), lora_request=reqs[0])


def test_expert_lora_matches_merged_expert_weights():
    """Adapters on routed experts (gate / up / down of every expert) plus attention projections:
    mixed batch of adapter and plain requests equals engines with the deltas merged into the weights."""
    kw = dict(device="cpu", seed=0, block_size=16, max_model_len=128, max_num_seqs=8)
    llm = LLM("tiny-moe", enable_lora=True, max_loras=2, max_lora_rank=8, **kw)
    cfg = llm.cfg.model
    assert llm.engine.runner.lora_manager.moe_layers and not llm.engine.runner.lora_manager.graph_safe
    g = torch.Generator().manual_seed(5)
    rank, alpha = 4, 8.0
    H, I = cfg.hidden_size, cfg.moe_intermediate_size
    ad = _adapter(cfg, rank, 9, targets=("q_proj", "o_proj"))
    for li in range(cfg.num_hidden_layers):
        for e in range(cfg.num_experts):
            base = f"base_model.model.model.layers.{li}.mlp.experts.{e}"
            for name, (k, n) in (("gate_proj", (H, I)), ("up_proj", (H, I)), ("down_proj", (I, H))):
                ad[f"{base}.{name}.lora_A.weight"] = torch.randn(rank, k, generator=g) * 0.3
                ad[f"{base}.{name}.lora_B.weight"] = torch.randn(n, rank, generator=g) * 0.3
    req = LoRARequest("moe", 7, tensors=ad, rank=rank, alpha=alpha)
    rng = np.random.default_rng(1)
    prompts = [rng.integers(1, 500, size=n).tolist() for n in (23, 9, 31)]
    sp = SamplingParams(max_tokens=5, temperature=0.0, ignore_eos=True)
    toks = [o.outputs[0].token_ids for o in llm.generate(prompts, sp, lora_request=[req, None, req])]

    def oracle(adapter, idx):
        ref = LLM("tiny-moe", **kw)
        if adapter is not None:
            ref.engine.runner.model.load_weights(_merged_state(ref, adapter, rank, alpha).items())
        return [o.outputs[0].token_ids for o in ref.generate([prompts[i] for i in idx], sp)]
    assert [toks[0], toks[2]] == oracle(ad, [0, 2])
    assert [toks[1]] == oracle(None, [1])
    assert toks[0] != oracle(None, [0])[0]


_EP_WORKER = """
import json, os, sys
import numpy as np, torch
sys.path.insert(0, {root!r})
from vllm_ascend_b200 import LLM, SamplingParams
from vllm_ascend_b200.lora.manager import LoRARequest
ep = int(os.environ.get("WORLD_SIZE", "1")) > 1
llm = LLM("tiny-moe", device="cpu", seed=0, block_size=16, max_model_len=128, max_num_seqs=8, enable_lora=True,
          max_loras=2, max_lora_rank=8, tensor_parallel_size=2 if ep else 1, enable_expert_parallel=ep)
cfg = llm.cfg.model
mgr = llm.engine.runner.lora_manager
assert mgr.moe_layers
if ep:
    ms = next(iter(mgr.moe_layers.values()))
    assert ms.num_experts == cfg.num_experts // 2 and not ms.sharded and ms.expert_map.count(-1) == cfg.num_experts // 2
g = torch.Generator().manual_seed(5)
rank, alpha = 4, 8.0
H, I = cfg.hidden_size, cfg.moe_intermediate_size
ad = dict()
for li in range(cfg.num_hidden_layers):
    for e in range(cfg.num_experts):
        base = "base_model.model.model.layers.%d.mlp.experts.%d" % (li, e)
        for name, (k, n) in (("gate_proj", (H, I)), ("up_proj", (H, I)), ("down_proj", (I, H))):
            ad[base + "." + name + ".lora_A.weight"] = torch.randn(rank, k, generator=g) * 0.3
            ad[base + "." + name + ".lora_B.weight"] = torch.randn(n, rank, generator=g) * 0.3
req = LoRARequest("moe", 7, tensors=ad, rank=rank, alpha=alpha)
rng = np.random.default_rng(1)
prompts = [rng.integers(1, 500, size=n).tolist() for n in (23, 9, 31)]
sp = SamplingParams(max_tokens=5, temperature=0.0, ignore_eos=True)
toks = [o.outputs[0].token_ids for o in llm.generate(prompts, sp, lora_request=[req, None, req])]
if int(os.environ.get("RANK", "0")) == 0:
    rt = llm.engine.runner.moe_runtime
    print("RESULT " + json.dumps([toks, dict((k.name, v) for k, v in rt.counts.items()) if rt else None]), flush=True)
llm.shutdown()
sys.stdout.flush()
os._exit(0)
"""


@pytest.mark.parametrize("method", ["allgather", "alltoall"])
def test_expert_lora_under_expert_parallelism_matches_single_rank(method):
    """Each EP rank keeps the adapters of its own experts; the adapter slot travels with the token on
    both the all-gather and the all-to-all path."""
    import json
    import os
    import socket
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    script = _EP_WORKER.format(root=root)

    def run(world):
        with socket.socket() as s:
            s.bind(("127.0.0.1", 0))
            port = s.getsockname()[1]
        env = dict(os.environ, MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), WORLD_SIZE=str(world),
                   OMP_NUM_THREADS="2", VLLM_B200_MOE_COMM=method)
        procs = [subprocess.Popen([sys.executable, "-c", script], env=dict(env, RANK=str(r), LOCAL_RANK=str(r)),
                                  stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True) for r in range(world)]
        outs = [p.communicate(timeout=300) for p in procs]
        for p, (o, e) in zip(procs, outs):
            assert p.returncode == 0, e[-3000:]
        return json.loads([l for l in outs[0][0].splitlines() if l.startswith("RESULT ")][-1][7:])
    single, _ = run(1)
    ep, counts = run(2)
    assert ep == single
    assert counts[method.upper()] > 0
