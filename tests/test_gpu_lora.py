"""LoRA kernels on the GPU against fp32 math; engine with adapters under CUDA graphs."""
import numpy as np
import pytest
import torch

from vllm_ascend_b200 import _native
from vllm_ascend_b200.lora import ops as lops

pytestmark = pytest.mark.gpu


def _ref(x, A, Bs, tok_slots, y0, scale, r, offs):
    want = y0.float().clone()
    for t in range(x.shape[0]):
        s = int(tok_slots[t])
        if s < 0:
            continue
        v = scale * (A[s].float() @ x[t].float())
        for i, (B, off) in enumerate(zip(Bs, offs)):
            want[t, off:off + B.shape[1]] += B[s].float() @ v[i * r:(i + 1) * r]
    return want


@pytest.mark.parametrize("r", [8, 16, 64])
def test_bgmv_sgmv_kernels(r):
    dev = torch.device("cuda")
    g = torch.Generator(device="cpu").manual_seed(r)
    K, S = 4096, 4
    Ns = [4096, 1024, 1024]
    lens = [1, 37, 8, 130, 3]
    slots = [2, 0, -1, 3, 1]
    T = sum(lens)
    x = (torch.randn(T, K, generator=g) * 0.5).to(torch.bfloat16).to(dev)
    A = (torch.randn(S, 3 * r, K, generator=g) * 0.05).to(torch.bfloat16).to(dev)
    Bs = [(torch.randn(S, n, r, generator=g) * 0.05).to(torch.bfloat16).to(dev) for n in Ns]
    y0 = (torch.randn(T, sum(Ns), generator=g)).to(torch.bfloat16).to(dev)
    tok_slots = torch.tensor(np.repeat(slots, lens), dtype=torch.int32, device=dev)
    offs = [0, Ns[0], Ns[0] + Ns[1]]
    want = _ref(x.cpu(), A.cpu(), [b.cpu() for b in Bs], tok_slots.cpu(), y0.cpu(), 0.5, r, offs)
    # bgmv
    v = lops.bgmv_shrink(x, A, tok_slots, 0.5)
    y = y0.clone()
    for i, (B, off) in enumerate(zip(Bs, offs)):
        lops.bgmv_expand(v, B, tok_slots, y, off, i * r)
    torch.cuda.synchronize()
    _native.check_status(dev)
    assert (y.float().cpu() - want).abs().max() < 0.06
    # rows without an adapter are untouched bit for bit
    none = (tok_slots < 0).cpu()
    assert torch.equal(y.cpu()[none], y0.cpu()[none])
    # sgmv
    starts = np.concatenate([[0], np.cumsum(lens)[:-1]])
    seg = lops.Segments(starts, lens, slots, dev)
    v2 = lops.sgmv_shrink(x, A, seg, 0.5)
    y2 = y0.clone()
    for i, (B, off) in enumerate(zip(Bs, offs)):
        lops.sgmv_expand(v2, B, seg, y2, off, i * r)
    torch.cuda.synchronize()
    _native.check_status(dev)
    assert (y2.float().cpu() - want).abs().max() < 0.06
    act = ~none
    assert torch.allclose(v2.cpu()[act], v.cpu()[act], rtol=1e-3, atol=1e-3)


def test_engine_lora_graph_equals_eager():
    import sys, os
    sys.path.insert(0, os.path.dirname(__file__))
    from test_lora_cpu import _adapter
    from test_gpu_engine import _cfg
    from vllm_ascend_b200.engine.llm import LLM
    from vllm_ascend_b200.engine.request import SamplingParams
    from vllm_ascend_b200.lora.manager import LoRARequest
    cfg = _cfg("bfloat16")
    ad = _adapter(cfg, 8, 3)
    ad = {k: v * 0.3 for k, v in ad.items()}
    req = LoRARequest("a", 1, tensors=ad, rank=8, alpha=8.0)
    rng = np.random.default_rng(0)
    prompts = [rng.integers(0, 2048, size=n).tolist() for n in (150, 40, 200)]
    sp = SamplingParams(temperature=0.0, max_tokens=10, ignore_eos=True)
    outs = {}
    for eager in (True, False):
        llm = LLM(_cfg("bfloat16"), device="cuda", max_model_len=512, max_num_seqs=8, max_num_batched_tokens=256,
                  num_gpu_blocks_override=40, enforce_eager=eager, cudagraph_capture_sizes=[2, 4],
                  enable_lora=True, max_loras=2, max_lora_rank=8)
        outs[eager] = [o.outputs[0].token_ids for o in llm.generate(prompts, sp, lora_request=[req, None, req])]
        if not eager:
            assert llm.engine.runner.stats["graph_replays"] > 0
        base = [o.outputs[0].token_ids for o in llm.generate(prompts, sp)]
        assert base[1] == outs[eager][1]            # the request without adapter is unaffected
        assert base[0] != outs[eager][0]            # the adapter changes the output
    assert outs[True] == outs[False]


def test_expert_lora_on_gpu():
    """Adapters on routed experts through the batched LoRA kernels with (slot, expert) indices; plain
    requests of the same batch are untouched, graph decode still serves steps without adapters."""
    from vllm_ascend_b200.config import ModelConfig
    from vllm_ascend_b200.engine.llm import LLM
    from vllm_ascend_b200.engine.request import SamplingParams
    from vllm_ascend_b200.lora.manager import LoRARequest

    def cfg():
        return ModelConfig(name="moe-t", architecture="Qwen3MoeForCausalLM", vocab_size=2048, hidden_size=512,
                           intermediate_size=1024, num_hidden_layers=2, num_attention_heads=8, num_key_value_heads=2,
                           head_dim=128, qk_norm=True, rope_theta=1e6, dtype="bfloat16", init_std=0.05,
                           num_experts=8, num_experts_per_tok=2, moe_intermediate_size=256)
    c = cfg()
    g = torch.Generator().manual_seed(0)
    rank, H, I = 8, c.hidden_size, c.moe_intermediate_size
    ad = {}
    for li in range(c.num_hidden_layers):
        for e in range(c.num_experts):
            base = f"base_model.model.model.layers.{li}.mlp.experts.{e}"
            for name, (k, n) in (("gate_proj", (H, I)), ("up_proj", (H, I)), ("down_proj", (I, H))):
                ad[f"{base}.{name}.lora_A.weight"] = torch.randn(rank, k, generator=g) * 0.1
                ad[f"{base}.{name}.lora_B.weight"] = torch.randn(n, rank, generator=g) * 0.1
    req = LoRARequest("moe", 1, tensors=ad, rank=rank, alpha=16.0)
    rng = np.random.default_rng(0)
    prompts = [rng.integers(0, 2048, size=n).tolist() for n in (150, 40, 200)]
    sp = SamplingParams(temperature=0.0, max_tokens=8, ignore_eos=True)
    llm = LLM(cfg(), device="cuda", max_model_len=512, max_num_seqs=8, max_num_batched_tokens=256,
              num_gpu_blocks_override=40, cudagraph_capture_sizes=[2, 4], enable_lora=True, max_loras=2, max_lora_rank=8)
    mixed = [o.outputs[0].token_ids for o in llm.generate(prompts, sp, lora_request=[req, None, req])]
    replays = llm.engine.runner.stats["graph_replays"]
    base = [o.outputs[0].token_ids for o in llm.generate(prompts, sp)]
    assert llm.engine.runner.stats["graph_replays"] > replays       # adapter-free decode steps replay graphs
    assert base[1][0] == mixed[1][0]
    assert base[0] != mixed[0] and base[2] != mixed[2]
    from vllm_ascend_b200 import _native
    _native.check_status(torch.device("cuda"))
