"""Gated DeltaNet kernels against their PyTorch definitions; hybrid model on the engine."""
import numpy as np
import pytest
import torch

from vllm_ascend_b200 import _native
from vllm_ascend_b200.ops import linear_attn as la

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _seqs():
    lens = [1, 37, 128, 5]
    cu = torch.tensor(np.concatenate([[0], np.cumsum(lens)]), dtype=torch.int32)
    slots = torch.tensor([3, 0, 5, 1], dtype=torch.int32)
    has_init = torch.tensor([1, 0, 1, 0], dtype=torch.int32)
    return lens, cu, slots, has_init


@pytest.mark.parametrize("K", [4, 3])
def test_causal_conv1d_kernel(K):
    g = torch.Generator().manual_seed(0)
    lens, cu, slots, has_init = _seqs()
    T, C = sum(lens), 384
    x = torch.randn(T, C, generator=g).bfloat16()
    w = (torch.randn(C, K, generator=g) * 0.5).bfloat16()
    b = torch.randn(C, generator=g).bfloat16()
    st = torch.randn(6, K - 1, C, generator=g).bfloat16()
    st_ref = st.clone().float()
    want = la.causal_conv1d_ref(x.float(), w.float(), b.float(), st_ref, cu, slots, has_init)
    st_dev = st.to(DEV)
    got = la.causal_conv1d(x.to(DEV), w.to(DEV), b.to(DEV), st_dev, cu.to(DEV), slots.to(DEV), has_init.to(DEV))
    torch.cuda.synchronize()
    _native.check_status(torch.device(DEV))
    assert torch.allclose(got.float().cpu(), want, atol=3e-2, rtol=3e-2)
    assert torch.allclose(st_dev.float().cpu(), st_ref, atol=1e-2)


@pytest.mark.parametrize("Hk,Hv,DK,DV", [(2, 4, 128, 128), (4, 4, 64, 64), (2, 2, 64, 128)])
def test_gated_delta_rule_kernel(Hk, Hv, DK, DV):
    g = torch.Generator().manual_seed(1)
    lens, cu, slots, has_init = _seqs()
    T = sum(lens)
    q = torch.randn(T, Hk, DK, generator=g).bfloat16()
    k = torch.randn(T, Hk, DK, generator=g).bfloat16()
    v = torch.randn(T, Hv, DV, generator=g).bfloat16()
    gg = -torch.rand(T, Hv, generator=g) * 0.3
    beta = torch.rand(T, Hv, generator=g)
    S = torch.randn(6, Hv, DK, DV, generator=g) * 0.1
    S_ref = S.clone()
    want = la.gated_delta_rule_ref(q.float(), k.float(), v.float(), gg, beta, S_ref, cu, slots, has_init, DK ** -0.5)
    S_dev = S.to(DEV)
    got = la.gated_delta_rule(q.to(DEV), k.to(DEV), v.to(DEV), gg.to(DEV), beta.to(DEV), S_dev, cu.to(DEV),
                              slots.to(DEV), has_init.to(DEV), DK ** -0.5)
    torch.cuda.synchronize()
    _native.check_status(torch.device(DEV))
    assert (got.float().cpu() - want).abs().max() < 3e-2
    assert (S_dev.cpu() - S_ref).abs().max() < 2e-2


def test_chunk_parallel_delta_rule_on_device(monkeypatch):
    """bf16 inputs on the device (the form is opt-in there): the chunked form (fp32 matrix products) and the recurrence kernel
    both against the fp32 definition, mixed step routed by sequence length."""
    monkeypatch.setenv("VLLM_B200_GDN_CHUNK_MIN", "64")
    g = torch.Generator().manual_seed(4)
    lens = [300, 1, 64, 130, 2]
    cu_h = np.concatenate([[0], np.cumsum(lens)]).astype(np.int64)
    cu = torch.tensor(cu_h, dtype=torch.int32)
    slots = torch.tensor([3, 0, 5, 1, 2], dtype=torch.int32)
    has_init = torch.tensor([1, 1, 0, 1, 0], dtype=torch.int32)
    Hk, Hv, DK, DV = 2, 4, 128, 128
    T = sum(lens)
    q = torch.randn(T, Hk, DK, generator=g).bfloat16()
    k = torch.randn(T, Hk, DK, generator=g).bfloat16()
    v = torch.randn(T, Hv, DV, generator=g).bfloat16()
    gg = -torch.rand(T, Hv, generator=g) * 0.3
    beta = torch.rand(T, Hv, generator=g)
    S = torch.randn(6, Hv, DK, DV, generator=g) * 0.1
    S_ref = S.clone()
    want = la.gated_delta_rule_ref(q.float(), k.float(), v.float(), gg, beta, S_ref, cu, slots, has_init, DK ** -0.5)
    S_dev = S.to(DEV)
    got = la.gated_delta_rule(q.to(DEV), k.to(DEV), v.to(DEV), gg.to(DEV), beta.to(DEV), S_dev, cu.to(DEV),
                              slots.to(DEV), has_init.to(DEV), DK ** -0.5, cu_cpu=cu_h)
    torch.cuda.synchronize()
    _native.check_status(torch.device(DEV))
    assert (got.float().cpu() - want).abs().max() < 3e-2
    assert (S_dev.cpu() - S_ref).abs().max() < 2e-2


def test_hybrid_model_on_engine_graph_equals_eager():
    from vllm_ascend_b200.config import ModelConfig
    from vllm_ascend_b200.engine.llm import LLM
    from vllm_ascend_b200.engine.request import SamplingParams

    def cfg():
        return ModelConfig(name="gdn-t", architecture="Qwen3NextForCausalLM", vocab_size=2048, hidden_size=512,
                           intermediate_size=1024, num_hidden_layers=4, num_attention_heads=8,
                           num_key_value_heads=2, head_dim=128, qk_norm=True, rope_theta=1e6, dtype="bfloat16",
                           init_std=0.05, full_attention_interval=2, linear_num_key_heads=2,
                           linear_num_value_heads=4, linear_key_head_dim=128, linear_value_head_dim=128)
    rng = np.random.default_rng(0)
    prompts = [rng.integers(0, 2048, size=n).tolist() for n in (150, 40, 300)]
    sp = SamplingParams(temperature=0.0, max_tokens=10, ignore_eos=True)
    outs = {}
    for eager in (True, False):
        llm = LLM(cfg(), device="cuda", max_model_len=512, max_num_seqs=8, max_num_batched_tokens=256,
                  num_gpu_blocks_override=40, enforce_eager=eager, cudagraph_capture_sizes=[2, 4])
        outs[eager] = [o.outputs[0].token_ids for o in llm.generate(prompts, sp)]
        if not eager:
            assert llm.engine.runner.stats["graph_replays"] > 0
        # a second pass reuses the state rows of finished requests
        assert [o.outputs[0].token_ids for o in llm.generate(prompts, sp)] == outs[eager]
    assert outs[True] == outs[False]
    _native.check_status(torch.device("cuda"))
