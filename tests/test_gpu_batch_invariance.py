"""Batch invariance on the GPU: the value computed for a row must not depend on how many other rows
share the launch.  The GEMM kernels pick tile shapes (1-CTA / paired-CTA, tile width) from the problem
size; every shape accumulates an output element over K in one order, which is what these tests pin."""
import numpy as np
import pytest
import torch

from vllm_ascend_b200 import _native, ops

pytestmark = pytest.mark.gpu
DEV = "cuda"
SIZES = (1, 8, 100, 128, 255, 256, 300, 768, 1000, 2048, 4096)


@pytest.mark.parametrize("N,K", [(4096, 4096), (6144, 4096), (4096, 12288), (1536, 512)])
def test_gemm_rows_do_not_depend_on_the_row_count(N, K):
    g = torch.Generator(device="cpu").manual_seed(0)
    x = (torch.randn(4096, K, generator=g) * 0.5).bfloat16().to(DEV)
    w = (torch.randn(N, K, generator=g) * 0.05).bfloat16().to(DEV)
    bias = torch.randn(N, generator=g).bfloat16().to(DEV)
    full = ops.linear(x, w, bias)
    for m in SIZES:
        part = ops.linear(x[:m], w, bias)
        assert torch.equal(part, full[:m]), f"rows differ at M={m}"
    # rows taken from the middle of the batch as a batch of their own
    assert torch.equal(ops.linear(x[1000:1003].contiguous(), w, bias), full[1000:1003])
    torch.cuda.synchronize()
    _native.check_status(torch.device(DEV))


def test_swiglu_gemm_norm_and_activation_rows_do_not_depend_on_the_row_count():
    g = torch.Generator(device="cpu").manual_seed(1)
    K, I = 2048, 3072
    x = (torch.randn(2048, K, generator=g) * 0.5).bfloat16().to(DEV)
    w = (torch.randn(2 * I, K, generator=g) * 0.05).bfloat16().to(DEV)
    nw = torch.rand(K, generator=g).bfloat16().to(DEV)
    res = torch.randn(2048, K, generator=g).bfloat16().to(DEV)
    full = ops.linear_swiglu(x, w)
    fn, fr = ops.rms_norm(x, nw, 1e-6, residual=res.clone())
    for m in (1, 8, 128, 256, 300, 768, 2048):
        assert torch.equal(ops.linear_swiglu(x[:m], w), full[:m]), m
        pn, pr = ops.rms_norm(x[:m], nw, 1e-6, residual=res[:m].clone())
        assert torch.equal(pn, fn[:m]) and torch.equal(pr, fr[:m]), m
    torch.cuda.synchronize()
    _native.check_status(torch.device(DEV))


def test_engine_in_batch_invariant_mode_gives_a_request_the_same_tokens_alone_and_in_a_batch(monkeypatch):
    from test_gpu_engine import _cfg
    from vllm_ascend_b200 import batch_invariant
    from vllm_ascend_b200.engine.llm import LLM
    from vllm_ascend_b200.engine.request import SamplingParams
    monkeypatch.setenv("VLLM_B200_BATCH_INVARIANT", "1")
    try:
        rng = np.random.default_rng(7)
        prompts = [rng.integers(0, 2048, size=n).tolist() for n in (150, 40, 333, 129, 64, 90)]
        sp = SamplingParams(temperature=0.0, max_tokens=12, ignore_eos=True, logprobs=3)
        llm = LLM(_cfg("bfloat16"), device="cuda", max_model_len=512, max_num_seqs=8, max_num_batched_tokens=1024,
                  num_gpu_blocks_override=64, enforce_eager=True, enable_prefix_caching=False)
        assert batch_invariant.is_batch_invariant()
        assert not getattr(llm.engine.runner.model, "norm_folded", False)
        together = llm.generate(prompts, sp)
        for i in (0, 2, 5):
            alone = llm.generate([prompts[i]], sp)[0]
            assert alone.outputs[0].token_ids == together[i].outputs[0].token_ids
            assert alone.outputs[0].logprobs == together[i].outputs[0].logprobs
    finally:
        batch_invariant.disable_batch_invariant_mode()
