"""Hyper-connection ops: definitions against hand-written arithmetic, the doubly stochastic mixing matrix,
and a decoder that runs on widened residual streams through the engine."""
import numpy as np
import torch

from vllm_ascend_b200.ops import hyper_connection as hc


def _inputs(T=5, m=4, H=32, seed=0):
    g = torch.Generator().manual_seed(seed)
    x = (torch.rand(T, m, H, generator=g) * 2).bfloat16()
    fn = torch.rand((2 + m) * m, m * H, generator=g) / (m * H)
    scale = torch.rand(3, generator=g) * 2
    base = torch.rand((2 + m) * m, generator=g) * 2
    return x, fn, scale, base


def test_hc_pre_matches_stepwise_arithmetic():
    m = 4
    x, fn, scale, base = _inputs(m=m)
    y, post, comb = hc.hc_pre(x, fn, scale, base, m, sinkhorn_iters=20)
    assert y.shape == (5, 32) and y.dtype == torch.bfloat16
    assert post.shape == (5, m) and comb.shape == (5, m, m) and post.dtype == comb.dtype == torch.float32
    for t in range(5):
        flat = x[t].float().reshape(-1)
        mixes = fn @ flat / torch.sqrt((flat * flat).mean() + 1e-6)
        pre = torch.sigmoid(mixes[:m] * scale[0] + base[:m]) + 1e-6
        assert torch.allclose(y[t].float(), (pre[:, None] * x[t].float()).sum(0).bfloat16().float(), atol=1e-2)
        assert torch.allclose(post[t], 2 * torch.sigmoid(mixes[m:2 * m] * scale[1] + base[m:2 * m]), atol=1e-6)
    # Sinkhorn: rows and columns of the mixing matrix sum to one
    assert torch.allclose(comb.sum(-1), torch.ones(5, m), atol=1e-3)
    assert torch.allclose(comb.sum(-2), torch.ones(5, m), atol=1e-3)
    assert (comb > 0).all()
    one = hc.hc_pre(x, fn, scale, base, m, sinkhorn_iters=1)[2]       # one pass: columns only
    assert torch.allclose(one.sum(-2), torch.ones(5, m), atol=1e-4) and not torch.allclose(one.sum(-1), torch.ones(5, m), atol=1e-3)


def test_hc_post_and_head():
    m, T, H = 3, 4, 16
    g = torch.Generator().manual_seed(1)
    y = torch.randn(T, H, generator=g)
    res = torch.randn(T, m, H, generator=g)
    post = torch.rand(T, m, generator=g)
    comb = torch.rand(T, m, m, generator=g)
    out = hc.hc_post(y, res, post, comb)
    for t in range(T):
        for i in range(m):
            want = post[t, i] * y[t] + sum(comb[t, j, i] * res[t, j] for j in range(m))
            assert torch.allclose(out[t, i], want, atol=1e-5)
    # identity mixing and zero write weights leave the streams alone
    eye = torch.eye(m).expand(T, m, m)
    assert torch.allclose(hc.hc_post(y, res, torch.zeros(T, m), eye), res)
    fn = torch.rand(m, m * H, generator=g) / (m * H)
    head = hc.hc_head(res, fn, torch.tensor([1.5]), torch.rand(m, generator=g))
    assert head.shape == (T, H)
    flat = res[0].reshape(-1)
    pre = torch.sigmoid(fn @ flat / torch.sqrt((flat * flat).mean() + 1e-6) * 1.5 + torch.zeros(m)) + 1e-6
    assert head.shape == (T, H) and torch.isfinite(head).all()


def test_decoder_on_widened_streams_through_the_engine():
    """A dense decoder with hc_mult = 2: chunked prefill + batching + decode equal a pass that recomputes every
    prefix from scratch, and the model differs from the plain residual one."""
    from vllm_ascend_b200.config import get_model_config
    from vllm_ascend_b200.engine.llm import LLM
    from vllm_ascend_b200.engine.request import SamplingParams
    import dataclasses
    base = get_model_config("tiny-qwen")
    cfg = dataclasses.replace(base, hc_mult=2, hc_sinkhorn_iters=4)
    kw = dict(device="cpu", seed=0, block_size=16, max_model_len=96, max_num_seqs=4)
    rng = np.random.default_rng(3)
    prompts = [rng.integers(1, 900, size=n).tolist() for n in (37, 9)]
    sp = SamplingParams(max_tokens=5, temperature=0.0, ignore_eos=True)
    llm = LLM(cfg, max_num_batched_tokens=24, **kw)
    got = [o.outputs[0].token_ids for o in llm.generate(prompts, sp)]
    want = []
    for p in prompts:
        toks = []
        for _ in range(5):
            one = LLM(cfg, max_num_batched_tokens=128, **kw)
            toks.append(one.generate([p + toks], SamplingParams(max_tokens=1, temperature=0.0, ignore_eos=True))[0]
                        .outputs[0].token_ids[0])
        want.append(toks)
    assert got == want
    plain = [o.outputs[0].token_ids for o in LLM(base, max_num_batched_tokens=24, **kw).generate(prompts, sp)]
    assert plain != got
    names = [n for n, _ in llm.engine.runner.model.named_parameters()]
    assert "model.layers.0.hc_attn_fn" in names and "model.hc_head_fn" in names
