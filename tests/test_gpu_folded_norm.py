"""RMSNorm folded into the neighbouring GEMMs: same model function as the unfolded kernels."""
import numpy as np
import pytest
import torch

from vllm_ascend_b200 import _native, ops

pytestmark = pytest.mark.gpu
DEV = "cuda"


def test_gemm_scales_rows_and_accumulates_sum_of_squares():
    g = torch.Generator(device="cpu").manual_seed(0)
    M, K, N, H = 520, 512, 768, 512
    x = (torch.randn(M, K, generator=g) * 2.0).bfloat16().to(DEV)
    w = (torch.randn(N, K, generator=g) * 0.1).bfloat16().to(DEV)
    res = torch.randn(M, N, generator=g).bfloat16().to(DEV)
    ss_in = (x.float() ** 2).sum(-1).contiguous()
    ss_out = torch.full((M + 8,), 3.0, dtype=torch.float32, device=DEV)        # keeps what was there and adds
    zero = torch.full((M + 8,), 7.0, dtype=torch.float32, device=DEV)
    out = ops.linear_norm_folded(x, w, residual=res, ss_in=ss_in, norm_dim=H, eps=1e-6, ss_out=ss_out, zero=zero)
    torch.cuda.synchronize()
    _native.check_status(torch.device(DEV))
    rstd = torch.rsqrt(ss_in / H + 1e-6)
    want = (x.float() @ w.float().t()) * rstd[:, None] + res.float()
    assert float((out.float() - want).abs().max() / want.abs().max()) < 2e-2
    want_ss = 3.0 + (out.float() ** 2).sum(-1)
    assert float(((ss_out[:M] - want_ss) / want_ss).abs().max()) < 1e-3
    assert float(ss_out[M:].min()) == 3.0 and float(zero[:M].abs().max()) == 0.0 and float(zero[M:].min()) == 7.0
    # SwiGLU epilogue: both halves are scaled before the activation
    I = 256
    w2 = (torch.randn(2 * I, K, generator=g) * 0.1).bfloat16().to(DEV)
    act = ops.linear_norm_folded(x, w2, swiglu=True, ss_in=ss_in, norm_dim=H, eps=1e-6)
    hh = (x.float() @ w2.float().t()) * rstd[:, None]
    want2 = torch.nn.functional.silu(hh[:, :I]) * hh[:, I:]
    assert float((act.float() - want2).abs().max()) < 0.02 * float(want2.abs().max()) + 0.02


def test_engine_with_folded_norms_matches_the_unfolded_engine(monkeypatch):
    from test_gpu_engine import _cfg
    from vllm_ascend_b200 import envs
    from vllm_ascend_b200.engine.llm import LLM
    from vllm_ascend_b200.engine.request import SamplingParams
    rng = np.random.default_rng(3)
    prompts = [rng.integers(0, 2048, size=n).tolist() for n in (300, 280, 17)]
    sp = SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True, logprobs=5)
    kw = dict(device="cuda", max_model_len=512, max_num_seqs=8, max_num_batched_tokens=1024,
              num_gpu_blocks_override=64, enforce_eager=True)

    def run(fold):
        monkeypatch.setitem(envs.env_variables, "VLLM_B200_FOLD_NORM", lambda: "1" if fold else "0")
        cfg = _cfg("bfloat16")
        llm = LLM(cfg, **kw)
        model = llm.engine.runner.model
        assert bool(getattr(model, "norm_folded", False)) == fold
        if not fold:
            # give the norms real weights, then build the folded engine from the same parameters
            g = torch.Generator(device="cpu").manual_seed(9)
            for L in model.layers:
                for n in (L.input_layernorm, L.post_attention_layernorm):
                    n.weight.copy_((torch.rand(n.weight.shape, generator=g) + 0.5).to(n.weight.dtype))
        return llm

    plain = run(False)
    state = {k: v.clone() for k, v in plain.engine.runner.model.named_parameters()}
    want = plain.generate(prompts, sp)
    folded = run(True)
    model = folded.engine.runner.model
    for k, v in model.named_parameters():
        v.copy_(state[k])
    from vllm_ascend_b200.models.folded import fold_norms
    fold_norms(model)
    assert all(bool((L.input_layernorm.weight == 1).all()) for L in model.layers)
    got = folded.generate(prompts, sp)
    _native.check_status(torch.device(DEV))
    for a, b in zip(got, want):
        la, lb = a.outputs[0].logprobs[0], b.outputs[0].logprobs[0]
        common = set(la) & set(lb)
        assert len(common) >= 3 and max(abs(la[t] - lb[t]) for t in common) < 0.1, (la, lb)
    same = sum(x == y for a, b in zip(got, want) for x, y in zip(a.outputs[0].token_ids, b.outputs[0].token_ids))
    assert same >= 0.8 * 18
