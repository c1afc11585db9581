"""RMSNorm folded into the neighbouring GEMMs: same model function as the unfolded kernels."""
import numpy as np
import pytest
import torch

from vllm_ascend_b200 import _native, ops

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _stats(rows, feats, per_row):
    """Row-statistics buffer holding ``per_row`` as two unequal partials."""
    buf = ops.alloc_row_stats(rows, feats, DEV)
    n = per_row.numel()
    view = buf[:buf.stats_rows * buf.stats_parts].view(buf.stats_parts, buf.stats_rows)
    view[0, :n] = per_row * 0.25
    view[1, :n] = per_row * 0.75
    view[2, :n] = 1e9                                   # beyond the part count: must not be read
    buf[buf.stats_rows * buf.stats_parts:].view(torch.int32)[0] = 2
    return buf


def test_gemm_scales_rows_and_writes_sum_of_squares_partials():
    g = torch.Generator(device="cpu").manual_seed(0)
    M, K, N, H = 520, 512, 768, 512
    x = (torch.randn(M, K, generator=g) * 2.0).bfloat16().to(DEV)
    w = (torch.randn(N, K, generator=g) * 0.1).bfloat16().to(DEV)
    res = torch.randn(M, N, generator=g).bfloat16().to(DEV)
    ss_rows = (x.float() ** 2).sum(-1).contiguous()
    ss_in = _stats(M + 8, N, ss_rows)
    ss_out = ops.alloc_row_stats(M + 8, N, DEV)
    ss_out.fill_(5.0)                                     # stale values of an earlier step
    out = ops.linear_norm_folded(x, w, residual=res, ss_in=ss_in, norm_dim=H, eps=1e-6, ss_out=ss_out)
    torch.cuda.synchronize()
    _native.check_status(torch.device(DEV))
    rstd = torch.rsqrt(ss_rows / H + 1e-6)
    want = (x.float() @ w.float().t()) * rstd[:, None] + res.float()
    assert float((out.float() - want).abs().max() / want.abs().max()) < 2e-2
    R, P = ss_out.stats_rows, ss_out.stats_parts
    parts = int(ss_out[R * P:].view(torch.int32)[0])
    assert 1 <= parts <= P
    got_ss = ss_out[:R * P].view(P, R)[:parts, :M].sum(0)
    want_ss = (out.float() ** 2).sum(-1)
    assert float(((got_ss - want_ss) / want_ss).abs().max()) < 1e-3
    # bit-for-bit repeatable: the statistics are stores summed in a fixed order, not atomics
    ss_again = ops.alloc_row_stats(M + 8, N, DEV)
    out2 = ops.linear_norm_folded(x, w, residual=res, ss_in=ss_in, norm_dim=H, eps=1e-6, ss_out=ss_again)
    torch.cuda.synchronize()
    assert torch.equal(out, out2)
    assert torch.equal(ss_again[:R * P].view(P, R)[:parts, :M], ss_out[:R * P].view(P, R)[:parts, :M])
    ss_in = _stats(M + 8, N, ss_rows)
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
    # the folded engine repeats itself exactly
    folded.reset_prefix_cache()             # same step shapes as the first pass
    again = folded.generate(prompts, sp)
    assert [o.outputs[0].token_ids for o in again] == [o.outputs[0].token_ids for o in got]
    assert [o.outputs[0].logprobs[0] for o in again] == [o.outputs[0].logprobs[0] for o in got]
