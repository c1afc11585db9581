"""The fusion plan is live: with a fusion switched off the layers run the op sequence it replaces, and the
tokens do not change."""
import numpy as np

from vllm_ascend_b200 import ops
from vllm_ascend_b200.compilation import fusion
from vllm_ascend_b200.engine.llm import LLM
from vllm_ascend_b200.engine.request import SamplingParams
from vllm_ascend_b200.platform_config import clear_b200_config


def _tokens(additional, monkeypatch, counts):
    real_qk, real_sw, real_norm = ops.qknorm_rope_kvwrite, ops.linear_swiglu, ops.rms_norm

    def qk(*a, **k):
        counts["qk"] += 1
        return real_qk(*a, **k)

    def sw(*a, **k):
        counts["swiglu"] += 1
        return real_sw(*a, **k)

    def norm(x, w, eps, residual=None, *a, **k):
        counts["norm_with_residual" if residual is not None else "norm_plain"] += 1
        return real_norm(x, w, eps, residual, *a, **k)
    from vllm_ascend_b200.models.layers import GQAAttention
    real_attend = GQAAttention.attend

    def attend(self, *a, **k):
        counts["attend"] += 1
        return real_attend(self, *a, **k)
    monkeypatch.setattr(GQAAttention, "attend", attend)
    monkeypatch.setattr(ops, "qknorm_rope_kvwrite", qk)
    monkeypatch.setattr(ops, "linear_swiglu", sw)
    monkeypatch.setattr(ops, "rms_norm", norm)
    llm = LLM("tiny-qwen", device="cpu", seed=0, block_size=16, max_model_len=128, max_num_seqs=4,
              max_num_batched_tokens=64, additional_config=additional)
    rng = np.random.default_rng(1)
    prompts = [rng.integers(1, 900, size=n).tolist() for n in (40, 9)]
    out = [o.outputs[0].token_ids for o in llm.generate(prompts, SamplingParams(max_tokens=6, temperature=0.0,
                                                                                 ignore_eos=True))]
    clear_b200_config()
    return out


def test_unfused_sequences_give_the_fused_tokens(monkeypatch):
    on = dict(qk=0, swiglu=0, norm_with_residual=0, norm_plain=0, attend=0)
    want = _tokens(None, monkeypatch, on)
    on = dict(on)                       # the wrappers of this run stay installed under the next ones
    plan = fusion.get_plan()
    assert all(plan.enabled(f.name) for f in fusion.FUSIONS) and len(plan.describe()) == len(fusion.FUSIONS)
    off = dict(qk=0, swiglu=0, norm_with_residual=0, norm_plain=0, attend=0)
    got = _tokens({"fusion_config": {"fuse_norm_quant": False, "fuse_qknorm_rope": False, "fuse_muls_add": False,
                                     "fuse_gemm_comm": False}}, monkeypatch, off)
    assert got == want
    assert on["swiglu"] > 0 and off["swiglu"] == 0                       # gate_up GEMM, then SiLU-mul
    assert on["qk"] == on["attend"] > 0 and off["qk"] == 3 * off["attend"] > 0     # norm, rotary, cache write as three passes
    assert on["norm_with_residual"] > 0 and off["norm_with_residual"] == 0 and off["norm_plain"] > on["norm_plain"]
