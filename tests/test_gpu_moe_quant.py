"""Native MoE kernels and block-scaled fp8 GEMMs vs PyTorch references."""
import pytest
import torch

from vllm_ascend_b200 import _native, ops
from vllm_ascend_b200.ops import fused_moe, moe_native, reference as ref
from vllm_ascend_b200.quantization import schemes

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.mark.parametrize("E,k,scoring,n_group,topk_group,bias", [
    (128, 8, "softmax", 1, 1, False), (256, 8, "sigmoid", 8, 4, True), (8, 2, "softmax", 1, 1, False),
    (64, 6, "sigmoid", 4, 2, False), (160, 6, "softmax", 1, 1, True)])
def test_gating_topk(E, k, scoring, n_group, topk_group, bias):
    torch.manual_seed(E + k)
    T = 77
    logits = torch.randn(T, E, device=DEV) * 2
    b = torch.randn(E, device=DEV) * 0.1 if bias else None
    w, ids = moe_native.gating_topk(logits, k, scoring, True, n_group, topk_group, b, 2.5)
    ew, eids = fused_moe.gating_topk_ref(logits, k, scoring, True, n_group, topk_group, b, 2.5)
    assert torch.equal(ids.sort(-1).values, eids.sort(-1).values)
    order = ids.long().argsort(-1)
    eorder = eids.long().argsort(-1)
    assert torch.allclose(w.gather(1, order), ew.gather(1, eorder), rtol=1e-4, atol=1e-6)


@pytest.mark.parametrize("T,E,k,H,I,local", [(64, 8, 2, 256, 128, None), (300, 16, 4, 512, 256, (4, 12)),
                                             (1, 8, 2, 128, 128, None), (1000, 128, 8, 2048, 768, None)])
def test_fused_experts_native_matches_reference(T, E, k, H, I, local):
    torch.manual_seed(T)
    x = (torch.randn(T, H, device=DEV) * 0.5).bfloat16()
    Elocal = E if local is None else local[1] - local[0]
    w13 = (torch.randn(Elocal, 2 * I, H, device=DEV) * 0.05).bfloat16()
    w2 = (torch.randn(Elocal, H, I, device=DEV) * 0.05).bfloat16()
    logits = torch.randn(T, E, device=DEV)
    tw, ids = fused_moe.gating_topk_ref(logits, k)
    emap = None
    if local is not None:
        emap = torch.full((E,), -1, dtype=torch.int32, device=DEV)
        emap[local[0]:local[1]] = torch.arange(Elocal, dtype=torch.int32, device=DEV)
    got = moe_native.fused_experts(x, w13, w2, tw, ids, emap)
    torch.cuda.synchronize()
    _native.check_status(torch.device(DEV))
    exp = fused_moe.fused_experts_ref(x.float(), w13.float(), w2.float(), tw, ids, emap)
    assert (got.float() - exp).abs().max() < 0.03 * exp.abs().max() + 0.02


@pytest.mark.parametrize("M,N,K", [(128, 128, 128), (300, 512, 1024), (4096, 4096, 4096), (5, 1536, 7168), (777, 136, 256)])
def test_fp8_block_gemm(M, N, K):
    torch.manual_seed(M)
    x = (torch.randn(M, K, device=DEV) * 0.5).bfloat16()
    w = torch.randn(N, K, device=DEV) * 0.1
    w8, ws = schemes.quantize_weight_block_fp8(w)
    got = schemes.fp8_block_linear(x, w8, ws)
    torch.cuda.synchronize()
    _native.check_status(torch.device(DEV))
    exp = ref.block_fp8_linear(x, w8, ws, out_dtype=torch.float32)
    assert (got.float() - exp).abs().max() < 0.01 * exp.abs().max() + 0.02
    full = x.float() @ w.t()
    assert (got.float() - full).abs().max() < 0.08 * full.abs().max()


def test_fp8_experts_native_matches_reference():
    torch.manual_seed(9)
    T, E, k, H, I = 200, 8, 2, 512, 256
    x = (torch.randn(T, H, device=DEV) * 0.5).bfloat16()

    class Blk:
        pass
    blk = Blk()
    blk.w13 = torch.randn(E, 2 * I, H, device=DEV) * 0.05
    blk.w2 = torch.randn(E, H, I, device=DEV) * 0.05
    sch = schemes.Fp8BlockMoE()
    sch.convert(blk)
    tw, ids = fused_moe.gating_topk_ref(torch.randn(T, E, device=DEV), k)
    got = moe_native.fused_experts_fp8(x, blk.w13, blk.w13_scale, blk.w2, blk.w2_scale, tw, ids, None)
    torch.cuda.synchronize()
    _native.check_status(torch.device(DEV))
    xc, twc, idc = x.cpu(), tw.cpu(), ids.cpu()
    blk.w13, blk.w13_scale, blk.w2, blk.w2_scale = (t.cpu() for t in (blk.w13, blk.w13_scale, blk.w2, blk.w2_scale))
    exp = sch.apply_experts(xc, blk.w13, blk.w2, twc, idc, None)
    assert (got.float().cpu() - exp.float()).abs().max() < 0.04 * exp.float().abs().max() + 0.02


@pytest.mark.parametrize("H,with_res", [(4096, True), (1024, False), (12288, True)])
def test_fused_norm_quant_matches_unfused(H, with_res):
    torch.manual_seed(0)
    T = 77
    x = torch.randn(T, H, device=DEV).bfloat16()
    w = (1 + 0.1 * torch.randn(H, device=DEV)).bfloat16()
    res = torch.randn(T, H, device=DEV).bfloat16() if with_res else None
    r1 = res.clone() if with_res else None
    r2 = res.clone() if with_res else None
    y, ro = ops.rms_norm(x.clone(), w, 1e-6, r1)
    q_ref, s_ref = ops.quant_fp8_group128(y)
    qa, ro2 = ops.rms_norm_quant_fp8(x.clone(), w, 1e-6, r2)
    torch.cuda.synchronize()
    assert torch.equal(qa.scales, s_ref)
    assert torch.equal(qa.q.view(torch.uint8), q_ref.view(torch.uint8))
    if with_res:
        assert torch.equal(ro2, ro)


def test_fused_silu_mul_quant_matches_unfused():
    torch.manual_seed(1)
    T, I = 65, 3072
    x = torch.randn(T, 2 * I, device=DEV).bfloat16()
    q_ref, s_ref = ops.quant_fp8_group128(ops.silu_and_mul(x))
    qa = ops.silu_and_mul_quant_fp8(x)
    torch.cuda.synchronize()
    # the two paths may round silu differently by one bf16 ulp: compare dequantised values
    a = q_ref.float().view(T, I // 128, 128) * s_ref.unsqueeze(-1)
    b = qa.q.float().view(T, I // 128, 128) * qa.scales.unsqueeze(-1)
    assert (a - b).abs().max() <= 0.07 * a.abs().max()
    assert (a - b).abs().mean() < 2e-3


def test_fp8_model_uses_fused_producers_and_matches_unfused(monkeypatch):
    """A dense model quantised to block fp8: generation with the fused norm/activation
    producers equals generation with the separate quant kernel."""
    import numpy as np
    from vllm_ascend_b200.config import ModelConfig
    from vllm_ascend_b200.engine.llm import LLM
    from vllm_ascend_b200.engine.request import SamplingParams
    from vllm_ascend_b200.models import layers

    def cfg():
        return ModelConfig(name="t8", architecture="Qwen3ForCausalLM", vocab_size=2048, hidden_size=512,
                           intermediate_size=1024, num_hidden_layers=2, num_attention_heads=8,
                           num_key_value_heads=2, head_dim=128, qk_norm=True, rope_theta=1e6,
                           dtype="bfloat16", init_std=0.05, quantization="fp8")
    rng = np.random.default_rng(0)
    prompts = [rng.integers(0, 2048, size=n).tolist() for n in (90, 33)]
    sp = SamplingParams(temperature=0.0, max_tokens=8, ignore_eos=True)
    kw = dict(device="cuda", max_model_len=256, max_num_seqs=4, max_num_batched_tokens=128,
              num_gpu_blocks_override=16, enforce_eager=True)
    c0 = ops.launch_counter[0]
    fused = [o.outputs[0].token_ids for o in LLM(cfg(), **kw).generate(prompts, sp)]
    n_fused = ops.launch_counter[0] - c0
    monkeypatch.setattr(layers, "wants_quant_act", lambda linear: False)
    c0 = ops.launch_counter[0]
    plain = [o.outputs[0].token_ids for o in LLM(cfg(), **kw).generate(prompts, sp)]
    n_plain = ops.launch_counter[0] - c0
    assert fused == plain
    assert n_fused < n_plain          # fewer launches: the quant passes disappeared


@pytest.mark.parametrize("T,H", [(300, 4096), (5, 128), (64, 12288)])
def test_quant_fp8_per_token_kernel(T, H):
    torch.manual_seed(T)
    x = (torch.randn(T, H, device=DEV) * torch.rand(T, 1, device=DEV) * 3).bfloat16()
    c0 = _native.launch_counter[0]
    q, s = ops.quant_fp8_per_token(x)
    assert _native.launch_counter[0] == c0 + 1
    eq, es = ref.quant_fp8_per_token(x.cpu())
    assert torch.allclose(s.cpu(), es, rtol=1e-6)
    # identical except where the product lands on a rounding boundary of e4m3
    diff = (q.float().cpu() - eq.float()).abs()
    assert (diff > 0).float().mean() < 5e-3 and (diff <= 0.13 * eq.float().abs() + 1e-3).all()


@pytest.mark.parametrize("M,N,K", [(128, 128, 128), (300, 512, 1024), (4096, 4096, 4096), (5, 1536, 7168), (777, 136, 256)])
def test_fp8_channel_gemm(M, N, K):
    torch.manual_seed(M)
    x = (torch.randn(M, K, device=DEV) * 0.5).bfloat16()
    w = torch.randn(N, K, device=DEV) * 0.1 * (torch.rand(N, 1, device=DEV) + 0.2)
    bias = torch.randn(N, device=DEV).bfloat16()
    ws = (w.abs().amax(dim=1) / 448.0).clamp_min(1e-10)
    w8 = (w / ws.unsqueeze(1)).to(torch.float8_e4m3fn)
    got = schemes.fp8_channel_linear(x, w8, ws, bias)
    torch.cuda.synchronize()
    _native.check_status(torch.device(DEV))
    xq, xs = ops.quant_fp8_per_token(x)              # the GEMM is checked on the kernel's own quantised input
    exp = (xq.float() @ w8.float().t()) * xs.unsqueeze(1) * ws.unsqueeze(0) + bias.float()
    assert (got.float() - exp).abs().max() < 0.01 * exp.abs().max() + 0.02
    full = x.float() @ w.t() + bias.float()
    assert (got.float() - full).abs().max() < 0.08 * full.abs().max()


def test_fp8_channel_linear_scheme_and_experts_on_gpu():
    from vllm_ascend_b200 import quantization as Q
    from vllm_ascend_b200.models.layers import Linear
    torch.manual_seed(3)
    lin = Linear((torch.randn(384, 512, device=DEV) * 0.1).bfloat16(), (torch.randn(384, device=DEV) * 0.1).bfloat16())
    x = torch.randn(2, 33, 512, device=DEV).bfloat16()
    exp = x.float() @ lin.weight.float().t() + lin.bias.float()
    sch = Q.get_scheme_class("W8A8FP8_DYNAMIC", "linear")()
    sch.convert(lin)
    lin.quant = Q.LinearMethod(sch)
    c0 = _native.launch_counter[0]
    got = lin(x)
    assert _native.launch_counter[0] == c0 + 2            # per-token quant + GEMM, no fallback
    assert got.shape == exp.shape and (got.float() - exp).abs().max() < 0.08 * exp.abs().max()

    T, E, k, H, I = 200, 8, 2, 512, 256
    xt = (torch.randn(T, H, device=DEV) * 0.5).bfloat16()
    blk = type("B", (), {})()
    blk.w13 = torch.randn(E, 2 * I, H, device=DEV) * 0.05
    blk.w2 = torch.randn(E, H, I, device=DEV) * 0.05
    tw, ids = fused_moe.gating_topk_ref(torch.randn(T, E, device=DEV), k)
    want = fused_moe.fused_experts_ref(xt.float(), blk.w13, blk.w2, tw, ids, None)
    ms = Q.get_scheme_class("W8A8FP8_DYNAMIC", "moe")()
    ms.convert(blk)
    assert blk.w13.dtype == torch.float8_e4m3fn and blk.w13_scale.shape == (E, 2 * I)
    got = ms.apply_experts(xt, blk.w13, blk.w2, tw, ids, None)
    torch.cuda.synchronize()
    _native.check_status(torch.device(DEV))
    assert (got.float() - want).abs().max() < 0.1 * want.abs().max() + 0.02
    # local-expert subset (expert parallel layout): experts 2..5 live here
    emap = torch.full((E,), -1, dtype=torch.int32, device=DEV)
    emap[2:6] = torch.arange(4, dtype=torch.int32, device=DEV)
    sub = type("B", (), {})()
    sub.w13, sub.w2, sub.w13_scale, sub.w2_scale = blk.w13[2:6].contiguous(), blk.w2[2:6].contiguous(), \
        blk.w13_scale[2:6].contiguous(), blk.w2_scale[2:6].contiguous()
    ms2 = Q.get_scheme_class("W8A8FP8_DYNAMIC", "moe")()
    ms2.block_ref = sub
    part = ms2.apply_experts(xt, sub.w13, sub.w2, tw, ids, emap)
    mask = ((ids >= 2) & (ids < 6)).to(tw.dtype)
    want_part = fused_moe.fused_experts_ref(xt.float(), (blk.w13[2:6].float() * blk.w13_scale[2:6].unsqueeze(-1)),
                                            (blk.w2[2:6].float() * blk.w2_scale[2:6].unsqueeze(-1)), tw * mask,
                                            (ids - 2).clamp(0, 3), None)
    assert (part.float() - want_part).abs().max() < 0.1 * want_part.abs().max() + 0.02
