"""sm_100a elementwise kernels vs plain PyTorch fp32 restatements."""
import pytest
import torch

from vllm_ascend_b200 import ops
from vllm_ascend_b200.ops import reference as ref

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.mark.parametrize("T,H", [(1, 128), (7, 4096), (300, 5120), (33, 8192)])
@pytest.mark.parametrize("with_res", [False, True])
def test_rms_norm(T, H, with_res):
    torch.manual_seed(0)
    x = torch.randn(T, H, device=DEV).bfloat16()
    w = (1 + 0.1 * torch.randn(H, device=DEV)).bfloat16()
    res = torch.randn(T, H, device=DEV).bfloat16() if with_res else None
    exp_out, exp_res = ref.rms_norm(x.float(), w.float(), 1e-6, None if res is None else res.float())
    if with_res:  # the kernel rounds the sum to bf16 before normalising
        exp_out, exp_res = ref.rms_norm(x, w, 1e-6, res.clone())
    r2 = res.clone() if with_res else None
    out, r_out = ops.rms_norm(x, w, 1e-6, r2)
    assert torch.allclose(out.float(), exp_out.float(), atol=3e-2, rtol=2e-2)
    if with_res:
        assert torch.equal(r_out, exp_res)


def test_rms_norm_strided_input_and_gemma():
    x_full = torch.randn(16, 1024, device=DEV).bfloat16()
    x = x_full[:, :512]
    w = torch.randn(512, device=DEV).bfloat16() * 0.1
    out, _ = ops.rms_norm(x, w, 1e-5, None, gemma=True)
    exp, _ = ref.rms_norm(x.float(), w.float(), 1e-5, None, gemma=True)
    assert torch.allclose(out.float(), exp, atol=3e-2, rtol=2e-2)


@pytest.mark.parametrize("T,I", [(1, 64), (513, 12288), (4096, 768)])
def test_silu_and_mul(T, I):
    x = torch.randn(T, 2 * I, device=DEV).bfloat16()
    out = ops.silu_and_mul(x)
    assert torch.allclose(out.float(), ref.silu_and_mul(x.float()), atol=2e-2, rtol=2e-2)
    lim = ops.silu_and_mul(x, limit=1.0)
    assert torch.allclose(lim.float(), ref.silu_and_mul(x.float(), 1.0), atol=2e-2, rtol=2e-2)


def test_embedding_with_vocab_shard():
    w = torch.randn(1000, 256, device=DEV).bfloat16()
    ids = torch.randint(0, 3000, (77,), device=DEV)
    out = ops.embedding(ids, w, 1000, 2000)
    assert torch.equal(out, ref.embedding(ids, w, 1000, 2000))


@pytest.mark.parametrize("Hq,Hkv,D,rot", [(32, 8, 128, 128), (4, 2, 64, 64), (8, 8, 128, 64)])
@pytest.mark.parametrize("layout", ["NHD", "HND"])
@pytest.mark.parametrize("qk_norm", [True, False])
def test_qknorm_rope_kvwrite(Hq, Hkv, D, rot, qk_norm, layout):
    torch.manual_seed(1)
    T, bs, nb = 67, 16, 12
    qkv = torch.randn(T, (Hq + 2 * Hkv) * D, device=DEV).bfloat16()
    pos = torch.randint(0, 500, (T,), device=DEV)
    cs = ref.build_cos_sin_cache(rot, 512, 1e6, None, DEV)
    qn = (1 + 0.1 * torch.randn(D, device=DEV)).bfloat16() if qk_norm else None
    kn = (1 + 0.1 * torch.randn(D, device=DEV)).bfloat16() if qk_norm else None
    slots = torch.randperm(nb * bs, device=DEV)[:T]
    slots[5] = -1
    kc = ops.alloc_kv_cache(nb, bs, Hkv, D, torch.bfloat16, DEV, layout)
    vc = ops.alloc_kv_cache(nb, bs, Hkv, D, torch.bfloat16, DEV, layout)
    exp = qkv.clone().float()
    ekc, evc = kc.clone().float(), vc.clone().float()
    ref.qknorm_rope_kvwrite(exp, pos, cs, rot, None if qn is None else qn.float(),
                            None if kn is None else kn.float(), 1e-6, ekc, evc, slots, Hq, Hkv, D)
    ops.qknorm_rope_kvwrite(qkv, pos, cs, rot, qn, kn, 1e-6, kc, vc, slots, Hq, Hkv, D)
    assert torch.allclose(qkv.float(), exp, atol=6e-2, rtol=3e-2)
    assert torch.allclose(kc.float(), ekc, atol=6e-2, rtol=3e-2)
    assert torch.allclose(vc.float(), evc, atol=1e-6)
    assert float(kc[slots[6] // bs, slots[6] % bs].abs().sum()) > 0


def test_quant_fp8_group128():
    x = torch.randn(65, 1024, device=DEV).bfloat16() * 3
    q, s = ops.quant_fp8_group128(x)
    eq, es = ref.quant_fp8_group128(x)
    assert torch.allclose(s, es, rtol=1e-5)
    deq = q.float().view(65, 8, 128) * s.unsqueeze(-1)
    assert torch.allclose(deq.view(65, 1024), x.float(), atol=0.2, rtol=0.07)


@pytest.mark.parametrize("kind,gated", [("gelu", True), ("gelu_tanh", True), ("quick_gelu", False), ("gelu", False),
                                        ("swiglu_oai", True)])
def test_activation_family(kind, gated):
    torch.manual_seed(0)
    x = (torch.randn(33, 2048, device=DEV) * 2).bfloat16()
    got = ops.activation(x, kind, gated)
    want = ref.activation(x.float(), kind, gated)
    assert got.shape == want.shape
    assert torch.allclose(got.float(), want, atol=3e-2, rtol=2e-2)


@pytest.mark.parametrize("group,before", [(0, True), (128, True), (128, False)])
def test_rms_norm_gated(group, before):
    torch.manual_seed(1)
    x = torch.randn(19, 1024, device=DEV).bfloat16()
    z = torch.randn(19, 1024, device=DEV).bfloat16()
    w = (1 + 0.1 * torch.randn(group or 1024, device=DEV)).bfloat16()
    got = ops.rms_norm_gated(x, z, w, 1e-6, group, before)
    want = ref.rms_norm_gated(x.float(), z.float(), w.float(), 1e-6, group, before)
    assert torch.allclose(got.float(), want, atol=4e-2, rtol=3e-2)
