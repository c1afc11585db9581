"""Dispatcher ops: schemas exist, the CPU key computes the PyTorch definitions, the meta key
propagates shapes and dtypes without data (FakeTensorMode)."""
import torch

from vllm_ascend_b200 import ops
from vllm_ascend_b200.ops import torch_bindings as tb


def test_ops_are_defined_once_with_schemas():
    names = tb.register()
    assert tb.register() == names                       # idempotent
    for n in tb.SCHEMAS:
        assert hasattr(torch.ops.b200, n), n
    s = str(torch.ops.b200.add_rms_norm.default._schema)
    assert "residual" in s and "->" in s


def test_cpu_key_matches_the_op_functions():
    tb.register()
    g = torch.Generator().manual_seed(0)
    x = torch.randn(6, 64, generator=g)
    w = torch.randn(64, generator=g)
    r = torch.randn(6, 64, generator=g)
    assert torch.equal(torch.ops.b200.rms_norm(x, w, 1e-6), ops.rms_norm(x, w, 1e-6)[0])
    y, r2 = torch.ops.b200.add_rms_norm(x, r, w, 1e-6)
    y0, r0 = ops.rms_norm(x, w, 1e-6, residual=r)
    assert torch.equal(y, y0) and torch.equal(r2, r0)
    W = torch.randn(32, 64, generator=g)
    b = torch.randn(32, generator=g)
    torch.testing.assert_close(torch.ops.b200.linear(x, W, b, None), x @ W.t() + b)
    torch.testing.assert_close(torch.ops.b200.silu_and_mul(x, 0.0),
                               torch.nn.functional.silu(x[:, :32]) * x[:, 32:])
    bt = torch.tensor([[4, 9], [2, 7]], dtype=torch.int32)
    out = torch.ops.b200.slot_mapping(bt, torch.tensor([0, 1], dtype=torch.int32), torch.tensor([17, 3]), 16, 10)
    assert out.tolist() == [9 * 16 + 1, 2 * 16 + 3]
    var = torch.zeros(4, 3)
    torch.ops.b200.scatter_nd_update_(var, torch.tensor([[2]]), torch.ones(1, 3))
    assert var[2].tolist() == [1, 1, 1]


def test_paged_attention_op_on_cpu_equals_dense_attention():
    tb.register()
    g = torch.Generator().manual_seed(1)
    Hq, Hkv, D, bs = 4, 2, 32, 16
    lens = [20, 7]
    kc = torch.randn(8, bs, Hkv, D, generator=g)
    vc = torch.randn(8, bs, Hkv, D, generator=g)
    bt = torch.tensor([[1, 2], [3, 0]], dtype=torch.int32)
    q = torch.randn(sum(lens), Hq, D, generator=g)
    qsl = torch.tensor([0, 20, 27], dtype=torch.int32)
    sl = torch.tensor(lens, dtype=torch.int32)
    out = torch.ops.b200.paged_attention(q, kc, vc, bt, sl, qsl, 20, 20, D ** -0.5, True, 0)
    off = 0
    for i, n in enumerate(lens):
        k = torch.cat([kc[b] for b in bt[i].tolist()])[:n].repeat_interleave(Hq // Hkv, dim=1)
        v = torch.cat([vc[b] for b in bt[i].tolist()])[:n].repeat_interleave(Hq // Hkv, dim=1)
        s = torch.einsum("qhd,khd->hqk", q[off:off + n], k) * D ** -0.5
        s = s.masked_fill(torch.triu(torch.ones(n, n, dtype=torch.bool), 1), float("-inf"))
        ref = torch.einsum("hqk,khd->qhd", s.softmax(-1), v)
        torch.testing.assert_close(out[off:off + n], ref, rtol=1e-4, atol=1e-4)
        off += n


def test_meta_functions_propagate_shapes_under_fake_tensors():
    tb.register()
    from torch._subclasses.fake_tensor import FakeTensorMode
    with FakeTensorMode():
        x = torch.empty(10, 256, dtype=torch.bfloat16)
        w = torch.empty(256, dtype=torch.bfloat16)
        W = torch.empty(512, 256, dtype=torch.bfloat16)
        assert torch.ops.b200.rms_norm(x, w, 1e-6).shape == (10, 256)
        a, b = torch.ops.b200.add_rms_norm(x, x, w, 1e-6)
        assert a.shape == b.shape == (10, 256)
        assert torch.ops.b200.linear(x, W, None, None).shape == (10, 512)
        assert torch.ops.b200.linear_swiglu(x, W).shape == (10, 256)
        q, s = torch.ops.b200.quant_fp8_group128(x, False)
        assert q.dtype == torch.float8_e4m3fn and s.shape == (10, 2) and s.dtype == torch.float32
        q, s = torch.ops.b200.quant_fp8_per_token(x)
        assert s.shape == (10,)
        lg = torch.empty(10, 1000)
        assert torch.ops.b200.argmax(lg).shape == (10,) and torch.ops.b200.argmax(lg).dtype == torch.int64
        qq = torch.empty(10, 8, 128, dtype=torch.bfloat16)
        kc = torch.empty(4, 128, 2, 128, dtype=torch.bfloat16)
        o = torch.ops.b200.paged_attention(qq, kc, kc, torch.empty(2, 2, dtype=torch.int32),
                                           torch.empty(2, dtype=torch.int32), torch.empty(3, dtype=torch.int32),
                                           5, 100, 0.1, True, 0)
        assert o.shape == (10, 8, 128) and o.dtype == torch.bfloat16
        assert torch.ops.b200.sign_bits_pack(x).shape == (320,)
        assert torch.ops.b200.sign_bits_unpack(torch.empty(4, dtype=torch.uint8), 30, 1.0, torch.bfloat16).dtype \
            == torch.bfloat16
        assert torch.ops.b200.expand_block_table(torch.empty(3, 5, dtype=torch.int32), 4).shape == (3, 20)
        assert torch.ops.b200.bincount(torch.empty(7, dtype=torch.int64), None, 2, 50).shape == (2, 50)


def test_opcheck_of_a_functional_and_a_mutating_op():
    tb.register()
    x = torch.randn(4, 16)
    w = torch.ones(16)
    torch.library.opcheck(torch.ops.b200.rms_norm.default, (x, w, 1e-6),
                          test_utils=("test_schema", "test_faketensor"))
    var = torch.zeros(4, 3)
    torch.library.opcheck(torch.ops.b200.scatter_nd_update_.default, (var, torch.tensor([[1]]), torch.ones(1, 3)),
                          test_utils=("test_schema", "test_faketensor"))
