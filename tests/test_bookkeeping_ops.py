"""Bookkeeping ops: the host definitions against hand-computed cases, and (on a GPU) the CUDA kernels
against the host definitions."""
import pytest
import torch

from vllm_ascend_b200.ops import bookkeeping as bk


def _cases(dev):
    g = torch.Generator().manual_seed(3)
    R, B, bs, nblk = 5, 7, 16, 200
    bt = torch.randint(0, nblk, (R, B), generator=g, dtype=torch.int32)
    bt[3, 5:] = -1
    T = 300
    req = torch.randint(-1, R, (T,), generator=g, dtype=torch.int32)
    pos = torch.randint(0, B * bs + 10, (T,), generator=g, dtype=torch.int64)     # some beyond the table
    return bt.to(dev), req.to(dev), pos.to(dev), bs, nblk


def test_slot_mapping_host_definition():
    bt = torch.tensor([[4, 9, -1], [2, 7, 5]], dtype=torch.int32)
    req = torch.tensor([0, 0, 1, -1, 1, 0], dtype=torch.int32)
    pos = torch.tensor([0, 17, 40, 3, 100, 35], dtype=torch.int64)
    out = bk.slot_mapping(bt, req, pos, 16, 10)
    assert out.tolist() == [64, 9 * 16 + 1, 5 * 16 + 8, -1, -1, -1]


def test_expand_block_table_host_definition():
    bt = torch.tensor([[3, -1], [0, 5]], dtype=torch.int32)
    assert bk.expand_block_table(bt, 2).tolist() == [[6, 7, -1, -1], [0, 1, 10, 11]]


def test_bincount_and_scatter_host_definitions():
    ids = torch.tensor([1, 1, 3, 9, -1, 2], dtype=torch.int64)
    rows = torch.tensor([0, 0, 1, 1, 0, 5], dtype=torch.int32)
    c = bk.bincount(ids, rows, 2, 4)
    assert c.tolist() == [[0, 2, 0, 0], [0, 0, 0, 1]]
    var = torch.zeros(3, 2, 4)
    idx = torch.tensor([[2, 1], [0, 0], [3, 0]], dtype=torch.int64)
    upd = torch.arange(12, dtype=torch.float32).view(3, 4)
    bk.scatter_nd_update(var, idx, upd)
    assert var[2, 1].tolist() == [0, 1, 2, 3] and var[0, 0].tolist() == [4, 5, 6, 7] and var.sum() == 6 + 22


def test_sign_bits_round_trip_host():
    x = torch.tensor([1.0, -2.0, 0.0, -0.0, 3.0, -1.0, -1.0, 5.0, -7.0, 2.0])
    p = bk.sign_bits_pack(x)
    assert p.tolist() == [0b01101010, 0b00000001]
    y = bk.sign_bits_unpack(p, 10, scale=0.5)
    assert torch.equal(y, torch.where(torch.signbit(x), -0.5, 0.5))


@pytest.mark.gpu
def test_kernels_equal_host_definitions():
    dev = torch.device("cuda:0")
    bt, req, pos, bs, nblk = _cases(dev)
    from vllm_ascend_b200 import _native
    got = bk.slot_mapping(bt, req, pos, bs, nblk)
    ref = bk.slot_mapping(bt.cpu(), req.cpu(), pos.cpu(), bs, nblk)
    assert torch.equal(got.cpu(), ref)
    # out-of-range rows were recorded in the status word: read and clear it
    st = _native.status_word(dev)
    assert int(st.item()) == 2
    st.zero_()
    assert torch.equal(bk.expand_block_table(bt, 4).cpu(), bk.expand_block_table(bt.cpu(), 4))
    g = torch.Generator().manual_seed(5)
    ids = torch.randint(-2, 1100, (5000,), generator=g, dtype=torch.int64)
    rows = torch.randint(0, 6, (5000,), generator=g, dtype=torch.int32)
    assert torch.equal(bk.bincount(ids.to(dev), rows.to(dev), 6, 1024).cpu(), bk.bincount(ids, rows, 6, 1024))
    var = torch.randn(9, 5, 24, generator=g).bfloat16()
    perm = torch.randperm(45, generator=g)[:20]
    idx = torch.stack([perm // 5, perm % 5], dim=1).contiguous()
    upd = torch.randn(20, 24, generator=g).bfloat16()
    a = bk.scatter_nd_update(var.clone().to(dev), idx.to(dev), upd.to(dev)).cpu()
    assert torch.equal(a, bk.scatter_nd_update(var.clone(), idx, upd))
    for dt in (torch.float32, torch.bfloat16):
        x = torch.randn(1003, generator=g).to(dt)
        p = bk.sign_bits_pack(x.to(dev))
        assert torch.equal(p.cpu(), bk.sign_bits_pack(x))
        assert torch.equal(bk.sign_bits_unpack(p, 1003, 2.0, dt).cpu(), bk.sign_bits_unpack(p.cpu(), 1003, 2.0, dt))
    torch.cuda.synchronize()


@pytest.mark.gpu
def test_swap_blocks_through_the_copy_kernel():
    from vllm_ascend_b200.attention.backend import B200AttentionBackend
    dev = torch.device("cuda:0")
    g = torch.Generator().manual_seed(7)
    src = torch.randn(12, 16, 4, 64, generator=g).bfloat16().to(dev)
    host = torch.zeros(6, 16, 4, 64, dtype=torch.bfloat16).pin_memory()
    pairs = torch.tensor([[1, 0], [7, 3], [11, 5]])
    B200AttentionBackend.swap_blocks(src, host, pairs)
    torch.cuda.synchronize()
    for s, d in pairs.tolist():
        assert torch.equal(host[d], src[s].cpu())
    back = torch.zeros_like(src)
    B200AttentionBackend.swap_blocks(host, back, torch.tensor([[0, 2], [3, 9]]))
    torch.cuda.synchronize()
    assert torch.equal(back[2].cpu(), host[0]) and torch.equal(back[9].cpu(), host[3])
    # HND view (permuted heads / tokens) as the destination
    hnd = torch.zeros(12, 4, 16, 64, dtype=torch.bfloat16, device=dev).permute(0, 2, 1, 3)
    B200AttentionBackend.swap_blocks(src, hnd, torch.tensor([[4, 4]]))
    torch.cuda.synchronize()
    assert torch.equal(hnd[4], src[4])


@pytest.mark.gpu
def test_engine_tokens_equal_with_device_slot_mapping(monkeypatch):
    import numpy as np
    from vllm_ascend_b200.config import ModelConfig
    from vllm_ascend_b200.engine.llm import LLM
    from vllm_ascend_b200.engine.request import SamplingParams
    cfg = dict(name="t", architecture="Qwen3ForCausalLM", vocab_size=2048, hidden_size=512, intermediate_size=1024,
               num_hidden_layers=2, num_attention_heads=8, num_key_value_heads=2, head_dim=128, qk_norm=True,
               rope_theta=1e6, dtype="bfloat16", init_std=0.05)
    rng = np.random.default_rng(0)
    prompts = [rng.integers(0, 2048, size=n).tolist() for n in (150, 40, 333)]
    sp = SamplingParams(temperature=0.0, max_tokens=10, ignore_eos=True)
    outs = {}
    for flag in ("0", "1"):
        monkeypatch.setenv("VLLM_B200_DEVICE_SLOT_MAPPING", flag)
        llm = LLM(ModelConfig(**cfg), device="cuda", max_model_len=512, max_num_seqs=8, max_num_batched_tokens=256,
                  num_gpu_blocks_override=40, cudagraph_capture_sizes=[2, 4])
        outs[flag] = [list(o.outputs[0].token_ids) for o in llm.generate(prompts, sp)]
        if flag == "1":
            assert llm.engine.runner._use_device_slots()
        del llm
    assert outs["0"] == outs["1"]
