"""Sampling kernels vs the sort-based PyTorch reference."""
import pytest
import torch

from vllm_ascend_b200 import ops
from vllm_ascend_b200.ops import reference as ref

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_argmax(dtype):
    x = torch.randn(37, 151936, device=DEV).to(dtype)
    assert torch.equal(ops.argmax(x), x.float().argmax(-1))


def test_argmax_ties_odd_widths_and_unaligned_rows():
    """The first maximum wins, whatever mix of vector and scalar loads reads the row."""
    g = torch.Generator(device="cpu").manual_seed(0)
    for V in (8, 9, 1000, 1003, 4099):
        x = torch.randint(-3, 4, (5, V), generator=g).to(torch.bfloat16).to(DEV)       # many ties
        assert torch.equal(ops.argmax(x), x.float().argmax(-1)), V
    wide = torch.randint(-3, 4, (6, 2051), generator=g).to(torch.bfloat16).to(DEV)
    view = wide[:, 3:]                       # rows start 6 bytes off a 16-byte boundary
    assert torch.equal(ops.argmax(view), view.float().argmax(-1))
    top = torch.zeros(2, 4096, dtype=torch.bfloat16, device=DEV)
    top[0, 4095] = 1.0
    top[1, 0] = 1.0
    assert ops.argmax(top).tolist() == [4095, 0]


def test_penalties_match_reference():
    torch.manual_seed(0)
    B, V = 9, 5000
    logits = torch.randn(B, V, device=DEV)
    prompt = torch.randint(0, V, (B, 40), device=DEV)
    prompt[:, 30:] = V
    outp = torch.randint(0, V, (B, 25), device=DEV)
    outp[:, 20:] = V
    outp[:, 3] = outp[:, 2]           # repeated output token -> frequency counts 2
    rep = torch.rand(B, device=DEV) + 1.0
    freq = torch.rand(B, device=DEV)
    pres = torch.rand(B, device=DEV)
    rep[0], freq[0], pres[0] = 1.0, 0.0, 0.0
    exp = ref.apply_penalties(logits.clone(), prompt, outp, rep, freq, pres)
    got = ops.apply_penalties(logits.clone(), prompt, outp, rep, freq, pres)
    assert torch.allclose(got, exp, atol=1e-5)


def test_top_k_one_and_temperature_zero_are_greedy():
    torch.manual_seed(1)
    B, V = 16, 32000
    logits = torch.randn(B, V, device=DEV) * 3
    am = logits.argmax(-1)
    t = torch.ones(B, device=DEV)
    k = torch.ones(B, dtype=torch.int32, device=DEV)
    p = torch.ones(B, device=DEV)
    got = ops.sample(logits.clone(), t, k, p, None, None, None)
    assert torch.equal(got, am)
    got0 = ops.sample(logits.clone(), torch.zeros(B, device=DEV), torch.zeros(B, dtype=torch.int32, device=DEV), p)
    assert torch.equal(got0, am)


def test_samples_stay_inside_the_top_k_top_p_set():
    torch.manual_seed(2)
    B, V = 64, 20000
    logits = torch.randn(B, V, device=DEV) * 2
    t = torch.full((B,), 0.8, device=DEV)
    k = torch.randint(1, 50, (B,), dtype=torch.int32, device=DEV)
    p = torch.rand(B, device=DEV) * 0.6 + 0.3
    probs = torch.softmax(logits / 0.8, -1)
    keep = ref.top_k_top_p_filter(probs, k.long(), p) > 0
    seeds = torch.arange(B, dtype=torch.int64, device=DEV)
    for off in range(4):
        offsets = torch.full((B,), off, dtype=torch.int64, device=DEV)
        got = ops.sample(logits.clone(), t, k, p, None, seeds, offsets)
        assert bool(keep.gather(1, got.unsqueeze(1)).all())


def test_sampling_distribution_matches_probabilities():
    # 4096 identical rows: empirical frequencies of the top tokens follow softmax
    V, B = 1000, 4096
    torch.manual_seed(3)
    row = torch.randn(V, device=DEV) * 2
    logits = row.unsqueeze(0).repeat(B, 1).contiguous()
    t = torch.ones(B, device=DEV)
    k = torch.zeros(B, dtype=torch.int32, device=DEV)
    p = torch.ones(B, device=DEV)
    seeds = torch.arange(B, dtype=torch.int64, device=DEV) * 7919 + 13
    got = ops.sample(logits, t, k, p, None, seeds, torch.zeros(B, dtype=torch.int64, device=DEV))
    freq = torch.bincount(got, minlength=V).float() / B
    probs = torch.softmax(row, -1)
    top = probs.topk(5).indices
    assert torch.allclose(freq[top], probs[top], atol=0.03)


def test_seeded_sampling_is_reproducible():
    logits = torch.randn(8, 5000, device=DEV)
    t = torch.ones(8, device=DEV)
    k = torch.zeros(8, dtype=torch.int32, device=DEV)
    p = torch.full((8,), 0.9, device=DEV)
    seeds = torch.arange(8, dtype=torch.int64, device=DEV)
    off = torch.zeros(8, dtype=torch.int64, device=DEV)
    a = ops.sample(logits.clone(), t, k, p, None, seeds, off)
    b = ops.sample(logits.clone(), t, k, p, None, seeds, off)
    assert torch.equal(a, b)
