"""Chunk-parallel gated delta rule against the per-token recurrence (CPU, fp32), and the routing
that sends long sequences of a step to the chunked form and short ones to the recurrence."""
import numpy as np
import pytest
import torch

from vllm_ascend_b200.ops import linear_attn as la


def _case(lens, Hk=2, Hv=4, DK=16, DV=24, seed=0):
    g = torch.Generator().manual_seed(seed)
    cu = np.concatenate([[0], np.cumsum(lens)]).astype(np.int64)
    T, B = int(cu[-1]), len(lens)
    q = torch.randn(T, Hk, DK, generator=g)
    k = torch.randn(T, Hk, DK, generator=g)
    v = torch.randn(T, Hv, DV, generator=g)
    gate = -torch.rand(T, Hv, generator=g) * 0.5
    beta = torch.rand(T, Hv, generator=g)
    slots = torch.randperm(B + 2, generator=g)[:B].to(torch.int32)
    has_init = (torch.rand(B, generator=g) > 0.4).to(torch.int32)
    has_init[torch.tensor(lens) == 0] = 1           # a sequence without tokens keeps its state in both forms
    state = torch.randn(B + 2, Hv, DK, DV, generator=g) * 0.5
    return q, k, v, gate, beta, state, cu, slots, has_init


@pytest.mark.parametrize("chunk", [16, 64])
@pytest.mark.parametrize("lens", [[1, 70, 3, 200, 64, 0, 129], [5], [64, 64], [63, 65, 1]])
def test_chunked_form_equals_recurrence(lens, chunk):
    q, k, v, gate, beta, state, cu, slots, has_init = _case(lens)
    s_ref, s_ch = state.clone(), state.clone()
    cu_t = torch.tensor(cu, dtype=torch.int32)
    want = la.gated_delta_rule_ref(q, k, v, gate, beta, s_ref, cu_t, slots, has_init, 0.25)
    got = la.gated_delta_rule_chunked(q, k, v, gate, beta, s_ch, cu, slots, has_init, 0.25, chunk=chunk)
    assert (want - got).abs().max() < 1e-4
    assert (s_ref - s_ch).abs().max() < 1e-4
    # slots nobody used keep their contents
    unused = sorted(set(range(state.shape[0])) - set(int(s) for s, n in zip(slots, lens) if n > 0))
    assert torch.equal(s_ch[unused], state[unused])


def test_chunked_form_with_strong_decay_stays_finite():
    """Differences of cumulative log-decays are only exponentiated below the diagonal, where they are
    <= 0: a decay of e^-20 per token over a 64-token chunk must not overflow."""
    q, k, v, gate, beta, state, cu, slots, has_init = _case([130], seed=3)
    gate = torch.full_like(gate, -20.0)
    s_ref, s_ch = state.clone(), state.clone()
    want = la.gated_delta_rule_ref(q, k, v, gate, beta, s_ref, torch.tensor(cu, dtype=torch.int32), slots, has_init, 1.0)
    got = la.gated_delta_rule_chunked(q, k, v, gate, beta, s_ch, cu, slots, has_init, 1.0)
    assert torch.isfinite(got).all() and (want - got).abs().max() < 1e-4


def test_subset_of_sequences_leaves_other_rows_and_states_alone():
    lens = [80, 2, 100]
    q, k, v, gate, beta, state, cu, slots, has_init = _case(lens, seed=5)
    s_ref, s_ch = state.clone(), state.clone()
    want = la.gated_delta_rule_ref(q, k, v, gate, beta, s_ref, torch.tensor(cu, dtype=torch.int32), slots, has_init, 0.5)
    out = torch.full_like(v, 7.0)
    la.gated_delta_rule_chunked(q, k, v, gate, beta, s_ch, cu, slots, has_init, 0.5, seqs=[0, 2], out=out)
    assert (out[:80] - want[:80]).abs().max() < 1e-4 and (out[82:] - want[82:]).abs().max() < 1e-4
    assert torch.equal(out[80:82], torch.full_like(out[80:82], 7.0))
    assert torch.equal(s_ch[int(slots[1])], state[int(slots[1])])


def test_router_sends_long_sequences_to_the_chunked_form(monkeypatch):
    lens = [1, 70, 3, 200, 1, 64]
    q, k, v, gate, beta, state, cu, slots, has_init = _case(lens, seed=9)
    cu_t = torch.tensor(cu, dtype=torch.int32)
    calls = []
    real = la.gated_delta_rule_chunked

    def spy(*a, **kw):
        calls.append(sorted(int(x) for x in kw["seqs"]))
        return real(*a, **kw)
    monkeypatch.setattr(la, "gated_delta_rule_chunked", spy)
    s_ref, s_mix = state.clone(), state.clone()
    want = la.gated_delta_rule_ref(q, k, v, gate, beta, s_ref, cu_t, slots, has_init, 0.25)
    got = la.gated_delta_rule(q, k, v, gate, beta, s_mix, cu_t, slots, has_init, 0.25, cu_cpu=cu)
    assert calls == [[1, 3, 5]]
    assert (want - got).abs().max() < 1e-4 and (s_ref - s_mix).abs().max() < 1e-4
    # switched off: the recurrence serves everything
    monkeypatch.setenv("VLLM_B200_GDN_CHUNK_MIN", "0")
    calls.clear()
    s_off = state.clone()
    off = la.gated_delta_rule(q, k, v, gate, beta, s_off, cu_t, slots, has_init, 0.25, cu_cpu=cu)
    assert calls == [] and torch.equal(off, want)


def test_hybrid_engine_tokens_do_not_depend_on_the_form(monkeypatch):
    from vllm_ascend_b200.engine.llm import LLM
    from vllm_ascend_b200.engine.request import SamplingParams
    rng = np.random.default_rng(2)
    prompts = [rng.integers(1, 500, size=n).tolist() for n in (45, 7, 60)]
    sp = SamplingParams(max_tokens=5, temperature=0.0, ignore_eos=True)
    outs = {}
    for chunk_min in ("0", "8"):
        monkeypatch.setenv("VLLM_B200_GDN_CHUNK_MIN", chunk_min)
        llm = LLM("tiny-gdn", device="cpu", seed=0, block_size=16, max_model_len=96, max_num_seqs=4,
                  max_num_batched_tokens=32)
        outs[chunk_min] = [o.outputs[0].token_ids for o in llm.generate(prompts, sp)]
    assert outs["0"] == outs["8"]


@pytest.mark.parametrize("lens", [[1, 70, 3, 200, 64, 1, 129], [1, 1, 1], [65]])
def test_lightning_attention_batched_forms_equal_the_recurrence(lens):
    g = torch.Generator().manual_seed(11)
    H, D = 4, 16
    cu = np.concatenate([[0], np.cumsum(lens)]).astype(np.int64)
    T, B = int(cu[-1]), len(lens)
    q, k, v = (torch.randn(T, H, D, generator=g) * 0.5 for _ in range(3))
    log_decay = -torch.tensor([0.5, 0.1, 0.02, 1.5])
    slots = torch.randperm(B + 2, generator=g)[:B].to(torch.int32)
    has_init = (torch.rand(B, generator=g) > 0.4).to(torch.int32)
    state = torch.randn(B + 2, H, D, D, generator=g) * 0.5
    s_ref, s_got = state.clone(), state.clone()
    cu_t = torch.tensor(cu, dtype=torch.int32)
    want = la.lightning_attention_ref(q, k, v, log_decay, s_ref, cu_t, slots, has_init)
    got = la.lightning_attention(q, k, v, log_decay, s_got, cu_t, slots, has_init, cu_cpu=cu, chunk=64)
    assert (want - got).abs().max() < 1e-4
    assert (s_ref - s_got).abs().max() < 1e-4
    small = state.clone()
    got16 = la.lightning_attention(q, k, v, log_decay, small, cu_t, slots, has_init, cu_cpu=cu, chunk=16)
    assert (want - got16).abs().max() < 1e-4 and (s_ref - small).abs().max() < 1e-4


@pytest.mark.parametrize("Hk", [4, 1, 2])
def test_gated_linear_attention_with_per_token_decay_and_grouped_keys(Hk):
    """The Mamba-2 shape of the op: scalar decay per token and head, keys / queries shared by groups of heads."""
    g_ = torch.Generator().manual_seed(21)
    lens = [1, 40, 130, 1, 2]
    H, N, P = 4, 8, 12
    cu = np.concatenate([[0], np.cumsum(lens)]).astype(np.int64)
    T, B = int(cu[-1]), len(lens)
    q, k = torch.randn(T, Hk, N, generator=g_) * 0.5, torch.randn(T, Hk, N, generator=g_) * 0.5
    v = torch.randn(T, H, P, generator=g_)
    gate = -torch.rand(T, H, generator=g_) * 2.0
    slots = torch.randperm(B + 1, generator=g_)[:B].to(torch.int32)
    has_init = torch.tensor([1, 0, 1, 0, 1], dtype=torch.int32)
    state = torch.randn(B + 1, H, N, P, generator=g_) * 0.5
    s_ref, s_got = state.clone(), state.clone()
    cu_t = torch.tensor(cu, dtype=torch.int32)
    want = la.gated_linear_attention_ref(q, k, v, gate, s_ref, cu_t, slots, has_init)
    got = la.gated_linear_attention(q, k, v, gate, s_got, cu_t, slots, has_init, cu_cpu=cu, chunk=32)
    assert (want - got).abs().max() < 1e-4 and (s_ref - s_got).abs().max() < 1e-4


@pytest.mark.parametrize("chunk", [8, 16])
def test_kda_chunked_form_equals_the_per_channel_recurrence(chunk):
    g_ = torch.Generator().manual_seed(31)
    lens = [1, 21, 40, 16]
    H, DK, DV = 3, 8, 12
    cu = np.concatenate([[0], np.cumsum(lens)]).astype(np.int64)
    T, B = int(cu[-1]), len(lens)
    q, k = torch.randn(T, H, DK, generator=g_), torch.randn(T, H, DK, generator=g_)
    v = torch.randn(T, H, DV, generator=g_)
    gate = -torch.rand(T, H, DK, generator=g_) * 3.0                    # a different decay for every key channel
    beta = torch.rand(T, H, generator=g_)
    slots = torch.tensor([2, 0, 4, 1], dtype=torch.int32)
    has_init = torch.tensor([1, 0, 1, 1], dtype=torch.int32)
    state = torch.randn(5, H, DK, DV, generator=g_) * 0.5
    s_ref, s_got = state.clone(), state.clone()
    want = la.kda_recurrent_ref(q, k, v, gate, beta, s_ref, torch.tensor(cu, dtype=torch.int32), slots, has_init, 0.3)
    got = la.kda_chunked(q, k, v, gate, beta, s_got, cu, slots, has_init, 0.3, chunk=chunk)
    assert (want - got).abs().max() < 1e-4 and (s_ref - s_got).abs().max() < 1e-4
    assert torch.equal(s_got[3], state[3])                              # the unused slot
    # with the same decay on every channel it is the scalar-gated delta rule
    flat = gate[:, :, :1].expand(-1, -1, DK).contiguous()
    a, b = state.clone(), state.clone()
    x = la.kda_recurrent_ref(q, k, v, flat, beta, a, torch.tensor(cu, dtype=torch.int32), slots, has_init, 0.3)
    y = la.gated_delta_rule_ref(q, k, v, flat[:, :, 0], beta, b, torch.tensor(cu, dtype=torch.int32), slots, has_init, 0.3)
    assert (x - y).abs().max() < 1e-5 and (a - b).abs().max() < 1e-5
