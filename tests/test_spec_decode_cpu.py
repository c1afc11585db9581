"""Speculative decoding on CPU: proposers, rejection sampling rules, and engine equivalence
(greedy speculative generation must equal plain greedy generation token for token)."""
import numpy as np
import pytest
import torch

from vllm_ascend_b200 import LLM, SamplingParams
from vllm_ascend_b200.sample.rejection_sampler import (RejectionSampler, block_verify_accept_len,
                                                       entropy_threshold, rejection_sample_ref)
from vllm_ascend_b200.spec_decode.ngram import NgramProposer, find_ngram_continuation
from vllm_ascend_b200.spec_decode.suffix import SuffixProposer


def test_ngram_lookup():
    t = np.array([5, 6, 7, 8, 9, 1, 2, 6, 7, 8], dtype=np.int32)
    assert find_ngram_continuation(t, 2, 4, 3).tolist() == [9, 1, 2]       # suffix 6 7 8 seen before
    assert find_ngram_continuation(t, 4, 5, 3).tolist() == []              # no 4-gram repeats
    assert find_ngram_continuation(np.array([1, 2, 3], dtype=np.int32), 1, 3, 2).tolist() == []
    # the most recent occurrence wins
    t2 = np.array([1, 2, 3, 9, 1, 2, 4, 9, 1, 2], dtype=np.int32)
    assert find_ngram_continuation(t2, 2, 2, 1).tolist() == [4]
    p = NgramProposer(3, 2, 4, max_model_len=12)
    table = np.zeros((2, 16), dtype=np.int32)
    table[1, :10] = t
    assert [x.tolist() for x in p.propose(table, np.array([10]), np.array([1]))] == [[9]]   # capped by max_model_len


def test_suffix_proposer_learns_across_requests():
    p = SuffixProposer(3, key_len=2)
    table = np.zeros((2, 32), dtype=np.int32)
    table[0, :8] = [1, 2, 3, 4, 5, 6, 7, 8]
    p.propose(table, np.array([8]), np.array([0]))
    table[1, :4] = [9, 9, 3, 4]
    out = p.propose(table, np.array([4]), np.array([1]))
    assert out[0].tolist() == [5, 6, 7]


def test_rejection_greedy_and_padding():
    draft = torch.tensor([4, 5, 6, 7, 8], dtype=torch.int32)
    cu = torch.tensor([0, 3, 3, 5], dtype=torch.int32)
    argmax = torch.tensor([4, 5, 9, 7, 8], dtype=torch.int32)
    bonus = torch.tensor([11, 12, 13], dtype=torch.int32)
    out, num = rejection_sample_ref(draft, cu, argmax, bonus, None, None, None, None, torch.ones(3, dtype=torch.bool), 3)
    assert out.tolist() == [[4, 5, 9, -1], [12, -1, -1, -1], [7, 8, 13, -1]]
    assert num.tolist() == [3, 1, 3]


def test_rejection_random_preserves_target_distribution():
    """One draft position, deterministic proposal (no draft probs): emitted token must be
    distributed as the target distribution."""
    torch.manual_seed(0)
    V, N = 6, 20000
    pt = torch.tensor([0.05, 0.4, 0.1, 0.25, 0.15, 0.05])
    x = 1
    draft = torch.full((N,), x, dtype=torch.int32)
    cu = torch.arange(N + 1, dtype=torch.int32)
    probs = pt.expand(N, V).contiguous()
    bonus = torch.full((N,), -7, dtype=torch.int32)
    out, num = rejection_sample_ref(draft, cu, probs.argmax(-1).int(), bonus, probs, None, torch.rand(N),
                                    torch.empty(N, V).exponential_(), torch.zeros(N, dtype=torch.bool), 1)
    first = out[:, 0]
    freq = torch.bincount(first.long(), minlength=V).float() / N
    assert (freq - pt).abs().max() < 0.02
    accepted = (num == 2)
    assert abs(float(accepted.float().mean()) - 0.4) < 0.02
    assert (out[accepted, 1] == -7).all()
    # with draft probabilities: p_d = one-hot on another token x2 with p_t(x2) = 0.1 < 1
    pd = torch.zeros(N, V)
    pd[:, 2] = 1.0
    draft2 = torch.full((N,), 2, dtype=torch.int32)
    out2, _ = rejection_sample_ref(draft2, cu, probs.argmax(-1).int(), bonus, probs, pd, torch.rand(N),
                                   torch.empty(N, V).exponential_(), torch.zeros(N, dtype=torch.bool), 1)
    freq2 = torch.bincount(out2[:, 0].long(), minlength=V).float() / N
    assert (freq2 - pt).abs().max() < 0.02


def test_block_and_entropy_rules():
    pt = torch.tensor([0.9, 0.2, 0.9])
    pd = torch.tensor([1.0, 1.0, 1.0])
    assert block_verify_accept_len(pt, pd, torch.tensor([0.5, 0.5, 0.1])) == 3     # joint ratio .9*.2*.9=.162 >= .1
    assert block_verify_accept_len(pt, pd, torch.tensor([0.95, 0.5, 0.5])) == 0
    conf = torch.tensor([0.97, 0.01, 0.01, 0.01])
    flat = torch.full((4,), 0.25)
    assert entropy_threshold(conf, 1.0, 0.9) > entropy_threshold(flat, 1.0, 0.9)
    assert entropy_threshold(conf, 0.0, 0.6) == 0.6
    rs = RejectionSampler("entropy_verify", 1.0, 0.5)
    logits = torch.log(torch.stack([conf, flat]))
    out, num = rs(torch.tensor([0, 2], dtype=torch.int32), torch.tensor([0, 2], dtype=torch.int32), logits,
                  torch.tensor([3], dtype=torch.int32), torch.zeros(1, dtype=torch.bool), torch.ones(1), 2)
    assert out[0, :2].tolist() == [0, 2] and int(num[0]) == 3      # both clear their thresholds
    with pytest.raises(ValueError):
        RejectionSampler("nope")


@pytest.mark.parametrize("method", ["ngram", "suffix"])
def test_engine_speculative_greedy_equals_plain_greedy(method):
    kw = dict(device="cpu", seed=0, block_size=16, max_model_len=160, max_num_seqs=4, max_num_batched_tokens=48)
    rng = np.random.default_rng(0)
    # repetitive prompts so that lookups hit
    base = rng.integers(1, 400, size=12).tolist()
    prompts = [base * 3 + base[:5], rng.integers(1, 400, size=30).tolist(), (base[::-1] * 2)[:20]]
    sp = SamplingParams(max_tokens=24, temperature=0.0, ignore_eos=True)
    want = [o.outputs[0].token_ids for o in LLM("tiny-qwen", **kw).generate(prompts, sp)]
    llm = LLM("tiny-qwen", speculative_config={"method": method, "num_speculative_tokens": 3,
                                               "prompt_lookup_min": 1, "prompt_lookup_max": 4}, **kw)
    got = [o.outputs[0].token_ids for o in llm.generate(prompts, sp)]
    assert got == want
    st = llm.engine.runner.spec_stats
    assert st["verify_steps"] > 0 and st["draft_tokens"] > 0
    assert llm.engine.scheduler.num_draft_tokens == st["draft_tokens"]
    # KV bookkeeping survived rejections: a second pass with the same engine is still right
    got2 = [o.outputs[0].token_ids for o in llm.generate(prompts, sp)]
    assert got2 == want


def test_engine_speculative_random_sampling_runs_and_respects_max_tokens():
    llm = LLM("tiny-qwen", device="cpu", seed=0, block_size=16, max_model_len=128, max_num_seqs=4,
              speculative_config={"method": "ngram", "num_speculative_tokens": 4, "prompt_lookup_min": 1})
    prompts = [[7, 8, 9] * 8, [3, 4] * 10]
    outs = llm.generate(prompts, SamplingParams(max_tokens=17, temperature=0.8, top_k=20, seed=1, ignore_eos=True))
    assert all(len(o.outputs[0].token_ids) == 17 for o in outs)


@pytest.mark.parametrize("method", ["draft_model", "eagle", "eagle3", "medusa"])
def test_engine_model_based_proposers_keep_greedy_output(method):
    kw = dict(device="cpu", seed=0, block_size=16, max_model_len=160, max_num_seqs=4, max_num_batched_tokens=40)
    rng = np.random.default_rng(1)
    prompts = [rng.integers(1, 400, size=n).tolist() for n in (45, 9, 70)]      # 70 > token budget: chunked prefill
    sp = SamplingParams(max_tokens=14, temperature=0.0, ignore_eos=True)
    want = [o.outputs[0].token_ids for o in LLM("tiny-qwen", **kw).generate(prompts, sp)]
    spec = {"method": method, "num_speculative_tokens": 3}
    if method == "draft_model":
        spec["model"] = "tiny-qwen"          # same weights as the target: every draft must be accepted
    llm = LLM("tiny-qwen", speculative_config=spec, **kw)
    got = [o.outputs[0].token_ids for o in llm.generate(prompts, sp)]
    assert got == want
    st = llm.engine.runner.spec_stats
    assert st["draft_tokens"] > 0
    if method == "draft_model":
        assert st["accepted_tokens"] == st["draft_tokens"]
        # far fewer target steps than tokens
        assert st["verify_steps"] <= 5
    assert llm.engine.runner.proposer.stats["draft_forwards"] > 0


def test_eagle3_head_reads_three_residual_streams_and_loads_hf_names(tmp_path):
    from vllm_ascend_b200.spec_decode.draft_model import Eagle3Head
    llm = LLM("tiny-qwen", device="cpu", seed=0, block_size=16, max_model_len=128, max_num_seqs=4,
              speculative_config={"method": "eagle3", "num_speculative_tokens": 2, "draft_vocab_size": 128})
    target = llm.engine.runner.model
    head = llm.engine.runner.proposer.model
    assert isinstance(head, Eagle3Head) and len(target.aux_layers) == 3
    assert head.fc_weight.shape == (target.cfg.hidden_size, 3 * target.cfg.hidden_size)
    assert head.layers[0].self_attn.qkv_proj.weight.shape[1] == 2 * target.cfg.hidden_size
    llm.generate([[1, 2, 3, 4, 5, 6]], SamplingParams(max_tokens=4, temperature=0.0, ignore_eos=True))
    assert target.aux_hidden.shape[-1] == 3 * target.cfg.hidden_size
    # checkpoint names of the published heads: split q/k/v and gate/up, reduced vocabulary + d2t
    H, D = target.cfg.hidden_size, target.cfg.head_dim
    nq, nkv, I = target.cfg.num_attention_heads * D, target.cfg.num_key_value_heads * D, target.cfg.intermediate_size
    g = torch.Generator().manual_seed(3)
    ck = {"fc.weight": torch.randn(H, 3 * H, generator=g), "midlayer.self_attn.q_proj.weight": torch.randn(nq, 2 * H, generator=g),
          "midlayer.self_attn.k_proj.weight": torch.randn(nkv, 2 * H, generator=g),
          "midlayer.self_attn.v_proj.weight": torch.randn(nkv, 2 * H, generator=g),
          "midlayer.self_attn.o_proj.weight": torch.randn(H, nq, generator=g),
          "midlayer.mlp.gate_proj.weight": torch.randn(I, H, generator=g), "midlayer.mlp.up_proj.weight": torch.randn(I, H, generator=g),
          "midlayer.mlp.down_proj.weight": torch.randn(H, I, generator=g), "midlayer.hidden_norm.weight": torch.rand(H, generator=g),
          "midlayer.input_layernorm.weight": torch.rand(H, generator=g), "midlayer.post_attention_layernorm.weight": torch.rand(H, generator=g),
          "norm.weight": torch.rand(H, generator=g), "lm_head.weight": torch.randn(128, H, generator=g),
          "d2t": torch.arange(128) * 3}
    loaded = head.load_weights(ck.items())
    assert loaded == set(ck)
    qkv = head.layers[0].self_attn.qkv_proj.weight
    assert torch.equal(qkv[nq:nq + nkv], ck["midlayer.self_attn.k_proj.weight"])
    assert torch.equal(head.layers[0].mlp.gate_up_proj.weight[I:], ck["midlayer.mlp.up_proj.weight"])
    toks = head.draft_tokens(torch.randn(5, H, generator=g))
    assert ((toks % 4) == 0).all() and toks.max() < 128 * 4             # index + d2t[index] = 4 * index


def test_mtp_head_on_mla_moe_target_keeps_greedy_output_and_loads_layer_n(tmp_path):
    """DeepSeek-style target (MLA + MoE): the MTP module is a full decoder layer of the target's kind
    with its own latent cache; speculative decoding leaves greedy output unchanged; tensors of layer
    N in a checkpoint stream go to the module."""
    from vllm_ascend_b200.spec_decode.draft_model import MTPHead
    kw = dict(device="cpu", seed=0, block_size=16, max_model_len=160, max_num_seqs=4, max_num_batched_tokens=40)
    rng = np.random.default_rng(1)
    prompts = [rng.integers(1, 400, size=n).tolist() for n in (45, 9, 70)]
    sp = SamplingParams(max_tokens=12, temperature=0.0, ignore_eos=True)
    want = [o.outputs[0].token_ids for o in LLM("tiny-deepseek", **kw).generate(prompts, sp)]
    llm = LLM("tiny-deepseek", speculative_config={"method": "mtp", "num_speculative_tokens": 2}, **kw)
    got = [o.outputs[0].token_ids for o in llm.generate(prompts, sp)]
    assert got == want
    head = llm.engine.runner.proposer.model
    assert isinstance(head, MTPHead) and hasattr(head.layers[0].self_attn, "dc") and hasattr(head.layers[0].mlp, "w13")
    assert llm.engine.runner.spec_stats["draft_tokens"] > 0
    N, H = head.idx, llm.cfg.model.hidden_size
    g = torch.Generator().manual_seed(0)
    E, I = llm.cfg.model.num_experts, llm.cfg.model.moe_intermediate_size
    ck = {f"model.layers.{N}.enorm.weight": torch.rand(H, generator=g), f"model.layers.{N}.hnorm.weight": torch.rand(H, generator=g),
          f"model.layers.{N}.eh_proj.weight": torch.randn(H, 2 * H, generator=g),
          f"model.layers.{N}.shared_head.norm.weight": torch.rand(H, generator=g),
          f"model.layers.{N}.shared_head.head.weight": torch.randn(llm.cfg.model.vocab_size, H, generator=g),
          f"model.layers.{N}.input_layernorm.weight": torch.rand(H, generator=g),
          f"model.layers.{N}.mlp.experts.3.down_proj.weight": torch.randn(H, I, generator=g),
          f"model.layers.{N}.self_attn.o_proj.weight": torch.randn(H, head.layers[0].self_attn.o_proj.weight.shape[1], generator=g),
          "model.layers.0.input_layernorm.weight": torch.rand(H, generator=g)}
    loaded = head.load_weights(ck.items())
    assert loaded == {k for k in ck if k.startswith(f"model.layers.{N}.")}
    assert torch.equal(head.eh_proj_weight, ck[f"model.layers.{N}.eh_proj.weight"])
    assert torch.equal(head.layers[0].mlp.w2[3], ck[f"model.layers.{N}.mlp.experts.3.down_proj.weight"])
    assert torch.equal(head.layers[0].input_layernorm.weight, ck[f"model.layers.{N}.input_layernorm.weight"])


def test_dynamic_speculation_length_follows_acceptance():
    from vllm_ascend_b200.platform_config import clear_b200_config
    from vllm_ascend_b200.spec_decode.dynamic import DynamicSpecController
    c = DynamicSpecController(6, {"budget_threshold": 0.3, "ema_alpha": 0.5, "initial_acceptance": 0.7})
    assert c.budget("a") == 3                              # 0.7^3 = 0.34 >= 0.3 > 0.7^4
    for _ in range(6):
        c.update("a", 4, 4)
    assert c.budget("a") == 6
    for _ in range(8):
        c.update("a", 4, 0)
    assert c.budget("a") == 1
    c.forget("a")
    assert c.budget("a") == 3
    # engine: a random EAGLE head is almost never right, so its budget collapses to the minimum while
    # greedy output stays exact
    kw = dict(device="cpu", seed=0, block_size=16, max_model_len=160, max_num_seqs=4, max_num_batched_tokens=40)
    prompts = [[7, 8, 9, 10, 11, 12] * 3, [3, 4, 5] * 4]
    sp = SamplingParams(max_tokens=20, temperature=0.0, ignore_eos=True)
    want = [o.outputs[0].token_ids for o in LLM("tiny-qwen", **kw).generate(prompts, sp)]
    spec = {"method": "eagle", "num_speculative_tokens": 4}
    fixed = LLM("tiny-qwen", speculative_config=spec, **kw)
    assert [o.outputs[0].token_ids for o in fixed.generate(prompts, sp)] == want
    dyn = LLM("tiny-qwen", speculative_config=spec, additional_config={
        "dynamic_spec_config": {"method": "acceptance", "method_params": {"ema_alpha": 0.6}}}, **kw)
    assert [o.outputs[0].token_ids for o in dyn.generate(prompts, sp)] == want
    assert dyn.engine.runner.spec_stats["draft_tokens"] < fixed.engine.runner.spec_stats["draft_tokens"]
    clear_b200_config()


def test_shared_verify_budget_goes_to_the_most_promising_draft_prefixes():
    from vllm_ascend_b200.platform_config import clear_b200_config
    from vllm_ascend_b200.spec_decode.dynamic import DynamicSpecController, VerifyBudgetAllocator
    a = VerifyBudgetAllocator(6, {"initial_verify_budget_per_req": 3, "budget_update_interval": 2,
                                  "budget_threshold": 0.3, "min_verify_tokens": 1})
    probs = np.array([[0.99] * 6,            # drafts that almost surely pass
                      [0.2] * 6,             # hopeless ones
                      [0.9, 0.9, 0.1, 0.9, 0.9, 0.9]])
    lens = a.allocate(probs)
    # 3 requests x budget 3 = 9 verify tokens: everyone gets one, the other six go where survival is highest
    assert lens.sum() == 9 and lens.tolist() == [6, 1, 2]
    # second step: the budget is re-estimated: positions with survival >= 0.3 are 6 + 0 + 2 -> mean 2.67 -> 3 (odd)
    lens = a.allocate(probs)
    assert a.budget_k == 3 and lens.tolist() == [6, 1, 2]
    good = np.full((2, 6), 0.95)
    a.allocate(good)
    a.allocate(good)                           # update step: 6 positions each -> 6 (the maximum; no odd bump past it)
    assert a.budget_k == 6 and a.allocate(good).tolist() == [6, 6]
    even = VerifyBudgetAllocator(6, {"budget_update_interval": 1, "budget_threshold": 0.5})
    even.allocate(np.array([[0.9, 0.9, 0.9, 0.9, 0.1, 0.1]]))      # 4 positions above 0.5 -> bumped to 5
    assert even.budget_k == 5
    # controller: the per-request estimates stand in when the proposer has no confidences
    c = DynamicSpecController(4, {"shared_budget": True, "initial_verify_budget_per_req": 2, "ema_alpha": 1.0})
    c.update("hot", 4, 4)
    c.update("cold", 4, 0)
    assert c.budgets(["hot", "cold"]) == [3, 1]
    assert DynamicSpecController(4, {}).budgets(["x"]) == [DynamicSpecController(4, {}).budget("x")]
    # engine run on the shared budget: exact greedy output
    kw = dict(device="cpu", seed=0, block_size=16, max_model_len=160, max_num_seqs=4, max_num_batched_tokens=40)
    prompts = [[7, 8, 9, 10, 11, 12] * 3, [3, 4, 5] * 4]
    sp = SamplingParams(max_tokens=16, temperature=0.0, ignore_eos=True)
    want = [o.outputs[0].token_ids for o in LLM("tiny-qwen", **kw).generate(prompts, sp)]
    dyn = LLM("tiny-qwen", speculative_config={"method": "ngram", "num_speculative_tokens": 4}, additional_config={
        "dynamic_spec_config": {"method": "acceptance", "method_params": {"shared_budget": True}}}, **kw)
    assert [o.outputs[0].token_ids for o in dyn.generate(prompts, sp)] == want
    assert dyn.engine.runner.dynamic_spec.allocator is not None
    clear_b200_config()


def test_extract_hidden_states_records_every_position(tmp_path):
    kw = dict(device="cpu", seed=0, block_size=16, max_model_len=160, max_num_seqs=4, max_num_batched_tokens=24)
    prompts = [[7, 8, 9, 10, 11, 12] * 6, [3, 4, 5] * 4]
    sp = SamplingParams(max_tokens=5, temperature=0.0, ignore_eos=True)
    want = [o.outputs[0].token_ids for o in LLM("tiny-qwen", **kw).generate(prompts, sp)]
    llm = LLM("tiny-qwen", speculative_config={"method": "extract_hidden_states", "layers": [0, 1],
                                               "output_dir": str(tmp_path)}, **kw)
    outs = llm.generate(prompts, sp)
    assert [o.outputs[0].token_ids for o in outs] == want                  # nothing is drafted
    H = llm.cfg.model.hidden_size
    for o, p in zip(outs, prompts):
        rec = torch.load(tmp_path / f"{o.request_id}.pt")
        # every computed position: the prompt and all generated tokens but the last one
        assert rec["hidden_states"].shape == (len(p) + 5 - 1, 2 * H)
        assert rec["token_ids"] == p + o.outputs[0].token_ids
    mem = LLM("tiny-qwen", speculative_config={"method": "extract_hidden_states"}, **kw)
    o = mem.generate(prompts[:1], sp)[0]
    assert mem.engine.runner.proposer.results[o.request_id].shape == (len(prompts[0]) + 4, H)
