"""End-to-end CPU fp32 checks of the engine plumbing (scheduler, paged cache,
model runner) against independent oracles: HF transformers for the dense
families and a cache-free recomputation for every family."""
import numpy as np
import pytest
import torch

from vllm_ascend_b200.config import get_model_config
from vllm_ascend_b200.engine.llm import LLM
from vllm_ascend_b200.engine.request import SamplingParams
from vllm_ascend_b200.models.transformer import export_hf_state_dict


def _prompts(n, length, vocab, seed=0):
    rng = np.random.default_rng(seed)
    return [rng.integers(0, vocab, size=length).tolist() for _ in range(n)]


def _hf_greedy(hf_model, prompt, n_new):
    ids = torch.tensor([prompt])
    out = []
    with torch.no_grad():
        for _ in range(n_new):
            logits = hf_model(ids).logits[0, -1]
            t = int(logits.argmax())
            out.append(t)
            ids = torch.cat([ids, torch.tensor([[t]])], dim=1)
    return out


def _make_hf(cfg, sd):
    import transformers
    common = dict(vocab_size=cfg.vocab_size, hidden_size=cfg.hidden_size,
                  intermediate_size=cfg.intermediate_size, num_hidden_layers=cfg.num_hidden_layers,
                  num_attention_heads=cfg.num_attention_heads,
                  num_key_value_heads=cfg.num_key_value_heads, head_dim=cfg.head_dim,
                  rms_norm_eps=cfg.rms_norm_eps, rope_theta=cfg.rope_theta,
                  max_position_embeddings=4096, tie_word_embeddings=False,
                  attention_bias=False, torch_dtype=torch.float32)
    if cfg.architecture == "Qwen3ForCausalLM":
        hc = transformers.Qwen3Config(**common)
        hc.rope_parameters = {"rope_type": "default", "rope_theta": cfg.rope_theta}
        m = transformers.Qwen3ForCausalLM(hc)
    else:
        hc = transformers.LlamaConfig(**common)
        hc.rope_parameters = {"rope_type": "default", "rope_theta": cfg.rope_theta}
        m = transformers.LlamaForCausalLM(hc)
    missing, unexpected = m.load_state_dict(sd, strict=False)
    assert not [k for k in missing if "rotary" not in k], missing
    assert not unexpected, unexpected
    return m.eval().float()


@pytest.mark.parametrize("preset", ["tiny-qwen", "tiny-llama"])
def test_greedy_matches_hf(preset):
    """Config 1 of the benchmark list: 4 prompts x 32 tokens, 16 greedy tokens, block 16."""
    cfg = get_model_config(preset)
    llm = LLM(cfg, device="cpu", max_model_len=128, max_num_seqs=8, max_num_batched_tokens=48,
              block_size=16)
    prompts = _prompts(4, 32, cfg.vocab_size)
    outs = llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=16, ignore_eos=True))
    hf = _make_hf(cfg, export_hf_state_dict(llm.engine.runner.model))
    for p, o in zip(prompts, outs):
        assert o.outputs[0].token_ids == _hf_greedy(hf, p, 16)
        assert o.outputs[0].finish_reason == "length"


def _recompute_greedy(model, prompt, n_new, block_size=16):
    """Cache-free oracle: every step re-runs the whole sequence as one prefill."""
    from vllm_ascend_b200.attention.metadata import AttentionMetadata
    cfg = model.cfg
    out = []
    ids = list(prompt)
    for _ in range(n_new):
        T = len(ids)
        nblk = (T + block_size - 1) // block_size + 1
        caches = []
        for L in model.layers:
            if cfg.use_mla:
                shapes = [(nblk, block_size, 1, cfg.kv_lora_rank), (nblk, block_size, 1, cfg.qk_rope_head_dim)]
            else:
                a = L.self_attn
                shapes = [(nblk, block_size, a.Hkv, a.D)] * 2
            caches.append(tuple(torch.zeros(s) for s in shapes))
        pos = torch.arange(T)
        meta = AttentionMetadata(
            num_reqs=1, num_actual_tokens=T, max_query_len=T, max_seq_len=T,
            query_start_loc=torch.tensor([0, T], dtype=torch.int32),
            seq_lens=torch.tensor([T], dtype=torch.int32),
            block_table=torch.arange(1, nblk, dtype=torch.int32).unsqueeze(0),
            slot_mapping=pos + block_size, positions=pos,
            query_start_loc_cpu=np.array([0, T]), seq_lens_cpu=np.array([T]))
        with torch.no_grad():
            h = model.forward(torch.tensor(ids), meta, caches)
            t = int(model.compute_logits(h[-1:]).argmax())
        out.append(t)
        ids.append(t)
    return out


@pytest.mark.parametrize("preset", ["tiny-moe", "tiny-deepseek"])
def test_greedy_matches_recompute(preset):
    cfg = get_model_config(preset)
    llm = LLM(cfg, device="cpu", max_model_len=128, max_num_seqs=4, max_num_batched_tokens=24,
              block_size=16)
    prompts = _prompts(3, 20, cfg.vocab_size, seed=1)
    outs = llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=8, ignore_eos=True))
    for p, o in zip(prompts, outs):
        assert o.outputs[0].token_ids == _recompute_greedy(llm.engine.runner.model, p, 8)


def test_chunked_prefill_and_preemption_are_transparent():
    cfg = get_model_config("tiny-qwen")
    sp = SamplingParams(temperature=0.0, max_tokens=12, ignore_eos=True)
    prompts = _prompts(6, 40, cfg.vocab_size, seed=3)
    big = LLM(cfg, device="cpu", max_model_len=128, max_num_seqs=8, max_num_batched_tokens=512, block_size=16)
    ref = [o.outputs[0].token_ids for o in big.generate(prompts, sp)]
    # tiny token budget -> chunked prefill; tiny pool -> recompute preemption
    small = LLM(cfg, device="cpu", max_model_len=128, max_num_seqs=8, max_num_batched_tokens=16,
                block_size=16, num_gpu_blocks_override=14)
    small.engine.scheduler.reserve_full = False      # over-admit so decode must preempt
    got = [o.outputs[0].token_ids for o in small.generate(prompts, sp)]
    assert got == ref
    assert small.engine.scheduler.num_preemptions > 0
    # with whole-sequence reservation the same pool never preempts
    calm = LLM(cfg, device="cpu", max_model_len=128, max_num_seqs=8, max_num_batched_tokens=16,
               block_size=16, num_gpu_blocks_override=14)
    assert [o.outputs[0].token_ids for o in calm.generate(prompts, sp)] == ref
    assert calm.engine.scheduler.num_preemptions == 0


def test_prefix_caching_reuses_blocks_and_keeps_outputs():
    cfg = get_model_config("tiny-qwen")
    sp = SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True)
    shared = _prompts(1, 48, cfg.vocab_size, seed=5)[0]
    prompts = [shared + t for t in _prompts(3, 8, cfg.vocab_size, seed=6)]
    plain = LLM(cfg, device="cpu", max_model_len=128, max_num_seqs=4, block_size=16)
    ref = [o.outputs[0].token_ids for o in plain.generate(prompts, sp)]
    pc = LLM(cfg, device="cpu", max_model_len=128, max_num_seqs=4, block_size=16,
             enable_prefix_caching=True)
    first = pc.generate(prompts[:1], sp)
    rest = pc.generate(prompts[1:], sp)
    assert [o.outputs[0].token_ids for o in first + rest] == ref
    assert all(o.num_cached_tokens == 48 for o in rest)


def test_stop_token_and_sampling_params_validation():
    cfg = get_model_config("tiny-qwen")
    llm = LLM(cfg, device="cpu", max_model_len=128, max_num_seqs=4, block_size=16)
    p = _prompts(1, 16, cfg.vocab_size, seed=9)
    full = llm.generate(p, SamplingParams(temperature=0.0, max_tokens=10, ignore_eos=True))[0].outputs[0].token_ids
    stop_at = full[3]
    out = llm.generate(p, SamplingParams(temperature=0.0, max_tokens=10, stop_token_ids=[stop_at]))[0]
    assert out.outputs[0].token_ids == full[:full.index(stop_at) + 1]
    assert out.outputs[0].finish_reason == "stop"
    with pytest.raises(ValueError):
        SamplingParams(top_p=0.0)
    with pytest.raises(ValueError):
        SamplingParams(temperature=-1)


def test_random_sampling_is_seeded_and_respects_top_k():
    cfg = get_model_config("tiny-qwen")
    llm = LLM(cfg, device="cpu", max_model_len=128, max_num_seqs=4, block_size=16, seed=7)
    p = _prompts(2, 16, cfg.vocab_size, seed=11)
    sp = SamplingParams(temperature=1.0, top_k=1, max_tokens=6, ignore_eos=True)
    greedy = SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True)
    a = [o.outputs[0].token_ids for o in llm.generate(p, sp)]
    g = [o.outputs[0].token_ids for o in llm.generate(p, greedy)]
    assert a == g          # top_k=1 is greedy whatever the noise


@pytest.mark.parametrize("prefix_caching", [False, True])
def test_async_scheduling_matches_synchronous_engine(prefix_caching):
    """One-step lookahead: scheduling and input preparation of step N+1 happen before step N's
    tokens are read; generated tokens, stop handling and block accounting must not change."""
    kw = dict(device="cpu", seed=0, block_size=16, max_model_len=96, max_num_seqs=4, max_num_batched_tokens=32,
              enable_prefix_caching=prefix_caching)
    rng = np.random.default_rng(3)
    prompts = [rng.integers(1, 500, size=n).tolist() for n in (40, 5, 23, 61, 9, 33)]
    sps = [SamplingParams(max_tokens=m, temperature=0.0, ignore_eos=True) for m in (7, 1, 12, 3, 20, 2)]
    sync = LLM("tiny-qwen", async_scheduling=False, **kw)
    want = [o.outputs[0].token_ids for o in sync.generate(prompts, sps)]
    llm = LLM("tiny-qwen", async_scheduling=True, **kw)
    assert llm.engine.async_scheduling
    got = [o.outputs[0].token_ids for o in llm.generate(prompts, sps)]
    assert got == want
    assert [len(g) for g in got] == [7, 1, 12, 3, 20, 2]
    pool = llm.engine.scheduler.pool
    assert pool.num_free_blocks == sync.engine.scheduler.pool.num_free_blocks
    assert not llm.engine.scheduler.running and llm.engine._inflight is None
    # stop tokens are honoured although the following step was already launched
    stop = want[2][4]
    sp = SamplingParams(max_tokens=12, temperature=0.0, stop_token_ids=[stop])
    a = llm.generate([prompts[2]], sp)[0].outputs[0].token_ids
    b = sync.generate([prompts[2]], sp)[0].outputs[0].token_ids
    assert a == b and a[-1] == stop
    # random sampling with a seed runs through the same path
    sp = SamplingParams(max_tokens=6, temperature=0.9, top_k=50, seed=11, ignore_eos=True)
    assert len(llm.generate(prompts[:2], sp)[1].outputs[0].token_ids) == 6


def test_weight_offload_with_prefetch_keeps_outputs():
    kw = dict(device="cpu", seed=0, block_size=16, max_model_len=96, max_num_seqs=4)
    rng = np.random.default_rng(8)
    prompts = [rng.integers(1, 500, size=n).tolist() for n in (30, 11)]
    sp = SamplingParams(max_tokens=6, temperature=0.0, ignore_eos=True)
    want = [o.outputs[0].token_ids for o in LLM("tiny-qwen", **kw).generate(prompts, sp)]
    llm = LLM("tiny-qwen", additional_config={"weight_offload_config": {
        "enabled": True, "group_size": 2, "num_in_group": 1, "prefetch_step": 1}}, **kw)
    off = llm.engine.worker.offloader
    assert off is not None and off.bytes_offloaded > 0 and len(off.layers) >= 1
    got = [o.outputs[0].token_ids for o in llm.generate(prompts, sp)]
    assert got == want
    assert off.stats["prefetches"] >= len(off.layers) * 6
    from vllm_ascend_b200.platform_config import clear_b200_config
    clear_b200_config()


def test_hybrid_linear_attention_model_matches_cache_free_recompute():
    """Gated DeltaNet hybrid: chunked prefill, batching and decode through the per-sequence
    recurrent states must equal a pass that recomputes every prefix from scratch."""
    kw = dict(device="cpu", seed=0, block_size=16, max_model_len=96, max_num_seqs=4)
    rng = np.random.default_rng(12)
    prompts = [rng.integers(1, 500, size=n).tolist() for n in (37, 9, 50)]
    sp = SamplingParams(max_tokens=6, temperature=0.0, ignore_eos=True)
    llm = LLM("tiny-gdn", max_num_batched_tokens=24, **kw)                  # several chunks per prompt
    assert any(getattr(L.self_attn, "is_linear_attention", False) for L in llm.engine.runner.model.layers)
    got = [o.outputs[0].token_ids for o in llm.generate(prompts, sp)]
    # oracle: one request at a time, whole prompt in one step, fresh engine per continuation length
    want = []
    for p in prompts:
        toks = []
        for _ in range(6):
            one = LLM("tiny-gdn", max_num_batched_tokens=128, **kw)
            t = one.generate([p + toks], SamplingParams(max_tokens=1, temperature=0.0, ignore_eos=True))
            toks.append(t[0].outputs[0].token_ids[0])
        want.append(toks)
    assert got == want
    # rows are reused by later requests: states must not leak between them
    again = [o.outputs[0].token_ids for o in llm.generate(prompts[::-1], sp)]
    assert again == want[::-1]


def test_logit_processors_and_logprobs():
    """allowed_token_ids, bad words (single- and multi-token), logit_bias, min_tokens and logprobs
    act on the distribution the way the public API promises."""
    llm = LLM("tiny-qwen", device="cpu", max_model_len=128, max_num_seqs=8, max_num_batched_tokens=64, block_size=16)
    prompt = [5, 6, 7, 8, 9]
    base = llm.generate([prompt], SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True, logprobs=3))[0].outputs[0]
    toks = base.token_ids
    assert len(base.logprobs) == 6
    for t, lp in zip(toks, base.logprobs):
        assert t in lp and len(lp) in (3, 4) and max(lp.values()) == lp[t] <= 0.0       # greedy: the top entry
    # allowed ids: only these tokens can appear
    allowed = [11, 12, 13]
    out = llm.generate([prompt], SamplingParams(temperature=0.0, max_tokens=5, ignore_eos=True,
                                                allowed_token_ids=allowed))[0].outputs[0].token_ids
    assert set(out) <= set(allowed)
    # single-token bad word: the greedy first token is replaced by the runner-up
    second = sorted(base.logprobs[0].items(), key=lambda kv: -kv[1])[1][0]
    out = llm.generate([prompt], SamplingParams(temperature=0.0, max_tokens=3, ignore_eos=True,
                                                bad_words_token_ids=[[toks[0]]]))[0].outputs[0].token_ids
    assert out[0] == second and toks[0] not in out
    # multi-token bad word: banned only after its prefix was generated
    out = llm.generate([prompt], SamplingParams(temperature=0.0, max_tokens=4, ignore_eos=True,
                                                bad_words_token_ids=[[toks[0], toks[1]]]))[0].outputs[0].token_ids
    assert out[0] == toks[0] and out[1] != toks[1]
    # a large bias forces a token
    out = llm.generate([prompt], SamplingParams(temperature=0.0, max_tokens=3, ignore_eos=True,
                                                logit_bias={77: 1000.0}))[0].outputs[0].token_ids
    assert out == [77, 77, 77]
    # min_tokens keeps a stop token away until the minimum is reached
    stop = toks[1]
    early = llm.generate([prompt], SamplingParams(temperature=0.0, max_tokens=8, stop_token_ids=[stop]))[0].outputs[0].token_ids
    late = llm.generate([prompt], SamplingParams(temperature=0.0, max_tokens=8, stop_token_ids=[stop],
                                                 min_tokens=4))[0].outputs[0].token_ids
    assert len(early) == 2 and early[-1] == stop
    assert len(late) >= 4 and stop not in late[:4]


def test_prompt_embeds_and_embedding_api():
    """Prompt embeddings equal to the model's own token embeddings reproduce the token-id run; embed()
    returns the last prompt token's final hidden state."""
    llm = LLM("tiny-qwen", device="cpu", max_model_len=128, max_num_seqs=8, max_num_batched_tokens=16, block_size=16)
    model = llm.engine.runner.model
    rng = np.random.default_rng(4)
    prompts = [rng.integers(1, 400, size=n).tolist() for n in (21, 5, 40)]
    sp = SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True)
    want = [o.outputs[0].token_ids for o in llm.generate(prompts, sp)]
    embeds = [model.embed_input_ids(torch.tensor(p)) for p in prompts]
    got = llm.generate([{"prompt_embeds": e} for e in embeds[:2]] + [prompts[2]], sp)
    assert [o.outputs[0].token_ids for o in got] == want
    with pytest.raises(ValueError):
        llm.generate([{"prompt_embeds": torch.zeros(3, 7)}], sp)
    vecs = llm.embed(prompts)
    assert len(vecs) == 3 and all(abs(float(v.norm()) - 1.0) < 1e-5 for v in vecs)
    # oracle: full forward of one prompt, last row of the final hidden states
    from test_engine_cpu import _recompute_greedy  # noqa: F401
    again = llm.embed([prompts[1]], normalize=False)[0]
    assert torch.allclose(torch.nn.functional.normalize(again, dim=-1), vecs[1], atol=1e-5)
    assert not torch.allclose(vecs[0], vecs[1])


def test_sparse_mla_model_with_lightning_indexer():
    """DeepSeek-V3.2 style layers: with index_topk at least the context length the indexer keeps every
    key and the model equals dense MLA on the same weights; a small top-k changes the continuation,
    and decoding equals a cache-free recomputation that applies the same selection."""
    from vllm_ascend_b200.config import get_model_config
    rng = np.random.default_rng(6)
    prompts = [rng.integers(1, 500, size=n).tolist() for n in (40, 13, 57)]
    sp = SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True)
    kw = dict(device="cpu", max_model_len=128, max_num_seqs=4, max_num_batched_tokens=32, block_size=16)

    def run(topk):
        cfg = get_model_config("tiny-deepseek-sparse")
        cfg.index_topk = topk
        llm = LLM(cfg, **kw)
        return llm, [o.outputs[0].token_ids for o in llm.generate(prompts, sp)]
    dense_llm, dense = run(0)
    full_llm, full = run(128)
    # the dense model has no indexer parameters: copy the shared ones so both use the same weights
    shared = dict(dense_llm.engine.runner.model.named_parameters())
    src = dict(full_llm.engine.runner.model.named_parameters())
    assert any("indexer" in k for k in src) and not any("indexer" in k for k in shared)
    assert all(torch.equal(shared[k], src[k]) for k in shared)
    assert full == dense
    _, small = run(8)
    assert small != dense and all(len(t) == 6 for t in small)
    # chunked prefill + decode of the sparse model equals one-shot prefill of the same engine settings
    cfg = get_model_config("tiny-deepseek-sparse")
    cfg.index_topk = 8
    one = LLM(cfg, device="cpu", max_model_len=128, max_num_seqs=4, max_num_batched_tokens=128, block_size=16)
    assert [o.outputs[0].token_ids for o in one.generate(prompts, sp)] == small


def test_sparse_attention_with_host_resident_kv():
    """sparse_kv_offload: latent KV on the host, per-sequence device pools refilled from the indexer's
    selection; same tokens as the engine that keeps the KV in the paged device cache."""
    from vllm_ascend_b200.config import get_model_config
    rng = np.random.default_rng(6)
    prompts = [rng.integers(1, 500, size=n).tolist() for n in (40, 13, 57)]
    sp = SamplingParams(temperature=0.0, max_tokens=8, ignore_eos=True)
    kw = dict(device="cpu", max_model_len=128, max_num_seqs=4, max_num_batched_tokens=32, block_size=16)

    def cfg():
        c = get_model_config("tiny-deepseek-sparse")
        c.index_topk = 8
        return c
    want = [o.outputs[0].token_ids for o in LLM(cfg(), **kw).generate(prompts, sp)]
    llm = LLM(cfg(), additional_config={"sparse_kv_offload_config": {"enabled": True, "device_slots_per_seq": 12}}, **kw)
    runner = llm.engine.runner
    assert runner.sparse_offload is not None and runner.kv_caches[0][0].shape[0] == 1      # placeholders on the device
    got = [o.outputs[0].token_ids for o in llm.generate(prompts, sp)]
    assert got == want
    st = runner.sparse_offload[0].mgr.stats()
    assert st["hits"] > 0 and st["misses"] > 0 and st["evictions"] > 0
    # rows are reused by later requests: a second batch still matches
    assert [o.outputs[0].token_ids for o in llm.generate(prompts[::-1], sp)] == want[::-1]
    from vllm_ascend_b200.platform_config import clear_b200_config
    clear_b200_config()


def test_async_engine_steps_synchronously_for_token_dependent_sampling():
    """Penalties and multi-token bad words read the newest token: an asynchronous engine falls back
    to synchronous steps while such a request is alive and returns to lookahead afterwards."""
    kw = dict(device="cpu", max_model_len=128, max_num_seqs=8, max_num_batched_tokens=64, block_size=16)
    prompts = [[5, 6, 7, 8, 9], [20, 21, 22]]
    sps = [SamplingParams(temperature=0.0, max_tokens=8, ignore_eos=True, repetition_penalty=1.3, presence_penalty=0.5),
           SamplingParams(temperature=0.0, max_tokens=12, ignore_eos=True)]
    want = [o.outputs[0].token_ids for o in LLM("tiny-qwen", async_scheduling=False, **kw).generate(prompts, sps)]
    llm = LLM("tiny-qwen", async_scheduling=True, **kw)
    assert llm.engine.async_scheduling
    got = [o.outputs[0].token_ids for o in llm.generate(prompts, sps)]
    assert got == want
    assert not llm.engine._needs_sync()


def test_n_samples_per_prompt():
    llm = LLM("tiny-qwen", device="cpu", max_model_len=128, max_num_seqs=8, max_num_batched_tokens=64, block_size=16,
              enable_prefix_caching=True)
    prompt = list(range(5, 45))
    out = llm.generate([prompt, [7, 8, 9]], [SamplingParams(n=3, temperature=1.0, top_k=50, seed=11, max_tokens=8, ignore_eos=True),
                                             SamplingParams(temperature=0.0, max_tokens=4, ignore_eos=True)])
    assert [len(o.outputs) for o in out] == [3, 1]
    assert [c.index for c in out[0].outputs] == [0, 1, 2]
    toks = [tuple(c.token_ids) for c in out[0].outputs]
    assert len(set(toks)) > 1 and all(len(t) == 8 for t in toks)                # independent random streams
    again = llm.generate([prompt], SamplingParams(n=3, temperature=1.0, top_k=50, seed=11, max_tokens=8, ignore_eos=True))
    assert [tuple(c.token_ids) for c in again[0].outputs] == toks               # reproducible with the seed
    assert again[0].num_cached_tokens > 0 or llm.engine.scheduler.pool.hits > 0  # siblings share the cached prompt
    assert not llm.engine.scheduler.requests


def test_beam_search_keeps_best_cumulative_logprob():
    """Width 1 is greedy decoding; wider beams never score below it; the reported cumulative
    log-probability equals the teacher-forced sum of the chosen tokens' log-probabilities."""
    from vllm_ascend_b200 import LLM, SamplingParams
    llm = LLM("tiny-qwen", device="cpu", seed=0, block_size=16, max_model_len=128, max_num_seqs=16)
    rng = np.random.default_rng(3)
    prompts = [rng.integers(1, 500, size=n).tolist() for n in (11, 7)]
    greedy = llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=5, ignore_eos=True, logprobs=1))
    one = llm.beam_search(prompts, beam_width=1, max_tokens=5, ignore_eos=True)
    wide = llm.beam_search(prompts, beam_width=3, max_tokens=5, ignore_eos=True)
    for g, b1, b3, p in zip(greedy, one, wide, prompts):
        toks = g.outputs[0].token_ids
        g_cum = sum(lp[t] for lp, t in zip(g.outputs[0].logprobs, toks))
        assert b1[0]["tokens"] == toks and abs(b1[0]["cum_logprob"] - g_cum) < 1e-4
        assert len(b3) == 3 and b3[0]["cum_logprob"] >= g_cum - 1e-5
        assert [b["score"] for b in b3] == sorted((b["score"] for b in b3), reverse=True)
        assert len({tuple(b["tokens"]) for b in b3}) == 3
        # teacher-forced rescoring of the best beam
        best, cum = b3[0]["tokens"], 0.0
        for j, t in enumerate(best):
            o = llm.generate([p + best[:j]], SamplingParams(temperature=0.0, max_tokens=1, ignore_eos=True, logprobs=500))
            cum += o[0].outputs[0].logprobs[0][t]
        assert abs(cum - b3[0]["cum_logprob"]) < 1e-3


def test_prompt_logprobs_match_teacher_forcing_across_chunks():
    """Prompt log-probabilities computed chunk by chunk during prefill equal the generation
    log-probabilities of the same tokens given the same prefixes."""
    from vllm_ascend_b200 import LLM, SamplingParams
    llm = LLM("tiny-qwen", device="cpu", seed=0, block_size=16, max_model_len=128, max_num_seqs=8,
              max_num_batched_tokens=16)
    rng = np.random.default_rng(4)
    prompt = rng.integers(1, 500, size=37).tolist()
    # warm the prefix cache with the same prompt: the logprob request must not reuse it
    llm.generate([prompt], SamplingParams(temperature=0.0, max_tokens=1))
    out = llm.generate([prompt, prompt[:9]], SamplingParams(temperature=0.0, max_tokens=2, prompt_logprobs=2))
    plp = out[0].prompt_logprobs
    assert len(plp) == 37 and plp[0] is None and all(e is not None for e in plp[1:])
    assert out[0].num_cached_tokens == 0 and len(out[1].prompt_logprobs) == 9
    for pos in (1, 15, 16, 17, 31, 36):
        o = llm.generate([prompt[:pos]], SamplingParams(temperature=0.0, max_tokens=1, logprobs=llm.cfg.model.vocab_size))
        ref_lp = o[0].outputs[0].logprobs[0]
        assert abs(plp[pos][prompt[pos]] - ref_lp[prompt[pos]]) < 1e-4
        top = sorted(ref_lp.items(), key=lambda kv: -kv[1])[:2]
        for t, v in top:
            assert abs(plp[pos][t] - v) < 1e-4
    plain = llm.generate([prompt], SamplingParams(temperature=0.0, max_tokens=2))
    assert plain[0].prompt_logprobs is None and plain[0].outputs[0].token_ids == out[0].outputs[0].token_ids


def test_deferred_sampling_applies_an_allowed_token_mask():
    """The forward pass and the sampling of a step can be separated: a constraint on the logits that
    arrives after the forward was launched (a host engine's grammar bitmask) is applied before sampling."""
    import torch
    cfg = get_model_config("tiny-qwen")
    llm = LLM(cfg, device="cpu", max_model_len=128, max_num_seqs=4, max_num_batched_tokens=64, block_size=16)
    eng = llm.engine
    prompts = _prompts(2, 12, cfg.vocab_size, seed=5)
    sp = SamplingParams(temperature=0.0, max_tokens=4, ignore_eos=True)
    rids = [eng.add_request(p, sp) for p in prompts]
    so = eng.scheduler.schedule()
    h = eng.runner.execute_async(so, None, defer_sampling=True)
    assert h.tokens is None and h.h_sel is not None
    allowed = torch.zeros(cfg.vocab_size, dtype=torch.bool)
    allowed[[5, 7, 300]] = True
    logits = eng.runner.model.compute_logits(h.h_sel).float()
    eng.runner.finish_sampling(h, {rids[0]: allowed})
    assert h.h_sel is None and h.tokens is not None
    sampled = eng.runner.collect(h)
    i0 = h.index[rids[0]]
    want0 = max((5, 7, 300), key=lambda t: float(logits[i0, t]))
    assert sampled[rids[0]] == [want0]
    assert sampled[rids[1]] == [int(logits[h.index[rids[1]]].argmax())]           # unconstrained row untouched
    eng.scheduler.update_from_output(so, sampled)
    # the engine carries on normally from there
    while eng.has_unfinished():
        eng.step()
    assert all(len(eng.scheduler.requests[r].output_token_ids) == 4 for r in rids)


def test_grammar_bitmask_rows_unpack_to_token_masks():
    import numpy as np
    import torch
    from types import SimpleNamespace as NS
    from vllm_ascend_b200.worker.vllm_worker import B200VllmWorker
    w = B200VllmWorker.__new__(B200VllmWorker)
    w.runner = NS(mcfg=NS(vocab_size=70))
    w.device = torch.device("cpu")
    bm = np.zeros((2, 3), dtype=np.int32)
    bm[0, 0] = np.array([(1 << 3) | (1 << 31)], dtype=np.uint32).view(np.int32)[0]       # tokens 3 and 31
    bm[0, 2] = 1 << 5                          # token 69
    bm[1, 1] = -1                              # tokens 32..63
    out = w._unpack_bitmask(["a", "b"], bm)
    assert torch.nonzero(out["a"]).flatten().tolist() == [3, 31, 69]
    assert torch.nonzero(out["b"]).flatten().tolist() == list(range(32, 64))
    assert out["a"].shape == (70,)
