"""Engine on a GPU (bf16, native kernels, CUDA graphs) checked against the CPU fp32
path running the same weights."""
import numpy as np
import pytest
import torch

from vllm_ascend_b200 import envs
from vllm_ascend_b200.config import ModelConfig
from vllm_ascend_b200.engine.llm import LLM
from vllm_ascend_b200.engine.request import SamplingParams

pytestmark = pytest.mark.gpu


def _cfg(dtype):
    return ModelConfig(name="t", architecture="Qwen3ForCausalLM", vocab_size=2048, hidden_size=512,
                       intermediate_size=1024, num_hidden_layers=3, num_attention_heads=8,
                       num_key_value_heads=2, head_dim=128, qk_norm=True, rope_theta=1e6,
                       dtype=dtype, init_std=0.05)


def _teacher_forced_gap(cpu_llm, prompt, gpu_tokens):
    """For every generated position: logit gap (CPU fp32) between the CPU argmax and
    the token the GPU chose.  Zero when they agree."""
    from test_engine_cpu import _recompute_greedy  # noqa: F401  (oracle lives there)
    from vllm_ascend_b200.attention.metadata import AttentionMetadata
    model = cpu_llm.engine.runner.model
    ids = list(prompt) + list(gpu_tokens)
    T = len(ids)
    bs = 16
    nblk = (T + bs - 1) // bs + 1
    caches = [tuple(torch.zeros(nblk, bs, L.self_attn.Hkv, L.self_attn.D) for _ in range(2))
              for L in model.layers]
    pos = torch.arange(T)
    meta = AttentionMetadata(
        num_reqs=1, num_actual_tokens=T, max_query_len=T, max_seq_len=T,
        query_start_loc=torch.tensor([0, T], dtype=torch.int32), seq_lens=torch.tensor([T], dtype=torch.int32),
        block_table=torch.arange(1, nblk, dtype=torch.int32).unsqueeze(0), slot_mapping=pos + bs,
        positions=pos, query_start_loc_cpu=np.array([0, T]), seq_lens_cpu=np.array([T]))
    with torch.no_grad():
        h = model.forward(torch.tensor(ids), meta, caches)
        logits = model.compute_logits(h[len(prompt) - 1:T - 1]).float()
    chosen = logits.gather(1, torch.tensor(gpu_tokens).unsqueeze(1)).squeeze(1)
    return (logits.max(-1).values - chosen)


@pytest.mark.parametrize("eager", [True, False])
def test_gpu_generation_follows_cpu_fp32(eager):
    rng = np.random.default_rng(0)
    prompts = [rng.integers(0, 2048, size=n).tolist() for n in (150, 40, 333, 129)]
    sp = SamplingParams(temperature=0.0, max_tokens=12, ignore_eos=True)
    gpu = LLM(_cfg("bfloat16"), device="cuda", max_model_len=512, max_num_seqs=8,
              max_num_batched_tokens=256, num_gpu_blocks_override=40, enforce_eager=eager,
              cudagraph_capture_sizes=[2, 4, 8])
    outs = gpu.generate(prompts, sp)
    if not eager:
        assert gpu.engine.runner.stats["graph_replays"] > 0
    assert gpu.engine.runner.total_launches() > 0
    cpu = LLM(_cfg("float32"), device="cpu", max_model_len=512, max_num_seqs=8, block_size=16)
    for p, o in zip(prompts, outs):
        toks = o.outputs[0].token_ids
        assert len(toks) == 12
        gap = _teacher_forced_gap(cpu, p, toks)
        # bf16 rounding may flip near-ties only
        assert float(gap.max()) < 0.35, gap


def test_gpu_random_sampling_runs_and_is_seeded():
    rng = np.random.default_rng(1)
    prompts = [rng.integers(0, 2048, size=64).tolist() for _ in range(4)]
    sp = SamplingParams(temperature=0.9, top_k=40, top_p=0.9, max_tokens=8, ignore_eos=True, seed=5,
                        repetition_penalty=1.1)
    gpu = LLM(_cfg("bfloat16"), device="cuda", max_model_len=256, max_num_seqs=8,
              max_num_batched_tokens=256, num_gpu_blocks_override=24, enforce_eager=True)
    a = [o.outputs[0].token_ids for o in gpu.generate(prompts, sp)]
    b = [o.outputs[0].token_ids for o in gpu.generate(prompts, sp)]
    assert a == b


def test_sleep_mode_frees_memory_and_restores_weights():
    """Level-1 sleep offloads weights to the host and drops the KV cache: device memory is
    returned to the driver while asleep, and after wake-up the engine generates the same tokens."""
    rng = np.random.default_rng(5)
    prompts = [rng.integers(0, 2048, size=n).tolist() for n in (100, 37)]
    sp = SamplingParams(temperature=0.0, max_tokens=8, ignore_eos=True)
    llm = LLM(_cfg("bfloat16"), device="cuda", max_model_len=512, max_num_seqs=8, max_num_batched_tokens=256,
              num_gpu_blocks_override=40, enforce_eager=True, enable_sleep_mode=True)
    first = [o.outputs[0].token_ids for o in llm.generate(prompts, sp)]
    torch.cuda.synchronize()
    free_awake, _ = torch.cuda.mem_get_info()
    llm.sleep(level=1)
    free_asleep, _ = torch.cuda.mem_get_info()
    assert llm.engine.sleep_level == 1
    assert free_asleep - free_awake > 20 << 20, (free_awake, free_asleep)      # weights + KV left the device
    llm.wake_up()
    assert llm.engine.sleep_level == 0
    second = [o.outputs[0].token_ids for o in llm.generate(prompts, sp)]
    assert second == first
    # waking up in two stages: weights first (e.g. to receive an update), KV cache later
    llm.sleep(level=1)
    llm.wake_up(tags=["weights"])
    assert llm.engine.sleep_level == 1
    llm.wake_up(tags=["kv_cache"])
    assert llm.engine.sleep_level == 0
    assert [o.outputs[0].token_ids for o in llm.generate(prompts, sp)] == first


def test_weight_offload_prefetch_on_gpu():
    from vllm_ascend_b200.platform_config import clear_b200_config
    rng = np.random.default_rng(6)
    prompts = [rng.integers(0, 2048, size=n).tolist() for n in (120, 45)]
    sp = SamplingParams(temperature=0.0, max_tokens=8, ignore_eos=True)
    kw = dict(device="cuda", max_model_len=512, max_num_seqs=8, max_num_batched_tokens=256,
              num_gpu_blocks_override=40)
    want = [o.outputs[0].token_ids for o in LLM(_cfg("bfloat16"), enforce_eager=True, **kw).generate(prompts, sp)]
    llm = LLM(_cfg("bfloat16"), additional_config={"weight_offload_config": {
        "enabled": True, "group_size": 1, "num_in_group": 1, "prefetch_step": 2}}, **kw)
    try:
        off = llm.engine.worker.offloader
        assert off is not None and len(off.layers) == 3 and off.num_slots == 3
        got = [o.outputs[0].token_ids for o in llm.generate(prompts, sp)]
        assert got == want
        assert llm.engine.runner.stats["graph_replays"] == 0
        assert off.stats["bytes"] > 0
    finally:
        clear_b200_config()


def test_training_consistent_attention_is_independent_of_batching():
    """With the single-kernel attention backend and split-free decode, a request's tokens do not
    depend on what else is in the batch or on how its prompt was chunked (GEMM kernels accumulate
    every output in one fixed order), which plain mode does not promise."""
    import os
    saved_env = dict(os.environ)
    rng = np.random.default_rng(11)
    prompts = [rng.integers(0, 2048, size=n).tolist() for n in (200, 37, 150, 90)]
    sp = SamplingParams(temperature=0.0, max_tokens=12, ignore_eos=True)
    add = {"rl_config": {"enabled": True, "enable_training_consistency": True, "enable_batch_invariant": True}}

    def run(batch_tokens, which):
        llm = LLM(_cfg("bfloat16"), device="cuda", max_model_len=512, max_num_seqs=8,
                  max_num_batched_tokens=batch_tokens, num_gpu_blocks_override=40, additional_config=add)
        return [o.outputs[0].token_ids for o in llm.generate([prompts[i] for i in which], sp)]
    try:
        together = run(512, [0, 1, 2, 3])
        chunked = run(64, [0, 1, 2, 3])
        alone = [run(512, [i])[0] for i in range(4)]
    finally:
        from vllm_ascend_b200.platform_config import clear_b200_config
        from vllm_ascend_b200.attention.backend import set_training_consistent_attention
        from vllm_ascend_b200.batch_invariant import disable_batch_invariant_mode
        set_training_consistent_attention(False)
        disable_batch_invariant_mode()
        clear_b200_config()
        os.environ.clear()
        os.environ.update(saved_env)
    assert together == chunked == alone
