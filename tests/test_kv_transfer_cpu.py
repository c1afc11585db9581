"""Disaggregated prefill on CPU: a producer engine and a consumer engine in one process talk
over the ZMQ side channel (tcp transport, fp32 tiny model); failures are injected on the host."""
import time

import numpy as np
import pytest

from vllm_ascend_b200 import LLM, SamplingParams
from vllm_ascend_b200.distributed.kv_transfer import plan_head_slices
from vllm_ascend_b200.platform_config import clear_b200_config


def _mk(role, engine_id, extra=None, additional=None, **kw):
    ktc = {"kv_connector": "NVLinkConnector", "kv_role": role, "engine_id": engine_id,
           "kv_connector_extra_config": dict(extra or {})}
    return LLM("tiny-qwen", device="cpu", seed=0, block_size=16, max_model_len=256, max_num_seqs=8,
               kv_transfer_config=ktc, additional_config=additional, **kw)


def _prompts(n, lo=20, hi=70, seed=1):
    rng = np.random.default_rng(seed)
    return [rng.integers(1, 500, size=int(rng.integers(lo, hi))).tolist() for _ in range(n)]


def _drain(llm, steps=50):
    for _ in range(steps):
        llm.engine.kv_connector.reap(llm.engine.scheduler)
        if llm.engine.kv_connector.num_delayed == 0:
            return
        time.sleep(0.02)


@pytest.fixture(autouse=True)
def _clear():
    yield
    clear_b200_config()


def test_plan_head_slices():
    # equal TP: one-to-one
    assert plan_head_slices(4, 4, 8, 2) == [(2, 0, 0, 2)]
    # prefill TP4 -> decode TP2: each decode rank pulls from two prefill ranks
    assert plan_head_slices(4, 2, 8, 1) == [(2, 0, 0, 2), (3, 0, 2, 2)]
    # prefill TP2 -> decode TP4: half of a prefill rank's heads
    assert plan_head_slices(2, 4, 8, 3) == [(1, 2, 0, 2)]
    # replicated heads on the prefill side (TP8, 4 KV heads) -> decode TP2
    s = plan_head_slices(8, 2, 4, 1)
    assert [(x[1], x[2], x[3]) for x in s] == [(0, 0, 1), (0, 1, 1)]
    assert [x[0] for x in s] == [2 * 2 + 1, 3 * 2 + 1]
    # every head is covered exactly once for a range of shapes
    for tp_s, tp_d, h in [(1, 8, 8), (8, 1, 8), (2, 8, 4), (8, 4, 2), (4, 4, 1)]:
        for r in range(tp_d):
            sl = plan_head_slices(tp_s, tp_d, h, r)
            n_local = max(h // tp_d, 1)
            assert sorted(d0 + i for _, _, d0, n in sl for i in range(n)) == list(range(n_local))


def test_prefill_then_remote_decode_matches_monolithic():
    prompts = _prompts(5)
    sp = SamplingParams(max_tokens=8, temperature=0.0, ignore_eos=True)
    mono = LLM("tiny-qwen", device="cpu", seed=0, block_size=16, max_model_len=256, max_num_seqs=8)
    want = [o.outputs[0].token_ids for o in mono.generate(prompts, sp)]

    pre = _mk("kv_producer", "P0")
    dec = _mk("kv_consumer", "D0")
    try:
        sp1 = SamplingParams(max_tokens=1, temperature=0.0, ignore_eos=True)
        outs = pre.generate([{"prompt_token_ids": p, "kv_transfer_params": {"do_remote_decode": True}}
                             for p in prompts], sp1)
        assert all(o.kv_transfer_params and o.kv_transfer_params["do_remote_prefill"] for o in outs)
        assert [o.outputs[0].token_ids[0] for o in outs] == [w[0] for w in want]
        assert pre.engine.kv_connector.num_delayed == len(prompts)
        free_before = pre.engine.scheduler.pool.num_free_blocks

        got = dec.generate([{"prompt_token_ids": p, "kv_transfer_params": o.kv_transfer_params}
                            for p, o in zip(prompts, outs)], sp)
        assert [o.outputs[0].token_ids for o in got] == want
        c = dec.engine.kv_connector
        assert c.stats["pulled_requests"] == len(prompts) and c.stats["failed"] == 0
        # the decode engine computed one prompt token per request, not the whole prompt
        assert dec.engine.runner.stats["prefill_tokens"] <= len(prompts) \
            if "prefill_tokens" in dec.engine.runner.stats else True
        # the producer frees the blocks once the consumer said it is done
        _drain(pre)
        assert pre.engine.kv_connector.num_delayed == 0
        assert pre.engine.scheduler.pool.num_free_blocks > free_before
        assert pre.engine.kv_connector.stats["released"] == len(prompts)
    finally:
        pre.engine.kv_connector.close()
        dec.engine.kv_connector.close()


def test_unclaimed_blocks_expire():
    pre = _mk("kv_producer", "P1", extra={"abort_timeout_s": 0.05})
    try:
        sp1 = SamplingParams(max_tokens=1, temperature=0.0, ignore_eos=True)
        total = pre.engine.scheduler.pool.num_free_blocks
        pre.generate([{"prompt_token_ids": p, "kv_transfer_params": {"do_remote_decode": True}}
                      for p in _prompts(3)], sp1)
        assert pre.engine.kv_connector.num_delayed == 3
        assert pre.engine.scheduler.pool.num_free_blocks < total
        time.sleep(0.1)
        pre.engine.kv_connector.reap(pre.engine.scheduler)
        assert pre.engine.kv_connector.num_delayed == 0
        assert pre.engine.kv_connector.stats["expired"] == 3
        assert pre.engine.scheduler.pool.num_free_blocks == total
    finally:
        pre.engine.kv_connector.close()


def test_pull_failure_falls_back_to_local_prefill():
    """The producer stops answering (dropped messages): the decode engine's recompute
    scheduler prefills locally and the output is still the monolithic one."""
    prompts = _prompts(3, seed=3)
    sp = SamplingParams(max_tokens=6, temperature=0.0, ignore_eos=True)
    mono = LLM("tiny-qwen", device="cpu", seed=0, block_size=16, max_model_len=256, max_num_seqs=8)
    want = [o.outputs[0].token_ids for o in mono.generate(prompts, sp)]
    pre = _mk("kv_producer", "P2")
    dec = _mk("kv_consumer", "D2", extra={"side_channel_timeout_ms": 200},
              additional={"scheduler_config": {"recompute_scheduler_enable": True}})
    try:
        sp1 = SamplingParams(max_tokens=1, temperature=0.0, ignore_eos=True)
        outs = pre.generate([{"prompt_token_ids": p, "kv_transfer_params": {"do_remote_decode": True}}
                             for p in prompts], sp1)
        pre.engine.kv_connector.drop_all_messages = True
        got = dec.generate([{"prompt_token_ids": p, "kv_transfer_params": o.kv_transfer_params}
                            for p, o in zip(prompts, outs)], sp)
        assert [o.outputs[0].token_ids for o in got] == want
        assert dec.engine.kv_connector.stats["failed"] == len(prompts)
        assert dec.engine.scheduler.num_recomputes == len(prompts)
    finally:
        pre.engine.kv_connector.close()
        dec.engine.kv_connector.close()


def test_unknown_remote_request_is_a_failure_not_a_crash():
    dec = _mk("kv_consumer", "D3", extra={"side_channel_timeout_ms": 200},
              additional={"scheduler_config": {"recompute_scheduler_enable": True}})
    pre = _mk("kv_producer", "P3")
    try:
        p = _prompts(1, seed=5)[0]
        bogus = {"do_remote_prefill": True, "remote_block_ids": [0, 1, 2, 3, 4], "remote_engine_id": "P3",
                 "remote_host": "127.0.0.1", "remote_port": pre.engine.kv_connector.base_port,
                 "remote_tp_size": 1, "remote_block_size": 16, "remote_request_id": "nope"}
        out = dec.generate([{"prompt_token_ids": p, "kv_transfer_params": bogus}],
                           SamplingParams(max_tokens=4, temperature=0.0, ignore_eos=True))
        assert len(out[0].outputs[0].token_ids) == 4
        assert dec.engine.kv_connector.stats["failed"] == 1
    finally:
        pre.engine.kv_connector.close()
        dec.engine.kv_connector.close()


def test_cpu_offload_restores_prefix_after_gpu_cache_is_gone():
    from vllm_ascend_b200.platform_config import clear_b200_config
    ktc = {"kv_connector": "CPUOffloadingConnector", "kv_connector_extra_config": {"num_cpu_blocks": 64}}
    llm = LLM("tiny-qwen", device="cpu", seed=0, block_size=16, max_model_len=256, max_num_seqs=4,
              kv_transfer_config=ktc)
    c = llm.engine.kv_connector
    prompts = _prompts(3, lo=60, hi=90, seed=9)
    sp = SamplingParams(max_tokens=6, temperature=0.0, ignore_eos=True)
    first = [o.outputs[0].token_ids for o in llm.generate(prompts, sp)]
    assert c.stats["saved_blocks"] >= sum(len(p) // 16 for p in prompts)
    # overwrite the device cache: whatever the second pass reuses must come from the host
    for kc, vc in llm.engine.runner.kv_caches:
        kc.normal_()
        vc.normal_()
    before = llm.engine.runner.stats.get("steps", 0)
    second = [o.outputs[0].token_ids for o in llm.generate(prompts, sp)]
    assert second == first
    assert c.stats["hit_tokens"] == sum((len(p) - 1) // 16 * 16 for p in prompts)
    assert c.stats["loaded_blocks"] == c.stats["hit_tokens"] // 16
    mono = LLM("tiny-qwen", device="cpu", seed=0, block_size=16, max_model_len=256, max_num_seqs=4)
    assert [o.outputs[0].token_ids for o in mono.generate(prompts, sp)] == first


def test_cpu_offload_lru_eviction_and_multi_connector():
    ktc = {"kv_connector": "MultiConnector", "kv_connector_extra_config": {"connectors": [
        {"kv_connector": "CPUOffloadingConnector", "kv_connector_extra_config": {"num_cpu_blocks": 4}}]}}
    llm = LLM("tiny-qwen", device="cpu", seed=0, block_size=16, max_model_len=256, max_num_seqs=4,
              kv_transfer_config=ktc)
    c = llm.engine.kv_connector.connectors[0]
    sp = SamplingParams(max_tokens=2, temperature=0.0, ignore_eos=True)
    for seed in range(3):
        llm.generate(_prompts(1, lo=64, hi=65, seed=20 + seed), sp)
    assert len(c.lru) <= 4 and c.stats["evicted_blocks"] > 0
    assert not c.free or len(c.lru) + len(c.free) == 4


def test_sparse_kv_offload_resident_set():
    """Native LRU bookkeeping: hits keep their slot, misses evict the least recently used token,
    tokens needed by the current step are never evicted, copies bring the right rows."""
    import numpy as np
    import torch
    from vllm_ascend_b200.distributed.kv_transfer.sparse_kv_offload import SparseKVOffloadManager
    m = SparseKVOffloadManager(max_seqs=3, max_tokens_per_seq=64, slots_per_seq=4, width=8,
                               dtype=torch.float32, device="cpu", num_threads=2)
    try:
        for row in range(3):
            m.append(row, 0, torch.arange(64 * 8, dtype=torch.float32).view(64, 8) + 1000 * row)
        rows = np.array([0, 2])
        s1 = m.step(rows, np.array([[5, 9, 1, -1], [7, 7, 3, 2]]))
        assert (s1[0, 3] == -1) and len(set(s1[0, :3].tolist())) == 3
        assert s1[1, 0] == s1[1, 1]                                   # same token, same slot
        for b, row in enumerate(rows):
            for j, tok in enumerate([[5, 9, 1], [7, 7, 3, 2]][b]):
                assert torch.equal(m.pool[row, s1[b, j]], m.host[row, tok])
        st = m.stats()
        assert st["misses"] == 6 and st["hits"] == 0
        # second step: 9 and 1 hit, 20 and 21 miss; one free slot is left, then the LRU token 5 goes
        s2 = m.step(np.array([0]), np.array([[9, 1, 20, 21]]))
        assert s2[0, 0] == s1[0, 1] and s2[0, 1] == s1[0, 2]
        assert s2[0, 3] == s1[0, 0]                                   # token 21 took token 5's slot
        assert torch.equal(m.pool[0, s2[0, 2]], m.host[0, 20])
        st = m.stats()
        assert st["hits"] == 2 and st["evictions"] == 1
        # five distinct tokens cannot be resident in four slots
        import pytest
        m.step(np.array([1]), np.array([[1, 2, 3, 4]]))
        with pytest.raises(RuntimeError):
            m.step(np.array([1]), np.array([[5, 6, 7, 8, 9]]))
        m.release(0)
        s3 = m.step(np.array([0]), np.array([[9, -1, -1, -1]]))
        assert m.stats()["misses"] > st["misses"]                     # state of the row was dropped
    finally:
        m.close()


def test_kv_pool_shares_prefixes_between_engines():
    """Engine A publishes the blocks of its finished requests to the store; engine B, which has
    never seen the prompts, loads them instead of prefilling."""
    from vllm_ascend_b200.distributed.kv_transfer.kv_pool import KVStoreServer
    store = KVStoreServer(capacity_bytes=64 << 20)
    try:
        def mk():
            return LLM("tiny-qwen", device="cpu", seed=0, block_size=16, max_model_len=256, max_num_seqs=4,
                       kv_transfer_config={"kv_connector": "KVPoolConnector",
                                           "kv_connector_extra_config": {"store_port": store.port}})
        a, b = mk(), mk()
        prompts = _prompts(3, lo=50, hi=90, seed=31)
        sp = SamplingParams(max_tokens=5, temperature=0.0, ignore_eos=True)
        want = [o.outputs[0].token_ids for o in a.generate(prompts, sp)]
        a.engine.kv_connector.flush()
        assert a.engine.kv_connector.stats["published_blocks"] >= sum(len(p) // 16 for p in prompts)
        got = [o.outputs[0].token_ids for o in b.generate(prompts, sp)]
        assert got == want
        cb = b.engine.kv_connector
        assert cb.stats["hit_tokens"] == sum((len(p) - 1) // 16 * 16 for p in prompts)
        assert cb.stats["loaded_blocks"] == cb.stats["hit_tokens"] // 16
        st = store._handle({"op": "stats"})
        assert st["blocks"] > 0 and st["hits"] == cb.stats["loaded_blocks"]
        # a tiny store evicts, lookups then simply miss
        small = KVStoreServer(capacity_bytes=1)
        small._handle({"op": "put", "hashes": [b"x"], "payloads": [b"123"]})
        assert small._handle({"op": "exists", "hashes": [b"x"]})["mask"] == [False]
        small.close()
    finally:
        store.close()


@pytest.mark.parametrize("backend,layerwise", [("memory", False), ("file", False), ("file", True), ("memory", True)])
def test_kv_pool_backends_and_layerwise_keys(backend, layerwise, tmp_path):
    """The same sharing through the other built-in stores, block-wise and layer-wise."""
    extra = {"backend": backend, "layerwise": layerwise, "name": f"t-{backend}-{layerwise}", "path": str(tmp_path / "kv")}

    def mk():
        return LLM("tiny-qwen", device="cpu", seed=0, block_size=16, max_model_len=256, max_num_seqs=4,
                   kv_transfer_config={"kv_connector": "KVPoolConnector", "kv_connector_extra_config": extra})
    a, b = mk(), mk()
    prompts = _prompts(2, lo=50, hi=90, seed=33)
    sp = SamplingParams(max_tokens=5, temperature=0.0, ignore_eos=True)
    want = [o.outputs[0].token_ids for o in a.generate(prompts, sp)]
    a.engine.kv_connector.flush()
    got = [o.outputs[0].token_ids for o in b.generate(prompts, sp)]
    assert got == want
    cb = b.engine.kv_connector
    assert cb.stats["hit_tokens"] == sum((len(p) - 1) // 16 * 16 for p in prompts) > 0
    st = cb.backend.stats()
    layers = len(cb.layers)
    per_block = layers if layerwise else 1
    assert st["blocks"] >= a.engine.kv_connector.stats["published_blocks"] * per_block > 0
    assert st["hits"] == cb.stats["loaded_blocks"] * per_block
    a.engine.kv_connector.close()
    cb.close()


def test_kv_store_backend_registry_and_file_eviction(tmp_path):
    from vllm_ascend_b200.distributed.kv_transfer import kv_store_backends as kb
    with pytest.raises(ValueError, match="unknown KV store backend"):
        kb.create_kv_store_backend({"backend": "nope"})
    made = []
    kb.register_kv_store_backend("mine", lambda e: made.append(e) or kb.MemoryBackend("mine-store", 1 << 20))
    be = kb.create_kv_store_backend({"backend": "mine", "x": 1})
    assert made == [{"backend": "mine", "x": 1}] and be.put([b"k"], [b"v"]) and be.get([b"k"]) == [b"v"]
    assert be.get([b"k", b"missing"]) is None
    # file store: capacity of three payloads, the least recently used file goes first
    fb = kb.FileBackend(str(tmp_path / "s"), capacity_bytes=300)
    for i in range(3):
        fb.put([b"k%d" % i], [bytes([i]) * 100])
        time.sleep(0.02)
    assert fb.get([b"k0"]) == [b"\x00" * 100]            # touch k0: k1 is now the oldest
    time.sleep(0.02)
    fb.put([b"k3"], [b"\x03" * 100])
    assert fb.exists([b"k0", b"k1", b"k2", b"k3"]) == [True, False, True, True]
    assert fb.stats()["evictions"] == 1 and fb.stats()["used"] == 300
    # a second process-like client on the same directory sees the same blocks
    assert kb.FileBackend(str(tmp_path / "s")).get([b"k3"]) == [b"\x03" * 100]


def test_layerwise_push_connector():
    """The decode engine allocates first and waits; the prefill engine pushes every layer's KV
    into the decode cache while it prefills (chunked), then signals completion."""
    from vllm_ascend_b200.distributed.kv_transfer.nvlink_connector import _LOCAL_ENGINES
    prompts = _prompts(3, lo=40, hi=90, seed=13)
    sp = SamplingParams(max_tokens=6, temperature=0.0, ignore_eos=True)
    mono = LLM("tiny-qwen", device="cpu", seed=0, block_size=16, max_model_len=256, max_num_seqs=8)
    want = [o.outputs[0].token_ids for o in mono.generate(prompts, sp)]

    def mk(role, eid):
        return LLM("tiny-qwen", device="cpu", seed=0, block_size=16, max_model_len=256, max_num_seqs=8,
                   max_num_batched_tokens=32,        # several prefill chunks per prompt
                   kv_transfer_config={"kv_connector": "LayerwiseConnector", "kv_role": role, "engine_id": eid})
    pre, dec = mk("kv_producer", "PL"), mk("kv_consumer", "DL")
    try:
        dc, pc = dec.engine.kv_connector, pre.engine.kv_connector
        rids = []
        for i, p in enumerate(prompts):
            rids.append(dec.engine.add_request(p, sp, kv_transfer_params={
                "do_remote_prefill": True, "layerwise": True, "key": f"k{i}"}))
        dec.engine.step()                                   # allocates the blocks, then waits
        assert len(dc._targets) == 3 and not dec.engine.scheduler.running
        reqs = {r: dec.engine.scheduler.requests[r] for r in rids}
        sp1 = SamplingParams(max_tokens=1, temperature=0.0, ignore_eos=True)
        outs = pre.generate([{"prompt_token_ids": p, "kv_transfer_params": {
            "do_remote_decode": True, "layerwise": True,
            "push_to": {"engine_id": "DL", "host": "127.0.0.1", "port": dc.base_port, "key": f"k{i}"}}}
            for i, p in enumerate(prompts)], sp1)
        assert all(o.kv_transfer_params["pushed"] for o in outs)
        assert pc.stats["pushed_requests"] == 3 and pc.stats["pushed_layers"] >= 2 * 2
        assert pre.engine.scheduler.pool.num_free_blocks == pre.engine.scheduler.pool.num_blocks - 1
        while dec.engine.has_unfinished():
            dec.engine.step()
        assert [reqs[r].output_token_ids for r in rids] == want
        assert dc.stats["pulled_requests"] == 3 and not dc._targets
        # the decode engine computed one prompt token per request itself, the rest was pushed
    finally:
        pre.engine.kv_connector.close()
        dec.engine.kv_connector.close()


def test_hybrid_connector_moves_kv_and_recurrent_state():
    """Gated-DeltaNet hybrid: the decode engine gets the attention layers' KV blocks, the linear
    layers' conv / delta-rule state rows and the first sampled token, and continues exactly as a
    monolithic engine would; the prefill engine holds the batch row until the pull is acknowledged."""
    def mk(role, eid):
        ktc = None if role is None else {"kv_connector": "HybridConnector", "kv_role": role, "engine_id": eid}
        return LLM("tiny-gdn", device="cpu", seed=0, block_size=16, max_model_len=256, max_num_seqs=4,
                   max_num_batched_tokens=48, kv_transfer_config=ktc)
    prompts = _prompts(3, seed=5)
    sp = SamplingParams(max_tokens=6, temperature=0.0, ignore_eos=True)
    want = [o.outputs[0].token_ids for o in mk(None, "M").generate(prompts, sp)]
    pre, dec = mk("kv_producer", "HP"), mk("kv_consumer", "HD")
    try:
        sp1 = SamplingParams(max_tokens=1, temperature=0.0, ignore_eos=True)
        outs = pre.generate([{"prompt_token_ids": p, "kv_transfer_params": {"do_remote_decode": True}}
                             for p in prompts], sp1)
        rows = [o.kv_transfer_params["remote_state_row"] for o in outs]
        assert len(set(rows)) == 3
        free_rows = pre.engine.scheduler._free_rows
        assert not set(rows) & set(free_rows)                   # held back with the states in them
        got = dec.generate([{"prompt_token_ids": p, "kv_transfer_params": o.kv_transfer_params}
                            for p, o in zip(prompts, outs)], sp)
        assert [o.outputs[0].token_ids for o in got] == want
        c = dec.engine.kv_connector
        assert c.stats["pulled_requests"] == 3 and c.stats["pulled_states"] == 3 and c.stats["failed"] == 0
        pre.engine.kv_connector.reap(pre.engine.scheduler)
        assert pre.engine.kv_connector.num_delayed == 0
        assert set(rows) <= set(pre.engine.scheduler._free_rows)
    finally:
        pre.engine.kv_connector.close()
        dec.engine.kv_connector.close()


def test_sparse_attention_remote_d2h_connector():
    """Prefill engine with paged sparse-attention caches -> decode engine whose latent KV is
    host-resident: the prompt's rows land in the host store, index keys in the paged index cache, and
    decoding continues as on a monolithic engine."""
    from vllm_ascend_b200.config import get_model_config
    from vllm_ascend_b200.platform_config import clear_b200_config

    def cfg():
        c = get_model_config("tiny-deepseek-sparse")
        c.index_topk = 8
        return c

    def mk(role, eid, offload):
        ktc = None if role is None else {"kv_connector": "SfaRemoteD2HConnector", "kv_role": role, "engine_id": eid}
        add = {"sparse_kv_offload_config": {"enabled": True, "device_slots_per_seq": 16}} if offload else None
        return LLM(cfg(), device="cpu", seed=0, block_size=16, max_model_len=256, max_num_seqs=4,
                   max_num_batched_tokens=48, kv_transfer_config=ktc, additional_config=add)
    prompts = _prompts(3, seed=8)
    sp = SamplingParams(max_tokens=6, temperature=0.0, ignore_eos=True)
    want = [o.outputs[0].token_ids for o in mk(None, "M", False).generate(prompts, sp)]
    pre = mk("kv_producer", "SP", False)
    try:
        sp1 = SamplingParams(max_tokens=1, temperature=0.0, ignore_eos=True)
        outs = pre.generate([{"prompt_token_ids": p, "kv_transfer_params": {"do_remote_decode": True}}
                             for p in prompts], sp1)
        dec = mk("kv_consumer", "SD", True)          # built last: the offload setting is process-wide config
        try:
            got = dec.generate([{"prompt_token_ids": p, "kv_transfer_params": o.kv_transfer_params}
                                for p, o in zip(prompts, outs)], sp)
            assert [o.outputs[0].token_ids for o in got] == want
            c = dec.engine.kv_connector
            assert c.stats["pulled_requests"] == 3 and c.stats["failed"] == 0
            assert c.stats["host_rows"] == sum(len(p) - 1 for p in prompts) * dec.cfg.model.num_hidden_layers
            pre.engine.kv_connector.reap(pre.engine.scheduler)
            assert pre.engine.kv_connector.num_delayed == 0
        finally:
            dec.engine.kv_connector.close()
    finally:
        pre.engine.kv_connector.close()
        clear_b200_config()


def test_block_keys_separate_multimodal_content_adapters_and_engines():
    """Blocks are shared only between requests whose KV really is the same: equal placeholder ids with
    other pixels, another adapter, or another model / cache layout give other keys; prompt-embedding
    requests (ids are placeholders, no content hash) are never looked up nor published."""
    from types import SimpleNamespace as NS
    import numpy as np
    from vllm_ascend_b200.engine.block_pool import BlockPool
    ids = np.arange(64, dtype=np.int32)
    mm = lambda h, modality="image": NS(hash=h, modality=modality)
    req = lambda **kw: NS(prompt_token_ids=ids, output_token_ids=[], lora_request=None, mm_inputs=[], **kw)
    base = BlockPool.request_key_extra(req())
    a, b = req(), req()
    a.mm_inputs, b.mm_inputs = [mm("img-a")], [mm("img-b")]
    ka, kb = BlockPool.request_key_extra(a), BlockPool.request_key_extra(b)
    assert len({base, ka, kb}) == 3
    c = req()
    c.lora_request = NS(lora_int_id=3)
    assert BlockPool.request_key_extra(c) not in (base, ka, kb)
    e = req()
    e.mm_inputs = [mm("embeds-req-1", "embeds")]
    assert BlockPool.request_key_extra(e) is None
    # a store shared by engines: another model or cache dtype changes every key
    import torch
    cfg = lambda name, bs=16: NS(model=NS(architecture="Qwen3ForCausalLM", name=name, model_path=None,
                                         num_hidden_layers=2, hidden_size=64, num_attention_heads=4,
                                         num_key_value_heads=2, head_dim=16, vocab_size=100, seed=0,
                                         quantization=None), cache=NS(block_size=bs))
    t16 = [torch.zeros(4, 16, 2, 16, dtype=torch.bfloat16)]
    t8 = [torch.zeros(4, 16, 2, 16, dtype=torch.float8_e4m3fn)]
    f = BlockPool.store_fingerprint
    assert f(cfg("a"), t16) == f(cfg("a"), t16)
    assert len({f(cfg("a"), t16), f(cfg("b"), t16), f(cfg("a"), t8)}) == 3
    # the connectors route through the same helper
    from vllm_ascend_b200.distributed.kv_transfer.kv_pool import KVPoolConnector
    conn = KVPoolConnector.__new__(KVPoolConnector)
    conn.block_size, conn._fingerprint = 16, f(cfg("a"), t16)
    assert conn._hashes(e, 64) == []
    ha, hb = conn._hashes(a, 64), conn._hashes(b, 64)
    assert len(ha) == 4 and ha[0] != hb[0]
    conn2 = KVPoolConnector.__new__(KVPoolConnector)
    conn2.block_size, conn2._fingerprint = 16, f(cfg("b"), t16)
    assert conn2._hashes(a, 64)[0] != ha[0]


@pytest.mark.parametrize("keep", [False, True])
def test_recompute_cpu_offload_keeps_preempted_requests_kv_on_the_host(keep):
    """A pool too small for the batch forces recompute preemption; with the connector the preempted
    requests' blocks come back from the host instead of being prefilled again, and outputs do not
    change."""
    from vllm_ascend_b200.config import get_model_config
    cfg = get_model_config("tiny-qwen")
    rng = np.random.default_rng(3)
    prompts = [rng.integers(0, cfg.vocab_size, size=40).tolist() for _ in range(6)]
    sp = SamplingParams(temperature=0.0, max_tokens=12, ignore_eos=True)
    big = LLM(cfg, device="cpu", max_model_len=128, max_num_seqs=8, max_num_batched_tokens=512, block_size=16)
    ref = [o.outputs[0].token_ids for o in big.generate(prompts, sp)]

    def small(ktc):
        llm = LLM(cfg, device="cpu", max_model_len=128, max_num_seqs=8, max_num_batched_tokens=16, block_size=16,
                  num_gpu_blocks_override=14, kv_transfer_config=ktc, enable_prefix_caching=False)
        llm.engine.scheduler.reserve_full = False          # over-admit so decode must preempt
        return llm
    plain = small(None)
    assert [o.outputs[0].token_ids for o in plain.generate(prompts, sp)] == ref
    assert plain.engine.scheduler.num_preemptions > 0
    steps_plain = plain.engine.runner.stats.get("steps", 0)
    llm = small({"kv_connector": "RecomputeCPUOffloadConnector",
                 "kv_connector_extra_config": {"cpu_bytes_to_use": 8 << 20, "enable_offload_prefix_caching": keep}})
    got = [o.outputs[0].token_ids for o in llm.generate(prompts, sp)]
    assert got == ref
    c = llm.engine.kv_connector
    assert llm.engine.scheduler.num_preemptions > 0
    assert c.stats["preempted_saved"] > 0 and c.stats["resumed_hits"] > 0 and c.stats["loaded_blocks"] > 0
    if not keep:
        # host blocks of finished requests went back to the free list
        assert len(c.free) == c.num_cpu_blocks and not c.lru and not c._owned
    else:
        assert c.lru
    with pytest.raises(ValueError, match="boolean"):
        small({"kv_connector": "RecomputeCPUOffloadConnector",
               "kv_connector_extra_config": {"enable_offload_prefix_caching": "yes"}})


def test_ucm_connector_delegates_to_an_external_cache_manager(monkeypatch):
    """A stand-in for the external package: a dispatcher class that declares only ``stats`` itself and
    keeps the real connector (the pool over a process-local store) as ``.connector``.  Every hook of
    the contract must reach the inner connector: the second engine loads what the first published."""
    import sys
    import types

    from vllm_ascend_b200.distributed.kv_transfer.kv_pool import KVPoolConnector
    from vllm_ascend_b200.distributed.kv_transfer.ucm_connector import UCMConnector
    calls = []

    class Dispatcher:
        def __init__(self, engine_cfg, runner):
            import copy
            cfg = copy.copy(engine_cfg)
            cfg.kv_transfer_config = {"kv_connector": "KVPoolConnector",
                                      "kv_connector_extra_config": {"backend": "memory", "name": "ucm-fake"}}
            self.connector = KVPoolConnector(cfg, runner)

        def stats(self):
            calls.append("stats")
            return dict(self.connector.stats, manager="fake")

    mod = types.ModuleType("fake_ucm")
    mod.Manager = Dispatcher
    monkeypatch.setitem(sys.modules, "fake_ucm", mod)
    extra = {"ucm_connector_module": "fake_ucm", "ucm_connector_class": "Manager"}

    def mk():
        return LLM("tiny-qwen", device="cpu", seed=0, block_size=16, max_model_len=256, max_num_seqs=4,
                   kv_transfer_config={"kv_connector": "UCMConnectorV1", "kv_connector_extra_config": extra})
    a, b = mk(), mk()
    assert isinstance(b.engine.kv_connector, UCMConnector)
    prompts = _prompts(2, lo=50, hi=90, seed=41)
    sp = SamplingParams(max_tokens=4, temperature=0.0, ignore_eos=True)
    want = [o.outputs[0].token_ids for o in a.generate(prompts, sp)]
    a.engine.kv_connector._engine.connector.flush()
    got = [o.outputs[0].token_ids for o in b.generate(prompts, sp)]
    assert got == want
    st = b.engine.kv_connector.stats()
    assert calls == ["stats"] and st["manager"] == "fake"
    assert st["hit_tokens"] == sum((len(p) - 1) // 16 * 16 for p in prompts) > 0
    a.engine.kv_connector.close()
    b.engine.kv_connector.close()
    # a missing package is reported with the names that were tried
    with pytest.raises(ImportError, match="no_such_ucm.UCMConnector"):
        LLM("tiny-qwen", device="cpu", seed=0, block_size=16, max_model_len=64, max_num_seqs=2,
            kv_transfer_config={"kv_connector": "UCMConnector",
                                "kv_connector_extra_config": {"ucm_connector_module": "no_such_ucm"}})


def test_recompute_scheduler_hands_requests_back_under_kv_pressure():
    """Decode node, pool too small for the batch, no host copy to park the victim on: the victim finishes
    with stop reason "recomputed" and the tokens it produced (a prefix of the full answer), ahead of the
    regular outputs of its step; continuing from prompt + those tokens gives the full answer."""
    from vllm_ascend_b200.config import get_model_config
    from vllm_ascend_b200.core.recompute import RecomputeScheduler
    cfg = get_model_config("tiny-qwen")
    rng = np.random.default_rng(3)
    prompts = [rng.integers(0, cfg.vocab_size, size=40).tolist() for _ in range(6)]
    sp = SamplingParams(temperature=0.0, max_tokens=12, ignore_eos=True)
    big = LLM(cfg, device="cpu", max_model_len=128, max_num_seqs=8, max_num_batched_tokens=512, block_size=16)
    ref = [o.outputs[0].token_ids for o in big.generate(prompts, sp)]
    llm = LLM(cfg, device="cpu", max_model_len=128, max_num_seqs=8, max_num_batched_tokens=16, block_size=16,
              num_gpu_blocks_override=14, enable_prefix_caching=False,
              kv_transfer_config={"kv_connector": "NVLinkConnector", "kv_role": "kv_consumer", "engine_id": "dec-hb",
                                  "kv_connector_extra_config": {"recompute_hand_back": True}},
              additional_config={"scheduler_config": {"recompute_scheduler_enable": True}})
    s = llm.engine.scheduler
    assert isinstance(s, RecomputeScheduler) and s.hand_back
    s.reserve_full = False
    rids = [llm.engine.add_request(p, sp) for p in prompts]
    finished_order = []
    while llm.engine.has_unfinished():
        step_done = llm.engine.step()
        # hand-backs lead the step's list
        kinds = [r.stop_reason == "recomputed" for r in step_done]
        assert kinds == sorted(kinds, reverse=True)
        finished_order += step_done
    assert len(finished_order) == len(prompts) and s.pool.num_free_blocks == s.pool.num_blocks - 1
    handed = [r for r in finished_order if r.stop_reason == "recomputed"]
    assert handed and set(s.recomputed_requests) == {r.request_id for r in handed}
    for r in finished_order:
        want = ref[rids.index(r.request_id)]
        got = list(r.output_token_ids or [])
        if r.stop_reason == "recomputed":
            assert r.status.name == "FINISHED_STOPPED" and len(got) < len(want) and got == want[:len(got)]
            # what the proxy does next: the rest from prompt + produced tokens
            rest = big.generate([prompts[rids.index(r.request_id)] + got],
                                SamplingParams(temperature=0.0, max_tokens=12 - len(got), ignore_eos=True))
            assert got + rest[0].outputs[0].token_ids == want
        else:
            assert got == want
    llm.engine.kv_connector.close()
