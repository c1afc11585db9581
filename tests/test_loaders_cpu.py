"""Peer-to-peer weight loading (netloader, rfork) and RL weight transfer on CPU (gloo)."""
import threading

import numpy as np
import pytest
import torch

from vllm_ascend_b200 import LLM, SamplingParams
from vllm_ascend_b200.distributed.weight_transfer import NCCLWeightTransferEngine, packed
from vllm_ascend_b200.model_loader.rfork import RForkLoader, RForkPlanner

KW = dict(device="cpu", block_size=16, max_model_len=64, max_num_seqs=2)
PROMPT = [[5, 6, 7, 8, 9, 10, 11]]
SP = SamplingParams(max_tokens=5, temperature=0.0, ignore_eos=True)


def _tokens(llm):
    return llm.generate(PROMPT, SP)[0].outputs[0].token_ids


def test_packed_buckets_roundtrip():
    g = torch.Generator().manual_seed(0)
    tensors = {f"w{i}": torch.randn(*shape, generator=g).to(dt) for i, (shape, dt) in enumerate(
        [((3, 5), torch.float32), ((7,), torch.bfloat16), ((64, 33), torch.float32), ((2, 2, 2), torch.float16)])}
    meta = [(n, t.dtype, tuple(t.shape)) for n, t in tensors.items()]
    buckets = packed.plan_buckets(meta, 1024)
    assert len(buckets) >= 2 and sum(len(b) for b in buckets) == 4
    for entries in buckets:
        buf = packed.pack(entries, tensors, "cpu")
        assert buf.numel() % 256 == 0
        for name, t in packed.unpack(entries, buf):
            assert torch.equal(t, tensors[name])


def test_netloader_pulls_weights_from_a_running_instance():
    src = LLM("tiny-qwen", seed=123, **KW)
    want = _tokens(src)
    source = src.serve_weights()
    try:
        new = LLM("tiny-qwen", seed=7, load_format="netloader",
                  model_loader_extra_config={"source_port": source.port, "backend": "gloo"}, **KW)
        assert new.engine.runner.loaded_from_peer
        assert _tokens(new) == want
        assert source.served == 1
        # a dead source: fall back to the default (random-init) weights, do not fail
        fb = LLM("tiny-qwen", seed=7, load_format="netloader",
                 model_loader_extra_config={"source_port": 1, "backend": "gloo"}, **KW)
        assert not fb.engine.runner.loaded_from_peer
        assert _tokens(fb) == _tokens(LLM("tiny-qwen", seed=7, **KW))
    finally:
        source.close()


def test_rfork_planner_picks_least_busy_seed_and_loader_forks():
    planner = RForkPlanner()
    src = LLM("tiny-qwen", seed=5, **KW)
    source = src.serve_weights()
    try:
        ld = RForkLoader("127.0.0.1", planner.port, "tiny-qwen", backend="gloo")
        assert not ld.load(src.engine.runner.model)            # no seed yet -> fallback signal
        ld.register_as_seed("127.0.0.1", source.port)
        new = LLM("tiny-qwen", seed=99, load_format="rfork",
                  model_loader_extra_config={"planner_port": planner.port, "backend": "gloo"}, **KW)
        assert new.engine.runner.loaded_from_peer and _tokens(new) == _tokens(src)
        k = ("tiny-qwen", 1, "127.0.0.1", source.port)
        assert planner.seeds[k]["inflight"] == 0 and planner.seeds[k]["served"] == 1
        # least-busy selection
        planner._handle({"op": "register", "model_id": "tiny-qwen", "tp_size": 1, "host": "h2", "port": 2})
        planner.seeds[k]["inflight"] = 3
        assert planner._handle({"op": "acquire", "model_id": "tiny-qwen", "tp_size": 1})["host"] == "h2"
    finally:
        source.close()
        planner.close()


def test_rl_weight_transfer_updates_a_live_engine():
    from test_tp_cpu import _free_port
    trainer_model = LLM("tiny-qwen", seed=42, **KW)
    worker = LLM("tiny-qwen", seed=1, **KW)
    assert _tokens(worker) != _tokens(trainer_model)
    port = _free_port()
    res = {}

    def trainer():
        eng = NCCLWeightTransferEngine("127.0.0.1", port, 0, 2, backend="gloo", bucket_bytes=1 << 16)
        eng.send_weights(trainer_model.engine.runner.model.named_parameters())
        res["sent"] = eng.stats

    t = threading.Thread(target=trainer)
    t.start()
    eng = NCCLWeightTransferEngine("127.0.0.1", port, 1, 2, backend="gloo", bucket_bytes=1 << 16)
    w = worker.engine.worker
    w.start_weight_update()
    params = dict(w.runner.model.named_parameters())

    def apply(pairs):
        n = 0
        for name, tensor in pairs:
            params[name].copy_(tensor)
            n += 1
        return n
    n = eng.receive_weights(apply)
    w.finish_weight_update()
    t.join()
    assert n == len(params) and res["sent"]["buckets"] == eng.stats["buckets"] > 1
    worker.reset_prefix_cache()
    assert _tokens(worker) == _tokens(trainer_model)


def test_sharded_state_roundtrip_and_reload_weights(tmp_path):
    import torch
    from safetensors.torch import save_file
    from vllm_ascend_b200 import LLM, SamplingParams
    from vllm_ascend_b200.models.transformer import export_hf_state_dict
    kw = dict(device="cpu", block_size=16, max_model_len=128, max_num_seqs=4)
    sp = SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True)
    prompt = [[5, 6, 7, 8, 9, 10]]
    a = LLM("tiny-moe", seed=0, **kw)
    want = a.generate(prompt, sp)[0].outputs[0].token_ids
    files = a.save_sharded_state(str(tmp_path / "sharded"), max_bytes=1 << 18)
    assert len(files) > 1                                         # split into parts
    from vllm_ascend_b200.config import get_model_config
    cfg = get_model_config("tiny-moe")
    cfg.seed = 123                                                # other random weights, then overwritten
    b = LLM(cfg, load_format="sharded_state", model_loader_extra_config={"path": str(tmp_path / "sharded")}, **kw)
    assert b.engine.runner.loaded_from_peer
    assert b.generate(prompt, sp)[0].outputs[0].token_ids == want
    # in-place reload from an HF-layout checkpoint directory
    c = LLM(get_model_config("tiny-moe"), **kw)
    ck = tmp_path / "hf"
    ck.mkdir()
    sd = {k: v.contiguous() for k, v in export_hf_state_dict(a.engine.runner.model).items()}
    save_file(sd, str(ck / "model.safetensors"))
    for _, t in c.engine.runner.model.named_parameters():
        t.zero_()
    ptrs = [t.data_ptr() for _, t in c.engine.runner.model.named_parameters()]
    assert c.reload_weights(str(ck)) == len(sd)
    assert ptrs == [t.data_ptr() for _, t in c.engine.runner.model.named_parameters()]
    assert c.generate(prompt, sp)[0].outputs[0].token_ids == want
    with pytest.raises(FileNotFoundError):
        LLM("tiny-moe", load_format="sharded_state", model_loader_extra_config={"path": str(tmp_path / "none")}, **kw)
