"""Platform plugin surface, forward context, CPU binding, health probe, logger, profiling spans."""
import logging
import os

import pytest
import torch

import vllm_ascend_b200 as pkg
from vllm_ascend_b200 import cpu_binding
from vllm_ascend_b200.platform_config import clear_b200_config, get_b200_config


@pytest.fixture(autouse=True)
def _clear():
    yield
    clear_b200_config()


def test_entry_points_and_platform_class_paths():
    import importlib
    path = pkg.register()
    mod, cls = path.rsplit(".", 1)
    P = getattr(importlib.import_module(mod), cls)
    import torch
    if torch.cuda.is_available():
        assert P.device_type == "cuda" and P.dispatch_key == "CUDA" and P.dist_backend == "nccl"
    else:       # the platform also loads without a GPU: the whole stack then runs on the host
        assert P.device_type == "cpu" and P.dispatch_key == "CPU" and P.dist_backend == "gloo"
    assert "fp8" in P.supported_quantization
    assert P.is_sleep_mode_available() and P.support_static_graph_mode() and P.opaque_attention_op()
    # every class path the platform hands out resolves to a real class
    for getter in (P.get_punica_wrapper, P.get_device_communicator_cls, P.get_static_graph_wrapper_cls,
                   P.get_pass_manager_cls, P.get_compile_backend):
        m, c = getter().rsplit(".", 1)
        assert hasattr(importlib.import_module(m), c), getter
    for key in [dict(use_mla=False), dict(use_mla=True), dict(use_mla=True, use_sparse=True)]:
        m, c = P.get_attn_backend_cls(None, **key).rsplit(".", 1)
        assert hasattr(importlib.import_module(m), c)
    with pytest.raises(ValueError):
        P.get_attn_backend_cls(None, use_mla=False, use_sparse=True)


def test_platform_check_and_update_config_on_a_host_config():
    from types import SimpleNamespace as NS
    from vllm_ascend_b200.platform import B200Platform
    vc = NS(additional_config={"scheduler_config": {"short_request_first_config": {"enabled": True}}},
            parallel_config=NS(tensor_parallel_size=2, data_parallel_size=1, enable_expert_parallel=False,
                               worker_cls="auto", enable_dbo=True, use_sequence_parallel_moe=True,
                               data_parallel_rank=0),
            scheduler_config=NS(max_num_seqs=64, scheduler_cls=None),
            compilation_config=NS(cudagraph_mode="FULL", cudagraph_capture_sizes=[1, 3, 8],
                                  max_cudagraph_capture_size=None, use_inductor=True),
            model_config=NS(enforce_eager=False, hf_config=NS(num_experts=0), disable_cascade_attn=False),
            cache_config=NS(block_size=None), kv_transfer_config=None, speculative_config=None)
    B200Platform.check_and_update_config(vc)
    assert vc.parallel_config.worker_cls.endswith("B200VllmWorker")
    assert vc.parallel_config.enable_dbo is False and vc.compilation_config.use_inductor is False
    assert vc.compilation_config.cudagraph_capture_sizes == [2, 4, 8]      # TP multiples for SP
    import torch
    assert vc.cache_config.block_size == (128 if torch.cuda.is_available() else 16)
    assert vc.scheduler_config.scheduler_cls.endswith("ShortRequestFirstScheduler")
    assert get_b200_config().scheduler_config.short_request_first_config.enabled
    vc.compilation_config = NS(cudagraph_capture_sizes=None, max_cudagraph_capture_size=None)
    B200Platform.apply_config_platform_defaults(vc)
    assert vc.compilation_config.max_cudagraph_capture_size == 64


def test_forward_context_extras_and_moe_selection():
    from vllm_ascend_b200.forward_context import (get_forward_context, has_forward_context,
                                                  set_forward_context)
    from vllm_ascend_b200.ops.moe_comm import MoECommType
    assert not has_forward_context()
    with set_forward_context(None, num_tokens=5, tp_size=4, sp_enabled=True, is_moe=True, ep_size=8,
                             num_tokens_across_dp=[5, 300], fused_moe_available=True,
                             fused_moe_capacity=512) as ctx:
        assert get_forward_context() is ctx
        assert ctx.padded_length == 8 and ctx.max_tokens_across_dp == 300
        assert ctx.moe_comm_type is MoECommType.FUSED
        assert ctx.fused_moe_mask.sum() == 5 and ctx.fused_moe_mask.numel() == 512
        with set_forward_context(None, num_tokens=4096, is_moe=True, ep_size=8, fused_moe_available=True) as inner:
            assert inner.moe_comm_type is MoECommType.ALLTOALL
        assert get_forward_context() is ctx
    assert not has_forward_context()
    with pytest.raises(RuntimeError):
        get_forward_context()


def test_cpu_binding_plan_with_fake_topology():
    files = {
        "/sys/devices/system/node/online": "0-1\n",
        "/sys/devices/system/node/node0/cpulist": "0-15\n",
        "/sys/devices/system/node/node1/cpulist": "16-31\n",
        "/sys/bus/pci/devices/0000:1b:00.0/numa_node": "0\n",
        "/sys/bus/pci/devices/0000:43:00.0/numa_node": "0\n",
        "/sys/bus/pci/devices/0000:9b:00.0/numa_node": "1\n",
    }
    topo = cpu_binding.discover(4, read=files.get, pci_bus_ids=["00000000:1B:00.0", "00000000:43:00.0",
                                                                 "00000000:9B:00.0", ""])
    topo.allowed = list(range(32))
    assert topo.gpu_node == {0: 0, 1: 0, 2: 1, 3: -1}
    p = cpu_binding.plan(topo, 4)
    assert p[0] == list(range(2, 9)) and p[1] == list(range(9, 16))      # node 0 minus 2 reserved, halved
    assert p[2] == list(range(18, 32))
    assert p[3] == list(range(24, 32))                                   # unknown node: even slice of all
    got = {}
    cpus = cpu_binding.bind_cpus(1, 4, topo=topo, setaffinity=lambda pid, s: got.update(pid=pid, cpus=s))
    assert got["cpus"] == set(range(9, 16)) and cpus == list(range(9, 16))
    assert cpu_binding.format_cpu_list([0, 1, 2, 5, 7, 8]) == "0-2,5,7-8"
    assert cpu_binding.parse_cpu_list("0-2,5,7-8") == [0, 1, 2, 5, 7, 8]


def test_gpu_health_against_fake_nvml():
    from vllm_ascend_b200.observability import health

    class Fake:
        NVML_TEMPERATURE_GPU, NVML_CLOCK_SM = 0, 1
        NVML_MEMORY_ERROR_TYPE_UNCORRECTED, NVML_VOLATILE_ECC = 1, 0
        ecc = 0
        calls = []

        def nvmlInit(self): self.calls.append("init")
        def nvmlShutdown(self): self.calls.append("shutdown")
        def nvmlDeviceGetHandleByIndex(self, i): return i
        def nvmlDeviceGetTemperature(self, h, k): return 55
        def nvmlDeviceGetPowerUsage(self, h): return 700000
        def nvmlDeviceGetClockInfo(self, h, k): return 1700
        def nvmlDeviceGetCurrentClocksEventReasons(self, h): return 0x4 | 0x40
        def nvmlDeviceGetTotalEccErrors(self, h, a, b): return self.ecc

    fake = Fake()
    health.set_nvml_for_testing(lambda: fake)
    try:
        h = health.gpu_health(0)
        assert h["ok"] and h["temperature_c"] == 55 and h["power_w"] == 700.0
        assert sorted(h["throttle"]) == ["hw_thermal_slowdown", "sw_power_cap"]
        fake.ecc = 3
        h = health.gpu_health(0)
        assert not h["ok"] and "ECC" in h["reason"]
        # only read-only calls were made
        assert set(fake.calls) == {"init", "shutdown"}
    finally:
        health.set_nvml_for_testing(None)


def test_file_logging(tmp_path, monkeypatch):
    from vllm_ascend_b200 import logger as lg
    monkeypatch.setenv("VLLM_B200_LOG_PATH", str(tmp_path))
    lg.configure_logging(force=True)
    lg.logger.warning("hello from the test")
    for h in lg.logger.handlers:
        h.flush()
    files = list(tmp_path.glob("vllm_b200_*.log"))
    assert files and "hello from the test" in files[0].read_text()
    monkeypatch.delenv("VLLM_B200_LOG_PATH")
    for h in list(lg.logger.handlers):
        if isinstance(h, logging.handlers.RotatingFileHandler):
            lg.logger.removeHandler(h)
            h.close()


def test_service_profiling_config_and_spans(tmp_path, monkeypatch):
    from vllm_ascend_b200.profiler import service_profiling as sp
    monkeypatch.setenv("VLLM_B200_SERVICE_PROFILING_DIR", str(tmp_path))
    path = sp.generate_service_profiling_config()
    assert os.path.exists(path) and "engine.step" in open(path).read()
    names = sp.install_spans(path, nvtx=False)
    try:
        assert "scheduler.schedule" in names
        from vllm_ascend_b200 import LLM, SamplingParams
        llm = LLM("tiny-qwen", device="cpu", seed=0, block_size=16, max_model_len=64, max_num_seqs=2)
        llm.generate([[1, 2, 3, 4]], SamplingParams(max_tokens=3, temperature=0.0, ignore_eos=True))
        assert sp.totals["engine.step"][0] >= 3 and sp.totals["runner.execute"][1] > 0
        m = llm.get_metrics()
        assert m["steps"] >= 3 and m["kv_blocks_free"] == m["kv_blocks_total"] or m["kv_usage"] >= 0
    finally:
        sp.uninstall_spans()


def test_batch_invariant_mode_pins_split_factor(monkeypatch):
    from vllm_ascend_b200 import batch_invariant as bi, ops
    monkeypatch.delenv("VLLM_B200_BATCH_INVARIANT", raising=False)
    bi.disable_batch_invariant_mode()
    assert ops.choose_num_splits(4, 8, 8192) > 1
    bi.enable_batch_invariant_mode()
    try:
        assert ops.choose_num_splits(4, 8, 8192) == 1 and bi.is_batch_invariant()
        assert os.environ["NCCL_ALGO"] == "Ring"
    finally:
        bi.disable_batch_invariant_mode()
    assert ops.choose_num_splits(4, 8, 8192) > 1


def test_utils_predicates_and_op_table():
    import importlib
    from types import SimpleNamespace as NS
    from vllm_ascend_b200 import utils
    cfg = NS(parallel=NS(enable_sequence_parallel=True, tensor_parallel_size=2, data_parallel_size=2,
                         enable_expert_parallel=True),
             model=NS(is_moe=True), additional_config={"finegrained_tp_config": {"lmhead_tensor_parallel_size": 2}})
    assert utils.enable_sp(cfg) and utils.is_moe_model(cfg) and utils.lmhead_tp_enable(cfg)
    assert not utils.oproj_tp_enable(cfg)
    assert not utils.should_skip_allreduce_across_dp_group(cfg, True)
    cfg.model.is_moe = False
    assert utils.should_skip_allreduce_across_dp_group(cfg, True)


def _dyntra_pair(threshold=0.1, **cfg):
    import numpy as np  # noqa: F401
    from vllm_ascend_b200.config import CacheConfig, SchedulerConfig
    from vllm_ascend_b200.core.dyntra_lb import DyntraLBScheduler
    from vllm_ascend_b200.platform_config import init_b200_config
    init_b200_config({"scheduler_config": {"dyntra_lb_config": dict({"enabled": True, "imbalance_threshold": threshold},
                                                                      **cfg)}}, refresh=True)
    sc = SchedulerConfig(max_num_seqs=8, max_num_batched_tokens=64, max_model_len=256)
    cc = CacheConfig(block_size=16)
    return [DyntraLBScheduler(sc, cc, 64, rank=r, world=2, gather_fn=lambda v: [v]) for r in range(2)]


def _dyntra_lockstep(s):
    """Emulates the two all-gathers of a balancing step for schedulers living in one process: the ranks
    are run one after the other against a bus that returns all contributions of the phase."""
    reports = [x.report() for x in s]
    boxes = []
    for r, x in enumerate(s):
        phase = {"n": 0}

        def g(v, phase=phase):
            phase["n"] += 1
            if phase["n"] == 1:
                return reports
            boxes.append(v)
            return []                       # deliveries happen below, once every rank has posted
        x._gather = g
        x.balance()
    from vllm_ascend_b200.core.dyntra_lb import _unpack
    for box in boxes:
        for dst, payload in box:
            s[dst]._adopt(_unpack(payload))


def test_dyntra_lb_plan_is_deterministic_and_narrows_the_gap():
    from vllm_ascend_b200.core.dyntra_lb import RankReport, plan_balance
    reps = [RankReport(running=[10, 10, 10], movable_running=[10, 10], waiting=[4, 6, 8], pool_blocks=100),
            RankReport(running=[5], movable_running=[5], waiting=[], pool_blocks=100),
            RankReport(running=[20, 4], movable_running=[4], waiting=[2], pool_blocks=100)]
    a = plan_balance(reps, 0.05, 4)
    b = plan_balance(reps, 0.05, 4)
    assert [(m.out_blk, m.out_to, m.in_blk, m.freeze) for m in a] == [(m.out_blk, m.out_to, m.in_blk, m.freeze) for m in b]
    loads = [r.load for r in reps]
    after = list(loads)
    for i, m in enumerate(a):
        after[i] += sum(m.in_blk) - sum(m.out_blk)
    assert sum(after) == sum(loads) and max(after) - min(after) < max(loads) - min(loads)
    assert sum(len(m.out_blk) for m in a) == sum(len(m.in_blk) for m in a) > 0
    assert a[0].out_blk and all(d != 0 for d in a[0].out_to)
    assert len(a[0].out_blk) <= 4
    # waiting requests go before running ones
    assert set(a[0].out_blk) <= {4, 6, 8} or set([4, 6, 8]) <= set(a[0].out_blk)
    # inside the threshold nothing moves
    calm = plan_balance([RankReport(running=[10], waiting=[], pool_blocks=100),
                         RankReport(running=[8], waiting=[], pool_blocks=100)], 0.05, 4)
    assert not any(m.out_blk or m.freeze for m in calm)


def test_dyntra_lb_moves_waiting_requests_to_the_idle_rank():
    """Two schedulers stand for two DP ranks."""
    import numpy as np
    from vllm_ascend_b200.engine.request import Request, SamplingParams
    s = _dyntra_pair()
    for i in range(10):                 # everything arrives at rank 0
        req = Request(f"r{i}", np.arange(100, dtype=np.int32), SamplingParams(max_tokens=4))
        req.client_index, req.origin_rank = i, 0
        s[0].add_request(req)
    before = len(s[0].waiting)
    for _ in range(4):
        _dyntra_lockstep(s)
    assert s[0].migrated_out > 0 and s[1].migrated_in == s[0].migrated_out
    assert len(s[0].waiting) + len(s[1].waiting) == before
    assert abs(s[0].pressure() - s[1].pressure()) < before * 7 / 64
    moved = list(s[1].waiting)
    assert all(r.origin_rank == 0 and r.client_index is not None for r in moved)
    # the oldest requests stay where they arrived
    assert s[0].waiting[0].request_id == "r0"


def test_dyntra_lb_pauses_running_requests_and_the_receiver_resumes_them():
    import numpy as np
    from vllm_ascend_b200.engine.request import Request, RequestStatus, SamplingParams
    s = _dyntra_pair(threshold=0.05, long_req_block_threshold=5)
    lens = [40, 40, 40, 40, 120]                      # the last one is long (8 blocks > 5): it stays
    for i, n in enumerate(lens):
        req = Request(f"r{i}", np.arange(n, dtype=np.int32), SamplingParams(max_tokens=16))
        req.client_index, req.origin_rank = i, 0
        s[0].add_request(req)
    s[0].world = 1                                     # admit everything without balancing first
    for _ in range(8):
        out = s[0].schedule()
        for req, n in out.scheduled:
            req.num_computed_tokens += n
            if req.num_computed_tokens >= req.num_tokens:
                req.output_token_ids = (req.output_token_ids or []) + [7]
                req.num_output_tokens += 1
    s[0].world = 2
    assert len(s[0].running) == 5 and not s[0].waiting
    assert all(r.num_output_tokens > 0 for r in s[0].running)
    free_before = s[0].pool.num_free_blocks
    _dyntra_lockstep(s)
    assert s[0].paused_running > 0 and s[0].migrated_out == s[0].paused_running == s[1].migrated_in
    assert s[0].pool.num_free_blocks > free_before                       # the paused requests' blocks came back
    assert "r4" in s[0].requests and all(r.request_id != "r4" for r in s[1].waiting)
    got = list(s[1].waiting)
    assert all(r.status == RequestStatus.PREEMPTED and r.num_output_tokens > 0 and r.output_token_ids for r in got)
    assert all(r.request_id not in s[0].requests for r in got)
    # the receiver schedules prompt + generated tokens of a resumed request
    out = s[1].schedule.__wrapped__(s[1]) if hasattr(s[1].schedule, "__wrapped__") else None
    s[1].world = 1
    out = s[1].schedule()
    first = out.scheduled[0]
    assert first[0].request_id == got[0].request_id and first[1] == min(64, got[0].num_tokens)
    # a frozen rank admits nothing new
    s[0].lb_freeze = True
    fresh = Request("new", np.arange(20, dtype=np.int32), SamplingParams(max_tokens=4))
    s[0].add_request(fresh)
    s[0].world = 1
    s[0].schedule()
    assert fresh.status == RequestStatus.WAITING and fresh not in s[0].running


def test_training_consistent_attention_backend_selection():
    from vllm_ascend_b200.attention.backend import B200FABackend, training_consistent_attention
    from vllm_ascend_b200.engine.llm import LLM
    from vllm_ascend_b200.engine.request import SamplingParams
    from vllm_ascend_b200.platform import B200Platform
    add = {"rl_config": {"enabled": True, "enable_training_consistency": True}}
    llm = LLM("tiny-qwen", device="cpu", max_model_len=128, max_num_seqs=4, max_num_batched_tokens=32,
              block_size=16, additional_config=add)
    assert training_consistent_attention()
    assert B200Platform.get_attn_backend_cls(use_mla=False).endswith("B200FABackend")
    with pytest.raises(ValueError):
        B200Platform.get_attn_backend_cls(use_mla=True)
    assert B200FABackend.get_name() == "B200_TCGEN05_CONSISTENT"
    a = [o.outputs[0].token_ids for o in llm.generate([[1, 2, 3, 4, 5]], SamplingParams(temperature=0.0, max_tokens=4))]
    plain = LLM("tiny-qwen", device="cpu", max_model_len=128, max_num_seqs=4, max_num_batched_tokens=32, block_size=16)
    assert not training_consistent_attention()
    assert a == [o.outputs[0].token_ids for o in plain.generate([[1, 2, 3, 4, 5]], SamplingParams(temperature=0.0, max_tokens=4))]


def _ns(**kw):
    from types import SimpleNamespace as NS
    return NS(**kw)


def test_pipeline_refuses_unrunnable_parallel_layouts():
    from vllm_ascend_b200 import platform as P
    with pytest.raises(ValueError, match="prefill context parallelism"):
        P._validate_parallel_config(_ns(parallel_config=_ns(tensor_parallel_size=4, prefill_context_parallel_size=2,
                                                            decode_context_parallel_size=1)))
    with pytest.raises(ValueError, match="must divide"):
        P._validate_parallel_config(_ns(parallel_config=_ns(tensor_parallel_size=4, prefill_context_parallel_size=1,
                                                            decode_context_parallel_size=3)))
    with pytest.raises(ValueError, match="speculative"):
        P._validate_parallel_config(_ns(
            parallel_config=_ns(tensor_parallel_size=4, prefill_context_parallel_size=1, decode_context_parallel_size=2),
            speculative_config=_ns(num_speculative_tokens_per_batch_size={1: 3})))
    P._validate_parallel_config(_ns(parallel_config=_ns(tensor_parallel_size=4, prefill_context_parallel_size=1,
                                                        decode_context_parallel_size=2), speculative_config=None))


def test_pipeline_detects_quantization_from_the_checkpoint_dir(tmp_path):
    import json
    from vllm_ascend_b200 import platform as P
    (tmp_path / "quant_model_description.json").write_text(json.dumps({"model.layers.0.mlp.down_proj.weight": "FLOAT"}))
    mc = _ns(model=str(tmp_path), quantization=None, hf_config=None)
    P._auto_detect_quantization(_ns(model_config=mc))
    assert mc.quantization == "ascend"
    mc2 = _ns(model=str(tmp_path), quantization="fp8", hf_config=None)
    P._auto_detect_quantization(_ns(model_config=mc2))
    assert mc2.quantization == "fp8"                      # an explicit choice is kept
    other = tmp_path / "plain"
    other.mkdir()
    mc3 = _ns(model=str(other), quantization=None, hf_config=_ns(quantization_config={"quant_method": "compressed-tensors"}))
    P._auto_detect_quantization(_ns(model_config=mc3))
    assert mc3.quantization == "compressed-tensors"


def test_pipeline_ties_cp_interleave_to_block_size_under_kv_transfer():
    from vllm_ascend_b200 import platform as P
    bad = _ns(parallel_config=_ns(prefill_context_parallel_size=1, decode_context_parallel_size=2,
                                  cp_kv_cache_interleave_size=1),
              cache_config=_ns(block_size=128), kv_transfer_config=_ns())
    with pytest.raises(ValueError, match="interleave"):
        P._validate_cp_kv(bad)
    bad.kv_transfer_config = None
    P._validate_cp_kv(bad)


def test_balance_scheduler_freezes_admission_while_any_replica_is_full():
    from vllm_ascend_b200.config import CacheConfig, SchedulerConfig
    from vllm_ascend_b200.core.balance import BalanceScheduler
    from vllm_ascend_b200.engine.request import Request, SamplingParams
    peers = {"v": [0, 0]}
    sc = SchedulerConfig(max_num_seqs=4, max_num_batched_tokens=64, max_model_len=256)
    s = BalanceScheduler(sc, CacheConfig(block_size=16), 64, gather_fn=lambda v: [v] + peers["v"][1:], world=2)
    assert s.collective_schedule

    def add(i):
        s.add_request(Request(request_id=f"r{i}", prompt_token_ids=list(range(1, 9)),
                              sampling_params=SamplingParams(max_tokens=8, temperature=0.0, ignore_eos=True)))
    add(0)
    add(1)
    peers["v"] = [0, 4]                      # the other replica ended its last step at the cap
    out = s.schedule()
    assert not out.scheduled and len(s.waiting) == 2 and s.frozen_steps == 1 and s.peer_running == [0, 4]
    peers["v"] = [0, 3]                      # it finished one: admission resumes
    out = s.schedule()
    assert len(out.scheduled) == 2 and not s.waiting and s.frozen_steps == 1
    # optional lead rule: two ahead of the least loaded replica, which still has room -> wait
    lead = BalanceScheduler(sc, CacheConfig(block_size=16), 64, gather_fn=lambda v: [v, 0], world=2, max_lead=2)
    for i in range(3):
        lead.add_request(Request(request_id=f"q{i}", prompt_token_ids=list(range(1, 9)),
                                 sampling_params=SamplingParams(max_tokens=8, temperature=0.0, ignore_eos=True)))
    assert len(lead.schedule().scheduled) == 2 and len(lead.waiting) == 1
    # a single replica never gathers
    solo = BalanceScheduler(sc, CacheConfig(block_size=16), 64, gather_fn=lambda v: 1 / 0, world=1)
    assert not solo.collective_schedule and solo.schedule() is not None
