"""Tensor / expert parallel sharding logic on CPU ranks (gloo, world size 2)."""
import json
import os
import socket
import subprocess
import sys
import textwrap

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

WORKER = textwrap.dedent("""
    import json, os, sys
    import numpy as np
    sys.path.insert(0, {root!r})
    from vllm_ascend_b200.config import get_model_config
    from vllm_ascend_b200.engine.llm import LLM
    from vllm_ascend_b200.engine.request import SamplingParams
    preset, tp, ep, pp, dcp = sys.argv[1], int(sys.argv[2]), sys.argv[3] == "1", int(sys.argv[4]), int(sys.argv[5])
    pcp = int(sys.argv[6])
    fg = json.loads(sys.argv[7]) if len(sys.argv) > 7 else None
    cfg = get_model_config(preset)
    llm = LLM(cfg, device="cpu", tensor_parallel_size=tp, enable_expert_parallel=ep, pipeline_parallel_size=pp, decode_context_parallel_size=dcp,
              prefill_context_parallel_size=pcp,
              additional_config=json.loads(os.environ["ADDCFG"]) if os.environ.get("ADDCFG") else (dict(cp_kv_cache_interleave_size=4) if dcp > 1 else (dict(finegrained_tp_config=fg) if fg else None)),
              max_model_len=128, max_num_seqs=4, max_num_batched_tokens=32, block_size=16)
    rng = np.random.default_rng(2)
    lens = [int(x) for x in os.environ["PROMPT_LENS"].split(",")] if os.environ.get("PROMPT_LENS") else [24] * 3
    prompts = [rng.integers(0, cfg.vocab_size, size=n).tolist() for n in lens]
    want_lp = os.environ.get("LOGPROBS") == "1"
    outs = llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True,
                                                logprobs=2 if want_lp else None))
    if want_lp and int(os.environ.get("RANK", "0")) == 0:
        print("LOGPROBS " + json.dumps([[sorted((int(k), round(float(v), 4)) for k, v in d.items())
                                         for d in o.outputs[0].logprobs] for o in outs]), flush=True)
    if fg:                 # data parallel: every rank reports the prompts it served
        print("PART " + json.dumps(dict((str(o.prompt_token_ids[:3]), o.outputs[0].token_ids) for o in outs)), flush=True)
    if int(os.environ.get("RANK", "0")) == 0:
        print("RESULT " + json.dumps([o.outputs[0].token_ids for o in outs]), flush=True)
    # orderly teardown: groups destroyed on every rank, then leave without running the
    # interpreter's atexit handlers against helper threads of the process-group backend
    llm.shutdown()
    sys.stdout.flush()
    os._exit(0)
""")


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _run(preset, world, tp, ep=False, pp=1, dcp=1, pcp=1, fg=None, addcfg=None, prompt_lens=None):
    script = WORKER.format(root=ROOT)
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", MASTER_PORT=str(_free_port()),
               WORLD_SIZE=str(world), OMP_NUM_THREADS="2")
    if prompt_lens:
        env["PROMPT_LENS"] = ",".join(str(n) for n in prompt_lens)
    if addcfg:
        env["ADDCFG"] = json.dumps(addcfg)
    procs = []
    for r in range(world):
        e = dict(env, RANK=str(r), LOCAL_RANK=str(r))
        procs.append(subprocess.Popen([sys.executable, "-c", script, preset, str(tp), "1" if ep else "0", str(pp), str(dcp), str(pcp)] + ([json.dumps(fg)] if fg else []),
                                      env=e, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True))
    outs = [p.communicate(timeout=300) for p in procs]
    for p, (o, e) in zip(procs, outs):
        assert p.returncode == 0, e[-3000:]
    if fg:
        merged = {}
        for o, _ in outs:
            for l in o.splitlines():
                if l.startswith("PART "):
                    merged.update(json.loads(l[5:]))
        return merged
    line = [l for l in outs[0][0].splitlines() if l.startswith("RESULT ")][-1]
    return json.loads(line[7:])


@pytest.mark.parametrize("preset", ["tiny-qwen", "tiny-moe", "tiny-deepseek", "tiny-mqa"])
def test_tp2_matches_tp1(preset):
    assert _run(preset, 2, 2) == _run(preset, 1, 1)


def _run_logprobs(preset, world, tp, **kw):
    os.environ["LOGPROBS"] = "1"
    try:
        script_out = {}
        orig = subprocess.Popen

        class Capture(orig):
            def communicate(self, *a, **k):
                o, e = super().communicate(*a, **k)
                for l in o.splitlines():
                    if l.startswith("LOGPROBS "):
                        script_out["lp"] = json.loads(l[9:])
                return o, e
        subprocess.Popen = Capture
        toks = _run(preset, world, tp, **kw)
        return toks, script_out.get("lp")
    finally:
        subprocess.Popen = orig
        os.environ.pop("LOGPROBS", None)


@pytest.mark.parametrize("kw", [dict(pp=2), dict(pcp=2)])
def test_logprobs_reach_every_rank_under_pipeline_and_prefill_context_parallelism(kw):
    tp = 1
    want_t, want_lp = _run_logprobs("tiny-qwen", 1, 1)
    got_t, got_lp = _run_logprobs("tiny-qwen", 2, tp, **kw)
    assert got_t == want_t and got_lp is not None and len(got_lp) == len(want_lp)
    for a, b in zip(got_lp, want_lp):
        assert len(a) == len(b) == 6
        for da, db in zip(a, b):
            assert [k for k, _ in da] == [k for k, _ in db]
            assert max(abs(x[1] - y[1]) for x, y in zip(da, db)) < 1e-3


def test_expert_parallel_matches_single_rank():
    # EP over 2 ranks (DP attention: tp=1, experts sharded over the 2 ranks)
    assert _run("tiny-moe", 2, 1, ep=True) == _run("tiny-moe", 1, 1)


@pytest.mark.parametrize("preset", ["tiny-qwen", "tiny-moe"])
def test_pipeline_parallel_matches_single_rank(preset):
    assert _run(preset, 2, 1, pp=2) == _run(preset, 1, 1)


@pytest.mark.parametrize("tp,pp", [(1, 2), (2, 1)])
def test_profiling_chunk_scheduler_decides_alike_on_every_rank(tp, pp):
    """Chunk sizes come from measured durations, and every rank has its own scheduler copy: the ranks agree
    on each duration (start-up profile and online samples), so pipeline stages / TP ranks stay in step and the
    tokens are those of one rank."""
    add = {"scheduler_config": {"profiling_chunk_config": {"enabled": True, "min_chunk": 8}}}
    assert _run("tiny-qwen", 2, tp, pp=pp, addcfg=add) == _run("tiny-qwen", 1, 1)


def test_short_request_first_aging_is_decided_once_for_all_ranks():
    """A waiting limit of a few microseconds makes the aging decision depend on each rank's clock; the ranks
    share rank 0's answer, so two TP ranks stay in step (the run ends, with the single-rank tokens)."""
    add = {"scheduler_config": {"short_request_first_config": {"enabled": True, "threshold": 16,
                                                               "long_max_wait_ms": 0.005}}}
    lens = [40, 8, 30, 6, 50, 10, 12, 44]          # long and short prompts, more requests than batch rows
    assert _run("tiny-qwen", 2, 2, addcfg=add, prompt_lens=lens) == _run("tiny-qwen", 1, 1, prompt_lens=lens)


def test_decode_context_parallel_matches_single_rank():
    # MLA latent cache sharded along the sequence over the 2 TP ranks
    assert _run("tiny-deepseek", 2, 2, dcp=2) == _run("tiny-deepseek", 1, 1)


def test_replicated_shared_experts_match_single_rank():
    # whole shared expert on every TP rank, each runs half of the rows, rows all-gathered
    assert _run("tiny-deepseek", 2, 2, addcfg={"enable_shared_expert_dp": True}) == _run("tiny-deepseek", 1, 1)


SHARED_WORKER = textwrap.dedent("""
    import json, os, sys
    import torch, torch.distributed as dist
    sys.path.insert(0, {root!r})
    from vllm_ascend_b200.config import get_model_config
    from vllm_ascend_b200.models.layers import ParamFactory, SwiGLUMLP, TPComm
    from vllm_ascend_b200.ops.shared_experts import SharedExpertParallelMode as M, SharedExperts
    from vllm_ascend_b200.parallel import state as pstate
    dist.init_process_group("gloo")
    rank, tp = dist.get_rank(), dist.get_world_size()
    pstate.initialize_model_parallel(tp=tp)
    cfg = get_model_config("tiny-qwen")
    pf = ParamFactory(cfg, torch.device("cpu"), torch.float32)
    H, I, T = 64, 96, 10
    comm = TPComm(pstate.get_tp_group())
    one = TPComm(pstate.single_rank_group())
    full = SwiGLUMLP(pf, "shared", H, I, one, reduce_results=False)                 # whole weights
    shard = SwiGLUMLP(pf, "shared", H, I, comm, reduce_results=False)              # this rank's shard
    gate = pf.normal("shared_gate", (1, H))
    g = torch.Generator().manual_seed(1)
    x = torch.randn(T, H, generator=g)
    want = SharedExperts(full, one, True, gate).forward(x)
    rows = T // tp
    mine = x[rank * rows:(rank + 1) * rows]
    out = {{}}
    ex_tp, ex_dp = SharedExperts(shard, comm, False, gate), SharedExperts(full, comm, True, gate)
    out["modes"] = [ex_tp.mode(False).name, ex_dp.mode(False).name, ex_tp.mode(True).name, ex_dp.mode(True).name]
    out["tp"] = float((ex_tp.forward(x) - want).abs().max())
    part = ex_tp.forward(x, reduce=False)
    out["tp_partial_differs"] = float((part - want).abs().max()) > 1e-3
    out["dp"] = float((ex_dp.forward(x) - want).abs().max())
    out["dp_odd"] = float((ex_dp.forward(x[:7]) - want[:7]).abs().max())            # rows not divisible by tp
    out["sp"] = float((ex_tp.forward(mine, activations_sharded=True) - want[rank * rows:(rank + 1) * rows]).abs().max())
    out["sp_sedp"] = float((ex_dp.forward(mine, activations_sharded=True) - want[rank * rows:(rank + 1) * rows]).abs().max())
    ex_tp.validate_split(torch.device("cpu"), torch.float32, H)
    res = [None] * tp
    dist.all_gather_object(res, out)
    if rank == 0:
        print("RESULT " + json.dumps(res), flush=True)
    dist.barrier()
    dist.destroy_process_group()
    sys.stdout.flush()
    os._exit(0)
""")


def test_shared_experts_four_parallel_modes_agree():
    script = SHARED_WORKER.format(root=ROOT)
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", MASTER_PORT=str(_free_port()), WORLD_SIZE="2", OMP_NUM_THREADS="2")
    procs = [subprocess.Popen([sys.executable, "-c", script], env=dict(env, RANK=str(r), LOCAL_RANK=str(r)),
                              stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True) for r in range(2)]
    outs = [p.communicate(timeout=300) for p in procs]
    for p, (o, e) in zip(procs, outs):
        assert p.returncode == 0, e[-3000:]
    res = json.loads([l for l in outs[0][0].splitlines() if l.startswith("RESULT ")][-1][7:])
    for r in res:
        assert r["modes"] == ["TENSOR_PARALLEL", "DATA_PARALLEL_ONLY", "SEQUENCE_PARALLEL_ONLY", "SEQUENCE_PARALLEL_SEDP"]
        assert r["tp_partial_differs"]
        for k in ("tp", "dp", "dp_odd", "sp", "sp_sedp"):
            assert r[k] < 1e-4, (k, r)


def test_gqa_decode_context_parallel_matches_single_rank():
    # one KV head replicated over the 2 TP ranks; its cache sharded along the sequence between them
    assert _run("tiny-mqa", 2, 2, dcp=2) == _run("tiny-mqa", 1, 1)


def test_dcp_local_lengths_count_the_tokens_a_rank_stores():
    from vllm_ascend_b200.attention.dcp import local_seq_lens, owner_and_offset
    for bs, d, inter in ((16, 2, 1), (16, 2, 4), (8, 4, 2), (16, 4, 16)):
        for sl in (0, 1, 5, 16, 31, 32, 33, 100, 257):
            pos = np.arange(sl)
            owner, local = owner_and_offset(pos % (bs * d), bs, d, inter)
            for r in range(d):
                n = int(local_seq_lens(np.array([sl]), bs, d, r, inter)[0])
                assert n == int((owner == r).sum()), (bs, d, inter, sl, r)
                # the rank's tokens fill its blocks densely: local index == running count
                mine = np.nonzero(owner == r)[0]
                idx = (mine // (bs * d)) * bs + local[mine]
                assert (idx == np.arange(n)).all()


@pytest.mark.parametrize("preset,world,tp", [("tiny-qwen", 2, 1), ("tiny-moe", 2, 1), ("tiny-qwen", 4, 2)])
def test_prefill_context_parallel_matches_single_rank(preset, world, tp):
    # prompt chunks split head-tail over the PCP ranks, K / V all-gathered per layer, rank 0 samples
    assert _run(preset, world, tp, pcp=2) == _run(preset, 1, 1)


def test_pcp_partition_covers_every_token_once_and_balances_work():
    from vllm_ascend_b200.attention.pcp import build_plan, split_ranges
    starts, q_lens = np.array([0, 16, 40], dtype=np.int32), np.array([37, 1, 8], dtype=np.int32)
    cu = np.concatenate([[0], np.cumsum(q_lens)]).astype(np.int32)
    plan = build_plan(starts, q_lens, cu, 4)
    cover = np.concatenate(plan.local_idx)
    split = np.concatenate([np.arange(cu[0], cu[1]), np.arange(cu[2], cu[3])])     # requests 0 and 2 are split
    for t in split:
        assert (cover == t).sum() == 1
    assert (cover == cu[1]).sum() == 4                                             # the decode is replicated
    # causal cost of a rank = sum over its queries of the key count: head + tail pieces even it out
    cost = [sum(sum(range(a + 1, b + 1)) for a, b in split_ranges(0, 4096, 4, r)) for r in range(4)]
    assert max(cost) / min(cost) < 1.01
    assert any(e[2] == 37 for e in plan.entries[0]) and all(e[2] != 37 or e[0] != 0 for r in (1, 2, 3) for e in plan.entries[r])


@pytest.mark.parametrize("preset", ["tiny-qwen", "tiny-llama"])
def test_finegrained_tp_over_dp_replicas_matches_single_rank(preset):
    """Two DP replicas (tp=1) share o_proj, MLP, LM head and embedding shards; replicas serve
    different prompts with different token counts per step."""
    fg = dict(oproj_tensor_parallel_size=2, mlp_tensor_parallel_size=2, lmhead_tensor_parallel_size=2,
              embedding_tensor_parallel_size=2)
    got = _run(preset, 2, 1, fg=fg)
    want = _run(preset, 1, 1)
    assert len(got) == 3 and sorted(got.values()) == sorted(want)


SUSPEND_WORKER = textwrap.dedent("""
    import json, os, sys
    import numpy as np
    sys.path.insert(0, {root!r})
    from vllm_ascend_b200.config import get_model_config
    from vllm_ascend_b200.engine.llm import LLM
    from vllm_ascend_b200.engine.request import SamplingParams
    from vllm_ascend_b200.parallel import state as pstate
    cfg = get_model_config("tiny-moe")
    llm = LLM(cfg, device="cpu", tensor_parallel_size=2, enable_expert_parallel=True, max_model_len=128, max_num_seqs=4,
              max_num_batched_tokens=32, block_size=16)
    rng = np.random.default_rng(2)
    prompts = [rng.integers(0, cfg.vocab_size, size=24).tolist() for _ in range(3)]
    sp = SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True)
    before = [o.outputs[0].token_ids for o in llm.generate(prompts, sp)]
    tp = pstate.get_tp_group()
    destroyed = pstate.suspend_groups()
    assert destroyed >= 2 and tp.device_group is None and pstate.groups_suspended()
    assert pstate.suspend_groups() == 0
    restored = pstate.restore_groups()
    assert restored == destroyed and tp.device_group is not None and pstate.get_tp_group() is tp
    after = [o.outputs[0].token_ids for o in llm.generate(prompts, sp)]
    if int(os.environ.get("RANK", "0")) == 0:
        print("RESULT " + json.dumps([before, after, destroyed]), flush=True)
    llm.shutdown()
    sys.stdout.flush()
    os._exit(0)
""")


def test_groups_destroyed_for_sleep_come_back_in_the_same_coordinators():
    """The sleep path with extra cleanup destroys every model-parallel communicator and wake-up
    re-creates them inside the coordinator objects the layers already hold."""
    script = SUSPEND_WORKER.format(root=ROOT)
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", MASTER_PORT=str(_free_port()), WORLD_SIZE="2", OMP_NUM_THREADS="2")
    procs = [subprocess.Popen([sys.executable, "-c", script], env=dict(env, RANK=str(r), LOCAL_RANK=str(r)),
                              stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True) for r in range(2)]
    outs = [p.communicate(timeout=300) for p in procs]
    for p, (o, e) in zip(procs, outs):
        assert p.returncode == 0, e[-3000:]
    before, after, destroyed = json.loads([l for l in outs[0][0].splitlines() if l.startswith("RESULT ")][-1][7:])
    assert before == after and destroyed >= 2


DYNTRA_WORKER = textwrap.dedent("""
    import json, os, sys
    import numpy as np
    sys.path.insert(0, {root!r})
    from vllm_ascend_b200.config import get_model_config
    from vllm_ascend_b200.engine.llm import LLM
    from vllm_ascend_b200.engine.request import SamplingParams
    dp = int(sys.argv[1])
    policy = sys.argv[2] if len(sys.argv) > 2 else "dyntra"
    add = None
    if dp > 1 and policy == "dyntra":
        add = {{"scheduler_config": {{"dyntra_lb_config": {{"enabled": True, "imbalance_threshold": 0.02,
                                                            "max_migrations_per_step": 2}}}}}}
    elif dp > 1:
        add = {{"scheduler_config": {{"enable_balance_scheduling": True}}}}
    cfg = get_model_config("tiny-qwen")
    llm = LLM(cfg, device="cpu", data_parallel_size=dp, additional_config=add, max_model_len=256, max_num_seqs=4,
              max_num_batched_tokens=64, block_size=16, num_gpu_blocks_override=64)
    rng = np.random.default_rng(5)
    # even prompts (rank 0's share) are long, odd ones short: rank 0 is the loaded one
    prompts = [rng.integers(0, cfg.vocab_size, size=(90 if i % 2 == 0 else 8)).tolist() for i in range(12)]
    outs = llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=10, ignore_eos=True))
    s = llm.engine.scheduler
    stats = [getattr(s, "migrated_out", 0), getattr(s, "migrated_in", 0), getattr(s, "paused_running", 0),
             getattr(s, "frozen_steps", -1), type(s).__name__]
    print("STATS%s " % os.environ.get("RANK", "0") + json.dumps(stats), flush=True)
    if int(os.environ.get("RANK", "0")) == 0:
        print("RESULT " + json.dumps([o.outputs[0].token_ids for o in outs]), flush=True)
    llm.shutdown()
    sys.stdout.flush()
    os._exit(0)
""")


def _run_dyntra(dp, policy="dyntra"):
    script = DYNTRA_WORKER.format(root=ROOT)
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", MASTER_PORT=str(_free_port()), WORLD_SIZE=str(dp), OMP_NUM_THREADS="2")
    procs = [subprocess.Popen([sys.executable, "-c", script, str(dp), policy],
                              env=dict(env, RANK=str(r), LOCAL_RANK=str(r)),
                              stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True) for r in range(dp)]
    outs = [p.communicate(timeout=300) for p in procs]
    for p, (o, e) in zip(procs, outs):
        assert p.returncode == 0, e[-3000:]
    res = json.loads([l for l in outs[0][0].splitlines() if l.startswith("RESULT ")][-1][7:])
    stats = {}
    for o, _ in outs:
        for l in o.splitlines():
            if l.startswith("STATS"):
                stats[int(l[5])] = json.loads(l[7:])
    return res, stats


def test_dyntra_lb_balances_data_parallel_engines_without_changing_outputs():
    want, _ = _run_dyntra(1)
    got, stats = _run_dyntra(2)
    assert got == want
    # the loaded rank handed requests to the other one (waiting or paused running ones)
    assert stats[0][0] > 0 and stats[1][1] == stats[0][0] + stats[1][0] - stats[0][1]


def test_balance_scheduling_on_two_data_parallel_engines():
    """Two replicas with different loads (one finishes its share early and keeps stepping with nothing to
    do): the per-step gather never blocks, admission freezes while a replica is full, tokens are those of a
    single engine."""
    want, _ = _run_dyntra(1)
    got, stats = _run_dyntra(2, "balance")
    assert got == want
    assert stats[0][4] == stats[1][4] == "BalanceScheduler"
    assert stats[0][3] > 0 or stats[1][3] > 0
