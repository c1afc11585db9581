"""TP/full weight switching on two gloo ranks: a row-parallel and a column-parallel layer (bf16 and
128 x 128 block-scaled fp8) run with the all-gathered weight and give the unsharded layer's answer;
afterwards they hold their shards again; layers of equal geometry share the pooled full buffer."""
import json
import os
import socket
import subprocess
import sys
import textwrap

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

WORKER = textwrap.dedent("""
    import json, os, sys
    import torch, torch.distributed as dist
    sys.path.insert(0, {root!r})
    from types import SimpleNamespace as NS
    from vllm_ascend_b200.quantization import schemes
    from vllm_ascend_b200.quantization.tp_weight_switch import TPWeightSwitch, split_for_tp, supports
    from vllm_ascend_b200.ops import reference as ref
    dist.init_process_group("gloo")
    rank, tp = dist.get_rank(), dist.get_world_size()
    group = NS(world_size=tp, rank_in_group=rank, device_group=dist.group.WORLD)
    g = torch.Generator().manual_seed(0)
    N, K = 256, 512
    w = torch.randn(N, K, generator=g) * 0.1
    b = torch.randn(N, generator=g)
    x = torch.randn(5, K, generator=g)
    out = {{}}
    pool = {{}}
    # ---- bf16 / float layers
    row = NS(weight=split_for_tp(w, tp, rank, 1), bias=None, quant=None, name="row")
    col = NS(weight=split_for_tp(w, tp, rank, 0), bias=split_for_tp(b, tp, rank, 0), quant=None, name="col")
    col2 = NS(weight=split_for_tp(w * 2, tp, rank, 0), bias=split_for_tp(b, tp, rank, 0), quant=None, name="col2")
    sr, sc, sc2 = (TPWeightSwitch(row, group, "input", pool, "k"), TPWeightSwitch(col, group, "output", pool, "k"),
                   TPWeightSwitch(col2, group, "output", pool, "k"))
    sr.start_gather(); sc.start_gather()          # started ahead, consumed later
    with sr.full() as L:
        out["row"] = float((x @ L.weight.t() - x @ w.t()).abs().max())
    with sc.full() as L:
        out["col"] = float((x @ L.weight.t() + L.bias - (x @ w.t() + b)).abs().max())
        shared = L.weight.data_ptr()
    with sc2.full() as L:                         # same geometry: same pooled buffer, other contents
        out["col2"] = float((x @ L.weight.t() - x @ (2 * w).t()).abs().max())
        out["pooled"] = L.weight.data_ptr() == shared
    out["back"] = list(row.weight.shape) == [N, K // tp] and list(col.weight.shape) == [N // tp, K]
    # ---- block-scaled fp8: weight and scales travel together
    q, s = schemes.quantize_weight_block_fp8(w)
    fq = NS(weight=split_for_tp(q.view(torch.uint8), tp, rank, 1).view(torch.float8_e4m3fn),
            weight_scale_inv=split_for_tp(s, tp, rank, 1), bias=None, quant=schemes.Fp8BlockLinear(), name="fp8row")
    out["fp8_supported"] = supports(fq)
    sf = TPWeightSwitch(fq, group, "input", pool, "k")
    with sf.full() as L:
        deq = ref.dequant_block_fp8_weight(L.weight, L.weight_scale_inv)
        out["fp8"] = float((deq - ref.dequant_block_fp8_weight(q, s)).abs().max())
    out["fp8_back"] = list(fq.weight_scale_inv.shape) == [N // 128, K // 128 // tp]
    out["unsupported"] = not supports(NS(quant=NS(scheme_name="W4A16")))
    if rank == 0:
        print("RESULT " + json.dumps(out), flush=True)
    dist.barrier()
    dist.destroy_process_group()
""")


def test_tp_weight_switch_gathers_full_weights_and_restores_shards():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), WORLD_SIZE="2", OMP_NUM_THREADS="2")
    procs = [subprocess.Popen([sys.executable, "-c", WORKER.format(root=ROOT)], env=dict(env, RANK=str(r)),
                              stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True) for r in range(2)]
    outs = [p.communicate(timeout=300) for p in procs]
    for p, (o, e) in zip(procs, outs):
        assert p.returncode == 0, e[-3000:]
    r = json.loads([l for l in outs[0][0].splitlines() if l.startswith("RESULT ")][-1][7:])
    assert r["row"] < 1e-5 and r["col"] < 1e-5 and r["col2"] < 1e-5
    assert r["pooled"] and r["back"]
    assert r["fp8_supported"] and r["fp8"] == 0.0 and r["fp8_back"]
    assert r["unsupported"]
