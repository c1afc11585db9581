#!/usr/bin/env python
"""Per-kernel micro-benchmarks with roofline fractions.

    python benchmarks/kernel_bench.py gemm --m 8192 --n 4096 --k 4096
    python benchmarks/kernel_bench.py attn-decode --batch 256 --ctx 1152
    python benchmarks/kernel_bench.py attn-prefill --batch 8 --seq 1024
    python benchmarks/kernel_bench.py norm --tokens 8192 --hidden 4096
    python benchmarks/kernel_bench.py all

Timing: CUDA events on the launching stream, warm-up first, a buffer larger than
L2 is rewritten between timed iterations.  Fractions are "of measured": the
denominators come from MEASURED_PEAKS.json at the repository root (copy bandwidth
and cuBLAS bf16 throughput measured on this machine type); when the file is absent
the fallback 6650 GB/s / 1590 TFLOP/s is used and marked "of fallback".
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

from vllm_ascend_b200 import _native, ops  # noqa: E402


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return d["hbm_gbs"], d["bf16_tflops"], "of measured"
    return 6650.0, 1590.0, "of fallback"


_flush = None


def timeit(fn, iters=20, warm=5, flush=True):
    global _flush
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    if flush and _flush is None:
        _flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    ts = []
    for _ in range(iters):
        if flush:
            _flush.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1))
    ts.sort()
    return ts[len(ts) // 2]


def timeit_between(fn, between, iters=20, warm=5):
    """Median device time of ``fn`` when ``between`` (untimed) runs before every timed launch."""
    for _ in range(warm):
        between()
        fn()
    torch.cuda.synchronize()
    evs = []
    for _ in range(iters):
        between()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        evs.append((e0, e1))
    torch.cuda.synchronize()
    ts = sorted(e0.elapsed_time(e1) for e0, e1 in evs)
    return ts[len(ts) // 2]


def bench_gemm(a):
    M, N, K = a.m, a.n, a.k
    x = (torch.randn(M, K, device="cuda") * 0.1).bfloat16()
    w = (torch.randn(N, K, device="cuda") * 0.1).bfloat16()
    out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
    if a.raster:
        _native.register_signature("b200_gemm_2cta_set_raster", [ctypes.c_int])
        _native.lib().b200_gemm_2cta_set_raster(a.raster)
    _native.register_signature("b200_gemm_2cta_set_bn", [ctypes.c_int])
    _native.lib().b200_gemm_2cta_set_bn(a.tile_n)       # 0: the kernel chooses its tile width
    _native.register_signature("b200_gemm_2cta_set_l2_prefetch", [ctypes.c_int])
    _native.lib().b200_gemm_2cta_set_l2_prefetch(a.l2_prefetch)      # 0: off
    ms = timeit(lambda: ops.linear(x, w, out=out, bn=a.bn), a.iters, flush=not a.no_flush)
    ms_lib = timeit(lambda: torch.nn.functional.linear(x, w), a.iters, flush=not a.no_flush) if a.compare else None
    hbm, tf, tag = peaks()
    fl = 2.0 * M * N * K
    line = (f"gemm M={M} N={N} K={K} bn={a.bn or 'auto'} tile_n={a.tile_n or 'auto'} l2pf={a.l2_prefetch}: {ms:.4f} ms  {fl / ms / 1e9:.0f} TFLOP/s "
            f"({fl / ms / 1e9 / tf:.2f} {tag})")
    if ms_lib:
        line += f"  | cuBLAS {ms_lib:.4f} ms {fl / ms_lib / 1e9:.0f} TFLOP/s"
    print(line, flush=True)


def bench_gemm_fp8(a):
    """Block-scaled fp8 GEMM (1x128 activation scales, 128x128 weight scales) incl. and excl. the
    activation quantisation pass."""
    from vllm_ascend_b200.quantization import schemes
    M, N, K = a.m, a.n, a.k
    x = (torch.randn(M, K, device="cuda") * 0.1).bfloat16()
    w = (torch.randn(N, K, device="cuda") * 0.1).bfloat16()
    w8, ws = schemes.quantize_weight_block_fp8(w)
    xq, xs = ops.quant_fp8_group128(x)
    ms_all = timeit(lambda: schemes.fp8_block_linear(x, w8, ws), a.iters)
    ms_gemm = timeit(lambda: schemes.fp8_block_linear(None, w8, ws, quant=(xq, xs)), a.iters)
    hbm, tf, tag = peaks()
    fl = 2.0 * M * N * K
    print(f"gemm-fp8 M={M} N={N} K={K}: quant+gemm {ms_all:.4f} ms {fl / ms_all / 1e9:.0f} TFLOP/s | gemm only "
          f"{ms_gemm:.4f} ms {fl / ms_gemm / 1e9:.0f} TFLOP/s ({fl / ms_gemm / 1e9 / tf:.2f} of the bf16 {tag} peak)",
          flush=True)
    _native.check_status(torch.device("cuda"))


def bench_attn_decode(a):
    from gpu_utils import make_paged_case
    B, ctx = a.batch, a.ctx
    if a.ragged:
        # serving-like batch: context lengths spread over +-ragged tokens around ctx
        import numpy as np
        lens = np.random.default_rng(0).integers(ctx - a.ragged, ctx + a.ragged, size=B)
        ctxs = [int(x) - 1 for x in lens]
    else:
        ctxs = [ctx - 1] * B
    q, kc, vc, meta = make_paged_case([1] * B, ctxs, a.hq, a.hkv, a.d, a.block_size, seed=0,
                                      layout=a.kv_layout)
    out = torch.empty_like(q)
    scale = a.d ** -0.5
    meta.tile_seq = meta.tile_qoff = None
    bytes_kv = 2.0 * float(sum(c + 1 for c in ctxs)) * a.hkv * a.d * 2
    between = None
    if a.interleave_gemm:
        # a compute-bound GEMM between the timed launches keeps the GPU at its power cap, the
        # clock regime the kernel meets inside a serving step
        ga = torch.randn(8192, 4096, device="cuda", dtype=torch.bfloat16)
        gb = torch.randn(12288, 4096, device="cuda", dtype=torch.bfloat16)
        gout = torch.empty(8192, 12288, device="cuda", dtype=torch.bfloat16)
        between = lambda: [ops.linear(ga, gb, out=gout) for _ in range(a.interleave_gemm)]
    hbm, tf, tag = peaks()
    for name, fn in (
        ("cuda-core", lambda ns: ops.paged_decode(q, kc, vc, meta.block_table, meta.seq_lens, scale, out, 0, ns)),
        ("tcgen05", lambda ns: ops.paged_attention_tc(q, kc, vc, meta, scale, out, True, 0, ns)),
        ("tcgen05-decode", lambda ns: ops.paged_attention_decode_tc(q, kc, vc, meta, scale, out, 0, ns)),
    ):
        if a.impl not in ("both", name):
            continue
        if name == "cuda-core" and a.kv_layout != "NHD":
            continue        # that kernel reads [blocks, tokens, heads, D] caches only
        ns = a.splits or ops.choose_num_splits(B, a.hkv, ctx)
        ms = timeit(lambda: fn(ns), a.iters) if between is None else timeit_between(lambda: fn(ns), between, a.iters)
        print(f"attn-decode[{name}/{a.kv_layout}] B={B} ctx={ctx}{' ragged' if a.ragged else ''}"
              f"{' between GEMMs' if between else ''} Hq={a.hq} Hkv={a.hkv} D={a.d} splits={ns}: "
              f"{ms:.4f} ms  {bytes_kv / ms / 1e6:.0f} GB/s ({bytes_kv / ms / 1e6 / hbm:.2f} {tag})",
              flush=True)
    _native.check_status(torch.device("cuda"))


def bench_mla_decode(a):
    """Absorbed-weight MLA decode: B sequences of ctx tokens, H heads, one query token each."""
    from vllm_ascend_b200.attention.mla import mla_decode_native
    dev = torch.device("cuda")
    B, ctx, H, bs = a.batch, a.ctx, a.heads, a.block_size
    nblk = (ctx + bs - 1) // bs
    total = B * nblk + 1
    g = torch.Generator(device="cuda").manual_seed(0)
    lat = (torch.randn(total, bs, 512, device=dev, generator=g) * 0.5).bfloat16()
    pe = (torch.randn(total, bs, 64, device=dev, generator=g) * 0.5).bfloat16()
    bt = (torch.randperm(total - 1, device=dev, generator=g) + 1).int().view(B, nblk)
    q = (torch.randn(B, H, 576, device=dev, generator=g) * 0.3).bfloat16()
    row_seq = torch.arange(B, dtype=torch.int32, device=dev)
    row_kv = torch.full((B,), ctx, dtype=torch.int32, device=dev)
    scale = 576 ** -0.5
    hbm, tf, tag = peaks()
    ms = timeit(lambda: mla_decode_native(q, lat, pe, row_seq, row_kv, bt, scale, a.splits, ctx), a.iters)
    kv_bytes = B * ctx * 576 * 2.0
    flops = 2.0 * B * ctx * H * (576 + 512)
    print(f"mla-decode B={B} ctx={ctx} H={H}: {ms:.4f} ms  KV {kv_bytes / ms / 1e6:.0f} GB/s "
          f"({kv_bytes / ms / 1e6 / hbm:.2f} {tag})  {flops / ms / 1e9:.0f} TFLOP/s ({flops / ms / 1e9 / tf:.2f} {tag})",
          flush=True)
    _native.check_status(dev)


def bench_gdn(a):
    """Gated delta rule: decode (B sequences, one token each: state traffic bound) and one prefill
    chunk (sequential over tokens: latency bound)."""
    from vllm_ascend_b200.ops import linear_attn as la
    dev = torch.device("cuda")
    Hk, Hv, DK, DV = 16, 32, 128, 128
    hbm, tf, tag = peaks()
    g = torch.Generator(device="cuda").manual_seed(0)
    for B, q_len in ((a.batch, 1), (max(1, a.batch // 64), a.seq)):
        T = B * q_len
        q = torch.randn(T, Hk, DK, device=dev, generator=g).bfloat16()
        k = torch.randn(T, Hk, DK, device=dev, generator=g).bfloat16()
        v = torch.randn(T, Hv, DV, device=dev, generator=g).bfloat16()
        gg = -torch.rand(T, Hv, device=dev, generator=g) * 0.3
        beta = torch.rand(T, Hv, device=dev, generator=g)
        S = torch.randn(B + 1, Hv, DK, DV, device=dev, generator=g) * 0.1
        cu = torch.arange(0, T + 1, q_len, dtype=torch.int32, device=dev)
        slots = torch.arange(B, dtype=torch.int32, device=dev)
        init = torch.ones(B, dtype=torch.int32, device=dev)
        ms = timeit(lambda: la.gated_delta_rule(q, k, v, gg, beta, S, cu, slots, init, DK ** -0.5), a.iters)
        state_bytes = 2.0 * B * Hv * DK * DV * 4
        print(f"gated-delta-rule B={B} q_len={q_len} Hv={Hv} {DK}x{DV}: {ms:.4f} ms  state {state_bytes / ms / 1e6:.0f} GB/s "
              f"({state_bytes / ms / 1e6 / hbm:.2f} {tag})  {T / ms * 1e3:.0f} tok/s", flush=True)
        if q_len >= 64:
            cu_h = cu.cpu().numpy()
            ms_c = timeit(lambda: la.gated_delta_rule_chunked(q, k, v, gg, beta, S, cu_h, slots, init, DK ** -0.5),
                          max(3, a.iters // 4))
            print(f"gated-delta-rule chunk-parallel form, same case: {ms_c:.4f} ms  {T / ms_c * 1e3:.0f} tok/s "
                  f"({ms / ms_c:.1f}x the recurrence)", flush=True)
    _native.check_status(dev)


def bench_attn_prefill(a):
    from gpu_utils import make_paged_case
    B, S = a.batch, a.seq
    q, kc, vc, meta = make_paged_case([S] * B, [a.ctx] * B, a.hq, a.hkv, a.d, a.block_size, seed=0,
                                      layout=a.kv_layout)
    out = torch.empty_like(q)
    scale = a.d ** -0.5
    ms = timeit(lambda: ops.paged_attention_tc(q, kc, vc, meta, scale, out, True, 0, 1), a.iters)
    # causal: each query sees ctx + (i+1) keys
    pairs = B * (S * a.ctx + S * (S + 1) / 2.0)
    fl = 4.0 * pairs * a.hq * a.d
    hbm, tf, tag = peaks()
    print(f"attn-prefill B={B} S={S} ctx={a.ctx} Hq={a.hq} Hkv={a.hkv} D={a.d}: {ms:.4f} ms  "
          f"{fl / ms / 1e9:.0f} TFLOP/s ({fl / ms / 1e9 / tf:.2f} {tag})", flush=True)
    _native.check_status(torch.device("cuda"))


def bench_norm(a):
    T, H = a.tokens, a.hidden
    x = torch.randn(T, H, device="cuda").bfloat16()
    r = torch.randn(T, H, device="cuda").bfloat16()
    w = torch.ones(H, device="cuda").bfloat16()
    out = torch.empty_like(x)
    hbm, tf, tag = peaks()
    ms = timeit(lambda: ops.rms_norm(x, w, 1e-6, r, out=out), a.iters)
    by = 4.0 * T * H * 2
    print(f"add+rmsnorm T={T} H={H}: {ms:.4f} ms  {by / ms / 1e6:.0f} GB/s ({by / ms / 1e6 / hbm:.2f} {tag})")
    g = torch.randn(T, 2 * a.inter, device="cuda").bfloat16()
    ms = timeit(lambda: ops.silu_and_mul(g), a.iters)
    by = 3.0 * T * a.inter * 2
    print(f"silu_and_mul T={T} I={a.inter}: {ms:.4f} ms  {by / ms / 1e6:.0f} GB/s ({by / ms / 1e6 / hbm:.2f} {tag})",
          flush=True)


def bench_rope(a):
    """Split-QKV + q/k RMSNorm + RoPE + paged KV write (one pass over the fused QKV rows)."""
    from vllm_ascend_b200.models.layers import get_cos_sin_cache
    T, Hq, Hkv, D = a.tokens, a.hq, a.hkv, a.d
    qkv = torch.randn(T, (Hq + 2 * Hkv) * D, device="cuda").bfloat16()
    pos = torch.arange(T, device="cuda", dtype=torch.int64) % 4096
    cs = get_cos_sin_cache(D, 8192, 1e6, None, torch.device("cuda"))
    nb = (T + 127) // 128 + 1
    kc = ops.alloc_kv_cache(nb, 128, Hkv, D, torch.bfloat16, "cuda")
    vc = ops.alloc_kv_cache(nb, 128, Hkv, D, torch.bfloat16, "cuda")
    slots = torch.arange(T, device="cuda", dtype=torch.int64) + 128
    w = torch.ones(D, device="cuda").bfloat16()
    hbm, tf, tag = peaks()
    ms = timeit(lambda: ops.qknorm_rope_kvwrite(qkv, pos, cs, D, w, w, 1e-6, kc, vc, slots, Hq, Hkv, D), a.iters)
    by = T * D * 2.0 * (2 * (Hq + Hkv) + 3 * Hkv)       # q, k read + written in place; v read; k, v cache written
    print(f"qknorm+rope+kvwrite T={T} Hq={Hq} Hkv={Hkv} D={D}: {ms:.4f} ms  {by / ms / 1e6:.0f} GB/s "
          f"({by / ms / 1e6 / hbm:.2f} {tag})", flush=True)
    _native.check_status(torch.device("cuda"))


def bench_sampler(a):
    """Greedy argmax over the vocabulary, and temperature / top-k / top-p sampling (radix select)."""
    B, V = a.batch, a.vocab
    logits = torch.randn(B, V, device="cuda").bfloat16()
    hbm, tf, tag = peaks()
    ms = timeit(lambda: ops.argmax(logits), a.iters)
    print(f"argmax B={B} V={V}: {ms:.4f} ms  {B * V * 2 / ms / 1e6:.0f} GB/s ({B * V * 2 / ms / 1e6 / hbm:.2f} {tag})")
    temp = torch.full((B,), 0.8, device="cuda")
    tk = torch.full((B,), 50, device="cuda", dtype=torch.int32)
    tp = torch.full((B,), 0.9, device="cuda")
    seeds = torch.arange(B, device="cuda", dtype=torch.int64)
    offs = torch.zeros(B, device="cuda", dtype=torch.int64)
    lf = logits.float()

    def run():
        ops.sample(lf.clone(), temp, tk, tp, None, seeds, offs)
    ms_clone = timeit(lambda: lf.clone(), a.iters)
    ms = timeit(run, a.iters) - ms_clone
    print(f"sample top-k/top-p B={B} V={V}: {ms:.4f} ms (clone of the logits subtracted)  "
          f"{B * V * 4 / ms / 1e6:.0f} GB/s of fp32 logits per pass", flush=True)


def bench_moe(a):
    """Grouped GEMM + SwiGLU over experts (rows already sorted by expert)."""
    from vllm_ascend_b200.ops import moe_native
    E, K, I, rows = a.experts, a.k, a.inter, a.m
    w13 = (torch.randn(E, 2 * I, K, device="cuda") * 0.05).bfloat16()
    w2 = (torch.randn(E, K, I, device="cuda") * 0.05).bfloat16()
    x = (torch.randn(rows, K, device="cuda") * 0.1).bfloat16()
    per = rows // E
    offsets = torch.arange(0, E + 1, device="cuda", dtype=torch.int32) * per
    offsets[-1] = rows
    hbm, tf, tag = peaks()
    h = moe_native.grouped_gemm(x, w13, offsets, True)
    ms1 = timeit(lambda: moe_native.grouped_gemm(x, w13, offsets, True), a.iters)
    ms2 = timeit(lambda: moe_native.grouped_gemm(h, w2, offsets, False), a.iters)
    f1, f2 = 2.0 * rows * 2 * I * K, 2.0 * rows * K * I
    b1 = (w13.numel() + x.numel() + h.numel()) * 2.0
    print(f"moe grouped gemm1+swiglu E={E} rows={rows} K={K} I={I}: {ms1:.4f} ms {f1 / ms1 / 1e9:.0f} TFLOP/s "
          f"({f1 / ms1 / 1e9 / tf:.2f} {tag}), weights+acts {b1 / ms1 / 1e6:.0f} GB/s ({b1 / ms1 / 1e6 / hbm:.2f} {tag})")
    print(f"moe grouped gemm2 : {ms2:.4f} ms {f2 / ms2 / 1e9:.0f} TFLOP/s ({f2 / ms2 / 1e9 / tf:.2f} {tag})", flush=True)
    _native.check_status(torch.device("cuda"))


def bench_kv_copy(a):
    """Paged KV block gather/scatter between two caches (all layers in one launch)."""
    from vllm_ascend_b200.attention.backend import B200AttentionBackend
    nb, bs, H, D = a.blocks, 128, a.hkv, a.d
    src = torch.randn(nb, bs, H, D, device="cuda").bfloat16()
    dst = torch.zeros_like(src)
    perm = torch.randperm(nb)
    pairs = torch.stack([torch.arange(nb), perm], dim=1)
    hbm, tf, tag = peaks()
    ms = timeit(lambda: B200AttentionBackend.swap_blocks(src, dst, pairs), a.iters)
    by = 2.0 * src.numel() * 2
    print(f"kv block copy blocks={nb} x {bs * H * D * 2 >> 10} KiB: {ms:.4f} ms  {by / ms / 1e6:.0f} GB/s "
          f"({by / ms / 1e6 / hbm:.2f} {tag})", flush=True)
    _native.check_status(torch.device("cuda"))


def bench_gemm_folded(a):
    """Paired-CTA GEMM with the RMSNorm fold: consumer (row scale from partial statistics) and producer
    (residual add + per-tile sum of squares) forms against the plain kernel."""
    M, N, K = a.m, a.n, a.k
    x = (torch.randn(M, K, device="cuda") * 0.5).bfloat16()
    w = (torch.randn(N, K, device="cuda") * 0.05).bfloat16()
    res = torch.randn(M, N, device="cuda").bfloat16()
    out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
    ss_in = ops.alloc_row_stats(M + 8, max(N, K), "cuda")
    ss_out = ops.alloc_row_stats(M + 8, max(N, K), "cuda")
    R, P = ss_in.stats_rows, ss_in.stats_parts
    ss_in[:R * P].view(P, R)[:8, :M] = (x.float() ** 2).sum(-1) / 8
    ss_in[R * P:].view(torch.int32)[0] = 8
    hbm, tf, tag = peaks()
    fl = 2.0 * M * N * K
    ms0 = timeit(lambda: ops.linear_norm_folded(x, w, out=out), a.iters)
    ms1 = timeit(lambda: ops.linear_norm_folded(x, w, out=out, ss_in=ss_in, norm_dim=K, eps=1e-6), a.iters)
    ms2 = timeit(lambda: ops.linear_norm_folded(x, w, residual=res, out=out, ss_out=ss_out), a.iters)
    print(f"gemm-folded M={M} N={N} K={K}: plain {ms0:.4f} ms {fl / ms0 / 1e9:.0f} TFLOP/s | row-scaled "
          f"{ms1:.4f} ms {fl / ms1 / 1e9:.0f} | +residual+statistics {ms2:.4f} ms {fl / ms2 / 1e9:.0f} "
          f"({fl / ms2 / 1e9 / tf:.2f} {tag})", flush=True)
    _native.check_status(torch.device("cuda"))


def bench_quant(a):
    """Producers of the fp8 GEMM's activation operand: add + RMSNorm + 1x128 quant, SiLU-mul + quant."""
    T, H, I = a.tokens, a.hidden, a.inter
    x = torch.randn(T, H, device="cuda").bfloat16()
    r = torch.randn(T, H, device="cuda").bfloat16()
    w = torch.ones(H, device="cuda").bfloat16()
    hbm, tf, tag = peaks()
    ms = timeit(lambda: ops.rms_norm_quant_fp8(x, w, 1e-6, r), a.iters)
    by = T * H * (2 + 2 + 2 + 1) + T * (H // 128) * 4.0          # x, residual in / residual out, fp8 out, scales
    print(f"add+rmsnorm+quant T={T} H={H}: {ms:.4f} ms  {by / ms / 1e6:.0f} GB/s ({by / ms / 1e6 / hbm:.2f} {tag})")
    g = torch.randn(T, 2 * I, device="cuda").bfloat16()
    ms = timeit(lambda: ops.silu_and_mul_quant_fp8(g), a.iters)
    by = T * I * (4 + 1) + T * (I // 128) * 4.0
    print(f"silu_mul+quant T={T} I={I}: {ms:.4f} ms  {by / ms / 1e6:.0f} GB/s ({by / ms / 1e6 / hbm:.2f} {tag})")
    ms = timeit(lambda: ops.quant_fp8_group128(x), a.iters)
    by = T * H * 3 + T * (H // 128) * 4.0
    print(f"quant 1x128 T={T} H={H}: {ms:.4f} ms  {by / ms / 1e6:.0f} GB/s ({by / ms / 1e6 / hbm:.2f} {tag})", flush=True)
    _native.check_status(torch.device("cuda"))


def bench_moe_route(a):
    """Router top-k (softmax scoring, renormalised) over the expert logits."""
    from vllm_ascend_b200.ops import moe_native
    T, E, k = a.tokens, a.experts, a.topk
    logits = torch.randn(T, E, device="cuda")
    ms = timeit(lambda: moe_native.gating_topk(logits, k, "softmax", True, 1, 1, None, 1.0), a.iters)
    print(f"moe gating top-{k} T={T} E={E}: {ms:.4f} ms  {T * E * 4 / ms / 1e6:.0f} GB/s of logits", flush=True)


def bench_indexer(a):
    """Lightning indexer (scores of every query token against its sequence's index keys + top-k), decode rows."""
    from gpu_utils import make_paged_case
    from vllm_ascend_b200.attention import sfa
    B, ctx, G = a.batch, a.ctx, a.heads
    _, kc, _, meta = make_paged_case([1] * B, [ctx] * B, 1, 1, 128, 128, device="cuda", seed=0)
    kc = kc.cuda()
    meta.positions = torch.full((B,), ctx, dtype=torch.int64, device="cuda")
    g = torch.Generator(device="cuda").manual_seed(0)
    q_idx = (torch.randn(B, G, 128, device="cuda", generator=g) * 0.3).bfloat16()
    w = torch.rand(B, G, device="cuda", generator=g)
    ms = timeit(lambda: sfa.lightning_indexer_native(q_idx, w, kc, meta, a.topk), a.iters)
    hbm, tf, tag = peaks()
    key_bytes = float(B) * (ctx + 1) * 128 * 2
    fl = 2.0 * B * G * (ctx + 1) * 128
    print(f"indexer B={B} ctx={ctx} G={G} topk={a.topk}: {ms:.4f} ms (scores + top-k)  keys {key_bytes / ms / 1e6:.0f} GB/s "
          f"({key_bytes / ms / 1e6 / hbm:.2f} {tag})  {fl / ms / 1e9:.1f} TFLOP/s", flush=True)
    _native.check_status(torch.device("cuda"))


def bench_mla_pre(a):
    """Fused MLA pre-process (latent norm + rope key + cache scatter + query rope), DeepSeek-V3 head geometry."""
    from vllm_ascend_b200.ops import reference as ref
    T, H, dn, dr, dc = a.tokens, a.heads, 128, 64, 512
    q = torch.randn(T, H, dn + dr, device="cuda").bfloat16()
    kv = torch.randn(T, dc + dr, device="cuda").bfloat16()
    w = torch.ones(dc, device="cuda").bfloat16()
    pos = torch.arange(T, device="cuda") % 4096
    cs = ref.build_cos_sin_cache(dr, 8192, 1e4, None, torch.device("cuda"))
    nb = (T + 127) // 128 + 1
    lat = torch.zeros(nb, 128, 1, dc, device="cuda", dtype=torch.bfloat16)
    pe = torch.zeros(nb, 128, 1, dr, device="cuda", dtype=torch.bfloat16)
    slots = torch.arange(T, device="cuda") + 128
    hbm, tf, tag = peaks()
    ms = timeit(lambda: ops.mla_preprocess(q, kv, w, 1e-6, pos, cs, slots, lat, pe, dn, dr), a.iters)
    by = T * (2.0 * H * dr * 2 + (dc + dr) * 2 * 2)
    print(f"mla preprocess T={T} H={H}: {ms:.4f} ms  {by / ms / 1e6:.0f} GB/s of touched bytes "
          f"({by / ms / 1e6 / hbm:.2f} {tag})", flush=True)
    _native.check_status(torch.device("cuda"))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("what", choices=["gemm", "gemm-fp8", "gemm-folded", "attn-decode", "attn-prefill", "mla-decode", "gdn",
                                     "norm", "rope", "sampler", "moe", "kv-copy", "quant", "moe-route", "mla-pre", "indexer", "all"])
    ap.add_argument("--topk", type=int, default=8)
    ap.add_argument("--l2-prefetch", type=int, default=0,
                    help="paired-CTA GEMM: k-blocks the L2 prefetch runs ahead (0 = off)")
    ap.add_argument("--vocab", type=int, default=151936)
    ap.add_argument("--experts", type=int, default=128)
    ap.add_argument("--blocks", type=int, default=2048)
    ap.add_argument("--m", type=int, default=8192)
    ap.add_argument("--n", type=int, default=4096)
    ap.add_argument("--k", type=int, default=4096)
    ap.add_argument("--bn", type=int, default=0)
    ap.add_argument("--raster", type=int, default=0, help="M-tiles per raster group of the paired-CTA GEMM")
    ap.add_argument("--compare", action="store_true")
    ap.add_argument("--no-flush", action="store_true", help="gemm: leave the operands in L2 between timed launches")
    ap.add_argument("--tile-n", type=int, default=0, help="paired-CTA GEMM: fixed tile width (128..256 step 16)")
    ap.add_argument("--batch", type=int, default=256)
    ap.add_argument("--ctx", type=int, default=1152)
    ap.add_argument("--seq", type=int, default=1024)
    ap.add_argument("--hq", type=int, default=32)
    ap.add_argument("--hkv", type=int, default=8)
    ap.add_argument("--d", type=int, default=128)
    ap.add_argument("--heads", type=int, default=128)
    ap.add_argument("--block-size", type=int, default=128)
    ap.add_argument("--splits", type=int, default=0)
    ap.add_argument("--impl", default="both")
    ap.add_argument("--tokens", type=int, default=8192)
    ap.add_argument("--hidden", type=int, default=4096)
    ap.add_argument("--inter", type=int, default=12288)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--kv-layout", default="HND", choices=["NHD", "HND"])
    ap.add_argument("--ragged", type=int, default=0, help="attn-decode: spread of the context lengths (+-tokens)")
    ap.add_argument("--interleave-gemm", type=int, default=0,
                    help="attn-decode: run this many large GEMMs (untimed) between the timed launches")
    a = ap.parse_args()
    if a.what in ("gemm", "all"):
        if a.what == "all":
            a.compare = True
            for (m, n, k) in [(8192, 6144, 4096), (8192, 4096, 4096), (8192, 24576, 4096),
                              (8192, 4096, 12288), (768, 6144, 4096), (768, 24576, 4096),
                              (768, 4096, 12288), (768, 151936, 4096)]:
                a.m, a.n, a.k = m, n, k
                bench_gemm(a)
        else:
            bench_gemm(a)
    if a.what == "quant":
        bench_quant(a)
    if a.what == "moe-route":
        bench_moe_route(a)
    if a.what == "mla-pre":
        bench_mla_pre(a)
    if a.what == "rope":
        bench_rope(a)
    if a.what == "sampler":
        bench_sampler(a)
    if a.what == "moe":
        bench_moe(a)
    if a.what == "kv-copy":
        bench_kv_copy(a)
    if a.what == "gemm-folded":
        bench_gemm_folded(a)
    if a.what in ("attn-decode", "all"):
        if a.what == "all":
            for b, c in [(768, 1152), (256, 1152), (32, 4096), (4, 32768)]:
                a.batch, a.ctx = b, c
                a.ctx = min(a.ctx, 8192) if b * c > 2_000_000 else a.ctx
                bench_attn_decode(a)
        else:
            bench_attn_decode(a)
    if a.what == "indexer":
        bench_indexer(a)
    if a.what == "gdn":
        bench_gdn(a)
    if a.what in ("attn-prefill", "all"):
        if a.what == "all":
            a.ctx = 0
            for b, s in [(8, 1024), (2, 4096), (1, 8192)]:
                a.batch, a.seq = b, s
                bench_attn_prefill(a)
        else:
            a.ctx = 0 if a.ctx == 1152 else a.ctx
            bench_attn_prefill(a)
    if a.what == "gemm-fp8":
        bench_gemm_fp8(a)
    if a.what == "mla-decode":
        bench_mla_decode(a)
    if a.what in ("norm", "all"):
        bench_norm(a)


if __name__ == "__main__":
    main()
