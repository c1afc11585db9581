"""Paged attention kernels (tcgen05 unified kernel, CUDA-core decode) vs fp32 reference."""
import numpy as np
import pytest
import torch

from vllm_ascend_b200 import _native, ops
from vllm_ascend_b200.ops import reference as ref
from gpu_utils import make_paged_case

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _ref(q, kc, vc, meta, scale, causal=True, window=0):
    return ref.paged_attention(q.float().cpu(), kc.float().cpu(), vc.float().cpu(),
                               meta.query_start_loc_cpu, meta.seq_lens_cpu, meta.block_table.cpu(),
                               scale, causal, window)


def _run_tc(q, kc, vc, meta, scale, window=0, num_splits=1, thr=8.0):
    out = torch.full_like(q, float("nan"))
    ops.paged_attention_tc(q, kc, vc, meta, scale, out, True, window, num_splits, thr)
    torch.cuda.synchronize()
    _native.check_status(torch.device(DEV))
    return out


CASES = [
    # q_lens, ctx_lens, Hq, Hkv, D, block_size
    ([128], [0], 4, 4, 128, 128),                # one tile, MHA
    ([32], [0], 4, 1, 128, 128),                 # one packed-GQA tile
    ([200, 77, 1024], [0, 0, 0], 8, 2, 128, 128),  # varlen causal prefill
    ([64, 300], [500, 37], 8, 2, 128, 128),      # chunked prefill with context
    ([1, 1, 1, 1, 1], [5, 127, 128, 700, 1300], 8, 2, 128, 128),  # decode
    ([3, 2, 4], [100, 260, 9], 8, 2, 128, 128),  # spec-decode style short queries
    ([150, 90], [0, 40], 4, 2, 128, 16),         # small pages (several TMA loads per tile)
    ([150, 1], [10, 333], 4, 2, 64, 32),         # head_dim 64
    ([96], [64], 32, 8, 128, 256),               # pages larger than a tile
]


@pytest.mark.parametrize("layout", ["NHD", "HND"])
@pytest.mark.parametrize("case", CASES)
def test_attn_tc_matches_reference(case, layout):
    q_lens, ctx, Hq, Hkv, D, bs = case
    q, kc, vc, meta = make_paged_case(q_lens, ctx, Hq, Hkv, D, bs, seed=len(q_lens), layout=layout)
    scale = D ** -0.5
    out = _run_tc(q, kc, vc, meta, scale)
    exp = _ref(q, kc, vc, meta, scale)
    err = (out.float().cpu() - exp).abs().max().item()
    assert err < 2e-2, f"max abs err {err}"


def test_attn_tc_exact_rescale_and_lazy_rescale_agree():
    q, kc, vc, meta = make_paged_case([256, 64], [900, 0], 8, 2, 128, 128, seed=3)
    q = q * 4        # large score spread so the running max moves a lot
    scale = 128 ** -0.5
    exp = _ref(q, kc, vc, meta, scale)
    for thr in (0.0, 8.0):
        out = _run_tc(q, kc, vc, meta, scale, thr=thr)
        assert (out.float().cpu() - exp).abs().max().item() < 3e-2


def test_attn_tc_split_kv_decode():
    q, kc, vc, meta = make_paged_case([1] * 6, [40, 1000, 2047, 129, 3000, 5], 8, 2, 128, 128, seed=4)
    scale = 128 ** -0.5
    exp = _ref(q, kc, vc, meta, scale)
    for ns in (2, 4, 7):
        out = _run_tc(q, kc, vc, meta, scale, num_splits=ns)
        assert (out.float().cpu() - exp).abs().max().item() < 2e-2


def test_attn_tc_sliding_window():
    q, kc, vc, meta = make_paged_case([300, 1], [200, 700], 4, 2, 128, 128, seed=5)
    scale = 128 ** -0.5
    out = _run_tc(q, kc, vc, meta, scale, window=160)
    exp = _ref(q, kc, vc, meta, scale, window=160)
    assert (out.float().cpu() - exp).abs().max().item() < 2e-2


@pytest.mark.parametrize("Hq,Hkv,D,bs", [(32, 8, 128, 128), (8, 8, 128, 16), (16, 2, 64, 32), (4, 2, 128, 256)])
@pytest.mark.parametrize("ns", [1, 3])
def test_cuda_core_decode(Hq, Hkv, D, bs, ns):
    ctx = [0, 17, 128, 999, 2500]
    q, kc, vc, meta = make_paged_case([1] * len(ctx), ctx, Hq, Hkv, D, bs, seed=7)
    scale = D ** -0.5
    out = torch.full_like(q, float("nan"))
    ops.paged_decode(q, kc, vc, meta.block_table, meta.seq_lens, scale, out, 0, ns)
    torch.cuda.synchronize()
    _native.check_status(torch.device(DEV))
    exp = _ref(q, kc, vc, meta, scale)
    assert (out.float().cpu() - exp).abs().max().item() < 2e-2


DEC_CASES = [
    # q_lens, ctx_lens, Hq, Hkv, block_size
    ([1, 1, 1, 1, 1, 1], [0, 5, 127, 128, 700, 1300], 32, 8, 128),
    ([1, 1, 1], [31, 1000, 257], 8, 8, 16),          # MHA, small pages
    ([4, 2, 1, 3], [100, 260, 9, 1151], 8, 2, 128),  # spec-decode style (G=4: up to 4 tokens)
    ([2, 1], [500, 3], 64, 8, 256),                  # G=8: up to 2 tokens
    ([1, 1], [2000, 77], 16, 1, 128),                # G=16
]


@pytest.mark.parametrize("layout", ["NHD", "HND"])
@pytest.mark.parametrize("case", DEC_CASES)
@pytest.mark.parametrize("ns", [1, 3])
def test_attn_decode_tc(case, ns, layout):
    q_lens, ctx, Hq, Hkv, bs = case
    q, kc, vc, meta = make_paged_case(q_lens, ctx, Hq, Hkv, 128, bs, seed=11, layout=layout)
    scale = 128 ** -0.5
    out = torch.full_like(q, float("nan"))
    ops.paged_attention_decode_tc(q, kc, vc, meta, scale, out, 0, ns)
    torch.cuda.synchronize()
    _native.check_status(torch.device(DEV))
    exp = _ref(q, kc, vc, meta, scale)
    assert (out.float().cpu() - exp).abs().max().item() < 2e-2


def test_attn_decode_tc_sliding_window():
    q, kc, vc, meta = make_paged_case([1, 2, 1], [900, 300, 40], 8, 2, 128, 128, seed=12)
    scale = 128 ** -0.5
    out = torch.full_like(q, float("nan"))
    ops.paged_attention_decode_tc(q, kc, vc, meta, scale, out, 200, 1)
    torch.cuda.synchronize()
    exp = _ref(q, kc, vc, meta, scale, window=200)
    assert (out.float().cpu() - exp).abs().max().item() < 2e-2


def test_attn_decode_tc_large_score_spread_triggers_rescale():
    q, kc, vc, meta = make_paged_case([1, 2, 1], [1500, 700, 130], 8, 2, 128, 128, seed=13)
    q = q * 6          # running max jumps by far more than the lazy-rescale threshold
    scale = 128 ** -0.5
    out = torch.full_like(q, float("nan"))
    ops.paged_attention_decode_tc(q, kc, vc, meta, scale, out, 0, 1)
    torch.cuda.synchronize()
    _native.check_status(torch.device(DEV))
    exp = _ref(q, kc, vc, meta, scale)
    assert (out.float().cpu() - exp).abs().max().item() < 3e-2


def _lse_ref(q, kc, vc, meta, scale, lens):
    """fp32 log-sum-exp of the scaled scores of every (query token, head) over the first ``lens[b]``
    keys of its sequence, and the attention output over those keys."""
    T, Hq, D = q.shape
    Hkv = kc.shape[2]
    G = Hq // Hkv
    bs = kc.shape[1]
    lse = torch.full((T, Hq), float("-inf"))
    out = torch.zeros(T, Hq, D)
    kcf, vcf, bt = kc.float().cpu(), vc.float().cpu(), meta.block_table.cpu()
    for b in range(meta.num_reqs):
        n = int(lens[b])
        qs, qe = int(meta.query_start_loc_cpu[b]), int(meta.query_start_loc_cpu[b + 1])
        if n == 0 or qe == qs:
            continue
        nb = (n + bs - 1) // bs
        k = torch.cat([kcf[int(i)] for i in bt[b, :nb]])[:n].repeat_interleave(G, dim=1)
        v = torch.cat([vcf[int(i)] for i in bt[b, :nb]])[:n].repeat_interleave(G, dim=1)
        s = torch.einsum("qhd,khd->qhk", q[qs:qe].float().cpu(), k) * scale
        lse[qs:qe] = torch.logsumexp(s, -1)
        out[qs:qe] = torch.einsum("qhk,khd->qhd", s.softmax(-1), v)
    return out, lse


@pytest.mark.parametrize("ns", [1, 3])
def test_attn_decode_tc_returns_log_sum_exp_and_takes_local_lengths(ns):
    q, kc, vc, meta = make_paged_case([1, 1, 1, 1], [640, 5, 300, 1290], 16, 2, 128, 128, seed=21)
    scale = 128 ** -0.5
    # a context-parallel rank sees fewer keys than the sequence holds; one sequence has none here
    local = np.array([333, 0, 128, 700], dtype=np.int32)
    lens = torch.from_numpy(local).to(DEV)
    out = torch.full_like(q, float("nan"))
    lse = torch.full((q.shape[0], q.shape[1]), float("nan"), dtype=torch.float32, device=DEV)
    ops.paged_attention_decode_tc(q, kc, vc, meta, scale, out, 0, ns, max_q_len=1, lse_out=lse, seq_lens=lens)
    torch.cuda.synchronize()
    _native.check_status(torch.device(DEV))
    exp_o, exp_l = _lse_ref(q, kc, vc, meta, scale, local)
    assert torch.isinf(lse[1]).all() and (lse[1] < 0).all() and (out[1] == 0).all()
    keep = [0, 2, 3]
    assert (lse[keep].cpu() - exp_l[keep]).abs().max().item() < 2e-2
    assert (out.float().cpu() - exp_o).abs().max().item() < 2e-2


def test_partials_of_two_key_shards_merge_to_full_attention():
    """Two 'ranks' hold the even / odd keys of every sequence densely under the same block table
    (interleave 1): their decode results merged by log-sum-exp equal attention over all keys."""
    q, kc, vc, meta = make_paged_case([1, 1, 1], [1023, 37, 300], 8, 1, 128, 128, seed=22)
    scale = 128 ** -0.5
    T, Hq, D = q.shape
    bs = kc.shape[1]
    full = meta.seq_lens_cpu
    po = torch.empty(T, Hq, 2, D, dtype=torch.float32, device=DEV)
    pl = torch.empty(T, Hq, 2, dtype=torch.float32, device=DEV)
    bt = meta.block_table.cpu()
    for r in range(2):
        kr, vr = torch.zeros_like(kc), torch.zeros_like(vc)
        local = np.zeros(len(full), dtype=np.int32)
        for b, n in enumerate(full):
            nb = (int(n) + bs - 1) // bs
            ids = bt[b, :nb].long().to(DEV)
            ks = kc[ids].reshape(-1, *kc.shape[2:])[:int(n)][r::2]
            vs = vc[ids].reshape(-1, *vc.shape[2:])[:int(n)][r::2]
            local[b] = ks.shape[0]
            flat_k = kr[ids].reshape(-1, *kc.shape[2:])
            flat_v = vr[ids].reshape(-1, *vc.shape[2:])
            flat_k[:ks.shape[0]] = ks
            flat_v[:vs.shape[0]] = vs
            kr[ids] = flat_k.view(nb, bs, *kc.shape[2:])
            vr[ids] = flat_v.view(nb, bs, *vc.shape[2:])
        o = torch.empty_like(q)
        l = torch.empty(T, Hq, dtype=torch.float32, device=DEV)
        ops.paged_attention_decode_tc(q, kr, vr, meta, scale, o, 0, 1, max_q_len=1, lse_out=l,
                                      seq_lens=torch.from_numpy(local).to(DEV))
        po[:, :, r] = o.float()
        pl[:, :, r] = l
    merged_lse = torch.empty(T, Hq, dtype=torch.float32, device=DEV)
    merged = ops.merge_attn_partials(po, pl, lse_out=merged_lse)
    torch.cuda.synchronize()
    _native.check_status(torch.device(DEV))
    exp = _ref(q, kc, vc, meta, scale)
    assert (merged.float().cpu() - exp).abs().max().item() < 2e-2
    _, exp_l = _lse_ref(q, kc, vc, meta, scale, full)
    assert (merged_lse.cpu() - exp_l).abs().max().item() < 2e-2
    # the PyTorch definition of the merge agrees with the kernel
    host = ops.merge_attn_partials(po.cpu(), pl.cpu())
    assert (host - merged.float().cpu()).abs().max().item() < 1e-2
