"""Helpers shared by the GPU kernel tests."""
import numpy as np
import torch

from vllm_ascend_b200.attention.metadata import AttentionMetadata, build_tile_worklist


def make_paged_case(q_lens, ctx_lens, Hq, Hkv, D, block_size, device="cuda", seed=0,
                    dtype=torch.bfloat16, shuffle_blocks=True, tok_per_tile=None, layout="NHD"):
    """Random q + paged K/V caches for sequences with `ctx_lens[i]` cached tokens and
    `q_lens[i]` new query tokens (whose K/V are already in the cache)."""
    g = torch.Generator(device="cpu").manual_seed(seed)
    q_lens = np.asarray(q_lens, dtype=np.int32)
    seq_lens = q_lens + np.asarray(ctx_lens, dtype=np.int32)
    B = len(q_lens)
    T = int(q_lens.sum())
    nblk_per = (seq_lens + block_size - 1) // block_size
    total = int(nblk_per.sum()) + 1
    perm = torch.randperm(total - 1, generator=g) + 1 if shuffle_blocks else torch.arange(1, total)
    max_blocks = int(nblk_per.max()) + 1
    bt = torch.zeros(B, max_blocks, dtype=torch.int32)
    o = 0
    for b in range(B):
        n = int(nblk_per[b])
        bt[b, :n] = perm[o:o + n].to(torch.int32)
        o += n
    k_cache = (torch.randn(total, block_size, Hkv, D, generator=g) * 0.5).to(dtype)
    v_cache = (torch.randn(total, block_size, Hkv, D, generator=g) * 0.5).to(dtype)
    q = (torch.randn(T, Hq, D, generator=g) * 0.5).to(dtype)
    cu = np.zeros(B + 1, dtype=np.int32)
    np.cumsum(q_lens, out=cu[1:])
    meta = AttentionMetadata(
        num_reqs=B, num_actual_tokens=T, max_query_len=int(q_lens.max()),
        max_seq_len=int(seq_lens.max()),
        query_start_loc=torch.from_numpy(cu).to(device), seq_lens=torch.from_numpy(seq_lens).to(device),
        block_table=bt.to(device), slot_mapping=torch.zeros(T, dtype=torch.int64, device=device),
        positions=torch.zeros(T, dtype=torch.int64, device=device),
        query_start_loc_cpu=cu, seq_lens_cpu=seq_lens)
    if tok_per_tile is None:
        tok_per_tile = 128 // (Hq // Hkv)
    if int(q_lens.max()) > tok_per_tile or True:
        ts, tq = build_tile_worklist(q_lens, tok_per_tile, seq_lens)
        meta.tile_seq = torch.from_numpy(ts).to(device)
        meta.tile_qoff = torch.from_numpy(tq).to(device)
        meta.num_tiles = len(ts)
    k_cache, v_cache = k_cache.to(device), v_cache.to(device)
    if layout == "HND":      # same logical tensor, heads-major physical order
        k_cache = k_cache.permute(0, 2, 1, 3).contiguous().permute(0, 2, 1, 3)
        v_cache = v_cache.permute(0, 2, 1, 3).contiguous().permute(0, 2, 1, 3)
    return q.to(device), k_cache, v_cache, meta


def rel_err(a: torch.Tensor, b: torch.Tensor) -> float:
    a, b = a.float(), b.float()
    return float((a - b).abs().max() / b.abs().max().clamp_min(1e-6))
