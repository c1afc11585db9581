"""Op entry points.  CUDA bf16 tensors go to the hand-written sm_100a kernels;
CPU (and non-bf16) tensors run the PyTorch restatement in ``reference``.

A CUDA bf16 tensor never falls back silently: if the native library is missing
the call raises.  The only library paths are explicit opt-outs through
``envs.VLLM_B200_GEMM`` / ``VLLM_B200_PREFILL_ATTN`` (kept for validation).

The op set corresponds to the reference's OOT custom-op table
(vllm_ascend/utils.py:703-732) and ``DeviceOperator`` routes
(vllm_ascend/device/device_op.py:43-965).
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import _native, envs
from . import reference as ref

_BF16 = torch.bfloat16

#: number of launches of this package's own kernels (bench.py reports it)
launch_counter = _native.launch_counter


def _use_native(t: torch.Tensor) -> bool:
    return t.is_cuda and t.dtype == _BF16


def kv_layout(cache: torch.Tensor) -> int:
    """Physical layout of a paged cache whose logical shape is [blocks, tokens, heads, D]:
    0 = stored in that order, 1 = stored as [blocks, heads, tokens, D] (each head's page is
    one contiguous run, which is what the per-head TMA page loads prefer)."""
    if cache.is_contiguous():
        return 0
    if cache.permute(0, 2, 1, 3).is_contiguous():
        return 1
    raise ValueError("unsupported KV-cache strides")


def alloc_kv_cache(num_blocks: int, block_size: int, heads: int, dim: int, dtype, device,
                   layout: str = "HND", arena=None) -> torch.Tensor:
    """Zero-filled cache with logical shape [blocks, tokens, heads, dim].  ``arena`` (an
    object with ``take(shape, dtype)`` returning zeroed storage) replaces the torch
    allocator, e.g. an IPC-exportable arena for disaggregated prefill."""
    hnd = layout == "HND" and heads > 1
    shape = (num_blocks, heads, block_size, dim) if hnd else (num_blocks, block_size, heads, dim)
    t = arena.take(shape, dtype) if arena is not None else torch.zeros(shape, dtype=dtype, device=device)
    return t.permute(0, 2, 1, 3) if hnd else t


# ---------------------------------------------------------------- norms / activations
def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float,
             residual: Optional[torch.Tensor] = None, gemma: bool = False,
             out: Optional[torch.Tensor] = None):
    """Returns (normed, residual_out).  With ``residual`` the sum x+residual is
    written back into ``residual`` (in place) — the fused add+RMSNorm of
    vllm_ascend/ops/layernorm.py:63-85."""
    if not _use_native(x):
        return ref.rms_norm(x, weight, eps, residual, gemma)
    H = x.shape[-1]
    x2 = x.reshape(-1, H) if x.stride(-1) == 1 else x.contiguous().view(-1, H)
    T = x2.shape[0]
    if out is None:
        out = torch.empty((T, H), dtype=x.dtype, device=x.device)
    if residual is not None:
        assert residual.is_contiguous()
    rc = _native.lib().b200_rms_norm(x2.data_ptr(), _native.ptr(residual), weight.data_ptr(),
                                     out.data_ptr(), T, H, eps, int(gemma), x2.stride(0),
                                     out.stride(0), _native.stream_ptr())
    _native.check(rc, "rms_norm")
    launch_counter[0] += 1
    return out.view(x.shape), residual


def layer_norm(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], eps: float) -> torch.Tensor:
    """LayerNorm over the last dimension (vision-tower blocks and mergers)."""
    H = x.shape[-1]
    if not _use_native(x) or H % 8 or H > 32768:
        return ref.layer_norm(x, weight, bias, eps)
    x2 = x.reshape(-1, H) if x.stride(-1) == 1 else x.contiguous().view(-1, H)
    if x2.stride(0) % 8:
        x2 = x2.contiguous()
    out = torch.empty((x2.shape[0], H), dtype=x.dtype, device=x.device)
    rc = _native.lib().b200_layer_norm(x2.data_ptr(), weight.data_ptr(), _native.ptr(bias), out.data_ptr(),
                                       x2.shape[0], H, eps, x2.stride(0), out.stride(0), _native.stream_ptr())
    _native.check(rc, "layer_norm")
    launch_counter[0] += 1
    return out.view(x.shape)


def silu_and_mul(x: torch.Tensor, limit: float = 0.0,
                 out: Optional[torch.Tensor] = None) -> torch.Tensor:
    if not _use_native(x):
        return ref.silu_and_mul(x, limit)
    I = x.shape[-1] // 2
    x2 = x.view(-1, 2 * I)
    T = x2.shape[0]
    if out is None:
        out = torch.empty((T, I), dtype=x.dtype, device=x.device)
    rc = _native.lib().b200_silu_and_mul(x2.data_ptr(), out.data_ptr(), T, I, limit,
                                         _native.stream_ptr())
    _native.check(rc, "silu_and_mul")
    launch_counter[0] += 1
    return out.view(*x.shape[:-1], I)


def embedding(ids: torch.Tensor, weight: torch.Tensor, vocab_start: int = 0,
              vocab_end: Optional[int] = None, out: Optional[torch.Tensor] = None):
    if vocab_end is None:
        vocab_end = vocab_start + weight.shape[0]
    if not _use_native(weight):
        return ref.embedding(ids, weight, vocab_start, vocab_end)
    T, H = ids.numel(), weight.shape[1]
    if out is None:
        out = torch.empty((T, H), dtype=weight.dtype, device=weight.device)
    ids = ids.to(torch.int64)
    rc = _native.lib().b200_embedding(ids.data_ptr(), weight.data_ptr(), out.data_ptr(), T, H,
                                      vocab_start, vocab_end, _native.stream_ptr())
    _native.check(rc, "embedding")
    launch_counter[0] += 1
    return out


def qknorm_rope_kvwrite(qkv: torch.Tensor, positions: torch.Tensor, cos_sin: torch.Tensor,
                        rot_dim: int, q_norm_w, k_norm_w, eps: float,
                        k_cache: Optional[torch.Tensor], v_cache: Optional[torch.Tensor],
                        slot_mapping: Optional[torch.Tensor], Hq: int, Hkv: int, D: int,
                        mrope_axis: Optional[torch.Tensor] = None) -> None:
    """Split-QKV + per-head q/k RMSNorm + neox RoPE + paged KV-cache write, one pass, in place.
    With ``mrope_axis`` (int32 [rot_dim/2]) positions is [3, N] and each rotary pair follows the
    temporal / height / width position its table entry names (multimodal rotary embedding)."""
    native_ok = (_use_native(qkv) and D in (32, 64, 96, 128, 256) and rot_dim <= D
                 and (rot_dim == 0 or (rot_dim // 2) % 32 == 0)
                 and (k_cache is None or k_cache.dtype == _BF16))
    if not native_ok:
        if qkv.is_cuda and qkv.dtype == _BF16 and D in (64, 128):
            raise RuntimeError("qknorm_rope_kvwrite: unsupported rotary shape for the native kernel")
        return ref.qknorm_rope_kvwrite(qkv, positions, cos_sin, rot_dim, q_norm_w, k_norm_w, eps,
                                       k_cache, v_cache, slot_mapping, Hq, Hkv, D, mrope_axis)
    T = qkv.shape[0]
    num_slots = 0 if k_cache is None else k_cache.shape[0] * k_cache.shape[1]
    if mrope_axis is not None:
        rc = _native.lib().b200_qknorm_mrope_kvwrite(
            qkv.data_ptr(), qkv.stride(0), positions.data_ptr(), positions.stride(0),
            mrope_axis.data_ptr(), cos_sin.data_ptr(), rot_dim,
            _native.ptr(q_norm_w), _native.ptr(k_norm_w), eps, _native.ptr(k_cache),
            _native.ptr(v_cache), _native.ptr(slot_mapping), T, Hq, Hkv, D, num_slots,
            0 if k_cache is None else k_cache.shape[1], 0 if k_cache is None else kv_layout(k_cache),
            _native.status_word(qkv.device).data_ptr(), _native.stream_ptr())
        _native.check(rc, "qknorm_mrope_kvwrite")
        launch_counter[0] += 1
        return
    rc = _native.lib().b200_qknorm_rope_kvwrite(
        qkv.data_ptr(), qkv.stride(0), positions.data_ptr(), cos_sin.data_ptr(), rot_dim,
        _native.ptr(q_norm_w), _native.ptr(k_norm_w), eps, _native.ptr(k_cache),
        _native.ptr(v_cache), _native.ptr(slot_mapping), T, Hq, Hkv, D, num_slots,
        0 if k_cache is None else k_cache.shape[1], 0 if k_cache is None else kv_layout(k_cache),
        _native.status_word(qkv.device).data_ptr(), _native.stream_ptr())
    _native.check(rc, "qknorm_rope_kvwrite")
    launch_counter[0] += 1


# ---------------------------------------------------------------- GEMM
def linear(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None,
           residual: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None,
           bn: int = 0) -> torch.Tensor:
    """y = x @ weight.T (+bias) (+residual).  x [..., K], weight [N, K]."""
    K = x.shape[-1]
    N = weight.shape[0]
    if (not _use_native(x)) or weight.dtype != _BF16:
        y = torch.nn.functional.linear(x, weight.to(x.dtype), bias)
        if residual is not None:
            y = y + residual
        return y
    x2 = x.reshape(-1, K)
    if x2.stride(-1) != 1 or (x2.stride(0) % 8) != 0:
        x2 = x2.contiguous()
    M = x2.shape[0]
    if envs.VLLM_B200_GEMM == "cublas" or (K % 8) or (N % 8):
        y = torch.nn.functional.linear(x2, weight, bias)
        if residual is not None:
            y = y + residual.view(M, N)
        return y.view(*x.shape[:-1], N)
    if out is None:
        out = torch.empty((M, N), dtype=x.dtype, device=x.device)
    if M == 0:
        return out.view(*x.shape[:-1], N)
    res2 = None
    if residual is not None:
        res2 = residual.view(M, N)
        assert res2.stride(0) == out.stride(0) and res2.stride(1) == 1
    min2 = envs.VLLM_B200_GEMM_2CTA_MIN_M
    if bn == 512 or (bn == 0 and min2 > 0 and M >= min2 and N >= 256):
        # paired-CTA kernel: 256 x 256 tiles issued with tcgen05 cta_group::2
        rc = _native.lib().b200_gemm_bf16_2cta(
            x2.data_ptr(), weight.data_ptr(), out.data_ptr(), _native.ptr(bias),
            _native.ptr(res2), M, N, K, x2.stride(0), weight.stride(0), out.stride(0), 0,
            _native.status_word(x.device).data_ptr(), _native.stream_ptr())
    else:
        rc = _native.lib().b200_gemm_bf16(
            x2.data_ptr(), weight.data_ptr(), out.data_ptr(), _native.ptr(bias), _native.ptr(res2),
            M, N, K, x2.stride(0), weight.stride(0), out.stride(0), bn,
            _native.status_word(x.device).data_ptr(), 0, _native.stream_ptr())
    _native.check(rc, "gemm_bf16")
    launch_counter[0] += 1
    return out.view(*x.shape[:-1], N)


def alloc_row_stats(rows: int, max_out_features: int, device) -> torch.Tensor:
    """Row-statistics buffer of the folded-norm GEMMs: fp32 [parts][rows] partial sums of squares
    (one part per 128 output columns at most) followed by the int32 part count."""
    parts = (max_out_features + 127) // 128
    buf = torch.zeros(parts * rows + 4, dtype=torch.float32, device=device)
    buf.stats_rows, buf.stats_parts = rows, parts          # geometry travels with the tensor
    return buf


def linear_norm_folded(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None,
                       residual: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None,
                       swiglu: bool = False, ss_in: Optional[torch.Tensor] = None, norm_dim: int = 0,
                       eps: float = 1e-6, ss_out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Paired-CTA GEMM with the RMSNorm around it folded in (CUDA, bf16, x [M, K] with M >= 1).

    ``ss_in`` / ``ss_out`` are buffers of ``alloc_row_stats`` (same geometry).  ``ss_in`` holds the
    partial sums of squares of x's rows: the result rows are scaled by rsqrt(sum / norm_dim + eps),
    i.e. the GEMM runs on the un-normalised rows and ``weight`` already carries the norm weight.
    ``ss_out`` receives, per column tile, the sum of squares of every stored output row (the
    statistics of the NEXT norm).  Partials are summed in a fixed order: a step repeats bit for bit.
    ``residual`` may alias ``out``."""
    M, K = x.shape
    N = weight.shape[0] // 2 if swiglu else weight.shape[0]
    if weight.dim() != 2 or weight.shape[1] != K or N == 0 or not weight.is_cuda:
        raise ValueError(f"weight {tuple(weight.shape)} on {weight.device} does not fit rows of {K} columns "
                         "(offloaded or unloaded layer?)")
    rows = parts = 0
    for name, t in (("ss_in", ss_in), ("ss_out", ss_out)):
        if t is None:
            continue
        r_, p_ = getattr(t, "stats_rows", 0), getattr(t, "stats_parts", 0)
        if t.dtype != torch.float32 or r_ < M or p_ < 1 or t.numel() < r_ * p_ + 1 or (rows and (r_, p_) != (rows, parts)):
            raise ValueError(f"{name} must be a row-statistics buffer (alloc_row_stats) of at least {M} rows")
        rows, parts = r_, p_
    if ss_out is not None and parts * 128 < N:
        raise ValueError(f"row-statistics buffer has {parts} parts; {N} output columns need {(N + 127) // 128}")
    if out is None:
        out = torch.empty((M, N), dtype=x.dtype, device=x.device)
    rc = _native.lib().b200_gemm_bf16_2cta_norm(
        x.data_ptr(), weight.data_ptr(), out.data_ptr(), _native.ptr(bias), _native.ptr(residual), M, N, K,
        x.stride(0), weight.stride(0), out.stride(0), int(swiglu), _native.ptr(ss_in), int(norm_dim), float(eps),
        _native.ptr(ss_out), rows, parts, _native.status_word(x.device).data_ptr(), _native.stream_ptr())
    _native.check(rc, "gemm_2cta_norm")
    launch_counter[0] += 1
    return out


def linear_swiglu(x: torch.Tensor, weight: torch.Tensor, out: Optional[torch.Tensor] = None,
                  two_cta: bool = False) -> torch.Tensor:
    """silu(x @ Wg^T) * (x @ Wu^T) with weight = [Wg; Wu] ([2I, K]) in one GEMM: the tile pairs
    128 gate columns with the matching 128 up columns and the epilogue applies SiLU-mul
    (the reference fuses the same pair in its grouped-matmul+swiglu op, csrc/gmm)."""
    I = weight.shape[0] // 2
    K = x.shape[-1]
    if not (_use_native(x) and weight.dtype == _BF16 and I % 128 == 0 and K % 8 == 0
            and envs.VLLM_B200_GEMM != "cublas"):
        return silu_and_mul(linear(x, weight))
    x2 = x.reshape(-1, K)
    if x2.stride(-1) != 1 or (x2.stride(0) % 8) != 0:
        x2 = x2.contiguous()
    M = x2.shape[0]
    if out is None:
        out = torch.empty((M, I), dtype=x.dtype, device=x.device)
    min2 = envs.VLLM_B200_GEMM_2CTA_MIN_M
    if M > 0 and (two_cta or (min2 > 0 and M >= min2)):
        rc = _native.lib().b200_gemm_bf16_2cta(
            x2.data_ptr(), weight.data_ptr(), out.data_ptr(), None, None, M, I, K, x2.stride(0),
            weight.stride(0), out.stride(0), 1, _native.status_word(x.device).data_ptr(),
            _native.stream_ptr())
        _native.check(rc, "gemm_swiglu_2cta")
        launch_counter[0] += 1
    elif M > 0:
        rc = _native.lib().b200_gemm_swiglu_bf16(
            x2.data_ptr(), weight.data_ptr(), out.data_ptr(), M, I, K, x2.stride(0),
            weight.stride(0), out.stride(0), _native.status_word(x.device).data_ptr(),
            _native.stream_ptr())
        _native.check(rc, "gemm_swiglu")
        launch_counter[0] += 1
    return out.view(*x.shape[:-1], I)


# ---------------------------------------------------------------- attention
_scratch: dict = {}


def _get_scratch(device, nbytes: int) -> torch.Tensor:
    """Grow-only per-device scratch (split-KV partials)."""
    key = (device.type, device.index)
    buf = _scratch.get(key)
    if buf is None or buf.numel() < nbytes:
        buf = torch.empty(max(nbytes, 1 << 20), dtype=torch.uint8, device=device)
        _scratch[key] = buf
    return buf


def reserve_attention_scratch(device, nbytes: int) -> None:
    """Pre-size the split-KV scratch (must happen before CUDA-graph capture)."""
    _get_scratch(torch.device(device), nbytes)


def paged_attention_tc(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, meta,
                       scale: float, out: torch.Tensor, causal: bool = True, window: int = 0,
                       num_splits: int = 1, rescale_threshold: float = 8.0,
                       v_lbo: int = 0, v_sbo: int = 0) -> torch.Tensor:
    """tcgen05 kernel over all query tokens of the batch (prefill, decode or mixed)."""
    T, Hq, D = q.shape
    NB, BS, Hkv, _ = k_cache.shape
    G = Hq // Hkv
    if meta.tile_seq is None and meta.max_query_len > 128 // G:
        raise ValueError("attention work list required when a sequence has more than 128/G query tokens")
    num_tiles = meta.num_tiles if meta.tile_seq is not None else meta.num_reqs
    scratch = None
    if num_splits > 1:
        nbytes = T * Hq * num_splits * (D + 1) * 4
        scratch = _get_scratch(q.device, nbytes)
    rc = _native.lib().b200_attn_fwd_tc(
        q.data_ptr(), q.stride(0), T, k_cache.data_ptr(), v_cache.data_ptr(), NB, BS,
        meta.query_start_loc.data_ptr(), meta.seq_lens.data_ptr(), meta.block_table.data_ptr(),
        meta.block_table.stride(0), _native.ptr(meta.tile_seq), _native.ptr(meta.tile_qoff),
        num_tiles, Hq, Hkv, D, scale, int(causal), int(window), num_splits, out.data_ptr(),
        out.stride(0), _native.ptr(scratch), rescale_threshold, v_lbo, v_sbo, kv_layout(k_cache),
        _native.status_word(q.device).data_ptr(), _native.stream_ptr())
    _native.check(rc, "attn_fwd_tc")
    launch_counter[0] += 1 + (1 if num_splits > 1 else 0)
    return out


_dec_prefetch_set = None


def paged_attention_decode_tc(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, meta,
                              scale: float, out: torch.Tensor, window: int = 0,
                              num_splits: int = 1, num_seqs: Optional[int] = None,
                              timeline: Optional[torch.Tensor] = None, max_q_len: int = 0,
                              lse_out: Optional[torch.Tensor] = None,
                              seq_lens: Optional[torch.Tensor] = None) -> torch.Tensor:
    """tcgen05 flash-decode (keys on the MMA M axis): the first ``num_seqs`` sequences of the
    batch, each with at most 16/G query tokens; ``q``/``out`` hold exactly their tokens.
    ``lse_out`` (fp32 [T, Hq]) receives the log-sum-exp over the keys seen, ``seq_lens`` replaces
    the metadata's lengths (a context-parallel rank attends over the keys it stores)."""
    T, Hq, D = q.shape
    if num_seqs is None:
        num_seqs = meta.num_reqs
    NB, BS, Hkv, _ = k_cache.shape
    global _dec_prefetch_set
    if _dec_prefetch_set != envs.VLLM_B200_DECODE_L2_PREFETCH:
        _dec_prefetch_set = envs.VLLM_B200_DECODE_L2_PREFETCH
        _native.lib().b200_attn_decode_set_l2_prefetch(int(_dec_prefetch_set))
    scratch = None
    if num_splits > 1:
        scratch = _get_scratch(q.device, T * Hq * num_splits * (D + 1) * 4)
    if lse_out is not None and (lse_out.dtype != torch.float32 or lse_out.numel() < T * Hq
                                or not lse_out.is_contiguous()):
        raise ValueError("lse_out must be a contiguous fp32 tensor of T x Hq elements")
    sl = meta.seq_lens if seq_lens is None else seq_lens
    rc = _native.lib().b200_attn_decode_tc_lse(
        q.data_ptr(), q.stride(0), T, k_cache.data_ptr(), v_cache.data_ptr(), NB, BS,
        meta.query_start_loc.data_ptr(), sl.data_ptr(), meta.block_table.data_ptr(),
        meta.block_table.stride(0), num_seqs, Hq, Hkv, D, scale, int(window), num_splits,
        max_q_len if max_q_len else min(meta.max_query_len, 16 // (Hq // Hkv)), out.data_ptr(),
        out.stride(0), _native.ptr(scratch), kv_layout(k_cache), _native.ptr(lse_out),
        _native.status_word(q.device).data_ptr(), _native.ptr(timeline), _native.stream_ptr())
    _native.check(rc, "attn_decode_tc")
    launch_counter[0] += 1 + (1 if num_splits > 1 else 0)
    return out


def merge_attn_partials(partial_o: torch.Tensor, partial_lse: torch.Tensor, out: Optional[torch.Tensor] = None,
                        lse_out: Optional[torch.Tensor] = None, out_dtype=None) -> torch.Tensor:
    """partial_o fp32 [T, H, S, D] (each normalised over its own keys), partial_lse fp32 [T, H, S] ->
    [T, H, D]: the attention result over the union of the S key sets."""
    T, H, S, D = partial_o.shape
    if not partial_o.is_cuda:
        m = partial_lse.max(dim=-1, keepdim=True).values.clamp(min=-1e30)
        w = torch.exp(partial_lse - m)
        w = torch.where(torch.isfinite(partial_lse), w, torch.zeros_like(w))
        den = w.sum(-1)
        res = (partial_o * w.unsqueeze(-1)).sum(2) / den.clamp(min=1e-30).unsqueeze(-1)
        if lse_out is not None:
            lse_out.copy_(torch.where(den > 0, m.squeeze(-1) + torch.log(den.clamp(min=1e-30)),
                                      torch.full_like(den, float("-inf"))))
        res = res.to(out_dtype or partial_o.dtype)
        if out is not None:
            out.copy_(res)
            return out
        return res
    if out is None:
        out = torch.empty((T, H, D), dtype=_BF16, device=partial_o.device)
    if not (partial_o.is_contiguous() and partial_lse.is_contiguous() and partial_lse.dtype == torch.float32
            and out.dtype == _BF16 and out.stride(2) == 1 and out.stride(1) == D):
        raise ValueError("merge_attn_partials takes contiguous fp32 partials and a bf16 [T, H, D] output")
    rc = _native.lib().b200_merge_attn_partials(partial_o.data_ptr(), partial_lse.data_ptr(), T, H, S, D,
                                                out.data_ptr(), out.stride(0), _native.ptr(lse_out),
                                                _native.stream_ptr())
    _native.check(rc, "merge_attn_partials")
    launch_counter[0] += 1
    return out


def paged_decode(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                 block_table: torch.Tensor, seq_lens: torch.Tensor, scale: float,
                 out: torch.Tensor, window: int = 0, num_splits: int = 1) -> torch.Tensor:
    """CUDA-core flash-decode: one query token per sequence (q [B, Hq, D])."""
    B, Hq, D = q.shape
    NB, BS, Hkv, _ = k_cache.shape
    if kv_layout(k_cache) != 0:
        raise ValueError("the CUDA-core decode kernel reads [blocks, tokens, heads, D] caches only")
    scratch = None
    if num_splits > 1:
        scratch = _get_scratch(q.device, B * Hq * num_splits * (D + 1) * 4)
    rc = _native.lib().b200_paged_decode(
        q.data_ptr(), q.stride(0), k_cache.data_ptr(), v_cache.data_ptr(), block_table.data_ptr(),
        block_table.stride(0), seq_lens.data_ptr(), B, Hq, Hkv, D, BS, scale, int(window),
        num_splits, out.data_ptr(), out.stride(0), _native.ptr(scratch), NB,
        _native.status_word(q.device).data_ptr(), _native.stream_ptr())
    _native.check(rc, "paged_decode")
    launch_counter[0] += 1 + (1 if num_splits > 1 else 0)
    return out


def choose_num_splits(num_seqs: int, Hkv: int, max_seq_len: int, sm_count: int = 148,
                      tile: int = 128) -> int:
    """Split-KV factor: enough CTAs to fill the GPU, never more splits than KV tiles.  In
    batch-invariant mode the factor is 1: the merge order must not depend on the batch."""
    from ..batch_invariant import is_batch_invariant
    if is_batch_invariant():
        return 1
    ctas = max(1, num_seqs * Hkv)
    if ctas >= 2 * sm_count:
        return 1
    want = (2 * sm_count + ctas - 1) // ctas
    max_tiles = max(1, (max_seq_len + tile - 1) // tile)
    return max(1, min(want, max_tiles, 32))


def paged_attention_consistent(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, meta,
                               scale: float, out: torch.Tensor) -> torch.Tensor:
    """Every batch shape through the tile kernel with one KV split (training-consistent mode)."""
    if not _use_native(q):
        return ref.paged_attention(q, k_cache, v_cache, meta.query_start_loc_cpu, meta.seq_lens_cpu,
                                   meta.block_table, scale, True, 0, out=out)
    T, Hq, D = q.shape
    G = Hq // k_cache.shape[2]
    if D not in (64, 128) or 128 % G:
        raise RuntimeError("training-consistent attention needs head_dim 64 or 128 and a group size dividing 128")
    if meta.tile_seq is None and meta.max_query_len > 128 // G:
        raise RuntimeError("training-consistent attention needs the tile work list for long queries")
    nd = meta.num_decodes
    if meta.tile_seq is not None and nd > 0:
        # the work list of a mixed step covers the prefill sequences; decodes get their own launch of
        # the same kernel (tile i = sequence i)
        import copy
        dm = copy.copy(meta)
        dm.tile_seq = dm.tile_qoff = None
        dm.num_reqs, dm.max_query_len = nd, 1
        paged_attention_tc(q, k_cache, v_cache, dm, scale, out, True, 0, 1)
        if meta.num_tiles > 0:
            paged_attention_tc(q, k_cache, v_cache, meta, scale, out, True, 0, 1)
        return out
    return paged_attention_tc(q, k_cache, v_cache, meta, scale, out, True, 0, 1)


def paged_attention(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, meta,
                    scale: float, out: Optional[torch.Tensor] = None, causal: bool = True,
                    window: int = 0) -> torch.Tensor:
    """Attention of every scheduled token over its sequence's paged KV."""
    T, Hq, D = q.shape
    if out is None:
        out = torch.empty((T, Hq, v_cache.shape[-1]), dtype=q.dtype, device=q.device)
    from ..attention.backend import training_consistent_attention
    if training_consistent_attention() and causal and window == 0:
        return paged_attention_consistent(q, k_cache, v_cache, meta, scale, out)
    if not _use_native(q):
        return ref.paged_attention(q, k_cache, v_cache, meta.query_start_loc_cpu,
                                   meta.seq_lens_cpu, meta.block_table, scale, causal, window,
                                   out=out)
    Hkv = k_cache.shape[2]
    G = Hq // Hkv
    is_decode = meta.max_query_len == 1
    tc_ok = D in (64, 128) and 128 % G == 0 and v_cache.shape[-1] == D
    mode = envs.VLLM_B200_DECODE_ATTN
    dec_ok = (mode == "native" and D == 128 and 16 % G == 0 and causal
              and v_cache.shape[-1] == D)
    if dec_ok and meta.max_query_len <= 16 // G:
        return paged_attention_decode_tc(q, k_cache, v_cache, meta, scale, out, window,
                                         num_splits=meta.num_splits if is_decode else 1)
    if (dec_ok and tc_ok and meta.num_decodes > 0 and meta.tile_seq is not None
            and envs.VLLM_B200_PREFILL_ATTN == "tcgen05"):
        # mixed batch: the leading decode sequences stream their KV through the decode
        # kernel, the work list of the prefill kernel covers the remaining sequences
        nd, ndt = meta.num_decodes, meta.num_decode_tokens
        paged_attention_decode_tc(q[:ndt], k_cache, v_cache, meta, scale, out[:ndt], window,
                                  num_splits=1, num_seqs=nd, max_q_len=1)
        if meta.num_tiles > 0:
            paged_attention_tc(q, k_cache, v_cache, meta, scale, out, causal, window)
        return out
    if is_decode:
        if mode == "tcgen05" and tc_ok:
            return paged_attention_tc(q, k_cache, v_cache, meta, scale, out, causal, window,
                                      num_splits=meta.num_splits)
        if D in (64, 128) and G in (1, 2, 4, 8) and k_cache.is_contiguous():
            return paged_decode(q, k_cache, v_cache, meta.block_table, meta.seq_lens, scale, out,
                                window, num_splits=meta.num_splits)
        if tc_ok:
            return paged_attention_tc(q, k_cache, v_cache, meta, scale, out, causal, window,
                                      num_splits=meta.num_splits)
    if envs.VLLM_B200_PREFILL_ATTN == "tcgen05" and tc_ok:
        return paged_attention_tc(q, k_cache, v_cache, meta, scale, out, causal, window)
    # explicit opt-out: PyTorch path (validation only)
    return ref.paged_attention(q, k_cache, v_cache, meta.query_start_loc_cpu, meta.seq_lens_cpu,
                               meta.block_table, scale, causal, window, out=out)


def mla_preprocess(q: torch.Tensor, kv: torch.Tensor, norm_w: torch.Tensor, eps: float, positions: torch.Tensor,
                   cos_sin: torch.Tensor, slot_mapping: Optional[torch.Tensor], lat_cache: Optional[torch.Tensor],
                   pe_cache: Optional[torch.Tensor], dn: int, dr: int, want_outputs: bool = False):
    """Fused MLA pre-processing: RMSNorm of the latent part of ``kv`` [T, dc + dr] and interleaved RoPE
    of its rope part, both scattered into their paged caches at ``slot_mapping`` (slot < 0: skipped);
    interleaved RoPE of the last ``dr`` columns of every head of ``q`` [T, H, dn + dr] in place.
    Returns (latent [T, dc], k_pe [T, dr]) when ``want_outputs`` else None."""
    T, H, D = q.shape
    dc = kv.shape[1] - dr
    native = (_use_native(q) and kv.dtype == _BF16 and q.stride(2) == 1 and q.stride(1) == D and kv.stride(1) == 1
              and cos_sin.dtype == torch.float32 and cos_sin.shape[1] == dr and dn % 2 == 0 and dr % 2 == 0
              and q.stride(0) % 2 == 0
              and (lat_cache is None or (lat_cache.dtype == _BF16 and lat_cache.is_contiguous()
                                         and pe_cache.is_contiguous())))
    if not native:
        latent = ref.rms_norm(kv[:, :dc].contiguous(), norm_w, eps)[0]
        k_pe = ref.apply_rope_interleaved(kv[:, dc:].reshape(T, 1, dr), positions, cos_sin, dr).view(T, dr)
        q[..., dn:] = ref.apply_rope_interleaved(q[..., dn:], positions, cos_sin, dr)
        if slot_mapping is not None and lat_cache is not None:
            valid = (slot_mapping >= 0).unsqueeze(-1)
            idx = slot_mapping.clamp(min=0)
            lf, pf_ = lat_cache.view(-1, dc), pe_cache.view(-1, dr)
            lf.index_copy_(0, idx, torch.where(valid, latent.to(lf.dtype), lf[idx]))
            pf_.index_copy_(0, idx, torch.where(valid, k_pe.to(pf_.dtype), pf_[idx]))
        return (latent, k_pe) if want_outputs else None
    latent = torch.empty((T, dc), dtype=q.dtype, device=q.device) if want_outputs else None
    k_pe = torch.empty((T, dr), dtype=q.dtype, device=q.device) if want_outputs else None
    num_slots = 0 if lat_cache is None else lat_cache.numel() // dc
    use_slots = slot_mapping is not None and lat_cache is not None
    rc = _native.lib().b200_mla_preprocess(
        q.data_ptr(), q.stride(0), T, H, dn, dr, kv.data_ptr(), kv.stride(0), dc, norm_w.data_ptr(), float(eps),
        positions.data_ptr(), cos_sin.data_ptr(), cos_sin.shape[0], _native.ptr(slot_mapping) if use_slots else None,
        _native.ptr(lat_cache), _native.ptr(pe_cache), num_slots, _native.ptr(latent), _native.ptr(k_pe),
        _native.status_word(q.device).data_ptr(), _native.stream_ptr())
    _native.check(rc, "mla_preprocess")
    launch_counter[0] += 1
    return (latent, k_pe) if want_outputs else None


# ---------------------------------------------------------------- sampling
def argmax(logits: torch.Tensor) -> torch.Tensor:
    if not logits.is_cuda or logits.dtype not in (_BF16, torch.float32):
        return logits.argmax(dim=-1)
    B, V = logits.shape
    out = torch.empty(B, dtype=torch.int64, device=logits.device)
    rc = _native.lib().b200_argmax(logits.data_ptr(), 0 if logits.dtype == _BF16 else 1,
                                   logits.stride(0), B, V, out.data_ptr(), _native.stream_ptr())
    _native.check(rc, "argmax")
    launch_counter[0] += 1
    return out


def to_float_logits(logits: torch.Tensor) -> torch.Tensor:
    if logits.dtype == torch.float32:
        return logits
    if not (logits.is_cuda and logits.dtype == _BF16):
        return logits.float()
    B, V = logits.shape
    out = torch.empty((B, V), dtype=torch.float32, device=logits.device)
    rc = _native.lib().b200_cast_bf16_f32(logits.data_ptr(), logits.stride(0), out.data_ptr(),
                                          out.stride(0), B, V, _native.stream_ptr())
    _native.check(rc, "cast")
    launch_counter[0] += 1
    return out


def apply_penalties(logits: torch.Tensor, prompt_ids, output_ids, rep, freq, pres) -> torch.Tensor:
    """fp32 logits [B, V], in place on CUDA."""
    if not logits.is_cuda:
        return ref.apply_penalties(logits, prompt_ids, output_ids, rep, freq, pres)
    B, V = logits.shape
    rc = _native.lib().b200_apply_penalties(
        logits.data_ptr(), logits.stride(0), B, V, prompt_ids.data_ptr(), prompt_ids.shape[1],
        output_ids.data_ptr(), output_ids.shape[1], rep.data_ptr(), freq.data_ptr(),
        pres.data_ptr(), _native.stream_ptr())
    _native.check(rc, "apply_penalties")
    launch_counter[0] += 1
    return logits


def sample(logits_f32: torch.Tensor, temperature, top_k, top_p, min_p=None, seeds=None,
           offsets=None, generator=None) -> torch.Tensor:
    """Top-k/top-p/min-p + exponential-race sampling (destroys ``logits_f32`` on CUDA)."""
    if not logits_f32.is_cuda:
        return ref.sample(logits_f32, temperature, top_k.to(torch.int64), top_p, min_p, generator, seeds, offsets)
    B, V = logits_f32.shape
    out = torch.empty(B, dtype=torch.int64, device=logits_f32.device)
    rc = _native.lib().b200_sample(
        logits_f32.data_ptr(), logits_f32.stride(0), B, V, _native.ptr(temperature),
        _native.ptr(top_k), _native.ptr(top_p), _native.ptr(min_p), _native.ptr(seeds),
        _native.ptr(offsets), out.data_ptr(), _native.stream_ptr())
    _native.check(rc, "sample")
    launch_counter[0] += 1
    return out


def quant_fp8_group128(x: torch.Tensor, pow2_scale: bool = False):
    if not _use_native(x):
        return ref.quant_fp8_group128(x, pow2_scale)
    T, H = x.shape
    q = torch.empty((T, H), dtype=torch.float8_e4m3fn, device=x.device)
    s = torch.empty((T, H // 128), dtype=torch.float32, device=x.device)
    rc = _native.lib().b200_quant_fp8_group128(x.data_ptr(), q.data_ptr(), s.data_ptr(), T, H,
                                               int(pow2_scale), _native.stream_ptr())
    _native.check(rc, "quant_fp8_group128")
    launch_counter[0] += 1
    return q, s


def quant_fp8_per_token(x: torch.Tensor):
    """[T, H] -> (e4m3 [T, H], scale [T] fp32 = row amax / 448): the dynamic per-token activation
    quantisation of the per-channel W8A8 schemes."""
    if not _use_native(x) or x.shape[-1] % 8:
        return ref.quant_fp8_per_token(x)
    if x.stride(-1) != 1 or x.stride(0) % 8:
        x = x.contiguous()
    T, H = x.shape
    q = torch.empty((T, H), dtype=torch.float8_e4m3fn, device=x.device)
    s = torch.empty((T,), dtype=torch.float32, device=x.device)
    rc = _native.lib().b200_quant_fp8_per_token(x.data_ptr(), x.stride(0), q.data_ptr(), s.data_ptr(), T, H,
                                                _native.stream_ptr())
    _native.check(rc, "quant_fp8_per_token")
    launch_counter[0] += 1
    return q, s


class QuantAct:
    """A block-scaled fp8 activation: values [T, H] e4m3 and scales [T, H / 128] fp32, produced by
    a fused norm / activation kernel and consumed by the fp8 GEMM without an extra quant pass."""
    __slots__ = ("q", "scales", "shape", "dtype")

    def __init__(self, q: torch.Tensor, scales: torch.Tensor, dtype=torch.bfloat16):
        self.q, self.scales, self.shape, self.dtype = q, scales, q.shape, dtype

    def dequant(self) -> torch.Tensor:
        T, H = self.q.shape
        return (self.q.float().view(T, H // 128, 128) * self.scales.unsqueeze(-1)).view(T, H).to(self.dtype)


def rms_norm_quant_fp8(x: torch.Tensor, weight: torch.Tensor, eps: float,
                       residual: Optional[torch.Tensor] = None, gemma: bool = False):
    """Fused (add +) RMSNorm + 1x128 fp8 quantisation.  Returns (QuantAct, residual_out)."""
    H = x.shape[-1]
    if not _use_native(x) or H % 128:
        y, res = rms_norm(x, weight, eps, residual, gemma)
        return QuantAct(*quant_fp8_group128(y.reshape(-1, H)), dtype=x.dtype), res
    x2 = x.reshape(-1, H) if x.stride(-1) == 1 else x.contiguous().view(-1, H)
    T = x2.shape[0]
    q = torch.empty((T, H), dtype=torch.float8_e4m3fn, device=x.device)
    s = torch.empty((T, H // 128), dtype=torch.float32, device=x.device)
    if residual is not None:
        assert residual.is_contiguous()
    rc = _native.lib().b200_rms_norm_quant_fp8(x2.data_ptr(), _native.ptr(residual), weight.data_ptr(), q.data_ptr(),
                                               s.data_ptr(), T, H, eps, int(gemma), x2.stride(0), _native.stream_ptr())
    _native.check(rc, "rms_norm_quant_fp8")
    launch_counter[0] += 1
    return QuantAct(q, s, x.dtype), (residual if residual is not None else x)


def silu_and_mul_quant_fp8(x: torch.Tensor, limit: float = 0.0) -> QuantAct:
    """Fused SiLU(gate) * up + 1x128 fp8 quantisation of [T, 2I] -> QuantAct [T, I]."""
    I = x.shape[-1] // 2
    if not _use_native(x) or I % 128 or not x.is_contiguous():
        y = silu_and_mul(x) if limit <= 0 else ref.silu_and_mul(x, limit)
        return QuantAct(*quant_fp8_group128(y.reshape(-1, I)), dtype=x.dtype)
    x2 = x.view(-1, 2 * I)
    T = x2.shape[0]
    q = torch.empty((T, I), dtype=torch.float8_e4m3fn, device=x.device)
    s = torch.empty((T, I // 128), dtype=torch.float32, device=x.device)
    rc = _native.lib().b200_silu_mul_quant_fp8(x2.data_ptr(), q.data_ptr(), s.data_ptr(), T, I, limit,
                                               _native.stream_ptr())
    _native.check(rc, "silu_mul_quant_fp8")
    launch_counter[0] += 1
    return QuantAct(q, s, x.dtype)


_ACT_KINDS = {"gelu": 1, "gelu_tanh": 2, "quick_gelu": 3, "swiglu_oai": 4}


def activation(x: torch.Tensor, kind: str, gated: bool = False, alpha: float = 1.702, limit: float = 7.0):
    """GELU (erf / tanh), QuickGELU, and the clamped "swiglu-oai" gate; ``gated`` inputs are [gate | up]."""
    I = x.shape[-1] // 2 if gated else x.shape[-1]
    if not _use_native(x) or I % 8 or not x.is_contiguous():
        return ref.activation(x, kind, gated, alpha, limit)
    x2 = x.view(-1, x.shape[-1])
    out = torch.empty((x2.shape[0], I), dtype=x.dtype, device=x.device)
    rc = _native.lib().b200_activation(x2.data_ptr(), out.data_ptr(), x2.shape[0], I, _ACT_KINDS[kind], int(gated),
                                       alpha, limit, _native.stream_ptr())
    _native.check(rc, "activation")
    launch_counter[0] += 1
    return out.view(*x.shape[:-1], I)


def rms_norm_gated(x: torch.Tensor, z: torch.Tensor, weight: torch.Tensor, eps: float, group: int = 0,
                   norm_before_gate: bool = True) -> torch.Tensor:
    """Gated RMSNorm of linear-attention blocks: rmsnorm(x) * w * silu(z), per ``group`` columns."""
    H = x.shape[-1]
    g = group or H
    if not _use_native(x) or not (x.is_contiguous() and z.is_contiguous()) or H % g:
        return ref.rms_norm_gated(x, z, weight, eps, group, norm_before_gate)
    out = torch.empty_like(x)
    rows = x.numel() // g
    rc = _native.lib().b200_rms_norm_gated(x.data_ptr(), z.data_ptr(), weight.data_ptr(), out.data_ptr(), rows, g,
                                           eps, int(norm_before_gate), _native.stream_ptr())
    _native.check(rc, "rms_norm_gated")
    launch_counter[0] += 1
    return out
