"""Tensor parallelism with the collectives fused into the GEMMs.

Instead of ``row-parallel GEMM -> all-reduce`` the decoder runs with a
sequence-sharded residual stream:

    o_proj / down_proj  : GEMM -> reduce-scatter, the GEMM epilogue stores bf16 partial
                          rows straight into the owning rank's staging buffer (NVLink)
    add + RMSNorm       : the owner sums the partials, adds its residual shard,
                          normalises and pushes the rows into every peer's gather buffer
    qkv / gate_up / head: all-gather -> GEMM, the TMA producer waits for each source
                          rank's epoch flag and starts with the locally produced rows

which is the reference's ``MLPColumnParallelOp`` / ``MLPRowParallelOp`` dataflow
(vllm_ascend/ops/linear_op.py:152-191) and its matmul+reduce-scatter fusion
(vllm_ascend/device/device_op.py:164-190) with the transfers issued from inside the
kernels.  All flags are epochs in peer-mapped memory; waits are bounded and a
timeout surfaces as a Python exception after the step.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from .. import _native, ops
from ..ops import launch_counter
from .state import GroupCoordinator
from .symm_mem import SymmetricMemory


class FusedTPContext:
    def __init__(self, group: GroupCoordinator, device: torch.device, max_tokens: int, hidden: int):
        self.group = group
        self.n = group.world_size
        self.rank = group.rank_in_group
        self.device = device
        self.H = hidden
        self.max_rows_local = (max_tokens + self.n - 1) // self.n
        self.max_tokens = self.max_rows_local * self.n
        nbytes = self.max_tokens * hidden * 2
        from .. import envs
        mode = envs.VLLM_B200_NVLS
        if mode == "auto" and self.n > envs.VLLM_B200_NVLS_AUTO_MAX_RANKS:
            mode = "0"          # group sizes the multicast path has not been validated on use peer stores
        self.symm = SymmetricMemory(group, device, 2 * nbytes + 4096, multicast=mode != "0")
        self.off_ag = self.symm.region(nbytes)
        self.off_rs = self.symm.region(nbytes)
        # NVSwitch multicast (NVLS).  "push" (the default where multicast exists): the all-gather push
        # of the normalised rows is one multimem.st per 16 bytes, replicated by the switch, so a rank
        # sends 1 x instead of (N-1) x its rows; the reduce-scatter stays in the GEMM epilogue, where
        # the peer stores overlap the tensor-core work.  "full": the partial sums stay in every
        # rank's own buffer and the owner sums them inside the switch (multimem.ld_reduce); that
        # moves the reduce-scatter traffic out of the GEMM into the (exposed) reduce kernel and
        # measured slower at TP2 (17.7k vs 18.1k tok/s on the Qwen3-8B workload).
        self.nvls = self.symm.mc_ptr != 0 and mode != "0"
        self.nvls_full = self.nvls and mode == "full"
        self.mc_ag = self.symm.mc_ptr + self.off_ag if self.nvls else 0
        self.mc_rs = self.symm.mc_ptr + self.off_rs if self.nvls else 0
        self.ag_ptrs = self.symm.ptr_array(self.off_ag)
        self.rs_ptrs = self.symm.ptr_array(self.off_rs)
        self.ctl_ptrs = self.symm.ctl_ptrs
        self.ag_local = self.symm.tensor(self.off_ag, (self.max_tokens, hidden), torch.bfloat16)
        self.rs_local_ptr = self.symm.local_ptr + self.off_rs
        self.residual = torch.zeros((self.max_rows_local, hidden), dtype=torch.bfloat16, device=device)
        self.status = _native.status_word(device)
        self.rows_local = 0
        self.T = 0

    # ------------------------------------------------------------------
    def begin(self, num_tokens: int) -> tuple[int, int]:
        """Fix the shard geometry of this forward pass: returns (padded tokens, rows per rank)."""
        self.rows_local = (num_tokens + self.n - 1) // self.n
        self.T = self.rows_local * self.n
        assert self.T <= self.max_tokens
        return self.T, self.rows_local

    def norm_push(self, weight: torch.Tensor, eps: float, first: bool = False,
                  skip_norm: bool = False) -> None:
        """first=True : residual holds the embedding rows -> normalise and push.
        first=False: sum the peers' GEMM partials, add the residual shard, normalise, push."""
        lib = _native.lib()
        rl = self.rows_local
        if self.nvls_full:
            rc = lib.b200_nvls_reduce_add_norm_push(
                None if first else self.mc_rs, 0 if first else 1, self.residual.data_ptr() if first else None,
                None if first else self.residual.data_ptr(), weight.data_ptr(), eps, self.mc_ag, self.ctl_ptrs,
                rl, self.H, self.rank, self.n, int(skip_norm), _native.stream_ptr())
            _native.check(rc, "nvls_reduce_add_norm_push")
            launch_counter[0] += 1
            return
        mc = self.mc_ag if self.nvls else None
        if first:
            rc = lib.b200_reduce_add_norm_push_mc(None, 0, self.residual.data_ptr(), None,
                                                  weight.data_ptr(), eps, self.ag_ptrs, self.ctl_ptrs,
                                                  rl, self.H, self.rank, self.n, int(skip_norm), mc,
                                                  _native.stream_ptr())
        else:
            rc = lib.b200_reduce_add_norm_push_mc(self.rs_local_ptr, self.n, None,
                                                  self.residual.data_ptr(), weight.data_ptr(), eps,
                                                  self.ag_ptrs, self.ctl_ptrs, rl, self.H, self.rank,
                                                  self.n, int(skip_norm), mc, _native.stream_ptr())
        _native.check(rc, "reduce_add_norm_push")
        launch_counter[0] += 1

    def _two_cta(self, n_cols: int) -> bool:
        """The paired-CTA kernel (256 x 256 tiles) pays off from a few hundred rows on."""
        from .. import envs
        m = envs.VLLM_B200_GEMM_2CTA_MIN_M
        return m > 0 and self.T >= m and n_cols >= 256

    def ag_gemm(self, weight: torch.Tensor, bias: Optional[torch.Tensor] = None,
                swiglu: bool = False) -> torch.Tensor:
        """[T, N_local] = gathered normalised hidden [T, H] @ weight^T; with ``swiglu`` the weight
        is [gate; up] and the result is silu(gate) * up ([T, N_local / 2])."""
        N = weight.shape[0] // 2 if swiglu else weight.shape[0]
        out = torch.empty((self.T, N), dtype=torch.bfloat16, device=self.device)
        if self._two_cta(N) and (not swiglu or N % 128 == 0):
            rc = _native.lib().b200_gemm_ag_bf16_2cta(
                self.ag_local.data_ptr(), weight.data_ptr(), out.data_ptr(), _native.ptr(bias),
                self.T, N, self.H, self.H, weight.stride(0), N, self.symm.local_ptr, self.rank, self.n,
                self.rows_local, int(swiglu), self.status.data_ptr(), _native.stream_ptr())
            _native.check(rc, "gemm_ag_2cta")
            launch_counter[0] += 1
            return out
        if swiglu:
            from .. import ops
            return ops.silu_and_mul(self.ag_gemm(weight, bias))
        rc = _native.lib().b200_gemm_ag_bf16(
            self.ag_local.data_ptr(), weight.data_ptr(), out.data_ptr(), _native.ptr(bias),
            self.T, N, self.H, self.H, weight.stride(0), N, self.symm.local_ptr, self.rank, self.n,
            self.rows_local, 0, self.status.data_ptr(), _native.stream_ptr())
        _native.check(rc, "gemm_ag")
        launch_counter[0] += 1
        return out

    def gemm_rs(self, x: torch.Tensor, weight: torch.Tensor,
                bias: Optional[torch.Tensor] = None) -> None:
        """x [T, K_local] @ weight^T -> partial rows stored into their owners' staging."""
        assert x.shape[0] == self.T and weight.shape[0] == self.H
        b = _native.ptr(bias) if self.rank == 0 else None
        if self.nvls_full:
            # the partial rows stay in this rank's own (multicast-bound) buffer; peers learn that
            # they are complete and sum them inside the switch
            if self._two_cta(self.H):
                rc = _native.lib().b200_gemm_pub_bf16_2cta(
                    x.data_ptr(), weight.data_ptr(), self.rs_local_ptr, b, self.T, self.H, x.shape[1], x.stride(0),
                    weight.stride(0), self.H, self.ctl_ptrs, self.rank, self.n, self.status.data_ptr(),
                    _native.stream_ptr())
            else:
                rc = _native.lib().b200_gemm_pub_bf16(
                    x.data_ptr(), weight.data_ptr(), self.rs_local_ptr, b, self.T, self.H, x.shape[1], x.stride(0),
                    weight.stride(0), self.H, self.ctl_ptrs, self.rank, self.n, 0, self.status.data_ptr(),
                    _native.stream_ptr())
            _native.check(rc, "gemm_pub")
            launch_counter[0] += 1
            return
        if self._two_cta(self.H):
            rc = _native.lib().b200_gemm_rs_bf16_2cta(
                x.data_ptr(), weight.data_ptr(), b, self.T, self.H, x.shape[1], x.stride(0), weight.stride(0),
                self.rs_ptrs, self.ctl_ptrs, self.rank, self.n, self.rows_local, self.status.data_ptr(),
                _native.stream_ptr())
            _native.check(rc, "gemm_rs_2cta")
        else:
            rc = _native.lib().b200_gemm_rs_bf16(
                x.data_ptr(), weight.data_ptr(), b, self.T, self.H, x.shape[1], x.stride(0), weight.stride(0),
                self.rs_ptrs, self.ctl_ptrs, self.rank, self.n, self.rows_local, 0, self.status.data_ptr(),
                _native.stream_ptr())
            _native.check(rc, "gemm_rs")
        launch_counter[0] += 1

    def gathered(self) -> torch.Tensor:
        """Waits for every rank's push of the current epoch; returns the [T, H] gather buffer."""
        rc = _native.lib().b200_ag_wait(self.symm.local_ptr, self.rank, self.n,
                                        _native.stream_ptr())
        _native.check(rc, "ag_wait")
        launch_counter[0] += 1
        return self.ag_local[:self.T]

    def check(self) -> None:
        st = self.symm.read_status()
        if st != 0:
            raise _native.NativeError(
                f"fused TP kernel reported status {_native.STATUS_NAMES.get(st, st)} "
                "(a peer did not signal within the wait budget)")


def forward_sp(model, ctx: FusedTPContext, input_ids: torch.Tensor, meta, kv_caches: list) -> torch.Tensor:
    """Forward pass of a dense GQA decoder with the sequence-sharded residual stream."""
    T = input_ids.shape[0]
    Tp, rl = ctx.begin(T)
    r = ctx.rank
    lo = min(r * rl, T)
    hi = min((r + 1) * rl, T)
    res = ctx.residual[:rl]
    if hi - lo < rl:
        res.zero_()
    if hi > lo:
        ops.embedding(input_ids[lo:hi], model.full_embedding, 0, model.full_embedding.shape[0],
                      out=res[:hi - lo])
    layers = model.layers
    ctx.norm_push(layers[0].input_layernorm.weight, layers[0].input_layernorm.eps, first=True)
    for i, layer in enumerate(layers):
        a = layer.self_attn
        qkv = ctx.ag_gemm(a.qkv_proj.weight, a.qkv_proj.bias)
        k_cache, v_cache = kv_caches[i]
        ops.qknorm_rope_kvwrite(qkv[:T], meta.positions, a.cos_sin, a.rot_dim, a.q_norm, a.k_norm,
                                a.cfg.rms_norm_eps, k_cache, v_cache, meta.slot_mapping, a.Hq,
                                a.Hkv, a.D)
        attn = torch.empty((Tp, a.Hq * a.D), dtype=qkv.dtype, device=qkv.device)
        if Tp > T:
            attn[T:].zero_()
        q = qkv[:T, :a.Hq * a.D].view(T, a.Hq, a.D)
        ops.paged_attention(q, k_cache, v_cache, meta, a.scale, out=attn[:T].view(T, a.Hq, a.D),
                            causal=True, window=a.window)
        ctx.gemm_rs(attn, a.o_proj.weight, a.o_proj.bias)
        ctx.norm_push(layer.post_attention_layernorm.weight, layer.post_attention_layernorm.eps)
        act = ctx.ag_gemm(layer.mlp.gate_up_proj.weight, swiglu=True)
        ctx.gemm_rs(act, layer.mlp.down_proj.weight)
        nxt = layers[i + 1].input_layernorm if i + 1 < len(layers) else model.norm
        ctx.norm_push(nxt.weight, nxt.eps)
        if model.layer_hook is not None:
            model.layer_hook(i)
    return ctx.gathered()[:T]


def supports(model) -> bool:
    from ..models.layers import GQAAttention, SwiGLUMLP
    cfg = model.cfg
    return (not cfg.use_mla and not cfg.is_moe and model.dtype == torch.bfloat16
            and not cfg.mrope_section and not cfg.is_hybrid and cfg.embed_scale == 1.0
            and cfg.residual_multiplier == 1.0 and cfg.logits_scaling == 1.0 and not cfg.qk_norm_full
            and not cfg.deepnorm_factors and cfg.hc_mult <= 1 and cfg.pre_norm
            and cfg.hidden_act in ("silu", "swish") and not cfg.attn_output_gate and not cfg.sandwich_norm
            and cfg.partial_rotary_factor == 1.0
            and model.is_first and model.is_last
            and all(isinstance(L.self_attn, GQAAttention) and isinstance(L.mlp, SwiGLUMLP)
                    and L.self_attn.qkv_proj.quant is None for L in model.layers))


def attach(model, engine_cfg, device: torch.device) -> Optional[FusedTPContext]:
    """Switch a TP-sharded dense model to the fused sequence-parallel forward."""
    if not supports(model):
        return None
    comm = model.comm
    if comm.size <= 1:
        return None
    max_tokens = max(engine_cfg.scheduler.max_num_batched_tokens, engine_cfg.scheduler.max_num_seqs)
    ctx = FusedTPContext(comm.group, device, max_tokens + comm.size, model.cfg.hidden_size)
    # the residual stream is sharded by token, so every rank looks up its own rows in a
    # replicated embedding table (no collective for the embedding)
    emb = model.embed_tokens
    full = comm.all_gather(emb.weight, dim=0)[:model.cfg.vocab_size].contiguous()
    model.full_embedding = full
    model.sp_ctx = ctx
    return ctx


def calibrate(runner, group: GroupCoordinator) -> dict:
    """``VLLM_B200_TP_COMM=auto``: time one forward pass per step class (a full prefill chunk, a
    decode batch) with the fused peer-memory dataflow and with the NCCL all-reduce dataflow, take
    the maximum over the TP ranks, and keep the faster one for that class.  The choice is stored
    on the model (``sp_prefill`` / ``sp_decode``); a fused pass that raises keeps NCCL."""
    import torch.distributed as dist
    model = runner.model
    ctx = model.sp_ctx
    out = {}
    if ctx is None:
        return out
    classes = {"prefill": (min(8, runner.max_seqs), max(1, min(runner.max_tokens // min(8, runner.max_seqs),
                                                             runner.max_model_len - 1))),
               "decode": (min(256, runner.max_seqs), 1)}
    for name, (B, q) in classes.items():
        times = {}
        for path in ("fused", "nccl"):
            model.sp_ctx = ctx if path == "fused" else None
            try:
                meta, T, Tp, _, _ = runner._dummy_meta(B, q)
                meta.slot_mapping.fill_(-1)
                for _ in range(2):
                    runner._forward(Tp, meta)
                ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                ev0.record()
                for _ in range(3):
                    runner._forward(Tp, meta)
                ev1.record()
                torch.cuda.synchronize()
                if path == "fused":
                    ctx.check()
                t = torch.tensor([ev0.elapsed_time(ev1) / 3], dtype=torch.float64)
            except Exception as e:                      # keep serving on the NCCL path
                from ..logger import logger
                logger.warning("fused TP path failed during calibration (%s): using NCCL", e)
                t = torch.tensor([float("inf")], dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group.cpu_group)
            times[path] = float(t)
        model.sp_ctx = ctx
        out[name] = {"fused_ms": times["fused"], "nccl_ms": times["nccl"],
                     "choice": "fused" if times["fused"] <= times["nccl"] * 1.02 else "nccl"}
    model.sp_prefill = out["prefill"]["choice"] == "fused"
    model.sp_decode = out["decode"]["choice"] == "fused"
    return out
