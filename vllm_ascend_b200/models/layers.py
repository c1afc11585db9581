"""Building blocks shared by every decoder family: TP-sharded linears, norms,
rotary tables, the paged GQA attention layer and the SwiGLU MLP.

Parity notes: the linear classes mirror the reference's per-layer communication
group selection (vllm_ascend/ops/linear.py:114-575, ops/linear_op.py:152-357):
column-parallel layers may all-gather their input and row-parallel layers end in
all-reduce or reduce-scatter, chosen by the layer's ``TPComm``.
"""
from __future__ import annotations

import hashlib
import math
from typing import Optional

import torch

from .. import ops
from ..config import ModelConfig
from ..ops import reference as ref
from ..parallel import state as pstate


# ---------------------------------------------------------------- parameters
class ParamFactory:
    """Creates (shards of) parameters.  Random init is seeded per parameter name so
    every TP rank slices the same full tensor; small tensors are drawn on the CPU so
    CPU and GPU instances of a test model hold identical weights."""

    def __init__(self, cfg: ModelConfig, device: torch.device, dtype: torch.dtype):
        self.cfg, self.device, self.dtype = cfg, device, dtype
        self.meta_only = False

    def _gen(self, name: str, dev) -> torch.Generator:
        h = int.from_bytes(hashlib.sha256(f"{self.cfg.seed}:{name}".encode()).digest()[:7], "little")
        g = torch.Generator(device=dev)
        g.manual_seed(h)
        return g

    def normal(self, name: str, shape, shard_dim: Optional[int] = None, shard_rank: int = 0,
               shard_world: int = 1, std: Optional[float] = None, dtype=None) -> torch.Tensor:
        std = self.cfg.init_std if std is None else std
        dtype = dtype or self.dtype
        numel = math.prod(shape)
        dev = torch.device("cpu") if numel <= (1 << 26) else self.device
        full = torch.empty(shape, dtype=torch.float32 if dev.type == "cpu" else dtype, device=dev)
        full.normal_(0.0, std, generator=self._gen(name, dev))
        if shard_dim is not None and shard_world > 1:
            size = shape[shard_dim] // shard_world
            full = full.narrow(shard_dim, shard_rank * size, size)
        return full.to(device=self.device, dtype=dtype).contiguous()

    def ones(self, shape, dtype=None) -> torch.Tensor:
        return torch.ones(shape, dtype=dtype or self.dtype, device=self.device)

    def zeros(self, shape, dtype=None) -> torch.Tensor:
        return torch.zeros(shape, dtype=dtype or self.dtype, device=self.device)


# ---------------------------------------------------------------- TP communication
class TPComm:
    """Collective that follows a row-parallel GEMM / precedes a column-parallel one.

    ``mode``: "allreduce" (upstream default), or "sp" — sequence-parallel residual
    stream where row-parallel ends in reduce-scatter and column-parallel starts with
    all-gather (the reference's MLP/O-proj fine-grained TP ops).  The fused
    GEMM+collective kernels plug in through ``parallel.fused_linear``.
    """

    def __init__(self, group: Optional[pstate.GroupCoordinator] = None, mode: str = "allreduce"):
        self.group = group or pstate.get_tp_group()
        self.mode = mode
        self.fused = None          # set by parallel.fused_linear.attach()

    @property
    def size(self) -> int:
        return self.group.world_size

    @property
    def rank(self) -> int:
        return self.group.rank_in_group

    def all_reduce(self, t: torch.Tensor) -> torch.Tensor:
        if self.size == 1:
            return t
        if self.fused is not None and t.is_cuda:
            return self.fused.all_reduce(t)
        return self.group.all_reduce(t)

    def all_gather(self, t: torch.Tensor, dim: int = 0) -> torch.Tensor:
        return self.group.all_gather(t, dim)

    def reduce_scatter(self, t: torch.Tensor, dim: int = 0) -> torch.Tensor:
        return self.group.reduce_scatter(t, dim)


# ---------------------------------------------------------------- linear layers
class Linear:
    """y = x W^T (+b).  ``weight`` is [N_local, K_local]."""

    def __init__(self, weight: torch.Tensor, bias: Optional[torch.Tensor] = None, name: str = ""):
        self.weight = weight
        self.bias = bias
        self.name = name
        self.quant = None           # quantization.LinearMethod or None
        self.lora = None            # lora.manager.LoRALayerState or None

    def _lora_on(self) -> bool:
        return self.lora is not None and self.lora.punica.any_active

    def __call__(self, x: torch.Tensor, residual: Optional[torch.Tensor] = None) -> torch.Tensor:
        if self.quant is not None:
            y = self.quant.apply(self, x, residual)
        else:
            if isinstance(x, ops.QuantAct):
                x = x.dequant()
            y = ops.linear(x, self.weight, self.bias, residual)
        if self._lora_on():
            y = self.lora.apply(x, y)
        return y

    def named_tensors(self):
        yield "weight", self.weight
        if self.bias is not None:
            yield "bias", self.bias
        if self.quant is not None:
            yield from self.quant.named_tensors(self)


class ColumnParallelLinear(Linear):
    """Output dim sharded over TP.  ``output_sizes`` lists merged sub-matrices
    (qkv, gate_up) so checkpoint shards land in the right rows."""

    def __init__(self, pf: ParamFactory, name: str, in_size: int, output_sizes: list[int],
                 comm: TPComm, bias: bool = False, gather_output: bool = False):
        tp, r = comm.size, comm.rank
        parts = [pf.normal(f"{name}.{i}", (n, in_size), 0, r, tp) for i, n in enumerate(output_sizes)]
        w = torch.cat(parts, dim=0) if len(parts) > 1 else parts[0]
        b = pf.zeros((w.shape[0],)) if bias else None
        super().__init__(w, b, name)
        self.comm = comm
        self.output_sizes = output_sizes
        self.local_sizes = [n // tp for n in output_sizes]
        self.gather_output = gather_output

    def __call__(self, x, residual=None):
        y = super().__call__(x, residual)
        if self.gather_output and self.comm.size > 1:
            y = self.comm.all_gather(y, dim=-1)
        return y


class RowParallelLinear(Linear):
    """Input dim sharded over TP; the partial sums are reduced by ``comm``."""

    def __init__(self, pf: ParamFactory, name: str, in_size: int, out_size: int, comm: TPComm,
                 bias: bool = False, reduce_results: bool = True):
        w = pf.normal(name, (out_size, in_size), 1, comm.rank, comm.size)
        b = pf.zeros((out_size,)) if bias else None
        super().__init__(w, b, name)
        self.comm = comm
        self.reduce_results = reduce_results

    def __call__(self, x, residual=None):
        if self.comm.size == 1:
            return super().__call__(x, residual)
        # residual/bias must be added once, not per rank
        if self.quant is not None:
            y = self.quant.apply(self, x, None, skip_bias=self.comm.rank != 0)
        else:
            y = ops.linear(x, self.weight, self.bias if self.comm.rank == 0 else None)
        if self._lora_on():         # partial delta of this rank's input shard, reduced with y
            y = self.lora.apply(x, y)
        if self.reduce_results:
            y = self.comm.all_reduce(y)
        if residual is not None:
            y = y + residual
        return y


class RMSNorm:
    def __init__(self, pf: ParamFactory, size: int, eps: float, gemma: bool = False):
        self.weight = pf.ones((size,))
        self.eps = eps
        self.gemma = gemma

    def __call__(self, x, residual=None, quant_out: bool = False):
        """With ``quant_out`` the normalised activations come back as block-scaled fp8
        (``ops.QuantAct``) from one fused kernel, for a consumer that is an fp8 GEMM."""
        if residual is not None and not _plan().enabled("add_rmsnorm"):
            # the sequence the fused kernel replaces: add, then normalise
            residual = x + residual
            x, _ = (ops.rms_norm_quant_fp8 if quant_out else ops.rms_norm)(residual, self.weight, self.eps, None, self.gemma)
            return x, residual
        if quant_out:
            return ops.rms_norm_quant_fp8(x, self.weight, self.eps, residual, self.gemma)
        return ops.rms_norm(x, self.weight, self.eps, residual, self.gemma)


def wants_quant_act(linear) -> bool:
    """True when ``linear`` can consume fp8 activations produced by a fused kernel."""
    q = getattr(linear, "quant", None)
    return bool(q is not None and getattr(q, "accepts_quant_act", False) and linear.weight.is_cuda
                and getattr(linear, "lora", None) is None)


class VocabParallelEmbedding:
    """Vocab sharded over TP, masked lookup + all-reduce
    (vllm_ascend/ops/vocab_parallel_embedding.py:229-257)."""

    def __init__(self, pf: ParamFactory, name: str, vocab: int, hidden: int, comm: TPComm):
        self.comm = comm
        self.vocab = vocab
        pad = (-vocab) % (comm.size * 8)
        self.padded_vocab = vocab + pad
        self.shard = self.padded_vocab // comm.size
        self.start = comm.rank * self.shard
        full_rows = min(max(vocab - self.start, 0), self.shard)
        w = pf.zeros((self.shard, hidden))
        if full_rows > 0:
            src = pf.normal(name, (self.padded_vocab, hidden), 0, comm.rank, comm.size)
            w[:full_rows] = src[:full_rows]
        self.weight = w

    def __call__(self, ids: torch.Tensor) -> torch.Tensor:
        out = ops.embedding(ids, self.weight, self.start, self.start + self.shard)
        if self.comm.size > 1:
            out = self.comm.all_reduce(out)
        return out


class ParallelLMHead:
    """Logits = hidden @ W^T with the vocab sharded over TP and gathered."""

    def __init__(self, embed: VocabParallelEmbedding, weight: Optional[torch.Tensor] = None):
        self.embed = embed
        self.weight = weight if weight is not None else embed.weight
        self.comm = embed.comm

    def __call__(self, hidden: torch.Tensor) -> torch.Tensor:
        logits = ops.linear(hidden, self.weight)
        if self.comm.size > 1:
            logits = self.comm.all_gather(logits, dim=-1)
        return logits[..., :self.embed.vocab]

    def greedy_tokens(self, hidden: torch.Tensor) -> torch.Tensor:
        """Arg-max over the full vocabulary without gathering the logits: every rank reduces its
        own vocabulary shard to (max value, index) and only those pairs are all-gathered — the
        "reduce sample" path of vllm_ascend/sample/sampler.py:87-107, 168-204."""
        logits = ops.linear(hidden, self.weight)                       # [B, V / tp]
        n, r = self.comm.size, self.comm.rank
        shard = logits.shape[-1]
        first = r * shard
        if first + shard > self.embed.vocab:                           # padded tail of the last shard
            logits = logits.clone()
            logits[:, max(self.embed.vocab - first, 0):] = float("-inf")
        idx = ops.argmax(logits)
        val = logits.float().gather(1, idx.view(-1, 1)).squeeze(1)
        if n == 1:
            return idx
        pair = torch.stack([val, (idx + first).to(torch.float32)], dim=1)          # ids < 2^24: exact in fp32
        allp = self.comm.all_gather(pair.contiguous(), dim=0).view(n, -1, 2)       # [tp, B, 2]
        vals, ids = allp[..., 0], allp[..., 1]
        best = vals.max(dim=0, keepdim=True).values
        # ties resolve to the lowest index, as a single arg-max over the whole row would
        cand = torch.where(vals == best, ids, torch.full_like(ids, float("inf")))
        return cand.min(dim=0).values.to(torch.int64)


# ---------------------------------------------------------------- rotary tables
_ROPE_CACHE: dict = {}


def get_cos_sin_cache(rot_dim: int, max_pos: int, theta: float, scaling, device) -> torch.Tensor:
    key = (rot_dim, max_pos, theta, str(scaling), str(device))
    t = _ROPE_CACHE.get(key)
    if t is None:
        t = ref.build_cos_sin_cache(rot_dim, max_pos, theta, scaling, device)
        _ROPE_CACHE[key] = t
    return t


# ---------------------------------------------------------------- attention + MLP
def _plan():
    from ..compilation.fusion import get_plan
    return get_plan()


class GQAAttention:
    """qkv proj -> fused (q/k RMSNorm + RoPE + paged KV write) -> paged attention -> o proj."""

    def __init__(self, pf: ParamFactory, cfg: ModelConfig, layer_idx: int, comm: TPComm,
                 max_pos: int):
        self.cfg = cfg
        self.layer_idx = layer_idx
        tp = comm.size
        self.D = cfg.head_dim
        self.Hq = cfg.num_attention_heads // tp
        self.total_kv = cfg.num_key_value_heads
        # kv heads are replicated when there are fewer of them than TP ranks
        self.Hkv = max(1, self.total_kv // tp)
        prefix = f"model.layers.{layer_idx}.self_attn"
        kv_out = self.total_kv * self.D if self.total_kv >= tp else tp * self.D
        self.kv_replicas = 1 if self.total_kv >= tp else tp // self.total_kv
        self.out_gate = bool(cfg.attn_output_gate)
        sizes = [cfg.num_attention_heads * self.D, kv_out, kv_out]
        if self.out_gate:       # [q | k | v | gate]: the fused rope / cache-write kernel still sees q, k, v first
            sizes.append(cfg.num_attention_heads * self.D)
        self.qkv_proj = ColumnParallelLinear(pf, f"{prefix}.qkv_proj", cfg.hidden_size, sizes, comm,
                                             bias=cfg.attention_bias)
        if self.kv_replicas > 1 and self.qkv_proj.weight.device.type != "meta":
            # random init: ranks that replicate a KV head must hold the same rows (those of the
            # unsharded model), as they do after loading a checkpoint
            kv_rank = comm.rank // self.kv_replicas
            with torch.no_grad():
                for i in (1, 2):
                    rows = pf.normal(f"{prefix}.qkv_proj.{i}", (self.total_kv * self.D, cfg.hidden_size), 0, kv_rank,
                                     self.total_kv)
                    at = self.Hq * self.D + (i - 1) * self.D
                    self.qkv_proj.weight[at:at + self.D].copy_(rows)
        self.o_proj = RowParallelLinear(pf, f"{prefix}.o_proj", cfg.num_attention_heads * self.D,
                                        cfg.hidden_size, comm)
        self.q_norm = pf.ones((self.D,)) if cfg.qk_norm else None
        self.k_norm = pf.ones((self.D,)) if cfg.qk_norm else None
        self.comm = comm
        self.qk_norm_full = bool(cfg.qk_norm_full)
        if self.qk_norm_full:      # this rank's slice of the [all heads x D] weights
            self.q_norm = pf.ones((self.Hq * self.D,))
            self.k_norm = pf.ones((self.Hkv * self.D,))
        self.scale = self.D ** -0.5 if cfg.attention_multiplier is None else float(cfg.attention_multiplier)
        self.rot_dim = int(self.D * cfg.partial_rotary_factor) // 2 * 2
        if cfg.no_rope_layers and layer_idx < len(cfg.no_rope_layers) and not cfg.no_rope_layers[layer_idx]:
            self.rot_dim = 0
        self.cos_sin = get_cos_sin_cache(self.rot_dim, max_pos, cfg.rope_theta, cfg.rope_scaling,
                                         pf.device)
        self.window = cfg.sliding_window or 0
        # the attention implementation comes from the platform's backend table (paged tcgen05
        # kernels, or the training-consistent single-kernel backend when the RL config asks for it)
        from ..attention.backend import get_attn_backend
        self.backend = get_attn_backend()
        self.impl = self.backend.get_impl_cls()(self.Hq, self.D, self.scale, self.Hkv,
                                                sliding_window=self.window or None)
        self.mrope_axis = None
        if cfg.mrope_section:
            assert 2 * sum(cfg.mrope_section) == self.rot_dim, "mrope sections must cover rot_dim / 2 pairs"
            self.mrope_axis = ref.mrope_axis_table(cfg.mrope_section, cfg.mrope_interleaved).to(pf.device)

    def __call__(self, x: torch.Tensor, meta, kv_cache) -> torch.Tensor:
        return self.o_proj(self.attend(self.qkv_proj(x), meta, kv_cache))

    def attend(self, qkv: torch.Tensor, meta, kv_cache) -> torch.Tensor:
        """Everything between the two projections: q/k norm + rotary + KV write, paged attention,
        output gate.  qkv [T, (Hq + 2 Hkv) D (+ gate)] -> [T, Hq D]."""
        k_cache, v_cache = kv_cache
        mpos = getattr(meta, "mrope_positions", None) if self.mrope_axis is not None else None
        pcp = getattr(meta, "pcp", None)
        qkv_in = qkv
        if self.out_gate:          # the kernel walks (Hq + 2 Hkv) heads per row; the gate columns follow them
            qkv = qkv[:, :(self.Hq + 2 * self.Hkv) * self.D]
        if self.qk_norm_full:
            self._norm_over_all_heads(qkv)
        elif not _plan().enabled("qknorm_rope") and mpos is None and pcp is None:
            # the three passes the fused kernel replaces: q / k norm, rotary, cache write
            eps = self.cfg.rms_norm_eps
            if self.q_norm is not None:
                ops.qknorm_rope_kvwrite(qkv, meta.positions, self.cos_sin, 0, self.q_norm, self.k_norm, eps,
                                        None, None, None, self.Hq, self.Hkv, self.D)
            ops.qknorm_rope_kvwrite(qkv, meta.positions, self.cos_sin, self.rot_dim, None, None, eps,
                                    None, None, None, self.Hq, self.Hkv, self.D)
            ops.qknorm_rope_kvwrite(qkv, meta.positions, self.cos_sin, 0, None, None, eps,
                                    k_cache, v_cache, meta.slot_mapping, self.Hq, self.Hkv, self.D)
            return self._after_kv_write(qkv_in, meta, kv_cache)
        ops.qknorm_rope_kvwrite(qkv, meta.positions if mpos is None else mpos, self.cos_sin,
                                self.rot_dim, None if self.qk_norm_full else self.q_norm,
                                None if self.qk_norm_full else self.k_norm, self.cfg.rms_norm_eps,
                                k_cache if pcp is None else None, v_cache if pcp is None else None,
                                meta.slot_mapping, self.Hq, self.Hkv, self.D,
                                mrope_axis=None if mpos is None else self.mrope_axis)
        if pcp is not None:
            # prefill context parallel: this rank rotated its share of the tokens; the cache gets
            # the K / V rows of all ranks
            from ..attention.pcp import gather_kv_into_cache
            gather_kv_into_cache(qkv[:, self.Hq * self.D:], pcp, k_cache, v_cache, self.Hkv, self.D,
                                 self.cfg.rms_norm_eps, self.cos_sin)
        return self._after_kv_write(qkv_in, meta, kv_cache)

    def _after_kv_write(self, qkv: torch.Tensor, meta, kv_cache) -> torch.Tensor:
        k_cache, v_cache = kv_cache
        T = qkv.shape[0]
        q = qkv[:, :self.Hq * self.D].view(T, self.Hq, self.D)
        from ..parallel import state as pstate
        dcp = pstate.get_dcp_group()
        if dcp.world_size > 1:
            # the KV cache holds this rank's share of every sequence
            from ..attention.dcp import gqa_attention_dcp
            o = gqa_attention_dcp(q, k_cache, v_cache, meta, self.scale, dcp, getattr(meta, "dcp_interleave", 1))
        else:
            o = self.impl.forward(q, k_cache, v_cache, meta)
        o = o.view(T, self.Hq * self.D)
        if self.out_gate:
            o = o * torch.sigmoid(qkv[:, (self.Hq + 2 * self.Hkv) * self.D:].float()).to(o.dtype)
        return o


def _norm_over_all_heads(self, qkv: torch.Tensor) -> None:
    """RMSNorm of q over all query heads together, and of k over all KV heads (MiniMax-M2), in place.
    Under TP a rank holds some of the heads: the sums of squares of both vectors travel in one
    all-reduce ([T, 2] fp32); replicated KV heads count once."""
    cfg = self.cfg
    nq, nk = self.Hq * self.D, self.Hkv * self.D
    q, k = qkv[:, :nq], qkv[:, nq:nq + nk]
    qf, kf = q.float(), k.float()
    ss = torch.stack([(qf * qf).sum(-1), (kf * kf).sum(-1) / self.kv_replicas], dim=-1)
    if self.comm.size > 1:
        ss = self.comm.group.all_reduce(ss)
    inv_q = torch.rsqrt(ss[:, :1] / (cfg.num_attention_heads * self.D) + cfg.rms_norm_eps)
    inv_k = torch.rsqrt(ss[:, 1:] / (self.total_kv * self.D) + cfg.rms_norm_eps)
    q.copy_((qf * inv_q).to(q.dtype) * self.q_norm)
    k.copy_((kf * inv_k).to(k.dtype) * self.k_norm)


GQAAttention._norm_over_all_heads = _norm_over_all_heads


_GATED_ACTS = {"silu": None, "swish": None, "gelu_pytorch_tanh": "gelu_tanh", "gelu_tanh": "gelu_tanh",
               "gelu_new": "gelu_tanh", "gelu": "gelu"}


class PlainMLP:
    """Ungated MLP: act(x W_up) -> W_down, with ReLU^2 (Arcee), GELU, SiLU or ReLU."""

    _ACTS = {"relu2": lambda t: torch.relu(t).square(), "relu": torch.relu, "silu": torch.nn.functional.silu,
             "gelu": torch.nn.functional.gelu,
             "gelu_pytorch_tanh": lambda t: torch.nn.functional.gelu(t, approximate="tanh")}

    def __init__(self, pf: ParamFactory, prefix: str, hidden: int, inter: int, comm: TPComm, act: str = "relu2"):
        if act not in self._ACTS:
            raise ValueError(f"unsupported MLP activation {act!r}")
        self.fn = self._ACTS[act]
        self.up_proj = ColumnParallelLinear(pf, f"{prefix}.up_proj", hidden, [inter], comm)
        self.down_proj = RowParallelLinear(pf, f"{prefix}.down_proj", inter, hidden, comm)

    def __call__(self, x: torch.Tensor) -> torch.Tensor:
        return self.down_proj(self.fn(self.up_proj(x)))


class SwiGLUMLP:
    """Gated MLP: act(x W_gate) * (x W_up) -> W_down; SiLU (fused into the GEMM epilogue) or GELU gates."""

    def __init__(self, pf: ParamFactory, prefix: str, hidden: int, inter: int, comm: TPComm,
                 reduce_results: bool = True, act: str = "silu"):
        if act not in _GATED_ACTS:
            raise ValueError(f"unsupported MLP activation {act!r}")
        self.act = _GATED_ACTS[act]
        self.gate_up_proj = ColumnParallelLinear(pf, f"{prefix}.gate_up_proj", hidden,
                                                 [inter, inter], comm)
        self.down_proj = RowParallelLinear(pf, f"{prefix}.down_proj", inter, hidden, comm,
                                           reduce_results=reduce_results)

    def __call__(self, x: torch.Tensor) -> torch.Tensor:
        gu = self.gate_up_proj
        if self.act is not None:
            return self.down_proj(ops.activation(gu(x).contiguous(), self.act, gated=True))
        if gu.quant is None and gu.bias is None and not gu.gather_output and not gu._lora_on() \
                and _plan().enabled("gemm_swiglu"):
            return self.down_proj(ops.linear_swiglu(x, gu.weight))
        if wants_quant_act(self.down_proj):
            return self.down_proj(ops.silu_and_mul_quant_fp8(gu(x)))
        return self.down_proj(ops.silu_and_mul(gu(x)))
