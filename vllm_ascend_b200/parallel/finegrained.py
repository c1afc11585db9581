"""Fine-grained tensor parallelism for data-parallel deployments.

With DP attention every replica holds full copies of o_proj, the dense MLP, the LM head and the
embedding.  Fine-grained TP shards each of those over its own group of ranks that spans DP
replicas, trading a collective over the group's tokens for the weight memory:

  mlp_tp    all-gather(tokens) -> gate_up shard -> SiLU-mul -> down shard -> reduce-scatter(tokens)
  otp       all-to-all (head columns out, tokens in) -> o_proj shard -> reduce-scatter(tokens)
  lmtp      all-gather(rows) -> vocab-shard logits -> all-to-all (rows back, vocab shards in)
  embed_tp  all-gather(ids) -> masked lookup in the vocab shard -> reduce-scatter(tokens)

Replicas schedule different token counts, so every tensor is padded to the step's maximum over
the DP group (the engine's per-step DP sync provides it) before a collective.  Same dataflow as
the reference's custom linear ops (vllm_ascend/ops/linear_op.py:152-273 MLPColumnParallelOp /
MLPRowParallelOp / OProjRowParallelOp; ops/vocab_parallel_embedding.py:170-391) over the groups of
vllm_ascend/distributed/parallel_state.py:95-134.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from . import state as pstate


@dataclass
class FGState:
    otp: Optional[pstate.GroupCoordinator] = None
    lmtp: Optional[pstate.GroupCoordinator] = None
    embed_tp: Optional[pstate.GroupCoordinator] = None
    mlp_tp: Optional[pstate.GroupCoordinator] = None
    max_tokens: int = 0          # pad target of token-shaped tensors in this step
    max_rows: int = 0            # pad target of the rows that reach the LM head in this step

    @property
    def any(self) -> bool:
        return any(g is not None for g in (self.otp, self.lmtp, self.embed_tp, self.mlp_tp))


_FG: Optional[FGState] = None


def init_from_groups() -> Optional[FGState]:
    """Picks up the fine-grained groups created by ``initialize_model_parallel``."""
    global _FG
    extra = pstate.get_state().extra
    st = FGState()
    for name in ("otp", "lmtp", "embed_tp", "mlp_tp"):
        g = extra.get(name)
        if g is not None and g.world_size > 1:
            setattr(st, name, g)
    _FG = st if st.any else None
    return _FG


def get_fg() -> Optional[FGState]:
    return _FG


def reset() -> None:
    global _FG
    _FG = None


def _pad_rows(x: torch.Tensor, n: int) -> torch.Tensor:
    if x.shape[0] == n:
        return x.contiguous()
    if x.shape[0] > n:
        raise RuntimeError(f"fine-grained TP: {x.shape[0]} rows exceed this step's pad target {n}")
    out = x.new_zeros((n, *x.shape[1:]))
    out[:x.shape[0]] = x
    return out


class FGMLP:
    """Dense SwiGLU MLP sharded over the mlp_tp group."""

    def __init__(self, inner, group):
        self.inner, self.group = inner, group          # inner: SwiGLUMLP(reduce_results=False) over the group
        self.gate_up_proj, self.down_proj = inner.gate_up_proj, inner.down_proj

    def __call__(self, x):
        fg = get_fg()
        T = x.shape[0]
        xg = self.group.all_gather(_pad_rows(x, max(fg.max_tokens, 1)), dim=0)
        y = self.inner(xg)                               # partial sums over the group
        return self.group.reduce_scatter(y.contiguous(), dim=0)[:T]


class FGOProj:
    """o_proj sharded along its input (head) dimension over the otp group."""

    def __init__(self, inner, group):
        self.inner, self.group = inner, group          # inner: RowParallelLinear(reduce_results=False)
        self.weight, self.bias, self.quant, self.lora = inner.weight, inner.bias, inner.quant, inner.lora

    def named_tensors(self):
        return self.inner.named_tensors()

    def __call__(self, x, residual=None):
        fg = get_fg()
        T, n = x.shape[0], self.group.world_size
        Tm = max(fg.max_tokens, 1)
        xp = _pad_rows(x, Tm)                                            # [Tm, K]
        K = xp.shape[1]
        # column block j goes to rank j; rank j receives its block of everybody's tokens
        send = xp.view(Tm, n, K // n).transpose(0, 1).contiguous()      # [n, Tm, K/n]
        recv = self.group.all_to_all_single(send.view(n * Tm, K // n))  # [n * Tm, K/n], source-major
        y = self.inner(recv)                                            # [n * Tm, H] partial
        y = self.group.reduce_scatter(y.contiguous(), dim=0)[:T]
        return y if residual is None else y + residual


class FGLMHead:
    """LM head with the vocabulary sharded over the lmtp group."""

    def __init__(self, head, group):
        self.head, self.group = head, group           # head: ParallelLMHead over a TPComm(group) embedding
        self.embed, self.weight, self.comm = head.embed, head.weight, head.comm

    def _local_logits(self, hidden):
        from .. import ops
        fg = get_fg()
        n_rows = hidden.shape[0]
        Rm = max(fg.max_rows, 1)
        hg = self.group.all_gather(_pad_rows(hidden, Rm), dim=0)         # [n * Rm, H]
        return ops.linear(hg, self.weight), n_rows, Rm                  # [n * Rm, V / n]

    def __call__(self, hidden):
        logits, n_rows, Rm = self._local_logits(hidden)
        n = self.group.world_size
        back = self.group.all_to_all_single(logits.contiguous())        # block j: my rows, vocab shard j
        full = back.view(n, Rm, -1).transpose(0, 1).reshape(Rm, -1)
        return full[:n_rows, :self.embed.vocab]

    def greedy_tokens(self, hidden):
        return self(hidden).argmax(dim=-1)


class FGEmbedding:
    """Embedding with the vocabulary sharded over the embed_tp group."""

    def __init__(self, inner, group):
        self.inner, self.group = inner, group
        self.weight, self.vocab, self.comm = inner.weight, inner.vocab, inner.comm
        self.shard, self.start, self.padded_vocab = inner.shard, inner.start, inner.padded_vocab

    def __call__(self, ids):
        from .. import ops
        fg = get_fg()
        T = ids.shape[0]
        ig = self.group.all_gather(_pad_rows(ids, max(fg.max_tokens, 1)), dim=0)
        part = ops.embedding(ig, self.weight, self.start, self.start + self.shard)
        return self.group.reduce_scatter(part.contiguous(), dim=0)[:T]
