"""Medusa proposer: K small heads on top of the target's last hidden state, head j predicting
the token j+1 positions ahead.  No draft KV cache and no extra forward pass of a model: one
residual block and one LM-head projection per head on the sampled rows
(the "medusa" method of vllm_ascend/spec_decode/__init__.py:33-58).
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import ops
from ..models.layers import ParamFactory


class MedusaHead:
    """h -> h + SiLU(W h + b), then the shared LM head."""

    def __init__(self, pf: ParamFactory, name: str, hidden: int, num_blocks: int = 1):
        self.blocks = [(pf.normal(f"{name}.blocks.{i}.weight", (hidden, hidden)), pf.zeros((hidden,)))
                       for i in range(num_blocks)]

    def __call__(self, h: torch.Tensor) -> torch.Tensor:
        for w, b in self.blocks:
            h = h + torch.nn.functional.silu(ops.linear(h, w, b))
        return h

    def named_tensors(self):
        for i, (w, b) in enumerate(self.blocks):
            yield f"blocks.{i}.weight", w
            yield f"blocks.{i}.bias", b


class MedusaProposer:
    name = "medusa"
    needs_hidden_states = True

    def __init__(self, num_speculative_tokens: int, spec_cfg: dict, runner):
        self.k, self.runner = num_speculative_tokens, runner
        model = runner.model
        pf = ParamFactory(runner.mcfg, runner.device, model.embed_tokens.weight.dtype)
        self.heads = [MedusaHead(pf, f"medusa.{j}", runner.mcfg.hidden_size,
                                 int(spec_cfg.get("num_residual_blocks", 1))) for j in range(self.k)]
        self.lm_head = model.lm_head
        self.stats = {"draft_forwards": 0}

    def load_weights(self, weights) -> int:
        """HF medusa naming: ``<head>.<block>.linear.{weight,bias}``."""
        params = {f"{j}.{n}": t for j, h in enumerate(self.heads) for n, t in h.named_tensors()}
        n = 0
        for name, w in weights:
            key = name.replace("linear.", "").replace("medusa_head.", "")
            if key in params:
                params[key].copy_(w)
                n += 1
        return n

    def note_step_start(self, so) -> None:
        self._starts = {req.request_id: req.num_computed_tokens for req, _ in so.scheduled}

    @torch.inference_mode()
    def propose_step(self, so, sampled: dict, hidden: Optional[torch.Tensor], scheduler) -> None:
        live, rows = [], []
        off = 0
        for req, n in so.scheduled:
            off_req, off = off, off + n
            if req.request_id not in sampled or req.status.name != "RUNNING":
                continue
            # the hidden state that produced the newest token: last accepted position of this step
            start = self._starts.get(req.request_id, 0)
            last = req.num_computed_tokens - 1 - start
            if last < 0 or last >= n:
                continue
            live.append(req)
            rows.append(off_req + last)
        if not live:
            return
        h = hidden[torch.tensor(rows, dtype=torch.int64, device=hidden.device)]
        drafts = []
        for head in self.heads:
            drafts.append(ops.argmax(self.lm_head(head(h))))
        self.stats["draft_forwards"] += 1
        toks = torch.stack(drafts, dim=1).cpu().numpy()            # [B, k]
        for req, t in zip(live, toks):
            room = min(self.k, self.runner.max_model_len - req.num_tokens - 1,
                       req.sampling_params.max_tokens - req.num_output_tokens - 1)
            req.spec_token_ids = [int(x) for x in t[:max(room, 0)]]
