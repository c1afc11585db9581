"""Pseudo proposer that records hidden states instead of drafting.

Runs in the proposer slot of the engine (it sees every step's hidden states in scheduling order) but
never proposes a token.  For every request it accumulates the final hidden state, or the residual
streams of the configured layers, of each position the target model computed, and on completion
hands ``[num_tokens, width]`` to a sink: a directory (one ``<request id>.pt`` per request), or an
in-memory dict.  Used to collect training data for draft heads (the role of the reference's
extract-hidden-states proposer, vllm_ascend/spec_decode/extract_hidden_states_proposer.py, which
stores the states through a KV connector).
"""
from __future__ import annotations

import os
from typing import Optional

import torch


class ExtractHiddenStatesProposer:
    name = "extract_hidden_states"
    method = "extract_hidden_states"

    def __init__(self, spec_cfg: dict, runner):
        self.runner = runner
        self.layers = tuple(spec_cfg.get("layers") or ())
        self.output_dir: Optional[str] = spec_cfg.get("output_dir")
        if self.output_dir:
            os.makedirs(self.output_dir, exist_ok=True)
        if self.layers:
            runner.model.aux_layers = self.layers
        self.uses_aux = bool(self.layers)
        self.chunks: dict[str, list] = {}
        self.results: dict[str, torch.Tensor] = {}
        self.stats = {"requests": 0, "rows": 0}
        self._step_start: dict = {}

    def note_step_start(self, so) -> None:
        self._step_start = {req.request_id: req.num_computed_tokens for req, _ in so.scheduled}

    @torch.inference_mode()
    def propose_step(self, so, sampled: dict, hidden: Optional[torch.Tensor], scheduler) -> None:
        src = self.runner.model.aux_hidden if self.uses_aux else hidden
        off = 0
        for req, n in so.scheduled:
            rows = src[off:off + n].float().cpu()
            off += n
            self.chunks.setdefault(req.request_id, []).append(rows)
            self.stats["rows"] += n
            req.spec_token_ids = []
            if req.is_finished:
                out = torch.cat(self.chunks.pop(req.request_id))
                self.stats["requests"] += 1
                if self.output_dir:
                    torch.save({"request_id": req.request_id, "token_ids": req.prompt_token_ids.tolist()
                                + list(req.output_token_ids or []), "hidden_states": out},
                               os.path.join(self.output_dir, f"{req.request_id}.pt"))
                else:
                    self.results[req.request_id] = out
