"""Runner-side multimodal state: encoder execution, encoder-output cache, embedding merge and
3-axis rotary positions.

Per step, for every scheduled chunk that overlaps a placeholder run, the item's encoder output is
taken from the cache (or computed: all missing items of the step go through the vision tower in
one batch, or are fetched from a remote encoder through the EC connector) and the overlapping rows
are written over the token embeddings.  An item's output is dropped once the request has computed
past its run.  Follows the reference's flow in worker/model_runner_v1.py:1846-1990
(_execute_mm_encoder / _gather_mm_embeddings / mrope position preparation).
"""
from __future__ import annotations

from typing import Optional

import numpy as np
import torch


class MultimodalState:
    def __init__(self, runner, ec_connector=None):
        self.runner = runner
        dev = runner.device
        n = runner.input_ids.shape[0]
        self.mrope_positions = torch.zeros((3, n), dtype=torch.int64, device=dev)
        self._h_mrope = torch.zeros((3, n), dtype=torch.int64, pin_memory=runner.is_cuda)
        self.delta_cpu = np.zeros(runner.max_seqs + 1, dtype=np.int64)
        self.encoder_cache: dict[tuple, torch.Tensor] = {}
        self.ec_connector = ec_connector
        self.encoder_graphs = None                 # optional EncoderGraphManager
        self._patches: list[tuple[int, int, torch.Tensor]] = []
        self.deepstack = None                      # set by inputs_embeds for models with deepstack features
        self.stats = {"encoder_runs": 0, "encoder_items": 0, "encoder_cache_hits": 0, "remote_items": 0}

    # -- per-step preparation -------------------------------------------------
    def prepare(self, reqs, starts, q_lens, cu, pos, req_idx, T: int, Tp: int, meta) -> None:
        for r in reqs:
            self.delta_cpu[r.row] = getattr(r, "mrope_delta", 0)
        rows = np.fromiter((r.row for r in reqs), dtype=np.int64, count=len(reqs))
        base = pos + self.delta_cpu[rows][req_idx]
        hm = self._h_mrope
        hm[:, :T] = torch.from_numpy(np.broadcast_to(base, (3, T)).copy())
        self._patches = []
        need: list[tuple] = []
        for i, r in enumerate(reqs):
            if not getattr(r, "mm_inputs", None):
                continue
            s, e = int(starts[i]), int(starts[i] + q_lens[i])
            self.release(r, s)
            P = r.num_prompt_tokens
            if s < P and r.mrope_positions is not None:
                pe = min(e, P)
                hm[:, cu[i]:cu[i] + pe - s] = torch.from_numpy(r.mrope_positions[:, s:pe])
            for k, it in enumerate(r.mm_inputs):
                if it.offset < e and it.end > s:
                    need.append((r, k, it, i, s, e))
        if Tp > T:
            hm[:, T:Tp] = 0
        self.mrope_positions[:, :Tp].copy_(hm[:, :Tp], non_blocking=True)
        meta.mrope_positions = self.mrope_positions[:, :Tp]
        if not need:
            return
        self._run_encoder([(r, k, it) for r, k, it, *_ in need])
        for r, k, it, i, s, e in need:
            emb = self.encoder_cache[(r.request_id, k)]
            lo, hi = max(s, it.offset), min(e, it.end)
            self._patches.append((int(cu[i]) + lo - s, int(cu[i]) + hi - s, emb[lo - it.offset:hi - it.offset]))

    def _run_encoder(self, wanted: list) -> None:
        missing = []
        for r, k, it in wanted:
            key = (r.request_id, k)
            if key in self.encoder_cache:
                self.stats["encoder_cache_hits"] += 1
                continue
            if it.embeds is not None:
                self.encoder_cache[key] = it.embeds.to(self.runner.device, self.runner.model.dtype)
                continue
            if self.ec_connector is not None:
                got = self.ec_connector.load(it.hash, self.runner.device, self.runner.model.dtype)
                if got is not None:
                    self.encoder_cache[key] = got
                    self.stats["remote_items"] += 1
                    continue
            if it.pixel_values is None:
                raise RuntimeError(f"{r.request_id}: encoder input {k} has neither pixels nor a cached output")
            missing.append((key, it))
        if not missing:
            return
        model = self.runner.model
        audio = [(key, it) for key, it in missing if it.modality == "audio"]
        missing = [(key, it) for key, it in missing if it.modality != "audio"]
        if audio:
            out = model.embed_audio([it.pixel_values for _, it in audio], [it.grid_thw[0] for _, it in audio])
            self._store(audio, out)
        if not missing:
            return
        px = torch.cat([it.pixel_values for _, it in missing]).to(self.runner.device, model.dtype)
        grid = np.array([it.grid_thw for _, it in missing], dtype=np.int64)
        if self.encoder_graphs is not None:
            out = self.encoder_graphs.run(px, grid)
        else:
            out = model.embed_multimodal(px, grid)
        self._store(missing, out)

    def _store(self, items: list, out: torch.Tensor) -> None:
        self.stats["encoder_runs"] += 1
        self.stats["encoder_items"] += len(items)
        off = 0
        for key, it in items:
            self.encoder_cache[key] = out[off:off + it.length]
            off += it.length
            if self.ec_connector is not None and self.ec_connector.is_producer:
                self.ec_connector.save(it.hash, self.encoder_cache[key])

    # -- forward-time merge -------------------------------------------------------
    def inputs_embeds(self, input_ids: torch.Tensor) -> Optional[torch.Tensor]:
        """Token embeddings with this step's encoder rows written in; None for text-only steps."""
        self.deepstack = None
        if not self._patches:
            return None
        h = self.runner.model.embed_input_ids(input_ids)
        H = h.shape[-1]
        L = getattr(self.runner.model, "num_deepstack", 0)
        rows, feats = [], []
        for a, b, emb in self._patches:
            h[a:b] = emb[:, :H].to(h.dtype)
            if L and emb.shape[-1] == (1 + L) * H:
                rows.append(torch.arange(a, b, device=h.device))
                feats.append(emb[:, H:].to(h.dtype).view(b - a, L, H))
        if rows:
            # (token rows [n], features [L, n, H]) the decoder adds after its first L layers
            self.deepstack = (torch.cat(rows), torch.cat(feats).transpose(0, 1).contiguous())
        self._patches = []
        return h

    # -- lifetime ---------------------------------------------------------------------
    def release(self, req, computed: Optional[int] = None) -> None:
        """Drop outputs the request has moved past (all of them when it finishes)."""
        for k, it in enumerate(req.mm_inputs):
            if computed is None or it.end <= computed:
                self.encoder_cache.pop((req.request_id, k), None)
