"""Sparse MLA attention over host-resident KV.

With ``sparse_kv_offload_config.enabled`` the latent / rope-key rows of every sequence live in
pinned host memory and the device keeps, per sequence, a small pool of the rows the indexer
selected recently (LRU bookkeeping in native code, ``csrc/sparse_kv_offload.cpp``).  Per layer and
step: the new tokens' rows go to the host, the indexer's selection is read back, the pool is
refilled with the misses, and attention runs over the pool rows.  Index keys stay in a paged
device cache because the indexer scores all of them every step.  The per-layer host round trip makes
this a capacity feature (context length x batch beyond HBM), not a fast path.

Role of the reference's sparse KV offload for its sparse-attention backend
(vllm_ascend/distributed/kv_transfer/sparse_kv_offload/sparse_kv_offload_manager.py with
attention/sfa_v1.py reading the resident set).
"""
from __future__ import annotations

import numpy as np
import torch

from ..distributed.kv_transfer.sparse_kv_offload import SparseKVOffloadManager


class SparseOffloadLayer:
    def __init__(self, max_seqs: int, max_tokens_per_seq: int, slots_per_seq: int, dc: int, dr: int, dtype, device,
                 num_threads: int = 4):
        self.dc, self.dr = dc, dr
        self.mgr = SparseKVOffloadManager(max_seqs, max_tokens_per_seq, slots_per_seq, dc + dr, dtype, device,
                                          num_threads)

    @property
    def host(self) -> torch.Tensor:
        return self.mgr.host

    def append(self, tok_rows: np.ndarray, positions: np.ndarray, latent: torch.Tensor, k_pe: torch.Tensor) -> None:
        """Rows of this step's tokens -> host store (tokens with a negative row are padding)."""
        keep = tok_rows >= 0
        vals = torch.cat([latent, k_pe], dim=-1).to(self.mgr.host.dtype).cpu()
        if not keep.all():
            vals, tok_rows, positions = vals[torch.from_numpy(keep)], tok_rows[keep], positions[keep]
        self.mgr.host[torch.from_numpy(tok_rows.astype(np.int64)), torch.from_numpy(positions.astype(np.int64))] = vals

    def release(self, row: int) -> None:
        self.mgr.release(row)

    def attend(self, q_lat: torch.Tensor, q_pe: torch.Tensor, tok_rows: np.ndarray, indices: torch.Tensor,
               scale: float) -> torch.Tensor:
        """q_lat [T,H,dc], q_pe [T,H,dr], indices [T, topk] token positions (-1 padded) -> o_lat [T,H,dc]."""
        T = q_lat.shape[0]
        idx_cpu = indices.cpu().numpy()
        out = torch.zeros_like(q_lat)
        # the resident set is per sequence: tokens of one sequence are served one after the other
        occ = np.zeros(T, dtype=np.int64)
        seen: dict = {}
        for t, r in enumerate(tok_rows.tolist()):
            occ[t] = seen.get(r, 0)
            seen[r] = occ[t] + 1
        for rnd in range(int(occ.max()) + 1 if T else 0):
            sel = np.nonzero((occ == rnd) & (tok_rows >= 0))[0]
            if sel.size == 0:
                continue
            rows = tok_rows[sel].astype(np.int64)
            slots = self.mgr.step(rows, idx_cpu[sel])                              # [n, topk] int64, -1 padded
            rows_d = torch.from_numpy(rows).to(q_lat.device)
            kv = self.mgr.pool[rows_d[:, None], slots.clamp(min=0)].float()           # [n, topk, dc + dr]
            kl, kp = kv[..., :self.dc], kv[..., self.dc:]
            sel_d = torch.from_numpy(sel).to(q_lat.device)
            s = (torch.einsum("nhc,nkc->nhk", q_lat[sel_d].float(), kl)
                 + torch.einsum("nhr,nkr->nhk", q_pe[sel_d].float(), kp)) * scale
            s = s.masked_fill((slots < 0)[:, None, :], float("-inf"))
            p = torch.softmax(s, dim=-1)
            out[sel_d] = torch.einsum("nhk,nkc->nhc", p, kl).to(out.dtype)
        return out
