"""Sparse-attention KV offload: the full KV of every sequence stays in pinned host memory, the
GPU holds a per-sequence pool of token slots that is refilled with whatever the indexer selects.

``SparseKVOffloadManager.step(seq_ids, topk)`` maps each selected token to a device slot
(native LRU bookkeeping in ``csrc/sparse_kv_offload.cpp``), copies the misses host→device and
returns the slot indices the sparse attention kernel should read.  Role of
vllm_ascend/distributed/kv_transfer/sparse_kv_offload/sparse_kv_offload_manager.py.
"""
from __future__ import annotations

import ctypes
from ctypes import POINTER, c_int, c_long, c_void_p

import numpy as np
import torch

from ... import _native

_native.register_signature("b200_sko_create", [c_int], restype=c_void_p)
_native.register_signature("b200_sko_destroy", [c_void_p], restype=None)
_native.register_signature("b200_sko_release", [c_void_p, c_long], restype=None)
_native.register_signature("b200_sko_update", [c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p,
                                               c_void_p, c_void_p, c_int])
_native.register_signature("b200_sko_stats", [c_void_p, c_void_p], restype=None)


class SparseKVOffloadManager:
    def __init__(self, max_seqs: int, max_tokens_per_seq: int, slots_per_seq: int, width: int,
                 dtype=torch.bfloat16, device="cuda", num_threads: int = 4):
        self.device = torch.device(device)
        self.slots_per_seq, self.width, self.num_threads = slots_per_seq, width, num_threads
        pin = self.device.type == "cuda"
        # host: every token of every sequence row; device: the resident pools
        self.host = torch.zeros((max_seqs, max_tokens_per_seq, width), dtype=dtype, pin_memory=pin)
        self.pool = torch.zeros((max_seqs, slots_per_seq, width), dtype=dtype, device=self.device)
        self.lib = _native.lib()
        self.h = self.lib.b200_sko_create(slots_per_seq)
        if not self.h:
            raise ValueError("slots_per_seq must be positive")

    def append(self, row: int, position: int, values: torch.Tensor) -> None:
        """Store newly computed KV rows [n, width] of sequence ``row`` on the host."""
        n = values.shape[0]
        self.host[row, position:position + n].copy_(values, non_blocking=True)

    def step(self, rows: np.ndarray, topk: np.ndarray) -> torch.Tensor:
        """rows [B] sequence rows, topk [B, k] selected token positions (-1 padded) ->
        device slot indices [B, k] (int64, -1 padded) into ``pool[row]``."""
        rows = np.ascontiguousarray(rows, dtype=np.int64)
        topk = np.ascontiguousarray(topk, dtype=np.int32)
        B, k = topk.shape
        slots = np.empty((B, k), dtype=np.int32)
        miss_tok = np.empty((B, k), dtype=np.int32)
        miss_slot = np.empty((B, k), dtype=np.int32)
        miss_cnt = np.empty(B, dtype=np.int32)
        rc = self.lib.b200_sko_update(self.h, rows.ctypes.data, B, topk.ctypes.data, k, slots.ctypes.data,
                                      miss_tok.ctypes.data, miss_slot.ctypes.data, miss_cnt.ctypes.data,
                                      self.num_threads)
        if rc != 0:
            raise RuntimeError(f"sequence row {rows[rc - 1]} selects more distinct tokens than its "
                               f"{self.slots_per_seq} device slots")
        total = int(miss_cnt.sum())
        if total:
            r = np.repeat(rows, miss_cnt)
            mask = np.arange(k)[None, :] < miss_cnt[:, None]
            src_tok, dst_slot = miss_tok[mask], miss_slot[mask]
            src = self.host[torch.from_numpy(r), torch.from_numpy(src_tok.astype(np.int64))]
            if self.device.type == "cuda":
                src = src.pin_memory().to(self.device, non_blocking=True)
            self.pool[torch.from_numpy(r).to(self.device), torch.from_numpy(dst_slot.astype(np.int64)).to(self.device)] = src
        return torch.from_numpy(slots.astype(np.int64)).to(self.device)

    def release(self, row: int) -> None:
        self.lib.b200_sko_release(self.h, int(row))

    def stats(self) -> dict:
        out = (c_long * 3)()
        self.lib.b200_sko_stats(self.h, out)
        return {"hits": out[0], "misses": out[1], "evictions": out[2]}

    def close(self) -> None:
        if self.h:
            self.lib.b200_sko_destroy(self.h)
            self.h = None
