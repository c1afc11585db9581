"""KV offload to pinned host memory, keyed by prefix hash.

Full blocks of finished requests are copied device→host on a side stream (the GPU blocks
are freed only after the copy), and a later request whose prompt starts with the same
tokens gets those blocks copied back host→device instead of recomputing them.  The copies
are one gather/scatter kernel over all layers writing or reading the pinned host buffers
directly (unified addressing), the B200 form of the reference's batched async block swaps
(vllm_ascend/distributed/kv_transfer/kv_pool/kv_offload/native/cpu_npu.py:56-328 and the
``swap_blocks_batch`` op); the scheduler side follows the simple CPU offload connector
(lookup by block hash, LRU host pool).
"""
from __future__ import annotations

import time
from collections import OrderedDict
from typing import Optional

import numpy as np
import torch

from ... import _native
from ...engine.block_pool import BlockPool
from ...logger import logger
from .base import ConnectorMetadata, KVConnectorBase


class CPUOffloadConnector(KVConnectorBase):
    def __init__(self, engine_cfg, runner):
        ktc = dict(engine_cfg.kv_transfer_config or {})
        extra = dict(ktc.get("kv_connector_extra_config") or {})
        self.runner = runner
        self.block_size = engine_cfg.cache.block_size
        self.tensors = [t for pair in runner.kv_caches for t in pair]
        self._fingerprint = BlockPool.store_fingerprint(engine_cfg, self.tensors)
        self.is_cuda = self.tensors[0].is_cuda
        per_block = sum(t[0].numel() * t.element_size() for t in self.tensors)
        n = int(extra.get("num_cpu_blocks", 0))
        if n <= 0:
            n = max(1, int(float(extra.get("cpu_bytes", 1 << 30)) // per_block))
        self.num_cpu_blocks = n
        # host mirror of every cache tensor, dense [blocks, tokens, heads, dim]
        self.host = [torch.zeros((n,) + tuple(t.shape[1:]), dtype=t.dtype, pin_memory=self.is_cuda)
                     for t in self.tensors]
        self.lru: "OrderedDict[bytes, int]" = OrderedDict()      # block hash -> host block
        self.free = list(range(n))
        self._pending_load: list[tuple[list, list]] = []          # (host blocks, gpu blocks)
        self._saving: list[tuple[object, list, list, list]] = []  # (event, gpu blocks, hashes, host blocks)
        self._scheduler = None
        self.stats = {"saved_blocks": 0, "loaded_blocks": 0, "hit_tokens": 0, "evicted_blocks": 0}
        if self.is_cuda:
            import vllm_ascend_b200.distributed.kv_transfer.nvlink_connector  # noqa: F401  (kernel signature)
            self.stream = torch.cuda.Stream(device=self.tensors[0].device)
            self._groups = self._make_groups()

    # ------------------------------------------------------------------ copies
    def _make_groups(self):
        from .nvlink_connector import _group_tensors
        dev = self.tensors[0].device
        out = []
        for g in _group_tensors(self.tensors):
            hs = [self.host[i] for i in g.indices]
            e = hs[0].element_size()
            hstr = (hs[0].stride(0) * e, hs[0].stride(1) * e, hs[0].stride(2) * e)
            dptr = torch.tensor([self.tensors[i].data_ptr() for i in g.indices], dtype=torch.int64, device=dev)
            hptr = torch.tensor([h.data_ptr() for h in hs], dtype=torch.int64, device=dev)
            out.append((g, dptr, hptr, hstr))
        return out

    def _copy(self, src_blocks: list, dst_blocks: list, to_host: bool, stream) -> None:
        if not src_blocks:
            return
        if not self.is_cuda:
            s, d = torch.as_tensor(src_blocks), torch.as_tensor(dst_blocks)
            for t, h in zip(self.tensors, self.host):
                if to_host:
                    h[d] = t[s]
                else:
                    t[d] = h[s]
            return
        dev = self.tensors[0].device
        lib = _native.lib()
        with torch.cuda.stream(stream):
            sb = torch.tensor(src_blocks, dtype=torch.int32).pin_memory().to(dev, non_blocking=True)
            db = torch.tensor(dst_blocks, dtype=torch.int32).pin_memory().to(dev, non_blocking=True)
            for g, dptr, hptr, hstr in self._groups:
                sp, dp = (dptr, hptr) if to_host else (hptr, dptr)
                ss, ds = (g.strides, hstr) if to_host else (hstr, g.strides)
                ns, nd = (int(self.tensors[0].shape[0]), self.num_cpu_blocks) if to_host else \
                    (self.num_cpu_blocks, int(self.tensors[0].shape[0]))
                rc = lib.b200_kv_block_copy(sp.data_ptr(), dp.data_ptr(), sb.data_ptr(), db.data_ptr(),
                                            len(src_blocks), len(g.indices), self.block_size, g.hd_bytes, g.heads,
                                            0, 0, ss[0], ss[1], ss[2], ds[0], ds[1], ds[2], ns, nd,
                                            _native.status_word(dev).data_ptr(), stream.cuda_stream)
                _native.check(rc, "kv_block_copy (offload)")
                _native.count_launch()
            self._keep = (sb, db)

    # ------------------------------------------------------------------ host pool
    def _take_host_block(self) -> Optional[int]:
        if self.free:
            return self.free.pop()
        if self.lru:
            _, b = self.lru.popitem(last=False)
            self.stats["evicted_blocks"] += 1
            return b
        return None

    def _hashes(self, req, num_tokens: int) -> list[bytes]:
        toks = np.concatenate([req.prompt_token_ids, np.asarray(req.output_token_ids or [], dtype=np.int32)])
        extra = BlockPool.request_key_extra(req, self._fingerprint)
        if extra is None:               # nothing of this request may be looked up or published
            return []
        out, parent = [], None
        for i in range(num_tokens // self.block_size):
            parent = BlockPool.hash_block(parent, toks[i * self.block_size:(i + 1) * self.block_size], extra)
            out.append(parent)
        return out

    # ------------------------------------------------------------------ scheduler side
    def get_num_new_matched_tokens(self, req, num_computed_tokens: int) -> tuple[int, bool]:
        bs = self.block_size
        hashes = self._hashes(req, self._lookup_tokens(req))       # the last token is always computed
        first = num_computed_tokens // bs
        n = 0
        for h in hashes[first:]:
            if h not in self.lru:
                break
            n += 1
        return n * bs, False

    def update_state_after_alloc(self, req, block_ids: list, num_external_tokens: int) -> None:
        if num_external_tokens <= 0:
            return
        bs = self.block_size
        first = req.num_cached_tokens // bs
        n = num_external_tokens // bs
        hashes = self._hashes(req, (first + n) * bs)[first:first + n]
        host = []
        for h in hashes:
            self.lru.move_to_end(h)
            host.append(self.lru[h])
        self._pending_load.append((host, list(block_ids[first:first + n])))
        self.stats["hit_tokens"] += num_external_tokens

    def build_connector_meta(self, scheduler_output) -> ConnectorMetadata:
        return ConnectorMetadata(reqs_to_recv={i: j for i, j in enumerate(self._pending_load)})

    def _lookup_tokens(self, req) -> int:
        return req.num_prompt_tokens - 1

    def request_finished(self, req, block_ids: list) -> tuple[bool, Optional[dict]]:
        """Offload the request's full blocks that the host does not hold yet."""
        return self._save_blocks(req, block_ids), None

    def _save_blocks(self, req, block_ids: list) -> bool:
        """Copy the request's full blocks the host does not hold yet; True when the GPU blocks must
        stay allocated until the copy has finished (the connector frees them then)."""
        n_full = min(req.num_computed_tokens, req.num_tokens) // self.block_size
        if n_full == 0 or not block_ids:
            return False
        hashes = self._hashes(req, n_full * self.block_size)
        self._note_owner(req, hashes)
        src, dst, hs = [], [], []
        for h, b in zip(hashes, block_ids):
            if h in self.lru:
                self.lru.move_to_end(h)
                continue
            hb = self._take_host_block()
            if hb is None:
                break
            src.append(b)
            dst.append(hb)
            hs.append(h)
        if not src:
            return False
        if not self.is_cuda:
            self._copy(src, dst, True, None)
            for h, hb in zip(hs, dst):
                self.lru[h] = hb
            self.stats["saved_blocks"] += len(src)
            return False
        # the blocks were written on the compute stream: order the copy after it
        self.stream.wait_stream(torch.cuda.current_stream())
        self._copy(src, dst, True, self.stream)
        ev = torch.cuda.Event()
        ev.record(self.stream)
        self._saving.append((ev, list(block_ids), hs, dst))
        return True                # free after the copy finished

    def _note_owner(self, req, hashes: list) -> None:
        pass

    # ------------------------------------------------------------------ worker side
    def start_load_kv(self, scheduler_output) -> None:
        jobs, self._pending_load = self._pending_load, []
        for host, gpu in jobs:
            # on the compute stream, so the forward pass of this step sees the blocks
            self._copy(host, gpu, False, torch.cuda.current_stream() if self.is_cuda else None)
            self.stats["loaded_blocks"] += len(gpu)

    def step_finished(self, scheduler_output, scheduler) -> None:
        self._scheduler = scheduler
        still = []
        for ev, blocks, hs, dst in self._saving:
            if ev.query():
                for h, hb in zip(hs, dst):
                    self.lru[h] = hb
                self.stats["saved_blocks"] += len(hs)
                scheduler.pool.free(blocks)
            else:
                still.append((ev, blocks, hs, dst))
        self._saving = still

    def reap(self, scheduler) -> None:
        if self.is_cuda:
            self.stream.synchronize()
        self.step_finished(None, scheduler)

    @property
    def num_delayed(self) -> int:
        return len(self._saving)

    def close(self) -> None:
        if self.is_cuda and self._saving:
            self.stream.synchronize()
            if self._scheduler is not None:
                self.step_finished(None, self._scheduler)



class RecomputeCPUOffloadConnector(CPUOffloadConnector):
    """Host copies of the KV of *preempted* requests.

    When the scheduler preempts a request for lack of GPU blocks, everything it computed would be
    recomputed on resume.  This connector copies the request's full blocks (prompt and generated
    tokens) to pinned host memory before they are freed and copies them back when the request is
    scheduled again, so a resume costs a host-to-device copy instead of a prefill.  Host blocks of a
    request are released when it finishes; with ``enable_offload_prefix_caching`` they stay in the
    LRU pool (and finished requests are offloaded too), which adds the prefix-sharing behaviour of the
    plain offload connector.

    Behaviour of the reference's ``RecomputeCPUOffloadConnectorV1``
    (vllm_ascend/distributed/kv_transfer/kv_pool/recompute_cpu_offload/recompute_cpu_offload_connector.py:
    "CPU KV cache preservation for recompute-preempted requests", ``cpu_bytes_to_use`` and
    ``enable_offload_prefix_caching`` options)."""

    def __init__(self, engine_cfg, runner):
        ktc = dict(engine_cfg.kv_transfer_config or {})
        extra = dict(ktc.get("kv_connector_extra_config") or {})
        if "cpu_bytes_to_use" in extra and "cpu_bytes" not in extra:
            extra["cpu_bytes"] = extra["cpu_bytes_to_use"]
            engine_cfg.kv_transfer_config = dict(ktc, kv_connector_extra_config=extra)
        super().__init__(engine_cfg, runner)
        keep = extra.get("enable_offload_prefix_caching", False)
        if not isinstance(keep, bool):
            raise ValueError(f"enable_offload_prefix_caching must be a boolean, got {keep!r}")
        self.keep_finished = keep
        self._owned: dict[str, set] = {}
        self.stats.update(preempted_saved=0, resumed_hits=0)

    def _lookup_tokens(self, req) -> int:
        return req.num_tokens - 1                   # a resumed request also finds its generated tokens

    def _note_owner(self, req, hashes: list) -> None:
        self._owned.setdefault(req.request_id, set()).update(hashes)

    def request_preempted(self, req, block_ids: list) -> bool:
        """Called by the scheduler before it frees a preempted request's blocks.  Returns True when
        the blocks must stay allocated until the copy has finished."""
        before = self.stats["saved_blocks"] + sum(len(hs) for _, _, hs, _ in self._saving)
        delay = self._save_blocks(req, block_ids)
        after = self.stats["saved_blocks"] + sum(len(hs) for _, _, hs, _ in self._saving)
        self.stats["preempted_saved"] += after - before
        return delay

    def update_state_after_alloc(self, req, block_ids: list, num_external_tokens: int) -> None:
        if num_external_tokens > 0 and req.request_id in self._owned:
            self.stats["resumed_hits"] += num_external_tokens // self.block_size
        super().update_state_after_alloc(req, block_ids, num_external_tokens)

    def request_finished(self, req, block_ids: list) -> tuple[bool, Optional[dict]]:
        if self.keep_finished:
            return super().request_finished(req, block_ids)
        # copies still in flight for this request land in the pool first
        if self.is_cuda and any(h in self._owned.get(req.request_id, ()) for _, _, hs, _ in self._saving for h in hs):
            self.stream.synchronize()
            if self._scheduler is not None:
                self.step_finished(None, self._scheduler)
        for h in self._owned.pop(req.request_id, ()):
            hb = self.lru.pop(h, None)
            if hb is not None:
                self.free.append(hb)
        return False, None
