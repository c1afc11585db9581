"""Disaggregated-prefill KV connector for NVLink/NVSwitch nodes.

A prefill engine keeps the blocks of a finished ``do_remote_decode`` request alive and
returns ``kv_transfer_params`` naming them; the decode engine that receives those
parameters PULLS the blocks straight into its own paged cache and starts decoding after
recomputing only the last prompt token.

Transports, picked per remote engine:
  * ``local`` — both engines live in this process: one gather/scatter kernel.
  * ``ipc``   — same node, other process: the prefill cache arena is mapped through CUDA
    IPC and the same kernel reads it over NVLink (no staging, no CPU copy).
  * ``tcp``   — anything else (other node, CPU tensors): host-staged payload over the side
    channel.

Behavioural parity with vllm_ascend/distributed/kv_transfer/kv_p2p/mooncake_connector.py
(scheduler contract 1843-2001, delayed free 1973-2001 and 361-571, heterogeneous TP head
slices 1271-1296, failure reporting consumed by core/recompute_scheduler.py).
"""
from __future__ import annotations

import ctypes
import queue
import socket
import threading
import time
from concurrent.futures import ThreadPoolExecutor
from ctypes import c_int, c_long, c_void_p
from dataclasses import dataclass, field
from typing import Optional

import numpy as np
import torch

from ... import _native, envs
from ...logger import logger
from .base import ConnectorMetadata, KVConnectorBase, plan_head_slices
from .side_channel import SideChannelError, SideChannelServer, request as sc_request

P, I, L = c_void_p, c_int, c_long
_native.register_signature("b200_kv_block_copy", [P, P, P, P, I, I, I, I, I, I, I, L, L, L, L, L, L, L, L, P, P])
_native.register_signature("b200_copy_blocks", [P, P, I, L, P])

# (engine_id, tp_rank) -> connector, for engines that share this process
_LOCAL_ENGINES: dict[tuple[str, int], "NVLinkConnector"] = {}
_LOCAL_HOSTS = ("127.0.0.1", "localhost", "0.0.0.0")


class KVArena:
    """One ``cudaMalloc`` allocation holding every layer's K/V cache, so a single CUDA IPC
    handle exports the whole cache to decode engines on the same node."""

    def __init__(self, nbytes: int, device: torch.device):
        from ...parallel.symm_mem import _RawCudaBuffer
        lib = _native.lib()
        self.nbytes = (nbytes + 1023) // 1024 * 1024
        p = c_void_p()
        with torch.cuda.device(device):
            _native.check(lib.b200_symm_alloc(self.nbytes, ctypes.byref(p)), "kv arena alloc")
        self.ptr = p.value
        self._keep = _RawCudaBuffer(self.ptr, self.nbytes)
        self.bytes = torch.as_tensor(self._keep, device=device)
        self.bytes.zero_()
        self._offset = 0
        self._handle: Optional[bytes] = None

    def take(self, shape, dtype) -> torch.Tensor:
        n = int(np.prod(shape)) * torch.empty((), dtype=dtype).element_size()
        off = self._offset
        self._offset += (n + 255) // 256 * 256
        if self._offset > self.nbytes:
            raise RuntimeError("KV arena exhausted")
        return self.bytes[off:off + n].view(dtype).view(*shape)

    def ipc_handle(self) -> bytes:
        if self._handle is None:
            h = (ctypes.c_ubyte * 64)()
            _native.check(_native.lib().b200_ipc_get_handle(self.ptr, h), "ipc_get_handle")
            self._handle = bytes(h)
        return self._handle

    @staticmethod
    def bytes_needed(shapes, dtype) -> int:
        e = torch.empty((), dtype=dtype).element_size()
        return sum((int(np.prod(s)) * e + 255) // 256 * 256 for s in shapes)


@dataclass
class TransferJob:
    request_id: str
    local_blocks: list
    remote_blocks: list
    params: dict
    state: str = "queued"            # queued -> inflight -> done | failed
    events: list = field(default_factory=list)
    futures: list = field(default_factory=list)
    error: Optional[str] = None
    t_start: float = 0.0
    pulled_from: list = field(default_factory=list)     # (host, port) to notify when done


@dataclass
class _TensorGroup:
    """Cache tensors with identical geometry; one kernel launch moves a group."""
    indices: list
    heads: int
    hd_bytes: int
    strides: tuple          # bytes: (block, token, head)
    ptrs: Optional[torch.Tensor] = None    # device int64 array of base pointers


def _group_tensors(tensors: list) -> list[_TensorGroup]:
    groups: dict = {}
    for i, t in enumerate(tensors):
        e = t.element_size()
        key = (t.shape[2], t.shape[3] * e, (t.stride(0) * e, t.stride(1) * e, t.stride(2) * e))
        groups.setdefault(key, []).append(i)
    return [_TensorGroup(idx, k[0], k[1], k[2]) for k, idx in groups.items()]


class NVLinkConnector(KVConnectorBase):
    def __init__(self, engine_cfg, runner):
        ktc = dict(engine_cfg.kv_transfer_config or {})
        extra = dict(ktc.get("kv_connector_extra_config") or {})
        self.cfg = engine_cfg
        self.runner = runner
        self.role = ktc.get("kv_role", "kv_both")
        self.engine_id = str(ktc.get("engine_id") or f"engine-{id(self):x}")
        self.host = ktc.get("kv_ip", "127.0.0.1")
        self.base_port = int(ktc.get("kv_port", 0))
        self.transport = extra.get("transport", "auto")
        self.timeout_ms = int(extra.get("side_channel_timeout_ms", 5000))
        self.abort_timeout_s = float(extra.get("abort_timeout_s", envs.VLLM_B200_KV_ABORT_REQUEST_TIMEOUT))
        self.block_size = engine_cfg.cache.block_size
        from ...parallel import state as pstate
        self.tp_group = pstate.get_tp_group()
        self.tp_size = self.tp_group.world_size
        self.tp_rank = self.tp_group.rank_in_group
        self.num_kv_heads = 1 if runner.mcfg.use_mla else runner.mcfg.num_key_value_heads
        # producer state
        self._delayed: dict[str, tuple[list, float]] = {}       # rid -> (block ids, deadline)
        self._done_q: "queue.Queue[tuple[str, int, int]]" = queue.Queue()
        self._done_seen: dict[str, set] = {}
        # consumer state
        self._pending: list[TransferJob] = []
        self._inflight: dict[str, TransferJob] = {}
        self._ready: set[str] = set()
        self._failed: list[str] = []
        self._synced_this_step = False
        self._remote_meta: dict[tuple[str, int], dict] = {}
        self._pool = ThreadPoolExecutor(max_workers=int(extra.get("num_threads", 4)),
                                        thread_name_prefix="kv-pull")
        self.stats = {"pulled_requests": 0, "pulled_blocks": 0, "failed": 0, "bytes": 0,
                      "released": 0, "expired": 0}
        # failure-injection knobs for host-side tests
        self.drop_done_messages = False
        self.drop_all_messages = False
        self.tensors: list[torch.Tensor] = []
        self.groups: list[_TensorGroup] = []
        self.server: Optional[SideChannelServer] = None
        self.stream = None
        self.register_kv_caches(runner.kv_caches)
        port = self.base_port + self.tp_rank if self.base_port else 0
        self.server = SideChannelServer(self.host, port, self._handle)
        self.port = self.server.port
        if not self.base_port:
            self.base_port = self.port - self.tp_rank
        self.server.start()
        _LOCAL_ENGINES[(self.engine_id, self.tp_rank)] = self

    # ------------------------------------------------------------------ caches
    def register_kv_caches(self, kv_caches: list) -> None:
        self.tensors = [t for pair in kv_caches for t in pair]
        self.groups = _group_tensors(self.tensors)
        self.is_cuda = bool(self.tensors) and self.tensors[0].is_cuda
        if self.is_cuda:
            dev = self.tensors[0].device
            self.stream = torch.cuda.Stream(device=dev)
            for g in self.groups:
                g.ptrs = torch.tensor([self.tensors[i].data_ptr() for i in g.indices],
                                      dtype=torch.int64, device=dev)
        self.arena: Optional[KVArena] = getattr(self.runner, "kv_arena", None)

    def _meta(self) -> dict:
        t0 = self.tensors[0]
        m = {"ok": True, "engine_id": self.engine_id, "tp_size": self.tp_size, "tp_rank": self.tp_rank,
             "block_size": self.block_size, "num_blocks": int(t0.shape[0]),
             "num_kv_heads": self.num_kv_heads, "dtype": str(t0.dtype), "cuda": self.is_cuda,
             "device_index": t0.device.index if self.is_cuda else -1,
             "hostname": socket.gethostname(),
             "tensors": [{"heads": int(t.shape[2]), "dim": int(t.shape[3]),
                          "strides": [t.stride(0) * t.element_size(), t.stride(1) * t.element_size(),
                                      t.stride(2) * t.element_size()],
                          "offset": (t.data_ptr() - self.arena.ptr) if self.arena else -1}
                         for t in self.tensors]}
        if self.arena is not None:
            m["ipc_handle"] = self.arena.ipc_handle()
            m["arena_bytes"] = self.arena.nbytes
        return m

    # ------------------------------------------------------------------ side-channel handler
    def _handle(self, msg: dict) -> Optional[dict]:
        if self.drop_all_messages:
            return None
        op = msg.get("op")
        if op == "meta":
            return self._meta()
        if op == "done":
            if self.drop_done_messages:
                return None
            self._done_q.put((msg["request_id"], int(msg.get("from_rank", 0)), int(msg.get("tp_size", 1))))
            return {"ok": True}
        if op == "read":
            return self._serve_read(msg)
        return {"ok": False, "error": f"unknown op {op!r}"}

    def _serve_read(self, msg: dict) -> dict:
        rid = msg["request_id"]
        if rid not in self._delayed:
            return {"ok": False, "error": f"request {rid} is not held here (expired or unknown)"}
        blocks = torch.as_tensor(msg["block_ids"], dtype=torch.long)
        h0, nh = int(msg["head0"]), int(msg["num_heads"])
        payload = []
        if self.is_cuda:
            dev = self.tensors[0].device
            with torch.cuda.device(dev), torch.cuda.stream(self._serve_stream()):
                idx = blocks.to(dev)
                for t in self.tensors:
                    hh0, hn = (h0, nh) if t.shape[2] > 1 else (0, 1)
                    payload.append(t[idx][:, :, hh0:hh0 + hn].contiguous().view(torch.uint8).cpu())
                torch.cuda.current_stream().synchronize()
        else:
            for t in self.tensors:
                hh0, hn = (h0, nh) if t.shape[2] > 1 else (0, 1)
                payload.append(t[blocks][:, :, hh0:hh0 + hn].contiguous().view(torch.uint8))
        return {"ok": True, "data": [p.numpy().tobytes() for p in payload]}

    def _serve_stream(self):
        if not hasattr(self, "_srv_stream"):
            self._srv_stream = torch.cuda.Stream(device=self.tensors[0].device)
        return self._srv_stream

    # ------------------------------------------------------------------ scheduler side
    def get_num_new_matched_tokens(self, req, num_computed_tokens: int) -> tuple[int, bool]:
        p = req.kv_transfer_params
        if not p or not p.get("do_remote_prefill") or self.role == "kv_producer":
            return 0, False
        # everything but the last prompt token comes from the prefill engine; the last token is
        # recomputed locally so this engine samples the first output token itself
        n = req.num_prompt_tokens - 1 - num_computed_tokens
        if n <= 0 or not p.get("remote_block_ids"):
            return 0, False
        return n, True

    def update_state_after_alloc(self, req, block_ids: list, num_external_tokens: int) -> None:
        p = req.kv_transfer_params
        if num_external_tokens <= 0 or not p or not p.get("do_remote_prefill"):
            return
        p["do_remote_prefill"] = False          # consumed: never matched again
        first = req.num_cached_tokens // self.block_size
        last = (req.num_prompt_tokens - 1 + self.block_size - 1) // self.block_size
        remote = list(p["remote_block_ids"])
        job = TransferJob(req.request_id, list(block_ids[first:last]), remote[first:last], dict(p))
        if int(p.get("remote_block_size", self.block_size)) != self.block_size:
            job.state, job.error = "failed", "prefill and decode engines use different block sizes"
        elif len(job.remote_blocks) != len(job.local_blocks):
            job.state, job.error = "failed", "remote block list does not cover the prompt"
        self._pending.append(job)
        self._inflight[req.request_id] = job

    def build_connector_meta(self, scheduler_output) -> Optional[ConnectorMetadata]:
        self._synced_this_step = False
        meta = ConnectorMetadata()
        meta.reqs_to_recv = {j.request_id: j for j in self._pending}
        meta.reqs_to_send = {rid: b for rid, (b, _) in self._delayed.items()}
        return meta

    def request_finished(self, req, block_ids: list) -> tuple[bool, Optional[dict]]:
        from ...engine.request import RequestStatus
        p = req.kv_transfer_params
        job = self._inflight.pop(req.request_id, None)
        if job is not None:          # aborted while its KV was still being pulled
            for fut in job.futures:  # the blocks go back to the pool: nothing may still write them
                try:
                    fut.result(timeout=self.timeout_ms / 1000)
                except Exception:
                    pass
            for ev in job.events:
                ev.synchronize()
            self._notify_done(job)
        if not p or not p.get("do_remote_decode") or self.role == "kv_consumer":
            return False, None
        if req.status != RequestStatus.FINISHED_LENGTH or not block_ids:
            return False, None       # stopped/aborted during prefill: nothing worth handing over
        nblk = (req.num_prompt_tokens + self.block_size - 1) // self.block_size
        keep = list(block_ids[:nblk])
        self._delayed[req.request_id] = (list(block_ids), time.monotonic() + self.abort_timeout_s)
        out = {"do_remote_prefill": True, "do_remote_decode": False, "remote_block_ids": keep,
               "remote_engine_id": self.engine_id, "remote_host": self.host,
               "remote_port": self.base_port, "remote_tp_size": self.tp_size,
               "remote_pcp_size": 1, "remote_dcp_size": 1, "remote_block_size": self.block_size,
               "remote_request_id": req.request_id, "num_prompt_blocks": nblk,
               "last_token_id": int(req.output_token_ids[-1]) if req.output_token_ids else None}
        return True, out

    def is_ready(self, req) -> bool:
        self._sync_step()
        if req.request_id in self._ready:
            self._ready.discard(req.request_id)
            return True
        return False

    def take_failed_requests(self) -> list[str]:
        self._sync_step()
        out, self._failed = self._failed, []
        return out

    def _sync_step(self) -> None:
        """Once per scheduling step: poll the transfers and, under TP, make every rank see the
        same set of finished/failed requests so the SPMD schedulers stay in lock-step."""
        if self._synced_this_step or not self._inflight:
            return
        self._synced_this_step = True
        done, failed = [], []
        for rid, job in self._inflight.items():
            self._poll(job)
            if job.state == "done":
                done.append(rid)
            elif job.state == "failed":
                failed.append(rid)
        if self.tp_size > 1:
            gathered = self.tp_group.all_gather_object((done, failed))
            failed_all = set().union(*[set(f) for _, f in gathered])
            done_all = set(gathered[0][0]).intersection(*[set(d) for d, _ in gathered[1:]])
            # a rank that finished a pull another rank failed must not keep its result
            done, failed = sorted(done_all - failed_all), sorted(failed_all)
        for rid in failed:
            job = self._inflight.pop(rid)
            logger.warning("KV pull for %s failed: %s", rid, job.error or "failed on another rank")
            self._notify_done(job)          # let the prefill engine free its copy
            self._failed.append(rid)
            self.stats["failed"] += 1
        for rid in done:
            job = self._inflight.pop(rid)
            self._notify_done(job)
            self._ready.add(rid)
            self.stats["pulled_requests"] += 1
            self.stats["pulled_blocks"] += len(job.local_blocks)

    def _poll(self, job: TransferJob) -> None:
        if job.state != "inflight":
            return
        for fut in job.futures:
            if not fut.done():
                return
            err = fut.exception()
            if err is not None:
                job.state, job.error = "failed", f"{type(err).__name__}: {err}"
                return
        if all(e.query() for e in job.events):
            job.state = "done"

    def _notify_done(self, job: TransferJob) -> None:
        targets = job.pulled_from or self._targets_of(job.params)
        msg = {"op": "done", "request_id": job.params.get("remote_request_id", job.request_id),
               "from_rank": self.tp_rank, "tp_size": self.tp_size}
        for key in targets:
            local = _LOCAL_ENGINES.get(key) if isinstance(key[0], str) else None
            if local is not None:
                if not (local.drop_done_messages or local.drop_all_messages):
                    local._done_q.put((msg["request_id"], self.tp_rank, self.tp_size))
                continue
            host, port = key
            self._pool.submit(self._send_done, host, port, msg)

    def _send_done(self, host, port, msg) -> None:
        try:
            sc_request(host, port, msg, self.timeout_ms)
        except SideChannelError as e:      # the producer's own timeout frees the blocks
            logger.warning("could not tell %s:%s that %s was pulled: %s", host, port, msg["request_id"], e)

    def _targets_of(self, params: dict) -> list:
        out = []
        for src_rank, *_ in self._slices(int(params.get("remote_tp_size", 1))):
            key = (str(params.get("remote_engine_id")), src_rank)
            out.append(key if key in _LOCAL_ENGINES
                       else (params.get("remote_host", "127.0.0.1"), int(params.get("remote_port", 0)) + src_rank))
        return out

    def _slices(self, remote_tp: int):
        if self.num_kv_heads <= 1 and self.runner.mcfg.use_mla:
            return [(self.tp_rank % remote_tp, 0, 0, 1)]       # latent cache is replicated
        return plan_head_slices(remote_tp, self.tp_size, self.num_kv_heads, self.tp_rank)

    # ------------------------------------------------------------------ worker side
    def start_load_kv(self, scheduler_output) -> None:
        jobs, self._pending = self._pending, []
        for job in jobs:
            if job.state == "failed":
                continue
            job.t_start = time.monotonic()
            job.state = "inflight"
            try:
                self._launch(job)
            except Exception as e:        # an unreachable or inconsistent peer fails the pull, not the engine
                job.state, job.error = "failed", f"{type(e).__name__}: {e}"

    def _launch(self, job: TransferJob) -> None:
        p = job.params
        remote_tp = int(p.get("remote_tp_size", 1))
        eid = str(p.get("remote_engine_id"))
        host, port0 = p.get("remote_host", "127.0.0.1"), int(p.get("remote_port", 0))
        for src_rank, src_h0, dst_h0, nh in self._slices(remote_tp):
            key = (eid, src_rank)
            mode, local = self._resolve_mode(key, host, port0 + src_rank)
            job.pulled_from.append(key if local is not None else (host, port0 + src_rank))
            if mode == "local":
                if local is None:
                    raise SideChannelError(f"engine {eid} rank {src_rank} is not in this process")
                srcs = [(g.ptrs, g) for g in local.groups]
                self._copy_kernel(job, srcs, int(local.tensors[0].shape[0]), src_h0, dst_h0, nh)
            elif mode == "ipc":
                meta = self._get_meta(key, host, port0 + src_rank)
                srcs = self._ipc_sources(key, meta)
                self._copy_kernel(job, srcs, int(meta["num_blocks"]), src_h0, dst_h0, nh)
            else:
                job.futures.append(self._pool.submit(self._pull_tcp, job, host, port0 + src_rank, src_h0, dst_h0, nh))

    def _resolve_mode(self, key, host, port):
        """("local" | "ipc" | "tcp", connector of the source when it lives in this process)."""
        local = _LOCAL_ENGINES.get(key)
        mode = self.transport
        if mode == "auto":
            mode = "local" if (local is not None and local.is_cuda == self.is_cuda and self.is_cuda) else None
        if mode is None:
            meta = self._get_meta(key, host, port)
            same_node = meta.get("hostname") == socket.gethostname()
            mode = "ipc" if (self.is_cuda and meta.get("cuda") and same_node and meta.get("ipc_handle")
                             and local is None) else "tcp"
        return mode, local

    def _get_meta(self, key, host, port) -> dict:
        meta = self._remote_meta.get(key)
        if meta is None:
            local = _LOCAL_ENGINES.get(key)
            meta = local._meta() if local is not None else sc_request(host, port, {"op": "meta"}, self.timeout_ms)
            if int(meta["block_size"]) != self.block_size:
                raise SideChannelError("prefill and decode engines use different block sizes")
            if len(meta["tensors"]) != len(self.tensors):
                raise SideChannelError("prefill and decode engines hold different numbers of cache tensors")
            self._remote_meta[key] = meta
        return meta

    def _ipc_sources(self, key, meta) -> list:
        cached = meta.get("_sources")
        if cached is not None:
            return cached
        buf = (ctypes.c_ubyte * 64).from_buffer_copy(meta["ipc_handle"])
        q = c_void_p()
        with torch.cuda.device(self.tensors[0].device):
            _native.check(_native.lib().b200_ipc_open(buf, ctypes.byref(q)), f"ipc_open({key})")
        meta["_base"] = q.value
        srcs = []
        for g in self.groups:
            tm = [meta["tensors"][i] for i in g.indices]
            rg = _TensorGroup(g.indices, tm[0]["heads"], g.hd_bytes, tuple(tm[0]["strides"]))
            if any(tuple(t["strides"]) != rg.strides or t["heads"] != rg.heads for t in tm):
                raise SideChannelError("remote cache tensors of one group differ in geometry")
            rg.ptrs = torch.tensor([q.value + t["offset"] for t in tm], dtype=torch.int64,
                                   device=self.tensors[0].device)
            srcs.append((rg.ptrs, rg))
        meta["_sources"] = srcs
        return srcs

    def _copy_kernel(self, job: TransferJob, srcs: list, src_num_blocks: int, src_h0, dst_h0, nh) -> None:
        dev = self.tensors[0].device
        n = len(job.local_blocks)
        if n == 0:
            return
        lib = _native.lib()
        # the compute stream may still be writing other blocks of the cache, never these ones:
        # the pull only has to start after the blocks were allocated, which is host-side
        with torch.cuda.device(dev), torch.cuda.stream(self.stream):
            sb = torch.tensor(job.remote_blocks, dtype=torch.int32).pin_memory().to(dev, non_blocking=True)
            db = torch.tensor(job.local_blocks, dtype=torch.int32).pin_memory().to(dev, non_blocking=True)
            status = _native.status_word(dev)
            for (src_ptrs, sg), g in zip(srcs, self.groups):
                h_s0, h_d0, h_n = (src_h0, dst_h0, nh) if g.heads > 1 or sg.heads > 1 else (0, 0, 1)
                rc = lib.b200_kv_block_copy(
                    src_ptrs.data_ptr(), g.ptrs.data_ptr(), sb.data_ptr(), db.data_ptr(), n, len(g.indices),
                    self.block_size, g.hd_bytes, h_n, h_s0, h_d0,
                    sg.strides[0], sg.strides[1], sg.strides[2], g.strides[0], g.strides[1], g.strides[2],
                    src_num_blocks, int(self.tensors[0].shape[0]), status.data_ptr(),
                    self.stream.cuda_stream)
                _native.check(rc, "kv_block_copy")
                self.stats["bytes"] += n * len(g.indices) * self.block_size * h_n * g.hd_bytes
            ev = torch.cuda.Event()
            ev.record(self.stream)
            job.events.append(ev)
            job._keep = (sb, db)

    def _pull_tcp(self, job: TransferJob, host, port, src_h0, dst_h0, nh) -> None:
        reply = sc_request(host, port, {"op": "read", "request_id": job.params.get("remote_request_id"),
                                        "block_ids": list(job.remote_blocks), "head0": src_h0,
                                        "num_heads": nh}, self.timeout_ms)
        data = reply["data"]
        if len(data) != len(self.tensors):
            raise SideChannelError("payload does not match the local cache")
        idx = torch.as_tensor(job.local_blocks, dtype=torch.long)
        n = len(job.local_blocks)
        ctx = torch.cuda.stream(self.stream) if self.is_cuda else _nullctx()
        if self.is_cuda:
            torch.cuda.set_device(self.tensors[0].device)
        with ctx:
            for t, raw in zip(self.tensors, data):
                d0, hn = (dst_h0, nh) if t.shape[2] > 1 else (0, 1)
                src = torch.frombuffer(bytearray(raw), dtype=torch.uint8).view(t.dtype) \
                    .view(n, t.shape[1], hn, t.shape[3])
                t[idx.to(t.device), :, d0:d0 + hn] = src.to(t.device)
                self.stats["bytes"] += len(raw)
            if self.is_cuda:
                self.stream.synchronize()

    def step_finished(self, scheduler_output, scheduler) -> None:
        """Producer housekeeping after every engine step: free the blocks of requests every
        decode rank has pulled, and of requests nobody claimed before the abort timeout."""
        if not self._delayed:
            while not self._done_q.empty():
                self._done_q.get_nowait()
            return
        fresh = []
        while True:
            try:
                fresh.append(self._done_q.get_nowait())
            except queue.Empty:
                break
        now = time.monotonic()
        expired = [rid for rid, (_, dl) in self._delayed.items() if now > dl]
        if self.tp_size > 1:
            gathered = self.tp_group.all_gather_object((fresh, expired))
            fresh = [x for f, _ in gathered for x in f]
            expired = list(gathered[0][1])            # rank 0's clock decides
        for rid, from_rank, peer_tp in fresh:
            seen = self._done_seen.setdefault(rid, set())
            seen.add(from_rank)
            if len(seen) >= peer_tp and rid in self._delayed:
                blocks, _ = self._delayed.pop(rid)
                scheduler.pool.free(blocks)
                self._done_seen.pop(rid, None)
                self.stats["released"] += 1
        for rid in expired:
            if rid in self._delayed:
                blocks, _ = self._delayed.pop(rid)
                scheduler.pool.free(blocks)
                self._done_seen.pop(rid, None)
                self.stats["expired"] += 1
                logger.warning("no decode engine claimed the KV of %s within %.0f s; freed", rid, self.abort_timeout_s)

    def reap(self, scheduler) -> None:
        """Run the producer housekeeping outside a step (an idle prefill engine)."""
        self.step_finished(None, scheduler)

    @property
    def num_delayed(self) -> int:
        return len(self._delayed)

    def close(self) -> None:
        _LOCAL_ENGINES.pop((self.engine_id, self.tp_rank), None)
        if self.server is not None:
            self.server.stop()
        self._pool.shutdown(wait=False)
        lib = _native.lib() if self.is_cuda else None
        for meta in self._remote_meta.values():
            if meta.get("_base") and lib is not None:
                lib.b200_ipc_close(meta["_base"])
        self._remote_meta.clear()


class _nullctx:
    def __enter__(self):
        return self

    def __exit__(self, *a):
        return False
