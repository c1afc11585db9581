"""Layer-wise push connector: the prefill engine streams each layer's KV into the decode
engine's cache while the following layers are still computing, so the transfer hides behind
the prefill instead of following it.

Flow (vllm_ascend/distributed/kv_transfer/kv_p2p/mooncake_layerwise_connector.py; the
handshake of docs/.../disaggregated_prefill.md:49-56):
  1. the decode engine receives the request first (``do_remote_prefill`` + ``layerwise``),
     allocates its blocks and publishes them under the request key on its side channel;
  2. the prefill engine receives the same prompt with ``do_remote_decode``, ``layerwise`` and
     ``push_to`` (decode engine id / host / port / key), looks the target blocks up, and after
     every layer of every prefill chunk launches one block-copy kernel for that layer's K and V
     on a side stream (same process: direct pointers; same node: the decode arena mapped
     through CUDA IPC, stores over NVLink);
  3. after the last layer it tells the decode engine that the push is complete; the decode
     engine then computes the last prompt token and decodes.
"""
from __future__ import annotations

import time
from typing import Optional

import torch

from ... import _native
from ...logger import logger
from .base import ConnectorMetadata
from .nvlink_connector import _LOCAL_ENGINES, NVLinkConnector, TransferJob
from .side_channel import SideChannelError, request as sc_request


class LayerwiseConnector(NVLinkConnector):
    def __init__(self, engine_cfg, runner):
        super().__init__(engine_cfg, runner)
        self._targets: dict[str, TransferJob] = {}      # decode side: key -> job waiting for a push
        self._pushes: dict[str, dict] = {}              # prefill side: request id -> push state
        self._step_pushes: list[dict] = []
        self._push_done: list[tuple] = []               # (event, request id, state) awaiting completion
        self.stats.update({"pushed_layers": 0, "pushed_requests": 0})
        runner.model.layer_hook = self.save_kv_layer

    # ------------------------------------------------------------------ side channel
    def _handle(self, msg: dict) -> Optional[dict]:
        op = msg.get("op")
        if self.drop_all_messages:
            return None
        if op == "push_target":
            job = self._targets.get(msg["key"])
            if job is None:
                return {"ok": False, "error": "no request is waiting under this key (yet)"}
            return {"ok": True, "blocks": job.local_blocks, "meta": self._meta()}
        if op == "push_done":
            job = self._targets.pop(msg["key"], None)
            if job is not None:
                job.state = "done" if msg.get("success", True) else "failed"
                job.error = msg.get("error")
            return {"ok": True}
        return super()._handle(msg)

    # ------------------------------------------------------------------ decode side
    def update_state_after_alloc(self, req, block_ids: list, num_external_tokens: int) -> None:
        p = req.kv_transfer_params
        if not (p and p.get("layerwise")):
            return super().update_state_after_alloc(req, block_ids, num_external_tokens)
        if num_external_tokens <= 0 or not p.get("do_remote_prefill"):
            return
        p["do_remote_prefill"] = False
        last = (req.num_prompt_tokens - 1 + self.block_size - 1) // self.block_size
        job = TransferJob(req.request_id, list(block_ids[:last]), [], dict(p), state="inflight")
        job.t_start = time.monotonic()
        self._targets[p.get("key", req.request_id)] = job
        self._inflight[req.request_id] = job

    def get_num_new_matched_tokens(self, req, num_computed_tokens: int) -> tuple[int, bool]:
        p = req.kv_transfer_params
        if p and p.get("layerwise") and p.get("do_remote_prefill") and self.role != "kv_producer":
            n = req.num_prompt_tokens - 1          # a pushed prefix cannot be mixed with a cached one
            return (n, True) if n > 0 and num_computed_tokens == 0 else (0, False)
        return super().get_num_new_matched_tokens(req, num_computed_tokens)

    def _poll(self, job: TransferJob) -> None:
        if job.params.get("layerwise"):
            if job.state == "inflight" and time.monotonic() - job.t_start > self.abort_timeout_s:
                job.state, job.error = "failed", "the prefill engine never pushed this request"
            return
        super()._poll(job)

    def _notify_done(self, job: TransferJob) -> None:
        if job.params.get("layerwise"):
            self._targets.pop(job.params.get("key", job.request_id), None)
            return
        super()._notify_done(job)

    # ------------------------------------------------------------------ prefill side
    def _resolve_target(self, req) -> Optional[dict]:
        st = self._pushes.get(req.request_id)
        if st is not None:
            return st
        to = req.kv_transfer_params["push_to"]
        key = (str(to["engine_id"]), 0)
        local = _LOCAL_ENGINES.get(key)
        try:
            if local is not None:
                reply = local._handle({"op": "push_target", "key": to["key"]})
                if not reply.get("ok"):
                    raise SideChannelError(reply.get("error"))
            else:
                reply = sc_request(to["host"], int(to["port"]), {"op": "push_target", "key": to["key"]},
                                   self.timeout_ms)
        except SideChannelError as e:
            logger.warning("layerwise push of %s: %s", req.request_id, e)
            return None
        meta = reply["meta"]
        if local is not None:
            dsts = [(g.ptrs, g) for g in local.groups]
        else:
            self._remote_meta.setdefault(key, meta)
            dsts = self._ipc_sources(key, self._remote_meta[key])
        st = {"dst_blocks": reply["blocks"], "dsts": dsts, "dst_num_blocks": int(meta["num_blocks"]), "to": to,
              "local": local, "pushed_tokens": 0, "failed": False}
        self._pushes[req.request_id] = st
        return st

    def build_connector_meta(self, scheduler_output) -> Optional[ConnectorMetadata]:
        meta = super().build_connector_meta(scheduler_output)
        self._step_pushes = []
        if self.role == "kv_consumer":
            return meta
        bs = self.block_size
        for req, n in scheduler_output.scheduled:
            p = req.kv_transfer_params
            if not (p and p.get("layerwise") and p.get("do_remote_decode") and p.get("push_to")):
                continue
            if req.num_computed_tokens >= req.num_prompt_tokens:
                continue
            st = self._resolve_target(req)
            if st is None:
                continue
            first = req.num_computed_tokens // bs
            last = min((req.num_computed_tokens + n + bs - 1) // bs, len(st["dst_blocks"]))
            if last > first:
                self._step_pushes.append({"req": req, "state": st, "src": req.block_ids[first:last],
                                          "dst": st["dst_blocks"][first:last],
                                          "final": req.num_computed_tokens + n >= req.num_prompt_tokens})
        return meta

    def save_kv_layer(self, layer_idx: int) -> None:
        """Called by the model after layer ``layer_idx`` wrote its K/V for this step."""
        if not self._step_pushes:
            return
        for job in self._step_pushes:
            self._push_layer(job, layer_idx)
        self.stats["pushed_layers"] += 1

    def _push_layer(self, job: dict, layer_idx: int) -> None:
        st = job["state"]
        k_src, v_src = self.runner.kv_caches[layer_idx]
        n = len(job["src"])
        if not self.is_cuda:
            local = st["local"]
            if local is None:
                st["failed"] = True
                return
            s = torch.as_tensor(job["src"], dtype=torch.long)
            d = torch.as_tensor(job["dst"], dtype=torch.long)
            kd, vd = local.runner.kv_caches[layer_idx]
            kd[d] = k_src[s]
            vd[d] = v_src[s]
            return
        dev = k_src.device
        ev = torch.cuda.Event()
        ev.record()                                   # layer's KV writes are in the compute stream
        self.stream.wait_event(ev)
        lib = _native.lib()
        with torch.cuda.stream(self.stream):
            if "sb" not in job:
                job["sb"] = torch.tensor(job["src"], dtype=torch.int32).pin_memory().to(dev, non_blocking=True)
                job["db"] = torch.tensor(job["dst"], dtype=torch.int32).pin_memory().to(dev, non_blocking=True)
            # position of this layer's K and V inside the tensor groups
            for (dst_ptrs, dg), g in zip(st["dsts"], self.groups):
                for which, t in ((0, k_src), (1, v_src)):
                    ti = 2 * layer_idx + which
                    if ti not in g.indices:
                        continue
                    j = g.indices.index(ti)
                    rc = lib.b200_kv_block_copy(
                        g.ptrs.data_ptr() + 8 * j, dst_ptrs.data_ptr() + 8 * j, job["sb"].data_ptr(),
                        job["db"].data_ptr(), n, 1, self.block_size, g.hd_bytes, g.heads, 0, 0,
                        g.strides[0], g.strides[1], g.strides[2], dg.strides[0], dg.strides[1], dg.strides[2],
                        int(self.tensors[0].shape[0]), st["dst_num_blocks"],
                        _native.status_word(dev).data_ptr(), self.stream.cuda_stream)
                    _native.check(rc, "kv_block_copy (layer push)")
                    self.stats["bytes"] += n * self.block_size * g.heads * g.hd_bytes

    def step_finished(self, scheduler_output, scheduler) -> None:
        super().step_finished(scheduler_output, scheduler)
        for job in self._step_pushes:
            if job["final"]:
                ev = None
                if self.is_cuda:
                    ev = torch.cuda.Event()
                    ev.record(self.stream)
                self._push_done.append((ev, job["req"].request_id, job["state"]))
        self._step_pushes = []
        still = []
        for ev, rid, st in self._push_done:
            if ev is not None and not ev.query():
                still.append((ev, rid, st))
                continue
            self._finish_push(rid, st)
        self._push_done = still

    def _finish_push(self, rid: str, st: dict) -> None:
        self._pushes.pop(rid, None)
        msg = {"op": "push_done", "key": st["to"]["key"], "success": not st["failed"]}
        if st["local"] is not None:
            st["local"]._handle(msg)
        else:
            self._pool.submit(self._send_done, st["to"]["host"], int(st["to"]["port"]), msg)
        self.stats["pushed_requests"] += 1

    def request_finished(self, req, block_ids: list):
        p = req.kv_transfer_params
        if p and p.get("layerwise") and p.get("do_remote_decode"):
            # the KV left on the side stream while the layers ran: once those copies are complete
            # the decode engine may start and the blocks can be reused right away
            st = self._pushes.get(req.request_id)
            if st is not None:
                if self.is_cuda:
                    self.stream.synchronize()
                self._step_pushes = [j for j in self._step_pushes if j["req"] is not req]
                self._push_done = [x for x in self._push_done if x[1] != req.request_id]
                self._finish_push(req.request_id, st)
            return False, {"do_remote_prefill": False, "layerwise": True, "pushed": st is not None}
        return super().request_finished(req, block_ids)

    def flush(self) -> None:
        if self.is_cuda:
            self.stream.synchronize()
        for ev, rid, st in self._push_done:
            self._finish_push(rid, st)
        self._push_done = []
