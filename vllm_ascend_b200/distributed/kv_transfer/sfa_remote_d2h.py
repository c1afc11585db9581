"""P→D connector for sparse-attention decode engines that keep their KV on the host.

The decode engine runs with ``sparse_kv_offload_config`` (latent KV host-resident, per-sequence
device pools, paged index keys).  Pulling a prompt's KV therefore has two destinations: the latent /
rope-key rows go straight into the sequence's pinned host store and never occupy device KV blocks,
the index keys go into the engine's paged index cache.  The prefill engine is an ordinary
sparse-attention engine; it serves the rows of a finished request layer by layer and frees its
blocks when the decode side acknowledges, exactly like the block connector it extends.

Role of the reference's remote-D2H connector for PD-disaggregated sparse attention
(vllm_ascend/distributed/kv_transfer/kv_p2p/sfa_pd_rd2h/: decode pulls the bulk MLA KV into the
CPU offload pool, the indexer KV lands in HBM).
"""
from __future__ import annotations

import torch

from .nvlink_connector import _LOCAL_ENGINES, NVLinkConnector, TransferJob
from .side_channel import SideChannelError
from .side_channel import request as sc_request


class SfaRemoteD2HConnector(NVLinkConnector):
    def __init__(self, engine_cfg, runner):
        if not runner.mcfg.use_sparse:
            raise ValueError("SfaRemoteD2HConnector serves sparse-attention (index_topk) models")
        super().__init__(engine_cfg, runner)
        self.stats.update({"host_rows": 0})

    # ------------------------------------------------------------------ decode (consumer) side
    def update_state_after_alloc(self, req, block_ids: list, num_external_tokens: int) -> None:
        n_before = len(self._pending)
        super().update_state_after_alloc(req, block_ids, num_external_tokens)
        if len(self._pending) > n_before:
            job = self._pending[-1]
            job.local_row, job.num_tokens = int(req.row), int(req.num_prompt_tokens - 1)
            if self.runner.sparse_offload is None and job.state != "failed":
                job.state, job.error = "failed", "the decode engine runs without sparse_kv_offload_config"

    def _launch(self, job: TransferJob) -> None:
        p = job.params
        remote_tp = int(p.get("remote_tp_size", 1))
        src_rank = self.tp_rank % remote_tp                 # the latent cache is replicated over TP
        key = (str(p.get("remote_engine_id")), src_rank)
        host, port = p.get("remote_host", "127.0.0.1"), int(p.get("remote_port", 0)) + src_rank
        job.pulled_from.append(key if key in _LOCAL_ENGINES else (host, port))
        job.futures.append(self._pool.submit(self._pull_sparse, job, key, host, port))

    def _pull_sparse(self, job: TransferJob, key, host, port) -> None:
        msg = {"op": "read_sparse", "request_id": job.params.get("remote_request_id"),
               "block_ids": list(job.remote_blocks), "num_tokens": job.num_tokens}
        local = _LOCAL_ENGINES.get(key)
        reply = local._serve_sparse(msg) if local is not None else sc_request(host, port, msg, self.timeout_ms)
        if not reply.get("ok"):
            raise SideChannelError(reply.get("error", "read_sparse failed"))
        layers = reply["layers"]
        caches, stores = self.runner.kv_caches, self.runner.sparse_offload
        if len(layers) != len(stores):
            raise SideChannelError("prefill and decode engines have different layer counts")
        n, bs = job.num_tokens, self.block_size
        pos = torch.arange(n)
        slots = torch.as_tensor(job.local_blocks, dtype=torch.long)[pos // bs] * bs + pos % bs
        for (lat, pe, idx), store, cache in zip(layers, stores, caches):
            dt = store.host.dtype
            lat_t = torch.frombuffer(bytearray(lat), dtype=torch.uint8).view(dt).view(n, store.dc)
            pe_t = torch.frombuffer(bytearray(pe), dtype=torch.uint8).view(dt).view(n, store.dr)
            store.host[job.local_row, :n] = torch.cat([lat_t, pe_t], dim=-1)           # remote -> host, no device hop
            ic = cache[2]
            idx_t = torch.frombuffer(bytearray(idx), dtype=torch.uint8).view(ic.dtype).view(n, ic.shape[-1])
            ic.view(-1, ic.shape[-1])[slots.to(ic.device)] = idx_t.to(ic.device)
            self.stats["bytes"] += len(lat) + len(pe) + len(idx)
        if self.is_cuda:
            torch.cuda.current_stream(caches[0][2].device).synchronize()
        self.stats["host_rows"] += n * len(layers)

    # ------------------------------------------------------------------ prefill (producer) side
    def _handle(self, msg: dict):
        if msg.get("op") == "read_sparse" and not self.drop_all_messages:
            return self._serve_sparse(msg)
        return super()._handle(msg)

    def _serve_sparse(self, msg: dict) -> dict:
        rid = msg["request_id"]
        if rid not in self._delayed:
            return {"ok": False, "error": f"request {rid} is not held here (expired or unknown)"}
        n = int(msg["num_tokens"])
        out = []
        for caches in self.runner.kv_caches:
            if len(caches) < 3:
                return {"ok": False, "error": "the prefill engine has no index-key cache"}
            blocks = torch.as_tensor(msg["block_ids"], dtype=torch.long).to(caches[0].device)
            rows = []
            for c in caches[:3]:
                g = c[blocks]                                        # [nb, bs, 1, w]
                rows.append(g.reshape(-1, g.shape[-1])[:n].contiguous().view(torch.uint8).cpu().numpy().tobytes())
            out.append(rows)
        return {"ok": True, "layers": out}
