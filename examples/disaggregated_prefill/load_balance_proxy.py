"""Load-aware proxy for disaggregated prefill / decode instances, with elastic instance pools.

    python examples/disaggregated_prefill/load_balance_proxy.py --port 9000 \
        --prefill http://127.0.0.1:8100 --prefill http://127.0.0.1:8101 \
        --decode http://127.0.0.1:8200 --decode http://127.0.0.1:8201

What it adds over the round-robin ``proxy.py``:

* **Least-loaded placement.**  Each instance carries a load score: a prefill instance is charged
  ``len(prompt)`` while it computes (prefill cost grows with the prompt), a decode instance
  ``len(prompt) + max_tokens`` while the request lives there (KV it has to hold).  A request goes to
  the instance with the smallest score; ties break by arrival order.
* **Streaming.**  ``"stream": true`` requests are relayed chunk by chunk (server-sent events) from the
  decode instance.
* **Retry on another instance.**  A prefill or decode instance that fails a request (connection error or
  5xx) is marked suspect, the request is retried on the next-best instance (bounded), and the suspect
  is probed in the background before it takes traffic again.
* **Elastic pools.**  ``POST /instances/add`` / ``POST /instances/remove`` change the pools at run
  time; a new instance joins a waiting list and becomes schedulable once its ``/health`` answers; a
  removed instance finishes the requests it has and receives no new ones.
* ``GET /status`` shows every instance with role, state, load and counters.

Role and flow of the reference's load-balancing proxies
(examples/disaggregated_prefill_v1/load_balance_proxy_server_example.py: request-length scores, heap of
instances per role, instance add / remove with a waiting list and health retries, SSE relay).
"""
from __future__ import annotations

import argparse
import itertools
import threading
from dataclasses import dataclass, field
from typing import Iterator, Optional

import requests
import uvicorn
from fastapi import FastAPI, HTTPException
from fastapi.responses import StreamingResponse

ACTIVE, WAITING, SUSPECT, DRAINING = "active", "waiting", "suspect", "draining"


@dataclass
class Instance:
    url: str
    role: str                       # "prefill" | "decode"
    state: str = ACTIVE
    load: float = 0.0
    inflight: int = 0
    served: int = 0
    failed: int = 0
    order: int = 0                  # arrival order, tie-break
    probes: int = 0
    tags: dict = field(default_factory=dict)


def prefill_score(prompt_len: int) -> float:
    return float(max(1, prompt_len))


def decode_score(prompt_len: int, max_tokens: int) -> float:
    return float(max(1, prompt_len + max_tokens))


class Pools:
    """Thread-safe instance table with least-loaded selection."""

    def __init__(self, prefill: list[str], decode: list[str]):
        self._lock = threading.Lock()
        self._order = itertools.count()
        self.instances: dict[str, Instance] = {}
        for u in prefill:
            self._add(u, "prefill", ACTIVE)
        for u in decode:
            self._add(u, "decode", ACTIVE)

    def _add(self, url: str, role: str, state: str) -> Instance:
        inst = Instance(url.rstrip("/"), role, state, order=next(self._order))
        self.instances[inst.url] = inst
        return inst

    # ------------------------------------------------------------------ selection
    def acquire(self, role: str, load: float, exclude: tuple = ()) -> Optional[Instance]:
        with self._lock:
            cands = [i for i in self.instances.values()
                     if i.role == role and i.state == ACTIVE and i.url not in exclude]
            if not cands:
                return None
            best = min(cands, key=lambda i: (i.load, i.order))
            best.load += load
            best.inflight += 1
            return best

    def release(self, inst: Instance, load: float, ok: bool) -> None:
        with self._lock:
            inst.load = max(0.0, inst.load - load)
            inst.inflight = max(0, inst.inflight - 1)
            if ok:
                inst.served += 1
            else:
                inst.failed += 1
                if inst.state == ACTIVE:
                    inst.state = SUSPECT
            if inst.state == DRAINING and inst.inflight == 0:
                self.instances.pop(inst.url, None)

    # ------------------------------------------------------------------ membership
    def add(self, role: str, url: str) -> str:
        if role not in ("prefill", "decode"):
            raise ValueError("role must be 'prefill' or 'decode'")
        with self._lock:
            url = url.rstrip("/")
            if url in self.instances:
                if self.instances[url].state == DRAINING:
                    self.instances[url].state = WAITING
                return self.instances[url].state
            return self._add(url, role, WAITING).state

    def remove(self, url: str) -> bool:
        with self._lock:
            inst = self.instances.get(url.rstrip("/"))
            if inst is None:
                return False
            if inst.inflight == 0:
                self.instances.pop(inst.url)
            else:
                inst.state = DRAINING
            return True

    def probe_pending(self, check, max_probes: int = 0) -> None:
        """Health-check waiting and suspect instances; healthy ones become active.  With
        ``max_probes`` > 0 a waiting instance that never answered is dropped after that many tries."""
        with self._lock:
            pending = [i for i in self.instances.values() if i.state in (WAITING, SUSPECT)]
        for inst in pending:
            ok = check(inst.url)
            with self._lock:
                if inst.url not in self.instances or inst.state not in (WAITING, SUSPECT):
                    continue
                inst.probes += 1
                if ok:
                    inst.state, inst.probes = ACTIVE, 0
                elif max_probes and inst.state == WAITING and inst.probes >= max_probes:
                    self.instances.pop(inst.url)

    def snapshot(self) -> list[dict]:
        with self._lock:
            return [dict(url=i.url, role=i.role, state=i.state, load=i.load, inflight=i.inflight, served=i.served,
                         failed=i.failed) for i in sorted(self.instances.values(), key=lambda x: x.order)]


def _health(url: str, timeout: float = 3.0) -> bool:
    try:
        return requests.get(url + "/health", timeout=timeout).status_code == 200
    except requests.RequestException:
        return False


def _prompt_len(body: dict) -> int:
    p = body.get("prompt")
    if isinstance(p, list):
        return len(p)
    if isinstance(p, str):
        return max(1, len(p) // 4)          # rough token estimate for text prompts
    msgs = body.get("messages")
    if isinstance(msgs, list):
        return max(1, sum(len(str(m.get("content", ""))) for m in msgs) // 4)
    return 1


def build_proxy(prefill_urls: list[str], decode_urls: list[str], timeout: float = 600.0, max_retries: int = 2,
                probe_interval: float = 1.0, max_probes: int = 0, max_recompute_hops: int = 4) -> FastAPI:
    app = FastAPI(title="pd-load-balance-proxy")
    pools = Pools(prefill_urls, decode_urls)
    app.state.pools = pools
    stats = {"recomputed": 0}
    app.state.stats = stats
    stop = threading.Event()

    def prober():
        while not stop.wait(probe_interval):
            pools.probe_pending(_health, max_probes)

    threading.Thread(target=prober, daemon=True).start()
    app.state.stop = stop

    def run_prefill(body: dict, n_prompt: int, path: str) -> dict:
        """max_tokens=1 on the least-loaded prefill instance; returns the kv_transfer_params."""
        load, tried = prefill_score(n_prompt), []
        for _ in range(max_retries + 1):
            inst = pools.acquire("prefill", load, tuple(tried))
            if inst is None:
                break
            ok = False
            try:
                pre = dict(body, max_tokens=1, stream=False, kv_transfer_params={"do_remote_decode": True})
                r = requests.post(inst.url + path, json=pre, timeout=timeout)
                if r.status_code == 200:
                    ok = True
                    return r.json().get("kv_transfer_params")
                if r.status_code < 500:              # the request itself is wrong: no point in retrying
                    ok = True
                    raise HTTPException(r.status_code, f"prefill instance: {r.text}")
            except requests.RequestException:
                pass
            finally:
                pools.release(inst, load, ok)
            tried.append(inst.url)
        raise HTTPException(503, f"no prefill instance could serve the request (tried {tried})")

    def relay_stream(r: requests.Response, inst: Instance, load: float) -> Iterator[bytes]:
        ok = False
        try:
            for chunk in r.iter_content(chunk_size=None):
                if chunk:
                    yield chunk
            ok = True
        finally:
            r.close()
            pools.release(inst, load, ok)

    def run_decode(body: dict, ktp, n_prompt: int, path: str):
        load, tried = decode_score(n_prompt, int(body.get("max_tokens") or 16)), []
        stream = bool(body.get("stream"))
        for _ in range(max_retries + 1):
            inst = pools.acquire("decode", load, tuple(tried))
            if inst is None:
                break
            handed_over = False
            ok = False
            try:
                dec = dict(body, kv_transfer_params=ktp)
                r = requests.post(inst.url + path, json=dec, timeout=timeout, stream=stream)
                if r.status_code == 200:
                    if stream:
                        handed_over = True           # released when the relay ends
                        return StreamingResponse(relay_stream(r, inst, load), media_type="text/event-stream")
                    ok = True
                    return r.json()
                if r.status_code < 500:
                    ok = True
                    raise HTTPException(r.status_code, f"decode instance: {r.text}")
            except requests.RequestException:
                pass
            finally:
                if not handed_over:
                    pools.release(inst, load, ok)
            tried.append(inst.url)
        raise HTTPException(503, f"no decode instance could serve the request (tried {tried})")

    def handle(body: dict, path: str):
        n_prompt = _prompt_len(body)
        ktp = run_prefill(body, n_prompt, path)
        out = run_decode(body, ktp, n_prompt, path)
        # A decode instance under KV pressure hands a request back (stop_reason "recomputed") with the
        # tokens it produced: continue from prompt + those tokens through a fresh prefill, and join
        # the pieces.  (Streaming responses are relayed as they are: the client sees the stop reason.)
        done_ids: list = []
        done_text = ""
        hops = 0
        while isinstance(out, dict) and path == "/v1/completions" and hops < max_recompute_hops:
            ch = (out.get("choices") or [{}])[0]
            if ch.get("stop_reason") != "recomputed" or "prompt_token_ids" not in out:
                break
            hops += 1
            stats["recomputed"] += 1
            done_ids += list(ch.get("token_ids") or [])
            done_text += ch.get("text") or ""
            left = int(body.get("max_tokens") or 16) - len(done_ids)
            if left <= 0:
                ch["finish_reason"], ch["stop_reason"] = "length", None
                break
            again = dict(body, prompt=list(out["prompt_token_ids"]) + list(ch.get("token_ids") or []), max_tokens=left)
            again.pop("kv_transfer_params", None)
            n2 = _prompt_len(again)
            out = run_decode(again, run_prefill(again, n2, path), n2, path)
            body = dict(again, max_tokens=int(body.get("max_tokens") or 16))
        if done_ids and isinstance(out, dict):
            ch = (out.get("choices") or [{}])[0]
            ch["token_ids"] = done_ids + list(ch.get("token_ids") or [])
            if ch.get("text") is not None:
                ch["text"] = done_text + ch["text"]
            u = out.get("usage") or {}
            u["prompt_tokens"] = n_prompt
            u["completion_tokens"] = len(ch["token_ids"])
            u["total_tokens"] = n_prompt + len(ch["token_ids"])
            out["usage"] = u
        return out

    @app.post("/v1/completions")
    def completions(body: dict):
        return handle(body, "/v1/completions")

    @app.post("/v1/chat/completions")
    def chat(body: dict):
        return handle(body, "/v1/chat/completions")

    @app.post("/instances/add")
    def add_instance(body: dict):
        try:
            state = pools.add(body.get("role", ""), body["url"])
        except (KeyError, ValueError) as e:
            raise HTTPException(400, str(e))
        return {"url": body["url"], "state": state}

    @app.post("/instances/remove")
    def remove_instance(body: dict):
        if not pools.remove(body.get("url", "")):
            raise HTTPException(404, "unknown instance")
        return {"url": body["url"], "removed": True}

    @app.get("/status")
    def status():
        return {"instances": pools.snapshot()}

    @app.get("/health")
    def health():
        snap = pools.snapshot()
        for role in ("prefill", "decode"):
            if not any(i["role"] == role and i["state"] == ACTIVE for i in snap):
                raise HTTPException(503, f"no active {role} instance")
        return {"status": "ok", "instances": snap}

    @app.on_event("shutdown")
    def _shutdown():
        stop.set()

    return app


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--host", default="127.0.0.1")
    ap.add_argument("--port", type=int, default=9000)
    ap.add_argument("--prefill", action="append", default=[])
    ap.add_argument("--decode", action="append", default=[])
    ap.add_argument("--max-retries", type=int, default=2)
    ap.add_argument("--probe-interval", type=float, default=1.0)
    a = ap.parse_args()
    uvicorn.run(build_proxy(a.prefill, a.decode, max_retries=a.max_retries, probe_interval=a.probe_interval),
                host=a.host, port=a.port, log_level="warning")
