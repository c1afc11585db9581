"""Load-aware P/D proxy against scripted backends: placement by load, retry on another instance,
elastic add / remove with health-gated activation, SSE relay."""
import importlib.util
import os
import sys
import threading
import time

import requests
from fastapi import FastAPI, HTTPException
from fastapi.responses import StreamingResponse

from test_api_server_cpu import _Server

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _load():
    spec = importlib.util.spec_from_file_location(
        "lb_proxy", os.path.join(ROOT, "examples", "disaggregated_prefill", "load_balance_proxy.py"))
    mod = importlib.util.module_from_spec(spec)
    sys.modules["lb_proxy"] = mod           # dataclasses resolve annotations through sys.modules
    spec.loader.exec_module(mod)
    return mod


def _backend(name, log, fail=None, delay=0.0, healthy=None):
    """Scripted instance: records what it was asked, answers like an engine server."""
    app = FastAPI()
    healthy = healthy if healthy is not None else {"ok": True}

    @app.get("/health")
    def health():
        if not healthy["ok"]:
            raise HTTPException(503, "starting")
        return {"status": "ok"}

    @app.post("/v1/completions")
    def completions(body: dict):
        log.append((name, body.get("max_tokens"), bool(body.get("kv_transfer_params", {}).get("do_remote_decode")),
                    body.get("kv_transfer_params")))
        if fail and fail["on"]:
            raise HTTPException(500, "boom")
        if delay:
            time.sleep(delay)
        if body.get("kv_transfer_params", {}).get("do_remote_decode"):
            return {"choices": [{"token_ids": [1]}], "kv_transfer_params": {"remote_engine_id": name, "blocks": [3]}}
        if body.get("stream"):
            def gen():
                for i in range(3):
                    yield f"data: {{\"choices\": [{{\"token_ids\": [{i}]}}], \"by\": \"{name}\"}}\n\n".encode()
                yield b"data: [DONE]\n\n"
            return StreamingResponse(gen(), media_type="text/event-stream")
        return {"choices": [{"token_ids": [7, 8]}], "served_by": name, "pulled_from": body["kv_transfer_params"]}
    return app


def test_pools_pick_the_least_loaded_instance_and_release_load():
    lb = _load()
    pools = lb.Pools(["http://p0", "http://p1"], ["http://d0"])
    a = pools.acquire("prefill", 100.0)
    b = pools.acquire("prefill", 10.0)
    c = pools.acquire("prefill", 10.0)
    assert (a.url, b.url, c.url) == ("http://p0", "http://p1", "http://p1")      # 100 vs 0, then 100 vs 10
    pools.release(a, 100.0, ok=True)
    assert pools.acquire("prefill", 1.0).url == "http://p0"
    # a failure takes the instance out until a probe succeeds
    pools.release(b, 10.0, ok=False)
    assert pools.acquire("prefill", 1.0, exclude=("http://p0",)) is None
    pools.probe_pending(lambda url: True)
    assert pools.acquire("prefill", 1.0, exclude=("http://p0",)).url == "http://p1"
    # removal with requests in flight drains instead of dropping
    d = pools.acquire("decode", 5.0)
    assert pools.remove("http://d0") and pools.acquire("decode", 1.0) is None
    assert any(i["state"] == lb.DRAINING for i in pools.snapshot())
    pools.release(d, 5.0, ok=True)
    assert not any(i["url"] == "http://d0" for i in pools.snapshot())


def test_proxy_routes_retries_and_grows():
    lb = _load()
    log = []
    p0_fail = {"on": True}
    late_health = {"ok": False}
    p0 = _Server(_backend("p0", log, fail=p0_fail))
    p1 = _Server(_backend("p1", log))
    d0 = _Server(_backend("d0", log, delay=0.3))
    d1 = _Server(_backend("d1", log, healthy=late_health))
    proxy = _Server(lb.build_proxy([p0.url, p1.url], [d0.url], probe_interval=0.1))
    try:
        body = {"prompt": list(range(50)), "max_tokens": 8}
        r = requests.post(proxy.url + "/v1/completions", json=body, timeout=30)
        assert r.status_code == 200, r.text
        out = r.json()
        # p0 failed, the request was retried on p1; the decode side got p1's transfer parameters
        assert [e[0] for e in log] == ["p0", "p1", "d0"]
        assert out["served_by"] == "d0" and out["pulled_from"]["remote_engine_id"] == "p1"
        assert log[1][1] == 1 and log[1][2] and log[2][1] == 8
        st = {i["url"]: i for i in requests.get(proxy.url + "/status", timeout=5).json()["instances"]}
        assert st[p0.url]["failed"] == 1 and st[p0.url]["state"] in (lb.SUSPECT, lb.ACTIVE)
        # p0 recovers: the background probe brings it back
        p0_fail["on"] = False
        for _ in range(50):
            st = {i["url"]: i for i in requests.get(proxy.url + "/status", timeout=5).json()["instances"]}
            if st[p0.url]["state"] == lb.ACTIVE:
                break
            time.sleep(0.1)
        assert st[p0.url]["state"] == lb.ACTIVE
        # a new decode instance waits until its health check answers
        assert requests.post(proxy.url + "/instances/add", json={"role": "decode", "url": d1.url},
                             timeout=5).json()["state"] == lb.WAITING
        time.sleep(0.4)
        st = {i["url"]: i for i in requests.get(proxy.url + "/status", timeout=5).json()["instances"]}
        assert st[d1.url]["state"] == lb.WAITING
        late_health["ok"] = True
        for _ in range(50):
            st = {i["url"]: i for i in requests.get(proxy.url + "/status", timeout=5).json()["instances"]}
            if st[d1.url]["state"] == lb.ACTIVE:
                break
            time.sleep(0.1)
        assert st[d1.url]["state"] == lb.ACTIVE
        # two concurrent requests: the second goes to the decode instance that is not busy
        log.clear()
        outs = [None, None]

        def go(i):
            outs[i] = requests.post(proxy.url + "/v1/completions", json=body, timeout=30).json()
        ts = [threading.Thread(target=go, args=(i,)) for i in range(2)]
        ts[0].start()
        time.sleep(0.1)
        ts[1].start()
        [t.join() for t in ts]
        assert {o["served_by"] for o in outs} == {"d0", "d1"}
        # streaming is relayed chunk by chunk
        r = requests.post(proxy.url + "/v1/completions", json=dict(body, stream=True), stream=True, timeout=30)
        lines = [l.decode() for l in r.iter_lines() if l]
        assert lines[-1] == "data: [DONE]" and len(lines) == 4
        # removal: no new traffic
        assert requests.post(proxy.url + "/instances/remove", json={"url": d0.url}, timeout=5).status_code == 200
        log.clear()
        requests.post(proxy.url + "/v1/completions", json=body, timeout=30)
        assert [e[0] for e in log if e[0].startswith("d")] == ["d1"]
        assert requests.post(proxy.url + "/instances/remove", json={"url": "http://nowhere"}, timeout=5).status_code == 404
        # a malformed request is not retried on every instance
        log.clear()
    finally:
        for s in (p0, p1, d0, d1, proxy):
            s.stop()


def test_proxy_continues_a_request_a_decode_instance_handed_back():
    """First decode answer: three tokens and stop_reason "recomputed"; the proxy prefills prompt + those
    tokens again, asks for the remaining tokens and joins the pieces."""
    lb = _load()
    seen = []

    def engine(role):
        app = FastAPI()

        @app.get("/health")
        def health():
            return {"status": "ok"}

        @app.post("/v1/completions")
        def completions(body: dict):
            seen.append((role, list(body["prompt"]), body["max_tokens"]))
            if body.get("kv_transfer_params", {}).get("do_remote_decode"):
                return {"choices": [{"token_ids": [0]}], "kv_transfer_params": {"n": len(body["prompt"])}}
            first = sum(1 for r, _, _ in seen if r == "decode") == 1
            if first:
                return {"choices": [{"token_ids": [11, 12, 13], "text": "abc", "finish_reason": "stop",
                                     "stop_reason": "recomputed"}],
                        "prompt_token_ids": list(body["prompt"]),
                        "usage": {"prompt_tokens": 4, "completion_tokens": 3, "total_tokens": 7}}
            return {"choices": [{"token_ids": [14, 15], "text": "de", "finish_reason": "length", "stop_reason": None}],
                    "usage": {"prompt_tokens": 7, "completion_tokens": 2, "total_tokens": 9}}
        return app
    p, d = _Server(engine("prefill")), _Server(engine("decode"))
    proxy = lb.build_proxy([p.url], [d.url], probe_interval=0.05)
    px = _Server(proxy)
    try:
        r = requests.post(px.url + "/v1/completions", json={"prompt": [1, 2, 3, 4], "max_tokens": 5}, timeout=30)
        assert r.status_code == 200, r.text
        out = r.json()
    finally:
        proxy.state.stop.set()
        for srv in (px, p, d):
            srv.stop()
    ch = out["choices"][0]
    assert ch["token_ids"] == [11, 12, 13, 14, 15] and ch["text"] == "abcde" and ch["finish_reason"] == "length"
    assert out["usage"] == {"prompt_tokens": 4, "completion_tokens": 5, "total_tokens": 9}
    assert seen == [("prefill", [1, 2, 3, 4], 1), ("decode", [1, 2, 3, 4], 5),
                    ("prefill", [1, 2, 3, 4, 11, 12, 13], 1), ("decode", [1, 2, 3, 4, 11, 12, 13], 2)]
    assert proxy.state.stats["recomputed"] == 1
