"""Round-robin proxy for disaggregated prefill / decode instances.

    python examples/disaggregated_prefill/proxy.py --port 9000 \
        --prefill http://127.0.0.1:8100 --prefill http://127.0.0.1:8101 \
        --decode http://127.0.0.1:8200

Each completion request is first sent to a prefill instance with ``max_tokens=1`` and
``kv_transfer_params={"do_remote_decode": true}``; the ``kv_transfer_params`` it returns (the
blocks it keeps for the decode side) travel with the original request to a decode instance,
whose answer goes back to the client.  If the decode instance reports that it had to re-prefill
locally, the answer is still complete: that fallback lives in the decode engine's scheduler.
Same flow as the reference's proxies (examples/disaggregated_prefill_v1/*.py).
"""
from __future__ import annotations

import argparse
import itertools

import requests
import uvicorn
from fastapi import FastAPI, HTTPException


def build_proxy(prefill_urls: list[str], decode_urls: list[str], timeout: float = 600.0) -> FastAPI:
    app = FastAPI(title="pd-proxy")
    p_iter, d_iter = itertools.cycle(prefill_urls), itertools.cycle(decode_urls)
    app.state.counts = {"prefill": {u: 0 for u in prefill_urls}, "decode": {u: 0 for u in decode_urls}}

    @app.post("/v1/completions")
    def completions(body: dict):
        p_url, d_url = next(p_iter), next(d_iter)
        pre = dict(body, max_tokens=1, kv_transfer_params={"do_remote_decode": True})
        r = requests.post(p_url + "/v1/completions", json=pre, timeout=timeout)
        if r.status_code != 200:
            raise HTTPException(r.status_code, f"prefill instance: {r.text}")
        app.state.counts["prefill"][p_url] += 1
        ktp = r.json().get("kv_transfer_params")
        dec = dict(body, kv_transfer_params=ktp)
        r = requests.post(d_url + "/v1/completions", json=dec, timeout=timeout)
        if r.status_code != 200:
            raise HTTPException(r.status_code, f"decode instance: {r.text}")
        app.state.counts["decode"][d_url] += 1
        return r.json()

    @app.get("/health")
    def health():
        bad = []
        for u in prefill_urls + decode_urls:
            try:
                if requests.get(u + "/health", timeout=5).status_code != 200:
                    bad.append(u)
            except requests.RequestException:
                bad.append(u)
        if bad:
            raise HTTPException(503, f"unhealthy: {bad}")
        return {"status": "ok", "routed": app.state.counts}

    return app


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--host", default="127.0.0.1")
    ap.add_argument("--port", type=int, default=9000)
    ap.add_argument("--prefill", action="append", required=True)
    ap.add_argument("--decode", action="append", required=True)
    a = ap.parse_args()
    uvicorn.run(build_proxy(a.prefill, a.decode), host=a.host, port=a.port, log_level="warning")
