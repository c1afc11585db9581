"""HTTP serving: completion endpoint, metrics, and the prefill/decode proxy end to end (CPU)."""
import importlib.util
import os
import socket
import threading
import time

import numpy as np
import pytest
import requests
import uvicorn

from vllm_ascend_b200 import LLM, SamplingParams
from vllm_ascend_b200.entrypoints.api_server import build_app

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


class _Server:
    def __init__(self, app):
        self.port = _port()
        self.server = uvicorn.Server(uvicorn.Config(app, host="127.0.0.1", port=self.port, log_level="error"))
        self.thread = threading.Thread(target=self.server.run, daemon=True)
        self.thread.start()
        for _ in range(200):
            try:
                requests.get(self.url + "/health", timeout=0.5)
                break
            except requests.RequestException:
                time.sleep(0.05)

    @property
    def url(self):
        return f"http://127.0.0.1:{self.port}"

    def stop(self):
        self.server.should_exit = True
        self.thread.join(timeout=5)


def _llm(role=None, eid=None):
    ktc = None if role is None else {"kv_connector": "NVLinkConnector", "kv_role": role, "engine_id": eid}
    return LLM("tiny-qwen", device="cpu", seed=0, block_size=16, max_model_len=256, max_num_seqs=8,
               kv_transfer_config=ktc)


def test_completions_metrics_and_pd_proxy():
    spec = importlib.util.spec_from_file_location("pd_proxy", os.path.join(ROOT, "examples", "disaggregated_prefill",
                                                                            "proxy.py"))
    proxy_mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(proxy_mod)
    rng = np.random.default_rng(4)
    prompts = [rng.integers(1, 500, size=n).tolist() for n in (40, 21, 66)]
    want = [o.outputs[0].token_ids for o in
            _llm().generate(prompts, SamplingParams(max_tokens=6, temperature=0.0, ignore_eos=True))]
    mono, pre, dec = _llm(), _llm("kv_producer", "P-http"), _llm("kv_consumer", "D-http")
    servers = [_Server(build_app(x, model_name="tiny-qwen")) for x in (mono, pre, dec)]
    proxy = _Server(proxy_mod.build_proxy([servers[1].url], [servers[2].url]))
    try:
        body = {"prompt": prompts[0], "max_tokens": 6, "temperature": 0.0, "ignore_eos": True}
        r = requests.post(servers[0].url + "/v1/completions", json=body, timeout=60).json()
        assert r["choices"][0]["token_ids"] == want[0] and r["choices"][0]["finish_reason"] == "length"
        assert r["usage"] == {"prompt_tokens": 40, "completion_tokens": 6, "total_tokens": 46}
        assert requests.post(servers[0].url + "/v1/completions", json={"prompt": "text"}, timeout=10).status_code == 400
        mono.set_guided_vocabulary([None] + [chr(97 + i % 26) * (1 + i // 26) for i in range(mono.cfg.model.vocab_size - 1)],
                                   eos_token_id=0)
        r = requests.post(servers[0].url + "/v1/completions",
                          json=dict(body, guided_choice=["abba", "cc"], max_tokens=12, ignore_eos=False), timeout=60).json()
        vocab = [""] + [chr(97 + i % 26) * (1 + i // 26) for i in range(mono.cfg.model.vocab_size - 1)]
        assert "".join(vocab[t] for t in r["choices"][0]["token_ids"]) in ("abba", "cc")
        r = requests.post(servers[0].url + "/v1/completions", json=dict(body, prompt_logprobs=1), timeout=60).json()
        plp = r["choices"][0]["prompt_logprobs"]
        assert len(plp) == 40 and plp[0] is None and str(prompts[0][5]) in plp[5]
        m = requests.get(servers[0].url + "/metrics", timeout=10).text
        assert "vllm_b200_steps" in m and "vllm_b200_kv_blocks_free" in m
        assert requests.get(servers[0].url + "/v1/models", timeout=10).json()["data"][0]["id"] == "tiny-qwen"
        # concurrent requests through the proxy: prefill on one engine, decode on the other
        out = [None] * len(prompts)

        def go(i):
            b = {"prompt": prompts[i], "max_tokens": 6, "temperature": 0.0, "ignore_eos": True}
            out[i] = requests.post(proxy.url + "/v1/completions", json=b, timeout=120).json()
        ts = [threading.Thread(target=go, args=(i,)) for i in range(len(prompts))]
        [t.start() for t in ts]
        [t.join() for t in ts]
        assert [o["choices"][0]["token_ids"] for o in out] == want
        assert dec.engine.kv_connector.stats["pulled_requests"] == len(prompts)
        assert requests.get(proxy.url + "/health", timeout=20).json()["routed"]["decode"][servers[2].url] == 3
    finally:
        for s in servers + [proxy]:
            s.stop()
        pre.engine.kv_connector.close()
        dec.engine.kv_connector.close()


def test_streaming_chat_and_embeddings_endpoints():
    import json
    llm = _llm()
    prompt = [5, 6, 7, 8, 9, 10]
    want = llm.generate([prompt], SamplingParams(max_tokens=7, temperature=0.0, ignore_eos=True))[0].outputs[0].token_ids
    vec = llm.embed([prompt])[0]
    srv = _Server(build_app(llm, None, "tiny"))
    try:
        # server-sent events: the chunks concatenate to the non-streaming answer, then [DONE]
        r = requests.post(srv.url + "/v1/completions", json={"prompt": prompt, "max_tokens": 7, "temperature": 0.0,
                                                             "ignore_eos": True, "stream": True}, stream=True, timeout=60)
        assert r.status_code == 200 and r.headers["content-type"].startswith("text/event-stream")
        toks, finish, done = [], None, False
        for line in r.iter_lines():
            if not line:
                continue
            payload = line.decode()[len("data: "):]
            if payload == "[DONE]":
                done = True
                break
            ch = json.loads(payload)["choices"][0]
            toks += ch["token_ids"]
            finish = ch["finish_reason"] or finish
        assert done and toks == want and finish == "length"
        # chat endpoint with a pre-templated prompt (no tokenizer on this server)
        r = requests.post(srv.url + "/v1/chat/completions", json={
            "messages": [{"role": "user", "content": "hi"}], "prompt_token_ids": prompt, "max_tokens": 7,
            "temperature": 0.0, "ignore_eos": True, "logprobs": True, "top_logprobs": 2}, timeout=60)
        assert r.status_code == 200, r.text
        body = r.json()
        assert body["object"] == "chat.completion"
        ch = body["choices"][0]
        assert ch["message"]["token_ids"] == want and len(ch["logprobs"]) == 7
        r = requests.post(srv.url + "/v1/chat/completions", json={"messages": [{"role": "user", "content": "hi"}]},
                          timeout=60)
        assert r.status_code == 400
        # embeddings
        r = requests.post(srv.url + "/v1/embeddings", json={"input": [prompt, [1, 2, 3]]}, timeout=60)
        assert r.status_code == 200, r.text
        data = r.json()["data"]
        assert len(data) == 2 and np.allclose(data[0]["embedding"], vec.numpy(), atol=1e-5)
    finally:
        srv.stop()
        srv.server.config.app.state.engine_loop.stop()
