"""OpenAI-style completion server on top of the engine (the standalone counterpart of running
the reference under ``vllm serve``).

    python -m vllm_ascend_b200.entrypoints.api_server --model qwen3-8b --port 8000

One background thread owns the engine and steps it; HTTP handlers enqueue requests and wait
for their completion.  Prompts are token-id lists (``prompt`` may also be text when a
tokenizer directory is given).  ``kv_transfer_params`` are accepted and returned, which is
what a prefill/decode proxy needs.  ``stream: true`` answers with server-sent events (one chunk per
engine step that produced tokens); ``/v1/chat/completions`` applies the tokenizer's chat template (or
takes ``prompt_token_ids`` templated by the caller); ``/v1/embeddings`` returns last-token-pooled,
normalised hidden states.  ``/metrics`` exposes the engine counters in the Prometheus text format,
``/health`` runs the worker health check.
"""
from __future__ import annotations

import argparse
import asyncio
import queue
import threading
import time
import uuid
from typing import Optional

from fastapi import FastAPI, HTTPException
from fastapi.responses import PlainTextResponse

from ..engine.request import RequestError, RequestStatus, SamplingParams

_FINISH = {RequestStatus.FINISHED_STOPPED: "stop", RequestStatus.FINISHED_LENGTH: "length",
           RequestStatus.FINISHED_ABORTED: "abort"}


class EngineLoop(threading.Thread):
    """Owns the engine: drains the submission queue, steps while there is work."""

    def __init__(self, llm):
        super().__init__(daemon=True, name="engine-loop")
        self.llm, self.engine = llm, llm.engine
        self.inbox: "queue.Queue" = queue.Queue()
        self.waiters: dict[str, tuple] = {}          # request id -> (asyncio future, loop, request)
        self.streams: dict[str, list] = {}           # request id -> [asyncio queue, tokens already sent]
        self.stop_flag = threading.Event()
        self.error: Optional[BaseException] = None

    def submit(self, prompt_ids, sp: SamplingParams, kv_params, fut, loop, stream_q=None) -> str:
        rid = f"cmpl-{uuid.uuid4().hex[:16]}"
        self.inbox.put((rid, prompt_ids, sp, kv_params, fut, loop, stream_q))
        return rid

    def run(self) -> None:
        eng = self.engine
        while not self.stop_flag.is_set():
            try:
                block = not eng.has_unfinished()
                while True:
                    item = self.inbox.get(timeout=0.05) if block else self.inbox.get_nowait()
                    rid, ids, sp, kvp, fut, loop, sq = item
                    try:
                        eng.add_request(ids, sp, request_id=rid, kv_transfer_params=kvp)
                        self.waiters[rid] = (fut, loop, eng.scheduler.requests[rid])
                        if sq is not None:
                            self.streams[rid] = [sq, 0]
                    except Exception as e:
                        loop.call_soon_threadsafe(fut.set_exception, e)
                    block = False
            except queue.Empty:
                pass
            if not eng.has_unfinished():
                continue
            try:
                eng.step()
            except RequestError as e:            # one request's fault: abort it, keep serving the others
                eng.scheduler.abort_request(e.request_id)
                self.streams.pop(e.request_id, None)
                w = self.waiters.pop(e.request_id, None)
                eng.scheduler.requests.pop(e.request_id, None)
                if w is not None:
                    w[1].call_soon_threadsafe(w[0].set_exception, ValueError(str(e)))
                continue
            except BaseException as e:           # fail every waiter, stop serving
                self.error = e
                for fut, loop, _ in self.waiters.values():
                    loop.call_soon_threadsafe(fut.set_exception, RuntimeError(f"engine failed: {e}"))
                self.waiters.clear()
                return
            for rid, st in self.streams.items():     # streaming requests get their new tokens every step
                _, loop, req = self.waiters[rid]
                toks = req.output_token_ids or []
                if len(toks) > st[1]:
                    loop.call_soon_threadsafe(st[0].put_nowait, list(toks[st[1]:]))
                    st[1] = len(toks)
            for rid in [r for r, (_, _, req) in self.waiters.items() if req.is_finished]:
                self.streams.pop(rid, None)
                fut, loop, req = self.waiters.pop(rid)
                eng.scheduler.requests.pop(rid, None)
                loop.call_soon_threadsafe(fut.set_result, req)

    def stop(self) -> None:
        self.stop_flag.set()


def _guided(body: dict):
    """``guided_regex`` / ``guided_choice`` / ``guided_json`` (or an OpenAI ``response_format`` with a
    JSON schema) -> GuidedDecodingParams."""
    from ..sample.guided import GuidedDecodingParams
    if body.get("guided_regex") is not None:
        return GuidedDecodingParams(regex=str(body["guided_regex"]))
    if body.get("guided_choice") is not None:
        return GuidedDecodingParams(choice=list(body["guided_choice"]))
    if body.get("guided_json") is not None:
        return GuidedDecodingParams(json=body["guided_json"])
    rf = body.get("response_format") or {}
    if rf.get("type") == "json_schema":
        js = rf.get("json_schema") or {}
        return GuidedDecodingParams(json=js.get("schema", js))
    return None


def _sampling_params(body: dict) -> SamplingParams:
    lp = body.get("logprobs")
    if isinstance(lp, bool):                       # chat API: boolean + top_logprobs
        lp = int(body.get("top_logprobs") or 0) if lp else None
    if int(body.get("n") or 1) != 1:
        raise HTTPException(400, "n > 1 is served by LLM.generate; the HTTP server returns one choice per request")
    try:
        return _sampling_params_unchecked(body, lp)
    except (ValueError, TypeError) as e:
        raise HTTPException(400, f"bad sampling parameters: {e}")


def _sampling_params_unchecked(body: dict, lp) -> SamplingParams:
    return SamplingParams(
        max_tokens=int(body.get("max_tokens") or body.get("max_completion_tokens") or 16),
        temperature=float(body.get("temperature", 1.0)),
        top_p=float(body.get("top_p", 1.0)), top_k=int(body.get("top_k", 0) or 0),
        seed=body.get("seed"), ignore_eos=bool(body.get("ignore_eos", False)),
        stop_token_ids=list(body.get("stop_token_ids") or []),
        min_p=float(body.get("min_p", 0.0)), min_tokens=int(body.get("min_tokens", 0)),
        presence_penalty=float(body.get("presence_penalty", 0.0)),
        frequency_penalty=float(body.get("frequency_penalty", 0.0)),
        repetition_penalty=float(body.get("repetition_penalty", 1.0)),
        logprobs=lp,
        prompt_logprobs=(int(body["prompt_logprobs"]) if body.get("prompt_logprobs") is not None else None),
        logit_bias={int(k): float(v) for k, v in (body.get("logit_bias") or {}).items()} or None,
        allowed_token_ids=body.get("allowed_token_ids"),
        bad_words_token_ids=body.get("bad_words_token_ids"),
        guided_decoding=_guided(body))


def build_app(llm, tokenizer=None, model_name: str = "model") -> FastAPI:
    app = FastAPI(title="vllm_ascend_b200")
    if tokenizer is not None and llm.engine.guided is None and hasattr(tokenizer, "decode"):
        try:
            llm.set_guided_vocabulary(tokenizer)
        except Exception:                          # a tokenizer that cannot decode single ids: guided requests are refused
            pass
    loop_thread = EngineLoop(llm)
    loop_thread.start()
    app.state.engine_loop = loop_thread

    @app.get("/health")
    async def health():
        if loop_thread.error is not None:
            raise HTTPException(500, f"engine failed: {loop_thread.error}")
        try:
            llm.engine.check_health()
        except Exception as e:
            raise HTTPException(500, str(e))
        return {"status": "ok"}

    @app.get("/v1/models")
    async def models():
        return {"object": "list", "data": [{"id": model_name, "object": "model"}]}

    @app.get("/metrics", response_class=PlainTextResponse)
    async def metrics():
        from ..observability.metrics import collect
        lines = []
        for k, v in collect(llm.engine).items():
            if isinstance(v, (int, float)):
                lines.append(f"# TYPE vllm_b200_{k} gauge\nvllm_b200_{k} {float(v)}")
        return "\n".join(lines) + "\n"

    @app.post("/v1/completions")
    async def completions(body: dict):
        prompt = body.get("prompt")
        if isinstance(prompt, str):
            if tokenizer is None:
                raise HTTPException(400, "text prompts need a tokenizer; send token ids")
            ids = tokenizer.encode(prompt)
        elif isinstance(prompt, list) and prompt and all(isinstance(t, int) for t in prompt):
            ids = prompt
        else:
            raise HTTPException(400, "prompt must be a string or a list of token ids")
        sp = _sampling_params(body)
        if body.get("stream"):
            return await _stream(ids, sp, body, chat=False)
        aloop = asyncio.get_running_loop()
        fut = aloop.create_future()
        t0 = time.time()
        rid = loop_thread.submit(ids, sp, body.get("kv_transfer_params"), fut, aloop)
        try:
            req = await fut
        except Exception as e:
            raise HTTPException(400 if isinstance(e, ValueError) else 500, str(e))
        toks = list(req.output_token_ids or [])
        text = tokenizer.decode(toks) if tokenizer is not None else None
        return {"id": rid, "object": "text_completion", "created": int(t0), "model": model_name,
                "choices": [{"index": 0, "text": text, "token_ids": toks,
                             "finish_reason": _FINISH.get(req.status), "stop_reason": req.stop_reason,
                             "logprobs": ([{str(k): v for k, v in e.items()} for e in req.logprobs]
                                          if req.logprobs else None),
                             "prompt_logprobs": ([None if e is None else {str(k): v for k, v in e.items()}
                                                  for e in req.prompt_logprobs]
                                                 if getattr(req, "prompt_logprobs", None) else None)}],
                "usage": {"prompt_tokens": req.num_prompt_tokens, "completion_tokens": len(toks),
                          "total_tokens": req.num_prompt_tokens + len(toks)},
                "kv_transfer_params": req.kv_transfer_params,
                # a request handed back under KV pressure: the proxy continues it elsewhere from these
                **({"prompt_token_ids": [int(t) for t in req.prompt_token_ids]}
                   if req.stop_reason == "recomputed" else {})}

    async def _stream(ids, sp, body, chat: bool):
        """Server-sent events: one chunk per engine step that produced tokens, then ``[DONE]``."""
        import json

        from fastapi.responses import StreamingResponse
        aloop = asyncio.get_running_loop()
        fut, q = aloop.create_future(), asyncio.Queue()
        t0 = int(time.time())
        rid = loop_thread.submit(ids, sp, body.get("kv_transfer_params"), fut, aloop, q)
        obj = "chat.completion.chunk" if chat else "text_completion"

        def chunk(toks, finish=None):
            text = tokenizer.decode(toks) if (tokenizer is not None and toks) else ("" if tokenizer is not None else None)
            ch = {"index": 0, "token_ids": toks, "finish_reason": finish}
            if chat:
                ch["delta"] = {"content": text} if toks else {}
            else:
                ch["text"] = text
            return "data: " + json.dumps({"id": rid, "object": obj, "created": t0, "model": model_name,
                                          "choices": [ch]}) + "\n\n"

        async def gen():
            while True:
                getter = asyncio.ensure_future(q.get())
                done, _ = await asyncio.wait({getter, fut}, return_when=asyncio.FIRST_COMPLETED)
                if getter in done:
                    yield chunk(getter.result())
                    continue
                getter.cancel()
                if fut.exception() is not None:
                    yield "data: " + json.dumps({"error": str(fut.exception())}) + "\n\n"
                    break
                while not q.empty():
                    yield chunk(q.get_nowait())
                yield chunk([], _FINISH.get(fut.result().status))
                break
            yield "data: [DONE]\n\n"
        return StreamingResponse(gen(), media_type="text/event-stream")

    @app.post("/v1/chat/completions")
    async def chat_completions(body: dict):
        msgs = body.get("messages")
        if not isinstance(msgs, list) or not msgs:
            raise HTTPException(400, "messages must be a non-empty list")
        if body.get("prompt_token_ids"):
            ids = list(body["prompt_token_ids"])          # pre-templated by the caller
        elif tokenizer is None:
            raise HTTPException(400, "chat messages need a tokenizer; send prompt_token_ids")
        else:
            ids = tokenizer.apply_chat_template(msgs, add_generation_prompt=True, tokenize=True)
            ids = list(ids["input_ids"] if isinstance(ids, dict) else ids)
        sp = _sampling_params(body)
        if body.get("stream"):
            return await _stream(ids, sp, body, chat=True)
        aloop = asyncio.get_running_loop()
        fut = aloop.create_future()
        t0 = time.time()
        rid = loop_thread.submit(ids, sp, body.get("kv_transfer_params"), fut, aloop)
        try:
            req = await fut
        except Exception as e:
            raise HTTPException(400 if isinstance(e, ValueError) else 500, str(e))
        toks = list(req.output_token_ids or [])
        text = tokenizer.decode(toks) if tokenizer is not None else None
        return {"id": rid.replace("cmpl", "chatcmpl"), "object": "chat.completion", "created": int(t0),
                "model": model_name,
                "choices": [{"index": 0, "message": {"role": "assistant", "content": text, "token_ids": toks},
                             "finish_reason": _FINISH.get(req.status),
                             "logprobs": ([{str(k): v for k, v in e.items()} for e in req.logprobs]
                                          if req.logprobs else None)}],
                "usage": {"prompt_tokens": req.num_prompt_tokens, "completion_tokens": len(toks),
                          "total_tokens": req.num_prompt_tokens + len(toks)}}

    @app.post("/v1/embeddings")
    async def embeddings(body: dict):
        inp = body.get("input")
        items = inp if isinstance(inp, list) and inp and isinstance(inp[0], (list, str)) else [inp]
        ids_list = []
        for it in items:
            if isinstance(it, str):
                if tokenizer is None:
                    raise HTTPException(400, "text inputs need a tokenizer; send token ids")
                ids_list.append(tokenizer.encode(it))
            elif isinstance(it, list) and it and all(isinstance(t, int) for t in it):
                ids_list.append(it)
            else:
                raise HTTPException(400, "input must be text, a token-id list, or a list of those")
        sp = SamplingParams(temperature=0.0, max_tokens=1, ignore_eos=True, extra_args={"pooling": True})
        aloop = asyncio.get_running_loop()
        futs = []
        for ids in ids_list:
            fut = aloop.create_future()
            loop_thread.submit(ids, sp, None, fut, aloop)
            futs.append(fut)
        reqs = [await f for f in futs]
        import torch
        data = [{"object": "embedding", "index": i,
                 "embedding": torch.nn.functional.normalize(r.pooled, dim=-1).tolist()} for i, r in enumerate(reqs)]
        return {"object": "list", "model": model_name, "data": data,
                "usage": {"prompt_tokens": sum(r.num_prompt_tokens for r in reqs)}}

    return app


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", required=True)
    ap.add_argument("--host", default="127.0.0.1")
    ap.add_argument("--port", type=int, default=8000)
    ap.add_argument("--tokenizer", default=None)
    ap.add_argument("--max-model-len", type=int, default=4096)
    ap.add_argument("--max-num-seqs", type=int, default=256)
    ap.add_argument("--kv-transfer-config", default=None, help="JSON")
    ap.add_argument("--additional-config", default=None, help="JSON")
    ap.add_argument("--device", default=None)
    args = ap.parse_args()
    import json

    import uvicorn

    from ..engine.llm import LLM
    llm = LLM(args.model, device=args.device, max_model_len=args.max_model_len, max_num_seqs=args.max_num_seqs,
              kv_transfer_config=json.loads(args.kv_transfer_config) if args.kv_transfer_config else None,
              additional_config=json.loads(args.additional_config) if args.additional_config else None)
    tok = None
    if args.tokenizer:
        from transformers import AutoTokenizer
        tok = AutoTokenizer.from_pretrained(args.tokenizer)
    uvicorn.run(build_app(llm, tok, args.model), host=args.host, port=args.port, log_level="warning")


if __name__ == "__main__":
    main()
