"""OpenAI- and Anthropic-compatible HTTP server on top of the continuous-batching engine.

Routes (crates/pmetal-serve/src/server.rs:41-100, routes.rs:30-1060, anthropic.rs, sse.rs):
``POST /v1/chat/completions`` (streaming SSE and non-streaming, tools passed to the chat template and tool calls parsed
back out of the answer, ``logprobs`` / ``top_logprobs``, stop strings matched on the decoded text with the last tokens
held back from a stream until they can no longer be part of a stop string: routes.rs:162,235-335,558-605),
``POST /v1/completions``, ``POST /v1/embeddings`` (mean-pooled, L2-normalised final hidden states),
``POST /v1/messages`` (Anthropic), ``GET /v1/models``, ``GET /v1/metrics``, ``GET /health``.
A semaphore bounds in-flight requests and bodies larger than 2 MiB are rejected, as in the reference."""
from __future__ import annotations

import asyncio
import json
import time
import uuid
from typing import Any, AsyncIterator, Dict, List, Optional

try:                                    # module level so that FastAPI can resolve the handlers' annotations
    from fastapi import Request as HttpRequest
except ImportError:                     # pragma: no cover - the server needs fastapi, the rest of the package does not
    HttpRequest = None

from ..data.chat_templates import ChatTemplate, Message
from ..data.tokenizer import StreamDecoder
from ..models.sampling import SamplingParams
from .engine import ContinuousBatchEngine, Request

MAX_BODY = 2 << 20


def _params(body: Dict[str, Any], default_max: int = 256) -> SamplingParams:
    temp = float(body.get("temperature", 0.7))
    stop_ids = [int(x) for x in body.get("stop_token_ids", [])]
    return SamplingParams(temperature=temp, top_k=int(body.get("top_k", 0) or 0), top_p=float(body.get("top_p", 1.0)),
                          min_p=float(body.get("min_p", 0.0)),
                          repetition_penalty=float(body.get("repetition_penalty", 1.0)),
                          frequency_penalty=float(body.get("frequency_penalty", 0.0)),
                          presence_penalty=float(body.get("presence_penalty", 0.0)),
                          max_tokens=int(body.get("max_tokens") or body.get("max_completion_tokens") or default_max),
                          do_sample=temp > 0, seed=body.get("seed"), stop_token_ids=stop_ids)


def try_parse_tool_calls(text: str) -> Optional[List[dict]]:
    """Tool calls in a model answer (crates/pmetal-serve/src/types.rs:474-519): the whole answer must be one JSON
    value, either ``{"tool_calls": [{"function": {"name", "arguments"}, ...}]}`` or a bare ``{"name", "arguments"}``.
    Returns OpenAI-style tool-call objects or None when the text is ordinary prose."""
    t = text.strip()
    if not t.startswith(("{", "[")):
        return None
    try:
        v = json.loads(t)
    except json.JSONDecodeError:
        return None
    if not isinstance(v, dict):
        return None

    def call(name, arguments, cid=None, kind="function"):
        args = arguments if isinstance(arguments, str) else json.dumps(arguments)
        return {"id": cid or "call_" + uuid.uuid4().hex[:24], "type": kind, "function": {"name": name, "arguments": args}}
    if isinstance(v.get("tool_calls"), list):
        out = []
        for tc in v["tool_calls"]:
            fn = tc.get("function") if isinstance(tc, dict) else None
            if isinstance(fn, dict) and isinstance(fn.get("name"), str):
                out.append(call(fn["name"], fn.get("arguments"), tc.get("id"), tc.get("type") or "function"))
        return out or None
    if isinstance(v.get("name"), str):
        return [call(v["name"], v.get("arguments"))]
    return None


def _stop_list(stop) -> List[str]:
    if not stop:
        return []
    return [s for s in ([stop] if isinstance(stop, str) else list(stop)) if isinstance(s, str) and s]


def _content_text(content) -> str:
    if isinstance(content, str):
        return content
    if isinstance(content, list):          # OpenAI / Anthropic content parts
        return "".join(p.get("text", "") for p in content if isinstance(p, dict) and p.get("type") in ("text", None))
    return "" if content is None else str(content)


class ServerState:
    def __init__(self, engine: ContinuousBatchEngine, tokenizer, template: Optional[ChatTemplate] = None,
                 model_name: str = "pmetal-b200", max_concurrent: int = 256):
        self.engine, self.tok, self.template, self.model_name = engine, tokenizer, template or ChatTemplate("chatml"), model_name
        self.sem = asyncio.Semaphore(max_concurrent)
        self.started = time.time()

    def encode_chat(self, messages: List[dict], tools=None, no_thinking: bool = False) -> List[int]:
        msgs = [Message(m.get("role", "user"), _content_text(m.get("content")), m.get("tool_calls"), m.get("tool_call_id"),
                        m.get("name")) for m in messages]
        return self.tok.encode_with_special_tokens(self.template.apply_inference(msgs, no_thinking, tools))

    def adapter_of(self, body: Dict[str, Any]) -> Optional[str]:
        """Adapter a request asks for: the ``adapter`` field, or a ``model`` that names a loaded adapter."""
        ad = self.engine.adapters
        name = body.get("adapter")
        if name:
            return str(name)
        m = body.get("model")
        if ad is not None and isinstance(m, str) and m in ad.names:
            return m
        return None

    async def run(self, prompt: List[int], params: SamplingParams, stop=None, want_logprobs=False,
                  top_logprobs: int = 0, adapter: Optional[str] = None) -> Request:
        loop = asyncio.get_running_loop()
        fut = loop.create_future()
        req = Request(prompt, params, [], want_logprobs or top_logprobs > 0, stop_strings=_stop_list(stop),
                      decode=self.tok.decode, top_logprobs=top_logprobs, adapter=adapter,
                      on_done=lambda r: loop.call_soon_threadsafe(fut.set_result, r))
        self.engine.submit(req)
        return await fut

    async def stream(self, prompt: List[int], params: SamplingParams, stop=None,
                     adapter: Optional[str] = None) -> AsyncIterator[tuple]:
        """Yields (text piece, finish_reason or None). With stop strings the newest tokens are held back (as many
        tokens as the longest stop string has characters) so that text which turns out to be the beginning of a stop
        string is never sent; when the request ends, only the tokens the engine kept are flushed."""
        loop = asyncio.get_running_loop()
        q: asyncio.Queue = asyncio.Queue()
        stops = _stop_list(stop)
        hold = max((len(x) for x in stops), default=0)
        req = Request(prompt, params, [], False, stop_strings=stops, decode=self.tok.decode, adapter=adapter,
                      on_token=lambda t, lp: loop.call_soon_threadsafe(q.put_nowait, ("tok", t)),
                      on_done=lambda r: loop.call_soon_threadsafe(q.put_nowait, ("done", (r.finish_reason, len(r.output)))))
        self.engine.submit(req)
        dec = StreamDecoder(self.tok)
        pending: List[int] = []
        sent = 0

        def release(tok: int) -> str:
            return "" if tok in self.engine.eos else (dec.push(tok) or "")
        while True:
            kind, val = await q.get()
            if kind == "done":
                reason, kept = val
                for tok in pending[:max(kept - sent, 0)]:
                    piece = release(tok)
                    if piece:
                        yield piece, None
                yield "", reason
                return
            pending.append(val)
            while len(pending) > hold:
                piece = release(pending.pop(0))
                sent += 1
                if piece:
                    yield piece, None

    def text_of(self, req: Request) -> str:
        ids = [t for t in req.output if t not in self.engine.eos]
        return self.tok.decode(ids)

    @staticmethod
    def finish(reason: Optional[str]) -> str:
        return "length" if reason == "length" else "stop"


def create_app(state: ServerState):
    from fastapi import FastAPI, HTTPException
    from fastapi.responses import JSONResponse, StreamingResponse
    app = FastAPI(title="pmetal-b200")

    async def body_of(r: HttpRequest) -> dict:
        raw = await r.body()
        if len(raw) > MAX_BODY:
            raise HTTPException(413, "request body exceeds 2 MiB")
        try:
            return json.loads(raw or b"{}")
        except json.JSONDecodeError as e:
            raise HTTPException(400, f"invalid JSON: {e}") from None

    def sse(obj) -> bytes:
        return b"data: " + (obj if isinstance(obj, bytes) else json.dumps(obj).encode()) + b"\n\n"

    @app.get("/health")
    async def health():
        return {"status": "ok", "uptime_s": round(time.time() - state.started, 1)}

    @app.get("/v1/models")
    async def models():
        data = [{"id": state.model_name, "object": "model", "created": int(state.started), "owned_by": "pmetal"}]
        ad = state.engine.adapters
        for name in (ad.names if ad is not None else []):         # every loaded adapter is addressable as a model
            if name:
                data.append({"id": name, "object": "model", "created": int(state.started), "owned_by": "pmetal",
                             "parent": state.model_name})
        return {"object": "list", "data": data}

    @app.get("/v1/metrics")
    async def metrics():
        d = state.engine.stats.as_dict()
        d.update(active_slots=len(state.engine.slots), queued=len(state.engine.queue),
                 free_kv_blocks=state.engine.cache.num_free())
        return d

    @app.post("/v1/chat/completions")
    async def chat(r: HttpRequest):
        body = await body_of(r)
        if not isinstance(body.get("messages"), list) or not body["messages"]:
            raise HTTPException(400, "messages must be a non-empty list")
        prompt = state.encode_chat(body["messages"], body.get("tools"), bool(body.get("no_thinking")))
        params = _params(body)
        rid, created = "chatcmpl-" + uuid.uuid4().hex[:24], int(time.time())
        async with state.sem:
            if body.get("stream"):
                async def gen():
                    base = {"id": rid, "object": "chat.completion.chunk", "created": created, "model": state.model_name}
                    yield sse({**base, "choices": [{"index": 0, "delta": {"role": "assistant", "content": ""},
                                                    "finish_reason": None}]})
                    whole = []
                    async for piece, fin in state.stream(prompt, params, body.get("stop"), adapter=state.adapter_of(body)):
                        if fin is None:
                            whole.append(piece)
                            yield sse({**base, "choices": [{"index": 0, "delta": {"content": piece}, "finish_reason": None}]})
                        else:
                            calls = try_parse_tool_calls("".join(whole)) if body.get("tools") else None
                            if calls:               # tool-aware clients get the structured call in the closing chunk
                                yield sse({**base, "choices": [{"index": 0, "delta": {"tool_calls": [
                                    {"index": i, **c} for i, c in enumerate(calls)]}, "finish_reason": "tool_calls"}]})
                            else:
                                yield sse({**base, "choices": [{"index": 0, "delta": {}, "finish_reason": state.finish(fin)}]})
                    yield sse(b"[DONE]")
                return StreamingResponse(gen(), media_type="text/event-stream")
            top_n = min(int(body.get("top_logprobs") or 0), 20) if body.get("logprobs") else 0
            req = await state.run(prompt, params, body.get("stop"), bool(body.get("logprobs")), top_n, adapter=state.adapter_of(body))
        text = state.text_of(req)
        calls = try_parse_tool_calls(text) if body.get("tools") else None
        if calls:                                   # a structured call replaces the text (routes.rs:304-309)
            choice = {"index": 0, "message": {"role": "assistant", "content": None, "tool_calls": calls},
                      "finish_reason": "tool_calls"}
        else:
            choice = {"index": 0, "message": {"role": "assistant", "content": text},
                      "finish_reason": state.finish(req.finish_reason)}
        if body.get("logprobs"):
            content = []
            for i, (t, lp) in enumerate(zip(req.output, req.logprobs)):
                piece = state.tok.decode([t])
                entry = {"token": piece, "logprob": lp, "bytes": list(piece.encode("utf-8"))}
                if top_n:
                    alts = req.top_entries[i] if i < len(req.top_entries) else []
                    entry["top_logprobs"] = [{"token": state.tok.decode([a]), "logprob": alp,
                                              "bytes": list(state.tok.decode([a]).encode("utf-8"))} for a, alp in alts]
                content.append(entry)
            choice["logprobs"] = {"content": content}
        return {"id": rid, "object": "chat.completion", "created": created, "model": state.model_name, "choices": [choice],
                "usage": {"prompt_tokens": len(prompt), "completion_tokens": len(req.output),
                          "total_tokens": len(prompt) + len(req.output),
                          "prompt_tokens_details": {"cached_tokens": req.cached_tokens}}}

    @app.post("/v1/completions")
    async def completions(r: HttpRequest):
        body = await body_of(r)
        text = body.get("prompt")
        if isinstance(text, list):
            text = text[0] if text else ""
        if not isinstance(text, str):
            raise HTTPException(400, "prompt must be a string")
        prompt = state.tok.encode(text) or [0]
        params = _params(body, 16)
        rid, created = "cmpl-" + uuid.uuid4().hex[:24], int(time.time())
        async with state.sem:
            if body.get("stream"):
                async def gen():
                    base = {"id": rid, "object": "text_completion", "created": created, "model": state.model_name}
                    async for piece, fin in state.stream(prompt, params, body.get("stop"), adapter=state.adapter_of(body)):
                        yield sse({**base, "choices": [{"index": 0, "text": piece,
                                                        "finish_reason": None if fin is None else state.finish(fin)}]})
                    yield sse(b"[DONE]")
                return StreamingResponse(gen(), media_type="text/event-stream")
            n_lp = body.get("logprobs")
            top_n = min(int(n_lp), 20) if isinstance(n_lp, int) and not isinstance(n_lp, bool) else 0
            req = await state.run(prompt, params, body.get("stop"), bool(n_lp), top_n, adapter=state.adapter_of(body))
        choice = {"index": 0, "text": state.text_of(req), "finish_reason": state.finish(req.finish_reason)}
        if n_lp:                                    # legacy completions layout (routes.rs:446-471)
            toks = [state.tok.decode([t]) for t in req.output]
            choice["logprobs"] = {"tokens": toks, "token_logprobs": list(req.logprobs),
                                  "top_logprobs": [{state.tok.decode([a]): alp for a, alp in alts}
                                                   for alts in req.top_entries] if top_n else None}
        return {"id": rid, "object": "text_completion", "created": created, "model": state.model_name,
                "choices": [choice],
                "usage": {"prompt_tokens": len(prompt), "completion_tokens": len(req.output),
                          "total_tokens": len(prompt) + len(req.output)}}

    @app.post("/v1/embeddings")
    async def embeddings(r: HttpRequest):
        import torch
        body = await body_of(r)
        inp = body.get("input")
        texts = [inp] if isinstance(inp, str) else list(inp or [])
        if not texts:
            raise HTTPException(400, "input must be a string or a list of strings")
        model = state.engine.model
        out = []
        total = 0
        for i, t in enumerate(texts):
            ids = state.tok.encode(t) or [0]
            total += len(ids)
            x = torch.tensor(ids, dtype=torch.int64, device=state.engine.device)
            T = x.numel()
            with torch.no_grad():
                if hasattr(state.engine, "gen"):       # fast decoder: flat token batch with positions and document starts
                    h = model.forward_hidden(x, torch.arange(T, dtype=torch.int32, device=x.device),
                                             torch.tensor([0, T], dtype=torch.int32, device=x.device),
                                             torch.zeros(T, dtype=torch.int32, device=x.device))
                else:                                  # config-driven architectures take [batch, tokens]
                    h = model.forward_hidden(x[None])[0]
            e = torch.nn.functional.normalize(h.float().mean(0), dim=0)
            out.append({"object": "embedding", "index": i, "embedding": e.tolist()})
        return {"object": "list", "data": out, "model": state.model_name, "usage": {"prompt_tokens": total, "total_tokens": total}}

    @app.post("/v1/messages")
    async def anthropic_messages(r: HttpRequest):
        body = await body_of(r)
        msgs = list(body.get("messages") or [])
        if not msgs:
            raise HTTPException(400, "messages must be a non-empty list")
        if body.get("system"):
            msgs = [{"role": "system", "content": _content_text(body["system"])}] + msgs
        prompt = state.encode_chat(msgs, body.get("tools"))
        if "max_tokens" not in body:
            raise HTTPException(400, "max_tokens is required")
        params = _params(body)
        mid = "msg_" + uuid.uuid4().hex[:24]
        stop = body.get("stop_sequences")
        async with state.sem:
            if body.get("stream"):
                async def gen():
                    def ev(name, obj):
                        return f"event: {name}\ndata: {json.dumps(obj)}\n\n".encode()
                    yield ev("message_start", {"type": "message_start", "message": {
                        "id": mid, "type": "message", "role": "assistant", "model": state.model_name, "content": [],
                        "stop_reason": None, "usage": {"input_tokens": len(prompt), "output_tokens": 0}}})
                    yield ev("content_block_start", {"type": "content_block_start", "index": 0,
                                                     "content_block": {"type": "text", "text": ""}})
                    n = 0
                    async for piece, fin in state.stream(prompt, params, stop, adapter=state.adapter_of(body)):
                        if fin is None:
                            n += 1
                            yield ev("content_block_delta", {"type": "content_block_delta", "index": 0,
                                                             "delta": {"type": "text_delta", "text": piece}})
                        else:
                            yield ev("content_block_stop", {"type": "content_block_stop", "index": 0})
                            yield ev("message_delta", {"type": "message_delta", "delta": {
                                "stop_reason": "max_tokens" if fin == "length" else "end_turn"},
                                "usage": {"output_tokens": n}})
                    yield ev("message_stop", {"type": "message_stop"})
                return StreamingResponse(gen(), media_type="text/event-stream")
            req = await state.run(prompt, params, stop, adapter=state.adapter_of(body))
        return {"id": mid, "type": "message", "role": "assistant", "model": state.model_name,
                "content": [{"type": "text", "text": state.text_of(req)}],
                "stop_reason": "max_tokens" if req.finish_reason == "length" else "end_turn", "stop_sequence": None,
                "usage": {"input_tokens": len(prompt), "output_tokens": len(req.output)}}

    @app.exception_handler(KeyError)
    async def unknown_adapter(_, exc):
        return JSONResponse(status_code=404, content={"error": {"message": str(exc.args[0] if exc.args else exc),
                                                                "type": "invalid_request_error"}})

    @app.exception_handler(RuntimeError)
    async def runtime_error(_, exc):
        return JSONResponse(status_code=503, content={"error": {"message": str(exc), "type": "server_error"}})

    return app


def serve(model, tokenizer, template=None, host: str = "127.0.0.1", port: int = 8080, eos_ids=(), model_name="pmetal-b200",
          max_slots: int = 64, num_blocks: int = 8192, max_queue: int = 1024, cache_options: Optional[dict] = None,
          channel=None, adapters=None, engine=None):
    """Blocking: starts the engine thread and the HTTP server. ``cache_options`` (quant / window / sink) go to
    ``DecoderLM.new_cache``. With a model cut over several ranks, ``channel`` (serve/replica.py) is the leader's end of
    the step channel: the ranks that follow are released when the server stops. ``engine`` replaces the paged
    continuous-batching engine (``serve/portable_engine.py`` for the config-driven architectures)."""
    import uvicorn
    if engine is None:
        engine = ContinuousBatchEngine(model, eos_ids, max_slots=max_slots, num_blocks=num_blocks, max_queue=max_queue,
                                       cache_options=cache_options, adapters=adapters)
    engine.start()
    try:
        uvicorn.run(create_app(ServerState(engine, tokenizer, template, model_name)), host=host, port=port, log_level="info")
    finally:
        engine.shutdown()
        if channel is not None:
            channel.stop()
