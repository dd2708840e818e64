"""The rest of the reference's inference-facing HTTP surface, registered on the same app
(rust/engine/src/server.rs:697-718 and server/api/{responses,batches}.rs):

* OpenAI Responses API (``/v1/responses``, ``/v1/responses/{id}``), Files (``/v1/files``...) and
  Batches (``/v1/batches``...): a batch is a JSONL file of requests to ``/v1/chat/completions``,
  ``/v1/completions`` or ``/v1/embeddings`` that runs in the background on the same engine;
* scoring endpoints on a decoder: ``/v1/rerank`` (+ ``/rerank``), ``/v1/score``, ``/pooling``,
  ``/classify`` - all built on the hidden state of the last prompt token (decoder-as-encoder
  embeddings) or on the next-token distribution;
* llama.cpp ``/infill`` (fill-in-the-middle prompt), ``/slots/{id}``, ``/lora-adapters``,
  ``/is_sleeping``, ``/v1/models/{id}``, ``/embeddings``, ``/``;
* Ollama model management (``/api/pull`` ``/api/push`` ``/api/create`` ``/api/copy``
  ``/api/delete`` ``/api/blobs/{digest}``) for a server that holds exactly one local model: the
  calls succeed for that model and answer 404 / 501 otherwise, since nothing can be downloaded;
* middleware: CORS (``cors_origins``) and a token-bucket rate limit per API key or client address
  (``rate_limit_rps``), like the reference's ``server/http.rs``.

``register(app, ctx)`` gets the closures of ``create_app`` through ``ctx`` so every route here goes
through the same admission, stop-string, cache and metrics path as the core routes.
"""
from __future__ import annotations

import asyncio
import json
import math
import time
import uuid
from collections import OrderedDict
from typing import Dict, List, Optional

from fastapi import HTTPException, Request as HttpRequest
from fastapi.responses import JSONResponse, Response, StreamingResponse

from ..runtime.request import SamplingParams


class TokenBucket:
    """Per-client token bucket: `rps` requests per second with a burst of 2 x rps (at least 1)."""

    def __init__(self, rps: float):
        self.rps = float(rps)
        self.burst = max(1.0, 2.0 * self.rps)
        self.state: "OrderedDict[str, tuple]" = OrderedDict()

    def allow(self, key: str, now: Optional[float] = None) -> bool:
        now = time.monotonic() if now is None else now
        level, t = self.state.get(key, (self.burst, now))
        level = min(self.burst, level + (now - t) * self.rps)
        ok = level >= 1.0
        self.state[key] = (level - 1.0 if ok else level, now)
        self.state.move_to_end(key)
        while len(self.state) > 4096:
            self.state.popitem(last=False)
        return ok


def install_middleware(app, cors_origins: Optional[List[str]] = None, rate_limit_rps: float = 0.0) -> None:
    open_paths = ("/health", "/ready", "/metrics", "/version")
    if rate_limit_rps and rate_limit_rps > 0:
        bucket = TokenBucket(rate_limit_rps)

        @app.middleware("http")
        async def _rate_limit(request: HttpRequest, call_next):
            if request.url.path not in open_paths:
                who = request.headers.get("authorization") or request.headers.get("x-api-key") or \
                    (request.client.host if request.client else "anon")
                if not bucket.allow(who):
                    return JSONResponse({"error": {"message": "rate limit exceeded", "type": "rate_limit_error"}}, 429,
                                        headers={"retry-after": "1"})
            return await call_next(request)
    if cors_origins:
        allow_all = "*" in cors_origins

        @app.middleware("http")
        async def _cors(request: HttpRequest, call_next):
            origin = request.headers.get("origin")
            ok = origin is not None and (allow_all or origin in cors_origins)
            if request.method == "OPTIONS" and ok:
                resp = Response(status_code=204)
            else:
                resp = await call_next(request)
            if ok:
                resp.headers["access-control-allow-origin"] = "*" if allow_all else origin
                resp.headers["access-control-allow-methods"] = "GET, POST, DELETE, OPTIONS"
                resp.headers["access-control-allow-headers"] = request.headers.get("access-control-request-headers", "*")
                resp.headers["vary"] = "origin"
            return resp


def _cos(a: List[float], b: List[float]) -> float:
    na = math.sqrt(sum(x * x for x in a)) or 1.0
    nb = math.sqrt(sum(x * x for x in b)) or 1.0
    return sum(x * y for x, y in zip(a, b)) / (na * nb)


def _responses_input_to_messages(body: dict) -> List[dict]:
    msgs: List[dict] = []
    if body.get("instructions"):
        msgs.append({"role": "system", "content": str(body["instructions"])})
    inp = body.get("input")
    if isinstance(inp, str):
        msgs.append({"role": "user", "content": inp})
    elif isinstance(inp, list):
        for item in inp:
            if not isinstance(item, dict):
                raise HTTPException(400, "input items must be objects")
            if item.get("type") in (None, "message"):
                c = item.get("content")
                if isinstance(c, list):
                    c = "".join(p.get("text", "") for p in c if isinstance(p, dict) and p.get("type") in ("input_text", "output_text", "text"))
                msgs.append({"role": item.get("role", "user"), "content": c or ""})
            elif item.get("type") == "function_call_output":
                msgs.append({"role": "tool", "content": str(item.get("output", "")), "tool_call_id": item.get("call_id")})
    if not msgs:
        raise HTTPException(400, "input must be a string or a non-empty list of messages")
    return msgs


def register(app, ctx) -> None:
    """ctx: namespace with engine, worker, tokenizer, model_name, started, generate, collect, embed_one,
    encode_prompt, chat_prompt, sampling_from, attach_guided, shape_message, usage, sse."""
    engine, tokenizer, model_name = ctx.engine, ctx.tokenizer, ctx.model_name
    responses: "OrderedDict[str, dict]" = OrderedDict()
    files: Dict[str, dict] = {}
    batches: Dict[str, dict] = {}

    # ------------------------------------------------------------------ small ones
    @app.get("/")
    async def root():
        return {"name": "fllm_b200", "model": model_name, "status": "ok" if ctx.worker.ready() else "unavailable"}

    @app.get("/v1/models/{mid:path}")
    async def model_by_id(mid: str):
        if mid != model_name:
            raise HTTPException(404, f"model {mid!r} is not served here")
        return {"id": model_name, "object": "model", "created": int(ctx.started), "owned_by": "fllm_b200",
                "max_model_len": engine.cfg.max_model_len}

    @app.get("/is_sleeping")
    async def is_sleeping():
        return {"is_sleeping": False}

    @app.get("/lora-adapters")
    async def lora_adapters():
        return []                                   # adapters are merged into the weights at load time

    @app.post("/lora-adapters")
    async def lora_adapters_set(body: list = []):
        if body:
            raise HTTPException(501, "adapters are merged at load time (merge-lora); hot-swapping is not available")
        return []

    @app.get("/slots/{sid}")
    async def slot(sid: int):
        run = list(engine.scheduler.running)
        if not 0 <= sid < engine.cfg.max_num_seqs:
            raise HTTPException(404, "no such slot")
        if sid < len(run):
            r = run[sid]
            return {"id": sid, "is_processing": True, "n_ctx": engine.cfg.max_model_len, "n_past": r.num_computed,
                    "n_decoded": len(r.output), "request_id": r.request_id}
        return {"id": sid, "is_processing": False, "n_ctx": engine.cfg.max_model_len}

    # ------------------------------------------------------------------ Responses API
    def _response_object(rid, text, n_in, n_out, status="completed", reason="stop", body=None):
        msg, has_calls = ctx.shape_message(text)
        output = []
        if msg.get("reasoning_content"):
            output.append({"type": "reasoning", "id": "rs_" + uuid.uuid4().hex[:24],
                           "summary": [{"type": "summary_text", "text": msg["reasoning_content"]}]})
        for c in msg.get("tool_calls") or []:
            output.append({"type": "function_call", "id": "fc_" + uuid.uuid4().hex[:24], "call_id": c.get("id"),
                           "name": c["function"]["name"], "arguments": c["function"]["arguments"], "status": "completed"})
        if msg.get("content") or not output:
            output.append({"type": "message", "id": "msg_" + uuid.uuid4().hex[:24], "role": "assistant", "status": "completed",
                           "content": [{"type": "output_text", "text": msg.get("content") or "", "annotations": []}]})
        return {"id": rid, "object": "response", "created_at": int(time.time()), "status": status, "model": model_name,
                "output": output, "output_text": msg.get("content") or "",
                "incomplete_details": {"reason": "max_output_tokens"} if reason == "length" else None,
                "usage": {"input_tokens": n_in, "output_tokens": n_out, "total_tokens": n_in + n_out},
                "metadata": (body or {}).get("metadata") or {}, "previous_response_id": (body or {}).get("previous_response_id")}

    def _remember(obj: dict, messages: List[dict]) -> None:
        responses[obj["id"]] = {"object": obj, "messages": messages}
        while len(responses) > 512:
            responses.popitem(last=False)

    @app.post("/v1/responses")
    async def create_response(body: dict):
        msgs = _responses_input_to_messages(body)
        prev = body.get("previous_response_id")
        if prev:
            ent = responses.get(prev)
            if ent is None:
                raise HTTPException(404, f"response {prev!r} not found")
            msgs = ent["messages"] + msgs
        ids = ctx.chat_prompt(msgs, body.get("tools"))
        b2 = dict(body)
        if body.get("max_output_tokens") is not None:
            b2["max_tokens"] = body["max_output_tokens"]
        fmt = (body.get("text") or {}).get("format") or {}
        if fmt.get("type") in ("json_object", "json_schema"):
            b2["response_format"] = {"type": fmt["type"], "json_schema": {"schema": fmt.get("schema"), "name": fmt.get("name", "out")}}
        sp = ctx.sampling_from(b2, 512)
        ctx.attach_guided(sp, b2)
        rid = "resp_" + uuid.uuid4().hex
        if body.get("stream"):
            async def gen():
                seq = 0

                def ev(kind, **data):
                    nonlocal seq
                    seq += 1
                    return f"event: {kind}\ndata: {json.dumps(dict(data, type=kind, sequence_number=seq))}\n\n"
                shell = _response_object(rid, "", len(ids), 0, status="in_progress", body=body)
                yield ev("response.created", response=shell)
                item_id = "msg_" + uuid.uuid4().hex[:24]
                yield ev("response.output_item.added", output_index=0,
                         item={"type": "message", "id": item_id, "role": "assistant", "status": "in_progress", "content": []})
                text, n, reason = [], 0, "stop"
                async for piece in ctx.generate(ids, sp):
                    n += len(piece["tokens"])
                    if piece["text"]:
                        text.append(piece["text"])
                        yield ev("response.output_text.delta", item_id=item_id, output_index=0, content_index=0, delta=piece["text"])
                    if piece["finished"]:
                        reason = piece["reason"] or reason
                full = "".join(text)
                yield ev("response.output_text.done", item_id=item_id, output_index=0, content_index=0, text=full)
                obj = _response_object(rid, full, len(ids), n, reason=reason, body=body)
                if body.get("store", True):
                    _remember(obj, msgs + [{"role": "assistant", "content": full}])
                yield ev("response.completed", response=obj)
            return StreamingResponse(gen(), media_type="text/event-stream")
        text, toks, reason = await ctx.collect(ids, sp)
        obj = _response_object(rid, text, len(ids), len(toks), reason=reason, body=body)
        if body.get("store", True):
            _remember(obj, msgs + [{"role": "assistant", "content": text}])
        return obj

    @app.get("/v1/responses/{rid}")
    async def get_response(rid: str):
        ent = responses.get(rid)
        if ent is None:
            raise HTTPException(404, f"response {rid!r} not found")
        return ent["object"]

    @app.delete("/v1/responses/{rid}")
    async def delete_response(rid: str):
        if responses.pop(rid, None) is None:
            raise HTTPException(404, f"response {rid!r} not found")
        return {"id": rid, "object": "response", "deleted": True}

    # ------------------------------------------------------------------ Files
    def _file_meta(f: dict) -> dict:
        return {k: f[k] for k in ("id", "object", "bytes", "created_at", "filename", "purpose")}

    def _new_file(data: bytes, filename: str, purpose: str) -> dict:
        fid = "file-" + uuid.uuid4().hex[:24]
        files[fid] = {"id": fid, "object": "file", "bytes": len(data), "created_at": int(time.time()),
                      "filename": filename, "purpose": purpose, "data": data}
        return files[fid]

    @app.post("/v1/files")
    async def upload_file(request: HttpRequest):
        ctype = request.headers.get("content-type", "")
        if ctype.startswith("multipart/form-data"):
            try:
                form = await request.form()
            except Exception as e:                         # python-multipart missing or a malformed body
                raise HTTPException(400, f"cannot read the multipart body: {e}")
            up = form.get("file")
            if up is None:
                raise HTTPException(400, "multipart field 'file' is required")
            data = await up.read()
            return _file_meta(_new_file(data, getattr(up, "filename", "upload") or "upload", str(form.get("purpose") or "batch")))
        body = await request.json()
        content = body.get("content")
        if content is None:
            raise HTTPException(400, "send multipart/form-data with a 'file' part, or JSON {filename, purpose, content}")
        data = content.encode() if isinstance(content, str) else json.dumps(content).encode()
        return _file_meta(_new_file(data, str(body.get("filename") or "upload.jsonl"), str(body.get("purpose") or "batch")))

    @app.get("/v1/files")
    async def list_files():
        return {"object": "list", "data": [_file_meta(f) for f in files.values()]}

    @app.get("/v1/files/{fid}")
    async def get_file(fid: str):
        if fid not in files:
            raise HTTPException(404, f"file {fid!r} not found")
        return _file_meta(files[fid])

    @app.get("/v1/files/{fid}/content")
    async def file_content(fid: str):
        if fid not in files:
            raise HTTPException(404, f"file {fid!r} not found")
        return Response(files[fid]["data"], media_type="application/octet-stream")

    @app.delete("/v1/files/{fid}")
    async def delete_file(fid: str):
        if files.pop(fid, None) is None:
            raise HTTPException(404, f"file {fid!r} not found")
        return {"id": fid, "object": "file", "deleted": True}

    # ------------------------------------------------------------------ Batches
    async def _batch_line(url: str, body: dict) -> dict:
        if url == "/v1/chat/completions":
            ids = ctx.chat_prompt(body.get("messages") or [], body.get("tools"))
            sp = ctx.sampling_from(body, 256)
            ctx.attach_guided(sp, body)
            text, toks, reason = await ctx.collect(ids, sp)
            msg, has_calls = ctx.shape_message(text)
            return {"id": "chatcmpl-" + uuid.uuid4().hex, "object": "chat.completion", "created": int(time.time()), "model": model_name,
                    "choices": [{"index": 0, "message": msg, "finish_reason": "tool_calls" if has_calls else reason}],
                    "usage": ctx.usage(len(ids), len(toks))}
        if url == "/v1/completions":
            ids = ctx.encode_prompt(body.get("prompt", ""))
            sp = ctx.sampling_from(body, 16)
            text, toks, reason = await ctx.collect(ids, sp)
            return {"id": "cmpl-" + uuid.uuid4().hex, "object": "text_completion", "created": int(time.time()), "model": model_name,
                    "choices": [{"index": 0, "text": text, "token_ids": toks, "finish_reason": reason}],
                    "usage": ctx.usage(len(ids), len(toks))}
        if url == "/v1/embeddings":
            ids = ctx.encode_prompt(body.get("input", ""))
            vec = await ctx.embed_one(ids)
            return {"object": "list", "model": model_name, "data": [{"object": "embedding", "index": 0, "embedding": vec}],
                    "usage": {"prompt_tokens": len(ids), "total_tokens": len(ids)}}
        raise HTTPException(400, f"batches cannot call {url!r}")

    def _batch_meta(b: dict) -> dict:
        return {k: v for k, v in b.items() if k not in ("task",)}

    async def _run_batch(b: dict, lines: List[dict]) -> None:
        out, errs = [], []
        b["status"] = "in_progress"
        b["in_progress_at"] = int(time.time())
        sem = asyncio.Semaphore(max(1, engine.cfg.max_num_seqs))

        async def one(i, line):
            if b["status"] == "cancelling":
                return
            async with sem:
                cid = line.get("custom_id", str(i))
                try:
                    if line.get("method", "POST") != "POST":
                        raise HTTPException(400, "only POST lines are supported")
                    res = await _batch_line(line.get("url", b["endpoint"]), line.get("body") or {})
                    out.append({"id": "batch_req_" + uuid.uuid4().hex[:20], "custom_id": cid,
                                "response": {"status_code": 200, "request_id": uuid.uuid4().hex, "body": res}, "error": None})
                    b["request_counts"]["completed"] += 1
                except HTTPException as e:
                    errs.append({"id": "batch_req_" + uuid.uuid4().hex[:20], "custom_id": cid, "response": None,
                                 "error": {"code": str(e.status_code), "message": str(e.detail)}})
                    b["request_counts"]["failed"] += 1
                except Exception as e:
                    errs.append({"id": "batch_req_" + uuid.uuid4().hex[:20], "custom_id": cid, "response": None,
                                 "error": {"code": "500", "message": f"{type(e).__name__}: {e}"}})
                    b["request_counts"]["failed"] += 1
        await asyncio.gather(*[one(i, l) for i, l in enumerate(lines)])
        if out:
            b["output_file_id"] = _new_file("\n".join(json.dumps(o) for o in out).encode(), f"{b['id']}_output.jsonl", "batch_output")["id"]
        if errs:
            b["error_file_id"] = _new_file("\n".join(json.dumps(o) for o in errs).encode(), f"{b['id']}_errors.jsonl", "batch_output")["id"]
        if b["status"] == "cancelling":
            b["status"], b["cancelled_at"] = "cancelled", int(time.time())
        else:
            b["status"], b["completed_at"] = "completed", int(time.time())

    @app.post("/v1/batches")
    async def create_batch(body: dict):
        fid = body.get("input_file_id")
        if fid not in files:
            raise HTTPException(404, f"input file {fid!r} not found")
        endpoint = body.get("endpoint", "/v1/chat/completions")
        if endpoint not in ("/v1/chat/completions", "/v1/completions", "/v1/embeddings"):
            raise HTTPException(400, f"unsupported endpoint {endpoint!r}")
        lines = []
        for n, raw in enumerate(files[fid]["data"].decode("utf-8", "replace").splitlines()):
            if raw.strip():
                try:
                    lines.append(json.loads(raw))
                except json.JSONDecodeError as e:
                    raise HTTPException(400, f"line {n + 1} of the input file is not JSON: {e}")
        bid = "batch_" + uuid.uuid4().hex[:24]
        b = {"id": bid, "object": "batch", "endpoint": endpoint, "errors": None, "input_file_id": fid,
             "completion_window": body.get("completion_window", "24h"), "status": "validating", "output_file_id": None,
             "error_file_id": None, "created_at": int(time.time()), "in_progress_at": None, "completed_at": None,
             "cancelled_at": None, "request_counts": {"total": len(lines), "completed": 0, "failed": 0},
             "metadata": body.get("metadata")}
        batches[bid] = b
        b["task"] = asyncio.get_running_loop().create_task(_run_batch(b, lines))
        return _batch_meta(b)

    @app.get("/v1/batches")
    async def list_batches():
        return {"object": "list", "data": [_batch_meta(b) for b in batches.values()]}

    @app.get("/v1/batches/{bid}")
    async def get_batch(bid: str):
        if bid not in batches:
            raise HTTPException(404, f"batch {bid!r} not found")
        return _batch_meta(batches[bid])

    @app.post("/v1/batches/{bid}/cancel")
    async def cancel_batch(bid: str):
        if bid not in batches:
            raise HTTPException(404, f"batch {bid!r} not found")
        b = batches[bid]
        if b["status"] in ("validating", "in_progress"):
            b["status"] = "cancelling"
        return _batch_meta(b)

    # ------------------------------------------------------------------ scoring on a decoder
    def _texts(x) -> List[str]:
        if isinstance(x, str):
            return [x]
        if isinstance(x, list) and all(isinstance(t, str) for t in x):
            return list(x)
        if isinstance(x, list) and all(isinstance(t, dict) and "text" in t for t in x):
            return [t["text"] for t in x]
        raise HTTPException(400, "expected a string or a list of strings")

    async def _embed_text(t: str) -> List[float]:
        return await ctx.embed_one(tokenizer.encode(t, add_bos=True))

    async def _rerank(body: dict):
        query = body.get("query")
        docs = _texts(body.get("documents") or [])
        if not isinstance(query, str) or not docs:
            raise HTTPException(400, "query (string) and documents (non-empty list) are required")
        qv, *dv = await asyncio.gather(_embed_text(query), *[_embed_text(d) for d in docs])
        scored = sorted(({"index": i, "relevance_score": _cos(qv, v)} for i, v in enumerate(dv)), key=lambda r: -r["relevance_score"])
        top = body.get("top_n") or body.get("top_k")
        if top:
            scored = scored[: int(top)]
        if body.get("return_documents", False):
            for r in scored:
                r["document"] = {"text": docs[r["index"]]}
        n_tok = len(tokenizer.encode(query, add_bos=True)) + sum(len(tokenizer.encode(d, add_bos=True)) for d in docs)
        return {"id": "rerank-" + uuid.uuid4().hex, "model": model_name, "results": scored,
                "usage": {"total_tokens": n_tok}}

    @app.post("/v1/rerank")
    async def rerank_v1(body: dict):
        return await _rerank(body)

    @app.post("/rerank")
    async def rerank(body: dict):
        return await _rerank(body)

    @app.post("/v1/score")
    async def score(body: dict):
        a, b = _texts(body.get("text_1")), _texts(body.get("text_2"))
        if len(a) == 1:
            a = a * len(b)
        if len(a) != len(b):
            raise HTTPException(400, "text_1 must be one text or as many as text_2")
        va = await asyncio.gather(*[_embed_text(t) for t in a])
        vb = await asyncio.gather(*[_embed_text(t) for t in b])
        return {"id": "score-" + uuid.uuid4().hex, "object": "list", "model": model_name,
                "data": [{"index": i, "object": "score", "score": _cos(x, y)} for i, (x, y) in enumerate(zip(va, vb))],
                "usage": {"total_tokens": sum(len(tokenizer.encode(t, add_bos=True)) for t in a + b)}}

    @app.post("/pooling")
    async def pooling(body: dict):
        texts = _texts(body.get("input"))
        vecs = await asyncio.gather(*[_embed_text(t) for t in texts])
        return {"id": "pool-" + uuid.uuid4().hex, "object": "list", "model": model_name,
                "data": [{"index": i, "object": "pooling", "data": v} for i, v in enumerate(vecs)]}

    @app.post("/classify")
    async def classify(body: dict):
        """Zero-shot classification on a generative model: the probability of each label's first token right after
        the input (and an optional instruction), renormalised over the labels."""
        texts = _texts(body.get("input"))
        labels = body.get("labels")
        if not (isinstance(labels, list) and labels and all(isinstance(l, str) for l in labels)):
            raise HTTPException(400, "labels (non-empty list of strings) are required for a model without a classification head")
        first = [tokenizer.encode(" " + l, add_bos=False)[0] if tokenizer.encode(" " + l, add_bos=False) else 0 for l in labels]
        out = []
        for i, t in enumerate(texts):
            ids = tokenizer.encode((body.get("instruction") or "") + t, add_bos=True)
            sp = SamplingParams(max_tokens=1, temperature=0.0, ignore_eos=True, allowed_token_ids=sorted(set(first)),
                                logprobs=True, top_logprobs=min(20, len(set(first))))
            lp = {}
            async for piece in ctx.generate(ids, sp):
                for alt in (piece.get("top_logprobs") or []):
                    lp.update({int(a): float(b) for a, b in alt})
            raw = [math.exp(lp.get(f, -30.0)) for f in first]
            z = sum(raw) or 1.0
            probs = [r / z for r in raw]
            best = max(range(len(labels)), key=lambda j: probs[j])
            out.append({"index": i, "label": labels[best], "probs": probs, "num_classes": len(labels)})
        return {"id": "classify-" + uuid.uuid4().hex, "object": "list", "model": model_name, "data": out}

    @app.post("/embeddings")
    async def embeddings_alias(body: dict):
        texts = _texts(body.get("input") if body.get("input") is not None else body.get("content"))
        vecs = await asyncio.gather(*[_embed_text(t) for t in texts])
        return {"object": "list", "model": model_name,
                "data": [{"object": "embedding", "index": i, "embedding": v} for i, v in enumerate(vecs)]}

    # ------------------------------------------------------------------ llama.cpp infill
    def _special(*names) -> Optional[int]:
        for n in names:
            try:
                ids = tokenizer.encode(n, add_bos=False)
            except Exception:
                continue
            if len(ids) == 1:
                return ids[0]
        return None

    @app.post("/infill")
    async def infill(body: dict):
        prefix, suffix = str(body.get("input_prefix", "")), str(body.get("input_suffix", ""))
        pre = _special("<|fim_prefix|>", "<fim_prefix>", "<PRE>", "▁<PRE>")
        suf = _special("<|fim_suffix|>", "<fim_suffix>", "<SUF>", "▁<SUF>")
        mid = _special("<|fim_middle|>", "<fim_middle>", "<MID>", "▁<MID>")
        if None not in (pre, suf, mid):
            ids = [pre] + tokenizer.encode(prefix, add_bos=False) + [suf] + tokenizer.encode(suffix, add_bos=False) + [mid]
        else:                                         # no fill-in-the-middle tokens in this vocabulary: continue the prefix
            ids = tokenizer.encode(str(body.get("prompt", "")) + prefix, add_bos=True)
        sp = ctx.sampling_from(body, 128, "llamacpp")
        if body.get("stream"):
            async def gen():
                async for piece in ctx.generate(ids, sp):
                    yield f"data: {json.dumps({'content': piece['text'], 'stop': piece['finished']})}\n\n"
            return StreamingResponse(gen(), media_type="text/event-stream")
        text, toks, reason = await ctx.collect(ids, sp)
        return {"content": text, "stop": True, "tokens_predicted": len(toks), "tokens_evaluated": len(ids),
                "stopped_limit": reason == "length", "stopped_eos": reason == "stop", "model": model_name}

    # ------------------------------------------------------------------ Ollama model management (one local model)
    def _known(name: Optional[str]) -> bool:
        return bool(name) and name.split(":")[0] in (model_name, model_name.split(":")[0])

    @app.post("/api/pull")
    async def ollama_pull(body: dict):
        name = body.get("model") or body.get("name")
        if not _known(name):
            raise HTTPException(404, f"model {name!r} is not available: this server holds {model_name!r} and cannot download")
        return {"status": "success"}

    @app.post("/api/push")
    async def ollama_push(body: dict):
        raise HTTPException(501, "pushing models to a registry is not available")

    @app.post("/api/create")
    async def ollama_create(body: dict):
        raise HTTPException(501, "creating models from a Modelfile is not available; start the server with the model to serve")

    @app.post("/api/copy")
    async def ollama_copy(body: dict):
        if not _known(body.get("source")):
            raise HTTPException(404, f"model {body.get('source')!r} not found")
        raise HTTPException(501, "model aliases are not available")

    @app.delete("/api/delete")
    async def ollama_delete(body: dict):
        name = body.get("model") or body.get("name")
        if not _known(name):
            raise HTTPException(404, f"model {name!r} not found")
        raise HTTPException(501, "the served model cannot be deleted while the server runs")

    @app.head("/api/blobs/{digest}")
    async def ollama_blob_head(digest: str):
        raise HTTPException(404, "no such blob")

    @app.post("/api/blobs/{digest}")
    async def ollama_blob_post(digest: str):
        raise HTTPException(501, "blob uploads are not available")
