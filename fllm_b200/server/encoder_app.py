"""HTTP front end of an encoder model (BERT / RoBERTa / XLM-R): embeddings, pooling, classification, and
cross-encoder scoring / reranking, in the request shapes of the OpenAI, vLLM, Cohere / Jina and TEI APIs
(rust/engine/src/encoder_server.rs:1233-1266 lists the same routes for the reference's encoder server).
Requests are batched by a token budget and run on a worker thread; the model call itself is synchronous."""
import asyncio
import threading
import time
from typing import List, Optional, Sequence

import torch


class EncoderService:
    """Tokenise, batch by token budget, run."""

    def __init__(self, encoder, tokenizer, max_batch_tokens: int = 8192):
        self.enc, self.tok, self.max_batch_tokens = encoder, tokenizer, max_batch_tokens
        self.lock = threading.Lock()
        self.requests = 0
        self.tokens = 0

    # ---- tokenisation with the model's special tokens
    def ids(self, text, pair=None):
        tk = getattr(self.tok, "tk", None)
        if tk is not None:                                    # a tokenizers.Tokenizer: its post-processor adds [CLS] / [SEP]
            e = tk.encode(text, pair, add_special_tokens=True) if pair is not None else tk.encode(text, add_special_tokens=True)
            ids, types = list(e.ids), list(e.type_ids)
        else:
            ids = self.tok.encode(text) + (self.tok.encode(pair) if pair is not None else [])
            types = [0] * len(ids)
        limit = self.enc.cfg.max_position - self.enc.cfg.position_offset
        return ids[:limit], types[:limit]

    def _batches(self, items):
        batch, n = [], 0
        for it in items:
            if batch and n + len(it[0]) > self.max_batch_tokens:
                yield batch
                batch, n = [], 0
            batch.append(it)
            n += len(it[0])
        if batch:
            yield batch

    def _run(self, items, fn):
        outs = []
        with self.lock:
            for b in self._batches(items):
                outs.append(fn([x[0] for x in b], [x[1] for x in b]))
                self.tokens += sum(len(x[0]) for x in b)
        self.requests += 1
        return torch.cat(outs, 0)

    def embed(self, texts: Sequence, pooling: Optional[str] = None, normalize: bool = True) -> "tuple[List[List[float]], int]":
        items = [self.ids(t) if isinstance(t, str) else (list(t), [0] * len(t)) for t in texts]
        v = self._run(items, lambda s, ty: self.enc.embed(s, ty, pooling, normalize).float().cpu())
        return v.tolist(), sum(len(i[0]) for i in items)

    def classify(self, texts: Sequence[str], pairs: Optional[Sequence[str]] = None) -> "tuple[List[List[float]], int]":
        items = [self.ids(t, pairs[i] if pairs is not None else None) for i, t in enumerate(texts)]
        v = self._run(items, lambda s, ty: self.enc.classify(s, ty).float().cpu())
        return v.tolist(), sum(len(i[0]) for i in items)

    def score(self, query: str, docs: Sequence[str]) -> "tuple[List[float], int]":
        """Relevance of every document to the query: the cross-encoder head when the checkpoint has one (sigmoid of
        a single logit, or the probability of the last label), else the cosine of the two embeddings."""
        if self.enc.w.cls_w is not None:
            lg, n = self.classify([query] * len(docs), list(docs))
            t = torch.tensor(lg)
            s = torch.sigmoid(t[:, 0]) if t.shape[1] == 1 else torch.softmax(t, -1)[:, -1]
            return s.tolist(), n
        v, n = self.embed([query] + list(docs))
        t = torch.tensor(v)
        return (t[1:] @ t[0]).tolist(), n


def create_encoder_app(service: EncoderService, model_name: str, api_key: Optional[str] = None):
    from fastapi import FastAPI, HTTPException, Request
    from fastapi.responses import JSONResponse

    app = FastAPI(title="fllm_b200 encoder")
    started = time.time()

    def check(req: Request):
        if api_key and req.headers.get("authorization", "") != f"Bearer {api_key}":
            raise HTTPException(401, "invalid api key")

    async def body_of(req: Request) -> dict:
        check(req)
        try:
            b = await req.json()
        except Exception:
            raise HTTPException(400, "body is not JSON")
        if not isinstance(b, dict):
            raise HTTPException(400, "body must be an object")
        return b

    def as_list(x, what):
        if isinstance(x, str):
            return [x]
        if isinstance(x, list) and x and all(isinstance(i, (str, list)) for i in x):
            return x
        raise HTTPException(400, f"{what} must be a string or a non-empty list")

    async def call(fn, *a):
        try:
            return await asyncio.get_running_loop().run_in_executor(None, fn, *a)
        except ValueError as e:
            raise HTTPException(400, str(e))

    @app.get("/health")
    @app.get("/ready")
    async def health():
        return {"status": "ok"}

    @app.get("/v1/models")
    async def models():
        return {"object": "list", "data": [{"id": model_name, "object": "model", "created": int(started), "owned_by": "fllm_b200",
                                            "task": "classify" if service.enc.w.cls_w is not None else "embed"}]}

    @app.get("/info")
    async def info():
        c = service.enc.cfg
        return {"model_id": model_name, "model_type": c.arch, "max_input_length": c.max_position - c.position_offset,
                "hidden_size": c.hidden_size, "requests": service.requests, "tokens": service.tokens}

    @app.post("/tokenize")
    async def tokenize(req: Request):
        b = await body_of(req)
        ids, types = service.ids(b.get("text") or b.get("content") or b.get("prompt") or "", b.get("text_pair"))
        return {"tokens": ids, "token_type_ids": types, "count": len(ids)}

    @app.post("/v1/embeddings")
    @app.post("/embeddings")
    async def embeddings(req: Request):
        b = await body_of(req)
        texts = as_list(b.get("input"), "input")
        vecs, n = await call(service.embed, texts, b.get("pooling"), b.get("normalize", True))
        dims = b.get("dimensions")
        if dims:
            vecs = [v[:int(dims)] for v in vecs]
        return {"object": "list", "model": model_name,
                "data": [{"object": "embedding", "index": i, "embedding": v} for i, v in enumerate(vecs)],
                "usage": {"prompt_tokens": n, "total_tokens": n}}

    @app.post("/embed")                                         # TEI
    async def tei_embed(req: Request):
        b = await body_of(req)
        vecs, _ = await call(service.embed, as_list(b.get("inputs"), "inputs"), None, b.get("normalize", True))
        return JSONResponse(vecs)

    @app.post("/pooling")
    async def pooling(req: Request):
        b = await body_of(req)
        vecs, n = await call(service.embed, as_list(b.get("input"), "input"), b.get("pooling"), False)
        return {"object": "list", "model": model_name, "data": [{"object": "pooling", "index": i, "data": v} for i, v in enumerate(vecs)],
                "usage": {"prompt_tokens": n, "total_tokens": n}}

    @app.post("/classify")
    async def classify(req: Request):
        b = await body_of(req)
        texts = as_list(b.get("input"), "input")
        if service.enc.w.cls_w is None:
            raise HTTPException(400, "this model has no classification head")
        lg, n = await call(service.classify, texts, None)
        data = []
        for i, row in enumerate(lg):
            p = torch.softmax(torch.tensor(row), -1).tolist() if len(row) > 1 else [float(torch.sigmoid(torch.tensor(row[0])))]
            data.append({"index": i, "label": int(max(range(len(p)), key=p.__getitem__)), "probs": p, "num_classes": len(p)})
        return {"object": "list", "model": model_name, "data": data, "usage": {"prompt_tokens": n, "total_tokens": n}}

    @app.post("/v1/score")
    @app.post("/score")
    async def score(req: Request):
        b = await body_of(req)
        q, docs = b.get("text_1"), as_list(b.get("text_2"), "text_2")
        if not isinstance(q, str):
            raise HTTPException(400, "text_1 must be a string")
        s, n = await call(service.score, q, docs)
        return {"object": "list", "model": model_name, "data": [{"object": "score", "index": i, "score": v} for i, v in enumerate(s)],
                "usage": {"prompt_tokens": n, "total_tokens": n}}

    @app.post("/v1/rerank")
    @app.post("/rerank")
    async def rerank(req: Request):
        b = await body_of(req)
        q = b.get("query")
        docs = b.get("documents") or b.get("texts")
        if not isinstance(q, str) or not isinstance(docs, list) or not docs:
            raise HTTPException(400, "query (string) and documents (list) are required")
        texts = [d if isinstance(d, str) else str(d.get("text", "")) for d in docs]
        s, n = await call(service.score, q, texts)
        order = sorted(range(len(s)), key=lambda i: -s[i])[: int(b.get("top_n") or len(s))]
        res = [{"index": i, "relevance_score": s[i], **({"document": {"text": texts[i]}} if b.get("return_documents") else {})} for i in order]
        return {"id": f"rerank-{int(time.time() * 1000)}", "model": model_name, "results": res, "usage": {"total_tokens": n}}

    return app


def serve_encoder(encoder, tokenizer, host: str, port: int, model_name: str, api_key: Optional[str] = None,
                  log_level: str = "warning", ssl_certfile: Optional[str] = None, ssl_keyfile: Optional[str] = None):
    import uvicorn
    app = create_encoder_app(EncoderService(encoder, tokenizer), model_name, api_key)
    uvicorn.run(app, host=host, port=port, log_level=log_level, ssl_certfile=ssl_certfile, ssl_keyfile=ssl_keyfile)
