"""Replica router: one HTTP front for several engine servers (data-parallel replicas).

Every replica is a complete server (``python -m fllm_b200 serve``) on its own GPU or GPU group; the
router forwards each request to one of them:

* ``prefix``       requests whose prompts share a prefix go to the same replica (rendezvous hashing on
                   the first characters of the prompt / conversation), so that replica's prefix cache
                   keeps hitting; a replica that is not ready is skipped and the choice falls to the
                   next one in the request's hash order;
* ``least_loaded`` the ready replica with the fewest requests in flight;
* ``round_robin``.

Streaming responses (SSE / NDJSON) are passed through chunk by chunk; a request that fails before
its first byte is retried once on another replica. ``/health``, ``/ready``, ``/metrics`` and
``/v1/models`` are answered by the router itself (rust/router/src/main.rs is the reference's
``fllm-router``).
"""
from __future__ import annotations

import asyncio
import hashlib
import itertools
import json
import time
from typing import Dict, List, Optional

import httpx
from fastapi import FastAPI, Request, Response
from fastapi.responses import JSONResponse, PlainTextResponse, StreamingResponse

POLICIES = ("prefix", "least_loaded", "round_robin")
_HOP = {"connection", "keep-alive", "transfer-encoding", "content-length", "host", "content-encoding"}


class Replica:
    def __init__(self, name: str, client: httpx.AsyncClient):
        self.name, self.client = name, client
        self.inflight = 0
        self.ready = True
        self.served = self.failed = 0
        self.last_check = 0.0


def _affinity_key(path: str, body: Optional[dict], prefix_chars: int) -> str:
    """What two requests must share to land on the same replica."""
    if not body:
        return path
    if isinstance(body.get("messages"), list):
        text = json.dumps(body["messages"], sort_keys=True)
    else:
        p = body.get("prompt", body.get("inputs", body.get("content", body.get("input", ""))))
        text = p if isinstance(p, str) else json.dumps(p)
    return (str(body.get("cache_salt", "")) + "|" + text)[: prefix_chars + 64]


def create_router(replicas: Dict[str, httpx.AsyncClient], policy: str = "prefix", prefix_chars: int = 256,
                  health_period_s: float = 2.0) -> FastAPI:
    if policy not in POLICIES:
        raise ValueError(f"policy must be one of {POLICIES}")
    if not replicas:
        raise ValueError("at least one replica")
    reps = [Replica(n, c) for n, c in replicas.items()]
    rr = itertools.count()
    app = FastAPI(title="fllm_b200 router")
    app.state.replicas = reps

    async def refresh(rep: Replica) -> None:
        now = time.monotonic()
        if now - rep.last_check < health_period_s:
            return
        rep.last_check = now
        try:
            r = await rep.client.get("/ready", timeout=2.0)
            rep.ready = r.status_code == 200
        except Exception:
            rep.ready = False

    def order(key: str) -> List[Replica]:
        if policy == "round_robin":
            i = next(rr) % len(reps)
            return reps[i:] + reps[:i]
        if policy == "least_loaded":
            return sorted(reps, key=lambda r: (r.inflight, r.name))
        # rendezvous hashing: each replica scores the key, highest score first
        score = lambda r: hashlib.sha256((r.name + "\0" + key).encode()).digest()
        return sorted(reps, key=score, reverse=True)

    @app.get("/health")
    async def health():
        return {"status": "ok", "replicas": len(reps)}

    @app.get("/ready")
    async def ready():
        await asyncio.gather(*[refresh(r) for r in reps])
        ok = any(r.ready for r in reps)
        return JSONResponse({"ready": ok, "replicas": {r.name: r.ready for r in reps}}, 200 if ok else 503)

    @app.get("/metrics")
    async def metrics():
        lines = []
        for r in reps:
            lab = f'{{replica="{r.name}"}}'
            lines += [f"fllm_router_inflight{lab} {r.inflight}", f"fllm_router_served_total{lab} {r.served}",
                      f"fllm_router_failed_total{lab} {r.failed}", f"fllm_router_ready{lab} {1 if r.ready else 0}"]
        return PlainTextResponse("\n".join(lines) + "\n")

    @app.api_route("/{path:path}", methods=["GET", "POST", "DELETE"])
    async def forward(path: str, request: Request):
        raw = await request.body()
        body = None
        if raw and request.headers.get("content-type", "").startswith("application/json"):
            try:
                body = json.loads(raw)
            except ValueError:
                return JSONResponse({"error": {"message": "invalid JSON body"}}, 400)
        await asyncio.gather(*[refresh(r) for r in reps])
        key = _affinity_key("/" + path, body if isinstance(body, dict) else None, prefix_chars)
        candidates = [r for r in order(key) if r.ready] or order(key)
        headers = {k: v for k, v in request.headers.items() if k.lower() not in _HOP}
        last_err: Optional[str] = None
        for rep in candidates[:2]:                       # one retry on another replica
            rep.inflight += 1
            try:
                req = rep.client.build_request(request.method, "/" + path, content=raw, headers=headers,
                                               params=dict(request.query_params), timeout=None)
                resp = await rep.client.send(req, stream=True)
            except Exception as e:                       # connect / send failure: nothing reached the client yet
                rep.inflight -= 1
                rep.failed += 1
                rep.ready = False
                last_err = f"{type(e).__name__}: {e}"
                continue
            out_headers = {k: v for k, v in resp.headers.items() if k.lower() not in _HOP}
            out_headers["x-fllm-replica"] = rep.name

            async def relay(resp=resp, rep=rep):
                try:
                    async for chunk in resp.aiter_raw():
                        yield chunk
                    rep.served += 1
                except Exception:
                    rep.failed += 1
                    raise
                finally:
                    rep.inflight -= 1
                    await resp.aclose()
            return StreamingResponse(relay(), status_code=resp.status_code, headers=out_headers,
                                     media_type=resp.headers.get("content-type"))
        return JSONResponse({"error": {"message": f"no replica could take the request ({last_err})",
                                       "type": "service_unavailable"}}, 503)

    return app


def serve_router(urls: List[str], host: str = "127.0.0.1", port: int = 8080, policy: str = "prefix",
                 log_level: str = "info") -> None:
    import uvicorn
    clients = {u: httpx.AsyncClient(base_url=u, timeout=None) for u in urls}
    uvicorn.run(create_router(clients, policy), host=host, port=port, log_level=log_level)
