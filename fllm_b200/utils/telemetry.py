"""Request spans exported as OTLP/HTTP JSON, and an operator profiler.

``SpanExporter`` batches finished spans (128 per request or every 2 s, whichever comes first) and posts
them from a background thread to ``<endpoint>/v1/traces`` in the OpenTelemetry protocol's JSON
encoding; nothing is exported when no endpoint is configured (``OTEL_EXPORTER_OTLP_ENDPOINT`` or the
constructor argument). Export failures are counted, never raised into the serving path
(rust/engine/src/telemetry.rs:1-20 is the reference's exporter).

``OpProfiler`` wraps the operator object: a CUDA-event pair around every call, a table of calls / total /
mean per operator and token-count class, printed on demand (``FLLM_PROFILE=1`` in the CLI; the
reference's ``FLLM_CUDA_PROFILE``, rust/engine/cuda/linear.cu:757-789).
"""
from __future__ import annotations

import json
import os
import queue
import secrets
import threading
import time
import urllib.request
from typing import Dict, List, Optional


def _attr(k: str, v) -> dict:
    if isinstance(v, bool):
        return {"key": k, "value": {"boolValue": v}}
    if isinstance(v, int):
        return {"key": k, "value": {"intValue": str(v)}}
    if isinstance(v, float):
        return {"key": k, "value": {"doubleValue": v}}
    return {"key": k, "value": {"stringValue": str(v)}}


class Span:
    __slots__ = ("name", "trace_id", "span_id", "start_ns", "end_ns", "attrs", "events", "ok")

    def __init__(self, name: str, trace_id: Optional[str] = None):
        self.name = name
        self.trace_id = trace_id or secrets.token_hex(16)
        self.span_id = secrets.token_hex(8)
        self.start_ns = time.time_ns()
        self.end_ns = 0
        self.attrs: Dict[str, object] = {}
        self.events: List[tuple] = []
        self.ok = True

    def event(self, name: str) -> None:
        self.events.append((name, time.time_ns()))

    def to_otlp(self) -> dict:
        return {"traceId": self.trace_id, "spanId": self.span_id, "name": self.name, "kind": 2,
                "startTimeUnixNano": str(self.start_ns), "endTimeUnixNano": str(self.end_ns or time.time_ns()),
                "attributes": [_attr(k, v) for k, v in self.attrs.items()],
                "events": [{"name": n, "timeUnixNano": str(t)} for n, t in self.events],
                "status": {"code": 1 if self.ok else 2}}


class SpanExporter:
    def __init__(self, endpoint: Optional[str] = None, service: str = "fllm_b200", batch: int = 128, period_s: float = 2.0):
        self.endpoint = (endpoint or os.environ.get("OTEL_EXPORTER_OTLP_ENDPOINT") or "").rstrip("/")
        self.service, self.batch, self.period_s = service, batch, period_s
        self.q: "queue.Queue[Span]" = queue.Queue(maxsize=8192)
        self.exported = self.dropped = self.failed_posts = 0
        self._stop = threading.Event()
        self.thread = None
        if self.endpoint:
            self.thread = threading.Thread(target=self._run, name="fllm-otlp", daemon=True)
            self.thread.start()

    @property
    def enabled(self) -> bool:
        return bool(self.endpoint)

    def start_span(self, name: str, **attrs) -> Span:
        s = Span(name)
        s.attrs.update(attrs)
        return s

    def end_span(self, span: Span, ok: bool = True, **attrs) -> None:
        span.end_ns = time.time_ns()
        span.ok = ok
        span.attrs.update(attrs)
        if not self.enabled:
            return
        try:
            self.q.put_nowait(span)
        except queue.Full:
            self.dropped += 1

    def _payload(self, spans: List[Span]) -> bytes:
        return json.dumps({"resourceSpans": [{
            "resource": {"attributes": [_attr("service.name", self.service)]},
            "scopeSpans": [{"scope": {"name": "fllm_b200.server"}, "spans": [s.to_otlp() for s in spans]}]}]}).encode()

    def _post(self, spans: List[Span]) -> None:
        req = urllib.request.Request(self.endpoint + "/v1/traces", data=self._payload(spans),
                                     headers={"Content-Type": "application/json"}, method="POST")
        try:
            with urllib.request.urlopen(req, timeout=5) as r:
                r.read()
            self.exported += len(spans)
        except Exception:
            self.failed_posts += 1
            self.dropped += len(spans)

    def _run(self) -> None:
        pending: List[Span] = []
        deadline = time.monotonic() + self.period_s
        while not self._stop.is_set() or not self.q.empty() or pending:
            try:
                pending.append(self.q.get(timeout=max(0.01, min(0.2, deadline - time.monotonic()))))
            except queue.Empty:
                pass
            now = time.monotonic()
            if pending and (len(pending) >= self.batch or now >= deadline or self._stop.is_set()):
                self._post(pending[: self.batch])
                pending = pending[self.batch:]
            if now >= deadline:
                deadline = now + self.period_s

    def shutdown(self, timeout: float = 5.0) -> None:
        self._stop.set()
        if self.thread is not None:
            self.thread.join(timeout)

    def stats(self) -> dict:
        return {"enabled": self.enabled, "exported": self.exported, "dropped": self.dropped,
                "failed_posts": self.failed_posts, "queued": self.q.qsize()}


class OpProfiler:
    """Proxy around an operator object (``NativeOps`` / ``RefOps``) that times every call."""

    def __init__(self, ops):
        object.__setattr__(self, "_ops", ops)
        object.__setattr__(self, "_rows", {})
        object.__setattr__(self, "_pending", [])

    def __getattr__(self, name):
        target = getattr(self._ops, name)
        if not callable(target) or name.startswith("_") or name in ("check_status", "scratch_bf16"):
            return target
        import torch

        def timed(*a, **k):
            first = a[0] if a else None
            rows = int(first.shape[0]) if hasattr(first, "shape") and len(first.shape) else 0
            cls = "<=16" if rows <= 16 else "<=128" if rows <= 128 else ">128"
            cuda = torch.cuda.is_available() and getattr(first, "is_cuda", False)
            if cuda:
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                out = target(*a, **k)
                e1.record()
                self._pending.append((name, cls, e0, e1))
            else:
                t0 = time.perf_counter()
                out = target(*a, **k)
                self._add(name, cls, (time.perf_counter() - t0) * 1e3)
            return out
        return timed

    def __setattr__(self, name, value):
        setattr(self._ops, name, value)

    def _add(self, name, cls, ms):
        r = self._rows.setdefault((name, cls), [0, 0.0])
        r[0] += 1
        r[1] += ms

    def table(self) -> str:
        if self._pending:
            import torch
            torch.cuda.synchronize()
            for name, cls, e0, e1 in self._pending:
                self._add(name, cls, e0.elapsed_time(e1))
            self._pending.clear()
        lines = [f"{'operator':20s} {'rows':>6s} {'calls':>8s} {'total ms':>10s} {'mean us':>9s}"]
        for (name, cls), (n, ms) in sorted(self._rows.items(), key=lambda kv: -kv[1][1]):
            lines.append(f"{name:20s} {cls:>6s} {n:8d} {ms:10.2f} {ms / n * 1e3:9.1f}")
        return "\n".join(lines)
