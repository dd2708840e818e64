"""Prometheus text exposition without a client library: counters, gauges and histograms under
``fllm_*`` names with ``vllm:*`` aliases for dashboards built for that server
(rust/engine/src/metrics.rs; docs/telemetry.md:27-32)."""
from __future__ import annotations

import threading
from typing import Dict, List, Sequence, Tuple

_BUCKETS_S = (0.001, 0.005, 0.01, 0.02, 0.04, 0.06, 0.08, 0.1, 0.25, 0.5, 0.75, 1.0, 2.5, 5.0, 7.5, 10.0, 20.0, 40.0, 80.0)


class Histogram:
    def __init__(self, buckets: Sequence[float] = _BUCKETS_S):
        self.buckets = list(buckets)
        self.counts = [0] * (len(self.buckets) + 1)
        self.total, self.n = 0.0, 0

    def observe(self, v: float) -> None:
        self.total += v
        self.n += 1
        for i, b in enumerate(self.buckets):
            if v <= b:
                self.counts[i] += 1
                return
        self.counts[-1] += 1

    def quantile(self, q: float) -> float:
        if not self.n:
            return 0.0
        target, acc = q * self.n, 0
        for i, c in enumerate(self.counts):
            acc += c
            if acc >= target:
                return self.buckets[i] if i < len(self.buckets) else self.buckets[-1]
        return self.buckets[-1]


class Metrics:
    ALIASES = {
        "fllm_requests_total": "vllm:request_success_total",
        "fllm_prompt_tokens_total": "vllm:prompt_tokens_total",
        "fllm_generation_tokens_total": "vllm:generation_tokens_total",
        "fllm_time_to_first_token_seconds": "vllm:time_to_first_token_seconds",
        "fllm_inter_token_latency_seconds": "vllm:time_per_output_token_seconds",
        "fllm_e2e_request_latency_seconds": "vllm:e2e_request_latency_seconds",
        "fllm_requests_running": "vllm:num_requests_running",
        "fllm_requests_waiting": "vllm:num_requests_waiting",
        "fllm_kv_cache_usage": "vllm:gpu_cache_usage_perc",
    }

    def __init__(self):
        self.lock = threading.Lock()
        self.counters: Dict[str, float] = {}
        self.gauges: Dict[str, float] = {}
        self.hists: Dict[str, Histogram] = {}

    def inc(self, name: str, v: float = 1.0) -> None:
        with self.lock:
            self.counters[name] = self.counters.get(name, 0.0) + v

    def set(self, name: str, v: float) -> None:
        with self.lock:
            self.gauges[name] = v

    def observe(self, name: str, v: float) -> None:
        with self.lock:
            self.hists.setdefault(name, Histogram()).observe(v)

    def render(self) -> str:
        out: List[str] = []

        def emit(name: str, kind: str, rows: List[Tuple[str, float]]):
            for n in (name, self.ALIASES.get(name)):
                if not n:
                    continue
                out.append(f"# TYPE {n} {kind}")
                for suffix, v in rows:
                    out.append(f"{n}{suffix} {v}")

        with self.lock:
            for k, v in sorted(self.counters.items()):
                emit(k, "counter", [("", v)])
            for k, v in sorted(self.gauges.items()):
                emit(k, "gauge", [("", v)])
            for k, h in sorted(self.hists.items()):
                rows, acc = [], 0
                for b, c in zip(h.buckets, h.counts):
                    acc += c
                    rows.append((f'_bucket{{le="{b}"}}', acc))
                rows.append(('_bucket{le="+Inf"}', h.n))
                rows.append(("_sum", h.total))
                rows.append(("_count", h.n))
                emit(k, "histogram", rows)
        return "\n".join(out) + "\n"
