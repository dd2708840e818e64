"""HTTP load generator for a running server (``python -m fllm_b200 bench-serve``): N requests at a fixed
concurrency against ``/v1/completions`` with streaming, reporting request throughput, output token
throughput, time to first token and inter-token latency percentiles (the reference's ``bench-serve``,
rust/engine/src/bin/bench_serve.rs)."""
from __future__ import annotations

import asyncio
import json
import random
import statistics
import time
from typing import List, Optional

import httpx


def _pct(xs: List[float], q: float) -> Optional[float]:
    if not xs:
        return None
    xs = sorted(xs)
    return xs[min(len(xs) - 1, int(q * len(xs)))]


async def run_load(client: httpx.AsyncClient, num_prompts: int = 32, concurrency: int = 8, prompt_len: int = 64,
                   max_tokens: int = 32, vocab: int = 1000, seed: int = 0, model: str = "") -> dict:
    rng = random.Random(seed)
    prompts = [[rng.randrange(vocab) for _ in range(prompt_len)] for _ in range(num_prompts)]
    sem = asyncio.Semaphore(concurrency)
    ttft, itl, lat, out_tokens, errors = [], [], [], [0], [0]

    async def one(ids):
        async with sem:
            t0 = time.perf_counter()
            last = None
            try:
                async with client.stream("POST", "/v1/completions", json={
                        "model": model, "prompt": ids, "max_tokens": max_tokens, "temperature": 0, "ignore_eos": True,
                        "stream": True}, timeout=None) as r:
                    if r.status_code != 200:
                        errors[0] += 1
                        return
                    async for line in r.aiter_lines():
                        if not line.startswith("data: {"):
                            continue
                        n = len(json.loads(line[6:])["choices"][0].get("token_ids") or [])
                        if not n:
                            continue
                        now = time.perf_counter()
                        if last is None:
                            ttft.append(now - t0)
                        else:
                            itl.append((now - last) / n)
                        last = now
                        out_tokens[0] += n
                lat.append(time.perf_counter() - t0)
            except Exception:
                errors[0] += 1
    t_start = time.perf_counter()
    await asyncio.gather(*[one(p) for p in prompts])
    wall = time.perf_counter() - t_start
    ms = lambda v: None if v is None else round(v * 1e3, 2)
    return {"requests": num_prompts, "errors": errors[0], "concurrency": concurrency, "wall_s": round(wall, 3),
            "request_per_s": round((num_prompts - errors[0]) / wall, 2), "output_tok_per_s": round(out_tokens[0] / wall, 1),
            "input_tok_per_s": round((num_prompts - errors[0]) * prompt_len / wall, 1),
            "ttft_ms": {"p50": ms(_pct(ttft, 0.5)), "p99": ms(_pct(ttft, 0.99))},
            "itl_ms": {"p50": ms(_pct(itl, 0.5)), "p99": ms(_pct(itl, 0.99)), "mean": ms(statistics.fmean(itl)) if itl else None},
            "e2e_ms": {"p50": ms(_pct(lat, 0.5)), "p99": ms(_pct(lat, 0.99))}}


def main(url: str, **kw) -> dict:
    async def go():
        async with httpx.AsyncClient(base_url=url) as c:
            return await run_load(c, **kw)
    return asyncio.run(go())
