"""Replica router in front of two in-process engine servers (ASGI transports instead of sockets)."""
import json

import httpx
import pytest
from fastapi.testclient import TestClient

from fllm_b200.config import EngineConfig, preset
from fllm_b200.runtime import LLMEngine
from fllm_b200.server.app import create_app
from fllm_b200.server.router import create_router
from fllm_b200.tokenizer import ByteTokenizer


def _backend(seed):
    cfg = preset("qwen3-tiny")
    cfg.vocab_size = 512
    eng = LLMEngine(cfg, EngineConfig(max_num_seqs=4, max_num_batched_tokens=64, max_model_len=256, num_kv_blocks=64),
                    device="cpu", eos_token_id=257, seed=seed)
    return create_app(eng, ByteTokenizer(512), "tiny")


class _Dead(httpx.AsyncBaseTransport):
    async def handle_async_request(self, request):
        raise httpx.ConnectError("replica is down")


@pytest.fixture(scope="module")
def stack():
    apps = {"a": _backend(0), "b": _backend(0)}
    ctxs = [TestClient(a) for a in apps.values()]           # runs the lifespans (engine worker threads)
    for c in ctxs:
        c.__enter__()
    yield apps
    for c in ctxs:
        c.__exit__(None, None, None)


def _router(apps, policy, extra=None):
    clients = {n: httpx.AsyncClient(transport=httpx.ASGITransport(app=a), base_url="http://" + n) for n, a in apps.items()}
    clients.update(extra or {})
    return TestClient(create_router(clients, policy, health_period_s=0.0))


def test_prefix_affinity_is_sticky_and_spreads(stack):
    with _router(stack, "prefix") as c:
        seen = {}
        for i in range(12):
            body = {"prompt": f"conversation {i % 4} " + "x" * 40, "max_tokens": 2, "temperature": 0}
            r = c.post("/v1/completions", json=body)
            assert r.status_code == 200 and r.json()["choices"][0]["token_ids"]
            seen.setdefault(i % 4, set()).add(r.headers["x-fllm-replica"])
        assert all(len(v) == 1 for v in seen.values())        # same prefix -> same replica
        assert len(set().union(*seen.values())) == 2           # and both replicas get work
        assert c.get("/ready").json()["ready"] is True
        assert "fllm_router_served_total" in c.get("/metrics").text


def test_round_robin_and_streaming_passthrough(stack):
    with _router(stack, "round_robin") as c:
        names = [c.post("/v1/completions", json={"prompt": "p", "max_tokens": 1, "temperature": 0}).headers["x-fllm-replica"]
                 for _ in range(4)]
        assert names[0] != names[1] and names[0] == names[2]
        with c.stream("POST", "/v1/chat/completions", json={"messages": [{"role": "user", "content": "hi"}],
                                                             "max_tokens": 4, "temperature": 0, "stream": True}) as r:
            lines = [l for l in r.iter_lines() if l.startswith("data: ")]
        assert lines[-1] == "data: [DONE]" and len(lines) >= 3
        json.loads(lines[0][6:])


def test_a_dead_replica_is_skipped_and_reported(stack):
    dead = {"z-dead": httpx.AsyncClient(transport=_Dead(), base_url="http://dead")}
    with _router({"a": stack["a"]}, "round_robin", dead) as c:
        for _ in range(4):
            r = c.post("/v1/completions", json={"prompt": "p", "max_tokens": 1, "temperature": 0})
            assert r.status_code == 200 and r.headers["x-fllm-replica"] == "a"
        rd = c.get("/ready").json()
        assert rd["ready"] is True and rd["replicas"]["z-dead"] is False
    with _router({}, "round_robin", dead) as c:
        assert c.post("/v1/completions", json={"prompt": "p"}).status_code == 503
        assert c.get("/ready").status_code == 503


def test_disaggregated_prefill_and_decode_servers_agree_with_one_server(stack):
    """Server A processes the prompt and exports the request; server B imports it and decodes."""
    a, b = TestClient(stack["a"]), TestClient(stack["b"])
    body = {"prompt": "disaggregate this prompt please", "max_tokens": 8, "temperature": 0}
    whole = a.post("/v1/completions", json=body).json()["choices"][0]["token_ids"]
    blob = a.post("/admin/disagg/export", json=body)
    assert blob.status_code == 200
    blob = blob.json()
    assert len(blob["output"]) == 1 and blob["kv"]["shape"][2] >= 1
    done = b.post("/admin/disagg/import", json=blob).json()
    assert done["choices"][0]["token_ids"] == whole
    assert done["usage"]["completion_tokens"] == len(whole)
    # a blob for another KV layout is refused
    bad = dict(blob, block_size=32)
    assert b.post("/admin/disagg/import", json=bad).status_code == 400


def test_bench_serve_load_generator_against_an_in_process_server(stack):
    import asyncio
    from fllm_b200.server.bench_serve import run_load

    async def go():
        async with httpx.AsyncClient(transport=httpx.ASGITransport(app=stack["a"]), base_url="http://a") as c:
            return await run_load(c, num_prompts=6, concurrency=3, prompt_len=12, max_tokens=5, vocab=256)
    rep = asyncio.run(go())
    assert rep["errors"] == 0 and rep["requests"] == 6
    assert rep["output_tok_per_s"] > 0 and rep["ttft_ms"]["p50"] is not None and rep["e2e_ms"]["p99"] >= rep["ttft_ms"]["p50"]
