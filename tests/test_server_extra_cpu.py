"""The wider HTTP surface on a tiny random model (CPU reference ops): Responses, Files, Batches, rerank / score /
pooling / classify, infill, model management stubs, CORS and the rate limit."""
import json
import time

import pytest
from fastapi.testclient import TestClient

from fllm_b200.config import EngineConfig, preset
from fllm_b200.runtime import LLMEngine
from fllm_b200.server.app import create_app
from fllm_b200.server.extra_routes import TokenBucket
from fllm_b200.tokenizer import ByteTokenizer


def _engine():
    cfg = preset("qwen3-tiny")
    cfg.vocab_size = 512
    return LLMEngine(cfg, EngineConfig(max_num_seqs=8, max_num_batched_tokens=64, max_model_len=512, num_kv_blocks=128),
                     device="cpu", eos_token_id=257)


@pytest.fixture(scope="module")
def client():
    app = create_app(_engine(), ByteTokenizer(512), "tiny", cors_origins=["https://a.example"])
    with TestClient(app) as c:
        yield c


def test_responses_api_roundtrip_and_stream(client):
    r = client.post("/v1/responses", json={"input": "hello", "max_output_tokens": 6, "temperature": 0}).json()
    assert r["object"] == "response" and r["status"] == "completed"
    assert r["output"][-1]["content"][0]["type"] == "output_text" and r["usage"]["output_tokens"] <= 6
    assert client.get(f"/v1/responses/{r['id']}").json()["id"] == r["id"]
    # continue the stored conversation
    r2 = client.post("/v1/responses", json={"input": [{"role": "user", "content": [{"type": "input_text", "text": "more"}]}],
                                            "previous_response_id": r["id"], "max_output_tokens": 4, "temperature": 0}).json()
    assert r2["usage"]["input_tokens"] > r["usage"]["input_tokens"]
    assert client.post("/v1/responses", json={"input": "x", "previous_response_id": "resp_nope"}).status_code == 404
    with client.stream("POST", "/v1/responses", json={"input": "hello", "max_output_tokens": 6, "temperature": 0, "stream": True}) as s:
        events = [l[7:] for l in s.iter_lines() if l.startswith("event: ")]
        assert events[0] == "response.created" and events[-1] == "response.completed"
    assert client.delete(f"/v1/responses/{r['id']}").json()["deleted"] is True
    assert client.get(f"/v1/responses/{r['id']}").status_code == 404


def test_files_and_batches(client):
    lines = [{"custom_id": "a", "method": "POST", "url": "/v1/chat/completions",
              "body": {"messages": [{"role": "user", "content": "hi"}], "max_tokens": 4, "temperature": 0}},
             {"custom_id": "b", "method": "POST", "url": "/v1/completions", "body": {"prompt": "abc", "max_tokens": 3, "temperature": 0}},
             {"custom_id": "c", "method": "POST", "url": "/v1/nope", "body": {}}]
    f = client.post("/v1/files", json={"filename": "in.jsonl", "purpose": "batch", "content": "\n".join(json.dumps(l) for l in lines)}).json()
    assert f["object"] == "file" and f["bytes"] > 0
    assert any(x["id"] == f["id"] for x in client.get("/v1/files").json()["data"])
    b = client.post("/v1/batches", json={"input_file_id": f["id"], "endpoint": "/v1/chat/completions"}).json()
    assert b["object"] == "batch" and b["request_counts"]["total"] == 3
    for _ in range(200):
        b = client.get(f"/v1/batches/{b['id']}").json()
        if b["status"] == "completed":
            break
        time.sleep(0.05)
    assert b["status"] == "completed" and b["request_counts"] == {"total": 3, "completed": 2, "failed": 1}
    out = [json.loads(l) for l in client.get(f"/v1/files/{b['output_file_id']}/content").text.splitlines()]
    assert {o["custom_id"] for o in out} == {"a", "b"} and all(o["response"]["status_code"] == 200 for o in out)
    err = [json.loads(l) for l in client.get(f"/v1/files/{b['error_file_id']}/content").text.splitlines()]
    assert err[0]["custom_id"] == "c"
    assert client.post("/v1/batches", json={"input_file_id": "file-none"}).status_code == 404
    assert client.delete(f"/v1/files/{f['id']}").json()["deleted"] is True
    assert client.post(f"/v1/batches/{b['id']}/cancel").json()["status"] == "completed"


def test_scoring_endpoints(client):
    rr = client.post("/v1/rerank", json={"query": "apple", "documents": ["apple", "zebra crossing", "apple pie"], "top_n": 2,
                                         "return_documents": True}).json()
    assert len(rr["results"]) == 2 and rr["results"][0]["relevance_score"] >= rr["results"][1]["relevance_score"]
    assert rr["results"][0]["index"] == 0 and abs(rr["results"][0]["relevance_score"] - 1.0) < 1e-3       # identical text
    assert client.post("/rerank", json={"query": "q", "documents": []}).status_code == 400
    sc = client.post("/v1/score", json={"text_1": "same", "text_2": ["same", "other"]}).json()
    assert abs(sc["data"][0]["score"] - 1.0) < 1e-3 and sc["data"][1]["score"] < 1.0
    pl = client.post("/pooling", json={"input": ["ab", "cd"]}).json()
    assert len(pl["data"]) == 2 and len(pl["data"][0]["data"]) == 512
    cl = client.post("/classify", json={"input": "great movie", "labels": ["good", "bad"]}).json()
    assert cl["data"][0]["label"] in ("good", "bad") and abs(sum(cl["data"][0]["probs"]) - 1.0) < 1e-3
    assert client.post("/classify", json={"input": "x"}).status_code == 400
    assert len(client.post("/embeddings", json={"input": "hey"}).json()["data"][0]["embedding"]) == 512


def test_infill_models_slots_and_management_stubs(client):
    r = client.post("/infill", json={"input_prefix": "def f(", "input_suffix": "):", "n_predict": 4, "temperature": 0}).json()
    assert r["tokens_predicted"] <= 4 and r["stop"] is True
    assert client.get("/v1/models/tiny").json()["id"] == "tiny" and client.get("/v1/models/other").status_code == 404
    assert client.get("/").json()["model"] == "tiny"
    assert client.get("/slots/0").json()["is_processing"] is False and client.get("/slots/99").status_code == 404
    assert client.get("/is_sleeping").json() == {"is_sleeping": False} and client.get("/lora-adapters").json() == []
    assert client.post("/api/pull", json={"model": "tiny"}).json()["status"] == "success"
    assert client.post("/api/pull", json={"model": "llama3"}).status_code == 404
    assert client.post("/api/create", json={}).status_code == 501
    assert client.request("DELETE", "/api/delete", json={"model": "nope"}).status_code == 404


def test_cors_headers(client):
    ok = client.get("/v1/models", headers={"origin": "https://a.example"})
    assert ok.headers["access-control-allow-origin"] == "https://a.example"
    assert "access-control-allow-origin" not in client.get("/v1/models", headers={"origin": "https://evil.example"}).headers
    pre = client.options("/v1/chat/completions", headers={"origin": "https://a.example", "access-control-request-method": "POST"})
    assert pre.status_code == 204


def test_rate_limit_bucket_and_middleware():
    b = TokenBucket(2.0)                     # burst 4
    assert [b.allow("k", now=0.0) for _ in range(5)] == [True, True, True, True, False]
    assert b.allow("k", now=0.6) is True and b.allow("other", now=0.6) is True
    app = create_app(_engine(), ByteTokenizer(512), "tiny", rate_limit_rps=1.0)
    with TestClient(app) as c:
        codes = [c.get("/v1/models").status_code for _ in range(4)]
        assert codes[:2] == [200, 200] and 429 in codes
        assert c.get("/health").status_code == 200          # never limited
