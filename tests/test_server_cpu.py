"""HTTP API on a tiny random model (CPU reference ops): OpenAI, Anthropic, Ollama, llama.cpp and
TGI dialects on one app, streaming, stop strings, health / readiness, metrics, panic containment."""
import json
import time

import pytest
import torch
from fastapi.testclient import TestClient

from fllm_b200.config import EngineConfig, preset
from fllm_b200.runtime import LLMEngine
from fllm_b200.server.app import create_app
from fllm_b200.tokenizer import ByteTokenizer, render_chat


@pytest.fixture(scope="module")
def client():
    cfg = preset("qwen3-tiny")
    cfg.vocab_size = 512
    eng = LLMEngine(cfg, EngineConfig(max_num_seqs=8, max_num_batched_tokens=64, max_model_len=512, num_kv_blocks=128),
                    device="cpu", eos_token_id=257)
    app = create_app(eng, ByteTokenizer(512), "tiny")
    with TestClient(app) as c:
        yield c


def test_health_ready_models_metrics(client):
    assert client.get("/health").json()["status"] == "ok"
    assert client.get("/ready").status_code == 200
    assert client.get("/v1/models").json()["data"][0]["id"] == "tiny"
    assert client.get("/api/tags").json()["models"][0]["name"] == "tiny"
    assert "version" in client.get("/version").json()


def test_completions_greedy_is_deterministic(client):
    body = {"model": "tiny", "prompt": "hello world", "max_tokens": 8, "temperature": 0}
    a = client.post("/v1/completions", json=body).json()
    b = client.post("/v1/completions", json=body).json()
    assert a["choices"][0]["token_ids"] == b["choices"][0]["token_ids"]
    assert a["usage"]["completion_tokens"] == len(a["choices"][0]["token_ids"]) <= 8
    assert a["choices"][0]["finish_reason"] in ("length", "stop")
    ids = client.post("/v1/completions", json={"prompt": [1, 2, 3, 4], "max_tokens": 3, "temperature": 0}).json()
    assert len(ids["choices"][0]["token_ids"]) <= 3


def test_chat_stream_matches_non_stream(client):
    body = {"messages": [{"role": "user", "content": "hi"}], "max_tokens": 6, "temperature": 0}
    full = client.post("/v1/chat/completions", json=body).json()["choices"][0]["message"]["content"]
    with client.stream("POST", "/v1/chat/completions", json=dict(body, stream=True)) as r:
        chunks = [json.loads(l[6:]) for l in r.iter_lines() if l.startswith("data: {")]
    text = "".join(c["choices"][0]["delta"].get("content", "") for c in chunks)
    assert text == full
    assert chunks[-1]["choices"][0]["finish_reason"] is not None


def test_anthropic_and_ollama_and_llamacpp_and_tgi(client):
    m = client.post("/v1/messages", json={"max_tokens": 5, "messages": [{"role": "user", "content": "yo"}], "temperature": 0}).json()
    assert m["type"] == "message" and m["content"][0]["type"] == "text" and m["usage"]["output_tokens"] <= 5
    assert client.post("/v1/messages", json={"messages": []}).status_code == 400
    n = client.post("/v1/messages/count_tokens", json={"messages": [{"role": "user", "content": "yo"}]}).json()
    assert n["input_tokens"] > 2
    o = client.post("/api/generate", json={"prompt": "abc", "stream": False, "options": {"num_predict": 4, "temperature": 0}}).json()
    assert o["done"] and o["eval_count"] <= 4
    lines = client.post("/api/chat", json={"messages": [{"role": "user", "content": "x"}], "options": {"num_predict": 3}}).text.strip().split("\n")
    assert json.loads(lines[-1])["done"] is True
    l = client.post("/completion", json={"prompt": "abc", "n_predict": 4, "temperature": 0}).json()
    assert l["tokens_predicted"] <= 4
    t = client.post("/generate", json={"inputs": "abc", "parameters": {"max_new_tokens": 3}}).json()
    assert "generated_text" in t
    s = client.post("/generate", json={"text": "abc", "sampling_params": {"max_new_tokens": 3}}).json()
    assert s["meta_info"]["completion_tokens"] <= 3
    tok = client.post("/tokenize", json={"content": "hi"}).json()["tokens"]
    assert client.post("/detokenize", json={"tokens": tok}).json()["content"] == "hi"


def test_stop_string_and_validation(client):
    body = {"prompt": "hello", "max_tokens": 24, "temperature": 0}
    full = client.post("/v1/completions", json=body).json()["choices"][0]["text"]
    if len(full) >= 4:
        stop = full[2:4]
        cut = client.post("/v1/completions", json=dict(body, stop=[stop])).json()["choices"][0]
        assert cut["text"] == full[: full.index(stop)] and cut["finish_reason"] == "stop"
    assert client.post("/v1/completions", json={"prompt": "x", "temperature": -1}).status_code == 400
    assert client.post("/v1/chat/completions", json={"messages": []}).status_code == 400


def test_metrics_and_admin(client):
    client.post("/v1/completions", json={"prompt": "count me", "max_tokens": 2})
    txt = client.get("/metrics").text
    assert "fllm_generation_tokens_total" in txt and "vllm:generation_tokens_total" in txt
    assert "fllm_time_to_first_token_seconds_bucket" in txt
    assert "model" in client.get("/admin/config").json()
    assert "prefix_hits" in client.get("/admin/prefix-cache").json()


def test_step_failure_is_contained(client):
    w = client.app.state.worker
    w.inject_failure = 1
    r = client.post("/v1/completions", json={"prompt": "boom", "max_tokens": 4})
    assert r.status_code == 500 and "internal error" in r.text
    ok = client.post("/v1/completions", json={"prompt": "fine", "max_tokens": 2})
    assert ok.status_code == 200
    assert "fllm_worker_panics_total" in client.get("/metrics").text


def test_drain_makes_server_unready(client):
    client.post("/admin/drain", json={"enable": True})
    assert client.get("/ready").status_code == 503
    assert client.post("/v1/completions", json={"prompt": "x", "max_tokens": 1}).status_code == 503
    client.post("/admin/drain", json={"enable": False})
    assert client.get("/ready").status_code == 200


def test_chat_template_rendering():
    s = render_chat(None, [{"role": "system", "content": "s"}, {"role": "user", "content": [{"type": "text", "text": "u"}]}])
    assert s == "<|im_start|>system\ns<|im_end|>\n<|im_start|>user\nu<|im_end|>\n<|im_start|>assistant\n"
    t = render_chat("{{ messages | tojson }}", [{"role": "user", "content": "é"}])
    assert json.loads(t)[0]["content"] == "é"
