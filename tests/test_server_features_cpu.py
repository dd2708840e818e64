"""Structured output, output parsers and the response cache (CPU)."""
import asyncio
import json

import numpy as np
import pytest

from fllm_b200.runtime.grammar import GuidedJson, TokenTrie, json_complete, json_feed, json_start
from fllm_b200.server.cache import ResponseCache, request_key
from fllm_b200.server.parsers import ReasoningStream, parse_tool_calls, split_reasoning


# ------------------------------------------------------------------ JSON recogniser
@pytest.mark.parametrize("doc", ['{}', '{"a": 1}', ' {"a":[1,2.5e-3,true,null,"x\\n\\u00e9"],"b":{"c":[]}} ',
                                 '{"k":"v","n":-0.5}', '{"a":[ ]}'])
def test_valid_json_objects_are_accepted(doc):
    st = json_feed(json_start(True), doc)
    assert st is not None and json_complete(st)
    json.loads(doc)


@pytest.mark.parametrize("doc", ['[1]', '{"a" 1}', '{"a":01}', '{,}', '{"a":tru }', '{"a":"\\x"}', '{"a":1}}', '{"a":1,}'])
def test_invalid_prefixes_are_rejected(doc):
    assert json_feed(json_start(True), doc) is None


def test_top_level_values_and_numbers_end_implicitly():
    st = json_feed(json_start(False), "12.5")
    assert st is not None and json_complete(st)
    assert json_feed(json_start(False), "[1, 2") is not None and not json_complete(json_feed(json_start(False), "[1, 2"))


class _Tok:
    """Tiny vocabulary with multi-character pieces."""
    pieces = ['{', '}', '"', 'a', 'b', '":', ' ', '1', '23', ',', '{"', 'tr', 'ue', '[', ']', '</s>', 'x}', '":1}']
    vocab_size = len(pieces)
    eos_token_id = 15

    def decode(self, ids):
        return "".join(self.pieces[i] for i in ids)


def test_guided_json_masks_follow_the_grammar():
    tok = _Tok()
    trie = TokenTrie.from_tokenizer(tok)
    g = GuidedJson(trie, tok, [tok.eos_token_id])

    def allowed():
        m = g.mask_words(tok.vocab_size)
        return {tok.pieces[i] for i in range(tok.vocab_size) if (int(m[i >> 5]) >> (i & 31)) & 1}
    assert allowed() == {'{', ' ', '{"'}                    # an object must start
    g.advance(10)                                           # {"
    assert allowed() >= {'a', 'b', '"', '":', ' ', '1', '23', ',', '{', '}', 'tr', 'ue', '[', ']', 'x}', '":1}'} - {'</s>'}
    assert '</s>' not in allowed()
    g.advance(3)                                            # a
    g.advance(17)                                           # ":1}
    assert g.complete and allowed() == {' ', '</s>'}
    # random walks under the mask always produce parseable JSON once complete
    rng = np.random.default_rng(0)
    for _ in range(50):
        g = GuidedJson(trie, tok, [tok.eos_token_id])
        out = []
        for _ in range(40):
            m = g.mask_words(tok.vocab_size)
            ids = [i for i in range(tok.vocab_size) if (int(m[i >> 5]) >> (i & 31)) & 1]
            assert ids, "the grammar must never dead-end"
            t = tok.eos_token_id if (g.complete and rng.random() < 0.7) else int(rng.choice(ids))
            if t == tok.eos_token_id:
                break
            out.append(t)
            g.advance(t)
        if g.complete:
            assert isinstance(json.loads(tok.decode(out)), dict)


# ------------------------------------------------------------------ parsers
def test_split_reasoning_and_stream_agree():
    text = "<think>\nfirst, add.\n</think>\n\nThe answer is 4."
    r, a = split_reasoning(text)
    assert r == "first, add." and a == "The answer is 4."
    assert split_reasoning("plain answer") == (None, "plain answer")
    assert split_reasoning("thinking only</think>done") == (None, "thinking only</think>done")
    assert split_reasoning("thinking only</think>done", "think_open") == ("thinking only", "done")
    assert split_reasoning("<think>a</think>b", "think_open") == ("a", "b")
    for cut in (1, 3, 7, 11):
        rs = ReasoningStream()
        pieces = [text[i:i + cut] for i in range(0, len(text), cut)]
        rr, cc = "", ""
        for i, p in enumerate(pieces):
            x, y = rs.push(p, i == len(pieces) - 1)
            rr += x
            cc += y
        assert rr.strip() == "first, add." and cc == "The answer is 4."


def test_tool_call_styles():
    h = 'Sure.\n<tool_call>\n{"name": "get_weather", "arguments": {"city": "Paris"}}\n</tool_call>'
    rest, calls = parse_tool_calls(h, "hermes")
    assert rest == "Sure." and calls[0]["function"]["name"] == "get_weather"
    assert json.loads(calls[0]["function"]["arguments"]) == {"city": "Paris"}
    rest, calls = parse_tool_calls('{"name": "f", "parameters": {"x": 1}}; {"name": "g", "parameters": {}}', "llama3_json")
    assert rest == "" and [c["function"]["name"] for c in calls] == ["f", "g"]
    rest, calls = parse_tool_calls('ok [TOOL_CALLS] [{"name": "f", "arguments": {"x": 2}}]', "mistral")
    assert rest == "ok" and json.loads(calls[0]["function"]["arguments"]) == {"x": 2}
    # malformed markup stays text
    assert parse_tool_calls("<tool_call>{not json}</tool_call>", "hermes") == ("<tool_call>{not json}</tool_call>", [])
    assert parse_tool_calls("just text", "llama3_json") == ("just text", [])


# ------------------------------------------------------------------ response cache
def test_response_cache_keys_ttl_lru_and_coalescing():
    from fllm_b200.runtime import SamplingParams
    greedy, sampled = SamplingParams(temperature=0.0), SamplingParams(temperature=0.8)
    assert request_key("m", [1, 2], sampled) is None
    assert request_key("m", [1, 2], SamplingParams(temperature=0.8, seed=3)) is not None
    k1, k2 = request_key("m", [1, 2], greedy), request_key("m", [1, 3], greedy)
    assert k1 != k2 and k1 == request_key("m", [1, 2], SamplingParams(temperature=0.0))
    assert k1 != request_key("m", [1, 2], SamplingParams(temperature=0.0, cache_salt="tenant-b"))
    now = [0.0]
    c = ResponseCache(max_entries=2, ttl_s=10.0, clock=lambda: now[0])
    c.put("a", 1); c.put("b", 2); c.put("c", 3)
    assert c.get("a") is None and c.get("b") == 2 and c.get("c") == 3
    now[0] = 11.0
    assert c.get("b") is None

    async def scenario():
        cache, runs = ResponseCache(), []

        async def compute():
            runs.append(1)
            await asyncio.sleep(0.01)
            return "result"
        got = await asyncio.gather(*[cache.get_or_compute("k", compute) for _ in range(5)])
        assert got == ["result"] * 5 and len(runs) == 1 and cache.coalesced == 4
        assert await cache.get_or_compute("k", compute) == "result" and len(runs) == 1 and cache.hits == 1
        assert await cache.get_or_compute(None, compute) == "result" and len(runs) == 2
    asyncio.run(scenario())


# ------------------------------------------------------------------ through the HTTP API
@pytest.fixture(scope="module")
def client():
    from fastapi.testclient import TestClient
    from fllm_b200.config import EngineConfig, preset
    from fllm_b200.runtime import LLMEngine
    from fllm_b200.server.app import create_app
    from fllm_b200.tokenizer import ByteTokenizer
    cfg = preset("qwen3-tiny")
    cfg.vocab_size = 512
    eng = LLMEngine(cfg, EngineConfig(max_num_seqs=8, max_num_batched_tokens=64, max_model_len=512, num_kv_blocks=128),
                    device="cpu", eos_token_id=257)
    app = create_app(eng, ByteTokenizer(512), "tiny", tool_parser="hermes", reasoning_parser="think")
    with TestClient(app) as c:
        yield c


def test_json_mode_output_is_always_a_json_prefix(client):
    for temp, seed in ((0.0, None), (1.0, 7), (1.5, 11)):
        body = {"messages": [{"role": "user", "content": "give me json"}], "max_tokens": 24, "temperature": temp,
                "response_format": {"type": "json_object"}}
        if seed is not None:
            body["seed"] = seed
        r = client.post("/v1/chat/completions", json=body).json()
        text = r["choices"][0]["message"]["content"] or ""
        st = json_feed(json_start(True), text)
        assert st is not None, text                       # a random model cannot leave the grammar
        if r["choices"][0]["finish_reason"] == "stop":
            assert isinstance(json.loads(text), dict)
    o = client.post("/api/generate", json={"prompt": "x", "format": "json", "stream": False,
                                           "options": {"num_predict": 12, "temperature": 0}}).json()
    assert json_feed(json_start(True), o["response"]) is not None


def test_banned_words_given_as_text_and_rare_samplers_through_http(client):
    """`bad_words` strings are tokenised by the server (byte tokenizer: one token per byte) and never show
    up in the text; typical_p / DRY / mirostat fields are accepted on the OpenAI and Ollama routes."""
    body = {"prompt": "ban test", "max_tokens": 12, "temperature": 0}
    base = client.post("/v1/completions", json=body).json()["choices"][0]
    first = base["token_ids"][0]
    if first < 256:
        word = bytes([first]).decode("latin-1")
        got = client.post("/v1/completions", json={**body, "bad_words": [word]}).json()["choices"][0]
        assert first not in got["token_ids"]
    r = client.post("/v1/completions", json={**body, "temperature": 1.0, "seed": 3, "typical_p": 0.9, "dry_multiplier": 0.8,
                                             "dry_sequence_breakers": ["\n"], "mirostat": 2, "mirostat_tau": 3.0})
    assert r.status_code == 200 and len(r.json()["choices"][0]["token_ids"]) >= 1
    o = client.post("/api/generate", json={"prompt": "x", "stream": False,
                                           "options": {"num_predict": 6, "temperature": 0.8, "seed": 1, "typical_p": 0.5, "mirostat": 2}})
    assert o.status_code == 200
    bad = client.post("/v1/completions", json={**body, "typical_p": 0.0})
    assert bad.status_code in (400, 422)


def test_identical_greedy_requests_hit_the_response_cache(client):
    before = client.get("/admin/cache").json()["responses"]
    body = {"prompt": "cache me", "max_tokens": 6, "temperature": 0}
    a = client.post("/v1/completions", json=body).json()
    b = client.post("/v1/completions", json=body).json()
    after = client.get("/admin/cache").json()["responses"]
    assert a["choices"][0]["token_ids"] == b["choices"][0]["token_ids"]
    assert after["hits"] == before["hits"] + 1 and after["entries"] >= 1
    assert client.post("/admin/cache").json()["dropped_responses"] >= 1


def test_embeddings_routes_return_normalised_last_token_states(client):
    r = client.post("/v1/embeddings", json={"input": ["hello", "hello", "other text"]}).json()
    vecs = [d["embedding"] for d in r["data"]]
    assert len(vecs) == 3 and len(vecs[0]) == 64 or len(vecs[0]) > 0
    assert abs(sum(v * v for v in vecs[0]) - 1.0) < 1e-3
    assert max(abs(a - b) for a, b in zip(vecs[0], vecs[1])) < 1e-5       # same text, same vector
    assert max(abs(a - b) for a, b in zip(vecs[0], vecs[2])) > 1e-3
    assert r["usage"]["prompt_tokens"] > 0
    o = client.post("/api/embed", json={"input": "hello"}).json()
    assert max(abs(a - b) for a, b in zip(o["embeddings"][0], vecs[0])) < 1e-5
    assert len(client.post("/api/embeddings", json={"prompt": "hello"}).json()["embedding"]) == len(vecs[0])


def test_request_spans_reach_an_otlp_collector_and_failures_stay_out_of_the_serving_path():
    import http.server
    import threading
    from fastapi.testclient import TestClient
    from fllm_b200.config import EngineConfig, preset
    from fllm_b200.runtime import LLMEngine
    from fllm_b200.server.app import create_app
    from fllm_b200.tokenizer import ByteTokenizer
    from fllm_b200.utils.telemetry import SpanExporter
    got = []

    class Collector(http.server.BaseHTTPRequestHandler):
        def do_POST(self):
            got.append((self.path, json.loads(self.rfile.read(int(self.headers["Content-Length"])))))
            self.send_response(200)
            self.end_headers()
            self.wfile.write(b"{}")

        def log_message(self, *a):
            pass
    srv = http.server.HTTPServer(("127.0.0.1", 0), Collector)
    threading.Thread(target=srv.serve_forever, daemon=True).start()
    cfg = preset("qwen3-tiny")
    cfg.vocab_size = 512
    eng = LLMEngine(cfg, EngineConfig(max_num_seqs=4, max_num_batched_tokens=64, max_model_len=256, num_kv_blocks=64),
                    device="cpu", eos_token_id=257)
    app = create_app(eng, ByteTokenizer(512), "tiny", otlp_endpoint=f"http://127.0.0.1:{srv.server_port}")
    with TestClient(app) as c:
        for i in range(3):
            assert c.post("/v1/completions", json={"prompt": f"span {i}", "max_tokens": 3, "temperature": 0}).status_code == 200
        assert c.get("/admin/telemetry").json()["enabled"] is True
    srv.shutdown()                                   # the app's shutdown flushed the exporter before this
    spans = [s for path, body in got for rs in body["resourceSpans"] for ss in rs["scopeSpans"] for s in ss["spans"]]
    assert got and got[0][0] == "/v1/traces" and len(spans) == 3
    s0 = spans[0]
    assert s0["name"] == "llm.request" and len(s0["traceId"]) == 32 and len(s0["spanId"]) == 16
    assert int(s0["endTimeUnixNano"]) >= int(s0["startTimeUnixNano"])
    keys = {a["key"] for a in s0["attributes"]}
    assert {"llm.prompt_tokens", "llm.completion_tokens", "llm.finish_reason"} <= keys
    assert any(e["name"] == "first_token" for e in s0["events"])
    # a dead collector: spans are dropped and counted, nothing raises
    ex = SpanExporter("http://127.0.0.1:9", batch=2, period_s=0.05)
    for _ in range(3):
        ex.end_span(ex.start_span("x"))
    ex.shutdown()
    assert ex.exported == 0 and ex.dropped == 3 and ex.failed_posts >= 1
    off = SpanExporter("")
    off.end_span(off.start_span("y"))
    assert not off.enabled and off.q.qsize() == 0


def test_operator_profiler_counts_calls_by_operator_and_size():
    import torch
    from fllm_b200.ops.reference import RefOps
    from fllm_b200.utils.telemetry import OpProfiler
    p = OpProfiler(RefOps())
    w = torch.randn(8, 16).to(torch.bfloat16)
    for rows in (4, 4, 200):
        p.linear(torch.randn(rows, 16).to(torch.bfloat16), w)
    table = p.table()
    assert "linear" in table and "<=16" in table and ">128" in table
    assert [l for l in table.splitlines() if l.startswith("linear") and "<=16" in l][0].split()[2] == "2"


def test_logprobs_and_alternatives_on_both_openai_routes(client):
    """Greedy decoding: the chosen token is the first alternative, its log-probability equals that alternative's,
    alternatives are sorted, and probabilities are <= 1. The completions route takes `logprobs: N`."""
    import math
    r = client.post("/v1/chat/completions", json={"messages": [{"role": "user", "content": "hi"}], "max_tokens": 5,
                                                  "temperature": 0, "logprobs": True, "top_logprobs": 3}).json()
    content = r["choices"][0]["logprobs"]["content"]
    assert 1 <= len(content) <= 5
    for ent in content:
        alts = ent["top_logprobs"]
        assert len(alts) == 3 and alts[0]["token"] == ent["token"]
        assert abs(alts[0]["logprob"] - ent["logprob"]) < 1e-3
        assert alts[0]["logprob"] >= alts[1]["logprob"] >= alts[2]["logprob"]
        assert ent["logprob"] <= 1e-6 and sum(math.exp(a["logprob"]) for a in alts) <= 1.0 + 1e-4
        assert isinstance(ent["bytes"], list)
    c = client.post("/v1/completions", json={"prompt": "abc", "max_tokens": 4, "temperature": 0, "logprobs": 2}).json()
    lp = c["choices"][0]["logprobs"]
    n = len(c["choices"][0]["token_ids"])
    assert len(lp["tokens"]) == len(lp["token_logprobs"]) == len(lp["top_logprobs"]) == len(lp["text_offset"]) == n
    assert all(len(d) <= 2 and len(d) >= 1 for d in lp["top_logprobs"]) and lp["text_offset"][0] == 0
    plain = client.post("/v1/completions", json={"prompt": "abc", "max_tokens": 4, "temperature": 0}).json()
    assert plain["choices"][0]["logprobs"] is None and plain["choices"][0]["token_ids"] == c["choices"][0]["token_ids"]
    assert client.post("/v1/completions", json={"prompt": "abc", "logprobs": True, "top_logprobs": 50}).status_code in (400, 422)


def test_beam_search_over_http_returns_ranked_hypotheses(client):
    body = {"prompt": "beam", "max_tokens": 4, "use_beam_search": True, "n": 3, "length_penalty": 0.0}
    r = client.post("/v1/completions", json=body)
    assert r.status_code == 200
    ch = r.json()["choices"]
    assert len(ch) == 3 and [c["index"] for c in ch] == [0, 1, 2]
    scores = [c["beam_score"] for c in ch]
    assert scores == sorted(scores, reverse=True) and all(s <= 0 for s in scores)
    assert len({tuple(c["token_ids"]) for c in ch}) == 3
    greedy = client.post("/v1/completions", json={"prompt": "beam", "max_tokens": 4, "temperature": 0, "ignore_eos": True}).json()
    one = client.post("/v1/completions", json={**body, "n": 1, "ignore_eos": True}).json()["choices"][0]
    assert one["token_ids"] == greedy["choices"][0]["token_ids"]
    assert client.post("/v1/completions", json={**body, "n": 50}).status_code == 400


def test_kv_tier_admin_route(client):
    r = client.get("/admin/kv-tier").json()
    assert r["enabled"] is False and r["restored_blocks"] == 0


def test_n_choices_are_n_requests_with_consecutive_seeds(client):
    body = {"prompt": "many", "max_tokens": 6, "temperature": 1.0, "seed": 5, "n": 3}
    a = client.post("/v1/completions", json=body).json()
    b = client.post("/v1/completions", json=body).json()
    assert [c["index"] for c in a["choices"]] == [0, 1, 2]
    assert [c["token_ids"] for c in a["choices"]] == [c["token_ids"] for c in b["choices"]]       # seeded: repeats
    assert len({tuple(c["token_ids"]) for c in a["choices"]}) >= 2                               # seeds differ per choice
    single = client.post("/v1/completions", json={**body, "n": 1, "seed": 6}).json()
    assert single["choices"][0]["token_ids"] == a["choices"][1]["token_ids"]
    assert a["usage"]["completion_tokens"] == sum(len(c["token_ids"]) for c in a["choices"])
    chat = client.post("/v1/chat/completions", json={"messages": [{"role": "user", "content": "hi"}], "max_tokens": 4,
                                                     "temperature": 0, "n": 2}).json()
    assert len(chat["choices"]) == 2 and chat["choices"][0]["message"] == chat["choices"][1]["message"]
    assert client.post("/v1/completions", json={**body, "n": 100}).status_code == 400


def test_guided_choice_outputs_exactly_one_of_the_strings(client):
    choices = ["yes", "no", "maybe so"]
    for temp, seed in ((0.0, None), (1.0, 1), (1.0, 2), (1.5, 3)):
        body = {"prompt": "answer:", "max_tokens": 16, "temperature": temp, "guided_choice": choices}
        if seed is not None:
            body["seed"] = seed
        r = client.post("/v1/completions", json=body).json()["choices"][0]
        assert r["text"] in choices and r["finish_reason"] == "stop", r
    assert client.post("/v1/completions", json={"prompt": "x", "guided_choice": [""]}).status_code == 400


_SCHEMA = {"type": "object", "properties": {"name": {"type": "string"}, "age": {"type": "integer"}, "ok": {"type": "boolean"},
                                            "kind": {"enum": ["a", "bb", 3]}, "tags": {"type": "array"},
                                            "opt": {"type": ["number", "null"]}},
           "required": ["name", "age", "kind"], "additionalProperties": False}


def _schema_feed(step, text):
    st = step.start()
    for ch in text:
        st = step(st, ch)
        if st is None:
            return None
    return st


def test_json_schema_step_accepts_and_rejects_by_the_schema():
    from fllm_b200.runtime.grammar import JsonSchemaStep
    step = JsonSchemaStep(_SCHEMA)
    good = ['{"name":"x","age":12,"kind":"bb"}', '{"kind":3,"age":-4,"name":"e\\n","ok":true,"tags":[1,{"a":2}],"opt":null}',
            ' { "age" : 7 , "name" : "" , "kind" : "a" , "opt" : 1.5e3 } ', '{"kind":3 ,"age":0,"name":"q"}']
    for g in good:
        st = _schema_feed(step, g)
        assert st is not None and json_complete(st[0]), g
        doc = json.loads(g)
        assert set(_SCHEMA["required"]) <= set(doc) and set(doc) <= set(_SCHEMA["properties"])
    dead = ['{"name":"x","age":12}', '{"name":1', '{"age":1.', '{"age":1e', '{"kind":"c', '{"zzz', '{"name":"x","name"',
            '{"age":12,"kind":"a","name":"q","tags":[],"ok":false,"opt":2,', '{"kind":"b"', '{"kind":33', '{"ok":1', '{}',
            '{"opt":"s', '{"tags":{', '{"na\\u']
    for b in dead:
        assert _schema_feed(step, b) is None, b
    # open schemas take undeclared keys but still type the declared ones and wait for the required ones
    open_step = JsonSchemaStep({"type": "object", "properties": {"n": {"type": "integer"}}, "required": ["n"]})
    assert json_complete(_schema_feed(open_step, '{"extra":[1],"n":5}')[0])
    assert _schema_feed(open_step, '{"extra":1}') is None and _schema_feed(open_step, '{"n":"') is None
    with pytest.raises(ValueError):
        JsonSchemaStep({"type": "array"})


def test_json_schema_response_format_is_enforced_through_the_sampler(client):
    from fllm_b200.runtime.grammar import JsonSchemaStep
    step = JsonSchemaStep(_SCHEMA)
    finished = 0
    for temp, seed in ((0.0, None), (1.0, 3), (1.3, 4), (1.0, 5)):
        body = {"messages": [{"role": "user", "content": "fill the form"}], "max_tokens": 96, "temperature": temp,
                "response_format": {"type": "json_schema", "json_schema": {"name": "form", "schema": _SCHEMA}}}
        if seed is not None:
            body["seed"] = seed
        r = client.post("/v1/chat/completions", json=body).json()["choices"][0]
        text = r["message"]["content"] or ""
        assert _schema_feed(step, text) is not None, text          # never leaves the schema
        if r["finish_reason"] == "stop":
            doc = json.loads(text)
            assert {"name", "age", "kind"} <= set(doc) <= set(_SCHEMA["properties"])
            assert isinstance(doc["name"], str) and isinstance(doc["age"], int) and doc["kind"] in ("a", "bb", 3)
            finished += 1
    o = client.post("/api/generate", json={"prompt": "x", "format": _SCHEMA, "stream": False,
                                           "options": {"num_predict": 24, "temperature": 0}}).json()
    assert _schema_feed(step, o["response"]) is not None


def test_forced_tool_call_grammar(client):
    from fllm_b200.runtime.grammar import GuidedToolCall, TokenTrie
    from fllm_b200.tokenizer import ByteTokenizer
    tok = ByteTokenizer(512)
    g = GuidedToolCall(TokenTrie.from_tokenizer(tok), tok, [tok.eos_token_id], ["get_weather", "get_time"])

    def feed(text):
        st = g.state
        for ch in text:
            st = g.schema_step(st, ch)
            if st is None:
                return None
        return st
    full = '<tool_call>\n{"name": "get_time", "arguments": {"tz": "UTC", "n": [1, 2]}}\n</tool_call>'
    st = feed(full)
    assert st == ("post", len("</tool_call>"))
    for bad in ('hello', '<tool_call>\n{"name": "other', '<tool_call>\n{"arguments": 1', '<tool_call>\n{"name": "get_time"}',
                full + "x", '<tool_call>\n{"name": "get_time", "arguments": {}}<x'):
        assert feed(bad) is None, bad
    calls = parse_tool_calls(full, "hermes")[1]
    assert calls[0]["function"]["name"] == "get_time" and json.loads(calls[0]["function"]["arguments"])["tz"] == "UTC"
    tools = [{"type": "function", "function": {"name": "get_weather", "parameters": {"type": "object"}}},
             {"type": "function", "function": {"name": "get_time", "parameters": {"type": "object"}}}]
    for choice in ("required", {"type": "function", "function": {"name": "get_time"}}):
        r = client.post("/v1/chat/completions", json={"messages": [{"role": "user", "content": "time?"}], "tools": tools,
                                                      "tool_choice": choice, "max_tokens": 120, "temperature": 0})
        assert r.status_code == 200
        ch = r.json()["choices"][0]
        if ch["finish_reason"] == "tool_calls":
            names = [c["function"]["name"] for c in ch["message"]["tool_calls"]]
            assert names and all(n in ("get_weather", "get_time") for n in names)
            if isinstance(choice, dict):
                assert names == ["get_time"]
        else:                                                # ran out of tokens inside the call: still a prefix of the markup
            assert (ch["message"].get("content") or "").startswith("<tool_call>")
