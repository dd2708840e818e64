"""GBNF grammars, regular expressions and nested JSON schemas through one pushdown recogniser, and their use as
sampler constraints through the HTTP API on a tiny random model."""
import json
import re

import pytest

from fllm_b200.runtime.grammar_gbnf import GrammarError, GrammarMachine, machine_from, parse_gbnf, regex_to_gbnf, schema_to_gbnf

ARITH = '''
# sums of numbers and bracketed sums
root ::= expr
expr ::= term (("+" | "-") term)*
term ::= [0-9]+ | "(" expr ")"
'''


def test_gbnf_recogniser():
    m = GrammarMachine(parse_gbnf(ARITH))
    assert all(m.matches(t) for t in ("1", "1+2", "(1+23)-4", "((7))"))
    assert not any(m.matches(t) for t in ("", "1+", "a", "(1", "1 + 2"))
    st = m.start()
    for ch in "(12":
        st = m.step(st, ch)
    assert st is not None and not m.accepting(st) and m.step(st, ")") is not None and m.step(st, "x") is None
    with pytest.raises(GrammarError):
        parse_gbnf("expr ::= [0-9]+")                       # no root
    with pytest.raises(GrammarError):
        parse_gbnf('root ::= missing "x"')
    rep = GrammarMachine(parse_gbnf('root ::= "a"{2,3} [^x]? "\\n"'))
    assert rep.matches("aa\n") and rep.matches("aaab\n") and not rep.matches("a\n") and not rep.matches("aaaaa\n") and not rep.matches("aax\n")


@pytest.mark.parametrize("pattern", [r"\d{3}-[a-c]+(x|yz)?", r"(ab|cd)*e", r"[A-Z][a-z]{1,3}\s\w+", r"-?(0|[1-9]\d*)(\.\d+)?", r"a.c"])
def test_regex_agrees_with_python_re(pattern):
    m = machine_from("regex", pattern)
    for t in ("123-abc", "123-abyz", "12-a", "123-d", "abcde", "e", "abe", "Abc d_1", "Abcde x", "-12.50", "0", "01", "abc", "a\nc", "ac", ""):
        assert m.matches(t) == (re.fullmatch(pattern, t) is not None), (pattern, t)
    assert regex_to_gbnf(pattern).startswith("root ::= ")


SCHEMA = {"type": "object",
          "properties": {"name": {"type": "string", "minLength": 1}, "age": {"type": "integer"},
                         "tags": {"type": "array", "items": {"enum": ["a", "b"]}, "minItems": 1, "maxItems": 2},
                         "addr": {"type": "object", "properties": {"zip": {"type": "string", "pattern": "\\d{5}"}}, "required": ["zip"],
                                  "additionalProperties": False},
                         "kind": {"const": "user"}, "score": {"type": ["number", "null"]}},
          "required": ["name", "addr"], "additionalProperties": False}


def test_nested_json_schema():
    m = machine_from("json_schema", SCHEMA)
    good = ['{"name":"x","addr":{"zip":"12345"}}',
            '{ "name": "x", "age": 3, "tags": ["a", "b"], "addr": {"zip": "00000"}, "kind": "user", "score": null }',
            '{"name":"x","addr":{"zip":"12345"},"score":-1.5e3}']
    bad = ['{"name":"x"}', '{"name":"","addr":{"zip":"12345"}}', '{"name":"x","addr":{"zip":"1234"}}',
           '{"name":"x","age":1.5,"addr":{"zip":"12345"}}', '{"name":"x","addr":{"zip":"12345"},"z":1}',
           '{"name":"x","tags":[],"addr":{"zip":"12345"}}', '{"name":"x","tags":["a","b","a"],"addr":{"zip":"12345"}}',
           '{"name":"x","addr":{"zip":"12345","more":1}}', '{"name":"x","addr":{"zip":"12345"},"kind":"admin"}']
    for t in good:
        json.loads(t)
        assert m.matches(t), t
    for t in bad:
        assert not m.matches(t), t
    rec = {"$defs": {"node": {"type": "object", "properties": {"v": {"type": "integer"},
                                                                 "next": {"anyOf": [{"$ref": "#/$defs/node"}, {"type": "null"}]}},
                              "required": ["v", "next"], "additionalProperties": False}}, "$ref": "#/$defs/node"}
    rm = machine_from("json_schema", rec)
    assert rm.matches('{"v":1,"next":{"v":2,"next":null}}') and not rm.matches('{"v":1,"next":{"v":2}}')
    free = machine_from("json_schema", {"type": "object", "properties": {"a": {"type": "number"}}})
    assert free.matches('{"a":1,"other":[1,{"x":null}]}') and free.matches("{}") and not free.matches('{"a":"s"}')
    assert "root ::=" in schema_to_gbnf(SCHEMA)


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
    with TestClient(create_app(eng, ByteTokenizer(512), "tiny")) as c:
        yield c


def test_constraints_through_the_api(client):
    r = client.post("/v1/completions", json={"prompt": "id: ", "max_tokens": 24, "temperature": 0.9, "seed": 1,
                                             "guided_regex": r"[A-F]{2}-\d{4}"}).json()
    assert re.fullmatch(r"[A-F]{2}-\d{4}", r["choices"][0]["text"]), r["choices"][0]["text"]
    g = client.post("/v1/completions", json={"prompt": "sum: ", "max_tokens": 6, "temperature": 0.9, "seed": 2, "guided_grammar": ARITH}).json()
    text = g["choices"][0]["text"]
    m = GrammarMachine(parse_gbnf(ARITH))
    st = m.start()
    for ch in text:
        st = m.step(st, ch)
        assert st is not None, text                         # every generated prefix stays inside the grammar
    schema = {"type": "object", "properties": {"ok": {"type": "boolean"}, "n": {"type": "array", "items": {"type": "integer"}, "maxItems": 2}},
              "required": ["ok", "n"], "additionalProperties": False}
    j = client.post("/v1/chat/completions", json={"messages": [{"role": "user", "content": "go"}], "max_tokens": 60, "temperature": 0.8,
                                                  "seed": 3, "response_format": {"type": "json_schema", "json_schema": {"name": "x", "schema": schema}}}).json()
    out = j["choices"][0]["message"]["content"]
    sm = machine_from("json_schema", schema)
    st = sm.start()
    for ch in out:
        st = sm.step(st, ch)
        assert st is not None, out                          # never leaves the schema's language
    if j["choices"][0]["finish_reason"] == "stop":          # (a random model may spend the budget on digits)
        doc = json.loads(out)
        assert isinstance(doc["ok"], bool) and isinstance(doc["n"], list) and len(doc["n"]) <= 2 and set(doc) == {"ok", "n"}
    assert client.post("/v1/completions", json={"prompt": "x", "guided_grammar": "nonsense ::="}).status_code == 400
