"""Property / fuzz tests of the parsers that read untrusted bytes or text (hypothesis)."""
import json
import os
import struct

import numpy as np
import pytest
from hypothesis import HealthCheck, given, settings
from hypothesis import strategies as st

from fllm_b200.formats.gguf import GgufError, GgufReader
from fllm_b200.formats.safetensors_io import SafetensorsError, SafetensorsFile
from fllm_b200.runtime.grammar import json_complete, json_feed, json_start
from fllm_b200.server.parsers import ReasoningStream, parse_tool_calls, split_reasoning

# derandomised: the same examples on every run, so the suite is reproducible; no example database on disk
FAST = settings(max_examples=150, deadline=None, derandomize=True, database=None,
                suppress_health_check=[HealthCheck.function_scoped_fixture])


@FAST
@given(st.binary(min_size=0, max_size=400))
def test_gguf_reader_rejects_garbage_with_its_own_error(tmp_path, blob):
    path = os.path.join(tmp_path, "x.gguf")
    with open(path, "wb") as f:
        f.write(blob)
    with pytest.raises((GgufError, ValueError)):
        GgufReader(path)


@FAST
@given(st.binary(min_size=0, max_size=200), st.integers(0, 2 ** 20))
def test_gguf_reader_survives_a_valid_magic_with_corrupt_body(tmp_path, tail, count):
    path = os.path.join(tmp_path, "y.gguf")
    with open(path, "wb") as f:
        f.write(b"GGUF" + struct.pack("<IQQ", 3, count, count) + tail)
    try:
        r = GgufReader(path)
        r.close()
    except (GgufError, ValueError):
        pass


@FAST
@given(st.binary(min_size=0, max_size=300))
def test_safetensors_reader_rejects_garbage(tmp_path, blob):
    path = os.path.join(tmp_path, "m.safetensors")
    with open(path, "wb") as f:
        f.write(blob)
    try:
        f = SafetensorsFile(path)
        for k in f.keys():
            f.tensor(k)
        f.close()
    except (SafetensorsError, ValueError):
        pass


_json_values = st.recursive(
    st.none() | st.booleans() | st.integers(-10 ** 9, 10 ** 9) | st.floats(allow_nan=False, allow_infinity=False) | st.text(max_size=8),
    lambda kids: st.lists(kids, max_size=4) | st.dictionaries(st.text(max_size=5), kids, max_size=4), max_leaves=12)


@FAST
@given(st.dictionaries(st.text(max_size=5), _json_values, max_size=4), st.booleans())
def test_every_serialised_json_object_is_accepted_by_the_recogniser(obj, pretty):
    doc = json.dumps(obj, indent=1 if pretty else None, ensure_ascii=False)
    s = json_feed(json_start(True), doc)
    assert s is not None and json_complete(s), doc


@FAST
@given(st.text(max_size=60))
def test_recogniser_agrees_with_json_loads_on_complete_documents(text):
    s = json_feed(json_start(False), text)
    accepted = s is not None and json_complete(s)
    def strict(t):          # python's json accepts the NaN / Infinity literals, the standard (and the recogniser) do not
        def no_constants(name):
            raise ValueError(name)
        return json.loads(t, parse_constant=no_constants)
    try:
        strict(text)
        valid = True
    except (ValueError, RecursionError):
        valid = False
    assert accepted == valid, text


@FAST
@given(st.text(max_size=120), st.sampled_from(["hermes", "llama3_json", "mistral"]))
def test_tool_parsers_never_raise_and_keep_text_when_nothing_parses(text, style):
    rest, calls = parse_tool_calls(text, style)
    assert isinstance(rest, str) and isinstance(calls, list)
    if not calls:
        assert rest == text
    for c in calls:
        json.loads(c["function"]["arguments"])


@FAST
@given(st.text(alphabet="<>/think \nab", max_size=80), st.integers(1, 9), st.sampled_from(["think", "think_open"]))
def test_streaming_reasoning_split_equals_the_one_shot_split(text, cut, style):
    r, a = split_reasoning(text, style)
    rs = ReasoningStream(style)
    pieces = [text[i:i + cut] for i in range(0, len(text), cut)] or [""]
    rr, cc = "", ""
    for i, p in enumerate(pieces):
        x, y = rs.push(p, i == len(pieces) - 1)
        rr += x
        cc += y
    assert (rr.strip() or None) == r
    assert cc.strip() == a.strip()


_FORM = {"type": "object",
         "properties": {"name": {"type": "string"}, "age": {"type": "integer"}, "ok": {"type": "boolean"},
                        "kind": {"enum": ["a", "bb", 3, None]}, "tags": {"type": "array"}, "opt": {"type": ["number", "null"]},
                        "meta": {"type": "object"}},
         "required": ["name", "age", "kind"], "additionalProperties": False}
_json_any = st.recursive(st.none() | st.booleans() | st.integers(-1000, 1000) | st.text(max_size=6),
                         lambda ch: st.lists(ch, max_size=3) | st.dictionaries(st.text(max_size=4), ch, max_size=3), max_leaves=6)
_form_docs = st.fixed_dictionaries(
    {"name": st.text(max_size=8), "age": st.integers(-10**6, 10**6), "kind": st.sampled_from(["a", "bb", 3, None])},
    optional={"ok": st.booleans(), "tags": st.lists(_json_any, max_size=3),
              "opt": st.none() | st.integers(-99, 99) | st.floats(-1e3, 1e3, allow_nan=False).map(lambda x: round(x, 3)),
              "meta": st.dictionaries(st.text(max_size=4), _json_any, max_size=3)})


def _form_feed(step, text):
    s = step.start()
    for ch in text:
        s = step(s, ch)
        if s is None:
            return None
    return s


@FAST
@given(_form_docs, st.sampled_from([(",", ":"), (", ", ": "), (" , ", " : ")]), st.booleans(), st.randoms(use_true_random=False))
def test_schema_step_accepts_every_conforming_document(doc, seps, ascii_only, rnd):
    """Documents built from the schema, in any key order and spacing, are accepted and complete."""
    from fllm_b200.runtime.grammar import JsonSchemaStep
    keys = list(doc)
    rnd.shuffle(keys)
    text = json.dumps({k: doc[k] for k in keys}, separators=seps, ensure_ascii=ascii_only)
    s = _form_feed(JsonSchemaStep(_FORM), text)
    assert s is not None and json_complete(s[0]), text


@FAST
@given(_form_docs, st.sampled_from(["drop_required", "wrong_type", "extra_key", "bad_enum", "dup_key"]))
def test_schema_step_never_completes_a_violating_document(doc, how):
    from fllm_b200.runtime.grammar import JsonSchemaStep
    d = dict(doc)
    if how == "drop_required":
        del d["age"]
        text = json.dumps(d)
    elif how == "wrong_type":
        d["age"] = "12"
        text = json.dumps(d)
    elif how == "extra_key":
        d["zzz"] = 1
        text = json.dumps(d)
    elif how == "bad_enum":
        d["kind"] = "c"
        text = json.dumps(d)
    else:
        text = json.dumps(d)[:-1] + ', "name": "again"}'
    s = _form_feed(JsonSchemaStep(_FORM), text)
    assert s is None or not json_complete(s[0]), text
