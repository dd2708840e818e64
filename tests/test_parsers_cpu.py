"""Tool-call dialects and reasoning styles: each format's markup becomes OpenAI-shaped calls / a
(reasoning, answer) split; malformed markup stays in the text."""
import json

import pytest

from fllm_b200.server.parsers import REASONING_PARSERS, TOOL_PARSERS, ReasoningStream, parse_tool_calls, split_reasoning

BAR, LOW = "｜", "▁"
CASES = {
    "hermes": ('ok <tool_call>{"name": "get_w", "arguments": {"city": "Paris"}}</tool_call>', "ok"),
    "llama3": ('<|python_tag|>{"name": "get_w", "parameters": {"city": "Paris"}}', ""),
    "mistral": ('[TOOL_CALLS] [{"name": "get_w", "arguments": {"city": "Paris"}}]', ""),
    "qwen3_coder": ("ok <tool_call>\n<function=get_w>\n<parameter=city>\nParis\n</parameter>\n</function>\n</tool_call>", "ok"),
    "glm": ("<tool_call>get_w\n<arg_key>city</arg_key>\n<arg_value>Paris</arg_value>\n</tool_call>", ""),
    "deepseek": (f"hi<{BAR}tool{LOW}calls{LOW}begin{BAR}><{BAR}tool{LOW}call{LOW}begin{BAR}>function<{BAR}tool{LOW}sep{BAR}>get_w\n"
                 f"```json\n{{\"city\": \"Paris\"}}\n```<{BAR}tool{LOW}call{LOW}end{BAR}><{BAR}tool{LOW}calls{LOW}end{BAR}>", "hi"),
    "deepseek_v31": (f"<{BAR}tool{LOW}calls{LOW}begin{BAR}><{BAR}tool{LOW}call{LOW}begin{BAR}>get_w<{BAR}tool{LOW}sep{BAR}>"
                     f"{{\"city\": \"Paris\"}}<{BAR}tool{LOW}call{LOW}end{BAR}><{BAR}tool{LOW}calls{LOW}end{BAR}>", ""),
    "kimi": ('x<|tool_calls_section_begin|><|tool_call_begin|>functions.get_w:0<|tool_call_argument_begin|>{"city": "Paris"}'
             "<|tool_call_end|><|tool_calls_section_end|>", "x"),
    "gpt_oss": ('<|channel|>analysis<|message|>hm<|end|><|start|>assistant<|channel|>commentary to=functions.get_w '
                '<|constrain|>json<|message|>{"city": "Paris"}<|call|>', ""),
    "pythonic": ('[get_w(city="Paris")]', ""),
    "llama4_pythonic": ('<|python_start|>[get_w(city="Paris")]<|python_end|>', ""),
    "lfm2": ('<|tool_call_start|>[get_w(city="Paris")]<|tool_call_end|>done', "done"),
    "xlam": ('```json\n[{"name": "get_w", "arguments": {"city": "Paris"}}]\n```', ""),
    "granite3": ('<|tool_call|>[{"name": "get_w", "arguments": {"city": "Paris"}}]', ""),
    "phi4": ('functools[{"name": "get_w", "arguments": {"city": "Paris"}}]', ""),
    "minimax": ('<tool_calls>\n{"name": "get_w", "arguments": {"city": "Paris"}}\n</tool_calls>', ""),
}


@pytest.mark.parametrize("style", sorted(CASES))
def test_each_dialect_yields_the_call(style):
    text, rest_want = CASES[style]
    rest, calls = parse_tool_calls(text, style)
    assert rest == rest_want
    assert len(calls) == 1 and calls[0]["type"] == "function" and calls[0]["id"].startswith("call_")
    assert calls[0]["function"]["name"] == "get_w" and json.loads(calls[0]["function"]["arguments"]) == {"city": "Paris"}


def test_every_registered_dialect_has_a_case_and_plain_text_passes_through():
    assert set(CASES) | {"llama3_json"} == set(TOOL_PARSERS)
    for style in TOOL_PARSERS:
        assert parse_tool_calls("just words, no markup", style) == ("just words, no markup", [])
        for broken in ("<tool_call>{oops", "[f(", "<|tool_call|>[{", "functools[", "<tool_calls>\n{"):
            rest, calls = parse_tool_calls(broken, style)
            assert calls == [] and rest == broken


def test_several_calls_and_typed_parameters():
    rest, calls = parse_tool_calls('[a(x=1, y=[1, 2], z={"k": -2.5}, t=True), b()]', "pythonic")
    assert [c["function"]["name"] for c in calls] == ["a", "b"]
    assert json.loads(calls[0]["function"]["arguments"]) == {"x": 1, "y": [1, 2], "z": {"k": -2.5}, "t": True}
    rest, calls = parse_tool_calls("<tool_call>\n<function=f>\n<parameter=n>\n3\n</parameter>\n<parameter=s>\nabc\n</parameter>\n</function>\n</tool_call>", "qwen3_coder")
    assert json.loads(calls[0]["function"]["arguments"]) == {"n": 3, "s": "abc"}


@pytest.mark.parametrize("style,text,want", [
    ("think", "<think>a</think>\nb", ("a", "b")), ("think_open", "a</think>b", ("a", "b")),
    ("mistral", "[THINK]a[/THINK]b", ("a", "b")), ("seed", "<seed:think>a</seed:think>b", ("a", "b")),
    ("minimax_m3", "<mm:think>a</mm:think>b", ("a", "b")), ("ifm", "<ifm|think>a</ifm|think>b", ("a", "b")),
    ("gemma4", "<|channel>thought a<channel|>b", ("a", "b")),
    ("granite", "Here is my thought process: a Here is my response: b", ("a", " b")),
    ("hunyuan", "<think>a</think><answer>b</answer>", ("a", "b")),
    ("gpt_oss", "<|channel|>analysis<|message|>a<|end|><|start|>assistant<|channel|>final<|message|>b", ("a", "b")),
    ("think", "no tags", (None, "no tags")),
])
def test_reasoning_styles(style, text, want):
    assert style in REASONING_PARSERS
    assert split_reasoning(text, style) == want


@pytest.mark.parametrize("style", ["think", "mistral", "seed", "minimax_m3"])
def test_streaming_split_equals_one_shot(style):
    from fllm_b200.server.parsers import _REASONING_TAGS
    o, c = _REASONING_TAGS[style]
    text = f"{o}step one, step two{c}\n\nThe answer."
    for width in (1, 3, 7):
        rs = ReasoningStream(style)
        r_all, c_all = "", ""
        pieces = [text[i:i + width] for i in range(0, len(text), width)]
        for i, p in enumerate(pieces):
            r, cc = rs.push(p, i == len(pieces) - 1)
            r_all += r
            c_all += cc
        assert (r_all.strip(), c_all) == split_reasoning(text, style)
