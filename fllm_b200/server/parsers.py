"""Output parsers of the chat API: reasoning blocks and tool calls.

* Reasoning (``--reasoning-parser``): ``think`` splits ``<think> ... </think>`` off the front of the
  answer into ``reasoning_content`` (DeepSeek-R1 / Qwen3 style); ``think_open`` is for chat templates
  that already end with the opening tag, so that the model only writes the closing one.
  ``ReasoningStream`` is the incremental form used while streaming; both forms give the same split.
* Tool calls (``--tool-parser``): ``hermes`` (``<tool_call>{json}</tool_call>``, Qwen / Hermes),
  ``llama3_json`` (the whole answer, or what follows ``<|python_tag|>``, is
  ``{"name": ..., "parameters": {...}}``, several separated by ``;``), ``mistral``
  (``[TOOL_CALLS] [{...}, ...]``). Each returns the remaining text and OpenAI-shaped ``tool_calls``.


Further reasoning styles are tag pairs of other model families (``mistral`` ``[THINK]``, ``seed``
``<seed:think>``, ``minimax_m3`` ``<mm:think>``, ``ifm``, ``gemma4`` channel markers), the prose markers of
``granite``, ``hunyuan`` (``<think>`` then ``<answer>``) and the Harmony channels of ``gpt_oss``
(``analysis`` = reasoning, ``final`` = answer). Further tool dialects: ``qwen3_coder`` and ``glm`` (XML
parameters), ``deepseek`` / ``deepseek_v31`` (fullwidth-bar markers), ``kimi``, ``gpt_oss`` (Harmony
``to=functions.NAME``), ``pythonic`` / ``llama4_pythonic`` / ``lfm2`` (Python call lists), ``xlam``,
``granite3``, ``phi4``, ``minimax`` (JSON lists / lines behind a marker). A parser never raises:
what it cannot decode stays in the text.

The reference's counterparts: rust/engine/src/tool_parsers.rs:1997-2018 (the dialect registry),
rust/engine/src/reasoning.rs:9-21 (the reasoning families).
"""
from __future__ import annotations

import json
import re
import uuid
from typing import List, Optional, Tuple

# style -> (opening tag, closing tag); "think_open" = the template already wrote the opening tag
_REASONING_TAGS = {
    "think": ("<think>", "</think>"), "think_open": ("<think>", "</think>"), "mistral": ("[THINK]", "[/THINK]"),
    "seed": ("<seed:think>", "</seed:think>"), "minimax_m3": ("<mm:think>", "</mm:think>"),
    "ifm": ("<ifm|think>", "</ifm|think>"), "gemma4": ("<|channel>thought", "<channel|>"),
    "granite": ("Here is my thought process:", "Here is my response:"),
}
REASONING_PARSERS = tuple(_REASONING_TAGS) + ("hunyuan", "gpt_oss")
TOOL_PARSERS = ("hermes", "llama3_json", "llama3", "mistral", "qwen3_coder", "glm", "deepseek", "deepseek_v31", "kimi",
                "gpt_oss", "pythonic", "llama4_pythonic", "lfm2", "xlam", "granite3", "phi4", "minimax")


# ------------------------------------------------------------------------------ reasoning
def _split_harmony(text: str) -> Tuple[Optional[str], str]:
    """gpt-oss Harmony: ``<|channel|>analysis<|message|>...<|end|>`` blocks are reasoning, the ``final`` channel is
    the answer; text outside any channel is answer text."""
    reasoning, answer = [], []
    pos = 0
    pat = re.compile(r"<\|channel\|>(\w+)[^<]*<\|message\|>(.*?)(?:<\|end\|>|<\|return\|>|<\|call\|>|(?=<\|start\|>)|$)", re.S)
    for m in pat.finditer(text):
        answer.append(re.sub(r"<\|start\|>\w*", "", text[pos:m.start()]))
        (reasoning if m.group(1) == "analysis" else answer if m.group(1) == "final" else []).append(m.group(2))
        pos = m.end()
    answer.append(re.sub(r"<\|start\|>\w*", "", text[pos:]))
    r = "".join(reasoning).strip()
    return (r or None), "".join(answer).strip()


def split_reasoning(text: str, style: str = "think") -> Tuple[Optional[str], str]:
    """-> (reasoning or None, answer)."""
    if style not in REASONING_PARSERS:
        raise ValueError(f"unknown reasoning parser {style!r}")
    if style == "gpt_oss":
        return _split_harmony(text)
    if style == "hunyuan":
        r, rest = split_reasoning(text, "think")
        m = re.search(r"<answer>(.*?)(?:</answer>|$)", rest, re.S)
        return r, (m.group(1).strip() if m else rest)
    open_t, close_t = _REASONING_TAGS[style]
    body = text
    if body.lstrip().startswith(open_t):
        body = body.lstrip()[len(open_t):]
    elif style != "think_open":
        return None, text
    if close_t not in body:
        return body.strip() or None, ""            # the budget ran out inside the block
    r, _, rest = body.partition(close_t)
    return (r.strip() or None), rest.lstrip("\n")


class ReasoningStream:
    """Feed text pieces, get (reasoning_delta, content_delta) pairs. Holds back a tail that could be
    the beginning of a tag so that tags split across pieces are still recognised."""

    def __init__(self, style: str = "think"):
        if style not in REASONING_PARSERS:
            raise ValueError(f"unknown reasoning parser {style!r}")
        # channel / answer-tag styles are split once the text is complete; while streaming they pass through
        self.open_t, self.close_t = _REASONING_TAGS.get(style, ("\x00never\x00", "\x00never\x00"))
        self.in_reasoning = False
        self.decided = False                        # whether the opening tag question is settled
        self.assume_open = style == "think_open"    # no opening tag seen: the template supplied it
        self.strip_nl = False                       # drop the newlines that follow the closing tag
        self.buf = ""

    def _holdback(self, s: str, tag: str) -> int:
        for k in range(min(len(tag) - 1, len(s)), 0, -1):
            if tag.startswith(s[-k:]):
                return k
        return 0

    def push(self, piece: str, final: bool = False) -> Tuple[str, str]:
        self.buf += piece
        reasoning, content = "", ""
        while True:
            if not self.decided:
                s = self.buf.lstrip()
                if s.startswith(self.open_t):
                    self.buf = s[len(self.open_t):]
                    self.in_reasoning = self.decided = True
                    continue
                if self.open_t.startswith(s) and not final:
                    break                            # could still become the opening tag
                self.decided = True
                self.in_reasoning = self.assume_open
                continue
            if self.in_reasoning:
                i = self.buf.find(self.close_t)
                if i >= 0:
                    reasoning += self.buf[:i]
                    self.buf = self.buf[i + len(self.close_t):]
                    self.in_reasoning = False
                    self.strip_nl = True
                    continue
                keep = 0 if final else self._holdback(self.buf, self.close_t)
                reasoning += self.buf[: len(self.buf) - keep]
                self.buf = self.buf[len(self.buf) - keep:]
                break
            if self.strip_nl:
                self.buf = self.buf.lstrip("\n")
                if self.buf:
                    self.strip_nl = False
            content += self.buf
            self.buf = ""
            break
        return reasoning, content


# ------------------------------------------------------------------------------ tool calls
def _call(name: str, arguments) -> dict:
    if not isinstance(arguments, str):
        arguments = json.dumps(arguments if arguments is not None else {})
    return {"id": "call_" + uuid.uuid4().hex[:24], "type": "function",
            "function": {"name": name, "arguments": arguments}}


def _from_obj(o) -> Optional[dict]:
    if isinstance(o, dict) and isinstance(o.get("name"), str):
        return _call(o["name"], o.get("arguments", o.get("parameters", {})))
    return None


def parse_tool_calls(text: str, style: str) -> Tuple[str, List[dict]]:
    """-> (text without the call markup, tool_calls). Malformed calls stay in the text."""
    calls: List[dict] = []
    if style == "hermes":
        def take(m):
            try:
                c = _from_obj(json.loads(m.group(1)))
            except json.JSONDecodeError:
                c = None
            if c is None:
                return m.group(0)
            calls.append(c)
            return ""
        rest = re.sub(r"<tool_call>\s*(.*?)\s*</tool_call>", take, text, flags=re.S)
        return rest.strip() if calls else text, calls
    if style == "llama3_json":
        body = text.split("<|python_tag|>", 1)[1] if "<|python_tag|>" in text else text
        parts = [p for p in (s.strip() for s in body.split(";")) if p]
        for p in parts:
            try:
                c = _from_obj(json.loads(p))
            except json.JSONDecodeError:
                c = None
            if c is None:
                return text, []
            calls.append(c)
        return ("", calls) if calls else (text, [])
    if style == "mistral":
        tag = "[TOOL_CALLS]"
        if tag not in text:
            return text, []
        head, _, tail = text.partition(tag)
        try:
            arr = json.loads(tail.strip())
        except json.JSONDecodeError:
            return text, []
        for o in arr if isinstance(arr, list) else [arr]:
            c = _from_obj(o)
            if c is None:
                return text, []
            calls.append(c)
        return head.strip(), calls
    if style == "llama3":
        return parse_tool_calls(text, "llama3_json")
    if style in _XML_STYLES or style in _MARKER_JSON or style in ("pythonic", "llama4_pythonic", "lfm2", "xlam", "gpt_oss",
                                                                    "deepseek", "deepseek_v31", "kimi"):
        try:
            return _parse_more(text, style)
        except Exception:                          # a parser never fails a request
            return text, []
    raise ValueError(f"unknown tool parser {style!r}")


_XML_STYLES = ("qwen3_coder", "glm")
# style -> (opening marker, optional closing marker): what follows is a JSON list (or JSON objects, one per line)
_MARKER_JSON = {"granite3": ("<|tool_call|>", None), "phi4": ("functools", None), "minimax": ("<tool_calls>", "</tool_calls>")}


def _json_or_text(v: str):
    v = v.strip()
    try:
        return json.loads(v)
    except (json.JSONDecodeError, ValueError):
        return v


def _py_value(node):
    import ast
    if isinstance(node, ast.Constant):
        return node.value
    if isinstance(node, (ast.List, ast.Tuple)):
        return [_py_value(e) for e in node.elts]
    if isinstance(node, ast.Dict):
        return {_py_value(k): _py_value(v) for k, v in zip(node.keys, node.values)}
    if isinstance(node, ast.UnaryOp) and isinstance(node.op, ast.USub):
        return -_py_value(node.operand)
    if isinstance(node, ast.Name) and node.id in ("true", "false", "null", "none"):
        return {"true": True, "false": False}.get(node.id)
    raise ValueError("unsupported literal")


def _pythonic_calls(src: str) -> List[dict]:
    """``[f(a=1, b="x"), g()]`` -> calls; raises on anything that is not a list of keyword-argument calls."""
    import ast
    tree = ast.parse(src.strip(), mode="eval").body
    items = tree.elts if isinstance(tree, (ast.List, ast.Tuple)) else [tree]
    out = []
    for c in items:
        if not isinstance(c, ast.Call) or c.args:
            raise ValueError("not a keyword-argument call")
        name = ast.unparse(c.func)
        out.append(_call(name, {k.arg: _py_value(k.value) for k in c.keywords}))
    return out


def _parse_more(text: str, style: str) -> Tuple[str, List[dict]]:
    calls: List[dict] = []
    if style == "qwen3_coder":
        def take(m):
            fm = re.search(r"<function=([^>\n]+)>(.*?)</function>", m.group(1), re.S)
            if not fm:
                return m.group(0)
            args = {k.strip(): _json_or_text(v) for k, v in re.findall(r"<parameter=([^>\n]+)>\n?(.*?)\n?</parameter>", fm.group(2), re.S)}
            calls.append(_call(fm.group(1).strip(), args))
            return ""
        rest = re.sub(r"<tool_call>(.*?)</tool_call>", take, text, flags=re.S)
        return (rest.strip(), calls) if calls else (text, [])
    if style == "glm":
        def take(m):
            body = m.group(1).strip()
            name = body.split("\n", 1)[0].split("<", 1)[0].strip()
            if not name:
                return m.group(0)
            args = {k.strip(): _json_or_text(v) for k, v in
                    re.findall(r"<arg_key>(.*?)</arg_key>\s*<arg_value>(.*?)</arg_value>", body, re.S)}
            calls.append(_call(name, args))
            return ""
        rest = re.sub(r"<tool_call>(.*?)</tool_call>", take, text, flags=re.S)
        return (rest.strip(), calls) if calls else (text, [])
    if style in ("deepseek", "deepseek_v31"):
        begin, end = "<\uff5ctool\u2581calls\u2581begin\uff5c>", "<\uff5ctool\u2581calls\u2581end\uff5c>"
        cb, ce, sep = "<\uff5ctool\u2581call\u2581begin\uff5c>", "<\uff5ctool\u2581call\u2581end\uff5c>", "<\uff5ctool\u2581sep\uff5c>"
        if begin not in text:
            return text, []
        head, _, tail = text.partition(begin)
        block = tail.split(end, 1)[0]
        for part in block.split(cb)[1:]:
            part = part.split(ce, 1)[0]
            a, _, b = part.partition(sep)
            if style == "deepseek":                 # "function<sep>NAME\n```json\n{...}\n```"
                name, _, js = b.partition("\n")
                js = re.sub(r"^```(?:json)?\s*|\s*```\s*$", "", js.strip())
            else:                                   # "NAME<sep>{...}"
                name, js = a, b
            calls.append(_call(name.strip(), json.loads(js)))
        return head.strip(), calls
    if style == "kimi":
        if "<|tool_calls_section_begin|>" not in text:
            return text, []
        head, _, tail = text.partition("<|tool_calls_section_begin|>")
        for m in re.finditer(r"<\|tool_call_begin\|>\s*([^<]+?)\s*<\|tool_call_argument_begin\|>(.*?)<\|tool_call_end\|>", tail, re.S):
            name = m.group(1).strip()
            name = name.split(".", 1)[1] if name.startswith("functions.") else name
            calls.append(_call(name.rsplit(":", 1)[0], json.loads(m.group(2))))
        return (head.strip(), calls) if calls else (text, [])
    if style == "gpt_oss":
        pat = re.compile(r"(?:<\|start\|>assistant)?<\|channel\|>(?:commentary|analysis)\s+to=functions\.([\w.\-]+)[^<]*(?:<\|constrain\|>\w+)?"
                         r"<\|message\|>(.*?)(?:<\|call\|>|$)", re.S)
        rest = text
        for m in pat.finditer(text):
            calls.append(_call(m.group(1), json.loads(m.group(2))))
            rest = rest.replace(m.group(0), "")
        if not calls:
            return text, []
        return _split_harmony(rest)[1], calls
    if style in ("pythonic", "llama4_pythonic", "lfm2"):
        wrap = {"llama4_pythonic": ("<|python_start|>", "<|python_end|>"), "lfm2": ("<|tool_call_start|>", "<|tool_call_end|>")}.get(style)
        body, head, tail = text.strip(), "", ""
        if wrap and wrap[0] in text:
            head, _, r = text.partition(wrap[0])
            body, _, tail = r.partition(wrap[1])
        if not (body.strip().startswith("[") and body.strip().endswith("]")):
            return text, []
        calls = _pythonic_calls(body)
        return (head + tail).strip(), calls
    if style == "xlam":
        body = re.sub(r"^```(?:json)?\s*|\s*```\s*$", "", text.strip())
        arr = json.loads(body)
        arr = arr.get("tool_calls", arr) if isinstance(arr, dict) else arr
        for o in arr if isinstance(arr, list) else [arr]:
            c = _from_obj(o)
            if c is None:
                return text, []
            calls.append(c)
        return ("", calls) if calls else (text, [])
    if style in _MARKER_JSON:
        open_m, close_m = _MARKER_JSON[style]
        if open_m not in text:
            return text, []
        head, _, tail = text.partition(open_m)
        after = ""
        if close_m and close_m in tail:
            tail, _, after = tail.partition(close_m)
        tail = tail.strip()
        try:
            arr = json.loads(tail)
            arr = arr if isinstance(arr, list) else [arr]
        except json.JSONDecodeError:                # one JSON object per line
            arr = [json.loads(l) for l in tail.splitlines() if l.strip()]
        for o in arr:
            c = _from_obj(o)
            if c is None:
                return text, []
            calls.append(c)
        return (head + after).strip(), calls
    return text, []
