"""Output parsers of the chat API: reasoning blocks and tool calls.

* Reasoning (``--reasoning-parser``): ``think`` splits ``<think> ... </think>`` off the front of the
  answer into ``reasoning_content`` (DeepSeek-R1 / Qwen3 style); ``think_open`` is for chat templates
  that already end with the opening tag, so that the model only writes the closing one.
  ``ReasoningStream`` is the incremental form used while streaming; both forms give the same split.
* Tool calls (``--tool-parser``): ``hermes`` (``<tool_call>{json}</tool_call>``, Qwen / Hermes),
  ``llama3_json`` (the whole answer, or what follows ``<|python_tag|>``, is
  ``{"name": ..., "parameters": {...}}``, several separated by ``;``), ``mistral``
  (``[TOOL_CALLS] [{...}, ...]``). Each returns the remaining text and OpenAI-shaped ``tool_calls``.

The reference's counterparts: rust/engine/src/tool_parser.rs, rust/engine/src/reasoning.rs.
"""
from __future__ import annotations

import json
import re
import uuid
from typing import List, Optional, Tuple

REASONING_PARSERS = ("think", "think_open")
TOOL_PARSERS = ("hermes", "llama3_json", "mistral")


# ------------------------------------------------------------------------------ reasoning
def split_reasoning(text: str, style: str = "think") -> Tuple[Optional[str], str]:
    """-> (reasoning or None, answer)."""
    if style not in REASONING_PARSERS:
        raise ValueError(f"unknown reasoning parser {style!r}")
    open_t, close_t = "<think>", "</think>"
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
        self.open_t, self.close_t = "<think>", "</think>"
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
    raise ValueError(f"unknown tool parser {style!r}")
