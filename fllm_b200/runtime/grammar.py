"""Structured output: JSON-constrained decoding.

A character-level incremental JSON recogniser (``json_step``) is walked over a trie of the
tokenizer's pieces to find, for the current state, every token whose characters keep the output a
prefix of a valid JSON document. The result is a bit mask (one bit per vocabulary entry) handed to
the sampler's allowed-token input, so the constraint costs nothing on the device side. Masks are
cached per recogniser state: the state is a small hashable tuple and the same states (inside a
string, after a comma in an object, ...) come back all the time.

The reference delegates this to xgrammar / llguidance (rust/engine/src/structured.rs); here the
recogniser covers ``response_format: {"type": "json_object"}`` (OpenAI), ``format: "json"`` (Ollama)
and ``json_schema`` requests: ``JsonSchemaStep`` enforces properties / required / additionalProperties /
type / enum / const on the top-level object; nested values are any JSON of the declared type.
``GuidedChoice`` constrains the output to one of a list of strings (``guided_choice``) through the same
trie walk with its own step function.
"""
from __future__ import annotations

from typing import Dict, Iterable, List, Optional, Sequence, Tuple

import numpy as np

# state = (mode, aux, stack); stack is a str of 'o' / 'a' (innermost last)
State = Tuple[str, object, str]
_WS = " \t\n\r"
_DIG = "0123456789"
_HEX = "0123456789abcdefABCDEF"
_NUM_END = ("N0", "NI", "NF", "NE")          # modes in which a number may end


def json_start(require_object: bool = True) -> State:
    return ("V{" if require_object else "V", None, "")


def _after_value(stack: str) -> State:
    return ("A", None, stack) if stack else ("D", None, "")


def json_step(st: State, ch: str) -> Optional[State]:
    """The state after reading `ch`, or None when `ch` cannot follow."""
    mode, aux, stack = st
    if mode in ("V", "V{"):
        if ch in _WS:
            return st
        if ch == "{":
            return ("K", None, stack + "o")
        if mode == "V{":
            return None
        if ch == "[":
            return ("V]", None, stack + "a")
        if ch == '"':
            return ("S", "v", stack)
        if ch == "-":
            return ("N-", None, stack)
        if ch == "0":
            return ("N0", None, stack)
        if ch in _DIG:
            return ("NI", None, stack)
        if ch == "t":
            return ("L", "rue", stack)
        if ch == "f":
            return ("L", "alse", stack)
        if ch == "n":
            return ("L", "ull", stack)
        return None
    if mode == "V]":                             # first element of an array, or its end
        if ch == "]":
            return _after_value(stack[:-1])
        if ch in _WS:
            return st
        return json_step(("V", None, stack), ch)
    if mode == "S":
        if ch == '"':
            return ("C", None, stack) if aux == "k" else _after_value(stack)
        if ch == "\\":
            return ("E", aux, stack)
        return st if ord(ch) >= 0x20 else None
    if mode == "E":
        if ch in '"\\/bfnrt':
            return ("S", aux, stack)
        if ch == "u":
            return ("U", (aux, 4), stack)
        return None
    if mode == "U":
        kind, left = aux
        if ch not in _HEX:
            return None
        return ("S", kind, stack) if left == 1 else ("U", (kind, left - 1), stack)
    if mode == "L":
        if ch != aux[0]:
            return None
        return ("L", aux[1:], stack) if len(aux) > 1 else _after_value(stack)
    if mode == "N-":
        return ("N0", None, stack) if ch == "0" else ("NI", None, stack) if ch in _DIG else None
    if mode in _NUM_END or mode in ("N.", "Ne", "Ns"):
        if mode in ("NI", "NF", "NE") and ch in _DIG:
            return st
        if mode in ("N0", "NI") and ch == ".":
            return ("N.", None, stack)
        if mode == "N.":
            return ("NF", None, stack) if ch in _DIG else None
        if mode in ("N0", "NI", "NF") and ch in "eE":
            return ("Ne", None, stack)
        if mode == "Ne":
            return ("Ns", None, stack) if ch in "+-" else ("NE", None, stack) if ch in _DIG else None
        if mode == "Ns":
            return ("NE", None, stack) if ch in _DIG else None
        # a complete number ends at the first character that is not part of it
        return json_step(_after_value(stack), ch)
    if mode == "A":
        if ch in _WS:
            return st
        top = stack[-1]
        if ch == ",":
            return ("K2", None, stack) if top == "o" else ("V", None, stack)
        if ch == "}" and top == "o" or ch == "]" and top == "a":
            return _after_value(stack[:-1])
        return None
    if mode in ("K", "K2"):
        if ch in _WS:
            return st
        if ch == '"':
            return ("S", "k", stack)
        if ch == "}" and mode == "K":
            return _after_value(stack[:-1])
        return None
    if mode == "C":
        if ch in _WS:
            return st
        return ("V", None, stack) if ch == ":" else None
    if mode == "D":
        return st if ch in _WS else None
    return None


def json_complete(st: State) -> bool:
    return st[0] == "D" or (st[0] in _NUM_END and not st[2])


def json_feed(st: Optional[State], text: str) -> Optional[State]:
    for ch in text:
        if st is None:
            return None
        st = json_step(st, ch)
    return st


class TokenTrie:
    """Trie over the text of every ordinary token. Tokens whose text is empty, contains the
    replacement character (a partial UTF-8 sequence) or that are control tokens are left out."""

    def __init__(self, pieces: Sequence[Optional[str]]):
        self.vocab = len(pieces)
        self.children: List[Dict[str, int]] = [{}]
        self.ids: List[List[int]] = [[]]
        for tid, text in enumerate(pieces):
            if not text or "�" in text:
                continue
            node = 0
            for ch in text:
                nxt = self.children[node].get(ch)
                if nxt is None:
                    nxt = len(self.children)
                    self.children[node][ch] = nxt
                    self.children.append({})
                    self.ids.append([])
                node = nxt
            self.ids[node].append(tid)

    @classmethod
    def from_tokenizer(cls, tokenizer, special_ids: Iterable[int] = ()) -> "TokenTrie":
        special = set(int(s) for s in special_ids)
        for name in ("bos_token_id", "eos_token_id"):
            v = getattr(tokenizer, name, None)
            if v is not None:
                special.add(int(v))
        pieces = [None if i in special else tokenizer.decode([i]) for i in range(tokenizer.vocab_size)]
        return cls(pieces)

    def allowed(self, st, step=None) -> List[int]:
        """Tokens all of whose characters can follow state `st` under `step(state, ch) -> state | None`
        (the JSON recogniser by default)."""
        step = step or json_step
        out: List[int] = []
        stack = [(0, st)]
        children, ids = self.children, self.ids
        while stack:
            node, s = stack.pop()
            for ch, nxt in children[node].items():
                s2 = step(s, ch)
                if s2 is None:
                    continue
                if ids[nxt]:
                    out.extend(ids[nxt])
                if children[nxt]:
                    stack.append((nxt, s2))
        return out


class GuidedJson:
    """Per-request constraint object: ``mask_words`` for the sampler, ``advance`` after each token."""

    def __init__(self, trie: TokenTrie, tokenizer, eos_ids: Sequence[int], require_object: bool = True,
                 cache: Optional[dict] = None):
        self.trie, self.tok = trie, tokenizer
        self.eos_ids = [int(e) for e in eos_ids if e is not None]
        self.state: Optional[State] = json_start(require_object)
        self.cache = cache if cache is not None else {}

    @property
    def complete(self) -> bool:
        return self.state is not None and json_complete(self.state)

    def mask_words(self, vocab: int) -> np.ndarray:
        words = (vocab + 31) // 32
        key = (self.state, vocab)
        m = self.cache.get(key)
        if m is None:
            m = np.zeros(words, dtype=np.uint32)
            if self.state is not None:
                ids = np.asarray([t for t in self.trie.allowed(self.state) if t < vocab], dtype=np.int64)
                if ids.size:
                    np.bitwise_or.at(m, ids >> 5, (np.uint32(1) << (ids & 31).astype(np.uint32)))
            if self.state is None or json_complete(self.state):
                for e in self.eos_ids:
                    if e < vocab:
                        m[e >> 5] |= np.uint32(1 << (e & 31))
            if len(self.cache) > 4096:
                self.cache.clear()
            self.cache[key] = m
        return m

    def advance(self, token_id: int) -> None:
        if token_id in self.eos_ids or self.state is None:
            return
        self.state = json_feed(self.state, self.tok.decode([int(token_id)]))


class GuidedChoice:
    """Constraint "the output is exactly one of these strings" (``guided_choice``): the state is the text
    produced so far, a character may follow while some choice still starts with the result, and the end
    of sequence is allowed once the text equals a choice."""

    def __init__(self, trie: TokenTrie, tokenizer, eos_ids: Sequence[int], choices: Sequence[str]):
        self.trie, self.tok = trie, tokenizer
        self.eos_ids = [int(e) for e in eos_ids if e is not None]
        self.choices = [str(c) for c in choices if str(c)]
        if not self.choices:
            raise ValueError("guided_choice needs at least one non-empty string")
        self.state: Optional[str] = ""
        self.cache: dict = {}

    def _step(self, prefix: str, ch: str) -> Optional[str]:
        nxt = prefix + ch
        return nxt if any(c.startswith(nxt) for c in self.choices) else None

    @property
    def complete(self) -> bool:
        return self.state is not None and self.state in self.choices

    def mask_words(self, vocab: int) -> np.ndarray:
        key = (self.state, vocab)
        m = self.cache.get(key)
        if m is None:
            m = np.zeros((vocab + 31) // 32, dtype=np.uint32)
            if self.state is not None:
                ids = np.asarray([t for t in self.trie.allowed(self.state, self._step) if t < vocab], dtype=np.int64)
                if ids.size:
                    np.bitwise_or.at(m, ids >> 5, (np.uint32(1) << (ids & 31).astype(np.uint32)))
            if self.state is None or self.complete:
                for e in self.eos_ids:
                    if e < vocab:
                        m[e >> 5] |= np.uint32(1 << (e & 31))
            self.cache[key] = m
        return m

    def advance(self, token_id: int) -> None:
        if token_id in self.eos_ids or self.state is None:
            return
        st: Optional[str] = self.state
        for ch in self.tok.decode([int(token_id)]):
            st = self._step(st, ch) if st is not None else None
        self.state = st


# ----------------------------------------------------------------------------- JSON schema (top-level object)
_TYPE_FIRST = {"string": '"', "number": "-0123456789", "integer": "-0123456789", "boolean": "tf", "null": "n",
               "object": "{", "array": "["}
_NUM_MODES = ("N-", "N0", "NI", "N.", "NF", "Ne", "Ns", "NE")


class JsonSchemaStep:
    """The JSON recogniser plus the keywords of an object schema that matter most for tool calls and
    structured outputs, enforced on the TOP-LEVEL object: ``properties`` (with ``additionalProperties:
    false`` only declared keys can be written, each once), ``required`` (the object cannot close before
    they are all present), and per property ``type`` (also a list of types), ``enum`` and ``const``
    (the value's JSON text must be one of the listed literals). Nested values are any JSON of the
    declared type. State = (json state, key text being written, key whose value is open, keys done,
    value text for enum matching); it is hashable, so masks are cached per state like the plain ones."""

    def __init__(self, schema: dict):
        import json as _json
        if not isinstance(schema, dict) or schema.get("type", "object") != "object":
            raise ValueError("json_schema: the top level must be an object schema")
        self.props: Dict[str, dict] = {str(k): (v if isinstance(v, dict) else {}) for k, v in (schema.get("properties") or {}).items()}
        self.required = frozenset(str(k) for k in (schema.get("required") or ()))
        self.closed = schema.get("additionalProperties") is False
        unknown = self.required - set(self.props)
        if self.closed and unknown:
            raise ValueError(f"json_schema: required keys without a property: {sorted(unknown)}")
        self.literals: Dict[str, Tuple[str, ...]] = {}
        for k, p in self.props.items():
            vals = p["enum"] if isinstance(p.get("enum"), list) else ([p["const"]] if "const" in p else None)
            if vals is not None:
                self.literals[k] = tuple(_json.dumps(v, ensure_ascii=False, separators=(",", ":")) for v in vals)

    def start(self):
        return (json_start(True), None, None, frozenset(), None)

    def _first_chars(self, key: str) -> Optional[str]:
        p = self.props.get(key)
        if p is None:
            return None
        if key in self.literals:
            return "".join(sorted({lit[0] for lit in self.literals[key]}))
        t = p.get("type")
        if t is None:
            return None
        types = t if isinstance(t, list) else [t]
        return "".join(_TYPE_FIRST.get(x, "") for x in types) or None

    def __call__(self, st, ch: str):
        js, kbuf, key, seen, vbuf = st
        mode, aux, stack = js
        js2 = json_step(js, ch)
        if js2 is None:
            return None
        top = stack == "o"
        if top and mode in ("K", "K2") and ch == '"':
            return (js2, "", key, seen, None)
        if top and mode == "S" and aux == "k":                       # inside a top-level key
            if ch == '"':
                if self.closed and (kbuf not in self.props or kbuf in seen):
                    return None
                if kbuf in seen:
                    return None                                       # a key is written once
                return (js2, None, kbuf, seen, None)
            if ch == "\\":
                return None if self.closed else (js2, None, key, seen, None)
            if kbuf is None:
                return (js2, None, key, seen, None)                   # free-form key (after an escape)
            nk = kbuf + ch
            if self.closed and not any(k.startswith(nk) and k not in seen for k in self.props):
                return None
            return (js2, nk, key, seen, None)
        if top and mode == "V" and key is not None and ch not in _WS:   # first character of the key's value
            first = self._first_chars(key)
            if first is not None and ch not in first:
                return None
            if key in self.literals:
                vbuf = ""
        if key is not None and vbuf is not None and (len(stack) > 1 or top) and not (top and mode in ("A",)):
            # the value's text must stay a prefix of one of the allowed literals, and end exactly on one
            in_value = not (top and mode in ("C", "K", "K2"))
            ended_number = top and mode in _NUM_END and json_step(_after_value(stack), ch) is not None and ch not in _DIG + ".eE"
            if in_value and not ended_number and not (top and mode == "V" and ch in _WS):
                nv = vbuf + ch
                if not any(l.startswith(nv) for l in self.literals[key]):
                    return None
                vbuf = nv
        p = self.props.get(key) if key is not None else None
        if top and p is not None and mode in _NUM_MODES and ch in ".eE":
            t = p.get("type")
            if t == "integer" or (isinstance(t, list) and "integer" in t and "number" not in t):
                return None
        mode2, _, stack2 = js2
        if key is not None and ((stack2 == "o" and mode2 in ("A", "K2")) or stack2 == ""):
            if not (top and mode == "V" and ch in _WS) and not (stack2 == "o" and mode2 == "A" and mode == "A"):
                if vbuf is not None and key in self.literals:
                    done_text = vbuf if not (top and mode in _NUM_END and ch in ",} \t\n\r") else vbuf
                    if done_text not in self.literals[key]:
                        return None
                seen = seen | {key}
                key, vbuf = None, None
        if top and stack2 == "" and not self.required <= seen:
            return None                                               # closing before every required key is present
        if top and mode2 == "K2" and stack2 == "o" and mode != "K2" and self.closed and all(k in seen for k in self.props):
            return None                                               # a comma with no key left to write
        return (js2, kbuf if (top and mode == "S" and aux == "k") else None, key, seen, vbuf)


class GuidedJsonSchema(GuidedJson):
    """``response_format: {"type": "json_schema", ...}``: the JSON constraint plus ``JsonSchemaStep``."""

    def __init__(self, trie: TokenTrie, tokenizer, eos_ids: Sequence[int], schema: dict, cache: Optional[dict] = None):
        super().__init__(trie, tokenizer, eos_ids, True, {} if cache is None else cache)
        self.schema_step = JsonSchemaStep(schema)
        self.state = self.schema_step.start()

    @property
    def complete(self) -> bool:
        return self.state is not None and json_complete(self.state[0])

    def mask_words(self, vocab: int) -> np.ndarray:
        key = (self.state, vocab)
        m = self.cache.get(key)
        if m is None:
            m = np.zeros((vocab + 31) // 32, dtype=np.uint32)
            if self.state is not None:
                ids = np.asarray([t for t in self.trie.allowed(self.state, self.schema_step) if t < vocab], dtype=np.int64)
                if ids.size:
                    np.bitwise_or.at(m, ids >> 5, (np.uint32(1) << (ids & 31).astype(np.uint32)))
            if self.state is None or self.complete:
                for e in self.eos_ids:
                    if e < vocab:
                        m[e >> 5] |= np.uint32(1 << (e & 31))
            if len(self.cache) > 4096:
                self.cache.clear()
            self.cache[key] = m
        return m

    def advance(self, token_id: int) -> None:
        if token_id in self.eos_ids or self.state is None:
            return
        st = self.state
        for ch in self.tok.decode([int(token_id)]):
            st = self.schema_step(st, ch) if st is not None else None
        self.state = st


class GuidedToolCall(GuidedJsonSchema):
    """A forced tool call in the Hermes / Qwen markup: ``<tool_call>`` + a JSON object
    ``{"name": one of the offered functions, "arguments": {...}}`` + ``</tool_call>``
    (``tool_choice: "required"`` or a named function; the reference builds such grammars in
    rust/engine/src/tool_grammar.rs:1-8). State = (phase, inner): the literal prefix character by character, the
    schema-constrained JSON, then the literal suffix; the end of sequence is allowed after the suffix."""

    PREFIX, SUFFIX = "<tool_call>\n", "</tool_call>"

    def __init__(self, trie: TokenTrie, tokenizer, eos_ids: Sequence[int], names: Sequence[str]):
        names = [str(n) for n in names if str(n)]
        if not names:
            raise ValueError("tool_choice needs at least one function name")
        schema = {"type": "object", "properties": {"name": {"enum": names}, "arguments": {"type": "object"}},
                  "required": ["name", "arguments"], "additionalProperties": False}
        super().__init__(trie, tokenizer, eos_ids, schema)
        inner = self.schema_step

        def step(st, ch):
            phase, x = st
            if phase == "pre":
                if self.PREFIX[x] != ch:
                    return None
                return ("pre", x + 1) if x + 1 < len(self.PREFIX) else ("json", inner.start())
            if phase == "json":
                nxt = inner(x, ch)
                if nxt is not None:
                    return ("json", nxt)
                if json_complete(x[0]) and ch == self.SUFFIX[0]:
                    return ("post", 1)
                return None
            if phase == "post":
                if x >= len(self.SUFFIX) or self.SUFFIX[x] != ch:
                    return None
                return ("post", x + 1)
            return None
        self.schema_step = step
        self.state = ("pre", 0)

    @property
    def complete(self) -> bool:
        return self.state is not None and self.state[0] == "post" and self.state[1] == len(self.SUFFIX)
