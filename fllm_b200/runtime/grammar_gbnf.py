"""General grammar-constrained decoding: GBNF grammars, regular expressions and full (nested)
JSON schemas, all run by one character-level pushdown machine over the tokenizer's trie.

The reference hands these to llguidance (rust/engine/src/structured.rs:1, tool_grammar.rs:1-8:
JSON schema, GBNF / Lark, regex, tool-call grammars). Here:

* ``parse_gbnf`` reads llama.cpp's GBNF (``root ::= ...``; literals, character classes, rule
  references, groups, ``* + ? {m,n}``, alternation, comments) into rules whose alternatives are
  sequences of single-character terminals and rule references (repetitions and groups become
  helper rules);
* ``regex_to_rules`` compiles a regular expression (literals, ``.``, classes, ``\\d \\w \\s`` escapes,
  groups, alternation, ``* + ? {m,n}``, anchors ignored - the whole output must match) to the same
  rule form;
* ``schema_to_gbnf`` writes a JSON schema as GBNF: nested objects (properties in declaration order,
  required ones mandatory, ``additionalProperties`` honoured), arrays (``items``, ``minItems`` /
  ``maxItems``), ``enum`` / ``const``, ``anyOf`` / ``oneOf``, ``type`` lists, string ``pattern`` /
  ``minLength`` / ``maxLength``, integer vs number, local ``$ref`` / ``$defs``;
* ``GrammarMachine`` is the recogniser: a state is a frozen set of stacks of rule positions (hashable,
  so masks are cached per state exactly like the JSON recogniser's); ``GuidedGrammar`` adapts it to
  the sampler's allowed-token mask.
"""
from __future__ import annotations

import json
import re
from typing import Dict, FrozenSet, List, Optional, Sequence, Tuple

import numpy as np

# element: ("c", ((lo, hi), ...), negated)  one character of a class  |  ("r", rule_name)
Elem = tuple
Rules = Dict[str, List[Tuple[Elem, ...]]]


class GrammarError(ValueError):
    pass


def _lit(s: str) -> Tuple[Elem, ...]:
    return tuple(("c", ((ch, ch),), False) for ch in s)


_ESC = {"n": "\n", "r": "\r", "t": "\t", "\\": "\\", '"': '"', "'": "'", "[": "[", "]": "]", "-": "-", "/": "/", "0": "\0"}


class _GbnfParser:
    def __init__(self, text: str):
        self.s, self.i = text, 0
        self.rules: Rules = {}
        self.n_aux = 0

    def err(self, msg: str):
        line = self.s.count("\n", 0, self.i) + 1
        raise GrammarError(f"grammar line {line}: {msg}")

    def ws(self, newlines: bool = True):
        while self.i < len(self.s):
            c = self.s[self.i]
            if c == "#":
                while self.i < len(self.s) and self.s[self.i] != "\n":
                    self.i += 1
            elif c in " \t" or (newlines and c in "\r\n"):
                self.i += 1
            else:
                break

    def name(self) -> str:
        m = re.compile(r"[A-Za-z_][\w\-]*").match(self.s, self.i)
        if not m:
            self.err("rule name expected")
        self.i = m.end()
        return m.group(0)

    def aux(self, base: str) -> str:
        self.n_aux += 1
        return f"{base}~{self.n_aux}"

    def char(self) -> str:
        c = self.s[self.i]
        if c != "\\":
            self.i += 1
            return c
        self.i += 1
        e = self.s[self.i]
        self.i += 1
        if e == "x":
            v = self.s[self.i:self.i + 2]; self.i += 2
            return chr(int(v, 16))
        if e == "u":
            v = self.s[self.i:self.i + 4]; self.i += 4
            return chr(int(v, 16))
        if e == "U":
            v = self.s[self.i:self.i + 8]; self.i += 8
            return chr(int(v, 16))
        if e in _ESC:
            return _ESC[e]
        self.err(f"unknown escape \\{e}")

    def repeat(self, item: Tuple[Elem, ...], lo: int, hi: Optional[int], base: str) -> Tuple[Elem, ...]:
        """item{lo,hi} as elements (hi None = unbounded)."""
        if len(item) != 1 or item[0][0] != "r":
            sub = self.aux(base)
            self.rules[sub] = [item]
            item = (("r", sub),)
        seq = item * lo
        if hi is None:
            star = self.aux(base)
            self.rules[star] = [item + (("r", star),), ()]
            return seq + (("r", star),)
        opt_chain: Tuple[Elem, ...] = ()
        for _ in range(hi - lo):                       # (x (x (x)?)?)?
            o = self.aux(base)
            self.rules[o] = [item + opt_chain, ()]
            opt_chain = (("r", o),)
        return seq + opt_chain

    def sequence(self, base: str) -> Tuple[Elem, ...]:
        out: Tuple[Elem, ...] = ()
        while True:
            self.ws(newlines=False)
            if self.i >= len(self.s):
                break
            c = self.s[self.i]
            if c == '"':
                self.i += 1
                lit = []
                while self.i < len(self.s) and self.s[self.i] != '"':
                    lit.append(self.char())
                if self.i >= len(self.s):
                    self.err("unterminated literal")
                self.i += 1
                item = _lit("".join(lit))
            elif c == "[":
                self.i += 1
                neg = self.s[self.i] == "^"
                if neg:
                    self.i += 1
                ranges = []
                while self.i < len(self.s) and self.s[self.i] != "]":
                    a = self.char()
                    if self.s[self.i] == "-" and self.s[self.i + 1] != "]":
                        self.i += 1
                        b = self.char()
                        ranges.append((a, b))
                    else:
                        ranges.append((a, a))
                if self.i >= len(self.s):
                    self.err("unterminated character class")
                self.i += 1
                item = (("c", tuple(ranges), neg),)
            elif c == ".":
                self.i += 1
                item = (("c", (), True),)                       # anything
            elif c == "(":
                self.i += 1
                sub = self.aux(base)
                self.rules[sub] = self.alternatives(sub)
                self.ws()
                if self.i >= len(self.s) or self.s[self.i] != ")":
                    self.err("')' expected")
                self.i += 1
                item = (("r", sub),)
            elif c.isalpha() or c == "_":
                save = self.i
                nm = self.name()
                self.ws(newlines=False)
                if self.s.startswith("::=", self.i):              # the next rule starts here
                    self.i = save
                    break
                item = (("r", nm),)
            else:
                break
            # postfix operators
            if self.i < len(self.s) and self.s[self.i] in "*+?":
                op = self.s[self.i]
                self.i += 1
                item = self.repeat(item, 1 if op == "+" else 0, 1 if op == "?" else None, base)
            elif self.i < len(self.s) and self.s[self.i] == "{":
                m = re.compile(r"\{(\d+)(,(\d*))?\}").match(self.s, self.i)
                if not m:
                    self.err("bad repetition")
                self.i = m.end()
                lo = int(m.group(1))
                hi = lo if m.group(2) is None else (int(m.group(3)) if m.group(3) else None)
                item = self.repeat(item, lo, hi, base)
            out += item
        return out

    def alternatives(self, base: str) -> List[Tuple[Elem, ...]]:
        alts = [self.sequence(base)]
        while True:
            self.ws()
            if self.i < len(self.s) and self.s[self.i] == "|":
                self.i += 1
                self.ws()
                alts.append(self.sequence(base))
            else:
                return alts

    def parse(self) -> Rules:
        self.ws()
        while self.i < len(self.s):
            nm = self.name()
            self.ws(newlines=False)
            if not self.s.startswith("::=", self.i):
                self.err("'::=' expected")
            self.i += 3
            self.ws()
            self.rules[nm] = self.alternatives(nm)
            self.ws()
        if "root" not in self.rules:
            raise GrammarError("the grammar has no 'root' rule")
        for alts in self.rules.values():
            for alt in alts:
                for e in alt:
                    if e[0] == "r" and e[1] not in self.rules:
                        raise GrammarError(f"undefined rule {e[1]!r}")
        return self.rules


def parse_gbnf(text: str) -> Rules:
    return _GbnfParser(text).parse()


# ----------------------------------------------------------------------------- regular expressions
_CLASS_ESC = {"d": (("0", "9"),), "w": (("a", "z"), ("A", "Z"), ("0", "9"), ("_", "_")), "s": ((" ", " "), ("\t", "\t"), ("\n", "\n"), ("\r", "\r"))}


def regex_to_gbnf(pattern: str) -> str:
    """Rewrite a regular expression as a GBNF ``root`` rule (same operators, GBNF spelling)."""
    out, i, n = [], 0, len(pattern)

    def cls_body(esc: str, neg_outer: bool = False) -> str:
        body = {"d": "0-9", "w": "a-zA-Z0-9_", "s": " \\t\\n\\r"}[esc.lower()]
        return ("[^" if esc.isupper() != neg_outer else "[") + body + "]"
    while i < n:
        c = pattern[i]
        if c == "\\":
            e = pattern[i + 1] if i + 1 < n else "\\"
            i += 2
            if e in "dwsDWS":
                out.append(cls_body(e))
            elif e in "nrt":
                out.append(f'"\\{e}"')
            else:
                out.append(json.dumps(e))
        elif c == "[":
            j = i + 1
            if j < n and pattern[j] == "^":
                j += 1
            if j < n and pattern[j] == "]":
                j += 1
            while j < n and pattern[j] != "]":
                j += 2 if pattern[j] == "\\" else 1
            body = pattern[i:j + 1]
            body = body.replace("\\d", "0-9").replace("\\w", "a-zA-Z0-9_").replace("\\s", " \\t\\n\\r")
            out.append(body)
            i = j + 1
        elif c in "*+?":
            out[-1] = out[-1].rstrip() + c                       # postfix operators attach to their operand
            i += 1
        elif c in "(|":
            out.append(" " + c + " ")
            i += 1
        elif c == ")":
            out.append(c)
            i += 1
        elif c == ".":
            out.append("[^\\n]")                                  # like most regex dialects: any character but a newline
            i += 1
        elif c == "{":
            j = pattern.index("}", i)
            out[-1] = out[-1].rstrip() + pattern[i:j + 1]
            i = j + 1
        elif c in "^$":
            i += 1                                                # the whole output must match anyway
        else:
            out.append(json.dumps(c))
            i += 1
        out[-1] += " "
    return "root ::= " + "".join(out)


# ----------------------------------------------------------------------------- JSON schema -> GBNF
_PRIMS = {
    "ws": '([ \\t\\n\\r] [ \\t\\n\\r]?)?',          # at most two: unbounded white space lets a sampler stall inside it
    "string": '"\\"" char* "\\""',
    "char": '[^"\\\\\\x00-\\x1f] | "\\\\" (["\\\\/bfnrt] | "u" [0-9a-fA-F] [0-9a-fA-F] [0-9a-fA-F] [0-9a-fA-F])',
    "integer": '"-"? ("0" | [1-9] [0-9]*)',
    "number": 'integer ("." [0-9]+)? ([eE] [-+]? [0-9]+)?',
    "boolean": '"true" | "false"',
    "null": '"null"',
    "value": 'object | array | string | number | boolean | null',
    "object": '"{" ws (string ws ":" ws value (ws "," ws string ws ":" ws value)*)? ws "}"',
    "array": '"[" ws (value (ws "," ws value)*)? ws "]"',
}


class _SchemaCompiler:
    def __init__(self, root_schema: dict):
        self.root_schema = root_schema
        self.rules: Dict[str, str] = {}
        self.n = 0
        self.refs: Dict[str, str] = {}

    def prim(self, name: str) -> str:
        if name not in self.rules:
            self.rules[name] = _PRIMS[name]
            for dep in re.findall(r"\b(ws|string|char|integer|number|boolean|null|value|object|array)\b", _PRIMS[name]):
                if dep != name:
                    self.prim(dep)
        return name

    def fresh(self, hint: str) -> str:
        self.n += 1
        return re.sub(r"[^A-Za-z0-9]", "-", hint)[:24].strip("-") + f"-{self.n}"

    def literal(self, v) -> str:
        return json.dumps(json.dumps(v, ensure_ascii=False), ensure_ascii=False)

    def add(self, hint: str, body: str) -> str:
        nm = self.fresh(hint or "r")
        self.rules[nm] = body
        return nm

    def resolve(self, ref: str) -> dict:
        if not ref.startswith("#/"):
            raise GrammarError(f"only local references are supported, not {ref!r}")
        node = self.root_schema
        for part in ref[2:].split("/"):
            node = node[part.replace("~1", "/").replace("~0", "~")]
        return node

    def visit(self, sch, hint: str = "v") -> str:
        if sch is True or sch == {} or sch is None:
            return self.prim("value")
        if sch is False:
            raise GrammarError("a false schema matches nothing")
        if "$ref" in sch:
            ref = sch["$ref"]
            if ref not in self.refs:
                nm = self.fresh("ref")
                self.refs[ref] = nm
                self.rules[nm] = ""                              # placeholder: recursive schemas refer to it
                self.rules[nm] = self.visit(self.resolve(ref), hint)
            return self.refs[ref]
        if "const" in sch:
            return self.add(hint, self.literal(sch["const"]))
        if "enum" in sch:
            return self.add(hint, " | ".join(self.literal(v) for v in sch["enum"]))
        for key in ("anyOf", "oneOf"):
            if key in sch:
                return self.add(hint, " | ".join(self.visit(s, hint) for s in sch[key]))
        if "allOf" in sch and len(sch["allOf"]) == 1:
            return self.visit(sch["allOf"][0], hint)
        t = sch.get("type")
        if isinstance(t, list):
            return self.add(hint, " | ".join(self.visit(dict(sch, type=x), hint) for x in t))
        if t == "object" or (t is None and "properties" in sch):
            return self.object(sch, hint)
        if t == "array" or (t is None and "items" in sch):
            return self.array(sch, hint)
        if t == "string":
            return self.string(sch, hint)
        if t in ("integer", "number", "boolean", "null"):
            return self.prim(t)
        return self.prim("value")

    def string(self, sch: dict, hint: str) -> str:
        if "pattern" in sch:
            sub = regex_to_gbnf(sch["pattern"])[len("root ::= "):]
            return self.add(hint, f'"\\"" ({sub}) "\\""')
        lo, hi = sch.get("minLength", 0), sch.get("maxLength")
        if lo or hi is not None:
            self.prim("char")
            rep = f"{{{lo},{hi if hi is not None else ''}}}"
            return self.add(hint, f'"\\"" char{rep} "\\""')
        return self.prim("string")

    def array(self, sch: dict, hint: str) -> str:
        ws = self.prim("ws")
        item = self.visit(sch.get("items", True), hint + "-item")
        lo, hi = int(sch.get("minItems", 0)), sch.get("maxItems")
        more = f'({ws} "," {ws} {item})'
        if hi is not None and int(hi) == 0:
            return self.add(hint, f'"[" {ws} "]"')
        if lo == 0:
            tail = f"{more}*" if hi is None else f"{more}{{0,{int(hi) - 1}}}"
            return self.add(hint, f'"[" {ws} ({item} {tail})? {ws} "]"')
        tail = f"{more}{{{lo - 1},{'' if hi is None else int(hi) - 1}}}"
        return self.add(hint, f'"[" {ws} {item} {tail} {ws} "]"')

    def other_key(self, names: List[str], hint: str) -> str:
        """A JSON string that is none of `names` (a declared property cannot come back as an "additional" one):
        walk the trie of the names; leaving the trie frees the rest of the string, ending on a complete name is barred."""
        self.prim("char")
        trie: dict = {}
        for nm in names:
            node = trie
            for ch in nm:
                node = node.setdefault(ch, {})
            node[None] = True

        def lit_char(ch: str) -> str:
            return json.dumps(ch) if ch not in '"\\' else json.dumps("\\" + ch)      # inside a JSON string: \" and \\

        def cls_char(ch: str) -> str:
            return "\\" + ch if ch in "]\\^-" else ch

        def walk(node: dict) -> str:
            alts = []
            for ch, child in node.items():
                if ch is not None:
                    alts.append(f"{lit_char(ch)} {walk(child)}")
            taken = "".join(cls_char(ch) for ch in node if ch is not None and ch not in '"\\')
            alts.append(f'[^"\\\\\\x00-\\x1f{taken}] char*')
            if "\\" not in node:
                alts.append('"\\\\" (["\\\\/bfnrt] | "u" [0-9a-fA-F] [0-9a-fA-F] [0-9a-fA-F] [0-9a-fA-F]) char*')
            if None not in node:
                alts.append('""')
            return self.add(hint + "-k", " | ".join(alts))
        return self.add(hint + "-key", f'"\\"" {walk(trie)} "\\""')

    def object(self, sch: dict, hint: str) -> str:
        ws = self.prim("ws")
        props = list((sch.get("properties") or {}).items())
        required = set(sch.get("required") or [])
        extra = sch.get("additionalProperties", True)
        kv = {}
        for k, v in props:
            kv[k] = self.add(f"{hint}-{k}-kv", f'{self.literal(k)} {ws} ":" {ws} {self.visit(v, hint + "-" + k)}')
        extra_kv = None
        if extra is not False and extra is not None:
            val = self.visit(extra if isinstance(extra, dict) else True, hint + "-extra")
            key = self.other_key([k for k, _ in props], hint) if props else self.prim("string")
            extra_kv = self.add(hint + "-extra-kv", f'{key} {ws} ":" {ws} {val}')
        sep = f'{ws} "," {ws}'
        # properties in declaration order; an optional one may be skipped; every tail rule says what may still follow
        names = [k for k, _ in props]

        def tail_rule(i: int, first: bool) -> str:
            """Rule for "the members from property i on", given whether a member has been written before."""
            key = ("tail", i, first)
            if key in memo:
                return memo[key]
            nm = self.fresh(f"{hint}-rest")
            memo[key] = nm
            alts = []
            lead = "" if first else sep + " "
            for j in range(i, len(names)):
                alts.append(f"{lead}{kv[names[j]]} {tail_rule(j + 1, False)}")
                if names[j] in required:
                    break
            else:
                if extra_kv:
                    more = self.add(hint + "-more", f"({sep} {extra_kv})*")
                    alts.append(f"{lead}{extra_kv} {more}")
                alts.append("")                                   # nothing more
            self.rules[nm] = " | ".join(a if a else '""' for a in alts)
            return nm
        memo: Dict[tuple, str] = {}
        return self.add(hint, f'"{{" {ws} {tail_rule(0, True)} {ws} "}}"')


def schema_to_gbnf(schema: dict) -> str:
    c = _SchemaCompiler(schema)
    root = c.visit(schema, "root")
    lines = [f"root ::= {root}"]
    lines += [f"{k} ::= {v}" for k, v in c.rules.items()]
    return "\n".join(lines)


# ----------------------------------------------------------------------------- the machine
Stack = Tuple[Tuple[str, int, int], ...]            # frames (rule, alternative, position), innermost last


def _match(elem: Elem, ch: str) -> bool:
    _, ranges, neg = elem
    hit = any(lo <= ch <= hi for lo, hi in ranges)
    return hit != neg


class GrammarMachine:
    """Pushdown recogniser over characters. ``start()`` -> state; ``step(state, ch)`` -> state or None;
    ``accepting(state)``. A state is a frozenset of stacks whose top element is a terminal (or that are empty)."""

    def __init__(self, rules: Rules, max_stacks: int = 4096):
        self.rules = rules
        self.max_stacks = max_stacks

    def _advance(self, stack: Stack, out: set, seen: set) -> None:
        """Expand `stack` until its top is a terminal; completed frames pop."""
        if stack in seen:
            return
        seen.add(stack)
        if len(out) > self.max_stacks:
            raise GrammarError("the grammar is too ambiguous for this recogniser")
        if not stack:
            out.add(stack)
            return
        rule, alt, pos = stack[-1]
        seq = self.rules[rule][alt]
        if pos >= len(seq):
            self._advance(stack[:-1], out, seen)
            return
        e = seq[pos]
        if e[0] == "c":
            out.add(stack)
            return
        base = stack[:-1] + ((rule, alt, pos + 1),)            # where to continue after the referenced rule
        for k in range(len(self.rules[e[1]])):
            self._advance(base + ((e[1], k, 0),), out, seen)

    def start(self) -> FrozenSet[Stack]:
        out: set = set()
        seen: set = set()
        for k in range(len(self.rules["root"])):
            self._advance((("root", k, 0),), out, seen)
        return frozenset(out)

    def step(self, state: FrozenSet[Stack], ch: str) -> Optional[FrozenSet[Stack]]:
        out: set = set()
        seen: set = set()
        for st in state:
            if not st:
                continue
            rule, alt, pos = st[-1]
            if _match(self.rules[rule][alt][pos], ch):
                self._advance(st[:-1] + ((rule, alt, pos + 1),), out, seen)
        return frozenset(out) if out else None

    @staticmethod
    def accepting(state: Optional[FrozenSet[Stack]]) -> bool:
        return state is not None and () in state

    def matches(self, text: str) -> bool:
        st = self.start()
        for ch in text:
            st = self.step(st, ch)
            if st is None:
                return False
        return self.accepting(st)


def machine_from(kind: str, spec) -> GrammarMachine:
    """kind: "gbnf" (text), "regex" (pattern) or "json_schema" (dict)."""
    if kind == "gbnf":
        return GrammarMachine(parse_gbnf(spec))
    if kind == "regex":
        return GrammarMachine(parse_gbnf(regex_to_gbnf(spec)))
    if kind == "json_schema":
        return GrammarMachine(parse_gbnf(schema_to_gbnf(spec)))
    raise GrammarError(f"unknown grammar kind {kind!r}")


class GuidedGrammar:
    """Per-request constraint object for the sampler (same protocol as ``grammar.GuidedJson``)."""

    def __init__(self, trie, tokenizer, eos_ids: Sequence[int], machine: GrammarMachine, cache: Optional[dict] = None):
        self.trie, self.tok, self.machine = trie, tokenizer, machine
        self.eos_ids = [int(e) for e in eos_ids if e is not None]
        self.state = machine.start()
        self.cache = cache if cache is not None else {}

    @property
    def complete(self) -> bool:
        return self.machine.accepting(self.state)

    def mask_words(self, vocab: int) -> np.ndarray:
        key = (self.state, vocab)
        m = self.cache.get(key)
        if m is None:
            m = np.zeros((vocab + 31) // 32, dtype=np.uint32)
            if self.state is not None:
                ids = np.asarray([t for t in self.trie.allowed(self.state, self.machine.step) if t < vocab], dtype=np.int64)
                if ids.size:
                    np.bitwise_or.at(m, ids >> 5, (np.uint32(1) << (ids & 31).astype(np.uint32)))
            if self.state is None or self.complete:
                for e in self.eos_ids:
                    if e < vocab:
                        m[e >> 5] |= np.uint32(1 << (e & 31))
            if len(self.cache) > 2048:
                self.cache.clear()
            self.cache[key] = m
        return m

    def advance(self, token_id: int) -> None:
        if token_id in self.eos_ids or self.state is None:
            return
        st = self.state
        for ch in self.tok.decode([int(token_id)]):
            st = self.machine.step(st, ch) if st is not None else None
        self.state = st
