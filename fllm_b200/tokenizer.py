"""Tokenizers and chat templates.

* ``HFTokenizer``    a ``tokenizer.json`` (Hugging Face ``tokenizers``), with the chat template and
                     special tokens of ``tokenizer_config.json`` when present;
* ``GgufTokenizer``  the vocabulary embedded in a GGUF file (``tokenizer.ggml.*``): byte-level BPE with
                     merges and the model family's pre-tokenizer pattern (``gpt2``), SentencePiece BPE
                     driven by the piece scores (``llama``), or unigram Viterbi (``t5`` / ``unigram``);
                     control tokens written in the text (``<|im_start|>``) map to their ids;
* ``TiktokenTokenizer``  a ``*.tiktoken`` rank file (base64 token, rank per line) with byte-level BPE;
* ``ByteTokenizer``  bytes + a few specials; lets random-weight models be served and tested.

The reference embeds BPE / SPM / unigram tokenizers and renders chat templates with a Jinja
engine (rust/engine/src/tokenizer.rs, rust/engine/src/chat_template.rs:1-6); here the Jinja
engine is ``jinja2`` with a ``tojson`` filter that matches Python's ``json.dumps``.
"""
from __future__ import annotations

import json
import os
from typing import Dict, List, Optional, Sequence

DEFAULT_CHAT_TEMPLATE = (
    "{% for m in messages %}<|im_start|>{{ m['role'] }}\n{{ m['content'] }}<|im_end|>\n{% endfor %}"
    "{% if add_generation_prompt %}<|im_start|>assistant\n{% endif %}")


def render_chat(template: Optional[str], messages: List[dict], add_generation_prompt: bool = True,
                tools: Optional[list] = None, **extra) -> str:
    import jinja2
    env = jinja2.Environment(trim_blocks=True, lstrip_blocks=True)
    env.filters["tojson"] = lambda v, indent=None: json.dumps(v, ensure_ascii=False, indent=indent)
    env.globals["raise_exception"] = lambda msg: (_ for _ in ()).throw(ValueError(msg))
    norm = []
    for m in messages:
        c = m.get("content")
        if isinstance(c, list):               # OpenAI content parts -> text
            c = "".join(p.get("text", "") for p in c if isinstance(p, dict) and p.get("type") in ("text", None))
        norm.append({**m, "content": c if c is not None else ""})
    return env.from_string(template or DEFAULT_CHAT_TEMPLATE).render(
        messages=norm, add_generation_prompt=add_generation_prompt, tools=tools, bos_token="", eos_token="", **extra)


class ByteTokenizer:
    """ids 0..255 are bytes; 256 = <bos>, 257 = <eos>."""
    bos_token_id, eos_token_id = 256, 257
    chat_template = DEFAULT_CHAT_TEMPLATE

    def __init__(self, vocab_size: int = 512):
        if vocab_size < 258:
            raise ValueError("ByteTokenizer needs a vocabulary of at least 258 ids")
        self.vocab_size = vocab_size

    def encode(self, text: str, add_bos: bool = False) -> List[int]:
        ids = list(text.encode("utf-8"))
        return ([self.bos_token_id] if add_bos else []) + ids

    def decode(self, ids: Sequence[int]) -> str:
        return bytes(i for i in ids if 0 <= i < 256).decode("utf-8", errors="replace")


class HFTokenizer:
    def __init__(self, path: str):
        from tokenizers import Tokenizer
        tj = path if path.endswith(".json") else os.path.join(path, "tokenizer.json")
        self.tk = Tokenizer.from_file(tj)
        self.vocab_size = self.tk.get_vocab_size()
        self.chat_template, self.bos_token_id, self.eos_token_id = None, None, None
        cfg = os.path.join(os.path.dirname(tj), "tokenizer_config.json")
        if os.path.exists(cfg):
            c = json.load(open(cfg))
            self.chat_template = c.get("chat_template")
            for name in ("bos_token", "eos_token"):
                tok = c.get(name)
                tok = tok.get("content") if isinstance(tok, dict) else tok
                if tok is not None:
                    setattr(self, name + "_id", self.tk.token_to_id(tok))

    def encode(self, text: str, add_bos: bool = False) -> List[int]:
        ids = self.tk.encode(text, add_special_tokens=False).ids
        if add_bos and self.bos_token_id is not None:
            ids = [self.bos_token_id] + ids
        return ids

    def decode(self, ids: Sequence[int]) -> str:
        return self.tk.decode(list(ids), skip_special_tokens=True)


def _bytes_to_unicode() -> Dict[int, str]:
    bs = list(range(33, 127)) + list(range(161, 173)) + list(range(174, 256))
    cs = bs[:]
    n = 0
    for b in range(256):
        if b not in bs:
            bs.append(b)
            cs.append(256 + n)
            n += 1
    return dict(zip(bs, map(chr, cs)))


# pre-tokenizer patterns by ``tokenizer.ggml.pre`` (the families llama.cpp names); anything else uses GPT-2's
_PRE_GPT2 = r"'s|'t|'re|'ve|'m|'ll|'d| ?\p{L}+| ?\p{N}+| ?[^\s\p{L}\p{N}]+|\s+(?!\S)|\s+"
_PRE_LLAMA3 = (r"(?i:'s|'t|'re|'ve|'m|'ll|'d)|[^\r\n\p{L}\p{N}]?\p{L}+|\p{N}{1,3}| ?[^\s\p{L}\p{N}]+[\r\n]*|\s*[\r\n]+|"
               r"\s+(?!\S)|\s+")
_PRE_QWEN2 = (r"(?i:'s|'t|'re|'ve|'m|'ll|'d)|[^\r\n\p{L}\p{N}]?\p{L}+|\p{N}| ?[^\s\p{L}\p{N}]+[\r\n]*|\s*[\r\n]+|"
              r"\s+(?!\S)|\s+")
_PRE_O200K = (r"[^\r\n\p{L}\p{N}]?[\p{Lu}\p{Lt}\p{Lm}\p{Lo}\p{M}]*[\p{Ll}\p{Lm}\p{Lo}\p{M}]+(?i:'s|'t|'re|'ve|'m|'ll|'d)?|"
              r"[^\r\n\p{L}\p{N}]?[\p{Lu}\p{Lt}\p{Lm}\p{Lo}\p{M}]+[\p{Ll}\p{Lm}\p{Lo}\p{M}]*(?i:'s|'t|'re|'ve|'m|'ll|'d)?|"
              r"\p{N}{1,3}| ?[^\s\p{L}\p{N}]+[\r\n/]*|\s*[\r\n]+|\s+(?!\S)|\s+")
PRE_PATTERNS = {"default": _PRE_GPT2, "gpt-2": _PRE_GPT2, "llama-bpe": _PRE_LLAMA3, "llama3": _PRE_LLAMA3, "smaug-bpe": _PRE_LLAMA3,
                "qwen2": _PRE_QWEN2, "deepseek-r1-qwen": _PRE_QWEN2, "gpt-4o": _PRE_O200K, "tekken": _PRE_O200K, "o200k": _PRE_O200K}


def _byte_bpe(parts: List[bytes], ranks: Dict[bytes, int]) -> List[bytes]:
    """Byte-level BPE by rank (lowest rank merges first), as tiktoken files define it."""
    while len(parts) > 1:
        best, bi = None, -1
        for i in range(len(parts) - 1):
            r = ranks.get(parts[i] + parts[i + 1])
            if r is not None and (best is None or r < best):
                best, bi = r, i
        if best is None:
            break
        parts = parts[:bi] + [parts[bi] + parts[bi + 1]] + parts[bi + 2:]
    return parts


def rwkv_unescape(text: str) -> bytes:
    """Bytes of one RWKV "world" vocabulary entry as llama.cpp files store it: the Python ``repr`` of the byte string
    without its quotes (``\\x00``, ``\\n``, ``\\t``, ``\\r``, ``\\\\``, ``\\'``, ``\\"``; everything else stands for itself,
    non-ASCII characters as their UTF-8 bytes)."""
    out = bytearray()
    i, n = 0, len(text)
    simple = {"n": 10, "t": 9, "r": 13, "\\": 92, "'": 39, '"': 34, "a": 7, "b": 8, "f": 12, "v": 11, "0": 0}
    while i < n:
        ch = text[i]
        if ch == "\\" and i + 1 < n:
            nx = text[i + 1]
            hx = text[i + 2:i + 4]
            if nx == "x" and len(hx) == 2 and all(c in "0123456789abcdefABCDEF" for c in hx):
                out.append(int(text[i + 2:i + 4], 16))
                i += 4
                continue
            if nx in simple:
                out.append(simple[nx])
                i += 2
                continue
        out.extend(ch.encode("utf-8"))
        i += 1
    return bytes(out)


class RwkvVocab:
    """The RWKV "world" tokenizer (``tokenizer.ggml.model == "rwkv"``; rust/engine/src/tokenizer_rwkv.rs:1-5): the
    vocabulary is a list of byte strings and a text is cut greedily into the longest entry at every byte position,
    with no pre-tokenisation and no merges. The entries sit in a byte trie stored as flat arrays (first child per
    byte through one dict per node would cost a Python object per node; here a node is a row of ``next`` keyed by
    ``node * 256 + byte``), so a lookup is one dict probe per byte."""

    def __init__(self, escaped: Sequence[str]):
        self.entries: List[bytes] = [rwkv_unescape(t) for t in escaped]
        self.next: Dict[int, int] = {}
        self.terminal: List[int] = [-1]                   # node -> token id, -1 when no entry ends here
        for tid, e in enumerate(self.entries):
            if not e:
                continue
            node = 0
            for b in e:
                key = node * 256 + b
                nx = self.next.get(key)
                if nx is None:
                    nx = len(self.terminal)
                    self.next[key] = nx
                    self.terminal.append(-1)
                node = nx
            if self.terminal[node] < 0:                   # the first of two equal entries keeps the id
                self.terminal[node] = tid

    def encode_bytes(self, data: bytes, unk: int = 0) -> List[int]:
        ids: List[int] = []
        i, n = 0, len(data)
        nxt, term = self.next, self.terminal
        while i < n:
            node, best, best_end = 0, -1, i
            j = i
            while j < n:
                node = nxt.get(node * 256 + data[j])
                if node is None:
                    break
                j += 1
                if term[node] >= 0:
                    best, best_end = term[node], j
            if best < 0:                                  # a byte with no entry: the world vocabulary has all 256
                ids.append(unk)
                i += 1
            else:
                ids.append(best)
                i = best_end
        return ids

    def decode_bytes(self, ids: Sequence[int]) -> bytes:
        return b"".join(self.entries[i] for i in ids if 0 <= i < len(self.entries))


class GgufTokenizer:
    """Vocabulary embedded in a GGUF file (rust/engine/src/tokenizer.rs reads the same keys)."""

    def __init__(self, metadata: dict):
        self.model = metadata.get("tokenizer.ggml.model", "llama")
        self.tokens: List[str] = list(metadata.get("tokenizer.ggml.tokens", []))
        if not self.tokens:
            raise ValueError("the GGUF file embeds no tokenizer")
        self.vocab_size = len(self.tokens)
        self.index = {t: i for i, t in enumerate(self.tokens)}
        self.bos_token_id = metadata.get("tokenizer.ggml.bos_token_id")
        self.eos_token_id = metadata.get("tokenizer.ggml.eos_token_id")
        self.unk_token_id = metadata.get("tokenizer.ggml.unknown_token_id", 0)
        self.chat_template = metadata.get("tokenizer.chat_template")
        self.add_space_prefix = bool(metadata.get("tokenizer.ggml.add_space_prefix", True))
        merges = metadata.get("tokenizer.ggml.merges", [])
        self.ranks = {tuple(m.split(" ", 1)): i for i, m in enumerate(merges)}
        scores = metadata.get("tokenizer.ggml.scores")
        self.scores = [float(x) for x in scores] if scores is not None and len(scores) == len(self.tokens) else None
        types = metadata.get("tokenizer.ggml.token_type")
        self.types = [int(t) for t in types] if types is not None and len(types) == len(self.tokens) else None
        # control (3) and user-defined (4) tokens are matched literally in the text before anything else
        self.special = {t: i for i, t in enumerate(self.tokens)
                        if self.types is not None and self.types[i] in (3, 4) and len(t) > 1}
        self.pre = PRE_PATTERNS.get(str(metadata.get("tokenizer.ggml.pre", "default")), _PRE_GPT2)
        self.b2u = _bytes_to_unicode()
        self.u2b = {v: k for k, v in self.b2u.items()}
        self.max_piece = max((len(t) for t in self.tokens), default=1)
        self._special_re = None
        self.rwkv = RwkvVocab(self.tokens) if self.model == "rwkv" else None
        if self.rwkv is not None:
            self.special = {}                             # the world vocabulary has no control tokens inside text

    # ------------------------------------------------------------------ pieces
    def _bpe(self, word: List[str]) -> List[str]:
        while len(word) > 1:
            best, bi = None, -1
            for i in range(len(word) - 1):
                r = self.ranks.get((word[i], word[i + 1]))
                if r is not None and (best is None or r < best):
                    best, bi = r, i
            if best is None:
                break
            word = word[:bi] + [word[bi] + word[bi + 1]] + word[bi + 2:]
        return word

    def _byte_ids(self, ch: str) -> List[int]:
        return [self.index.get(f"<0x{b:02X}>", self.unk_token_id) for b in ch.encode("utf-8")]

    def _spm_bpe(self, s: str) -> List[int]:
        """SentencePiece BPE: start from characters, always merge the adjacent pair whose concatenation is the
        piece with the highest score (leftmost among equals); characters without a piece fall back to bytes."""
        import heapq
        sym = list(s)
        n = len(sym)
        prev, nxt = list(range(-1, n - 1)), list(range(1, n + 1))
        alive = [True] * n
        heap = []

        def push(i):
            j = nxt[i]
            if j >= n:
                return
            t = self.index.get(sym[i] + sym[j])
            if t is not None:
                heapq.heappush(heap, (-self.scores[t], i, sym[i], sym[j]))
        for i in range(n - 1):
            push(i)
        while heap:
            _, i, a, b = heapq.heappop(heap)
            j = nxt[i] if alive[i] else n
            if not alive[i] or j >= n or not alive[j] or sym[i] != a or sym[j] != b:
                continue                              # stale entry
            sym[i] = a + b
            alive[j] = False
            nxt[i] = nxt[j]
            if nxt[j] < n:
                prev[nxt[j]] = i
            if prev[i] >= 0:
                push(prev[i])
            push(i)
        ids: List[int] = []
        i = 0
        while i < n:
            if alive[i]:
                t = self.index.get(sym[i])
                ids.extend([t] if t is not None else [b for ch in sym[i] for b in self._byte_ids(ch)])
            i += 1
        return ids

    def _unigram(self, s: str) -> List[int]:
        """Viterbi segmentation maximising the sum of the pieces' log-probabilities; unknown characters cost a
        fixed penalty and become bytes (or <unk>)."""
        n = len(s)
        best = [float("-inf")] * (n + 1)
        back = [(0, -1)] * (n + 1)
        best[0] = 0.0
        unk_pen = min(self.scores) - 10.0
        for i in range(n):
            if best[i] == float("-inf"):
                continue
            for L in range(1, min(self.max_piece, n - i) + 1):
                t = self.index.get(s[i:i + L])
                if t is not None and (self.types is None or self.types[t] not in (3,)):
                    sc = best[i] + self.scores[t]
                    if sc > best[i + L]:
                        best[i + L], back[i + L] = sc, (i, t)
            if best[i] + unk_pen > best[i + 1]:
                best[i + 1], back[i + 1] = best[i] + unk_pen, (i, -1)
        out: List[int] = []
        i = n
        while i > 0:
            j, t = back[i]
            out.append(t if t >= 0 else -(i))           # negative: position of an unknown character (end index)
            i = j
        ids: List[int] = []
        for t in reversed(out):
            ids.extend([t] if t >= 0 else self._byte_ids(s[-t - 1]))
        return ids

    def _greedy(self, s: str) -> List[int]:
        ids: List[int] = []
        i = 0
        while i < len(s):
            for n in range(min(self.max_piece, len(s) - i), 0, -1):
                t = self.index.get(s[i:i + n])
                if t is not None:
                    ids.append(t)
                    i += n
                    break
            else:
                ids.extend(self._byte_ids(s[i]))
                i += 1
        return ids

    def _encode_plain(self, text: str) -> List[int]:
        if not text:
            return []
        if self.rwkv is not None:
            return self.rwkv.encode_bytes(text.encode("utf-8"), self.unk_token_id or 0)
        if self.model == "gpt2":
            import regex
            ids: List[int] = []
            for piece in regex.findall(self.pre, text):
                word = [self.b2u[b] for b in piece.encode("utf-8")]
                for tok in self._bpe(word):
                    if tok in self.index:
                        ids.append(self.index[tok])
                    else:
                        ids.extend(self.index.get(ch, self.unk_token_id) for ch in tok)
            return ids
        s = text.replace(" ", "\u2581")
        if self.add_space_prefix and not s.startswith("\u2581"):
            s = "\u2581" + s
        if self.scores is None:
            return self._greedy(s)
        return self._unigram(s) if self.model in ("t5", "unigram") else self._spm_bpe(s)

    # ------------------------------------------------------------------ public
    def encode(self, text: str, add_bos: bool = False) -> List[int]:
        ids: List[int] = [self.bos_token_id] if add_bos and self.bos_token_id is not None else []
        if not self.special:
            return ids + self._encode_plain(text)
        if self._special_re is None:
            import re
            self._special_re = re.compile("|".join(re.escape(t) for t in sorted(self.special, key=len, reverse=True)))
        pos = 0
        for m in self._special_re.finditer(text):
            ids += self._encode_plain(text[pos:m.start()])
            ids.append(self.special[m.group(0)])
            pos = m.end()
        return ids + self._encode_plain(text[pos:])

    def decode(self, ids: Sequence[int], skip_special: bool = True) -> str:
        keep = [i for i in ids if 0 <= i < self.vocab_size and
                not (skip_special and self.types is not None and self.types[i] == 3)]
        if self.rwkv is not None:
            return self.rwkv.decode_bytes(keep).decode("utf-8", errors="replace")
        if self.model == "gpt2":
            raw = "".join(self.tokens[i] for i in keep)
            return bytes(self.u2b.get(ch, 32) for ch in raw).decode("utf-8", errors="replace")
        out = bytearray()
        for i in keep:
            t = self.tokens[i]
            if len(t) == 6 and t.startswith("<0x") and t.endswith(">"):
                out.append(int(t[3:5], 16))
            else:
                out.extend(t.replace("\u2581", " ").encode("utf-8"))
        s = out.decode("utf-8", errors="replace")
        return s[1:] if self.add_space_prefix and s.startswith(" ") else s


class TiktokenTokenizer:
    """A ``*.tiktoken`` vocabulary: one ``base64(token bytes) rank`` pair per line; ids = ranks, special tokens
    follow the ranks. Encoding is byte-level BPE by rank inside the pieces of a pre-tokenizer pattern."""

    def __init__(self, path: str, pattern: str = _PRE_LLAMA3, special_tokens: Optional[List[str]] = None):
        import base64
        self.ranks: Dict[bytes, int] = {}
        for line in open(path, "rb").read().splitlines():
            if line.strip():
                tok, rank = line.split()
                self.ranks[base64.b64decode(tok)] = int(rank)
        self.by_id = {v: k for k, v in self.ranks.items()}
        base = max(self.by_id) + 1 if self.by_id else 0
        self.special = {t: base + i for i, t in enumerate(special_tokens or ["<|begin_of_text|>", "<|end_of_text|>"])}
        self.special_by_id = {v: k for k, v in self.special.items()}
        self.vocab_size = base + len(self.special)
        self.bos_token_id = self.special.get("<|begin_of_text|>")
        self.eos_token_id = self.special.get("<|end_of_text|>")
        self.chat_template = None
        self.pattern = pattern

    def encode(self, text: str, add_bos: bool = False) -> List[int]:
        import re
        import regex
        ids: List[int] = [self.bos_token_id] if add_bos and self.bos_token_id is not None else []
        sp = re.compile("|".join(re.escape(t) for t in sorted(self.special, key=len, reverse=True))) if self.special else None
        pos = 0
        spans = [(m.start(), m.end(), m.group(0)) for m in sp.finditer(text)] if sp else []
        for a, b, tok in spans + [(len(text), len(text), None)]:
            for piece in regex.findall(self.pattern, text[pos:a]):
                raw = piece.encode("utf-8")
                ids.extend(self.ranks[p] for p in _byte_bpe([bytes([c]) for c in raw], self.ranks) if p in self.ranks)
            if tok is not None:
                ids.append(self.special[tok])
            pos = b
        return ids

    def decode(self, ids: Sequence[int]) -> str:
        return b"".join(self.by_id.get(i, b"") for i in ids).decode("utf-8", errors="replace")


def load_tokenizer(path: Optional[str], vocab_size: int):
    if path:
        if path.endswith(".gguf"):
            from .formats.gguf import GgufReader
            r = GgufReader(path)
            try:
                return GgufTokenizer(r.metadata)
            finally:
                r.close()
        if path.endswith(".tiktoken"):
            return TiktokenTokenizer(path)
        return HFTokenizer(path)
    return ByteTokenizer(vocab_size)
