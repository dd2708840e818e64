"""Tokenizers and chat templates.

* ``HFTokenizer``    a ``tokenizer.json`` (Hugging Face ``tokenizers``), with the chat template and
                     special tokens of ``tokenizer_config.json`` when present;
* ``GgufTokenizer``  the vocabulary embedded in a GGUF file (``tokenizer.ggml.*``): byte-level BPE
                     with merges, or a greedy longest-match over the SentencePiece-style vocabulary;
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


class GgufTokenizer:
    """Vocabulary embedded in a GGUF file. ``gpt2`` models use byte-level BPE with the stored
    merges; other models use greedy longest-match over the piece table with byte fallback."""

    def __init__(self, metadata: dict):
        self.model = metadata.get("tokenizer.ggml.model", "llama")
        self.tokens: List[str] = list(metadata.get("tokenizer.ggml.tokens", []))
        if not self.tokens:
            raise ValueError("the GGUF file embeds no tokenizer")
        self.vocab_size = len(self.tokens)
        self.index = {t: i for i, t in enumerate(self.tokens)}
        self.bos_token_id = metadata.get("tokenizer.ggml.bos_token_id")
        self.eos_token_id = metadata.get("tokenizer.ggml.eos_token_id")
        self.chat_template = metadata.get("tokenizer.chat_template")
        merges = metadata.get("tokenizer.ggml.merges", [])
        self.ranks = {tuple(m.split(" ", 1)): i for i, m in enumerate(merges)}
        self.b2u = _bytes_to_unicode()
        self.u2b = {v: k for k, v in self.b2u.items()}
        self.max_piece = max((len(t) for t in self.tokens), default=1)

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

    def encode(self, text: str, add_bos: bool = False) -> List[int]:
        ids: List[int] = [self.bos_token_id] if add_bos and self.bos_token_id is not None else []
        if self.model == "gpt2":
            import regex
            pat = regex.compile(r"'s|'t|'re|'ve|'m|'ll|'d| ?\p{L}+| ?\p{N}+| ?[^\s\p{L}\p{N}]+|\s+(?!\S)|\s+")
            for piece in pat.findall(text):
                word = [self.b2u[b] for b in piece.encode("utf-8")]
                for tok in self._bpe(word):
                    if tok in self.index:
                        ids.append(self.index[tok])
                    else:
                        ids.extend(self.index.get(ch, 0) for ch in tok)
            return ids
        s = text.replace(" ", "▁")
        if not s.startswith("▁"):
            s = "▁" + s
        i = 0
        while i < len(s):
            for n in range(min(self.max_piece, len(s) - i), 0, -1):
                t = self.index.get(s[i:i + n])
                if t is not None:
                    ids.append(t)
                    i += n
                    break
            else:
                for b in s[i].encode("utf-8"):
                    ids.append(self.index.get(f"<0x{b:02X}>", 0))
                i += 1
        return ids

    def decode(self, ids: Sequence[int]) -> str:
        if self.model == "gpt2":
            raw = "".join(self.tokens[i] for i in ids if 0 <= i < self.vocab_size)
            return bytes(self.u2b.get(ch, 32) for ch in raw).decode("utf-8", errors="replace")
        out = bytearray()
        for i in ids:
            if not 0 <= i < self.vocab_size:
                continue
            t = self.tokens[i]
            if len(t) == 6 and t.startswith("<0x") and t.endswith(">"):
                out.append(int(t[3:5], 16))
            else:
                out.extend(t.replace("▁", " ").encode("utf-8"))
        s = out.decode("utf-8", errors="replace")
        return s[1:] if s.startswith(" ") else s


def load_tokenizer(path: Optional[str], vocab_size: int):
    if path:
        if path.endswith(".gguf"):
            from .formats.gguf import GgufReader
            r = GgufReader(path)
            try:
                return GgufTokenizer(r.metadata)
            finally:
                r.close()
        return HFTokenizer(path)
    return ByteTokenizer(vocab_size)
