"""GGUF-embedded tokenizers against their reference implementations: SentencePiece BPE and unigram models trained
on the spot and re-expressed as GGUF metadata must segment text exactly like ``sentencepiece`` does; byte-level BPE
with special tokens; tiktoken rank files."""
import base64
import io
import os

import pytest

from fllm_b200.tokenizer import GgufTokenizer, TiktokenTokenizer, load_tokenizer

CORPUS = ["the quick brown fox jumps over the lazy dog", "hello world, hello tokenizer", "pack my box with five dozen liquor jugs",
          "tensor cores multiply matrices quickly", "a paged key value cache holds the attention state",
          "low latency decoding needs fused kernels", "the scheduler batches requests continuously"] * 20
# (no runs of spaces: sentencepiece's default normaliser collapses them, a GGUF vocabulary carries no normaliser)
SENTENCES = ["hello world", "the quick tensor fox", "paged attention kernels!", "unseen wörds and 123 numbers", " leading space",
             "a scheduler for continuous batching"]


def _spm_to_metadata(sp, model_name):
    n = sp.get_piece_size()
    toks, scores, types = [], [], []
    for i in range(n):
        toks.append(sp.id_to_piece(i))
        scores.append(sp.get_score(i))
        types.append(2 if sp.is_unknown(i) else 3 if sp.is_control(i) else 6 if sp.is_byte(i) else 1)
    return {"tokenizer.ggml.model": model_name, "tokenizer.ggml.tokens": toks, "tokenizer.ggml.scores": scores,
            "tokenizer.ggml.token_type": types, "tokenizer.ggml.bos_token_id": sp.bos_id(), "tokenizer.ggml.eos_token_id": sp.eos_id(),
            "tokenizer.ggml.unknown_token_id": sp.unk_id()}


@pytest.mark.parametrize("kind,gguf_model", [("bpe", "llama"), ("unigram", "t5")])
def test_sentencepiece_models_segment_identically(kind, gguf_model):
    spm = pytest.importorskip("sentencepiece")
    model = io.BytesIO()
    spm.SentencePieceTrainer.train(sentence_iterator=iter(CORPUS), model_writer=model, vocab_size=400, model_type=kind,
                                   byte_fallback=True, character_coverage=1.0, minloglevel=2, hard_vocab_limit=False)
    sp = spm.SentencePieceProcessor(model_proto=model.getvalue())
    tk = GgufTokenizer(_spm_to_metadata(sp, gguf_model))
    for s in SENTENCES:
        want = sp.encode(s)
        assert tk.encode(s) == want, (s, [sp.id_to_piece(i) for i in want], [tk.tokens[i] for i in tk.encode(s)])
        assert tk.decode(want) == sp.decode(want)
    assert tk.encode("hello", add_bos=True)[0] == sp.bos_id()


def test_byte_level_bpe_with_special_tokens_and_family_pattern():
    from fllm_b200.tokenizer import _bytes_to_unicode
    b2u = _bytes_to_unicode()
    vocab = [b2u[b] for b in range(256)] + ["he", "ll", "hell", "hello", "Ġw", "<|im_start|>", "<|im_end|>"]
    md = {"tokenizer.ggml.model": "gpt2", "tokenizer.ggml.tokens": vocab, "tokenizer.ggml.merges": ["h e", "l l", "he ll", "hell o", "Ġ w"],
          "tokenizer.ggml.token_type": [1] * 261 + [3, 3], "tokenizer.ggml.pre": "qwen2", "tokenizer.ggml.eos_token_id": 262}
    tk = GgufTokenizer(md)
    ids = tk.encode("<|im_start|>hello world 12<|im_end|>")
    assert ids[0] == 261 and ids[-1] == 262 and vocab[ids[1]] == "hello"
    assert [vocab[i] for i in ids[-3:-1]] == ["1", "2"]               # qwen2 splits digits one by one
    assert tk.decode(ids) == "hello world 12" and tk.decode(ids, skip_special=False).startswith("<|im_start|>")
    md["tokenizer.ggml.pre"] = "llama-bpe"
    assert len(GgufTokenizer(md).encode("1234")) == 4                  # no merges for digits here, but one piece of three + one
    assert GgufTokenizer(md).decode(GgufTokenizer(md).encode("naïve café")) == "naïve café"


def test_tiktoken_rank_file(tmp_path):
    rows = [bytes([b]) for b in range(256)] + [b"he", b"ll", b"hell", b"hello", b" w", b" wo", b" wor", b" worl", b" world"]
    p = tmp_path / "v.tiktoken"
    p.write_bytes(b"\n".join(base64.b64encode(t) + b" " + str(i).encode() for i, t in enumerate(rows)))
    tk = load_tokenizer(str(p), 0)
    assert isinstance(tk, TiktokenTokenizer) and tk.vocab_size == len(rows) + 2
    ids = tk.encode("<|begin_of_text|>hello world")
    assert ids == [tk.bos_token_id, 259, 264] and tk.decode(ids) == "hello world"
    tiktoken = pytest.importorskip("tiktoken")
    enc = tiktoken.Encoding("t", pat_str=tk.pattern, mergeable_ranks=tk.ranks, special_tokens=tk.special)
    for s in ("hello world hello", "say hello, world!", "héllo wörld"):
        assert tk.encode(s) == enc.encode(s)


def test_rwkv_world_vocabulary_greedy_longest_match():
    """Entries are Python byte reprs; encoding takes the longest entry at each byte position; every byte has an
    entry, so any text round-trips (rust/engine/src/tokenizer_rwkv.rs:134-155 checks the same two properties)."""
    from fllm_b200.tokenizer import GgufTokenizer, rwkv_unescape
    assert rwkv_unescape(r"\x00") == b"\x00" and rwkv_unescape(r"\n") == b"\n" and rwkv_unescape(r"\\") == b"\\"
    assert rwkv_unescape(r"\'") == b"'" and rwkv_unescape(r"\xc3\xbc") == "ü".encode() and rwkv_unescape("a b") == b"a b"

    def esc(b: bytes) -> str:
        return repr(b)[2:-1]
    single = [bytes([i]) for i in range(256)]
    words = [b"he", b"hello", b"hell", b" world", b" wor", "ü".encode(), "üb".encode(), b"\n\n", b"it's"]
    tokens = ["<eot>"] + [esc(b) for b in single] + [esc(w) for w in words]
    tok = GgufTokenizer({"tokenizer.ggml.model": "rwkv", "tokenizer.ggml.tokens": tokens})
    ids = tok.encode("hello world")
    assert ids == [1 + 256 + 1, 1 + 256 + 3]
    assert tok.encode("hellx") == [1 + 256 + 2, 1 + ord("x")]
    assert tok.encode("über") == [1 + 256 + 6, 1 + ord("e"), 1 + ord("r")]
    assert tok.encode("it's\n\n") == [1 + 256 + 8, 1 + 256 + 7]
    for text in ["hello world", "über\n\nhell", "日本語 ok", "it's \\ fine"]:
        assert tok.decode(tok.encode(text)) == text
