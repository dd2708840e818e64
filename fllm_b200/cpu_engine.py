"""CPU engine for GGUF models with packed weights (batch 1, greedy, paged f16 KV in
16-token blocks) and the writer of the synthetic tiny-Llama GGUF used as the end-to-end
fixture (the reference's ``make-tiny-model`` sub-command). The compute is the native
``csrc_cpu/cpu_engine.cpp``; this file maps GGUF tensors into it without copying."""
from __future__ import annotations

import ctypes
import time
from typing import List, Optional, Sequence

import numpy as np

from .config import ModelConfig, RopeScaling, preset
from .formats import quant
from .formats.gguf import TYPE_ID, GgufReader, GgufWriter
from .ops._lib import load_cpu


class _CpuConfig(ctypes.Structure):
    _fields_ = [(n, ctypes.c_int) for n in ("n_layers", "hidden", "n_heads", "n_kv_heads", "head_dim", "ffn",
                                            "vocab", "block_size", "num_blocks", "rope_style", "tie_embeddings")] + \
               [("eps", ctypes.c_float), ("rope_theta", ctypes.c_float)]


def write_tiny_llama_gguf(path: str, cfg: Optional[ModelConfig] = None, seed: int = 0, qtype: int = quant.Q4_K,
                          qtype_for=None) -> ModelConfig:
    """N(0, 0.02) weights from `seed`, quantised to `qtype`; norm weights f32 = 1. `qtype_for(name)` may name another
    type for single tensors (a Q4_K_M file keeps attn_v and ffn_down in Q6_K)."""
    cfg = cfg or preset("tiny-llama")
    rng = np.random.default_rng(seed)
    w = GgufWriter(path)
    w.add("general.architecture", "llama")
    w.add("general.name", cfg.name)
    for k, v in (("block_count", cfg.num_layers), ("embedding_length", cfg.hidden_size),
                 ("attention.head_count", cfg.num_heads), ("attention.head_count_kv", cfg.num_kv_heads),
                 ("attention.key_length", cfg.head_dim), ("feed_forward_length", cfg.intermediate_size),
                 ("vocab_size", cfg.vocab_size), ("context_length", cfg.max_position)):
        w.add(f"llama.{k}", int(v))
    w.add("llama.attention.layer_norm_rms_epsilon", float(cfg.rms_eps))
    w.add("llama.rope.freq_base", float(cfg.rope_theta))
    w.add("fllm.rope_style", 0 if cfg.rope_style == "neox" else 1)
    w.add("fllm.tie_embeddings", bool(cfg.tie_embeddings))
    tname = {quant.Q4_K: "Q4_K", quant.Q6_K: "Q6_K", quant.Q8_0: "Q8_0", quant.Q5_K: "Q5_K"}[qtype]

    def mat(name, rows, cols):
        x = (rng.standard_normal((rows, cols), dtype=np.float32) * 0.02)
        # rows that the block size does not divide fall back: Q8_0 for multiples of 32, else f16
        # (the 688-wide FFN input of the tiny model is neither a multiple of 256 nor of 32)
        if cols % 256 == 0:
            qt = qtype_for(name) if qtype_for is not None and qtype_for(name) is not None else qtype
            tn = {quant.Q4_K: "Q4_K", quant.Q6_K: "Q6_K", quant.Q8_0: "Q8_0", quant.Q5_K: "Q5_K"}[qt]
        elif cols % 32 == 0:
            qt, tn = quant.Q8_0, "Q8_0"
        else:
            qt, tn = quant.F16, "F16"
        w.add_tensor(name, (rows, cols), TYPE_ID[tn], quant.quantize(x, qt))

    def ones(name, n):
        w.add_tensor(name, (n,), TYPE_ID["F32"], np.ones(n, dtype=np.float32))

    H, D = cfg.hidden_size, cfg.head_dim
    mat("token_embd.weight", cfg.vocab_size, H)
    for l in range(cfg.num_layers):
        p = f"blk.{l}."
        ones(p + "attn_norm.weight", H)
        mat(p + "attn_q.weight", cfg.num_heads * D, H)
        mat(p + "attn_k.weight", cfg.num_kv_heads * D, H)
        mat(p + "attn_v.weight", cfg.num_kv_heads * D, H)
        mat(p + "attn_output.weight", H, cfg.num_heads * D)
        ones(p + "ffn_norm.weight", H)
        mat(p + "ffn_gate.weight", cfg.intermediate_size, H)
        mat(p + "ffn_up.weight", cfg.intermediate_size, H)
        mat(p + "ffn_down.weight", H, cfg.intermediate_size)
    ones("output_norm.weight", H)
    if not cfg.tie_embeddings:
        mat("output.weight", cfg.vocab_size, H)
    w.write()
    return cfg


def config_from_gguf(r: GgufReader) -> ModelConfig:
    m = r.metadata
    arch = m.get("general.architecture", "llama")
    g = lambda k, d=None: m.get(f"{arch}.{k}", d)
    heads = int(g("attention.head_count"))
    hidden = int(g("embedding_length"))
    vocab = g("vocab_size")
    if vocab is None:
        vocab = r.tensors["token_embd.weight"].shape[0]
    head_dim = int(g("attention.key_length", hidden // heads))
    rot = g("rope.dimension_count")
    scaling = RopeScaling()
    kind = g("rope.scaling.type")
    if kind in ("linear", "yarn"):
        scaling = RopeScaling(kind=kind, factor=float(g("rope.scaling.factor", 1.0)),
                              original_max_position=int(g("rope.scaling.original_context_length", g("context_length", 4096))),
                              beta_fast=float(m.get("fllm.rope.yarn_beta_fast", 32.0)), beta_slow=float(m.get("fllm.rope.yarn_beta_slow", 1.0)),
                              truncate=bool(m.get("fllm.rope.yarn_truncate", True)), attn_factor=m.get("fllm.rope.yarn_attn_factor"))
    elif "rope_freqs.weight" in r.tensors:         # one divisor per frequency (Llama-3 style scaling, stored as a tensor)
        scaling = RopeScaling(kind="factors", freq_factors=[float(v) for v in r.tensor_f32("rope_freqs.weight").reshape(-1)])
    return ModelConfig(
        rope_scaling=scaling, rotary_dim=int(rot) if rot is not None and int(rot) != head_dim else None,
        arch="llama" if arch not in ("qwen3", "gpt_oss") else arch, name=str(m.get("general.name", arch)),
        vocab_size=int(vocab), hidden_size=hidden, num_layers=int(g("block_count")), num_heads=heads,
        num_kv_heads=int(g("attention.head_count_kv", heads)), head_dim=int(g("attention.key_length", hidden // heads)),
        intermediate_size=int(g("feed_forward_length")), rms_eps=float(g("attention.layer_norm_rms_epsilon", 1e-5)),
        rope_theta=float(g("rope.freq_base", 10000.0)), max_position=int(g("context_length", 4096)),
        rope_style="neox" if int(m.get("fllm.rope_style", 1 if arch == "llama" else 0)) == 0 else "pair",
        tie_embeddings=bool(m.get("fllm.tie_embeddings", "output.weight" not in r.tensors)),
        qk_norm=(arch == "qwen3"))


class CpuEngine:
    def __init__(self, gguf_path: str, num_blocks: int = 64, block_size: int = 16):
        self.lib = load_cpu()
        self.reader = GgufReader(gguf_path)
        self.cfg = config_from_gguf(self.reader)
        c = self.cfg
        self.block_size, self.num_blocks = block_size, num_blocks
        cc = _CpuConfig(c.num_layers, c.hidden_size, c.num_heads, c.num_kv_heads, c.head_dim, c.intermediate_size,
                        c.vocab_size, block_size, num_blocks, 0 if c.rope_style == "neox" else 1,
                        int(c.tie_embeddings), c.rms_eps, c.rope_theta)
        self.lib.fllm_cpu_create.restype = ctypes.c_void_p
        self.lib.fllm_cpu_set_tensor.argtypes = [ctypes.c_void_p, ctypes.c_char_p, ctypes.c_int, ctypes.c_void_p,
                                                 ctypes.c_int64, ctypes.c_int64]
        self.lib.fllm_cpu_forward.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_int,
                                              ctypes.c_void_p, ctypes.c_void_p]
        self.lib.fllm_cpu_generate.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_int,
                                               ctypes.c_void_p, ctypes.c_void_p]
        self.lib.fllm_cpu_destroy.argtypes = [ctypes.c_void_p]
        self.h = ctypes.c_void_p(self.lib.fllm_cpu_create(ctypes.byref(cc)))
        self._views = []
        for name, t in self.reader.tensors.items():
            view = self.reader.tensor_bytes(name)
            self._views.append(view)
            rows = int(np.prod(t.shape[:-1])) if len(t.shape) > 1 else 1
            if self.lib.fllm_cpu_set_tensor(self.h, name.encode(), t.ggml_type, view.ctypes.data, rows, t.shape[-1]):
                raise ValueError(f"tensor {name}: type {t.type_name} is not supported by the CPU engine")

    def _table(self, n_tokens: int) -> np.ndarray:
        nb = -(-n_tokens // self.block_size)
        if nb > self.num_blocks:
            raise MemoryError("sequence does not fit the CPU KV pool")
        return np.arange(nb, dtype=np.int32)

    def logits(self, tokens: Sequence[int], pos0: int = 0, total: Optional[int] = None) -> np.ndarray:
        toks = np.asarray(tokens, dtype=np.int32)
        table = self._table(total or (pos0 + len(toks)))
        out = np.empty(self.cfg.vocab_size, dtype=np.float32)
        rc = self.lib.fllm_cpu_forward(self.h, toks.ctypes.data, len(toks), pos0, table.ctypes.data, out.ctypes.data)
        if rc:
            raise RuntimeError("cpu forward failed (missing tensor?)")
        return out

    def generate(self, prompt: Sequence[int], n_out: int) -> List[int]:
        toks = np.asarray(prompt, dtype=np.int32)
        table = self._table(len(toks) + n_out)
        out = np.empty(n_out, dtype=np.int32)
        rc = self.lib.fllm_cpu_generate(self.h, toks.ctypes.data, len(toks), n_out, table.ctypes.data, out.ctypes.data)
        if rc < 0:
            raise RuntimeError("cpu generate failed")
        return out.tolist()

    def bench(self, prompt_len: int = 128, n_out: int = 64, seed: int = 0) -> dict:
        rng = np.random.default_rng(seed)
        prompt = rng.integers(0, self.cfg.vocab_size, prompt_len).tolist()
        t0 = time.perf_counter()
        self.logits(prompt)
        t1 = time.perf_counter()
        toks = self.generate(prompt, n_out)
        t2 = time.perf_counter()
        decode_s = (t2 - t1) - (t1 - t0)          # generate() repeats the prompt pass
        return {"prompt_tok_s": prompt_len / (t1 - t0), "decode_tok_s": n_out / max(decode_s, 1e-9), "tokens": toks}

    def close(self) -> None:
        if self.h:
            self.lib.fllm_cpu_destroy(self.h)
            self.h = None
        self._views.clear()
        try:
            self.reader.close()
        except BufferError:
            pass
