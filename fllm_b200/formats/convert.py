"""Checkpoint tooling: Hugging Face checkpoint -> GGUF (``convert``), re-quantisation of a GGUF
(``quantize``), metadata edits (``gguf-set``), sharding (``gguf-split`` / ``gguf-merge``) and LoRA
merging (``merge-lora``).

Same jobs as the reference's ``fllm-checkpoint`` crate (rust/checkpoint/src/convert.rs:1290
``convert_checkpoint``, requant.rs ``quantize_gguf``, gguf_tools.rs split / merge / set / merge-lora,
tokenizer_import.rs); the tensor names and metadata keys written here are the GGUF conventions of
llama.cpp, so the files load in either engine. Quantisation runs through the native codecs
(``csrc_cpu/quant.cpp``) row by row; a tensor whose row length the requested type cannot tile falls
back to Q8_0, then F16, like ``cpu_engine.write_tiny_llama_gguf`` does. One-dimensional tensors
(norm weights, biases) and the MoE router stay F32.
"""
from __future__ import annotations

import json
import os
import re
from typing import Dict, Iterable, List, Optional, Tuple

import numpy as np
import torch

from . import quant
from .gguf import GGML_TYPES, TYPE_ID, GgufReader, GgufWriter

# Hugging Face module name -> GGUF tensor name (per layer)
_LAYER_MAP = {
    "input_layernorm.weight": "attn_norm.weight", "post_attention_layernorm.weight": "ffn_norm.weight",
    "self_attn.q_proj.weight": "attn_q.weight", "self_attn.k_proj.weight": "attn_k.weight",
    "self_attn.v_proj.weight": "attn_v.weight", "self_attn.o_proj.weight": "attn_output.weight",
    "self_attn.q_proj.bias": "attn_q.bias", "self_attn.k_proj.bias": "attn_k.bias", "self_attn.v_proj.bias": "attn_v.bias",
    "self_attn.o_proj.bias": "attn_output.bias", "self_attn.q_norm.weight": "attn_q_norm.weight",
    "self_attn.k_norm.weight": "attn_k_norm.weight", "mlp.gate_proj.weight": "ffn_gate.weight",
    "mlp.up_proj.weight": "ffn_up.weight", "mlp.down_proj.weight": "ffn_down.weight",
    "pre_feedforward_layernorm.weight": "ffn_norm.weight", "post_feedforward_layernorm.weight": "post_ffw_norm.weight",
    "mlp.gate.weight": "ffn_gate_inp.weight", "block_sparse_moe.gate.weight": "ffn_gate_inp.weight",
}
_TOP_MAP = {"model.embed_tokens.weight": "token_embd.weight", "model.norm.weight": "output_norm.weight",
            "lm_head.weight": "output.weight"}
_ARCH = {"llama": "llama", "mistral": "llama", "qwen2": "qwen2", "qwen3": "qwen3", "gemma": "gemma", "gemma2": "gemma2",
         "phi3": "phi3", "mixtral": "llama", "qwen2_moe": "qwen2moe", "qwen3_moe": "qwen3moe", "gpt_oss": "gpt_oss"}


def gguf_name(hf_name: str) -> Optional[str]:
    if hf_name in _TOP_MAP:
        return _TOP_MAP[hf_name]
    m = re.match(r"model\.layers\.(\d+)\.(.+)$", hf_name)
    if not m:
        return None
    layer, rest = m.group(1), m.group(2)
    if rest in _LAYER_MAP:
        return f"blk.{layer}.{_LAYER_MAP[rest]}"
    e = re.match(r"(?:mlp|block_sparse_moe)\.experts\.(\d+)\.(gate_proj|up_proj|down_proj|w1|w3|w2)\.weight$", rest)
    if e:
        kind = {"gate_proj": "gate", "w1": "gate", "up_proj": "up", "w3": "up", "down_proj": "down", "w2": "down"}[e.group(2)]
        return f"blk.{layer}.ffn_{kind}.{e.group(1)}.weight"
    return None


def pick_type(want: str, shape: Tuple[int, ...], name: str) -> str:
    """The type a tensor is stored in when the file is quantised to `want`."""
    if len(shape) < 2 or name.endswith("ffn_gate_inp.weight") or "norm" in name:
        return "F32"
    if want in ("F32", "F16", "BF16"):
        return want
    cols = shape[-1]
    for t in (want, "Q8_0", "F16"):
        if cols % GGML_TYPES[TYPE_ID[t]][1] == 0:
            return t
    return "F16"


def encode_tensor(x: np.ndarray, type_name: str) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.float32)
    if type_name == "F32":
        return x.view(np.uint8).reshape(-1)
    rows = int(np.prod(x.shape[:-1])) if x.ndim > 1 else 1
    return quant.quantize(x.reshape(rows, x.shape[-1]), quant.TYPE_NAMES[type_name]).reshape(-1)


def _tokenizer_metadata(directory: str, w: GgufWriter, vocab_size: int) -> bool:
    """Copy a ``tokenizer.json`` BPE vocabulary (tokens, merges, special ids) into GGUF metadata."""
    path = os.path.join(directory, "tokenizer.json")
    if not os.path.exists(path):
        return False
    tj = json.load(open(path, encoding="utf-8"))
    model = tj.get("model") or {}
    vocab = model.get("vocab")
    if not isinstance(vocab, dict):
        return False
    tokens = [""] * max(vocab_size, max(vocab.values()) + 1)
    for tok, i in vocab.items():
        tokens[i] = tok
    types = [1] * len(tokens)                     # 1 normal, 3 control
    for a in tj.get("added_tokens") or []:
        if a["id"] >= len(tokens):
            tokens.extend([""] * (a["id"] + 1 - len(tokens)))
            types.extend([1] * (a["id"] + 1 - len(types)))
        tokens[a["id"]] = a["content"]
        types[a["id"]] = 3 if a.get("special") else 4
    merges = [m if isinstance(m, str) else " ".join(m) for m in (model.get("merges") or [])]
    w.add("tokenizer.ggml.model", "gpt2" if model.get("type", "BPE") == "BPE" else "llama")
    w.add("tokenizer.ggml.tokens", tokens)
    w.add("tokenizer.ggml.token_type", np.asarray(types, dtype=np.int32))
    if merges:
        w.add("tokenizer.ggml.merges", merges)
    cfg_path = os.path.join(directory, "tokenizer_config.json")
    if os.path.exists(cfg_path):
        tc = json.load(open(cfg_path, encoding="utf-8"))
        tmpl = tc.get("chat_template")
        if isinstance(tmpl, str):
            w.add("tokenizer.chat_template", tmpl)
        inv = {t: i for i, t in enumerate(tokens)}
        for key, field in (("bos_token", "bos_token_id"), ("eos_token", "eos_token_id"), ("pad_token", "padding_token_id")):
            v = tc.get(key)
            v = v.get("content") if isinstance(v, dict) else v
            if isinstance(v, str) and v in inv:
                w.add(f"tokenizer.ggml.{field}", int(inv[v]))
    return True


def convert_checkpoint(directory: str, out_path: str, out_type: str = "F16") -> dict:
    """Hugging Face directory (config.json + *.safetensors [+ tokenizer.json]) -> one GGUF file."""
    from ..config import ModelConfig
    from .safetensors_io import open_checkpoint
    out_type = out_type.upper()
    if out_type not in quant.TYPE_NAMES:
        raise ValueError(f"unknown output type {out_type!r}; one of {sorted(quant.TYPE_NAMES)}")
    hf = json.load(open(os.path.join(directory, "config.json")))
    cfg = ModelConfig.from_hf_config(hf)
    arch = _ARCH.get(hf.get("model_type", "llama"), "llama")
    ck = open_checkpoint(directory)
    w = GgufWriter(out_path)
    w.add("general.architecture", arch)
    w.add("general.name", str(hf.get("_name_or_path") or os.path.basename(os.path.normpath(directory))))
    w.add("general.file_type", int(TYPE_ID.get(out_type, 1)))
    for k, v in (("block_count", cfg.num_layers), ("embedding_length", cfg.hidden_size), ("attention.head_count", cfg.num_heads),
                 ("attention.head_count_kv", cfg.num_kv_heads), ("attention.key_length", cfg.head_dim),
                 ("attention.value_length", cfg.head_dim), ("feed_forward_length", cfg.moe_intermediate_size if cfg.is_moe else cfg.intermediate_size),
                 ("vocab_size", cfg.vocab_size), ("context_length", cfg.max_position)):
        w.add(f"{arch}.{k}", int(v))
    if cfg.is_moe:
        w.add(f"{arch}.expert_count", int(cfg.num_experts))
        w.add(f"{arch}.expert_used_count", int(cfg.experts_per_token))
    if cfg.sliding_window:
        w.add(f"{arch}.attention.sliding_window", int(cfg.sliding_window))
    w.add(f"{arch}.attention.layer_norm_rms_epsilon", float(cfg.rms_eps))
    w.add(f"{arch}.rope.freq_base", float(cfg.rope_theta))
    w.add("fllm.rope_style", 0 if cfg.rope_style == "neox" else 1)
    w.add("fllm.tie_embeddings", bool(cfg.tie_embeddings))
    if cfg.rotary_dim and cfg.rotary_dim != cfg.head_dim:
        w.add(f"{arch}.rope.dimension_count", int(cfg.rotary_dim))
    rs = cfg.rope_scaling
    if rs.kind in ("linear", "yarn"):            # the keys llama.cpp reads; the YaRN ramp ends and factor under keys of this project
        w.add(f"{arch}.rope.scaling.type", rs.kind)
        w.add(f"{arch}.rope.scaling.factor", float(rs.factor))
        w.add(f"{arch}.rope.scaling.original_context_length", int(rs.original_max_position))
        if rs.kind == "yarn":
            w.add("fllm.rope.yarn_beta_fast", float(rs.beta_fast))
            w.add("fllm.rope.yarn_beta_slow", float(rs.beta_slow))
            w.add("fllm.rope.yarn_truncate", bool(rs.truncate))
            if rs.attn_factor is not None:
                w.add("fllm.rope.yarn_attn_factor", float(rs.attn_factor))
    elif rs.kind in ("llama3", "factors"):       # one divisor per frequency, the tensor llama.cpp calls rope_freqs
        from ..config import RopeScaling, rope_inv_freq as rope_frequencies
        import copy
        plain = copy.copy(cfg)
        plain.rope_scaling = RopeScaling()
        div = np.asarray(rope_frequencies(plain)[0], dtype=np.float64) / np.asarray(rope_frequencies(cfg)[0], dtype=np.float64)
        w.add_tensor("rope_freqs.weight", (len(div),), TYPE_ID["F32"], div.astype(np.float32))
    has_tok = _tokenizer_metadata(directory, w, cfg.vocab_size)
    counts: Dict[str, int] = {}
    skipped: List[str] = []
    for hf_name in sorted(ck):
        f, n = ck[hf_name]
        name = gguf_name(hf_name)
        if name is None:
            skipped.append(hf_name)
            continue
        if name == "output.weight" and cfg.tie_embeddings:
            continue
        t = f.tensor(n)
        if not t.is_floating_point() or t.element_size() < 2:
            raise ValueError(f"{hf_name}: packed checkpoints are loaded directly, not converted (dtype {t.dtype})")
        x = t.float().numpy()
        tname = pick_type(out_type, tuple(x.shape), name)
        w.add_tensor(name, tuple(x.shape), TYPE_ID[tname], encode_tensor(x, tname))
        counts[tname] = counts.get(tname, 0) + 1
    w.write()
    return {"output": out_path, "architecture": arch, "tensors": counts, "skipped": skipped, "tokenizer": has_tok}


def _copy_meta(r: GgufReader, w: GgufWriter, skip: Iterable[str] = ()) -> None:
    skip = set(skip) | {"general.alignment"}
    for k, v in r.metadata.items():
        if k not in skip:
            w.add(k, v, r.value_types.get(k) if hasattr(r, "value_types") else None)


def quantize_gguf(in_path: str, out_path: str, out_type: str) -> dict:
    """Re-encode every 2-D weight of a GGUF in another type (through fp32)."""
    out_type = out_type.upper()
    if out_type not in quant.TYPE_NAMES:
        raise ValueError(f"unknown output type {out_type!r}; one of {sorted(quant.TYPE_NAMES)}")
    r = GgufReader(in_path)
    w = GgufWriter(out_path)
    _copy_meta(r, w, skip=("general.file_type",))
    w.add("general.file_type", int(TYPE_ID.get(out_type, 1)))
    counts: Dict[str, int] = {}
    for name, info in r.tensors.items():
        tname = pick_type(out_type, tuple(info.shape), name)
        if tname == info.type_name:
            w.add_tensor(name, tuple(info.shape), info.ggml_type, r.tensor_bytes(name))
        else:
            w.add_tensor(name, tuple(info.shape), TYPE_ID[tname], encode_tensor(r.tensor_f32(name), tname))
        counts[tname] = counts.get(tname, 0) + 1
    w.write()
    r.close()
    return {"output": out_path, "tensors": counts}


def gguf_set(in_path: str, out_path: str, edits: Dict[str, object], remove: Iterable[str] = ()) -> dict:
    """Copy a GGUF with metadata keys changed / added / removed; tensors are copied byte for byte."""
    r = GgufReader(in_path)
    w = GgufWriter(out_path)
    _copy_meta(r, w, skip=list(edits) + list(remove))
    for k, v in edits.items():
        w.add(k, v)
    for name, info in r.tensors.items():
        w.add_tensor(name, tuple(info.shape), info.ggml_type, r.tensor_bytes(name))
    w.write()
    r.close()
    return {"output": out_path, "set": sorted(edits), "removed": sorted(remove)}


def gguf_split(in_path: str, out_prefix: str, max_tensors: int = 128) -> List[str]:
    """Cut a GGUF into shards ``<prefix>-0000N-of-0000M.gguf`` (llama.cpp's naming): every shard carries
    ``split.no`` / ``split.count`` / ``split.tensors.count``; the first one carries the model's metadata."""
    r = GgufReader(in_path)
    names = list(r.tensors)
    groups = [names[i:i + max_tensors] for i in range(0, len(names), max_tensors)] or [[]]
    outs = []
    for i, grp in enumerate(groups):
        path = f"{out_prefix}-{i + 1:05d}-of-{len(groups):05d}.gguf"
        w = GgufWriter(path)
        if i == 0:
            _copy_meta(r, w, skip=("split.no", "split.count", "split.tensors.count"))
        w.add("split.no", i)
        w.add("split.count", len(groups))
        w.add("split.tensors.count", len(names))
        for n in grp:
            info = r.tensors[n]
            w.add_tensor(n, tuple(info.shape), info.ggml_type, r.tensor_bytes(n))
        w.write()
        outs.append(path)
    r.close()
    return outs


def gguf_merge(first_shard: str, out_path: str) -> dict:
    """Inverse of :func:`gguf_split`: give the first shard, get one file."""
    m = re.match(r"(.*)-(\d{5})-of-(\d{5})\.gguf$", first_shard)
    if not m:
        raise ValueError("shard names look like <prefix>-00001-of-0000N.gguf")
    prefix, count = m.group(1), int(m.group(3))
    w = GgufWriter(out_path)
    total = 0
    readers = []
    for i in range(count):
        r = GgufReader(f"{prefix}-{i + 1:05d}-of-{count:05d}.gguf")
        readers.append(r)
        if int(r.metadata.get("split.no", i)) != i:
            raise ValueError(f"shard {i + 1} does not carry split.no = {i}")
        if i == 0:
            _copy_meta(r, w, skip=("split.no", "split.count", "split.tensors.count"))
        for n, info in r.tensors.items():
            w.add_tensor(n, tuple(info.shape), info.ggml_type, r.tensor_bytes(n))
            total += 1
    want = int(readers[0].metadata.get("split.tensors.count", total))
    if want != total:
        raise ValueError(f"shards hold {total} tensors, the first one announces {want}")
    w.write()
    for r in readers:
        r.close()
    return {"output": out_path, "tensors": total, "shards": count}


def merge_lora_gguf(base_path: str, lora_dir: str, out_path: str, out_type: Optional[str] = None) -> dict:
    """W' = W + (alpha / r) * B @ A for every adapted projection of a PEFT LoRA (``adapter_config.json`` +
    ``adapter_model.safetensors``), written as a new GGUF. The reference merges adapters at load time
    (rust/engine/src/model.rs:207,415) and as a tool (rust/checkpoint/src/gguf_tools.rs)."""
    from .safetensors_io import SafetensorsFile
    acfg = json.load(open(os.path.join(lora_dir, "adapter_config.json")))
    scale = float(acfg.get("lora_alpha", acfg.get("r", 1))) / float(acfg.get("r", 1))
    sf = SafetensorsFile(os.path.join(lora_dir, "adapter_model.safetensors"))
    pairs: Dict[str, Dict[str, torch.Tensor]] = {}
    for key in sf.keys():
        m = re.match(r"(?:base_model\.model\.)?(.*)\.lora_([AB])(?:\.default)?\.weight$", key)
        if m:
            pairs.setdefault(m.group(1) + ".weight", {})[m.group(2)] = sf.tensor(key).float()
    r = GgufReader(base_path)
    w = GgufWriter(out_path)
    _copy_meta(r, w)
    deltas = {}
    for hf_name, ab in pairs.items():
        name = gguf_name(hf_name)
        if name is None or name not in r.tensors or "A" not in ab or "B" not in ab:
            continue
        deltas[name] = (ab["B"] @ ab["A"]) * scale
    merged = 0
    for name, info in r.tensors.items():
        if name in deltas:
            x = r.tensor_f32(name) + deltas[name].numpy().reshape(info.shape)
            tname = pick_type((out_type or info.type_name).upper(), tuple(info.shape), name)
            w.add_tensor(name, tuple(info.shape), TYPE_ID[tname], encode_tensor(x, tname))
            merged += 1
        else:
            w.add_tensor(name, tuple(info.shape), info.ggml_type, r.tensor_bytes(name))
    w.write()
    r.close()
    sf.close()
    return {"output": out_path, "merged": merged, "adapter_tensors": len(pairs), "scale": scale}
