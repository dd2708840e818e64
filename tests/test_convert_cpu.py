"""Checkpoint tooling: HF -> GGUF conversion, re-quantisation, metadata edits, split / merge, LoRA merge, and the
block codecs of the remaining GGML types against the fp32 values they encode."""
import json
import os

import numpy as np
import pytest
import torch

from fllm_b200.config import preset
from fllm_b200.formats import quant
from fllm_b200.formats.convert import (convert_checkpoint, gguf_merge, gguf_set, gguf_split, merge_lora_gguf, quantize_gguf)
from fllm_b200.formats.gguf import GgufReader
from fllm_b200.formats.loader import load_gguf, load_hf_checkpoint
from fllm_b200.formats.safetensors_io import save_file
from fllm_b200.models.weights import init_random_weights


def _write_hf(dirpath, cfg, w):
    D, I = cfg.head_dim, cfg.intermediate_size
    nq, nk = cfg.num_heads * D, cfg.num_kv_heads * D
    t = {"model.embed_tokens.weight": w.embed, "model.norm.weight": w.final_norm, "lm_head.weight": w.lm_head}
    for l, lw in enumerate(w.layers):
        p = f"model.layers.{l}."
        t.update({p + "input_layernorm.weight": lw.attn_norm, p + "post_attention_layernorm.weight": lw.ffn_norm,
                  p + "self_attn.q_proj.weight": lw.wqkv[:nq], p + "self_attn.k_proj.weight": lw.wqkv[nq:nq + nk],
                  p + "self_attn.v_proj.weight": lw.wqkv[nq + nk:], p + "self_attn.o_proj.weight": lw.wo,
                  p + "self_attn.q_norm.weight": lw.q_norm, p + "self_attn.k_norm.weight": lw.k_norm,
                  p + "mlp.gate_proj.weight": lw.w_gate_up[:I], p + "mlp.up_proj.weight": lw.w_gate_up[I:],
                  p + "mlp.down_proj.weight": lw.w_down})
    save_file({k: v.contiguous() for k, v in t.items()}, os.path.join(dirpath, "model.safetensors"))
    json.dump({"model_type": "qwen3", "vocab_size": cfg.vocab_size, "hidden_size": cfg.hidden_size,
               "num_hidden_layers": cfg.num_layers, "num_attention_heads": cfg.num_heads, "num_key_value_heads": cfg.num_kv_heads,
               "head_dim": D, "intermediate_size": I, "rms_norm_eps": cfg.rms_eps, "rope_theta": cfg.rope_theta,
               "max_position_embeddings": 4096, "tie_word_embeddings": False}, open(os.path.join(dirpath, "config.json"), "w"))


@pytest.fixture(scope="module")
def hf_dir(tmp_path_factory):
    d = str(tmp_path_factory.mktemp("hf"))
    cfg = preset("qwen3-tiny")
    _write_hf(d, cfg, init_random_weights(cfg, "cpu", seed=5))
    return d, cfg


def test_convert_bf16_reloads_as_the_same_model(hf_dir, tmp_path):
    d, cfg = hf_dir
    out = str(tmp_path / "m.gguf")
    rep = convert_checkpoint(d, out, "BF16")              # the checkpoint is bf16: this conversion is lossless
    assert rep["architecture"] == "qwen3" and rep["skipped"] == [] and rep["tensors"]["BF16"] > 0 and rep["tensors"]["F32"] > 0
    cfg_g, w_g, _ = load_gguf(out, "cpu")
    cfg_h, w_h, _ = load_hf_checkpoint(d, "cpu")
    assert (cfg_g.num_layers, cfg_g.head_dim, cfg_g.qk_norm, cfg_g.rope_style) == (cfg_h.num_layers, cfg_h.head_dim, True, cfg_h.rope_style)
    for a, b in zip(w_g.layers, w_h.layers):
        assert torch.equal(a.wqkv, b.wqkv) and torch.equal(a.w_gate_up, b.w_gate_up) and torch.equal(a.q_norm, b.q_norm)
    assert torch.equal(w_g.lm_head, w_h.lm_head)


@pytest.mark.parametrize("scaling", [
    dict(rope_type="llama3", factor=8.0, low_freq_factor=1.0, high_freq_factor=4.0, original_max_position_embeddings=64),
    dict(rope_type="yarn", factor=32.0, beta_fast=32.0, beta_slow=1.0, truncate=False, original_max_position_embeddings=128),
    dict(rope_type="linear", factor=4.0)])
def test_convert_keeps_the_rope_scaling(hf_dir, tmp_path, scaling):
    """The converted file rotates with the frequencies of the directory it came from: Llama-3 scaling as one divisor
    per frequency (the rope_freqs tensor), linear and YaRN scaling as metadata (with the YaRN ramp's rounding mode)."""
    from fllm_b200.config import rope_inv_freq
    d, _ = hf_dir
    d2 = str(tmp_path / "scaled")
    os.makedirs(d2)
    os.symlink(os.path.join(d, "model.safetensors"), os.path.join(d2, "model.safetensors"))
    hf = json.load(open(os.path.join(d, "config.json")))
    json.dump(dict(hf, rope_scaling=scaling), open(os.path.join(d2, "config.json"), "w"))
    out = str(tmp_path / "scaled.gguf")
    convert_checkpoint(d2, out, "BF16")
    cfg_g, _, _ = load_gguf(out, "cpu")
    cfg_h, _, _ = load_hf_checkpoint(d2, "cpu")
    assert cfg_h.rope_scaling.kind == scaling["rope_type"]
    assert cfg_g.rope_scaling.kind == ("factors" if scaling["rope_type"] == "llama3" else scaling["rope_type"])
    (fg, ag), (fh, ah) = rope_inv_freq(cfg_g), rope_inv_freq(cfg_h)
    assert ag == pytest.approx(ah) and fg == pytest.approx(fh, rel=1e-6)
    assert fh != pytest.approx(rope_inv_freq(load_hf_checkpoint(d, "cpu")[0])[0], rel=1e-3)      # the scaling does something


@pytest.mark.parametrize("qt", ["Q4_K", "Q5_0", "Q3_K", "IQ4_NL"])
def test_convert_quantised_and_requantise(hf_dir, tmp_path, qt):
    d, cfg = hf_dir
    out = str(tmp_path / f"m-{qt}.gguf")
    rep = convert_checkpoint(d, out, qt)
    assert rep["tensors"].get(qt, 0) > 0
    r = GgufReader(out)
    x = r.tensor_f32("blk.0.attn_q.weight")
    ref = load_hf_checkpoint(d, "cpu")[1].layers[0].wqkv[: cfg.num_heads * cfg.head_dim].float().numpy()
    assert np.abs(x - ref).max() < 0.35 * np.abs(ref).max()
    r.close()
    out2 = str(tmp_path / "m-q8.gguf")
    rep2 = quantize_gguf(out, out2, "Q8_0")
    assert rep2["tensors"]["Q8_0"] > 0
    r2 = GgufReader(out2)
    assert r2.tensors["blk.0.attn_q.weight"].type_name == "Q8_0" and r2.metadata["qwen3.block_count"] == cfg.num_layers
    r2.close()


def test_set_split_merge_roundtrip(hf_dir, tmp_path):
    d, cfg = hf_dir
    base = str(tmp_path / "b.gguf")
    convert_checkpoint(d, base, "F16")
    edited = str(tmp_path / "e.gguf")
    gguf_set(base, edited, {"general.name": "renamed", "fllm.note": 7}, remove=["general.file_type"])
    r = GgufReader(edited)
    assert r.metadata["general.name"] == "renamed" and r.metadata["fllm.note"] == 7 and "general.file_type" not in r.metadata
    n_tensors = len(r.tensors)
    r.close()
    shards = gguf_split(edited, str(tmp_path / "s"), max_tensors=7)
    assert len(shards) == -(-n_tensors // 7)
    merged = str(tmp_path / "merged.gguf")
    rep = gguf_merge(shards[0], merged)
    assert rep["tensors"] == n_tensors
    a, b = GgufReader(edited), GgufReader(merged)
    assert list(a.tensors) == list(b.tensors) and b.metadata["general.name"] == "renamed" and "split.no" not in b.metadata
    for n in a.tensors:
        assert bytes(a.tensor_bytes(n)) == bytes(b.tensor_bytes(n))
    a.close(), b.close()


def test_merge_lora(hf_dir, tmp_path):
    d, cfg = hf_dir
    base = str(tmp_path / "b.gguf")
    convert_checkpoint(d, base, "F32")
    lora = tmp_path / "lora"
    lora.mkdir()
    g = torch.Generator().manual_seed(0)
    nq, H, r_ = cfg.num_heads * cfg.head_dim, cfg.hidden_size, 4
    A, B = torch.randn(r_, H, generator=g) * 0.1, torch.randn(nq, r_, generator=g) * 0.1
    save_file({"base_model.model.model.layers.1.self_attn.q_proj.lora_A.weight": A,
               "base_model.model.model.layers.1.self_attn.q_proj.lora_B.weight": B}, str(lora / "adapter_model.safetensors"))
    json.dump({"r": r_, "lora_alpha": 8}, open(lora / "adapter_config.json", "w"))
    out = str(tmp_path / "merged.gguf")
    rep = merge_lora_gguf(base, str(lora), out)
    assert rep["merged"] == 1 and rep["scale"] == 2.0
    a, b = GgufReader(base), GgufReader(out)
    want = a.tensor_f32("blk.1.attn_q.weight") + (2.0 * (B @ A)).numpy()
    assert np.allclose(b.tensor_f32("blk.1.attn_q.weight"), want, atol=1e-6)
    assert bytes(a.tensor_bytes("blk.0.attn_q.weight")) == bytes(b.tensor_bytes("blk.0.attn_q.weight"))
    a.close(), b.close()


@pytest.mark.parametrize("name,tol", [("Q4_1", 0.12), ("Q5_0", 0.08), ("Q5_1", 0.07), ("Q2_K", 0.6), ("Q3_K", 0.3), ("IQ4_NL", 0.15),
                                      ("IQ4_XS", 0.15)])
def test_block_codecs_round_trip(name, tol):
    rng = np.random.default_rng(1)
    x = (rng.standard_normal((6, 768)) * 0.05).astype(np.float32)
    t = quant.TYPE_NAMES[name]
    packed = quant.quantize(x, t)
    assert packed.shape == (6, quant.row_bytes(t, 768))
    y = quant.dequantize(packed, t, 6, 768)
    assert np.sqrt(((y - x) ** 2).mean()) < tol * np.sqrt((x ** 2).mean())
    gguf = pytest.importorskip("gguf")            # bit-exact against the format's own numpy decoder when it is installed
    ref = gguf.quants.dequantize(packed, getattr(gguf.GGMLQuantizationType, name))
    assert np.array_equal(ref.astype(np.float32), y)
