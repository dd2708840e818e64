"""GGUF round trip, packed codecs and the CPU engine on the synthetic tiny-Llama Q4_K file."""
import os

import numpy as np
import pytest
import torch

from fllm_b200.formats import quant
from fllm_b200.formats.gguf import GgufError, GgufReader, GgufWriter, TYPE_ID


@pytest.mark.parametrize("qt,tol", [(quant.Q4_K, 0.09), (quant.Q5_K, 0.05), (quant.Q6_K, 0.025), (quant.Q8_0, 0.006),
                                    (quant.Q4_0, 0.12), (quant.MXFP4, 0.2), (quant.NVFP4, 0.15),
                                    (quant.BF16, 0.005), (quant.F16, 0.001), (quant.FP8_E4M3, 0.04)])
def test_codec_round_trip_error(qt, tol):
    rng = np.random.default_rng(0)
    x = rng.standard_normal((7, 512), dtype=np.float32) * 0.02
    y = quant.dequantize(quant.quantize(x, qt), qt, 7, 512)
    rel = np.linalg.norm(x - y) / np.linalg.norm(x)
    assert rel < tol, rel


def test_q4k_layout_matches_spec():
    """One hand-built block: d=1, dmin=0, scales all 1 -> values equal the 4-bit codes."""
    blk = bytearray(144)
    blk[0:2] = np.float16(1.0).tobytes()
    blk[2:4] = np.float16(0.0).tobytes()
    sc = [1] * 8
    mn = [0] * 8
    packed = bytearray(12)
    for j in range(4):
        packed[j] = sc[j]
        packed[j + 4] = mn[j]
    for j in range(4, 8):
        packed[j + 4] = (sc[j] & 0xF) | ((mn[j] & 0xF) << 4)
    blk[4:16] = packed
    codes = np.arange(256) % 16
    for j in range(4):
        for l in range(32):
            blk[16 + 32 * j + l] = int(codes[64 * j + l]) | (int(codes[64 * j + 32 + l]) << 4)
    y = quant.dequantize(np.frombuffer(bytes(blk), dtype=np.uint8), quant.Q4_K, 1, 256)
    assert np.array_equal(y[0], codes.astype(np.float32))


def test_e4m3_and_e2m1_are_exact_on_representable_values():
    vals = np.array([[0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0, -0.5, -6.0, 448.0, -448.0, 0.015625, 2.0 ** -9, 240.0, 1.75]],
                    dtype=np.float32)
    y = quant.dequantize(quant.quantize(vals, quant.FP8_E4M3), quant.FP8_E4M3, 1, 16)
    assert np.array_equal(y, vals)


def test_gguf_round_trip(tmp_path):
    p = str(tmp_path / "t.gguf")
    w = GgufWriter(p)
    w.add("general.architecture", "llama")
    w.add("llama.block_count", 2)
    w.add("x.f", 1.5)
    w.add("x.s", ["a", "bc"])
    w.add("x.arr", np.arange(5, dtype=np.int32))
    a = np.random.default_rng(1).standard_normal((4, 256), dtype=np.float32)
    w.add_tensor("a.weight", (4, 256), TYPE_ID["Q4_K"], quant.quantize(a, quant.Q4_K))
    w.add_tensor("b", (3,), TYPE_ID["F32"], np.array([1, 2, 3], dtype=np.float32))
    w.write()
    r = GgufReader(p)
    assert r.metadata["llama.block_count"] == 2 and r.metadata["x.s"] == ["a", "bc"]
    assert list(r.metadata["x.arr"]) == [0, 1, 2, 3, 4]
    assert r.tensors["a.weight"].shape == (4, 256) and r.tensors["a.weight"].type_name == "Q4_K"
    assert np.array_equal(r.tensor_bytes("a.weight"), quant.quantize(a, quant.Q4_K).reshape(-1))
    assert np.allclose(r.tensor_f32("b"), [1, 2, 3])
    for t in r.tensors.values():
        assert t.offset % 32 == 0


def test_gguf_rejects_garbage(tmp_path):
    p = tmp_path / "bad.gguf"
    p.write_bytes(b"GGUF" + b"\x03\0\0\0" + b"\xff" * 40)
    with pytest.raises(GgufError):
        GgufReader(str(p))
    p.write_bytes(b"NOPE")
    with pytest.raises(GgufError):
        GgufReader(str(p))


def test_cpu_engine_tiny_llama(tmp_path):
    """The Q4_K CPU engine is bit-stable and agrees with a float decoder on dequantised weights."""
    from fllm_b200.config import preset
    from fllm_b200.cpu_engine import CpuEngine, write_tiny_llama_gguf
    cfg = preset("tiny-llama")
    cfg.vocab_size = 2048
    path = str(tmp_path / "tiny.gguf")
    write_tiny_llama_gguf(path, cfg, seed=0)
    eng = CpuEngine(path)
    rng = np.random.default_rng(0)
    prompt = rng.integers(0, cfg.vocab_size, 40).tolist()
    a = eng.generate(prompt, 16)
    b = eng.generate(prompt, 16)
    assert a == b and len(a) == 16
    # logits vs a dense float forward over the dequantised tensors
    from fllm_b200.models.weights import DecoderWeights, LayerWeights
    from oracle import dense_forward
    r = eng.reader
    f = lambda n: torch.from_numpy(r.tensor_f32(n).copy())
    layers = []
    for l in range(cfg.num_layers):
        pre = f"blk.{l}."
        layers.append(LayerWeights(
            attn_norm=f(pre + "attn_norm.weight"),
            wqkv=torch.cat([f(pre + "attn_q.weight"), f(pre + "attn_k.weight"), f(pre + "attn_v.weight")], 0),
            wo=f(pre + "attn_output.weight"), ffn_norm=f(pre + "ffn_norm.weight"),
            w_gate_up=torch.cat([f(pre + "ffn_gate.weight"), f(pre + "ffn_up.weight")], 0),
            w_down=f(pre + "ffn_down.weight")))
    emb = f("token_embd.weight")
    w = DecoderWeights(embed=emb, layers=layers, final_norm=f("output_norm.weight"), lm_head=emb)
    want = dense_forward(cfg, w, prompt, round_bf16=False)[-1].numpy()
    got = eng.logits(prompt)
    err = np.abs(got - want).max()
    assert err < 0.05 * np.abs(want).max() + 1e-3, err
    eng.close()


def test_safetensors_round_trip_and_hf_loader(tmp_path):
    """A tiny HF-style checkpoint (config.json + safetensors) loads into the engine's fused layout,
    cut for tensor parallelism, and generates the same text as the dense oracle."""
    import json
    from fllm_b200.config import EngineConfig, preset
    from fllm_b200.formats.loader import load_model
    from fllm_b200.formats.safetensors_io import SafetensorsError, SafetensorsFile, save_file
    from fllm_b200.models.weights import init_random_weights
    from fllm_b200.runtime import LLMEngine, SamplingParams
    from oracle import greedy_generate
    cfg = preset("qwen3-tiny")
    w = init_random_weights(cfg, "cpu", seed=5)
    D, H, I = cfg.head_dim, cfg.hidden_size, cfg.intermediate_size
    tensors = {"model.embed_tokens.weight": w.embed, "model.norm.weight": w.final_norm, "lm_head.weight": w.lm_head}
    for l, lw in enumerate(w.layers):
        p = f"model.layers.{l}."
        q, k, v = lw.wqkv.split([cfg.q_size, cfg.kv_size, cfg.kv_size])
        tensors.update({p + "self_attn.q_proj.weight": q, p + "self_attn.k_proj.weight": k, p + "self_attn.v_proj.weight": v,
                        p + "self_attn.o_proj.weight": lw.wo, p + "self_attn.q_norm.weight": lw.q_norm,
                        p + "self_attn.k_norm.weight": lw.k_norm, p + "mlp.gate_proj.weight": lw.w_gate_up[:I],
                        p + "mlp.up_proj.weight": lw.w_gate_up[I:], p + "mlp.down_proj.weight": lw.w_down,
                        p + "input_layernorm.weight": lw.attn_norm, p + "post_attention_layernorm.weight": lw.ffn_norm})
    d = tmp_path / "ckpt"
    d.mkdir()
    save_file(tensors, str(d / "model.safetensors"), {"format": "pt"})
    json.dump({"model_type": "qwen3", "vocab_size": cfg.vocab_size, "hidden_size": H, "num_hidden_layers": cfg.num_layers,
               "num_attention_heads": cfg.num_heads, "num_key_value_heads": cfg.num_kv_heads, "head_dim": D,
               "intermediate_size": I, "rms_norm_eps": cfg.rms_eps, "rope_theta": cfg.rope_theta,
               "max_position_embeddings": 4096, "tie_word_embeddings": False}, open(d / "config.json", "w"))
    f = SafetensorsFile(str(d / "model.safetensors"))
    assert torch.equal(f.tensor("model.norm.weight"), w.final_norm) and f.meta["format"] == "pt"
    cfg2, w2, tok = load_model(str(d), "cpu")
    assert cfg2.qk_norm and cfg2.num_kv_heads == cfg.num_kv_heads and tok is None
    assert torch.equal(w2.layers[1].wqkv, w.layers[1].wqkv) and torch.equal(w2.layers[0].w_gate_up, w.layers[0].w_gate_up)
    _, half, _ = load_model(str(d), "cpu", tp=2, tp_rank=1)
    ref_half = init_random_weights(cfg, "cpu", seed=5, tp=2, tp_rank=1)
    assert torch.equal(half.layers[0].wqkv, ref_half.layers[0].wqkv) and torch.equal(half.layers[0].w_down, ref_half.layers[0].w_down)
    assert torch.equal(half.lm_head, ref_half.lm_head)
    eng = LLMEngine(cfg2, EngineConfig(max_num_batched_tokens=64, max_model_len=128, num_kv_blocks=32), device="cpu", weights=w2)
    prompt = list(range(3, 30))
    assert eng.generate([prompt], SamplingParams(max_tokens=5))[0] == greedy_generate(cfg, w, prompt, 5)
    bad = tmp_path / "bad.safetensors"
    bad.write_bytes(b"\xff" * 16)
    with pytest.raises(SafetensorsError):
        SafetensorsFile(str(bad))


def test_gguf_loader_feeds_the_torch_engine(tmp_path):
    """The same GGUF file drives the packed CPU engine and (expanded to bf16) the torch engine."""
    from fllm_b200.config import EngineConfig, preset
    from fllm_b200.cpu_engine import CpuEngine, write_tiny_llama_gguf
    from fllm_b200.formats.loader import load_model
    from fllm_b200.runtime import LLMEngine, SamplingParams
    cfg = preset("tiny-llama")
    cfg.vocab_size = 1024
    path = str(tmp_path / "t.gguf")
    write_tiny_llama_gguf(path, cfg, seed=2)
    cfg2, w, tok = load_model(path, "cpu")
    assert cfg2.hidden_size == 256 and w.layers[0].wqkv.shape == (cfg.q_size + 2 * cfg.kv_size, 256)
    eng = LLMEngine(cfg2, EngineConfig(max_num_batched_tokens=64, max_model_len=128, num_kv_blocks=32), device="cpu", weights=w)
    prompt = list(range(5, 40))
    a = eng.generate([prompt], SamplingParams(max_tokens=6))[0]
    c = CpuEngine(path)
    b = c.generate(prompt, 6)
    c.close()
    assert sum(x == y for x, y in zip(a, b)) >= 4       # int8-activation dots vs bf16 math: near ties may flip


def write_gpt_oss_checkpoint(tmp_path, cfg, w):
    """Writes `w` (full, single-rank weights of a gpt-oss style config) as a Hugging Face directory whose
    experts are MXFP4 `_blocks` / `_scales`; returns the de-quantised gate_up stacks per layer."""
    import json
    import torch
    from fllm_b200.formats.safetensors_io import save_file
    from fllm_b200.ops.fp4 import MXFP4, dequantize_fp4, quantize_mxfp4
    D, hq, hkv, H, I, E = cfg.head_dim, cfg.num_heads, cfg.num_kv_heads, cfg.hidden_size, cfg.moe_intermediate_size, cfg.num_experts
    t = {"model.embed_tokens.weight": w.embed, "model.norm.weight": w.final_norm, "lm_head.weight": w.lm_head}
    want_gu = []
    for l, lw in enumerate(w.layers):
        p = f"model.layers.{l}."
        q, k, v = lw.wqkv[: hq * D], lw.wqkv[hq * D: (hq + hkv) * D], lw.wqkv[(hq + hkv) * D:]
        bq, bk, bv = lw.bqkv[: hq * D], lw.bqkv[hq * D: (hq + hkv) * D], lw.bqkv[(hq + hkv) * D:]
        t.update({p + "input_layernorm.weight": lw.attn_norm, p + "post_attention_layernorm.weight": lw.ffn_norm,
                  p + "self_attn.q_proj.weight": q, p + "self_attn.k_proj.weight": k, p + "self_attn.v_proj.weight": v,
                  p + "self_attn.q_proj.bias": bq, p + "self_attn.k_proj.bias": bk, p + "self_attn.v_proj.bias": bv,
                  p + "self_attn.o_proj.weight": lw.wo, p + "self_attn.o_proj.bias": lw.bo,
                  p + "self_attn.sinks": lw.sinks.to(torch.bfloat16),
                  p + "mlp.router.weight": lw.router_w, p + "mlp.router.bias": lw.router_b,
                  p + "mlp.experts.gate_up_proj_bias": lw.exp_gate_up_b, p + "mlp.experts.down_proj_bias": lw.exp_down_b})
        for name, stack in (("gate_up_proj", lw.exp_gate_up), ("down_proj", lw.exp_down)):
            Ee, R, K = stack.shape
            codes, scales, _ = quantize_mxfp4(stack.reshape(Ee * R, K).float())
            t[p + f"mlp.experts.{name}_blocks"] = codes.view(Ee, R, K // 32, 16)
            t[p + f"mlp.experts.{name}_scales"] = scales.view(Ee, R, K // 32)
            if name == "gate_up_proj":
                want_gu.append(dequantize_fp4(codes, scales, MXFP4).view(Ee, R, K).to(torch.bfloat16))
    save_file({k: v.contiguous().cpu() for k, v in t.items()}, str(tmp_path / "model.safetensors"))
    hf = {"model_type": "gpt_oss", "vocab_size": cfg.vocab_size, "hidden_size": H, "num_hidden_layers": cfg.num_layers,
          "num_attention_heads": hq, "num_key_value_heads": hkv, "head_dim": D, "intermediate_size": I,
          "rms_norm_eps": cfg.rms_eps, "rope_theta": cfg.rope_theta, "max_position_embeddings": cfg.max_position,
          "num_local_experts": E, "num_experts_per_tok": cfg.experts_per_token, "sliding_window": 128,
          "layer_types": ["sliding_attention", "full_attention"], "attention_bias": True,
          "rope_scaling": {"rope_type": "yarn", "factor": 32.0, "beta_fast": 32.0, "beta_slow": 1.0,
                           "original_max_position_embeddings": 4096}}
    json.dump(hf, open(tmp_path / "config.json", "w"))
    return want_gu


def test_gpt_oss_checkpoint_with_mxfp4_experts_loads(tmp_path):
    """A synthetic gpt-oss style HF checkpoint (router, sinks, biases, experts as MXFP4 `_blocks` /
    `_scales`) loads into the decoder layout: dense tensors bit-equal, experts equal to the MXFP4
    de-quantisation of what was written, and the model runs."""
    import torch
    from fllm_b200.config import EngineConfig, preset
    from fllm_b200.formats.loader import load_hf_checkpoint
    from fllm_b200.models.weights import init_random_weights
    from fllm_b200.runtime import LLMEngine, SamplingParams
    cfg = preset("gpt-oss-tiny")
    w = init_random_weights(cfg, device="cpu", seed=4)
    E = cfg.num_experts
    want_gu = write_gpt_oss_checkpoint(tmp_path, cfg, w)
    cfg2, w2, _ = load_hf_checkpoint(str(tmp_path), device="cpu")
    assert cfg2.is_moe and cfg2.num_experts == E and cfg2.act == "swiglu_oai"
    for l in range(cfg.num_layers):
        a, b = w.layers[l], w2.layers[l]
        assert torch.equal(a.wqkv, b.wqkv) and torch.equal(a.wo, b.wo) and torch.equal(a.bqkv, b.bqkv)
        assert torch.equal(a.router_w, b.router_w) and torch.equal(a.exp_down_b, b.exp_down_b)
        assert torch.allclose(a.sinks, b.sinks, atol=1e-2)
        assert torch.equal(b.exp_gate_up, want_gu[l])
        assert ((b.exp_down.float() - a.exp_down.float()).norm() / a.exp_down.float().norm()).item() < 0.2
    eng = LLMEngine(cfg2, EngineConfig(max_num_seqs=2, max_num_batched_tokens=32, max_model_len=64, num_kv_blocks=16),
                    device="cpu", weights=w2)
    out = eng.generate([[5, 6, 7, 8, 9]], SamplingParams(max_tokens=4))
    assert len(out[0]) == 4


def _write_llama_like(tmp_path, cfg, w, hf_extra, moe_style=None):
    """HF-style directory for a llama-like (optionally per-expert MoE) model from single-rank weights."""
    import json
    from fllm_b200.formats.safetensors_io import save_file
    D, hq, hkv, H = cfg.head_dim, cfg.num_heads, cfg.num_kv_heads, cfg.hidden_size
    t = {"model.embed_tokens.weight": w.embed, "model.norm.weight": w.final_norm}
    if not cfg.tie_embeddings:
        t["lm_head.weight"] = w.lm_head
    for l, lw in enumerate(w.layers):
        p = f"model.layers.{l}."
        t.update({p + "input_layernorm.weight": lw.attn_norm, p + "post_attention_layernorm.weight": lw.ffn_norm,
                  p + "self_attn.q_proj.weight": lw.wqkv[: hq * D], p + "self_attn.k_proj.weight": lw.wqkv[hq * D: (hq + hkv) * D],
                  p + "self_attn.v_proj.weight": lw.wqkv[(hq + hkv) * D:], p + "self_attn.o_proj.weight": lw.wo})
        if cfg.attn_bias:
            t.update({p + "self_attn.q_proj.bias": lw.bqkv[: hq * D], p + "self_attn.k_proj.bias": lw.bqkv[hq * D: (hq + hkv) * D],
                      p + "self_attn.v_proj.bias": lw.bqkv[(hq + hkv) * D:]})
        if cfg.qk_norm:
            t.update({p + "self_attn.q_norm.weight": lw.q_norm, p + "self_attn.k_norm.weight": lw.k_norm})
        if moe_style:
            I = cfg.moe_intermediate_size
            base, names, router = ((p + "block_sparse_moe.", ("w1", "w3", "w2"), "block_sparse_moe.gate.weight") if moe_style == "mixtral"
                                   else (p + "mlp.", ("gate_proj", "up_proj", "down_proj"), "mlp.gate.weight"))
            t[p + router] = lw.router_w
            for e in range(cfg.num_experts):
                t[f"{base}experts.{e}.{names[0]}.weight"] = lw.exp_gate_up[e, :I]
                t[f"{base}experts.{e}.{names[1]}.weight"] = lw.exp_gate_up[e, I:]
                t[f"{base}experts.{e}.{names[2]}.weight"] = lw.exp_down[e]
        else:
            I = cfg.intermediate_size
            t.update({p + "mlp.gate_proj.weight": lw.w_gate_up[:I], p + "mlp.up_proj.weight": lw.w_gate_up[I:],
                      p + "mlp.down_proj.weight": lw.w_down})
    save_file({k: v.contiguous() for k, v in t.items()}, str(tmp_path / "model.safetensors"))
    hf = {"vocab_size": cfg.vocab_size, "hidden_size": H, "num_hidden_layers": cfg.num_layers, "num_attention_heads": hq,
          "num_key_value_heads": hkv, "head_dim": D, "intermediate_size": cfg.intermediate_size, "rms_norm_eps": cfg.rms_eps,
          "rope_theta": cfg.rope_theta, "max_position_embeddings": 4096, "tie_word_embeddings": cfg.tie_embeddings}
    hf.update(hf_extra)
    json.dump(hf, open(tmp_path / "config.json", "w"))


@pytest.mark.parametrize("family", ["mixtral", "qwen3_moe", "qwen2", "gemma"])
def test_model_families_load_from_hf_style_checkpoints(tmp_path, family):
    """Per-expert MoE layouts (Mixtral, Qwen-MoE), implicit q/k/v biases (Qwen2) and Gemma's conventions
    (1 + w norms, scaled embeddings, GeGLU, tied head) map onto the one decoder and reproduce the
    generation of the weights they were written from."""
    import torch
    from fllm_b200.config import EngineConfig, ModelConfig
    from fllm_b200.formats.loader import load_hf_checkpoint
    from fllm_b200.models.weights import init_random_weights
    from fllm_b200.runtime import LLMEngine, SamplingParams
    base = dict(vocab_size=512, hidden_size=128, num_layers=2, num_heads=4, num_kv_heads=2, head_dim=32,
                intermediate_size=192, rms_eps=1e-6, rope_theta=10000.0)
    if family == "mixtral":
        cfg = ModelConfig(**base, num_experts=4, experts_per_token=2, moe_intermediate_size=192, router_kind="softmax_topk")
        extra, style = {"model_type": "mixtral", "num_local_experts": 4, "num_experts_per_tok": 2}, "mixtral"
    elif family == "qwen3_moe":
        cfg = ModelConfig(**base, arch="qwen3", qk_norm=True, num_experts=4, experts_per_token=2, moe_intermediate_size=96,
                          router_kind="softmax_all")
        extra, style = {"model_type": "qwen3_moe", "num_experts": 4, "num_experts_per_tok": 2, "moe_intermediate_size": 96, "norm_topk_prob": True}, "qwen"
    elif family == "qwen2":
        cfg = ModelConfig(**base, attn_bias=True)
        extra, style = {"model_type": "qwen2"}, None
    else:
        cfg = ModelConfig(**base, act="geglu", norm_weight_offset=1.0, embed_scale=128 ** 0.5, tie_embeddings=True)
        extra, style = {"model_type": "gemma"}, None
    w = init_random_weights(cfg, device="cpu", seed=9)
    for lw in w.layers:
        lw.bo = None                       # none of these families has an o_proj bias
    _write_llama_like(tmp_path, cfg, w, extra, style)
    cfg2, w2, _ = load_hf_checkpoint(str(tmp_path), device="cpu")
    for field in ("num_experts", "experts_per_token", "router_kind", "attn_bias", "qk_norm", "act", "norm_weight_offset",
                  "tie_embeddings"):
        assert getattr(cfg2, field) == getattr(cfg, field), field
    assert abs(cfg2.embed_scale - cfg.embed_scale) < 1e-6
    if style:
        assert torch.equal(w2.layers[1].exp_gate_up, w.layers[1].exp_gate_up) and torch.equal(w2.layers[0].exp_down, w.layers[0].exp_down)
    ec = EngineConfig(max_num_seqs=2, max_num_batched_tokens=32, max_model_len=64, num_kv_blocks=16)
    prompt = [[3, 1, 4, 1, 5, 9, 2, 6]]
    sp = SamplingParams(max_tokens=6)
    assert LLMEngine(cfg2, ec, device="cpu", weights=w2).generate(prompt, sp) == LLMEngine(cfg, ec, device="cpu", weights=w).generate(prompt, sp)


def _quant_groups(w, g):
    """Asymmetric 4-bit groups of size g along K: (q uint8 [N, K], scale [N, K/g], zero [N, K/g] integers)."""
    N, K = w.shape
    x = w.float().view(N, K // g, g)
    lo, hi = x.amin(-1), x.amax(-1)
    s = ((hi - lo) / 15.0).clamp_min(1e-8).half().float()
    z = torch.round(-lo / s).clamp(0, 15)
    q = torch.round(x / s.unsqueeze(-1) + z.unsqueeze(-1)).clamp(0, 15).to(torch.uint8).view(N, K)
    return q, s, z


def test_awq_and_gptq_tensors_unpack_to_the_values_their_formula_gives():
    """Pack random codes the way AutoAWQ / AutoGPTQ lay them out, read them back, and compare the Int4Weight
    with (q - zero) * scale; activation-reordered GPTQ groups fall back to a dense tensor with the same values."""
    from fllm_b200.formats.int4_checkpoints import int4_linear, pack_awq, pack_gptq, unpack_awq, unpack_gptq
    from fllm_b200.ops.int4 import Int4Weight
    torch.manual_seed(0)
    N, K, g = 48, 256, 128
    w = torch.randn(N, K)
    q, s, z = _quant_groups(w, g)
    want = (q.float() - z.repeat_interleave(g, 1)) * s.repeat_interleave(g, 1)
    scales_file = s.t().contiguous().half()
    qw, qz = pack_awq(q, z)
    assert qw.shape == (K, N // 8) and qz.shape == (K // g, N // 8) and qw.dtype == torch.int32
    # nibble 1 of the first word is output channel 2 (AutoAWQ's order 0 2 4 6 1 3 5 7)
    assert (int(qw[0, 0]) >> 4) & 0xF == int(q[2, 0])
    q2, s2, z2 = unpack_awq(qw, qz, scales_file)
    assert torch.equal(q2, q) and torch.equal(z2, z) and torch.equal(s2, s)
    a = int4_linear("awq", qw, qz, scales_file)
    assert isinstance(a, Int4Weight) and a.shape == (N, K)
    assert (a.dense() - want).abs().max().item() <= 0.02 * want.abs().max().item()      # scale / min rounded to bf16
    for fmt, off in (("gptq", 1), ("gptq_v2", 0)):
        zz = z.clamp(1, 15) if off else z                     # the old layout cannot store zero = 0 (it stores zero - 1)
        want_g = (q.float() - zz.repeat_interleave(g, 1)) * s.repeat_interleave(g, 1)
        gw, gz = pack_gptq(q, zz, off)
        assert gw.shape == (K // 8, N) and (int(gw[0, 5]) >> 8) & 0xF == int(q[5, 2])   # nibble j = input row 8r + j
        q3, s3, z3 = unpack_gptq(gw, gz, scales_file, off)
        assert torch.equal(q3, q) and torch.equal(z3, zz)
        b = int4_linear("gptq", gw, gz, scales_file, torch.arange(K, dtype=torch.int32) // g, fmt)
        assert isinstance(b, Int4Weight)
        assert (b.dense() - want_g).abs().max().item() <= 0.02 * want_g.abs().max().item()
    perm = torch.randperm(K)
    g_idx = (perm // g).to(torch.int32)                      # act-order: rows of a group are scattered
    gw, gz = pack_gptq(q, z.clamp(1, 15), 1)
    d = int4_linear("gptq", gw, gz, scales_file, g_idx, "gptq", torch.float32)
    assert isinstance(d, torch.Tensor)
    idx = g_idx.long()
    assert torch.allclose(d, (q.float() - z.clamp(1, 15)[:, idx]) * s[:, idx])


@pytest.mark.parametrize("method", ["awq", "gptq"])
def test_int4_hf_checkpoint_loads_packed_and_generates_like_its_dequantised_twin(tmp_path, method):
    """A llama-like checkpoint whose projections are AWQ / GPTQ tensors: the loader keeps them as Int4Weight
    (also under TP2 cuts) and the engine produces the tokens of the same model with dequantised weights."""
    import json
    from fllm_b200.config import EngineConfig, preset
    from fllm_b200.formats.int4_checkpoints import pack_awq, pack_gptq
    from fllm_b200.formats.loader import load_hf_checkpoint
    from fllm_b200.formats.safetensors_io import save_file
    from fllm_b200.models.weights import init_random_weights
    from fllm_b200.ops.int4 import Int4Weight
    from fllm_b200.runtime import LLMEngine, SamplingParams
    cfg = preset("tiny-llama")
    cfg.vocab_size, cfg.intermediate_size = 512, 512
    w = init_random_weights(cfg, "cpu", seed=4)
    D, hq, hkv, I, g = cfg.head_dim, cfg.num_heads, cfg.num_kv_heads, cfg.intermediate_size, 64
    t = {"model.embed_tokens.weight": w.embed, "model.norm.weight": w.final_norm, "lm_head.weight": w.lm_head}

    def put(name, mat):
        q, s, z = _quant_groups(mat, g)
        if method == "gptq":
            z = z.clamp(1, 15)
            q = torch.round(mat.float().view(mat.shape[0], -1, g) / s.unsqueeze(-1) + z.unsqueeze(-1)).clamp(0, 15).to(torch.uint8).view(mat.shape)
            qw, qz = pack_gptq(q, z, 1)
            t[name + ".g_idx"] = torch.arange(mat.shape[1], dtype=torch.int32) // g
        else:
            qw, qz = pack_awq(q, z)
        t[name + ".qweight"], t[name + ".qzeros"], t[name + ".scales"] = qw, qz, s.t().contiguous().half()
        return ((q.float() - z.repeat_interleave(g, 1)) * s.repeat_interleave(g, 1))

    for l, lw in enumerate(w.layers):
        p = f"model.layers.{l}."
        t[p + "input_layernorm.weight"], t[p + "post_attention_layernorm.weight"] = lw.attn_norm, lw.ffn_norm
        parts = {"self_attn.q_proj": lw.wqkv[: hq * D], "self_attn.k_proj": lw.wqkv[hq * D: (hq + hkv) * D],
                 "self_attn.v_proj": lw.wqkv[(hq + hkv) * D:], "self_attn.o_proj": lw.wo,
                 "mlp.gate_proj": lw.w_gate_up[:I], "mlp.up_proj": lw.w_gate_up[I:], "mlp.down_proj": lw.w_down}
        deq = {k: put(p + k, v) for k, v in parts.items()}
        lw.wqkv = torch.cat([deq["self_attn.q_proj"], deq["self_attn.k_proj"], deq["self_attn.v_proj"]], 0)
        lw.wo, lw.w_down = deq["self_attn.o_proj"], deq["mlp.down_proj"]
        lw.w_gate_up = torch.cat([deq["mlp.gate_proj"], deq["mlp.up_proj"]], 0)
    save_file({k: v.contiguous() for k, v in t.items()}, str(tmp_path / "model.safetensors"))
    hf = {"model_type": "llama", "vocab_size": cfg.vocab_size, "hidden_size": cfg.hidden_size, "num_hidden_layers": cfg.num_layers,
          "num_attention_heads": hq, "num_key_value_heads": hkv, "head_dim": D, "intermediate_size": I, "rms_norm_eps": cfg.rms_eps,
          "rope_theta": cfg.rope_theta, "max_position_embeddings": 4096, "tie_word_embeddings": False,
          "quantization_config": {"quant_method": method, "bits": 4, "group_size": g, "checkpoint_format": "gptq"}}
    json.dump(hf, open(tmp_path / "config.json", "w"))
    cfg2, w2, _ = load_hf_checkpoint(str(tmp_path), device="cpu")
    for lw in w2.layers:
        assert all(isinstance(getattr(lw, n), Int4Weight) for n in ("wqkv", "wo", "w_gate_up", "w_down"))
    lw0 = w2.layers[0]
    assert (lw0.wqkv.dense() - w.layers[0].wqkv.float()).abs().max().item() <= 0.03 * w.layers[0].wqkv.abs().max().item()
    ec = EngineConfig(max_num_seqs=2, max_num_batched_tokens=32, max_model_len=64, num_kv_blocks=16)
    prompt = [[3, 1, 4, 1, 5, 9, 2, 6]]
    logits = []
    for cc, ww in ((cfg2, w2), (cfg, w)):
        eng = LLMEngine(cc, ec, device="cpu", weights=ww)
        eng.add_request(prompt[0], SamplingParams(max_tokens=1))
        step = eng.scheduler.schedule()
        logits.append(eng.decoder.forward(eng._build_batch(step))[-1].float())
    err = (logits[0] - logits[1]).abs().max().item() / (logits[1].abs().max().item() + 1e-6)
    assert err < 0.05, err
    _, w_r1, _ = load_hf_checkpoint(str(tmp_path), device="cpu", tp=2, tp_rank=1)
    half = w2.layers[0].w_down.shape[1] // 2
    assert w_r1.layers[0].w_down.shape == (cfg.hidden_size, half)
    if half % 64 == 0:
        assert isinstance(w_r1.layers[0].w_down, Int4Weight)
        assert torch.equal(w_r1.layers[0].w_down.dense(), w2.layers[0].w_down.dense()[:, half:])


def test_phi3_fused_projections_load_like_the_split_ones(tmp_path):
    """Phi-3 stores q|k|v and gate|up as single tensors: same weights and tokens as the split llama form."""
    import json
    from fllm_b200.config import EngineConfig, preset
    from fllm_b200.formats.loader import load_hf_checkpoint
    from fllm_b200.formats.safetensors_io import save_file
    from fllm_b200.models.weights import init_random_weights
    from fllm_b200.runtime import LLMEngine, SamplingParams
    cfg = preset("tiny-llama")
    cfg.vocab_size = 512
    w = init_random_weights(cfg, "cpu", seed=6)
    t = {"model.embed_tokens.weight": w.embed, "model.norm.weight": w.final_norm, "lm_head.weight": w.lm_head}
    for l, lw in enumerate(w.layers):
        p = f"model.layers.{l}."
        t.update({p + "input_layernorm.weight": lw.attn_norm, p + "post_attention_layernorm.weight": lw.ffn_norm,
                  p + "self_attn.qkv_proj.weight": lw.wqkv, p + "self_attn.o_proj.weight": lw.wo,
                  p + "mlp.gate_up_proj.weight": lw.w_gate_up, p + "mlp.down_proj.weight": lw.w_down})
    save_file({k: v.contiguous() for k, v in t.items()}, str(tmp_path / "model.safetensors"))
    hf = {"model_type": "phi3", "vocab_size": cfg.vocab_size, "hidden_size": cfg.hidden_size, "num_hidden_layers": cfg.num_layers,
          "num_attention_heads": cfg.num_heads, "num_key_value_heads": cfg.num_kv_heads, "intermediate_size": cfg.intermediate_size,
          "rms_norm_eps": cfg.rms_eps, "rope_theta": cfg.rope_theta, "max_position_embeddings": 4096, "tie_word_embeddings": False}
    json.dump(hf, open(tmp_path / "config.json", "w"))
    cfg2, w2, _ = load_hf_checkpoint(str(tmp_path), device="cpu")
    assert cfg2.head_dim == cfg.head_dim
    for a, b in zip(w2.layers, w.layers):
        assert torch.equal(a.wqkv, b.wqkv) and torch.equal(a.w_gate_up, b.w_gate_up) and torch.equal(a.w_down, b.w_down)
    _, w_r1, _ = load_hf_checkpoint(str(tmp_path), device="cpu", tp=2, tp_rank=1)
    I = cfg.intermediate_size
    assert torch.equal(w_r1.layers[0].w_gate_up[: I // 2], w.layers[0].w_gate_up[I // 2: I])
    ec = EngineConfig(max_num_seqs=2, max_num_batched_tokens=32, max_model_len=64, num_kv_blocks=16)
    sp = SamplingParams(max_tokens=5)
    prompt = [[3, 1, 4, 1, 5, 9, 2, 6]]
    assert LLMEngine(cfg2, ec, device="cpu", weights=w2).generate(prompt, sp) == LLMEngine(cfg, ec, device="cpu", weights=w).generate(prompt, sp)


def test_gemma2_post_norms_scale_and_window_pattern(tmp_path):
    """Gemma-2: the attention and FFN outputs go through their own RMSNorm before the residual add, the softmax
    scale comes from query_pre_attn_scalar, layers alternate sliding / full attention. The engine must match the
    dense oracle, and an HF-style checkpoint (four norm tensors per layer) must load into the same model."""
    import json
    from fllm_b200.config import EngineConfig, preset
    from fllm_b200.formats.loader import load_hf_checkpoint
    from fllm_b200.formats.safetensors_io import save_file
    from fllm_b200.models.weights import init_random_weights
    from fllm_b200.runtime import LLMEngine, SamplingParams
    from oracle import dense_forward, greedy_generate
    cfg = preset("tiny-llama")
    cfg.vocab_size, cfg.intermediate_size = 512, 512
    cfg.post_norms, cfg.attn_scale, cfg.act = True, 24.0 ** -0.5, "geglu"
    cfg.norm_weight_offset, cfg.embed_scale, cfg.tie_embeddings = 1.0, float(cfg.hidden_size) ** 0.5, True
    cfg.attn_softcap, cfg.logit_softcap, cfg.sliding_window, cfg.window_pattern = 50.0, 30.0, 16, [1, 0]
    w = init_random_weights(cfg, "cpu", seed=8)
    w.lm_head = w.embed
    for lw in w.layers:                                   # (1 + w) norms: keep the effective weights near one
        lw.post_attn_norm, lw.post_ffn_norm = lw.post_attn_norm - 1.0, lw.post_ffn_norm - 1.0
        lw.attn_norm, lw.ffn_norm = lw.attn_norm - 1.0, lw.ffn_norm - 1.0
    w.final_norm = w.final_norm - 1.0
    ec = EngineConfig(max_num_seqs=2, max_num_batched_tokens=32, max_model_len=96, num_kv_blocks=16)
    prompt = [int(t) for t in torch.randint(0, 512, (40,), generator=torch.Generator().manual_seed(1))]
    eng = LLMEngine(cfg, ec, device="cpu", weights=w)
    assert eng.generate([prompt], SamplingParams(max_tokens=5))[0] == greedy_generate(cfg, w, prompt, 5)
    # the post norms matter: without them the logits differ
    a = dense_forward(cfg, w, prompt)[-1]
    saved = [(lw.post_attn_norm, lw.post_ffn_norm) for lw in w.layers]
    for lw in w.layers:
        lw.post_attn_norm = lw.post_ffn_norm = None
    assert (dense_forward(cfg, w, prompt)[-1] - a).abs().max() > 1e-3
    for lw, (pa, pf) in zip(w.layers, saved):
        lw.post_attn_norm, lw.post_ffn_norm = pa, pf
    D, hq, hkv, I = cfg.head_dim, cfg.num_heads, cfg.num_kv_heads, cfg.intermediate_size
    t = {"model.embed_tokens.weight": w.embed, "model.norm.weight": w.final_norm}
    for l, lw in enumerate(w.layers):
        p = f"model.layers.{l}."
        t.update({p + "input_layernorm.weight": lw.attn_norm, p + "post_attention_layernorm.weight": lw.post_attn_norm,
                  p + "pre_feedforward_layernorm.weight": lw.ffn_norm, p + "post_feedforward_layernorm.weight": lw.post_ffn_norm,
                  p + "self_attn.q_proj.weight": lw.wqkv[: hq * D], p + "self_attn.k_proj.weight": lw.wqkv[hq * D: (hq + hkv) * D],
                  p + "self_attn.v_proj.weight": lw.wqkv[(hq + hkv) * D:], p + "self_attn.o_proj.weight": lw.wo,
                  p + "mlp.gate_proj.weight": lw.w_gate_up[:I], p + "mlp.up_proj.weight": lw.w_gate_up[I:],
                  p + "mlp.down_proj.weight": lw.w_down})
    save_file({k: v.contiguous() for k, v in t.items()}, str(tmp_path / "model.safetensors"))
    hf = {"model_type": "gemma2", "vocab_size": 512, "hidden_size": cfg.hidden_size, "num_hidden_layers": cfg.num_layers,
          "num_attention_heads": hq, "num_key_value_heads": hkv, "head_dim": D, "intermediate_size": I,
          "rms_norm_eps": cfg.rms_eps, "rope_theta": cfg.rope_theta, "max_position_embeddings": 4096,
          "query_pre_attn_scalar": 24, "sliding_window": 16, "attn_logit_softcapping": 50.0, "final_logit_softcapping": 30.0}
    json.dump(hf, open(tmp_path / "config.json", "w"))
    cfg2, w2, _ = load_hf_checkpoint(str(tmp_path), device="cpu")
    assert cfg2.post_norms and abs(cfg2.attn_scale - 24.0 ** -0.5) < 1e-9 and cfg2.window_pattern == [1, 0]
    assert cfg2.layer_window(0) == 16 and cfg2.layer_window(1) == 0 and cfg2.act == "geglu" and cfg2.tie_embeddings
    assert torch.equal(w2.layers[1].post_ffn_norm, w.layers[1].post_ffn_norm)
    eng2 = LLMEngine(cfg2, ec, device="cpu", weights=w2)
    assert eng2.generate([prompt], SamplingParams(max_tokens=5))[0] == eng.generate([prompt], SamplingParams(max_tokens=5))[0]


def test_planar_device_forms_of_q5k_q6k_q80_equal_the_codecs():
    """The re-laid planes of the 5 / 6 / 8-bit GGUF types decode to exactly what the file blocks decode to, keep
    the file's bits per weight, survive row and column cuts, and stack with other weight kinds."""
    import numpy as np
    import torch
    from fllm_b200.formats import quant as Q
    from fllm_b200.ops.int4 import Int4Weight
    from fllm_b200.ops.intk import IntKWeight, StackedWeight
    from fllm_b200.ops.reference import RefOps
    rng = np.random.default_rng(0)
    for name, tid, bpw in (("Q8_0", Q.Q8_0, 8.5), ("Q6_K", Q.Q6_K, 6.5625), ("Q5_K", Q.Q5_K, 5.625)):
        w = (rng.standard_normal((48, 512)) * 0.05).astype(np.float32)
        raw = Q.quantize(w, tid)
        want = Q.dequantize(raw, tid, 48, 512)
        k = IntKWeight.from_gguf(name, raw, 48, 512)
        assert np.array_equal(k.dense().numpy(), want)
        assert abs(k.nbytes() * 8 / (48 * 512) - bpw) < 0.01
        cut = k.rows(slice(8, 24)).cols(slice(256, 512))
        assert np.array_equal(cut.dense().numpy(), want[8:24, 256:512])
    K = 512
    ws = [(rng.standard_normal((n, K)) * 0.05).astype(np.float32) for n in (64, 32, 32)]
    st = StackedWeight([Int4Weight.from_gguf("Q4_K", Q.quantize(ws[0], Q.Q4_K), 64, K),
                        IntKWeight.from_gguf("Q6_K", Q.quantize(ws[1], Q.Q6_K), 32, K), torch.from_numpy(ws[2]).bfloat16()])
    x = torch.randn(3, K).bfloat16()
    y = RefOps().linear(x, st)
    ref = x.float() @ st.dense().t()
    assert st.shape == (128, K) and float((y.float() - ref).abs().max() / ref.abs().max()) < 1e-2


def test_pytorch_zip_checkpoints_are_read_without_running_their_pickle(tmp_path):
    import collections
    import os
    import pickle
    import zipfile
    import pytest
    import torch
    from fllm_b200.formats.safetensors_io import open_checkpoint
    from fllm_b200.formats.torch_zip import TorchZipError, TorchZipFile
    sd = collections.OrderedDict(a=torch.randn(3, 4), b=torch.randn(5, 6).bfloat16(), c=torch.arange(10)[2:8],
                                 t=torch.randn(4, 6).t(), s=torch.tensor(3.5), p=torch.nn.Parameter(torch.randn(2, 2)),
                                 h=torch.randn(7).half())
    d = tmp_path / "ck"
    d.mkdir()
    torch.save(sd, str(d / "pytorch_model.bin"))
    ck = open_checkpoint(str(d))
    assert set(ck) == set(sd)
    for k, v in sd.items():
        got = ck[k][0].tensor(k)
        assert got.dtype == v.dtype and torch.equal(got, v.detach()), k

    class Evil:
        def __reduce__(self):
            return (os.system, ("true",))
    bad = str(tmp_path / "bad.bin")
    with zipfile.ZipFile(bad, "w") as z:
        z.writestr("archive/data.pkl", pickle.dumps({"x": Evil()}))
    with pytest.raises(TorchZipError):
        TorchZipFile(bad)
    with open(str(tmp_path / "junk.bin"), "wb") as f:
        f.write(b"not a zip at all")
    with pytest.raises(TorchZipError):
        TorchZipFile(str(tmp_path / "junk.bin"))


@pytest.mark.parametrize("family", ["mlx4", "mlx8", "bnb_nf4", "bnb_nf4_double"])
def test_mlx_affine_and_bitsandbytes_layers_load(tmp_path, family):
    """A llama-like checkpoint whose projections are MLX affine tensors (uint32 words, scales, biases) or bitsandbytes
    4-bit tensors (nibble pairs, absmax per 64 values, optionally double-quantised): packed the way the formats define,
    read back by the loader; 4-bit MLX layers stay packed, the others are expanded; logits follow the dequantised twin."""
    import json
    from fllm_b200.config import EngineConfig, preset
    from fllm_b200.formats.extra_quant import NF4_MAP
    from fllm_b200.formats.loader import load_hf_checkpoint
    from fllm_b200.formats.safetensors_io import save_file
    from fllm_b200.models.weights import init_random_weights
    from fllm_b200.ops.int4 import Int4Weight
    from fllm_b200.runtime import LLMEngine, SamplingParams
    cfg = preset("tiny-llama")
    cfg.vocab_size, cfg.intermediate_size = 512, 512
    w = init_random_weights(cfg, "cpu", seed=8)
    D, hq, hkv, I, g = cfg.head_dim, cfg.num_heads, cfg.num_kv_heads, cfg.intermediate_size, 64
    t = {"model.embed_tokens.weight": w.embed, "model.norm.weight": w.final_norm, "lm_head.weight": w.lm_head}
    nf4 = torch.tensor(NF4_MAP)

    def put(name, mat):
        mat = mat.float()
        N, K = mat.shape
        if family.startswith("mlx"):
            bits = 4 if family == "mlx4" else 8
            grp = mat.view(N, K // g, g)
            lo, hi = grp.min(-1).values, grp.max(-1).values
            s = ((hi - lo) / (2 ** bits - 1)).clamp_min(1e-8).half().float()
            b = lo.half().float()
            q = torch.round((grp - b[..., None]) / s[..., None]).clamp(0, 2 ** bits - 1).to(torch.int64).view(N, K)
            per = 32 // bits
            words = (q.view(N, K // per, per) << (torch.arange(per) * bits)).sum(-1)
            t[name + ".weight"] = words.to(torch.uint32) if hasattr(torch, "uint32") else words.to(torch.int32)
            t[name + ".scales"], t[name + ".biases"] = s.half(), b.half()
            return (q.view(N, K // g, g).float() * s[..., None] + b[..., None]).view(N, K)
        flat = mat.reshape(-1, 64)
        absmax = flat.abs().max(-1).values.clamp_min(1e-8)
        code = ((flat / absmax[:, None])[..., None] - nf4).abs().argmin(-1)                   # nearest codebook entry
        pairs = code.view(-1, 2)
        t[name + ".weight"] = ((pairs[:, 0] << 4) | pairs[:, 1]).to(torch.uint8).view(-1, 1)
        t[name + ".weight.quant_map"] = nf4.clone()
        state = {"quant_type": "nf4", "blocksize": 64, "dtype": "bfloat16", "shape": [N, K]}
        used = absmax
        if family.endswith("double"):
            offset = float(absmax.mean())
            res = (absmax - offset).reshape(-1, 256) if absmax.numel() % 256 == 0 else None
            assert res is not None
            nmax = res.abs().max(-1).values.clamp_min(1e-8)
            nmap = torch.linspace(-1, 1, 256)
            ncode = ((res / nmax[:, None])[..., None] - nmap).abs().argmin(-1)
            t[name + ".weight.absmax"] = ncode.reshape(-1).to(torch.uint8)
            t[name + ".weight.nested_absmax"], t[name + ".weight.nested_quant_map"] = nmax, nmap
            state.update(nested_blocksize=256, nested_offset=offset, nested_dtype="float32")
            used = (nmap[ncode] * nmax[:, None]).reshape(-1) + offset
        else:
            t[name + ".weight.absmax"] = absmax
        t[name + ".weight.quant_state.bitsandbytes__nf4"] = torch.tensor(list(json.dumps(state).encode()), dtype=torch.uint8)
        return (nf4[code] * used[:, None]).view(N, K)

    for l, lw in enumerate(w.layers):
        p = f"model.layers.{l}."
        t[p + "input_layernorm.weight"], t[p + "post_attention_layernorm.weight"] = lw.attn_norm, lw.ffn_norm
        parts = {"self_attn.q_proj": lw.wqkv[: hq * D], "self_attn.k_proj": lw.wqkv[hq * D: (hq + hkv) * D],
                 "self_attn.v_proj": lw.wqkv[(hq + hkv) * D:], "self_attn.o_proj": lw.wo,
                 "mlp.gate_proj": lw.w_gate_up[:I], "mlp.up_proj": lw.w_gate_up[I:], "mlp.down_proj": lw.w_down}
        deq = {k: put(p + k, v) for k, v in parts.items()}
        lw.wqkv = torch.cat([deq["self_attn.q_proj"], deq["self_attn.k_proj"], deq["self_attn.v_proj"]], 0).bfloat16()
        lw.wo, lw.w_down = deq["self_attn.o_proj"].bfloat16(), deq["mlp.down_proj"].bfloat16()
        lw.w_gate_up = torch.cat([deq["mlp.gate_proj"], deq["mlp.up_proj"]], 0).bfloat16()
    save_file({k: v.contiguous() for k, v in t.items()}, str(tmp_path / "model.safetensors"))
    hf = {"model_type": "llama", "vocab_size": cfg.vocab_size, "hidden_size": cfg.hidden_size, "num_hidden_layers": cfg.num_layers,
          "num_attention_heads": hq, "num_key_value_heads": hkv, "head_dim": D, "intermediate_size": I, "rms_norm_eps": cfg.rms_eps,
          "rope_theta": cfg.rope_theta, "max_position_embeddings": 4096, "tie_word_embeddings": False}
    if family.startswith("mlx"):
        hf["quantization"] = {"group_size": g, "bits": 4 if family == "mlx4" else 8}
    else:
        hf["quantization_config"] = {"quant_method": "bitsandbytes", "load_in_4bit": True, "bnb_4bit_quant_type": "nf4",
                                     "bnb_4bit_use_double_quant": family.endswith("double")}
    json.dump(hf, open(tmp_path / "config.json", "w"))
    cfg2, w2, _ = load_hf_checkpoint(str(tmp_path), device="cpu")
    packed = all(isinstance(getattr(lw, n), Int4Weight) for lw in w2.layers for n in ("wqkv", "wo", "w_gate_up", "w_down"))
    assert packed == (family == "mlx4")
    a, b = w2.layers[0].w_down, w.layers[0].w_down.float()
    a = a.dense().float() if isinstance(a, Int4Weight) else a.float()
    assert (a - b).abs().max().item() <= 0.02 * b.abs().max().item()
    ec = EngineConfig(max_num_seqs=2, max_num_batched_tokens=32, max_model_len=64, num_kv_blocks=16)
    logits = []
    for cc, ww in ((cfg2, w2), (cfg, w)):
        eng = LLMEngine(cc, ec, device="cpu", weights=ww)
        logits.append(eng.token_logits([3, 1, 4, 1, 5, 9, 2, 6]))
    err = (logits[0] - logits[1]).abs().max().item() / (logits[1].abs().max().item() + 1e-6)
    assert err < 0.05, err
