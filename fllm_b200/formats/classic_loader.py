"""Hugging Face checkpoints of the families built from LayerNorm, plain MLPs or parallel blocks (StarCoder2, StableLM,
Nemotron, Arcee, Phi, GPT-NeoX / Pythia, Cohere) into the decoder's weight containers (one rank).

The reference reads these families from GGUF files through the same decoder (rust/engine/src/rust_decoder.rs
``load_layers_ex``: `norm` kinds, `ffn` kinds, parallel residual); the tensor roles are the same, the names here are the
Hugging Face ones.
"""
from __future__ import annotations

import torch

from ..config import ModelConfig
from ..models.weights import DecoderWeights, LayerWeights

# per family: (layer prefix, attention prefix, q/k/v names or fused name, output name, first norm, second norm, MLP in, MLP out)
_NAMES = {
    "starcoder2": ("model.layers.{}.", "self_attn.", ("q_proj", "k_proj", "v_proj"), "o_proj", "input_layernorm", "post_attention_layernorm",
                   "mlp.c_fc", "mlp.c_proj"),
    "stablelm": ("model.layers.{}.", "self_attn.", ("q_proj", "k_proj", "v_proj"), "o_proj", "input_layernorm", "post_attention_layernorm",
                 None, "mlp.down_proj"),
    "nemotron": ("model.layers.{}.", "self_attn.", ("q_proj", "k_proj", "v_proj"), "o_proj", "input_layernorm", "post_attention_layernorm",
                 "mlp.up_proj", "mlp.down_proj"),
    "jais2": ("model.layers.{}.", "self_attn.", ("q_proj", "k_proj", "v_proj"), "o_proj", "input_layernorm", "post_attention_layernorm",
              "mlp.up_proj", "mlp.down_proj"),
    "arcee": ("model.layers.{}.", "self_attn.", ("q_proj", "k_proj", "v_proj"), "o_proj", "input_layernorm", "post_attention_layernorm",
              "mlp.up_proj", "mlp.down_proj"),
    "phi": ("model.layers.{}.", "self_attn.", ("q_proj", "k_proj", "v_proj"), "dense", "input_layernorm", None, "mlp.fc1", "mlp.fc2"),
    "gpt_neox": ("gpt_neox.layers.{}.", "attention.", "query_key_value", "dense", "input_layernorm", "post_attention_layernorm",
                 "mlp.dense_h_to_4h", "mlp.dense_4h_to_h"),
    "cohere": ("model.layers.{}.", "self_attn.", ("q_proj", "k_proj", "v_proj"), "o_proj", "input_layernorm", None, None, "mlp.down_proj"),
    "cohere2": ("model.layers.{}.", "self_attn.", ("q_proj", "k_proj", "v_proj"), "o_proj", "input_layernorm", None, None, "mlp.down_proj"),
    "olmo": ("model.layers.{}.", "self_attn.", ("q_proj", "k_proj", "v_proj"), "o_proj", None, None, None, "mlp.down_proj"),
    "gpt_bigcode": ("transformer.h.{}.", "attn.", "c_attn", "c_proj", "ln_1", "ln_2", "mlp.c_fc", "mlp.c_proj"),
    "falcon": ("transformer.h.{}.", "self_attention.", "query_key_value", "dense", "input_layernorm", "post_attention_layernorm",
               "mlp.dense_h_to_4h", "mlp.dense_4h_to_h"),
    "gpt2": ("transformer.h.{}.", "attn.", "c_attn", "c_proj", "ln_1", "ln_2", "mlp.c_fc", "mlp.c_proj"),
    "opt": ("model.decoder.layers.{}.", "self_attn.", ("q_proj", "k_proj", "v_proj"), "out_proj", "self_attn_layer_norm", "final_layer_norm",
            "fc1", "fc2"),
    "olmo2": ("model.layers.{}.", "self_attn.", ("q_proj", "k_proj", "v_proj"), "o_proj", None, None, None, "mlp.down_proj"),
    "exaone4": ("model.layers.{}.", "self_attn.", ("q_proj", "k_proj", "v_proj"), "o_proj", None, None, None, "mlp.down_proj"),
    "olmo3": ("model.layers.{}.", "self_attn.", ("q_proj", "k_proj", "v_proj"), "o_proj", None, None, None, "mlp.down_proj"),
}


def load_hf_classic(cfg: ModelConfig, get, device, dtype) -> DecoderWeights:
    """``get(name, required=True)`` returns a checkpoint tensor (or None)."""
    def dev(t):
        return t.to(device=device, dtype=dtype).contiguous()

    def opt(name):
        t = get(name, False)
        return dev(t) if t is not None else None

    lp, ap, qkv, o_name, n1, n2, mlp_in, mlp_out = _NAMES[cfg.arch]
    if cfg.arch == "falcon" and cfg.parallel_block:          # one shared norm, or a norm each under names of their own
        n1, n2 = ("ln_attn", "ln_mlp") if cfg.parallel_norms == 2 else ("input_layernorm", None)
    H, D, hq, hkv = cfg.hidden_size, cfg.head_dim, cfg.num_heads, cfg.num_kv_heads
    if cfg.arch == "gpt2":                      # GPT-2 stores its matrices as [in, out]
        inner = get

        def get(name, required=True):            # noqa: F811 (a transposing view of the reader for this family's matrices)
            t = inner(name, required)
            if t is not None and t.dim() == 2 and name.endswith(".weight") and (".attn.c_" in name or ".mlp.c_" in name):
                return t.t()
            return t
    layers = []
    for l in range(cfg.num_layers):
        p = lp.format(l)
        lw = LayerWeights(attn_norm=dev(get(p + n1 + ".weight")) if n1 else None, wqkv=None, wo=None,
                          ffn_norm=dev(get(p + n2 + ".weight")) if n2 else None)
        lw.attn_norm_b, lw.ffn_norm_b = opt(p + n1 + ".bias") if n1 else None, opt(p + n2 + ".bias") if n2 else None
        if cfg.arch == "olmo":                  # LayerNorm without parameters
            lw.attn_norm = lw.ffn_norm = torch.ones(H, device=device, dtype=dtype)
        if cfg.post_norms:                      # OLMo-2: the norms sit behind the blocks
            lw.post_attn_norm = dev(get(p + "post_attention_layernorm.weight"))
            lw.post_ffn_norm = dev(get(p + "post_feedforward_layernorm.weight"))
        if cfg.qk_norm:
            lw.q_norm, lw.k_norm = dev(get(p + ap + "q_norm.weight")), dev(get(p + ap + "k_norm.weight"))
        if cfg.qk_norm_full:
            lw.q_norm_full, lw.k_norm_full = dev(get(p + ap + "q_norm.weight")), dev(get(p + ap + "k_norm.weight"))
        if isinstance(qkv, tuple):
            lw.wqkv = dev(torch.cat([get(p + ap + n + ".weight") for n in qkv], 0))
            bs = [get(p + ap + n + ".bias", False) for n in qkv]
            if bs[0] is not None:
                lw.bqkv = dev(torch.cat(bs))
        elif cfg.arch == "falcon" and cfg.ssm["qkv_layout"] == "grouped":     # per key / value head: its query heads, its key, its value
            g = hq // hkv
            w = get(p + ap + qkv + ".weight").view(hkv, g + 2, D, H)
            lw.wqkv = dev(torch.cat([w[:, :g].reshape(hq * D, H), w[:, g].reshape(hkv * D, H), w[:, g + 1].reshape(hkv * D, H)], 0))
            bb = get(p + ap + qkv + ".bias", False)
            if bb is not None:
                bb = bb.view(hkv, g + 2, D)
                lw.bqkv = dev(torch.cat([bb[:, :g].reshape(-1), bb[:, g].reshape(-1), bb[:, g + 1].reshape(-1)]))
        elif cfg.arch == "gpt2" or (cfg.arch in ("gpt_bigcode", "falcon") and hkv == 1):      # one matrix: all q rows, all k rows, all v rows
            lw.wqkv, lw.bqkv = dev(get(p + ap + qkv + ".weight")), opt(p + ap + qkv + ".bias")
        else:                                   # GPT-NeoX: one matrix whose rows go head by head as (q, k, v)
            w = get(p + ap + qkv + ".weight").view(hq, 3, D, H)
            lw.wqkv = dev(torch.cat([w[:, 0].reshape(hq * D, H), w[:, 1].reshape(hq * D, H), w[:, 2].reshape(hq * D, H)], 0))
            bb = get(p + ap + qkv + ".bias", False)
            if bb is not None:
                bb = bb.view(hq, 3, D)
                lw.bqkv = dev(torch.cat([bb[:, 0].reshape(-1), bb[:, 1].reshape(-1), bb[:, 2].reshape(-1)]))
        lw.wo, lw.bo = dev(get(p + ap + o_name + ".weight")), opt(p + ap + o_name + ".bias")
        if cfg.mlp_kind == "plain":
            lw.w_gate_up, lw.b_up = dev(get(p + mlp_in + ".weight")), opt(p + mlp_in + ".bias")
        else:
            lw.w_gate_up = dev(torch.cat([get(p + "mlp.gate_proj.weight"), get(p + "mlp.up_proj.weight")], 0))
        lw.w_down, lw.b_down = dev(get(p + mlp_out + ".weight")), opt(p + mlp_out + ".bias")
        layers.append(lw)
    if cfg.arch == "falcon":
        embed, fin, head = "transformer.word_embeddings.weight", "transformer.ln_f", "lm_head.weight"
    elif cfg.arch in ("gpt2", "gpt_bigcode"):
        embed, fin, head = "transformer.wte.weight", "transformer.ln_f", "lm_head.weight"
    elif cfg.arch == "opt":
        embed, fin, head = "model.decoder.embed_tokens.weight", "model.decoder.final_layer_norm", "lm_head.weight"
    elif cfg.arch == "gpt_neox":
        embed, fin, head = "gpt_neox.embed_in.weight", "gpt_neox.final_layer_norm", "embed_out.weight"
    elif cfg.arch == "phi":
        embed, fin, head = "model.embed_tokens.weight", "model.final_layernorm", "lm_head.weight"
    else:
        embed, fin, head = "model.embed_tokens.weight", "model.norm", "lm_head.weight"
    e = dev(get(embed))
    hw = get(head, False)
    head_d = e if (hw is None or cfg.tie_embeddings) else dev(hw)
    mult = cfg.ssm.get("logit_mult", 1.0) if cfg.ssm else 1.0
    if mult != 1.0:                             # Cohere: logits * scale, as a head of its own
        head_d = dev((get(embed) if (hw is None or cfg.tie_embeddings) else hw).float() * mult)
    fin_w = torch.ones(H, device=device, dtype=dtype) if cfg.arch == "olmo" else dev(get(fin + ".weight"))
    w = DecoderWeights(embed=e, layers=layers, final_norm=fin_w, lm_head=head_d, vocab_start=0,
                       vocab_local=cfg.vocab_size)
    w.final_norm_b = opt(fin + ".bias")
    if cfg.learned_positions:
        w.pos_embed = dev(get("transformer.wpe.weight" if cfg.arch in ("gpt2", "gpt_bigcode") else "model.decoder.embed_positions.weight"))
    w.lm_head_b = opt("lm_head.bias")
    return w
