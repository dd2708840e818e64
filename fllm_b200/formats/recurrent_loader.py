"""Hugging Face checkpoints of the recurrent and hybrid families (model types ``mamba``, ``falcon_mamba``,
``mamba2``, ``bamba``, ``lfm2``) and of the latent-attention family (``deepseek_v2``, ``deepseek_v3`` with dense
feed-forward layers) into the decoder's weight containers.

The reference reads the same families from GGUF files in rust/engine/src/rust_decoder.rs (``load_layers_ex``) and
rust/engine/src/rust_decoder/hybrid.rs; the tensor roles are the same, the names here are the Hugging Face ones.
"""
from __future__ import annotations

import torch

from ..config import ModelConfig
from ..models.recurrent import pack_mamba1, pack_mamba2
from ..models.weights import DecoderWeights, LayerWeights


def load_hf_recurrent(cfg: ModelConfig, get, device, dtype) -> DecoderWeights:
    """``get(name, required=True)`` returns a checkpoint tensor (or None)."""
    def dev(t):
        return t.to(device=device, dtype=dtype).contiguous()

    def attention(lw, p, q_norm=None, k_norm=None, o_name="o_proj"):
        lw.wqkv = dev(torch.cat([get(p + f"{n}_proj.weight") for n in "qkv"], 0))
        lw.wo = dev(get(p + o_name + ".weight"))
        if cfg.attn_bias and get(p + "q_proj.bias", False) is not None:
            lw.bqkv = dev(torch.cat([get(p + f"{n}_proj.bias") for n in "qkv"]))
            bo = get(p + o_name + ".bias", False)
            lw.bo = dev(bo) if bo is not None else None
        if q_norm is not None:
            lw.q_norm, lw.k_norm = dev(get(q_norm)), dev(get(k_norm))

    def glu(lw, p, gate, up, down):
        lw.w_gate_up = dev(torch.cat([get(p + gate + ".weight"), get(p + up + ".weight")], 0))
        lw.w_down = dev(get(p + down + ".weight"))

    def deepseek_moe(lw, mp):
        """Router (+ selection bias), routed experts (one fused pair of tensors or one module per expert), shared experts."""
        lw.router_w = dev(get(mp + "gate.weight"))
        sel = get(mp + "gate.e_score_correction_bias", False)
        for alt in ("gate.moe_statics.e_score_correction_bias", "moe_statics.e_score_correction_bias"):      # ERNIE 4.5
            if sel is None:
                sel = get(mp + alt, False)
        if sel is not None:
            lw.router_select_b = sel.float().reshape(-1).to(device).contiguous()
        fused = get(mp + "experts.gate_up_proj", False)
        if fused is not None:
            lw.exp_gate_up, lw.exp_down = dev(fused), dev(get(mp + "experts.down_proj"))
        else:
            E = cfg.num_experts
            lw.exp_gate_up = dev(torch.stack([torch.cat([get(mp + f"experts.{e}.gate_proj.weight"),
                                                         get(mp + f"experts.{e}.up_proj.weight")], 0) for e in range(E)]))
            lw.exp_down = dev(torch.stack([get(mp + f"experts.{e}.down_proj.weight") for e in range(E)]))
        if cfg.shared_intermediate_size:
            lw.shared_gate_up = dev(torch.cat([get(mp + "shared_experts.gate_proj.weight"), get(mp + "shared_experts.up_proj.weight")], 0))
            lw.shared_down = dev(get(mp + "shared_experts.down_proj.weight"))

    s = cfg.ssm
    layers = []
    mt = cfg.arch_alias or cfg.arch
    # language model inside a multimodal wrapper: model.language_model.*
    root = "model.language_model." if get("model.language_model.embed_tokens.weight", False) is not None else "model."
    # Nemotron-H checkpoints: backbone.embedding(s) / backbone.layers; the in-memory module names say model.embeddings
    nemo_embed = next((n for n in ("backbone.embeddings.weight", "backbone.embedding.weight", "model.embeddings.weight",
                                   "model.embedding.weight") if get(n, False) is not None), None) if mt == "nemotron_h" else None
    nemo_root = (nemo_embed or "backbone.").split(".")[0] + "."
    for l in range(cfg.num_layers):
        kind = cfg.layer_kind(l)
        if mt in ("mamba", "falcon_mamba", "mamba2"):
            p = f"backbone.layers.{l}."
            lw = LayerWeights(attn_norm=dev(get(p + "norm.weight")), wqkv=None, wo=None, ffn_norm=None)
            m = p + "mixer."
            if kind == "mamba1":
                lw.mixer = pack_mamba1(get(m + "in_proj.weight"), get(m + "conv1d.weight"), get(m + "conv1d.bias", False),
                                       get(m + "x_proj.weight"), get(m + "dt_proj.weight"), get(m + "dt_proj.bias"),
                                       get(m + "A_log"), get(m + "D"), get(m + "out_proj.weight"), s["d_state"], s["dt_rank"],
                                       dtype, device, get(m + "in_proj.bias", False), get(m + "out_proj.bias", False))
            else:
                lw.mixer = pack_mamba2(get(m + "in_proj.weight"), get(m + "conv1d.weight"), get(m + "conv1d.bias", False),
                                       get(m + "dt_bias"), get(m + "A_log"), get(m + "D"), get(m + "norm.weight"),
                                       get(m + "out_proj.weight"), dtype, device, get(m + "in_proj.bias", False),
                                       get(m + "out_proj.bias", False))
        elif mt == "nemotron_h":
            p = f"{nemo_root}layers.{l}."
            lw = LayerWeights(attn_norm=dev(get(p + "norm.weight")), wqkv=None, wo=None, ffn_norm=None)
            m = p + "mixer."
            if kind == "mamba2":
                lw.mixer = pack_mamba2(get(m + "in_proj.weight"), get(m + "conv1d.weight"), get(m + "conv1d.bias", False),
                                       get(m + "dt_bias"), get(m + "A_log"), get(m + "D"), get(m + "norm.weight"),
                                       get(m + "out_proj.weight"), dtype, device, get(m + "in_proj.bias", False),
                                       get(m + "out_proj.bias", False))
            elif kind == "attention":
                attention(lw, m)
            elif cfg.ffn_kind(l) == "moe":          # two-matrix experts: the "gate / up" stack holds the up projections alone
                lw.router_w = dev(get(m + "gate.weight"))
                sel = get(m + "gate.e_score_correction_bias", False)
                if sel is not None:
                    lw.router_select_b = sel.float().reshape(-1).to(device).contiguous()
                up = get(m + "experts.up_proj", False)
                if up is not None:
                    lw.exp_gate_up, lw.exp_down = dev(up), dev(get(m + "experts.down_proj"))
                else:
                    E = cfg.num_experts
                    lw.exp_gate_up = dev(torch.stack([get(m + f"experts.{e}.up_proj.weight") for e in range(E)]))
                    lw.exp_down = dev(torch.stack([get(m + f"experts.{e}.down_proj.weight") for e in range(E)]))
                if cfg.shared_intermediate_size:
                    lw.shared_gate_up = dev(get(m + "shared_experts.up_proj.weight"))
                    lw.shared_down = dev(get(m + "shared_experts.down_proj.weight"))
                if cfg.moe_latent_size:
                    lw.moe_latent_in, lw.moe_latent_out = dev(get(m + "fc1_latent_proj.weight")), dev(get(m + "fc2_latent_proj.weight"))
            else:
                lw.w_gate_up, lw.w_down = dev(get(m + "up_proj.weight")), dev(get(m + "down_proj.weight"))
                if cfg.mlp_bias:
                    lw.b_up, lw.b_down = dev(get(m + "up_proj.bias")), dev(get(m + "down_proj.bias"))
        elif mt == "falcon_h1":                      # the mu-P multipliers become part of the matrices they scale
            p, mu = f"model.layers.{l}.", s["mup"]
            lw = LayerWeights(attn_norm=dev(get(p + "input_layernorm.weight")), wqkv=None, wo=None,
                              ffn_norm=dev(get(p + "pre_ff_layernorm.weight")))
            a = p + "self_attn."
            scale = {"q": mu["attn_in"], "k": mu["attn_in"] * mu["key"], "v": mu["attn_in"]}
            lw.wqkv = dev(torch.cat([get(a + f"{n}_proj.weight").float() * scale[n] for n in "qkv"], 0))
            lw.wo = dev(get(a + "o_proj.weight").float() * mu["attn_out"])
            if cfg.attn_bias and get(a + "q_proj.bias", False) is not None:
                lw.bqkv = dev(torch.cat([get(a + f"{n}_proj.bias").float() * (mu["key"] if n == "k" else 1.0) for n in "qkv"]))
                bo = get(a + "o_proj.bias", False)
                lw.bo = dev(bo.float() * mu["attn_out"]) if bo is not None else None
            m = p + "mamba."
            Di, GN, Hm = s["d_inner"], s["n_groups"] * s["d_state"], s["n_heads"]
            rows = torch.cat([torch.full((n,), float(v)) for n, v in zip((Di, Di, GN, GN, Hm), mu["ssm"])])     # z, x, B, C, dt
            w_in, b_in = get(m + "in_proj.weight").float(), get(m + "in_proj.bias", False)
            w_out, b_out = get(m + "out_proj.weight").float(), get(m + "out_proj.bias", False)
            lw.mixer = pack_mamba2(w_in * rows[:, None] * mu["ssm_in"], get(m + "conv1d.weight"), get(m + "conv1d.bias", False),
                                   get(m + "dt_bias"), get(m + "A_log"), get(m + "D"),
                                   get(m + "norm.weight", False) if s["gate_mode"] != "gate_only" else torch.ones(Di),
                                   w_out * mu["ssm_out"], dtype, device, b_in.float() * rows if b_in is not None else None,
                                   b_out.float() * mu["ssm_out"] if b_out is not None else None)
            f = p + "feed_forward."
            lw.w_gate_up = dev(torch.cat([get(f + "gate_proj.weight").float() * mu["mlp"][0], get(f + "up_proj.weight").float()], 0))
            lw.w_down = dev(get(f + "down_proj.weight").float() * mu["mlp"][1])
        elif mt == "bamba":
            p = f"model.layers.{l}."
            lw = LayerWeights(attn_norm=dev(get(p + "input_layernorm.weight")), wqkv=None, wo=None,
                              ffn_norm=dev(get(p + "pre_ff_layernorm.weight")))
            if kind == "attention":
                attention(lw, p + "self_attn.")
            else:
                m = p + "mamba."
                lw.mixer = pack_mamba2(get(m + "in_proj.weight"), get(m + "conv1d.weight"), get(m + "conv1d.bias", False),
                                       get(m + "dt_bias"), get(m + "A_log"), get(m + "D"), get(m + "norm.weight"),
                                       get(m + "out_proj.weight"), dtype, device, get(m + "in_proj.bias", False),
                                       get(m + "out_proj.bias", False))
            glu(lw, p + "feed_forward.", "gate_proj", "up_proj", "down_proj")
        elif mt == "lfm2":
            p = f"model.layers.{l}."
            lw = LayerWeights(attn_norm=dev(get(p + "operator_norm.weight")), wqkv=None, wo=None,
                              ffn_norm=dev(get(p + "ffn_norm.weight")))
            if kind == "attention":
                attention(lw, p + "self_attn.", p + "self_attn.q_layernorm.weight", p + "self_attn.k_layernorm.weight", "out_proj")
            else:
                m = p + "conv."
                cw = get(m + "conv.weight")
                lw.mixer = dict(in_proj=dev(get(m + "in_proj.weight")), conv_w=cw.reshape(cw.shape[0], -1).float().to(device).contiguous(),
                                out_proj=dev(get(m + "out_proj.weight")))
                for name, key in (("conv_b", "conv.bias"), ("in_proj_b", "in_proj.bias"), ("out_proj_b", "out_proj.bias")):
                    t = get(m + key, False)
                    if t is not None:
                        lw.mixer[name] = t.float().to(device).contiguous() if name == "conv_b" else dev(t)
            glu(lw, p + "feed_forward.", "w1", "w3", "w2")
        elif mt == "glm4_moe":
            p = f"model.layers.{l}."
            lw = LayerWeights(attn_norm=dev(get(p + "input_layernorm.weight")), wqkv=None, wo=None,
                              ffn_norm=dev(get(p + "post_attention_layernorm.weight")))
            if cfg.qk_norm:
                attention(lw, p + "self_attn.", p + "self_attn.q_norm.weight", p + "self_attn.k_norm.weight")
            else:
                attention(lw, p + "self_attn.")
            if cfg.ffn_kind(l) == "moe":
                deepseek_moe(lw, p + "mlp.")
            else:
                glu(lw, p + "mlp.", "gate_proj", "up_proj", "down_proj")
        elif mt == "granitemoehybrid":
            rm = s.get("residual_mult", 1.0)                  # block output * rm: folded into each block's last projection
            p = f"model.layers.{l}."
            lw = LayerWeights(attn_norm=dev(get(p + "input_layernorm.weight")), wqkv=None, wo=None,
                              ffn_norm=dev(get(p + "post_attention_layernorm.weight")))
            if kind == "attention":
                attention(lw, p + "self_attn.")
                lw.wo = dev(get(p + "self_attn.o_proj.weight").float() * rm)
                if lw.bo is not None:
                    lw.bo = dev(lw.bo.float() * rm)
            else:
                m = p + "mamba."
                ob = get(m + "out_proj.bias", False)
                lw.mixer = pack_mamba2(get(m + "in_proj.weight"), get(m + "conv1d.weight"), get(m + "conv1d.bias", False),
                                       get(m + "dt_bias"), get(m + "A_log"), get(m + "D"), get(m + "norm.weight"),
                                       get(m + "out_proj.weight").float() * rm, dtype, device, get(m + "in_proj.bias", False),
                                       ob.float() * rm if ob is not None else None)
            shared_in = get(p + "shared_mlp.input_linear.weight", False)
            shared_out = get(p + "shared_mlp.output_linear.weight").float() * rm if shared_in is not None else None
            if cfg.ffn_kind(l) == "moe":
                mp = p + "block_sparse_moe."
                lw.router_w = dev(get(mp + "router.layer.weight"))
                lw.exp_gate_up = dev(get(mp + "input_linear.weight"))
                lw.exp_down = dev(get(mp + "output_linear.weight").float() * rm)
                if shared_in is not None:
                    lw.shared_gate_up, lw.shared_down = dev(shared_in), dev(shared_out)
            else:
                lw.w_gate_up, lw.w_down = dev(shared_in), dev(shared_out)
        elif mt == "jamba":
            p = f"model.layers.{l}."
            lw = LayerWeights(attn_norm=dev(get(p + "input_layernorm.weight")), wqkv=None, wo=None,
                              ffn_norm=dev(get(p + "pre_ff_layernorm.weight")))
            if kind == "attention":
                attention(lw, p + "self_attn.")
            else:
                m = p + "mamba."
                lw.mixer = pack_mamba1(get(m + "in_proj.weight"), get(m + "conv1d.weight"), get(m + "conv1d.bias", False),
                                       get(m + "x_proj.weight"), get(m + "dt_proj.weight"), get(m + "dt_proj.bias"),
                                       get(m + "A_log"), get(m + "D"), get(m + "out_proj.weight"), s["d_state"], s["dt_rank"],
                                       dtype, device, get(m + "in_proj.bias", False), get(m + "out_proj.bias", False))
                for name, key in (("dt_norm_w", "dt_layernorm"), ("b_norm_w", "b_layernorm"), ("c_norm_w", "c_layernorm")):
                    lw.mixer[name] = dev(get(m + key + ".weight"))
            if cfg.ffn_kind(l) == "moe":
                mp = p + "feed_forward."
                lw.router_w = dev(get(mp + "router.weight"))
                fused = get(mp + "experts.gate_up_proj", False)
                if fused is not None:
                    lw.exp_gate_up, lw.exp_down = dev(fused), dev(get(mp + "experts.down_proj"))
                else:
                    E = cfg.num_experts
                    lw.exp_gate_up = dev(torch.stack([torch.cat([get(mp + f"experts.{e}.gate_proj.weight"),
                                                                 get(mp + f"experts.{e}.up_proj.weight")], 0) for e in range(E)]))
                    lw.exp_down = dev(torch.stack([get(mp + f"experts.{e}.down_proj.weight") for e in range(E)]))
            else:
                glu(lw, p + "feed_forward.", "gate_proj", "up_proj", "down_proj")
        elif mt in ("qwen3_next", "qwen3_5_text", "qwen3_5_moe_text"):
            from ..models.recurrent import pack_gated_delta
            p = f"{root}layers.{l}."
            lw = LayerWeights(attn_norm=dev(get(p + "input_layernorm.weight")), wqkv=None, wo=None,
                              ffn_norm=dev(get(p + "post_attention_layernorm.weight")))
            if kind == "attention":
                a, D, Hq = p + "self_attn.", cfg.head_dim, cfg.num_heads
                qg = get(a + "q_proj.weight").view(Hq, 2, D, cfg.hidden_size)         # per head: query rows, then gate rows
                lw.wqkv = dev(torch.cat([qg[:, 0].reshape(Hq * D, -1), get(a + "k_proj.weight"), get(a + "v_proj.weight")], 0))
                lw.w_attn_gate = dev(qg[:, 1].reshape(Hq * D, -1))
                lw.wo = dev(get(a + "o_proj.weight"))
                # the family's norms multiply by 1 + w; the fused QK-norm kernel multiplies by w
                lw.q_norm, lw.k_norm = dev(get(a + "q_norm.weight").float() + 1.0), dev(get(a + "k_norm.weight").float() + 1.0)
            else:
                m = p + "linear_attn."
                Hk, Hv, Dk, Dv = s["num_k_heads"], s["num_v_heads"], s["head_k_dim"], s["head_v_dim"]
                r = Hv // Hk
                Hd = cfg.hidden_size
                if get(m + "in_proj_qkv.weight", False) is not None:      # Qwen3.5: q | k | v rows in order, z / beta / a apart
                    qkv_w = get(m + "in_proj_qkv.weight")
                    parts = (qkv_w[:Hk * Dk], qkv_w[Hk * Dk:2 * Hk * Dk], qkv_w[2 * Hk * Dk:], get(m + "in_proj_z.weight"),
                             get(m + "in_proj_b.weight"), get(m + "in_proj_a.weight"))
                else:                                                      # Qwen3-Next: rows grouped per key head
                    qkvz = get(m + "in_proj_qkvz.weight").view(Hk, 2 * Dk + 2 * r * Dv, Hd)      # q | k | v | z
                    ba = get(m + "in_proj_ba.weight").view(Hk, 2 * r, Hd)
                    parts = (qkvz[:, :Dk].reshape(-1, Hd), qkvz[:, Dk:2 * Dk].reshape(-1, Hd), qkvz[:, 2 * Dk:2 * Dk + r * Dv].reshape(-1, Hd),
                             qkvz[:, 2 * Dk + r * Dv:].reshape(-1, Hd), ba[:, :r].reshape(-1, Hd), ba[:, r:].reshape(-1, Hd))
                lw.mixer = pack_gated_delta(*parts, get(m + "conv1d.weight"), get(m + "dt_bias"), get(m + "A_log"), get(m + "norm.weight"),
                                            get(m + "out_proj.weight"), dtype, device)
            if cfg.ffn_kind(l) == "moe":
                mp = p + "mlp."
                lw.router_w = dev(get(mp + "gate.weight"))
                fused = get(mp + "experts.gate_up_proj", False)
                if fused is not None:
                    lw.exp_gate_up, lw.exp_down = dev(fused), dev(get(mp + "experts.down_proj"))
                else:
                    E = cfg.num_experts
                    lw.exp_gate_up = dev(torch.stack([torch.cat([get(mp + f"experts.{e}.gate_proj.weight"),
                                                                 get(mp + f"experts.{e}.up_proj.weight")], 0) for e in range(E)]))
                    lw.exp_down = dev(torch.stack([get(mp + f"experts.{e}.down_proj.weight") for e in range(E)]))
                if cfg.shared_intermediate_size:
                    lw.shared_gate_up = dev(torch.cat([get(mp + "shared_expert.gate_proj.weight"), get(mp + "shared_expert.up_proj.weight")], 0))
                    lw.shared_down = dev(get(mp + "shared_expert.down_proj.weight"))
                    g1 = get(mp + "shared_expert_gate.weight")                         # [1, H] -> 8 rows for the GEMM's width rule
                    lw.shared_gate_w = dev(torch.cat([g1, torch.zeros(7, g1.shape[1], dtype=g1.dtype)], 0))
            else:
                glu(lw, p + "mlp.", "gate_proj", "up_proj", "down_proj")
        elif mt in ("deepseek_v2", "deepseek_v3"):
            from ..models.mla import pack_mla
            p = f"model.layers.{l}."
            lw = LayerWeights(attn_norm=dev(get(p + "input_layernorm.weight")), wqkv=None, wo=None,
                              ffn_norm=dev(get(p + "post_attention_layernorm.weight")))
            a = p + "self_attn."
            opt = lambda name: get(a + name, False)
            lw.mixer = pack_mla(opt("q_a_proj.weight"), opt("q_a_layernorm.weight"), opt("q_b_proj.weight"), opt("q_proj.weight"),
                                get(a + "kv_a_proj_with_mqa.weight"), get(a + "kv_a_layernorm.weight"), get(a + "kv_b_proj.weight"),
                                get(a + "o_proj.weight"), cfg, dtype, device)
            if cfg.ffn_kind(l) == "moe":
                deepseek_moe(lw, p + "mlp.")
            else:
                glu(lw, p + "mlp.", "gate_proj", "up_proj", "down_proj")
        else:
            raise ValueError(f"no recurrent loader for {mt!r}")
        layers.append(lw)
    if mt in ("mamba", "falcon_mamba", "mamba2"):
        embed, final = get("backbone.embeddings.weight"), get("backbone.norm_f.weight")
    elif mt == "nemotron_h":
        embed, final = get(nemo_embed or "backbone.embeddings.weight"), get(nemo_root + "norm_f.weight")
    elif mt in ("bamba", "jamba", "falcon_h1"):
        embed, final = get("model.embed_tokens.weight"), get("model.final_layernorm.weight")
    elif mt in ("qwen3_next", "qwen3_5_text", "qwen3_5_moe_text"):
        embed, final = get(root + "embed_tokens.weight"), get(root + "norm.weight")
    elif mt in ("deepseek_v2", "deepseek_v3", "granitemoehybrid", "glm4_moe"):
        embed, final = get("model.embed_tokens.weight"), get("model.norm.weight")
    else:
        embed, final = get("model.embed_tokens.weight"), get("model.embedding_norm.weight")
    head = get("lm_head.weight", False)
    embed_d = dev(embed)
    head_d = embed_d if (head is None or cfg.tie_embeddings) else dev(head)
    div = s.get("logits_div", 1.0) if s else 1.0
    if mt == "falcon_h1":                                    # logits * lm_head_multiplier
        div = 1.0 / s["mup"]["head"]
    if div != 1.0:                                           # logits / div: a head of its own, scaled once
        head_d = dev((embed if (head is None or cfg.tie_embeddings) else head).float() / div)
    return DecoderWeights(embed=embed_d, layers=layers, final_norm=dev(final), lm_head=head_d, vocab_start=0,
                          vocab_local=cfg.vocab_size)
