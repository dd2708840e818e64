"""Typed configuration: the architecture-independent decoder description, the
engine / scheduler knobs and the parallel layout, each constructible from CLI
flags, ``FLLM_*`` environment switches or JSON.

``ModelConfig`` plays the role of the reference's ``ModelConfig``
(rust/engine/src/config.rs:447-545): one description drives every decoder
family (Llama, Qwen3, gpt-oss, ...) instead of one class per architecture.
"""
from __future__ import annotations

import dataclasses
import json
import math
import os
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Sequence


@dataclass
class RopeScaling:
    kind: str = "none"            # none | linear | llama3 | yarn | factors (one divisor per frequency, as GGUF files store it)
    factor: float = 1.0
    low_freq_factor: float = 1.0
    high_freq_factor: float = 4.0
    original_max_position: int = 8192
    beta_fast: float = 32.0
    beta_slow: float = 1.0
    attn_factor: Optional[float] = None
    truncate: bool = True         # YaRN: the two correction dimensions are rounded outward (False: GPT-OSS keeps them fractional)
    freq_factors: Optional[List[float]] = None


@dataclass
class ModelConfig:
    arch: str = "llama"                  # llama | qwen3 | gpt_oss
    vocab_size: int = 32000
    hidden_size: int = 4096
    num_layers: int = 32
    num_heads: int = 32
    num_kv_heads: int = 8
    head_dim: int = 128
    intermediate_size: int = 11008
    rms_eps: float = 1e-5
    rope_theta: float = 10000.0
    rope_style: str = "neox"             # neox (rotate-half) | pair (interleaved)
    rotary_dim: Optional[int] = None     # partial rotary; None = head_dim
    rope_scaling: RopeScaling = field(default_factory=RopeScaling)
    max_position: int = 131072
    tie_embeddings: bool = False
    qk_norm: bool = False                # per-head RMSNorm on q and k (Qwen3)
    attn_bias: bool = False              # bias on q/k/v/o projections
    act: str = "swiglu"                  # swiglu | geglu | swiglu_oai
    swiglu_alpha: float = 1.702
    swiglu_limit: float = 7.0
    norm_weight_offset: float = 0.0      # 1.0 for Gemma-style (1 + w)
    embed_scale: float = 1.0
    logit_softcap: float = 0.0
    attn_softcap: float = 0.0
    sliding_window: int = 0              # 0 = full attention
    window_pattern: Optional[List[int]] = None   # per layer: 1 = windowed, 0 = full
    attn_sinks: bool = False             # learned per-head sink logit (gpt-oss)
    attn_scale: Optional[float] = None   # softmax scale when it is not head_dim ** -0.5 (Gemma-2: query_pre_attn_scalar ** -0.5)
    post_norms: bool = False             # Gemma-2: the attention and FFN outputs are normalised before the residual add
    # mixture of experts
    num_experts: int = 0
    experts_per_token: int = 0
    moe_intermediate_size: int = 0
    router_kind: str = "softmax_topk"    # softmax_topk | softmax_all | deepseek_v2 | deepseek_v3
    expert_bias: bool = False
    # DeepSeek routers: always-on shared experts (one dense GLU of this width, 0 = none), a factor on the routed
    # weights, group-limited selection (experts in `router_groups` groups, the best `router_topk_groups` kept) and
    # whether the selected weights are renormalised
    shared_intermediate_size: int = 0
    router_scale: float = 1.0
    router_groups: int = 1
    router_topk_groups: int = 1
    router_norm_topk: bool = False
    shared_gate: bool = False            # the shared experts' output is scaled by sigmoid(h . g) (Qwen3-Next)
    moe_latent_size: int = 0             # > 0: routed experts work on a down-projection of the hidden state (Nemotron-H)
    qk_norm_offset: float = 0.0          # 1.0: the per-head q / k norms multiply by 1 + w (Gemma-3)
    rope_local_theta: float = 0.0        # > 0: windowed layers rotate with this base and no scaling (Gemma-3)
    # block variants of the pre-Llama families: LayerNorm (with or without bias) instead of RMSNorm, a plain two-matrix MLP
    # (activation in `act`: gelu | gelu_tanh | relu2 | silu | relu) instead of the gated one, attention and MLP side by side
    # from one residual read (with one shared norm or one norm each), biases on the MLP and the head
    norm_kind: str = "rms"               # rms | layernorm | layernorm_nobias | none (OLMo-2: only the block outputs are normalised)
    learned_positions: bool = False      # a learned position table is added to the token embeddings (GPT-2, OPT)
    position_offset: int = 0
    qk_norm_full: bool = False           # RMSNorm over the whole q and the whole k projection (all heads at once, OLMo-2)
    clip_qkv: float = 0.0                # > 0: the q / k / v projections are clamped to [-clip, clip] (OLMo)
    mlp_kind: str = "glu"                # glu | plain
    parallel_block: bool = False
    parallel_norms: int = 1              # parallel blocks: 1 = attention and MLP read the same normed input, 2 = a norm each
    mlp_bias: bool = False
    rope_layers: Optional[List[int]] = None   # per layer: 1 = rotary embedding, 0 = none (SmolLM3); None = every layer
    use_rope: bool = True                # False: attention layers carry no position signal of their own (Jamba)
    attn_out_gate: bool = False          # the query projection also emits a gate: attention output * sigmoid(gate) (Qwen3-Next)
    # recurrent and hybrid families: the token mixer of each layer (None = attention everywhere) and whether the
    # layer has a gated FFN behind it ("glu") or is the mixer alone ("none"); `ssm` holds the mixer shapes
    # (d_inner, d_state, d_conv, n_groups, head_dim, n_heads, dt_rank, norm_groups, dt_min, dt_max, conv_bias,
    # num_k_heads, num_v_heads, head_k_dim, head_v_dim, bcdt_rms ...)
    layer_kinds: Optional[List[str]] = None      # attention | mla | mamba1 | mamba2 | gated_delta | shortconv | none (FFN-only block)
                                                 # | attention+mamba2 (both read the block's input, their outputs add: Falcon-H1)
    ffn_kinds: Optional[List[str]] = None        # glu | moe | none
    ssm: Dict[str, Any] = field(default_factory=dict)
    # multi-head latent attention (layer kind "mla"): q_lora_rank (0 = one query projection), kv_lora_rank,
    # qk_nope_head_dim, qk_rope_head_dim, v_head_dim; head_dim is then qk_nope + qk_rope and rotary_dim qk_rope
    mla: Dict[str, Any] = field(default_factory=dict)
    # weight format of the big matrices
    weight_format: str = "bf16"          # bf16 | fp8_block | nvfp4 | mxfp4 | mxfp8 | mxfp4_a8 | nvfp4_a4 | int8_w8a8 | fp8_w8a8 | q4_k | ...
    name: str = "model"
    arch_alias: str = ""                 # loader family when several model types share one (the Granite MoE variants)

    # ---- derived
    @property
    def q_size(self) -> int:
        return self.num_heads * self.head_dim

    @property
    def kv_size(self) -> int:
        return self.num_kv_heads * self.head_dim

    @property
    def rot_dim(self) -> int:
        return self.rotary_dim or self.head_dim

    @property
    def is_moe(self) -> bool:
        return self.num_experts > 0

    def layer_kind(self, layer: int) -> str:
        return self.layer_kinds[layer] if self.layer_kinds else "attention"

    def ffn_kind(self, layer: int) -> str:
        return self.ffn_kinds[layer] if self.ffn_kinds else "glu"

    @property
    def has_recurrent(self) -> bool:
        return bool(self.layer_kinds) and any(k not in ("attention", "mla", "none") for k in self.layer_kinds)

    def has_kv(self, layer: int) -> bool:
        """Whether the layer keeps keys and values (or latent rows) in the paged pool."""
        return self.layer_kind(layer) in ("attention", "mla", "attention+mamba2")

    @property
    def has_mla(self) -> bool:
        return bool(self.layer_kinds) and "mla" in self.layer_kinds

    def layer_window(self, layer: int) -> int:
        if self.sliding_window <= 0:
            return 0
        if self.window_pattern is None:
            return self.sliding_window
        return self.sliding_window if self.window_pattern[layer % len(self.window_pattern)] else 0

    def param_count(self) -> int:
        h = self.hidden_size
        attn = h * (self.q_size + 2 * self.kv_size) + self.q_size * h
        if self.is_moe:
            ffn = self.num_experts * 3 * h * self.moe_intermediate_size + h * self.num_experts
        else:
            ffn = 3 * h * self.intermediate_size
        emb = self.vocab_size * h * (1 if self.tie_embeddings else 2)
        return self.num_layers * (attn + ffn + 2 * h) + emb + h

    def to_dict(self) -> Dict[str, Any]:
        return dataclasses.asdict(self)

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "ModelConfig":
        d = dict(d)
        rs = d.pop("rope_scaling", None)
        known = {f.name for f in dataclasses.fields(cls)}
        cfg = cls(**{k: v for k, v in d.items() if k in known})
        if isinstance(rs, dict):
            cfg.rope_scaling = RopeScaling(**rs)
        elif isinstance(rs, RopeScaling):
            cfg.rope_scaling = rs
        return cfg

    @classmethod
    def from_hf_config(cls, hf: Dict[str, Any]) -> "ModelConfig":
        """Map a Hugging Face ``config.json`` to the decoder description."""
        mt = hf.get("model_type", "llama")
        if mt in ("glm4_moe_lite", "kimi_k2", "youtu"):    # DeepSeek-V3 under another name (Youtu: its dense form): the same tensors, router and latent attention
            hf = dict(hf, model_type="deepseek_v3")
            mt = "deepseek_v3"
        if mt == "gemma3" and isinstance(hf.get("text_config"), dict):     # the multimodal wrapper: its language model
            hf = dict(hf["text_config"], model_type="gemma3_text")
            mt = "gemma3_text"
        if mt in ("qwen3_5", "qwen3_5_moe") and isinstance(hf.get("text_config"), dict):
            hf = dict(hf["text_config"])
            mt = hf.setdefault("model_type", mt + "_text")
        rp = hf.get("rope_parameters") or {}
        rp_local = None
        if isinstance(rp.get("full_attention"), dict):                     # per layer type: global layers / windowed layers
            rp_local, rp = rp.get("sliding_attention") or {}, rp["full_attention"]
        if rp:                                 # newer configs keep the RoPE base and scaling in one dictionary
            hf = dict(hf)
            hf.setdefault("rope_theta", rp.get("rope_theta", 10000.0))
            if rp.get("rope_type", "default") != "default" and not hf.get("rope_scaling"):
                hf["rope_scaling"] = rp
            if rp.get("partial_rotary_factor") is not None:
                hf.setdefault("partial_rotary_factor", rp["partial_rotary_factor"])
        if mt in RECURRENT_MODEL_TYPES:
            return recurrent_from_hf(cls, hf)
        if mt in ("deepseek_v2", "deepseek_v3"):
            return mla_from_hf(cls, hf)
        if mt in CLASSIC_MODEL_TYPES:
            return classic_from_hf(cls, hf)
        if mt not in ATTENTION_MODEL_TYPES:
            raise ValueError(f"model_type {mt!r} is not among the families this engine runs "
                             f"({', '.join(sorted(ATTENTION_MODEL_TYPES + CLASSIC_MODEL_TYPES + RECURRENT_MODEL_TYPES + ('deepseek_v2', 'deepseek_v3')))})")
        heads = hf["num_attention_heads"]
        hidden = hf["hidden_size"]
        cfg = cls(
            arch={"qwen3": "qwen3", "gpt_oss": "gpt_oss"}.get(mt, "llama"),
            vocab_size=hf["vocab_size"], hidden_size=hidden, num_layers=hf["num_hidden_layers"],
            num_heads=heads, num_kv_heads=hf.get("num_key_value_heads", heads),
            head_dim=hf.get("head_dim") or hidden // heads,
            intermediate_size=hf.get("intermediate_size", 4 * hidden),
            rms_eps=hf.get("rms_norm_eps", 1e-5), rope_theta=hf.get("rope_theta", 10000.0),
            max_position=hf.get("max_position_embeddings", 8192),
            tie_embeddings=hf.get("tie_word_embeddings", False),
            qk_norm=(mt in ("qwen3", "qwen3_moe")),
            attn_bias=hf.get("attention_bias", mt in ("qwen2", "qwen2_moe")),     # Qwen2 has q/k/v biases without a flag
            name=hf.get("_name_or_path", mt) or mt,
        )
        rs = hf.get("rope_scaling") or {}
        kind = rs.get("rope_type") or rs.get("type")
        if kind in ("linear", "llama3", "yarn"):
            cfg.rope_scaling = RopeScaling(
                kind=kind, factor=rs.get("factor", 1.0),
                low_freq_factor=rs.get("low_freq_factor", 1.0),
                high_freq_factor=rs.get("high_freq_factor", 4.0),
                original_max_position=rs.get("original_max_position_embeddings", 8192),
                beta_fast=rs.get("beta_fast", 32.0), beta_slow=rs.get("beta_slow", 1.0),
                attn_factor=rs.get("attention_factor"), truncate=bool(rs.get("truncate", True)))
        if mt == "gpt_oss":
            cfg.act = "swiglu_oai"
            cfg.attn_sinks = True
            cfg.attn_bias = True
            cfg.expert_bias = True
            cfg.sliding_window = hf.get("sliding_window", 128)
            lt = hf.get("layer_types")
            cfg.window_pattern = ([1 if t == "sliding_attention" else 0 for t in lt] if lt else [1, 0])
            cfg.num_experts = hf.get("num_local_experts", 0)
            cfg.experts_per_token = hf.get("num_experts_per_tok", hf.get("experts_per_token", 4))
            cfg.moe_intermediate_size = hf.get("intermediate_size", hidden)
            cfg.swiglu_limit = hf.get("swiglu_limit", 7.0)
        elif hf.get("num_local_experts") or hf.get("num_experts"):
            cfg.num_experts = hf.get("num_local_experts") or hf.get("num_experts")
            cfg.experts_per_token = hf.get("num_experts_per_tok", 2)
            cfg.moe_intermediate_size = hf.get("moe_intermediate_size", cfg.intermediate_size)
            # Mixtral: softmax over the selected logits. Qwen-MoE: softmax over all experts, then the selected
            # probabilities renormalised (norm_topk_prob)
            cfg.router_kind = "softmax_topk" if mt == "mixtral" else "softmax_all"
            if mt in ("qwen2_moe", "qwen3_moe", "olmoe") and not hf.get("norm_topk_prob", False):
                # the selected probabilities are used as they are (Qwen1.5-MoE, Qwen2-57B-A14B): the score-weighted router
                cfg.router_kind, cfg.router_norm_topk, cfg.router_scale = "deepseek_v2", False, 1.0
        if mt == "minimax_m2":                # q and k normalised over all heads, partial rotary, sigmoid router with a selection bias
            cfg.qk_norm_full = bool(hf.get("use_qk_norm", True))
            cfg.router_kind, cfg.router_norm_topk, cfg.router_scale = "deepseek_v3", True, float(hf.get("routed_scaling_factor") or 1.0)
            rot = hf.get("rotary_dim") or int(cfg.head_dim * float(hf.get("partial_rotary_factor", 1.0)))
            cfg.rotary_dim = rot if rot != cfg.head_dim else None
        if mt == "olmoe":                     # OLMoE: q and k normalised over all heads, optional clamp of q / k / v
            cfg.qk_norm_full, cfg.clip_qkv = True, float(hf.get("clip_qkv") or 0.0)
        if mt in ("gemma", "gemma2", "gemma3_text", "vaultgemma"):
            cfg.norm_weight_offset = 1.0
            cfg.embed_scale = float(hidden) ** 0.5
            cfg.act = "geglu"
            cfg.tie_embeddings = hf.get("tie_word_embeddings", True)
            cfg.logit_softcap = float(hf.get("final_logit_softcapping") or 0.0)
            cfg.attn_softcap = float(hf.get("attn_logit_softcapping") or 0.0)
        if mt == "gemma3_text":               # Gemma-3: QK-norm with 1 + w weights, a RoPE base of their own for windowed layers
            cfg.qk_norm, cfg.qk_norm_offset = True, 1.0
            cfg.rope_local_theta = float((rp_local or {}).get("rope_theta", hf.get("rope_local_base_freq", 10000.0)))
            if not hf.get("layer_types") and hf.get("sliding_window"):
                pat = hf.get("sliding_window_pattern", 6)
                hf = dict(hf, layer_types=["full_attention" if (i + 1) % pat == 0 else "sliding_attention"
                                           for i in range(hf["num_hidden_layers"])])
        if mt in ("gemma2", "gemma3_text", "vaultgemma"):
            cfg.post_norms = mt != "vaultgemma"           # VaultGemma: Gemma-2 without the norms behind the blocks
            if hf.get("query_pre_attn_scalar"):
                cfg.attn_scale = float(hf["query_pre_attn_scalar"]) ** -0.5
            if hf.get("sliding_window"):
                cfg.sliding_window = int(hf["sliding_window"])
                lt = hf.get("layer_types")
                cfg.window_pattern = [1 if t == "sliding_attention" else 0 for t in lt] if lt else [1, 0]
        if mt in ("glm", "glm4", "ernie4_5", "helium"):       # these rotate neighbouring pairs (x[2i], x[2i+1])
            cfg.rope_style = "pair"
        if mt == "glm4":                      # GLM-4-0414: the attention and MLP outputs are normalised too
            cfg.post_norms = True
        if mt in ("glm", "glm4"):
            cfg.rotary_dim = int(cfg.head_dim * hf.get("partial_rotary_factor", 0.5)) or None
            cfg.attn_bias = hf.get("attention_bias", True)
        if mt == "smollm3" and hf.get("no_rope_layers"):          # 1 = the layer rotates, 0 = no position signal in that layer
            cfg.rope_layers = [int(v) for v in hf["no_rope_layers"]]
        if mt == "granite":                   # llama with four multipliers; the residual and logit ones are folded into weights at load
            cfg.embed_scale = float(hf.get("embedding_multiplier") or 1.0)
            if hf.get("attention_multiplier"):
                cfg.attn_scale = float(hf["attention_multiplier"])
        if mt in ("phi3", "phi"):
            cfg.rotary_dim = int(cfg.head_dim * hf.get("partial_rotary_factor", 1.0)) or None
        if hf.get("sliding_window") and hf.get("use_sliding_window", mt in ("mistral", "ministral", "cwm")):
            cfg.sliding_window = hf["sliding_window"]
            lt = hf.get("layer_types")
            if lt and cfg.window_pattern is None and any(t != "sliding_attention" for t in lt):
                cfg.window_pattern = [1 if t == "sliding_attention" else 0 for t in lt]
        return cfg


# decoder families whose layers are attention + gated FFN (or routed experts) and that the generic mapping covers; every one
# of them is checked against `transformers` in tests/test_hf_parity_cpu.py
ATTENTION_MODEL_TYPES = ("llama", "mistral", "ministral", "cwm", "qwen2", "qwen3", "qwen2_moe", "qwen3_moe", "olmoe", "minimax_m2", "mixtral", "gemma", "gemma2",
                         "gemma3_text", "vaultgemma", "phi3", "gpt_oss", "granite", "seed_oss", "glm", "glm4", "ernie4_5", "helium", "smollm3")


CLASSIC_MODEL_TYPES = ("starcoder2", "stablelm", "nemotron", "arcee", "phi", "gpt_neox", "cohere", "cohere2", "olmo", "olmo2", "olmo3", "exaone4", "falcon", "jais2", "gpt2",
                       "gpt_bigcode", "opt")
_ACT_NAMES = {"gelu": "gelu", "gelu_new": "gelu_tanh", "gelu_pytorch_tanh": "gelu_tanh", "gelu_fast": "gelu_tanh", "relu2": "relu2",
              "silu": "silu", "swish": "silu", "relu": "relu"}


def classic_from_hf(cls, hf: Dict[str, Any]) -> "ModelConfig":
    """Families built from LayerNorm, plain MLPs or parallel blocks (the reference covers them through the same decoder,
    rust/engine/src/config.rs fields `norm`, `ffn`, `parallel_residual`)."""
    mt = hf["model_type"]
    if mt in ("gpt2", "gpt_bigcode"):     # their own field names
        hf = dict(hf, hidden_size=hf["n_embd"], num_hidden_layers=hf["n_layer"], num_attention_heads=hf["n_head"],
                  intermediate_size=hf.get("n_inner") or 4 * hf["n_embd"], max_position_embeddings=hf.get("n_positions", 1024),
                  hidden_act=hf.get("activation_function", "gelu_new"))
    if mt == "falcon":                    # its own field names; three layouts of the fused q|k|v rows
        if hf.get("alibi"):
            raise NotImplementedError("falcon with ALiBi position biases is not supported")
        new = bool(hf.get("new_decoder_architecture", False))
        kv = (hf.get("num_kv_heads") or hf["num_attention_heads"]) if new else (1 if hf.get("multi_query", True) else hf["num_attention_heads"])
        hf = dict(hf, num_key_value_heads=kv, intermediate_size=hf.get("ffn_hidden_size") or 4 * hf["hidden_size"],
                  hidden_act=hf.get("activation", "gelu"))
    if mt == "opt":
        if hf.get("word_embed_proj_dim") not in (None, hf["hidden_size"]) or not hf.get("do_layer_norm_before", True):
            raise NotImplementedError("OPT with projected embeddings or post-LayerNorm blocks (350m) is not supported")
        hf = dict(hf, intermediate_size=hf["ffn_dim"], hidden_act=hf.get("activation_function", "relu"))
    hidden, L, heads = hf["hidden_size"], hf["num_hidden_layers"], hf["num_attention_heads"]
    head_dim = hf.get("head_dim") or hidden // heads
    act = _ACT_NAMES.get(hf.get("hidden_act", "gelu"), "gelu")
    cfg = cls(arch=mt, name=hf.get("_name_or_path") or mt, vocab_size=hf["vocab_size"], hidden_size=hidden, num_layers=L, num_heads=heads,
              num_kv_heads=hf.get("num_key_value_heads") or heads, head_dim=head_dim, intermediate_size=hf.get("intermediate_size", 4 * hidden),
              rope_theta=hf.get("rope_theta", 10000.0), max_position=hf.get("max_position_embeddings", 4096),
              tie_embeddings=hf.get("tie_word_embeddings", False))
    prf = hf.get("partial_rotary_factor", hf.get("rotary_pct"))
    if prf is not None and float(prf) < 1.0:
        cfg.rotary_dim = int(head_dim * float(prf)) or None
    if mt == "starcoder2":
        cfg.norm_kind, cfg.mlp_kind, cfg.act, cfg.rms_eps = "layernorm", "plain", act, hf.get("norm_epsilon", 1e-5)
        cfg.attn_bias = cfg.mlp_bias = bool(hf.get("use_bias", True))
        cfg.tie_embeddings = hf.get("tie_word_embeddings", True)
        if hf.get("sliding_window"):
            cfg.sliding_window = int(hf["sliding_window"])
    elif mt == "stablelm":
        if hf.get("qk_layernorm") or hf.get("use_parallel_residual"):
            raise NotImplementedError("stablelm with per-head QK LayerNorm or parallel residual is not supported")
        cfg.norm_kind, cfg.rms_eps, cfg.attn_bias = "layernorm", hf.get("layer_norm_eps", 1e-5), bool(hf.get("use_qkv_bias", False))
    elif mt == "nemotron":                # LayerNorm whose weight is stored minus one, squared-ReLU MLP
        cfg.norm_kind, cfg.norm_weight_offset, cfg.rms_eps = "layernorm", 1.0, hf.get("norm_eps", 1e-5)
        cfg.mlp_kind, cfg.act, cfg.attn_bias, cfg.mlp_bias = "plain", act, bool(hf.get("attention_bias", False)), bool(hf.get("mlp_bias", False))
    elif mt == "jais2":                   # Llama blocks with LayerNorm (weight and bias) and a squared-ReLU two-matrix MLP
        cfg.norm_kind, cfg.rms_eps = "layernorm", hf.get("layer_norm_eps", 1e-5)
        cfg.mlp_kind, cfg.act, cfg.attn_bias, cfg.mlp_bias = "plain", act, bool(hf.get("attention_bias", True)), bool(hf.get("mlp_bias", True))
    elif mt == "arcee":
        cfg.mlp_kind, cfg.act, cfg.rms_eps = "plain", act, hf.get("rms_norm_eps", 1e-5)
        cfg.attn_bias, cfg.mlp_bias = bool(hf.get("attention_bias", False)), bool(hf.get("mlp_bias", False))
    elif mt == "phi":
        if hf.get("qk_layernorm"):
            raise NotImplementedError("phi with QK LayerNorm is not supported")
        cfg.norm_kind, cfg.mlp_kind, cfg.act, cfg.rms_eps = "layernorm", "plain", act, hf.get("layer_norm_eps", 1e-5)
        cfg.parallel_block, cfg.parallel_norms, cfg.attn_bias, cfg.mlp_bias = True, 1, True, True
    elif mt == "gpt_neox":
        cfg.norm_kind, cfg.mlp_kind, cfg.act, cfg.rms_eps = "layernorm", "plain", act, hf.get("layer_norm_eps", 1e-5)
        cfg.parallel_block, cfg.parallel_norms = bool(hf.get("use_parallel_residual", True)), 2
        cfg.attn_bias, cfg.mlp_bias = bool(hf.get("attention_bias", True)), True
    elif mt in ("gpt2", "opt", "gpt_bigcode"):           # learned absolute positions, LayerNorm, plain MLP, biases everywhere, tied head
        cfg.norm_kind, cfg.mlp_kind, cfg.act = "layernorm", "plain", act
        cfg.rms_eps = hf.get("layer_norm_epsilon", 1e-5)
        cfg.use_rope, cfg.learned_positions, cfg.attn_bias, cfg.mlp_bias = False, True, True, True
        cfg.position_offset = 2 if mt == "opt" else 0            # OPT's table starts two rows in
        cfg.tie_embeddings = hf.get("tie_word_embeddings", True)
        if mt == "gpt_bigcode" and hf.get("multi_query", True):          # one key / value head for all query heads
            cfg.num_kv_heads = 1
    elif mt == "olmo":                    # LayerNorm without weights, optionally clamped q / k / v
        cfg.norm_kind, cfg.rms_eps, cfg.attn_bias = "layernorm_nobias", 1e-5, bool(hf.get("attention_bias", False))
        cfg.clip_qkv = float(hf.get("clip_qkv") or 0.0)
    elif mt in ("olmo2", "olmo3"):        # no norm in front of a block: its output is normalised instead; q and k normalised over all heads
        cfg.norm_kind, cfg.post_norms, cfg.qk_norm_full, cfg.rms_eps = "none", True, True, hf.get("rms_norm_eps", 1e-6)
        cfg.attn_bias = bool(hf.get("attention_bias", False))
        lt = hf.get("layer_types")
        if mt == "olmo3" and hf.get("sliding_window") and lt:
            cfg.sliding_window = int(hf["sliding_window"])
            cfg.window_pattern = [1 if t == "sliding_attention" else 0 for t in lt]
    elif mt == "falcon":
        new = bool(hf.get("new_decoder_architecture", False))
        cfg.norm_kind, cfg.mlp_kind, cfg.act, cfg.rms_eps = "layernorm", "plain", act, hf.get("layer_norm_epsilon", 1e-5)
        cfg.parallel_block = new or bool(hf.get("parallel_attn", True))
        cfg.parallel_norms = 2 if (new and (hf.get("num_ln_in_parallel_attn") or 2) == 2) else 1
        cfg.attn_bias = cfg.mlp_bias = bool(hf.get("bias", False))
        cfg.ssm = dict(qkv_layout="grouped" if new else ("flat" if cfg.num_kv_heads == 1 else "per_head"))
    elif mt == "exaone4":                 # blocks normalised at their output, per-head QK-norm, windowed layers rotate and global ones do not
        cfg.norm_kind, cfg.post_norms, cfg.qk_norm, cfg.rms_eps = "none", True, True, hf.get("rms_norm_eps", 1e-5)
        lt = hf.get("layer_types")
        if hf.get("sliding_window") and lt and "sliding_attention" in lt:
            cfg.sliding_window = int(hf["sliding_window"])
            cfg.window_pattern = [1 if t == "sliding_attention" else 0 for t in lt]
            cfg.rope_layers = list(cfg.window_pattern)
    elif mt in ("cohere", "cohere2"):
        if hf.get("use_qk_norm"):
            raise NotImplementedError("cohere with QK norm is not supported")
        cfg.norm_kind, cfg.rms_eps, cfg.parallel_block, cfg.parallel_norms = "layernorm_nobias", hf.get("layer_norm_eps", 1e-5), True, 1
        cfg.rope_style, cfg.tie_embeddings = "pair", hf.get("tie_word_embeddings", True)
        cfg.attn_bias = bool(hf.get("attention_bias", False))
        cfg.ssm = dict(logit_mult=float(hf.get("logit_scale") or 1.0))       # folded into the head at load
        if mt == "cohere2":               # windowed layers rotate, the global ones carry no position signal
            pat = hf.get("sliding_window_pattern", 4)
            lt = hf.get("layer_types") or ["sliding_attention" if (i + 1) % pat else "full_attention" for i in range(L)]
            cfg.window_pattern = [1 if t == "sliding_attention" else 0 for t in lt]
            cfg.rope_layers = list(cfg.window_pattern)
            cfg.sliding_window = int(hf.get("sliding_window") or 4096)
    return cfg


def _yarn_mscale(factor: float, m: float) -> float:
    return 1.0 if factor <= 1.0 or not m else 0.1 * m * math.log(factor) + 1.0


def mla_from_hf(cls, hf: Dict[str, Any]) -> "ModelConfig":
    """DeepSeek-V2 / V3 (rust/engine/src/config.rs reads the same shapes from GGUF metadata): latent attention in every
    layer, dense feed-forward layers first, then routed experts with always-on shared experts and the family's routers
    (V2: softmax scores, optionally group-limited; V3: sigmoid scores with a selection bias, groups ranked by their two
    best experts, renormalised weights)."""
    mt = hf["model_type"]
    L, hidden, heads = hf["num_hidden_layers"], hf["hidden_size"], hf["num_attention_heads"]
    dn, dr = hf.get("qk_nope_head_dim", 128), hf.get("qk_rope_head_dim", 64)
    cfg = cls(arch=mt, name=hf.get("_name_or_path") or mt, vocab_size=hf["vocab_size"], hidden_size=hidden, num_layers=L,
              num_heads=heads, num_kv_heads=1, head_dim=dn + dr, rotary_dim=dr, rope_style="pair",
              intermediate_size=hf["intermediate_size"], rms_eps=hf.get("rms_norm_eps", 1e-6),
              rope_theta=hf.get("rope_theta", 10000.0), max_position=hf.get("max_position_embeddings", 4096),
              tie_embeddings=hf.get("tie_word_embeddings", False), layer_kinds=["mla"] * L,
              mla=dict(q_lora_rank=hf.get("q_lora_rank") or 0, kv_lora_rank=hf.get("kv_lora_rank", 512), qk_nope_head_dim=dn,
                       qk_rope_head_dim=dr, v_head_dim=hf.get("v_head_dim", 128)))
    dense_first = hf.get("first_k_dense_replace", 0)
    if hf.get("n_routed_experts") and dense_first < L:
        step = hf.get("moe_layer_freq", 1) or 1
        cfg.ffn_kinds = ["moe" if (i >= dense_first and i % step == 0) else "glu" for i in range(L)]
        cfg.num_experts = hf["n_routed_experts"]
        cfg.experts_per_token = hf.get("num_experts_per_tok") or 2
        cfg.moe_intermediate_size = hf.get("moe_intermediate_size", cfg.intermediate_size)
        cfg.shared_intermediate_size = (hf.get("n_shared_experts") or 0) * cfg.moe_intermediate_size
        cfg.router_scale = float(hf.get("routed_scaling_factor", 1.0))
        cfg.router_norm_topk = bool(hf.get("norm_topk_prob", mt == "deepseek_v3"))
        grouped = mt == "deepseek_v3" or hf.get("topk_method") == "group_limited_greedy"
        cfg.router_groups = (hf.get("n_group") or 1) if grouped else 1
        cfg.router_topk_groups = (hf.get("topk_group") or 1) if grouped else 1
        cfg.router_kind = mt
    rs = hf.get("rope_scaling") or {}
    if (rs.get("rope_type") or rs.get("type")) == "yarn":
        f = float(rs.get("factor", 1.0))
        af = rs.get("attention_factor")
        if af is None and rs.get("mscale") and rs.get("mscale_all_dim"):
            af = _yarn_mscale(f, rs["mscale"]) / _yarn_mscale(f, rs["mscale_all_dim"])
        cfg.rope_scaling = RopeScaling(kind="yarn", factor=f, original_max_position=rs.get("original_max_position_embeddings", 4096),
                                       beta_fast=rs.get("beta_fast", 32.0), beta_slow=rs.get("beta_slow", 1.0), attn_factor=af,
                                       truncate=bool(rs.get("truncate", True)))
        if mt == "deepseek_v3" and rs.get("mscale_all_dim"):        # V3 also scales the softmax by mscale squared
            cfg.attn_scale = (dn + dr) ** -0.5 * _yarn_mscale(f, rs["mscale_all_dim"]) ** 2
    return cfg


RECURRENT_MODEL_TYPES = ("falcon_h1", "nemotron_h", "nemotron_h_moe", "mamba", "falcon_mamba", "mamba2", "bamba", "lfm2", "rwkv7", "qwen3_next", "qwen3_5_text", "qwen3_5_moe_text", "jamba", "granitemoehybrid", "granitemoe", "granitemoeshared", "glm4_moe", "ernie4_5_moe", "rwkv6")


def _limit(v, default: float) -> float:
    """One end of a time-step limit as a config file spells it: a number, or infinity as a string / tagged value."""
    if isinstance(v, dict):
        v = next(iter(v.values()), None)
    try:
        f = float(v)
    except (TypeError, ValueError):
        return default
    return max(min(f, 1e30), -1e30)


def nemotron_h_from_hf(cls, hf: Dict[str, Any]) -> "ModelConfig":
    """Nemotron-H (the reference lists it with the Mamba-2 hybrids in docs/architectures.md and reads its per-layer
    pattern in rust/engine/src/config.rs): every block is ONE of a Mamba-2 mixer, an attention without rotary
    embedding, a two-matrix relu^2 MLP, or a mixture of such MLPs (sigmoid router with a selection bias, optional
    latent projection around the routed experts, a shared MLP on the hidden state), behind one RMSNorm."""
    blocks = hf.get("layers_block_type")
    if not blocks:
        names = {"M": "mamba", "*": "attention", "-": "mlp", "E": "moe"}
        blocks = [names[c] for c in hf.get("hybrid_override_pattern", "")]
    if not blocks:
        raise ValueError("nemotron_h: the config names no block pattern (layers_block_type / hybrid_override_pattern)")
    hidden, heads = hf["hidden_size"], hf["num_attention_heads"]
    H, P = hf.get("mamba_num_heads", 128), hf.get("mamba_head_dim", 64)
    G = hf.get("n_groups", hf.get("mamba_n_groups", 8))
    lim = hf.get("time_step_limit") or hf.get("mamba_dt_limit") or (0.0, float("inf"))
    E = hf.get("n_routed_experts", 0) if "moe" in blocks else 0
    kind = {"mamba": "mamba2", "attention": "attention", "mlp": "none", "moe": "none"}
    ffn = {"mamba": "none", "attention": "none", "mlp": "glu", "moe": "moe"}
    return cls(arch="nemotron_h", name=hf.get("_name_or_path") or "nemotron_h", vocab_size=hf["vocab_size"], hidden_size=hidden,
               num_layers=len(blocks), num_heads=heads, num_kv_heads=hf.get("num_key_value_heads", heads),
               head_dim=hf.get("head_dim") or hf.get("attention_head_dim") or hidden // heads,
               max_position=hf.get("max_position_embeddings", 8192), use_rope=False,
               intermediate_size=hf.get("intermediate_size", 0), rms_eps=hf.get("layer_norm_epsilon", hf.get("rms_norm_eps", 1e-5)),
               tie_embeddings=hf.get("tie_word_embeddings", False), attn_bias=hf.get("attention_bias", False),
               mlp_kind="plain", act=hf.get("mlp_hidden_act", "relu2"), mlp_bias=bool(hf.get("mlp_bias", False)),
               layer_kinds=[kind[b] for b in blocks], ffn_kinds=[ffn[b] for b in blocks],
               num_experts=E, experts_per_token=hf.get("num_experts_per_tok", 2) if E else 0,
               moe_intermediate_size=hf.get("moe_intermediate_size", 0) if E else 0,
               shared_intermediate_size=(hf.get("moe_shared_expert_intermediate_size", 0) if hf.get("n_shared_experts", 1) else 0) if E else 0,
               moe_latent_size=(hf.get("moe_latent_size") or 0) if E else 0,
               router_kind="deepseek_v3", router_scale=float(hf.get("routed_scaling_factor", 1.0)),
               router_norm_topk=bool(hf.get("norm_topk_prob", True)), router_groups=hf.get("n_group") or 1,
               router_topk_groups=hf.get("topk_group") or 1,
               ssm=dict(d_inner=H * P, d_state=hf.get("ssm_state_size", 128), d_conv=hf.get("conv_kernel", hf.get("mamba_d_conv", 4)),
                        n_groups=G, head_dim=P, n_heads=H, norm_groups=G,
                        conv_bias=hf.get("use_conv_bias", True), proj_bias=hf.get("use_bias", hf.get("mamba_proj_bias", False)),
                        dt_min=_limit(lim[0], 0.0), dt_max=_limit(lim[1], 1e30)))


def recurrent_from_hf(cls, hf: Dict[str, Any]) -> "ModelConfig":
    """Recurrent and hybrid families (the reference describes them in rust/engine/src/config.rs next to the
    attention fields and in rust/engine/src/hybrid_config.rs): which mixer each layer runs and its shapes."""
    mt = hf["model_type"]
    if mt in ("nemotron_h", "nemotron_h_moe"):
        return nemotron_h_from_hf(cls, hf)
    hidden, L = hf["hidden_size"], hf["num_hidden_layers"]
    if mt in ("mamba", "falcon_mamba"):
        d_inner = hf.get("intermediate_size") or hf.get("expand", 2) * hidden
        rank = hf.get("time_step_rank", "auto")
        rank = -(-hidden // 16) if rank == "auto" else int(rank)
        return cls(arch=mt, name=hf.get("_name_or_path") or mt, vocab_size=hf["vocab_size"], hidden_size=hidden,
                   num_layers=L, num_heads=1, num_kv_heads=1, head_dim=64, intermediate_size=0,
                   rms_eps=hf.get("layer_norm_epsilon", 1e-5), tie_embeddings=hf.get("tie_word_embeddings", True),
                   layer_kinds=["mamba1"] * L, ffn_kinds=["none"] * L,
                   ssm=dict(d_inner=d_inner, d_state=hf.get("state_size", 16), d_conv=hf.get("conv_kernel", 4),
                            dt_rank=rank, conv_bias=hf.get("use_conv_bias", True), proj_bias=hf.get("use_bias", False),
                            bcdt_rms=(mt == "falcon_mamba"), mixer_rms_eps=hf.get("mixer_rms_eps", 1e-6)))
    if mt == "mamba2":
        H, P = hf.get("num_heads", 128), hf.get("head_dim", 64)
        lim = hf.get("time_step_limit") or (0.0, float("inf"))
        return cls(arch=mt, name=hf.get("_name_or_path") or mt, vocab_size=hf["vocab_size"], hidden_size=hidden,
                   num_layers=L, num_heads=1, num_kv_heads=1, head_dim=64, intermediate_size=0,
                   rms_eps=hf.get("layer_norm_epsilon", 1e-5), tie_embeddings=hf.get("tie_word_embeddings", False),
                   layer_kinds=["mamba2"] * L, ffn_kinds=["none"] * L,
                   ssm=dict(d_inner=H * P, d_state=hf.get("state_size", 128), d_conv=hf.get("conv_kernel", 4),
                            n_groups=hf.get("n_groups", 8), head_dim=P, n_heads=H, norm_groups=1,
                            conv_bias=hf.get("use_conv_bias", True), proj_bias=hf.get("use_bias", False),
                            dt_min=_limit(lim[0], 0.0), dt_max=_limit(lim[1], 1e30)))
    if mt == "rwkv6":
        N = hf.get("head_size", 64)
        inter = hf.get("intermediate_size") or int(hidden * 3.5) // 32 * 32
        return cls(arch=mt, name=hf.get("_name_or_path") or mt, vocab_size=hf["vocab_size"], hidden_size=hidden, num_layers=L,
                   num_heads=hidden // N, num_kv_heads=hidden // N, head_dim=N, intermediate_size=inter,
                   rms_eps=hf.get("layer_norm_epsilon", 1e-5), tie_embeddings=False, layer_kinds=["rwkv6"] * L, ffn_kinds=["none"] * L,
                   ssm=dict(head_dim=N, d_conv=2, head_size_divisor=hf.get("head_size_divisor", 8),
                            mix_rank=hf.get("time_mix_extra_dim", 32), decay_rank=hf.get("time_decay_extra_dim", 64)))
    if mt == "rwkv7":
        N = hf.get("head_dim", 64)
        inter = hf.get("intermediate_size") or int(hf.get("hidden_ratio", 4.0) * hidden)
        return cls(arch=mt, name=hf.get("_name_or_path") or mt, vocab_size=hf["vocab_size"], hidden_size=hidden, num_layers=L,
                   num_heads=hidden // N, num_kv_heads=hidden // N, head_dim=N, intermediate_size=inter,
                   rms_eps=hf.get("norm_eps", 1e-5), tie_embeddings=False, layer_kinds=["rwkv7"] * L, ffn_kinds=["none"] * L,
                   ssm=dict(head_dim=N, d_conv=2, decay_rank=hf.get("decay_low_rank_dim", 64), a_rank=hf.get("a_low_rank_dim", 64),
                            v_rank=hf.get("v_low_rank_dim", 32), gate_rank=hf.get("gate_low_rank_dim", 128)))
    heads = hf["num_attention_heads"]
    head_dim = hf.get("head_dim") or hidden // heads
    base = dict(arch=mt, name=hf.get("_name_or_path") or mt, vocab_size=hf["vocab_size"], hidden_size=hidden, num_layers=L,
                num_heads=heads, num_kv_heads=hf.get("num_key_value_heads", heads), head_dim=head_dim,
                rope_theta=hf.get("rope_theta", 10000.0), max_position=hf.get("max_position_embeddings", 8192))
    if mt == "falcon_h1":
        # Falcon-H1 (docs/architectures.md of the reference: Mamba-2 and attention side by side in every layer, the mu-P
        # multipliers folded into the weights): the loader scales the projections, `embed_scale` the embeddings
        H = hf.get("mamba_n_heads", 128)
        Di = hf.get("mamba_d_ssm") or hf.get("mamba_expand", 2) * hidden
        P = hf.get("mamba_d_head", "auto")
        P = Di // H if P in ("auto", None) else int(P)
        lim = hf.get("time_step_limit") or (0.0, float("inf"))
        rope = hf.get("rope_parameters") or {}
        base["rope_theta"] = rope.get("rope_theta", hf.get("rope_theta", 10000.0))
        gate_mode = "gate_only" if not hf.get("mamba_rms_norm", False) else \
            ("norm_before_gate" if hf.get("mamba_norm_before_gate", True) else "norm_after_gate")
        return cls(**base, intermediate_size=hf["intermediate_size"], rms_eps=hf.get("rms_norm_eps", 1e-5),
                   tie_embeddings=hf.get("tie_word_embeddings", False), attn_bias=hf.get("attention_bias", False),
                   embed_scale=float(hf.get("embedding_multiplier", 1.0)),
                   layer_kinds=["attention+mamba2"] * L,
                   ssm=dict(d_inner=Di, d_state=hf.get("mamba_d_state", 256), d_conv=hf.get("mamba_d_conv", 4),
                            n_groups=hf.get("mamba_n_groups", 1), head_dim=P, n_heads=H, norm_groups=hf.get("mamba_n_groups", 1),
                            gate_mode=gate_mode, conv_bias=hf.get("mamba_conv_bias", True), proj_bias=hf.get("mamba_proj_bias", False),
                            dt_min=_limit(lim[0], 0.0), dt_max=_limit(lim[1], 1e30),
                            mup=dict(ssm=list(hf.get("ssm_multipliers") or [1.0] * 5), ssm_in=float(hf.get("ssm_in_multiplier", 1.0)),
                                     ssm_out=float(hf.get("ssm_out_multiplier", 1.0)), attn_in=float(hf.get("attention_in_multiplier", 1.0)),
                                     attn_out=float(hf.get("attention_out_multiplier", 1.0)), key=float(hf.get("key_multiplier", 1.0)),
                                     mlp=list(hf.get("mlp_multipliers") or [1.0, 1.0]), head=float(hf.get("lm_head_multiplier", 1.0)))))
    if mt == "bamba":
        H = hf.get("mamba_n_heads", 128)
        P = hf.get("mamba_d_head", "auto")
        P = hf.get("mamba_expand", 2) * hidden // H if P == "auto" else int(P)
        attn = set(hf.get("attn_layer_indices") or [])
        lim = hf.get("time_step_limit") or (0.0, float("inf"))
        rot = int(head_dim * hf.get("partial_rotary_factor", 0.5))
        return cls(**base, intermediate_size=hf["intermediate_size"], rms_eps=hf.get("rms_norm_eps", 1e-5),
                   tie_embeddings=hf.get("tie_word_embeddings", False), attn_bias=hf.get("attention_bias", False),
                   rotary_dim=rot if rot != head_dim else None,
                   layer_kinds=["attention" if i in attn else "mamba2" for i in range(L)],
                   ssm=dict(d_inner=H * P, d_state=hf.get("mamba_d_state", 256), d_conv=hf.get("mamba_d_conv", 4),
                            n_groups=hf.get("mamba_n_groups", 1), head_dim=P, n_heads=H, norm_groups=1,
                            conv_bias=hf.get("mamba_conv_bias", True), proj_bias=hf.get("mamba_proj_bias", False),
                            dt_min=_limit(lim[0], 0.0), dt_max=_limit(lim[1], 1e30)))
    if mt in ("qwen3_next", "qwen3_5_text", "qwen3_5_moe_text"):
        kinds = hf.get("layer_types") or ["linear_attention" if (i + 1) % 4 else "full_attention" for i in range(L)]
        E, step, dense = hf.get("num_experts", 0), hf.get("decoder_sparse_step", 1) or 1, set(hf.get("mlp_only_layers") or [])
        rot = int(head_dim * hf.get("partial_rotary_factor", 0.25))
        return cls(**base, intermediate_size=hf.get("intermediate_size") or hf.get("moe_intermediate_size", 0), rms_eps=hf.get("rms_norm_eps", 1e-6),
                   tie_embeddings=hf.get("tie_word_embeddings", False), qk_norm=True, norm_weight_offset=1.0,
                   attn_out_gate=True, rotary_dim=rot if rot != head_dim else None,
                   layer_kinds=["attention" if k == "full_attention" else "gated_delta" for k in kinds],
                   ffn_kinds=["moe" if (E > 0 and i not in dense and (i + 1) % step == 0) else "glu" for i in range(L)],
                   num_experts=E, experts_per_token=hf.get("num_experts_per_tok", 10),
                   moe_intermediate_size=hf.get("moe_intermediate_size", 512),
                   router_kind="softmax_all" if hf.get("norm_topk_prob", True) else "deepseek_v2", router_norm_topk=False,
                   shared_intermediate_size=hf.get("shared_expert_intermediate_size", 0) if E else 0, shared_gate=bool(E),
                   ssm=dict(num_k_heads=hf.get("linear_num_key_heads", 16), num_v_heads=hf.get("linear_num_value_heads", 32),
                            head_k_dim=hf.get("linear_key_head_dim", 128), head_v_dim=hf.get("linear_value_head_dim", 128),
                            d_conv=hf.get("linear_conv_kernel_dim", 4), norm_eps=hf.get("rms_norm_eps", 1e-6)))
    if mt == "ernie4_5_moe":              # ERNIE 4.5: pair-style rotation, softmax router with a selection bias, renormalised weights
        E, start, step = hf.get("moe_num_experts", 0), hf.get("moe_layer_start_index", 1), hf.get("moe_layer_interval", 1) or 1
        end = hf.get("moe_layer_end_index", -1)
        end = L - 1 if end in (None, -1) else end
        I = hf.get("moe_intermediate_size", 1536)
        return cls(**base, arch_alias="glm4_moe", rope_style="pair", intermediate_size=hf["intermediate_size"],
                   rms_eps=hf.get("rms_norm_eps", 1e-5), tie_embeddings=hf.get("tie_word_embeddings", True),
                   attn_bias=bool(hf.get("use_bias", False)), layer_kinds=["attention"] * L,
                   ffn_kinds=["moe" if (E and start <= i <= end and (i + 1) % step == 0) else "glu" for i in range(L)],
                   num_experts=E, experts_per_token=hf.get("moe_k", 6), moe_intermediate_size=I,
                   shared_intermediate_size=(hf.get("moe_num_shared_experts") or 0) * I, router_kind="deepseek_v2", router_norm_topk=True)
    if mt == "glm4_moe":                  # GLM-4.5: llama-style attention (partial rotary, optional per-head QK-norm) + the DeepSeek-V3 router
        dense_first, E = hf.get("first_k_dense_replace", 1), hf.get("n_routed_experts", 0)
        rot = int(head_dim * hf.get("partial_rotary_factor", 0.5))
        return cls(**base, intermediate_size=hf["intermediate_size"], rms_eps=hf.get("rms_norm_eps", 1e-5),
                   tie_embeddings=hf.get("tie_word_embeddings", False), attn_bias=hf.get("attention_bias", False),
                   qk_norm=bool(hf.get("use_qk_norm", False)), rotary_dim=rot if rot != head_dim else None,
                   layer_kinds=["attention"] * L, ffn_kinds=["moe" if (E and i >= dense_first) else "glu" for i in range(L)],
                   num_experts=E, experts_per_token=hf.get("num_experts_per_tok", 8), moe_intermediate_size=hf.get("moe_intermediate_size", 1408),
                   shared_intermediate_size=(hf.get("n_shared_experts") or 0) * hf.get("moe_intermediate_size", 1408),
                   router_kind="deepseek_v3", router_scale=float(hf.get("routed_scaling_factor", 1.0)),
                   router_norm_topk=bool(hf.get("norm_topk_prob", True)), router_groups=hf.get("n_group") or 1,
                   router_topk_groups=hf.get("topk_group") or 1)
    if mt in ("granitemoehybrid", "granitemoe", "granitemoeshared"):
        H = hf.get("mamba_n_heads", 128)
        P = hf.get("mamba_d_head", "auto")
        P = hf.get("mamba_expand", 2) * hidden // H if P == "auto" else int(P)
        kinds = hf.get("layer_types") or ["mamba"] * L
        if mt != "granitemoehybrid":          # the attention-only members of the family
            kinds = ["attention"] * L
            hf = dict(hf, shared_intermediate_size=hf.get("shared_intermediate_size", 0) if mt == "granitemoeshared" else 0)
        E = hf.get("num_local_experts") or 0
        lim = hf.get("time_step_limit") or (0.0, float("inf"))
        # the residual and logit multipliers are folded into the weights by the loader (residual_mult, logits_div)
        return cls(**base, arch_alias="granitemoehybrid", intermediate_size=hf.get("shared_intermediate_size", 1024), rms_eps=hf.get("rms_norm_eps", 1e-6),
                   tie_embeddings=hf.get("tie_word_embeddings", False), attn_bias=hf.get("attention_bias", False),
                   embed_scale=float(hf.get("embedding_multiplier") or 1.0), attn_scale=float(hf.get("attention_multiplier") or head_dim ** -0.5),
                   use_rope=(hf.get("position_embedding_type") or "rope") == "rope",
                   layer_kinds=["attention" if k == "attention" else "mamba2" for k in kinds],
                   ffn_kinds=["moe" if E else "glu"] * L, num_experts=E, experts_per_token=hf.get("num_experts_per_tok", 2) if E else 0,
                   moe_intermediate_size=hf["intermediate_size"] if E else 0, router_kind="softmax_topk",
                   shared_intermediate_size=hf.get("shared_intermediate_size", 1024) if E else 0,
                   ssm=dict(d_inner=H * P, d_state=hf.get("mamba_d_state", 256), d_conv=hf.get("mamba_d_conv", 4),
                            n_groups=hf.get("mamba_n_groups", 1), head_dim=P, n_heads=H, norm_groups=1,
                            conv_bias=hf.get("mamba_conv_bias", True), proj_bias=hf.get("mamba_proj_bias", False),
                            dt_min=_limit(lim[0], 0.0), dt_max=_limit(lim[1], 1e30),
                            residual_mult=float(hf.get("residual_multiplier") or 1.0), logits_div=float(hf.get("logits_scaling") or 1.0)))
    if mt == "jamba":
        ap, ao = hf.get("attn_layer_period", 8), hf.get("attn_layer_offset", 4)
        ep, eo = hf.get("expert_layer_period", 2), hf.get("expert_layer_offset", 1)
        E = hf.get("num_experts", 16)
        rank = hf.get("mamba_dt_rank", "auto")
        rank = -(-hidden // 16) if rank == "auto" else int(rank)
        return cls(**base, intermediate_size=hf["intermediate_size"], rms_eps=hf.get("rms_norm_eps", 1e-6),
                   tie_embeddings=hf.get("tie_word_embeddings", False), use_rope=False,
                   layer_kinds=["attention" if i % ap == ao else "mamba1" for i in range(L)],
                   ffn_kinds=["moe" if (E > 1 and i % ep == eo) else "glu" for i in range(L)],
                   num_experts=E if E > 1 else 0, experts_per_token=hf.get("num_experts_per_tok", 2),
                   moe_intermediate_size=hf["intermediate_size"], router_kind="deepseek_v2", router_norm_topk=False,
                   ssm=dict(d_inner=hf.get("mamba_expand", 2) * hidden, d_state=hf.get("mamba_d_state", 16),
                            d_conv=hf.get("mamba_d_conv", 4), dt_rank=rank, conv_bias=hf.get("mamba_conv_bias", True),
                            proj_bias=hf.get("mamba_proj_bias", False), bcdt_rms=True, mixer_rms_eps=hf.get("rms_norm_eps", 1e-6)))
    if mt == "lfm2":
        inter = hf.get("intermediate_size") or hf.get("block_ff_dim", 4 * hidden)
        if hf.get("block_auto_adjust_ff_dim", True):                # the checkpoint's FFN width: 2/3, multiplier, rounded up
            inter = int(2 * inter / 3)
            if hf.get("block_ffn_dim_multiplier") is not None:
                inter = int(hf["block_ffn_dim_multiplier"] * inter)
            mult = hf.get("block_multiple_of", 256)
            inter = mult * ((inter + mult - 1) // mult)
        kinds = hf.get("layer_types")
        if not kinds:
            full = set(hf.get("full_attn_idxs") or range(L))
            kinds = ["full_attention" if i in full else "conv" for i in range(L)]
        return cls(**base, intermediate_size=inter, rms_eps=hf.get("norm_eps", 1e-5),
                   tie_embeddings=hf.get("tie_word_embeddings", True), qk_norm=True,
                   layer_kinds=["attention" if k == "full_attention" else "shortconv" for k in kinds],
                   ssm=dict(d_conv=hf.get("conv_L_cache", 3), conv_bias=hf.get("conv_bias", False)))
    raise ValueError(f"no recurrent mapping for model_type {mt!r}")


def rope_inv_freq(cfg: ModelConfig) -> "tuple[List[float], float]":
    """Per-pair inverse frequencies (length rot_dim/2) and the attention factor that
    multiplies cos/sin. Covers plain, linear, Llama-3 and YaRN scaling
    (rust/engine/src/rope.rs:1 builds the same families of tables)."""
    rot = cfg.rot_dim
    base = [cfg.rope_theta ** (-(2.0 * i) / rot) for i in range(rot // 2)]
    rs = cfg.rope_scaling
    attn = 1.0
    if rs.kind == "linear":
        base = [f / rs.factor for f in base]
    elif rs.kind == "factors":
        if len(rs.freq_factors or ()) != len(base):
            raise ValueError(f"rope frequency factors: {len(rs.freq_factors or ())} values for {len(base)} frequencies")
        base = [f / d for f, d in zip(base, rs.freq_factors)]
    elif rs.kind == "llama3":
        lo_wl = rs.original_max_position / rs.low_freq_factor
        hi_wl = rs.original_max_position / rs.high_freq_factor
        out = []
        for f in base:
            wl = 2 * math.pi / f
            if wl < hi_wl:
                out.append(f)
            elif wl > lo_wl:
                out.append(f / rs.factor)
            else:
                s = (rs.original_max_position / wl - rs.low_freq_factor) / (
                    rs.high_freq_factor - rs.low_freq_factor)
                out.append((1 - s) * f / rs.factor + s * f)
        base = out
    elif rs.kind == "yarn":
        def corr_dim(n_rot: float) -> float:
            return (rot * math.log(rs.original_max_position / (n_rot * 2 * math.pi))) / (
                2 * math.log(cfg.rope_theta))
        lo, hi = corr_dim(rs.beta_fast), corr_dim(rs.beta_slow)
        if rs.truncate:
            lo, hi = math.floor(lo), math.ceil(hi)
        lo, hi = max(lo, 0), min(hi, rot - 1)
        out = []
        for i, f in enumerate(base):
            ramp = min(max((i - lo) / max(hi - lo, 1e-3), 0.0), 1.0)
            extrap_w = 1.0 - ramp
            out.append(f / rs.factor * (1 - extrap_w) + f * extrap_w)
        base = out
        attn = rs.attn_factor if rs.attn_factor is not None else 0.1 * math.log(rs.factor) + 1.0
    return base, attn


# ---------------------------------------------------------------------------- presets
def preset(name: str) -> ModelConfig:
    """Named shapes used by the benchmarks and tests (random-init, no checkpoint)."""
    n = name.lower().replace("_", "-")
    if n in ("tiny-llama", "tiny"):
        return ModelConfig(arch="llama", name="tiny-llama", vocab_size=32000, hidden_size=256,
                           num_layers=2, num_heads=4, num_kv_heads=2, head_dim=64,
                           intermediate_size=688, rms_eps=1e-5, rope_theta=10000.0,
                           tie_embeddings=True, max_position=4096)
    if n in ("qwen3-8b",):
        return ModelConfig(arch="qwen3", name="qwen3-8b", vocab_size=151936, hidden_size=4096,
                           num_layers=36, num_heads=32, num_kv_heads=8, head_dim=128,
                           intermediate_size=12288, rms_eps=1e-6, rope_theta=1e6, qk_norm=True,
                           max_position=40960)
    if n in ("qwen3-tiny",):
        return ModelConfig(arch="qwen3", name="qwen3-tiny", vocab_size=4096, hidden_size=512,
                           num_layers=2, num_heads=8, num_kv_heads=2, head_dim=64,
                           intermediate_size=1024, rms_eps=1e-6, rope_theta=1e6, qk_norm=True,
                           max_position=4096)
    if n in ("llama3-70b", "llama-3-70b", "llama31-70b", "llama-3.1-70b"):
        return ModelConfig(arch="llama", name=n, vocab_size=128256, hidden_size=8192, num_layers=80,
                           num_heads=64, num_kv_heads=8, head_dim=128, intermediate_size=28672,
                           rms_eps=1e-5, rope_theta=5e5, max_position=131072)
    if n in ("llama32-1b", "llama-3.2-1b"):
        return ModelConfig(arch="llama", name=n, vocab_size=128256, hidden_size=2048, num_layers=16,
                           num_heads=32, num_kv_heads=8, head_dim=64, intermediate_size=8192,
                           rms_eps=1e-5, rope_theta=5e5, tie_embeddings=True, max_position=131072)
    if n in ("gpt-oss-120b", "gpt-oss-tiny"):
        tiny = n.endswith("tiny")
        return ModelConfig(arch="gpt_oss", name=n, vocab_size=4096 if tiny else 201088,
                           hidden_size=256 if tiny else 2880, num_layers=2 if tiny else 36,
                           num_heads=8 if tiny else 64, num_kv_heads=2 if tiny else 8, head_dim=64,
                           intermediate_size=256 if tiny else 2880, rms_eps=1e-5, rope_theta=150000.0,
                           act="swiglu_oai", attn_sinks=True, attn_bias=True, expert_bias=True,
                           sliding_window=128, window_pattern=[1, 0],
                           num_experts=8 if tiny else 128, experts_per_token=4,
                           moe_intermediate_size=256 if tiny else 2880, weight_format="bf16",
                           rope_scaling=RopeScaling(kind="yarn", factor=32.0, beta_fast=32.0,
                                                    beta_slow=1.0, original_max_position=4096, truncate=False),
                           max_position=131072)
    if n in ("mamba2-2.7b", "mamba2-tiny"):
        tiny = n.endswith("tiny")
        hidden, L, H = (256, 2, 8) if tiny else (2560, 64, 80)
        return ModelConfig(arch="mamba2", name=n, vocab_size=4096 if tiny else 50288, hidden_size=hidden, num_layers=L,
                           num_heads=1, num_kv_heads=1, head_dim=64, intermediate_size=0, tie_embeddings=True,
                           layer_kinds=["mamba2"] * L, ffn_kinds=["none"] * L,
                           ssm=dict(d_inner=H * 64, d_state=128, d_conv=4, n_groups=1, head_dim=64, n_heads=H,
                                    norm_groups=1, conv_bias=True, dt_min=0.0, dt_max=1e30))
    if n in ("falcon-mamba-7b", "mamba1-tiny"):
        tiny = n.endswith("tiny")
        hidden, L = (256, 2) if tiny else (4096, 64)
        return ModelConfig(arch="falcon_mamba", name=n, vocab_size=4096 if tiny else 65024, hidden_size=hidden, num_layers=L,
                           num_heads=1, num_kv_heads=1, head_dim=64, intermediate_size=0, tie_embeddings=False,
                           layer_kinds=["mamba1"] * L, ffn_kinds=["none"] * L,
                           ssm=dict(d_inner=2 * hidden, d_state=16, d_conv=4, dt_rank=hidden // 16, conv_bias=True,
                                    proj_bias=False, bcdt_rms=True, mixer_rms_eps=1e-6))
    if n in ("bamba-9b", "bamba-tiny"):
        tiny = n.endswith("tiny")
        hidden, L, H = (256, 3, 8) if tiny else (4096, 32, 128)
        attn = {1} if tiny else {9, 18, 27}
        return ModelConfig(arch="bamba", name=n, vocab_size=4096 if tiny else 128256, hidden_size=hidden, num_layers=L,
                           num_heads=4 if tiny else 32, num_kv_heads=2 if tiny else 8, head_dim=64 if tiny else 128,
                           rotary_dim=32 if tiny else 64, intermediate_size=512 if tiny else 14336,
                           layer_kinds=["attention" if i in attn else "mamba2" for i in range(L)],
                           ssm=dict(d_inner=H * 64, d_state=128, d_conv=4, n_groups=1, head_dim=64, n_heads=H,
                                    norm_groups=1, conv_bias=True, dt_min=0.0, dt_max=1e30))
    if n in ("deepseek-v2-lite-dense", "mla-tiny"):
        # the attention of DeepSeek-V2-Lite (16 heads, 512 + 64 latent rows) with dense feed-forward layers throughout
        tiny = n == "mla-tiny"
        hidden, L, H = (256, 2, 4) if tiny else (2048, 27, 16)
        return ModelConfig(arch="deepseek_v2", name=n, vocab_size=4096 if tiny else 102400, hidden_size=hidden, num_layers=L,
                           num_heads=H, num_kv_heads=1, head_dim=192, rotary_dim=64, rope_style="pair",
                           intermediate_size=512 if tiny else 10944, rms_eps=1e-6, layer_kinds=["mla"] * L,
                           mla=dict(q_lora_rank=0, kv_lora_rank=512, qk_nope_head_dim=128, qk_rope_head_dim=64, v_head_dim=128))
    if n == "rwkv6-tiny":
        return ModelConfig(arch="rwkv6", name=n, vocab_size=4096, hidden_size=256, num_layers=2, num_heads=4, num_kv_heads=4,
                           head_dim=64, intermediate_size=896, layer_kinds=["rwkv6"] * 2, ffn_kinds=["none"] * 2,
                           ssm=dict(head_dim=64, d_conv=2, head_size_divisor=8, mix_rank=32, decay_rank=64))
    if n in ("rwkv7-1.5b", "rwkv7-tiny"):
        tiny = n.endswith("tiny")
        hidden, L = (256, 2) if tiny else (2048, 24)
        ranks = dict(decay_rank=32, a_rank=32, v_rank=16, gate_rank=64) if tiny else dict(decay_rank=96, a_rank=96, v_rank=64, gate_rank=256)
        return ModelConfig(arch="rwkv7", name=n, vocab_size=4096 if tiny else 65536, hidden_size=hidden, num_layers=L,
                           num_heads=hidden // 64, num_kv_heads=hidden // 64, head_dim=64, intermediate_size=4 * hidden,
                           layer_kinds=["rwkv7"] * L, ffn_kinds=["none"] * L, ssm=dict(head_dim=64, d_conv=2, **ranks))
    if n in ("deepseek-v2-lite", "deepseek-moe-tiny"):
        tiny = n.endswith("tiny")
        hidden, L, H = (256, 3, 4) if tiny else (2048, 27, 16)
        return ModelConfig(arch="deepseek_v2", name=n, vocab_size=4096 if tiny else 102400, hidden_size=hidden, num_layers=L,
                           num_heads=H, num_kv_heads=1, head_dim=192, rotary_dim=64, rope_style="pair",
                           intermediate_size=512 if tiny else 10944, rms_eps=1e-6, layer_kinds=["mla"] * L,
                           ffn_kinds=["glu"] + ["moe"] * (L - 1), num_experts=8 if tiny else 64, experts_per_token=2 if tiny else 6,
                           moe_intermediate_size=128 if tiny else 1408, shared_intermediate_size=256 if tiny else 2816,
                           router_kind="deepseek_v2", router_scale=1.0, router_norm_topk=False,
                           mla=dict(q_lora_rank=0, kv_lora_rank=512, qk_nope_head_dim=128, qk_rope_head_dim=64, v_head_dim=128))
    raise KeyError(f"unknown model preset {name!r}")


# ---------------------------------------------------------------------------- engine / parallel
@dataclass
class ParallelConfig:
    """World = tp x pp ranks, stage-major numbering rank = stage * tp + tp_rank;
    expert parallelism reuses the tensor-parallel group
    (rust/engine/src/parallel/config.rs:93-100)."""
    tp: int = 1
    pp: int = 1
    expert_parallel: bool = False
    ep_dispatch: str = "allreduce"       # allreduce (partial sums reduced like a dense FFN) | alltoall (rows travel to the experts' ranks and back over peer memory)
    pipeline_microbatches: int = 0       # 0 = one per stage
    distributed_backend: str = "fused"   # fused (peer-memory kernels) | nccl (baseline)
    nnodes: int = 1
    node_rank: int = 0
    master_addr: str = "127.0.0.1"
    master_port: int = 29500

    @property
    def world(self) -> int:
        return self.tp * self.pp

    def coords(self, rank: int) -> "tuple[int, int]":
        return rank // self.tp, rank % self.tp      # (stage, tp_rank)

    def stage_layers(self, num_layers: int, stage: int) -> range:
        per, rem = divmod(num_layers, self.pp)
        start = stage * per + min(stage, rem)
        return range(start, start + per + (1 if stage < rem else 0))


@dataclass
class EngineConfig:
    max_num_seqs: int = 256
    max_num_batched_tokens: int = 2048   # chunked-prefill token budget per step
    block_size: int = 16
    num_kv_blocks: int = 0               # 0 = size from gpu_memory_utilization
    gpu_memory_utilization: float = 0.90
    max_model_len: int = 8192
    kv_cache_dtype: str = "bf16"         # bf16 | fp8_e4m3
    enable_prefix_caching: bool = True
    scheduling_policy: str = "fcfs"      # fcfs | priority
    preemption: str = "recompute"        # recompute | swap (KV of a preempted request parked in host memory)
    swap_space_gb: float = 4.0           # host memory for swapped-out KV
    state_cache_gb: float = 0.0          # recurrent models: host memory for state checkpoints on block boundaries (0 = no prefix reuse)
    kv_tier_host_gb: float = 0.0         # host memory for evicted prefix-cache blocks (0 = no tier)
    kv_tier_disk_dir: Optional[str] = None   # directory for blocks that fall out of the host tier (default: $FLLM_KV_DISK_DIR)
    kv_tier_disk_gb: float = 0.0
    decode_first: bool = True
    max_partial_prefills: int = 4
    watermark: float = 0.01
    use_cuda_graphs: bool = True
    graph_buckets: Sequence[int] = (1, 2, 4, 8, 16, 24, 32, 48, 64, 96, 128, 192, 256)
    async_scheduling: bool = True
    multi_step: int = 1
    speculative: str = "off"             # off | draft | ngram | suffix
    draft_tokens: int = 4
    seed: int = 0
    step_deadline_s: float = 120.0       # watchdog: a step slower than this fails the batch

    @classmethod
    def from_env(cls, **over: Any) -> "EngineConfig":
        cfg = cls(**over)
        env = os.environ
        if "FLLM_MAX_SEQS" in env:
            cfg.max_num_seqs = int(env["FLLM_MAX_SEQS"])
        if "FLLM_MAX_BATCHED_TOKENS" in env:
            cfg.max_num_batched_tokens = int(env["FLLM_MAX_BATCHED_TOKENS"])
        if "FLLM_CUDA_GRAPHS" in env:
            cfg.use_cuda_graphs = env["FLLM_CUDA_GRAPHS"] not in ("0", "false", "off")
        if "FLLM_ASYNC_SCHEDULING" in env:
            cfg.async_scheduling = env["FLLM_ASYNC_SCHEDULING"] not in ("0", "false", "off")
        if "FLLM_KV_BLOCKS" in env:
            cfg.num_kv_blocks = int(env["FLLM_KV_BLOCKS"])
        return cfg


def dump_effective(model: ModelConfig, engine: EngineConfig, par: ParallelConfig) -> str:
    return json.dumps({"model": model.to_dict(), "engine": dataclasses.asdict(engine),
                       "parallel": dataclasses.asdict(par)}, default=list, indent=1)
