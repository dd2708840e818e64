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
    kind: str = "none"            # none | linear | llama3 | yarn
    factor: float = 1.0
    low_freq_factor: float = 1.0
    high_freq_factor: float = 4.0
    original_max_position: int = 8192
    beta_fast: float = 32.0
    beta_slow: float = 1.0
    attn_factor: Optional[float] = None


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
    router_kind: str = "softmax_topk"    # softmax over the selected top-k logits
    expert_bias: bool = False
    # weight format of the big matrices
    weight_format: str = "bf16"          # bf16 | fp8_block | nvfp4 | mxfp4 | mxfp8 | mxfp4_a8 | nvfp4_a4 | int8_w8a8 | fp8_w8a8 | q4_k | ...
    name: str = "model"

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
                attn_factor=rs.get("attention_factor"))
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
        if mt in ("gemma", "gemma2"):
            cfg.norm_weight_offset = 1.0
            cfg.embed_scale = float(hidden) ** 0.5
            cfg.act = "geglu"
            cfg.tie_embeddings = hf.get("tie_word_embeddings", True)
            cfg.logit_softcap = float(hf.get("final_logit_softcapping") or 0.0)
            cfg.attn_softcap = float(hf.get("attn_logit_softcapping") or 0.0)
        if mt == "gemma2":
            cfg.post_norms = True
            if hf.get("query_pre_attn_scalar"):
                cfg.attn_scale = float(hf["query_pre_attn_scalar"]) ** -0.5
            if hf.get("sliding_window"):
                cfg.sliding_window = int(hf["sliding_window"])
                lt = hf.get("layer_types")
                cfg.window_pattern = [1 if t == "sliding_attention" else 0 for t in lt] if lt else [1, 0]
        if mt in ("phi3", "phi"):
            cfg.rotary_dim = int(cfg.head_dim * hf.get("partial_rotary_factor", 1.0)) or None
        if hf.get("sliding_window") and hf.get("use_sliding_window", mt == "mistral"):
            cfg.sliding_window = hf["sliding_window"]
        return cfg


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
        lo = max(math.floor(corr_dim(rs.beta_fast)), 0)
        hi = min(math.ceil(corr_dim(rs.beta_slow)), rot // 2 - 1)
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
                                                    beta_slow=1.0, original_max_position=4096),
                           max_position=131072)
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
