"""Decoder weights: containers, deterministic random initialisation and the
tensor-parallel sharding rules.

Sharding follows the reference's plan (rust/engine/src/parallel/plan.rs:26-45,
rust/engine/src/parallel/decoder_shard.rs:112-214): query heads are divided by
``tp``; KV heads are divided, or replicated when ``tp`` exceeds their count;
q/k/v/gate/up are cut by output rows (column-parallel), o/down by input columns
(row-parallel) with the bias kept on tp-rank 0; norms are replicated; the LM head
is cut by vocabulary rows in equal padded chunks; experts are either cut like a
dense FFN (expert-TP) or assigned whole to ranks (expert parallel).
"""
from __future__ import annotations

import hashlib
from dataclasses import dataclass, field
from typing import Dict, List, Optional

import torch

from ..config import ModelConfig


@dataclass
class LayerWeights:
    attn_norm: torch.Tensor
    wqkv: torch.Tensor
    wo: torch.Tensor
    ffn_norm: torch.Tensor
    bqkv: Optional[torch.Tensor] = None
    bo: Optional[torch.Tensor] = None
    q_norm: Optional[torch.Tensor] = None
    k_norm: Optional[torch.Tensor] = None
    sinks: Optional[torch.Tensor] = None
    post_attn_norm: Optional[torch.Tensor] = None   # Gemma-2: norm of the attention output before the residual add
    post_ffn_norm: Optional[torch.Tensor] = None    # Gemma-2: norm of the FFN output before the residual add
    w_gate_up: Optional[torch.Tensor] = None
    w_down: Optional[torch.Tensor] = None
    # mixture of experts
    router_w: Optional[torch.Tensor] = None
    router_b: Optional[torch.Tensor] = None
    exp_gate_up: Optional[torch.Tensor] = None      # [E_local, 2*I, H]
    exp_gate_up_b: Optional[torch.Tensor] = None    # [E_local, 2*I]
    exp_down: Optional[torch.Tensor] = None         # [E_local, H, I]
    exp_down_b: Optional[torch.Tensor] = None       # [E_local, H]
    router_select_b: Optional[torch.Tensor] = None  # [E] added to the scores for the selection only (DeepSeek-V3)
    shared_gate_up: Optional[torch.Tensor] = None   # [2*Is, H] always-on shared experts as one dense GLU
    shared_down: Optional[torch.Tensor] = None      # [H, Is]
    moe_latent_in: Optional[torch.Tensor] = None    # [latent, H], [H, latent]: projections around the routed experts
    moe_latent_out: Optional[torch.Tensor] = None
    shared_gate_w: Optional[torch.Tensor] = None    # [8, H] (row 0 used): sigmoid(h . w) scales the shared experts' output
    w_attn_gate: Optional[torch.Tensor] = None      # [hq*D, H] output gate of the attention (Qwen3-Next)
    # LayerNorm families: norm biases; plain MLPs keep their first matrix in w_gate_up and carry biases
    attn_norm_b: Optional[torch.Tensor] = None
    ffn_norm_b: Optional[torch.Tensor] = None
    b_up: Optional[torch.Tensor] = None
    q_norm_full: Optional[torch.Tensor] = None      # [hq*D] / [hkv*D]: norms over the whole projections (OLMo-2)
    k_norm_full: Optional[torch.Tensor] = None
    b_down: Optional[torch.Tensor] = None
    # recurrent layers (Mamba, delta rule, short convolution): the mixer's tensors by name; wqkv / wo stay None
    mixer: Optional[Dict[str, torch.Tensor]] = None
    # packed formats keep their payload here (format name -> tensors)
    packed: Dict[str, object] = field(default_factory=dict)
    # row order of w_gate_up: 0 = gate half then up half; 16 = blocks of 16 gate rows followed by the 16 up
    # rows of the same features (set by the decoder on a GPU, where the GEMM epilogue applies the activation)
    glu_layout: int = 0


def gate_up_natural(lw: "LayerWeights") -> torch.Tensor:
    """The dense gate|up matrix in its natural row order (gate half, then up half), whatever order the
    decoder re-arranged it into for the GEMM epilogue."""
    w = lw.w_gate_up
    if getattr(lw, "glu_layout", 0) != 16:
        return w
    I = w.shape[0] // 2
    blk = w.view(I // 16, 2, 16, *w.shape[1:])
    return torch.cat([blk[:, 0].reshape(I, *w.shape[1:]), blk[:, 1].reshape(I, *w.shape[1:])], 0)


@dataclass
class DecoderWeights:
    embed: torch.Tensor
    layers: List[LayerWeights]
    final_norm: torch.Tensor
    lm_head: torch.Tensor               # [vocab_local(padded), H]
    vocab_start: int = 0
    vocab_local: int = 0
    final_norm_b: Optional[torch.Tensor] = None      # families whose blocks are LayerNorms (RWKV, GPT-NeoX, Phi, ...)
    lm_head_b: Optional[torch.Tensor] = None         # Phi
    pos_embed: Optional[torch.Tensor] = None         # [positions, H] learned absolute positions (GPT-2, OPT)

    def nbytes(self) -> int:
        n = 0
        seen = set()

        def add(t):
            nonlocal n
            if isinstance(t, torch.Tensor) and t.data_ptr() not in seen:
                seen.add(t.data_ptr())
                n += t.numel() * t.element_size()

        add(self.embed); add(self.final_norm); add(self.lm_head)
        for l in self.layers:
            for v in vars(l).values():
                add(v)
            for v in (l.mixer or {}).values():
                add(v)
        return n


@dataclass
class ShardSpec:
    """Per-rank head / column ranges for one tensor-parallel rank."""
    tp: int
    tp_rank: int
    hq_local: int
    hkv_local: int
    q_head_start: int
    kv_head_start: int
    inter_start: int
    inter_local: int
    vocab_chunk: int
    expert_start: int = 0
    expert_local: int = 0
    expert_parallel: bool = False


def attention_split(cfg: ModelConfig, tp: int, tp_rank: int):
    """(q heads, kv heads, first q head, first kv head) of one rank."""
    if cfg.num_heads % tp:
        raise ValueError(f"{cfg.num_heads} query heads cannot be divided over tp={tp}")
    hq = cfg.num_heads // tp
    if cfg.num_kv_heads >= tp:
        if cfg.num_kv_heads % tp:
            raise ValueError(f"{cfg.num_kv_heads} KV heads cannot be divided over tp={tp}")
        hkv = cfg.num_kv_heads // tp
        kv0 = tp_rank * hkv
    else:
        if tp % cfg.num_kv_heads:
            raise ValueError(f"tp={tp} must be a multiple of {cfg.num_kv_heads} KV heads")
        hkv = 1
        kv0 = tp_rank // (tp // cfg.num_kv_heads)
    return hq, hkv, tp_rank * hq, kv0


def expert_range(num_experts: int, tp: int, rank: int):
    """Contiguous expert range of a rank, remainder to the first ranks
    (rust/engine/src/parallel/ctx.rs:100-105)."""
    per, rem = divmod(num_experts, tp)
    start = rank * per + min(rank, rem)
    return start, per + (1 if rank < rem else 0)


def make_shard_spec(cfg: ModelConfig, tp: int = 1, tp_rank: int = 0, expert_parallel: bool = False,
                    align: int = 8) -> ShardSpec:
    hq, hkv, q0, kv0 = attention_split(cfg, tp, tp_rank)
    inter = cfg.moe_intermediate_size if cfg.is_moe else cfg.intermediate_size
    ep = bool(expert_parallel and cfg.is_moe and tp > 1)
    if ep:
        i0, il = 0, inter
    else:
        if inter % (tp * align):
            raise ValueError(f"intermediate size {inter} cannot be cut into {tp} aligned parts")
        il = inter // tp
        i0 = tp_rank * il
    chunk = -(-cfg.vocab_size // tp)
    chunk = -(-chunk // 128) * 128 if tp > 1 else cfg.vocab_size
    e0, el = expert_range(cfg.num_experts, tp, tp_rank) if ep else (0, cfg.num_experts)
    return ShardSpec(tp, tp_rank, hq, hkv, q0, kv0, i0, il, chunk, e0, el, ep)


def _randn(shape, gen, device, dtype, std=0.02):
    return (torch.randn(shape, generator=gen, device=device, dtype=torch.float32) * std).to(dtype)


def pack_layer(lw: LayerWeights, fmt: str) -> None:
    """Replace the big matrices of one layer by their packed form, in place: ``fp8_block`` (e4m3 codes + one fp32
    scale per 128 x 128), ``nvfp4`` (e2m1 + e4m3 scale per 16 + tensor scale), ``mxfp4`` (e2m1 + e8m0 scale per
    32; for mixture-of-experts layers only the expert stacks are packed, attention stays bf16 as in gpt-oss), or
    the block-scaled tensor-core pairs ``mxfp8`` / ``mxfp4_a8`` (MXFP8 / MXFP4 weights x MXFP8 activations) and
    ``nvfp4_a4`` (NVFP4 weights x NVFP4 activations).
    Matrices whose shape the format cannot tile stay bf16."""
    if fmt in ("bf16", "", None):
        return
    if fmt == "fp8_block":
        from ..ops.native import Fp8BlockWeight, quantize_weight_fp8_block
        for name in ("wqkv", "wo", "w_gate_up", "w_down"):
            w = getattr(lw, name, None)
            if isinstance(w, torch.Tensor) and w.dim() == 2 and w.shape[0] % 128 == 0 and w.shape[1] % 128 == 0:
                setattr(lw, name, Fp8BlockWeight(*quantize_weight_fp8_block(w)))
        return
    if fmt in ("nvfp4", "mxfp4"):
        from ..ops.fp4 import Fp4ExpertStack, Fp4Weight
        if lw.exp_gate_up is not None:
            if fmt == "mxfp4" and isinstance(lw.exp_gate_up, torch.Tensor) and lw.exp_gate_up.shape[2] % 64 == 0:
                lw.exp_gate_up = Fp4ExpertStack.from_dense(lw.exp_gate_up, fmt)
                lw.exp_down = Fp4ExpertStack.from_dense(lw.exp_down, fmt)
            return
        for name in ("wqkv", "wo", "w_gate_up", "w_down"):
            w = getattr(lw, name, None)
            if isinstance(w, torch.Tensor) and w.dim() == 2 and w.shape[1] % 64 == 0 and w.shape[0] % 8 == 0:
                setattr(lw, name, Fp4Weight.from_dense(w, fmt))
        return
    if fmt in ("int8_w8a8", "fp8_w8a8"):
        # per-channel 8-bit weights, activations quantised per token on the fly (tcgen05 kind::i8 / kind::f8f6f4)
        from ..ops.mx import W8A8Weight
        if lw.exp_gate_up is not None:
            return
        for name in ("wqkv", "wo", "w_gate_up", "w_down"):
            w = getattr(lw, name, None)
            if isinstance(w, torch.Tensor) and w.dim() == 2 and w.shape[1] % 128 == 0 and w.shape[0] % 8 == 0:
                setattr(lw, name, W8A8Weight.from_dense(w, "int8" if fmt == "int8_w8a8" else "fp8"))
        return
    if fmt in ("mxfp8", "mxfp4_a8", "nvfp4_a4"):
        # block-scaled tensor-core formats: MXFP8 or MXFP4 weights with activations quantised to MXFP8 on the fly,
        # or NVFP4 weights with activations quantised to NVFP4 per token
        from ..ops.mx import MxWeight, Nvfp4TcWeight
        if lw.exp_gate_up is not None:
            return
        for name in ("wqkv", "wo", "w_gate_up", "w_down"):
            w = getattr(lw, name, None)
            if isinstance(w, torch.Tensor) and w.dim() == 2 and w.shape[1] % 256 == 0 and w.shape[0] % 8 == 0:
                if fmt == "nvfp4_a4":
                    setattr(lw, name, Nvfp4TcWeight.from_dense(w))
                else:
                    setattr(lw, name, MxWeight.from_dense(w, "mxfp8" if fmt == "mxfp8" else "mxfp4"))
        return
    raise ValueError(f"random initialisation in weight format {fmt!r} is not available "
                     "(bf16, fp8_block, nvfp4, mxfp4, mxfp8, mxfp4_a8, nvfp4_a4, int8_w8a8, fp8_w8a8)")


def init_random_weights(cfg: ModelConfig, device="cpu", dtype=torch.bfloat16, seed: int = 0,
                        tp: int = 1, tp_rank: int = 0, expert_parallel: bool = False,
                        layers: Optional[range] = None, first_stage: bool = True,
                        last_stage: bool = True, weight_format: Optional[str] = None) -> DecoderWeights:
    """N(0, 0.02) weights, norm weights 1. Every tensor is drawn at full size from a
    generator seeded by (seed, layer, tensor) and then cut, so any (tp, pp) layout
    holds exactly the same model as the single-device one. ``weight_format`` (default: the
    model's own) packs every layer right after it is drawn, so a 70B-class model never exists
    in bf16 as a whole."""
    weight_format = weight_format if weight_format is not None else cfg.weight_format
    device = torch.device(device)
    if cfg.arch == "rwkv7":
        from .rwkv import random_rwkv7_state_dict, weights_from_state_dict
        if tp > 1 or (layers is not None and len(layers) != cfg.num_layers):
            raise NotImplementedError("RWKV models run on one rank and one pipeline stage")
        return weights_from_state_dict(cfg, random_rwkv7_state_dict(cfg, seed), device, dtype)
    if cfg.arch == "rwkv6":
        from .rwkv import random_rwkv6_state_dict, rwkv6_weights_from_state_dict
        if tp > 1 or (layers is not None and len(layers) != cfg.num_layers):
            raise NotImplementedError("RWKV models run on one rank and one pipeline stage")
        return rwkv6_weights_from_state_dict(cfg, random_rwkv6_state_dict(cfg, seed), device, dtype)
    sp = make_shard_spec(cfg, tp, tp_rank, expert_parallel)
    D, H = cfg.head_dim, cfg.hidden_size
    layers = range(cfg.num_layers) if layers is None else layers

    def gen_for(*key):
        g = torch.Generator(device=device)
        digest = hashlib.sha256(repr((seed,) + key).encode()).digest()
        g.manual_seed(int.from_bytes(digest[:6], "little"))
        return g

    def full(shape, *key, std=0.02):
        return _randn(shape, gen_for(*key), device, dtype, std)

    ones = lambda n: torch.ones(n, device=device, dtype=dtype)
    out_layers = []
    for li in layers:
        if cfg.layer_kind(li) != "attention":
            from .recurrent import init_random_mixer
            if tp > 1:
                raise NotImplementedError("recurrent and latent-attention layers are not cut over tensor-parallel ranks")
            has_ffn = cfg.ffn_kind(li) != "none"
            if cfg.layer_kind(li) == "mla":
                from .mla import init_random_mla
                mixer = init_random_mla(cfg, full, li, dtype, device)
            elif cfg.layer_kind(li) == "none":
                mixer = None
            else:
                mixer = init_random_mixer(cfg, cfg.layer_kind(li), full, li, dtype, device)
            lw = LayerWeights(attn_norm=ones(H), wqkv=None, wo=None, ffn_norm=ones(H) if has_ffn else None, mixer=mixer)
            if cfg.ffn_kind(li) == "moe":
                E, I, Is = cfg.num_experts, cfg.moe_intermediate_size, cfg.shared_intermediate_size
                lw.router_w = full((E, H), li, 20, std=0.5)
                if cfg.router_kind == "deepseek_v3":
                    lw.router_select_b = full((E,), li, 21, std=0.1).float()
                lw.exp_gate_up, lw.exp_down = full((E, 2 * I, H), li, 22), full((E, H, I), li, 23)
                if Is:
                    lw.shared_gate_up = torch.cat([full((Is, H), li, 26), full((Is, H), li, 27)], 0).contiguous()
                    lw.shared_down = full((H, Is), li, 28)
            elif has_ffn:
                I = cfg.intermediate_size
                lw.w_gate_up = torch.cat([full((I, H), li, 4), full((I, H), li, 5)], 0).contiguous()
                lw.w_down = full((H, I), li, 6)
            out_layers.append(lw)
            continue
        wq = full((cfg.q_size, H), li, 0)
        wk = full((cfg.kv_size, H), li, 1)
        wv = full((cfg.kv_size, H), li, 2)
        qs = slice(sp.q_head_start * D, (sp.q_head_start + sp.hq_local) * D)
        ks = slice(sp.kv_head_start * D, (sp.kv_head_start + sp.hkv_local) * D)
        wqkv = torch.cat([wq[qs], wk[ks], wv[ks]], 0).contiguous()
        wo = full((H, cfg.q_size), li, 3)[:, qs].contiguous()
        lw = LayerWeights(attn_norm=ones(H), wqkv=wqkv, wo=wo, ffn_norm=ones(H))
        del wq, wk, wv
        if cfg.attn_bias:
            bq = full((cfg.q_size,), li, 10)
            bk = full((cfg.kv_size,), li, 11)
            bv = full((cfg.kv_size,), li, 12)
            lw.bqkv = torch.cat([bq[qs], bk[ks], bv[ks]]).contiguous()
            bo = full((H,), li, 13)
            lw.bo = bo if tp_rank == 0 else torch.zeros_like(bo)
        if cfg.qk_norm:
            lw.q_norm, lw.k_norm = ones(D), ones(D)
        if cfg.post_norms:               # not all ones, so that a test sees whether they are applied
            lw.post_attn_norm = (1.0 + 0.5 * full((H,), li, 15, std=1.0)).contiguous()
            lw.post_ffn_norm = (1.0 + 0.5 * full((H,), li, 16, std=1.0)).contiguous()
        if cfg.attn_sinks:
            s = torch.randn(cfg.num_heads, generator=gen_for(li, 14), device=device) * 0.5
            lw.sinks = s[sp.q_head_start: sp.q_head_start + sp.hq_local].float().contiguous()
        if cfg.is_moe:
            E, I = cfg.num_experts, cfg.moe_intermediate_size
            lw.router_w = full((E, H), li, 20)
            lw.router_b = full((E,), li, 21) if cfg.expert_bias else None
            gu = full((E, 2 * I, H), li, 22)
            dn = full((E, H, I), li, 23)
            gub = full((E, 2 * I), li, 24) if cfg.expert_bias else None
            dnb = full((E, H), li, 25) if cfg.expert_bias else None
            if sp.expert_parallel:
                es = slice(sp.expert_start, sp.expert_start + sp.expert_local)
                lw.exp_gate_up, lw.exp_down = gu[es].contiguous(), dn[es].contiguous()
                lw.exp_gate_up_b = gub[es].contiguous() if gub is not None else None
                lw.exp_down_b = dnb[es].contiguous() if dnb is not None else None
            else:
                lw.exp_gate_up = _cut_gate_up(gu, cfg, sp, dim=1)
                lw.exp_down = dn[:, :, sp.inter_start: sp.inter_start + sp.inter_local].contiguous()
                lw.exp_gate_up_b = _cut_gate_up(gub, cfg, sp, dim=1) if gub is not None else None
                if dnb is not None:
                    lw.exp_down_b = dnb if tp_rank == 0 else torch.zeros_like(dnb)
        else:
            I = cfg.intermediate_size
            g = full((I, H), li, 4)
            u = full((I, H), li, 5)
            isl = slice(sp.inter_start, sp.inter_start + sp.inter_local)
            lw.w_gate_up = torch.cat([g[isl], u[isl]], 0).contiguous()
            lw.w_down = full((H, I), li, 6)[:, isl].contiguous()
        pack_layer(lw, weight_format)
        out_layers.append(lw)

    embed = full((cfg.vocab_size, H), "embed") if first_stage or cfg.tie_embeddings else \
        torch.empty(0, H, device=device, dtype=dtype)
    head_full = embed if cfg.tie_embeddings else (full((cfg.vocab_size, H), "head") if last_stage else None)
    v0 = tp_rank * sp.vocab_chunk if tp > 1 else 0
    if head_full is None:
        lm_head = torch.empty(0, H, device=device, dtype=dtype)
        v_local = 0
    elif tp > 1:
        v1 = min(v0 + sp.vocab_chunk, cfg.vocab_size)
        v_local = max(v1 - v0, 0)
        lm_head = torch.zeros(sp.vocab_chunk, H, device=device, dtype=dtype)
        if v_local:
            lm_head[:v_local] = head_full[v0:v1]
    else:
        lm_head, v_local = head_full, cfg.vocab_size
    if not first_stage and not cfg.tie_embeddings:
        embed = torch.empty(0, H, device=device, dtype=dtype)
    return DecoderWeights(embed=embed, layers=out_layers, final_norm=ones(H), lm_head=lm_head,
                          vocab_start=v0, vocab_local=v_local)


def _cut_gate_up(t, cfg: ModelConfig, sp: ShardSpec, dim: int):
    """Cut a fused gate/up tensor along `dim` (size 2*I). For the interleaved gpt-oss layout the
    (gate, up) pairs stay together; otherwise the gate half and the up half are cut separately."""
    I = t.shape[dim] // 2
    if cfg.act == "swiglu_oai":
        return t.narrow(dim, 2 * sp.inter_start, 2 * sp.inter_local).contiguous()
    g = t.narrow(dim, sp.inter_start, sp.inter_local)
    u = t.narrow(dim, I + sp.inter_start, sp.inter_local)
    return torch.cat([g, u], dim).contiguous()
