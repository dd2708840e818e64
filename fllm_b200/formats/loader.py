"""Model loading: a Hugging Face checkpoint directory (config.json + *.safetensors) or a GGUF file
-> (ModelConfig, DecoderWeights for this tensor-parallel rank, tokenizer path).

Projections are fused the way the kernels want them (q|k|v rows, gate|up rows) and cut for tensor
parallelism with the rules of ``models.weights``. Block-wise FP8 checkpoints (``weight_scale_inv``
tensors, 128 x 128 blocks) stay packed: the e4m3 bytes and their scales go to the GPU untouched
and run on the FP8 tensor cores. GGUF K-quants are consumed packed by the CPU engine; for the GPU
path they are expanded to bf16 once at load time
(rust/checkpoint/src/convert.rs:1290-1559 is the reference's importer).
"""
from __future__ import annotations

import json
import os
from typing import Optional, Tuple

import numpy as np
import torch

from ..config import CLASSIC_MODEL_TYPES, ModelConfig
from ..models.weights import DecoderWeights, LayerWeights, make_shard_spec


def _cut_rows(t: torch.Tensor, start: int, n: int) -> torch.Tensor:
    return t[start:start + n]


def load_hf_checkpoint(directory: str, device="cuda", tp: int = 1, tp_rank: int = 0, dtype=torch.bfloat16,
                       expert_parallel: bool = False):
    from .safetensors_io import open_checkpoint
    from ..ops.int4 import Int4Weight
    from .int4_checkpoints import int4_linear
    hf = json.load(open(os.path.join(directory, "config.json")))
    cfg = ModelConfig.from_hf_config(hf)
    qcfg = hf.get("quantization_config") or {}
    sp = make_shard_spec(cfg, tp, tp_rank, expert_parallel)
    ck = open_checkpoint(directory)
    D = cfg.head_dim

    def get(name, required=True):
        if name not in ck:
            if required:
                raise KeyError(f"checkpoint has no tensor {name!r}")
            return None
        f, n = ck[name]
        return f.tensor(n)

    def dev(t):
        return t.to(device=device, dtype=dtype if t.is_floating_point() and t.element_size() > 1 else t.dtype).contiguous()

    if cfg.arch in CLASSIC_MODEL_TYPES:
        if tp > 1:
            raise NotImplementedError(f"{cfg.arch} runs on one rank")
        from .classic_loader import load_hf_classic
        tok = directory if os.path.exists(os.path.join(directory, "tokenizer.json")) else None
        return cfg, load_hf_classic(cfg, get, device, dtype), tok
    if cfg.layer_kinds:
        if tp > 1:
            raise NotImplementedError("recurrent and latent-attention layers are not cut over tensor-parallel ranks")
        from .recurrent_loader import load_hf_recurrent
        tok = directory if os.path.exists(os.path.join(directory, "tokenizer.json")) else None
        if cfg.arch == "rwkv7":
            from ..models.rwkv import weights_from_state_dict
            return cfg, weights_from_state_dict(cfg, {k: get(k) for k in ck}, device, dtype), tok
        if cfg.arch == "rwkv6":
            from ..models.rwkv import rwkv6_weights_from_state_dict
            return cfg, rwkv6_weights_from_state_dict(cfg, {k: get(k) for k in ck}, device, dtype), tok
        return cfg, load_hf_recurrent(cfg, get, device, dtype), tok

    def has(name):
        return name + ".weight" in ck or name + ".qweight" in ck

    mlx_q = hf.get("quantization") if isinstance(hf.get("quantization"), dict) else None
    if mlx_q is None and isinstance(qcfg, dict) and "group_size" in qcfg and "bits" in qcfg and "quant_method" not in qcfg:
        mlx_q = qcfg

    def lin(name):
        """A projection by its module name: a tensor [N, K], or an Int4Weight for AWQ / GPTQ / MLX 4-bit tensors;
        bitsandbytes 4-bit layers are expanded."""
        if mlx_q is not None and name + ".scales" in ck and name + ".biases" in ck:
            from .extra_quant import mlx_linear
            per = mlx_q.get(name) if isinstance(mlx_q.get(name), dict) else mlx_q       # a layer may override bits / group
            return mlx_linear(get(name + ".weight"), get(name + ".scales"), get(name + ".biases"), int(per.get("bits", 4)),
                              int(per.get("group_size", 64)), dtype)
        if name + ".weight.absmax" in ck:
            from .extra_quant import bnb_linear
            w = bnb_linear(get, name, dtype)
            if w is not None:
                return w
        if name + ".qweight" in ck:
            return int4_linear(qcfg.get("quant_method", "gptq"), get(name + ".qweight"), get(name + ".qzeros"),
                               get(name + ".scales"), get(name + ".g_idx", False),
                               qcfg.get("checkpoint_format", "gptq"), dtype)
        return get(name + ".weight")

    def rows(w, sl):
        return w.rows(sl) if isinstance(w, Int4Weight) else w[sl]

    def cols(w, sl):
        if isinstance(w, Int4Weight):
            if sl.start % 64 == 0 and sl.stop % 64 == 0:
                return w.cols(sl)
            w = w.dense().to(dtype)
        return w[:, sl]

    def cat(parts):
        if all(isinstance(x, Int4Weight) for x in parts):
            return Int4Weight.cat(parts)
        return torch.cat([x.dense().to(dtype) if isinstance(x, Int4Weight) else x for x in parts], 0)

    def put(w):
        return w.to(device) if isinstance(w, Int4Weight) else dev(w)

    res_mult = float(hf.get("residual_multiplier") or 1.0) if hf.get("model_type") == "granite" else 1.0
    logit_div = float(hf.get("logits_scaling") or 1.0) if hf.get("model_type") == "granite" else 1.0
    qs = slice(sp.q_head_start * D, (sp.q_head_start + sp.hq_local) * D)
    ks = slice(sp.kv_head_start * D, (sp.kv_head_start + sp.hkv_local) * D)
    isl = slice(sp.inter_start, sp.inter_start + sp.inter_local)
    nq, nk, inter = cfg.num_heads * D, cfg.num_kv_heads * D, cfg.intermediate_size
    layers = []
    for l in range(cfg.num_layers):
        p = f"model.layers.{l}."
        if has(p + "self_attn.q_proj"):
            q, k, v = (lin(p + f"self_attn.{n}_proj") for n in "qkv")
        else:                                  # Phi-3: one fused q|k|v projection
            f = lin(p + "self_attn.qkv_proj")
            q, k, v = rows(f, slice(0, nq)), rows(f, slice(nq, nq + nk)), rows(f, slice(nq + nk, nq + 2 * nk))
        fp8 = isinstance(q, torch.Tensor) and q.dtype == torch.float8_e4m3fn
        if cfg.post_norms and has(p + "self_attn.q_proj") and (p + "post_self_attn_layernorm.weight") in ck:      # GLM-4
            lw = LayerWeights(attn_norm=dev(get(p + "input_layernorm.weight")), wqkv=None, wo=None,
                              ffn_norm=dev(get(p + "post_attention_layernorm.weight")),
                              post_attn_norm=dev(get(p + "post_self_attn_layernorm.weight")),
                              post_ffn_norm=dev(get(p + "post_mlp_layernorm.weight")))
        elif cfg.post_norms:                   # Gemma-2: post_attention_layernorm normalises the attention OUTPUT
            lw = LayerWeights(attn_norm=dev(get(p + "input_layernorm.weight")), wqkv=None, wo=None,
                              ffn_norm=dev(get(p + "pre_feedforward_layernorm.weight")),
                              post_attn_norm=dev(get(p + "post_attention_layernorm.weight")),
                              post_ffn_norm=dev(get(p + "post_feedforward_layernorm.weight")))
        else:
            # VaultGemma names its second norm like Gemma-2 does, without having the norms behind the blocks
            second = "pre_feedforward_layernorm" if (p + "pre_feedforward_layernorm.weight") in ck else "post_attention_layernorm"
            lw = LayerWeights(attn_norm=dev(get(p + "input_layernorm.weight")), wqkv=None, wo=None,
                              ffn_norm=dev(get(p + second + ".weight")))
        o = lin(p + "self_attn.o_proj")
        if cfg.is_moe:
            _load_moe_layer(cfg, sp, tp_rank, lw, p, get, dev)
            lw.wqkv = put(cat([rows(q, qs), rows(k, ks), rows(v, ks)]))
            lw.wo = put(cols(o, qs))
            g = u = d = None
        elif has(p + "mlp.gate_proj"):
            g, u, d = (lin(p + f"mlp.{n}_proj") for n in ("gate", "up", "down"))
        else:                                  # Phi-3: one fused gate|up projection
            f = lin(p + "mlp.gate_up_proj")
            g, u, d = rows(f, slice(0, inter)), rows(f, slice(inter, 2 * inter)), lin(p + "mlp.down_proj")
        if cfg.is_moe:
            pass
        elif fp8:
            def sc(name):
                return get(p + name + ".weight_scale_inv").float()
            def rows(t, s, sl):            # cut rows of codes and of their 128-row scale blocks
                return t[sl], s[sl.start // 128: -(-sl.stop // 128)]
            def cols(t, s, sl):
                return t[:, sl], s[:, sl.start // 128: -(-sl.stop // 128)]
            parts = [rows(q, sc("self_attn.q_proj"), qs), rows(k, sc("self_attn.k_proj"), ks), rows(v, sc("self_attn.v_proj"), ks)]
            lw.packed["wqkv"] = ("fp8_block", torch.cat([a for a, _ in parts]).view(torch.uint8).to(device).contiguous(),
                                 torch.cat([b for _, b in parts]).to(device).contiguous())
            a, b = cols(o, sc("self_attn.o_proj"), qs)
            lw.packed["wo"] = ("fp8_block", a.view(torch.uint8).to(device).contiguous(), b.to(device).contiguous())
            parts = [rows(g, sc("mlp.gate_proj"), isl), rows(u, sc("mlp.up_proj"), isl)]
            lw.packed["w_gate_up"] = ("fp8_block", torch.cat([a for a, _ in parts]).view(torch.uint8).to(device).contiguous(),
                                      torch.cat([b for _, b in parts]).to(device).contiguous())
            a, b = cols(d, sc("mlp.down_proj"), isl)
            lw.packed["w_down"] = ("fp8_block", a.view(torch.uint8).to(device).contiguous(), b.to(device).contiguous())
        else:
            lw.wqkv = put(cat([rows(q, qs), rows(k, ks), rows(v, ks)]))
            lw.wo = put(cols(o, qs))
            lw.w_gate_up = put(cat([rows(g, isl), rows(u, isl)]))
            lw.w_down = put(cols(d, isl))
        if cfg.attn_bias:
            bq, bk, bv = (get(p + f"self_attn.{n}_proj.bias", False) for n in "qkv")
            if bq is not None:
                lw.bqkv = dev(torch.cat([bq[qs], bk[ks], bv[ks]]))
            bo = get(p + "self_attn.o_proj.bias", False)
            if bo is not None:
                lw.bo = dev(bo if tp_rank == 0 else torch.zeros_like(bo))
        if cfg.qk_norm_full:                   # one norm over all heads of q, one over all heads of k (one rank)
            if tp > 1:
                raise NotImplementedError("QK-norm over all heads is not cut over tensor-parallel ranks")
            lw.q_norm_full, lw.k_norm_full = dev(get(p + "self_attn.q_norm.weight")), dev(get(p + "self_attn.k_norm.weight"))
        if cfg.qk_norm:
            lw.q_norm, lw.k_norm = dev(get(p + "self_attn.q_norm.weight")), dev(get(p + "self_attn.k_norm.weight"))
            if cfg.qk_norm_offset:             # the fused kernel multiplies by w: fold the 1 + w convention into it
                lw.q_norm, lw.k_norm = dev(lw.q_norm.float() + cfg.qk_norm_offset), dev(lw.k_norm.float() + cfg.qk_norm_offset)
        if res_mult != 1.0:                    # Granite: block output * multiplier, folded into the block's last projection
            for name in ("wo", "bo", "w_down"):
                t = getattr(lw, name, None)
                if isinstance(t, torch.Tensor):
                    setattr(lw, name, dev(t.float() * res_mult))
        if cfg.attn_sinks:
            sk = get(p + "self_attn.sinks", False)
            if sk is not None:
                lw.sinks = sk[sp.q_head_start: sp.q_head_start + sp.hq_local].float().to(device).contiguous()
        layers.append(lw)
    embed = get("model.embed_tokens.weight")
    head = get("lm_head.weight", False)
    if head is None or cfg.tie_embeddings:
        head = embed
    if logit_div != 1.0:                       # logits / divisor: a scaled head of its own
        head = head.float() / logit_div
    v0, vl = 0, cfg.vocab_size
    if tp > 1:
        v0 = tp_rank * sp.vocab_chunk
        v1 = min(v0 + sp.vocab_chunk, cfg.vocab_size)
        vl = max(v1 - v0, 0)
        hl = torch.zeros(sp.vocab_chunk, cfg.hidden_size, dtype=head.dtype)
        hl[:vl] = head[v0:v1]
        head = hl
    w = DecoderWeights(embed=dev(embed), layers=layers, final_norm=dev(get("model.norm.weight")), lm_head=dev(head),
                       vocab_start=v0, vocab_local=vl)
    tok = directory if os.path.exists(os.path.join(directory, "tokenizer.json")) else None
    return cfg, w, tok


def _mxfp4_stack(blocks: torch.Tensor, scales: torch.Tensor) -> torch.Tensor:
    """gpt-oss expert tensor: blocks uint8 [E, rows, K/32, 16] (two e2m1 per byte, low nibble first) and
    scales uint8 [E, rows, K/32] (e8m0) -> fp32 [E, rows, K]."""
    from ..ops.fp4 import MXFP4, dequantize_fp4
    E, R, G, _ = blocks.shape
    d = dequantize_fp4(blocks.reshape(E * R, G * 16), scales.reshape(E * R, G), MXFP4)
    return d.view(E, R, G * 32)


def _load_moe_layer(cfg, sp, tp_rank, lw, p, get, dev) -> None:
    """Router and experts of a gpt-oss style layer (`mlp.router`, `mlp.experts.{gate_up,down}_proj`): bf16
    tensors are taken as they are ([E, in, out] in the checkpoint), MXFP4 `_blocks` / `_scales` pairs
    ([E, out, in/32, 16]) are expanded to bf16. The grouped expert GEMM runs bf16 stacks."""
    from ..models.weights import _cut_gate_up
    if get(p + "mlp.router.weight", False) is None:
        return _load_per_expert_moe(cfg, sp, tp_rank, lw, p, get, dev)
    lw.router_w = dev(get(p + "mlp.router.weight"))
    rb = get(p + "mlp.router.bias", False)
    lw.router_b = dev(rb) if rb is not None else None

    # MXFP4 experts stay packed on a GPU when whole experts live on this rank (one GPU, or expert parallel)
    # and the grouped packed GEMM can address them (input width a multiple of 64)
    keep_packed = str(dev(torch.zeros(1)).device).startswith("cuda") and (sp.expert_parallel or sp.inter_local == cfg.moe_intermediate_size)

    def expert(name):
        blk = get(p + f"mlp.experts.{name}_blocks", False)
        if blk is not None:
            sc = get(p + f"mlp.experts.{name}_scales")
            if keep_packed and (blk.shape[2] * 32) % 64 == 0:
                from ..ops.fp4 import MXFP4, Fp4ExpertStack
                E, R, G, _ = blk.shape
                return Fp4ExpertStack(blk.reshape(E, R, G * 16), sc.reshape(E, R, G), MXFP4)
            return _mxfp4_stack(blk, sc)                                               # [E, out, in]
        return get(p + f"mlp.experts.{name}").float().transpose(1, 2)                # stored [E, in, out]
    gu, dn = expert("gate_up_proj"), expert("down_proj")
    if not isinstance(gu, torch.Tensor) or not isinstance(dn, torch.Tensor):
        es = slice(sp.expert_start, sp.expert_start + sp.expert_local) if sp.expert_parallel else slice(None)
        gub, dnb = get(p + "mlp.experts.gate_up_proj_bias", False), get(p + "mlp.experts.down_proj_bias", False)
        pick = lambda t: (t[es].to(dev(torch.zeros(1)).device) if not isinstance(t, torch.Tensor) else dev(t[es]))
        lw.exp_gate_up, lw.exp_down = pick(gu), pick(dn)
        lw.exp_gate_up_b = dev(gub[es]) if gub is not None else None
        lw.exp_down_b = dev(dnb[es]) if dnb is not None else None
        return
    gub, dnb = get(p + "mlp.experts.gate_up_proj_bias", False), get(p + "mlp.experts.down_proj_bias", False)
    if sp.expert_parallel:
        es = slice(sp.expert_start, sp.expert_start + sp.expert_local)
        lw.exp_gate_up, lw.exp_down = dev(gu[es]), dev(dn[es])
        lw.exp_gate_up_b = dev(gub[es]) if gub is not None else None
        lw.exp_down_b = dev(dnb[es]) if dnb is not None else None
    else:
        lw.exp_gate_up = dev(_cut_gate_up(gu, cfg, sp, dim=1))
        lw.exp_down = dev(dn[:, :, sp.inter_start: sp.inter_start + sp.inter_local])
        lw.exp_gate_up_b = dev(_cut_gate_up(gub, cfg, sp, dim=1)) if gub is not None else None
        if dnb is not None:
            lw.exp_down_b = dev(dnb if tp_rank == 0 else torch.zeros_like(dnb))


def _load_per_expert_moe(cfg, sp, tp_rank, lw, p, get, dev) -> None:
    """Mixtral (`block_sparse_moe.gate`, `experts.N.w1 / w3 / w2`) and Qwen-MoE (`mlp.gate`,
    `experts.N.gate_proj / up_proj / down_proj`): one tensor per expert and projection, stacked here
    into [E, 2I, H] (gate rows then up rows) and [E, H, I]."""
    from ..models.weights import _cut_gate_up
    if get(p + "block_sparse_moe.gate.weight", False) is not None:
        base, names, router = p + "block_sparse_moe.", ("w1", "w3", "w2"), "block_sparse_moe.gate.weight"
    else:
        base, names, router = p + "mlp.", ("gate_proj", "up_proj", "down_proj"), "mlp.gate.weight"
    lw.router_w = dev(get(p + router))
    lw.router_b = None
    sel = get(base + "e_score_correction_bias", False)            # MiniMax-M2: a bias that only steers the selection
    if sel is not None:
        lw.router_select_b = sel.float().reshape(-1).to(lw.router_w.device).contiguous()
    experts = range(sp.expert_start, sp.expert_start + sp.expert_local) if sp.expert_parallel else range(cfg.num_experts)
    fused = get(base + "experts.gate_up_proj", False)
    if fused is not None:                      # newer checkpoints: one [E, 2I, H] and one [E, H, I] tensor per layer
        es = slice(experts.start, experts.stop)
        gu, dn = fused[es], get(base + "experts.down_proj")[es]
    else:
        gu = torch.stack([torch.cat([get(f"{base}experts.{e}.{names[0]}.weight"), get(f"{base}experts.{e}.{names[1]}.weight")], 0)
                          for e in experts])
        dn = torch.stack([get(f"{base}experts.{e}.{names[2]}.weight") for e in experts])
    if sp.expert_parallel:
        lw.exp_gate_up, lw.exp_down = dev(gu), dev(dn)
    else:
        lw.exp_gate_up = dev(_cut_gate_up(gu, cfg, sp, dim=1))
        lw.exp_down = dev(dn[:, :, sp.inter_start: sp.inter_start + sp.inter_local])
    lw.exp_gate_up_b = lw.exp_down_b = None
    sg = get(base + "shared_expert.gate_proj.weight", False)
    if sg is not None:                         # Qwen2-MoE: an always-on expert whose output is scaled by sigmoid(h . g)
        su, sd = get(base + "shared_expert.up_proj.weight"), get(base + "shared_expert.down_proj.weight")
        Is = sg.shape[0]
        per = Is // sp.tp if (sp.tp > 1 and Is % (sp.tp * 8) == 0) else Is
        if sp.tp > 1 and per == Is:
            raise ValueError(f"the shared expert's width {Is} cannot be divided over tp={sp.tp}")
        sl = slice(sp.tp_rank * per, (sp.tp_rank + 1) * per) if sp.tp > 1 else slice(0, Is)
        lw.shared_gate_up, lw.shared_down = dev(torch.cat([sg[sl], su[sl]], 0)), dev(sd[:, sl])
        g1 = get(base + "shared_expert_gate.weight", False)
        if g1 is not None:
            lw.shared_gate_w = dev(torch.cat([g1, torch.zeros(7, g1.shape[1], dtype=g1.dtype)], 0))


def load_gguf(path: str, device="cuda", tp: int = 1, tp_rank: int = 0, dtype=torch.bfloat16, keep_packed: bool = True):
    """GGUF -> weights. On a GPU (`keep_packed`), 4-bit group types (Q4_K, Q4_0, Q4_1) stay packed as
    ``Int4Weight``, Q5_K / Q6_K / Q8_0 as ``IntKWeight`` planes, fused projections of mixed types as a
    ``StackedWeight``; every other type is expanded to bf16."""
    from ..cpu_engine import config_from_gguf
    from ..ops.int4 import Int4Weight
    from ..ops.intk import IntKWeight, StackedWeight
    from .gguf import GgufReader
    r = GgufReader(path)
    cfg = config_from_gguf(r)
    sp = make_shard_spec(cfg, tp, tp_rank)
    D = cfg.head_dim
    t = lambda n: torch.from_numpy(r.tensor_f32(n))
    dev = lambda x: x.to(device=device, dtype=dtype).contiguous()
    qs = slice(sp.q_head_start * D, (sp.q_head_start + sp.hq_local) * D)
    ks = slice(sp.kv_head_start * D, (sp.kv_head_start + sp.hkv_local) * D)
    isl = slice(sp.inter_start, sp.inter_start + sp.inter_local)
    packed_ok = keep_packed and torch.device(device).type == "cuda"

    def packed(name):
        """The tensor in its packed device form (4-bit group types, Q5_K / Q6_K / Q8_0 planes), or None."""
        info = r.tensors[name]
        if not packed_ok or len(info.shape) < 2:
            return None
        rows, cols = int(info.shape[-2]), int(info.shape[-1])
        if info.type_name in ("Q4_K", "Q4_0", "Q4_1") and cols % 64 == 0:
            return Int4Weight.from_gguf(info.type_name, r.tensor_bytes(name), rows, cols)
        if IntKWeight.supports(info.type_name, cols):
            return IntKWeight.from_gguf(info.type_name, r.tensor_bytes(name), rows, cols)
        return None

    def fused_rows(names, cuts):
        """Row-concatenation of row-cut tensors: one INT4 weight when every part has that form, a stack of
        differently typed parts when some are packed (a Q4_K_M file mixes Q4_K and Q6_K inside q|k|v), else bf16."""
        parts = [packed(n) for n in names]
        if all(isinstance(p, Int4Weight) for p in parts):
            return Int4Weight.cat([p.rows(c) for p, c in zip(parts, cuts)]).to(device)
        if any(p is not None for p in parts):
            return StackedWeight([p.rows(c).to(device) if p is not None else dev(t(n)[c])
                                  for p, n, c in zip(parts, names, cuts)])
        return dev(torch.cat([t(n)[c] for n, c in zip(names, cuts)], 0))

    def col_cut(name, cut):
        p = packed(name)
        unit = 64 if isinstance(p, Int4Weight) else (32 if getattr(p, "fmt", 0) == 8 else 256)
        if p is not None and cut.start % unit == 0 and cut.stop % unit == 0:
            return p.cols(cut).to(device)
        return dev(t(name)[:, cut])

    layers = []
    for l in range(cfg.num_layers):
        p = f"blk.{l}."
        lw = LayerWeights(
            attn_norm=dev(t(p + "attn_norm.weight")),
            wqkv=fused_rows([p + "attn_q.weight", p + "attn_k.weight", p + "attn_v.weight"], [qs, ks, ks]),
            wo=col_cut(p + "attn_output.weight", qs), ffn_norm=dev(t(p + "ffn_norm.weight")),
            w_gate_up=fused_rows([p + "ffn_gate.weight", p + "ffn_up.weight"], [isl, isl]),
            w_down=col_cut(p + "ffn_down.weight", isl))
        if p + "attn_q_norm.weight" in r.tensors:
            lw.q_norm, lw.k_norm = dev(t(p + "attn_q_norm.weight")), dev(t(p + "attn_k_norm.weight"))
        layers.append(lw)
    embed = t("token_embd.weight")
    head = t("output.weight") if "output.weight" in r.tensors and not cfg.tie_embeddings else embed
    v0, vl = 0, cfg.vocab_size
    if tp > 1:
        v0 = tp_rank * sp.vocab_chunk
        v1 = min(v0 + sp.vocab_chunk, cfg.vocab_size)
        vl = max(v1 - v0, 0)
        hl = torch.zeros(sp.vocab_chunk, cfg.hidden_size)
        hl[:vl] = head[v0:v1]
        head = hl
    w = DecoderWeights(embed=dev(embed), layers=layers, final_norm=dev(t("output_norm.weight")), lm_head=dev(head),
                       vocab_start=v0, vocab_local=vl)
    has_tok = "tokenizer.ggml.tokens" in r.metadata
    r.close()
    return cfg, w, (path if has_tok else None)


def load_model(path: str, device="cuda", tp: int = 1, tp_rank: int = 0):
    if path.endswith(".gguf"):
        return load_gguf(path, device, tp, tp_rank)
    return load_hf_checkpoint(path, device, tp, tp_rank)
