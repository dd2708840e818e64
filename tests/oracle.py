"""Independent dense (non-paged, whole-sequence) fp32 decoder used as the oracle for the
paged / scheduled / fused pipeline. It shares only the weight tensors with the engine."""
import math

import torch

from fllm_b200.models.weights import gate_up_natural
import torch.nn.functional as F

from fllm_b200.config import ModelConfig, rope_inv_freq


def _rms(x, w, eps, off=0.0):
    return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * (w.float() + off)


def _bf(x):
    return x.to(torch.bfloat16).float()


def dense_forward(cfg: ModelConfig, w, tokens, round_bf16=True):
    """Logits [len(tokens), vocab] of a full causal forward (single device weights)."""
    r = _bf if round_bf16 else (lambda t: t)
    T = len(tokens)
    ids = torch.tensor(tokens, dtype=torch.long, device=w.embed.device)
    x = w.embed[ids].float() * cfg.embed_scale
    inv, attn_f = rope_inv_freq(cfg)
    inv = torch.tensor(inv, dtype=torch.float32, device=x.device)
    pos = torch.arange(T, dtype=torch.float32, device=x.device)
    ang = pos[:, None] * inv[None]
    cos, sin = ang.cos() * attn_f, ang.sin() * attn_f
    D, hq, hkv = cfg.head_dim, cfg.num_heads, cfg.num_kv_heads
    rot = cfg.rot_dim

    def rope(t):
        a, b = t[..., : rot // 2], t[..., rot // 2: rot]
        c, s = cos[:, None], sin[:, None]
        if cfg.rope_style == "neox":
            out = torch.cat([a * c - b * s, b * c + a * s], -1)
        else:
            a, b = t[..., 0:rot:2], t[..., 1:rot:2]
            out = torch.stack([a * c - b * s, b * c + a * s], -1).flatten(-2)
        return torch.cat([out, t[..., rot:]], -1)

    for li, lw in enumerate(w.layers):
        h = r(_rms(x, lw.attn_norm, cfg.rms_eps, cfg.norm_weight_offset))
        qkv = h @ lw.wqkv.float().t()
        if lw.bqkv is not None:
            qkv = qkv + lw.bqkv.float()
        qkv = r(qkv).view(T, hq + 2 * hkv, D)
        q, k, v = qkv[:, :hq], qkv[:, hq:hq + hkv], qkv[:, hq + hkv:]
        if lw.q_norm is not None:
            q = r(_rms(q, lw.q_norm, cfg.rms_eps))
            k = r(_rms(k, lw.k_norm, cfg.rms_eps))
        q, k = r(rope(q)), r(rope(k))
        g = hq // hkv
        kk, vv = k.repeat_interleave(g, 1), v.repeat_interleave(g, 1)
        s = torch.einsum("thd,shd->hts", q, kk) * (cfg.attn_scale if cfg.attn_scale else D ** -0.5)
        if cfg.attn_softcap > 0:
            s = cfg.attn_softcap * torch.tanh(s / cfg.attn_softcap)
        i = torch.arange(T, device=x.device)
        mask = i[None, :] <= i[:, None]
        win = cfg.layer_window(li)
        if win > 0:
            mask = mask & (i[None, :] > i[:, None] - win)
        s = s.masked_fill(~mask[None], float("-inf"))
        if lw.sinks is not None:
            s = torch.cat([s, lw.sinks.float()[:, None, None].expand(hq, T, 1)], -1)
            p = torch.softmax(s, -1)[..., :-1]
        else:
            p = torch.softmax(s, -1)
        a = r(torch.einsum("hts,shd->thd", p, vv).reshape(T, hq * D))
        o = a @ lw.wo.float().t()
        if lw.bo is not None:
            o = o + lw.bo.float()
        if lw.post_attn_norm is not None:
            o = _rms(r(o), lw.post_attn_norm, cfg.rms_eps, cfg.norm_weight_offset)
        x = r(x + r(o))
        h = r(_rms(x, lw.ffn_norm, cfg.rms_eps, cfg.norm_weight_offset))
        if cfg.is_moe:
            from fllm_b200.models.moe import moe_reference
            d = moe_reference(cfg, lw, h)
        else:
            gu = r(h @ gate_up_natural(lw).float().t())
            I = gu.shape[1] // 2
            gate = F.gelu(gu[:, :I], approximate="tanh") if cfg.act == "geglu" else F.silu(gu[:, :I])
            act = r(gate * gu[:, I:])
            d = act @ lw.w_down.float().t()
        if lw.post_ffn_norm is not None:
            d = _rms(r(d), lw.post_ffn_norm, cfg.rms_eps, cfg.norm_weight_offset)
        x = r(x + r(d))
    h = r(_rms(x, w.final_norm, cfg.rms_eps, cfg.norm_weight_offset))
    return r(h @ w.lm_head.float().t())[:, : cfg.vocab_size]


def greedy_generate(cfg, w, prompt, n):
    toks = list(prompt)
    for _ in range(n):
        lg = dense_forward(cfg, w, toks)
        toks.append(int(lg[-1].argmax()))
    return toks[len(prompt):]
