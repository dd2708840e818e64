"""RWKV-6 ("Finch") and RWKV-7 ("Goose") as families of the decoder runner. RWKV-7: LayerNorm blocks, token shift, low-rank decay / value-mix /
in-context-learning-rate / gate branches, the generalised delta-rule state per head, a per-head GroupNorm with the
r.k bonus, and the squared-ReLU channel mix.

The reference runs the family in rust/engine/src/rust_decoder/rwkv.rs with the state update in rust/engine/cuda/rwkv.cu
and keeps a PyTorch transcription of the official recurrence in scripts/rwkv_reference.py. Tensor names are those of the
Hugging Face ``RWKV7ForCausalLM`` layout (``model.layers.N.attn.*``, ``attn_norm``, ``ffn_norm``, ``ffn.*``, ``pre_norm`` in
layer 0). RWKV-6 (``Rwkv6ForCausalLM`` layout: ``rwkv.blocks.N.attention.*``, ``ln1``, ``ln2``, ``feed_forward.*``, ``pre_ln`` in
block 0) has data-dependent mixing coefficients and decays from low-rank branches, a bonus vector for the current token,
a SiLU gate and a receptance-gated channel mix.

Token shift is a two-tap causal convolution with taps (+1, -1): its output is ``previous - current`` and its window
is the previous row, kept per sequence in the state pool, so chunked prefill and decode need no special case.
"""
from __future__ import annotations

from typing import Dict

import torch
import torch.nn.functional as F

from ..config import ModelConfig
from ..ops.recurrent import RWKV6, RWKV7

DECAY_SCALE = -0.6065306597126334            # -exp(-0.5): decay = exp(DECAY_SCALE * sigmoid(.)) lies in (0.545, 1)


def _ln(x, w, b, eps):
    return F.layer_norm(x.float(), (x.shape[-1],), w.float(), b.float(), eps).to(x.dtype)


def _shift_taps(C: int, device) -> torch.Tensor:
    t = torch.empty(C, 2, dtype=torch.float32, device=device)
    t[:, 0], t[:, 1] = 1.0, -1.0
    return t


def rwkv7_forward_hidden(dec, b):
    """All layers of this stage; returns (residual stream, None). ``dec.rstate`` holds, per layer, the two token-shift
    rows (``conv`` for the time mix, ``shift2`` for the channel mix) and the matrix state ``scan`` [slots, H, N, N]."""
    cfg, ops, st = dec.cfg, dec.ops, dec.rstate
    eps, N = cfg.rms_eps, cfg.ssm["head_dim"]
    C = cfg.hidden_size
    H = C // N
    qs, ss, pos = b.q_starts, b.seq_state, b.positions
    x = ops.embed(b.token_ids, dec.w.embed, 1.0)
    T = x.shape[0]
    taps = getattr(dec, "_shift_taps", None)
    if taps is None:
        taps = dec._shift_taps = _shift_taps(C, x.device)
    v_first = None
    lin = ops.linear

    def lora(m, name, v, act=None, bias=True):
        hmid = lin(v, m[name + "_a"])
        if act is not None:
            hmid = act(hmid.float()).to(v.dtype)
        return lin(hmid, m[name + "_b"], m.get(name + "_bias") if bias else None)

    for li, lw in zip(dec.layer_range, dec.w.layers):
        m = lw.mixer
        if "pre_norm_w" in m:
            x = _ln(x, m["pre_norm_w"], m["pre_norm_b"], eps)
        h = _ln(x, lw.attn_norm, m["attn_norm_b"], eps)
        xx = ops.causal_conv1d(h, taps, None, st.conv[li], qs, ss, pos, act=False, max_q_len=getattr(b, "max_q_len", 0))
        xr, xw, xk, xv, xa, xg = (h + xx * m["x_" + c] for c in "rwkvag")
        r, k, v = lin(xr, m["r_proj"]), lin(xk, m["k_proj"]), lin(xv, m["v_proj"])
        w = (DECAY_SCALE * torch.sigmoid(lora(m, "w", xw, torch.tanh).float())).contiguous()        # fp32 log decay
        if v_first is None:
            v_first = v
        else:
            v = v + (v_first - v) * torch.sigmoid(lora(m, "v", xv).float()).to(v.dtype)
        a = torch.sigmoid(lora(m, "a", xa).float())
        g = lora(m, "g", xg, torch.sigmoid, bias=False)
        kf = k.float()
        kk = F.normalize((kf * m["k_k"]).view(T, H, N), dim=-1, p=2.0, eps=1e-12).view(T, C)
        kf = kf * (1.0 + (a - 1.0) * m["k_a"])
        k2 = kf.to(h.dtype)
        y = ops.matrix_state_scan(RWKV7, r, k2, v, (-kk).to(h.dtype), (kk * a).to(h.dtype), w, None, None, st.scan[li], qs, ss, pos,
                                  H, N, N, 1, False, 1.0)
        yf = F.group_norm(y.float(), H, m["g_norm_w"], m["g_norm_b"], N * eps)
        bonus = (r.float().view(T, H, N) * kf.view(T, H, N) * m["r_k"]).sum(-1, keepdim=True) * v.float().view(T, H, N)
        y = ((yf + bonus.view(T, C)) * g.float()).to(h.dtype)
        x = x + lin(y, m["o_proj"])
        h2 = _ln(x, lw.ffn_norm, m["ffn_norm_b"], eps)
        xx2 = ops.causal_conv1d(h2, taps, None, st.shift2[li], qs, ss, pos, act=False, max_q_len=getattr(b, "max_q_len", 0))
        kx = h2 + xx2 * m["ffn_x_k"]
        x = x + lin(torch.relu(lin(kx, m["ffn_key"]).float()).square().to(h.dtype), m["ffn_value"])
    return x, None


def rwkv7_final_norm(dec, x):
    return _ln(x, dec.w.final_norm, dec.w.final_norm_b, dec.cfg.rms_eps)


# ------------------------------------------------------------------------------------------------ weights
def pack_rwkv7_layer(get, p: str, layer: int, dtype, device) -> Dict[str, torch.Tensor]:
    """``get(name, required=True)`` reads a checkpoint tensor; ``p`` is the layer prefix. Low-rank branches are stored
    as two linear weights [rank, C] and [C, rank] (+ bias); mixing vectors as fp32 rows."""
    bf = lambda t: t.to(device=device, dtype=dtype).contiguous()
    vec = lambda t: t.reshape(-1).to(device=device, dtype=dtype).contiguous()
    f32 = lambda t: t.float().to(device).contiguous()
    m = {"attn_norm_b": f32(get(p + "attn_norm.bias")), "ffn_norm_b": f32(get(p + "ffn_norm.bias"))}
    if get(p + "pre_norm.weight", False) is not None:
        m["pre_norm_w"], m["pre_norm_b"] = f32(get(p + "pre_norm.weight")), f32(get(p + "pre_norm.bias"))
    a = p + "attn."
    for c in "rwkvag":
        m["x_" + c] = vec(get(a + "x_" + c))
    for name in ("r_proj", "k_proj", "v_proj", "o_proj"):
        m[name] = bf(get(a + name + ".weight"))
    for name in ("w", "a", "v", "g"):
        if name == "v" and get(a + "v_lora.lora.0.weight", False) is None:
            continue                                         # layer 0 has no value mix
        m[name + "_a"] = bf(get(a + f"{name}_lora.lora.0.weight"))
        m[name + "_b"] = bf(get(a + f"{name}_lora.lora.2.weight"))
        bias = get(a + f"{name}_lora.lora.2.bias", False)
        if bias is not None:
            m[name + "_bias"] = bf(bias)
    m["k_k"], m["k_a"] = f32(get(a + "k_k").reshape(-1)), f32(get(a + "k_a").reshape(-1))
    m["r_k"] = f32(get(a + "r_k"))
    m["g_norm_w"], m["g_norm_b"] = f32(get(a + "g_norm.weight")), f32(get(a + "g_norm.bias"))
    m["ffn_x_k"] = vec(get(p + "ffn.x_k"))
    m["ffn_key"], m["ffn_value"] = bf(get(p + "ffn.key.weight")), bf(get(p + "ffn.value.weight"))
    return m


def random_rwkv7_state_dict(cfg: ModelConfig, seed: int = 0) -> Dict[str, torch.Tensor]:
    """A random checkpoint in the Hugging Face layout (fp32), with mixing coefficients, decays and norms in the ranges
    trained models use; ``init_random_weights`` and the tests build models from it."""
    g = torch.Generator().manual_seed(seed)
    rn = lambda *s, std=0.15: torch.randn(*s, generator=g) * std
    ru = lambda *s, lo=0.0, hi=1.0: lo + (hi - lo) * torch.rand(*s, generator=g)
    C, V, L, N, I = cfg.hidden_size, cfg.vocab_size, cfg.num_layers, cfg.ssm["head_dim"], cfg.intermediate_size
    H = C // N
    rk = cfg.ssm
    sd = {"model.embeddings.weight": rn(V, C, std=0.5), "lm_head.weight": rn(V, C, std=C ** -0.5),
          "model.norm.weight": ru(C, lo=0.8, hi=1.2), "model.norm.bias": rn(C, std=0.1)}
    for l in range(L):
        p = f"model.layers.{l}."
        for n in (["pre_norm"] if l == 0 else []) + ["attn_norm", "ffn_norm"]:
            sd[p + n + ".weight"], sd[p + n + ".bias"] = ru(C, lo=0.8, hi=1.2), rn(C, std=0.1)
        a = p + "attn."
        for c in "rwkvag":
            sd[a + "x_" + c] = ru(1, 1, C)
        for n in ("r_proj", "k_proj", "v_proj", "o_proj"):
            sd[a + n + ".weight"] = rn(C, C, std=C ** -0.5)
        for n, rank in (("w", rk["decay_rank"]), ("a", rk["a_rank"]), ("v", rk["v_rank"]), ("g", rk["gate_rank"])):
            if n == "v" and l == 0:
                continue
            sd[a + f"{n}_lora.lora.0.weight"] = rn(rank, C, std=C ** -0.5)
            sd[a + f"{n}_lora.lora.2.weight"] = rn(C, rank, std=rank ** -0.5)
            if n != "g":
                sd[a + f"{n}_lora.lora.2.bias"] = rn(C, std=0.5)
        sd[a + "k_k"], sd[a + "k_a"], sd[a + "r_k"] = ru(C, lo=0.5, hi=1.0), ru(C, lo=0.8, hi=1.2), rn(H, N, std=0.3)
        sd[a + "g_norm.weight"], sd[a + "g_norm.bias"] = ru(C, lo=0.8, hi=1.2), rn(C, std=0.1)
        sd[p + "ffn.x_k"] = ru(1, 1, C)
        sd[p + "ffn.key.weight"], sd[p + "ffn.value.weight"] = rn(I, C, std=C ** -0.5), rn(C, I, std=I ** -0.5)
    return sd


def weights_from_state_dict(cfg: ModelConfig, sd: Dict[str, torch.Tensor], device, dtype):
    from .weights import DecoderWeights, LayerWeights

    def get(name, required=True):
        if name not in sd:
            if required:
                raise KeyError(f"checkpoint has no tensor {name!r}")
            return None
        return sd[name]
    bf = lambda t: t.to(device=device, dtype=dtype).contiguous()
    layers = []
    for l in range(cfg.num_layers):
        p = f"model.layers.{l}."
        layers.append(LayerWeights(attn_norm=get(p + "attn_norm.weight").float().to(device), wqkv=None, wo=None,
                                   ffn_norm=get(p + "ffn_norm.weight").float().to(device),
                                   mixer=pack_rwkv7_layer(get, p, l, dtype, device)))
    w = DecoderWeights(embed=bf(get("model.embeddings.weight")), layers=layers, final_norm=get("model.norm.weight").float().to(device),
                       lm_head=bf(get("lm_head.weight")), vocab_start=0, vocab_local=cfg.vocab_size)
    w.final_norm_b = get("model.norm.bias").float().to(device)
    return w


# ================================================================================================ RWKV-6
def rwkv6_forward_hidden(dec, b):
    cfg, ops, st = dec.cfg, dec.ops, dec.rstate
    eps, N = cfg.rms_eps, cfg.ssm["head_dim"]
    C = cfg.hidden_size
    H = C // N
    qs, ss, pos = b.q_starts, b.seq_state, b.positions
    x = ops.embed(b.token_ids, dec.w.embed, 1.0)
    T = x.shape[0]
    taps = getattr(dec, "_shift_taps", None)
    if taps is None:
        taps = dec._shift_taps = _shift_taps(C, x.device)
    lin = ops.linear
    gn_eps = 1e-5 * cfg.ssm.get("head_size_divisor", 8) ** 2
    for li, lw in zip(dec.layer_range, dec.w.layers):
        m = lw.mixer
        if "pre_norm_w" in m:
            x = _ln(x, m["pre_norm_w"], m["pre_norm_b"], eps)
        h = _ln(x, lw.attn_norm, m["attn_norm_b"], eps)
        xx = ops.causal_conv1d(h, taps, None, st.conv[li], qs, ss, pos, act=False, max_q_len=getattr(b, "max_q_len", 0))
        lo = torch.tanh(lin(h + xx * m["maa_x"], m["maa_w1"]).float()).to(h.dtype)              # [T, 5 d]
        d = lo.shape[1] // 5
        xw, xk, xv, xr, xg = (h + xx * (m["maa_" + c] + lin(lo[:, j * d:(j + 1) * d].contiguous(), m["maa_w2_" + c]))
                              for j, c in enumerate("wkvrg"))
        r, k, v = lin(xr, m["r_proj"]), lin(xk, m["k_proj"]), lin(xv, m["v_proj"])
        gate = torch.nn.functional.silu(lin(xg, m["g_proj"]).float())
        wraw = m["decay"] + lin(torch.tanh(lin(xw, m["decay_w1"]).float()).to(h.dtype), m["decay_w2"]).float()
        w = (-torch.exp(wraw)).contiguous()                                                         # fp32 log decay
        y = ops.matrix_state_scan(RWKV6, r, k, v, None, None, w, m["bonus"], None, st.scan[li], qs, ss, pos, H, N, N, 1, False, 1.0)
        yf = F.group_norm(y.float(), H, m["g_norm_w"], m["g_norm_b"], gn_eps)
        x = x + lin((yf * gate).to(h.dtype), m["o_proj"])
        h2 = _ln(x, lw.ffn_norm, m["ffn_norm_b"], eps)
        xx2 = ops.causal_conv1d(h2, taps, None, st.shift2[li], qs, ss, pos, act=False, max_q_len=getattr(b, "max_q_len", 0))
        kk = torch.relu(lin(h2 + xx2 * m["ffn_maa_k"], m["ffn_key"]).float()).square().to(h.dtype)
        rr = torch.sigmoid(lin(h2 + xx2 * m["ffn_maa_r"], m["ffn_recept"]).float())
        x = x + (rr * lin(kk, m["ffn_value"]).float()).to(h.dtype)
    return x, None


def pack_rwkv6_layer(get, p: str, dtype, device) -> Dict[str, torch.Tensor]:
    bf = lambda t: t.to(device=device, dtype=dtype).contiguous()
    vec = lambda t: t.reshape(-1).to(device=device, dtype=dtype).contiguous()
    f32 = lambda t: t.float().to(device).contiguous()
    m = {"attn_norm_b": f32(get(p + "ln1.bias")), "ffn_norm_b": f32(get(p + "ln2.bias"))}
    if get(p + "pre_ln.weight", False) is not None:
        m["pre_norm_w"], m["pre_norm_b"] = f32(get(p + "pre_ln.weight")), f32(get(p + "pre_ln.bias"))
    a = p + "attention."
    m["maa_x"] = vec(get(a + "time_maa_x"))
    for c in "wkvrg":
        m["maa_" + c] = vec(get(a + "time_maa_" + c))
    m["maa_w1"] = bf(get(a + "time_maa_w1").t())                       # stored as x @ W: [C, 5 d] -> [5 d, C]
    w2 = get(a + "time_maa_w2")                                        # [5, d, C]
    for j, c in enumerate("wkvrg"):
        m["maa_w2_" + c] = bf(w2[j].t())
    m["decay"] = f32(get(a + "time_decay").reshape(-1))
    m["decay_w1"], m["decay_w2"] = bf(get(a + "time_decay_w1").t()), bf(get(a + "time_decay_w2").t())
    m["bonus"] = f32(get(a + "time_faaaa").reshape(-1))
    for name, key in (("r_proj", "receptance"), ("k_proj", "key"), ("v_proj", "value"), ("g_proj", "gate"), ("o_proj", "output")):
        m[name] = bf(get(a + key + ".weight"))
    m["g_norm_w"], m["g_norm_b"] = f32(get(a + "ln_x.weight")), f32(get(a + "ln_x.bias"))
    f = p + "feed_forward."
    m["ffn_maa_k"], m["ffn_maa_r"] = vec(get(f + "time_maa_k")), vec(get(f + "time_maa_r"))
    m["ffn_key"], m["ffn_recept"], m["ffn_value"] = bf(get(f + "key.weight")), bf(get(f + "receptance.weight")), bf(get(f + "value.weight"))
    return m


def random_rwkv6_state_dict(cfg: ModelConfig, seed: int = 0) -> Dict[str, torch.Tensor]:
    g = torch.Generator().manual_seed(seed)
    rn = lambda *s, std=0.15: torch.randn(*s, generator=g) * std
    ru = lambda *s, lo=0.0, hi=1.0: lo + (hi - lo) * torch.rand(*s, generator=g)
    C, V, L, N, I = cfg.hidden_size, cfg.vocab_size, cfg.num_layers, cfg.ssm["head_dim"], cfg.intermediate_size
    H, d, dd = C // N, cfg.ssm["mix_rank"], cfg.ssm["decay_rank"]
    sd = {"rwkv.embeddings.weight": rn(V, C, std=0.5), "head.weight": rn(V, C, std=C ** -0.5),
          "rwkv.ln_out.weight": ru(C, lo=0.8, hi=1.2), "rwkv.ln_out.bias": rn(C, std=0.1)}
    for l in range(L):
        p = f"rwkv.blocks.{l}."
        for n in (["pre_ln"] if l == 0 else []) + ["ln1", "ln2"]:
            sd[p + n + ".weight"], sd[p + n + ".bias"] = ru(C, lo=0.8, hi=1.2), rn(C, std=0.1)
        a = p + "attention."
        for c in "xwkvrg":
            sd[a + "time_maa_" + c] = ru(1, 1, C)
        sd[a + "time_maa_w1"], sd[a + "time_maa_w2"] = rn(C, 5 * d, std=C ** -0.5), rn(5, d, C, std=d ** -0.5)
        sd[a + "time_decay"] = rn(1, 1, C, std=1.0) - 1.0
        sd[a + "time_decay_w1"], sd[a + "time_decay_w2"] = rn(C, dd, std=C ** -0.5), rn(dd, C, std=dd ** -0.5)
        sd[a + "time_faaaa"] = rn(H, N, std=0.3)
        for n in ("receptance", "key", "value", "gate", "output"):
            sd[a + n + ".weight"] = rn(C, C, std=C ** -0.5)
        sd[a + "ln_x.weight"], sd[a + "ln_x.bias"] = ru(C, lo=0.8, hi=1.2), rn(C, std=0.1)
        f = p + "feed_forward."
        sd[f + "time_maa_k"], sd[f + "time_maa_r"] = ru(1, 1, C), ru(1, 1, C)
        sd[f + "key.weight"], sd[f + "receptance.weight"], sd[f + "value.weight"] = rn(I, C, std=C ** -0.5), rn(C, C, std=C ** -0.5), rn(C, I, std=I ** -0.5)
    return sd


def rwkv6_weights_from_state_dict(cfg: ModelConfig, sd: Dict[str, torch.Tensor], device, dtype):
    from .weights import DecoderWeights, LayerWeights

    def get(name, required=True):
        if name not in sd:
            if required:
                raise KeyError(f"checkpoint has no tensor {name!r}")
            return None
        return sd[name]
    bf = lambda t: t.to(device=device, dtype=dtype).contiguous()
    layers = []
    for l in range(cfg.num_layers):
        p = f"rwkv.blocks.{l}."
        layers.append(LayerWeights(attn_norm=get(p + "ln1.weight").float().to(device), wqkv=None, wo=None,
                                   ffn_norm=get(p + "ln2.weight").float().to(device), mixer=pack_rwkv6_layer(get, p, dtype, device)))
    w = DecoderWeights(embed=bf(get("rwkv.embeddings.weight")), layers=layers, final_norm=get("rwkv.ln_out.weight").float().to(device),
                       lm_head=bf(get("head.weight")), vocab_start=0, vocab_local=cfg.vocab_size)
    w.final_norm_b = get("rwkv.ln_out.bias").float().to(device)
    return w
