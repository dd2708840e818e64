"""Recurrent token mixers of the hybrid families: Mamba-1, Mamba-2, the gated delta rule and the gated short
convolution, as layer kinds of the one decoder runner.

The reference runs these layers from rust/engine/src/rust_decoder/hybrid.rs (layer dispatch), the recurrent halves of
rust/engine/src/rust_decoder.rs and rust/engine/cuda/{mamba1,mamba2,deltanet,shortconv}.cu, with the per-sequence
states kept beside the paged KV pool (rust/engine/src/mem/state_cache.rs). Here a layer's state is one row of a pool
per layer (``RecurrentState``); the engine gives every running sequence a row, and a sequence whose step starts at
position 0 starts from zeros, which covers fresh prompts, chunked prefill (later chunks continue the row) and
recomputation after preemption alike.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch
import torch.nn.functional as F

from ..config import ModelConfig
from ..ops.recurrent import GATED_DELTA

RECURRENT_KINDS = ("mamba1", "mamba2", "gated_delta", "shortconv")


def pad8(n: int) -> int:
    return (n + 7) // 8 * 8


def _state_kind(kind: str) -> str:
    return "mamba2" if kind == "attention+mamba2" else kind


def conv_channels(cfg: ModelConfig, kind: str) -> int:
    s = cfg.ssm
    if kind == "mamba1":
        return s["d_inner"]
    if kind == "mamba2":
        return s["d_inner"] + 2 * s["n_groups"] * s["d_state"]
    if kind == "gated_delta":
        return 2 * s["num_k_heads"] * s["head_k_dim"] + s["num_v_heads"] * s["head_v_dim"]
    if kind in ("shortconv", "rwkv7", "rwkv6"):
        return cfg.hidden_size
    raise ValueError(kind)


def scan_state_shape(cfg: ModelConfig, kind: str):
    s = cfg.ssm
    if kind == "mamba1":
        return (s["d_inner"], s["d_state"])
    if kind == "mamba2":
        return (s["n_heads"], s["head_dim"], s["d_state"])
    if kind == "gated_delta":
        return (s["num_v_heads"], s["head_v_dim"], s["head_k_dim"])
    if kind in ("rwkv7", "rwkv6"):
        return (cfg.hidden_size // s["head_dim"], s["head_dim"], s["head_dim"])
    return None


class RecurrentState:
    """State pools of this stage's recurrent layers: per layer a convolution window [slots, W - 1, C] in the activation type (bf16 on a GPU) and (except
    for the short convolution) an fp32 scan state [slots, ...]. The last row is the scratch row of padding sequences."""

    def __init__(self, cfg: ModelConfig, layer_range: range, slots: int, device, act_dtype=torch.bfloat16):
        self.slots = slots
        self.conv: Dict[int, torch.Tensor] = {}
        self.scan: Dict[int, torch.Tensor] = {}
        self.shift2: Dict[int, torch.Tensor] = {}          # RWKV: the channel mix has a token shift of its own
        W = cfg.ssm.get("d_conv", 4)
        for li in layer_range:
            kind = _state_kind(cfg.layer_kind(li))
            if kind in ("attention", "mla", "none"):
                continue
            if kind in ("rwkv7", "rwkv6"):
                self.shift2[li] = torch.zeros(slots, W - 1, cfg.hidden_size, dtype=act_dtype, device=device)
            self.conv[li] = torch.zeros(slots, W - 1, conv_channels(cfg, kind), dtype=act_dtype, device=device)
            shape = scan_state_shape(cfg, kind)
            if shape is not None:
                self.scan[li] = torch.zeros(slots, *shape, dtype=torch.float32, device=device)

    @staticmethod
    def bytes_per_slot(cfg: ModelConfig, layer_range: range) -> int:
        n = 0
        W = cfg.ssm.get("d_conv", 4)
        for li in layer_range:
            kind = _state_kind(cfg.layer_kind(li))
            if kind in ("attention", "mla", "none"):
                continue
            n += (W - 1) * conv_channels(cfg, kind) * (4 if kind in ("rwkv7", "rwkv6") else 2)
            shape = scan_state_shape(cfg, kind)
            if shape is not None:
                k = 4
                for d in shape:
                    k *= d
                n += k
        return n

    def nbytes(self) -> int:
        return sum(t.numel() * t.element_size() for d in (self.conv, self.scan, self.shift2) for t in d.values())


def _batch_meta(b):
    if b.q_starts is None or getattr(b, "seq_state", None) is None:
        raise RuntimeError("a recurrent layer needs q_starts and seq_state in the step batch")
    return b.q_starts, b.seq_state, b.positions


def _rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    xf = x.float()
    return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)).to(x.dtype)


def mamba1_mixer(dec, li: int, lw, h: torch.Tensor, b) -> torch.Tensor:
    """in_proj -> (x, z); x = silu(conv(x)); (B, C, dt) = x_proj(x); dt = dt_proj(dt); selective scan gated by
    silu(z); out_proj. The loader stores x_proj's rows as [B | C | dt] with dt padded to 8 columns, so that every
    slice of its output starts on a 16-byte boundary."""
    s, m, ops = dec.cfg.ssm, lw.mixer, dec.ops
    qs, ss, pos = _batch_meta(b)
    Di, N = s["d_inner"], s["d_state"]
    xz = ops.linear(h, m["in_proj"], m.get("in_proj_b"))
    x = ops.causal_conv1d(xz[:, :Di], m["conv_w"], m.get("conv_b"), dec.rstate.conv[li], qs, ss, pos, act=True, max_q_len=getattr(b, "max_q_len", 0))
    bcd = ops.linear(x, m["x_proj"])
    Bm, Cm, dtl = bcd[:, :N], bcd[:, N:2 * N], bcd[:, 2 * N:]
    if s.get("bcdt_rms"):
        eps = s.get("mixer_rms_eps", 1e-6)
        R = s["dt_rank"]
        dtn, Bm, Cm = _rms(dtl[:, :R], eps), _rms(Bm, eps), _rms(Cm, eps)
        if "dt_norm_w" in m:                           # Jamba: the three norms carry weights
            dtn, Bm, Cm = dtn * m["dt_norm_w"], Bm * m["b_norm_w"], Cm * m["c_norm_w"]
        dtl = torch.nn.functional.pad(dtn, (0, dtl.shape[1] - R))
    dt = ops.linear(dtl, m["dt_proj"])
    y = ops.mamba1_scan(x, dt, Bm, Cm, xz[:, Di:2 * Di], m["A"], m["D"], m["dt_bias"], dec.rstate.scan[li], qs, ss, pos,
                        getattr(b, "max_q_len", 0))
    return ops.linear(y, m["out_proj"], m.get("out_proj_b"))


def mamba2_mixer(dec, li: int, lw, h: torch.Tensor, b) -> torch.Tensor:
    """in_proj -> (z, xBC, dt); xBC = silu(conv(xBC)) -> (x, B, C); SSD scan; rmsnorm(y * silu(z)); out_proj."""
    s, m, ops = dec.cfg.ssm, lw.mixer, dec.ops
    qs, ss, pos = _batch_meta(b)
    Di, N, G, H, P = s["d_inner"], s["d_state"], s["n_groups"], s["n_heads"], s["head_dim"]
    C = Di + 2 * G * N
    zxd = ops.linear(h, m["in_proj"], m.get("in_proj_b"))
    xbc = ops.causal_conv1d(zxd[:, Di:Di + C], m["conv_w"], m.get("conv_b"), dec.rstate.conv[li], qs, ss, pos, act=True, max_q_len=getattr(b, "max_q_len", 0))
    y = ops.mamba2_scan(xbc[:, :Di], zxd[:, Di + C:Di + C + H], xbc[:, Di:Di + G * N], xbc[:, Di + G * N:], m["A"], m["D"],
                        m["dt_bias"], dec.rstate.scan[li], qs, ss, pos, H, P, G, N, s.get("dt_min", 0.0),
                        s.get("dt_max", 1e30), getattr(b, "max_q_len", 0), None, getattr(b, "host_seqs", None))
    mode = s.get("gate_mode", "norm_after_gate")
    if mode == "gate_only":                       # Falcon-H1 without the mixer norm: y * silu(z)
        y = y * F.silu(zxd[:, :Di])
    else:
        y = ops.gated_rmsnorm(y, zxd[:, :Di], m["norm_w"], s.get("norm_eps", dec.cfg.rms_eps), Di // s.get("norm_groups", 1),
                              mode == "norm_before_gate")
    return ops.linear(y, m["out_proj"], m.get("out_proj_b"))


def gated_delta_mixer(dec, li: int, lw, h: torch.Tensor, b) -> torch.Tensor:
    """in_proj -> (q, k, v | z | beta, a); (q, k, v) = silu(conv(q, k, v)); log decay = -exp(A_log) softplus(a + dt_bias)
    and step size = sigmoid(beta), both computed inside the scan;
    delta rule with L2-normalised q, k; per-head rmsnorm(y) * w * silu(z); out_proj."""
    s, m, ops = dec.cfg.ssm, lw.mixer, dec.ops
    qs, ss, pos = _batch_meta(b)
    Hk, Hv, Dk, Dv = s["num_k_heads"], s["num_v_heads"], s["head_k_dim"], s["head_v_dim"]
    K, V = Hk * Dk, Hv * Dv
    proj = ops.linear(h, m["in_proj"])                                  # [q | k | v | z | beta | a] (+ padding)
    qkv = ops.causal_conv1d(proj[:, :2 * K + V], m["conv_w"], m.get("conv_b"), dec.rstate.conv[li], qs, ss, pos, act=True, max_q_len=getattr(b, "max_q_len", 0))
    z = proj[:, 2 * K + V:2 * K + 2 * V]
    o = 2 * K + 2 * V                                                   # the step-size and decay logits go to the scan raw
    y = ops.matrix_state_scan(GATED_DELTA, qkv[:, :K], qkv[:, K:2 * K], qkv[:, 2 * K:], None, None, None, None, proj[:, o:o + Hv],
                              dec.rstate.scan[li], qs, ss, pos, Hv, Dk, Dv, Hv // Hk, True, Dk ** -0.5,
                              gate_raw=proj[:, o + Hv:o + 2 * Hv], gate_A=m["A"], gate_dt_bias=m["dt_bias"])
    y = ops.gated_rmsnorm(y, z, m["norm_w"], s.get("norm_eps", dec.cfg.rms_eps), Dv, True)
    return ops.linear(y, m["out_proj"])


def shortconv_mixer(dec, li: int, lw, h: torch.Tensor, b) -> torch.Tensor:
    """in_proj -> (B, C, x); y = C * conv(B * x); out_proj (the LFM2 operator)."""
    m, ops = lw.mixer, dec.ops
    qs, ss, pos = _batch_meta(b)
    Hd = dec.cfg.hidden_size
    bcx = ops.linear(h, m["in_proj"], m.get("in_proj_b"))
    bx = bcx[:, :Hd] * bcx[:, 2 * Hd:3 * Hd]
    y = ops.causal_conv1d(bx, m["conv_w"], m.get("conv_b"), dec.rstate.conv[li], qs, ss, pos, act=False, max_q_len=getattr(b, "max_q_len", 0))
    return ops.linear(bcx[:, Hd:2 * Hd] * y, m["out_proj"], m.get("out_proj_b"))


MIXERS = {"mamba1": mamba1_mixer, "mamba2": mamba2_mixer, "gated_delta": gated_delta_mixer, "shortconv": shortconv_mixer}


# ------------------------------------------------------------------------------------------------ weights
def pad_rows(w: torch.Tensor, n: int) -> torch.Tensor:
    if w.shape[0] == n:
        return w.contiguous()
    out = torch.zeros(n, *w.shape[1:], dtype=w.dtype, device=w.device)
    out[:w.shape[0]] = w
    return out


def pad_cols(w: torch.Tensor, n: int) -> torch.Tensor:
    if w.shape[1] == n:
        return w.contiguous()
    out = torch.zeros(w.shape[0], n, dtype=w.dtype, device=w.device)
    out[:, :w.shape[1]] = w
    return out


def pack_mamba1(in_proj, conv_w, conv_b, x_proj, dt_proj, dt_bias, A_log, D, out_proj, N: int, R: int, dtype, device,
                in_proj_b=None, out_proj_b=None) -> Dict[str, torch.Tensor]:
    """Mixer tensors in checkpoint layout (x_proj rows [dt | B | C]) -> the runner's layout."""
    Rp = pad8(R)
    xp = torch.cat([x_proj[R:R + 2 * N], pad_rows(x_proj[:R], Rp)], 0)
    f32 = lambda t: t.float().to(device).contiguous()
    bf = lambda t: t.to(device=device, dtype=dtype).contiguous()
    m = dict(in_proj=bf(in_proj), conv_w=f32(conv_w.reshape(conv_w.shape[0], -1)), x_proj=bf(xp),
             dt_proj=bf(pad_cols(dt_proj, Rp)), dt_bias=f32(dt_bias), A=f32(-torch.exp(A_log.float())), D=f32(D),
             out_proj=bf(out_proj))
    if conv_b is not None:
        m["conv_b"] = f32(conv_b)
    if in_proj_b is not None:
        m["in_proj_b"] = bf(in_proj_b)
    if out_proj_b is not None:
        m["out_proj_b"] = bf(out_proj_b)
    return m


def pack_mamba2(in_proj, conv_w, conv_b, dt_bias, A_log, D, norm_w, out_proj, dtype, device, in_proj_b=None,
                out_proj_b=None) -> Dict[str, torch.Tensor]:
    f32 = lambda t: t.float().to(device).contiguous()
    bf = lambda t: t.to(device=device, dtype=dtype).contiguous()
    m = dict(in_proj=bf(pad_rows(in_proj, pad8(in_proj.shape[0]))), conv_w=f32(conv_w.reshape(conv_w.shape[0], -1)),
             dt_bias=f32(dt_bias), A=f32(-torch.exp(A_log.float())), D=f32(D), norm_w=bf(norm_w), out_proj=bf(out_proj))
    if conv_b is not None:
        m["conv_b"] = f32(conv_b)
    if in_proj_b is not None:
        m["in_proj_b"] = bf(pad_rows(in_proj_b, pad8(in_proj.shape[0])))
    if out_proj_b is not None:
        m["out_proj_b"] = bf(out_proj_b)
    return m


def pack_gated_delta(q, k, v, z, b, a, conv_w, dt_bias, A_log, norm_w, out_proj, dtype, device) -> Dict[str, torch.Tensor]:
    """Projection rows already separated by role ([Hk*Dk], [Hk*Dk], [Hv*Dv], [Hv*Dv], [Hv], [Hv]) -> one in_proj."""
    f32 = lambda t: t.float().to(device).contiguous()
    bf = lambda t: t.to(device=device, dtype=dtype).contiguous()
    fused = torch.cat([q, k, v, z, b, a], 0)
    return dict(in_proj=bf(pad_rows(fused, pad8(fused.shape[0]))), conv_w=f32(conv_w.reshape(conv_w.shape[0], -1)),
                dt_bias=f32(dt_bias), A=f32(-torch.exp(A_log.float())), norm_w=bf(norm_w), out_proj=bf(out_proj))


def init_random_mixer(cfg: ModelConfig, kind: str, full, li: int, dtype, device) -> Dict[str, torch.Tensor]:
    """Random mixer weights in the ranges trained checkpoints use (decays in (0, 1), positive steps); ``full(shape,
    *key, std=)`` draws a seeded normal tensor."""
    s, H = cfg.ssm, cfg.hidden_size
    W = s.get("d_conv", 4)
    if kind == "mamba1":
        Di, N, R = s["d_inner"], s["d_state"], s["dt_rank"]
        A_log = torch.log(torch.arange(1, N + 1, dtype=torch.float32, device=device)).repeat(Di, 1)
        return pack_mamba1(full((2 * Di, H), li, 30), full((Di, W), li, 31, std=0.3), full((Di,), li, 32, std=0.1),
                           full((R + 2 * N, Di), li, 33, std=0.05), full((Di, R), li, 34, std=R ** -0.5),
                           full((Di,), li, 35, std=0.5).float() - 3.0, A_log, torch.ones(Di, device=device),
                           full((H, Di), li, 36), N, R, dtype, device)
    if kind == "mamba2":
        Di, N, G, Hn = s["d_inner"], s["d_state"], s["n_groups"], s["n_heads"]
        A_log = torch.log(torch.linspace(1.0, 16.0, Hn, device=device))
        return pack_mamba2(full((2 * Di + 2 * G * N + Hn, H), li, 30), full((Di + 2 * G * N, W), li, 31, std=0.3),
                           full((Di + 2 * G * N,), li, 32, std=0.1), full((Hn,), li, 35, std=0.5).float() - 3.0, A_log,
                           torch.ones(Hn, device=device), torch.ones(Di, device=device), full((H, Di), li, 36), dtype, device)
    if kind == "gated_delta":
        Hk, Hv, Dk, Dv = s["num_k_heads"], s["num_v_heads"], s["head_k_dim"], s["head_v_dim"]
        K, V = Hk * Dk, Hv * Dv
        return pack_gated_delta(full((K, H), li, 30), full((K, H), li, 31), full((V, H), li, 32), full((V, H), li, 33),
                                full((Hv, H), li, 34), full((Hv, H), li, 35), full((2 * K + V, W), li, 36, std=0.3),
                                torch.ones(Hv, device=device), torch.log(torch.linspace(1.0, 16.0, Hv, device=device)),
                                torch.ones(Dv, device=device), full((H, V), li, 37), dtype, device)
    if kind == "shortconv":
        m = dict(in_proj=full((3 * H, H), li, 30), conv_w=full((H, W), li, 31, std=0.3).float(), out_proj=full((H, H), li, 32))
        if s.get("conv_bias"):
            m["conv_b"] = full((H,), li, 33, std=0.1).float()
        return m
    raise ValueError(f"unknown recurrent layer kind {kind!r}")
