"""Mixture-of-experts feed-forward: router top-k, expert FFNs, weighted combine.

``moe_reference`` is the fp32 PyTorch oracle. ``moe_ffn`` is what the decoder calls: on a GPU it
runs route -> align -> gather -> grouped tcgen05 GEMM (gate/up) -> GLU -> grouped GEMM (down) ->
combine, all sizes staying on the device. Under tensor parallelism each rank holds either a
column slice of every expert (expert-TP) or a contiguous range of whole experts (expert
parallel, rust/engine/src/parallel/decoder_shard.rs:165-211); in both cases the rank's output is
a partial sum that the caller reduces like a dense FFN output.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn.functional as F


def _act(cfg, gu: torch.Tensor) -> torch.Tensor:
    if cfg.mlp_kind == "plain":                  # experts of two matrices: the activation alone
        return {"gelu": F.gelu, "gelu_tanh": lambda t: F.gelu(t, approximate="tanh"), "relu2": lambda t: F.relu(t).square(),
                "silu": F.silu, "relu": F.relu}[cfg.act](gu)
    if cfg.act == "swiglu_oai":
        g, u = gu[..., 0::2], gu[..., 1::2]
        g = g.clamp(max=cfg.swiglu_limit)
        u = u.clamp(min=-cfg.swiglu_limit, max=cfg.swiglu_limit)
        return g * torch.sigmoid(cfg.swiglu_alpha * g) * (u + 1)
    I = gu.shape[-1] // 2
    g, u = gu[..., :I], gu[..., I:]
    return (F.silu(g) if cfg.act == "swiglu" else F.gelu(g, approximate="tanh")) * u


def route_deepseek(cfg, logits: torch.Tensor, bias: Optional[torch.Tensor]):
    """The DeepSeek routers in plain tensor ops (the selection is [T, E]-sized work). V2: softmax scores, experts
    outside the best groups (by their best expert) masked, top-k, weights = scores. V3: sigmoid scores, selection on
    scores + bias with groups ranked by the sum of their two best, weights = unbiased scores, renormalised. Both scale
    the weights by ``router_scale``."""
    k, E, G = cfg.experts_per_token, cfg.num_experts, max(cfg.router_groups, 1)
    lf = logits.float()
    if cfg.router_kind == "deepseek_v3":
        scores = torch.sigmoid(lf)
        choice = scores + (bias.float() if bias is not None else 0.0)
        group_rank = choice.view(-1, G, E // G).topk(min(2, E // G), dim=-1)[0].sum(-1)
    else:
        scores = torch.softmax(lf, -1)
        choice = scores + bias.float() if bias is not None else scores         # ERNIE 4.5: a selection bias on softmax scores
        group_rank = choice.view(-1, G, E // G).max(-1).values
    if G > 1:
        keep = torch.zeros_like(group_rank).scatter_(1, group_rank.topk(cfg.router_topk_groups, dim=-1)[1], 1.0)
        choice = choice.masked_fill(keep[:, :, None].expand(-1, G, E // G).reshape(-1, E) == 0, 0.0)
    ids = choice.topk(k, dim=-1)[1]
    w = scores.gather(1, ids)
    if cfg.router_norm_topk:
        w = w / (w.sum(-1, keepdim=True) + 1e-20)
    return ids.int(), (w * cfg.router_scale).contiguous()


def route_reference(cfg, logits: torch.Tensor, bias: Optional[torch.Tensor] = None):
    """Top-k ids [T, k] and weights [T, k] (fp32)."""
    if cfg.router_kind in ("deepseek_v2", "deepseek_v3"):
        return route_deepseek(cfg, logits, bias)
    k = cfg.experts_per_token
    lf = logits.float()
    vals, ids = torch.topk(lf, k, dim=-1)
    if cfg.router_kind == "softmax_topk":
        w = torch.softmax(vals, -1)
    else:
        p = torch.softmax(lf, -1).gather(-1, ids)
        w = p / p.sum(-1, keepdim=True)
    return ids.int(), w


def moe_reference(cfg, lw, h: torch.Tensor, expert_lo: int = 0, round_bf16: bool = True,
                  xe: Optional[torch.Tensor] = None) -> torch.Tensor:
    """fp32 math on the experts stored in `lw` (global ids expert_lo .. expert_lo + E_local). ``xe``: the rows the
    experts read when they are not the rows the router reads (a latent projection)."""
    r = (lambda t: t.to(torch.bfloat16).float()) if round_bf16 else (lambda t: t)
    hf = h.float()
    logits = hf @ lw.router_w.float().t()
    if xe is not None:
        hf = xe.float()
    select_bias = getattr(lw, "router_select_b", None)
    if lw.router_b is not None:
        logits = logits + lw.router_b.float()
    ids, w = route_reference(cfg, r(logits), select_bias)
    out = torch.zeros(h.shape[0], lw.exp_down.shape[1], dtype=torch.float32, device=h.device)
    e_local = lw.exp_gate_up.shape[0]
    for e in range(e_local):
        sel = (ids == e + expert_lo)
        tok = sel.any(-1).nonzero().flatten()
        if tok.numel() == 0:
            continue
        gu = hf[tok] @ lw.exp_gate_up[e].float().t()
        if lw.exp_gate_up_b is not None:
            gu = gu + lw.exp_gate_up_b[e].float()
        a = r(_act(cfg, r(gu)))
        y = a @ lw.exp_down[e].float().t()
        if lw.exp_down_b is not None:
            y = y + lw.exp_down_b[e].float()
        wt = (w * sel.float()).sum(-1)[tok]
        out[tok] += r(y) * wt[:, None]
    return out


def _token_tile(rows_per_expert: float) -> int:
    for bn in (16, 32, 64):
        if rows_per_expert <= bn:
            return bn
    return 128


def _dense_experts(lw):
    """LayerWeights view with packed expert stacks expanded (oracle / CPU path)."""
    if isinstance(lw.exp_gate_up, torch.Tensor) and isinstance(lw.exp_down, torch.Tensor):
        return lw
    import copy
    d = copy.copy(lw)
    if not isinstance(lw.exp_gate_up, torch.Tensor):
        d.exp_gate_up = lw.exp_gate_up.dense().to(torch.bfloat16)
    if not isinstance(lw.exp_down, torch.Tensor):
        d.exp_down = lw.exp_down.dense().to(torch.bfloat16)
    return d


def _grouped(k_ops, ops, x, w, bias, y, tile_e, tile_r, ntiles, bn):
    """Grouped expert GEMM on a bf16 stack or on a packed 4-bit stack."""
    if isinstance(w, torch.Tensor):
        k_ops.moe_grouped_linear(x, w, bias, y, tile_e, tile_r, ntiles, bn, ops.status)
    else:
        k_ops.moe_grouped_linear_w4(x, w.codes, w.scales, w.fmt, w.alpha, bias, y, tile_e, tile_r, ntiles, bn, ops.status)


def _router_logits(ops, lw, h: torch.Tensor) -> torch.Tensor:
    """Router scores [T, E] (a view when the GEMM needs the expert count padded to a multiple of 8, e.g. 60 experts)."""
    E = lw.router_w.shape[0]
    if E % 8 == 0:
        return ops.linear(h, lw.router_w, lw.router_b)
    pad = getattr(lw, "_router_pad", None)
    if pad is None:
        Ep = (E + 7) // 8 * 8
        wp = torch.zeros(Ep, lw.router_w.shape[1], dtype=lw.router_w.dtype, device=lw.router_w.device)
        wp[:E] = lw.router_w
        bp = None
        if lw.router_b is not None:
            bp = torch.zeros(Ep, dtype=lw.router_b.dtype, device=lw.router_b.device)
            bp[:E] = lw.router_b
        pad = lw._router_pad = (wp, bp)
    return ops.linear(h, pad[0], pad[1])[:, :E]


def moe_ffn(dec, lw, h: torch.Tensor, xe: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``h``: the rows the router reads; ``xe``: the rows the experts read and write when they differ (None: ``h``)."""
    cfg, ops, sp = dec.cfg, dec.ops, dec.spec
    lo = sp.expert_start if sp.expert_parallel else 0
    if not hasattr(ops, "k") or not h.is_cuda:
        return moe_reference(cfg, _dense_experts(lw), h, lo, h.dtype != torch.float32, xe).to(h.dtype)
    k_ops = ops.k
    T, H = (h if xe is None else xe).shape
    k = cfg.experts_per_token
    e_local = lw.exp_gate_up.shape[0]
    logits = _router_logits(ops, lw, h)
    ids = torch.empty(T, k, dtype=torch.int32, device=h.device)
    wts = torch.empty(T, k, dtype=torch.float32, device=h.device)
    if cfg.router_kind in ("deepseek_v2", "deepseek_v3"):
        if cfg.router_groups <= 1 and cfg.num_experts <= 256 and k <= 8:        # one kernel; grouped selection stays in tensor ops
            k_ops.moe_route_scored(logits, getattr(lw, "router_select_b", None), k, 2 if cfg.router_kind == "deepseek_v3" else 1,
                                   bool(cfg.router_norm_topk), float(cfg.router_scale), ids, wts)
        else:
            ids, wts = route_deepseek(cfg, logits, getattr(lw, "router_select_b", None))
    elif cfg.num_experts > 256 or k > 8:         # beyond the routing kernel's register budget: the same rule in tensor ops
        ids, wts = route_reference(cfg, logits)
        wts = wts.contiguous()
    else:
        k_ops.moe_route(logits, None, k, cfg.router_kind != "softmax_topk", ids, wts)
    share = e_local / cfg.num_experts
    bn = _token_tile(T * k * share / max(e_local, 1))
    rows_cap = -(-(T * k + e_local * (bn - 1)) // bn) * bn
    max_tiles = rows_cap // bn
    i32 = dict(dtype=torch.int32, device=h.device)
    row_of = torch.empty(T, k, **i32)
    token_of = torch.empty(rows_cap, **i32)
    tile_e, tile_r = torch.empty(max_tiles, **i32), torch.empty(max_tiles, **i32)
    ntiles = torch.zeros(2, **i32)
    k_ops.moe_align(ids, cfg.num_experts, lo, lo + e_local, bn, row_of, token_of, tile_e, tile_r, ntiles)
    xp = torch.empty(rows_cap, H, dtype=h.dtype, device=h.device)
    k_ops.moe_gather(h if xe is None else xe, token_of, xp)
    gu = torch.empty(rows_cap, lw.exp_gate_up.shape[1], dtype=h.dtype, device=h.device)
    _grouped(k_ops, ops, xp, lw.exp_gate_up, lw.exp_gate_up_b, gu, tile_e, tile_r, ntiles, bn)
    act = ops.act_(gu, cfg.act) if cfg.mlp_kind == "plain" else ops.glu(gu, dec.act_kind, cfg.swiglu_alpha, cfg.swiglu_limit)
    y = torch.empty(rows_cap, H, dtype=h.dtype, device=h.device)
    _grouped(k_ops, ops, act, lw.exp_down, lw.exp_down_b, y, tile_e, tile_r, ntiles, bn)
    out = torch.empty(T, H, dtype=h.dtype, device=h.device)
    k_ops.moe_combine(y, row_of, wts, out)
    ops.launches += 6
    return out


def moe_ffn_alltoall(dec, lw, h: torch.Tensor) -> torch.Tensor:
    """Expert parallelism with all-to-all dispatch. Activations are replicated across the group, so
    each rank treats an equal slice of the rows as its own, sends those rows to the ranks that hold
    their experts, receives the expert outputs back, forms the weighted sum for its rows and
    all-gathers the result. Every (token, expert) pair is computed once in the whole group and only
    routed rows cross NVLink (rust/engine/src/parallel/decoder_shard.rs:442-508)."""
    from ..comm.ep_a2a import moe_ffn_a2a_phases
    ep, tp = dec.ep_a2a, dec.tp
    T, H = h.shape
    per = -(-T // ep.ranks)
    own = torch.zeros(per, H, dtype=h.dtype, device=h.device)          # rows past T stay zero (padding)
    lo = min(ep.rank * per, T)
    n = max(min(lo + per, T) - lo, 0)
    if n:
        own[:n] = h[lo:lo + n]
    out = None
    for out in moe_ffn_a2a_phases(dec, lw, ep, own):
        pass
    return tp.all_gather(out.contiguous()).reshape(ep.ranks * per, H)[:T]
