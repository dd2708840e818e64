"""Roofline planner over TP x PP x EP layouts (``plan-cluster``).

Same idea as the reference's estimator (rust/engine/src/parallel/cluster_plan.rs:53-67 GPU
presets incl. b200, :523-660 the estimate, :506-521 what is runnable): per decode step the time
of a layout is max(weight + KV bytes / HBM bandwidth, FLOPs / tensor peak) per stage, plus the
collectives (bytes over the link + a fixed latency each), plus pipeline bubbles. It ranks
layouts; it does not replace a measurement.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List

from ..config import ModelConfig


@dataclass
class GpuPreset:
    name: str
    mem_gib: float
    hbm_gbs: float
    link_gbs: float          # per direction per GPU
    bf16_tflops: float
    collective_us: float     # fixed cost of one small collective


GPU_PRESETS: Dict[str, GpuPreset] = {
    # measured on this pool where available (copy bandwidth, cuBLAS bf16, peer copy); datasheet otherwise
    "b200": GpuPreset("b200", 179.0, 6450.0, 770.0, 1400.0, 8.0),
    "h100": GpuPreset("h100", 79.0, 3000.0, 400.0, 750.0, 10.0),
    "a100": GpuPreset("a100", 79.0, 1800.0, 250.0, 280.0, 12.0),
}


def _divisors(n: int) -> List[int]:
    return [d for d in range(1, n + 1) if n % d == 0]


def runnable(cfg: ModelConfig, tp: int, pp: int, ep: bool) -> "tuple[bool, str]":
    if cfg.num_heads % tp:
        return False, "query heads not divisible by tp"
    if cfg.num_kv_heads >= tp and cfg.num_kv_heads % tp:
        return False, "kv heads not divisible by tp"
    if cfg.num_kv_heads < tp and tp % cfg.num_kv_heads:
        return False, "tp not a multiple of kv heads"
    if pp > cfg.num_layers:
        return False, "more stages than layers"
    if ep and not cfg.is_moe:
        return False, "expert parallelism needs a mixture-of-experts model"
    inter = cfg.moe_intermediate_size if cfg.is_moe else cfg.intermediate_size
    if not ep and inter % (tp * 8):
        return False, "ffn width not divisible by tp * 8"
    return True, ""


def estimate(cfg: ModelConfig, gpu: GpuPreset, tp: int, pp: int, ep: bool, batch: int, ctx: int,
             weight_bits: float = 16, kv_bits: float = 16) -> dict:
    H, L = cfg.hidden_size, cfg.num_layers
    attn_w = H * (cfg.q_size + 2 * cfg.kv_size) + cfg.q_size * H
    if cfg.is_moe:
        I, E, k = cfg.moe_intermediate_size, cfg.num_experts, cfg.experts_per_token
        ffn_total = E * 3 * H * I
        touched = min(E, batch * k)                      # experts that see at least one token
        ffn_read = touched * 3 * H * I
        ffn_flops_tok = k * 3 * H * I * 2
    else:
        ffn_total = ffn_read = 3 * H * cfg.intermediate_size
        ffn_flops_tok = ffn_total * 2
    head = cfg.vocab_size * H
    wbytes = weight_bits / 8
    per_layer_read = (attn_w + ffn_read) / tp * wbytes
    kv_per_layer = batch * ctx * 2 * max(cfg.kv_size // tp, cfg.head_dim) * kv_bits / 8
    layers_stage = -(-L // pp)
    mem_gib = ((attn_w + ffn_total) / tp * wbytes * layers_stage + head / tp * wbytes * 2
               + kv_per_layer * layers_stage) / 2 ** 30
    t_mem = (per_layer_read + kv_per_layer) / (gpu.hbm_gbs * 1e9)
    flops = batch * ((attn_w * 2 + ffn_flops_tok) / tp + 4 * ctx * cfg.q_size / tp)
    t_mma = flops / (gpu.bf16_tflops * 1e12)
    t_layer = max(t_mem, t_mma)
    # two reduce-scatter + all-gather pairs per layer (or all-to-all pairs for experts)
    msg = batch * H * 2
    t_coll = 0.0
    if tp > 1:
        per = 2 * (msg * (tp - 1) / tp / (gpu.link_gbs * 1e9) * 2 + gpu.collective_us * 1e-6)
        if ep:
            per = per / 2 + (2 * batch * cfg.experts_per_token * H * 2 / (gpu.link_gbs * 1e9) + 2 * gpu.collective_us * 1e-6)
        t_coll = per
    t_stage = layers_stage * (t_layer + t_coll)
    t_head = max(head / tp * wbytes / (gpu.hbm_gbs * 1e9), batch * head * 2 / tp / (gpu.bf16_tflops * 1e12))
    hop = (msg / (gpu.link_gbs * 1e9) + gpu.collective_us * 1e-6) if pp > 1 else 0.0
    step = t_stage * pp + t_head + hop * (pp - 1)      # one micro-batch: stages run one after another
    return {"tp": tp, "pp": pp, "ep": ep, "gpus": tp * pp, "ms_per_step": round(step * 1e3, 3),
            "tok_s": round(batch / step, 1), "mem_gib_per_gpu": round(mem_gib, 1), "fits": mem_gib < gpu.mem_gib * 0.92,
            "bound": "memory" if t_mem >= t_mma else "tensor", "collective_share": round(t_coll / (t_layer + t_coll), 3)}


def plan_cluster(cfg: ModelConfig, gpus: int, gpu: GpuPreset, batch: int = 64, ctx: int = 2048,
                 weight_bits: float = 16) -> List[dict]:
    out = []
    for tp in _divisors(gpus):
        if tp > 8:
            continue
        pp = gpus // tp
        for ep in ([False, True] if cfg.is_moe and tp > 1 else [False]):
            ok, why = runnable(cfg, tp, pp, ep)
            if not ok:
                continue
            out.append(estimate(cfg, gpu, tp, pp, ep, batch, ctx, weight_bits))
    out.sort(key=lambda p: (not p["fits"], p["ms_per_step"]))
    return out
