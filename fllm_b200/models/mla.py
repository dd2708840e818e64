"""Multi-head latent attention (DeepSeek-V2 / V3 family) as a layer kind of the decoder runner.

A token is cached as one row: the normalised KV latent (``kv_lora_rank`` values) followed by the rotated shared key
part (``qk_rope_head_dim`` values). The key up-projection is absorbed into the query and the value up-projection
is applied after the softmax, so attention itself is multi-query over those rows for prefill and decode alike
(the reference keeps an expanded prefill path in rust/engine/cuda/mla.cu next to the latent one in
rust/engine/cuda/mla_latent.cu / mla_decode.cu and rust/engine/src/rust_decoder/mla_latent.rs; here the latent form
is the only one).
"""
from __future__ import annotations

from typing import Dict

import torch

from ..config import ModelConfig


class MlaCache:
    """Paged latent pool [layers, blocks, block_size, width]."""

    def __init__(self, num_layers: int, num_blocks: int, block_size: int, width: int, device, dtype=torch.bfloat16):
        self.num_blocks, self.block_size, self.width = num_blocks, block_size, width
        self.store = torch.zeros(num_layers, num_blocks, block_size, width, device=device, dtype=dtype)

    def layer(self, i: int) -> torch.Tensor:
        return self.store[i]

    @staticmethod
    def bytes_per_block(num_layers: int, block_size: int, width: int, elem: int = 2) -> int:
        return num_layers * block_size * width * elem


def mla_block(dec, li: int, lw, h: torch.Tensor, b) -> torch.Tensor:
    cfg, m, ops = dec.cfg, lw.mixer, dec.ops
    c = cfg.mla
    H, dn, dr, dv, R = cfg.num_heads, c["qk_nope_head_dim"], c["qk_rope_head_dim"], c["v_head_dim"], c["kv_lora_rank"]
    T = h.shape[0]
    if "q_a" in m:
        q = ops.linear(ops.rmsnorm(ops.linear(h, m["q_a"]), None, m["q_a_norm"], cfg.rms_eps), m["q_b"])
    else:
        q = ops.linear(h, m["q_proj"])
    q = q.view(T, H, dn + dr)
    ckv = ops.linear(h, m["kv_a"])                                     # [T, pad8(R + dr)]
    cache = dec.kv.layer(dec.kv_index[li])
    q_pe = ops.mla_prepare(ckv, q, dn, b.positions, b.slots, dec.inv_freq, dec.attn_factor, m["kv_a_norm"], cfg.rms_eps, cache)
    q_abs = torch.bmm(q[:, :, :dn].transpose(0, 1), m["w_uk"])                                # [H, T, R]
    o_lat = ops.attention_mla(q_abs, q_pe, cache, b.block_tables, b.row_seq, b.positions, dec.scale, b.max_kv_len)     # [H, T, R]
    o = torch.bmm(o_lat, m["w_uv"]).transpose(0, 1).reshape(T, H * dv)
    return ops.linear(o, m["wo"], m.get("bo"))


def pack_mla(q_a, q_a_norm, q_b, q_proj, kv_a, kv_a_norm, kv_b, o_proj, cfg: ModelConfig, dtype, device) -> Dict[str, torch.Tensor]:
    """Checkpoint tensors -> the runner's layout: kv_b [H * (dn + dv), R] is cut into the absorbed key matrix
    w_uk [H, dn, R] and the value matrix w_uv [H, R, dv]; kv_a is padded to a multiple of 8 rows."""
    c = cfg.mla
    H, dn, dv, R = cfg.num_heads, c["qk_nope_head_dim"], c["v_head_dim"], c["kv_lora_rank"]
    bf = lambda t: t.to(device=device, dtype=dtype).contiguous()
    kvb = kv_b.view(H, dn + dv, R)
    rows = (kv_a.shape[0] + 7) // 8 * 8
    kva = torch.zeros(rows, kv_a.shape[1], dtype=kv_a.dtype)
    kva[:kv_a.shape[0]] = kv_a
    m = dict(kv_a=bf(kva), kv_a_norm=bf(kv_a_norm), w_uk=bf(kvb[:, :dn, :]), w_uv=bf(kvb[:, dn:, :].transpose(1, 2)), wo=bf(o_proj))
    if q_proj is not None:
        m["q_proj"] = bf(q_proj)
    else:
        m.update(q_a=bf(q_a), q_a_norm=bf(q_a_norm), q_b=bf(q_b))
    return m


def init_random_mla(cfg: ModelConfig, full, li: int, dtype, device) -> Dict[str, torch.Tensor]:
    c = cfg.mla
    H, dn, dr, dv, R, Hd = cfg.num_heads, c["qk_nope_head_dim"], c["qk_rope_head_dim"], c["v_head_dim"], c["kv_lora_rank"], cfg.hidden_size
    ql = c.get("q_lora_rank")
    ones = lambda n: torch.ones(n, dtype=dtype)
    cpu = lambda t: t.cpu()
    if ql:
        q = dict(q_a=cpu(full((ql, Hd), li, 40)), q_a_norm=ones(ql), q_b=cpu(full((H * (dn + dr), ql), li, 41)), q_proj=None)
    else:
        q = dict(q_a=None, q_a_norm=None, q_b=None, q_proj=cpu(full((H * (dn + dr), Hd), li, 40)))
    return pack_mla(q["q_a"], q["q_a_norm"], q["q_b"], q["q_proj"], cpu(full((R + dr, Hd), li, 42)), ones(R),
                    cpu(full((H * (dn + dv), R), li, 43)), cpu(full((Hd, H * dv), li, 44)), cfg, dtype, device)
