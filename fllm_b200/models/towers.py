"""Pre-LayerNorm encoder towers of multimodal models: the SigLIP vision transformer (patches of an image) and the
Whisper audio encoder (two 1-D convolutions over a log-mel spectrogram). Both end in the hidden states a language
model's projector consumes; the projector and the placement of these states among text tokens are not part of this
module.

The reference keeps these towers in rust/engine/src/vision/** (SigLIP, Qwen-VL towers) and its Whisper encoder beside
them. The blocks share one runner: projections through ``ops.linear`` (bias in the GEMM epilogue), bidirectional
attention through the decoder's prefill kernels over a scratch paged pool (head widths the kernels do not have, such
as SigLIP-so400m's 72, go through PyTorch's attention), LayerNorm / GELU / the input stems in PyTorch.
"""
from __future__ import annotations

import json
import math
import os
from dataclasses import dataclass
from typing import List, Optional

import torch
import torch.nn.functional as F

from .decoder import StepBatch


@dataclass
class TowerConfig:
    kind: str = "siglip"               # siglip | whisper
    hidden_size: int = 768
    num_layers: int = 12
    num_heads: int = 12
    intermediate_size: int = 3072
    layer_norm_eps: float = 1e-6
    act: str = "gelu_tanh"             # gelu_tanh (SigLIP) | gelu (Whisper)
    # vision stem
    image_size: int = 224
    patch_size: int = 16
    num_channels: int = 3
    # audio stem
    num_mel_bins: int = 80
    max_source_positions: int = 1500

    @property
    def head_dim(self) -> int:
        return self.hidden_size // self.num_heads

    @classmethod
    def from_hf(cls, d: dict) -> "TowerConfig":
        mt = d.get("model_type", "")
        if mt in ("siglip", "siglip2") and "vision_config" in d:
            d, mt = d["vision_config"], "siglip_vision_model"
        if mt in ("siglip_vision_model", "siglip2_vision_model"):
            return cls(kind="siglip", hidden_size=d.get("hidden_size", 768), num_layers=d.get("num_hidden_layers", 12),
                       num_heads=d.get("num_attention_heads", 12), intermediate_size=d.get("intermediate_size", 3072),
                       layer_norm_eps=d.get("layer_norm_eps", 1e-6), act="gelu_tanh" if "tanh" in d.get("hidden_act", "gelu_pytorch_tanh") else "gelu",
                       image_size=d.get("image_size", 224), patch_size=d.get("patch_size", 16), num_channels=d.get("num_channels", 3))
        if mt == "whisper":
            return cls(kind="whisper", hidden_size=d["d_model"], num_layers=d["encoder_layers"], num_heads=d["encoder_attention_heads"],
                       intermediate_size=d["encoder_ffn_dim"], layer_norm_eps=1e-5, act="gelu", num_mel_bins=d.get("num_mel_bins", 80),
                       max_source_positions=d.get("max_source_positions", 1500))
        raise ValueError(f"not a tower this engine knows: model_type={mt!r}")


@dataclass
class TowerLayer:
    ln1_w: torch.Tensor
    ln1_b: torch.Tensor
    wqkv: torch.Tensor
    bqkv: torch.Tensor
    wo: torch.Tensor
    bo: torch.Tensor
    ln2_w: torch.Tensor
    ln2_b: torch.Tensor
    w_in: torch.Tensor
    b_in: torch.Tensor
    w_out: torch.Tensor
    b_out: torch.Tensor


@dataclass
class TowerWeights:
    layers: List[TowerLayer]
    final_ln_w: torch.Tensor
    final_ln_b: torch.Tensor
    pos: torch.Tensor                           # [positions, hidden]
    patch_w: Optional[torch.Tensor] = None      # SigLIP: [hidden, channels * patch * patch] (the patch convolution as a matrix)
    patch_b: Optional[torch.Tensor] = None
    conv1_w: Optional[torch.Tensor] = None      # Whisper: [hidden, mel, 3], [hidden, hidden, 3]
    conv1_b: Optional[torch.Tensor] = None
    conv2_w: Optional[torch.Tensor] = None
    conv2_b: Optional[torch.Tensor] = None


def load_hf_tower(path: str, device="cpu", dtype=torch.bfloat16):
    """A Hugging Face SigLIP (vision part) or Whisper (encoder part) directory -> (config, weights)."""
    from ..formats.safetensors_io import open_checkpoint
    cfg = TowerConfig.from_hf(json.load(open(os.path.join(path, "config.json"))))
    ck = open_checkpoint(path)
    names = set(ck.keys())
    t = lambda n: ck[n][0].tensor(ck[n][1]).to(device=device, dtype=dtype).contiguous()
    H = cfg.hidden_size
    if cfg.kind == "siglip":
        root = next((p for p in ("vision_model.", "vision_tower.vision_model.", "model.vision_model.", "")
                     if p + "embeddings.patch_embedding.weight" in names), None)
        if root is None:
            raise ValueError("no SigLIP vision tower in this checkpoint")
        lp, attn, names_qkv, o_name, fc1, fc2 = root + "encoder.layers.{}.", "self_attn.", ("q_proj", "k_proj", "v_proj"), "out_proj", "mlp.fc1", "mlp.fc2"
        ln1, ln2 = "layer_norm1", "layer_norm2"
    else:
        root = next((p for p in ("model.encoder.", "encoder.") if p + "conv1.weight" in names), None)
        if root is None:
            raise ValueError("no Whisper encoder in this checkpoint")
        lp, attn, names_qkv, o_name, fc1, fc2 = root + "layers.{}.", "self_attn.", ("q_proj", "k_proj", "v_proj"), "out_proj", "fc1", "fc2"
        ln1, ln2 = "self_attn_layer_norm", "final_layer_norm"
    layers = []
    for i in range(cfg.num_layers):
        p = lp.format(i)
        ws = [t(p + attn + n + ".weight") for n in names_qkv]
        bs = [t(p + attn + n + ".bias") if p + attn + n + ".bias" in names else torch.zeros(H, device=device, dtype=dtype) for n in names_qkv]
        layers.append(TowerLayer(t(p + ln1 + ".weight"), t(p + ln1 + ".bias"), torch.cat(ws, 0).contiguous(), torch.cat(bs, 0).contiguous(),
                                 t(p + attn + o_name + ".weight"), t(p + attn + o_name + ".bias"), t(p + ln2 + ".weight"), t(p + ln2 + ".bias"),
                                 t(p + fc1 + ".weight"), t(p + fc1 + ".bias"), t(p + fc2 + ".weight"), t(p + fc2 + ".bias")))
    if cfg.kind == "siglip":
        pw = t(root + "embeddings.patch_embedding.weight")
        w = TowerWeights(layers, t(root + "post_layernorm.weight"), t(root + "post_layernorm.bias"),
                         t(root + "embeddings.position_embedding.weight"), patch_w=pw.reshape(pw.shape[0], -1).contiguous(),
                         patch_b=t(root + "embeddings.patch_embedding.bias"))
    else:
        w = TowerWeights(layers, t(root + "layer_norm.weight"), t(root + "layer_norm.bias"), t(root + "embed_positions.weight"),
                         conv1_w=t(root + "conv1.weight"), conv1_b=t(root + "conv1.bias"), conv2_w=t(root + "conv2.weight"),
                         conv2_b=t(root + "conv2.bias"))
    for f in {id(v[0]): v[0] for v in ck.values()}.values():
        f.close()
    return cfg, w


class Tower:
    BLOCK = 16

    def __init__(self, cfg: TowerConfig, weights: TowerWeights, ops, device):
        self.cfg, self.w, self.ops = cfg, weights, ops
        self.device = torch.device(device)
        self.inv_freq = torch.zeros(max(cfg.head_dim // 2, 1), dtype=torch.float32, device=self.device)   # no rotation
        self._pool = None
        self.kernel_attention = cfg.head_dim in (64, 128, 256)

    # ------------------------------------------------------------------ stems
    def vision_stem(self, pixels: torch.Tensor) -> torch.Tensor:
        """pixels [B, channels, size, size] -> patch embeddings + positions [B, patches, hidden]."""
        cfg, w = self.cfg, self.w
        B, C, Hh, Ww = pixels.shape
        p = cfg.patch_size
        if C != cfg.num_channels or Hh % p or Ww % p or (Hh // p) * (Ww // p) != w.pos.shape[0]:
            raise ValueError(f"images must be {cfg.num_channels} x {cfg.image_size} x {cfg.image_size}")
        patches = pixels.to(w.patch_w.dtype).unfold(2, p, p).unfold(3, p, p)             # [B, C, gh, gw, p, p]
        patches = patches.permute(0, 2, 3, 1, 4, 5).reshape(B * w.pos.shape[0], C * p * p).contiguous()
        x = self.ops.linear(patches, w.patch_w, w.patch_b)                                # the patch convolution as one GEMM
        return (x.view(B, -1, cfg.hidden_size).float() + w.pos.float()).to(x.dtype)

    def audio_stem(self, mel: torch.Tensor) -> torch.Tensor:
        """mel [B, mel bins, frames] -> [B, frames / 2, hidden] (GELU after each convolution, fixed positions added)."""
        w = self.w
        x = F.gelu(F.conv1d(mel.to(w.conv1_w.dtype), w.conv1_w, w.conv1_b, padding=1).float())
        x = F.gelu(F.conv1d(x.to(w.conv2_w.dtype), w.conv2_w, w.conv2_b, stride=2, padding=1).float())
        x = x.permute(0, 2, 1)
        if x.shape[1] > w.pos.shape[0]:
            raise ValueError(f"at most {2 * w.pos.shape[0]} frames")
        return (x + w.pos[:x.shape[1]].float()).to(w.conv1_w.dtype)

    # ------------------------------------------------------------------ blocks
    def _attention(self, qkv: torch.Tensor, B: int, n: int, meta) -> torch.Tensor:
        cfg, ops = self.cfg, self.ops
        nh, D = cfg.num_heads, cfg.head_dim
        if not self.kernel_attention:
            q, k, v = qkv.view(B, n, 3, nh, D).permute(2, 0, 3, 1, 4)
            return F.scaled_dot_product_attention(q, k, v).permute(0, 2, 1, 3).reshape(B * n, nh * D)
        kc, vc, slots, row_seq, vis, zeros_pos = meta["pool"] + meta["rows"]
        q = ops.rope_kv_write(qkv, zeros_pos, slots, self.inv_freq, None, None, kc, vc, nh, nh, D, D, 0, 1e-6, 1.0)
        return ops.attention(q, kc, vc, meta["batch"].block_tables, row_seq, vis, nh, nh, D, D ** -0.5, meta=meta["batch"],
                             bidirectional=True).contiguous()

    def _meta(self, B: int, n: int):
        if not self.kernel_attention:
            return None
        dev, bs = self.device, self.BLOCK
        nblk = -(-n // bs)
        if self._pool is None or self._pool.shape[1] < B * nblk:
            self._pool = torch.zeros(2, max(B * nblk, 64), self.cfg.num_heads, bs, self.cfg.head_dim,
                                     dtype=self.w.final_ln_w.dtype, device=dev)
        tables = torch.arange(B * nblk, dtype=torch.int32, device=dev).view(B, nblk)
        ar = torch.arange(n, dtype=torch.int32, device=dev)
        slots = (torch.arange(B, dtype=torch.int32, device=dev)[:, None] * (nblk * bs) + ar[None, :]).reshape(-1).contiguous()
        row_seq = torch.arange(B, dtype=torch.int32, device=dev).repeat_interleave(n).contiguous()
        vis = torch.full((B * n,), n - 1, dtype=torch.int32, device=dev)
        batch = StepBatch(None, vis, slots, row_seq, tables, None, num_seqs=B, num_tokens=B * n, max_kv_len=n, all_decode=False,
                          seq_lens=torch.full((B,), n, dtype=torch.int32, device=dev),
                          q_starts=torch.arange(0, B * n + 1, n, dtype=torch.int32, device=dev), max_q_len=n, min_q_len=n)
        return {"pool": (self._pool[0], self._pool[1]), "rows": (slots, row_seq, vis, torch.zeros(B * n, dtype=torch.int32, device=dev)),
                "batch": batch}

    @torch.inference_mode()
    def forward(self, inputs: torch.Tensor) -> torch.Tensor:
        """Images [B, C, size, size] (SigLIP) or log-mel spectrograms [B, mel, frames] (Whisper) -> last hidden states
        [B, positions, hidden] (after the final LayerNorm)."""
        cfg, ops = self.cfg, self.ops
        x = self.vision_stem(inputs) if cfg.kind == "siglip" else self.audio_stem(inputs)
        B, n, H = x.shape
        x = x.reshape(B * n, H).contiguous()
        meta = self._meta(B, n)
        act = (lambda t: F.gelu(t, approximate="tanh")) if cfg.act == "gelu_tanh" else F.gelu
        ln = lambda t, wt, bt: F.layer_norm(t.float(), (H,), wt.float(), bt.float(), cfg.layer_norm_eps).to(t.dtype)
        for lw in self.w.layers:
            a = self._attention(ops.linear(ln(x, lw.ln1_w, lw.ln1_b), lw.wqkv, lw.bqkv), B, n, meta)
            x = (x.float() + ops.linear(a, lw.wo, lw.bo).float()).to(x.dtype)
            f = act(ops.linear(ln(x, lw.ln2_w, lw.ln2_b), lw.w_in, lw.b_in).float()).to(x.dtype)
            x = (x.float() + ops.linear(f, lw.w_out, lw.b_out).float()).to(x.dtype)
        return ln(x, self.w.final_ln_w, self.w.final_ln_b).view(B, n, H)
