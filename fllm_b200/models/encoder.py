"""BERT-family encoders (BERT, RoBERTa, XLM-RoBERTa): bidirectional attention over packed sequences, post-LayerNorm
blocks, learned positions, CLS / mean pooling, optional pooler + classifier head (cross-encoder rerankers).

The projections run through ``ops.linear`` (the tcgen05 GEMMs, bias in the epilogue) and the attention through
``ops.attention(..., bidirectional=True)``: keys and values of a batch are written into a scratch paged pool by the
same kernel the decoder uses (with a zero frequency table, so nothing is rotated) and the prefill attention
kernels run without their causal mask. LayerNorm, GELU and the embedding sums are plain PyTorch. The reference's
counterpart is its encoder server (rust/engine/src/encoder.rs, rust/engine/src/encoder_server.rs:1233-1266,
rust/engine/cuda/attn_encoder.cu:41).
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass
from typing import List, Optional, Sequence

import torch
import torch.nn.functional as F

from .decoder import StepBatch


@dataclass
class EncoderConfig:
    arch: str = "bert"                 # bert | roberta | xlm-roberta
    vocab_size: int = 30522
    hidden_size: int = 768
    num_layers: int = 12
    num_heads: int = 12
    intermediate_size: int = 3072
    max_position: int = 512
    type_vocab_size: int = 2
    layer_norm_eps: float = 1e-12
    pad_token_id: int = 0
    num_labels: int = 0                # > 0: a classifier head follows the pooler
    pooling: str = "cls"               # cls | mean
    hidden_act: str = "gelu"

    @property
    def head_dim(self) -> int:
        return self.hidden_size // self.num_heads

    @property
    def position_offset(self) -> int:
        """RoBERTa-style checkpoints number positions from padding_idx + 1."""
        return self.pad_token_id + 1 if self.arch in ("roberta", "xlm-roberta") else 0

    @classmethod
    def from_hf(cls, d: dict) -> "EncoderConfig":
        arch = d.get("model_type", "bert")
        if arch not in ("bert", "roberta", "xlm-roberta"):
            raise ValueError(f"not an encoder this engine knows: model_type={arch!r}")
        n_labels = 0
        archs = " ".join(d.get("architectures") or [])
        if "SequenceClassification" in archs:
            n_labels = len(d.get("id2label") or {}) or int(d.get("num_labels", 1))
        return cls(arch=arch, vocab_size=d["vocab_size"], hidden_size=d["hidden_size"], num_layers=d["num_hidden_layers"],
                   num_heads=d["num_attention_heads"], intermediate_size=d["intermediate_size"],
                   max_position=d.get("max_position_embeddings", 512), type_vocab_size=d.get("type_vocab_size", 2),
                   layer_norm_eps=d.get("layer_norm_eps", 1e-12), pad_token_id=d.get("pad_token_id", 0) or 0,
                   num_labels=n_labels, hidden_act=d.get("hidden_act", "gelu"))


@dataclass
class EncoderLayer:
    wqkv: torch.Tensor
    bqkv: torch.Tensor
    wo: torch.Tensor
    bo: torch.Tensor
    ln1_w: torch.Tensor
    ln1_b: torch.Tensor
    w_in: torch.Tensor
    b_in: torch.Tensor
    w_out: torch.Tensor
    b_out: torch.Tensor
    ln2_w: torch.Tensor
    ln2_b: torch.Tensor


@dataclass
class EncoderWeights:
    word: torch.Tensor
    pos: torch.Tensor
    typ: torch.Tensor
    emb_ln_w: torch.Tensor
    emb_ln_b: torch.Tensor
    layers: List[EncoderLayer]
    pooler_w: Optional[torch.Tensor] = None
    pooler_b: Optional[torch.Tensor] = None
    cls_w: Optional[torch.Tensor] = None       # [num_labels, hidden] (RoBERTa heads: dense + out_proj)
    cls_b: Optional[torch.Tensor] = None
    cls_dense_w: Optional[torch.Tensor] = None
    cls_dense_b: Optional[torch.Tensor] = None


def init_random_encoder(cfg: EncoderConfig, device="cpu", dtype=torch.bfloat16, seed: int = 0) -> EncoderWeights:
    g = torch.Generator().manual_seed(seed)
    r = lambda *s: (torch.randn(*s, generator=g) * 0.02).to(device=device, dtype=dtype)
    one = lambda n: torch.ones(n, device=device, dtype=dtype)
    zero = lambda n: torch.zeros(n, device=device, dtype=dtype)
    H, I = cfg.hidden_size, cfg.intermediate_size
    layers = [EncoderLayer(r(3 * H, H), r(3 * H), r(H, H), r(H), one(H), zero(H), r(I, H), r(I), r(H, I), r(H), one(H), zero(H))
              for _ in range(cfg.num_layers)]
    w = EncoderWeights(r(cfg.vocab_size, H), r(cfg.max_position, H), r(cfg.type_vocab_size, H), one(H), zero(H), layers,
                       r(H, H), r(H))
    if cfg.num_labels:
        w.cls_w, w.cls_b = r(cfg.num_labels, H), r(cfg.num_labels)
    return w


def load_hf_encoder(path: str, device="cpu", dtype=torch.bfloat16):
    """A Hugging Face BERT / RoBERTa / XLM-R directory (config.json + safetensors) -> (config, weights)."""
    from ..formats.safetensors_io import open_checkpoint
    cfg = EncoderConfig.from_hf(json.load(open(os.path.join(path, "config.json"))))
    ck = open_checkpoint(path)
    names = set(ck.keys())
    prefix = next((p for p in ("bert.", "roberta.", "") if p + "embeddings.word_embeddings.weight" in names), None)
    if prefix is None:
        raise ValueError("no encoder embeddings in this checkpoint")
    t = lambda n: ck[n][0].tensor(ck[n][1]).to(device=device, dtype=dtype).contiguous()
    has = lambda n: n in names
    layers = []
    for i in range(cfg.num_layers):
        p = f"{prefix}encoder.layer.{i}."
        q, k, v = (t(p + f"attention.self.{n}.weight") for n in ("query", "key", "value"))
        bq, bk, bv = (t(p + f"attention.self.{n}.bias") for n in ("query", "key", "value"))
        layers.append(EncoderLayer(
            torch.cat([q, k, v], 0).contiguous(), torch.cat([bq, bk, bv], 0).contiguous(),
            t(p + "attention.output.dense.weight"), t(p + "attention.output.dense.bias"),
            t(p + "attention.output.LayerNorm.weight"), t(p + "attention.output.LayerNorm.bias"),
            t(p + "intermediate.dense.weight"), t(p + "intermediate.dense.bias"),
            t(p + "output.dense.weight"), t(p + "output.dense.bias"),
            t(p + "output.LayerNorm.weight"), t(p + "output.LayerNorm.bias")))
    e = prefix + "embeddings."
    w = EncoderWeights(t(e + "word_embeddings.weight"), t(e + "position_embeddings.weight"),
                       t(e + "token_type_embeddings.weight"), t(e + "LayerNorm.weight"), t(e + "LayerNorm.bias"), layers)
    if has(prefix + "pooler.dense.weight"):
        w.pooler_w, w.pooler_b = t(prefix + "pooler.dense.weight"), t(prefix + "pooler.dense.bias")
    if has("classifier.weight"):
        w.cls_w, w.cls_b = t("classifier.weight"), t("classifier.bias")
    elif has("classifier.out_proj.weight"):
        w.cls_dense_w, w.cls_dense_b = t("classifier.dense.weight"), t("classifier.dense.bias")
        w.cls_w, w.cls_b = t("classifier.out_proj.weight"), t("classifier.out_proj.bias")
    for f in {id(v[0]): v[0] for v in ck.values()}.values():
        f.close()
    return cfg, w


class Encoder:
    BLOCK = 16

    def __init__(self, cfg: EncoderConfig, weights: EncoderWeights, ops, device):
        self.cfg, self.w, self.ops = cfg, weights, ops
        self.device = torch.device(device)
        self.inv_freq = torch.zeros(cfg.head_dim // 2, dtype=torch.float32, device=self.device)   # no rotation
        self._pool = None

    def _kv_pool(self, blocks: int):
        if self._pool is None or self._pool.shape[1] < blocks:
            self._pool = torch.zeros(2, max(blocks, 64), self.cfg.num_heads, self.BLOCK, self.cfg.head_dim,
                                     dtype=self.w.word.dtype, device=self.device)
        return self._pool[0], self._pool[1]

    @torch.inference_mode()
    def forward(self, seqs: Sequence[Sequence[int]], type_ids: Optional[Sequence[Sequence[int]]] = None) -> torch.Tensor:
        """Token hidden states of a batch of sequences, packed: [sum(len), hidden]."""
        cfg, w, ops, dev = self.cfg, self.w, self.ops, self.device
        lens = [len(s) for s in seqs]
        if not lens or min(lens) < 1:
            raise ValueError("empty sequence")
        if max(lens) + cfg.position_offset > cfg.max_position:
            raise ValueError(f"sequence longer than the model's {cfg.max_position - cfg.position_offset} positions")
        T, B, bs = sum(lens), len(lens), self.BLOCK
        ids = torch.tensor([t for s in seqs for t in s], dtype=torch.long, device=dev)
        pos = torch.cat([torch.arange(n) for n in lens]).to(dev)
        typ = torch.tensor([t for s in (type_ids or [[0] * n for n in lens]) for t in s], dtype=torch.long, device=dev)
        x = w.word[ids].float() + w.pos[pos + cfg.position_offset].float() + w.typ[typ].float()
        x = F.layer_norm(x, (cfg.hidden_size,), w.emb_ln_w.float(), w.emb_ln_b.float(), cfg.layer_norm_eps).to(w.word.dtype)
        # paged scratch pool: every sequence starts on a block boundary
        nblk = [-(-n // bs) for n in lens]
        first = [0]
        for n in nblk:
            first.append(first[-1] + n)
        kc, vc = self._kv_pool(first[-1])
        tables = torch.zeros(B, max(nblk), dtype=torch.int32)
        slots, row_seq, last_pos, q_starts = [], [], [], [0]
        for i, n in enumerate(lens):
            tables[i, :nblk[i]] = torch.arange(first[i], first[i] + nblk[i], dtype=torch.int32)
            slots += list(range(first[i] * bs, first[i] * bs + n))
            row_seq += [i] * n
            last_pos += [n - 1] * n                      # every row sees the whole sequence
            q_starts.append(q_starts[-1] + n)
        i32 = lambda a: torch.tensor(a, dtype=torch.int32, device=dev)
        slots_t, row_seq_t, vis = i32(slots), i32(row_seq), i32(last_pos)
        meta = StepBatch(None, vis, slots_t, row_seq_t, tables.to(dev), None, num_seqs=B, num_tokens=T, max_kv_len=max(lens),
                         all_decode=False, seq_lens=i32(lens), q_starts=i32(q_starts), max_q_len=max(lens), min_q_len=min(lens))
        H, nh, D = cfg.hidden_size, cfg.num_heads, cfg.head_dim
        zeros_pos = torch.zeros(T, dtype=torch.int32, device=dev)
        for lw in w.layers:
            qkv = ops.linear(x, lw.wqkv, lw.bqkv)
            q = ops.rope_kv_write(qkv, zeros_pos, slots_t, self.inv_freq, None, None, kc, vc, nh, nh, D, D, 0, 1e-6, 1.0)
            a = ops.attention(q, kc, vc, meta.block_tables, row_seq_t, vis, nh, nh, D, D ** -0.5, meta=meta, bidirectional=True)
            o = ops.linear(a.contiguous(), lw.wo, lw.bo)
            x = F.layer_norm(x.float() + o.float(), (H,), lw.ln1_w.float(), lw.ln1_b.float(), cfg.layer_norm_eps).to(x.dtype)
            f = F.gelu(ops.linear(x, lw.w_in, lw.b_in).float()).to(x.dtype)
            f = ops.linear(f, lw.w_out, lw.b_out)
            x = F.layer_norm(x.float() + f.float(), (H,), lw.ln2_w.float(), lw.ln2_b.float(), cfg.layer_norm_eps).to(x.dtype)
        self._last_starts = q_starts
        return x

    @torch.inference_mode()
    def embed(self, seqs, type_ids=None, pooling: Optional[str] = None, normalize: bool = True) -> torch.Tensor:
        """One vector per sequence: [B, hidden] fp32 (CLS token or mean over tokens; L2-normalised on request)."""
        x = self.forward(seqs, type_ids).float()
        st = self._last_starts
        if (pooling or self.cfg.pooling) == "mean":
            out = torch.stack([x[st[i]:st[i + 1]].mean(0) for i in range(len(seqs))])
        else:
            out = x[torch.tensor(st[:-1], device=x.device)]
        return F.normalize(out, dim=-1) if normalize else out

    @torch.inference_mode()
    def classify(self, seqs, type_ids=None) -> torch.Tensor:
        """Logits of the sequence-classification head ([B, num_labels]): pooler (dense + tanh on CLS) then the
        classifier for BERT, dense + tanh + out_proj for RoBERTa heads. A cross-encoder's relevance score is label 0."""
        w = self.w
        if w.cls_w is None:
            raise ValueError("this checkpoint has no classification head")
        x = self.forward(seqs, type_ids).float()
        cls = x[torch.tensor(self._last_starts[:-1], device=x.device)]
        if w.cls_dense_w is not None:
            h = torch.tanh(cls @ w.cls_dense_w.float().t() + w.cls_dense_b.float())
        elif w.pooler_w is not None:
            h = torch.tanh(cls @ w.pooler_w.float().t() + w.pooler_b.float())
        else:
            h = cls
        return h @ w.cls_w.float().t() + w.cls_b.float()
