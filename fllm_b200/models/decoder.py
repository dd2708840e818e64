"""One decoder runner for every supported family (Llama, Qwen3, gpt-oss).

The step contract is the reference's ragged batch (``RustDecoder::forward_with_hidden``,
rust/engine/src/rust_decoder.rs:8480): token ids, positions, KV slots, block tables and
the rows whose logits are wanted. The layer loop is the one of
rust/engine/src/rust_decoder.rs:4467-6050, re-cut for bf16 activations and fused
kernels: each norm consumes the previous projection's output as a residual delta, QK
norm + RoPE + KV write are one kernel, and under tensor parallelism the projection
outputs are combined either by the fused peer-memory kernels or by a library
all-reduce (baseline).
"""
from __future__ import annotations

import os
from dataclasses import dataclass
from typing import List, Optional

import torch

from ..config import ModelConfig, rope_inv_freq
from .weights import DecoderWeights, ShardSpec, make_shard_spec

ACT_KIND = {"swiglu": 0, "geglu": 1, "swiglu_oai": 2}


@dataclass
class StepBatch:
    """Device-side description of one engine step."""
    token_ids: torch.Tensor          # [T] int32
    positions: torch.Tensor          # [T] int32, position of each token in its sequence
    slots: torch.Tensor              # [T] int32, KV slot = block * block_size + offset (-1 = skip)
    row_seq: torch.Tensor            # [T] int32, index into block_tables
    block_tables: torch.Tensor       # [B, max_blocks] int32
    logit_rows: torch.Tensor         # [R] int32, token rows whose logits are needed
    # host-side facts used to pick kernels (never read by kernels)
    num_seqs: int = 0
    num_tokens: int = 0
    max_kv_len: int = 0
    all_decode: bool = False
    max_q_len: int = 1
    min_q_len: int = 1
    seq_lens: Optional[torch.Tensor] = None      # [B] int32 visible KV length per sequence
    q_starts: Optional[torch.Tensor] = None      # [B+1] int32 first token row of each sequence
    seq_state: Optional[torch.Tensor] = None     # [B] int32 row of the recurrent-state pools (hybrid families)
    host_seqs: Optional[list] = None             # the same on the host for steps with long prompt chunks: (first row, rows, state row, fresh)


class KVCache:
    """Paged KV pool: one K and one V tensor per local layer,
    [num_blocks, kv_heads_local, block_size, head_dim]."""

    def __init__(self, num_layers: int, num_blocks: int, kv_heads: int, block_size: int, head_dim: int,
                 device, dtype=torch.bfloat16):
        """dtype torch.float8_e4m3fn halves the pool (values stored unscaled; written by the rope kernel,
        read by the generic attention kernel)."""
        self.num_blocks, self.block_size = num_blocks, block_size
        self.store = torch.zeros(num_layers, 2, num_blocks, kv_heads, block_size, head_dim,
                                 device=device, dtype=dtype)

    def k(self, layer: int) -> torch.Tensor:
        return self.store[layer, 0]

    def v(self, layer: int) -> torch.Tensor:
        return self.store[layer, 1]

    @staticmethod
    def bytes_per_block(num_layers, kv_heads, block_size, head_dim, elem=2) -> int:
        return num_layers * 2 * kv_heads * block_size * head_dim * elem


class Decoder:
    def __init__(self, cfg: ModelConfig, weights: DecoderWeights, kv: KVCache, ops, spec: Optional[ShardSpec] = None,
                 tp_group=None, layer_range: Optional[range] = None, first_stage: bool = True,
                 last_stage: bool = True, rstate=None):
        self.cfg, self.w, self.kv, self.ops = cfg, weights, kv, ops
        self.rstate = rstate          # models.recurrent.RecurrentState when some layer is recurrent
        self.spec = spec or make_shard_spec(cfg)
        self.tp = tp_group            # object with all_reduce / all_gather (or None)
        self.layer_range = layer_range or range(cfg.num_layers)
        self.first_stage, self.last_stage = first_stage, last_stage
        # the KV pool holds only this stage's attention layers
        self.kv_index = {li: i for i, li in enumerate(l for l in self.layer_range if cfg.has_kv(l))}
        dev = weights.final_norm.device
        inv, attn = rope_inv_freq(cfg)
        if not cfg.use_rope:                       # a zero frequency table turns the rotation into the identity
            inv = [0.0] * len(inv)
        self.inv_freq = torch.tensor(inv, dtype=torch.float32, device=dev)
        self.inv_freq_local = None
        self._inv_freq_zero = None
        if cfg.rope_local_theta > 0:               # windowed layers: their own base, never scaled
            rot = cfg.rot_dim
            self.inv_freq_local = torch.tensor([cfg.rope_local_theta ** (-(2.0 * i) / rot) for i in range(rot // 2)],
                                               dtype=torch.float32, device=dev)
        self.attn_factor = attn
        self.scale = cfg.attn_scale if cfg.attn_scale else cfg.head_dim ** -0.5
        self.rope_style = 0 if cfg.rope_style == "neox" else 1
        self.act_kind = ACT_KIND.get(cfg.act, 0)
        # packed payloads loaded from a checkpoint become weight objects that pick their own kernel
        for lw in self.w.layers:
            for name, packed in list(lw.packed.items()):
                if packed[0] == "fp8_block":
                    from ..ops.native import Fp8BlockWeight
                    setattr(lw, name, Fp8BlockWeight(packed[1], packed[2]))
                elif packed[0] in ("nvfp4", "mxfp4"):
                    from ..ops.fp4 import FMT_NAMES, Fp4Weight
                    setattr(lw, name, Fp4Weight(packed[1], packed[2], FMT_NAMES[packed[0]], packed[3] if len(packed) > 3 else 1.0))
        # the GEMMs take row counts in multiples of 8: a head with an odd vocabulary (added tokens) gets zero rows; the
        # logits beyond vocab_local are cut off by the consumers
        head = self.w.lm_head
        if dev.type == "cuda" and isinstance(head, torch.Tensor) and head.shape[0] % 8 and head.shape[0] > 0:
            padded = torch.zeros((head.shape[0] + 7) // 8 * 8, head.shape[1], dtype=head.dtype, device=head.device)
            padded[:head.shape[0]] = head
            self.w.lm_head = padded
            if self.w.lm_head_b is not None:
                self.w.lm_head_b = torch.nn.functional.pad(self.w.lm_head_b, (0, padded.shape[0] - head.shape[0]))
        self.capture_hidden, self.last_hidden = False, None
        # FLLM_NVTX=1: named ranges per layer half for timeline profilers
        self._nvtx = os.environ.get("FLLM_NVTX", "0") not in ("", "0") and dev.type == "cuda"
        self.ep_a2a = None            # comm.ep_a2a.EpAllToAll when expert parallelism dispatches rows all-to-all
        self._reduced = False
        self._dense_weights = all(isinstance(getattr(lw, n, None), torch.Tensor) for lw in self.w.layers
                                  for n in ("wqkv", "wo", "w_gate_up", "w_down") if getattr(lw, n, None) is not None)
        # split-K reductions of the projections are left to the kernel that consumes them (norm / rope)
        # (only the RMSNorm, rope and gated-activation kernels take partials: LayerNorm families and parallel blocks do not defer)
        self._defer = (hasattr(ops, "k") and dev.type == "cuda" and cfg.norm_kind == "rms" and not cfg.parallel_block
                       and not cfg.qk_norm_full and not cfg.clip_qkv)
        if self._defer:
            self._block_gate_up()

    def _block_gate_up(self) -> None:
        """Re-order the rows of every dense gate|up matrix into blocks of 16 gate rows followed by the 16 up
        rows of the same features (once per weight object, in place), so that the GEMM epilogue holds a
        feature's gate and up values in one warp and applies the activation itself."""
        if self.cfg.is_moe or self.cfg.act not in ("swiglu", "geglu"):
            return
        for lw in self.w.layers:
            w = lw.w_gate_up
            if not isinstance(w, torch.Tensor) or getattr(lw, "glu_layout", 0) or (w.shape[0] // 2) % 16:
                continue
            I, K = w.shape[0] // 2, w.shape[1]
            blocked = torch.stack([w[:I].view(I // 16, 16, K), w[I:].view(I // 16, 16, K)], 1).reshape(2 * I, K)
            w.copy_(blocked)
            del blocked
            lw.glu_layout = 16

    # ------------------------------------------------------------------ pieces
    def _reduce(self, x: torch.Tensor) -> torch.Tensor:
        if self._reduced:
            self._reduced = False
            return x
        if self.tp is not None and self.tp.size > 1:
            return self.tp.all_reduce(x)
        return x

    def _attention_block(self, li: int, lw, h: torch.Tensor, b: StepBatch) -> torch.Tensor:
        cfg, sp, ops = self.cfg, self.spec, self.ops
        gated = lw.w_attn_gate is not None
        qkv = ops.linear(h, lw.wqkv, lw.bqkv, defer=self._defer and not gated)
        if lw.q_norm_full is not None:             # RMSNorm over all heads of q and of k at once, before the rotation
            nq, nk = sp.hq_local * cfg.head_dim, sp.hkv_local * cfg.head_dim
            qkv[:, :nq] = ops.rmsnorm(qkv[:, :nq].contiguous(), None, lw.q_norm_full, cfg.rms_eps, 0.0)
            qkv[:, nq:nq + nk] = ops.rmsnorm(qkv[:, nq:nq + nk].contiguous(), None, lw.k_norm_full, cfg.rms_eps, 0.0)
        if cfg.clip_qkv > 0:                       # after the full-width norms where a family has both (OLMoE)
            qkv = ops.materialize(qkv).clamp_(-cfg.clip_qkv, cfg.clip_qkv)
        local = self.kv_index[li]
        kc, vc = self.kv.k(local), self.kv.v(local)
        local_rope = self.inv_freq_local is not None and cfg.layer_window(li) > 0
        inv = self.inv_freq_local if local_rope else self.inv_freq
        if cfg.rope_layers is not None and not cfg.rope_layers[li]:
            if self._inv_freq_zero is None:
                self._inv_freq_zero = torch.zeros_like(self.inv_freq)
            inv = self._inv_freq_zero
        q = ops.rope_kv_write(qkv, b.positions, b.slots, inv, lw.q_norm, lw.k_norm,
                              kc, vc, sp.hq_local, sp.hkv_local, cfg.head_dim, cfg.rot_dim, self.rope_style,
                              cfg.rms_eps, 1.0 if local_rope else self.attn_factor)
        a = ops.attention(q, kc, vc, b.block_tables, b.row_seq, b.positions, sp.hq_local, sp.hkv_local,
                          cfg.head_dim, self.scale, cfg.layer_window(li), lw.sinks, cfg.attn_softcap,
                          meta=b)
        if gated:                                # the attention output passes through a sigmoid gate of its own projection
            a = (a.float() * torch.sigmoid(ops.linear(h, lw.w_attn_gate).float())).to(a.dtype)
        return ops.linear(a, lw.wo, lw.bo, defer=self._defer_out(lw.post_attn_norm))

    def _defer_out(self, post_norm) -> bool:
        """May a row-parallel projection hand its split-K partials to the next norm? Only when nothing
        sits between the two: no all-reduce, no output norm, no pipeline hand-over."""
        return (self._defer and post_norm is None and (self.tp is None or self.tp.size == 1)
                and self.first_stage and self.last_stage)

    def _norm(self, x, delta, w, b=None):
        """The block norm of the family: RMSNorm, or LayerNorm with / without bias; `delta` is added to `x` in place first."""
        cfg = self.cfg
        if cfg.norm_kind == "rms" or (cfg.norm_kind == "none" and w is not None):     # (the final norm of a "none" family is an RMSNorm)
            return self.ops.rmsnorm(x, delta, w, cfg.rms_eps, cfg.norm_weight_offset)
        if cfg.norm_kind == "none":                # the block reads the residual stream as it is
            if delta is not None:
                x.add_(self.ops.materialize(delta))
            return x
        return self.ops.layernorm(x, delta, w, b, cfg.rms_eps, cfg.norm_weight_offset)

    def _ffn_block(self, lw, h: torch.Tensor) -> torch.Tensor:
        cfg, ops = self.cfg, self.ops
        if lw.router_w is not None:
            from .moe import moe_ffn, moe_ffn_alltoall
            if self.ep_a2a is not None:
                self._reduced = True                 # rows come back complete: nothing left to reduce
                return moe_ffn_alltoall(self, lw, h)
            if lw.moe_latent_in is not None:         # the router reads the hidden state, the experts a projection of it
                y = ops.linear(moe_ffn(self, lw, h, ops.linear(h, lw.moe_latent_in)), lw.moe_latent_out)
            else:
                y = moe_ffn(self, lw, h)
            if lw.shared_gate_up is not None:        # always-on shared experts: one dense MLP beside the routed ones
                if cfg.mlp_kind == "plain":
                    act = ops.act_(ops.linear(h, lw.shared_gate_up), cfg.act)
                else:
                    act = ops.linear_glu(h, lw.shared_gate_up, None, self.act_kind, cfg.swiglu_alpha, cfg.swiglu_limit, 0)
                ys = ops.linear(act, lw.shared_down)
                if lw.shared_gate_w is not None:
                    ys = (ys.float() * torch.sigmoid(ops.linear(h, lw.shared_gate_w)[:, :1].float())).to(ys.dtype)
                y = y + ys
            return y
        if cfg.mlp_kind == "plain":               # two matrices and an activation between them
            u = ops.act_(ops.linear(h, lw.w_gate_up, lw.b_up), cfg.act)
            return ops.linear(u, lw.w_down, lw.b_down)
        act = ops.linear_glu(h, lw.w_gate_up, None, self.act_kind, cfg.swiglu_alpha, cfg.swiglu_limit,
                             getattr(lw, "glu_layout", 0))
        return ops.linear(act, lw.w_down, defer=self._defer_out(lw.post_ffn_norm))

    # ------------------------------------------------------------------ forward
    def forward_hidden(self, b: StepBatch, hidden_in: Optional[torch.Tensor] = None,
                       delta_in: Optional[torch.Tensor] = None):
        """Runs this stage's layers. Returns (residual, pending_delta): the residual
        stream and the last projection output that has not been added yet."""
        cfg, ops = self.cfg, self.ops
        if cfg.arch == "rwkv7":
            from .rwkv import rwkv7_forward_hidden
            return rwkv7_forward_hidden(self, b)
        if cfg.arch == "rwkv6":
            from .rwkv import rwkv6_forward_hidden
            return rwkv6_forward_hidden(self, b)
        if self.first_stage:
            x = ops.embed(b.token_ids, self.w.embed, cfg.embed_scale)
            if cfg.learned_positions:              # the same row gather on the position table
                pos_ids = b.positions + cfg.position_offset if cfg.position_offset else b.positions
                x = x + ops.embed(pos_ids, self.w.pos_embed, 1.0)
            delta = None
        else:
            x, delta = hidden_in, delta_in
        nvtx = self._nvtx
        for li, lw in zip(self.layer_range, self.w.layers):
            if nvtx:
                torch.cuda.nvtx.range_push(f"layer{li}.attn")
            h = self._norm(x, delta, lw.attn_norm, lw.attn_norm_b)
            kind = cfg.layer_kind(li)
            if cfg.parallel_block:                    # attention and MLP side by side from one read of the residual
                o = ops.materialize(self._reduce(self._attention_block(li, lw, h, b)))
                h2 = h if cfg.parallel_norms == 1 else self._norm(x, None, lw.ffn_norm, lw.ffn_norm_b)
                delta = o + ops.materialize(self._reduce(self._ffn_block(lw, h2)))
                if nvtx:
                    torch.cuda.nvtx.range_pop()
                continue
            if kind == "none":                        # a block that is only a feed-forward network behind its norm
                delta = self._reduce(self._ffn_block(lw, h))
                if nvtx:
                    torch.cuda.nvtx.range_pop()
                continue
            if kind == "attention":
                o = self._reduce(self._attention_block(li, lw, h, b))
            elif kind == "attention+mamba2":          # two mixers on one normed input
                from .recurrent import mamba2_mixer
                o = ops.materialize(self._reduce(self._attention_block(li, lw, h, b))) + mamba2_mixer(self, li, lw, h, b)
            elif kind == "mla":
                from .mla import mla_block
                o = mla_block(self, li, lw, h, b)
            else:
                from .recurrent import MIXERS
                o = MIXERS[kind](self, li, lw, h, b)
            if cfg.ffn_kind(li) == "none":            # a mixer-only layer (Mamba): its output is the residual delta
                delta = o
                if nvtx:
                    torch.cuda.nvtx.range_pop()
                continue
            if lw.post_attn_norm is not None:
                o = ops.rmsnorm(o, None, lw.post_attn_norm, cfg.rms_eps, cfg.norm_weight_offset)
            if nvtx:
                torch.cuda.nvtx.range_pop()
                torch.cuda.nvtx.range_push(f"layer{li}.ffn")
            h = self._norm(x, o, lw.ffn_norm, lw.ffn_norm_b)
            delta = self._reduce(self._ffn_block(lw, h))
            if lw.post_ffn_norm is not None:
                delta = ops.rmsnorm(delta, None, lw.post_ffn_norm, cfg.rms_eps, cfg.norm_weight_offset)
            if nvtx:
                torch.cuda.nvtx.range_pop()
        return x, delta

    # ------------------------------------------------------------------ fused tensor parallel
    @property
    def fused_tp(self) -> bool:
        return (self.tp is not None and getattr(self.tp, "backend", "") == "fused" and self.tp.size > 1
                and not self.cfg.is_moe and not self.cfg.post_norms and self.first_stage and self.last_stage
                and self._dense_weights and not self.cfg.layer_kinds and not self.cfg.rope_local_theta and self.cfg.rope_layers is None
                and self.cfg.norm_kind == "rms" and self.cfg.mlp_kind == "glu" and not self.cfg.parallel_block)

    def forward_fused(self, b: StepBatch) -> torch.Tensor:
        """Whole forward with the sequence-sharded residual: every projection output leaves the
        GPU from the GEMM epilogue (reduce-scatter over peer memory), one small kernel reduces,
        adds the residual, normalises and pushes the rows to all ranks, and the next GEMM's TMA
        producer waits for those rows. Returns the local vocabulary slice of the logits."""
        cfg, ops, tp, sp = self.cfg, self.ops, self.tp, self.spec
        T = b.token_ids.shape[0]
        bc = tp.use_bcast(T)
        if bc:                       # residual replicated: all rows on every rank
            x = ops.embed(b.token_ids, self.w.embed, cfg.embed_scale)
        else:                        # residual sequence-sharded: only the rows this rank owns
            lo, hi = tp.my_rows(T)
            if hi > lo:
                x = ops.embed(b.token_ids[lo:hi].contiguous(), self.w.embed, cfg.embed_scale)
            else:
                x = torch.zeros(1, cfg.hidden_size, dtype=self.w.embed.dtype, device=self.w.embed.device)
        h_all = tp.ag_local[:T]      # normalised activations of all rows (local buffer)

        def col_linear(w, bias=None):
            # broadcast mode: the norm kernel already reduced everything locally -> plain GEMM;
            # scatter/gather mode: the GEMM's TMA producer waits for the peers' rows
            return ops.linear(h_all, w, bias) if bc else tp.linear_ag(T, w, bias)

        partials = False
        for li, lw in zip(self.layer_range, self.w.layers):
            tp.norm(x, T, partials, lw.attn_norm, cfg.rms_eps, cfg.norm_weight_offset, bc)
            # (Measured on 2 and 4 GPUs: handing split-K partials to the rope kernel and running the gated activation
            # in the gate_up epilogue, which are neutral on one GPU, cost 0.16 / 0.47 ms per step here, where the
            # per-rank matrices are small and the consumers have few rows to spread the sums over. So this path
            # keeps the plain GEMM + reduce and the separate activation kernel.)
            qkv = col_linear(lw.wqkv, lw.bqkv)
            local = li - self.layer_range.start
            kc, vc = self.kv.k(local), self.kv.v(local)
            q = ops.rope_kv_write(qkv, b.positions, b.slots, self.inv_freq, lw.q_norm, lw.k_norm, kc, vc,
                                  sp.hq_local, sp.hkv_local, cfg.head_dim, cfg.rot_dim, self.rope_style,
                                  cfg.rms_eps, self.attn_factor)
            a = ops.attention(q, kc, vc, b.block_tables, b.row_seq, b.positions, sp.hq_local, sp.hkv_local,
                              cfg.head_dim, self.scale, cfg.layer_window(li), lw.sinks, cfg.attn_softcap, meta=b)
            tp.linear_rs(a, lw.wo, lw.bo, bc)
            tp.norm(x, T, True, lw.ffn_norm, cfg.rms_eps, cfg.norm_weight_offset, bc)
            layout = getattr(lw, "glu_layout", 0)
            act = ops.glu(col_linear(lw.w_gate_up), self.act_kind, cfg.swiglu_alpha, cfg.swiglu_limit, layout)
            tp.linear_rs(act, lw.w_down, None, bc)
            partials = True
            if hasattr(ops, "launches"):
                ops.launches += 4 if bc else 6       # the kernels launched through `tp` (upper bound)
        tp.norm(x, T, partials, self.w.final_norm, cfg.rms_eps, cfg.norm_weight_offset, bc)
        if bc:
            hs = h_all if (b.all_decode and b.logit_rows.numel() == T) else ops.gather_rows(h_all, b.logit_rows)
            lg = ops.linear(hs, self.w.lm_head)
            if hasattr(ops, "launches"):
                ops.launches += 1
            if cfg.logit_softcap > 0:
                lg = ops.softcap_(lg, cfg.logit_softcap)
            return lg
        # the head runs on every row (it is the consumer that retires the gathered rows); the
        # wanted rows are selected afterwards
        lg = tp.linear_ag(T, self.w.lm_head)
        if hasattr(ops, "launches"):
            ops.launches += 2
        if not (b.all_decode and b.logit_rows.numel() == T):
            lg = lg.index_select(0, b.logit_rows.long())
        if cfg.logit_softcap > 0:
            lg = ops.softcap_(lg, cfg.logit_softcap)
        return lg

    def logits(self, x: torch.Tensor, delta: Optional[torch.Tensor], b: StepBatch) -> torch.Tensor:
        """Final norm + LM head on the requested rows -> [R, vocab_local]."""
        cfg, ops = self.cfg, self.ops
        if cfg.arch in ("rwkv7", "rwkv6"):
            from .rwkv import rwkv7_final_norm
            h = rwkv7_final_norm(self, x)
        else:
            h = self._norm(x, delta, self.w.final_norm, self.w.final_norm_b)
        if b.all_decode and b.logit_rows.numel() == h.shape[0]:
            hs = h                     # every row is a decode row: no gather needed
        else:
            hs = ops.gather_rows(h, b.logit_rows)
        if self.capture_hidden:
            self.last_hidden = hs                  # [logit rows, hidden]: the embeddings API reads it
        lg = ops.linear(hs, self.w.lm_head, self.w.lm_head_b)
        if cfg.logit_softcap > 0:
            lg = ops.softcap_(lg, cfg.logit_softcap)
        return lg

    def forward(self, b: StepBatch) -> torch.Tensor:
        if self.fused_tp:
            return self.forward_fused(b)
        x, delta = self.forward_hidden(b)
        return self.logits(x, delta, b)

    # ------------------------------------------------------------------ heads
    def greedy_tokens(self, logits_local: torch.Tensor) -> torch.Tensor:
        """Greedy token per row. With a vocabulary-parallel head only (value, index) pairs
        travel between ranks, never the logits
        (cf. rust/engine/src/parallel/decoder_shard.rs:546-585)."""
        tp = self.tp
        if tp is None or tp.size == 1:
            return self.ops.argmax(logits_local[:, : self.w.vocab_local] if logits_local.shape[1] != self.w.vocab_local else logits_local)
        view = logits_local[:, : max(self.w.vocab_local, 1)]
        _, pair = self.ops.argmax(view, id_offset=self.w.vocab_start, want_pairs=True)     # [R, 2] (value, id)
        if self.w.vocab_local == 0:
            pair[:, 0] = float("-inf")
        allp = tp.all_gather(pair)                                       # [tp, R, 2]; ids < 2^24 fit fp32 exactly
        # ties between ranks resolve to the lowest rank = lowest token id, like a global argmax
        return self.ops.argmax_pairs_select(allp)

    def full_logits(self, logits_local: torch.Tensor) -> torch.Tensor:
        tp = self.tp
        if tp is None or tp.size == 1:
            return logits_local[:, : self.cfg.vocab_size]
        allp = tp.all_gather(logits_local.contiguous())                  # [tp, R, chunk]
        return allp.permute(1, 0, 2).reshape(logits_local.shape[0], -1)[:, : self.cfg.vocab_size]
