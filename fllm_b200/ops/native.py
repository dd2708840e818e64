"""Python face of the sm_100a kernels (``torch.ops.fllm_b200``).

Every method mirrors :class:`fllm_b200.ops.reference.RefOps`; the model runner is
written once against this interface. There is no fallback inside this class: if
the library is missing the constructor raises.
"""
from __future__ import annotations

import struct
from typing import Optional

import torch

from ._lib import load_cuda
from .recurrent import RecurrentNative


class Deferred:
    """Handle to a projection whose split-K reduction was left to its consumer: the fp32 partial sums
    [splits][rows][cols] sit in the operator workspace (bias not added) until the next ``linear`` call.
    ``rmsnorm``, ``rope_kv_write`` and the gated activation accept it in place of a tensor and add the
    partials while they read them, which removes the reduction kernel from the chain."""
    __slots__ = ("splits", "rows", "cols", "bias")

    def __init__(self, splits: int, rows: int, cols: int, bias):
        self.splits, self.rows, self.cols, self.bias = splits, rows, cols, bias

    @property
    def shape(self):
        return (self.rows, self.cols)


class NativeOps(RecurrentNative):
    name = "sm100a"

    def __init__(self, device: torch.device, workspace_bytes: int = 96 << 20):
        self.k = load_cuda()
        self.device = torch.device(device)
        # first 64 KiB = split-K tile counters (must start at zero; the kernels re-zero them)
        self.workspace = torch.zeros(workspace_bytes, dtype=torch.uint8, device=self.device)
        self.status = torch.zeros(1, dtype=torch.int32, device=self.device)
        self.use_tc_attention = True
        self.attn_ws = None
        self.launches = 0            # kernels launched through this object (graph capture included)
        self._scratch = None
        self._argmax_ws = None

    def scratch_bf16(self, numel: int) -> torch.Tensor:
        """Grow-only bf16 scratch (expanded weights of packed formats during prefill). Stream-ordered
        reuse: the dense GEMM that reads it is queued before the next expansion overwrites it."""
        if self._scratch is None or self._scratch.numel() < numel:
            self._scratch = torch.empty(numel, dtype=torch.bfloat16, device=self.device)
        return self._scratch[:numel]

    # ---------------------------------------------------------------- dense
    def linear(self, x, w, bias=None, out=None, force_splits: int = 0, defer: bool = False):
        """y = x @ w^T (+ bias). With ``defer`` the call may return a :class:`Deferred` instead of a tensor
        (when the kernel picked split-K): pass it on to ``rmsnorm`` / ``rope_kv_write``."""
        if not isinstance(w, torch.Tensor):          # packed weight (FP8 block, FP4, ...): it knows its kernel
            return w.apply(self, x, bias, out)
        if out is None:
            out = torch.empty(x.shape[0], w.shape[0], dtype=x.dtype, device=x.device)
        if not defer:
            self.launches += self.k.linear(x, w, bias, out, self.workspace, self.status, force_splits)
            return out
        n, splits = self.k.linear_ex(x, w, bias, out, self.workspace, self.status, force_splits, 0, 16, 0.0, 0.0, True)
        self.launches += n
        return Deferred(splits, x.shape[0], w.shape[0], bias) if splits > 1 else out

    def materialize(self, y):
        """Tensor value of a projection result (adds a Deferred's partials with the stand-alone path)."""
        if not isinstance(y, Deferred):
            return y
        raise RuntimeError("a deferred projection can only be consumed by rmsnorm, rope_kv_write or a gated activation")

    def linear_glu(self, x, w, bias, act_kind=0, alpha=1.702, limit=7.0, layout=0, force_splits: int = 0):
        """act(x @ w^T + bias) for a fused gate|up weight, [T, N/2]. With a row layout the GEMM epilogue can
        pair up (blocks of 16, or the pairs of the clamped SwiGLU-OAI kind) the activation runs inside the GEMM;
        when the GEMM needs split-K the activation kernel adds the partial sums instead."""
        T, N = x.shape[0], w.shape[0]
        pd = 16 if layout == 16 else (1 if act_kind == 2 else 0)
        if not isinstance(w, torch.Tensor) or pd == 0 or N % 32:
            return self.glu(self.linear(x, w, bias), act_kind, alpha, limit, layout)
        out = torch.empty(T, N // 2, dtype=x.dtype, device=x.device)
        n, splits = self.k.linear_ex(x, w, bias, out, self.workspace, self.status, force_splits, act_kind + 1, pd,
                                     float(alpha), float(limit), True)
        self.launches += n
        if splits > 1:
            self.k.glu_ex(None, out, act_kind, float(alpha), float(limit), layout, self.workspace, splits, bias)
            self.launches += 1
        return out

    def embed(self, ids, table, scale=1.0):
        out = torch.empty(ids.numel(), table.shape[1], dtype=table.dtype, device=table.device)
        self.k.embed(ids, table, out, float(scale))
        self.launches += 1
        return out

    def rmsnorm(self, residual, delta, w, eps, w_offset=0.0):
        y = torch.empty_like(residual)
        if isinstance(delta, Deferred):
            self.k.rmsnorm_splitk(residual, self.workspace, delta.splits, delta.bias, w, y, float(eps), float(w_offset))
        else:
            self.k.rmsnorm(residual, delta, w, y, float(eps), float(w_offset))
        self.launches += 1
        return y

    def rope_kv_write(self, qkv, positions, slots, inv_freq, q_norm_w, k_norm_w, k_cache, v_cache,
                      hq, hkv, head_dim, rot_dim, rope_style, eps, attn_factor=1.0):
        """QK-norm + RoPE + paged KV write; returns the rotated queries [T, hq * head_dim]."""
        self.launches += 1
        if isinstance(qkv, Deferred):
            q = torch.empty(qkv.rows, hq * head_dim, dtype=torch.bfloat16, device=self.device)
            self.k.rope_kv_write_splitk(self.workspace, qkv.splits, qkv.bias, q, positions, slots, inv_freq, q_norm_w,
                                        k_norm_w, k_cache, v_cache, hq, hkv, head_dim, rot_dim, rope_style,
                                        float(eps), float(attn_factor))
            return q
        self.k.rope_kv_write(qkv, positions, slots, inv_freq, q_norm_w, k_norm_w, k_cache, v_cache,
                             hq, hkv, head_dim, rot_dim, rope_style, float(eps), float(attn_factor))
        return qkv[:, : hq * head_dim]

    def glu(self, x, act_kind=0, alpha=1.702, limit=7.0, layout=0):
        out = torch.empty(x.shape[0], x.shape[1] // 2, dtype=x.dtype, device=x.device)
        if layout:
            self.k.glu_ex(x, out, act_kind, float(alpha), float(limit), layout, None, 0, None)
        else:
            self.k.glu(x, out, act_kind, float(alpha), float(limit))
        self.launches += 1
        return out

    def gather_rows(self, x, rows):
        out = torch.empty(rows.numel(), x.shape[1], dtype=x.dtype, device=x.device)
        self.k.gather_rows(x, rows, out)
        self.launches += 1
        return out

    # ---------------------------------------------------------------- attention
    def attention(self, q, k_cache, v_cache, block_tables, row_seq, positions, hq, hkv, head_dim,
                  scale, window=0, sinks=None, softcap=0.0, meta=None, bidirectional=False):
        """bidirectional: no causal mask (encoders); `positions` must then hold the last position of each row's
        sequence (the generic kernel's visibility limit), the tensor-core kernels take the flag."""
        out = torch.empty(q.shape[0], hq * head_dim, dtype=q.dtype, device=q.device)
        kv8 = k_cache.element_size() == 1
        if (self.use_tc_attention and meta is not None and meta.q_starts is not None
                and head_dim in (64, 128) and hq // hkv <= 16
                and (not kv8 or (meta.max_q_len * (hq // hkv) <= 16 and not bidirectional))):
            # (an e4m3 KV cache: decode-shaped batches run the tensor-core decode kernel, which widens the pages to
            # f16 in shared memory; batches with prefill chunks fall through to the generic kernel)
            if self.attn_ws is None:
                self.attn_ws = torch.empty(64 << 20, dtype=torch.uint8, device=self.device)
            self.launches += self.k.attention_tc(
                q, k_cache, v_cache, block_tables, meta.q_starts, meta.seq_lens, out, meta.num_seqs,
                meta.max_q_len, meta.min_q_len, meta.max_kv_len, hq, hkv, head_dim, float(scale),
                int(window), sinks, float(softcap), self.attn_ws, self.status, bool(bidirectional))
            return out
        self.k.attention_generic(q, k_cache, v_cache, block_tables, row_seq, positions, out, hq, hkv,
                                 head_dim, float(scale), int(window), sinks, float(softcap))
        self.launches += 1
        return out

    def layernorm(self, residual, delta, w, b, eps, w_offset=0.0):
        """LayerNorm(residual (+= delta)) * (w + w_offset) + b in one kernel."""
        delta = self.materialize(delta) if delta is not None else None
        out = torch.empty_like(residual)
        self.k.add_layernorm(residual, delta, w, b, out, float(eps), float(w_offset))
        self.launches += 1
        return out

    ACTS = {"gelu": 0, "gelu_tanh": 1, "relu2": 2, "silu": 3, "relu": 4}

    def act_(self, x, kind: str):
        self.k.act_(x, self.ACTS[kind])
        self.launches += 1
        return x

    def softcap_(self, x, cap: float):
        """x = cap * tanh(x / cap) in place (final-logit soft-cap)."""
        self.k.softcap_(x, float(cap))
        self.launches += 1
        return x

    def attention_tree(self, q, k_cache, v_cache, block_tables, row_seq, positions, tree_mask, tree_base, hq, hkv,
                       head_dim, scale, window=0, sinks=None, softcap=0.0):
        """Attention for the nodes of draft trees: row t sees the first tree_base[t] tokens of its sequence and the
        tree nodes whose bit is set in tree_mask[t] (int64, bit i = node i, stored at position tree_base[t] + i);
        positions[t] = tree_base[t] + nodes - 1."""
        out = torch.empty(q.shape[0], hq * head_dim, dtype=q.dtype, device=q.device)
        self.k.attention_generic(q, k_cache, v_cache, block_tables, row_seq, positions, out, hq, hkv, head_dim,
                                 float(scale), int(window), sinks, float(softcap), tree_mask, tree_base)
        self.launches += 1
        return out

    # ---------------------------------------------------------------- sampling
    def argmax(self, logits, id_offset=0, want_vals=False, want_pairs=False):
        """Greedy id per row (lowest index among equal maxima). want_pairs: also [rows, 2] fp32
        (value, float(id)), the message a vocabulary-parallel head exchanges."""
        rows = logits.shape[0]
        ids = torch.empty(rows, dtype=torch.int32, device=logits.device)
        vals = torch.empty(rows, dtype=torch.float32, device=logits.device) if want_vals else None
        pairs = torch.empty(rows, 2, dtype=torch.float32, device=logits.device) if want_pairs else None
        if rows <= 1024:
            if self._argmax_ws is None:     # [row counters (zero between launches) | per-slice (value, index)]
                self._argmax_ws = torch.zeros(1024 * 4 + 1024 * 32 * 8 + 64, dtype=torch.uint8, device=self.device)
            self.k.argmax_split(logits, ids, vals, pairs, id_offset, self._argmax_ws)
        else:
            self.k.argmax(logits, ids, vals, id_offset)
            if want_pairs:
                pairs = torch.stack([vals if vals is not None else logits.float().max(-1).values, ids.float()], 1).contiguous()
        self.launches += 1
        if want_pairs:
            return ids, pairs
        return (ids, vals) if want_vals else ids

    def argmax_pairs_select(self, pairs):
        """[ranks, rows, 2] gathered (value, id) pairs -> winning id per row."""
        out = torch.empty(pairs.shape[1], dtype=torch.int32, device=pairs.device)
        self.k.argmax_pairs_select(pairs.contiguous(), out)
        self.launches += 1
        return out

    def sample(self, logits, params, pen_ids=None, pen_counts=None, bias_ids=None, bias_vals=None,
               allow_mask=None, want_logprobs=False):
        ids = torch.empty(logits.shape[0], dtype=torch.int32, device=logits.device)
        lp = torch.empty(logits.shape[0], dtype=torch.float32, device=logits.device) if want_logprobs else None
        self.k.sample(logits, params, pen_ids, pen_counts, bias_ids, bias_vals, allow_mask, ids, lp)
        self.launches += 1
        return (ids, lp) if want_logprobs else ids

    def spec_verify_greedy(self, draft_ids, target_ids, n_draft=None, row_start=None):
        """Greedy chain acceptance on the device. draft_ids [B, k]; target_ids [B, k+1] or, with row_start [B],
        the flat ids of a ragged step. -> (n_accept [B], out_tokens [B, k+1]: accepted drafts then the target's token)."""
        B, k = draft_ids.shape
        n_acc = torch.zeros(B, dtype=torch.int32, device=draft_ids.device)
        out = torch.full((B, k + 1), -1, dtype=torch.int32, device=draft_ids.device)
        self.k.spec_verify_greedy(draft_ids, target_ids, n_draft, n_acc, out, row_start)
        self.launches += 1
        return n_acc, out

    def spec_verify_sampled(self, target_logits, draft_logits, draft_ids, params, n_draft=None, row_start=None):
        """Exact speculative sampling on the device (accept with min(1, p/q), residual draw at the first
        rejection, bonus draw after the last acceptance). params: sampler rows (temperature, ..., draw, seed),
        one per sequence; draft_logits None = point-mass drafts."""
        B, k = draft_ids.shape
        dev = draft_ids.device
        prm = torch.frombuffer(bytearray(pack_sample_rows(params)), dtype=torch.uint8).to(dev)
        n_acc = torch.zeros(B, dtype=torch.int32, device=dev)
        out = torch.full((B, k + 1), -1, dtype=torch.int32, device=dev)
        self.k.spec_verify_sampled(target_logits, draft_logits, draft_ids, n_draft, prm, n_acc, out, row_start)
        self.launches += 1
        return n_acc, out

    def check_status(self) -> int:
        code = int(self.status.item())
        if code:
            self.status.zero_()
        return code


SAMPLE_ROW_FMT = "<6fiIQ"      # mirrors struct fllm::SampleRow (40 bytes)


def pack_sample_rows(rows) -> bytes:
    """rows: iterable of (temperature, top_p, min_p, repetition_penalty, presence_penalty,
    frequency_penalty, top_k, draw, seed)."""
    return b"".join(struct.pack(SAMPLE_ROW_FMT, *r) for r in rows)


def quantize_weight_fp8_block(w: torch.Tensor, block: int = 128):
    """bf16/fp32 [N, K] -> (e4m3 bytes [N, K] as uint8, fp32 scales [N/128, K/128]); amax / 448 per block."""
    N, K = w.shape
    wf = w.float().view(N // block, block, K // block, block)
    amax = wf.abs().amax(dim=(1, 3)).clamp_min(1e-10)
    scale = amax / 448.0
    q = (wf / scale[:, None, :, None]).to(torch.float8_e4m3fn)
    return q.view(N, K).view(torch.uint8).contiguous(), scale.contiguous()


class Fp8BlockWeight:
    """A weight stored as block-scaled e4m3 (codes [N, K] as bytes + fp32 scales per 128 x 128).
    ``ops.linear`` accepts it in place of a bf16 tensor: activations are quantised per token per
    128 values on the fly and the product runs on the FP8 tensor cores."""

    def __init__(self, wq: torch.Tensor, sw: torch.Tensor):
        self.wq, self.sw = wq, sw
        self.shape = wq.shape

    def apply(self, ops, x, bias=None, out=None):
        T, K = x.shape
        if not x.is_cuda:                                           # CPU oracle path
            wd = self.wq.view(torch.float8_e4m3fn).float().view(self.shape[0] // 128, 128, K // 128, 128) * self.sw[:, None, :, None]
            y = x.float() @ wd.view(self.shape[0], K).t()
            return (y + bias.float() if bias is not None else y).to(x.dtype)
        xq = torch.empty(T, K, dtype=torch.uint8, device=x.device)
        sx = torch.empty(T, K // 128, dtype=torch.float32, device=x.device)
        ops.k.quant_fp8_1x128(x.contiguous(), xq, sx)
        y = out if out is not None else torch.empty(T, self.shape[0], dtype=torch.bfloat16, device=x.device)
        ops.launches += 1 + ops.k.linear_fp8_block(xq, sx, self.wq, self.sw, bias, y, ops.status, ops.workspace)
        return y


class Fp8BlockLinear:
    def __init__(self, ops: NativeOps, wq: torch.Tensor, sw: torch.Tensor, bias=None):
        self.ops, self.w, self.bias = ops, Fp8BlockWeight(wq, sw), bias

    def __call__(self, x: torch.Tensor) -> torch.Tensor:
        return self.w.apply(self.ops, x, self.bias)
