"""Recurrent token mixers: the fp32 PyTorch statement of each op (``RecurrentRef``, mixed into the reference ops)
and the wrappers of the sm_100a kernels (``RecurrentNative``, mixed into the native ops).

Ops and their reference counterparts: depthwise causal convolution (rust/engine/cuda/shortconv.cu and the
convolution halves of mamba1.cu / mamba2.cu / deltanet.cu), Mamba-1 and Mamba-2 selective scans
(rust/engine/cuda/mamba1.cu, mamba2.cu), the matrix-state recurrences of RWKV-6 / RWKV-7 (rust/engine/cuda/rwkv.cu),
the gated delta rule (deltanet.cu) and its per-channel-decay form (kda.cu), and the gated RMSNorm after a scan.

Every op works on a ragged batch: ``q_starts`` [B + 1] (first token row of each sequence), ``seq_state`` [B] (row of
the state pool) and ``positions`` [T]; a sequence whose first token of the step sits at position 0 starts from zeros.
States are updated in place.
"""
from __future__ import annotations

import math
from typing import Optional

import torch
import torch.nn.functional as F

RWKV6, RWKV7, GATED_DELTA, KDA = 0, 1, 2, 3
# Mamba-2 prompt chunks from this many tokens on take the matrix form (``ssd_chunked``) instead of the token walk; 0 = never.
# Off by default: as a chain of PyTorch operators (about 40 launches per layer and sequence over [chunks, heads, 128, 128]
# tensors) it measured slower than the sequence-parallel scan kernel on a B200 (Mamba-2 2.7B prefill 15.3 k against
# 16.6 k tok/s); it is kept as the tested statement of the algorithm a fused kernel would implement.
SSD_MIN_TOKENS = int(__import__("os").environ.get("FLLM_SSD_MIN_TOKENS", "0"))
# Tokens per segment of the sequence-parallel Mamba scans (0: always one walk per sequence).
SCAN_SEG_LEN = int(__import__("os").environ.get("FLLM_SCAN_SEG_LEN", "128"))


def _seqs(q_starts, seq_state, positions):
    qs = q_starts.tolist()
    slots = seq_state.tolist()
    for s in range(len(slots)):
        t0, t1 = qs[s], qs[s + 1]
        if t1 > t0:
            yield t0, t1, slots[s], int(positions[t0]) == 0


def ssd_chunked(x, dt, Bm, Cm, A, D, dt_bias, h0, H, P, G, N, dt_min=0.0, dt_max=float("inf"), chunk=128):
    """One sequence of the Mamba-2 recurrence in its matrix form (the state-space duality of the Mamba-2 paper): inside
    chunks of ``chunk`` tokens the outputs are (C B^T masked by the decay between the two positions) X, a chunk hands
    B^T (decay to the chunk's end * X) to the next one, and the carried state enters each chunk through C. All of it is
    batched matrix products (tensor cores through the library GEMM on a GPU) instead of a walk over the tokens; the
    reference gets the same effect with its chunk-parallel scan (rust/engine/cuda/scan.cu, 64-token chunks).

    x [n, H*P], dt [n, H] (raw), Bm / Cm [n, G*N], h0 [H, P, N] fp32 or None. Returns (y [n, H*P] in x's type, final
    state [H, P, N] fp32)."""
    n = x.shape[0]
    r = H // G
    dev = x.device
    dtf = F.softplus(dt.float() + (dt_bias.float() if dt_bias is not None else 0.0)).clamp(dt_min, dt_max)     # [n, H]
    xf = x.float().view(n, H, P)
    Xd = xf * dtf[:, :, None]
    Ad = dtf * A.float()                                                     # [n, H], log decay per step (negative)
    Bf, Cf = Bm.float().view(n, G, N), Cm.float().view(n, G, N)
    pad = (-n) % chunk
    if pad:                                                                   # zero steps: decay 1, no input
        Xd = F.pad(Xd, (0, 0, 0, 0, 0, pad))
        Ad = F.pad(Ad, (0, 0, 0, pad))
        Bf, Cf = F.pad(Bf, (0, 0, 0, 0, 0, pad)), F.pad(Cf, (0, 0, 0, 0, 0, pad))
    c, Q = (n + pad) // chunk, chunk
    Xc = Xd.view(c, Q, G, r, P)
    Bc, Cc = Bf.view(c, Q, G, N), Cf.view(c, Q, G, N)
    Acs = torch.cumsum(Ad.view(c, Q, G, r), 1)                                # [c, Q, G, r] log decay from the chunk start
    # inside a chunk: y[l] += sum_{s <= l} (C[l] . B[s]) exp(Acs[l] - Acs[s]) X[s]
    CB = torch.einsum("clgn,csgn->cgls", Cc, Bc)                              # [c, G, Q, Q]
    diff = Acs.permute(0, 2, 3, 1)[..., :, None] - Acs.permute(0, 2, 3, 1)[..., None, :]        # [c, G, r, Q(l), Q(s)]
    tril = torch.ones(Q, Q, dtype=torch.bool, device=dev).tril()
    M = torch.exp(diff.masked_fill(~tril, float("-inf"))) * CB[:, :, None]
    Y = torch.matmul(M, Xc.permute(0, 2, 3, 1, 4))                            # [c, G, r, Q, P]
    # what a chunk adds to the state: sum_l B[l] (decay from l to the chunk end) X[l]
    to_end = torch.exp(Acs[:, -1:, :, :] - Acs)                               # [c, Q, G, r]
    add = torch.einsum("clgrp,clgn->cgrpn", Xc * to_end[..., None], Bc)       # [c, G, r, P, N]
    chunk_decay = torch.exp(Acs[:, -1])                                        # [c, G, r]
    h = h0.float().view(G, r, P, N) if h0 is not None else torch.zeros(G, r, P, N, dtype=torch.float32, device=dev)
    starts = []
    for ci in range(c):                                                        # the carried state: c short steps
        starts.append(h)
        h = h * chunk_decay[ci, :, :, None, None] + add[ci]
    S0 = torch.stack(starts)                                                   # [c, G, r, P, N] state entering each chunk
    Y = Y + torch.einsum("clgn,cgrpn->cgrlp", Cc, S0) * torch.exp(Acs).permute(0, 2, 3, 1)[..., None]
    y = Y.permute(0, 3, 1, 2, 4).reshape(c * Q, H, P)[:n]
    if D is not None:
        y = y + D.float()[:, None] * xf
    return y.reshape(n, H * P).to(x.dtype), h.reshape(H, P, N)


class RecurrentRef:
    def causal_conv1d(self, x, w, bias, state, q_starts, seq_state, positions, act=True, max_q_len=0):
        """y[t, c] = act(bias[c] + sum_j w[c, j] * x[t - (W - 1) + j, c]) inside each sequence; the W - 1 inputs before
        the step come from ``state`` [slots, W - 1, C], which ends up holding the last W - 1 inputs."""
        W = w.shape[1]
        y = torch.empty_like(x)
        for t0, t1, slot, fresh in _seqs(q_starts, seq_state, positions):
            hist = torch.zeros(W - 1, x.shape[1], dtype=torch.float32, device=x.device) if fresh else state[slot].float()
            full = torch.cat([hist, x[t0:t1].float()], 0)                      # [n + W - 1, C]
            acc = torch.zeros(t1 - t0, x.shape[1], dtype=torch.float32, device=x.device)
            for j in range(W):
                acc += full[j:j + t1 - t0] * w[:, j].float()
            if bias is not None:
                acc += bias.float()
            y[t0:t1] = (F.silu(acc) if act else acc).to(x.dtype)
            state[slot] = full[-(W - 1):].to(state.dtype)
        return y

    def mamba2_scan(self, x, dt, Bm, Cm, A, D, dt_bias, state, q_starts, seq_state, positions, H, P, G, N,
                    dt_min=0.0, dt_max=float("inf"), max_q_len=0, seg_len=None, host_seqs=None):
        """h = exp(dt A) h + dt x (x) B;  y = h C + D x per head; dt = clamp(softplus(dt + dt_bias))."""
        y = torch.empty_like(x)
        rep = H // G
        for t0, t1, slot, fresh in _seqs(q_starts, seq_state, positions):
            h = torch.zeros(H, P, N, dtype=torch.float32, device=x.device) if fresh else state[slot].clone()
            for t in range(t0, t1):
                d = F.softplus(dt[t].float() + (dt_bias if dt_bias is not None else 0.0)).clamp(dt_min, dt_max)      # [H]
                xv = x[t].float().view(H, P)
                Bv = Bm[t].float().view(G, N).repeat_interleave(rep, 0)
                Cv = Cm[t].float().view(G, N).repeat_interleave(rep, 0)
                h = h * torch.exp(d * A.float())[:, None, None] + (d[:, None] * xv)[:, :, None] * Bv[:, None, :]
                out = (h * Cv[:, None, :]).sum(-1)
                if D is not None:
                    out = out + D.float()[:, None] * xv
                y[t] = out.reshape(-1).to(x.dtype)
            state[slot] = h
        return y

    def mamba1_scan(self, x, dt, Bm, Cm, z, A, D, dt_bias, state, q_starts, seq_state, positions, max_q_len=0, seg_len=None):
        """h[d, n] = exp(dt[d] A[d, n]) h + dt[d] B[n] x[d];  y = (h C + D x) * silu(z)."""
        y = torch.empty_like(x)
        for t0, t1, slot, fresh in _seqs(q_starts, seq_state, positions):
            h = torch.zeros_like(state[slot]) if fresh else state[slot].clone()
            for t in range(t0, t1):
                d = F.softplus(dt[t].float() + (dt_bias if dt_bias is not None else 0.0))                          # [Dm]
                xv = x[t].float()
                h = h * torch.exp(d[:, None] * A.float()) + (d * xv)[:, None] * Bm[t].float()[None, :]
                out = (h * Cm[t].float()[None, :]).sum(-1)
                if D is not None:
                    out = out + D.float() * xv
                if z is not None:
                    out = out * F.silu(z[t].float())
                y[t] = out.to(x.dtype)
            state[slot] = h
        return y

    def matrix_state_scan(self, kind, r, k, v, a, b, w, u, beta, state, q_starts, seq_state, positions, H, DK, DV,
                          kv_ratio=1, l2norm=False, q_scale=1.0, gate_raw=None, gate_A=None, gate_dt_bias=None):
        """State S[v, k] per head; ``w`` holds log decays (fp32). See the kinds at the top of the module:
        RWKV-6  y = sum_k r (u k v + S), S = S d + k v;  RWKV-7  sa = S a, S = S d + sa b + v k, y = S r;
        delta rules  S = S d, m = S k, S += (v - m) beta k, y = S q * q_scale (q, k L2-normalised when asked)."""
        if w is None:            # gated delta rule with raw gates: step size and decay from their logits
            beta = torch.sigmoid(beta.float())
            w = gate_A.float() * F.softplus(gate_raw.float() + gate_dt_bias.float())
        y = torch.empty(r.shape[0], H * DV, dtype=r.dtype, device=r.device)
        for t0, t1, slot, fresh in _seqs(q_starts, seq_state, positions):
            S = torch.zeros(H, DV, DK, dtype=torch.float32, device=r.device) if fresh else state[slot].clone()
            for t in range(t0, t1):
                rv = r[t].float().view(-1, DK).repeat_interleave(kv_ratio, 0)                                   # [H, DK]
                kv = k[t].float().view(-1, DK).repeat_interleave(kv_ratio, 0)
                vv = v[t].float().view(H, DV)
                if kind == GATED_DELTA:
                    d = torch.exp(w[t].float())[:, None].expand(H, DK)
                else:
                    d = torch.exp(w[t].float().view(-1, DK)).repeat_interleave(kv_ratio, 0)
                if kind == RWKV6:
                    uu = u.float().view(-1, DK).repeat_interleave(kv_ratio, 0)
                    kvm = vv[:, :, None] * kv[:, None, :]
                    out = ((uu[:, None, :] * kvm + S) * rv[:, None, :]).sum(-1)
                    S = S * d[:, None, :] + kvm
                elif kind == RWKV7:
                    av = a[t].float().view(-1, DK).repeat_interleave(kv_ratio, 0)
                    bv = b[t].float().view(-1, DK).repeat_interleave(kv_ratio, 0)
                    sa = (S * av[:, None, :]).sum(-1)
                    S = S * d[:, None, :] + sa[:, :, None] * bv[:, None, :] + vv[:, :, None] * kv[:, None, :]
                    out = (S * rv[:, None, :]).sum(-1)
                else:
                    qs = torch.full((H, 1), float(q_scale), device=r.device)
                    if l2norm:
                        qs = qs * torch.rsqrt((rv * rv).sum(-1, keepdim=True) + 1e-6)
                        kv = kv * torch.rsqrt((kv * kv).sum(-1, keepdim=True) + 1e-6)
                    S = S * d[:, None, :]
                    m = (S * kv[:, None, :]).sum(-1)
                    delta = (vv - m) * beta[t].float()[:, None]
                    S = S + delta[:, :, None] * kv[:, None, :]
                    out = (S * rv[:, None, :]).sum(-1) * qs
                y[t] = out.reshape(-1).to(r.dtype)
            state[slot] = S
        return y

    def gated_rmsnorm(self, x, z, w, eps, group_size=0, norm_before_gate=False):
        """Mamba-2: rmsnorm(x * silu(z)) * w over groups; gated delta net: rmsnorm(x) * w * silu(z) (norm first).
        ``w`` may be shorter than the row (one weight vector per head): it repeats."""
        T, D = x.shape
        gs = group_size or D
        xf = x.float()
        gate = F.silu(z.float()) if z is not None else None
        if gate is not None and not norm_before_gate:
            xf = xf * gate
        xg = xf.view(T, D // gs, gs)
        xg = xg * torch.rsqrt(xg.pow(2).mean(-1, keepdim=True) + eps)
        wf = w.float().repeat(D // w.numel())
        out = xg.reshape(T, D) * wf
        if gate is not None and norm_before_gate:
            out = out * gate
        return out.to(x.dtype)


    def mla_prepare(self, ckv, q, rope_offset, positions, slots, inv_freq, attn_factor, norm_w, eps, cache):
        """Latent attention, per token: RMSNorm of the latent part of ``ckv`` [T, R + dr] and rotation of its last dr
        values (neighbouring pairs) into cache row ``slots[t]`` (negative: no write); returns the rotated rotary part
        of every head of ``q`` [T, H, head] as [T, H, dr]."""
        dr = 2 * inv_freq.numel()
        R = cache.shape[-1] - dr
        ang = positions[:ckv.shape[0]].float()[:, None] * inv_freq[None, :]
        cos, sin = torch.cos(ang) * attn_factor, torch.sin(ang) * attn_factor

        def rot(x):                                   # [T, ..., dr]
            xf = x.float().unflatten(-1, (-1, 2))
            a, b = xf[..., 0], xf[..., 1]
            c, s_ = cos, sin
            while c.dim() < a.dim():
                c, s_ = c.unsqueeze(1), s_.unsqueeze(1)
            return torch.stack([a * c - b * s_, a * s_ + b * c], -1).flatten(-2)
        lat = ckv[:, :R].float()
        lat = lat * torch.rsqrt(lat.pow(2).mean(-1, keepdim=True) + eps) * norm_w.float()
        row = torch.cat([lat, rot(ckv[:, R:R + dr])], -1).to(cache.dtype)
        keep = slots[:ckv.shape[0]] >= 0
        cache.view(-1, R + dr)[slots[:ckv.shape[0]][keep].long()] = row[keep]
        return rot(q[:, :, rope_offset:rope_offset + dr]).to(q.dtype)

    def attention_mla(self, q_abs, q_pe, cache, block_tables, row_seq, positions, scale, max_kv_len=0, tensor_cores=True, splits=None):
        """Latent attention: absorbed queries ``q_abs`` [H, T, R] and rotated parts ``q_pe`` [T, H, dr] against cache rows
        [blocks, block_size, R + dr]; the values are the first R entries of the same rows. Returns [H, T, R]."""
        H, T, R = q_abs.shape
        W = cache.shape[-1]
        bs = cache.shape[1]
        out = torch.empty(H, T, R, dtype=q_abs.dtype, device=q_abs.device)
        for t in range(T):
            n = int(positions[t]) + 1
            nblk = (n + bs - 1) // bs
            rows = cache[block_tables[int(row_seq[t]), :nblk].long()].reshape(nblk * bs, W)[:n].float()
            qt = torch.cat([q_abs[:, t].float(), q_pe[t].float()], -1)
            p = torch.softmax(qt @ rows.T * scale, -1)
            out[:, t] = (p @ rows[:, :R]).to(out.dtype)
        return out


class RecurrentNative:
    """Kernel wrappers; ``self.k`` is the loaded extension and ``self.launches`` the launch counter of the ops object."""

    def causal_conv1d(self, x, w, bias, state, q_starts, seq_state, positions, act=True, max_q_len=0):
        y = torch.empty(x.shape, dtype=x.dtype, device=x.device)
        self.k.causal_conv1d(x, w, bias, state, q_starts, seq_state, positions, y, bool(act), int(max_q_len))   # 0: bounded by the rows
        self.launches += 1
        return y

    def mamba2_scan(self, x, dt, Bm, Cm, A, D, dt_bias, state, q_starts, seq_state, positions, H, P, G, N,
                    dt_min=0.0, dt_max=float("inf"), max_q_len=0, seg_len=None, host_seqs=None):
        """``max_q_len`` (host-side bound on the tokens of a sequence in this step) lets long prompts of few sequences run
        sequence-parallel: segments of ``seg_len`` tokens side by side, a short combine pass, then the outputs.
        ``host_seqs`` (the step's sequences as (first row, rows, state row, fresh) known on the host) sends prompt chunks
        of ``SSD_MIN_TOKENS`` tokens or more through the matrix form (``ssd_chunked``: batched matrix products on tensor
        cores); the scan kernel then leaves those sequences alone."""
        y = torch.empty(x.shape, dtype=x.dtype, device=x.device)
        B = seq_state.numel()
        skip = 0
        if host_seqs:
            long = [q for q in host_seqs if SSD_MIN_TOKENS and q[1] >= SSD_MIN_TOKENS]
            for t0, n, slot, fresh in long:
                yv, hf = ssd_chunked(x[t0:t0 + n], dt[t0:t0 + n], Bm[t0:t0 + n], Cm[t0:t0 + n], A, D, dt_bias,
                                     None if fresh else state[slot], H, P, G, N, dt_min, min(dt_max, 3.0e38))
                y[t0:t0 + n] = yv
                state[slot] = hf
            if long:
                if len(long) == len(host_seqs):
                    return y
                skip, max_q_len = SSD_MIN_TOKENS, SSD_MIN_TOKENS - 1
        if seg_len is None:
            # CTAs that walk long sequences (a mixed step's decode rows finish at once and do not fill the GPU)
            ctas = max(1, min(B, x.shape[0] // 256)) * H * max(1, P * max(N // 16, 1) // 128)
            seg_len = SCAN_SEG_LEN if (max_q_len >= 512 and ctas < 4 * 148) else 0
        segs = -(-int(max_q_len) // seg_len) if seg_len else 1
        scratch = None
        if segs > 1:
            need = B * (segs * H * P * N + (segs - 1) * H)
            scratch = getattr(self, "_scan_scratch", None)
            if scratch is None or scratch.numel() < need:
                scratch = self._scan_scratch = torch.empty(need, dtype=torch.float32, device=x.device)
        self.k.mamba2_scan(x, dt, Bm, Cm, A, D, dt_bias, state, q_starts, seq_state, positions, y, H, P, G, N,
                           float(dt_min), float(min(dt_max, 3.0e38)), int(seg_len if segs > 1 else 0), int(segs), scratch, int(skip))
        self.launches += 3 if segs > 1 else 1
        return y

    def mamba1_scan(self, x, dt, Bm, Cm, z, A, D, dt_bias, state, q_starts, seq_state, positions, max_q_len=0, seg_len=None):
        """Long prompts of few sequences run sequence-parallel (``max_q_len``: host-side bound on a sequence's tokens in the step)."""
        y = torch.empty(x.shape, dtype=x.dtype, device=x.device)
        B, Dm, N = seq_state.numel(), x.shape[1], A.shape[1]
        if seg_len is None:
            ctas = max(1, min(B, x.shape[0] // 256)) * ((Dm + 127) // 128)          # those that walk long sequences
            seg_len = SCAN_SEG_LEN if (max_q_len >= 512 and ctas < 4 * 148) else 0
        segs = -(-int(max_q_len) // seg_len) if seg_len else 1
        scratch = None
        if segs > 1:
            need = B * Dm * (segs * N + segs - 1)
            scratch = getattr(self, "_scan_scratch", None)
            if scratch is None or scratch.numel() < need:
                scratch = self._scan_scratch = torch.empty(need, dtype=torch.float32, device=x.device)
        self.k.mamba1_scan(x, dt, Bm, Cm, z, A, D, dt_bias, state, q_starts, seq_state, positions, y,
                           int(seg_len if segs > 1 else 0), int(segs), scratch)
        self.launches += 3 if segs > 1 else 1
        return y

    def matrix_state_scan(self, kind, r, k, v, a, b, w, u, beta, state, q_starts, seq_state, positions, H, DK, DV,
                          kv_ratio=1, l2norm=False, q_scale=1.0, gate_raw=None, gate_A=None, gate_dt_bias=None):
        y = torch.empty(r.shape[0], H * DV, dtype=r.dtype, device=r.device)
        self.k.matrix_state_scan(int(kind), r, k, v, a, b, w, u, beta, state, q_starts, seq_state, positions, y, H, DK,
                                 DV, int(kv_ratio), bool(l2norm), float(q_scale), gate_raw, gate_A, gate_dt_bias)
        self.launches += 1
        return y

    def gated_rmsnorm(self, x, z, w, eps, group_size=0, norm_before_gate=False):
        y = torch.empty(x.shape, dtype=x.dtype, device=x.device)
        self.k.gated_rmsnorm(x, z, w, y, int(group_size or x.shape[1]), float(eps), bool(norm_before_gate))
        self.launches += 1
        return y

    def mla_prepare(self, ckv, q, rope_offset, positions, slots, inv_freq, attn_factor, norm_w, eps, cache):
        if cache.shape[-1] != 576 or inv_freq.numel() != 32:      # the kernels are built for the 512 + 64 rows of the DeepSeek family
            return RecurrentRef.mla_prepare(self, ckv, q, rope_offset, positions, slots, inv_freq, attn_factor, norm_w, eps, cache)
        q_pe = torch.empty(q.shape[0], q.shape[1], 64, dtype=q.dtype, device=q.device)
        self.k.mla_prepare(ckv, q, int(rope_offset), positions, slots, inv_freq, float(attn_factor), norm_w, float(eps), cache, q_pe)
        self.launches += 1
        return q_pe

    def attention_mla(self, q_abs, q_pe, cache, block_tables, row_seq, positions, scale, max_kv_len=0, tensor_cores=True, splits=None):
        """``max_kv_len`` (host-side bound on the context of the step's rows) sizes the split over key slices."""
        if cache.shape[-1] != 576 or q_abs.shape[-1] != 512:
            return RecurrentRef.attention_mla(self, q_abs, q_pe, cache, block_tables, row_seq, positions, scale)
        H, T = q_abs.shape[0], q_abs.shape[1]
        out = torch.empty(q_abs.shape, dtype=q_abs.dtype, device=q_abs.device)
        if not tensor_cores:
            self.k.attention_mla(q_abs, q_pe, cache, block_tables, row_seq, positions, out, True, float(scale), 0, None)
            self.launches += 1
            return out
        if splits is None:
            splits = int(self.k.attention_mla_splits(T, H, int(max_kv_len))) if max_kv_len else 1
        ws = None
        if splits > 1:
            need = int(self.k.attention_mla_workspace_bytes(T, H, splits))
            ws = getattr(self, "_mla_ws", None)
            if ws is None or ws.numel() < need:           # grow-only; the warm-up before a graph capture sizes it
                ws = self._mla_ws = torch.empty(need, dtype=torch.uint8, device=q_abs.device)
        self.k.attention_mla(q_abs, q_pe, cache, block_tables, row_seq, positions, out, True, float(scale), int(splits), ws)
        self.launches += 2 if splits > 1 else 1
        return out
