"""Plain PyTorch fp32 restatement of every op. It is the numerics oracle of the
CUDA kernels and the engine's compute path on machines without a GPU (tests,
gloo-rank parallel equivalence); it is never used when a GPU is present.
"""
from __future__ import annotations

import math
from typing import Optional

import numpy as np
import torch
import torch.nn.functional as F

from .recurrent import RecurrentRef


class RefOps(RecurrentRef):
    name = "reference"

    # ---------------------------------------------------------------- dense
    def linear(self, x, w, bias=None, out=None, force_splits: int = 0, defer: bool = False):
        if not isinstance(w, torch.Tensor):
            return w.apply(self, x, bias, out)
        y = x.float() @ w.float().t()
        if bias is not None:
            y = y + bias.float()
        y = y.to(x.dtype)
        if out is not None:
            out.copy_(y)
            return out
        return y

    def linear_glu(self, x, w, bias, act_kind=0, alpha=1.702, limit=7.0, layout=0, force_splits: int = 0):
        return self.glu(self.linear(x, w, bias), act_kind, alpha, limit, layout)

    def embed(self, ids, table, scale=1.0):
        x = table[ids.long()]
        if scale != 1.0:
            x = (x.float() * scale).to(table.dtype)
        return x

    def rmsnorm(self, residual, delta, w, eps, w_offset=0.0):
        """Returns y; when delta is given, residual += delta in place first."""
        if delta is not None:
            residual.copy_((residual.float() + delta.float()).to(residual.dtype))
        x = residual.float()
        inv = torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps)
        return (x * inv * (w.float() + w_offset)).to(residual.dtype)

    # ---------------------------------------------------------------- rope + kv
    def rope_kv_write(self, qkv, positions, slots, inv_freq, q_norm_w, k_norm_w, k_cache, v_cache,
                      hq, hkv, head_dim, rot_dim, rope_style, eps, attn_factor=1.0):
        T = qkv.shape[0]
        x = qkv.float().view(T, hq + 2 * hkv, head_dim)
        q, k, v = x[:, :hq], x[:, hq:hq + hkv], x[:, hq + hkv:]

        def norm(t, w):
            if w is None:
                return t
            inv = torch.rsqrt(t.pow(2).mean(-1, keepdim=True) + eps)
            return (t * inv * w.float()).to(qkv.dtype).float()

        q, k = norm(q, q_norm_w), norm(k, k_norm_w)
        ang = positions.float()[:, None] * inv_freq.float()[None, :]      # [T, rot/2]
        cos, sin = ang.cos() * attn_factor, ang.sin() * attn_factor

        def rot(t):
            r, rest = t[..., :rot_dim], t[..., rot_dim:]
            c, s = cos[:, None, :], sin[:, None, :]
            if rope_style == 0:
                a, b = r[..., : rot_dim // 2], r[..., rot_dim // 2:]
                r2 = torch.cat([a * c - b * s, b * c + a * s], -1)
            else:
                a, b = r[..., 0::2], r[..., 1::2]
                r2 = torch.stack([a * c - b * s, b * c + a * s], -1).flatten(-2)
            return torch.cat([r2, rest], -1)

        q, k = rot(q), rot(k)
        qkv.view(T, hq + 2 * hkv, head_dim)[:, :hq] = q.to(qkv.dtype)
        if slots is not None:
            bs = k_cache.shape[2]
            ok = slots >= 0
            sl = slots[ok].long()
            blk, off = sl // bs, sl % bs
            k_cache[blk, :, off] = k[ok].to(k_cache.dtype)
            v_cache[blk, :, off] = v[ok].to(v_cache.dtype)
        return qkv[:, : hq * head_dim]

    def glu(self, x, act_kind=0, alpha=1.702, limit=7.0, layout=0):
        """layout 16: columns come in blocks of 16 gate values followed by the 16 up values of the same
        features (the order the GEMM's gated epilogue pairs up)."""
        xf = x.float()
        if layout == 16:
            blk = xf.view(x.shape[0], -1, 2, 16)
            g, u = blk[:, :, 0].reshape(x.shape[0], -1), blk[:, :, 1].reshape(x.shape[0], -1)
            if act_kind == 2:
                g = g.clamp(max=limit)
                u = u.clamp(min=-limit, max=limit)
                y = g * torch.sigmoid(alpha * g) * (u + 1)
            else:
                y = (F.silu(g) if act_kind == 0 else F.gelu(g, approximate="tanh")) * u
            return y.to(x.dtype)
        if act_kind == 2:
            g, u = xf[:, 0::2], xf[:, 1::2]
            g = g.clamp(max=limit)
            u = u.clamp(min=-limit, max=limit)
            y = g * torch.sigmoid(alpha * g) * (u + 1)
        else:
            inter = x.shape[1] // 2
            g, u = xf[:, :inter], xf[:, inter:]
            y = (F.silu(g) if act_kind == 0 else F.gelu(g, approximate="tanh")) * u
        return y.to(x.dtype)

    def gather_rows(self, x, rows):
        return x[rows.long()].contiguous()

    # ---------------------------------------------------------------- attention
    def attention(self, q, k_cache, v_cache, block_tables, row_seq, positions, hq, hkv, head_dim,
                  scale, window=0, sinks=None, softcap=0.0, meta=None, bidirectional=False):
        """`positions[t]` is the last visible token of row t: a causal decoder passes the row's own position, an
        encoder (bidirectional) the last position of the row's sequence."""
        T = q.shape[0]
        bs = k_cache.shape[2]
        out = torch.empty(T, hq * head_dim, dtype=q.dtype, device=q.device)
        qf = q.float().view(T, hq, head_dim)
        g = hq // hkv
        for t in range(T):
            seq = int(row_seq[t])
            n = int(positions[t]) + 1
            begin = max(0, n - window) if window > 0 else 0
            nblk = (n + bs - 1) // bs
            blocks = block_tables[seq, :nblk].long()
            k = k_cache[blocks].float().permute(1, 0, 2, 3).reshape(hkv, nblk * bs, head_dim)[:, begin:n]
            v = v_cache[blocks].float().permute(1, 0, 2, 3).reshape(hkv, nblk * bs, head_dim)[:, begin:n]
            k = k.repeat_interleave(g, 0)
            v = v.repeat_interleave(g, 0)
            s = torch.einsum("hd,hnd->hn", qf[t], k) * scale
            if softcap > 0:
                s = softcap * torch.tanh(s / softcap)
            if sinks is not None:
                s = torch.cat([s, sinks.float()[:, None]], 1)
                p = torch.softmax(s, -1)[:, :-1]
            else:
                p = torch.softmax(s, -1)
            out[t] = torch.einsum("hn,hnd->hd", p, v).reshape(-1).to(q.dtype)
        return out

    def materialize(self, y):
        return y

    def layernorm(self, residual, delta, w, b, eps, w_offset=0.0):
        """Returns LayerNorm(residual) * (w + w_offset) + b; when delta is given, residual += delta in place first."""
        if delta is not None:
            residual.copy_((residual.float() + delta.float()).to(residual.dtype))
        x = residual.float()
        y = F.layer_norm(x, (x.shape[-1],), w.float() + w_offset, b.float() if b is not None else None, eps)
        return y.to(residual.dtype)

    def act_(self, x, kind: str):
        """Activation of a plain MLP, in place: gelu | gelu_tanh | relu2 | silu | relu."""
        xf = x.float()
        y = {"gelu": F.gelu, "gelu_tanh": lambda t: F.gelu(t, approximate="tanh"), "relu2": lambda t: F.relu(t).square(),
             "silu": F.silu, "relu": F.relu}[kind](xf)
        x.copy_(y.to(x.dtype))
        return x

    def softcap_(self, x, cap: float):
        x.copy_((cap * torch.tanh(x.float() / cap)).to(x.dtype))
        return x

    def attention_tree(self, q, k_cache, v_cache, block_tables, row_seq, positions, tree_mask, tree_base, hq, hkv,
                       head_dim, scale, window=0, sinks=None, softcap=0.0):
        """Rows are nodes of draft trees: the context plus the ancestors named by a 64-bit mask per row."""
        T = q.shape[0]
        bs = k_cache.shape[2]
        out = torch.empty(T, hq * head_dim, dtype=q.dtype, device=q.device)
        qf = q.float().view(T, hq, head_dim)
        g = hq // hkv
        for t in range(T):
            seq, n, base, mask = int(row_seq[t]), int(positions[t]) + 1, int(tree_base[t]), int(tree_mask[t]) & ((1 << 64) - 1)
            nblk = (n + bs - 1) // bs
            blocks = block_tables[seq, :nblk].long()
            k = k_cache[blocks].float().permute(1, 0, 2, 3).reshape(hkv, nblk * bs, head_dim)[:, :n]
            v = v_cache[blocks].float().permute(1, 0, 2, 3).reshape(hkv, nblk * bs, head_dim)[:, :n]
            vis = torch.tensor([j < base or ((mask >> (j - base)) & 1) == 1 for j in range(n)], device=q.device)
            s = torch.einsum("hd,hnd->hn", qf[t], k.repeat_interleave(g, 0)) * scale
            if softcap > 0:
                s = softcap * torch.tanh(s / softcap)
            s = s.masked_fill(~vis[None, :], float("-inf"))
            if sinks is not None:
                p = torch.softmax(torch.cat([s, sinks.float()[:, None]], 1), -1)[:, :-1]
            else:
                p = torch.softmax(s, -1)
            out[t] = torch.einsum("hn,hnd->hd", p, v.repeat_interleave(g, 0)).reshape(-1).to(q.dtype)
        return out

    # ---------------------------------------------------------------- sampling
    def argmax(self, logits, id_offset=0, want_vals=False, want_pairs=False):
        vals, ids = logits.float().max(-1)
        ids = (ids + id_offset).int()
        if want_pairs:
            return ids, torch.stack([vals, ids.float()], 1).contiguous()
        return (ids, vals) if want_vals else ids

    def argmax_pairs_select(self, pairs):
        """[ranks, rows, 2] (value, id) pairs -> id of the highest value per row, lowest rank among equals."""
        best = pairs[:, :, 0].argmax(0)
        return pairs[best, torch.arange(pairs.shape[1], device=pairs.device), 1].int()


    def spec_verify_greedy(self, draft_ids, target_ids, n_draft=None, row_start=None):
        B, k = draft_ids.shape
        d = draft_ids.cpu().tolist()
        t = target_ids.cpu().flatten().tolist()
        nd = n_draft.cpu().tolist() if n_draft is not None else [k] * B
        rs = row_start.cpu().tolist() if row_start is not None else [b * (k + 1) for b in range(B)]
        n_acc = torch.zeros(B, dtype=torch.int32)
        out = torch.full((B, k + 1), -1, dtype=torch.int32)
        for b in range(B):
            acc = 0
            while acc < min(nd[b], k) and d[b][acc] == t[rs[b] + acc]:
                out[b, acc] = d[b][acc]
                acc += 1
            out[b, acc] = t[rs[b] + acc]
            n_acc[b] = acc
        return n_acc.to(draft_ids.device), out.to(draft_ids.device)

    def spec_verify_sampled(self, target_logits, draft_logits, draft_ids, params, n_draft=None, row_start=None):
        """Host statement of the device rule with the same counter-based random numbers."""
        B, k = draft_ids.shape
        tl = target_logits.float().cpu()
        dl = draft_logits.float().cpu() if draft_logits is not None else None
        d = draft_ids.cpu().tolist()
        nd = n_draft.cpu().tolist() if n_draft is not None else [k] * B
        rs = row_start.cpu().tolist() if row_start is not None else [b * (k + 1) for b in range(B)]
        V = tl.shape[1]
        idx = np.arange(V, dtype=np.uint64)
        n_acc = torch.zeros(B, dtype=torch.int32)
        out = torch.full((B, k + 1), -1, dtype=torch.int32)

        def gumbel_pick(score, seed, draw):
            u = philox_uniform_np(seed, draw, idx)
            g = score - np.log(-np.log(u))
            return int(np.argmax(np.where(np.isfinite(score), g, -np.inf)))

        for b in range(B):
            temp, draw, seed = float(params[b][0]), int(params[b][7]), int(params[b][8])
            inv_t = 1.0 / temp if temp > 0 else 1.0
            acc, final = 0, -1
            for i in range(min(nd[b], k) + 1):
                trow = tl[rs[b] + i].double().numpy()
                amax = int(np.argmax(trow))
                lt = (trow - trow[amax]) * inv_t
                pt = np.exp(lt) / np.exp(lt).sum()
                if i == min(nd[b], k):
                    final = amax if temp <= 0 else gumbel_pick(lt, seed, draw + 2 * i + 1)
                    break
                x = d[b][i]
                if dl is not None:
                    drow = dl[b * k + i].double().numpy()
                    lq = (drow - drow.max()) * inv_t
                    q = np.exp(lq) / np.exp(lq).sum()
                else:
                    q = np.zeros(V)
                    q[x] = 1.0
                if temp <= 0:
                    ok = x == amax
                else:
                    u = float(philox_uniform_np(seed, draw + 2 * i, np.array([0xFFFFFFFF], dtype=np.uint64))[0])
                    ok = True if q[x] <= 0 else u < min(1.0, pt[x] / q[x])
                if ok:
                    out[b, acc] = x
                    acc += 1
                    continue
                if temp <= 0:
                    final = amax
                    break
                r = pt - q
                with np.errstate(divide="ignore"):
                    score = np.where(r > 0, np.log(np.maximum(r, 1e-300)), -np.inf)
                final = gumbel_pick(score, seed, draw + 2 * i + 1) if (r > 0).any() else amax
                break
            out[b, acc] = final
            n_acc[b] = acc
        return n_acc.to(draft_ids.device), out.to(draft_ids.device)


def philox_uniform_np(seed: int, draw: int, idx: "np.ndarray") -> "np.ndarray":
    """Vector form of philox_uniform over an array of indices."""
    M = np.uint64(0xFFFFFFFF)
    c0 = idx.astype(np.uint64) & M
    c1 = np.full_like(c0, np.uint64(draw & 0xFFFFFFFF))
    c2 = np.full_like(c0, np.uint64(0x9E3779B9))
    c3 = np.full_like(c0, np.uint64(0xBB67AE85))
    k0, k1 = seed & 0xFFFFFFFF, (seed >> 32) & 0xFFFFFFFF
    for _ in range(10):
        p0 = np.uint64(0xD2511F53) * c0
        p1 = np.uint64(0xCD9E8D57) * c2
        hi0, lo0 = p0 >> np.uint64(32), p0 & M
        hi1, lo1 = p1 >> np.uint64(32), p1 & M
        c0, c1, c2, c3 = (hi1 ^ c1 ^ np.uint64(k0)) & M, lo1, (hi0 ^ c3 ^ np.uint64(k1)) & M, lo0
        k0 = (k0 + 0x9E3779B9) & 0xFFFFFFFF
        k1 = (k1 + 0xBB67AE85) & 0xFFFFFFFF
    return ((c0 >> np.uint64(8)).astype(np.float64) + 0.5) / 16777216.0


def philox_uniform(seed: int, draw: int, idx: int) -> float:
    """Host restatement of the device sampler's counter-based uniform."""
    M = 0xFFFFFFFF
    c = [idx & M, draw & M, 0x9E3779B9, 0xBB67AE85]
    k0, k1 = seed & M, (seed >> 32) & M
    for _ in range(10):
        p0 = 0xD2511F53 * c[0]
        p1 = 0xCD9E8D57 * c[2]
        hi0, lo0 = p0 >> 32, p0 & M
        hi1, lo1 = p1 >> 32, p1 & M
        c = [(hi1 ^ c[1] ^ k0) & M, lo1, (hi0 ^ c[3] ^ k1) & M, lo0]
        k0 = (k0 + 0x9E3779B9) & M
        k1 = (k1 + 0xBB67AE85) & M
    return ((c[0] >> 8) + 0.5) / 16777216.0


def sample_reference(logits: torch.Tensor, temperature: float, top_k: int, top_p: float, min_p: float,
                     seed: int, draw: int) -> int:
    """Filter order and Gumbel-max draw of the device sampler, on one fp32 row."""
    x = logits.float().cpu()
    if temperature <= 0:
        return int(x.argmax())
    vmax = float(x.max())
    thr = -math.inf
    if min_p > 0:
        thr = max(thr, vmax + temperature * math.log(min_p))
    if 0 < top_k < x.numel():
        thr = max(thr, float(torch.topk(x, top_k).values[-1]))
    if 0 < top_p < 1:
        keep = x >= thr
        w = torch.where(keep, torch.exp((x - vmax) / temperature), torch.zeros_like(x))
        need = top_p * float(w.sum())
        sv, si = torch.sort(x, descending=True)
        cw = torch.cumsum(w[si], 0)
        j = int(torch.searchsorted(cw, torch.tensor(need * (1 - 1e-6))))
        j = min(j, x.numel() - 1)
        thr = max(thr, float(sv[j]))
    best, best_i = -math.inf, -1
    for i in torch.nonzero(x >= thr).flatten().tolist():
        u = philox_uniform(seed, draw, i)
        g = (float(x[i]) - vmax) / temperature - math.log(-math.log(u))
        if g > best:
            best, best_i = g, i
    return best_i
