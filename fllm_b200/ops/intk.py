"""GGUF Q5_K, Q6_K and Q8_0 weights kept packed on the GPU, and stacks of differently typed parts.

The file layouts (176 / 210-byte super-blocks with 6-bit or int8 sub-scales, 34-byte Q8_0 blocks) are not
aligned for vector loads, so they are re-laid once at load time into planes with the same number of bits per
weight (the reference does the same before its kernels: rust/engine/cuda/qgemm5k.cu:17, qgemm6k.cu:23,
qgemm8.cu):

* ``Q5_K``  low nibbles uint8 [N, K/2] (nibble order of ``ops.int4``: ``[v0 v2 v4 v6 v1 v3 v5 v7]`` per word),
  fifth bits uint32 [N, K/32] (nibble g of the word = bits of the four values the g-th nibble mask delivers),
  sub-scales uint8 [N, K/32, 2] = (scale, min), super-scales fp16 [N, K/256, 2] = (d, dmin);
  value = d * scale * q - dmin * min, q in 0..31.                                  5.625 bits / weight
* ``Q6_K``  low nibbles as above, two planes of high bits uint32 [N, K/32, 2], sub-scales int8 [N, K/16],
  super-scale fp16 [N, K/256]; value = d * scale * (q - 32), q in 0..63.            6.56 bits / weight
* ``Q8_0``  int8 codes [N, K], fp16 scale per 32 values; value = d * q.               8.5 bits / weight

Steps of at most 4 tokens multiply these planes directly (``csrc/gemv_wk.cu``: int8 activations, dp4a); longer
steps expand the matrix into bf16 scratch and run the dense GEMM, so the resident form stays packed either way.
``StackedWeight`` concatenates parts of different types along the output dimension (q|k|v, gate|up of a
Q4_K_M file mix Q4_K and Q6_K): each part multiplies into its slice of the output.
"""
from __future__ import annotations

from typing import List

import numpy as np
import torch

Q5K, Q6K, Q80 = 5, 6, 8
_ORDER = (0, 2, 4, 6, 1, 3, 5, 7)            # nibble j of a word holds value _ORDER[j]
_GROUP = ((0, 4, 1, 5), (2, 6, 3, 7))        # the values the two nibble masks of a word deliver, in byte order


def _f16(a: np.ndarray) -> np.ndarray:
    return np.ascontiguousarray(a).view(np.float16)


def _pack_low(q: np.ndarray) -> np.ndarray:
    """uint8 [N, K] (low 4 bits used) -> uint8 [N, K/2] in the kernel's nibble order."""
    N, K = q.shape
    g = (q & 0xF).reshape(N, K // 8, 8)[:, :, list(_ORDER)]
    return (g[:, :, 0::2] | (g[:, :, 1::2] << 4)).reshape(N, K // 2).astype(np.uint8)


def _pack_bit(bits: np.ndarray) -> np.ndarray:
    """uint8 [N, K] of 0/1 -> uint32 [N, K/32]: nibble g of a word holds the bits of mask group g of the block
    (g = 2 * word + half), bit i of the nibble = byte i of that group."""
    N, K = bits.shape
    b = bits.reshape(N, K // 32, 4, 8).astype(np.uint32)          # block, word, value in word
    out = np.zeros((N, K // 32), np.uint32)
    for w in range(4):
        for h in range(2):
            for i, v in enumerate(_GROUP[h]):
                out |= b[:, :, w, v] << np.uint32(4 * (2 * w + h) + i)
    return out


def _unpack_low(ql: np.ndarray) -> np.ndarray:
    N, K2 = ql.shape
    nib = np.stack([ql & 0xF, ql >> 4], -1).reshape(N, K2 // 4, 8)
    out = np.empty_like(nib)
    out[:, :, list(_ORDER)] = nib
    return out.reshape(N, K2 * 2)


def _unpack_bit(plane: np.ndarray) -> np.ndarray:
    N, G = plane.shape
    out = np.zeros((N, G, 4, 8), np.uint8)
    for w in range(4):
        for h in range(2):
            for i, v in enumerate(_GROUP[h]):
                out[:, :, w, v] = (plane >> np.uint32(4 * (2 * w + h) + i)) & 1
    return out.reshape(N, G * 32)


class IntKWeight:
    """A [N, K] matrix in the planar device form of Q5_K, Q6_K or Q8_0."""

    def __init__(self, fmt: int, shape, codes: torch.Tensor, high: torch.Tensor, sub: torch.Tensor, sup: torch.Tensor):
        self.fmt, self.shape = int(fmt), (int(shape[0]), int(shape[1]))
        self.codes, self.high, self.sub, self.sup = codes, high, sub, sup
        self.device = codes.device

    # ---------------------------------------------------------------- constructors
    @classmethod
    def from_gguf(cls, qtype_name: str, raw: np.ndarray, rows: int, cols: int, device="cpu") -> "IntKWeight":
        """raw: the tensor's bytes as stored in the file (uint8, row-major blocks)."""
        raw = np.ascontiguousarray(raw, dtype=np.uint8)
        if qtype_name == "Q8_0":
            b = raw.reshape(rows, cols // 32, 34)
            d = _f16(b[:, :, 0:2]).reshape(rows, cols // 32)
            q = np.ascontiguousarray(b[:, :, 2:34]).reshape(rows, cols)
            t = [torch.from_numpy(q.copy()), torch.zeros(1, dtype=torch.int32), torch.zeros(1, dtype=torch.uint8),
                 torch.from_numpy(d.copy())]
            fmt = Q80
        elif qtype_name == "Q6_K":
            nb = cols // 256
            b = raw.reshape(rows, nb, 210)
            ql, qh = b[:, :, 0:128], b[:, :, 128:192]
            sc = np.ascontiguousarray(b[:, :, 192:208]).view(np.int8).reshape(rows, nb * 16)
            d = _f16(b[:, :, 208:210]).reshape(rows, nb)
            q = np.empty((rows, nb, 256), np.uint8)                    # ggml's dequantize_row_q6_K index order
            for half in range(2):
                l = ql[:, :, 64 * half:64 * half + 64]
                h = qh[:, :, 32 * half:32 * half + 32]
                o = 128 * half
                q[:, :, o + 0:o + 32] = (l[:, :, 0:32] & 0xF) | (((h >> 0) & 3) << 4)
                q[:, :, o + 32:o + 64] = (l[:, :, 32:64] & 0xF) | (((h >> 2) & 3) << 4)
                q[:, :, o + 64:o + 96] = (l[:, :, 0:32] >> 4) | (((h >> 4) & 3) << 4)
                q[:, :, o + 96:o + 128] = (l[:, :, 32:64] >> 4) | (((h >> 6) & 3) << 4)
            q = q.reshape(rows, cols)
            high = np.stack([_pack_bit((q >> 4) & 1), _pack_bit((q >> 5) & 1)], -1)
            t = [torch.from_numpy(_pack_low(q)), torch.from_numpy(high.view(np.int32).copy()), torch.from_numpy(sc.copy()),
                 torch.from_numpy(d.copy())]
            fmt = Q6K
        elif qtype_name == "Q5_K":
            nb = cols // 256
            b = raw.reshape(rows, nb, 176)
            d = _f16(b[:, :, 0:2]).reshape(rows, nb)
            dmin = _f16(b[:, :, 2:4]).reshape(rows, nb)
            s = b[:, :, 4:16]
            sc6 = np.empty((rows, nb, 8), np.uint8)
            mn6 = np.empty((rows, nb, 8), np.uint8)
            sc6[:, :, :4] = s[:, :, 0:4] & 63
            mn6[:, :, :4] = s[:, :, 4:8] & 63
            sc6[:, :, 4:] = (s[:, :, 8:12] & 0xF) | ((s[:, :, 0:4] >> 6) << 4)
            mn6[:, :, 4:] = (s[:, :, 8:12] >> 4) | ((s[:, :, 4:8] >> 6) << 4)
            qh, qs = b[:, :, 16:48], b[:, :, 48:176].reshape(rows, nb, 4, 32)
            q = np.empty((rows, nb, 4, 2, 32), np.uint8)
            for j in range(4):                                         # sub-blocks 2j (low nibbles) and 2j + 1 (high)
                q[:, :, j, 0, :] = (qs[:, :, j] & 0xF) | (((qh >> (2 * j)) & 1) << 4)
                q[:, :, j, 1, :] = (qs[:, :, j] >> 4) | (((qh >> (2 * j + 1)) & 1) << 4)
            q = q.reshape(rows, cols)
            sub = np.stack([sc6.reshape(rows, nb * 8), mn6.reshape(rows, nb * 8)], -1)
            sup = np.stack([d, dmin], -1)
            t = [torch.from_numpy(_pack_low(q)), torch.from_numpy(_pack_bit((q >> 4) & 1).view(np.int32).copy()),
                 torch.from_numpy(sub.copy()), torch.from_numpy(sup.copy())]
            fmt = Q5K
        else:
            raise ValueError(f"{qtype_name} has no packed 5/6/8-bit device form")
        return cls(fmt, (rows, cols), *[x.contiguous().to(device) for x in t])

    @staticmethod
    def supports(qtype_name: str, cols: int) -> bool:
        return (qtype_name in ("Q5_K", "Q6_K") and cols % 256 == 0) or (qtype_name == "Q8_0" and cols % 32 == 0)

    # ---------------------------------------------------------------- cuts
    def rows(self, sl: slice) -> "IntKWeight":
        sl = slice(*sl.indices(self.shape[0]))
        pick = lambda x: x[sl] if x.dim() > 1 else x
        return IntKWeight(self.fmt, (sl.stop - sl.start, self.shape[1]), pick(self.codes), pick(self.high), pick(self.sub),
                          pick(self.sup))

    def cols(self, sl: slice) -> "IntKWeight":
        """A range of input features; its ends must fall on 256-value boundaries (32 for Q8_0)."""
        unit = 32 if self.fmt == Q80 else 256
        if sl.start % unit or sl.stop % unit:
            raise ValueError(f"column cuts of this weight must be multiples of {unit}")
        a, b = sl.start, sl.stop
        if self.fmt == Q80:
            return IntKWeight(self.fmt, (self.shape[0], b - a), self.codes[:, a:b].contiguous(), self.high, self.sub,
                              self.sup[:, a // 32:b // 32].contiguous())
        sub = self.sub[:, a // 16:b // 16] if self.fmt == Q6K else self.sub[:, a // 32:b // 32]
        return IntKWeight(self.fmt, (self.shape[0], b - a), self.codes[:, a // 2:b // 2].contiguous(),
                          self.high[:, a // 32:b // 32].contiguous(), sub.contiguous(), self.sup[:, a // 256:b // 256].contiguous())

    def to(self, device) -> "IntKWeight":
        return IntKWeight(self.fmt, self.shape, *[x.to(device) for x in (self.codes, self.high, self.sub, self.sup)])

    def contiguous(self) -> "IntKWeight":
        return IntKWeight(self.fmt, self.shape, *[x.contiguous() for x in (self.codes, self.high, self.sub, self.sup)])

    # ---------------------------------------------------------------- use
    def dense(self) -> torch.Tensor:
        """fp32 [N, K]: the values the kernels multiply with."""
        N, K = self.shape
        codes, high = self.codes.cpu().numpy(), self.high.cpu().numpy()
        sub, sup = self.sub.cpu().numpy(), self.sup.cpu().numpy().astype(np.float32)
        if self.fmt == Q80:
            w = codes.view(np.int8).astype(np.float32).reshape(N, K // 32, 32) * sup.reshape(N, K // 32, 1)
        elif self.fmt == Q6K:
            hp = high.view(np.uint32).reshape(N, K // 32, 2)
            q = _unpack_low(codes) | (_unpack_bit(hp[:, :, 0]) << 4) | (_unpack_bit(hp[:, :, 1]) << 5)
            s = sub.view(np.int8).astype(np.float32).reshape(N, K // 256, 16) * sup.reshape(N, K // 256, 1)
            w = (q.astype(np.float32) - 32.0).reshape(N, K // 16, 16) * s.reshape(N, K // 16, 1)
        else:
            q = _unpack_low(codes) | (_unpack_bit(high.view(np.uint32).reshape(N, K // 32)) << 4)
            sm = sub.astype(np.float32).reshape(N, K // 256, 8, 2)
            s = sm[..., 0] * sup[:, :, None, 0]
            m = sm[..., 1] * sup[:, :, None, 1]
            w = q.astype(np.float32).reshape(N, K // 32, 32) * s.reshape(N, K // 32, 1) - m.reshape(N, K // 32, 1)
        return torch.from_numpy(np.ascontiguousarray(w.reshape(N, K))).to(self.device)

    def nbytes(self) -> int:
        return sum(x.numel() * x.element_size() for x in (self.codes, self.high, self.sub, self.sup))

    def apply(self, ops, x, bias=None, out=None):
        T, K = x.shape
        N = self.shape[0]
        if not x.is_cuda or not hasattr(ops, "k"):
            y = x.float() @ self.dense().to(x.device).t()
            return (y + bias.float() if bias is not None else y).to(x.dtype)
        y = out if out is not None else torch.empty(T, N, dtype=torch.bfloat16, device=x.device)
        if T <= 4 and T * K * 1.5 <= 160 * 1024 and x.stride(0) % 8 == 0:
            ops.launches += ops.k.gemv_wk(x, self.codes, self.high, self.sub, self.sup, self.fmt, bias, y)
            return y
        dense = ops.scratch_bf16(N * K).view(N, K)
        ops.k.wk_dequant(self.codes, self.high, self.sub, self.sup, self.fmt, dense)
        ops.launches += 1
        return ops.linear(x, dense, bias, y)


class StackedWeight:
    """Parts with a common K stacked along the output dimension; each part may be of a different kind (a bf16
    tensor, an ``Int4Weight``, an ``IntKWeight``, ...). The product runs part by part into slices of one output."""

    def __init__(self, parts: List):
        self.parts = list(parts)
        self.shape = (sum(p.shape[0] for p in self.parts), self.parts[0].shape[1])
        self.device = getattr(self.parts[0], "device", None)

    def to(self, device) -> "StackedWeight":
        return StackedWeight([p.to(device) for p in self.parts])

    def dense(self) -> torch.Tensor:
        return torch.cat([p.float() if isinstance(p, torch.Tensor) else p.dense().float() for p in self.parts], 0)

    def nbytes(self) -> int:
        return sum(p.numel() * p.element_size() if isinstance(p, torch.Tensor) else p.nbytes() for p in self.parts)

    def apply(self, ops, x, bias=None, out=None):
        T = x.shape[0]
        y = out if out is not None else torch.empty(T, self.shape[0], dtype=x.dtype, device=x.device)
        r = 0
        for p in self.parts:
            n = p.shape[0]
            b = bias[r:r + n] if bias is not None else None
            got = ops.linear(x, p, b, out=y[:, r:r + n])
            if got.data_ptr() != y[:, r:r + n].data_ptr():            # a path that could not write in place
                y[:, r:r + n] = got
            r += n
        return y
