"""INT4 group-affine weights on the GPU: unsigned 4-bit codes with one (scale, min) pair per 32
values, ``value = q * scale - min``.

This is the device form of the GGUF types Q4_K, Q4_0, Q4_1 and of AWQ / GPTQ int4 groups: the file
layouts (144-byte super-blocks with 6-bit sub-scales, 18-byte blocks, column-packed int32 words)
are re-laid once at load time into two planar arrays

* ``codes``  uint8 [N, K/2]; inside every group of 8 values the nibbles are ordered
  [v0 v2 v4 v6 v1 v3 v5 v7], so that ``(word >> 4j) & 0x000F000F`` is the pair (v2j, v2j+1);
* ``sm``     bf16 [N, K/32, 2] = {scale, min}

and stay packed in HBM (4 bits + 1 bit of scale per weight). Steps of at most 4 tokens run the dp4a
kernel of ``csrc/gemv_w4.cu`` (int8 activations), steps of at most 128 tokens the packed tcgen05 GEMM of
``csrc/gemm_w4a16.cu`` (format 2); longer steps expand to bf16 scratch.
The reference keeps these types packed too and runs them through per-type kernels
(rust/engine/cuda/qgemm4k.cu, marlin_q4k.cu, mmvq.cu, marlin_vllm/*; device re-layout at
rust/engine/src/backend/cuda.rs:1798-1935).
"""
from __future__ import annotations

import numpy as np
import torch

INT4G = 2
GEMV_MAX_TOKENS = 4
_ORDER = (0, 2, 4, 6, 1, 3, 5, 7)          # nibble j of a word holds value _ORDER[j]


def pack_codes(q: torch.Tensor) -> torch.Tensor:
    """uint8 [N, K] values 0..15 -> uint8 [N, K/2] in the kernel's nibble order."""
    N, K = q.shape
    g = q.view(N, K // 8, 8)[:, :, list(_ORDER)]                     # nibble order
    return (g[:, :, 0::2] | (g[:, :, 1::2] << 4)).reshape(N, K // 2).contiguous()


def unpack_codes(codes: torch.Tensor) -> torch.Tensor:
    N, K2 = codes.shape
    nib = torch.stack([codes & 0xF, codes >> 4], -1).view(N, K2 // 4, 8)   # nibble j of each word
    out = torch.empty_like(nib)
    out[:, :, list(_ORDER)] = nib
    return out.view(N, K2 * 2)


class Int4Weight:
    def __init__(self, codes: torch.Tensor, sm: torch.Tensor):
        assert codes.dtype == torch.uint8 and sm.dtype == torch.bfloat16 and sm.shape[-1] == 2
        self.codes, self.sm = codes.contiguous(), sm.contiguous()
        self.shape = (codes.shape[0], codes.shape[1] * 2)
        self.device = codes.device

    # ---------------------------------------------------------------- constructors
    @classmethod
    def from_groups(cls, q: torch.Tensor, scale: torch.Tensor, minv: torch.Tensor) -> "Int4Weight":
        """q uint8 [N, K] (0..15); scale, minv float [N, K/g] for any group size g that is a multiple
        of 32 (AWQ / GPTQ: g = 128, minv = zero_point * scale)."""
        N, K = q.shape
        rep = (K // 32) // scale.shape[1]
        s = scale.float().repeat_interleave(rep, 1)
        m = minv.float().repeat_interleave(rep, 1)
        return cls(pack_codes(q), torch.stack([s, m], -1).to(torch.bfloat16))

    @classmethod
    def from_dense(cls, w: torch.Tensor, group: int = 32) -> "Int4Weight":
        """Asymmetric min-max quantisation per group (what a Q4_1 / AWQ-style quantiser does)."""
        N, K = w.shape
        g = w.float().view(N, K // group, group)
        lo, hi = g.amin(-1), g.amax(-1)
        s = ((hi - lo) / 15.0).clamp_min(1e-12).to(torch.bfloat16).float()      # the scale the kernel will use
        m = (-lo).to(torch.bfloat16).float()
        q = torch.round((g + m.unsqueeze(-1)) / s.unsqueeze(-1)).clamp_(0, 15).to(torch.uint8).view(N, K)
        return cls.from_groups(q, s, m)

    @classmethod
    def from_gguf(cls, qtype_name: str, raw: np.ndarray, rows: int, cols: int, device="cpu") -> "Int4Weight":
        """raw: the tensor's bytes as stored in the file (uint8, row-major blocks)."""
        if qtype_name == "Q4_K":
            q, s, m = _decode_q4_k(raw, rows, cols)
        elif qtype_name == "Q4_0":
            q, s, m = _decode_q4_0(raw, rows, cols)
        elif qtype_name == "Q4_1":
            q, s, m = _decode_q4_1(raw, rows, cols)
        else:
            raise ValueError(f"{qtype_name} has no INT4 group-affine form")
        w = cls.from_groups(torch.from_numpy(q), torch.from_numpy(s), torch.from_numpy(m))
        return cls(w.codes.to(device), w.sm.to(device))

    # ---------------------------------------------------------------- cuts (tensor parallelism, fused projections)
    @staticmethod
    def cat(parts: "list[Int4Weight]") -> "Int4Weight":
        """Stack along the output dimension (q|k|v, gate|up)."""
        return Int4Weight(torch.cat([p.codes for p in parts], 0), torch.cat([p.sm for p in parts], 0))

    def rows(self, sl: slice) -> "Int4Weight":
        return Int4Weight(self.codes[sl], self.sm[sl])

    def cols(self, sl: slice) -> "Int4Weight":
        """A range of input features; its ends must fall on 64-value boundaries."""
        if sl.start % 64 or sl.stop % 64:
            raise ValueError("column cuts of an INT4 weight must be multiples of 64")
        return Int4Weight(self.codes[:, sl.start // 2: sl.stop // 2], self.sm[:, sl.start // 32: sl.stop // 32])

    def to(self, device) -> "Int4Weight":
        return Int4Weight(self.codes.to(device), self.sm.to(device))

    # ---------------------------------------------------------------- use
    def dense(self) -> torch.Tensor:
        """fp32 [N, K] of q * scale - min with the bf16 scale / min the kernel multiplies with."""
        N, K = self.shape
        q = unpack_codes(self.codes).float().view(N, K // 32, 32)
        s, m = self.sm[..., 0].float().unsqueeze(-1), self.sm[..., 1].float().unsqueeze(-1)
        return (q * s - m).view(N, K)

    def nbytes(self) -> int:
        return self.codes.numel() + self.sm.numel() * 2

    def apply(self, ops, x, bias=None, out=None):
        T = x.shape[0]
        N, K = self.shape
        if not x.is_cuda:
            y = x.float() @ self.dense().to(torch.bfloat16).float().t()
            return (y + bias.float() if bias is not None else y).to(x.dtype)
        if T <= GEMV_MAX_TOKENS and K % 32 == 0 and T * K * 1.25 <= 160 * 1024 and x.stride(0) % 8 == 0:
            # a handful of tokens: integer dot products on the packed codes (csrc/gemv_w4.cu)
            y = out if out is not None else torch.empty(T, N, dtype=torch.bfloat16, device=x.device)
            ops.launches += ops.k.gemv_w4(x, self.codes, self.sm.view(torch.uint8).view(N, -1), INT4G, 1.0, bias, y)
            return y
        if T <= 128:
            y = out if out is not None else torch.empty(T, N, dtype=torch.bfloat16, device=x.device)
            ops.launches += ops.k.linear_w4a16(x, self.codes, self.sm.view(torch.uint8).view(N, -1), INT4G, 1.0, bias, y,
                                               ops.workspace, ops.status)
            return y
        dense = ops.scratch_bf16(N * K).view(N, K)
        ops.k.w4_dequant(self.codes, self.sm.view(torch.uint8).view(N, -1), INT4G, 1.0, dense)
        ops.launches += 1
        return ops.linear(x, dense, bias, out)


# -------------------------------------------------------------------- GGUF block decoders (numpy)
def _f16(a: np.ndarray) -> np.ndarray:
    return a.view(np.float16).astype(np.float32)


def _decode_q4_k(raw: np.ndarray, rows: int, cols: int):
    """144-byte super-blocks of 256 values: d, dmin (f16), 12 bytes of 6-bit (scale, min) for 8
    sub-blocks, 128 bytes of codes (sub-blocks 2j and 2j+1 share 32 bytes: low / high nibbles).
    value = d * sc * q - dmin * mn  (ggml's dequantize_row_q4_K)."""
    nb = cols // 256
    b = np.ascontiguousarray(raw, dtype=np.uint8).reshape(rows, nb, 144)
    d = _f16(np.ascontiguousarray(b[:, :, 0:2])).reshape(rows, nb)
    dmin = _f16(np.ascontiguousarray(b[:, :, 2:4])).reshape(rows, nb)
    sc = b[:, :, 4:16].astype(np.uint8)
    scale6 = np.empty((rows, nb, 8), np.uint8)
    min6 = np.empty((rows, nb, 8), np.uint8)
    scale6[:, :, :4] = sc[:, :, 0:4] & 63
    min6[:, :, :4] = sc[:, :, 4:8] & 63
    scale6[:, :, 4:] = (sc[:, :, 8:12] & 0xF) | ((sc[:, :, 0:4] >> 6) << 4)
    min6[:, :, 4:] = (sc[:, :, 8:12] >> 4) | ((sc[:, :, 4:8] >> 6) << 4)
    qs = b[:, :, 16:144].reshape(rows, nb, 4, 32)
    q = np.empty((rows, nb, 4, 2, 32), np.uint8)
    q[:, :, :, 0, :] = qs & 0xF
    q[:, :, :, 1, :] = qs >> 4
    s = (d[:, :, None] * scale6.astype(np.float32)).reshape(rows, nb * 8)
    m = (dmin[:, :, None] * min6.astype(np.float32)).reshape(rows, nb * 8)
    return q.reshape(rows, cols), s, m


def _decode_q4_0(raw: np.ndarray, rows: int, cols: int):
    """18-byte blocks of 32: d (f16) + 16 bytes (low nibbles = first 16 values). value = d * (q - 8)."""
    nb = cols // 32
    b = np.ascontiguousarray(raw, dtype=np.uint8).reshape(rows, nb, 18)
    d = _f16(np.ascontiguousarray(b[:, :, 0:2])).reshape(rows, nb)
    qs = b[:, :, 2:18]
    q = np.concatenate([qs & 0xF, qs >> 4], -1).reshape(rows, cols)
    return q, d, 8.0 * d


def _decode_q4_1(raw: np.ndarray, rows: int, cols: int):
    """20-byte blocks of 32: d, m (f16) + 16 bytes. value = d * q + m."""
    nb = cols // 32
    b = np.ascontiguousarray(raw, dtype=np.uint8).reshape(rows, nb, 20)
    d = _f16(np.ascontiguousarray(b[:, :, 0:2])).reshape(rows, nb)
    mn = _f16(np.ascontiguousarray(b[:, :, 2:4])).reshape(rows, nb)
    qs = b[:, :, 4:20]
    q = np.concatenate([qs & 0xF, qs >> 4], -1).reshape(rows, cols)
    return q, d, -mn
