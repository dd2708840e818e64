"""MX block-scaled weights (OCP microscaling): MXFP8 (e4m3 values) and MXFP4 (e2m1 codes, two per byte), one
e8m0 power-of-two scale per 32 values along K, multiplied by activations that are quantised on the fly to
MXFP8 (e4m3 + e8m0 per 32). The product runs on ``tcgen05.mma kind::mxf8f6f4.block_scale``
(``csrc/gemm_mx.cu``): packed bytes go from HBM through TMA straight into the tensor core, the scales through
tensor memory; no expansion stage and no scale arithmetic on the ALUs. ``Nvfp4TcWeight`` is the NVFP4 pair of the
same kernel family (``kind::mxf4nvf4``): e2m1 on both sides, e4m3 scales per 16 values.

The kernel reads scale factors in 512-byte atoms (128 rows x 4 K-slices; byte ``(r % 32) * 16 + (r // 32) * 4
+ j``); ``sf_atoms`` builds them from the row-major scales a checkpoint stores (gpt-oss ``*_scales``,
``quantize_mxfp4``). The reference has block-scaled FP4 MMAs for GeForce Blackwell only
(rust/engine/cuda/nvfp4.cu:132-307) and serves MXFP4 through look-up kernels (rust/engine/cuda/mxfp4_moe.cu).
"""
from __future__ import annotations

import torch

from .fp4 import MXFP4, NVFP4, Fp4Weight, _e2m1_codes, _pack, _unpack_values, quantize_mxfp4, quantize_nvfp4

KIND_E4M3, KIND_E2M1_A8, KIND_NVFP4 = 0, 1, 2

ATOM = 512


def sf_atoms(scales: torch.Tensor) -> torch.Tensor:
    """uint8 [R, K/32] row-major e8m0 -> uint8 [ceil(R/128), K/128, 512] atoms (rows padded with zeros)."""
    R, G = scales.shape
    assert G % 4 == 0, "K must be a multiple of 128"
    Rp = (R + 127) // 128 * 128
    s = torch.zeros(Rp, G, dtype=torch.uint8, device=scales.device)
    s[:R] = scales
    # [row block, quarter (r // 32), lane (r % 32), k block, slice] -> [row block, k block, lane, quarter, slice]
    s = s.view(Rp // 128, 4, 32, G // 4, 4).permute(0, 3, 2, 1, 4).contiguous()
    return s.view(Rp // 128, G // 4, ATOM)


def e8m0_to_float(s: torch.Tensor) -> torch.Tensor:
    return torch.exp2(s.float() - 127.0)


def quantize_mxfp8(w: torch.Tensor):
    """[N, K] -> (e4m3 bytes uint8 [N, K], e8m0 scales uint8 [N, K/32]); the scale is the smallest power of two
    that brings the block's largest magnitude under 448."""
    N, K = w.shape
    blk = w.float().view(N, K // 32, 32)
    amax = blk.abs().amax(-1)
    e = torch.where(amax > 0, torch.ceil(torch.log2(amax.clamp_min(2.0 ** -126) / 448.0)), torch.full_like(amax, -127.0))
    e = e.clamp(-127, 127)
    q = (blk * torch.exp2(-e).unsqueeze(-1)).clamp(-448, 448).to(torch.float8_e4m3fn)
    return q.view(N, K).view(torch.uint8).contiguous(), (e + 127).to(torch.uint8).contiguous()


def quantize_act_reference(x: torch.Tensor) -> torch.Tensor:
    """What the device quantiser makes of bf16 activations, dequantised back to fp32 (the values the MMA sees)."""
    q, s = quantize_mxfp8(x)
    T, K = x.shape
    return (q.view(torch.float8_e4m3fn).float().view(T, K // 32, 32) * e8m0_to_float(s).unsqueeze(-1)).view(T, K)


def quantize_act_nvfp4(x: torch.Tensor):
    """Host statement of the device NVFP4 activation quantiser: (codes uint8 [T, K/2], e4m3 scales uint8 [T, K/16],
    token scales fp32 [T]); value = code * block_scale * token_scale, token_scale = amax(token) / (6 * 448)."""
    T, K = x.shape
    xf = x.float()
    amax = xf.abs().amax(-1)
    ts = torch.where(amax > 0, amax / (6.0 * 448.0), torch.ones_like(amax))
    blk = xf.view(T, K // 16, 16)
    sb = (blk.abs().amax(-1) / 6.0 / ts.unsqueeze(-1)).clamp_max(448.0).to(torch.float8_e4m3fn)
    sbf = sb.float()
    inv = torch.where(sbf > 0, 1.0 / (sbf * ts.unsqueeze(-1)), torch.zeros_like(sbf))
    codes = _e2m1_codes(blk * inv.unsqueeze(-1)).view(T, K)
    return _pack(codes), sb.view(torch.uint8).contiguous(), ts


def dequantize_act_nvfp4(codes: torch.Tensor, scales: torch.Tensor, ts: torch.Tensor) -> torch.Tensor:
    T = codes.shape[0]
    K = codes.shape[1] * 2
    v = _unpack_values(codes).view(T, K // 16, 16) * scales.view(torch.float8_e4m3fn).float().unsqueeze(-1)
    return v.view(T, K) * ts.view(T, 1)


class Nvfp4TcWeight:
    """NVFP4 weights for the block-scaled tensor-core path (W4A4): the checkpoint's codes [N, K/2], e4m3 scales per
    16 values and tensor scale, multiplied by activations quantised to NVFP4 per token on the fly
    (``tcgen05.mma kind::mxf4nvf4.block_scale.block16``). K must be a multiple of 256."""

    def __init__(self, codes: torch.Tensor, scales: torch.Tensor, alpha: float):
        self.q, self.scales, self.alpha = codes.contiguous(), scales.contiguous(), float(alpha)
        self.shape = (codes.shape[0], codes.shape[1] * 2)
        self.device = codes.device
        self._atoms = None

    @classmethod
    def from_dense(cls, w: torch.Tensor) -> "Nvfp4TcWeight":
        return cls(*quantize_nvfp4(w))

    @classmethod
    def from_fp4(cls, w: Fp4Weight) -> "Nvfp4TcWeight":
        if w.fmt != NVFP4:
            raise ValueError("not an NVFP4 weight")
        return cls(w.codes, w.scales, w.alpha)

    def to(self, device) -> "Nvfp4TcWeight":
        return Nvfp4TcWeight(self.q.to(device), self.scales.to(device), self.alpha)

    @property
    def atoms(self) -> torch.Tensor:
        if self._atoms is None:
            self._atoms = sf_atoms(self.scales)
        return self._atoms

    def dense(self) -> torch.Tensor:
        from .fp4 import dequantize_fp4
        return dequantize_fp4(self.q, self.scales, NVFP4, self.alpha)

    def nbytes(self) -> int:
        return self.q.numel() + self.scales.numel()

    def apply(self, ops, x, bias=None, out=None):
        T, K = x.shape
        N = self.shape[0]
        if not x.is_cuda or not hasattr(ops, "k"):                  # PyTorch statement of the same arithmetic
            y = dequantize_act_nvfp4(*quantize_act_nvfp4(x)) @ self.dense().t()
            return (y + bias.float() if bias is not None else y).to(x.dtype)
        xq = torch.empty(T, K // 2, dtype=torch.uint8, device=x.device)
        sf = torch.empty(ops.k.mx_act_scale_bytes(T, K, KIND_NVFP4), dtype=torch.uint8, device=x.device)
        ts = torch.empty(T, dtype=torch.float32, device=x.device)
        ops.k.quant_nvfp4(x if x.stride(1) == 1 else x.contiguous(), xq, sf, ts)
        y = out if out is not None else torch.empty(T, N, dtype=torch.bfloat16, device=x.device)
        ops.launches += 1 + ops.k.linear_mx(xq, sf, self.q, self.atoms, KIND_NVFP4, self.alpha, ts, bias, y, ops.workspace,
                                            ops.status)
        return y


def quantize_rows_8bit(x: torch.Tensor, is_int8: bool):
    """Per-row symmetric 8-bit quantisation (what the device quantiser does to activations and what a per-channel
    W8A8 checkpoint holds for weights): (codes uint8 [R, K], fp32 scales [R]); value = code * scale."""
    xf = x.float()
    amax = xf.abs().amax(-1)
    qmax = 127.0 if is_int8 else 448.0
    scale = torch.where(amax > 0, amax / qmax, torch.ones_like(amax))
    v = xf * (1.0 / scale).unsqueeze(-1)
    if is_int8:
        q = torch.round(v).clamp(-127, 127).to(torch.int8).view(torch.uint8)
    else:
        q = v.clamp(-448, 448).to(torch.float8_e4m3fn).view(torch.uint8)
    return q.contiguous(), scale.contiguous()


def dequantize_rows_8bit(q: torch.Tensor, scale: torch.Tensor, is_int8: bool) -> torch.Tensor:
    v = q.view(torch.int8).float() if is_int8 else q.view(torch.float8_e4m3fn).float()
    return v * scale.view(-1, 1).float()


class W8A8Weight:
    """Per-channel 8-bit weights (int8 or e4m3 codes [N, K] + one fp32 scale per output feature) multiplied by
    activations quantised per token on the fly, on ``tcgen05.mma kind::i8`` (int32 accumulators) or ``kind::f8f6f4``:
    the W8A8 form of SmoothQuant / compressed-tensors INT8 and per-channel FP8 checkpoints
    (rust/engine/cuda/int8_gemm.cu, rust/engine/cuda/fp8_gemm.cu:44-78 in the reference). K % 128 == 0."""

    def __init__(self, q: torch.Tensor, scale: torch.Tensor, is_int8: bool):
        self.q, self.scale, self.is_int8 = q.contiguous(), scale.float().contiguous(), bool(is_int8)
        self.shape = tuple(q.shape)
        self.device = q.device

    @classmethod
    def from_dense(cls, w: torch.Tensor, fmt: str = "int8") -> "W8A8Weight":
        q, s = quantize_rows_8bit(w, fmt == "int8")
        return cls(q, s, fmt == "int8")

    def to(self, device) -> "W8A8Weight":
        return W8A8Weight(self.q.to(device), self.scale.to(device), self.is_int8)

    def dense(self) -> torch.Tensor:
        return dequantize_rows_8bit(self.q, self.scale, self.is_int8)

    def nbytes(self) -> int:
        return self.q.numel() + self.scale.numel() * 4

    def apply(self, ops, x, bias=None, out=None):
        T, K = x.shape
        N = self.shape[0]
        if not x.is_cuda or not hasattr(ops, "k"):
            y = dequantize_rows_8bit(*quantize_rows_8bit(x, self.is_int8), self.is_int8) @ self.dense().t()
            return (y + bias.float() if bias is not None else y).to(x.dtype)
        xq = torch.empty(T, K, dtype=torch.uint8, device=x.device)
        ts = torch.empty(T, dtype=torch.float32, device=x.device)
        ops.k.quant_rows_8bit(x if x.stride(1) == 1 else x.contiguous(), xq, ts, self.is_int8)
        y = out if out is not None else torch.empty(T, N, dtype=torch.bfloat16, device=x.device)
        ops.launches += 1 + ops.k.linear_w8a8(xq, ts, self.q, self.scale, self.is_int8, bias, y, ops.workspace, ops.status)
        return y


class MxWeight:
    """A [N, K] matrix in MXFP8 (``a4`` False: e4m3 bytes [N, K]) or MXFP4 (``a4`` True: codes [N, K/2])."""

    def __init__(self, q: torch.Tensor, scales: torch.Tensor, a4: bool):
        self.q, self.scales, self.a4 = q.contiguous(), scales.contiguous(), bool(a4)
        self.shape = (q.shape[0], q.shape[1] * (2 if a4 else 1))
        self.device = q.device
        self._atoms = None

    @classmethod
    def from_dense(cls, w: torch.Tensor, fmt: str = "mxfp8") -> "MxWeight":
        if fmt == "mxfp8":
            q, s = quantize_mxfp8(w)
            return cls(q, s, False)
        if fmt == "mxfp4":
            c, s, _ = quantize_mxfp4(w)
            return cls(c, s, True)
        raise ValueError(f"unknown MX format {fmt!r}")

    @classmethod
    def from_fp4(cls, w: Fp4Weight) -> "MxWeight":
        if w.fmt != MXFP4 or w.alpha != 1.0:
            raise ValueError("only MXFP4 weights carry power-of-two scales per 32 values")
        return cls(w.codes, w.scales, True)

    def to(self, device) -> "MxWeight":
        return MxWeight(self.q.to(device), self.scales.to(device), self.a4)

    @property
    def atoms(self) -> torch.Tensor:
        if self._atoms is None:
            self._atoms = sf_atoms(self.scales)
        return self._atoms

    def dense(self) -> torch.Tensor:
        N, K = self.shape
        v = _unpack_values(self.q) if self.a4 else self.q.view(torch.float8_e4m3fn).float()
        sc = e8m0_to_float(self.scales) * (self.scales != 0 if self.a4 else 1)
        return (v.view(N, K // 32, 32) * sc.unsqueeze(-1)).view(N, K)

    def nbytes(self) -> int:
        return self.q.numel() + self.scales.numel()

    def apply(self, ops, x, bias=None, out=None):
        T, K = x.shape
        N = self.shape[0]
        if not x.is_cuda or not hasattr(ops, "k"):                  # PyTorch statement of the same arithmetic
            y = quantize_act_reference(x) @ self.dense().t()
            return (y + bias.float() if bias is not None else y).to(x.dtype)
        xq = torch.empty(T, K, dtype=torch.uint8, device=x.device)
        sf = torch.empty(ops.k.mx_act_scale_bytes(T, K, KIND_E4M3), dtype=torch.uint8, device=x.device)
        ops.k.quant_mx(x if x.stride(1) == 1 else x.contiguous(), xq, sf)
        y = out if out is not None else torch.empty(T, N, dtype=torch.bfloat16, device=x.device)
        ops.launches += 1 + ops.k.linear_mx(xq, sf, self.q, self.atoms, KIND_E2M1_A8 if self.a4 else KIND_E4M3, 1.0, None, bias,
                                            y, ops.workspace, ops.status)
        return y
