"""FP4 weight formats: NVFP4 (e2m1 codes + one e4m3 scale per 16 values + an fp32 tensor scale)
and MXFP4 (e2m1 codes + one e8m0 power-of-two scale per 32 values).

Codes are packed two per byte, low nibble = even index, exactly as ModelOpt NVFP4 checkpoints
(``weight`` uint8 [N, K/2], ``weight_scale`` e4m3 [N, K/16], ``weight_scale_2`` fp32) and the
gpt-oss MXFP4 expert tensors (``*_blocks`` / ``*_scales``) store them, so checkpoint bytes go to
the GPU untouched. ``Fp4Weight.apply`` is what ``ops.linear`` calls when it meets such a weight:
steps of at most 128 tokens run the packed GEMM (the weights cross HBM as 4.5 / 4.25 bit each);
longer steps (prefill) expand the matrix to bf16 scratch once and run the dense GEMM, which is
compute-bound there anyway.

The reference's counterparts: rust/engine/cuda/nvfp4.cu:132-307 (GeForce-only mma.sync kernels),
rust/quant/src/nvfp4.rs (codec), rust/engine/cuda/marlin_vllm (the W4A16 default on sm_100).
"""
from __future__ import annotations

import torch

NVFP4, MXFP4 = 0, 1
FMT_NAMES = {"nvfp4": NVFP4, "mxfp4": MXFP4}
_GRID = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0)


def _e2m1_codes(x: torch.Tensor) -> torch.Tensor:
    """Nearest e2m1 code (ties to the even code) of values already divided by their scale."""
    a = x.abs().clamp_max(6.0)
    grid = torch.tensor(_GRID, dtype=torch.float32, device=x.device)
    mids = (grid[1:] + grid[:-1]) / 2
    idx = torch.bucketize(a, mids, right=False)                  # a == midpoint -> lower code
    tie_up = (a.unsqueeze(-1) == mids).any(-1) & (idx % 2 == 1)  # on a midpoint with an odd lower code: go up
    idx = idx + tie_up.to(idx.dtype)
    return (idx | ((x < 0).to(idx.dtype) << 3)).to(torch.uint8)


def _pack(codes: torch.Tensor) -> torch.Tensor:
    return (codes[..., 0::2] | (codes[..., 1::2] << 4)).contiguous()


def _unpack_values(packed: torch.Tensor) -> torch.Tensor:
    grid = torch.tensor(_GRID + tuple(-v for v in _GRID), dtype=torch.float32, device=packed.device)
    lo, hi = (packed & 0xF).long(), (packed >> 4).long()
    return torch.stack([grid[lo], grid[hi]], -1).flatten(-2)


def quantize_nvfp4(w: torch.Tensor):
    """[N, K] -> (codes uint8 [N, K/2], scales uint8 [N, K/16] holding e4m3, tensor scale float)."""
    N, K = w.shape
    wf = w.float()
    s2 = max(wf.abs().max().item() / (6.0 * 448.0), 1e-12)
    blk = wf.view(N, K // 16, 16)
    sb = (blk.abs().amax(-1) / 6.0 / s2).to(torch.float8_e4m3fn)
    sbf = sb.float().clamp_min(2.0 ** -9)
    codes = _e2m1_codes(blk / (sbf * s2).unsqueeze(-1)).view(N, K)
    return _pack(codes), sb.view(torch.uint8).contiguous(), float(s2)


def quantize_mxfp4(w: torch.Tensor):
    """[N, K] -> (codes uint8 [N, K/2], scales uint8 [N, K/32] holding e8m0, 1.0)."""
    N, K = w.shape
    blk = w.float().view(N, K // 32, 32)
    amax = blk.abs().amax(-1).clamp_min(2.0 ** -120)
    e = (torch.floor(torch.log2(amax)) - 2).clamp(-127, 127)     # e2m1's largest exponent is 2
    codes = _e2m1_codes(blk / torch.exp2(e).unsqueeze(-1)).view(N, K)
    return _pack(codes), (e + 127).to(torch.uint8).contiguous(), 1.0


def scales_to_float(scales: torch.Tensor, fmt: int) -> torch.Tensor:
    if fmt == NVFP4:
        return scales.view(torch.float8_e4m3fn).float()
    return torch.exp2(scales.float() - 127.0) * (scales != 0)


def dequantize_fp4(codes: torch.Tensor, scales: torch.Tensor, fmt: int, alpha: float = 1.0) -> torch.Tensor:
    """fp32 [N, K]: the exact values the packed GEMM multiplies with (before the tensor scale is
    applied to the fp32 accumulator)."""
    N = codes.shape[0]
    K = codes.shape[1] * 2
    bs = 16 if fmt == NVFP4 else 32
    v = _unpack_values(codes).view(N, K // bs, bs) * scales_to_float(scales, fmt).view(N, K // bs, 1)
    return v.view(N, K) * alpha


class Fp4Weight:
    """A [N, K] matrix held as packed FP4 codes + block scales (+ tensor scale)."""

    def __init__(self, codes: torch.Tensor, scales: torch.Tensor, fmt: int, alpha: float = 1.0):
        self.codes, self.scales, self.fmt, self.alpha = codes, scales, int(fmt), float(alpha)
        self.shape = (codes.shape[0], codes.shape[1] * 2)
        self.device = codes.device

    @classmethod
    def from_dense(cls, w: torch.Tensor, fmt="nvfp4") -> "Fp4Weight":
        f = FMT_NAMES[fmt] if isinstance(fmt, str) else fmt
        c, s, a = (quantize_nvfp4 if f == NVFP4 else quantize_mxfp4)(w)
        return cls(c, s, f, a)

    def dense(self) -> torch.Tensor:
        return dequantize_fp4(self.codes, self.scales, self.fmt, self.alpha)

    def nbytes(self) -> int:
        return self.codes.numel() + self.scales.numel()

    def apply(self, ops, x, bias=None, out=None):
        T = x.shape[0]
        N, K = self.shape
        if not x.is_cuda:                                        # CPU oracle path
            y = x.float() @ self.dense().to(x.device).t()
            return (y + bias.float() if bias is not None else y).to(x.dtype)
        if T <= 4 and K % 32 == 0 and T * K * 1.25 <= 160 * 1024 and x.stride(0) % 8 == 0:
            # a handful of tokens: integer dot products on the packed codes (csrc/gemv_w4.cu)
            y = out if out is not None else torch.empty(T, N, dtype=torch.bfloat16, device=x.device)
            ops.launches += ops.k.gemv_w4(x, self.codes, self.scales, self.fmt, self.alpha, bias, y)
            return y
        if T <= 128:
            y = out if out is not None else torch.empty(T, N, dtype=torch.bfloat16, device=x.device)
            ops.launches += ops.k.linear_w4a16(x, self.codes, self.scales, self.fmt, self.alpha, bias, y,
                                               ops.workspace, ops.status)
            return y
        dense = ops.scratch_bf16(N * K).view(N, K)
        ops.k.w4_dequant(self.codes, self.scales, self.fmt, self.alpha, dense)
        ops.launches += 1
        return ops.linear(x, dense, bias, out)


class Fp4ExpertStack:
    """The matrices of several experts held packed: codes [E, N, K/2], scales [E, N, K/block] (bytes).
    ``moe_ffn`` hands it to the grouped packed GEMM; gpt-oss checkpoints store their experts this way
    (MXFP4), so the bytes go from the file to the tensor core unexpanded."""

    def __init__(self, codes: torch.Tensor, scales: torch.Tensor, fmt: int, alpha: float = 1.0):
        self.codes, self.scales, self.fmt, self.alpha = codes.contiguous(), scales.contiguous(), int(fmt), float(alpha)
        self.shape = (codes.shape[0], codes.shape[1], codes.shape[2] * 2)
        self.device = codes.device

    @classmethod
    def from_dense(cls, stack: torch.Tensor, fmt="mxfp4") -> "Fp4ExpertStack":
        f = FMT_NAMES[fmt] if isinstance(fmt, str) else fmt
        E, N, K = stack.shape
        if f == NVFP4:
            raise ValueError("expert stacks use one scale format for all experts: MXFP4")
        c, s, _ = quantize_mxfp4(stack.reshape(E * N, K))
        return cls(c.view(E, N, K // 2), s.view(E, N, K // 32), f)

    def dense(self) -> torch.Tensor:
        E, N, K = self.shape
        return dequantize_fp4(self.codes.view(E * N, K // 2), self.scales.view(E * N, -1), self.fmt, self.alpha).view(E, N, K)

    def __getitem__(self, sl) -> "Fp4ExpertStack":
        return Fp4ExpertStack(self.codes[sl], self.scales[sl], self.fmt, self.alpha)

    def to(self, device) -> "Fp4ExpertStack":
        return Fp4ExpertStack(self.codes.to(device), self.scales.to(device), self.fmt, self.alpha)

    def nbytes(self) -> int:
        return self.codes.numel() + self.scales.numel()


def quantize_decoder_weights(weights, fmt: str = "nvfp4") -> int:
    """Replace the four projection matrices of every layer by FP4 weights (embedding, norms and
    the lm_head stay bf16). Returns the bytes now held for those projections."""
    total = 0
    for lw in weights.layers:
        for name in ("wqkv", "wo", "w_gate_up", "w_down"):
            w = getattr(lw, name, None)
            if isinstance(w, torch.Tensor) and w.dim() == 2 and w.shape[1] % 64 == 0 and w.shape[0] % 8 == 0:
                q = Fp4Weight.from_dense(w, fmt)
                setattr(lw, name, q)
                total += q.nbytes()
    return total
