"""Readers for 4-bit group-quantised Hugging Face checkpoints: AWQ (AutoAWQ "GEMM" layout) and GPTQ
(AutoGPTQ / GPTQModel layouts ``gptq`` and ``gptq_v2``).

Both store a linear layer ``y = x W^T`` as three tensors, laid out along the *input* dimension first:

=========  ======================================  ======================================
tensor     AWQ                                      GPTQ
=========  ======================================  ======================================
qweight    int32 [K, N/8]; nibble j of a word is    int32 [K/8, N]; nibble j of a word is
           output channel 8c + (0,2,4,6,1,3,5,7)[j]  input row 8r + j
qzeros     int32 [K/g, N/8], same nibble order      int32 [K/g, N/8], nibble j = channel 8c + j;
                                                    layout ``gptq`` stores zero - 1
scales     fp16 [K/g, N]                            fp16 [K/g, N]
g_idx      --                                       int32 [K]: group of every input row
=========  ======================================  ======================================

``w[n, k] = (q[n, k] - zero[n, k / g]) * scale[n, k / g]``. The readers unpack to one code per byte
``[N, K]`` plus per-group scale and ``min = zero * scale`` and hand them to ``Int4Weight.from_groups``,
which re-packs them for the tcgen05 packed GEMM, so the weights stay 4-bit in HBM. A GPTQ tensor
quantised with activation reordering (``desc_act``: ``g_idx`` is not ``k // g``) has groups that are
not contiguous along K; it is expanded to bf16 instead.

The reference runs these checkpoints through its Marlin kernels (rust/engine/cuda/marlin_vllm/*,
repacking in rust/engine/src/backend/cuda.rs:1798-1935).
"""
from __future__ import annotations

from typing import Optional, Union

import torch

from ..ops.int4 import Int4Weight

_AWQ_ORDER = (0, 2, 4, 6, 1, 3, 5, 7)


def _nibbles(words: torch.Tensor) -> torch.Tensor:
    """int32 [...]-> uint8 [..., 8]: nibble j of every word."""
    w = words.to(torch.int64) & 0xFFFFFFFF
    shifts = torch.arange(0, 32, 4, dtype=torch.int64, device=words.device)
    return ((w.unsqueeze(-1) >> shifts) & 0xF).to(torch.uint8)


def unpack_awq(qweight: torch.Tensor, qzeros: torch.Tensor, scales: torch.Tensor):
    """-> (q uint8 [N, K], scale float [N, K/g], zero float [N, K/g])."""
    K, n8 = qweight.shape
    N = n8 * 8
    inv = torch.empty(8, dtype=torch.long)
    inv[list(_AWQ_ORDER)] = torch.arange(8)                  # channel offset c -> nibble holding it
    q = _nibbles(qweight)[:, :, inv].reshape(K, N)           # [K, N] in channel order
    z = _nibbles(qzeros)[:, :, inv].reshape(qzeros.shape[0], N)
    return q.t().contiguous(), scales.float().t().contiguous(), z.float().t().contiguous()


def unpack_gptq(qweight: torch.Tensor, qzeros: torch.Tensor, scales: torch.Tensor, zero_offset: int = 1):
    """-> (q uint8 [N, K], scale float [N, K/g], zero float [N, K/g]); ``zero_offset`` is 1 for the
    ``gptq`` layout (zeros stored minus one) and 0 for ``gptq_v2``."""
    k8, N = qweight.shape
    K = k8 * 8
    q = _nibbles(qweight).permute(0, 2, 1).reshape(K, N)     # row 8r + j
    z = _nibbles(qzeros).reshape(qzeros.shape[0], N).float() + zero_offset
    return q.t().contiguous(), scales.float().t().contiguous(), z.t().contiguous()


def pack_awq(q: torch.Tensor, zero: torch.Tensor):
    """Inverse of ``unpack_awq`` for the integer tensors (tests and converters): q [N, K], zero [N, K/g]."""
    def pack(m):                                             # m: [rows, N] values 0..15
        r, N = m.shape
        g = m.view(r, N // 8, 8)[:, :, list(_AWQ_ORDER)].to(torch.int64)
        w = sum(g[:, :, j] << (4 * j) for j in range(8))
        return torch.where(w >= 2 ** 31, w - 2 ** 32, w).to(torch.int32)
    return pack(q.t().contiguous()), pack(zero.t().contiguous().to(torch.uint8))


def pack_gptq(q: torch.Tensor, zero: torch.Tensor, zero_offset: int = 1):
    """Inverse of ``unpack_gptq``: q [N, K], zero [N, K/g] -> (qweight [K/8, N], qzeros [K/g, N/8])."""
    N, K = q.shape
    qk = q.t().contiguous().view(K // 8, 8, N).to(torch.int64)
    w = sum(qk[:, j, :] << (4 * j) for j in range(8))
    zz = ((zero.t().contiguous().to(torch.int64) - zero_offset) & 0xF).view(-1, N // 8, 8)
    z = sum(zz[:, :, j] << (4 * j) for j in range(8))
    fix = lambda t: torch.where(t >= 2 ** 31, t - 2 ** 32, t).to(torch.int32)
    return fix(w), fix(z)


def int4_linear(method: str, qweight: torch.Tensor, qzeros: torch.Tensor, scales: torch.Tensor,
                g_idx: Optional[torch.Tensor] = None, checkpoint_format: str = "gptq",
                dtype=torch.bfloat16) -> Union[Int4Weight, torch.Tensor]:
    """One quantised linear layer as an ``Int4Weight`` [N, K] (or a dense tensor when its groups are
    not contiguous, or K is not a multiple of 32)."""
    if method == "awq":
        q, s, z = unpack_awq(qweight, qzeros, scales)
    elif method == "gptq":
        q, s, z = unpack_gptq(qweight, qzeros, scales, 0 if checkpoint_format == "gptq_v2" else 1)
    else:
        raise ValueError(f"unknown 4-bit checkpoint method {method!r}")
    N, K = q.shape
    groups = s.shape[1]
    g = K // groups
    contiguous = True
    if g_idx is not None and g_idx.numel() == K:
        contiguous = bool(torch.equal(g_idx.to(torch.int64).cpu(), torch.arange(K) // g))
    if contiguous and K % 32 == 0 and g % 32 == 0:
        return Int4Weight.from_groups(q, s, z * s)
    idx = g_idx.to(torch.int64).cpu() if g_idx is not None and g_idx.numel() == K else torch.arange(K) // g
    return ((q.float() - z[:, idx]) * s[:, idx]).to(dtype)
