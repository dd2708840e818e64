"""Readers of two more 4-bit checkpoint families stored in safetensors files.

* MLX affine quantisation (``mlx-community`` checkpoints; the reference runs it in rust/engine/cuda/mlx_affine.cu and
  rust/engine/src/cpu_mlx.rs): per linear layer ``weight`` uint32 [N, K * bits / 32] with the codes of a row packed
  low bits first, ``scales`` and ``biases`` [N, K / group]; w = scale * q + bias. 4-bit layers become the packed
  group format of the GPU kernels (codes + (scale, min) per 32 values) without leaving 4 bits; 2- and 8-bit layers
  are expanded at load.
* bitsandbytes 4-bit (NF4 / FP4; rust/engine/cuda/bnb.cuh, rust/engine/src/cpu_bnb.rs): ``weight`` uint8
  [numel / 2, 1] with the first value of a pair in the high nibble, one ``absmax`` per ``blocksize`` values (itself
  8-bit quantised against ``nested_absmax`` when double quantisation is on), a 16-entry ``quant_map``; w =
  quant_map[code] * absmax[block]. A codebook is not an affine grid, so these layers are expanded at load.
"""
from __future__ import annotations

import json
from typing import Optional

import torch

NF4_MAP = [-1.0, -0.6961928009986877, -0.5250730514526367, -0.39491748809814453, -0.28444138169288635,
           -0.18477343022823334, -0.09105003625154495, 0.0, 0.07958029955625534, 0.16093020141124725,
           0.24611230194568634, 0.33791524171829224, 0.44070982933044434, 0.5626170039176941, 0.7229568362236023, 1.0]
FP4_MAP = [0.0, 0.0052083333, 0.6666667, 1.0, 0.33333334, 0.5, 0.16666667, 0.25,
           -0.0, -0.0052083333, -0.6666667, -1.0, -0.33333334, -0.5, -0.16666667, -0.25]


def unpack_mlx_codes(weight: torch.Tensor, bits: int) -> torch.Tensor:
    """uint32 words [N, W] -> codes uint8 [N, W * 32 / bits] (bits in 2, 4, 8: codes never straddle a word)."""
    if bits not in (2, 4, 8):
        raise ValueError(f"MLX affine layers with {bits}-bit codes are not supported (2, 4 and 8 are)")
    w = weight.to(torch.int64) & 0xFFFFFFFF
    shifts = torch.arange(0, 32, bits, dtype=torch.int64)
    return ((w[:, :, None] >> shifts) & ((1 << bits) - 1)).reshape(w.shape[0], -1).to(torch.uint8)


def mlx_linear(weight: torch.Tensor, scales: torch.Tensor, biases: torch.Tensor, bits: int, group: int, dtype=torch.bfloat16):
    """One MLX affine layer: an ``Int4Weight`` when it is 4-bit with groups of a multiple of 32, else a dense tensor."""
    from ..ops.int4 import Int4Weight
    q = unpack_mlx_codes(weight, bits)
    N, K = q.shape
    if K // group != scales.shape[1]:
        raise ValueError(f"MLX layer: {K} columns in groups of {group} need {K // group} scales per row, found {scales.shape[1]}")
    if bits == 4 and group % 32 == 0 and K % 32 == 0:
        return Int4Weight.from_groups(q, scales.float(), -biases.float())           # w = s q - m with m = -bias
    s = scales.float().repeat_interleave(group, 1)
    b = biases.float().repeat_interleave(group, 1)
    return (q.float() * s + b).to(dtype)


def dequantize_bnb4(weight: torch.Tensor, absmax: torch.Tensor, shape, blocksize: int = 64, quant_map: Optional[torch.Tensor] = None,
                    quant_type: str = "nf4", nested_absmax: Optional[torch.Tensor] = None, nested_quant_map: Optional[torch.Tensor] = None,
                    nested_blocksize: int = 256, nested_offset: float = 0.0, dtype=torch.bfloat16) -> torch.Tensor:
    code = quant_map.float() if quant_map is not None else torch.tensor(NF4_MAP if quant_type == "nf4" else FP4_MAP)
    b = weight.reshape(-1).to(torch.int64)
    q = torch.stack([b >> 4, b & 15], 1).reshape(-1)
    n = 1
    for d in shape:
        n *= int(d)
    q = q[:n]
    am = absmax
    if nested_absmax is not None:                                 # double quantisation: absmax is an 8-bit code itself
        idx = torch.arange(am.numel()) // nested_blocksize
        am = nested_quant_map.float()[am.to(torch.int64)] * nested_absmax.float()[idx] + float(nested_offset)
    scale = am.float().repeat_interleave(blocksize)[:n]
    return (code[q] * scale).reshape(*shape).to(dtype)


def bnb_linear(get, name: str, dtype=torch.bfloat16) -> Optional[torch.Tensor]:
    """The dense weight of a bitsandbytes 4-bit layer named ``name`` (``get(tensor_name, required)`` reads the
    checkpoint), or None when the layer is not stored that way."""
    for qt in ("nf4", "fp4"):
        state = get(f"{name}.weight.quant_state.bitsandbytes__{qt}", False)
        if state is None:
            continue
        meta = json.loads(bytes(state.to(torch.uint8).tolist()).decode("utf-8"))
        nested = get(name + ".weight.nested_absmax", False)
        return dequantize_bnb4(get(name + ".weight"), get(name + ".weight.absmax"), meta["shape"], int(meta.get("blocksize", 64)),
                               get(name + ".weight.quant_map", False), qt, nested, get(name + ".weight.nested_quant_map", False),
                               int(meta.get("nested_blocksize", 256)), float(meta.get("nested_offset", 0.0)), dtype)
    return None
