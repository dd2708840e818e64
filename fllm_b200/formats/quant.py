"""ctypes face of the native codecs (``csrc_cpu/quant.cpp``): quantize / dequantize rows of
every packed type the engine knows, keeping the packed bytes as ``numpy`` uint8 arrays."""
from __future__ import annotations

import ctypes

import numpy as np

from ..ops._lib import load_cpu

F32, F16, Q4_0, Q8_0, Q4_K, Q5_K, Q6_K, Q8_K, BF16, MXFP4 = 0, 1, 2, 8, 12, 13, 14, 15, 30, 39
Q4_1, Q5_0, Q5_1, Q2_K, Q3_K, IQ4_NL, IQ4_XS = 3, 6, 7, 10, 11, 20, 23
TYPE_NAMES = {"F32": F32, "F16": F16, "BF16": BF16, "Q4_0": Q4_0, "Q4_1": Q4_1, "Q5_0": Q5_0, "Q5_1": Q5_1, "Q8_0": Q8_0,
              "Q2_K": Q2_K, "Q3_K": Q3_K, "Q4_K": Q4_K, "Q5_K": Q5_K, "Q6_K": Q6_K, "IQ4_NL": IQ4_NL, "IQ4_XS": IQ4_XS,
              "MXFP4": MXFP4}
NVFP4, FP8_E4M3 = 1001, 1002
_configured = False


def _lib():
    global _configured
    lib = load_cpu()
    if not _configured:
        lib.fllm_row_bytes.restype = ctypes.c_int64
        lib.fllm_row_bytes.argtypes = [ctypes.c_int, ctypes.c_int64]
        lib.fllm_quantize.argtypes = [ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64, ctypes.c_int64]
        lib.fllm_dequantize.argtypes = [ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64, ctypes.c_int64]
        _configured = True
    return lib


def row_bytes(qtype: int, ncols: int) -> int:
    n = _lib().fllm_row_bytes(qtype, ncols)
    if n < 0:
        raise ValueError(f"type {qtype} cannot hold rows of {ncols} values")
    return n


def quantize(x: np.ndarray, qtype: int) -> np.ndarray:
    """x: float32 [rows, cols] -> uint8 [rows, row_bytes]."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    rows, cols = x.shape
    out = np.empty((rows, row_bytes(qtype, cols)), dtype=np.uint8)
    if _lib().fllm_quantize(qtype, x.ctypes.data, out.ctypes.data, rows, cols):
        raise ValueError("quantize failed")
    return out


def dequantize(packed: np.ndarray, qtype: int, rows: int, cols: int) -> np.ndarray:
    packed = np.ascontiguousarray(packed).view(np.uint8)
    if packed.size != rows * row_bytes(qtype, cols):
        raise ValueError("packed size does not match rows x cols")
    out = np.empty((rows, cols), dtype=np.float32)
    if _lib().fllm_dequantize(qtype, packed.ctypes.data, out.ctypes.data, rows, cols):
        raise ValueError("dequantize failed")
    return out
