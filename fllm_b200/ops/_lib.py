"""Loading of the native libraries built by ``fllm_b200._build``.

On a machine with a GPU the CUDA library is mandatory: a missing or stale
``_C.so`` raises instead of silently running PyTorch math, so a passing GPU test
always means the hand-written kernels ran.
"""
from __future__ import annotations

import ctypes
import os
from pathlib import Path

import torch

_PKG = Path(__file__).resolve().parent.parent
_LIB_CUDA = _PKG / "_C.so"
_LIB_CPU = _PKG / "_cpu.so"
_state = {"cuda": None, "cpu": None}


def load_cuda(build_if_missing: bool = True):
    """Register ``torch.ops.fllm_b200``; returns the ops namespace."""
    if _state["cuda"] is not None:
        return _state["cuda"]
    if not _LIB_CUDA.exists():
        if not build_if_missing or os.environ.get("FLLM_NO_JIT_BUILD") == "1":
            raise RuntimeError(f"native library {_LIB_CUDA} is missing; run `python -m fllm_b200._build`")
        from .. import _build
        _build.build_cuda()
    torch.ops.load_library(str(_LIB_CUDA))
    _state["cuda"] = torch.ops.fllm_b200
    return _state["cuda"]


def have_cuda_lib() -> bool:
    try:
        load_cuda(build_if_missing=False)
        return True
    except Exception:
        return False


def load_cpu(build_if_missing: bool = True) -> ctypes.CDLL:
    if _state["cpu"] is not None:
        return _state["cpu"]
    alt = os.environ.get("FLLM_CPU_LIB")          # another build of the same library (the sanitizer build)
    if alt:
        _state["cpu"] = ctypes.CDLL(alt)
        return _state["cpu"]
    if not _LIB_CPU.exists():
        if not build_if_missing:
            raise RuntimeError(f"native library {_LIB_CPU} is missing; run `python -m fllm_b200._build`")
        from .. import _build
        _build.build_cpu()
    _state["cpu"] = ctypes.CDLL(str(_LIB_CPU))
    return _state["cpu"]


def loaded_libraries() -> list:
    return [str(p) for p, k in ((_LIB_CUDA, "cuda"), (_LIB_CPU, "cpu")) if _state[k] is not None]
