"""Operator layer: ``NativeOps`` (hand-written sm_100a kernels) and ``RefOps``
(PyTorch fp32 oracle). ``get_ops(device)`` picks the native path for CUDA devices
and fails loudly when its library is missing."""
from __future__ import annotations

import torch

from .reference import RefOps


def get_ops(device) -> object:
    device = torch.device(device)
    if device.type == "cuda":
        from .native import NativeOps
        return NativeOps(device)
    return RefOps()
