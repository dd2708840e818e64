"""Tensor-parallel runtime handed to the decoder: which collectives combine the
row-parallel projection outputs.

* ``fused``  peer-memory kernels (``fllm_b200.comm.symm``): partial sums are pushed
             into the owning rank's HBM over NVLink from inside our own kernels, with
             bounded flag waits; no library collective on the hot path;
* ``nccl``   ``torch.distributed`` all-reduce / all-gather - the baseline the fused path
             is measured against, and the path used on CPU ranks (gloo).
"""
from __future__ import annotations

import os
from typing import Optional

import torch

from ..comm.group import Group


class SingleRank:
    size, rank, backend = 1, 0, "none"

    def all_reduce(self, x):
        return x

    def all_gather(self, x):
        return x.unsqueeze(0)

    def close(self):
        pass


class LibraryTP:
    """Baseline: library collectives on the compute stream."""

    def __init__(self, group: Group):
        self.group, self.size, self.rank = group, group.size, group.rank
        self.backend = "nccl" if not group.deterministic else "gloo"

    def all_reduce(self, x):
        return self.group.all_reduce(x)

    def all_gather(self, x):
        return self.group.all_gather(x)

    def close(self):
        pass


def make_tp_runtime(world: int, rank: int, device, backend: str = "auto", group: Optional[Group] = None,
                    hidden: int = 0, max_tokens: int = 2048):
    if world <= 1:
        return SingleRank()
    group = group or Group()
    device = torch.device(device)
    if backend == "auto":
        backend = os.environ.get("FLLM_TP_BACKEND", "fused" if device.type == "cuda" else "nccl")
    if backend == "fused" and device.type == "cuda":
        try:
            from ..comm.symm import FusedTP
            rt = FusedTP(group, device, hidden, max_tokens)
            if rt.self_check():
                return rt
            rt.close()
        except Exception as e:                        # keep serving on the library path
            if rank == 0:
                print(f"[fllm_b200] fused tensor-parallel path unavailable ({e}); using NCCL", flush=True)
    return LibraryTP(group)
