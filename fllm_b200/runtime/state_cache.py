"""Recurrent-state checkpoints: the prefix cache of models whose layers carry a state instead of (or beside) KV.

A paged KV prefix can be shared block by block; a recurrent state cannot: it summarises the whole prefix. So a prompt
prefix is reusable only at positions where a copy of the state was kept. The engine keeps such copies at block
boundaries where prefill chunks end (the scheduler cuts chunks there), in host memory, under the chain hash of the
last block of the prefix; a later request whose prompt starts with the same blocks gets the copy written into its
state row and starts computing behind it. The reference keeps the same checkpoints in
rust/engine/src/mem/state_cache.rs (on block boundaries, beside the prefix cache).
"""
from __future__ import annotations

from collections import OrderedDict
from typing import Dict, List, Tuple

import torch


class StateCheckpoints:
    def __init__(self, rstate, budget_bytes: int):
        self.rstate = rstate
        self.budget = int(budget_bytes)
        self.used = 0
        self.items: "OrderedDict[bytes, Tuple[List[torch.Tensor], int]]" = OrderedDict()       # hash -> (rows, bytes), LRU first
        self.stats: Dict[str, int] = {"saved": 0, "restored": 0, "evicted": 0}

    def _pools(self) -> List[torch.Tensor]:
        r = self.rstate
        return [d[li] for d in (r.conv, r.scan, r.shift2) for li in sorted(d)]

    def has(self, h: bytes) -> bool:
        return h in self.items

    def save(self, h: bytes, slot: int) -> bool:
        """Copy row ``slot`` of every pool to host memory under ``h`` (after the kernels already queued on the stream)."""
        if h in self.items:
            self.items.move_to_end(h)
            return True
        rows = [p[slot].to("cpu", copy=True) for p in self._pools()]
        n = sum(t.numel() * t.element_size() for t in rows)
        if n > self.budget:
            return False
        while self.used + n > self.budget and self.items:
            _, (_, freed) = self.items.popitem(last=False)
            self.used -= freed
            self.stats["evicted"] += 1
        self.items[h] = (rows, n)
        self.used += n
        self.stats["saved"] += 1
        return True

    def restore(self, h: bytes, slot: int) -> bool:
        item = self.items.get(h)
        if item is None:
            return False
        self.items.move_to_end(h)
        for p, row in zip(self._pools(), item[0]):
            p[slot].copy_(row, non_blocking=False)
        self.stats["restored"] += 1
        return True
