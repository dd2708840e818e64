"""Host-memory and disk tier for prefix-cache blocks.

When the block manager has to reuse a cached prefix block, the block's KV (all layers, K and V) is
copied out and kept under its chain hash: first in host memory (LRU by bytes), and when that is full the
oldest entries move to one file per hash in a directory (LRU by bytes as well). A later request whose
prompt continues past the blocks still cached on the GPU gets the following blocks back from the tier
instead of recomputing them. Files carry a header with the KV layout, so a directory written by a
different model or cache dtype is ignored; files found at start-up are indexed, which re-warms the
cache after a restart (rust/engine/src/mem/kv_tier.rs:1-20 is the reference's tier; its directory comes
from FLLM_KV_DISK_DIR, which this class reads as a default too).
"""
from __future__ import annotations

import hashlib
import os
import struct
from collections import OrderedDict
from typing import Optional

import torch

_MAGIC = b"FLLMKVT1"


class KvTier:
    def __init__(self, signature: str, block_bytes: int, host_bytes: int = 0, disk_dir: Optional[str] = None,
                 disk_bytes: int = 0):
        self.sig = hashlib.sha256(signature.encode()).digest()[:16]
        self.block_bytes = int(block_bytes)
        self.host_cap, self.disk_cap = int(host_bytes), int(disk_bytes)
        self.host: "OrderedDict[bytes, torch.Tensor]" = OrderedDict()
        self.disk: "OrderedDict[bytes, int]" = OrderedDict()          # hash -> file size
        self.disk_dir = disk_dir if (disk_dir and self.disk_cap > 0) else None
        self.stats = {"stored": 0, "host_hits": 0, "disk_hits": 0, "spilled": 0, "dropped": 0, "rewarmed": 0}
        if self.disk_dir:
            os.makedirs(self.disk_dir, exist_ok=True)
            for name in sorted(os.listdir(self.disk_dir), key=lambda n: os.path.getmtime(os.path.join(self.disk_dir, n))):
                if not name.endswith(".kv"):
                    continue
                path = os.path.join(self.disk_dir, name)
                try:
                    with open(path, "rb") as f:
                        head = f.read(32)
                    ok = head[:8] == _MAGIC and head[8:24] == self.sig and struct.unpack("<Q", head[24:32])[0] == self.block_bytes
                    if ok:
                        self.disk[bytes.fromhex(name[:-3])] = os.path.getsize(path)
                        self.stats["rewarmed"] += 1
                except (OSError, ValueError):
                    continue
            self._trim_disk()

    # ------------------------------------------------------------------ queries
    @property
    def enabled(self) -> bool:
        return self.host_cap >= self.block_bytes or self.disk_dir is not None

    def has(self, h: bytes) -> bool:
        return h in self.host or h in self.disk

    def host_used(self) -> int:
        return len(self.host) * self.block_bytes

    def disk_used(self) -> int:
        return sum(self.disk.values())

    # ------------------------------------------------------------------ store / fetch
    def put(self, h: bytes, data: torch.Tensor) -> None:
        """data: the block's KV as a CPU uint8 tensor of block_bytes."""
        if not self.enabled or self.has(h):
            return
        assert data.numel() == self.block_bytes and data.dtype == torch.uint8
        self.stats["stored"] += 1
        if self.host_cap >= self.block_bytes:
            self.host[h] = data
            while self.host_used() > self.host_cap:
                old, blob = self.host.popitem(last=False)
                self._to_disk(old, blob)
        else:
            self._to_disk(h, data)

    def get(self, h: bytes) -> Optional[torch.Tensor]:
        blob = self.host.get(h)
        if blob is not None:
            self.host.move_to_end(h)
            self.stats["host_hits"] += 1
            return blob
        if h in self.disk:
            try:
                with open(self._path(h), "rb") as f:
                    f.seek(32)
                    raw = f.read(self.block_bytes)
                if len(raw) == self.block_bytes:
                    self.disk.move_to_end(h)
                    self.stats["disk_hits"] += 1
                    return torch.frombuffer(bytearray(raw), dtype=torch.uint8)
            except OSError:
                pass
            self.disk.pop(h, None)
        return None

    def clear(self) -> None:
        self.host.clear()
        for h in list(self.disk):
            self._unlink(h)
        self.disk.clear()

    # ------------------------------------------------------------------ disk
    def _path(self, h: bytes) -> str:
        return os.path.join(self.disk_dir, h.hex() + ".kv")

    def _unlink(self, h: bytes) -> None:
        try:
            os.remove(self._path(h))
        except OSError:
            pass

    def _to_disk(self, h: bytes, blob: torch.Tensor) -> None:
        if self.disk_dir is None:
            self.stats["dropped"] += 1
            return
        tmp = self._path(h) + ".tmp"
        try:
            with open(tmp, "wb") as f:
                f.write(_MAGIC + self.sig + struct.pack("<Q", self.block_bytes))
                f.write(blob.numpy().tobytes())
            os.replace(tmp, self._path(h))
        except OSError:
            self.stats["dropped"] += 1
            return
        self.disk[h] = 32 + self.block_bytes
        self.stats["spilled"] += 1
        self._trim_disk()

    def _trim_disk(self) -> None:
        while self.disk and self.disk_used() > self.disk_cap:
            old, _ = self.disk.popitem(last=False)
            self._unlink(old)
            self.stats["dropped"] += 1

    def info(self) -> dict:
        return dict(self.stats, host_blocks=len(self.host), disk_blocks=len(self.disk), host_bytes=self.host_used(),
                    disk_bytes=self.disk_used(), disk_dir=self.disk_dir)
