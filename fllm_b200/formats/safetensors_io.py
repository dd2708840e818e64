"""Minimal safetensors reader/writer (mmap, zero-copy): an 8-byte little-endian header length,
a JSON header {name: {dtype, shape, data_offsets}}, then raw tensor bytes. Packed payloads
(uint8 / int32 code tensors, fp8 bytes, scale tensors) are returned as they are stored, which is
how quantised checkpoints stay packed on their way to the GPU
(rust/checkpoint/src/safetensors.rs plays this role in the reference)."""
from __future__ import annotations

import json
import mmap
import os
import struct
import warnings
from typing import Dict, Iterable, List, Tuple

import numpy as np
import torch

_DT = {"F32": (np.float32, torch.float32), "F16": (np.float16, torch.float16), "BF16": (np.uint16, torch.bfloat16),
       "I32": (np.int32, torch.int32), "I64": (np.int64, torch.int64), "U8": (np.uint8, torch.uint8),
       "I8": (np.int8, torch.int8), "F8_E4M3": (np.uint8, torch.float8_e4m3fn), "F8_E5M2": (np.uint8, torch.float8_e5m2),
       "BOOL": (np.bool_, torch.bool), "I16": (np.int16, torch.int16), "F64": (np.float64, torch.float64),
       "U16": (np.uint16, torch.uint16), "U32": (np.uint32, torch.uint32), "U64": (np.uint64, torch.uint64)}
_NAME = {v[1]: k for k, v in _DT.items()}


class SafetensorsError(ValueError):
    pass


class SafetensorsFile:
    def __init__(self, path: str):
        self.path = path
        self._f = open(path, "rb")
        size = os.fstat(self._f.fileno()).st_size
        if size < 8:
            raise SafetensorsError("file too short")
        n, = struct.unpack("<Q", self._f.read(8))
        if n > size - 8 or n > (100 << 20):
            raise SafetensorsError("implausible header length")
        try:
            self.header = json.loads(self._f.read(n))
        except Exception as e:
            raise SafetensorsError(f"bad JSON header: {e}")
        self.meta = self.header.pop("__metadata__", {})
        self._base = 8 + n
        self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ)
        for name, t in self.header.items():
            a, b = t["data_offsets"]
            if t["dtype"] not in _DT or a > b or self._base + b > size:
                raise SafetensorsError(f"tensor {name!r} is malformed")

    def keys(self) -> List[str]:
        return list(self.header)

    def tensor(self, name: str) -> torch.Tensor:
        t = self.header[name]
        npdt, tdt = _DT[t["dtype"]]
        a, b = t["data_offsets"]
        arr = np.frombuffer(self._mm, dtype=npdt, count=(b - a) // np.dtype(npdt).itemsize, offset=self._base + a)
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")          # the mapping is read-only by design
            out = torch.from_numpy(arr.reshape(t["shape"]) if t["shape"] else arr.reshape(()))
        return out.view(tdt) if out.dtype != tdt else out

    def close(self) -> None:
        try:
            self._mm.close()
        except BufferError:
            pass
        self._f.close()


def open_checkpoint(directory: str) -> Dict[str, Tuple[SafetensorsFile, str]]:
    """name -> (file, name) over every *.safetensors of a checkpoint directory (index-aware); a directory that holds
    ``pytorch_model.bin`` files instead is read through ``formats.torch_zip``."""
    files = {}
    out: Dict[str, Tuple[SafetensorsFile, str]] = {}
    idx = os.path.join(directory, "model.safetensors.index.json")
    names = sorted(f for f in os.listdir(directory) if f.endswith(".safetensors"))
    if not names and not os.path.exists(idx):
        # a PyTorch zip checkpoint (pytorch_model.bin and shards): same interface, read without running its pickle
        from .torch_zip import open_torch_checkpoint
        return open_torch_checkpoint(directory)
    if os.path.exists(idx):
        wm = json.load(open(idx))["weight_map"]
        for tname, fname in wm.items():
            if fname not in files:
                files[fname] = SafetensorsFile(os.path.join(directory, fname))
            out[tname] = (files[fname], tname)
        return out
    for fname in names:
        f = SafetensorsFile(os.path.join(directory, fname))
        for k in f.keys():
            out[k] = (f, k)
    return out


def save_file(tensors: Dict[str, torch.Tensor], path: str, metadata: Dict[str, str] = None) -> None:
    header, blobs, off = {}, [], 0
    for name, t in tensors.items():
        t = t.contiguous().cpu()
        raw = t.view(torch.uint8).numpy().tobytes() if t.numel() else b""
        header[name] = {"dtype": _NAME[t.dtype], "shape": list(t.shape), "data_offsets": [off, off + len(raw)]}
        blobs.append(raw)
        off += len(raw)
    if metadata:
        header["__metadata__"] = metadata
    hj = json.dumps(header, separators=(",", ":")).encode()
    hj += b" " * ((-len(hj)) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hj)) + hj)
        for b in blobs:
            f.write(b)
