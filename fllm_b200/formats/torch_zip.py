"""Reader for PyTorch's zip checkpoints (``pytorch_model.bin``, ``*.pt`` written by ``torch.save``) without running
their pickle: a restricted unpickler accepts only the handful of constructors a state dict needs (ordered dicts,
tensor rebuild functions, storage type tags) and refuses everything else, and tensors are views of the archive's
storage files read on demand. Offers the interface of ``SafetensorsFile`` (``keys`` / ``tensor`` / ``close``), so
the checkpoint loaders take either. The reference reads these files in rust/checkpoint/src/pytorch.rs."""
from __future__ import annotations

import json
import os
import pickle
import zipfile
from typing import Dict, List, Tuple

import numpy as np
import torch

_DTYPES = {
    "FloatStorage": (torch.float32, np.float32), "HalfStorage": (torch.float16, np.float16),
    "BFloat16Storage": (torch.bfloat16, np.uint16), "DoubleStorage": (torch.float64, np.float64),
    "LongStorage": (torch.int64, np.int64), "IntStorage": (torch.int32, np.int32), "ShortStorage": (torch.int16, np.int16),
    "CharStorage": (torch.int8, np.int8), "ByteStorage": (torch.uint8, np.uint8), "BoolStorage": (torch.bool, np.bool_),
    "Float8_e4m3fnStorage": (torch.float8_e4m3fn, np.uint8), "Float8_e5m2Storage": (torch.float8_e5m2, np.uint8),
}


class TorchZipError(ValueError):
    pass


class _StorageTag:
    def __init__(self, name: str):
        self.name = name


class _LazyTensor:
    """What the unpickler builds in place of a tensor: where its bytes are and how to view them."""

    def __init__(self, key: str, dtype_name: str, offset: int, size: Tuple[int, ...], stride: Tuple[int, ...]):
        self.key, self.dtype_name, self.offset, self.size, self.stride = key, dtype_name, offset, tuple(size), tuple(stride)


def _rebuild_tensor_v2(storage, storage_offset, size, stride, requires_grad=False, backward_hooks=None, metadata=None):
    key, dtype_name = storage
    return _LazyTensor(key, dtype_name, int(storage_offset), tuple(int(s) for s in size), tuple(int(s) for s in stride))


def _rebuild_parameter(data, requires_grad=False, backward_hooks=None):
    return data


class _Unpickler(pickle.Unpickler):
    _ALLOWED = {
        ("collections", "OrderedDict"): __import__("collections").OrderedDict,
        ("torch._utils", "_rebuild_tensor_v2"): _rebuild_tensor_v2,
        ("torch._utils", "_rebuild_parameter"): _rebuild_parameter,
    }

    def find_class(self, module, name):
        if (module, name) in self._ALLOWED:
            return self._ALLOWED[(module, name)]
        if module == "torch" and name in _DTYPES:
            return _StorageTag(name)
        raise TorchZipError(f"refusing to unpickle {module}.{name}: not part of a plain state dict")

    def persistent_load(self, pid):
        # ('storage', storage type, key, location, numel)
        if not (isinstance(pid, tuple) and len(pid) >= 3 and pid[0] == "storage" and isinstance(pid[1], _StorageTag)):
            raise TorchZipError("unexpected persistent id in the checkpoint")
        return (str(pid[2]), pid[1].name)


class TorchZipFile:
    def __init__(self, path: str):
        self.path = path
        try:
            self.zf = zipfile.ZipFile(path)
        except zipfile.BadZipFile as e:
            raise TorchZipError(f"{path}: not a zip checkpoint ({e}); legacy (pre-1.6) pickles are not read") from e
        pkl = [n for n in self.zf.namelist() if n.endswith("/data.pkl") or n == "data.pkl"]
        if len(pkl) != 1:
            raise TorchZipError(f"{path}: expected one data.pkl, found {len(pkl)}")
        self.root = pkl[0][: -len("data.pkl")]
        try:
            with self.zf.open(pkl[0]) as f:
                obj = _Unpickler(f).load()
        except TorchZipError:
            raise
        except Exception as e:                      # truncated or hostile pickles
            raise TorchZipError(f"{path}: cannot read the state dict ({type(e).__name__}: {e})") from e
        if isinstance(obj, dict) and "state_dict" in obj and isinstance(obj["state_dict"], dict):
            obj = obj["state_dict"]
        if not isinstance(obj, dict):
            raise TorchZipError(f"{path}: the checkpoint is not a dictionary of tensors")
        self.entries: Dict[str, _LazyTensor] = {k: v for k, v in obj.items() if isinstance(v, _LazyTensor)}

    def keys(self) -> List[str]:
        return list(self.entries)

    def tensor(self, name: str) -> torch.Tensor:
        e = self.entries[name]
        tdt, ndt = _DTYPES[e.dtype_name]
        raw = self.zf.read(f"{self.root}data/{e.key}")
        flat = np.frombuffer(raw, dtype=ndt)
        n = 1
        for s in e.size:
            n *= s
        # contiguous tensors only need a slice; others go through as_strided on the whole storage
        t = torch.from_numpy(flat.copy())
        if tdt in (torch.bfloat16, torch.float8_e4m3fn, torch.float8_e5m2):
            t = t.view(tdt)
        if e.size == ():
            return t[e.offset].clone()
        need = e.offset + sum((s - 1) * st for s, st in zip(e.size, e.stride)) + 1 if n else e.offset
        if need > t.numel():
            raise TorchZipError(f"{self.path}: tensor {name} reaches past its storage")
        return torch.as_strided(t, e.size, e.stride, e.offset).contiguous()

    def close(self) -> None:
        self.zf.close()


def open_torch_checkpoint(directory: str) -> Dict[str, Tuple[TorchZipFile, str]]:
    """name -> (file, name) over ``pytorch_model.bin`` or its shards (``pytorch_model.bin.index.json``)."""
    out: Dict[str, Tuple[TorchZipFile, str]] = {}
    idx = os.path.join(directory, "pytorch_model.bin.index.json")
    files: Dict[str, TorchZipFile] = {}
    if os.path.exists(idx):
        for tname, fname in json.load(open(idx))["weight_map"].items():
            if fname not in files:
                files[fname] = TorchZipFile(os.path.join(directory, fname))
            out[tname] = (files[fname], tname)
        return out
    names = sorted(f for f in os.listdir(directory) if f.endswith(".bin") or f.endswith(".pt") or f.endswith(".pth"))
    for fname in names:
        f = TorchZipFile(os.path.join(directory, fname))
        for k in f.keys():
            out[k] = (f, k)
    return out
