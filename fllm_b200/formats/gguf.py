"""GGUF v3 reader (mmap, zero-copy tensor views) and writer.

The reader plays the role of the reference's ``MappedGguf`` (rust/gguf-probe/src/lib.rs:
576-900: metadata, tensor index, validated zero-copy tensor bytes); the writer is what
``rust/checkpoint/src/gguf.rs`` does for converted checkpoints. Packed tensors stay
packed: a tensor is handed out as a ``numpy`` byte view of the file plus its GGML type.
"""
from __future__ import annotations

import mmap
import struct
from dataclasses import dataclass
from typing import Any, BinaryIO, Dict, List, Optional, Tuple

import numpy as np

MAGIC = b"GGUF"
# value types
U8, I8, U16, I16, U32, I32, F32, BOOL, STR, ARR, U64, I64, F64 = range(13)
_SCALAR = {U8: "<B", I8: "<b", U16: "<H", I16: "<h", U32: "<I", I32: "<i", F32: "<f", BOOL: "<?",
           U64: "<Q", I64: "<q", F64: "<d"}

# GGML tensor types: id -> (name, block elements, block bytes)
GGML_TYPES: Dict[int, Tuple[str, int, int]] = {
    0: ("F32", 1, 4), 1: ("F16", 1, 2), 2: ("Q4_0", 32, 18), 3: ("Q4_1", 32, 20), 6: ("Q5_0", 32, 22),
    7: ("Q5_1", 32, 24), 8: ("Q8_0", 32, 34), 9: ("Q8_1", 32, 36), 10: ("Q2_K", 256, 84),
    11: ("Q3_K", 256, 110), 12: ("Q4_K", 256, 144), 13: ("Q5_K", 256, 176), 14: ("Q6_K", 256, 210),
    15: ("Q8_K", 256, 292), 16: ("IQ2_XXS", 256, 66), 17: ("IQ2_XS", 256, 74), 18: ("IQ3_XXS", 256, 98),
    19: ("IQ1_S", 256, 50), 20: ("IQ4_NL", 32, 18), 21: ("IQ3_S", 256, 110), 22: ("IQ2_S", 256, 82),
    23: ("IQ4_XS", 256, 136), 24: ("I8", 1, 1), 25: ("I16", 1, 2), 26: ("I32", 1, 4), 27: ("I64", 1, 8),
    28: ("F64", 1, 8), 29: ("IQ1_M", 256, 56), 30: ("BF16", 1, 2), 39: ("MXFP4", 32, 17),
}
TYPE_ID = {v[0]: k for k, v in GGML_TYPES.items()}


class GgufError(ValueError):
    pass


@dataclass
class TensorInfo:
    name: str
    shape: Tuple[int, ...]        # outermost first (rows, cols): GGUF stores innermost first
    ggml_type: int
    offset: int                   # absolute file offset
    nbytes: int

    @property
    def type_name(self) -> str:
        return GGML_TYPES[self.ggml_type][0]


def tensor_nbytes(ggml_type: int, shape: Tuple[int, ...]) -> int:
    if ggml_type not in GGML_TYPES:
        raise GgufError(f"unknown GGML type id {ggml_type}")
    _, bs, bb = GGML_TYPES[ggml_type]
    inner = shape[-1] if shape else 1
    if inner % bs:
        raise GgufError(f"row length {inner} is not a multiple of the block size {bs}")
    n = 1
    for d in shape:
        n *= d
    return n // bs * bb


class GgufReader:
    def __init__(self, path: str):
        self.path = path
        self._f = open(path, "rb")
        self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ)
        self._buf = memoryview(self._mm)
        self.metadata: Dict[str, Any] = {}
        self.value_types: Dict[str, int] = {}
        self.tensors: Dict[str, TensorInfo] = {}
        self._parse()

    # -------------------------------------------------------------- parsing
    def _need(self, pos: int, n: int) -> None:
        if n < 0 or pos + n > len(self._buf):
            raise GgufError("truncated GGUF file")

    def _scalar(self, pos: int, vt: int):
        fmt = _SCALAR[vt]
        n = struct.calcsize(fmt)
        self._need(pos, n)
        return struct.unpack_from(fmt, self._buf, pos)[0], pos + n

    def _string(self, pos: int):
        n, pos = self._scalar(pos, U64)
        if n > (1 << 30):
            raise GgufError("implausible string length")
        self._need(pos, n)
        return bytes(self._buf[pos:pos + n]).decode("utf-8", errors="replace"), pos + n

    def _value(self, pos: int, vt: int, depth: int = 0):
        if vt in _SCALAR:
            return self._scalar(pos, vt)
        if vt == STR:
            return self._string(pos)
        if vt == ARR:
            if depth > 4:
                raise GgufError("array nesting too deep")
            et, pos = self._scalar(pos, U32)
            n, pos = self._scalar(pos, U64)
            if n > (1 << 28):
                raise GgufError("implausible array length")
            if et in _SCALAR:
                fmt = _SCALAR[et]
                sz = struct.calcsize(fmt)
                self._need(pos, n * sz)
                arr = np.frombuffer(self._buf, dtype=np.dtype(fmt), count=n, offset=pos)
                return arr, pos + n * sz
            out = []
            for _ in range(n):
                v, pos = self._value(pos, et, depth + 1)
                out.append(v)
            return out, pos
        raise GgufError(f"unknown metadata value type {vt}")

    def _parse(self) -> None:
        self._need(0, 24)
        if bytes(self._buf[:4]) != MAGIC:
            raise GgufError("not a GGUF file")
        version, = struct.unpack_from("<I", self._buf, 4)
        if version not in (2, 3):
            raise GgufError(f"unsupported GGUF version {version}")
        n_tensors, n_kv = struct.unpack_from("<QQ", self._buf, 8)
        if n_tensors > (1 << 24) or n_kv > (1 << 24):
            raise GgufError("implausible header counts")
        pos = 24
        for _ in range(n_kv):
            key, pos = self._string(pos)
            vt, pos = self._scalar(pos, U32)
            val, pos = self._value(pos, vt)
            self.metadata[key] = val
            if vt != ARR:
                self.value_types[key] = vt           # so that a rewrite keeps u32 / i64 / f64 ... as they were
        infos = []
        for _ in range(n_tensors):
            name, pos = self._string(pos)
            nd, pos = self._scalar(pos, U32)
            if nd > 8:
                raise GgufError("too many tensor dimensions")
            dims = []
            for _ in range(nd):
                d, pos = self._scalar(pos, U64)
                dims.append(d)
            gt, pos = self._scalar(pos, U32)
            off, pos = self._scalar(pos, U64)
            infos.append((name, tuple(reversed(dims)), gt, off))
        align = int(self.metadata.get("general.alignment", 32)) or 32
        data_start = (pos + align - 1) // align * align
        for name, shape, gt, off in infos:
            nbytes = tensor_nbytes(gt, shape)
            absolute = data_start + off
            if off % align or absolute + nbytes > len(self._buf):
                raise GgufError(f"tensor {name!r} lies outside the file or is misaligned")
            self.tensors[name] = TensorInfo(name, shape, gt, absolute, nbytes)

    # -------------------------------------------------------------- access
    def tensor_bytes(self, name: str) -> np.ndarray:
        """Zero-copy uint8 view of a tensor's packed bytes."""
        t = self.tensors[name]
        return np.frombuffer(self._buf, dtype=np.uint8, count=t.nbytes, offset=t.offset)

    def tensor_f32(self, name: str) -> np.ndarray:
        """Dequantised copy (any supported type) through the native codecs."""
        from .quant import dequantize
        t = self.tensors[name]
        rows = int(np.prod(t.shape[:-1])) if len(t.shape) > 1 else 1
        return dequantize(self.tensor_bytes(name), t.ggml_type, rows, t.shape[-1]).reshape(t.shape)

    def close(self) -> None:
        """Unmap the file. Zero-copy views handed out by ``tensor_bytes`` keep the mapping alive: while one
        exists the mapping is left to the garbage collector instead."""
        try:
            self._buf.release()
            self._mm.close()
        except BufferError:
            pass
        self._f.close()


class GgufWriter:
    def __init__(self, path: str, alignment: int = 32):
        self.path, self.alignment = path, alignment
        self.meta: List[Tuple[str, int, Any]] = []
        self.tensors: List[Tuple[str, Tuple[int, ...], int, np.ndarray]] = []

    def add(self, key: str, value: Any, vtype: Optional[int] = None) -> None:
        if vtype is None:
            if isinstance(value, bool):
                vtype = BOOL
            elif isinstance(value, int):
                vtype = U32 if 0 <= value < (1 << 32) else I64
            elif isinstance(value, float):
                vtype = F32
            elif isinstance(value, str):
                vtype = STR
            elif isinstance(value, (list, tuple, np.ndarray)):
                vtype = ARR
            else:
                raise TypeError(f"cannot infer GGUF type of {type(value)}")
        self.meta.append((key, vtype, value))

    def add_tensor(self, name: str, shape: Tuple[int, ...], ggml_type: int, data: np.ndarray) -> None:
        data = np.ascontiguousarray(data).view(np.uint8).reshape(-1)
        if data.size != tensor_nbytes(ggml_type, tuple(shape)):
            raise GgufError(f"tensor {name!r}: {data.size} bytes do not match its shape and type")
        self.tensors.append((name, tuple(shape), ggml_type, data))

    @staticmethod
    def _s(s: str) -> bytes:
        b = s.encode()
        return struct.pack("<Q", len(b)) + b

    def _val(self, vt: int, v: Any) -> bytes:
        if vt in _SCALAR:
            return struct.pack(_SCALAR[vt], v)
        if vt == STR:
            return self._s(v)
        if vt == ARR:
            if isinstance(v, np.ndarray):
                et = {np.dtype("int32"): I32, np.dtype("uint32"): U32, np.dtype("float32"): F32,
                      np.dtype("int64"): I64, np.dtype("uint8"): U8}[v.dtype]
                return struct.pack("<IQ", et, v.size) + v.tobytes()
            v = list(v)
            if v and isinstance(v[0], str):
                return struct.pack("<IQ", STR, len(v)) + b"".join(self._s(x) for x in v)
            if v and isinstance(v[0], float):
                return struct.pack("<IQ", F32, len(v)) + struct.pack(f"<{len(v)}f", *v)
            return struct.pack("<IQ", I32, len(v)) + struct.pack(f"<{len(v)}i", *v)
        raise TypeError(vt)

    def write(self) -> None:
        head = bytearray(MAGIC + struct.pack("<IQQ", 3, len(self.tensors), len(self.meta) + 1))
        head += self._s("general.alignment") + struct.pack("<I", U32) + struct.pack("<I", self.alignment)
        for key, vt, v in self.meta:
            head += self._s(key) + struct.pack("<I", vt) + self._val(vt, v)
        off = 0
        offsets = []
        for name, shape, gt, data in self.tensors:
            head += self._s(name) + struct.pack("<I", len(shape))
            for d in reversed(shape):
                head += struct.pack("<Q", d)
            head += struct.pack("<IQ", gt, off)
            offsets.append(off)
            off = (off + data.size + self.alignment - 1) // self.alignment * self.alignment
        pad = (-len(head)) % self.alignment
        with open(self.path, "wb") as f:
            f.write(head + b"\0" * pad)
            for (name, shape, gt, data), o in zip(self.tensors, offsets):
                f.write(data.tobytes())
                f.write(b"\0" * ((-data.size) % self.alignment))
