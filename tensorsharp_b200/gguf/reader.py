"""Memory-mapped GGUF reader.

Reads header, key/value metadata and tensor infos, then exposes every tensor as a
zero-copy ``uint8`` view of the mapped file: quantised blocks are never decoded here,
they are handed to the device repacker byte-for-byte.

Parity: TensorSharp.Runtime/GgufReader.cs:78-119 (header, KV section, tensor infos,
``general.alignment``, data offset), :121-193 (typed getters that accept array-typed
scalars), :271-283 (mmap views).  GGUF dims are stored ne0-first; ``shape`` below is
the reversed (row-major, outermost first) form the models use
(TensorSharp.Models/ModelBase.cs:618-624).
"""
from __future__ import annotations

import mmap
import os
import struct
from dataclasses import dataclass
from typing import Any, Dict, List, Optional, Tuple

import numpy as np

from .constants import (GGUF_DEFAULT_ALIGNMENT, GGUF_MAGIC, GGMLType, GGUFValueType,
                        tensor_bytes)

_SCALAR_FMT = {
    GGUFValueType.UINT8: "<B", GGUFValueType.INT8: "<b",
    GGUFValueType.UINT16: "<H", GGUFValueType.INT16: "<h",
    GGUFValueType.UINT32: "<I", GGUFValueType.INT32: "<i",
    GGUFValueType.FLOAT32: "<f", GGUFValueType.UINT64: "<Q",
    GGUFValueType.INT64: "<q", GGUFValueType.FLOAT64: "<d",
    GGUFValueType.BOOL: "<?",
}
_NP_DTYPE = {
    GGUFValueType.UINT8: np.uint8, GGUFValueType.INT8: np.int8,
    GGUFValueType.UINT16: np.uint16, GGUFValueType.INT16: np.int16,
    GGUFValueType.UINT32: np.uint32, GGUFValueType.INT32: np.int32,
    GGUFValueType.FLOAT32: np.float32, GGUFValueType.UINT64: np.uint64,
    GGUFValueType.INT64: np.int64, GGUFValueType.FLOAT64: np.float64,
    GGUFValueType.BOOL: np.bool_,
}


class GGUFFormatError(ValueError):
    """Raised for a file that is not a readable GGUF (bad magic, truncated, bad type)."""


@dataclass
class GGUFTensorInfo:
    name: str
    ne: Tuple[int, ...]          # GGUF order, ne[0] is the contiguous (row) dimension
    ggml_type: GGMLType
    offset: int                  # relative to the start of the data section
    nbytes: int

    @property
    def shape(self) -> Tuple[int, ...]:
        """Row-major shape, outermost dimension first."""
        return tuple(reversed(self.ne))

    @property
    def n_elements(self) -> int:
        n = 1
        for d in self.ne:
            n *= d
        return n


class GGUFFile:
    """An open GGUF file.  Use as a context manager or call :meth:`close`."""

    def __init__(self, path: str):
        self.path = path
        self._fh = open(path, "rb")
        size = os.fstat(self._fh.fileno()).st_size
        if size < 24:
            self._fh.close()
            raise GGUFFormatError(f"{path}: file too small to be GGUF ({size} bytes)")
        self._mm = mmap.mmap(self._fh.fileno(), 0, access=mmap.ACCESS_READ)
        self._buf = memoryview(self._mm)
        self._size = size
        self.metadata: Dict[str, Any] = {}
        self.metadata_types: Dict[str, GGUFValueType] = {}
        self.tensors: Dict[str, GGUFTensorInfo] = {}
        self.version = 0
        self.alignment = GGUF_DEFAULT_ALIGNMENT
        self.data_offset = 0
        try:
            self._parse()
        except (struct.error, IndexError) as exc:
            self.close()
            raise GGUFFormatError(f"{path}: truncated or corrupt GGUF header ({exc})") from exc
        except Exception:
            self.close()
            raise

    # ------------------------------------------------------------------ parsing
    def _rd(self, fmt: str, pos: int):
        return struct.unpack_from(fmt, self._buf, pos)[0], pos + struct.calcsize(fmt)

    def _rd_str(self, pos: int):
        n, pos = self._rd("<Q", pos)
        if pos + n > self._size:
            raise GGUFFormatError(f"{self.path}: string runs past end of file")
        return bytes(self._buf[pos:pos + n]).decode("utf-8", errors="replace"), pos + n

    def _rd_value(self, vt: GGUFValueType, pos: int):
        if vt == GGUFValueType.STRING:
            return self._rd_str(pos)
        if vt == GGUFValueType.ARRAY:
            et, pos = self._rd("<I", pos)
            et = GGUFValueType(et)
            n, pos = self._rd("<Q", pos)
            if et == GGUFValueType.STRING:
                out = []
                for _ in range(n):
                    s, pos = self._rd_str(pos)
                    out.append(s)
                return out, pos
            if et == GGUFValueType.ARRAY:
                out = []
                for _ in range(n):
                    v, pos = self._rd_value(et, pos)
                    out.append(v)
                return out, pos
            dt = np.dtype(_NP_DTYPE[et])
            nb = dt.itemsize * n
            if pos + nb > self._size:
                raise GGUFFormatError(f"{self.path}: array runs past end of file")
            arr = np.frombuffer(self._buf, dtype=dt, count=n, offset=pos)
            return arr.tolist(), pos + nb
        if vt not in _SCALAR_FMT:
            raise GGUFFormatError(f"{self.path}: unknown metadata value type {int(vt)}")
        return self._rd(_SCALAR_FMT[vt], pos)

    def _parse(self) -> None:
        pos = 0
        magic, pos = self._rd("<I", pos)
        if magic != GGUF_MAGIC:
            raise GGUFFormatError(f"{self.path}: bad magic 0x{magic:08x}, not a GGUF file")
        self.version, pos = self._rd("<I", pos)
        if self.version < 2:
            raise GGUFFormatError(f"{self.path}: GGUF version {self.version} < 2 is unsupported")
        n_tensors, pos = self._rd("<Q", pos)
        n_kv, pos = self._rd("<Q", pos)
        for _ in range(n_kv):
            key, pos = self._rd_str(pos)
            vt, pos = self._rd("<I", pos)
            try:
                vt = GGUFValueType(vt)
            except ValueError as exc:
                raise GGUFFormatError(f"{self.path}: key {key!r} has unknown type {vt}") from exc
            val, pos = self._rd_value(vt, pos)
            self.metadata[key] = val
            self.metadata_types[key] = vt
        infos: List[GGUFTensorInfo] = []
        for _ in range(n_tensors):
            name, pos = self._rd_str(pos)
            nd, pos = self._rd("<I", pos)
            ne = []
            for _ in range(nd):
                d, pos = self._rd("<Q", pos)
                ne.append(int(d))
            tt, pos = self._rd("<I", pos)
            off, pos = self._rd("<Q", pos)
            try:
                gt = GGMLType(tt)
            except ValueError as exc:
                raise GGUFFormatError(f"{self.path}: tensor {name!r} has unknown ggml type {tt}") from exc
            infos.append(GGUFTensorInfo(name, tuple(ne), gt, int(off), tensor_bytes(gt, ne or (1,))))
        self.alignment = int(self.get_scalar("general.alignment", GGUF_DEFAULT_ALIGNMENT))
        a = self.alignment
        self.data_offset = (pos + a - 1) // a * a
        for ti in infos:
            if self.data_offset + ti.offset + ti.nbytes > self._size:
                raise GGUFFormatError(
                    f"{self.path}: tensor {ti.name!r} ({ti.nbytes} bytes at {ti.offset}) runs past end of file")
            self.tensors[ti.name] = ti

    # ------------------------------------------------------------------ metadata getters
    def get_scalar(self, key: str, default=None):
        """Value of ``key``; a one-element (or longer) array yields its first element."""
        v = self.metadata.get(key, None)
        if v is None:
            return default
        if isinstance(v, list):
            return v[0] if v else default
        return v

    def get_int(self, key: str, default: int = 0) -> int:
        v = self.get_scalar(key, None)
        return default if v is None else int(v)

    def get_float(self, key: str, default: float = 0.0) -> float:
        v = self.get_scalar(key, None)
        return default if v is None else float(v)

    def get_bool(self, key: str, default: bool = False) -> bool:
        v = self.get_scalar(key, None)
        return default if v is None else bool(v)

    def get_str(self, key: str, default: Optional[str] = None) -> Optional[str]:
        v = self.get_scalar(key, None)
        return default if v is None else str(v)

    def get_array(self, key: str, default=None):
        """Array value of ``key``; a scalar is wrapped into a one-element list."""
        v = self.metadata.get(key, None)
        if v is None:
            return default
        return v if isinstance(v, list) else [v]

    # ------------------------------------------------------------------ tensor access
    def has_tensor(self, name: str) -> bool:
        return name in self.tensors

    def tensor_bytes_view(self, name: str) -> np.ndarray:
        """Zero-copy ``uint8`` view of the tensor's raw blocks inside the mapped file."""
        ti = self.tensors[name]
        return np.frombuffer(self._buf, dtype=np.uint8, count=ti.nbytes,
                             offset=self.data_offset + ti.offset)

    def adjacent(self, first: str, second: str) -> bool:
        """True when ``second`` starts exactly where ``first`` ends, so the two can be viewed
        as one concatenated tensor without a copy (ModelBase.cs:24-202, concatenated views)."""
        a, b = self.tensors[first], self.tensors[second]
        return a.offset + a.nbytes == b.offset

    def close(self) -> None:
        buf = getattr(self, "_buf", None)
        if buf is not None:
            try:
                buf.release()
            except BufferError:
                pass
            self._buf = None
        mm = getattr(self, "_mm", None)
        if mm is not None:
            try:
                mm.close()
            except BufferError:
                pass  # numpy views still alive; the mapping is released with them
            self._mm = None
        fh = getattr(self, "_fh", None)
        if fh is not None:
            fh.close()
            self._fh = None

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()
        return False
