"""GGUF writer.

The reference only reads GGUF; a writer is needed here because the benchmark models
are random-initialised and serialised to GGUF before the engine loads them, so that the
loader, repacker and kernels all see the on-disk block layouts.

Layout written (GGUF v3): header, metadata KV, tensor infos, padding to
``general.alignment``, then each tensor's raw blocks padded to the alignment.
Parity for the layout rules: TensorSharp.Runtime/GgufReader.cs:78-119.
"""
from __future__ import annotations

import struct
from typing import Any, Callable, List, Sequence, Tuple, Union

import numpy as np

from .constants import (GGUF_DEFAULT_ALIGNMENT, GGUF_MAGIC, GGUF_VERSION, GGMLType,
                        GGUFValueType, tensor_bytes)

_SCALAR_FMT = {
    GGUFValueType.UINT8: "<B", GGUFValueType.INT8: "<b",
    GGUFValueType.UINT16: "<H", GGUFValueType.INT16: "<h",
    GGUFValueType.UINT32: "<I", GGUFValueType.INT32: "<i",
    GGUFValueType.FLOAT32: "<f", GGUFValueType.UINT64: "<Q",
    GGUFValueType.INT64: "<q", GGUFValueType.FLOAT64: "<d",
    GGUFValueType.BOOL: "<?",
}

TensorSource = Union[np.ndarray, bytes, Callable[[], Any]]


def _infer_type(v) -> GGUFValueType:
    if isinstance(v, bool):
        return GGUFValueType.BOOL
    if isinstance(v, int):
        return GGUFValueType.UINT32 if 0 <= v < 2 ** 32 else GGUFValueType.INT64
    if isinstance(v, float):
        return GGUFValueType.FLOAT32
    if isinstance(v, str):
        return GGUFValueType.STRING
    if isinstance(v, (list, tuple)):
        return GGUFValueType.ARRAY
    raise TypeError(f"cannot infer GGUF type for {type(v)}")


def _to_bytes(src) -> bytes:
    if callable(src):
        src = src()
    if isinstance(src, (bytes, bytearray, memoryview)):
        return bytes(src)
    if isinstance(src, np.ndarray):
        return np.ascontiguousarray(src).tobytes()
    # torch tensor (kept duck-typed so this module does not import torch)
    if hasattr(src, "detach"):
        t = src.detach().contiguous().cpu()
        return t.view(-1).view(dtype=__import__("torch").uint8).numpy().tobytes()
    raise TypeError(f"unsupported tensor source {type(src)}")


class GGUFWriter:
    def __init__(self, path: str, alignment: int = GGUF_DEFAULT_ALIGNMENT):
        self.path = path
        self.alignment = alignment
        self._kv: List[Tuple[str, GGUFValueType, Any, Any]] = []
        self._tensors: List[Tuple[str, Tuple[int, ...], GGMLType, int, TensorSource]] = []

    # ------------------------------------------------------------------ metadata
    def add(self, key: str, value, vtype: GGUFValueType = None, elem_type: GGUFValueType = None):
        """Add one metadata entry; types are inferred from the Python value unless given."""
        vtype = GGUFValueType(vtype) if vtype is not None else _infer_type(value)
        if vtype == GGUFValueType.ARRAY and elem_type is None:
            elem_type = _infer_type(value[0]) if len(value) else GGUFValueType.UINT32
            if elem_type == GGUFValueType.UINT32 and any((x < 0) for x in value):
                elem_type = GGUFValueType.INT32
        self._kv.append((key, vtype, value, elem_type))
        return self

    # ------------------------------------------------------------------ tensors
    def add_tensor(self, name: str, shape: Sequence[int], ggml_type: GGMLType, data: TensorSource):
        """Register a tensor.  ``shape`` is row-major (outermost first); it is stored
        reversed, ne0-first, as GGUF requires.  ``data`` is the raw block bytes (numpy
        array, bytes, torch tensor) or a zero-argument callable producing them at write
        time, which keeps peak host memory at one tensor for large synthetic models."""
        ne = tuple(int(d) for d in reversed(tuple(shape)))
        nbytes = tensor_bytes(GGMLType(ggml_type), ne)
        self._tensors.append((name, ne, GGMLType(ggml_type), nbytes, data))
        return self

    # ------------------------------------------------------------------ serialisation
    @staticmethod
    def _pack_str(s: str) -> bytes:
        b = s.encode("utf-8")
        return struct.pack("<Q", len(b)) + b

    def _pack_value(self, vt: GGUFValueType, v, et: GGUFValueType = None) -> bytes:
        if vt == GGUFValueType.STRING:
            return self._pack_str(v)
        if vt == GGUFValueType.ARRAY:
            out = [struct.pack("<IQ", int(et), len(v))]
            if et == GGUFValueType.STRING:
                out.extend(self._pack_str(x) for x in v)
            else:
                fmt = _SCALAR_FMT[et]
                out.append(struct.pack("<" + fmt[1] * len(v), *v) if len(v) else b"")
            return b"".join(out)
        return struct.pack(_SCALAR_FMT[vt], v)

    def write(self) -> int:
        """Serialise to ``self.path``; returns the file size in bytes."""
        a = self.alignment
        kv = list(self._kv)
        if not any(k == "general.alignment" for k, *_ in kv):
            kv.append(("general.alignment", GGUFValueType.UINT32, a, None))
        head = [struct.pack("<IIQQ", GGUF_MAGIC, GGUF_VERSION, len(self._tensors), len(kv))]
        for key, vt, v, et in kv:
            head.append(self._pack_str(key))
            head.append(struct.pack("<I", int(vt)))
            head.append(self._pack_value(vt, v, et))
        off = 0
        for name, ne, gt, nbytes, _ in self._tensors:
            head.append(self._pack_str(name))
            head.append(struct.pack("<I", len(ne)))
            head.append(struct.pack("<" + "Q" * len(ne), *ne))
            head.append(struct.pack("<IQ", int(gt), off))
            off += (nbytes + a - 1) // a * a
        blob = b"".join(head)
        pad = (-len(blob)) % a
        with open(self.path, "wb") as fh:
            fh.write(blob)
            fh.write(b"\0" * pad)
            for name, ne, gt, nbytes, src in self._tensors:
                raw = _to_bytes(src)
                if len(raw) != nbytes:
                    raise ValueError(f"tensor {name}: got {len(raw)} bytes, expected {nbytes} "
                                     f"for {gt.name} ne={ne}")
                fh.write(raw)
                fh.write(b"\0" * ((-nbytes) % a))
            return fh.tell()
