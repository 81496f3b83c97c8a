"""Quantised weight matrices as the kernels see them.

A :class:`QuantWeight` is a ``[N, K]`` matrix (``N`` output features, rows of ``K``
values) or a stack of ``E`` such matrices (mixture-of-experts), held either as raw GGUF
blocks on the host (CPU oracle path) or as 16-byte-aligned planes on the device.

Plane layouts per type (device):
  Q4_K / Q5_K : one plane, the GGUF blocks unchanged (144 / 176 bytes are multiples of 16)
  Q8_0        : int8 qs[N][K], half d[N][K/32]
  Q4_0        : u8 qs[N][K/2], half d[N][K/32]
  MXFP4       : u8 qs[N][K/2], u8 e8m0[N][K/32]
  Q6_K        : u8 ql[N][K/2], u8 qh[N][K/4], int8 sc[N][K/16], half d[N][K/256]
  BF16 / F16 / F32 : the values
Every other GGUF type is decoded to BF16 once at load time.

Parity: TensorSharp.Models/ModelBase.cs:24-202 (QuantizedWeight), :660-706 (one-time
device upload), TensorSharp.GGML.Native/ggml_ops_core.cpp:1199-1318 (preload).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional, Sequence

import torch

from ..gguf.constants import GGMLType, block_size, type_size
from . import codecs

_NATIVE = {GGMLType.Q4_K, GGMLType.Q5_K, GGMLType.Q6_K, GGMLType.Q8_0, GGMLType.Q4_0, GGMLType.MXFP4,
           GGMLType.BF16, GGMLType.F16, GGMLType.F32}
Q8_ACT_TYPES = {GGMLType.Q4_K, GGMLType.Q5_K, GGMLType.Q6_K, GGMLType.Q8_0, GGMLType.Q4_0, GGMLType.MXFP4}


def _split_planes(raw: torch.Tensor, t: GGMLType, rows: int, K: int) -> List[torch.Tensor]:
    """Re-arrange raw GGUF blocks (uint8, on any device) into aligned planes."""
    nb = rows * (K // block_size(t))
    b = raw.reshape(nb, type_size(t))
    if t in (GGMLType.Q4_K, GGMLType.Q5_K, GGMLType.BF16, GGMLType.F16, GGMLType.F32):
        return [raw.reshape(-1).contiguous()]
    if t == GGMLType.Q8_0:
        return [b[:, 2:34].contiguous().view(-1), b[:, 0:2].contiguous().view(-1)]
    if t == GGMLType.Q4_0:
        return [b[:, 2:18].contiguous().view(-1), b[:, 0:2].contiguous().view(-1)]
    if t == GGMLType.MXFP4:
        return [b[:, 1:17].contiguous().view(-1), b[:, 0:1].contiguous().view(-1)]
    if t == GGMLType.Q6_K:
        return [b[:, 0:128].contiguous().view(-1), b[:, 128:192].contiguous().view(-1),
                b[:, 192:208].contiguous().view(-1), b[:, 208:210].contiguous().view(-1)]
    raise NotImplementedError(t)


def _join_planes(planes: Sequence[torch.Tensor], t: GGMLType, rows: int, K: int) -> torch.Tensor:
    """Inverse of :func:`_split_planes` (used to run the torch codecs on device planes)."""
    nb = rows * (K // block_size(t))
    if t in (GGMLType.Q4_K, GGMLType.Q5_K, GGMLType.BF16, GGMLType.F16, GGMLType.F32):
        return planes[0]
    if t in (GGMLType.Q8_0, GGMLType.Q4_0):
        w = 32 if t == GGMLType.Q8_0 else 16
        return torch.cat([planes[1].view(nb, 2), planes[0].view(nb, w)], 1).view(-1)
    if t == GGMLType.MXFP4:
        return torch.cat([planes[1].view(nb, 1), planes[0].view(nb, 16)], 1).view(-1)
    if t == GGMLType.Q6_K:
        return torch.cat([planes[0].view(nb, 128), planes[1].view(nb, 64), planes[2].view(nb, 16),
                          planes[3].view(nb, 2)], 1).view(-1)
    raise NotImplementedError(t)


@dataclass
class QuantWeight:
    ggml_type: GGMLType
    N: int                       # rows per expert
    K: int
    planes: List[torch.Tensor]   # uint8 tensors (device layout, see module docstring)
    experts: int = 1
    name: str = ""
    _bf16_cache: Optional[torch.Tensor] = field(default=None, repr=False)

    @property
    def device(self) -> torch.device:
        return self.planes[0].device

    @property
    def rows(self) -> int:
        return self.N * self.experts

    @property
    def nbytes(self) -> int:
        return sum(p.numel() for p in self.planes)

    @property
    def uses_q8_activations(self) -> bool:
        return self.ggml_type in Q8_ACT_TYPES

    # ------------------------------------------------------------------ construction
    @staticmethod
    def from_raw(raw, ggml_type: GGMLType, shape: Sequence[int], device="cpu", name: str = "") -> "QuantWeight":
        """``raw``: GGUF block bytes (numpy or torch uint8); ``shape``: row-major
        ``[N, K]`` or ``[E, N, K]``."""
        t = GGMLType(ggml_type)
        shape = tuple(int(s) for s in shape)
        if len(shape) == 1:
            shape = (1,) + shape
        E = 1
        if len(shape) == 3:
            E, N, K = shape
        else:
            N, K = shape
        if not isinstance(raw, torch.Tensor):
            import warnings

            import numpy as np
            with warnings.catch_warnings():
                # read-only mmap views are fine: weights are never written through this tensor
                warnings.simplefilter("ignore", UserWarning)
                raw = torch.from_numpy(np.ascontiguousarray(raw))
        raw = raw.reshape(-1).view(torch.uint8)
        raw = raw.to(device, non_blocking=False)
        rows = E * N
        if t not in _NATIVE:
            vals = codecs.dequantize(raw, t).to(torch.bfloat16)
            return QuantWeight(GGMLType.BF16, N, K, [vals.contiguous().view(-1).view(torch.uint8)], E, name)
        return QuantWeight(t, N, K, _split_planes(raw, t, rows, K), E, name)

    @staticmethod
    def from_float(w: torch.Tensor, ggml_type: GGMLType, device=None, name: str = "") -> "QuantWeight":
        """Quantise a float matrix (``[N, K]`` or ``[E, N, K]``) to ``ggml_type``."""
        device = device if device is not None else w.device
        raw = codecs.quantize(w.to(device), ggml_type)
        return QuantWeight.from_raw(raw, ggml_type, tuple(w.shape), device, name)

    # ------------------------------------------------------------------ views / conversions
    def raw_blocks(self) -> torch.Tensor:
        """The weight as flat GGUF block bytes (inverse of the plane split)."""
        return _join_planes(self.planes, self.ggml_type, self.rows, self.K)

    def dequantize(self, dtype=torch.float32) -> torch.Tensor:
        """Decode with the torch codecs (oracle path; any device).  ``[rows, K]``."""
        return codecs.dequantize(self.raw_blocks(), self.ggml_type, (self.rows, self.K)).to(dtype)

    def expert(self, e: int) -> "QuantWeight":
        """View of one expert's ``[N, K]`` matrix (no copy).  The view object is created once per expert, so
        state attached to it (a decoded copy for the tensor-core path) lives as long as the stack does."""
        if self.experts == 1:
            return self
        views = self.__dict__.setdefault("_expert_views", {})
        if e in views:
            return views[e]
        out = []
        for p in self.planes:
            per = p.numel() // self.experts
            out.append(p[e * per:(e + 1) * per])
        views[e] = QuantWeight(self.ggml_type, self.N, self.K, out, 1, f"{self.name}.{e}")
        return views[e]

    def row_slice(self, start: int, stop: int) -> "QuantWeight":
        """Rows ``[start, stop)`` as a new weight sharing storage (tensor-parallel column shard)."""
        assert self.experts == 1
        out = []
        for p in self.planes:
            per = p.numel() // self.N
            out.append(p[start * per:stop * per])
        return QuantWeight(self.ggml_type, stop - start, self.K, out, 1, self.name)

    def col_slice(self, k0: int, k1: int) -> "QuantWeight":
        """Columns (input features) ``[k0, k1)`` of every row as a new, contiguous weight
        (tensor-parallel row shard).  The range must fall on block boundaries."""
        assert self.experts == 1 or True
        bs = block_size(self.ggml_type)
        if k0 % bs or k1 % bs:
            raise ValueError(f"col_slice [{k0}, {k1}) is not aligned to the {self.ggml_type.name} block of {bs}")
        rows = self.rows
        out = []
        for p in self.planes:
            per_row = p.numel() // rows
            per_k = per_row * bs // self.K            # plane bytes per block of `bs` values
            v = p.view(rows, per_row)
            out.append(v[:, (k0 // bs) * per_k:(k1 // bs) * per_k].contiguous().view(-1))
        return QuantWeight(self.ggml_type, self.N, k1 - k0, out, self.experts, self.name)

    @staticmethod
    def concat_rows(ws: Sequence["QuantWeight"], name: str = "") -> "QuantWeight":
        """Stack matrices with equal K and type along N (fused QKV / gate-up).
        Parity: Qwen3Model.cs:67-78 requires equal ggml types for the fusion."""
        t, K = ws[0].ggml_type, ws[0].K
        if any(w.ggml_type != t or w.K != K or w.experts != 1 for w in ws):
            raise ValueError("concat_rows needs equal type and K")
        planes = [torch.cat([w.planes[i] for w in ws]) for i in range(len(ws[0].planes))]
        return QuantWeight(t, sum(w.N for w in ws), K, planes, 1, name)

    @staticmethod
    def concat_rows_per_expert(ws: Sequence["QuantWeight"], name: str = "") -> "QuantWeight":
        """Per-expert row concatenation of expert stacks ``[E, N_i, K]`` -> ``[E, sum N_i, K]``
        (fused expert gate/up: concatenation, not interleave - GptOssModel.cs:126)."""
        t, K, E = ws[0].ggml_type, ws[0].K, ws[0].experts
        if any(w.ggml_type != t or w.K != K or w.experts != E for w in ws):
            raise ValueError("concat_rows_per_expert needs equal type, K and expert count")
        planes = []
        for i in range(len(ws[0].planes)):
            planes.append(torch.cat([w.planes[i].view(E, -1) for w in ws], 1).contiguous().view(-1))
        return QuantWeight(t, sum(w.N for w in ws), K, planes, E, name)

    def expert_range(self, e0: int, e1: int) -> "QuantWeight":
        """Experts ``[e0, e1)`` as a new stack sharing storage (expert-parallel shard)."""
        out = []
        for p in self.planes:
            per = p.numel() // self.experts
            out.append(p[e0 * per:e1 * per])
        return QuantWeight(self.ggml_type, self.N, self.K, out, e1 - e0, self.name)

    def to(self, device) -> "QuantWeight":
        return QuantWeight(self.ggml_type, self.N, self.K, [p.to(device) for p in self.planes], self.experts,
                           self.name)
