"""Paged KV cache, per-sequence block tables and batch assembly.

The reference keeps one contiguous F32 cache ``[kvHeads, maxSeqLen, headDim]`` per layer
for its single sequence (TensorSharp.Models/ModelBase.cs:1340 CopyToCache, :302-408
context sizing).  Here the cache is paged (``[n_pages * page_size, Hkv, Dh]`` bf16 per
layer) so that many sequences share one pool, a sequence can be truncated to any prefix
in O(1) (multi-turn prefix reuse, ModelBase.TruncateKVCache).  All layers of a sequence
share one block table, so a sliding-window layer keeps its pages and masks by position
(the reference's circular window caches, Gemma4Model.cs:1927, have no counterpart).  Layers that share KV with a donor layer (Gemma 4) alias the donor's
tensors.  Recurrent layers (GatedDeltaNet, Mamba2) get fixed-size state slots instead.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from ..ops.functional import Batch


class OutOfPagesError(RuntimeError):
    """The KV pool has no free page left for the requested growth."""


@dataclass
class SeqState:
    """One sequence's view of the pool."""
    seq_id: int
    slot: int                      # recurrent-state slot
    pages: List[int] = field(default_factory=list)
    length: int = 0                # tokens whose K/V are in the cache


class PagedKV:
    def __init__(self, layer_shapes: Sequence[Optional[Tuple[int, int]]], n_pages: int, page_size: int = 64,
                 device="cpu", dtype=torch.bfloat16, donors: Optional[Dict[int, int]] = None, max_seqs: int = 64):
        """``layer_shapes[l]`` is ``(Hkv, Dh)`` for attention layers, ``None`` for layers
        without a KV cache; ``donors[l] = m`` makes layer ``l`` read layer ``m``'s cache."""
        self.page_size = page_size
        self.n_pages = n_pages
        self.device = torch.device(device)
        self.dtype = dtype
        self.k: List[Optional[torch.Tensor]] = []
        self.v: List[Optional[torch.Tensor]] = []
        donors = donors or {}
        for l, shp in enumerate(layer_shapes):
            if shp is None or l in donors:
                self.k.append(None)
                self.v.append(None)
                continue
            hkv, dh = shp
            self.k.append(torch.zeros((n_pages * page_size, hkv, dh), dtype=dtype, device=self.device))
            self.v.append(torch.zeros((n_pages * page_size, hkv, dh), dtype=dtype, device=self.device))
        for l, m in donors.items():
            self.k[l], self.v[l] = self.k[m], self.v[m]
        self._free: List[int] = list(range(n_pages - 1, -1, -1))
        self._free_slots: List[int] = list(range(max_seqs - 1, -1, -1))
        self._next_id = 0
        self.max_seqs = max_seqs

    # ------------------------------------------------------------------ sequences
    @property
    def free_pages(self) -> int:
        return len(self._free)

    def new_seq(self) -> SeqState:
        if not self._free_slots:
            raise OutOfPagesError("no free sequence slot")
        s = SeqState(self._next_id, self._free_slots.pop())
        self._next_id += 1
        return s

    def free_seq(self, s: SeqState) -> None:
        self._free.extend(reversed(s.pages))
        s.pages.clear()
        s.length = 0
        if s.slot >= 0:
            self._free_slots.append(s.slot)
            s.slot = -1

    def reserve(self, s: SeqState, new_len: int) -> None:
        need = (new_len + self.page_size - 1) // self.page_size - len(s.pages)
        if need > len(self._free):
            raise OutOfPagesError(f"need {need} pages, {len(self._free)} free")
        for _ in range(max(0, need)):
            s.pages.append(self._free.pop())

    def truncate(self, s: SeqState, n_tokens: int) -> None:
        """Keep the first ``n_tokens`` tokens; whole pages past them return to the pool."""
        n_tokens = max(0, min(n_tokens, s.length))
        keep = (n_tokens + self.page_size - 1) // self.page_size
        while len(s.pages) > keep:
            self._free.append(s.pages.pop())
        s.length = n_tokens

    # ------------------------------------------------------------------ batches
    def build_batch(self, seqs: Sequence[SeqState], new_tokens: Sequence[Sequence[int]],
                    table_width: Optional[int] = None) -> Batch:
        """Reserve pages for the new tokens of each sequence and assemble the packed batch.
        Sequence lengths are advanced; the caller runs the model right after."""
        ps = self.page_size
        toks: List[int] = []
        pos: List[int] = []
        slots: List[int] = []
        cu = [0]
        lens: List[int] = []
        last: List[int] = []
        for s, nt in zip(seqs, new_tokens):
            n = len(nt)
            self.reserve(s, s.length + n)
            for i, t in enumerate(nt):
                p = s.length + i
                toks.append(int(t))
                pos.append(p)
                slots.append(s.pages[p // ps] * ps + p % ps)
            s.length += n
            cu.append(cu[-1] + n)
            lens.append(s.length)
            last.append(cu[-1] - 1)
        width = table_width or max(1, max(len(s.pages) for s in seqs))
        table = torch.zeros((len(seqs), width), dtype=torch.int32)
        for i, s in enumerate(seqs):
            if s.pages:
                table[i, :len(s.pages)] = torch.tensor(s.pages, dtype=torch.int32)
        dev = self.device
        max_q = max(cu[i + 1] - cu[i] for i in range(len(seqs)))
        return Batch(
            tokens=torch.tensor(toks, dtype=torch.int32).to(dev, non_blocking=True),
            positions=torch.tensor(pos, dtype=torch.int32).to(dev, non_blocking=True),
            slots=torch.tensor(slots, dtype=torch.int64).to(dev, non_blocking=True),
            cu_q=torch.tensor(cu, dtype=torch.int32).to(dev, non_blocking=True),
            kv_lens=torch.tensor(lens, dtype=torch.int32).to(dev, non_blocking=True),
            block_table=table.to(dev, non_blocking=True),
            last_idx=torch.tensor(last, dtype=torch.int64).to(dev, non_blocking=True),
            seq_slots=torch.tensor([s.slot for s in seqs], dtype=torch.int64).to(dev, non_blocking=True),
            max_q_len=max_q, max_kv_len=max(lens), is_decode=(max_q == 1 and len(toks) == len(seqs)),
            page_size=ps, h_cu_q=tuple(cu), h_kv_lens=tuple(lens))
