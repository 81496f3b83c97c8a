"""Paged KV cache, per-sequence block tables and batch assembly.

The reference keeps one contiguous F32 cache ``[kvHeads, maxSeqLen, headDim]`` per layer
for its single sequence (TensorSharp.Models/ModelBase.cs:1340 CopyToCache, :302-408
context sizing).  Here the cache is paged (``[n_pages * page_size, Hkv, Dh]`` bf16 per
layer) so that many sequences share one pool, a sequence can be truncated to any prefix
in O(1) (multi-turn prefix reuse, ModelBase.TruncateKVCache).  By default all layers of a
sequence share one block table, so a sliding-window layer keeps its pages and masks by position.
With ``window_layers`` and ``ring_chunk`` the window layers get a pool of their own in which a
sequence owns a ring of pages (the reference's circular window caches, Gemma4Model.cs:1927):
logical page j lives in ring page j mod R, R = pages for window + ring_chunk tokens + 1, so a
32 k context costs a window layer a few dozen pages instead of five hundred.  A forward call may
then add at most ``ring_chunk`` tokens to a sequence (the caller prefills in chunks), and a cache
can be cut back by at most ring capacity - window tokens (``can_truncate``).  Layers that share KV
with a donor layer (Gemma 4) alias the donor's tensors.  Recurrent layers (GatedDeltaNet, Mamba2)
get fixed-size state slots instead.
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
    wpages: List[int] = field(default_factory=list)     # ring pages in the window layers' pool (empty without a ring)


class PagedKV:
    def __init__(self, layer_shapes: Sequence[Optional[Tuple[int, int]]], n_pages: int, page_size: int = 64,
                 device="cpu", dtype=torch.bfloat16, donors: Optional[Dict[int, int]] = None, max_seqs: int = 64,
                 window_layers: Optional[Dict[int, int]] = None, ring_chunk: int = 0):
        """``layer_shapes[l]`` is ``(Hkv, Dh)`` for attention layers, ``None`` for layers
        without a KV cache; ``donors[l] = m`` makes layer ``l`` read layer ``m``'s cache.
        ``window_layers[l] = W`` with ``ring_chunk > 0`` gives those layers the ring pool."""
        self.page_size = page_size
        self.n_pages = n_pages
        self.device = torch.device(device)
        self.dtype = dtype
        self.k: List[Optional[torch.Tensor]] = []
        self.v: List[Optional[torch.Tensor]] = []
        donors = donors or {}
        self.window_layers = dict(window_layers or {}) if ring_chunk > 0 else {}
        self.window_layers = {l: w for l, w in self.window_layers.items() if w and w > 0 and l not in donors}
        self.ring_chunk = int(ring_chunk) if self.window_layers else 0
        self.ring_window = max(self.window_layers.values()) if self.window_layers else 0
        self.ring_pages = ((self.ring_window + self.ring_chunk + page_size - 1) // page_size + 1) if self.window_layers else 0
        self.n_wpages = min(n_pages, self.ring_pages * max(1, max_seqs)) if self.window_layers else 0
        for l, shp in enumerate(layer_shapes):
            if shp is None or l in donors:
                self.k.append(None)
                self.v.append(None)
                continue
            hkv, dh = shp
            rows = (self.n_wpages if l in self.window_layers else n_pages) * page_size
            self.k.append(torch.zeros((rows, hkv, dh), dtype=dtype, device=self.device))
            self.v.append(torch.zeros((rows, hkv, dh), dtype=dtype, device=self.device))
        self._wfree: List[int] = list(range(self.n_wpages - 1, -1, -1))
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

    @property
    def ring(self) -> bool:
        """Whether sliding-window layers keep a ring of pages."""
        return self.ring_pages > 0

    def is_window_layer(self, l: int) -> bool:
        return l in self.window_layers

    def can_truncate(self, s: SeqState, n_tokens: int) -> bool:
        """Whether the first ``n_tokens`` tokens can be kept and the rest dropped: always without a ring; with one, only
        while the window before the cut has not been overwritten by the tokens that are dropped."""
        if not self.ring or n_tokens <= 0 or n_tokens >= s.length or s.length <= self.ring_pages * self.page_size:
            return True
        return s.length - n_tokens <= self.ring_pages * self.page_size - self.ring_window

    def free_seq(self, s: SeqState) -> None:
        self._free.extend(reversed(s.pages))
        s.pages.clear()
        self._wfree.extend(reversed(s.wpages))
        s.wpages.clear()
        s.length = 0
        if s.slot >= 0:
            self._free_slots.append(s.slot)
            s.slot = -1

    def reserve(self, s: SeqState, new_len: int) -> None:
        need = (new_len + self.page_size - 1) // self.page_size - len(s.pages)
        if need > len(self._free):
            raise OutOfPagesError(f"need {need} pages, {len(self._free)} free")
        wneed = min(self.ring_pages, (new_len + self.page_size - 1) // self.page_size) - len(s.wpages) if self.ring else 0
        if wneed > len(self._wfree):
            raise OutOfPagesError(f"need {wneed} window pages, {len(self._wfree)} free")
        for _ in range(max(0, need)):
            s.pages.append(self._free.pop())
        for _ in range(max(0, wneed)):
            s.wpages.append(self._wfree.pop())

    def truncate(self, s: SeqState, n_tokens: int) -> None:
        """Keep the first ``n_tokens`` tokens; whole pages past them return to the pool."""
        n_tokens = max(0, min(n_tokens, s.length))
        keep = (n_tokens + self.page_size - 1) // self.page_size
        if self.ring and not self.can_truncate(s, n_tokens):
            raise RuntimeError(f"the window layers' ring no longer holds the {self.ring_window} tokens before position {n_tokens}")
        while len(s.pages) > keep:
            self._free.append(s.pages.pop())
        if self.ring and (n_tokens == 0 or s.length <= self.ring_pages * self.page_size):
            # nothing kept, or the ring never wrapped (pages map one to one): surplus ring pages go back
            while len(s.wpages) > min(keep, self.ring_pages):
                self._wfree.append(s.wpages.pop())
        s.length = n_tokens

    # ------------------------------------------------------------------ ring addressing
    def wslot(self, s: SeqState, p: int) -> int:
        """Flat slot of position ``p`` in the window layers' pool."""
        ps = self.page_size
        return s.wpages[(p // ps) % self.ring_pages] * ps + p % ps

    def wtable_row(self, s: SeqState, width: int) -> List[int]:
        """Block-table row of the window layers: logical page j -> ring page j mod R (0 where the ring has no page yet)."""
        R, n = self.ring_pages, len(s.wpages)
        return [s.wpages[j % R] if (j % R) < n else 0 for j in range(width)]

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
        wslots: List[int] = []
        for s, nt in zip(seqs, new_tokens):
            n = len(nt)
            if self.ring and n > self.ring_chunk:
                raise ValueError(f"{n} new tokens in one call, but the window layers' ring was sized for chunks of {self.ring_chunk}")
            self.reserve(s, s.length + n)
            for i, t in enumerate(nt):
                p = s.length + i
                toks.append(int(t))
                pos.append(p)
                slots.append(s.pages[p // ps] * ps + p % ps)
                if self.ring:
                    wslots.append(self.wslot(s, p))
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
        ring = {}
        if self.ring:
            ring = dict(slots_w=torch.tensor(wslots, dtype=torch.int64).to(dev, non_blocking=True),
                        block_table_w=torch.tensor([self.wtable_row(s, width) for s in seqs], dtype=torch.int32).to(dev, non_blocking=True))
        return Batch(**ring,
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
