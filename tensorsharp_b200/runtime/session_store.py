"""Persist a conversation's KV state: the token list, the cached next-token logits and the K / V rows of
one sequence, so that a later process can continue the chat without re-running the prompt.

The reference keeps KV reuse in memory only and loses it on reload or session switch
(TensorSharp.Server/ModelService.cs:124-157); its ``/save`` writes transcript text.  The file is a
``torch.save`` archive: ``{"arch", "n_layers", "tokens", "logits", "k": [...], "v": [...]}`` with layers that
have no cache of their own (none, or shared with a donor layer) stored as ``None``.
"""
from __future__ import annotations

from typing import List, Optional

import torch

from .kv_cache import KVCache


def _slots(kv, seq, n: int) -> torch.Tensor:
    ps = kv.page_size
    pos = torch.arange(n)
    pages = torch.tensor(seq.pages, dtype=torch.long)
    return (pages[pos // ps] * ps + pos % ps).to(kv.device)


def _rows(t: torch.Tensor, slots: torch.Tensor) -> torch.Tensor:
    """``t[slots]``; one-byte element types (the 8-bit cache) are indexed through their bytes."""
    if t.element_size() == 1:
        return t.view(torch.uint8)[slots].view(t.dtype)
    return t[slots]


def _set_rows(t: torch.Tensor, slots: torch.Tensor, rows: torch.Tensor) -> None:
    """``t[slots] = rows`` converted to the cache's element type (a session saved from a bf16 cache loads into an
    8-bit one and the other way round)."""
    rows = rows.to(t.device).to(t.dtype) if rows.dtype != t.dtype else rows.to(t.device)
    if t.element_size() == 1:
        t.view(torch.uint8)[slots] = rows.view(torch.uint8)
    else:
        t[slots] = rows


def save_session(path: str, model, cache: KVCache, seq=None) -> int:
    """Write the first ``cache.count`` positions of ``seq`` (default: the model's own sequence)."""
    if not getattr(model, "supports_kv_truncation", True):
        raise RuntimeError(f"{type(model).__name__} keeps recurrent state that is not part of the KV pool")
    if model.kv.ring:
        raise RuntimeError("the window layers keep only a ring of pages (TSB_KV_WINDOW_RING=1): their cache cannot be saved")
    seq = seq or model._seq()
    n = min(cache.count, seq.length)
    slots = _slots(model.kv, seq, n)
    seen = {}
    ks: List[Optional[torch.Tensor]] = []
    vs: List[Optional[torch.Tensor]] = []
    for k, v in zip(model.kv.k, model.kv.v):
        if k is None or id(k) in seen:
            ks.append(None)
            vs.append(None)
            continue
        seen[id(k)] = True
        ks.append(_rows(k, slots).cpu())
        vs.append(_rows(v, slots).cpu())
    logits = cache.next_logits
    torch.save({"arch": model.arch, "n_layers": len(ks), "tokens": list(cache.tokens)[:n],
                "logits": logits.detach().cpu() if isinstance(logits, torch.Tensor) and n == cache.count else None,
                "k": ks, "v": vs}, path)
    return n


def load_session(path: str, model, cache: KVCache, seq=None) -> int:
    """Restore into ``seq`` (emptied first); returns the number of tokens now cached."""
    d = torch.load(path, map_location="cpu", weights_only=False)
    if d["arch"] != model.arch or d["n_layers"] != len(model.kv.k):
        raise ValueError(f"session file was written by a different model ({d['arch']}, {d['n_layers']} layers)")
    if model.kv.ring:
        raise RuntimeError("the window layers keep only a ring of pages (TSB_KV_WINDOW_RING=1): a saved cache cannot be restored")
    seq = seq or model._seq()
    n = len(d["tokens"])
    model.kv.truncate(seq, 0)
    model.kv.reserve(seq, n)
    seq.length = n
    slots = _slots(model.kv, seq, n)
    seen = {}
    for l, (k, v) in enumerate(zip(model.kv.k, model.kv.v)):
        if k is None or id(k) in seen or d["k"][l] is None:
            continue
        seen[id(k)] = True
        _set_rows(k, slots, d["k"][l])
        _set_rows(v, slots, d["v"][l])
    cache.reset()
    lg = d["logits"]
    cache.record_append(d["tokens"], lg.to(model.device) if lg is not None else None)
    return n
