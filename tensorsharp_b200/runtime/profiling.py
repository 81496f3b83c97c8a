"""Per-phase timing and trace ranges.

The reference accumulates host tick counters around linear / attention / norm / embedding / lm_head calls
and prints them with PrintTimingStats (TensorSharp.Models/ModelBase.cs:229-234, :877-903, :1922-1930);
those include the device round trip of every call.  Here a phase is bracketed by CUDA events on the
launching stream (host clock on CPU), nothing synchronises until the table is read, and the same names
can be emitted as NVTX ranges for an external timeline tool.  Off unless ``TSB_PROFILE=1`` (timing) or
``TSB_NVTX=1`` (ranges), so the hot path pays one dictionary lookup.
"""
from __future__ import annotations

import contextlib
import os
import time
from collections import OrderedDict
from typing import Dict, List, Optional, Tuple

import torch


class PhaseTimer:
    def __init__(self, device=None, enabled: Optional[bool] = None, nvtx: Optional[bool] = None):
        self.device = torch.device(device) if device is not None else torch.device("cpu")
        self.enabled = os.environ.get("TSB_PROFILE", "0") == "1" if enabled is None else enabled
        self.nvtx = (os.environ.get("TSB_NVTX", "0") == "1" if nvtx is None else nvtx) and self.device.type == "cuda"
        self._pending: List[Tuple[str, object, object]] = []
        self._totals: "OrderedDict[str, List[float]]" = OrderedDict()

    @contextlib.contextmanager
    def phase(self, name: str):
        if not self.enabled and not self.nvtx:
            yield
            return
        if self.nvtx:
            torch.cuda.nvtx.range_push(name)
        if self.enabled:
            if self.device.type == "cuda":
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
            else:
                t0 = time.perf_counter()
        try:
            yield
        finally:
            if self.enabled:
                if self.device.type == "cuda":
                    e1.record()
                    self._pending.append((name, e0, e1))
                else:
                    self._add(name, (time.perf_counter() - t0) * 1e3)
            if self.nvtx:
                torch.cuda.nvtx.range_pop()

    def _add(self, name: str, ms: float) -> None:
        t = self._totals.setdefault(name, [0.0, 0])
        t[0] += ms
        t[1] += 1

    def _collect(self) -> None:
        if self._pending:
            torch.cuda.synchronize(self.device)
            for name, e0, e1 in self._pending:
                self._add(name, e0.elapsed_time(e1))
            self._pending = []

    def reset(self) -> None:
        self._pending, self._totals = [], OrderedDict()

    def stats(self) -> Dict[str, Dict[str, float]]:
        self._collect()
        return {k: {"total_ms": v[0], "calls": v[1], "avg_ms": v[0] / max(1, v[1])} for k, v in self._totals.items()}

    def table(self) -> str:
        s = self.stats()
        total = sum(v["total_ms"] for v in s.values()) or 1.0
        lines = [f"{'phase':<24}{'calls':>8}{'total ms':>12}{'avg ms':>10}{'share':>8}"]
        for k, v in s.items():
            lines.append(f"{k:<24}{int(v['calls']):>8}{v['total_ms']:>12.2f}{v['avg_ms']:>10.3f}{100 * v['total_ms'] / total:>7.1f}%")
        return "\n".join(lines)
