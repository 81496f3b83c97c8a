"""Sampling configuration and the token sampler.

The transformation order is the reference's (TensorSharp.Runtime/TokenSampler.cs:36-61):
greedy shortcut → penalties over the unique generated ids (repetition: divide when the
logit is positive else multiply; presence: subtract once; frequency: subtract × count)
→ arg-max when temperature ≤ 0 → ÷ temperature → softmax → min-p (zero below
min_p × max prob) → top-k (descending) → top-p (smallest prefix whose mass ≥ p) →
renormalise over the survivors → draw.  Defaults are SamplingConfig.cs:22-80
(temperature 0.8, top_k 40, top_p 0.9, min_p 0, repetition 1.1, seed −1).

The sampler runs on whatever device the logits live on: on CUDA the logits never leave
the device, only the chosen id does.  The random stream is Python's ``random.Random``
seeded like the reference seeds ``System.Random`` (the two generators differ, so equal
seeds reproduce runs of this engine, not of the reference).
"""
from __future__ import annotations

import random
from dataclasses import dataclass, replace
from typing import Dict, List, Optional, Sequence, Tuple

import torch


@dataclass
class SamplingConfig:
    temperature: float = 0.8
    top_k: int = 40
    top_p: float = 0.9
    min_p: float = 0.0
    repetition_penalty: float = 1.1
    presence_penalty: float = 0.0
    frequency_penalty: float = 0.0
    seed: int = -1
    stop_sequences: Optional[List[str]] = None
    max_tokens: int = 0

    @property
    def is_greedy(self) -> bool:
        return self.temperature <= 0 and self.top_k <= 0 and self.top_p >= 1.0 and self.min_p <= 0

    @property
    def has_penalties(self) -> bool:
        return self.repetition_penalty != 1.0 or self.presence_penalty != 0 or self.frequency_penalty != 0

    @staticmethod
    def default() -> "SamplingConfig":
        return SamplingConfig()

    @staticmethod
    def greedy() -> "SamplingConfig":
        return SamplingConfig(temperature=0.0, top_k=0, top_p=1.0, repetition_penalty=1.0)

    @staticmethod
    def creative() -> "SamplingConfig":
        return SamplingConfig(temperature=0.7, top_p=0.9, min_p=0.05)

    def clone(self) -> "SamplingConfig":
        return replace(self, stop_sequences=list(self.stop_sequences) if self.stop_sequences is not None else None)


class TokenSampler:
    def __init__(self, config: Optional[SamplingConfig] = None):
        self.config = config or SamplingConfig.default()
        self.rng = random.Random(self.config.seed) if self.config.seed >= 0 else random.Random()

    # ------------------------------------------------------------------ sampling
    def sample(self, logits: torch.Tensor, generated: Optional[Sequence[int]] = None) -> int:
        """Pick the next token from float logits ``[vocab]`` (any device)."""
        c = self.config
        if c.is_greedy and not c.has_penalties and not generated:
            return self._argmax(logits)
        scores = logits.float().clone()
        self._apply_penalties(scores, generated)
        if c.temperature <= 0:
            return self._argmax(scores)
        scores = scores * (1.0 / c.temperature)
        probs = torch.softmax(scores, -1)
        if c.min_p > 0:
            probs = torch.where(probs < c.min_p * probs.max(), torch.zeros_like(probs), probs)
        n = probs.numel()
        k = min(c.top_k, n) if c.top_k > 0 else n
        if k < n:
            cand_p, cand_i = torch.topk(probs, k)
        else:
            cand_p, cand_i = torch.sort(probs, descending=True, stable=True)
        if c.top_p < 1.0:
            cum = torch.cumsum(cand_p, 0)
            hit = torch.nonzero(cum >= c.top_p)
            cutoff = int(hit[0]) + 1 if hit.numel() else cand_p.numel()
            cand_p, cand_i = cand_p[:cutoff], cand_i[:cutoff]
        if cand_i.numel() == 0:
            return 0
        if cand_i.numel() == 1:
            return int(cand_i[0])
        total = float(cand_p.sum())
        if total <= 0:
            return int(cand_i[0])
        r = self.rng.random() * total
        cum = torch.cumsum(cand_p, 0)
        idx = int(torch.searchsorted(cum, torch.tensor(r, dtype=cum.dtype, device=cum.device)).clamp_max(cum.numel() - 1))
        return int(cand_i[idx])

    @staticmethod
    def _argmax(x: torch.Tensor) -> int:
        if x.is_cuda:
            from ..ops import functional as F
            return int(F.argmax(x.view(1, -1))[0])
        return int(torch.argmax(x))

    def _apply_penalties(self, scores: torch.Tensor, generated: Optional[Sequence[int]]) -> None:
        c = self.config
        if not generated or not c.has_penalties:
            return
        counts: Dict[int, int] = {}
        for t in generated:
            counts[t] = counts.get(t, 0) + 1
        ids = [t for t in counts if 0 <= t < scores.numel()]
        if not ids:
            return
        idx = torch.tensor(ids, dtype=torch.long, device=scores.device)
        cnt = torch.tensor([counts[t] for t in ids], dtype=scores.dtype, device=scores.device)
        v = scores[idx]
        if c.repetition_penalty != 1.0:
            v = torch.where(v > 0, v / c.repetition_penalty, v * c.repetition_penalty)
        if c.presence_penalty != 0:
            v = v - c.presence_penalty
        if c.frequency_penalty != 0:
            v = v - c.frequency_penalty * cnt
        scores[idx] = v

    # ------------------------------------------------------------------ stop sequences
    def check_stop_sequences(self, decoded: str) -> Tuple[str, bool]:
        """(text trimmed at the first stop sequence found, whether to stop).  Stop sequences
        are checked in list order, by substring (TokenSampler.cs:67-79)."""
        stops = self.config.stop_sequences
        if not stops:
            return decoded, False
        for s in stops:
            i = decoded.find(s)
            if i >= 0:
                return decoded[:i], True
        return decoded, False
