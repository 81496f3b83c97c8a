"""Token book-keeping of a session's KV cache and the reuse planner.

Behaviour matched to TensorSharp.Runtime/KVCache.cs: the cache remembers the exact token
sequence the model has seen plus the logits that followed it; ``plan_reuse`` (:187-215)
decides between
  * EXACT_MATCH  - the request is exactly the cached sequence: return the cached logits,
  * PARTIAL_REUSE - keep ``reused_prefix_length`` tokens, forward the remaining suffix,
  * RESET        - start over (nothing in common, or the model cannot truncate and the
                   request diverges inside the cached sequence).
A request that is a strict prefix-equal of the cache (all of it already cached, but no
stored logits) backs off by one token so that there is something to run.
"""
from __future__ import annotations

import enum
from dataclasses import dataclass
from typing import List, Optional, Sequence


class ReusePlanKind(enum.Enum):
    EXACT_MATCH = "ExactMatch"
    PARTIAL_REUSE = "PartialReuse"
    RESET = "Reset"


@dataclass(frozen=True)
class ReusePlan:
    kind: ReusePlanKind
    reused_prefix_length: int = 0
    tokens_to_forward: int = 0
    cached_logits: object = None

    @staticmethod
    def exact_match(logits) -> "ReusePlan":
        return ReusePlan(ReusePlanKind.EXACT_MATCH, 0, 0, logits)

    @staticmethod
    def reuse(prefix: int, to_forward: int) -> "ReusePlan":
        return ReusePlan(ReusePlanKind.PARTIAL_REUSE, prefix, to_forward, None)

    @staticmethod
    def reset(to_forward: int) -> "ReusePlan":
        return ReusePlan(ReusePlanKind.RESET, 0, to_forward, None)


class KVCache:
    def __init__(self):
        self._tokens: List[int] = []
        self._next_logits = None

    def __len__(self) -> int:
        return len(self._tokens)

    @property
    def count(self) -> int:
        return len(self._tokens)

    @property
    def tokens(self) -> Sequence[int]:
        return self._tokens

    @property
    def next_logits(self):
        return self._next_logits

    @property
    def is_empty(self) -> bool:
        return not self._tokens

    def common_prefix_length(self, other: Optional[Sequence[int]]) -> int:
        if not other or not self._tokens:
            return 0
        n = min(len(self._tokens), len(other))
        i = 0
        while i < n and self._tokens[i] == other[i]:
            i += 1
        return i

    def is_prefix_of(self, tokens: Optional[Sequence[int]]) -> bool:
        if tokens is None or len(tokens) < len(self._tokens):
            return False
        return all(a == b for a, b in zip(self._tokens, tokens))

    def try_get_exact_match_logits(self, tokens: Optional[Sequence[int]]):
        """The cached next-token logits (a copy) when ``tokens`` is exactly the cached sequence."""
        if self._next_logits is None or tokens is None or len(tokens) != len(self._tokens):
            return None
        if any(a != b for a, b in zip(self._tokens, tokens)):
            return None
        lg = self._next_logits
        return lg.clone() if hasattr(lg, "clone") else (lg.copy() if hasattr(lg, "copy") else lg)

    def reset(self) -> None:
        self._tokens.clear()
        self._next_logits = None

    def truncate_to(self, length: int) -> None:
        if length < 0:
            raise ValueError("Truncation length cannot be negative.")
        if length > len(self._tokens):
            raise ValueError("Truncation length exceeds cached token count.")
        if length < len(self._tokens):
            del self._tokens[length:]
            self._next_logits = None

    def record_append(self, new_tokens, next_logits) -> None:
        if new_tokens is None:
            return
        if isinstance(new_tokens, int):
            self._tokens.append(new_tokens)
        else:
            self._tokens.extend(int(t) for t in new_tokens)
        self._next_logits = next_logits

    def plan_reuse(self, input_tokens: Optional[Sequence[int]], supports_truncation: bool) -> ReusePlan:
        if not input_tokens:
            return ReusePlan.reset(0)
        cached = self.try_get_exact_match_logits(input_tokens)
        if cached is not None:
            return ReusePlan.exact_match(cached)
        common = self.common_prefix_length(input_tokens)
        if not supports_truncation and common < len(self._tokens):
            return ReusePlan.reset(len(input_tokens))
        if common == len(input_tokens):
            common = max(0, len(input_tokens) - 1)
        suffix = len(input_tokens) - common
        if common == 0:
            return ReusePlan.reset(len(input_tokens))
        return ReusePlan.reuse(common, suffix)
