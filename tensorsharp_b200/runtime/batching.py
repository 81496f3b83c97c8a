"""Continuous batching: many independent generations share every decode step.

The reference answers one request at a time (its queue admits a single running inference,
TensorSharp.Server/InferenceQueue.cs, and the CLI's JSONL mode loops over the requests,
TensorSharp.Cli/Program.cs:660).  On a B200 a decode step costs about the same for 16 sequences as for
one (the weights are streamed once either way), so this engine keeps up to ``max_batch`` sequences in
flight in the paged KV pool: a finished sequence frees its pages and the next waiting request is
prefilled and joins the running batch at the following step.  Sampling, end-of-sequence and stop
sequences are per request and follow the single-request loop exactly, so a request's output does not
depend on what it was batched with (greedy sampling: bit-for-bit on the CPU path).
"""
from __future__ import annotations

import time
from collections import deque
from dataclasses import dataclass, field
from typing import Callable, Deque, List, Optional, Sequence

from .sampling import SamplingConfig, TokenSampler


@dataclass
class GenRequest:
    tokens: Sequence[int]                         # prompt ids
    max_tokens: int
    sampling: SamplingConfig = field(default_factory=SamplingConfig.greedy)
    on_piece: Optional[Callable[[str], None]] = None
    tag: object = None                            # the caller's handle (request id, line number ...)
    # results
    ids: List[int] = field(default_factory=list)
    text: str = ""
    stopped: bool = False                         # ended on a stop sequence
    error: Optional[str] = None
    prefill_ms: float = 0.0
    total_ms: float = 0.0
    # engine state
    _seq: object = None
    _sampler: Optional[TokenSampler] = None
    _next: int = -1
    _t0: float = 0.0


class ContinuousBatcher:
    def __init__(self, model, max_batch: int = 8, prefill_chunk: int = 2048):
        if max_batch < 1:
            raise ValueError("max_batch must be at least 1")
        self.model, self.max_batch, self.prefill_chunk = model, max_batch, prefill_chunk
        self.steps = 0                 # decode steps run
        self.step_rows = 0             # sequences advanced over all steps (step_rows / steps = mean batch)
        self.graph_steps = 0
        # decode steps replay captured graphs (engine.py: BatchGraphStepper), as the merged steps of the concurrent
        # server do; TSB_GATHER_GRAPH=0 keeps them eager
        import os
        self._stepper = None
        if os.environ.get("TSB_GATHER_GRAPH", "1") != "0":
            from .engine import BatchGraphStepper
            self._stepper = BatchGraphStepper(model, max_batch)

    # ------------------------------------------------------------------ one request's life
    def _sync(self) -> None:
        if self.model.device.type == "cuda":
            import torch
            torch.cuda.synchronize(self.model.device)

    def _admit(self, r: GenRequest) -> bool:
        """Prefill ``r`` into a fresh sequence and draw its first token; False when it ended at once."""
        m = self.model
        r._t0 = time.perf_counter()
        r._sampler = TokenSampler(r.sampling)
        r._seq = m.new_sequence()
        toks = list(r.tokens)
        logits = None
        for i in range(0, len(toks), self.prefill_chunk):
            last = i + self.prefill_chunk >= len(toks)
            out = m.forward_batch(m.kv.build_batch([r._seq], [toks[i:i + self.prefill_chunk]]), want_logits=last)
            if last:
                logits = out[0]
        self._sync()
        r.prefill_ms = (time.perf_counter() - r._t0) * 1e3
        return self._consume(r, logits)

    def _consume(self, r: GenRequest, logits) -> bool:
        """Draw the next token of ``r`` from ``logits``; False when the request is finished."""
        tok = self.model.tokenizer
        if len(r.ids) >= r.max_tokens:
            return False
        nxt = r._sampler.sample(logits, r.ids)
        if tok.is_eos(nxt):
            return False
        r.ids.append(nxt)
        new_text = tok.decode(r.ids)
        if r.on_piece is not None and len(new_text) > len(r.text) and not new_text.endswith("�"):
            r.on_piece(new_text[len(r.text):])
        r.text = new_text
        if r.sampling.stop_sequences:
            trimmed, stop = r._sampler.check_stop_sequences(r.text)
            if stop:
                r.text, r.stopped = trimmed, True
                return False
        if len(r.ids) >= r.max_tokens:
            return False
        r._next = nxt
        return True

    def _finish(self, r: GenRequest) -> None:
        if r._seq is not None:
            self.model.free_sequence(r._seq)
            r._seq = None
        r.total_ms = (time.perf_counter() - r._t0) * 1e3

    # ------------------------------------------------------------------ the loop
    def run(self, requests: Sequence[GenRequest]) -> Sequence[GenRequest]:
        """Generate for every request; results are written into the request objects (order preserved)."""
        m = self.model
        waiting: Deque[GenRequest] = deque(requests)
        active: List[GenRequest] = []
        while waiting or active:
            while waiting and len(active) < self.max_batch:
                r = waiting.popleft()
                try:
                    if self._admit(r):
                        active.append(r)
                    else:
                        self._finish(r)
                except Exception as e:                      # one bad request must not end the batch
                    r.error = str(e)
                    self._finish(r)
            if not active:
                continue
            logits = None
            if self._stepper is not None:
                logits = self._stepper.step([r._seq for r in active], [r._next for r in active])
                self.graph_steps += logits is not None
            if logits is None:
                batch = m.kv.build_batch([r._seq for r in active], [[r._next] for r in active])
                logits = m.forward_batch(batch, True)
            self.steps += 1
            self.step_rows += len(active)
            still: List[GenRequest] = []
            for i, r in enumerate(active):
                if self._consume(r, logits[i]):
                    still.append(r)
                else:
                    self._finish(r)
            active = still
        return requests
