"""Merging the model calls of concurrent requests into shared steps.

A serving host keeps its request logic per request (prompt rendering, KV reuse across turns, stop
sequences, output parsing) and simply runs several of them at once, each in its own thread, each
against its own *slot*: a view of the one loaded model that owns one sequence of the paged KV pool.
When a slot calls ``forward`` the call is parked; a stepper thread collects the calls that are parked
at that moment (it waits a moment for the other busy slots to arrive, so that decode steps stay in
lockstep), packs them into one batch (prefill chunks and single decode tokens mix freely), runs the
graph once and hands every caller its own row of logits.  The request code cannot tell that it shared
the step; on a B200 a decode step for eight sequences costs about what it costs for one.  A call that carries image or
audio embeddings runs by itself (its spans are positions of its own prompt); a step in which every caller brings one
token replays a captured graph (engine.py: BatchGraphStepper; ``TSB_GATHER_GRAPH=0`` turns that off).

The reference runs one inference at a time (TensorSharp.Server/InferenceQueue.cs) and has no counterpart.
"""
from __future__ import annotations

import threading
import time
from typing import List, Optional, Sequence


class _Call:
    __slots__ = ("seq", "tokens", "want", "embeddings", "done", "result", "error")

    def __init__(self, seq, tokens, want, embeddings=None):
        self.seq, self.tokens, self.want, self.embeddings = seq, tokens, want, embeddings
        self.done = threading.Event()
        self.result = None
        self.error: Optional[BaseException] = None


class GatheredModel:
    """Owns the loaded model and the stepper thread; ``slot(i)`` gives the per-request views."""

    def __init__(self, model, n_slots: int, window_s: float = 0.002):
        self.model, self.n_slots, self.window_s = model, n_slots, window_s
        self._cv = threading.Condition()
        self._pending: List[_Call] = []
        self._busy = 0                    # slots currently inside a generation
        self._stop = False
        self.model_lock = threading.RLock()          # held while the graph runs and while a slot edits its cache
        self.steps = 0
        self.step_rows = 0
        self.graph_steps = 0
        # steps in which every caller brings one token replay a captured graph (engine.py: BatchGraphStepper): measured
        # on a B200 with eight clients 848 against 663 tok/s, and 408 against 112 tok/s for one client at a time;
        # TSB_GATHER_GRAPH=0 keeps the merged steps eager
        import os
        self._stepper = None
        if os.environ.get("TSB_GATHER_GRAPH", "1") != "0":
            from .engine import BatchGraphStepper
            self._stepper = BatchGraphStepper(model, n_slots)
        self._slots = [SlotModel(self, i) for i in range(n_slots)]
        self._thread = threading.Thread(target=self._run, name="tsb-gather", daemon=True)
        self._thread.start()

    def slot(self, i: int) -> "SlotModel":
        return self._slots[i]

    # ------------------------------------------------------------------ called by slots
    def enter(self) -> None:
        with self._cv:
            self._busy += 1

    def leave(self) -> None:
        with self._cv:
            self._busy = max(0, self._busy - 1)
            self._cv.notify_all()

    def submit(self, seq, tokens: Sequence[int], want: bool, embeddings=None):
        c = _Call(seq, list(tokens), want, embeddings)
        with self._cv:
            if self._stop:
                raise RuntimeError("the model has been closed")
            self._pending.append(c)
            self._cv.notify_all()
        c.done.wait()
        if c.error is not None:
            raise c.error
        return c.result

    # ------------------------------------------------------------------ the stepper
    def _take(self) -> List[_Call]:
        with self._cv:
            while not self._pending and not self._stop:
                self._cv.wait()
            if self._stop:
                calls, self._pending = self._pending, []
                return calls
            # wait briefly for the other busy slots, so that their decode tokens ride in this step
            deadline = time.monotonic() + self.window_s
            while len(self._pending) < max(1, self._busy) and not self._stop:
                left = deadline - time.monotonic()
                if left <= 0:
                    break
                self._cv.wait(left)
            calls, self._pending = self._pending, []
            return calls

    def _run(self) -> None:
        while True:
            calls = self._take()
            if self._stop:
                for c in calls:
                    c.error = RuntimeError("the model has been closed")
                    c.done.set()
                return
            # a call that carries image / audio embeddings runs by itself (the spans are positions of its own prompt);
            # all the others share one step
            alone = [c for c in calls if c.embeddings]
            shared = [c for c in calls if not c.embeddings]
            for group in [[c] for c in alone] + ([shared] if shared else []):
                self._step(group)
            for c in calls:
                c.done.set()

    def _step(self, calls: List[_Call]) -> None:
        try:
            with self.model_lock:
                m = self.model
                logits = None
                if calls[0].embeddings:
                    for emb, pos in calls[0].embeddings:
                        m.set_vision_embeddings(emb, pos)
                elif self._stepper is not None and all(len(c.tokens) == 1 for c in calls):
                    logits = self._stepper.step([c.seq for c in calls], [c.tokens[0] for c in calls])
                    self.graph_steps += logits is not None
                if logits is None:
                    batch = m.kv.build_batch([c.seq for c in calls], [c.tokens for c in calls])
                    logits = m.forward_batch(batch, any(c.want for c in calls))
                if m.device.type == "cuda":
                    import torch
                    torch.cuda.synchronize(m.device)
            self.steps += 1
            self.step_rows += len(calls)
            for i, c in enumerate(calls):
                c.result = logits[i] if (c.want and logits is not None) else None
        except BaseException as e:                     # hand the failure to every caller of this step
            for c in calls:
                c.error = e

    def close(self) -> None:
        with self._cv:
            self._stop = True
            self._cv.notify_all()
        self._thread.join(timeout=5)
        for s in self._slots:
            s.release()
        close = getattr(self.model, "close", None)
        if close is not None:
            close()


class SlotModel:
    """What one request sees: the single-sequence model API over one sequence of the shared pool."""

    def __init__(self, owner: GatheredModel, index: int):
        self.__dict__["_owner"] = owner
        self.__dict__["_index"] = index
        self.__dict__["_seq"] = None
        self.__dict__["_pending"] = []
        self.__dict__["_injector"] = None

    # configuration, tokenizer, architecture ... come from the shared model
    def __getattr__(self, name):
        return getattr(self.__dict__["_owner"].model, name)

    def _sequence(self):
        if self._seq is None:
            with self._owner.model_lock:
                self.__dict__["_seq"] = self._owner.model.new_sequence()
        return self._seq

    @property
    def multimodal(self):
        """This slot's injector (its own prepared spans and queue) over the encoders the shared model has loaded;
        ``None`` for text-only architectures."""
        shared = self._owner.model.multimodal
        if shared is None:
            return None
        if self._injector is None:
            from ..multimodal.injector import SlotInjector
            self.__dict__["_injector"] = SlotInjector(self, shared)
        return self._injector

    def set_vision_embeddings(self, embeddings, insert_position: int) -> None:
        self._pending.append((embeddings, int(insert_position)))

    set_audio_embeddings = set_vision_embeddings

    @property
    def cache_length(self) -> int:
        return self._seq.length if self._seq is not None else 0

    def forward(self, tokens: Sequence[int], want_logits: bool = True):
        emb, self.__dict__["_pending"] = self._pending, []
        return self._owner.submit(self._sequence(), tokens, want_logits, emb or None)

    def forward_refill(self, tokens: Sequence[int], chunk: int = 2048):
        tokens = list(tokens)
        out = None
        for i in range(0, len(tokens), chunk):
            out = self.forward(tokens[i:i + chunk], want_logits=i + chunk >= len(tokens))
        return out

    def reset_kv_cache(self) -> None:
        if self._seq is not None:
            with self._owner.model_lock:
                m = self._owner.model
                m.kv.truncate(self._seq, 0)
                m.reset_recurrent_state(self._seq.slot)

    def truncate_kv_cache(self, n_tokens: int) -> None:
        m = self._owner.model
        if self._seq is None or n_tokens >= self._seq.length:      # keeping the whole cache is not a truncation
            return
        if not m.supports_kv_truncation:
            raise RuntimeError(f"{type(m).__name__} cannot truncate its cache (recurrent state)")
        with self._owner.model_lock:
            m.kv.truncate(self._seq, n_tokens)

    def warm_up_kernels(self) -> None:
        if self._index == 0:
            with self._owner.model_lock:
                self._owner.model.warm_up_kernels()

    # a generation brackets itself so that the stepper knows how many callers to expect
    def __enter__(self):
        self._owner.enter()
        return self

    def __exit__(self, *exc):
        self._owner.leave()

    def release(self) -> None:
        if self._seq is not None:
            with self._owner.model_lock:
                self._owner.model.free_sequence(self._seq)
            self.__dict__["_seq"] = None

    def close(self) -> None:              # a slot does not own the model
        self.release()
