"""FIFO admission queue: one inference runs at a time (or ``capacity`` of them when the server batches
concurrent requests), later requests wait with a visible position.

Parity: TensorSharp.Server/InferenceQueue.cs (Enqueue :43, Release :76, RemoveCancelled :99,
ActivateNext :118, GetStatus :159, QueueTicket :189-262).  Tickets are context managers; a
waiting client polls ``position`` once a second (``wait(1.0)``) to stream queue progress.
"""
from __future__ import annotations

import collections
import threading
from dataclasses import dataclass
from typing import Deque, Optional

from ..runtime.logging import Ev, NULL_LOGGER


@dataclass
class QueueStatus:
    busy: bool
    pending_requests: int
    total_processed: int
    current_request_id: Optional[str]


class CancellationToken:
    """A flag the HTTP layer sets when the client goes away; callbacks run once on cancel."""

    def __init__(self):
        self._ev = threading.Event()
        self._cbs = []
        self._lock = threading.Lock()

    @property
    def cancelled(self) -> bool:
        return self._ev.is_set()

    def register(self, cb) -> None:
        with self._lock:
            if not self._ev.is_set():
                self._cbs.append(cb)
                return
        cb()

    def unregister(self, cb) -> None:
        with self._lock:
            if cb in self._cbs:
                self._cbs.remove(cb)

    def cancel(self) -> None:
        with self._lock:
            if self._ev.is_set():
                return
            self._ev.set()
            cbs, self._cbs = self._cbs, []
        for cb in cbs:
            cb()


NEVER = CancellationToken()


class QueueTicket:
    def __init__(self, queue: "InferenceQueue", ct: CancellationToken, request_id: Optional[str]):
        self._queue, self._ct, self.request_id = queue, ct, request_id
        self._ready = threading.Event()
        self._wake = threading.Event()          # set on ready or cancel: ends wait() early
        self.position = 0
        self.slot = -1                          # which of the queue's running slots this ticket holds once ready
        self.thread_id = threading.get_ident()  # the request thread that asked for it
        self._disposed = False
        self._queued = False
        ct.register(self._on_cancel)

    def _on_cancel(self) -> None:
        self._wake.set()
        self._queue._remove_cancelled(self)

    @property
    def is_ready(self) -> bool:
        return self._ready.is_set()

    @property
    def is_cancelled(self) -> bool:
        return self._ct.cancelled

    def _mark_ready(self) -> None:
        self._ready.set()
        self._wake.set()

    def wait(self, timeout: float) -> None:
        """Block until ready, cancelled, or ``timeout`` seconds have passed."""
        if not self.is_ready:
            self._wake.wait(timeout)

    def wait_until_ready(self) -> None:
        while not self.is_ready and not self.is_cancelled:
            self._wake.wait(1.0)

    def dispose(self) -> None:
        if self._disposed:
            return
        self._disposed = True
        self._ct.unregister(self._on_cancel)
        if self.is_ready:
            self._queue._release(self)
        else:
            self._queue._remove_cancelled(self)

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.dispose()


class InferenceQueue:
    def __init__(self, logger=None, capacity: int = 1):
        self._lock = threading.RLock()
        self._waiters: Deque[QueueTicket] = collections.deque()
        self._capacity = max(1, int(capacity))
        self._free_slots = list(range(self._capacity - 1, -1, -1))
        self._running = {}                      # ticket -> slot
        self._busy = False
        self._total = 0
        self._current: Optional[str] = None
        self._log = logger or NULL_LOGGER

    @property
    def pending_count(self) -> int:
        with self._lock:
            return len(self._waiters)

    @property
    def total_processed(self) -> int:
        return self._total

    @property
    def is_busy(self) -> bool:
        with self._lock:
            return self._busy

    def enqueue(self, ct: Optional[CancellationToken] = None, request_id: Optional[str] = None,
                prefer_slot: int = -1) -> QueueTicket:
        """``prefer_slot``: the running slot to take if it is free when this request starts (a chat session
        returning to the slot that still holds its KV cache); any free slot otherwise."""
        with self._lock:
            t = QueueTicket(self, ct or NEVER, request_id)
            t.prefer_slot = prefer_slot
            if len(self._running) < self._capacity:
                self._busy, self._current = True, request_id
                t.position = 0
                self._start(t)
                self._log.debug(Ev.QueueReady, "Inference slot acquired immediately for request {RequestId}",
                                RequestId=request_id or "(none)")
                return t
            self._waiters.append(t)
            t._queued = True
            t.position = len(self._waiters)
            self._log.info(Ev.QueueEnqueued, "Request {RequestId} queued at position {Position} (pending={PendingCount}, "
                           "current={CurrentRequestId})", RequestId=request_id or "(none)", Position=t.position,
                           PendingCount=len(self._waiters), CurrentRequestId=self._current or "(none)")
            return t

    def _release(self, done: QueueTicket) -> None:
        with self._lock:
            self._total += 1
            slot = self._running.pop(done, None)
            if slot is not None:
                self._free_slots.append(slot)
            if done._queued:
                self._discard(done)
            self._log.debug(Ev.QueueReleased, "Inference slot released for request {RequestId} (totalProcessed="
                            "{TotalProcessed}, pending={PendingCount})", RequestId=done.request_id or "(none)",
                            TotalProcessed=self._total, PendingCount=len(self._waiters))
            self._activate_next()

    def _discard(self, t: QueueTicket) -> None:
        try:
            self._waiters.remove(t)
        except ValueError:
            pass
        t._queued = False

    def _remove_cancelled(self, t: QueueTicket) -> None:
        with self._lock:
            if t._queued:
                self._discard(t)
                self._update_positions()
                self._log.info(Ev.QueueCancelled, "Cancelled queued request {RequestId} (pending={PendingCount})",
                               RequestId=t.request_id or "(none)", PendingCount=len(self._waiters))

    def _start(self, t: QueueTicket) -> None:
        want = getattr(t, "prefer_slot", -1)
        if want in self._free_slots:
            self._free_slots.remove(want)
            t.slot = want
        else:
            t.slot = self._free_slots.pop()
        self._running[t] = t.slot
        t._mark_ready()

    def slot_for_thread(self, thread_id: Optional[int] = None) -> int:
        """The running slot held by a ticket that ``thread_id`` (default: the caller) enqueued, or -1."""
        tid = threading.get_ident() if thread_id is None else thread_id
        with self._lock:
            for t, slot in self._running.items():
                if t.thread_id == tid:
                    return slot
        return -1

    def _activate_next(self) -> None:
        while self._waiters and len(self._running) < self._capacity:
            nxt = self._waiters.popleft()
            nxt._queued = False
            if nxt.is_cancelled:
                continue
            self._current = nxt.request_id
            nxt.position = 0
            self._start(nxt)
            self._update_positions()
            self._log.info(Ev.QueueReady, "Activated queued request {RequestId} (pending={PendingCount})",
                           RequestId=nxt.request_id or "(none)", PendingCount=len(self._waiters))
        if not self._running:
            self._busy, self._current = False, None

    def _update_positions(self) -> None:
        for i, t in enumerate(self._waiters):
            t.position = i + 1

    def get_status(self) -> QueueStatus:
        with self._lock:
            return QueueStatus(self._busy, len(self._waiters), self._total, self._current)
