"""Several requests at once: a pool of model services over one loaded model.

With ``--max-batch N`` the admission queue lets N requests run together.  Each running request is
served by its own ``ModelService`` (prompt rendering, KV reuse, stop sequences, metrics: all unchanged)
whose "model" is a slot of a ``GatheredModel``: one sequence of the shared KV pool, with every ``forward``
merged into the step the other running requests take at that moment (runtime/gather.py).  The pool has
the surface of a single ``ModelService`` so the HTTP layer does not change; which slot a call goes to
follows from the queue ticket that the calling request thread holds.

The reference serves strictly one request at a time (TensorSharp.Server/InferenceQueue.cs).
"""
from __future__ import annotations

from typing import Iterator, List, Optional

from ..runtime.gather import GatheredModel
from ..runtime.logging import NULL_LOGGER
from .model_service import ModelService, backend_device
from .options import canonicalize_backend


class ServicePool:
    def __init__(self, logger, queue, n_slots: int, max_context: Optional[int] = None, model_factory=None):
        self._log = logger or NULL_LOGGER
        self._queue, self._n = queue, max(1, int(n_slots))
        self._max_context, self._factory = max_context, model_factory
        self._gather: Optional[GatheredModel] = None
        self._session_slot = {}
        self._slots: List[ModelService] = [
            ModelService(logger, model_factory=self._slot_factory(i), max_context=max_context, max_sessions=1) for i in range(self._n)]

    def _slot_factory(self, i: int):
        def factory(path, device, **kw):
            return self._gather.slot(i)
        return factory

    # ------------------------------------------------------------------ model lifetime
    def load_model(self, model_path: str, mmproj_path: Optional[str], backend: Optional[str]) -> None:
        make = self._factory
        if make is None:
            from ..models.base import ModelBase
            make = ModelBase.create
        kw = {"max_seqs": self._n + 1}
        if self._max_context:
            kw["max_context"] = self._max_context
        b = canonicalize_backend(backend) or "cpu"
        real = make(model_path, backend_device(b if b in ("b200", "cpu") else "cpu"), **kw)
        previous, self._gather = self._gather, GatheredModel(real, self._n)
        for i, s in enumerate(self._slots):
            # each service lets go of its old slot and takes the new one; the first one also loads the multimodal
            # projector, once, into the shared model's injector (the other slots find the encoders there)
            s.load_model(model_path, mmproj_path if i == 0 else None, backend)
        if previous is not None:
            previous.close()

    def close(self) -> None:
        for s in self._slots:
            s.close()
        if self._gather is not None:
            self._gather.close()
            self._gather = None

    # ------------------------------------------------------------------ the single-service surface
    @property
    def is_loaded(self) -> bool:
        return self._gather is not None and self._slots[0].is_loaded

    @property
    def loaded_model_name(self):
        return self._slots[0].loaded_model_name

    @property
    def loaded_mmproj_name(self):
        return self._slots[0].loaded_mmproj_name

    @property
    def loaded_backend(self):
        return self._slots[0].loaded_backend

    @property
    def architecture(self):
        return self._slots[0].architecture

    @property
    def model(self):
        return self._gather.model if self._gather is not None else None

    @property
    def gather(self) -> Optional[GatheredModel]:
        return self._gather

    def __getattr__(self, name):
        # anything else (available_models, is_mmproj helpers ...) is the same on every slot
        return getattr(self._slots[0], name)

    def _mine(self, session=None) -> ModelService:
        slot = self._queue.slot_for_thread()
        slot = slot if 0 <= slot < self._n else 0
        if session is not None:
            self._session_slot[getattr(session, "id", None)] = slot
        return self._slots[slot]

    def preferred_slot(self, session) -> int:
        """The slot that served this chat session last (it still holds the session's KV cache), or -1."""
        return self._session_slot.get(getattr(session, "id", None), -1)

    def _bracket(self, svc: ModelService, it: Iterator) -> Iterator:
        slot_model = svc.model
        entered = slot_model is not None and hasattr(slot_model, "__enter__")
        if entered:
            slot_model.__enter__()
        try:
            yield from it
        finally:
            if entered:
                slot_model.__exit__(None, None, None)

    def chat_stream_with_metrics(self, *a, **k) -> Iterator:
        svc = self._mine(k.get("session"))
        return self._bracket(svc, svc.chat_stream_with_metrics(*a, **k))

    def chat_stream(self, *a, **k) -> Iterator:
        svc = self._mine()
        return self._bracket(svc, svc.chat_stream(*a, **k))

    def generate_stream(self, *a, **k) -> Iterator:
        svc = self._mine()
        return self._bracket(svc, svc.generate_stream(*a, **k))

    def reset_session(self, session) -> None:
        for s in self._slots:
            s.reset_session(session)

    def dispose_session(self, session) -> None:
        self._session_slot.pop(getattr(session, "id", None), None)
        for s in self._slots:
            s.dispose_session(session)
