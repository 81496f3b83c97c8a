"""Serving a model that spans several processes (tensor, pipeline or context parallel) from one front end.

The HTTP server, the CLI's interactive mode and the queue live on rank 0 only; the other ranks hold their
shards and must make exactly the calls rank 0 makes, in the same order, or the collectives and in-kernel
exchanges inside ``forward`` would not meet.  ``LeaderModel`` wraps rank 0's shard: every call that
touches the KV cache or runs the graph (forward, reset, truncate, sequence management, load / close) is
first announced to the followers, then executed locally.  ``follower_main`` is the other ranks' whole
program: receive a command, execute it on the local shard, repeat until told to stop.

Commands travel as small Python objects over ``torch.distributed.broadcast_object_list`` from rank 0 (host
side, a few hundred microseconds); the tensors of a step never do: each rank computes its own.  The
reference serves from a single process on a single device and has no counterpart.
"""
from __future__ import annotations

from typing import Any, Callable, Dict, Optional, Sequence



def _bcast(comm, obj: Any = None) -> Any:
    import torch.distributed as dist
    box = [obj]
    src = 0 if comm.group is None else dist.get_global_rank(comm.group, 0)
    dist.broadcast_object_list(box, src=src, group=comm.group, device=comm.device if comm.device.type == "cuda" else None)
    return box[0]


class LeaderModel:
    """Rank 0's shard, announcing every state-changing call to the followers before making it."""

    def __init__(self, model, comm, watchdog=None):
        self.__dict__["_model"] = model
        self.__dict__["_comm"] = comm
        self.__dict__["_watchdog"] = watchdog

    # everything not listed below (cfg, tokenizer, arch, kv, cache_length, ...) is the local shard's
    def __getattr__(self, name):
        return getattr(self.__dict__["_model"], name)

    def __setattr__(self, name, value):
        setattr(self.__dict__["_model"], name, value)

    def _tell(self, op: str, *args) -> None:
        # a follower that has gone quiet (or said it leaves) would make the broadcast below wait for ever: fail the
        # call with a typed error instead, before anything is launched
        wd = self._watchdog
        if wd is not None and wd.failed:
            from .errors import RankFailureError
            raise RankFailureError(wd.failed)
        _bcast(self._comm, (op, args))

    # ------------------------------------------------------------------ graph execution
    def forward(self, tokens: Sequence[int], want_logits: bool = True):
        tokens = [int(t) for t in tokens]
        self._tell("forward", tokens, bool(want_logits))
        return self._model.forward(tokens, want_logits)

    def forward_refill(self, tokens: Sequence[int], chunk: int = 2048):
        tokens = list(tokens)
        out = None
        for i in range(0, len(tokens), chunk):
            out = self.forward(tokens[i:i + chunk], want_logits=i + chunk >= len(tokens))
        return out

    def warm_up_kernels(self) -> None:
        self._tell("warm_up")
        self._model.warm_up_kernels()

    def recover_exchanges(self) -> int:
        """After an ``ExchangeTimeoutError``: every rank drops its in-kernel exchanges and symmetric buffers at the same
        point and rebuilds them on next use (ModelBase.recover_exchanges); weights stay resident, the caches are reset."""
        self._tell("recover")
        return self._model.recover_exchanges()

    # ------------------------------------------------------------------ cache and sequences
    def reset_kv_cache(self) -> None:
        self._tell("reset")
        self._model.reset_kv_cache()

    def truncate_kv_cache(self, n_tokens: int) -> None:
        self._tell("truncate", int(n_tokens))
        self._model.truncate_kv_cache(n_tokens)

    def new_sequence(self):
        self._tell("new_seq")
        return self._model.new_sequence()

    def free_sequence(self, seq) -> None:
        self._tell("free_seq", seq.seq_id)
        self._model.free_sequence(seq)

    def bind_sequence(self, seq) -> None:
        self._tell("bind_seq", seq.seq_id if seq is not None else None)
        self._model.bind_sequence(seq)

    # ------------------------------------------------------------------ image / audio embeddings
    @property
    def multimodal(self):
        """The injector runs on rank 0 only (it owns the encoders); its embeddings reach the model through
        :meth:`set_vision_embeddings` below, which also hands them to the followers."""
        if self._model.multimodal is None:
            return None
        inj = self.__dict__.get("_injector")
        if inj is None:
            from ..multimodal.injector import MultimodalInjector
            inj = self.__dict__["_injector"] = MultimodalInjector(self)
        return inj

    def set_vision_embeddings(self, embeddings, insert_position: int) -> None:
        self._tell("embed", embeddings.detach().float().cpu(), int(insert_position))
        self._model.set_vision_embeddings(embeddings, insert_position)

    set_audio_embeddings = set_vision_embeddings

    def close(self) -> None:
        self._tell("unload")
        close = getattr(self._model, "close", None)
        if close is not None:
            close()


def layout_create(mode: str) -> Optional[Callable]:
    """The ``create`` callable (for :func:`leader_factory` / :func:`follower_main`) of a parallel layout: ``tp`` cuts the
    weights across the ranks (the default, ``None``), ``pp`` gives each rank a range of layers, ``cp`` gives every rank
    the whole model and deals long prompts to them slice by slice."""
    mode = (mode or "tp").lower()
    if mode == "tp":
        return None
    if mode not in ("pp", "cp"):
        raise ValueError(f"unknown parallel layout {mode!r} (tp, pp or cp)")

    def create(path, device, *, tp_rank=0, tp_size=1, comm=None, **kw):
        from ..models.base import ModelBase
        if mode == "cp":
            return ModelBase.create(path, device, cp_comm=comm, **kw)
        from .pipeline import PipelinedModel
        return PipelinedModel(ModelBase.create(path, device, pp_rank=comm.rank, pp_size=comm.size, pp_comm=comm, **kw))
    return create


def start_watchdog(comm, timeout_s: float, store=None, on_failure: Optional[Callable] = None):
    """Heartbeats of this job's ranks over its key-value store (the process group's own store unless one is given):
    returns the started ``Watchdog``, or ``None`` when ``timeout_s`` is 0 or no store can be had."""
    if timeout_s <= 0:
        return None
    from .watchdog import Heartbeat, Watchdog
    if store is None:
        try:
            from torch.distributed.distributed_c10d import _get_default_store
            store = _get_default_store()
        except Exception:
            return None
    return Watchdog(Heartbeat(store, comm.rank, comm.size), timeout_s, on_failure=on_failure).start()


def leader_factory(comm, create: Optional[Callable] = None, watchdog=None) -> Callable:
    """A ``model_factory`` for ``ModelService`` (or any host) on rank 0: tells the followers which file to
    load, loads rank 0's shard and returns it wrapped."""
    def factory(path: str, device, **kw):
        from ..models.base import ModelBase
        plain = {k: v for k, v in kw.items() if isinstance(v, (int, float, str, bool, type(None)))}
        _bcast(comm, ("load", (path, plain)))
        make = create or ModelBase.create
        dev = comm.device if comm.device.type == "cuda" else device
        return LeaderModel(make(path, dev, tp_rank=comm.rank, tp_size=comm.size, comm=comm, **kw), comm, watchdog)
    return factory


def shutdown_followers(comm) -> None:
    _bcast(comm, ("stop", ()))


def follower_main(comm, create: Optional[Callable] = None, device=None) -> int:
    """Program of ranks 1 .. N-1: mirror rank 0's calls until it says stop.  Returns the number of
    commands executed."""
    from ..models.base import ModelBase
    make = create or ModelBase.create
    model = None
    seqs: Dict[int, Any] = {}
    n = 0
    while True:
        op, args = _bcast(comm)
        n += 1
        if op == "stop":
            return n
        if op == "load":
            path, kw = args
            model, seqs = None, {}
            dev = comm.device if comm.device.type == "cuda" else (device or "cpu")
            model = make(path, dev, tp_rank=comm.rank, tp_size=comm.size, comm=comm, **kw)
        elif op == "unload":
            model, seqs = None, {}
        elif model is None:
            raise RuntimeError(f"follower received {op!r} before a model was loaded")
        elif op == "forward":
            model.forward(args[0], args[1])
        elif op == "embed":
            model.set_vision_embeddings(args[0].to(model.device), args[1])
        elif op == "warm_up":
            model.warm_up_kernels()
        elif op == "recover":
            model.recover_exchanges()
        elif op == "reset":
            model.reset_kv_cache()
        elif op == "truncate":
            model.truncate_kv_cache(args[0])
        elif op == "new_seq":
            s = model.new_sequence()
            seqs[s.seq_id] = s
        elif op == "free_seq":
            s = seqs.pop(args[0], None) or (model._default_seq if model._default_seq is not None and model._default_seq.seq_id == args[0] else None)
            if s is not None:
                model.free_sequence(s)
        elif op == "bind_seq":
            model.bind_sequence(seqs.get(args[0]) if args[0] is not None else None)
        else:
            raise RuntimeError(f"unknown command {op!r}")
