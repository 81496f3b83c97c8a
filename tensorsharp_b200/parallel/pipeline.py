"""Pipeline parallelism: contiguous layer ranges on successive ranks, the residual stream handed from
stage to stage with point-to-point sends (NCCL on GPUs, gloo on CPU), the sampled token broadcast back
from the last stage so that every stage advances its own part of the KV cache.

The reference runs every model in one process on one device and has no counterpart.  A stage is a model
built with ``pp_rank`` / ``pp_size`` / ``pp_comm`` (see ``ModelBase``); all stages make the same
``forward`` calls, only the last one gets logits back.
"""
from __future__ import annotations

from typing import Callable, List, Optional, Sequence

import torch


def _global_rank(comm, r: int) -> int:
    if comm.group is None:
        return r
    import torch.distributed as dist
    return dist.get_global_rank(comm.group, r)


def send_hidden(comm, dst: int, h: torch.Tensor) -> None:
    import torch.distributed as dist
    dist.send(h.contiguous(), _global_rank(comm, dst), group=comm.group)


def recv_hidden(comm, src: int, shape, device) -> torch.Tensor:
    import torch.distributed as dist
    h = torch.empty(shape, dtype=torch.float32, device=device)
    dist.recv(h, _global_rank(comm, src), group=comm.group)
    return h


def broadcast_token(comm, token: Optional[int], device) -> int:
    """The last stage's choice, delivered to every stage."""
    import torch.distributed as dist
    t = torch.tensor([token if token is not None else 0], dtype=torch.int64, device=device)
    dist.broadcast(t, _global_rank(comm, comm.size - 1), group=comm.group)
    return int(t[0])


def generate(model, prompt: Sequence[int], max_tokens: int, pick: Optional[Callable[[torch.Tensor], int]] = None,
             eos_ids: Sequence[int] = (), prefill_chunk: int = 2048) -> List[int]:
    """Greedy (or ``pick``-driven) generation over a pipeline of stages; every rank calls this with the same
    arguments and every rank returns the same token list."""
    comm = model.pp_comm
    pick = pick or (lambda lg: int(lg.argmax()))
    eos = set(int(e) for e in eos_ids)
    logits = model.forward_refill(list(prompt), prefill_chunk)
    out: List[int] = []
    for _ in range(max_tokens):
        t = broadcast_token(comm, pick(logits) if model.is_last_stage else None, model.device)
        if t in eos:
            break
        out.append(t)
        logits = model.forward([t])
    return out


class PipelinedModel:
    """A pipeline stage with the plain single-process model surface: ``forward`` returns the logits on
    every rank (the last stage computes them and broadcasts the row), so a host that samples on the CPU
    with a shared seed (the CLI's loops, the server's token loop on rank 0 with followers mirroring it)
    runs unchanged on top of a pipeline.  Costs one broadcast of ``vocab`` floats per step."""

    def __init__(self, stage):
        self.__dict__["_stage"] = stage

    def __getattr__(self, name):
        return getattr(self.__dict__["_stage"], name)

    def __setattr__(self, name, value):
        setattr(self.__dict__["_stage"], name, value)

    def forward(self, tokens: Sequence[int], want_logits: bool = True):
        import torch.distributed as dist
        st = self._stage
        out = st.forward(tokens, want_logits)
        if not want_logits:
            return None
        comm = st.pp_comm
        if out is None:
            out = torch.empty(st.cfg.vocab, dtype=torch.float32, device=st.device)
        else:
            out = out[:st.cfg.vocab].float().contiguous()
        dist.broadcast(out, _global_rank(comm, comm.size - 1), group=comm.group)
        return out

    def forward_refill(self, tokens: Sequence[int], chunk: int = 2048):
        tokens = list(tokens)
        out = None
        for i in range(0, len(tokens), chunk):
            out = self.forward(tokens[i:i + chunk], want_logits=i + chunk >= len(tokens))
        return out

    def warm_up_kernels(self) -> None:
        n = max(1, min(8, self.max_context - 2))
        tok = min(self.cfg.vocab - 1, 100)
        self.forward([tok] * n)
        self.forward([tok])
        self.reset_kv_cache()
