"""Process-group plumbing and the shard arithmetic of tensor / expert parallelism.

The reference is single-device (TensorSharp.Models/ModelBase.cs:236-264 binds device 0
only) and has no collective of any kind, so everything here is new: one process per GPU,
``torch.distributed`` (NCCL on GPUs, Gloo on CPU ranks) for bootstrap and the baseline
collectives, and the same interface implemented in-process for single-rank runs and
unit tests.  The fused compute + collective kernels live in ``parallel/fused.py`` and use
this module only for rendezvous.
"""
from __future__ import annotations

from typing import List, Optional, Tuple

import torch


class Communicator:
    """Thin wrapper over a ``torch.distributed`` process group (or no group at all)."""

    def __init__(self, rank: int = 0, size: int = 1, device=None, group=None):
        self.rank, self.size = rank, size
        self.device = torch.device(device) if device is not None else torch.device("cpu")
        self.group = group
        self.bytes_reduced = 0          # payload bytes this rank contributed to all-reduces
        self.bytes_gathered = 0

    @property
    def active(self) -> bool:
        return self.size > 1

    def all_reduce(self, t: torch.Tensor) -> torch.Tensor:
        if self.size > 1:
            import torch.distributed as dist
            dist.all_reduce(t, group=self.group)
            self.bytes_reduced += t.numel() * t.element_size()
        return t

    def all_gather_cat(self, t: torch.Tensor, dim: int = -1) -> torch.Tensor:
        """Concatenate every rank's ``t`` along ``dim`` (equal shapes on all ranks)."""
        if self.size == 1:
            return t
        import torch.distributed as dist
        parts = [torch.empty_like(t) for _ in range(self.size)]
        dist.all_gather(parts, t.contiguous(), group=self.group)
        self.bytes_gathered += t.numel() * t.element_size() * (self.size - 1)
        return torch.cat(parts, dim)

    def all_gather_list(self, t: torch.Tensor) -> List[torch.Tensor]:
        if self.size == 1:
            return [t]
        import torch.distributed as dist
        parts = [torch.empty_like(t) for _ in range(self.size)]
        dist.all_gather(parts, t.contiguous(), group=self.group)
        return parts

    def barrier(self) -> None:
        if self.size > 1:
            import torch.distributed as dist
            dist.barrier(group=self.group)


def init_from_env(backend: Optional[str] = None) -> Communicator:
    """Join the job described by RANK / WORLD_SIZE / LOCAL_RANK / MASTER_* (torchrun)."""
    import os
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    cuda = torch.cuda.is_available()
    dev = torch.device("cuda", local) if cuda else torch.device("cpu")
    if cuda:
        torch.cuda.set_device(dev)
    if world > 1:
        import torch.distributed as dist
        if not dist.is_initialized():
            kw = {"device_id": dev} if cuda else {}
            dist.init_process_group(backend or ("nccl" if cuda else "gloo"), **kw)
    return Communicator(rank, world, dev)


# ---------------------------------------------------------------------------- shard arithmetic
def even_split(n: int, parts: int, rank: int) -> Tuple[int, int]:
    """[start, stop) of ``rank``'s share when ``n`` items are dealt as evenly as possible
    (the first ``n % parts`` ranks get one extra)."""
    base, rem = divmod(n, parts)
    start = rank * base + min(rank, rem)
    return start, start + base + (1 if rank < rem else 0)


def block_split(n: int, block: int, parts: int, rank: int) -> Tuple[int, int]:
    """Like :func:`even_split` but in units of ``block`` values, for a dimension that is the
    K axis of a block-quantised matrix (a 256-value K-quant super-block cannot be cut)."""
    if n % block:
        raise ValueError(f"{n} is not a multiple of the block size {block}")
    s, e = even_split(n // block, parts, rank)
    return s * block, e * block


def head_split(n_heads: int, n_kv_heads: int, parts: int, rank: int):
    """Query / KV head ranges of ``rank``.  KV heads are dealt evenly and each rank takes the query heads that attend
    to its KV heads, so no KV head is replicated; when there are fewer KV heads than ranks (and the ranks divide evenly
    among them) a KV head is held by several ranks, which share its group of query heads."""
    g = n_heads // n_kv_heads
    if n_kv_heads % parts == 0:
        k0, k1 = even_split(n_kv_heads, parts, rank)
        return (k0 * g, k1 * g), (k0, k1)
    if parts % n_kv_heads == 0 and g % (parts // n_kv_heads) == 0:
        rep = parts // n_kv_heads
        per = g // rep
        k = rank // rep
        q0 = k * g + (rank % rep) * per
        return (q0, q0 + per), (k, k + 1)
    raise ValueError(f"{n_kv_heads} KV heads (of {n_heads} query heads) cannot be split over {parts} ranks")
