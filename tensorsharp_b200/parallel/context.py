"""Context-parallel (sequence-sharded) causal attention for long prefills.

Rank r holds queries, keys and values of tokens ``[r * shard, (r + 1) * shard)``.  Every rank publishes
its K / V shard in a peer-mapped staging buffer; a rank pulls each lower rank's shard across NVLink once
(plain peer loads in a kernel of this library), runs the flash-attention kernel on the local copy with
every key visible, runs it causally on its own shard, and merges the partial outputs by their
log-sum-exp weights (csrc/context_parallel.cu).  Nothing like it exists in the reference, whose long
context path is single-device (Gemma4Model.cs:593-637 chunked prefill).
"""
from __future__ import annotations

import ctypes as C

import torch

from ..ops import native
from .symm import SymmetricBuffer, _lib


class ContextParallelAttention:
    def __init__(self, comm, max_shard: int, Hkv: int, Dh: int):
        self.comm, self.max_shard, self.Hkv, self.Dh = comm, int(max_shard), Hkv, Dh
        lib = _lib()
        for name in ("tsb_cp_struct_bytes", "tsb_cp_init", "tsb_cp_publish", "tsb_cp_pull", "tsb_cp_merge"):
            getattr(lib, name).restype = C.c_int
        lib.tsb_cp_region_bytes.restype = C.c_long
        kv_row = Hkv * Dh
        self.region = SymmetricBuffer(comm, lib.tsb_cp_region_bytes(C.c_long(self.max_shard), C.c_long(kv_row)))
        dev = comm.device
        self.local = torch.zeros(8, dtype=torch.int32, device=dev)
        self.ticket = torch.zeros(1, dtype=torch.int32, device=dev)
        self.struct = torch.zeros(lib.tsb_cp_struct_bytes(), dtype=torch.uint8, device=dev)
        arr = C.c_void_p * comm.size
        native.check(lib.tsb_cp_init(C.c_void_p(self.struct.data_ptr()), arr(*self.region.ptrs), C.c_void_p(self.local.data_ptr()),
                                     C.c_int(comm.rank), C.c_int(comm.size), C.c_long(self.max_shard), C.c_long(kv_row)), "cp_init")
        self.k_pull = torch.empty((self.max_shard, Hkv, Dh), dtype=torch.bfloat16, device=dev)
        self.v_pull = torch.empty_like(self.k_pull)
        comm.barrier()

    def attention(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float, softcap: float = 0.0) -> torch.Tensor:
        """``q`` ``[n, Hq, Dh]``, ``k`` / ``v`` ``[n, Hkv, Dh]`` bf16: this rank's shard (all shards the same
        length ``n``).  Returns ``[n, Hq, Dh]``: causal attention over the whole sequence."""
        from ..ops import kernels as kk
        lib = kk._lib()
        n, Hq, Dh = q.shape
        Hkv = k.shape[1]
        assert n <= self.max_shard and k.is_contiguous() and v.is_contiguous() and q.is_contiguous()
        dev = q.device
        sp = C.c_void_p(self.struct.data_ptr())
        elems = n * Hkv * Dh
        native.check(lib.tsb_cp_publish(sp, kk._p(k), kk._p(v), C.c_long(elems), kk._stream()), "cp_publish")
        kk._count(2)
        r = self.comm.rank
        S = r + 1
        parts = torch.empty((S, n, Hq, Dh), dtype=torch.bfloat16, device=dev)
        lse = torch.empty((S, n, Hq), dtype=torch.float32, device=dev)
        table = torch.zeros((1, 1), dtype=torch.int32, device=dev)
        lens = torch.tensor([n], dtype=torch.int32, device=dev)
        cu_q = torch.tensor([0, n], dtype=torch.int32, device=dev)
        seen_all = torch.tensor([n], dtype=torch.int32, device=dev)          # first query sits after the whole shard
        page = 1 << 30
        # own shard first (needs no transfer), then the remote ones as they arrive
        kk.attn_prefill(q, k, v, table, lens, cu_q, n, scale=scale, Hq=Hq, Hkv=Hkv, Dh=Dh, page_size=page, softcap=softcap,
                        out=parts[r], lse_out=lse[r])
        for s in range(r):
            native.check(lib.tsb_cp_pull(sp, C.c_int(s), kk._p(self.k_pull), kk._p(self.v_pull), C.c_long(elems),
                                         kk._p(self.ticket), kk._stream()), "cp_pull")
            kk._count(1)
            kk.attn_prefill(q, self.k_pull, self.v_pull, table, lens, cu_q, n, scale=scale, Hq=Hq, Hkv=Hkv, Dh=Dh,
                            page_size=page, softcap=softcap, out=parts[s], lse_out=lse[s], q_pos0=seen_all)
        if S == 1:
            return parts[0]
        out = torch.empty_like(q)
        native.check(lib.tsb_cp_merge(kk._p(parts), kk._p(lse), kk._p(out), C.c_int(S), C.c_long(n * Hq), C.c_int(Dh),
                                      kk._stream()), "cp_merge")
        kk._count(1)
        return out

    def status(self) -> int:
        torch.cuda.synchronize(self.comm.device)
        return int(self.local[4].item())

    def close(self) -> None:
        torch.cuda.synchronize(self.comm.device)
        self.region.close()


# ---------------------------------------------------------------------------------------------------
# Context-parallel prefill of a whole model: the pieces that are the same for every architecture.
# Each rank of the group holds all the weights and runs the layers on its slice of the prompt; after a
# layer's K / V rows are computed they are exchanged, so that every rank ends with the full cache and
# the decode steps that follow can run on every rank alike (or on any one of them).

def shard_bounds(T: int, size: int, rank: int):
    """Token range of ``rank`` when ``T`` prompt tokens are dealt to ``size`` ranks in order (sizes differ by one at most)."""
    base, rem = divmod(T, size)
    t0 = rank * base + min(rank, rem)
    return t0, t0 + base + (1 if rank < rem else 0)


def balanced_ranges(T: int, size: int, rank: int):
    """Token ranges of ``rank`` when the prompt is cut into ``2 * size`` pieces and rank r takes piece r and piece
    ``2 * size - 1 - r``: under a causal mask every rank then attends to about the same number of keys (with whole
    contiguous slices the last rank would do almost twice the average).  Falls back to one contiguous slice when the
    prompt has fewer than ``2 * size`` tokens."""
    if T < 2 * size:
        return [shard_bounds(T, size, rank)]
    return [shard_bounds(T, 2 * size, rank), shard_bounds(T, 2 * size, 2 * size - 1 - rank)]


def shard_batch(batch, t0, t1=None):
    """Tokens ``[t0, t1)`` of a one-sequence batch (or several such ranges, given as a list of pairs) as a batch of their
    own: each range is a packed row that sees the cache up to its own last position, as a chunk of a chunked prefill
    does; the rows share the sequence's block table."""
    from ..ops.functional import Batch
    ranges = [(t0, t1)] if t1 is not None else list(t0)
    assert batch.B == 1 and all(0 <= a < b <= batch.T for a, b in ranges)
    dev = batch.tokens.device
    lens = [b - a for a, b in ranges]
    kv = [batch.h_kv_lens[0] - (batch.T - b) for _, b in ranges]
    cu = [0]
    for n in lens:
        cu.append(cu[-1] + n)
    pick = lambda t: torch.cat([t[a:b] for a, b in ranges]).contiguous()                      # noqa: E731
    R = len(ranges)
    return Batch(tokens=pick(batch.tokens), positions=pick(batch.positions), slots=pick(batch.slots),
                 cu_q=torch.tensor(cu, dtype=torch.int32, device=dev), kv_lens=torch.tensor(kv, dtype=torch.int32, device=dev),
                 block_table=batch.block_table.expand(R, -1).contiguous(),
                 last_idx=torch.tensor([c - 1 for c in cu[1:]], dtype=torch.int64, device=dev),
                 seq_slots=batch.seq_slots.expand(R).contiguous(), max_q_len=max(lens), max_kv_len=max(kv), is_decode=False,
                 page_size=batch.page_size, h_cu_q=tuple(cu), h_kv_lens=tuple(kv))


def exchange_kv_shards(comm, batch, rank_bounds, k_cache: torch.Tensor, v_cache: torch.Tensor) -> None:
    """Every rank has written the K / V rows of its own tokens into its cache; fetch the other ranks' rows
    (one all-gather of the padded shards) and write them at the same tokens' slots of this rank's cache.
    ``rank_bounds[r]`` is rank r's range ``(t0, t1)`` or its list of ranges."""
    as_list = lambda x: [x] if isinstance(x[0], int) else list(x)                             # noqa: E731
    per_rank = [as_list(b) for b in rank_bounds]
    slots_of = lambda rs: torch.cat([batch.slots[a:b] for a, b in rs])                        # noqa: E731
    count = [sum(b - a for a, b in rs) for rs in per_rank]
    r = comm.rank
    n_max = max(count)
    mine = torch.zeros((2, n_max) + tuple(k_cache.shape[1:]), dtype=k_cache.dtype, device=k_cache.device)
    own = slots_of(per_rank[r])
    mine[0, :count[r]] = k_cache.index_select(0, own)
    mine[1, :count[r]] = v_cache.index_select(0, own)
    for s, part in enumerate(comm.all_gather_list(mine)):
        if s == r:
            continue
        idx = slots_of(per_rank[s])
        k_cache.index_copy_(0, idx, part[0, :count[s]])
        v_cache.index_copy_(0, idx, part[1, :count[s]])
