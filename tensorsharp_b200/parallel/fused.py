"""Fused compute + collective paths of tensor parallelism.

``TpExchange`` replaces "row-parallel GEMV, NCCL all-reduce, residual add, RMSNorm, activation
quantisation" (five launches and a library collective) by two kernels of this library: the GEMV
stores its partial sums, tagged with the exchange number, into every rank's mailbox over NVLink
as its rows finish (``linear_push``), and one kernel polls its own mailbox, adds the partials to
the residual stream in rank order, normalises and emits the next GEMV's quantised input
(``reduce_norm``).  The wire protocol is described in csrc/tp_fused.cuh.  Used for batches of
up to ``max_rows`` tokens (decode and short prefill); long prefill keeps the GEMM + NCCL path.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional

import torch

from ..ops import native
from ..ops.functional import Act
from ..quant.qweight import QuantWeight
from .symm import SymmetricBuffer, _lib


class TpExchange:
    def __init__(self, comm, max_rows: int, max_d: int):
        self.comm, self.max_rows, self.max_d = comm, int(max_rows), int(max_d)
        lib = _lib()
        n = comm.size
        self.mail = SymmetricBuffer(comm, lib.tsb_tp_mailbox_bytes(C.c_int(n), C.c_long(self.max_rows), C.c_long(self.max_d)))
        dev = comm.device
        self.counters = torch.zeros(8, dtype=torch.int32, device=dev)
        self.struct = torch.zeros(lib.tsb_tp_struct_bytes(), dtype=torch.uint8, device=dev)
        arr = C.c_void_p * n
        native.check(lib.tsb_tp_init(C.c_void_p(self.struct.data_ptr()), arr(*self.mail.ptrs),
                                     C.c_void_p(self.counters.data_ptr()), C.c_int(comm.rank), C.c_int(n),
                                     C.c_long(self.max_rows), C.c_long(self.max_d)), "tp_init")
        comm.barrier()
        self.exchanges = 0

    # ------------------------------------------------------------------ the two kernels
    def linear_push(self, a: Act, w: QuantWeight, bias: Optional[torch.Tensor] = None) -> None:
        """Partial ``a @ w^T`` of this rank (``w`` holds its slice of the input features) into
        every rank's mailbox."""
        from ..ops import functional as F
        from ..ops import kernels as k
        T = a.T
        if T > self.max_rows or w.N > self.max_d:
            raise ValueError(f"exchange sized for [{self.max_rows}, {self.max_d}], got [{T}, {w.N}]")
        if w.uses_q8_activations:
            F._ensure_q8(a)
            xq, xds, xb = a.q, a.ds, None
        else:
            xq, xds, xb = None, None, a.b.contiguous()
        ps = k._planes(w)
        lib = k._lib()
        lib.tsb_gemv_push.restype = C.c_int
        native.check(lib.tsb_gemv_push(ps[0], ps[1], ps[2], ps[3], C.c_int(int(w.ggml_type)), C.c_int(w.N), C.c_int(w.K),
                                       k._p(xq), k._p(xds), k._p(xb), None, k._p(bias), None, None, None, C.c_int(T),
                                       C.c_int(1), C.c_int(1), C.c_int(1), C.c_int(0),
                                       C.c_void_p(self.struct.data_ptr()), k._stream()), "gemv_push")
        k._count(1)

    def linear_push_fused(self, x: torch.Tensor, w: QuantWeight, bias: Optional[torch.Tensor] = None) -> None:
        """``linear_push`` for at most ``F.FUSED_MAX_M`` rows of a plain bf16 / f32 activation: the
        int8 quantisation of the input happens inside the projection kernel as well."""
        from ..ops import functional as F
        from ..ops import kernels as k
        if not F.can_fuse(x, w):
            return self.linear_push(F.as_act(x), w, bias)
        x = x.contiguous()
        kw = {"x_f32": x} if x.dtype == torch.float32 else {"x_bf16": x if x.dtype == torch.bfloat16 else x.to(torch.bfloat16)}
        k.fused_gemv(w, bias=bias, push=self.struct.data_ptr(), **kw)

    def reduce_norm(self, h: torch.Tensor, w: Optional[torch.Tensor], eps: float, want_q8: bool = True,
                    want_bf16: bool = True, norm: bool = True, parts: int = 1) -> Optional[Act]:
        """``h += sum of all ranks' partials`` (in place, f32), then ``RMSNorm(h) * w`` as the next
        projection's input.  With ``norm=False`` only the residual stream is updated.  ``parts`` > 1:
        every rank sent that many partial rows per token (mixture-of-experts slots)."""
        from ..ops import kernels as k
        assert h.dtype == torch.float32 and h.is_contiguous()
        T, D = h.shape
        yb = torch.empty((T, D), dtype=torch.bfloat16, device=h.device) if norm and want_bf16 else None
        yq = yds = None
        if norm and want_q8:
            yq = torch.empty((T, D), dtype=torch.int8, device=h.device)
            yds = torch.empty((T, D // 32, 2), dtype=torch.float32, device=h.device)
        lib = k._lib()
        lib.tsb_tp_reduce_norm.restype = C.c_int
        native.check(lib.tsb_tp_reduce_norm(C.c_void_p(self.struct.data_ptr()), k._p(h), k._p(w if norm else None),
                                            C.c_float(eps), C.c_int(T), C.c_int(D), C.c_int(parts), k._p(yb), k._p(yq),
                                            k._p(yds), k._stream()), "tp_reduce_norm")
        k._count(1)
        self.exchanges += 1
        return Act(yb, yq, yds) if norm else None

    def fits(self, y: torch.Tensor) -> bool:
        """Whether :meth:`all_reduce` takes ``y``: f32, contiguous, 2-D, within the mailbox's rows and row length."""
        return (y.is_cuda and y.dtype == torch.float32 and y.dim() == 2 and y.is_contiguous() and 0 < y.shape[0] <= self.max_rows
                and y.shape[1] <= self.max_d and y.shape[1] % 4 == 0 and y.data_ptr() % 16 == 0)

    def all_reduce(self, y: torch.Tensor) -> torch.Tensor:
        """Sum ``y`` [rows, D] over the ranks in place (rank order, so every rank holds the same bits): one kernel
        that stores its rows into every peer's mailbox and adds what the peers stored into its own."""
        from ..ops import kernels as k
        lib = k._lib()
        lib.tsb_tp_all_reduce.restype = C.c_int
        native.check(lib.tsb_tp_all_reduce(C.c_void_p(self.struct.data_ptr()), k._p(y), C.c_int(y.shape[0]), C.c_int(y.shape[1]),
                                           k._stream()), "tp_all_reduce")
        k._count(1)
        self.exchanges += 1
        self.comm.bytes_reduced += y.numel() * 4
        return y

    # ------------------------------------------------------------------ health
    def status(self) -> int:
        """0 when every wait so far was satisfied, else 1 + the rank whose flag did not arrive
        within the kernel's time limit (synchronises the device)."""
        torch.cuda.synchronize(self.comm.device)
        return int(self.counters[4].item())

    def check(self) -> None:
        """Raise ``ExchangeTimeoutError`` if any wait so far ran out (synchronises the device)."""
        from .errors import ExchangeTimeoutError
        code = self.status()
        if code:
            raise ExchangeTimeoutError("tensor-parallel mailbox exchange", code)

    def close(self) -> None:
        torch.cuda.synchronize(self.comm.device)
        self.mail.close()


def tensor_from_ptr(ptr: int, shape, dtype: torch.dtype, device) -> torch.Tensor:
    """A tensor aliasing raw device memory owned by someone else (the symmetric region)."""
    esize = torch.empty((), dtype=dtype).element_size()
    n = 1
    for d in shape:
        n *= int(d)

    class _Raw:
        __cuda_array_interface__ = {"shape": (n * esize,), "typestr": "|u1", "data": (int(ptr), False), "version": 3,
                                    "strides": None}
    return torch.as_tensor(_Raw(), device=device).view(dtype).view(*shape)


class TpSeqParallel:
    """Sequence-parallel prefill exchange (csrc/tp_fused.cuh, TpSeq): tokens are dealt to ranks in
    shards of ``shard`` rows (a multiple of the GEMM's 128-token tile).

    * ``gemm_rs``  row-parallel GEMM whose epilogue stores every tile into the token owner's
      accumulator over NVLink (GEMM -> reduce-scatter in one kernel; the owner adds the slots),
    * ``norm_gather``  the owner folds the sum into its shard of the residual stream, normalises and
      stores the rows into every rank's gathered buffer (all-gather inside the norm kernel),
    * ``gemm_ag``  column-parallel GEMM on the gathered buffer whose TMA producer waits per token
      tile for the shard it needs (all-gather -> GEMM).
    * ``norm_gather(local_only=True)`` + ``dispatch`` + ``push_rows(k_routed=...)`` + ``norm_gather(acc_k=...)``:
      expert-parallel dispatch and combine, in which a token's row travels only to the ranks that hold its experts and
      only their partial sums travel back.
    """

    def __init__(self, comm, max_tokens: int, hidden: int):
        self.comm, self.hidden = comm, int(hidden)
        n = comm.size
        self.shard = ((max_tokens + n - 1) // n + 127) // 128 * 128
        lib = _lib()
        for name in ("tsb_tpseq_struct_bytes", "tsb_tpseq_init", "tsb_tpseq_norm_gather", "tsb_tpseq_wait_all",
                     "tsb_gemm_bf16_tp", "tsb_tpseq_norm_ep", "tsb_tpseq_dispatch", "tsb_tpseq_push_rows_ep", "tsb_tpseq_route_kmax"):
            getattr(lib, name).restype = C.c_int
        lib.tsb_tpseq_region_bytes.restype = C.c_long
        lib.tsb_tpseq_route_offset.restype = C.c_long
        self.region = SymmetricBuffer(comm, lib.tsb_tpseq_region_bytes(C.c_int(n), C.c_int(self.shard), C.c_long(self.hidden)))
        dev = comm.device
        self.local = torch.zeros(16, dtype=torch.int32, device=dev)
        self.struct = torch.zeros(lib.tsb_tpseq_struct_bytes(), dtype=torch.uint8, device=dev)
        arr = C.c_void_p * n
        native.check(lib.tsb_tpseq_init(C.c_void_p(self.struct.data_ptr()), arr(*self.region.ptrs),
                                        C.c_void_p(self.local.data_ptr()), C.c_int(comm.rank), C.c_int(n),
                                        C.c_int(self.shard), C.c_long(self.hidden)), "tpseq_init")
        xoff = 256 + 2 * n * self.shard * self.hidden * 2
        self.xfull = tensor_from_ptr(self.region.local + xoff, (n * self.shard, self.hidden), torch.bfloat16, dev)
        # routing records of the expert dispatch: ids and weights of every token, row stride = the model's top-k
        self.route_kmax = int(lib.tsb_tpseq_route_kmax())
        roff = int(lib.tsb_tpseq_route_offset(C.c_int(n), C.c_int(self.shard), C.c_long(self.hidden)))
        cells = n * self.shard * self.route_kmax
        self._route_ids = tensor_from_ptr(self.region.local + roff, (cells,), torch.int32, dev)
        self._route_w = tensor_from_ptr(self.region.local + roff + cells * 4, (cells,), torch.float32, dev)
        self._route_ids.fill_(-1)
        self._route_w.zero_()
        torch.cuda.synchronize(dev)
        comm.barrier()

    @property
    def rows(self) -> slice:
        """This rank's rows of the token dimension."""
        return slice(self.comm.rank * self.shard, (self.comm.rank + 1) * self.shard)

    def _gemm(self, W: torch.Tensor, X: torch.Tensor, out, bias, T: int, rs: bool, ag: bool):
        from ..ops import kernels as k
        lib = k._lib()
        N, K = W.shape
        sp = C.c_void_p(self.struct.data_ptr())
        native.check(lib.tsb_gemm_bf16_tp(k._p(W), C.c_long(W.stride(0)), k._p(X), C.c_long(X.stride(0)), k._p(out),
                                          C.c_long(out.stride(0) if out is not None else 0),
                                          C.c_int(1 if (out is None or out.dtype == torch.float32) else 0), k._p(bias), None,
                                          C.c_int(T), C.c_int(N), C.c_int(K), sp if rs else None, sp if ag else None,
                                          C.c_int(self.shard), C.c_int(self.comm.size), C.c_int(self.comm.rank),
                                          k._p(k.gemm_status(X.device)),
                                          k._stream()), "gemm_bf16_tp")
        k._count(1)

    def gemm_rs(self, x: torch.Tensor, w: QuantWeight, bias: Optional[torch.Tensor] = None) -> None:
        """Partial ``x @ w^T`` of this rank, reduced into the token owners' accumulators."""
        from ..ops import functional as F
        if x.dtype != torch.bfloat16:
            x = x.to(torch.bfloat16)
        assert x.shape[0] <= self.comm.size * self.shard and w.N == self.hidden
        self._gemm(F._dequant_scratch(w), x.contiguous(), None, bias, x.shape[0], True, False)

    def norm_gather(self, h_shard: torch.Tensor, w: Optional[torch.Tensor], eps: float, has_acc: bool, *,
                    local_only: bool = False, acc_k: int = 0, experts_per_rank: int = 0) -> None:
        """``local_only``: keep the normalised rows here (``dispatch`` sends them on); ``acc_k``: the accumulators hold
        an expert combine, add only the slots of the ranks that own one of the row's ``acc_k`` chosen experts."""
        from ..ops import kernels as k
        assert h_shard.dtype == torch.float32 and h_shard.shape == (self.shard, self.hidden) and h_shard.is_contiguous()
        if local_only or acc_k:
            native.check(k._lib().tsb_tpseq_norm_ep(C.c_void_p(self.struct.data_ptr()), k._p(h_shard), k._p(w), C.c_float(eps),
                                                    C.c_int(self.shard), C.c_int(self.hidden), C.c_int(1 if has_acc else 0),
                                                    C.c_int(1 if local_only else 0), C.c_int(acc_k), C.c_int(experts_per_rank),
                                                    k._stream()), "tpseq_norm_ep")
        else:
            native.check(k._lib().tsb_tpseq_norm_gather(C.c_void_p(self.struct.data_ptr()), k._p(h_shard), k._p(w), C.c_float(eps),
                                                        C.c_int(self.shard), C.c_int(self.hidden), C.c_int(1 if has_acc else 0),
                                                        k._stream()), "tpseq_norm_gather")
        k._count(1)

    def dispatch(self, ids: torch.Tensor, weights: torch.Tensor, T: int, experts_per_rank: int) -> None:
        """Expert dispatch of this rank's shard: ``ids`` / ``weights`` ``[shard, k]`` are the router's choices for its
        (locally normalised) rows; each row goes to the ranks that own one of its experts, the routing records to all."""
        from ..ops import kernels as k
        kk = ids.shape[1]
        assert ids.shape == (self.shard, kk) == tuple(weights.shape) and kk <= self.route_kmax
        ids = ids.to(torch.int32).contiguous()
        weights = weights.float().contiguous()
        native.check(k._lib().tsb_tpseq_dispatch(C.c_void_p(self.struct.data_ptr()), k._p(ids), k._p(weights), C.c_int(kk),
                                                 C.c_int(experts_per_rank), C.c_int(T), C.c_int(self.shard), k._stream()),
                     "tpseq_dispatch")
        k._count(1)

    def routes(self, T: int, kk: int):
        """The routing records of the first ``T`` tokens as ``(ids [T, k] int32, weights [T, k] f32)`` views."""
        return self._route_ids[:T * kk].view(T, kk), self._route_w[:T * kk].view(T, kk)

    def gemm_ag(self, w: QuantWeight, T: int, bias: Optional[torch.Tensor] = None, out_dtype=torch.bfloat16) -> torch.Tensor:
        """``gathered[:T] @ w^T`` (+ bias); tiles start as soon as their shard has arrived."""
        from ..ops import functional as F
        out = torch.empty((T, w.N), dtype=out_dtype, device=self.xfull.device)
        self._gemm(F._dequant_scratch(w), self.xfull, out, bias, T, False, True)
        return out

    def push_rows(self, partial: torch.Tensor, T: int, *, k_routed: int = 0, e0: int = 0, e1: int = 0) -> None:
        """Reduce-scatter a partial ``[T, hidden]`` f32 sum that no GEMM epilogue produced (the summed
        outputs of this rank's experts): same destination and counters as ``gemm_rs``.  ``k_routed``: after a
        ``dispatch`` with that top-k, only the rows of tokens that chose one of the experts ``[e0, e1)`` are sent."""
        from ..ops import kernels as k
        assert partial.dtype == torch.float32 and partial.is_contiguous() and partial.shape[1] == self.hidden
        if k_routed:
            native.check(k._lib().tsb_tpseq_push_rows_ep(C.c_void_p(self.struct.data_ptr()), k._p(partial), C.c_int(T),
                                                         C.c_int(self.shard), C.c_int(self.comm.size), C.c_int(self.hidden),
                                                         C.c_int(k_routed), C.c_int(e0), C.c_int(e1), k._stream()),
                         "tpseq_push_rows_ep")
        else:
            native.check(k._lib().tsb_tpseq_push_rows(C.c_void_p(self.struct.data_ptr()), k._p(partial), C.c_int(T),
                                                      C.c_int(self.shard), C.c_int(self.comm.size), C.c_int(self.hidden),
                                                      k._stream()), "tpseq_push_rows")
        k._count(1)

    def wait_all(self) -> None:
        from ..ops import kernels as k
        native.check(k._lib().tsb_tpseq_wait_all(C.c_void_p(self.struct.data_ptr()), k._stream()), "tpseq_wait_all")
        k._count(1)

    def status(self) -> int:
        torch.cuda.synchronize(self.comm.device)
        return int(self.local[8].item())

    def check(self) -> None:
        from .errors import ExchangeTimeoutError
        code = self.status()
        if code:
            raise ExchangeTimeoutError("sequence-parallel prefill exchange", code)

    def close(self) -> None:
        torch.cuda.synchronize(self.comm.device)
        self.region.close()
