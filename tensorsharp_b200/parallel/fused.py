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
                    want_bf16: bool = True, norm: bool = True) -> Optional[Act]:
        """``h += sum of all ranks' partials`` (in place, f32), then ``RMSNorm(h) * w`` as the next
        projection's input.  With ``norm=False`` only the residual stream is updated."""
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
                                            C.c_float(eps), C.c_int(T), C.c_int(D), k._p(yb), k._p(yq), k._p(yds),
                                            k._stream()), "tp_reduce_norm")
        k._count(1)
        self.exchanges += 1
        return Act(yb, yq, yds) if norm else None

    # ------------------------------------------------------------------ health
    def status(self) -> int:
        """0 when every wait so far was satisfied, else 1 + the rank whose flag did not arrive
        within the kernel's time limit (synchronises the device)."""
        torch.cuda.synchronize(self.comm.device)
        return int(self.counters[4].item())

    def close(self) -> None:
        torch.cuda.synchronize(self.comm.device)
        self.mail.close()
