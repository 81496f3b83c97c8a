"""Symmetric device memory: one buffer per rank, every rank's buffer mapped into every process.

Each rank allocates plain device memory in the native library, exports it as a CUDA IPC handle,
the 64-byte handles are exchanged through the process group (host side, once), and every rank
opens its peers' handles.  Kernels of this library then load and store peer memory directly
over NVLink; no library kernel is ever given a peer pointer.  The reference has nothing like
this (single device: TensorSharp.Models/ModelBase.cs:236-264).
"""
from __future__ import annotations

import ctypes as C
from typing import List

import torch

from ..ops import native


GUARD = 256                  # bytes of guard band on either side of a symmetric buffer
CANARY = 0x5A5AC3C3


def _lib():
    lib = native.lib()
    for name in ("tsb_symm_alloc", "tsb_symm_free", "tsb_ipc_get_handle", "tsb_ipc_open", "tsb_ipc_close",
                 "tsb_ipc_handle_bytes", "tsb_tp_struct_bytes", "tsb_tp_init", "tsb_tp_status"):
        getattr(lib, name).restype = C.c_int
    lib.tsb_tp_mailbox_bytes.restype = C.c_long
    return lib


class SymmetricBuffer:
    """``nbytes`` of zeroed device memory on every rank; ``ptrs[r]`` is rank r's buffer as an
    address valid in this process (``ptrs[rank]`` is the local allocation)."""

    def __init__(self, comm, nbytes: int):
        import torch.distributed as dist
        self.comm, self.nbytes = comm, int(nbytes)
        lib = _lib()
        base = C.c_void_p()
        # a guard band on either side holds a known pattern; check_canaries() tells whether a kernel of
        # this rank or a peer wrote outside the buffer
        native.check(lib.tsb_symm_alloc(C.c_size_t(self.nbytes + 2 * GUARD), C.byref(base)), "symm_alloc")
        self._base = base.value
        self.local = self._base + GUARD
        self._guards = None
        try:
            from .fused import tensor_from_ptr
            dev = comm.device
            self._guards = (tensor_from_ptr(self._base, (GUARD // 4,), torch.int32, dev),
                            tensor_from_ptr(self.local + self.nbytes, (GUARD // 4,), torch.int32, dev))
            for gd in self._guards:
                gd.fill_(CANARY)
            torch.cuda.synchronize(dev)
        except Exception:
            self._guards = None
        hb = lib.tsb_ipc_handle_bytes()
        handle = (C.c_ubyte * hb)()
        native.check(lib.tsb_ipc_get_handle(C.c_void_p(self._base), handle), "ipc_get_handle")
        mine = bytes(handle)
        if comm.size > 1:
            handles: List[bytes] = [b""] * comm.size
            dist.all_gather_object(handles, mine, group=comm.group)
        else:
            handles = [mine]
        self.ptrs: List[int] = []
        self._opened: List[int] = []
        for r, h in enumerate(handles):
            if r == comm.rank:
                self.ptrs.append(self.local)
                continue
            p = C.c_void_p()
            buf = (C.c_ubyte * hb).from_buffer_copy(h)
            native.check(lib.tsb_ipc_open(buf, C.byref(p)), f"ipc_open(rank {r})")
            self.ptrs.append(p.value + GUARD)
            self._opened.append(p.value)
        comm.barrier()

    def check_canaries(self) -> bool:
        """True while both guard bands of the local buffer still hold their pattern."""
        if self._guards is None:
            return True
        torch.cuda.synchronize(self.comm.device)
        return all(bool((gd == CANARY).all()) for gd in self._guards)

    def close(self) -> None:
        lib = _lib()
        for p in self._opened:
            lib.tsb_ipc_close(C.c_void_p(p))
        self._opened = []
        self.comm.barrier()              # nobody still maps the memory that is about to be freed
        if self.local:
            self._guards = None
            lib.tsb_symm_free(C.c_void_p(self._base))
            self.local = self._base = 0
