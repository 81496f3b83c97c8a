"""Typed failures of the multi-GPU paths.  Device-side waits never trap: they write a status word
that the host turns into one of these after the step (csrc/tp_fused.cuh)."""


class ParallelError(RuntimeError):
    pass


class ExchangeTimeoutError(ParallelError):
    """A bounded wait inside an exchange kernel ran out.  ``code`` is the kernel's status word:
    1 + r: mailbox data of rank r missing; 10: reduce-scatter arrivals; 20 + r: gathered rows of rank r;
    30: staging half still being read; 40 + r: shard of rank r not published."""

    def __init__(self, where: str, code: int):
        super().__init__(f"{where}: a bounded device-side wait ran out (status {code}); the peer is late or gone")
        self.where, self.code = where, code


class RankFailureError(ParallelError):
    """One or more ranks stopped reporting heartbeats."""

    def __init__(self, stale):
        super().__init__(f"ranks {sorted(stale)} stopped responding")
        self.stale = sorted(stale)
