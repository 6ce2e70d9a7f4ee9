"""Python face of the C++ scheduler (csrc/host/scheduler.cpp).

The scheduler knows requests as lengths only: how many tokens are known and how
many are in the cache.  ``next()`` returns this step's entries, with pages
already reserved; the caller runs them, calls ``step_done()``, and for every
entry whose logits were wanted either ``append_token`` or ``finish``.
"""
from __future__ import annotations

from ctypes import c_int, c_longlong
from dataclasses import dataclass

from ..cache.page_table import PageTable, _lib


class SchedulerError(RuntimeError):
    pass


class RequestRejected(SchedulerError):
    """The request can never run: empty prompt, too long for the context or for the cache."""


@dataclass(frozen=True)
class ScheduledEntry:
    req: int
    start: int
    count: int
    wants_logits: bool


_REJECT = {-10: "empty prompt", -11: "prompt plus max_tokens exceeds the context limit",
           -12: "the request needs more cache pages than exist", -13: "request id already in use"}


class Scheduler:
    def __init__(self, table: PageTable, *, max_seqs: int, max_batch_tokens: int, prefill_chunk: int,
                 max_context: int = 0):
        self._lib = _lib()
        self._table = table  # keeps the C++ cache manager alive
        self.capacity = max_seqs
        self._h = self._lib.rmx_sched_create(table._h, max_seqs, max_batch_tokens, prefill_chunk, max_context)
        if not self._h:
            raise SchedulerError("max_seqs, max_batch_tokens and prefill_chunk must be positive")
        self._ids = (c_longlong * max_seqs)()
        self._start = (c_int * max_seqs)()
        self._count = (c_int * max_seqs)()
        self._wants = (c_int * max_seqs)()

    def __del__(self):
        h, self._h = getattr(self, "_h", None), None
        if h:
            self._lib.rmx_sched_destroy(h)

    def add(self, req: int, prompt_len: int, max_new_tokens: int) -> None:
        code = self._lib.rmx_sched_add(self._h, req, prompt_len, max_new_tokens)
        if code != 0:
            raise RequestRejected(f"request {req}: {_REJECT.get(code, code)}")

    def next(self) -> list:
        n = self._lib.rmx_sched_next(self._h, self._ids, self._start, self._count, self._wants, self.capacity)
        if n < 0:
            raise SchedulerError("more entries than max_seqs")
        return [ScheduledEntry(self._ids[i], self._start[i], self._count[i], bool(self._wants[i])) for i in range(n)]

    def step_done(self) -> None:
        if self._lib.rmx_sched_step_done(self._h) != 0:
            raise SchedulerError("step_done without a step in flight")

    def append_token(self, req: int) -> None:
        if self._lib.rmx_sched_append_token(self._h, req) != 0:
            raise SchedulerError(f"request {req} cannot take a token now")

    def finish(self, req: int) -> None:
        if self._lib.rmx_sched_finish(self._h, req) != 0:
            raise SchedulerError(f"request {req} is unknown")

    def take_preempted(self) -> list:
        buf = (c_longlong * self.capacity)()
        n = self._lib.rmx_sched_take_preempted(self._h, buf, self.capacity)
        return list(buf[:n])

    @property
    def waiting(self) -> int:
        return self._lib.rmx_sched_waiting(self._h)

    @property
    def running(self) -> int:
        return self._lib.rmx_sched_running(self._h)

    def idle(self) -> bool:
        return self.waiting == 0 and self.running == 0

    def computed(self, req: int) -> int:
        return self._lib.rmx_sched_computed(self._h, req)

    def total(self, req: int) -> int:
        return self._lib.rmx_sched_total(self._h, req)
