"""Python face of the C++ cache manager (csrc/host/cache_manager.cpp).

The manager keeps the books: for every live request its state slot, its length,
and per cache group its block table (logical page -> page id, -1 where a window
has passed).  It owns no tensors.
"""
from __future__ import annotations

import ctypes
from ctypes import c_int, c_longlong, c_void_p
from dataclasses import dataclass

from ..kernels.library import host_library


class CacheError(RuntimeError):
    pass


class OutOfPages(CacheError):
    """A request needs more pages than its group's pool has free."""


class OutOfSlots(CacheError):
    """More live requests than state slots."""


@dataclass(frozen=True)
class GroupGeometry:
    num_pages: int
    page_size: int
    window: int = 0


_ERRORS = {-1: "no pages", -2: "no state slot", -3: "unknown request", -4: "bad length", -5: "request already open",
           -6: "bad argument", -7: "invariant broken"}


def _lib():
    lib = host_library()
    if not getattr(lib, "_rmx_typed", False):
        lib.rmx_cm_create.restype = c_void_p
        lib.rmx_cm_create.argtypes = [c_int, c_void_p, c_void_p, c_void_p, c_int]
        lib.rmx_cm_destroy.argtypes = [c_void_p]
        for name in ("open", "close", "length", "reserved", "slot", "has", "release_reserved"):
            getattr(lib, f"rmx_cm_{name}").argtypes = [c_void_p, c_longlong]
        for name in ("reserve", "max_reservable", "commit", "pages_held"):
            getattr(lib, f"rmx_cm_{name}").argtypes = [c_void_p, c_longlong, c_int]
        lib.rmx_cm_table.argtypes = [c_void_p, c_longlong, c_int, c_void_p, c_int]
        lib.rmx_cm_peak_pages.argtypes = [c_void_p, c_int, c_int, c_int]
        lib.rmx_cm_free_pages.argtypes = [c_void_p, c_int]
        for name in ("free_slots", "live", "check"):
            getattr(lib, f"rmx_cm_{name}").argtypes = [c_void_p]
        lib.rmx_sched_create.restype = c_void_p
        lib.rmx_sched_create.argtypes = [c_void_p, c_int, c_int, c_int, c_int]
        lib.rmx_sched_destroy.argtypes = [c_void_p]
        lib.rmx_sched_add.argtypes = [c_void_p, c_longlong, c_int, c_int]
        lib.rmx_sched_next.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int]
        for name in ("step_done", "waiting", "running"):
            getattr(lib, f"rmx_sched_{name}").argtypes = [c_void_p]
        for name in ("append_token", "finish", "computed", "total"):
            getattr(lib, f"rmx_sched_{name}").argtypes = [c_void_p, c_longlong]
        lib.rmx_sched_take_preempted.argtypes = [c_void_p, c_void_p, c_int]
        lib._rmx_typed = True
    return lib


class PageTable:
    """Pages and state slots of the live requests."""

    def __init__(self, groups: list, max_requests: int):
        self.groups = [g if isinstance(g, GroupGeometry) else GroupGeometry(*g) for g in groups]
        self.max_requests = int(max_requests)
        self._lib = _lib()
        n = len(self.groups)
        arr = c_int * max(n, 1)
        self._h = self._lib.rmx_cm_create(
            n, arr(*[g.num_pages for g in self.groups]), arr(*[g.page_size for g in self.groups]),
            arr(*[g.window for g in self.groups]), self.max_requests)
        if not self._h:
            raise CacheError("bad cache geometry: pages >= 0, page size > 0, window >= 0, requests > 0")
        self._max_entries = [0] * n

    def __del__(self):
        h, self._h = getattr(self, "_h", None), None
        if h:
            self._lib.rmx_cm_destroy(h)

    def _fail(self, code, what, req):
        msg = f"{what} of request {req!r}: {_ERRORS.get(code, code)}"
        if code == -1:
            raise OutOfPages(msg)
        if code == -2:
            raise OutOfSlots(msg)
        raise CacheError(msg)

    def open(self, req: int) -> int:
        slot = self._lib.rmx_cm_open(self._h, req)
        if slot < 0:
            self._fail(slot, "open", req)
        return slot

    def has(self, req: int) -> bool:
        return bool(self._lib.rmx_cm_has(self._h, req))

    def reserve(self, req: int, new_len: int) -> None:
        code = self._lib.rmx_cm_reserve(self._h, req, new_len)
        if code < 0:
            self._fail(code, f"reserve({new_len})", req)

    def try_reserve(self, req: int, new_len: int) -> bool:
        code = self._lib.rmx_cm_reserve(self._h, req, new_len)
        if code == -1:
            return False
        if code < 0:
            self._fail(code, f"reserve({new_len})", req)
        return True

    def max_reservable(self, req: int, want: int) -> int:
        return self._lib.rmx_cm_max_reservable(self._h, req, want)

    def commit(self, req: int, new_len: int) -> int:
        freed = self._lib.rmx_cm_commit(self._h, req, new_len)
        if freed < 0:
            self._fail(freed, f"commit({new_len})", req)
        return freed

    def close(self, req: int) -> int:
        freed = self._lib.rmx_cm_close(self._h, req)
        if freed < 0:
            self._fail(freed, "close", req)
        return freed

    def release_reserved(self, req: int) -> int:
        return self._lib.rmx_cm_release_reserved(self._h, req)

    def length(self, req: int) -> int:
        n = self._lib.rmx_cm_length(self._h, req)
        if n < 0:
            self._fail(n, "length", req)
        return n

    def reserved(self, req: int) -> int:
        return self._lib.rmx_cm_reserved(self._h, req)

    def slot(self, req: int) -> int:
        s = self._lib.rmx_cm_slot(self._h, req)
        if s < 0:
            self._fail(s, "slot", req)
        return s

    def table(self, req: int, group: int) -> list:
        cap = max(16, -(-self.reserved(req) // self.groups[group].page_size))
        buf = (c_int * cap)()
        n = self._lib.rmx_cm_table(self._h, req, group, buf, cap)
        if n < 0:
            self._fail(n, "table", req)
        return list(buf[:n])

    def table_into(self, req: int, group: int, out_ptr: int, capacity: int) -> int:
        """Write the table straight into int32 memory at ``out_ptr``; returns the entry count."""
        n = self._lib.rmx_cm_table(self._h, req, group, c_void_p(out_ptr), capacity)
        if n < 0:
            self._fail(n, "table", req)
        return n

    def pages_held(self, req: int, group: int) -> int:
        return self._lib.rmx_cm_pages_held(self._h, req, group)

    def peak_pages(self, group: int, length: int, portion: int) -> int:
        return self._lib.rmx_cm_peak_pages(self._h, group, length, portion)

    def free_pages(self, group: int) -> int:
        return self._lib.rmx_cm_free_pages(self._h, group)

    def free_slots(self) -> int:
        return self._lib.rmx_cm_free_slots(self._h)

    def live(self) -> int:
        return self._lib.rmx_cm_live(self._h)

    def check(self) -> None:
        if self._lib.rmx_cm_check(self._h) != 0:
            raise CacheError("cache manager invariant broken: a page or slot is lost, held twice or freed twice")
