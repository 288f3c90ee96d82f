"""The cache manager seen from Python: a thin handle on the native one (csrc/host/cache_manager.h).

It hands out indices only. `KVArena` (cache/arena.py) owns the memory that the indices point
into, and the step function ships block tables and slot mappings to the GPU every step.
"""

from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

import numpy as np

from . import _host

CACHE_OK, CACHE_NO_PAGES, CACHE_BAD_REQUEST, CACHE_TOO_LONG, CACHE_BAD_ARG = 0, -1, -2, -3, -4
_STATUS = {
    CACHE_NO_PAGES: "not enough free pages",
    CACHE_BAD_REQUEST: "bad request slot (out of range, not open, or already open)",
    CACHE_TOO_LONG: "beyond max_seq_len",
    CACHE_BAD_ARG: "bad argument",
}


class CacheError(RuntimeError):
    def __init__(self, status: int, what: str):
        super().__init__(f"{what}: {_STATUS.get(status, f'status {status}')}")
        self.status = status


class OutOfPages(CacheError):
    pass


@dataclass(frozen=True)
class GroupSpec:
    """One cache group: layers whose pages live and die together."""

    page_size: int
    window: int = 0  # 0 = every position is kept; w > 0 = a query at p reads keys (p - w, p]
    num_pages: int = 1  # pages that can be handed out; page id 0 (the null page) is extra


def _ptr(a: np.ndarray):
    assert a.dtype == np.int32 and a.flags["C_CONTIGUOUS"], (a.dtype, a.flags)
    return a.ctypes.data_as(_host.I32P)


def group_array(groups: list[GroupSpec]):
    arr = (_host.GroupSpecC * len(groups))()
    for i, g in enumerate(groups):
        arr[i] = _host.GroupSpecC(g.page_size, g.window, g.num_pages)
    return arr


class CacheManager:
    def __init__(self, groups: list[GroupSpec], max_requests: int, max_seq_len: int, _borrowed=None):
        self._lib = _host.lib()
        self.groups = list(groups)
        self.max_requests = max_requests
        self.max_seq_len = max_seq_len
        self._owner = _borrowed  # a scheduler that owns the native object, or None
        if _borrowed is None:
            handle = self._lib.r2_cache_create(group_array(self.groups), len(self.groups), max_requests, max_seq_len)
            if not handle:
                raise ValueError(f"cache manager: {_host.last_error()}")
            self._h = C.c_void_p(handle)
        else:
            self._h = C.c_void_p(_borrowed._cache_handle())
        self.table_widths = [self._lib.r2_cache_table_width(self._h, g) for g in range(len(self.groups))]

    def __del__(self):
        if getattr(self, "_owner", None) is None and getattr(self, "_h", None):
            self._lib.r2_cache_destroy(self._h)
            self._h = None

    # ---- requests --------------------------------------------------------------------------
    def open(self, req: int) -> None:
        self._check(self._lib.r2_cache_open(self._h, req), f"open request {req}")

    def close(self, req: int) -> None:
        self._check(self._lib.r2_cache_close(self._h, req), f"close request {req}")

    def is_open(self, req: int) -> bool:
        return bool(self._lib.r2_cache_is_open(self._h, req))

    def reserve(self, req: int, n_computed: int, n_total: int) -> None:
        """Pages for positions up to n_total (exclusive) in every group, or none at all."""
        self._check(self._lib.r2_cache_reserve(self._h, req, n_computed, n_total),
                    f"reserve positions [{n_computed}, {n_total}) for request {req}")

    def can_reserve(self, req: int, n_computed: int, n_total: int, spare_pages: int = 0) -> bool:
        return bool(self._lib.r2_cache_can_reserve(self._h, req, n_computed, n_total, spare_pages))

    def slide(self, req: int, n_computed: int) -> None:
        """Window groups give back the pages that the window has passed."""
        self._check(self._lib.r2_cache_slide(self._h, req, n_computed), f"slide request {req}")

    # ---- queries ---------------------------------------------------------------------------
    def n_free(self, group: int = 0) -> int:
        return self._lib.r2_cache_n_free(self._h, group)

    def pages_held(self, req: int, group: int = 0) -> int:
        return self._lib.r2_cache_pages_held(self._h, req, group)

    def worst_pages(self, group: int, n_total: int, max_chunk: int, grain: int = 1) -> int:
        return self._lib.r2_cache_worst_pages(self._h, group, n_total, max_chunk, grain)

    def table(self, req: int, group: int = 0) -> np.ndarray:
        out = np.zeros(self.table_widths[group], dtype=np.int32)
        n = self._lib.r2_cache_table(self._h, req, group, _ptr(out), len(out))
        self._check(min(n, 0), f"table of request {req}")
        return out

    def check(self) -> str:
        """'' when every page is either free or in exactly one table."""
        buf = C.create_string_buffer(4096)
        self._lib.r2_cache_check(self._h, buf, len(buf))
        return buf.value.decode()

    # ---- batches ---------------------------------------------------------------------------
    def fill(self, batch) -> None:
        """Positions, slots and block tables of a StepBatch whose entries are set."""
        ptrs = getattr(batch, "_fill_ptrs", None)
        if ptrs is None:  # the arrays of a batch never move: their pointers are made once
            ptrs = batch._fill_ptrs = tuple(_ptr(a) for a in (
                batch.entry_req, batch.entry_start, batch.entry_rows, batch.positions, batch.row_entry, batch.q_start,
                batch.seq_lens, batch.state_slot, batch.fresh, batch.slot_mapping_flat, batch.block_tables_flat))
        status = self._lib.r2_cache_fill_batch(self._h, batch.n_entries, ptrs[0], ptrs[1], ptrs[2], batch.t_cap, batch.r_cap,
                                               *ptrs[3:])
        self._check(status, "fill batch")

    def _check(self, status: int, what: str) -> None:
        if status >= 0:
            return
        if status == CACHE_NO_PAGES:
            raise OutOfPages(status, what)
        raise CacheError(status, what)
