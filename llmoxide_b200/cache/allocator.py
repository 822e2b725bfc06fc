"""Host-side bookkeeping of the cache: which slot belongs to which live
sequence, which pages each slot holds in each group of layers, and each
sequence's own length.  No tensors here, so it is tested without a GPU.  The
bookkeeping itself is C++ (``csrc/host_runtime.cpp``, built with the C++
compiler alone); this class holds the handle and raises the typed errors.

A *slot* is one live sequence's entry.  A *page* holds ``PAGE`` consecutive
positions of one sequence for every layer of one *group* (layers with the same
needs: head count, head size, all keys or a window of them).  Position ``p``
of a sequence lives in its logical page ``p // PAGE``; the slot's page list
maps logical to physical pages.  A group with a window gives pages back as
soon as no later query can see them (the reference keeps a ring of exactly the
window for such layers, crates/model/src/cache.rs:10-37; pages reach the same
bound up to one page of slack, and let a whole prompt be written before it is
attended to).  Lengths only grow: there is no rewind
(crates/model/src/qwen35/cpu.rs:119-125,404).
"""

from __future__ import annotations

import ctypes
from ctypes import c_char_p, c_int, c_longlong, c_void_p
from typing import Optional

from ..errors import CacheExhausted, CacheMisuse, ContextOverflow

PAGE = 64

# codes of csrc/host_runtime.cpp
_MISUSE, _OVERFLOW_SEQ, _EXHAUSTED, _BAD_VALUE, _OVERFLOW_STEP, _TOO_SMALL = 1, 2, 3, 4, 5, 6
_lib = None


def pages_for(n_tokens: int) -> int:
    return (n_tokens + PAGE - 1) // PAGE


def host_library():
    """The host runtime, built on first use."""
    global _lib
    if _lib is None:
        from ..csrc.build import load_library

        lib = load_library("host_runtime")
        P = ctypes.POINTER
        lib.llmx_alloc_new.restype = c_void_p
        lib.llmx_alloc_new.argtypes = [c_int, c_int, P(c_int), c_int, c_longlong]
        lib.llmx_alloc_delete.argtypes = [c_void_p]
        lib.llmx_alloc_delete.restype = None
        for name in ("acquire", "check", "n_free_slots"):
            getattr(lib, f"llmx_alloc_{name}").argtypes = [c_void_p]
        for name in ("release", "unreserve", "n_free_pages"):
            getattr(lib, f"llmx_alloc_{name}").argtypes = [c_void_p, c_int]
        for name in ("reserve", "commit"):
            getattr(lib, f"llmx_alloc_{name}").argtypes = [c_void_p, c_int, c_longlong]
        lib.llmx_alloc_commit_many.argtypes = [c_void_p, c_int, c_void_p, c_void_p]
        lib.llmx_alloc_length.argtypes = [c_void_p, c_int]
        lib.llmx_alloc_length.restype = c_longlong
        lib.llmx_alloc_generation.argtypes = [c_void_p, c_int]
        lib.llmx_alloc_generation.restype = c_longlong
        lib.llmx_alloc_page_row.argtypes = [c_void_p, c_int, c_int, c_void_p, c_int]
        lib.llmx_host_error.argtypes = [c_char_p, c_int, P(c_longlong)]
        lib.llmx_pack_step.argtypes = [c_int] + [c_void_p] * 6 + [c_int] + [c_void_p] * 4 + [c_longlong, c_void_p]
        lib.llmx_plan_step.argtypes = [c_void_p, c_int] + [c_void_p] * 5 + [c_int, c_longlong, c_int, c_void_p,
                                                                              c_longlong, c_void_p]
        _lib = lib
    return _lib


def raise_host_error(code: int) -> None:
    """The typed error for a non-zero code of the host runtime, with its message."""
    lib = host_library()
    buf = ctypes.create_string_buffer(600)
    info = (c_longlong * 2)()
    lib.llmx_host_error(buf, 600, info)
    msg = buf.value.decode()
    if code == _MISUSE:
        raise CacheMisuse(msg)
    if code == _OVERFLOW_SEQ:
        raise ContextOverflow(int(info[0]), int(info[1]), "longest sequence the cache allows")
    if code == _EXHAUSTED:
        raise CacheExhausted(msg)
    if code == _OVERFLOW_STEP:
        raise ContextOverflow(int(info[0]), int(info[1]), "step limit (max_step_tokens)")
    raise ValueError(msg)


class CacheAllocator:
    """Slots, pages and lengths.  ``windows[g]`` is group g's window or None."""

    def __init__(self, n_slots: int, n_pages: int, windows: list, max_seq_len: Optional[int] = None):
        if n_slots <= 0 or n_pages <= 0:
            raise ValueError("the cache needs at least one slot and one page")
        self.n_slots, self.n_pages = n_slots, n_pages
        self.windows = list(windows)
        self.max_seq_len = max_seq_len if max_seq_len is not None else n_pages * PAGE
        self._lib = host_library()
        w = (c_int * len(self.windows))(*[int(x) if x else 0 for x in self.windows])
        self._h = self._lib.llmx_alloc_new(n_slots, n_pages, w, len(self.windows), self.max_seq_len)
        if not self._h:
            raise ValueError("the cache needs at least one slot, one page and one group")
        self._row = (c_int * max(1, n_pages))()

    def __del__(self):
        h, self._h = getattr(self, "_h", None), None
        if h and self._lib is not None:
            self._lib.llmx_alloc_delete(h)

    @property
    def handle(self):
        return self._h

    def _ok(self, code: int) -> None:
        if code:
            raise_host_error(code)

    # ---- slots -----------------------------------------------------------

    @property
    def n_free_slots(self) -> int:
        return self._lib.llmx_alloc_n_free_slots(self._h)

    def acquire(self) -> int:
        s = self._lib.llmx_alloc_acquire(self._h)
        if s < 0:
            raise_host_error(-s)
        return s

    def release(self, slot: int) -> None:
        self._ok(self._lib.llmx_alloc_release(self._h, slot))

    def length(self, slot: int) -> int:
        n = self._lib.llmx_alloc_length(self._h, slot)
        if n < 0:
            raise_host_error(_MISUSE)
        return int(n)

    def generation(self, slot: int) -> int:
        """How many owners the slot has had."""
        return int(self._lib.llmx_alloc_generation(self._h, slot))

    # ---- a step: reserve pages, then commit the new length ---------------

    def reserve(self, slot: int, n_new: int) -> None:
        """Makes sure positions length .. length+n_new-1 have pages in every
        group.  Raises before anything is changed if they do not fit."""
        self._ok(self._lib.llmx_alloc_reserve(self._h, slot, n_new))

    def unreserve(self, slot: int) -> None:
        """Takes back a reservation that no step will use: pages beyond those the slot's length needs return
        to their pools (a step that was refused for another sequence of its batch does this for the
        sequences it had already reserved for)."""
        self._ok(self._lib.llmx_alloc_unreserve(self._h, slot))

    def commit(self, slot: int, n_new: int) -> None:
        """The step wrote n_new positions: the length grows, and groups with a
        window give back the pages no later query can see."""
        self._ok(self._lib.llmx_alloc_commit(self._h, slot, n_new))

    def commit_many(self, slots, counts) -> None:
        n = len(slots)
        self._ok(self._lib.llmx_alloc_commit_many(self._h, n, (c_int * n)(*slots), (c_int * n)(*counts)))

    def page_row(self, slot: int, group: int) -> list:
        """Logical page -> physical page (-1 where a page was given back)."""
        n = self._lib.llmx_alloc_page_row(self._h, slot, group, self._row, len(self._row))
        if n < 0:
            raise_host_error(_MISUSE)
        return list(self._row[:n])

    def pages_held(self, group: int = 0) -> int:
        return self.n_pages - self._lib.llmx_alloc_n_free_pages(self._h, group)

    def check_consistent(self) -> None:
        """No page held twice or lost; used by tests."""
        self._ok(self._lib.llmx_alloc_check(self._h))
