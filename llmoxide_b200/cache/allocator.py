"""Host-side bookkeeping of the cache: which slot belongs to which live
sequence, which pages each slot holds in each group of layers, and each
sequence's own length.  No tensors here, so it is tested without a GPU.

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

from dataclasses import dataclass, field
from typing import Optional

from ..errors import CacheExhausted, CacheMisuse, ContextOverflow

PAGE = 64


def pages_for(n_tokens: int) -> int:
    return (n_tokens + PAGE - 1) // PAGE


class PagePool:
    """Free list of physical pages of one group."""

    def __init__(self, n_pages: int):
        self.n_pages = n_pages
        self._free = list(range(n_pages - 1, -1, -1))  # pop() hands out low ids first
        self._held = [False] * n_pages

    @property
    def n_free(self) -> int:
        return len(self._free)

    def take(self, n: int) -> list:
        if n > len(self._free):
            raise CacheExhausted(f"{n} more cache pages are needed, {len(self._free)} of {self.n_pages} are free")
        out = [self._free.pop() for _ in range(n)]
        for p in out:
            self._held[p] = True
        return out

    def give_back(self, pages) -> None:
        for p in pages:
            if not (0 <= p < self.n_pages) or not self._held[p]:
                raise CacheMisuse(f"page {p} is given back but is not held")
            self._held[p] = False
            self._free.append(p)


@dataclass
class SlotState:
    length: int = 0                    # positions written so far
    reserved: int = 0                  # positions that have pages (>= length)
    pages: list = field(default_factory=list)   # per group: logical page -> physical page or -1
    live: bool = False
    generation: int = 0                # counts owners of this slot


class CacheAllocator:
    """Slots, pages and lengths.  ``windows[g]`` is group g's window or None."""

    def __init__(self, n_slots: int, n_pages: int, windows: list, max_seq_len: Optional[int] = None):
        if n_slots <= 0 or n_pages <= 0:
            raise ValueError("the cache needs at least one slot and one page")
        self.n_slots, self.n_pages = n_slots, n_pages
        self.windows = list(windows)
        self.max_seq_len = max_seq_len if max_seq_len is not None else n_pages * PAGE
        self.pools = [PagePool(n_pages) for _ in self.windows]
        self.slots = [SlotState() for _ in range(n_slots)]
        self._free_slots = list(range(n_slots - 1, -1, -1))

    # ---- slots -----------------------------------------------------------

    @property
    def n_free_slots(self) -> int:
        return len(self._free_slots)

    def acquire(self) -> int:
        if not self._free_slots:
            raise CacheExhausted(f"all {self.n_slots} cache slots are held by live sequences")
        s = self._free_slots.pop()
        st = self.slots[s]
        st.length = st.reserved = 0
        st.pages = [[] for _ in self.windows]
        st.live = True
        st.generation += 1
        return s

    def release(self, slot: int) -> None:
        st = self._live(slot)
        for pool, pages in zip(self.pools, st.pages):
            pool.give_back([p for p in pages if p >= 0])
        st.pages = [[] for _ in self.windows]
        st.length = st.reserved = 0
        st.live = False
        self._free_slots.append(slot)

    def _live(self, slot: int) -> SlotState:
        if not (0 <= slot < self.n_slots):
            raise CacheMisuse(f"slot {slot} does not exist (there are {self.n_slots})")
        st = self.slots[slot]
        if not st.live:
            raise CacheMisuse(f"slot {slot} is not held by a live sequence (freed twice, or used after being freed)")
        return st

    def length(self, slot: int) -> int:
        return self._live(slot).length

    # ---- a step: reserve pages, then commit the new length ---------------

    def reserve(self, slot: int, n_new: int) -> None:
        """Makes sure positions length .. length+n_new-1 have pages in every
        group.  Raises before anything is changed if they do not fit."""
        st = self._live(slot)
        new_len = st.length + n_new
        if new_len > self.max_seq_len:
            raise ContextOverflow(new_len, self.max_seq_len, "longest sequence the cache allows")
        want = pages_for(new_len)
        for pool, pages in zip(self.pools, st.pages):
            need = want - len(pages)
            if need > pool.n_free:
                raise CacheExhausted(
                    f"slot {slot} needs {need} more cache pages for {new_len} positions, "
                    f"{pool.n_free} of {pool.n_pages} are free")
        for pool, pages in zip(self.pools, st.pages):
            pages.extend(pool.take(want - len(pages)))
        st.reserved = max(st.reserved, new_len)

    def unreserve(self, slot: int) -> None:
        """Takes back a reservation that no step will use: pages beyond those the slot's length needs return
        to their pools (a step that was refused for another sequence of its batch calls this for the
        sequences it had already reserved for)."""
        st = self._live(slot)
        keep = pages_for(st.length)
        for pool, pages in zip(self.pools, st.pages):
            pool.give_back([p for p in pages[keep:] if p >= 0])
            del pages[keep:]
        st.reserved = st.length

    def commit(self, slot: int, n_new: int) -> None:
        """The step wrote n_new positions: the length grows, and groups with a
        window give back the pages no later query can see."""
        st = self._live(slot)
        if st.length + n_new > st.reserved:
            raise CacheMisuse(f"slot {slot}: {n_new} positions are committed but only "
                              f"{st.reserved - st.length} were reserved")
        st.length += n_new
        for pool, pages, window in zip(self.pools, st.pages, self.windows):
            if window is None:
                continue
            # The next query sits at position `length` and sees keys from
            # length - (window - 1) on; whole pages below that are dead.
            first_visible = max(0, st.length - (window - 1))
            dead = first_visible // PAGE
            gone = [p for p in pages[:dead] if p >= 0]
            if gone:
                pool.give_back(gone)
                for i in range(dead):
                    pages[i] = -1

    def page_row(self, slot: int, group: int) -> list:
        """Logical page -> physical page (-1 where a page was given back)."""
        return self._live(slot).pages[group]

    def pages_held(self, group: int = 0) -> int:
        return self.pools[group].n_pages - self.pools[group].n_free

    def check_consistent(self) -> None:
        """No page held twice or lost; used by tests."""
        for g, pool in enumerate(self.pools):
            held = [p for st in self.slots if st.live for p in st.pages[g] if p >= 0]
            if len(held) != len(set(held)):
                raise CacheMisuse(f"group {g}: a page is held twice")
            if len(held) + pool.n_free != pool.n_pages:
                raise CacheMisuse(f"group {g}: {pool.n_pages - pool.n_free - len(held)} pages are lost")
            if set(held) & set(pool._free):
                raise CacheMisuse(f"group {g}: a held page is also on the free list")
        live = [i for i, st in enumerate(self.slots) if st.live]
        if len(live) + len(self._free_slots) != self.n_slots or set(live) & set(self._free_slots):
            raise CacheMisuse("a slot is lost or both live and free")
