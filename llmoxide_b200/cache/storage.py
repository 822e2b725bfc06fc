"""Device storage of the cache and the per-sequence state area.

Cache entries (one per ``LayerCall.cache`` id) with equal needs form a group
with storage and a page pool of its own: keys and values as
``[entry, page, kv head, row in page, dim]``.  Beside the keys and values,
every entry may own per-sequence state of fixed size, ``[slot, *shape]``,
zero-filled whenever a slot gets a new owner (the reference zeroes its
recurrent state on clear because it is cumulative,
crates/model/src/qwen35/state.rs:41-45,65-73).  The dense Qwen3 decoder has
no such state; the area exists, is addressed and is reset through the same
path, so that a mixer with state can use it.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from ..guard import guarded
from .allocator import PAGE, CacheAllocator


@dataclass(frozen=True)
class KVNeed:
    """Keys and values for every position (window None) or for the last
    ``window`` positions.  Values may be narrower or wider than keys
    (``v_head_dim``, default ``head_dim``), and an entry may keep its keys and
    values in a dtype of its own (default: the runtime's cache dtype)."""

    n_kv_heads: int
    head_dim: int
    window: Optional[int] = None
    v_head_dim: Optional[int] = None
    dtype: Optional[torch.dtype] = None


@dataclass(frozen=True)
class StateNeed:
    """Fixed-size state per sequence, float32 unless said otherwise."""

    shape: tuple
    dtype: torch.dtype = torch.float32


@dataclass
class CacheEntryView:
    """What one layer call sees of the cache."""

    group: Optional[int]            # index of the block table to use; None without keys/values
    k: Optional[torch.Tensor]       # [n_pages, G, PAGE, D]
    v: Optional[torch.Tensor]       # [n_pages, G, PAGE, D of the values]
    state: Optional[torch.Tensor]   # [n_slots, *shape]
    need: Optional[KVNeed]


class Cache:
    def __init__(self, needs: list, n_slots: int, max_tokens: int, dtype: torch.dtype, device,
                 max_seq_len: Optional[int] = None):
        """``needs[e] = (KVNeed | None, StateNeed | None)`` for cache entry e.
        ``max_tokens``: the most tokens live sequences hold at any time, each
        sequence's count rounded up to a multiple of PAGE."""
        self.n_slots, self.dtype, self.device = n_slots, dtype, device
        n_pages = max(1, (max_tokens + PAGE - 1) // PAGE)
        self.n_pages = n_pages
        self.groups: list = []          # KVNeed per group
        self._entry_group: list = []    # entry -> (group, index in group) or None
        members: dict = {}
        for kv, _ in needs:
            if kv is None:
                self._entry_group.append(None)
                continue
            if kv not in members:
                members[kv] = []
                self.groups.append(kv)
            g = self.groups.index(kv)
            self._entry_group.append((g, len(members[kv])))
            members[kv].append(len(self._entry_group) - 1)
        self.k_store, self.v_store = [], []
        for kv in self.groups:
            k_shape = (len(members[kv]), n_pages, kv.n_kv_heads, PAGE, kv.head_dim)
            v_shape = k_shape[:-1] + (kv.v_head_dim or kv.head_dim,)
            # (every long-lived buffer carries guard words behind it: guard.py)
            g = len(self.k_store)
            self.k_store.append(guarded(k_shape, kv.dtype or dtype, device, f"cache group {g} keys", zero=True))
            self.v_store.append(guarded(v_shape, kv.dtype or dtype, device, f"cache group {g} values", zero=True))
        self.state_store = [
            None if st is None else guarded((n_slots, *st.shape), st.dtype, device, f"cache entry {e} state", zero=True)
            for e, (_, st) in enumerate(needs)
        ]
        self.alloc = CacheAllocator(n_slots, n_pages, [kv.window for kv in self.groups] or [None],
                                    max_seq_len=max_seq_len)
        self._has_groups = bool(self.groups)

    # ---- slots -------------------------------------------------------------

    def acquire(self) -> int:
        slot = self.alloc.acquire()
        for st in self.state_store:
            if st is not None:
                st[slot].zero_()
        return slot

    def release(self, slot: int) -> None:
        self.alloc.release(slot)

    def length(self, slot: int) -> int:
        return self.alloc.length(slot)

    # ---- views ---------------------------------------------------------------

    def view(self, entry: int) -> CacheEntryView:
        eg = self._entry_group[entry]
        if eg is None:
            return CacheEntryView(None, None, None, self.state_store[entry], None)
        g, i = eg
        return CacheEntryView(g, self.k_store[g][i], self.v_store[g][i], self.state_store[entry], self.groups[g])

    def n_groups(self) -> int:
        return len(self.groups)

    def bytes(self) -> int:
        n = sum(t.numel() * t.element_size() for t in self.k_store + self.v_store)
        return n + sum(t.numel() * t.element_size() for t in self.state_store if t is not None)

    def wipe(self) -> None:
        """Overwrites every key, value and state (crates/model/src/qwen35/state.rs:75-92)."""
        for t in self.k_store + self.v_store + [s for s in self.state_store if s is not None]:
            t.zero_()
