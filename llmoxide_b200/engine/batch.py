"""One step's batch: which tokens of which sequences run, where they sit in
their sequences and in the cache, and whose logits are wanted.

Everything a kernel needs to know about the batch travels in ONE int32 buffer
(pinned on the host, one copy to the device per step): the packed token ids,
each token's sequence and position, each sequence's start in the packed row,
its cached length and slot, the rows whose logits are wanted, and one block
table per cache group.  The step function's semantics are the reference's
single-sequence forward applied per sequence (crates/model/src/qwen35/cpu.rs:
106-125): tokens are appended at the sequence's current length.
"""

from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np
import torch

from ..cache import PAGE
from ..guard import guarded


def _align(n: int, a: int = 4) -> int:
    return (n + a - 1) // a * a


@dataclass
class StepLayout:
    """Offsets (in int32 elements) of each array inside the step buffer."""

    n_tokens: int
    n_seqs: int
    n_want: int
    widths: tuple            # block-table width per cache group
    offsets: dict = field(default_factory=dict)
    total: int = 0

    @classmethod
    def make(cls, n_tokens, n_seqs, n_want, widths):
        lay = cls(n_tokens, n_seqs, n_want, tuple(widths))
        at = 0
        for name, n in (("tokens", n_tokens), ("token_seq", n_tokens), ("token_pos", n_tokens),
                        ("seq_start", n_seqs + 1), ("seq_past", n_seqs), ("seq_slot", n_seqs),
                        ("want_rows", n_want),
                        *((f"block_table{g}", n_seqs * w) for g, w in enumerate(widths))):
            lay.offsets[name] = (at, n)
            at = _align(at + n)
        lay.total = max(at, 4)
        return lay

    def key(self):
        return (self.n_tokens, self.n_seqs, self.n_want, self.widths)


@dataclass
class StepContext:
    """The batch as the parts see it: device views and a few host numbers."""

    n_tokens: int
    n_seqs: int
    max_new: int             # most new tokens of one sequence
    max_len: int             # longest sequence after this step
    is_decode: bool          # every sequence brings exactly one token
    tokens: torch.Tensor
    token_seq: torch.Tensor
    token_pos: torch.Tensor
    seq_start: torch.Tensor
    seq_past: torch.Tensor
    seq_slot: torch.Tensor
    want_rows: torch.Tensor
    block_tables: list
    widths: tuple
    probe: object = None     # callable(name, tensor) for named intermediates of the step, or None


N_FIXED = 7        # arrays before the block tables: tokens, token_seq, token_pos, seq_start, seq_past, seq_slot, want_rows
_NAMES = ("tokens", "token_seq", "token_pos", "seq_start", "seq_past", "seq_slot", "want_rows")


def layout_from_meta(meta) -> tuple:
    """(layout, facts) from the numbers the C++ packer returns (csrc/host_runtime.cpp, write_meta)."""
    n_tokens, n_seqs, n_want, total, max_new, max_len, is_decode, n_groups = (int(x) for x in meta[:8])
    offs = [int(x) for x in meta[8 : 8 + N_FIXED + n_groups]]
    widths = tuple(int(x) for x in meta[8 + N_FIXED + n_groups : 8 + N_FIXED + 2 * n_groups])
    lay = StepLayout(n_tokens, n_seqs, n_want, widths)
    sizes = (n_tokens, n_tokens, n_tokens, n_seqs + 1, n_seqs, n_seqs, n_want)
    for name, at, n in zip(_NAMES, offs, sizes):
        lay.offsets[name] = (at, n)
    for g, w in enumerate(widths):
        lay.offsets[f"block_table{g}"] = (offs[N_FIXED + g], n_seqs * w)
    lay.total = total
    return lay, dict(max_new=max_new, max_len=max_len, is_decode=bool(is_decode))


def flatten_entries(entries, wants):
    """The entries as the flat int32 arrays the C++ runtime takes; ``wants`` None: every entry's last token."""
    n = len(entries)
    slots = np.fromiter((s for s, _ in entries), dtype=np.int32, count=n)
    counts = np.fromiter((len(t) for _, t in entries), dtype=np.int32, count=n)
    toks = [t for _, t in entries]
    tokens = (np.concatenate([np.asarray(t, dtype=np.int64) for t in toks]) if n and counts.sum() else
              np.zeros(0, dtype=np.int64))
    if tokens.size and (tokens.min() < -(1 << 31) or tokens.max() >= (1 << 31)):
        raise ValueError("a token id does not fit 32 bits")
    tokens = np.ascontiguousarray(tokens, dtype=np.int32)
    if wants is None:
        want_counts = np.full(n, -1, dtype=np.int32)
        want_flat = np.zeros(1, dtype=np.int32)
    else:
        want_counts = np.fromiter((len(w) for w in wants), dtype=np.int32, count=n)
        flat = [x for w in wants for x in w]
        want_flat = np.asarray(flat if flat else [0], dtype=np.int32)
    return slots, counts, tokens, want_counts, want_flat


def build_host_arrays(entries, wants, lengths, page_rows, n_groups):
    """``entries``: [(slot, tokens)]; ``wants``: per entry the places among its
    tokens whose logits are wanted; ``lengths``: cached length per entry;
    ``page_rows[g][i]``: entry i's logical->physical page list in group g.
    Returns (layout, int32 array, host facts).  The packing itself is the C++
    runtime's (the engine's own steps go through its ``llmx_plan_step``, which
    also checks and reserves)."""
    from ..cache.allocator import host_library, raise_host_error

    lib = host_library()
    n = len(entries)
    slots, counts, tokens, want_counts, want_flat = flatten_entries(entries, wants)
    lens = np.asarray(lengths, dtype=np.int64)
    rows, row_off, row_len = [], [], []
    for g in range(n_groups):
        for i in range(n):
            row_off.append(len(rows))
            row_len.append(len(page_rows[g][i]))
            rows.extend(page_rows[g][i])
    rows = np.asarray(rows if rows else [0], dtype=np.int32)
    row_off = np.asarray(row_off, dtype=np.int64)
    row_len = np.asarray(row_len, dtype=np.int32)
    meta = np.zeros(8 + N_FIXED + 2 * n_groups, dtype=np.int64)
    cap = 4 * int(counts.sum()) + 8 * n + len(want_flat) + n * n_groups * (int(lens.max() + counts.max()) // PAGE + 8) + 64
    buf = np.zeros(cap, dtype=np.int32)
    ptr = lambda a: a.ctypes.data
    code = lib.llmx_pack_step(n, ptr(slots), ptr(counts), ptr(tokens), ptr(want_counts), ptr(want_flat), ptr(lens),
                              n_groups, ptr(rows), ptr(row_off), ptr(row_len), ptr(buf), cap, ptr(meta))
    if code:
        raise_host_error(code)
    lay, facts = layout_from_meta(meta)
    return lay, buf[: lay.total], facts


class StepBuffers:
    """Pinned host buffers and their device twin; all grow when needed.  The
    host side is a small ring: a buffer is written again only after the copy
    that last read it has finished on the device."""

    RING = 4

    def __init__(self, device, capacity: int = 1 << 14):
        self.device = device
        self._alloc(capacity)

    def _alloc(self, capacity):
        self.capacity = capacity
        self.hosts = [torch.empty(capacity, dtype=torch.int32).pin_memory() for _ in range(self.RING)]
        self.events = [None] * self.RING
        self.turn = 0
        self.dev = guarded((capacity,), torch.int32, self.device, "step buffer")

    def upload(self, lay: StepLayout, buf: np.ndarray, facts: dict) -> StepContext:
        """A packed step (``build_host_arrays``) through the next pinned buffer to the device."""
        if lay.total > self.capacity:
            self.grow(lay.total)
        host = self.next_host()
        host[: lay.total].copy_(torch.from_numpy(buf))
        return self.send(lay, facts)

    def grow(self, total: int) -> None:
        torch.cuda.current_stream().synchronize()
        self._alloc(max(total, 2 * self.capacity))

    def next_host(self) -> torch.Tensor:
        """The pinned buffer the next step is packed into (free again: the copy that last read it is done)."""
        i = self.turn
        if self.events[i] is not None:
            self.events[i].synchronize()
        return self.hosts[i]

    def send(self, lay: StepLayout, facts: dict) -> StepContext:
        """Copies the buffer ``next_host`` gave out to the device and hands out the step's views."""
        i = self.turn
        self.turn = (i + 1) % self.RING
        host = self.hosts[i]
        self.dev[: lay.total].copy_(host[: lay.total], non_blocking=True)
        ev = torch.cuda.Event()
        ev.record()
        self.events[i] = ev
        return self.context(lay, facts)

    def context(self, lay: StepLayout, facts: dict) -> StepContext:
        def view(name):
            at, n = lay.offsets[name]
            return self.dev[at : at + n]

        tables = [view(f"block_table{g}").view(lay.n_seqs, w) for g, w in enumerate(lay.widths)]
        return StepContext(
            n_tokens=lay.n_tokens, n_seqs=lay.n_seqs, max_new=facts["max_new"], max_len=facts["max_len"],
            is_decode=facts["is_decode"], tokens=view("tokens"), token_seq=view("token_seq"),
            token_pos=view("token_pos"), seq_start=view("seq_start"), seq_past=view("seq_past"),
            seq_slot=view("seq_slot"), want_rows=view("want_rows"), block_tables=tables, widths=lay.widths)
