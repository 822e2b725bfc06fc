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


def build_host_arrays(entries, wants, lengths, page_rows, n_groups):
    """``entries``: [(slot, tokens)]; ``wants``: per entry the places among its
    tokens whose logits are wanted; ``lengths``: cached length per entry;
    ``page_rows[g][i]``: entry i's logical->physical page list in group g.
    Returns (layout, int32 array, host facts)."""
    n_seqs = len(entries)
    counts = [len(t) for _, t in entries]
    n_tokens = sum(counts)
    seq_start = np.zeros(n_seqs + 1, dtype=np.int32)
    seq_start[1:] = np.cumsum(counts)
    tokens = np.concatenate([np.asarray(t, dtype=np.int64) for _, t in entries]).astype(np.int32)
    token_seq = np.repeat(np.arange(n_seqs, dtype=np.int32), counts)
    token_pos = np.concatenate(
        [np.arange(p, p + c, dtype=np.int32) for p, c in zip(lengths, counts)])
    want_rows = np.asarray(
        [seq_start[i] + w for i, ws in enumerate(wants) for w in ws], dtype=np.int32)
    final = [p + c for p, c in zip(lengths, counts)]
    widths = []
    tables = []
    for g in range(n_groups):
        width = max(1, max((f + PAGE - 1) // PAGE for f in final))
        # Round the width up so that a growing sequence changes the layout rarely.
        width = _align(width, 4)
        tab = np.full((n_seqs, width), -1, dtype=np.int32)
        for i in range(n_seqs):
            row = page_rows[g][i]
            tab[i, : len(row)] = row
        widths.append(width)
        tables.append(tab)
    lay = StepLayout.make(n_tokens, n_seqs, len(want_rows), widths)
    buf = np.zeros(lay.total, dtype=np.int32)

    def put(name, arr):
        at, n = lay.offsets[name]
        buf[at : at + n] = np.asarray(arr, dtype=np.int32).reshape(-1)

    put("tokens", tokens), put("token_seq", token_seq), put("token_pos", token_pos)
    put("seq_start", seq_start), put("seq_past", lengths), put("seq_slot", [s for s, _ in entries])
    put("want_rows", want_rows)
    for g, tab in enumerate(tables):
        put(f"block_table{g}", tab)
    facts = dict(max_new=max(counts), max_len=max(final), is_decode=all(c == 1 for c in counts))
    return lay, buf, facts


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
        if lay.total > self.capacity:
            torch.cuda.current_stream().synchronize()
            self._alloc(max(lay.total, 2 * self.capacity))
        i = self.turn
        self.turn = (i + 1) % self.RING
        if self.events[i] is not None:
            self.events[i].synchronize()
        host = self.hosts[i]
        host[: lay.total].copy_(torch.from_numpy(buf))
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
