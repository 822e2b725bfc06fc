"""Guard words behind long-lived device buffers.

Every buffer that kernels of this package index with numbers computed from a
batch (the step buffer, each cache group's keys and values, the per-sequence
state, the sampler's buffers, arrival counters) is allocated with 256 bytes
of a fixed pattern after it.  A kernel that writes past the end of such a
buffer changes the pattern, and ``check_all`` says which buffer it was.  The
reference checks its own device state for residue in the same spirit
(crates/gpu/src/qwen35.rs:534-574).  Short-lived scratch (split partials of a
matrix product, the decode attention's workspace) gets guards too when
``scratch_guards(True)`` is on, which costs one fill per allocation and is
meant for tests.

Nothing here runs on the hot path: the pattern is written when a buffer is
made and read only by ``check_all``.
"""

from __future__ import annotations

import weakref

import torch

from .errors import KernelError

GUARD_BYTES = 256
PATTERN = 0x5AC35AC3

_entries: list = []          # [weakref to the payload, guard view, name]
_hold_dead = False           # tests: keep a buffer's guard until it has been checked once after its owner let go
_scratch = False


class GuardError(KernelError):
    """A guard word behind a device buffer was overwritten."""


def hold_until_checked(on: bool) -> None:
    """With this on, the guard of a buffer whose owner has let go of it is kept until the next ``check_all``
    (which then looks at it one last time); off, such guards are dropped when the next buffer is made."""
    global _hold_dead
    _hold_dead = on


def scratch_guards(on: bool) -> None:
    global _scratch
    _scratch = on


def _prune() -> None:
    if not _hold_dead:
        _entries[:] = [e for e in _entries if e[0]() is not None]


def guarded(shape, dtype, device, name: str, zero: bool = False) -> torch.Tensor:
    """A tensor of ``shape`` with guard words after its last element."""
    _prune()
    shape = tuple(int(n) for n in (shape if isinstance(shape, (tuple, list, torch.Size)) else (shape,)))
    n = 1
    for k in shape:
        n *= k
    nbytes = n * torch.empty((), dtype=dtype).element_size()
    padded = (nbytes + GUARD_BYTES - 1) // GUARD_BYTES * GUARD_BYTES
    base = torch.empty(padded + GUARD_BYTES, dtype=torch.uint8, device=device)
    if zero:
        base[:padded].zero_()
    guard = base[padded:].view(torch.int32)
    guard.fill_(PATTERN)
    payload = base[:nbytes].view(dtype).view(shape)
    _entries.append([weakref.ref(payload), guard, name])
    return payload


def scratch(shape, dtype, device, name: str = "scratch") -> torch.Tensor:
    """Short-lived scratch: plain ``torch.empty``, or guarded when ``scratch_guards`` is on."""
    if _scratch:
        return guarded(shape, dtype, device, name)
    return torch.empty(shape, dtype=dtype, device=device)


def check_all() -> int:
    """Looks at every guard; raises ``GuardError`` naming the buffers whose guard changed.  Returns how many
    guards were looked at.  Buffers whose owner has let go are forgotten afterwards."""
    torch.cuda.synchronize()
    bad, keep = [], []
    n = len(_entries)
    for entry in _entries:
        ref, guard, name = entry
        wrong = (guard != PATTERN).nonzero()
        if wrong.numel():
            bad.append(f"{name} (guard word {int(wrong[0])} of {guard.numel()})")
        elif ref() is not None:
            keep.append(entry)
    _entries[:] = keep          # reported guards are forgotten too: one report per fault
    if bad:
        raise GuardError("something wrote past the end of: " + "; ".join(bad))
    return n


def n_guards() -> int:
    return len(_entries)
