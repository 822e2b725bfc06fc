"""Checkpoint -> tensors on the device, by tensor name, checked against the
model description before anything is copied.

The reference resolves every tensor by name up front and compares every
dimension with the configuration (crates/model/src/qwen35/weights.rs:71-203),
aliasing the head to the embedding table when the checkpoint has none
(weights.rs:79).  Here every problem of a checkpoint is collected into one
``WeightsError``: missing tensors, unexpected tensors, wrong shapes or dtypes.

Precision policy.  ``bfloat16``: a tensor stored in 16-bit floating point is
kept as bfloat16, a tensor stored in 32-bit stays float32, integer tables
become int32.  ``float32``: every floating-point tensor is widened to float32
(exact), so that the whole model runs in true 32-bit.
"""

from __future__ import annotations

import sys

import torch

from ..config.spec import ModelSpec
from ..errors import CheckpointFormatError, WeightsError
from .safetensors_io import open_checkpoint

_FLOATS = ("F32", "F16", "BF16")
_INTS = ("I64", "I32", "I16", "I8", "U8")


def check_checkpoint(spec: ModelSpec, entries: dict, where="") -> list:
    """Raises WeightsError unless the checkpoint holds exactly the tensors of
    ``spec`` with their shapes.  Returns notes about tensors that are ignored."""
    expected = {t.name: t for t in spec.tensors()}
    missing = [n for n in expected if n not in entries]
    unexpected, notes = [], []
    for n in entries:
        if n in expected:
            continue
        if spec.is_ignored(n):
            # the description names tensors a file may carry that the model does not use
            if n in spec.ignored_tensors:
                notes.append(f"{n} is present but the configuration does not use it; ignored")
            continue
        unexpected.append(n)
    wrong = []
    for n, t in expected.items():
        e = entries.get(n)
        if e is None:
            continue
        if tuple(e.shape) != tuple(t.shape):
            wrong.append((n, f"shape {list(e.shape)} != expected {list(t.shape)}"))
        elif t.role == "table" and e.dtype not in _INTS:
            wrong.append((n, f"dtype {e.dtype}, expected an integer table"))
        elif t.role != "table" and e.dtype not in _FLOATS:
            wrong.append((n, f"dtype {e.dtype}, expected floating point"))
    if missing or unexpected or wrong:
        raise WeightsError(sorted(missing), sorted(unexpected), wrong, where)
    return notes


def target_dtype(stored: torch.dtype, compute: str) -> torch.dtype:
    if not stored.is_floating_point:
        return torch.int32
    if compute == "float32" or stored == torch.float32:
        return torch.float32
    return torch.bfloat16


VERIFY_SPAN = 256      # elements read back at the head and at the tail of every uploaded tensor


def _verify_upload(name: str, host: torch.Tensor, dev: torch.Tensor) -> None:
    """Reads the first and last elements of an uploaded tensor back and compares them with what was sent
    (the reference checks head and tail spans of every buffer it uploads, crates/gpu/src/lib.rs:700-712)."""
    flat_h, flat_d = host.reshape(-1), dev.reshape(-1)
    n = flat_h.numel()
    for lo, hi in ((0, min(n, VERIFY_SPAN)), (max(0, n - VERIFY_SPAN), n)):
        want = flat_h[lo:hi].to(flat_d.dtype)
        got = flat_d[lo:hi].cpu()
        if not torch.equal(got.view(torch.uint8), want.contiguous().view(torch.uint8)):
            raise CheckpointFormatError(f"{name}: elements {lo}..{hi} read back from the device differ from the file")


def load_checkpoint(folder, spec: ModelSpec, dtype: str = "bfloat16", device="cuda",
                    progress=None, verify: bool = True) -> dict:
    """name -> tensor on ``device`` for every tensor of ``spec``; with ``verify`` the head and the tail of
    every tensor are read back and compared."""
    if dtype not in ("bfloat16", "float32"):
        raise ValueError(f"dtype {dtype!r}: expected 'bfloat16' or 'float32'")
    entries = open_checkpoint(folder)
    for note in check_checkpoint(spec, entries, where=str(folder)):
        print(f"[llmoxide_b200] {note}", file=sys.stderr)
    out = {}
    names = [t.name for t in spec.tensors()]
    for i, name in enumerate(names):
        e = entries[name]
        host = e.file.tensor(name)
        out[name] = host.to(device=device, dtype=target_dtype(host.dtype, dtype), copy=True)
        if verify:
            _verify_upload(name, host, out[name])
        if progress is not None:
            progress(i + 1, len(names), name)
    return out
