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
from ..errors import WeightsError
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


def load_checkpoint(folder, spec: ModelSpec, dtype: str = "bfloat16", device="cuda",
                    progress=None) -> dict:
    """name -> tensor on ``device`` for every tensor of ``spec``."""
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
        if progress is not None:
            progress(i + 1, len(names), name)
    return out
