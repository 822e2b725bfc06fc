"""Random-weights mode: from a configuration and a seed, either a model folder
on disk (config.json + model.safetensors) or the tensors directly on a device.

Matrices are N(0, 0.02); gains are 1 + N(0, 0.02).  The reference has only an
offline script for this (scripts/make-tiny-qwen35.py:96-102: seeded Gaussian
matrices, gains around 1).  Every tensor has a stream of its own, derived from
the seed and the tensor's name, so its values do not depend on which other
tensors exist or in which order they are made.
"""

from __future__ import annotations

import json
import zlib
from pathlib import Path

import numpy as np
import torch

from ..config.spec import ModelSpec
from .safetensors_io import SafetensorsWriter

MATRIX_STD = 0.02
GAIN_STD = 0.02
_CHUNK = 1 << 24


def _stream_seed(seed: int, name: str) -> int:
    return (int(seed) * 0x9E3779B1 + zlib.crc32(name.encode())) & 0x7FFFFFFFFFFFFFFF


def _storage_dtype(spec: ModelSpec, role: str, dtype=None) -> torch.dtype:
    if role == "table":
        return torch.int32
    name = dtype or spec.storage_dtype
    return {"bfloat16": torch.bfloat16, "float32": torch.float32}[name]


def _host_tensor(t, seed: int, dtype: torch.dtype) -> torch.Tensor:
    rng = np.random.Generator(np.random.PCG64(_stream_seed(seed, t.name)))
    n = int(np.prod(t.shape, dtype=np.int64))
    out = torch.empty(n, dtype=dtype)
    for lo in range(0, n, _CHUNK):
        m = min(_CHUNK, n - lo)
        x = rng.standard_normal(m, dtype=np.float32)
        if t.role == "vector":
            x = 1.0 + GAIN_STD * x
        else:
            x = MATRIX_STD * x
        out[lo : lo + m] = torch.from_numpy(x.astype(np.float32)).to(dtype)
    return out.view(t.shape)


def write_model_folder(folder, config, seed: int, dtype: str | None = None) -> Path:
    """Writes config.json and model.safetensors for ``config`` (a typed
    configuration with ``to_spec`` and ``to_dict``).  ``dtype`` overrides the
    storage dtype that the configuration names."""
    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    spec = config.to_spec()
    raw = config.to_dict()
    if dtype is not None:
        raw["torch_dtype"] = dtype
    (folder / "config.json").write_text(json.dumps(raw, indent=2) + "\n")
    tensors = spec.tensors()
    declared = [(t.name, _storage_dtype(spec, t.role, dtype), tuple(t.shape)) for t in tensors]
    with SafetensorsWriter(folder / "model.safetensors", declared,
                           {"format": "pt", "seed": seed, "generator": "llmoxide_b200.random_init"}) as w:
        for t, (_, dt, _) in zip(tensors, declared):
            w.write(t.name, _host_tensor(t, seed, dt))
    return folder


def random_tensors_on_device(spec: ModelSpec, seed: int, dtype: str = "bfloat16", device="cuda") -> dict:
    """The same distributions made on the device, for models too large to be
    worth a trip through the file system.  The values differ from
    ``write_model_folder``'s (another generator); use a folder where two
    implementations must see the same weights."""
    out = {}
    for t in spec.tensors():
        gen = torch.Generator(device=device)
        gen.manual_seed(_stream_seed(seed, t.name))
        # A gain stays float32 in either mode; a matrix follows ``dtype``.
        dt = torch.float32 if (dtype == "float32" or t.role == "vector") else torch.bfloat16
        x = torch.empty(t.shape, dtype=dt, device=device)
        x.normal_(0.0, 1.0, generator=gen)
        if t.role == "vector":
            x.mul_(GAIN_STD).add_(1.0)
        else:
            x.mul_(MATRIX_STD)
        out[t.name] = x
    return out
