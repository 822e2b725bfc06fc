"""Random-weights mode: from a configuration and a seed, either a model folder
on disk (config.json + model.safetensors) or the tensors directly on a device.
Both hold the same values, bit for bit, so a model made on the device has a
twin that any other implementation can read from a folder.

Matrices are N(0, 0.02); gains are 1 + N(0, 0.02).  The reference has only an
offline script for this (scripts/make-tiny-qwen35.py:96-102: seeded Gaussian
matrices, gains around 1).  The generator is counter-based: element i of a
tensor depends on the seed, the tensor's name and i alone, so a tensor's values
do not depend on which other tensors exist, in which order they are made, or
where (numpy here, one CUDA thread per element in csrc/random_init.cu).

    z = mix(stream + (i + 1) * 0x9E3779B97F4A7C15)          64-bit, wrapping
    a = z >> 48, f = ((z >> 32) & 0xffff) / 65536
    x = q[a] + (q[a + 1] - q[a]) * f                          q: 65537 quantiles of N(0, 1)
    value = mean + std * x   -> storage dtype

Each floating-point step is a single float32 operation, rounded once, on
either side.  The normal is cut at about 4.3 standard deviations (the outermost
quantiles) and is linear between neighbouring quantiles.
"""

from __future__ import annotations

import json
import os
import zlib
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

import numpy as np
import torch

from ..config.spec import ModelSpec
from .loader import target_dtype
from .safetensors_io import SafetensorsWriter

MATRIX_STD = 0.02
GAIN_STD = 0.02
_CHUNK = 1 << 22
_GOLDEN = np.uint64(0x9E3779B97F4A7C15)
_M1, _M2 = np.uint64(0xBF58476D1CE4E5B9), np.uint64(0x94D049BB133111EB)
_N_QUANTILES = 1 << 16


def _stream_seed(seed: int, name: str) -> int:
    """The 64-bit stream word of one tensor."""
    h = (int(seed) * 0x9E3779B1 + zlib.crc32(name.encode())) & 0xFFFFFFFFFFFFFFFF
    return (h * 0xD6E8FEB86659FD93 + 0x2545F4914F6CDD1D) & 0xFFFFFFFFFFFFFFFF


_quantiles_host = None
_quantiles_dev: dict = {}


def quantiles() -> np.ndarray:
    """q[a] = the a/65536 quantile of N(0, 1) as float32, a = 0..65536, the two ends moved in to the
    quantiles of 1/4 of a step; antisymmetric by construction."""
    global _quantiles_host
    if _quantiles_host is None:
        n = _N_QUANTILES
        p = torch.arange(1, n // 2 + 1, dtype=torch.float64) / n          # (0, 1/2]
        upper = -torch.special.ndtri(p).flip(0)                            # quantiles of [1/2, 1)
        upper = torch.cat([upper, -torch.special.ndtri(torch.tensor([0.25 / n], dtype=torch.float64))])
        upper = upper.to(torch.float32).numpy()
        upper[0] = 0.0
        _quantiles_host = np.concatenate([-upper[:0:-1], upper]).astype(np.float32)
        assert _quantiles_host.shape == (n + 1,)
    return _quantiles_host


def _mix(z: np.ndarray) -> np.ndarray:
    z = (z ^ (z >> np.uint64(30))) * _M1
    z = (z ^ (z >> np.uint64(27))) * _M2
    return z ^ (z >> np.uint64(31))


def host_values(stream: int, lo: int, n: int, mean: float, std: float) -> np.ndarray:
    """Elements lo .. lo+n-1 of a stream as float32 (before the storage dtype's rounding)."""
    q = quantiles()
    with np.errstate(over="ignore"):
        i = np.arange(lo + 1, lo + n + 1, dtype=np.uint64)
        z = _mix(np.uint64(stream) + i * _GOLDEN)
    a = (z >> np.uint64(48)).astype(np.int64)
    f = ((z >> np.uint64(32)) & np.uint64(0xFFFF)).astype(np.float32) * np.float32(1.0 / 65536.0)
    q0, q1 = q[a], q[a + 1]
    x = q0 + (q1 - q0) * f
    return np.float32(mean) + np.float32(std) * x


def _moments(role: str):
    return (1.0, GAIN_STD) if role == "vector" else (0.0, MATRIX_STD)


def _storage_dtype(spec: ModelSpec, role: str, dtype=None) -> torch.dtype:
    if role == "table":
        return torch.int32
    name = dtype or spec.storage_dtype
    return {"bfloat16": torch.bfloat16, "float32": torch.float32}[name]


def host_tensor(t, seed: int, dtype: torch.dtype) -> torch.Tensor:
    """One tensor of the description on the host, in ``dtype``."""
    stream = _stream_seed(seed, t.name)
    mean, std = _moments(t.role)
    n = int(np.prod(t.shape, dtype=np.int64))
    out = torch.empty(n, dtype=dtype)

    def fill(lo):
        m = min(_CHUNK, n - lo)
        out[lo : lo + m] = torch.from_numpy(host_values(stream, lo, m, mean, std)).to(dtype)

    if n <= _CHUNK:
        fill(0)
    else:       # numpy releases the interpreter lock inside its loops: large tensors use the cores there are
        with ThreadPoolExecutor(max_workers=min(16, os.cpu_count() or 1)) as pool:
            list(pool.map(fill, range(0, n, _CHUNK)))
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
            w.write(t.name, host_tensor(t, seed, dt))
    return folder


def random_tensors_on_device(spec: ModelSpec, seed: int, dtype: str = "bfloat16", device="cuda",
                             storage: str | None = None) -> dict:
    """What ``load_checkpoint`` would return for the folder that ``write_model_folder`` writes from the same
    description and seed (storage dtype ``storage``, default the description's), made on the device without
    a trip through the file system: every value is rounded to the storage dtype and kept in the dtype the
    precision policy gives it."""
    from .. import kernels

    device = torch.device(device)
    q = _quantiles_dev.get(device)
    if q is None:
        q = _quantiles_dev[device] = torch.from_numpy(quantiles()).to(device)
    out = {}
    for t in spec.tensors():
        stored = _storage_dtype(spec, t.role, storage)
        if not stored.is_floating_point:
            raise ValueError(f"{t.name}: integer tables have no random-weights rule")
        x = torch.empty(t.shape, dtype=target_dtype(stored, dtype), device=device)
        mean, std = _moments(t.role)
        kernels.fill_normal(x, _stream_seed(seed, t.name), q, mean, std, stored)
        out[t.name] = x
    return out
