"""Reader and writer for safetensors files, by tensor name.

File format: an 8-byte little-endian header length, a JSON header
``{name: {"dtype", "shape", "data_offsets": [begin, end]}}`` and the payload.
The reader maps the file and hands out tensors that borrow from the mapping,
checks every tensor's extent against the file before anything is read (the
reference checks its GGUF the same way, crates/gguf/src/lib.rs:496-508), and
follows ``model.safetensors.index.json`` when a checkpoint is split.
"""

from __future__ import annotations

import json
import struct
from pathlib import Path

import numpy as np
import torch

from ..errors import CheckpointFormatError

# safetensors dtype -> (numpy dtype used to map the bytes, torch dtype, bytes per element)
_DTYPES = {
    "F32": (np.float32, torch.float32, 4),
    "F16": (np.float16, torch.float16, 2),
    "BF16": (np.int16, torch.bfloat16, 2),
    "I64": (np.int64, torch.int64, 8),
    "I32": (np.int32, torch.int32, 4),
    "I16": (np.int16, torch.int16, 2),
    "I8": (np.int8, torch.int8, 1),
    "U8": (np.uint8, torch.uint8, 1),
    "BOOL": (np.bool_, torch.bool, 1),
}
_TORCH_TO_ST = {torch.float32: "F32", torch.float16: "F16", torch.bfloat16: "BF16",
                torch.int64: "I64", torch.int32: "I32", torch.int16: "I16",
                torch.int8: "I8", torch.uint8: "U8", torch.bool: "BOOL"}

_MAX_HEADER = 100 << 20


class TensorEntry:
    __slots__ = ("name", "dtype", "shape", "begin", "end", "file")

    def __init__(self, name, dtype, shape, begin, end, file):
        self.name, self.dtype, self.shape = name, dtype, tuple(shape)
        self.begin, self.end, self.file = begin, end, file

    @property
    def torch_dtype(self):
        return _DTYPES[self.dtype][1]

    def __repr__(self):
        return f"{self.name}: {self.dtype}{list(self.shape)}"


class SafetensorsFile:
    """One mapped file.  ``entries`` holds every tensor's description."""

    def __init__(self, path):
        self.path = Path(path)
        size = self.path.stat().st_size
        if size < 8:
            raise CheckpointFormatError(f"{self.path}: {size} bytes is too short for a safetensors header")
        with open(self.path, "rb") as f:
            (n,) = struct.unpack("<Q", f.read(8))
            if n > _MAX_HEADER or 8 + n > size:
                raise CheckpointFormatError(
                    f"{self.path}: header of {n} bytes runs past the end of the file ({size} bytes)")
            try:
                header = json.loads(f.read(n))
            except (json.JSONDecodeError, UnicodeDecodeError) as e:
                raise CheckpointFormatError(f"{self.path}: header is not valid JSON: {e}") from None
        if not isinstance(header, dict):
            raise CheckpointFormatError(f"{self.path}: header is not a JSON object")
        self.metadata = header.pop("__metadata__", None) or {}
        self._base = 8 + n
        payload = size - self._base
        self.entries = {}
        for name, info in header.items():
            try:
                dtype, shape = info["dtype"], list(info["shape"])
                begin, end = info["data_offsets"]
            except (KeyError, TypeError, ValueError):
                raise CheckpointFormatError(f"{self.path}: malformed entry for tensor {name!r}") from None
            if dtype not in _DTYPES:
                raise CheckpointFormatError(f"{self.path}: tensor {name!r} has unsupported dtype {dtype!r}")
            want = int(np.prod(shape, dtype=np.int64)) * _DTYPES[dtype][2] if shape else _DTYPES[dtype][2]
            if begin < 0 or end < begin or end - begin != want:
                raise CheckpointFormatError(
                    f"{self.path}: tensor {name!r} spans {end - begin} bytes, its shape {shape} needs {want}")
            if end > payload:
                raise CheckpointFormatError(
                    f"{self.path}: tensor {name!r} runs past the end of the file "
                    f"(needs {end} payload bytes, file has {payload}); the file is truncated")
            self.entries[name] = TensorEntry(name, dtype, shape, begin, end, self)
        self._map = None

    def _mapping(self):
        if self._map is None:
            self._map = np.memmap(self.path, dtype=np.uint8, mode="r")
        return self._map

    def tensor(self, name) -> torch.Tensor:
        """A CPU tensor that borrows from the mapping (read-only: copy before writing)."""
        e = self.entries[name]
        np_dtype, torch_dtype, _ = _DTYPES[e.dtype]
        raw = self._mapping()[self._base + e.begin : self._base + e.end]
        arr = raw.view(np_dtype).reshape(e.shape)
        import warnings
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")  # torch warns that the mapping is not writable
            t = torch.from_numpy(arr)
        return t.view(torch_dtype) if e.dtype == "BF16" else t


def open_checkpoint(folder) -> dict:
    """name -> TensorEntry over every file of a model folder.  A split
    checkpoint lists its files in model.safetensors.index.json."""
    folder = Path(folder)
    index = folder / "model.safetensors.index.json"
    if index.is_file():
        weight_map = json.loads(index.read_text()).get("weight_map", {})
        files = sorted(set(weight_map.values()))
    elif (folder / "model.safetensors").is_file():
        files = ["model.safetensors"]
    else:
        raise CheckpointFormatError(f"{folder}: no model.safetensors (or model.safetensors.index.json) found")
    entries = {}
    for fname in files:
        path = folder / fname
        if not path.is_file():
            raise CheckpointFormatError(f"{folder}: the index names {fname}, which does not exist")
        for name, e in SafetensorsFile(path).entries.items():
            if name in entries:
                raise CheckpointFormatError(f"{folder}: tensor {name!r} appears in more than one file")
            entries[name] = e
    return entries


class SafetensorsWriter:
    """Writes one file tensor by tensor, so that a model larger than host
    memory can be written: declare every tensor first, then stream the data
    in the declared order."""

    def __init__(self, path, declared, metadata=None):
        """``declared``: list of (name, torch dtype, shape)."""
        self.path = Path(path)
        header, offset = {}, 0
        self._order = []
        for name, dtype, shape in declared:
            st = _TORCH_TO_ST[dtype]
            nbytes = int(np.prod(shape, dtype=np.int64)) * _DTYPES[st][2] if len(shape) else _DTYPES[st][2]
            header[name] = {"dtype": st, "shape": list(shape), "data_offsets": [offset, offset + nbytes]}
            self._order.append((name, dtype, tuple(shape), nbytes))
            offset += nbytes
        if metadata:
            header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
        blob = json.dumps(header, separators=(",", ":")).encode()
        blob += b" " * (-len(blob) % 8)
        self._f = open(self.path, "wb")
        self._f.write(struct.pack("<Q", len(blob)))
        self._f.write(blob)
        self._next = 0

    def write(self, name, tensor: torch.Tensor) -> None:
        want_name, dtype, shape, nbytes = self._order[self._next]
        if name != want_name or tensor.dtype != dtype or tuple(tensor.shape) != shape:
            raise ValueError(f"expected {want_name} {dtype} {shape}, got {name} {tensor.dtype} {tuple(tensor.shape)}")
        t = tensor.detach().contiguous().cpu()
        if t.dtype == torch.bfloat16:
            t = t.view(torch.int16)
        data = t.numpy().tobytes()
        assert len(data) == nbytes
        self._f.write(data)
        self._next += 1

    def close(self) -> None:
        if self._next != len(self._order):
            raise ValueError(f"{len(self._order) - self._next} declared tensors were never written")
        self._f.close()

    def __enter__(self):
        return self

    def __exit__(self, exc_type, exc, tb):
        if exc_type is None:
            self.close()
        else:
            self._f.close()


def save_file(tensors: dict, path, metadata=None) -> None:
    declared = [(n, t.dtype, tuple(t.shape)) for n, t in tensors.items()]
    with SafetensorsWriter(path, declared, metadata) as w:
        for n, t in tensors.items():
            w.write(n, t)
