"""What every part is told about where it runs."""

from __future__ import annotations

from dataclasses import dataclass, field

import torch


@dataclass
class Runtime:
    dtype: str                 # "bfloat16" (serving precisions) or "float32" (true 32-bit everywhere)
    device: torch.device
    max_positions: int         # longest sequence the cache allows; sizes position tables
    tensor_cores: bool = True  # bfloat16 only: use the tcgen05 matrix product where it applies
    shared: dict = field(default_factory=dict)  # objects that parts of one model share (position tables)
    n_sm: int = 0              # streaming multiprocessors of the device (asked once; the split policies size grids by it)

    def __post_init__(self):
        if not self.n_sm:
            self.n_sm = kernels_n_sm(self.device)

    @property
    def act_dtype(self) -> torch.dtype:
        return torch.float32 if self.dtype == "float32" else torch.bfloat16

    @property
    def cache_dtype(self) -> torch.dtype:
        return self.act_dtype


_n_sm: dict = {}


def kernels_n_sm(device) -> int:
    """cudaDevAttrMultiProcessorCount of ``device``, asked once."""
    device = torch.device(device)
    if device.type != "cuda" or not torch.cuda.is_available():
        return 148          # no device to ask (descriptions built on a CPU box): the B200's count
    key = device.index if device.index is not None else torch.cuda.current_device()
    if key not in _n_sm:
        _n_sm[key] = int(torch.cuda.get_device_properties(key).multi_processor_count)
    return _n_sm[key]
