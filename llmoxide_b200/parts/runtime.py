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

    @property
    def act_dtype(self) -> torch.dtype:
        return torch.float32 if self.dtype == "float32" else torch.bfloat16

    @property
    def cache_dtype(self) -> torch.dtype:
        return self.act_dtype
