"""The head: logits = x W^T in float32 over the wanted rows only, W the
head's own matrix or, tied, the embedding's table
(crates/model/src/qwen35/cpu.rs:406-416, crates/model/src/qwen35/weights.rs:79);
with ``softcap`` c the logits become c * tanh(logits / c) (the dense Qwen3
description gives none)."""

from __future__ import annotations

import torch

from .. import kernels
from ..errors import ConfigError
from .linear import Linear
from .registry import register_head


@register_head("linear")
class LinearHead:
    def __init__(self, spec, weights: dict, rt, embedding):
        self.rt = rt
        if spec.get("tied"):
            table = getattr(embedding, "table", None)
            if table is None:
                raise ConfigError("the head is tied to the embedding, but the embedding part has no table to share")
            weight = table
        else:
            weight = weights.pop(spec.tensors["weight"].name)
        self.linear = Linear(weight, rt)
        cap = spec.get("softcap")
        self.softcap = None if cap is None else float(cap)

    def libraries(self) -> set:
        return {"elementwise"} | self.linear.libraries()

    def forward(self, x) -> torch.Tensor:
        logits = self.linear(x, out_dtype=torch.float32, splits_ok=True)
        if logits.dim() == 3:       # split partials of the reduction
            parts, logits = logits, torch.empty(logits.shape[1:], dtype=torch.float32, device=x.device)
            kernels.sum_splits(parts, logits)
        if self.softcap is not None:
            kernels.softcap(logits, self.softcap)
        return logits
