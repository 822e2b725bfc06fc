"""Token embedding: h[t,:] = E[tok_t,:] widened to float32, times ``scale``
when the description gives one (the reference's dense Qwen3 path has none,
crates/model/src/qwen35/cpu.rs:129-136)."""

from __future__ import annotations

from .. import kernels
from .registry import register_embedding


@register_embedding("gather")
class GatherEmbedding:
    def __init__(self, spec, weights: dict, rt):
        self.table = weights[spec.tensors["table"].name]       # left in ``weights``: a tied head shares it
        scale = spec.get("scale")
        self.scale = 1.0 if scale is None else float(scale)

    def libraries(self) -> set:
        return {"elementwise"}

    def forward(self, tokens, h) -> None:
        kernels.embed(self.table, tokens, h, self.scale)
