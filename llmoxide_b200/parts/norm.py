"""RMSNorm with a plain multiplicative gain: x / sqrt(mean(x^2) + eps) * g
(crates/model/src/ops.rs:40-59), fused with the residual add that precedes it."""

from __future__ import annotations

import torch

from .. import kernels
from .registry import register_norm


@register_norm("rms_norm")
class RMSNorm:
    def __init__(self, spec, weights: dict, rt):
        self.size, self.eps, self.rt = spec["size"], float(spec["eps"]), rt
        self.gain = weights[spec.tensors["gain"].name].to(torch.float32).contiguous()

    def libraries(self) -> set:
        return {"elementwise"}

    def add_forward(self, h, delta, rows=None, write_h=True, out_dtype=None):
        n = h.shape[0] if rows is None else rows.numel()
        out = torch.empty((n, self.size), dtype=out_dtype or self.rt.act_dtype, device=h.device)
        kernels.add_rms_norm(h, delta, self.gain, self.eps, out, rows=rows, write_h=write_h)
        return out
