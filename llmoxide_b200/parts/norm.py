"""RMSNorm with a plain multiplicative gain: x / sqrt(mean(x^2) + eps) * g
(crates/model/src/ops.rs:40-59), fused with the residual add that precedes it."""

from __future__ import annotations

import torch

from .. import kernels
from .row_scaled import RowScaled
from .registry import register_norm


@register_norm("rms_norm")
class RMSNorm:
    def __init__(self, spec, weights: dict, rt):
        self.size, self.eps, self.rt = spec["size"], float(spec["eps"]), rt
        self.gain = weights[spec.tensors["gain"].name].to(torch.float32).contiguous()

    def libraries(self) -> set:
        return {"elementwise"}

    ROW_SCALE_MAX_TOKENS = 64      # what the products' epilogues take

    def add_forward(self, h, delta, rows=None, write_h=True, out_dtype=None, row_scales_ok=False):
        """With ``row_scales_ok`` the caller's next products apply the norm's scale themselves; for a step of
        few tokens the result is then ``RowScaled`` (the norm in two halves, see ``parts.row_scaled``)."""
        if (row_scales_ok and rows is None and write_h and out_dtype in (None, torch.bfloat16)
                and self.rt.act_dtype == torch.bfloat16 and h.shape[0] <= self.ROW_SCALE_MAX_TOKENS
                and self.size % 4 == 0):
            T = h.shape[0]
            parts = (self.size + kernels.ADD_SLICE - 1) // kernels.ADD_SLICE
            x = torch.empty((T, self.size), dtype=torch.bfloat16, device=h.device)
            sumsq = torch.empty((parts, max(T, 8)), dtype=torch.float32, device=h.device)
            kernels.add_gain_sumsq(h, delta, self.gain, x, sumsq)
            return RowScaled(x, sumsq, parts, self.eps, self.size)
        n = h.shape[0] if rows is None else rows.numel()
        out = torch.empty((n, self.size), dtype=out_dtype or self.rt.act_dtype, device=h.device)
        kernels.add_rms_norm(h, delta, self.gain, self.eps, out, rows=rows, write_h=write_h)
        return out
