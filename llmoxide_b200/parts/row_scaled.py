"""Normalised rows whose scale has not been applied yet.

For a step of few tokens (a decode step) the RMSNorm before a matrix product
is split in two: the norm writes ``x`` = bf16(h * gain) and partial sums of
squares of h (``sumsq``, one row per slice of columns), and the product
multiplies its output row t by r[t] = 1 / sqrt(sum(sumsq[:, t]) / d + eps) in
its epilogue, which is the same thing because a product is linear in its input
rows: rmsnorm(h) * gain = x * r row by row.  The first half then needs no CTA
to wait for another, so every SM takes part in it.

A part that declares ``takes_row_scales = True`` accepts a ``RowScaled`` where
it would get rows, and hands it to its first products.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch


@dataclass
class RowScaled:
    x: torch.Tensor          # [T, d] bfloat16: h * gain
    sumsq: torch.Tensor      # [parts, stride >= T] float32
    n_parts: int
    eps: float
    d: int

    @property
    def shape(self):
        return self.x.shape

    @property
    def dtype(self):
        return self.x.dtype

    @property
    def device(self):
        return self.x.device
