"""Gated feed-forward: down(act(gate x) * (up x)), act = SiLU x/(1+exp(-x))
(crates/model/src/qwen35/cpu.rs:386-395, crates/model/src/ops.rs:176-178).
Gate and up are one matrix product over the rows [gate; up]."""

from __future__ import annotations

import torch

from .. import kernels
from ..errors import Unsupported
from .row_scaled import RowScaled
from .linear import Linear
from .registry import register_feed_forward


import os

# Above this many tokens the gate/up product applies the activation in its epilogue (no split of its
# reduction); at or below it the reduction is split and the activation sums the partials.  Measured at
# Qwen3-8B layer sizes the fused form is as fast or faster at every batch size, so it is the default.
FUSE_MIN_TOKENS = int(os.environ.get("LLMX_FUSE_MIN_TOKENS", "0"))


@register_feed_forward("gated_mlp")
class GatedMLP:
    def __init__(self, spec, weights: dict, rt):
        if spec.get("activation", "silu") != "silu":
            raise Unsupported(f"gated_mlp activation {spec.get('activation')!r}: only 'silu' is built")
        self.rt, self.F = rt, spec["intermediate_size"]
        t = spec.tensors
        wg, wu = weights.pop(t["gate"].name), weights.pop(t["up"].name)
        if wg.dtype != wu.dtype:
            wg, wu = wg.float(), wu.float()
        # One matrix for gate and up.  Where the width allows, rows go in blocks of 16 gate rows each
        # followed by the 16 up rows of the same features: a warp of the matrix product's epilogue (32 rows of
        # a tile) then holds both halves of 16 features, and the activation is one shuffle away.  Otherwise
        # gate rows, then up rows.
        self.block = 16 if self.F % 16 == 0 else 0
        if self.block:
            k = wg.shape[1]
            fused = torch.stack([wg.view(-1, 16, k), wu.view(-1, 16, k)], dim=1).reshape(2 * self.F, k)
        else:
            fused = torch.cat([wg, wu], dim=0)
        del wg, wu
        self.gate_up = Linear(fused, rt)
        del fused
        self.down = Linear(weights.pop(t["down"].name), rt)

    def libraries(self) -> set:
        return {"elementwise"} | self.gate_up.libraries() | self.down.libraries()

    @property
    def takes_row_scales(self) -> bool:
        """The gate|up product can apply a norm's row scales in its epilogue, ahead of the activation."""
        return self.gate_up._tc is not None

    adds_to_residual = True      # forward() takes ``residual`` and may return None: "already added"

    def forward(self, x, ctx, residual=None):
        tc = self.gate_up._tc
        scaled = isinstance(x, RowScaled)
        n_tokens = x.shape[0]
        if tc is not None and x.dtype == torch.bfloat16 and n_tokens > FUSE_MIN_TOKENS and (
                scaled or kernels.gemm_tc_supports(x, tc.weight)):
            # the activation is the epilogue of the gate/up product
            act = tc.gated(x, self.rt.act_dtype, self.block)
        else:
            assert not scaled
            gu = self.gate_up(x, splits_ok=True)
            act = torch.empty((n_tokens, self.F), dtype=self.rt.act_dtype, device=x.device)
            kernels.silu_gate(gu, act, self.block)
        if residual is not None and self.down.add_into(act, residual):
            return None
        return self.down(act, splits_ok=True)
