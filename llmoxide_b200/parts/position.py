"""Position encodings.  ``rope_neox`` rotates pairs (i, i + n_rot/2) of the
first n_rot dims of a head by angle pos * base^(-2i/n_rot).  The angle is a
float64 recurrence theta_{i+1} = theta_i * base^(-2/n_rot) starting at pos,
and only sin/cos are rounded to float32, as the reference computes it
(crates/model/src/ops.rs:142-159, base held as float32).  ``none`` rotates
nothing."""

from __future__ import annotations

import numpy as np
import torch

from .registry import register_position


@register_position("rope_neox")
class RotaryNeox:
    def __init__(self, spec, weights: dict, rt):
        self.n_rot, self.base, self.rt = int(spec["n_rot"]), float(spec["base"]), rt
        self.factors = spec.get("factors")  # optional per-pair divisors of the angle
        if self.n_rot % 2:
            raise ValueError(f"n_rot {self.n_rot} must be even")
        self._tables = None
        self.rotary_tables()        # made when the model is built (tens of milliseconds), not in its first step

    def rotary_tables(self):
        if self._tables is None:
            half, n = self.n_rot // 2, self.rt.max_positions
            theta_scale = float(np.float32(self.base)) ** (-2.0 / self.n_rot)
            theta = np.arange(n, dtype=np.float64)
            cos = np.empty((n, half), dtype=np.float32)
            sin = np.empty((n, half), dtype=np.float32)
            for i in range(half):
                angle = theta if self.factors is None else theta / float(np.float32(self.factors[i]))
                cos[:, i] = np.cos(angle).astype(np.float32)
                sin[:, i] = np.sin(angle).astype(np.float32)
                theta = theta * theta_scale
            dev = self.rt.device
            self._tables = (torch.from_numpy(cos).to(dev), torch.from_numpy(sin).to(dev), self.n_rot)
        return self._tables


@register_position("none")
class NoPosition:
    def __init__(self, spec, weights: dict, rt):
        pass

    def rotary_tables(self):
        return None
