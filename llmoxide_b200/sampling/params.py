"""Sampling options and the per-sequence random stream, with the reference's
names, meanings and defaults (crates/model/src/sample.rs:12-33,43-53,75-92)."""

from __future__ import annotations

from dataclasses import dataclass, replace

import numpy as np

_M64 = (1 << 64) - 1


@dataclass(frozen=True)
class Sampling:
    """temperature <= 0 is greedy.  top_k = 0 means no limit (whole
    vocabulary; needs top_p >= 1 on vocabularies above 1024).  repeat_penalty
    1.0 is off; it acts on the last ``repeat_window`` generated tokens."""

    temperature: float = 1.0
    top_k: int = 64
    top_p: float = 0.95
    repeat_penalty: float = 1.0
    repeat_window: int = 64
    seed: int = 0

    def is_greedy(self) -> bool:
        return self.temperature <= 0.0

    @classmethod
    def greedy(cls) -> "Sampling":
        return cls(temperature=0.0)

    def with_(self, **kw) -> "Sampling":
        return replace(self, **kw)


class Rng:
    """xorshift64*: state seed * 0x9E3779B97F4A7C15 | 1; a draw is the top 24
    bits of state * 0x2545F4914F6CDD1D as a float in [0, 1)."""

    def __init__(self, seed: int):
        self.state = ((int(seed) * 0x9E3779B97F4A7C15) & _M64) | 1

    def next_f32(self) -> float:
        x = self.state
        x ^= x >> 12
        x ^= (x << 25) & _M64
        x ^= x >> 27
        self.state = x
        return float(np.float32(((x * 0x2545F4914F6CDD1D) & _M64) >> 40) / np.float32(1 << 24))
