"""Runs the sampling kernels over a step's logits.  Per-row parameters travel
in one small pinned buffer; a batch in which every row is greedy and
unpenalised takes the argmax kernel alone."""

from __future__ import annotations

import numpy as np
import torch

from .. import kernels
from ..errors import Unsupported

MAX_TOP_K = 1024  # SMP_MAX_K in sampling.cu


class DeviceSampler:
    def __init__(self, device, vocab_size: int, max_rows: int = 64):
        self.device, self.vocab = device, vocab_size
        self._cap = 0
        self._grow(max_rows)
        self.status = torch.zeros(1, dtype=torch.int32, device=device)

    def _grow(self, rows: int, width: int = 64):
        self._cap, self._width = rows, width
        n = rows * (5 + width)
        self._host = torch.empty(n, dtype=torch.int32).pin_memory()
        self._dev = torch.empty(n, dtype=torch.int32, device=self.device)
        self.tokens = torch.empty(rows, dtype=torch.int32, device=self.device)
        self.tokens_host = torch.empty(rows, dtype=torch.int32).pin_memory()

    def check(self, s) -> None:
        if s.is_greedy():
            return
        if s.top_k < 0 or s.top_k > MAX_TOP_K and s.top_k < self.vocab:
            raise Unsupported(f"top_k {s.top_k}: the sampling kernel sorts up to {MAX_TOP_K} candidates; "
                              f"use 0 for no limit")
        if (s.top_k == 0 or s.top_k >= self.vocab) and s.top_p < 1.0 and self.vocab > MAX_TOP_K:
            raise Unsupported("top_p < 1 needs top_k <= 1024 on this vocabulary")

    def sample(self, logits: torch.Tensor, params: list, recents: list, uniforms: list) -> list:
        """One token per row.  ``params[i]`` is row i's Sampling, ``recents[i]``
        its generated tokens so far, ``uniforms[i]`` its draw in [0, 1)."""
        n = logits.shape[0]
        assert n == len(params) == len(recents) == len(uniforms)
        if all(p.is_greedy() and p.repeat_penalty == 1.0 for p in params):
            if n > self._cap:
                self._grow(max(n, 2 * self._cap), self._width)
            kernels.argmax(logits, self.tokens[:n])
        else:
            width = max(1, max(min(p.repeat_window, len(r)) for p, r in zip(params, recents)))
            if n > self._cap or width > self._width:
                self._grow(max(n, self._cap), max(width, self._width))
            W = self._width
            host = self._host.numpy()
            f = host.view(np.float32)
            for i, (p, r, u) in enumerate(zip(params, recents, uniforms)):
                f[i] = p.temperature
                host[n + i] = p.top_k if p.top_k < self.vocab else 0
                f[2 * n + i] = p.top_p
                f[3 * n + i] = p.repeat_penalty
                f[4 * n + i] = u
                row = host[5 * n + i * W : 5 * n + (i + 1) * W]
                row[:] = -1
                tail = r[max(0, len(r) - p.repeat_window):] if p.repeat_penalty != 1.0 else []
                row[: len(tail)] = tail
            total = n * (5 + W)
            self._dev[:total].copy_(self._host[:total], non_blocking=True)
            d = self._dev
            fl = d.view(torch.float32)
            kernels.sample(logits, fl[0:n], d[n : 2 * n], fl[2 * n : 3 * n], fl[3 * n : 4 * n],
                           d[5 * n : 5 * n + n * W].view(n, W), fl[4 * n : 5 * n], self.tokens[:n], self.status)
        self.tokens_host[:n].copy_(self.tokens[:n], non_blocking=True)
        torch.cuda.current_stream().synchronize()
        return self.tokens_host[:n].tolist()
