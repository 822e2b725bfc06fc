"""Runs the sampling kernels over a step's logits.  Per-row parameters travel
in one small pinned buffer; a batch in which every row is greedy and
unpenalised takes the argmax kernel alone.  A launch returns at once with a
handle; the host reads the tokens when it needs them, so the next step can
already be running (the generation loop launches one step ahead)."""

from __future__ import annotations

import os
import time

import numpy as np
import torch

from .. import kernels
from ..errors import KernelError, Unsupported
from ..guard import guarded

# How long the host waits for a step's tokens before it gives up with an error instead of waiting for ever.
STEP_TIMEOUT_S = float(os.environ.get("LLMX_STEP_TIMEOUT_S", "120"))

MAX_TOP_K = 1024  # SMP_MAX_K in sampling.cu
RING = 3          # launches whose results may be unread at the same time


class SampledTokens:
    """The tokens of one launch: on the device at once, on the host after
    ``tokens()`` has waited for the copy."""

    def __init__(self, dev, host, event, n):
        self.dev, self._host, self._event, self.n = dev, host, event, n

    def tokens(self) -> list:
        """Waits for the launch (polling, so that a step that never ends becomes an error, not a silent
        hang) and returns its tokens."""
        if not self._event.query():
            start = time.monotonic()
            while not self._event.query():
                waited = time.monotonic() - start
                if waited > STEP_TIMEOUT_S:
                    raise KernelError(
                        f"a step did not finish within {STEP_TIMEOUT_S:.0f} s (LLMX_STEP_TIMEOUT_S): a kernel "
                        f"waits for something that does not come, or the GPU is lost")
                if waited > 0.05:
                    time.sleep(0.001)          # a long step (a prompt): stop spinning
        kernels.check_status()      # a kernel of the step may have reported that a bounded wait ran out
        return self._host[: self.n].tolist()


class DeviceSampler:
    def __init__(self, device, vocab_size: int, max_rows: int = 64):
        self.device, self.vocab = device, vocab_size
        kernels.preload(["sampling"])      # before the step whose logits it will read is launched
        self._cap = 0
        self._turn = 0
        self._grow(max_rows)
        # what a sampling kernel cannot do is reported in the library's word, which the host reads with the tokens
        self.status = kernels.status_word("sampling")

    def _grow(self, rows: int, width: int = 64):
        torch.cuda.current_stream().synchronize()      # nothing in flight may still use the old buffers
        self._cap, self._width = rows, width
        n = rows * (5 + width)
        self._params_host = [torch.empty(n, dtype=torch.int32).pin_memory() for _ in range(RING)]
        self._params_dev = [guarded((n,), torch.int32, self.device, f"sampler parameters {i}") for i in range(RING)]
        self._tokens_dev = [guarded((rows,), torch.int32, self.device, f"sampled tokens {i}") for i in range(RING)]
        self._tokens_host = [torch.empty(rows, dtype=torch.int32).pin_memory() for _ in range(RING)]
        self._events = [None] * RING

    def check(self, s) -> None:
        if s.is_greedy():
            return
        if s.top_k < 0 or (MAX_TOP_K < s.top_k < self.vocab):
            raise Unsupported(f"top_k {s.top_k}: the sampling kernel sorts up to {MAX_TOP_K} candidates; "
                              f"use 0 for no limit")
        if (s.top_k == 0 or s.top_k >= self.vocab) and s.top_p < 1.0 and self.vocab > MAX_TOP_K:
            raise Unsupported("top_p < 1 needs top_k <= 1024 on this vocabulary")

    def launch(self, logits: torch.Tensor, params: list, recents: list, uniforms: list) -> SampledTokens:
        """One token per row.  ``params[i]`` is row i's Sampling, ``recents[i]``
        its generated tokens so far, ``uniforms[i]`` its draw in [0, 1)."""
        n = logits.shape[0]
        assert n == len(params) == len(recents) == len(uniforms)
        penalised = any(p.repeat_penalty != 1.0 for p in params)
        width = max(1, max(min(p.repeat_window, len(r)) for p, r in zip(params, recents))) if penalised else 1
        if n > self._cap or width > self._width:
            self._grow(max(n, 2 * self._cap if n > self._cap else self._cap), max(width, self._width))
        i = self._turn
        self._turn = (i + 1) % RING
        if self._events[i] is not None:
            self._events[i].synchronize()              # the slot's last launch has been read back
        out = self._tokens_dev[i]
        if all(p.is_greedy() for p in params) and not penalised:
            kernels.argmax(logits, out[:n])
        else:
            for p in params:
                self.check(p)
            W = self._width
            host = self._params_host[i].numpy()
            f = host.view(np.float32)
            for r, (p, rec, u) in enumerate(zip(params, recents, uniforms)):
                f[r] = p.temperature
                host[n + r] = p.top_k if p.top_k < self.vocab else 0
                f[2 * n + r] = p.top_p
                f[3 * n + r] = p.repeat_penalty
                f[4 * n + r] = u
                row = host[5 * n + r * W : 5 * n + (r + 1) * W]
                row[:] = -1
                tail = rec[max(0, len(rec) - p.repeat_window):] if p.repeat_penalty != 1.0 else []
                row[: len(tail)] = tail
            total = n * (5 + W)
            d = self._params_dev[i]
            d[:total].copy_(self._params_host[i][:total], non_blocking=True)
            fl = d.view(torch.float32)
            kernels.sample(logits, fl[0:n], d[n : 2 * n], fl[2 * n : 3 * n], fl[3 * n : 4 * n],
                           d[5 * n : 5 * n + n * W].view(n, W), fl[4 * n : 5 * n], out[:n], self.status)
        self._tokens_host[i][:n].copy_(out[:n], non_blocking=True)
        ev = torch.cuda.Event()
        ev.record()
        self._events[i] = ev
        return SampledTokens(out, self._tokens_host[i], ev, n)

    def sample(self, logits, params, recents, uniforms) -> list:
        return self.launch(logits, params, recents, uniforms).tokens()
