"""The library entry point, in the manner of the reference's facade
(llmoxide/src/session.rs:338-364,434-446; llmoxide/src/backend.rs:62-105):
``Session.load(folder, LoadOptions)`` or ``Session.random(config, seed)``,
then ``generate(requests)`` / ``complete(request)`` for token ids in and out,
``forward(tokens)`` for raw logits of one sequence, ``info()`` and ``wipe()``.
"""

from __future__ import annotations

from typing import Callable, Optional, Sequence

import torch

from . import kernels
from .engine.engine import Engine, LoadOptions
from .engine.generate import GenerationLoop, Limits, Outcome, Request
from .sampling.params import Sampling


class Session:
    def __init__(self, engine: Engine):
        self.engine = engine
        info = engine.info()
        self.limits = Limits(max_batch=info["max_batch"], max_tokens=info["max_tokens"],
                             max_step_tokens=engine.options.max_step_tokens, max_seq_len=info["max_seq_len"])
        self.default_sampling = Sampling(**engine.spec.default_sampling)
        self.loop = GenerationLoop(engine, self.limits, self.default_sampling, engine.spec.stop_ids)
        self._resident: Optional[int] = None   # slot of the sequence that forward() extends
        # A session generates, so it samples: the sampling kernels are built and loaded now, not in the middle of
        # the first request (trace replay, which samples nothing, drives the engine without a session).
        if engine.device.type == "cuda":
            kernels.preload(["sampling"])

    # ---- loading ---------------------------------------------------------------

    @classmethod
    def load(cls, folder, options: Optional[LoadOptions] = None, **kw) -> "Session":
        return cls(Engine.load(folder, options, **kw))

    @classmethod
    def random(cls, config, seed: int = 0, options: Optional[LoadOptions] = None, **kw) -> "Session":
        return cls(Engine.random(config, seed, options, **kw))

    # ---- generation --------------------------------------------------------------

    def generate(self, requests: Sequence, on_token: Optional[Callable] = None) -> list:
        """``requests``: Requests, or plain token-id lists (which then take the
        defaults).  Returns one Outcome per request, in order."""
        reqs = [r if isinstance(r, Request) else Request(prompt=list(r)) for r in requests]
        return self.loop.run(reqs, on_token)

    def complete(self, request, on_token: Optional[Callable] = None) -> Outcome:
        cb = None if on_token is None else (lambda _i, tok: on_token(tok))
        return self.generate([request], cb)[0]

    # ---- raw logits ------------------------------------------------------------------

    def forward(self, tokens: Sequence[int]) -> torch.Tensor:
        """Appends ``tokens`` to the resident sequence and returns the float32
        logits at the last one, as the reference's Backend::forward does
        (llmoxide/src/backend.rs:62-76).  ``wipe()`` starts a new sequence."""
        if self._resident is None:
            self._resident = self.engine.acquire()
        return self.engine.step([(self._resident, list(tokens))])[0]

    def wipe(self) -> None:
        """Forgets the resident sequence and overwrites the whole cache."""
        if self._resident is not None:
            self.engine.release(self._resident)
            self._resident = None
        self.engine.cache.wipe()

    def info(self) -> dict:
        return self.engine.info()

    @property
    def timings(self):
        return self.loop.timings
