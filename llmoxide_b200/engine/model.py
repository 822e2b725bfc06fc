"""The decoder as data: blocks built from a ``ModelSpec`` through the part
registries, run in the order of the spec's schedule.  Nothing here names an
architecture.

Forward of one step, in the reference's order
(crates/model/src/qwen35/cpu.rs:129-136,138-400,406-416): the embedding part
fills the float32 residual stream; the scheduled layer calls run on it; the
final norm and the head part run on the wanted rows only (the reference takes
the last row, cpu.rs:410-414)."""

from __future__ import annotations

import torch

from .. import kernels
from ..cache import Cache
from ..config.spec import ModelSpec
from ..parts import Runtime, build_block
from ..parts.block import build_part
from ..parts.registry import EMBEDDINGS, HEADS, NORMS


class DecoderModel:
    def __init__(self, spec: ModelSpec, weights: dict, rt: Runtime):
        """``weights``: name -> device tensor; the parts take theirs out of it."""
        self.spec, self.rt = spec, rt
        self.embedding = build_part(EMBEDDINGS, "embedding", spec.embedding, weights, rt)
        self.blocks = [build_block(b, weights, rt) for b in spec.blocks]
        self.final_norm = build_part(NORMS, "norm", spec.final_norm, weights, rt)
        self.head = build_part(HEADS, "head", spec.head, weights, rt, self.embedding)
        for t in spec.embedding.tensors.values():       # the embedding left its tensors in for a tied head
            weights.pop(t.name, None)
        self._check_schedule()
        # A part that reads device data on the host during its forward (it says
        # so with ``graph_safe = False``) keeps decode steps out of CUDA graphs.
        self.graph_safe = (all(getattr(p, "graph_safe", True) for b in self.blocks for p in vars(b).values())
                           and all(getattr(p, "graph_safe", True) for p in (self.embedding, self.head, self.final_norm)))

    def _check_schedule(self):
        writers = {}
        for call in self.spec.schedule:
            if not (0 <= call.layer < len(self.blocks)):
                raise ValueError(f"the schedule names layer {call.layer}; there are {len(self.blocks)}")
            if call.writes_cache:
                writers.setdefault(call.cache, call.layer)
        for call in self.spec.schedule:
            if call.cache not in writers:
                raise ValueError(f"cache entry {call.cache} is read but no scheduled call writes it")
            if self.blocks[call.layer].cache_need() != self.blocks[writers[call.cache]].cache_need():
                raise ValueError(f"layer {call.layer} reads cache entry {call.cache} whose writer has other needs")
        self._writers = writers

    def libraries(self) -> set:
        """The CUDA libraries this model's parts say they launch (a part without ``libraries()`` says
        nothing, and its libraries are loaded at their first use)."""
        libs = {"elementwise"}
        for part in (self.embedding, self.head, self.final_norm):
            libs |= getattr(part, "libraries", set)()
        for b in self.blocks:
            libs |= getattr(b, "libraries", set)()
        return libs

    def cache_needs(self) -> list:
        """Per cache entry: (KVNeed | None, StateNeed | None), from the entry's writer."""
        n = self.spec.n_cache_entries()
        missing = [e for e in range(n) if e not in self._writers]
        if missing:
            raise ValueError(f"cache entries {missing} are never written")
        return [self.blocks[self._writers[e]].cache_need() for e in range(n)]

    def forward(self, ctx, cache: Cache) -> torch.Tensor:
        """float32 logits [n_want, vocab] at ``ctx.want_rows``."""
        d = self.spec.hidden_size
        h = torch.empty((ctx.n_tokens, d), dtype=torch.float32, device=self.rt.device)
        self.embedding.forward(ctx.tokens, h)
        probe = ctx.probe
        if probe:
            probe("model.input_embed", h)
        pending = None
        for i, call in enumerate(self.spec.schedule):
            if probe:
                # a block reports by stage; the stage of the residual stream entering call i is the output of call i-1
                ctx.probe = (lambda name, t, i=i: probe(f"{name}-{i}", t) if name != "resid_in"
                             else (probe(f"l_out-{i - 1}", t) if i else None))
            pending = self.blocks[call.layer].forward(h, pending, ctx, cache.view(call.cache), call.writes_cache)
        ctx.probe = probe
        if probe and pending is not None:
            kernels.add_rms_norm(h, pending, self.final_norm.gain, self.final_norm.eps, None)     # h += the last delta
            pending = None
            probe(f"l_out-{len(self.spec.schedule) - 1}", h)
        n_want = ctx.want_rows.numel()
        if n_want == 0:
            return torch.empty((0, self.spec.vocab_size), dtype=torch.float32, device=self.rt.device)
        x = self.final_norm.add_forward(h, pending, rows=ctx.want_rows, write_h=False)
        if probe:
            probe("result_norm", x)
        return self.head.forward(x)
