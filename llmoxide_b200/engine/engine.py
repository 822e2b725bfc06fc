"""The engine: a model, its cache and the one step function.

``step`` takes a batch of sequences that all start together (whole prompts of
unequal lengths) or all go on (one token each, or several), runs only the
tokens it is given as one batch, from the cache, and returns the logits at
the wanted places.  Limits are checked before anything is launched, as the
reference checks its forward (crates/gpu/src/qwen35.rs:1212-1222,
crates/model/src/qwen35/cpu.rs:119-125).
"""

from __future__ import annotations

import sys
import time
from dataclasses import dataclass
from pathlib import Path
from typing import Optional

import numpy as np
import torch

from .. import kernels
from ..cache import PAGE, Cache
from ..config import read_config
from ..errors import CacheExhausted, CacheMisuse, ContextOverflow
from ..parts import Runtime
from ..weights import load_checkpoint, random_tensors_on_device
from ..cache.allocator import _TOO_SMALL, host_library, raise_host_error
from .batch import N_FIXED, StepBuffers, flatten_entries, layout_from_meta
from .model import DecoderModel


@dataclass
class LoadOptions:
    """How a model is loaded (the reference sizes context and batch at load
    time too, llmoxide/src/backend.rs:112-139).

    ``max_tokens``: the most tokens live sequences hold at any time, each
    sequence's count rounded up to a multiple of 64; it sizes the cache.
    ``max_batch``: most sequences alive at once (slots).
    ``max_step_tokens``: most tokens one step may bring.
    ``overlap_prompt_kernels``: let the kernels of a prompt step start before the kernel before them has
    ended, as those of decode steps always do (off by default; the rule is stated in ``Engine._overlaps``).
    ``graph_prompt_tokens``: prompt steps of up to this many tokens are bound by their ~300 launches, not by
    the GPU; one whose shape comes back is captured as a CUDA graph like a decode step (0: never)."""

    dtype: str = "bfloat16"
    max_tokens: int = 16384
    max_batch: int = 256
    max_step_tokens: int = 16384
    device: str = "cuda:0"
    tensor_cores: bool = True
    cuda_graphs: bool = True
    overlap_prompt_kernels: bool = False
    graph_prompt_tokens: int = 1024


class Engine:
    def __init__(self, config, weights: dict, options: LoadOptions):
        kernels.require_gpu()
        self.config, self.options = config, options
        self.spec = config.to_spec()
        self.device = torch.device(options.device)
        torch.cuda.set_device(self.device)
        max_seq = min(self.spec.max_positions, (options.max_tokens + PAGE - 1) // PAGE * PAGE)
        self.rt = Runtime(dtype=options.dtype, device=self.device, max_positions=max_seq,
                          tensor_cores=options.tensor_cores)
        self.model = DecoderModel(self.spec, weights, self.rt)
        # Every library the model will launch is built and made resident now, while the GPU is idle: a step
        # never has to stop for one.
        kernels.preload(sorted(self.model.libraries()))
        n_slots = max(1, min(options.max_batch, (options.max_tokens + PAGE - 1) // PAGE))
        self.cache = Cache(self.model.cache_needs(), n_slots, options.max_tokens, self.rt.cache_dtype,
                           self.device, max_seq_len=max_seq)
        # The step buffer is sized for the largest step up front (up to a bound), because growing it
        # moves it, and a captured decode graph reads it at a fixed address.
        width = (max_seq // PAGE + 8) * max(1, self.cache.n_groups())
        want = 4 * min(options.max_step_tokens, options.max_tokens) + 4 * n_slots + min(n_slots, 256) * width + 64
        self.buffers = StepBuffers(self.device, capacity=max(1 << 14, min(want, 1 << 22)))
        self.n_steps = 0
        self.host_seconds = 0.0
        self._sampler = None
        self._graphs: dict = {}
        self._prompt_graphs: dict = {}
        self._prompt_shapes: dict = {}      # prompt-step shape -> times seen
        self._graph_pool = torch.cuda.graph_pool_handle() if options.cuda_graphs else None

    # ---- loading -------------------------------------------------------------

    @classmethod
    def load(cls, folder, options: Optional[LoadOptions] = None, **kw) -> "Engine":
        """From a model folder (config.json + model.safetensors); the model is
        chosen by config.json's architecture name."""
        options = options or LoadOptions(**kw)
        kernels.require_gpu()
        config = read_config(folder)
        weights = load_checkpoint(folder, config.to_spec(), options.dtype, options.device)
        return cls(config, weights, options)

    @classmethod
    def random(cls, config, seed: int = 0, options: Optional[LoadOptions] = None, **kw) -> "Engine":
        """Random weights made on the device (see ``weights.random_init``)."""
        options = options or LoadOptions(**kw)
        kernels.require_gpu()
        if not hasattr(config, "to_spec"):
            config = read_config(config)
        weights = random_tensors_on_device(config.to_spec(), seed, options.dtype, options.device)
        return cls(config, weights, options)

    # ---- slots -----------------------------------------------------------------

    def acquire(self) -> int:
        return self.cache.acquire()

    def release(self, slot: int) -> None:
        self.cache.release(slot)

    def length(self, slot: int) -> int:
        return self.cache.length(slot)

    # ---- the step --------------------------------------------------------------

    def step(self, entries, want=None, probe=None) -> torch.Tensor:
        """``entries``: [(slot, token ids)]; every sequence brings at least one
        token, appended at its current length.  ``want``: per entry the places
        among its tokens whose logits are asked for (default: the last).
        Returns float32 logits [wanted, vocab] on the device, in the order of
        the entries and of ``want``.  ``probe(name, tensor)`` is called with the
        step's named intermediates over its packed tokens (the reference traces
        the same stages, crates/model/src/qwen35/cpu.rs:136-415); such a step
        runs eagerly, with every norm as one kernel."""
        logits, replayed = self._step(entries, want, probe=probe)
        # A replayed graph writes its logits to the same memory every time.
        return logits.clone() if replayed else logits

    def _step(self, entries, want=None, feed_tokens=None, probe=None):
        t_host = time.perf_counter()
        try:
            return self._step_inner(entries, want, feed_tokens, probe)
        finally:
            # the host's own time in steps (checks, step buffer, launches; no waiting for the GPU except
            # where a launch queue is full)
            self.host_seconds += time.perf_counter() - t_host

    def _step_inner(self, entries, want=None, feed_tokens=None, probe=None):
        lay, ctx = self._prepare(entries, want)
        ctx.probe = probe
        if feed_tokens is not None:
            ctx.tokens.copy_(feed_tokens)      # on the stream, after the step buffer's copy
        try:
            logits, replayed = self._run(lay, ctx, entries, probe)
        except BaseException:
            # A step that fails after its pages were reserved (out of device memory for its activations, a
            # kernel's refusal) gives the reservation back: the sequences keep their lengths and stay usable.
            for slot, _ in entries:
                self.cache.alloc.unreserve(slot)
            raise
        self.cache.alloc.commit_many([slot for slot, _ in entries], [len(toks) for _, toks in entries])
        self.n_steps += 1
        return logits, replayed

    def _run(self, lay, ctx, entries, probe):
        graphs = bool(self.options.cuda_graphs and self.model.graph_safe and probe is None)
        replayed = graphs and (ctx.is_decode or self._prompt_shape_came_back(lay, ctx))
        if replayed and ctx.is_decode:
            logits = self._graphed_forward(lay, ctx, [slot for slot, _ in entries])
        elif replayed:
            logits = self._graphed_prompt(lay, ctx)
            replayed = logits is not None
            if not replayed:
                logits = self._forward(ctx)
        else:
            logits = self._forward(ctx)
        return logits, replayed

    def _overlaps(self, ctx) -> bool:
        """Rule: the kernels of a prompt step run fully ordered.  Long steps gain nothing measurable from
        overlapping a kernel's start with the end of the one before, and kernels that take whole SMs in pairs
        must not wait on one another for resources.  Steps of up to 128 tokens launch what a decode step
        launches and would gain a tenth; they stay ordered too, because the one unexplained wrong result of
        this engine's tests came while they overlapped."""
        return ctx.is_decode or self.options.overlap_prompt_kernels

    def _forward(self, ctx):
        if self._overlaps(ctx):
            return self.model.forward(ctx, self.cache)
        kernels.set_overlap(False)
        try:
            return self.model.forward(ctx, self.cache)
        finally:
            kernels.set_overlap(True)

    def _prompt_key(self, lay, ctx):
        # what the launches of a prompt step depend on besides the step buffer's contents
        return (lay.key(), ctx.max_new, ctx.max_len, self.buffers.dev.data_ptr())

    def _prompt_shape_came_back(self, lay, ctx) -> bool:
        """Whether this prompt step is short enough to be bound by its launches and has a shape that ran
        before (a capture costs about two steps, so a shape is captured when it is seen the second time)."""
        if ctx.n_tokens > self.options.graph_prompt_tokens:
            return False
        if lay.n_want * self.spec.vocab_size > (1 << 24):
            return False                 # a graph keeps its logits: not 64 MB and more per shape
        key = self._prompt_key(lay, ctx)
        seen = self._prompt_shapes.pop(key, 0) + 1
        if len(self._prompt_shapes) >= 1024:
            self._prompt_shapes.pop(next(iter(self._prompt_shapes)))
        self._prompt_shapes[key] = seen          # (most recently seen last)
        return seen >= 2

    def _graphed_prompt(self, lay, ctx):
        """The forward of a short prompt step as a replayed graph (of fully ordered kernels where the rule
        of ``_overlaps`` says so), or None if it cannot be captured.  The shape ran eagerly before (every library and kernel it needs is loaded), so
        nothing runs at capture and state of fixed size advances once, at the replay."""
        key = self._prompt_key(lay, ctx)
        entry = self._prompt_graphs.pop(key, None)
        if entry is None:
            torch.cuda.current_stream().synchronize()
            before = kernels.launch_count
            graph = torch.cuda.CUDAGraph()
            kernels.set_overlap(self._overlaps(ctx))
            try:
                with torch.cuda.graph(graph, pool=self._graph_pool):
                    logits = self.model.forward(ctx, self.cache)
            except RuntimeError as e:
                print(f"[llmoxide_b200] prompt steps are not captured as CUDA graphs: {e}", file=sys.stderr)
                self.options.graph_prompt_tokens = 0
                torch.cuda.synchronize()
                return None
            finally:
                kernels.set_overlap(True)
            entry = (graph, logits, kernels.launch_count - before)
            if len(self._prompt_graphs) >= 16:
                self._prompt_graphs.pop(next(iter(self._prompt_graphs)))
        self._prompt_graphs[key] = entry          # (most recently used last)
        graph, logits, n_kernels = entry
        graph.replay()
        kernels.launch_count += n_kernels
        return logits

    def _prepare(self, entries, want):
        """The step's plan, made by the C++ runtime (csrc/host_runtime.cpp, llmx_plan_step): every check that
        can refuse the step (slot validity, empty sequences, token ids, wanted places, the step limit), then
        the reservation of pages for every sequence (taken back if one does not fit), then the step buffer,
        packed straight into pinned memory."""
        if not entries:
            raise ValueError("a step needs at least one sequence")
        lib = host_library()
        alloc = self.cache.alloc
        n_groups = max(1, self.cache.n_groups())
        slots, counts, tokens, want_counts, want_flat = flatten_entries(entries, want)
        meta = np.zeros(8 + N_FIXED + 2 * n_groups, dtype=np.int64)
        ptr = lambda a: a.ctypes.data
        for attempt in range(2):
            host = self.buffers.next_host()
            code = lib.llmx_plan_step(alloc.handle, len(entries), ptr(slots), ptr(counts), ptr(tokens), ptr(want_counts),
                                      ptr(want_flat), self.spec.vocab_size, self.options.max_step_tokens, n_groups,
                                      host.data_ptr(), self.buffers.capacity, ptr(meta))
            if code == _TOO_SMALL and attempt == 0:
                self.buffers.grow(int(meta[3]))          # (a captured decode graph reads the buffer at a fixed
                continue                                 # address: its key holds the address, so it is captured anew)
            if code:
                raise_host_error(code)
            break
        lay, facts = layout_from_meta(meta)
        return lay, self.buffers.send(lay, facts)

    def _graphed_forward(self, lay, ctx, slots):
        """Decode steps are launch-bound, so the whole forward of a decode
        step is captured once per batch shape as a CUDA graph and replayed.
        The step's inputs live in the step buffer at offsets that depend on
        the shape alone, so a replay reads the new step's data.  The first
        occurrence of a shape runs eagerly once (libraries load, workspaces
        get their sizes), is then captured (which executes nothing) and
        replayed.  Running a step twice rewrites the same keys and values,
        which is harmless, but would advance per-sequence state of fixed
        size twice: the state rows of the step's slots are put back after
        the eager run."""
        key = (lay.key(), self.buffers.dev.data_ptr())
        entry = self._graphs.get(key)
        if entry is None:
            rows = torch.as_tensor(slots, dtype=torch.long, device=self.device)
            saved = [(st, st[rows].clone()) for st in self.cache.state_store if st is not None]
            self.model.forward(ctx, self.cache)            # warm-up: loads libraries, sizes workspaces
            for st, old_rows in saved:
                st[rows] = old_rows
            torch.cuda.current_stream().synchronize()
            before = kernels.launch_count
            graph = torch.cuda.CUDAGraph()
            try:
                with torch.cuda.graph(graph, pool=self._graph_pool):
                    logits = self.model.forward(ctx, self.cache)
            except RuntimeError as e:
                # A part that reads device data on the host cannot be captured:
                # from here on this engine runs every step eagerly.
                print(f"[llmoxide_b200] decode steps are not captured as CUDA graphs: {e}", file=sys.stderr)
                self.options.cuda_graphs = False
                torch.cuda.synchronize()
                return self.model.forward(ctx, self.cache)
            entry = (graph, logits, kernels.launch_count - before)
            if len(self._graphs) >= 64:
                self._graphs.pop(next(iter(self._graphs)))
            self._graphs[key] = entry
        graph, logits, n_kernels = entry
        graph.replay()
        kernels.launch_count += n_kernels
        return logits

    def step_sample(self, entries, samplings, recents, uniforms) -> list:
        """One step, then one token per entry from the logits at its last
        token, chosen on the device.  Returns the token ids as a host list."""
        return self.launch_step_sample(entries, samplings, recents, uniforms).tokens()

    def launch_step_sample(self, entries, samplings, recents, uniforms, feed=None):
        """The same without waiting: returns a handle whose ``tokens()`` waits
        for the result.  With ``feed`` (the handle of the step before, over the
        same sequences in the same order) every entry's single token is taken
        on the device from that step's result, so this step can be launched
        before the host has seen those tokens."""
        if self._sampler is None:
            from ..sampling.device import DeviceSampler
            self._sampler = DeviceSampler(self.device, self.spec.vocab_size)
        if feed is None:
            logits, _ = self._step(entries)
        else:
            if feed.n != len(entries) or any(len(t) != 1 for _, t in entries):
                raise ValueError("a fed step takes one token per sequence of the step before")
            logits, _ = self._step(entries, feed_tokens=feed.dev[: feed.n])
        return self._sampler.launch(logits, samplings, recents, uniforms)

    def check_status(self) -> None:
        """Raises ``KernelError`` if a kernel of an earlier step reported a failure (a bounded wait that ran
        out).  ``step`` returns without waiting for the GPU, so a caller asks once it has read the step's
        logits; the generation loop and trace replay do."""
        kernels.check_status()

    # ---- facts -------------------------------------------------------------------

    def info(self) -> dict:
        """What the reference's ``Info`` carries (llmoxide/src/backend.rs:36-49)."""
        return dict(architecture=self.spec.architecture, dtype=self.options.dtype, device=str(self.device),
                    vocab_size=self.spec.vocab_size, hidden_size=self.spec.hidden_size,
                    n_layers=len(self.spec.blocks), stop_ids=tuple(self.spec.stop_ids),
                    max_tokens=self.cache.n_pages * PAGE, max_batch=self.cache.n_slots,
                    max_seq_len=self.cache.alloc.max_seq_len, cache_bytes=self.cache.bytes(),
                    summary=self.config.summary() if hasattr(self.config, "summary") else "")
