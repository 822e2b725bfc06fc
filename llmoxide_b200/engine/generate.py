"""The generation loop above the step function: batches of unequal prompts,
stop tokens, sequences that end earlier, and as many batches one after
another as there are requests.

For one sequence the loop is the reference's (llmoxide/src/session.rs:573-611):
``max_new = min(max_tokens, context - prompt)``; sample from the prompt's last
logits; a stop token is recorded, not fed back, and ends the sequence with
reason ``stop``; otherwise the token is recorded, the caller's callback may
cancel, and the token is fed back for the next logits; falling out of the
loop leaves reason ``length``.  Batching is this library's own: all prompts of
a batch run in one step, then the live sequences decode one token each; a
sequence that ends gives its slot back at once and the others go on in a
smaller batch.

The decisions live here without any tensor, so they are tested on the CPU
with a scripted backend.  A backend offers ``acquire() -> slot``,
``release(slot)`` and ``step_sample(entries, samplings, recents, uniforms) ->
[token]`` (run one step, sample one token per entry from its last logits).
"""

from __future__ import annotations

import time
from dataclasses import dataclass, field
from typing import Callable, Optional, Sequence

from ..cache.allocator import PAGE
from ..errors import CacheExhausted, ContextOverflow
from ..sampling.params import Rng, Sampling

STOP, LENGTH, CANCELLED = "stop", "length", "cancelled"


@dataclass
class Request:
    """What to generate (token ids in; the reference's Request carries
    messages, llmoxide/src/session.rs:83-112, whose text layer is not built)."""

    prompt: Sequence[int]
    max_tokens: int = 512
    sampling: Optional[Sampling] = None     # None: the model's recommended settings
    stop_ids: Sequence[int] = ()            # extra stop tokens beside the model's own


@dataclass
class Outcome:
    """llmoxide/src/session.rs:179-186, without the text fields."""

    tokens: list
    reason: str
    prompt_tokens: int
    generated: int
    cached_tokens: int = 0


@dataclass
class Limits:
    max_batch: int
    max_tokens: int          # page budget of the cache, in tokens
    max_step_tokens: int
    max_seq_len: int


@dataclass
class Timings:
    prefill_tokens: int = 0
    prefill_seconds: float = 0.0
    decode_tokens: int = 0
    decode_seconds: float = 0.0
    steps: int = 0


def max_new_tokens(prompt_len: int, max_tokens: int, limits: Limits) -> int:
    """The last sampled token is never fed back, so a sequence uses
    prompt + new - 1 positions."""
    if prompt_len == 0:
        raise ValueError("a request needs at least one prompt token")
    if prompt_len >= limits.max_seq_len:
        raise ContextOverflow(prompt_len, limits.max_seq_len)
    return max(0, min(max_tokens, limits.max_seq_len - prompt_len))


def _pages(n_tokens: int) -> int:
    return (n_tokens + PAGE - 1) // PAGE


def plan_batches(prompt_lens, new_lens, limits: Limits) -> list:
    """Requests in arrival order, cut into batches that start together: at
    most max_batch sequences whose pages at their final lengths fit the cache.
    Prompts that do not fit one step together are fed in several steps (each
    sequence's tokens in order), after which the whole batch decodes together:
    the step limit bounds a step, not the width of a batch.  A request too
    large for the cache alone still gets a batch of its own (the cache then
    refuses it)."""
    batches, cur, pages = [], [], 0
    budget = _pages(limits.max_tokens)
    for i, (p, n) in enumerate(zip(prompt_lens, new_lens)):
        need = _pages(p + max(0, n - 1))
        if cur and (len(cur) >= limits.max_batch or pages + need > budget):
            batches.append(cur)
            cur, pages = [], 0
        cur.append(i)
        pages += need
    if cur:
        batches.append(cur)
    return batches


class _Done:
    """A finished step in the shape of a handle (for backends that only step synchronously)."""

    def __init__(self, tokens):
        self._tokens = tokens

    def tokens(self):
        return self._tokens


class _Live:
    __slots__ = ("index", "slot", "sampling", "rng", "stops", "max_new", "out", "next_token")

    def __init__(self, index, slot, sampling, stops, max_new):
        self.index, self.slot, self.sampling, self.stops, self.max_new = index, slot, sampling, stops, max_new
        self.rng = Rng(sampling.seed)
        self.out: list = []
        self.next_token = None


class GenerationLoop:
    def __init__(self, backend, limits: Limits, default_sampling: Sampling, stop_ids=()):
        self.backend, self.limits = backend, limits
        self.default_sampling, self.stop_ids = default_sampling, frozenset(stop_ids)
        self.timings = Timings()

    def run(self, requests: Sequence[Request], on_token: Optional[Callable] = None) -> list:
        """Outcomes in the order of ``requests``.  ``on_token(index, token)``
        is called for every generated token that is not a stop token; a false
        return value cancels that sequence."""
        prompt_lens = [len(r.prompt) for r in requests]
        new_lens = [max_new_tokens(p, r.max_tokens, self.limits) for p, r in zip(prompt_lens, requests)]
        outcomes: list = [None] * len(requests)
        for batch in plan_batches(prompt_lens, new_lens, self.limits):
            self._run_batch(batch, requests, new_lens, outcomes, on_token)
        return outcomes

    # -----------------------------------------------------------------------

    def _run_batch(self, batch, requests, new_lens, outcomes, on_token):
        live = []
        for i in batch:
            r = requests[i]
            if new_lens[i] == 0:
                outcomes[i] = Outcome([], LENGTH, len(r.prompt), 0)
                continue
            sampling = r.sampling or self.default_sampling
            live.append(_Live(i, None, sampling, self.stop_ids | frozenset(r.stop_ids), new_lens[i]))
        if not live:
            return
        try:
            for s in live:
                s.slot = self.backend.acquire()
            t0 = time.perf_counter()
            self._prompt_steps(live, requests)
            self.timings.prefill_seconds += time.perf_counter() - t0
            self.timings.prefill_tokens += sum(len(requests[s.index].prompt) for s in live)
            t0 = time.perf_counter()
            live = self._decode(live, requests, outcomes, on_token)
            self.timings.decode_seconds += time.perf_counter() - t0
        finally:
            for s in live:
                if s.slot is not None and outcomes[s.index] is None:
                    self.backend.release(s.slot)
                    s.slot = None

    def _prompt_steps(self, live, requests):
        """All prompts in one step when they fit the step limit; otherwise
        in as many steps as needed, each sequence's tokens in order (the
        reference feeds long prompts in chunks, llmoxide/src/session.rs:636-656).
        Only the step that brings a prompt's last token is sampled from."""
        cap = self.limits.max_step_tokens
        fed = {s.index: 0 for s in live}
        while True:
            room, entries, finals = cap, [], []
            for s in live:
                prompt = requests[s.index].prompt
                left = len(prompt) - fed[s.index]
                if left == 0 or room == 0:
                    continue
                n = min(left, room)
                entries.append((s, list(prompt[fed[s.index] : fed[s.index] + n])))
                fed[s.index] += n
                room -= n
                finals.append(fed[s.index] == len(prompt))
            if not entries:
                return
            self._sample_step([s for (s, _), f in zip(entries, finals)], [(s.slot, t) for s, t in entries],
                              sampled=finals)

    def _sample_step(self, seqs, entries, sampled=None):
        samplings = [s.sampling for s in seqs]
        recents = [s.out for s in seqs]
        sampled = sampled or [True] * len(seqs)
        # A draw is taken only for a row that samples, so a sequence's random
        # stream does not depend on how its prompt was cut or batched.
        uniforms = [s.rng.next_f32() if (f and not s.sampling.is_greedy()) else 0.0 for s, f in zip(seqs, sampled)]
        tokens = self.backend.step_sample(entries, samplings, recents, uniforms)
        self.timings.steps += 1
        for s, tok, f in zip(seqs, tokens, sampled):
            s.next_token = int(tok) if f else None

    # ---- decoding, one step ahead ------------------------------------------

    def _launch(self, seqs, feed=None):
        """Starts a decode step for ``seqs`` (each brings its ``next_token``, or,
        with ``feed``, the token the step before is still computing)."""
        entries = [(s.slot, [0 if feed is not None else s.next_token]) for s in seqs]
        # A launch that the backend refuses (no room for a token that may not be needed) must leave every
        # sequence's random stream where it was: the draws are taken back, so that a sequence's tokens do
        # not depend on how full the cache was.
        states = [s.rng.state for s in seqs]
        uniforms = [0.0 if s.sampling.is_greedy() else s.rng.next_f32() for s in seqs]
        args = (entries, [s.sampling for s in seqs], [s.out for s in seqs], uniforms)
        try:
            if hasattr(self.backend, "launch_step_sample"):
                handle = self.backend.launch_step_sample(*args, feed=feed)
            else:
                handle = _Done(self.backend.step_sample(*args))
        except BaseException:
            for s, state in zip(seqs, states):
                s.rng.state = state
            raise
        self.timings.steps += 1
        self.timings.decode_tokens += len(seqs)
        return handle

    def _can_run_ahead(self, seqs) -> bool:
        """A second step may be launched before the first one's tokens are known
        when its inputs do not need them on the host: no repetition penalty
        (which reads the tokens), and no sequence that the first step's token
        ends by length.  A sequence that the first step ends by a stop token is
        only known afterwards; its share of the second step is thrown away."""
        if not hasattr(self.backend, "launch_step_sample"):
            return False
        return all(s.sampling.repeat_penalty == 1.0 and len(s.out) + 1 < s.max_new for s in seqs)

    def _decode(self, live, requests, outcomes, on_token):
        """The decode loop.  Every live sequence holds a ``next_token`` that is
        not yet recorded.  Returns the sequences still live (none, normally)."""
        live = self._settle(live, requests, outcomes, on_token)
        if not live:
            return live
        step = self._launch(live)
        while True:
            ahead = None
            if self._can_run_ahead(live):
                try:
                    ahead = self._launch(live, feed=step)
                except (ContextOverflow, CacheExhausted):
                    ahead = None                    # no room for a token that may not be needed: do not run ahead
            for s, tok in zip(live, step.tokens()):
                s.next_token = int(tok)
            before = live
            live = self._settle(before, requests, outcomes, on_token)
            if not live:
                return live
            if ahead is not None and len(live) < len(before):
                # Some sequence ended on the first step's token.  The second step already ran with it in
                # the batch; the other sequences' tokens are right all the same (a sequence's result does
                # not depend on its neighbours), so they are kept and the batch goes on without it.
                place = {id(s): i for i, s in enumerate(before)}
                toks = ahead.tokens()
                for s in live:
                    s.next_token = int(toks[place[id(s)]])
                live = self._settle(live, requests, outcomes, on_token)
                if not live:
                    return live
                ahead = None
            step = ahead if ahead is not None else self._launch(live)

    def _settle(self, live, requests, outcomes, on_token):
        """Records each sequence's new token and decides who goes on."""
        still = []
        for s in live:
            tok = s.next_token
            reason = None
            s.out.append(tok)
            if tok in s.stops:
                reason = STOP
            else:
                if on_token is not None and on_token(s.index, tok) is False:
                    reason = CANCELLED
                elif len(s.out) >= s.max_new:
                    reason = LENGTH
            if reason is None:
                still.append(s)
            else:
                outcomes[s.index] = Outcome(s.out, reason, len(requests[s.index].prompt), len(s.out))
                self.backend.release(s.slot)
                s.slot = None
        return still
