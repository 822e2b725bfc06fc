"""CPU tests: the cache's bookkeeping (no slot or page lost, held twice or
freed twice; windows give pages back) and the generation loop's decisions
with a scripted backend."""

import random

import pytest

from llmoxide_b200.cache import PAGE, CacheAllocator, pages_for
from llmoxide_b200.engine.generate import (CANCELLED, LENGTH, STOP, GenerationLoop, Limits, Request,
                                           max_new_tokens, plan_batches)
from llmoxide_b200.errors import CacheExhausted, CacheMisuse, ContextOverflow
from llmoxide_b200.sampling import Rng, Sampling

import plain_qwen3 as plain


# ---- cache ----------------------------------------------------------------------

def test_slots_are_given_back_and_used_again():
    a = CacheAllocator(n_slots=2, n_pages=4, windows=[None])
    s0, s1 = a.acquire(), a.acquire()
    assert {s0, s1} == {0, 1}
    with pytest.raises(CacheExhausted):
        a.acquire()
    a.reserve(s0, 70), a.commit(s0, 70)
    assert a.length(s0) == 70 and len(a.page_row(s0, 0)) == 2
    a.release(s0)
    s2 = a.acquire()
    assert s2 == s0 and a.length(s2) == 0 and a.page_row(s2, 0) == []
    a.check_consistent()


def test_double_free_and_use_after_free_are_errors():
    a = CacheAllocator(2, 4, [None])
    s = a.acquire()
    a.release(s)
    with pytest.raises(CacheMisuse):
        a.release(s)
    with pytest.raises(CacheMisuse):
        a.reserve(s, 1)
    with pytest.raises(CacheMisuse):
        a.length(5)
    s = a.acquire()
    a.reserve(s, 3)
    with pytest.raises(CacheMisuse):
        a.commit(s, 4)          # more than was reserved


def test_pages_run_out_without_changing_anything():
    a = CacheAllocator(2, 3, [None, 16])
    s0, s1 = a.acquire(), a.acquire()
    a.reserve(s0, 2 * PAGE), a.commit(s0, 2 * PAGE)
    with pytest.raises(CacheExhausted):
        a.reserve(s1, PAGE + 1)
    assert a.page_row(s1, 0) == [] and a.page_row(s1, 1) == []
    a.check_consistent()
    a.reserve(s1, PAGE)
    a.check_consistent()


def test_longest_sequence_is_enforced():
    a = CacheAllocator(1, 8, [None], max_seq_len=100)
    s = a.acquire()
    a.reserve(s, 100), a.commit(s, 100)
    with pytest.raises(ContextOverflow):
        a.reserve(s, 1)


def test_window_group_gives_dead_pages_back():
    w = 24
    a = CacheAllocator(1, 8, [None, w])
    s = a.acquire()
    a.reserve(s, 150), a.commit(s, 150)
    # next query at 150 sees keys from 127 on: pages 0 (0..63) is dead, page 1 (64..127) holds 127
    assert a.page_row(s, 0) == [0, 1, 2]
    assert a.page_row(s, 1)[0] == -1 and a.page_row(s, 1)[1] >= 0
    assert a.pages_held(1) == 2
    for _ in range(42):          # up to length 192: first visible 169 -> pages 0, 1 dead
        a.reserve(s, 1), a.commit(s, 1)
    assert a.page_row(s, 1)[:2] == [-1, -1] and a.pages_held(1) == 1
    a.check_consistent()
    a.release(s)
    assert a.pages_held(0) == 0 and a.pages_held(1) == 0


def test_random_traffic_never_loses_or_doubles_a_page():
    rng = random.Random(3)
    a = CacheAllocator(6, 40, [None, 50])
    live = {}
    for _ in range(3000):
        op = rng.random()
        if op < 0.15 and a.n_free_slots:
            live[a.acquire()] = 0
        elif op < 0.25 and live:
            s = rng.choice(list(live))
            a.release(s)
            del live[s]
        elif live:
            s = rng.choice(list(live))
            n = rng.choice([1, 1, 1, 7, 64, 130])
            try:
                a.reserve(s, n)
            except (CacheExhausted, ContextOverflow):
                continue
            a.commit(s, n)
            live[s] += n
            assert a.length(s) == live[s]
        a.check_consistent()
    for s in list(live):
        a.release(s)
    a.check_consistent()
    assert a.pages_held(0) == 0 and a.pages_held(1) == 0 and a.n_free_slots == 6


# ---- the generation loop ------------------------------------------------------------

class ScriptedBackend:
    """Answers each sequence with its own scripted tokens and records every
    step; checks that slots are acquired, used and released consistently."""

    def __init__(self, scripts, n_slots):
        self.scripts, self.n_slots = scripts, n_slots       # first prompt token -> list of tokens to emit
        self.free = list(range(n_slots))
        self.owner, self.fed, self.steps, self.released = {}, {}, [], []

    def acquire(self):
        slot = self.free.pop(0)
        self.fed[slot] = []
        return slot

    def release(self, slot):
        assert slot in self.fed, "released a slot that is not held"
        self.released.append((slot, list(self.fed.pop(slot))))
        self.free.append(slot)

    def step_sample(self, entries, samplings, recents, uniforms):
        self.steps.append([(slot, list(toks)) for slot, toks in entries])
        out = []
        for (slot, toks), recent in zip(entries, recents):
            assert slot in self.fed, "stepped a slot that is not held"
            self.fed[slot].extend(toks)
            key = self.fed[slot][0]
            out.append(self.scripts[key][len(recent)])
        return out


LIMITS = Limits(max_batch=3, max_tokens=64 * 8, max_step_tokens=100, max_seq_len=128)


def _loop(scripts, limits=LIMITS, stop_ids=(99,)):
    be = ScriptedBackend(scripts, limits.max_batch)
    return be, GenerationLoop(be, limits, Sampling.greedy(), stop_ids)


def test_stop_length_and_early_finishers():
    scripts = {1: [5, 6, 99, 7], 2: [8] * 10, 3: [99]}
    be, loop = _loop(scripts)
    outs = loop.run([Request([1, 10, 11], max_tokens=8), Request([2], max_tokens=4), Request([3, 30], max_tokens=8)])
    assert outs[0].tokens == [5, 6, 99] and outs[0].reason == STOP          # the stop token is recorded
    assert outs[1].tokens == [8, 8, 8, 8] and outs[1].reason == LENGTH
    assert outs[2].tokens == [99] and outs[2].reason == STOP and outs[2].prompt_tokens == 2
    # one prompt step with all three, then decode steps with the live ones only
    assert [len(s) for s in be.steps] == [3, 2, 2, 1]
    assert be.steps[0] == [(0, [1, 10, 11]), (1, [2]), (2, [3, 30])]
    assert be.steps[1] == [(0, [5]), (1, [8])]
    # the stop token is never fed back, and the last token of a length-limited sequence is not either
    fed = {f[0]: f for _, f in be.released}
    assert fed[1] == [1, 10, 11, 5, 6] and fed[2] == [2, 8, 8, 8] and fed[3] == [3, 30]
    assert sorted(be.free) == [0, 1, 2]


def test_batches_follow_one_another_and_reuse_slots():
    scripts = {i: [i] * 6 for i in range(1, 8)}
    be, loop = _loop(scripts)
    reqs = [Request([i], max_tokens=1 + i % 3) for i in range(1, 8)]
    outs = loop.run(reqs)
    assert [o.generated for o in outs] == [1 + i % 3 for i in range(1, 8)]
    assert len(be.released) == 7 and sorted(be.free) == [0, 1, 2]
    assert max(len(s) for s in be.steps) <= 3
    # 7 requests, at most 3 at a time: three batches
    assert plan_batches([1] * 7, [2] * 7, LIMITS) == [[0, 1, 2], [3, 4, 5], [6]]


def test_callback_cancels_one_sequence_only():
    scripts = {1: [5, 6, 7, 8], 2: [9, 9, 9, 9]}
    be, loop = _loop(scripts)
    seen = []

    def on_token(i, tok):
        seen.append((i, tok))
        return not (i == 0 and tok == 6)

    outs = loop.run([Request([1], max_tokens=4), Request([2], max_tokens=3)], on_token)
    assert outs[0].reason == CANCELLED and outs[0].tokens == [5, 6]
    assert outs[1].reason == LENGTH and outs[1].tokens == [9, 9, 9]
    assert (0, 5) in seen and (1, 9) in seen


def test_plan_batches_respects_pages_and_slots():
    lim = Limits(max_batch=8, max_tokens=64 * 4, max_step_tokens=100, max_seq_len=512)
    assert plan_batches([60, 60, 60], [1, 1, 1], lim) == [[0, 1, 2]]               # one batch, prompts over two steps
    assert plan_batches([10, 10, 10], [120, 120, 10], lim) == [[0], [1, 2]]        # pages: 3 + 3 > 4, 3 + 1 fit
    assert plan_batches([300], [1], lim) == [[0]]                                  # alone (the cache refuses it)
    wide = Limits(max_batch=8, max_tokens=64 * 64, max_step_tokens=4, max_seq_len=512)
    assert plan_batches([1] * 20, [1] * 20, wide) == [list(range(8)), list(range(8, 16)), list(range(16, 20))]


def test_prompts_beyond_one_step_are_fed_over_several_and_decode_together():
    scripts = {1: [5, 5, 5], 2: [6, 6, 6], 3: [7, 7, 7]}
    lim = Limits(max_batch=3, max_tokens=64 * 8, max_step_tokens=10, max_seq_len=128)
    be, loop = _loop(scripts, lim)
    reqs = [Request([1] + [20] * 6, max_tokens=3), Request([2] + [21] * 7, max_tokens=3), Request([3, 22], max_tokens=3)]
    outs = loop.run(reqs)
    assert [o.tokens for o in outs] == [[5, 5, 5], [6, 6, 6], [7, 7, 7]]
    # 7 + 8 + 2 prompt tokens under a step limit of 10: two prompt steps, then the three decode as one batch
    assert [sum(len(t) for _, t in st) for st in be.steps[:2]] == [10, 7]
    assert [len(st) for st in be.steps[2:]] == [3, 3]
    fed = {f[0]: f for _, f in be.released}
    assert fed[1][:7] == [1] + [20] * 6 and fed[2][:8] == [2] + [21] * 7 and fed[3][:2] == [3, 22]


def test_long_prompt_is_fed_in_chunks_and_sampled_once():
    scripts = {1: [7, 7, 7]}
    lim = Limits(max_batch=2, max_tokens=64 * 8, max_step_tokens=4, max_seq_len=256)
    be, loop = _loop(scripts, lim)
    prompt = [1] + list(range(20, 29))
    out = loop.run([Request(prompt, max_tokens=2)])[0]
    assert out.tokens == [7, 7]
    assert [t for s in be.steps[:3] for _, t in s] == [prompt[0:4], prompt[4:8], prompt[8:10]]
    assert be.steps[3] == [(0, [7])]


def test_limits_and_context_overflow():
    lim = Limits(2, 1024, 1024, 16)
    assert max_new_tokens(10, 512, lim) == 6
    with pytest.raises(ContextOverflow):
        max_new_tokens(16, 4, lim)
    with pytest.raises(ValueError):
        max_new_tokens(0, 4, lim)
    be, loop = _loop({1: [4] * 20}, lim)
    out = loop.run([Request([1] * 12, max_tokens=50)])[0]
    assert out.generated == 4 and out.reason == LENGTH
    assert len(be.released[0][1]) == 15            # 12 prompt + 3 fed back: position 15 is the last


def test_rng_matches_the_plain_implementation_and_is_per_sequence():
    a, b = Rng(42), plain.Rng(42)
    assert [a.next_f32() for _ in range(100)] == [b.next_f32() for _ in range(100)]
    scripts = {1: [5] * 5, 2: [6] * 5}
    be, loop = _loop(scripts)
    draws = []
    orig = be.step_sample
    be.step_sample = lambda e, s, r, u: (draws.append(list(u)), orig(e, s, r, u))[1]
    samp = Sampling(temperature=0.7, seed=9)
    loop.run([Request([1], 3, samp), Request([2], 3, samp.with_(seed=10))])
    r9, r10 = plain.Rng(9), plain.Rng(10)
    assert [d[0] for d in draws] == [r9.next_f32() for _ in range(3)]
    assert [d[1] for d in draws] == [r10.next_f32() for _ in range(3)]


class AheadBackend(ScriptedBackend):
    """A scripted backend that can be launched one step ahead: with ``feed`` a
    sequence's token is the one the step before produced."""

    class Handle:
        def __init__(self, tokens):
            self._tokens, self.n, self.read = tokens, len(tokens), False

        def tokens(self):
            self.read = True
            return self._tokens

    def __init__(self, scripts, n_slots):
        super().__init__(scripts, n_slots)
        self.fed_ahead = 0

    def launch_step_sample(self, entries, samplings, recents, uniforms, feed=None):
        if feed is not None:
            assert not feed.read, "a step is launched ahead before the step before has been read"
            entries = [(slot, [tok]) for (slot, _), tok in zip(entries, feed._tokens)]
            recents = [list(r) + [tok] for r, tok in zip(recents, feed._tokens)]
            self.fed_ahead += 1
        return self.Handle(self.step_sample(entries, samplings, recents, uniforms))


def test_running_one_step_ahead_changes_no_outcome():
    scripts = {1: [5, 6, 99, 7, 7, 7], 2: [8] * 12, 3: [4, 4, 4, 4, 99, 1], 4: [99]}
    reqs = [Request([1, 10], max_tokens=8), Request([2], max_tokens=9), Request([3, 30, 31], max_tokens=8),
            Request([4], max_tokens=3)]
    lim = Limits(max_batch=4, max_tokens=64 * 8, max_step_tokens=100, max_seq_len=128)
    plain_be = ScriptedBackend(scripts, 4)
    want = GenerationLoop(plain_be, lim, Sampling.greedy(), (99,)).run(reqs)
    be = AheadBackend(scripts, 4)
    got = GenerationLoop(be, lim, Sampling.greedy(), (99,)).run(reqs)
    assert [(o.tokens, o.reason) for o in got] == [(o.tokens, o.reason) for o in want]
    assert be.fed_ahead >= 4                       # steps really were launched ahead
    assert sorted(be.free) == [0, 1, 2, 3] and len(be.released) == 4
    # what each sequence was fed: its prompt, then its own tokens in order (a stop token may have been
    # fed by a step that was already running when it was read; nothing after it)
    for slot, fed in be.released:
        script, n_prompt = scripts[fed[0]], {1: 2, 2: 1, 3: 3, 4: 1}[fed[0]]
        assert fed[n_prompt:] == script[: len(fed) - n_prompt]
        assert 99 not in fed[n_prompt:-1]
    # with a repetition penalty the tokens are needed on the host first: nothing runs ahead
    be2 = AheadBackend(scripts, 4)
    GenerationLoop(be2, lim, Sampling(temperature=0.0, repeat_penalty=1.2), (99,)).run(reqs)
    assert be2.fed_ahead == 0
    # a sequence whose next token is its last by length is not run ahead
    be3 = AheadBackend({2: [8] * 12}, 1)
    out = GenerationLoop(be3, lim, Sampling.greedy(), (99,)).run([Request([2], max_tokens=2)])[0]
    assert out.tokens == [8, 8] and be3.fed_ahead == 0


def test_a_refused_launch_ahead_takes_no_draw():
    """The step launched ahead may be refused (no room for a token that may never be needed).  The draws taken
    for it are given back, so every sequence's uniforms are still its own stream in order."""

    class Refusing(AheadBackend):
        def __init__(self, scripts, n_slots, refuse_at):
            super().__init__(scripts, n_slots)
            self.refuse_at, self.calls, self.draws = set(refuse_at), 0, []

        def launch_step_sample(self, entries, samplings, recents, uniforms, feed=None):
            self.calls += 1
            if feed is not None and self.calls in self.refuse_at:
                raise CacheExhausted("scripted: no page for the step ahead")
            self.draws.append((feed is not None, list(uniforms)))
            return super().launch_step_sample(entries, samplings, recents, uniforms, feed=feed)

        def step_sample(self, entries, samplings, recents, uniforms):
            if len(entries[0][1]) > 1 or not self.steps:           # the prompt step (called directly by the loop)
                self.draws.append((False, list(uniforms)))
            return super().step_sample(entries, samplings, recents, uniforms)

    scripts = {1: [5] * 9, 2: [6] * 9}
    lim = Limits(max_batch=2, max_tokens=64 * 8, max_step_tokens=100, max_seq_len=128)
    samp = Sampling(temperature=0.7, seed=21)
    reqs = [Request([1, 3], 7, samp), Request([2, 4], 7, samp.with_(seed=22))]
    for refuse_at in ((), (2,), (2, 3, 5)):
        be = Refusing(scripts, 2, refuse_at)
        outs = GenerationLoop(be, lim, Sampling.greedy(), (99,)).run(reqs)
        assert [o.tokens for o in outs] == [[5] * 7, [6] * 7]
        # every sampled row's draw, in step order, is the sequence's own stream: nothing skipped, nothing twice
        r21, r22 = plain.Rng(21), plain.Rng(22)
        assert [d[0] for _, d in be.draws] == [r21.next_f32() for _ in be.draws], refuse_at
        assert [d[1] for _, d in be.draws] == [r22.next_f32() for _ in be.draws], refuse_at
        assert len(be.draws) == 7


def test_a_refused_step_leaves_the_cache_as_it_was():
    """Two sequences in one step, the second does not fit: the first one's new pages go back, and a later
    smaller step for it still finds a block-table row that matches its length."""
    a = CacheAllocator(n_slots=2, n_pages=4, windows=[None, 48])
    s0, s1 = a.acquire(), a.acquire()
    a.reserve(s0, 10), a.commit(s0, 10)
    a.reserve(s1, 2 * PAGE), a.commit(s1, 2 * PAGE)
    held = (a.pages_held(0), a.pages_held(1))
    a.reserve(s0, PAGE)                       # fits: one more page in each group
    with pytest.raises(CacheExhausted):
        a.reserve(s1, 2 * PAGE)               # does not: the step is refused as a whole
    a.unreserve(s0)
    assert (a.pages_held(0), a.pages_held(1)) == held
    assert len(a.page_row(s0, 0)) == pages_for(10) and a.length(s0) == 10
    a.check_consistent()
    a.reserve(s0, 1), a.commit(s0, 1)
    assert len(a.page_row(s0, 0)) == 1
    a.check_consistent()


def test_decode_attention_share_count_depends_on_the_shape_only():
    """Every sequence's keys are cut into as many shares as keep the whole grid resident at once (two CTAs per
    SM), never more than a full block table has 32-key tiles for; at most 8 (one thread-block cluster), or up to
    32 through the workspace where a small batch with a long context would leave most of the GPU idle."""
    from llmoxide_b200.kernels import decode_chunks

    for n_sm in (148, 132, 20):
        for n_seqs in (1, 2, 8, 16, 64, 300):
            for n_kv, group in ((8, 4), (1, 5), (2, 12), (8, 8)):
                for n_pages in (1, 3, 64, 640):
                    n = decode_chunks(n_seqs, n_kv, group, n_pages, n_sm)
                    base = n_seqs * n_kv * ((group + 7) // 8)
                    assert 1 <= n <= min(32, n_pages)
                    assert n == 1 or base * n <= 2 * n_sm
                    if n > 8:       # through the workspace only for a small batch with a long context
                        assert base * 8 <= n_sm and n_pages >= 8 * n
    assert decode_chunks(8, 8, 4, 64) == 4 and decode_chunks(64, 8, 4, 64) == 1 and decode_chunks(1, 8, 4, 64) == 8
    assert decode_chunks(1, 8, 4, 516) == 27 and decode_chunks(1, 8, 4, 132) == 16 and decode_chunks(2, 8, 4, 516) == 13


def test_bench_refuses_more_than_one_gpu_and_names_the_missing_reference():
    """The measurement's contract at its edges: more than one GPU is one line and exit code 2; the reference arm
    says in one JSON line why it cannot run, and exits 0."""
    import json
    import subprocess
    import sys
    from pathlib import Path

    bench = str(Path(__file__).resolve().parent.parent / "bench.py")
    many = subprocess.run([sys.executable, bench, "--gpus", "2"], capture_output=True, text=True, timeout=300)
    assert many.returncode == 2 and len(many.stdout.strip().splitlines()) == 1
    ref = subprocess.run([sys.executable, bench, "--impl", "reference"], capture_output=True, text=True, timeout=300)
    line = json.loads(ref.stdout.strip().splitlines()[-1])
    assert ref.returncode == 0 and line["impl"] == "reference" and line["unavailable"]
