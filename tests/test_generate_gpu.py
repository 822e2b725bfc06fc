"""GPU: generation through the entry point -- greedy against the plain
implementation, long decoding, the first tokens of a sequence, unequal
batches with early finishers and slots used again, temperature sampling that
is reproducible and independent of the batch, and the command line."""

import subprocess
import sys

import numpy as np
import pytest
import torch

import plain_qwen3 as plain
import replay_util as ru
from tiny_configs import ALL, make_folder, prompts

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    base = tmp_path_factory.mktemp("models")
    return {(n, d): make_folder(base, n, d) for n in ALL for d in ("float32", "bfloat16")}


def _session(folder, dtype, **kw):
    from llmoxide_b200 import LoadOptions, Session

    opts = dict(dtype=dtype, max_tokens=2048, max_batch=4)
    opts.update(kw)
    return Session.load(folder, LoadOptions(**opts))


@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_greedy_generation_matches_the_plain_implementation(folders, name):
    from llmoxide_b200 import Request, Sampling

    folder = folders[(name, "float32")]
    cfg, w = plain.read_model(folder)
    ps = prompts(cfg["vocab_size"], [3, 17, 1, 40, 9, 66, 5], seed=3)
    n_new = [12, 5, 20, 8, 1, 10, 30]
    stops = tuple(cfg["eos_token_id"]) if isinstance(cfg["eos_token_id"], list) else (cfg["eos_token_id"],)
    want = [plain.greedy_generate(cfg, w, p, n, stops) for p, n in zip(ps, n_new)]
    s = _session(folder, "float32", max_batch=3)           # 7 requests over 3 slots: slots are used again
    outs = s.generate([Request(p, max_tokens=n, sampling=Sampling.greedy()) for p, n in zip(ps, n_new)])
    for o, wt, n in zip(outs, want, n_new):
        assert o.tokens == wt
        assert o.reason == ("stop" if wt[-1] in stops else "length")
        assert o.generated == len(wt)
    s.engine.cache.alloc.check_consistent()
    assert s.engine.cache.alloc.pages_held() == 0 and s.engine.cache.alloc.n_free_slots == 3


def test_greedy_bfloat16_follows_float32_logits(folders):
    """bfloat16 may pick another token only where the float32 logits nearly tie."""
    from llmoxide_b200 import Request, Sampling

    folder = folders[("B", "bfloat16")]
    cfg, w = plain.read_model(folder)
    p = prompts(cfg["vocab_size"], [23], seed=4)[0]
    out = _session(folder, "bfloat16").generate([Request(p, 24, Sampling.greedy(), stop_ids=())])[0]
    ids = list(p)
    for tok in out.tokens:
        logits = plain.forward(cfg, w, ids)[-1].numpy()
        assert logits.max() - logits[tok] <= 2e-2 * np.abs(logits).max()
        ids.append(tok)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_and_first_tokens(folders, dtype):
    """One token at a time from the very first position, across several pages
    and, in configuration C, far beyond the window."""
    for name in ("A", "C"):
        folder = folders[(name, dtype)]
        vocab = ALL[name]["vocab_size"]
        toks = prompts(vocab, [ALL[name]["max_position_embeddings"] // 2 if name == "A" else 230], seed=8)[0]
        from llmoxide_b200.engine.engine import Engine, LoadOptions
        eng = Engine.load(folder, LoadOptions(dtype=dtype, max_tokens=512, max_batch=2))
        slot = eng.acquire()
        rows = [eng.step([(slot, [t])])[0].cpu().numpy() for t in toks]
        eng.release(slot)
        got = np.stack(rows)
        want = ru.expected_logits(folder, {"x": toks})["x"]
        for lo, hi in ((0, 4), (0, len(toks))):            # the first tokens, then all of them
            assert ru.rel_err(got[lo:hi], want[lo:hi]) <= ru.TOL[dtype], (name, lo, hi)
        if name == "C":
            assert eng.cache.alloc.pages_held(0) == 0 and eng.cache.alloc.pages_held(1) == 0


def test_temperature_sampling_is_seeded_and_batch_independent(folders):
    from llmoxide_b200 import Request, Sampling

    folder = folders[("B", "float32")]
    ps = prompts(ALL["B"]["vocab_size"], [9, 30, 2], seed=5)
    samp = Sampling(temperature=0.9, top_k=40, top_p=0.9, repeat_penalty=1.1, seed=21)
    s = _session(folder, "float32")
    reqs = [Request(p, 16, samp.with_(seed=21 + i), stop_ids=()) for i, p in enumerate(ps)]
    together = s.generate(reqs)
    alone = [s.generate([r])[0] for r in reqs]
    again = s.generate(reqs)
    for a, b, c in zip(together, alone, again):
        assert a.tokens == b.tokens == c.tokens
    other = s.generate([Request(ps[0], 16, samp.with_(seed=99), stop_ids=())])[0]
    assert other.tokens != together[0].tokens
    # against the plain sampler, step by step, on the plain logits of the engine's own prefix
    cfg, w = plain.read_model(folder)
    for i, o in enumerate(together):
        _check_sampled(cfg, w, ps[i], o.tokens, samp.with_(seed=21 + i))


def _check_sampled(cfg, w, prompt, tokens, samp):
    """Every token is what the plain sampler picks, with the sequence's next draw, from the plain
    implementation's logits after the prompt and the engine's own tokens before it."""
    rng, ids = plain.Rng(samp.seed), list(prompt)
    for n, tok in enumerate(tokens):
        logits = plain.forward(cfg, w, ids)[-1].numpy()
        want = plain.sample(logits, tokens[:n], temperature=samp.temperature, top_k=samp.top_k, top_p=samp.top_p,
                            repeat_penalty=samp.repeat_penalty, repeat_window=samp.repeat_window, u=rng.next_f32())
        assert tok == want, (n, tok, want, tokens)
        ids.append(tok)


def test_sampling_while_running_one_step_ahead(folders):
    """Without a repetition penalty the loop launches each decode step before it has read the tokens of the
    step before, so a sequence's draws are taken a step early, and on the survivors of a batch that loses a
    neighbour.  Three requests, one of which stops early (after its third token or later) on a stop token of
    its own."""
    from llmoxide_b200 import Request, Sampling

    folder = folders[("B", "float32")]
    cfg, w = plain.read_model(folder)
    ps = prompts(ALL["B"]["vocab_size"], [12, 5, 40], seed=6)
    samp = Sampling(temperature=0.8, top_k=30, top_p=0.95, repeat_penalty=1.0, seed=50)
    s = _session(folder, "float32")
    ahead = []
    launch = s.engine.launch_step_sample
    s.engine.launch_step_sample = lambda *a, feed=None: (ahead.append(feed is not None), launch(*a, feed=feed))[1]
    reqs = [Request(p, 14, samp.with_(seed=50 + i), stop_ids=()) for i, p in enumerate(ps)]
    free = s.generate(reqs)
    assert sum(ahead) >= 10                              # steps really were launched ahead
    for i, o in enumerate(free):
        assert o.generated == 14
        _check_sampled(cfg, w, ps[i], o.tokens, samp.with_(seed=50 + i))
    # the second request now stops at its fourth token; the others go on in a smaller batch, unchanged
    k = next(k for k in range(2, 14) if free[1].tokens[k] not in free[1].tokens[:k])
    reqs[1] = Request(ps[1], 14, samp.with_(seed=51), stop_ids=(free[1].tokens[k],))
    outs = s.generate(reqs)
    assert outs[1].tokens == free[1].tokens[: k + 1] and outs[1].reason == "stop"
    assert outs[0].tokens == free[0].tokens and outs[2].tokens == free[2].tokens
    s.engine.cache.alloc.check_consistent()
    assert s.engine.cache.alloc.pages_held() == 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_libraries_are_resident_before_the_first_step_and_prompts_may_overlap(folders, dtype):
    """The parts name the CUDA libraries they launch and the engine loads them when it is built; a prompt step
    gives the same tokens with and without the overlap of consecutive kernels."""
    from llmoxide_b200 import Request, Sampling, kernels
    from llmoxide_b200.csrc.build import LIBRARIES

    ps = prompts(ALL["D"]["vocab_size"], [70, 3, 140], seed=11)
    outs = []
    for overlap in (False, True):
        session = _session(folders[("D", dtype)], dtype, overlap_prompt_kernels=overlap)
        named = session.engine.model.libraries()
        assert named and named <= set(LIBRARIES)
        assert named <= kernels._libs_ready
        outs.append([o.tokens for o in session.generate([Request(p, 6, Sampling.greedy(), stop_ids=()) for p in ps])])
        assert "sampling" in kernels._libs_ready
        assert kernels._overlap is True          # switched back after the prompt step
    assert outs[0] == outs[1]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_prompt_shape_that_comes_back_is_replayed_as_a_graph(folders, dtype):
    """A short prompt step is bound by its launches: the second time a shape is seen it is captured and from
    then on replayed.  Same logits as the eager step, bit for bit, with other tokens in other slots each time;
    a longer shape and an engine with the option off stay eager."""
    from llmoxide_b200 import LoadOptions
    from llmoxide_b200.engine.engine import Engine

    folder = folders[("D", dtype)]
    eager = Engine.load(folder, LoadOptions(dtype=dtype, max_tokens=4096, max_batch=8, graph_prompt_tokens=0))
    graphed = Engine.load(folder, LoadOptions(dtype=dtype, max_tokens=4096, max_batch=8, graph_prompt_tokens=200))
    held = []
    for rep in range(4):
        ps = prompts(ALL["D"]["vocab_size"], [70, 3, 100], seed=20 + rep)
        outs = []
        for eng in (eager, graphed):
            slots = [eng.acquire() for _ in ps]
            before = eng.n_steps
            logits = eng.step(list(zip(slots, ps)), want=[[0, len(p) - 1] for p in ps])
            outs.append(logits.clone())
            # one decode step on top, so that the replayed prompt step's cache entries are read back
            outs.append(eng.step([(s, [7 + rep]) for s in slots]).clone())
            assert eng.n_steps == before + 2
            if rep % 2:
                held.append((eng, slots))          # the next round's pages lie elsewhere
            else:
                for s in slots:
                    eng.release(s)
        assert torch.equal(outs[0], outs[2]) and torch.equal(outs[1], outs[3]), rep
        assert len(graphed._prompt_graphs) == (1 if rep >= 1 else 0)
    graphed.check_status()
    assert not eager._prompt_graphs
    # beyond the limit: eager however often it comes back
    for rep in range(3):
        slot = graphed.acquire()
        graphed.step([(slot, prompts(ALL["D"]["vocab_size"], [230], seed=rep)[0])])
        graphed.release(slot)
    assert len(graphed._prompt_graphs) == 1
    for eng, slots in held:
        for s in slots:
            eng.release(s)
    for eng in (eager, graphed):
        eng.cache.alloc.check_consistent()
        assert eng.cache.alloc.pages_held() == 0


def test_a_step_that_fails_midway_gives_its_pages_back(folders):
    """A step that raises after its pages were reserved (here: the forward itself, as when the device runs out
    of memory for a step's activations) leaves the sequences as they were: same lengths, no page kept beyond
    them, and the next step gives the logits it would have given."""
    from llmoxide_b200 import LoadOptions
    from llmoxide_b200.engine.engine import Engine

    folder = folders[("B", "float32")]
    eng = Engine.load(folder, LoadOptions(dtype="float32", max_tokens=1024, max_batch=4))
    toks = prompts(ALL["B"]["vocab_size"], [150, 40], seed=9)
    want = ru.expected_logits(folder, {"a": toks[0], "b": toks[1]})
    a, b = eng.acquire(), eng.acquire()
    eng.step([(a, toks[0][:30]), (b, toks[1][:10])])
    held = eng.cache.alloc.pages_held()
    real = eng.model.forward

    def failing(ctx, cache):
        real(ctx, cache)
        raise RuntimeError("out of memory, say")

    eng.model.forward = failing
    with pytest.raises(RuntimeError):
        eng.step([(a, toks[0][30:]), (b, toks[1][10:])])          # would have taken two more pages for a
    eng.model.forward = real
    assert (eng.length(a), eng.length(b)) == (30, 10)
    assert eng.cache.alloc.pages_held() == held
    eng.cache.alloc.check_consistent()
    got = eng.step([(a, toks[0][30:]), (b, toks[1][10:])]).cpu().numpy()
    assert ru.rel_err(got[0:1], want["a"][-1:]) <= ru.TOL["float32"]
    assert ru.rel_err(got[1:2], want["b"][-1:]) <= ru.TOL["float32"]
    eng.release(a), eng.release(b)
    assert eng.cache.alloc.pages_held() == 0


def test_forward_and_wipe(folders):
    folder = folders[("A", "float32")]
    s = _session(folder, "float32")
    toks = prompts(ALL["A"]["vocab_size"], [11], seed=6)[0]
    want = ru.expected_logits(folder, {"x": toks})["x"]
    a = s.forward(toks[:6]).cpu().numpy()
    b = s.forward(toks[6:]).cpu().numpy()
    assert ru.rel_err(a[None], want[5:6]) <= ru.TOL["float32"]
    assert ru.rel_err(b[None], want[10:11]) <= ru.TOL["float32"]
    s.wipe()
    c = s.forward(toks[:6]).cpu().numpy()
    assert np.array_equal(a, c)
    assert s.info()["architecture"] == "Qwen3ForCausalLM"


def test_errors_before_any_launch(folders):
    from llmoxide_b200 import CacheExhausted, ContextOverflow, LoadOptions, Request, Session
    from llmoxide_b200.engine.engine import Engine

    folder = folders[("A", "float32")]
    eng = Engine.load(folder, LoadOptions(dtype="float32", max_tokens=128, max_batch=2, max_step_tokens=64))
    slot = eng.acquire()
    with pytest.raises(ValueError, match="vocabulary"):
        eng.step([(slot, [1, 256])])
    with pytest.raises(ContextOverflow):
        eng.step([(slot, [1] * 65)])                      # step limit
    with pytest.raises(ContextOverflow):
        eng.step([(slot, [1] * 60)]), eng.step([(slot, [1] * 60)]), eng.step([(slot, [1] * 60)])
    other = eng.acquire()
    with pytest.raises(CacheExhausted):
        eng.acquire()
    with pytest.raises(CacheExhausted):
        eng.step([(other, [1] * 10)])                     # the pages are held by the first sequence
    eng.release(slot), eng.release(other)
    eng.cache.alloc.check_consistent()
    with pytest.raises(ContextOverflow):
        Session(eng).generate([Request([1] * 128, 4)])


def test_command_line(folders):
    folder = folders[("A", "float32")]
    cfg, w = plain.read_model(folder)
    ps = prompts(cfg["vocab_size"], [4, 9], seed=7)
    text = ";".join(",".join(map(str, p)) for p in ps)
    p = subprocess.run([sys.executable, str(ru.ROOT / "bin" / "llmoxide"), str(folder), text, "6",
                        "--dtype", "float32", "--ignore-stop"], capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-3000:]
    lines = [l for l in p.stdout.splitlines() if l.startswith("ids: ")]
    want = [plain.greedy_generate(cfg, w, q, 6) for q in ps]
    assert [l.split("  (")[0] for l in lines] == [f"ids: {t}" for t in want]
    assert "prefill" in p.stderr and "tok/s" in p.stderr
    q = subprocess.run([sys.executable, str(ru.ROOT / "bin" / "llmoxide"), str(folder), "1,2", "--cpu"],
                       capture_output=True, text=True, timeout=600)
    assert q.returncode == 2 and "no CPU path" in q.stderr
