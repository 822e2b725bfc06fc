"""GPU: the same requests replayed whole, with the last 32 tokens one by one,
and in batches of unequal lengths with slots used again -- in true 32-bit and
in bfloat16, each compared with the plain implementation."""

import os

import numpy as np
import pytest
import torch

import replay_util as ru
from tiny_configs import ALL, drawn_config, make_folder, make_folder_of, prompts

pytestmark = pytest.mark.gpu

LENGTHS = {"A": [5, 9, 13, 70, 1, 41], "B": [1, 7, 16, 31, 130, 66], "C": [3, 90, 25, 64, 150, 49],
           "D": [200, 65, 1, 129, 330, 64], "E": [33, 257, 100, 2, 128, 70]}


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    base = tmp_path_factory.mktemp("models")
    return {(n, d): make_folder(base, n, d) for n in ALL for d in ("float32", "bfloat16")}


def _engine(folder, dtype, max_tokens=1024):
    from llmoxide_b200.engine.engine import Engine, LoadOptions

    return Engine.load(folder, LoadOptions(dtype=dtype, max_tokens=max_tokens, max_batch=8))


def _requests(name):
    toks = prompts(ALL[name]["vocab_size"], LENGTHS[name], seed=11)
    return {f"r{i}": t for i, t in enumerate(toks)}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D", "E"])
def test_three_cuttings_match_the_plain_implementation(folders, tmp_path, name, dtype):
    folder = folders[(name, dtype)]
    reqs = _requests(name)
    want = ru.expected_logits(folder, reqs)
    vocab = ALL[name]["vocab_size"]
    eng = _engine(folder, dtype, max_tokens=2048)
    results = {}
    for what, steps in (("whole", ru.trace_whole(reqs)),
                        ("last 32 one by one", ru.trace_tail_decode(reqs, 32)),
                        ("unequal batches", ru.trace_batches(reqs, 4)),
                        ("unequal batches of 3, short prompts", ru.trace_batches(reqs, 3, 0.2)),
                        ("prompts in chunks of 48", ru.trace_chunks(reqs, 48, 3)),
                        ("prompts in chunks of 64", ru.trace_chunks(reqs, 64, 4)),
                        ("chunks of 48 beside single tokens", ru.trace_chunks(reqs, 48, 3, mixed=True)),
                        ("chunks of 100 beside single tokens", ru.trace_chunks(reqs, 100, 6, tail=40, mixed=True))):
        out = tmp_path / what.replace(" ", "_").replace(",", "")
        ru.run_in_process(eng, steps, out)
        got = ru.collect(steps, out, vocab)
        ru.assert_matches(got, want, dtype, f"{name}/{dtype}/{what}")
        print(f"{name}/{dtype}/{what}: worst rel err {max(ru.rel_err(got[r], want[r]) for r in reqs):.2e}")
        results[what] = got
    if dtype == "float32":
        # In 32-bit the cuttings agree with one another far below the tolerance
        # against the plain implementation.
        for what, got in results.items():
            for rid in reqs:
                assert ru.rel_err(got[rid], results["whole"][rid]) <= 2e-6, (what, rid)


@pytest.mark.parametrize("seed", range(24))
def test_drawn_configurations(tmp_path, seed):
    """Configurations drawn from a seed (head sizes 16 ... 256, widths that are no multiple of 8 or 16, odd
    vocabularies, windows), in both dtypes: whole, the tail one by one, unequal batches, chunks beside single
    tokens.  A size a kernel does not take has to be refused or routed to a kernel that does, never computed
    wrongly."""
    cfg = drawn_config(seed)
    print(cfg)
    toks = prompts(cfg["vocab_size"], [150, 3, 67, 129, 40], seed=seed)
    reqs = {f"r{i}": t for i, t in enumerate(toks)}
    for dtype in ("float32", "bfloat16"):
        folder = make_folder_of(tmp_path, f"drawn{seed}", cfg, dtype)
        want = ru.expected_logits(folder, reqs)
        eng = _engine(folder, dtype, max_tokens=2048)
        for what, steps in (("whole", ru.trace_whole(reqs)),
                            ("last 32 one by one", ru.trace_tail_decode(reqs, 32)),
                            ("unequal batches of 3", ru.trace_batches(reqs, 3, 0.6)),
                            ("chunks of 48 beside single tokens", ru.trace_chunks(reqs, 48, 5, tail=20, mixed=True))):
            out = tmp_path / f"{dtype}_{what.replace(' ', '_')}"
            ru.run_in_process(eng, steps, out)
            got = ru.collect(steps, out, cfg["vocab_size"])
            ru.assert_matches(got, want, dtype, f"drawn {seed}/{dtype}/{what}")
        eng.check_status()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run_program(folders, tmp_path, dtype):
    """The program itself, as a user runs it: fewer pages than all requests
    together would need, so pages and slots are used again."""
    name = "B"
    folder = folders[(name, dtype)]
    reqs = _requests(name)
    want = ru.expected_logits(folder, reqs)
    steps = ru.trace_batches(reqs, 2)
    # two live requests at a time: the two longest are 130 and 66 tokens
    max_tokens = 192 + 128
    ru.run_trace_run(folder, dtype, steps, tmp_path / "out", max_tokens)
    got = ru.collect(steps, tmp_path / "out", ALL[name]["vocab_size"])
    ru.assert_matches(got, want, dtype, f"trace_run/{dtype}")


def test_steps_without_wanted_logits_write_no_file(folders, tmp_path):
    folder = folders[("A", "float32")]
    steps = [dict(step=0, entries=[dict(id="a", tokens=[1, 2, 3], want=[])], end=[]),
             dict(step=1, entries=[dict(id="a", tokens=[4], want=[0])], end=["a"])]
    eng = _engine(folder, "float32")
    ru.run_in_process(eng, steps, tmp_path)
    assert not (tmp_path / "0.f32").exists() and (tmp_path / "1.f32").exists()
    want = ru.expected_logits(folder, {"a": [1, 2, 3, 4]})["a"][3:]
    got = np.fromfile(tmp_path / "1.f32", dtype="<f4").reshape(1, -1)
    assert ru.rel_err(got, want) <= ru.TOL["float32"]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_layer_sizes_of_qwen3_8b(tmp_path_factory, dtype):
    """One layer at Qwen3-8B layer sizes: a prompt longer than the prompt kernels' tiles (so the
    CTA-pair matrix product, the gated epilogue and the tiled attention run), decoding with split
    reductions, and a batch of unequal lengths."""
    folder = make_folder(tmp_path_factory.mktemp("m8b"), "8B", "bfloat16")      # bfloat16 weights in both runs
    toks = prompts(1536, [200, 150, 37], seed=3)
    reqs = {f"r{i}": t for i, t in enumerate(toks)}
    want = ru.expected_logits(folder, reqs)
    eng = _engine(folder, dtype, max_tokens=1024)
    for what, steps in (("whole", ru.trace_whole(reqs)), ("last 32 one by one", ru.trace_tail_decode(reqs, 32)),
                        ("unequal batch", ru.trace_batches(reqs, 3, 0.8)),
                        ("prompts in chunks of 48", ru.trace_chunks(reqs, 48, 3)),
                        ("chunks of 64 beside single tokens", ru.trace_chunks(reqs, 64, 3, tail=40, mixed=True))):
        out = tmp_path_factory.mktemp("o")
        ru.run_in_process(eng, steps, out)
        got = ru.collect(steps, out, 1536)
        ru.assert_matches(got, want, dtype, f"8B layer/{dtype}/{what}")
        print(f"8B layer/{dtype}/{what}: worst rel err {max(ru.rel_err(got[r], want[r]) for r in reqs):.2e}")
    from llmoxide_b200 import kernels
    assert kernels.gemm_tc_status() == 0


def test_a_step_of_more_than_65535_tokens(folders):
    """Grid dimensions other than x end at 65535: a prompt step larger than that must still be right."""
    import plain_qwen3 as plain
    from llmoxide_b200.engine.engine import Engine, LoadOptions

    for dtype in ("float32", "bfloat16"):
        folder = folders[("E", dtype)]
        toks = prompts(ALL["E"]["vocab_size"], [950] * 70, seed=9)           # 66 500 tokens in one step
        eng = Engine.load(folder, LoadOptions(dtype=dtype, max_tokens=70 * 960, max_batch=70, max_step_tokens=70000))
        slots = [eng.acquire() for _ in toks]
        logits = eng.step(list(zip(slots, toks))).cpu().numpy()              # the last position of each
        cfg, w = plain.read_model(folder)
        for i in (0, 37, 69):
            want = plain.forward(cfg, w, toks[i])[-1].numpy()
            assert ru.rel_err(logits[i][None], want[None]) <= ru.TOL[dtype], (dtype, i)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_named_intermediates_find_the_first_stage_that_differs(folders, tmp_path, dtype):
    """A step can hand out its named intermediates (the reference's trace names).  Whole prompt against the
    plain implementation's trace, stage by stage; then a fault is put into the engine's weights (the gain of the
    second layer's pre-feed-forward norm), and walking the stages in order finds it at that stage."""
    import plain_qwen3 as plain

    name = "D"
    folder = folders[(name, dtype)]
    toks = prompts(ALL[name]["vocab_size"], [150], seed=5)[0]
    cfg, w = plain.read_model(folder)
    want = {}
    plain.forward(cfg, w, toks, trace=lambda n, x: want.__setitem__(n, x.numpy().copy()))
    order = list(want)
    assert order[:3] == ["model.input_embed", "attn_norm-0", "attn_output-0"] and order[-1] == "result_norm"
    tol = {"float32": 2e-5, "bfloat16": 3e-2}[dtype]

    def stages(eng):
        got = {}
        slot = eng.acquire()
        eng.step([(slot, toks)], [list(range(len(toks)))], probe=lambda n, t: got.__setitem__(n, t.float().cpu().numpy()))
        eng.release(slot)
        return got

    def first_bad(got):
        for n in order:
            if ru.rel_err(got[n], want[n]) > tol:
                return n
        return None

    eng = _engine(folder, dtype)
    got = stages(eng)
    assert set(order) <= set(got), sorted(set(order) - set(got))
    assert first_bad(got) is None, first_bad(got)
    eng.model.blocks[1].ff_norm.gain.mul_(1.5)
    assert first_bad(stages(eng)) == "attn_post_norm-1"
    # through the replay program's own class: one file per stage and step
    from llmoxide_b200.engine.replay import Replayer
    eng2 = _engine(folder, dtype)
    rp = Replayer(eng2, tmp_path / "dump", dump=True)
    rp.run_step(dict(step=0, entries=[dict(id="a", tokens=toks[:70], want=[69])], end=[]))
    rp.run_step(dict(step=1, entries=[dict(id="a", tokens=toks[70:71], want=[0])], end=["a"]))
    d = ALL[name]["hidden_size"]
    first = np.fromfile(tmp_path / "dump" / "0.l_out-1.f32", dtype="<f4").reshape(70, d)
    assert ru.rel_err(first, want["l_out-1"][:70]) <= tol
    second = np.fromfile(tmp_path / "dump" / "1.attn_residual-0.f32", dtype="<f4").reshape(1, d)
    assert ru.rel_err(second, want["attn_residual-0"][70:71]) <= tol


def test_a_damaged_upload_is_noticed(folders, monkeypatch):
    """The head and the tail of every tensor are read back after the copy to the device."""
    from llmoxide_b200.config import read_config
    from llmoxide_b200.errors import CheckpointFormatError
    from llmoxide_b200.weights import loader

    folder = folders[("A", "float32")]
    spec = read_config(folder).to_spec()
    good = loader.load_checkpoint(folder, spec, "float32", "cuda")
    assert len(good) == len(spec.tensors())
    real = torch.Tensor.to

    def lossy(self, *a, **kw):
        out = real(self, *a, **kw)
        if kw.get("device") is not None and out.is_cuda and out.numel() == 64 * 128:     # one matrix of A's layers
            out.view(-1)[-1] += 1.0
        return out

    monkeypatch.setattr(torch.Tensor, "to", lossy)
    with pytest.raises(CheckpointFormatError, match="read back"):
        loader.load_checkpoint(folder, spec, "float32", "cuda")
