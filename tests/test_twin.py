"""CPU: the plain implementation (the oracle of every other test) against a
second, independent writing of the model in C++, made from the reference's
other statement of the same forward pass (crates/lab/src/engine.rs:275-406);
and against small committed outputs, so that a change of the oracle or of the
random-weights generator does not pass unseen."""

import json
import shutil
from pathlib import Path

import numpy as np
import pytest

import plain_qwen3 as plain
from tiny_configs import ALL, make_folder, prompts
from twin_util import twin_logits

GOLDEN = Path(__file__).resolve().parent / "golden"

pytestmark = pytest.mark.skipif(shutil.which("g++") is None and shutil.which("c++") is None,
                                reason="the twin needs a C++ compiler")


@pytest.mark.parametrize("name", ["A", "B", "C", "D", "E"])
def test_plain_implementation_agrees_with_its_twin(tmp_path, name):
    """Whole sequences without a cache (plain) against a prompt step plus single-token steps over a cache
    (twin): 37 tokens, longer than C's window of 24, so the window's edge moves inside the run."""
    folder = make_folder(tmp_path, name, "float32")
    vocab = ALL[name]["vocab_size"]
    toks = prompts(vocab, [37], seed=21)[0]
    cfg, w = plain.read_model(folder)
    want = plain.forward(cfg, w, toks).numpy()
    for prefix in (37, 20, 1):
        got = twin_logits(folder, toks, prefix, vocab)
        err = np.abs(got - want).max(axis=1) / np.abs(want).max()
        assert err.max() <= 2e-6, (name, prefix, int(err.argmax()), float(err.max()))
        assert (got.argmax(axis=1) == want.argmax(axis=1)).all()


def test_bfloat16_folders_are_read_alike(tmp_path):
    folder = make_folder(tmp_path, "B", "bfloat16")
    toks = prompts(ALL["B"]["vocab_size"], [19], seed=2)[0]
    cfg, w = plain.read_model(folder)
    want = plain.forward(cfg, w, toks).numpy()
    got = twin_logits(folder, toks, 7, ALL["B"]["vocab_size"])
    assert np.abs(got - want).max() / np.abs(want).max() <= 2e-6


@pytest.mark.parametrize("name", ["A", "B"])
def test_committed_outputs(tmp_path, name):
    """tests/golden/make_golden.py wrote these from the twin; the plain implementation must still give them
    from a freshly made folder (same configuration, same seed)."""
    meta = json.loads((GOLDEN / f"tiny_{name}.json").read_text())
    folder = make_folder(tmp_path, name, "float32", seed=meta["seed"])
    cfg, w = plain.read_model(folder)
    got = plain.forward(cfg, w, meta["tokens"]).numpy()[meta["positions"]]
    want = np.fromfile(GOLDEN / f"tiny_{name}.f32", dtype="<f4").reshape(got.shape)
    assert np.abs(got - want).max() / np.abs(want).max() <= 2e-6
