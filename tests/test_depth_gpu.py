"""GPU: logits through depth at real widths.  Eight layers at Qwen3-8B layer
sizes with the full vocabulary of 151 936 (tied head, 2.2 B parameters), made
with the random-weights mode on the device; the plain implementation reads the
same values (the mode gives the same tensors on the device and in a folder,
tests/test_weights_gpu.py).  Every way of cutting the work, in true 32-bit and
in bfloat16.  This is where the split matrix product of the head and the sum
of its partials meet a logits test at the real width."""

import numpy as np
import pytest
import torch

import plain_qwen3 as plain
import replay_util as ru
from tiny_configs import LAYER_8B, prompts

pytestmark = pytest.mark.gpu

RAW = dict(LAYER_8B, num_hidden_layers=8, vocab_size=151936, tie_word_embeddings=True, torch_dtype="bfloat16")
SEED = 31


@pytest.fixture(scope="module")
def plain_logits():
    from llmoxide_b200 import read_config
    from llmoxide_b200.weights import random_tensors_on_device

    cfg = read_config(RAW)
    w = {k: v.float().cpu() for k, v in random_tensors_on_device(cfg.to_spec(), SEED, "bfloat16", "cuda").items()}
    torch.cuda.empty_cache()
    toks = prompts(RAW["vocab_size"], [150, 64, 97], seed=13)
    reqs = {f"r{i}": t for i, t in enumerate(toks)}
    raw = dict(cfg.to_dict())
    want = {rid: plain.forward(raw, w, t).numpy() for rid, t in reqs.items()}
    del w
    return cfg, reqs, want


@pytest.mark.parametrize("dtype", ["bfloat16", "float32"])
def test_eight_layers_at_qwen3_8b_sizes_with_the_full_vocabulary(plain_logits, tmp_path, dtype):
    from llmoxide_b200.engine.engine import Engine, LoadOptions

    cfg, reqs, want = plain_logits
    eng = Engine.random(cfg, SEED, LoadOptions(dtype=dtype, max_tokens=1024, max_batch=4))
    V = RAW["vocab_size"]
    results = {}
    for what, steps in (("whole", ru.trace_whole(reqs)), ("last 32 one by one", ru.trace_tail_decode(reqs, 32)),
                        ("unequal batch", ru.trace_batches(reqs, 3, 0.7)),
                        ("prompts in chunks of 48", ru.trace_chunks(reqs, 48, 3, tail=4)),
                        ("chunks of 64 beside single tokens", ru.trace_chunks(reqs, 64, 3, tail=12, mixed=True))):
        out = tmp_path / what.replace(" ", "_")
        ru.run_in_process(eng, steps, out)
        got = ru.collect(steps, out, V)
        ru.assert_matches(got, want, dtype, f"8 layers, full vocabulary/{dtype}/{what}")
        print(f"8 layers, full vocabulary/{dtype}/{what}: worst rel err "
              f"{max(ru.rel_err(got[r], want[r]) for r in reqs):.2e}")
        # the token a greedy sampler would take: the same wherever the plain logits do not nearly tie
        for rid in reqs:
            top2 = np.sort(want[rid], axis=1)[:, -2:]
            clear = (top2[:, 1] - top2[:, 0]) > 2 * ru.TOL[dtype] * np.abs(want[rid]).max()
            assert (got[rid].argmax(1)[clear] == want[rid].argmax(1)[clear]).all(), (what, rid)
        results[what] = got
        for f in out.iterdir():
            f.unlink()
    if dtype == "float32":
        for what, got in results.items():
            for rid in reqs:
                assert ru.rel_err(got[rid], results["whole"][rid]) <= 2e-6, (what, rid)
    eng.check_status()
