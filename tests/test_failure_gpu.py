"""GPU: failure detection.  A bounded wait that runs out is reported in the
library's status word, the engine turns it into ``KernelError`` where it has
waited for the step anyway, the kernel winds down through its normal exit and
the library stays usable.  The waits are made to run out on the host's terms:
a test switch makes one role of a kernel leave out a single arrival, and the
limit is set to half a millisecond; nothing traps, faults or spins past its
limit.  Also: the guard words behind device buffers and the fixture that
checks them."""

import math

import pytest
import torch

import plain_qwen3 as plain
import replay_util as ru
from tiny_configs import ALL, make_folder, prompts

pytestmark = pytest.mark.gpu

SHORT = 1_000_000        # clock cycles: about half a millisecond


def _reset(lib):
    from llmoxide_b200 import kernels

    kernels.test_waits(lib, 0, False)
    try:
        kernels.check_status()
    except Exception:
        pass
    # the library's own copy of the report is cleared by reading it
    {"gemm_tc": kernels.gemm_tc_status, "attention_decode": kernels.attention_decode_status,
     "attention_prefill_tc": kernels.attention_prefill_tc_status}[lib]()


def test_a_matrix_product_whose_wait_runs_out_is_reported_and_the_library_goes_on():
    from llmoxide_b200 import kernels
    from llmoxide_b200.errors import KernelError

    torch.manual_seed(0)
    x = (torch.randn(40, 256) * 0.5).bfloat16().cuda()
    w = (torch.randn(384, 256) * 0.5).bfloat16().cuda()
    want = x.float() @ w.float().t()
    out = torch.empty(40, 384, dtype=torch.bfloat16, device="cuda")
    kernels.gemm_tc(x, w, out)
    torch.cuda.synchronize()
    kernels.check_status()
    assert kernels.gemm_tc_status() == 0
    try:
        kernels.test_waits("gemm_tc", SHORT, True)
        for kw in (dict(), dict(n_split=2)):
            o = torch.empty((2, 40, 384), dtype=torch.float32, device="cuda") if kw else out
            kernels.gemm_tc(x, w, o, **kw)
            torch.cuda.synchronize()                # returns: every role gave up and the CTAs left
            with pytest.raises(KernelError, match="gemm_tc"):
                kernels.check_status()
            kernels.check_status()                  # the report was cleared
            assert kernels.gemm_tc_status() in (1, 3, 4)
        # the CTA-pair kernel of prompt-sized products
        xp = (torch.randn(300, 256) * 0.5).bfloat16().cuda()
        op = torch.empty(300, 384, dtype=torch.bfloat16, device="cuda")
        kernels.gemm_tc(xp, w, op, pair=True)
        torch.cuda.synchronize()
        with pytest.raises(KernelError, match="CTA pair"):
            kernels.check_status()
        assert kernels.gemm_tc_status() in (11, 13, 14)
    finally:
        _reset("gemm_tc")
    kernels.gemm_tc(x, w, out)                       # tensor memory was freed, the library works as before
    torch.cuda.synchronize()
    kernels.check_status()
    assert float((out.float() - want).abs().max() / want.abs().max()) < 6e-3
    kernels.gemm_tc(xp, w, op, pair=True)
    torch.cuda.synchronize()
    wantp = xp.float() @ w.float().t()
    assert float((op.float() - wantp).abs().max() / wantp.abs().max()) < 6e-3
    assert kernels.gemm_tc_status() == 0


def _decode_case(D, lengths, G=2, H=8):
    g = torch.Generator().manual_seed(3)
    n_pages = sum((n + 63) // 64 for n in lengths) + 1
    kc = torch.randn(n_pages, G, 64, D, generator=g).bfloat16().cuda()
    vc = torch.randn(n_pages, G, 64, D, generator=g).bfloat16().cuda()
    width = max((n + 63) // 64 for n in lengths)
    table = torch.zeros((len(lengths), width), dtype=torch.int32)
    nxt = 1
    for b, n in enumerate(lengths):
        for lp in range((n + 63) // 64):
            table[b, lp] = nxt
            nxt += 1
    q = torch.randn(len(lengths), H * D, generator=g).bfloat16().cuda()
    past = torch.tensor([n - 1 for n in lengths], dtype=torch.int32).cuda()
    return q, kc, vc, table.cuda(), past


@pytest.mark.parametrize("D", [128, 48])        # tensor copies; per-lane cp.async
def test_decode_attention_whose_copy_never_lands_is_reported(D):
    from llmoxide_b200 import kernels
    from llmoxide_b200.errors import KernelError

    H, G = 8, 2
    q, kc, vc, table, past = _decode_case(D, [300, 500])
    out = torch.empty_like(q)
    scale = 1 / math.sqrt(D)
    kernels.attention_decode(q, out, kc, vc, table, past, H, G, D, None, scale, n_chunks=2)
    torch.cuda.synchronize()
    good = out.clone()
    kernels.check_status()
    try:
        kernels.test_waits("attention_decode", SHORT, True)
        kernels.attention_decode(q, out, kc, vc, table, past, H, G, D, None, scale, n_chunks=2)
        torch.cuda.synchronize()
        with pytest.raises(KernelError, match="attention_decode"):
            kernels.check_status()
        assert kernels.attention_decode_status() == 1
    finally:
        _reset("attention_decode")
    kernels.attention_decode(q, out, kc, vc, table, past, H, G, D, None, scale, n_chunks=2)
    torch.cuda.synchronize()
    kernels.check_status()
    assert torch.equal(out, good)


def test_prompt_attention_whose_wait_runs_out_is_reported():
    from llmoxide_b200 import kernels
    from llmoxide_b200.errors import KernelError

    H, G, D, T = 4, 2, 128, 200
    g = torch.Generator().manual_seed(4)
    kc = torch.randn(6, G, 64, D, generator=g).bfloat16().cuda()
    vc = torch.randn(6, G, 64, D, generator=g).bfloat16().cuda()
    table = torch.tensor([[1, 2, 3, 4]], dtype=torch.int32).cuda()
    q = torch.randn(T, H * D, generator=g).bfloat16().cuda()
    out = torch.empty_like(q)
    start = torch.tensor([0, T], dtype=torch.int32).cuda()
    past = torch.zeros(1, dtype=torch.int32).cuda()
    args = (q, out, kc, vc, table, start, past, 1, T, H, G, D, None, 1 / math.sqrt(D))
    kernels.attention_prefill_tc(*args)
    torch.cuda.synchronize()
    good = out.clone()
    kernels.check_status()
    try:
        kernels.test_waits("attention_prefill_tc", SHORT, True)
        kernels.attention_prefill_tc(*args)
        torch.cuda.synchronize()
        with pytest.raises(KernelError, match="attention_prefill_tc"):
            kernels.check_status()
        assert kernels.attention_prefill_tc_status() in (1, 2, 5, 7)     # whichever role's wait ran out first
    finally:
        _reset("attention_prefill_tc")
    kernels.attention_prefill_tc(*args)
    torch.cuda.synchronize()
    kernels.check_status()
    assert torch.equal(out, good)
    assert kernels.attention_prefill_tc_status() == 0


def test_the_engine_raises_where_it_has_waited(tmp_path):
    """Through the product path: the generation loop (reading a step's tokens) and trace replay (reading a
    step's logits) raise ``KernelError``; afterwards the same engine gives right logits again."""
    from llmoxide_b200 import kernels
    from llmoxide_b200.engine.engine import Engine, LoadOptions
    from llmoxide_b200.engine.replay import Replayer
    from llmoxide_b200.errors import KernelError
    from llmoxide_b200.sampling import Sampling

    folder = make_folder(tmp_path, "D", "bfloat16")
    toks = prompts(ALL["D"]["vocab_size"], [90], seed=1)[0]
    eng = Engine.load(folder, LoadOptions(dtype="bfloat16", max_tokens=512, max_batch=2))
    slot = eng.acquire()
    eng.step_sample([(slot, toks[:40])], [Sampling.greedy()], [[]], [0.0])       # fine
    try:
        kernels.test_waits("gemm_tc", SHORT, True)
        with pytest.raises(KernelError, match="gemm_tc"):
            eng.step_sample([(slot, toks[40:41])], [Sampling.greedy()], [[]], [0.0])
        rp = Replayer(eng, tmp_path / "out")
        with pytest.raises(KernelError, match="bounded wait|ran out"):
            rp.run_step(dict(step=0, entries=[dict(id="x", tokens=toks[:20], want=[19])], end=[]))
        rp.run_step(dict(step=1, entries=[], end=["x"]))
    finally:
        _reset("gemm_tc")
    eng.release(slot)
    reqs = {"a": toks}
    steps = ru.trace_tail_decode(reqs, 8)
    ru.run_in_process(eng, steps, tmp_path / "again")
    got = ru.collect(steps, tmp_path / "again", ALL["D"]["vocab_size"])
    ru.assert_matches(got, ru.expected_logits(folder, reqs), "bfloat16", "after a reported failure")


def test_an_unserved_sampling_request_is_reported():
    """What the sampling kernel cannot do (top-p over more candidates than it sorts) is refused on the host
    first; handed to the kernel all the same, it reports through the status word."""
    from llmoxide_b200 import kernels
    from llmoxide_b200.errors import KernelError

    B, V = 2, 3000
    logits = torch.randn(B, V, device="cuda")
    f = lambda v: torch.full((B,), v, dtype=torch.float32, device="cuda")
    out = torch.zeros(B, dtype=torch.int32, device="cuda")
    kernels.preload(["sampling"])
    kernels.sample(logits, f(0.8), torch.zeros(B, dtype=torch.int32, device="cuda"), f(0.5), f(1.0), None, f(0.3), out,
                   kernels.status_word("sampling"))
    torch.cuda.synchronize()
    with pytest.raises(KernelError, match="sampling"):
        kernels.check_status()
    kernels.check_status()


# ---- guard words ------------------------------------------------------------------------

def test_guard_words_catch_a_write_past_the_end():
    """The corruption is made from the host (a guard word is overwritten by a copy), not by a kernel that
    runs out of bounds."""
    from llmoxide_b200 import guard

    guard.check_all()
    t = guard.guarded((1000,), torch.float32, "cuda", "a test buffer", zero=True)
    assert t.shape == (1000,) and float(t.abs().sum()) == 0.0
    n = guard.check_all()
    assert n >= 1
    # the word right behind the payload (rounded up to 256 bytes: 4000 -> 4096 bytes = word 1024 of the storage)
    whole = torch.empty(0, dtype=torch.int32, device="cuda").set_(t.untyped_storage(), 0, (1024 + 64,))
    assert int(whole[1024]) == guard.PATTERN
    whole[1024 + 5] = 7
    with pytest.raises(guard.GuardError, match="a test buffer"):
        guard.check_all()
    guard.check_all()            # reported once, then forgotten


def test_every_long_lived_buffer_of_an_engine_is_guarded(tmp_path):
    from llmoxide_b200 import guard
    from llmoxide_b200.engine.engine import Engine, LoadOptions
    from llmoxide_b200.sampling import Sampling

    guard.check_all()
    before = guard.n_guards()
    folder = make_folder(tmp_path, "C", "bfloat16")      # two cache groups: all keys, and a window
    eng = Engine.load(folder, LoadOptions(dtype="bfloat16", max_tokens=512, max_batch=4))
    slot = eng.acquire()
    eng.step_sample([(slot, [1, 2, 3])], [Sampling(temperature=0.5, top_k=5)], [[]], [0.3])
    names = [e[2] for e in guard._entries[before:]]
    for want in ("step buffer", "cache group 0 keys", "cache group 1 values", "sampled tokens 0"):
        assert want in names, names
    # scratch of a step gets guards on request: a whole prompt and decode steps run under them
    guard.scratch_guards(True)
    try:
        eng.step([(slot, list(range(4, 150)))])
        for t in range(5):
            eng.step([(slot, [t])])
        assert any("matrix product" in e[2] for e in guard._entries)
        guard.check_all()
    finally:
        guard.scratch_guards(False)
