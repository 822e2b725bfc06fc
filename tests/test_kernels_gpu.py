"""GPU: each kernel alone against its plain float32 reference, at sizes other
than the engine's, with inputs made so that a fault shows (a far key among
hundreds, a window's edge, a page boundary)."""

import math

import numpy as np
import pytest
import torch

import plain_qwen3 as plain

pytestmark = pytest.mark.gpu

DEV = "cuda"
PAGE = 64


def rel(got, want):
    got, want = got.float().cpu(), want.float().cpu()
    return float((got - want).abs().max() / want.abs().max())


def tol(dtype):
    return 2e-6 if dtype == torch.float32 else 6e-3   # one bfloat16 rounding is 2^-9 = 2e-3


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_embed(dtype):
    from llmoxide_b200 import kernels
    table = torch.randn(1000, 200).to(dtype)
    toks = torch.tensor([0, 999, 17, 17, 500], dtype=torch.int32)
    out = torch.empty(5, 200, dtype=torch.float32, device=DEV)
    kernels.embed(table.to(DEV), toks.to(DEV), out)
    assert torch.equal(out.cpu(), plain.embed(table.float(), toks.tolist()))


@pytest.mark.parametrize("delta_dtype, out_dtype", [(torch.float32, torch.float32), (torch.float32, torch.bfloat16),
                                                    (torch.bfloat16, torch.bfloat16)])
def test_add_rms_norm(delta_dtype, out_dtype):
    from llmoxide_b200 import kernels
    T, d, S = 7, 200, 3
    h = torch.randn(T, d)
    delta = torch.randn(S, T, d).to(delta_dtype)
    gain = 1 + 0.1 * torch.randn(d)
    eps = 1e-5
    want_h = h + delta.float().sum(0)
    want = plain.rms_norm(want_h, gain, eps)
    hd = h.to(DEV)
    out = torch.empty(T, d, dtype=out_dtype, device=DEV)
    kernels.add_rms_norm(hd, delta.to(DEV), gain.to(DEV), eps, out)
    assert rel(hd, want_h) < 2e-6
    assert rel(out, want) < tol(out_dtype)
    # gathered rows, residual left alone
    rows = torch.tensor([5, 0, 5], dtype=torch.int32, device=DEV)
    hd2 = h.to(DEV)
    out2 = torch.empty(3, d, dtype=out_dtype, device=DEV)
    kernels.add_rms_norm(hd2, delta.to(DEV), gain.to(DEV), eps, out2, rows=rows, write_h=False)
    assert torch.equal(hd2.cpu(), h)
    assert rel(out2, want[[5, 0, 5]]) < tol(out_dtype)
    # no delta at all: a plain norm
    out3 = torch.empty(T, d, dtype=out_dtype, device=DEV)
    kernels.add_rms_norm(hd2, None, gain.to(DEV), eps, out3)
    assert rel(out3, plain.rms_norm(h, gain, eps)) < tol(out_dtype)


def _paged(seqs_kv, G, D, dtype, n_pages=32, shuffle=True):
    """Scatter per-sequence k, v [L,G,D] into a paged cache with a shuffled
    page order; returns k_cache, v_cache, block table."""
    rng = np.random.default_rng(5)
    order = rng.permutation(n_pages) if shuffle else np.arange(n_pages)
    k_cache = torch.full((n_pages, G, PAGE, D), float("nan"), dtype=dtype)
    v_cache = torch.full((n_pages, G, PAGE, D), float("nan"), dtype=dtype)
    width = max((len(k) + PAGE - 1) // PAGE for k, _ in seqs_kv)
    table = torch.full((len(seqs_kv), width), -1, dtype=torch.int32)
    nxt = 0
    for i, (k, v) in enumerate(seqs_kv):
        for lp in range((len(k) + PAGE - 1) // PAGE):
            page = int(order[nxt]); nxt += 1
            table[i, lp] = page
            chunk = slice(lp * PAGE, min(len(k), (lp + 1) * PAGE))
            n = chunk.stop - chunk.start
            k_cache[page, :, :n] = k[chunk].transpose(0, 1).to(dtype)
            v_cache[page, :, :n] = v[chunk].transpose(0, 1).to(dtype)
    return k_cache, v_cache, table


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("window", [None, 37])
def test_attention_paged_whole_and_single_tokens(dtype, window):
    from llmoxide_b200 import kernels
    H, G, D = 6, 3, 48
    lens = [1, 100, 300]
    torch.manual_seed(0)
    qs = [torch.randn(L, H, D).to(dtype).float() for L in lens]
    ks = [torch.randn(L, G, D).to(dtype).float() for L in lens]
    vs = [torch.randn(L, G, D).to(dtype).float() for L in lens]
    # a far key among hundreds: key 3 of the last sequence answers query 290 of head 4 loudly
    ks[2][3, 2] = 0.0
    ks[2][3, 2, :8] = 4.0
    qs[2][290, 4] = 0.0
    qs[2][290, 4, :8] = 4.0
    want = [plain.causal_attention(q, k, v, G, window) for q, k, v in zip(qs, ks, vs)]
    if window is None:
        assert torch.allclose(want[2][290, 4], vs[2][3, 2], atol=1e-3)   # the far key dominates
    kc, vc, table = _paged(list(zip(ks, vs)), G, D, dtype)
    scale = 1 / math.sqrt(D)
    # (a) all tokens of all sequences in one launch
    q_all = torch.cat(qs).reshape(-1, H * D).to(dtype)
    seq = torch.cat([torch.full((L,), i, dtype=torch.int32) for i, L in enumerate(lens)])
    pos = torch.cat([torch.arange(L, dtype=torch.int32) for L in lens])
    out = torch.empty_like(q_all, device=DEV)
    kernels.attention_paged(q_all.to(DEV), out, kc.to(DEV), vc.to(DEV), table.to(DEV), seq.to(DEV), pos.to(DEV),
                            H, G, D, window, scale)
    want_all = torch.cat(want).reshape(-1, H * D)
    assert rel(out, want_all) < tol(dtype)
    # (b) only the last token of each sequence, as a decode step does
    last = torch.tensor([sum(lens[: i + 1]) - 1 for i in range(3)])
    out2 = torch.empty(3, H * D, dtype=dtype, device=DEV)
    kernels.attention_paged(q_all[last].to(DEV), out2, kc.to(DEV), vc.to(DEV), table.to(DEV),
                            torch.arange(3, dtype=torch.int32, device=DEV),
                            torch.tensor([L - 1 for L in lens], dtype=torch.int32, device=DEV),
                            H, G, D, window, scale)
    assert rel(out2, want_all[last]) < tol(dtype)
    if dtype == torch.float32:
        assert torch.equal(out2.cpu(), out.cpu()[last])     # bit-equal however the tokens are batched


def test_attention_window_edge_is_exact():
    """The key just outside the window must not be seen, the one just inside must."""
    from llmoxide_b200 import kernels
    H = G = 1
    D, L, w = 16, 200, 70
    k = torch.zeros(L, G, D)
    v = torch.zeros(L, G, D)
    q = torch.zeros(L, H, D)
    p = 199
    q[p, 0, 0] = 8.0
    inside, outside = p - (w - 1), p - w
    k[outside, 0, 0], v[outside, 0, 1] = 50.0, 1.0     # would dominate if seen
    k[inside, 0, 0], v[inside, 0, 2] = 5.0, 1.0
    kc, vc, table = _paged([(k, v)], G, D, torch.float32)
    out = torch.empty(1, D, device=DEV)
    args = (kc.to(DEV), vc.to(DEV), table.to(DEV), torch.zeros(1, dtype=torch.int32, device=DEV),
            torch.tensor([p], dtype=torch.int32, device=DEV), H, G, D)
    kernels.attention_paged(q[p].reshape(1, D).to(DEV), out, *args, w, 0.25)
    want = plain.causal_attention(q, k, v, G, w)[p, 0]
    assert want[1] == 0 and want[2] > 0.99
    assert rel(out[0], want) < 2e-6
    kernels.attention_paged(q[p].reshape(1, D).to(DEV), out, *args, w + 1, 0.25)
    assert out[0, 1].item() > 0.99


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("D, n_rot, n_split", [(80, 32, 1), (128, 128, 1), (128, 128, 3), (128, 64, 2), (16, 16, 1)])
def test_qk_norm_rope_cache(dtype, D, n_rot, n_split):
    from llmoxide_b200 import kernels
    H, G = 3, 1
    lens, past = [5, 70], [60, 0]             # the first sequence crosses a page boundary
    T = sum(lens)
    torch.manual_seed(1)
    if n_split == 1:
        qkv = torch.randn(T, (H + 2 * G) * D).to(dtype)
        x = qkv.float()
    else:                                     # float32 partials of a split reduction, summed in order
        qkv = torch.randn(n_split, T, (H + 2 * G) * D)
        x = qkv[0].clone()
        for s_ in range(1, n_split):
            x = x + qkv[s_]
    qg, kg = 1 + 0.1 * torch.randn(D), 1 + 0.1 * torch.randn(D)
    eps, base = 1e-5, 5000.0
    pos = torch.cat([torch.arange(p, p + L) for p, L in zip(past, lens)]).to(torch.int32)
    seq = torch.cat([torch.full((L,), i) for i, L in enumerate(lens)]).to(torch.int32)
    cos, sin = plain.rope_angles(list(range(256)), n_rot, base)
    table = torch.tensor([[3, 1], [0, 2]], dtype=torch.int32)
    kc = torch.zeros(4, G, PAGE, D, dtype=dtype, device=DEV)
    vc = torch.zeros_like(kc)
    q_out = torch.empty(T, H * D, dtype=dtype, device=DEV)
    kernels.qk_norm_rope_cache(qkv.to(DEV), q_out, kc, vc, table.to(DEV), seq.to(DEV), pos.to(DEV),
                               qg.to(DEV), kg.to(DEV), eps, cos.to(DEV), sin.to(DEV), n_rot, H, G, D, True)
    q = x[:, : H * D].view(T, H, D)
    k = x[:, H * D : (H + G) * D].view(T, G, D)
    v = x[:, (H + G) * D :].view(T, G, D)
    want_q = plain.rope_neox(plain.rms_norm(q, qg, eps), pos.tolist(), base, n_rot)
    want_k = plain.rope_neox(plain.rms_norm(k, kg, eps), pos.tolist(), base, n_rot)
    assert rel(q_out.view(T, H, D), want_q) < tol(dtype)
    for t in range(T):
        page = table[seq[t], pos[t] // PAGE]
        assert rel(kc[page, :, pos[t] % PAGE], want_k[t]) < tol(dtype), t
        assert torch.equal(vc[page, :, pos[t] % PAGE].float().cpu(), v[t].to(dtype).float()), t
    # without the cache write nothing is stored and q is the same
    kc2 = torch.zeros_like(kc)
    q2 = torch.empty_like(q_out)
    kernels.qk_norm_rope_cache(qkv.to(DEV), q2, kc2, kc2, table.to(DEV), seq.to(DEV), pos.to(DEV),
                               qg.to(DEV), kg.to(DEV), eps, cos.to(DEV), sin.to(DEV), n_rot, H, G, D, False)
    assert torch.equal(q2, q_out) and not kc2.any()


@pytest.mark.parametrize("xd, wd, yd", [(torch.float32,) * 3, (torch.bfloat16,) * 3,
                                         (torch.bfloat16, torch.float32, torch.bfloat16),
                                         (torch.bfloat16, torch.bfloat16, torch.float32)])
def test_gemm_fma(xd, wd, yd):
    from llmoxide_b200 import kernels
    M, N, K = 37, 130, 75
    x, w = torch.randn(M, K).to(xd), torch.randn(N, K).to(wd)
    out = torch.empty(M, N, dtype=yd, device=DEV)
    kernels.gemm_fma(x.to(DEV), w.to(DEV), out)
    want = plain.linear(x.double(), w.double()).float()
    assert rel(out, want) < (2e-6 if yd == torch.float32 else 6e-3)
    if xd == torch.float32:
        one = torch.empty(1, N, device=DEV)
        kernels.gemm_fma(x[11:12].to(DEV), w.to(DEV), one)
        assert torch.equal(one[0], out[11])        # a row does not depend on the rows around it


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_silu_gate_and_sum_splits(dtype):
    from llmoxide_b200 import kernels
    S, T, F = 2, 9, 70
    gu = torch.randn(S, T, 2 * F).to(dtype)
    act = torch.empty(T, F, dtype=dtype, device=DEV)
    kernels.silu_gate(gu.to(DEV), act)
    g = gu.float().sum(0)
    assert rel(act, plain.silu(g[:, :F]) * g[:, F:]) < tol(dtype)
    out = torch.empty(T, 2 * F, dtype=torch.float32, device=DEV)
    kernels.sum_splits(gu.to(DEV), out)
    assert rel(out, g) < 2e-6
    # blocks of 10 gate columns followed by the 10 up columns of the same features
    blocked = g.view(T, 2, F // 10, 10).permute(0, 2, 1, 3).reshape(T, 2 * F).to(dtype)
    act2 = torch.empty(T, F, dtype=dtype, device=DEV)
    kernels.silu_gate(blocked.to(DEV), act2, block=10)
    gb = blocked.float().view(T, F // 10, 2, 10)
    assert rel(act2, (plain.silu(gb[:, :, 0]) * gb[:, :, 1]).reshape(T, F)) < tol(dtype)


def test_argmax_takes_the_last_of_equal_maxima():
    from llmoxide_b200 import kernels
    V = 5003
    logits = torch.randn(4, V)
    logits[0, [7, 4000]] = 9.0
    logits[1, 0] = 9.0
    logits[2, V - 1] = 9.0
    logits[3, [10, 11, 12]] = float("inf")
    out = torch.empty(4, dtype=torch.int32, device=DEV)
    kernels.argmax(logits.to(DEV), out)
    assert out.tolist() == [4000, 0, V - 1, 12]
    assert out.tolist() == [plain.argmax(r.numpy()) for r in logits]


@pytest.mark.parametrize("n_rows, V", [(8, 151936), (1, 151936), (64, 32000), (300, 1000), (3, 4099)])
def test_argmax_in_slices(n_rows, V):
    """Rows cut into slices over many CTAs: equal maxima in different slices, a maximum at a slice's edge, rows
    without a finite number, NaNs, and both zeros; twice, since the kernel leaves its counters for the next call."""
    from llmoxide_b200 import kernels
    g = torch.Generator().manual_seed(n_rows + V)
    logits = torch.randn(n_rows, V, generator=g)
    logits[0, [5, V // 2, V - 3]] = 7.5                       # equal maxima far apart: the last one
    if n_rows > 1:
        logits[1] = float("-inf")                             # no finite number: the last index
        logits[-1, ::7] = float("nan")
    if n_rows > 2:
        logits[2] = -1.0
        logits[2, [3, V - 2]] = torch.tensor([-0.0, 0.0])     # the two zeros are one value: the later index
        logits[2, V - 2], logits[2, 3] = -0.0, 0.0
    want = [plain.argmax(np.where(np.isnan(r.numpy()), -np.inf, r.numpy())) if not np.isnan(r.numpy()).all() else 0
            for r in logits]
    dev = logits.to(DEV)
    for _ in range(2):
        out = torch.full((n_rows,), -1, dtype=torch.int32, device=DEV)
        kernels.argmax(dev, out)
        assert out.tolist() == want


@pytest.mark.parametrize("V, top_k, top_p, temp, pen", [
    (307, 20, 0.8, 0.7, 1.0), (5003, 64, 0.95, 1.0, 1.3), (5003, 1, 1.0, 1.0, 1.0),
    (5003, 1024, 1.0, 2.0, 1.0), (307, 0, 0.9, 1.5, 1.0), (151936, 20, 0.8, 0.7, 1.1),
])
def test_sample_matches_the_plain_sampler(V, top_k, top_p, temp, pen):
    from llmoxide_b200 import kernels
    B = 24
    g = torch.Generator().manual_seed(V + top_k)
    logits = (3 * torch.randn(B, V, generator=g)).float()
    logits[:, 5] = logits[:, 9]                      # equal logits: the lower id goes first
    logits[3, :50] = float("-inf")
    recent = torch.full((B, 8), -1, dtype=torch.int32)
    for b in range(B):
        top = torch.topk(logits[b], 3).indices
        recent[b, :3] = top.to(torch.int32)
        recent[b, 3] = top[0]                        # a token twice in the window is penalised twice
    u = torch.rand(B, generator=g)
    u[0], u[1] = 0.0, 0.9999999
    dev = lambda t: t.to(DEV)
    out = torch.empty(B, dtype=torch.int32, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    work = dev(logits.clone())
    kernels.sample(work, dev(torch.full((B,), temp)), dev(torch.full((B,), top_k, dtype=torch.int32)),
                   dev(torch.full((B,), top_p)), dev(torch.full((B,), pen)), dev(recent), dev(u), out, status)
    assert status.item() == 0
    got = out.tolist()
    mismatches = []
    for b in range(B):
        rec = [t for t in recent[b].tolist() if t >= 0]
        want = plain.sample(logits[b].numpy(), rec, temperature=temp, top_k=top_k, top_p=top_p,
                            repeat_penalty=pen, repeat_window=64, u=float(u[b]))
        if got[b] != want:
            mismatches.append((b, got[b], want))
    # expf on the device and exp on the host may differ in the last bit, which can
    # move a draw that sits on the edge between two tokens; more than one in 24 is a fault
    assert len(mismatches) <= 1, mismatches


@pytest.mark.parametrize("top_k", [64, 1024])
def test_sample_with_many_equal_logits_at_the_threshold(top_k):
    """Logits that take a dozen values only, so that the k-th largest is shared by a hundred others of which
    a few belong to the top k: those with the lowest ids.  With k = 64 the logits at or above the threshold's
    binade are few and the kernel sorts them all; with k = 1024 they are more than 1024 and it selects byte by
    byte and takes the equal ones in id order."""
    from llmoxide_b200 import kernels
    V, B = 5003, 16
    g = torch.Generator().manual_seed(top_k)
    logits = torch.round(2 * torch.randn(B, V, generator=g)).float()
    u = torch.rand(B, generator=g)
    u[0], u[1] = 0.0, 0.9999999                    # the first and the last of the kept tokens
    dev = lambda t: t.to(DEV)
    out = torch.empty(B, dtype=torch.int32, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    kernels.sample(dev(logits.clone()), dev(torch.ones(B)), dev(torch.full((B,), top_k, dtype=torch.int32)),
                   dev(torch.ones(B)), None, None, dev(u), out, status)
    assert status.item() == 0
    want = [plain.sample(logits[b].numpy(), [], temperature=1.0, top_k=top_k, top_p=1.0, repeat_penalty=1.0,
                         repeat_window=64, u=float(u[b])) for b in range(B)]
    wrong = [(b, g_, w) for b, (g_, w) in enumerate(zip(out.tolist(), want)) if g_ != w]
    assert len(wrong) <= 1, wrong                  # (a draw on the edge between two tokens may fall either way)
    # every chosen token is one of the top k in the order (value down, id up)
    for b, tok in enumerate(out.tolist()):
        order = sorted(range(V), key=lambda i: (-float(logits[b, i]), i))[:top_k]
        assert tok in order, (b, tok)


def test_sample_whole_vocabulary_follows_the_distribution():
    from llmoxide_b200 import kernels
    V, B = 3000, 4096
    base = torch.zeros(V)
    base[[10, 2000, 2999]] = torch.tensor([2.0, 1.0, 0.0])
    base[[0, 1, 2]] = -30.0
    base[3:10] = -40.0
    base[11:2000] = -50.0
    base[2001:2999] = -50.0
    logits = base.repeat(B, 1).clone()
    g = torch.Generator().manual_seed(1)
    u = torch.rand(B, generator=g)
    out = torch.empty(B, dtype=torch.int32, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    dev = lambda t: t.to(DEV)
    kernels.sample(dev(logits), dev(torch.ones(B)), dev(torch.zeros(B, dtype=torch.int32)), dev(torch.ones(B)),
                   None, None, dev(u), out, status)
    assert status.item() == 0
    counts = torch.bincount(out.cpu().long(), minlength=V).float() / B
    p = torch.softmax(base, 0)
    for t in (10, 2000, 2999):
        assert abs(counts[t] - p[t]) < 0.03, (t, counts[t], p[t])
    # the walk is in id order: small u lands on the lowest ids with mass
    assert out[u.argmin()].item() <= 10
    # top_p < 1 over a whole large vocabulary is refused, not approximated
    kernels.sample(dev(logits), dev(torch.ones(B)), dev(torch.zeros(B, dtype=torch.int32)),
                   dev(torch.full((B,), 0.5)), None, None, dev(u), out, status)
    assert status.item() != 0


@pytest.mark.parametrize("T, N, K", [(1, 256, 64), (8, 384, 512), (64, 200, 1000), (130, 520, 320),
                                     (300, 128, 4096), (5, 1000, 72),
                                     # more work units than resident CTAs: a CTA walks several units
                                     (8, 40000, 128), (600, 7680, 192), (300, 20480, 128), (40, 10240, 640)])
def test_gemm_tc(T, N, K):
    """The tcgen05 kernel against float64, plain, split and gated."""
    from llmoxide_b200 import kernels
    g = torch.Generator().manual_seed(T * N)
    x = torch.randn(T, K, generator=g).bfloat16()
    w = (torch.randn(N, K, generator=g) / math.sqrt(K)).bfloat16()
    x[:, K // 3] *= 30                     # one loud column: a misplaced K block shows
    want = x.double() @ w.double().t()
    xd, wd = x.to(DEV), w.to(DEV)
    assert kernels.gemm_tc_supports(xd, wd)
    out32 = torch.empty(T, N, dtype=torch.float32, device=DEV)
    kernels.gemm_tc(xd, wd, out32)
    assert rel(out32, want) < 1e-5
    out16 = torch.empty(T, N, dtype=torch.bfloat16, device=DEV)
    kernels.gemm_tc(xd, wd, out16)
    assert rel(out16, want) < 6e-3
    for s in (2, 3):
        parts = torch.full((s, T, N), float("nan"), dtype=torch.float32, device=DEV)
        kernels.gemm_tc(xd, wd, parts, n_split=s)
        assert rel(parts.sum(0), want) < 1e-5
    if N % 2 == 0:
        F = N // 2
        act = torch.empty(T, F, dtype=torch.bfloat16, device=DEV)
        kernels.gemm_tc(xd, wd, act, gated=True)
        gate, up = want[:, :F].float(), want[:, F:].float()
        assert rel(act, plain.silu(gate) * up) < 8e-3
    if N % 32 == 0:       # rows in blocks of 16 gate rows + the 16 up rows of the same features
        F = N // 2
        blocks = want.float().view(T, N // 32, 2, 16)
        act = torch.full((T, F), float("nan"), dtype=torch.bfloat16, device=DEV)
        kernels.gemm_tc(xd, wd, act, gated=2)
        assert rel(act, (plain.silu(blocks[:, :, 0]) * blocks[:, :, 1]).reshape(T, F)) < 8e-3
    assert kernels.gemm_tc_status() == 0


def test_gemm_tc_pair_token_tile_groups():
    """So many tokens that their activations no longer share L2: the CTA-pair kernel walks the token tiles
    in groups (here two groups of sixteen tiles, the last tile partly empty).  Neighbouring token tiles differ
    in loudness, so a tile computed for the wrong place shows."""
    from llmoxide_b200 import kernels
    T, N, K = 8000, 768, 4096
    g = torch.Generator().manual_seed(5)
    x = torch.randn(T, K, generator=g).bfloat16()
    x *= (1 + (torch.arange(T) // 256) % 7).to(torch.bfloat16)[:, None]
    w = (torch.randn(N, K, generator=g) / math.sqrt(K)).bfloat16()
    xd, wd = x.to(DEV), w.to(DEV)
    want = (xd.double() @ wd.double().t()).cpu()
    out = torch.full((T, N), float("nan"), dtype=torch.float32, device=DEV)
    kernels.gemm_tc(xd, wd, out, pair=True)
    assert kernels.gemm_tc_status() == 0
    assert rel(out, want) < 1e-5
    for tile in range(0, T, 256):
        assert rel(out[tile:tile + 256], want[tile:tile + 256]) < 1e-5, tile


@pytest.mark.parametrize("T, N, K", [(129, 256, 64), (300, 520, 320), (2048, 1024, 512), (600, 20480, 192),
                                     (1000, 200, 1000), (257, 4096 + 128, 4096),
                                     # more units than CTA pairs, and not a multiple of them: a last round partly empty
                                     (2048, 4096, 1024), (700, 9728, 520), (2048, 6144, 4096), (1500, 2560, 72)])
def test_gemm_tc_pair(T, N, K):
    """The CTA-pair (cta_group::2) kernel against float64, plain and gated."""
    from llmoxide_b200 import kernels
    g = torch.Generator().manual_seed(T + N)
    x = torch.randn(T, K, generator=g).bfloat16()
    w = (torch.randn(N, K, generator=g) / math.sqrt(K)).bfloat16()
    x[:, K // 3] *= 30
    x[T // 2] *= 5                         # one loud token: a swapped half of the token tile shows
    want = x.double() @ w.double().t()
    xd, wd = x.to(DEV), w.to(DEV)
    out32 = torch.full((T, N), float("nan"), dtype=torch.float32, device=DEV)
    kernels.gemm_tc(xd, wd, out32, pair=True)
    assert kernels.gemm_tc_status() == 0
    assert rel(out32, want) < 1e-5
    again = torch.full((T, N), float("nan"), dtype=torch.float32, device=DEV)
    kernels.gemm_tc(xd, wd, again, pair=True)          # the same bits every time
    assert torch.equal(again, out32)
    out16 = torch.empty(T, N, dtype=torch.bfloat16, device=DEV)
    kernels.gemm_tc(xd, wd, out16, pair=True)
    assert rel(out16, want) < 6e-3
    for n_split in (2, 3):        # the reduction cut into splits: float32 partials, one plane each
        if K >= 128 * n_split:
            parts = torch.full((n_split, T, N), float("nan"), dtype=torch.float32, device=DEV)
            kernels.gemm_tc(xd, wd, parts, n_split=n_split, pair=True)
            assert kernels.gemm_tc_status() == 0
            assert rel(parts.sum(0), want) < 1e-5, n_split
    if N % 4 == 0:        # Y += X W^T: one float32 addition per element, the same bits as adding the product
        base = torch.randn(T, N, generator=g).to(DEV)
        acc = base.clone()
        kernels.gemm_tc(xd, wd, acc, pair=True, accumulate=True)
        assert torch.equal(acc, base + out32)
    if N % 2 == 0:
        F = N // 2
        act = torch.full((T, F), float("nan"), dtype=torch.bfloat16, device=DEV)
        kernels.gemm_tc(xd, wd, act, gated=True, pair=True)
        gate, up = want[:, :F].float(), want[:, F:].float()
        assert rel(act, plain.silu(gate) * up) < 8e-3
    if N % 32 == 0:
        F = N // 2
        blocks = want.float().view(T, N // 32, 2, 16)
        act = torch.full((T, F), float("nan"), dtype=torch.bfloat16, device=DEV)
        kernels.gemm_tc(xd, wd, act, gated=2, pair=True)
        assert rel(act, (plain.silu(blocks[:, :, 0]) * blocks[:, :, 1]).reshape(T, F)) < 8e-3
    assert kernels.gemm_tc_status() == 0


def test_gemm_tc_refuses_what_it_cannot_do():
    from llmoxide_b200 import kernels
    x = torch.randn(4, 76).bfloat16().to(DEV)       # K not a multiple of 8
    w = torch.randn(16, 76).bfloat16().to(DEV)
    assert not kernels.gemm_tc_supports(x, w)
    with pytest.raises(Exception):
        kernels.gemm_tc(x, w, torch.empty(4, 16, dtype=torch.bfloat16, device=DEV))


def _attention_case(H, G, D, lens, pasts, window, seed=0, n_pages=64):
    """Sequences with ``pasts[i]`` cached positions and ``lens[i]`` new tokens;
    returns everything the bfloat16 attention kernels need and the plain result
    for the new tokens."""
    torch.manual_seed(seed)
    qs, ks, vs, want = [], [], [], []
    for L, P in zip(lens, pasts):
        n = P + L
        q = torch.randn(n, H, D).bfloat16().float()
        k = torch.randn(n, G, D).bfloat16().float()
        v = torch.randn(n, G, D).bfloat16().float()
        if n > 40:      # a far key among many answers one late query loudly
            k[2, G - 1] = 0.0
            k[2, G - 1, :8] = 3.0
            q[n - 1, H - 1] = 0.0
            q[n - 1, H - 1, :8] = 3.0
        full = plain.causal_attention(q, k, v, G, window)
        qs.append(q[P:]), ks.append(k), vs.append(v), want.append(full[P:])
    kc, vc, table = _paged(list(zip(ks, vs)), G, D, torch.bfloat16, n_pages=n_pages)
    starts = torch.tensor([0] + list(np.cumsum(lens)), dtype=torch.int32)
    q_all = torch.cat(qs).reshape(-1, H * D).bfloat16()
    return q_all, kc, vc, table, starts, torch.tensor(pasts, dtype=torch.int32), torch.cat(want).reshape(-1, H * D)


@pytest.mark.parametrize("H, G, D", [(8, 2, 128), (6, 6, 64), (5, 1, 128)])
@pytest.mark.parametrize("window", [None, 100])
def test_attention_prefill_tiled(H, G, D, window):
    from llmoxide_b200 import kernels
    lens, pasts = [1, 64, 200, 65, 130], [0, 0, 0, 70, 300]     # whole prompts and later chunks of prompts
    q, kc, vc, table, starts, past, want = _attention_case(H, G, D, lens, pasts, window)
    out = torch.full_like(q, float("nan"), device=DEV)
    kernels.attention_prefill(q.to(DEV), out, kc.to(DEV), vc.to(DEV), table.to(DEV), starts.to(DEV), past.to(DEV),
                              len(lens), max(lens), H, G, D, window, 1 / math.sqrt(D))
    assert not out.isnan().any()
    for i in range(len(lens)):
        lo, hi = starts[i], starts[i + 1]
        assert rel(out[lo:hi], want[lo:hi]) < 1.2e-2, (i, lens[i], pasts[i])


@pytest.mark.parametrize("H, G", [(8, 2), (5, 1), (3, 3)])
@pytest.mark.parametrize("window", [None, 100, 300])
def test_attention_prefill_tcgen05(H, G, window):
    from llmoxide_b200 import kernels
    D = 128
    lens, pasts = [1, 64, 200, 65, 130, 700], [0, 0, 0, 70, 300, 0]   # whole prompts and later chunks of prompts
    q, kc, vc, table, starts, past, want = _attention_case(H, G, D, lens, pasts, window)
    out = torch.full_like(q, float("nan"), device=DEV)
    kernels.attention_prefill_tc(q.to(DEV), out, kc.to(DEV), vc.to(DEV), table.to(DEV), starts.to(DEV), past.to(DEV),
                                 len(lens), max(lens), H, G, D, window, 1 / math.sqrt(D))
    assert kernels.attention_prefill_tc_status() == 0
    assert not out.isnan().any()
    for i in range(len(lens)):
        lo, hi = starts[i], starts[i + 1]
        assert rel(out[lo:hi], want[lo:hi]) < 1.2e-2, (i, lens[i], pasts[i])


@pytest.mark.parametrize("H, G, D", [(8, 2, 128), (6, 6, 64), (5, 1, 48), (16, 2, 80), (4, 4, 256), (24, 2, 16)])
@pytest.mark.parametrize("window", [None, 100])
def test_attention_decode_split(H, G, D, window):
    from llmoxide_b200 import kernels
    pasts = [0, 63, 64, 500, 1500, 129]
    lens = [1] * len(pasts)
    q, kc, vc, table, starts, past, want = _attention_case(H, G, D, lens, pasts, window)
    out = torch.full_like(q, float("nan"), device=DEV)
    kernels.attention_decode(q.to(DEV), out, kc.to(DEV), vc.to(DEV), table.to(DEV), past.to(DEV), H, G, D, window,
                             1 / math.sqrt(D))
    assert not out.isnan().any()
    for i in range(len(pasts)):
        assert rel(out[i], want[i]) < 1.2e-2, (i, pasts[i])
    # a wider block table (another split of the keys) gives the same result up to rounding
    wide = torch.full((len(pasts), 64), -1, dtype=torch.int32)
    wide[:, : table.shape[1]] = table
    out2 = torch.empty_like(out)
    kernels.attention_decode(q.to(DEV), out2, kc.to(DEV), vc.to(DEV), wide.to(DEV), past.to(DEV), H, G, D, window,
                             1 / math.sqrt(D))
    assert rel(out2, out) < 1e-2
    # and again: the arrival counters were left at zero
    out3 = torch.full_like(out, float("nan"))
    kernels.attention_decode(q.to(DEV), out3, kc.to(DEV), vc.to(DEV), table.to(DEV), past.to(DEV), H, G, D, window,
                             1 / math.sqrt(D))
    assert torch.equal(out3, out)
    # more than 8 shares: merged through the workspace by the CTA that arrives last; twice (the counters return to zero)
    for _ in range(2):
        out4 = torch.full_like(out, float("nan"))
        kernels.attention_decode(q.to(DEV), out4, kc.to(DEV), vc.to(DEV), table.to(DEV), past.to(DEV), H, G, D, window,
                                 1 / math.sqrt(D), n_chunks=11)
        assert rel(out4, out) < 1e-2
    # and one share
    out5 = torch.full_like(out, float("nan"))
    kernels.attention_decode(q.to(DEV), out5, kc.to(DEV), vc.to(DEV), table.to(DEV), past.to(DEV), H, G, D, window,
                             1 / math.sqrt(D), n_chunks=1)
    assert rel(out5, out) < 1e-2
    assert kernels.attention_decode_status() == 0


def test_attention_decode_many_sequences_one_share_each():
    """A batch that fills the GPU by itself: every sequence's keys stay in one CTA and nothing is merged."""
    from llmoxide_b200 import kernels
    H, G, D = 8, 4, 64
    pasts = [(37 * i) % 260 for i in range(80)]
    assert kernels.decode_chunks(len(pasts), G, H // G, 5) == 1
    q, kc, vc, table, starts, past, want = _attention_case(H, G, D, [1] * len(pasts), pasts, None, n_pages=256)
    out = torch.full_like(q, float("nan"), device=DEV)
    kernels.attention_decode(q.to(DEV), out, kc.to(DEV), vc.to(DEV), table.to(DEV), past.to(DEV), H, G, D, None,
                             1 / math.sqrt(D))
    assert not out.isnan().any()
    for i in range(len(pasts)):
        assert rel(out[i], want[i]) < 1.2e-2, (i, pasts[i])


# ---- the window's edge in the bfloat16 kernels ----------------------------------------------------

def _edge_case(D, past, n_new, window, rows):
    """One sequence, one head.  For every tested new token (``rows``, indices among the new tokens) the key
    just outside its window is loud and marks one output dim, the key just inside is a little less loud and
    marks another; each tested row listens on a dim of its own, so that the rows' edges (which may be
    neighbours) do not disturb one another.  Seeing the outside key, or missing the inside one, changes
    the marked outputs from (0, 1) to (1, 0) or (0, 0)."""
    n = past + n_new
    q = torch.zeros(n, 1, D)
    k = torch.zeros(n, 1, D)
    v = torch.zeros(n, 1, D)
    marks = []
    for j, r in enumerate(rows):
        pos = past + r
        inside, outside = pos - (window - 1), pos - window
        assert outside >= 0
        q[pos, 0, j] = 8.0
        k[outside, 0, j] = 50.0
        k[inside, 0, j] = 40.0
        v[outside, 0, 8 + 2 * j] = 1.0
        v[inside, 0, 9 + 2 * j] = 1.0
        marks.append((r, 8 + 2 * j, 9 + 2 * j))
    kc, vc, table = _paged([(k, v)], 1, D, torch.bfloat16, n_pages=(n + PAGE - 1) // PAGE + 3)
    return q[past:].reshape(n_new, D).bfloat16(), kc, vc, table, marks


def _assert_edge(out, marks, what):
    out = out.float().cpu()
    for r, dim_out, dim_in in marks:
        assert float(out[r, dim_out]) < 1e-3, (what, r, "the key just outside the window was seen")
        assert float(out[r, dim_in]) > 0.999, (what, r, "the key just inside the window was missed")


@pytest.mark.parametrize("off", [0, 31, 63])
@pytest.mark.parametrize("D", [128, 64, 48])
def test_window_edge_decode_attention(D, off):
    from llmoxide_b200 import kernels
    p = 700
    window = p - (128 + off) + 1                     # the first visible key sits at offset `off` of a page
    q, kc, vc, table, marks = _edge_case(D, p, 1, window, [0])
    for n_chunks in (1, 3, 8, 11):
        out = torch.full((1, D), float("nan"), dtype=torch.bfloat16, device=DEV)
        kernels.attention_decode(q.to(DEV), out, kc.to(DEV), vc.to(DEV), table.to(DEV),
                                 torch.tensor([p], dtype=torch.int32, device=DEV), 1, 1, D, window, 1 / math.sqrt(D),
                                 n_chunks=n_chunks)
        _assert_edge(out, marks, f"decode, {n_chunks} shares, offset {off}")


@pytest.mark.parametrize("off", [0, 31, 63])
@pytest.mark.parametrize("n_new", [2, 129])
@pytest.mark.parametrize("kernel, D", [("tcgen05", 128), ("tiled", 128), ("tiled", 64)])
def test_window_edge_prompt_attention(kernel, D, n_new, off):
    """A later portion of a prompt (``past`` > 0) of 2 tokens (the edge in the first key tile) and of 129
    (rows of two query tiles; the edge falls in tiles that only some rows mask)."""
    from llmoxide_b200 import kernels
    past = 400
    window = past - (128 + off) + 1
    rows = sorted({0, n_new - 1, n_new // 2})
    q, kc, vc, table, marks = _edge_case(D, past, n_new, window, rows)
    out = torch.full((n_new, D), float("nan"), dtype=torch.bfloat16, device=DEV)
    fn = kernels.attention_prefill_tc if kernel == "tcgen05" else kernels.attention_prefill
    fn(q.to(DEV), out, kc.to(DEV), vc.to(DEV), table.to(DEV), torch.tensor([0, n_new], dtype=torch.int32, device=DEV),
       torch.tensor([past], dtype=torch.int32, device=DEV), 1, n_new, 1, 1, D, window, 1 / math.sqrt(D))
    assert not out.isnan().any()
    _assert_edge(out, marks, f"{kernel} D={D}, {n_new} new tokens, offset {off}")


def test_softcap_and_scaled_embedding():
    from llmoxide_b200 import kernels
    x = torch.randn(7, 333) * 40
    d = x.to(DEV)
    kernels.softcap(d, 30.0)
    assert rel(d, 30.0 * torch.tanh(x / 30.0)) < 2e-6
    table = torch.randn(50, 72)
    toks = torch.tensor([3, 49, 0], dtype=torch.int32)
    out = torch.empty(3, 72, dtype=torch.float32, device=DEV)
    kernels.embed(table.to(DEV), toks.to(DEV), out, 8.5)
    assert torch.equal(out.cpu(), table[toks.long()] * 8.5)


@pytest.mark.parametrize("T, d, N2", [(8, 512, 768), (1, 200, 256), (64, 1152, 384), (37, 4096, 256), (5, 8200, 128)])
def test_norm_in_two_halves(T, d, N2):
    """The residual add + RMSNorm of a step of few tokens as two halves: sums of squares per slice from one
    kernel, the scale in the epilogue of the product that follows; against the same in plain float32.  The
    residual stream is bit-equal to what the one-kernel norm gives."""
    from llmoxide_b200 import kernels
    g = torch.Generator().manual_seed(T + d)
    w2 = (torch.randn(N2, d, generator=g) / math.sqrt(d)).bfloat16()
    h0 = torch.randn(T, d, generator=g) * 3
    gain = 1 + 0.1 * torch.randn(d, generator=g)
    eps = 1e-5
    w2d, gd = w2.to(DEV), gain.to(DEV)
    parts = (d + kernels.ADD_SLICE - 1) // kernels.ADD_SLICE
    for n_split, ddtype in ((0, None), (1, torch.bfloat16), (3, torch.float32), (9, torch.float32), (16, torch.float32)):
        delta = None if n_split == 0 else torch.randn(n_split, T, d, generator=g).to(ddtype)
        want_h = h0 if delta is None else h0 + delta.float().sum(0)
        want_y = plain.rms_norm(want_h, gain, eps) @ w2.float().t()
        dd = None if delta is None else delta.to(DEV)
        h = h0.to(DEV)
        x = torch.full((T, d), float("nan"), dtype=torch.bfloat16, device=DEV)
        sumsq = torch.full((parts, max(T, 8)), float("nan"), dtype=torch.float32, device=DEV)
        kernels.add_gain_sumsq(h, dd, gd, x, sumsq)
        h_ref, x_ref = h0.to(DEV), torch.empty((T, d), dtype=torch.bfloat16, device=DEV)
        kernels.add_rms_norm(h_ref, dd, gd, eps, x_ref)
        assert torch.equal(h, h_ref), n_split
        assert rel(sumsq[:, :T].sum(0), (want_h * want_h).sum(1)) < 1e-5
        assert rel(x, want_h * gain) < 6e-3
        y = torch.empty((T, N2), dtype=torch.float32, device=DEV)
        kernels.gemm_tc(x, w2d, y, scale=(sumsq, parts, eps, d))
        assert rel(y, want_y) < 6e-3, n_split
        if d // 64 >= 2:
            y2 = torch.empty((2, T, N2), dtype=torch.float32, device=DEV)
            kernels.gemm_tc(x, w2d, y2, n_split=2, scale=(sumsq, parts, eps, d))
            assert rel(y2.sum(0), want_y) < 6e-3
        if N2 % 128 == 0:        # the gated epilogue scales before the activation
            F = N2 // 2
            act = torch.empty((T, F), dtype=torch.bfloat16, device=DEV)
            kernels.gemm_tc(x, w2d, act, gated=True, scale=(sumsq, parts, eps, d))
            assert rel(act, plain.silu(want_y[:, :F]) * want_y[:, F:]) < 1e-2
            blocks = want_y.view(T, N2 // 32, 2, 16)
            kernels.gemm_tc(x, w2d, act, gated=2, scale=(sumsq, parts, eps, d))
            assert rel(act, (plain.silu(blocks[:, :, 0]) * blocks[:, :, 1]).reshape(T, F)) < 1e-2
    assert kernels.gemm_tc_status() == 0
