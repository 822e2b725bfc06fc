"""GPU: the decode attention entry point for callers that must not allocate
(a server that gave all device memory to its own pool, a latency-critical loop
that cannot afford cudaMalloc's device-wide synchronisation).  Its workspace
is a fixed array inside the library.  Called here through the exported C
symbol, several times in a row, and compared with the ordinary entry point
(whose workspace the caller allocates: the same kernel, the same shares and
the same merge order, so the outputs must be bit-equal) and with the plain
attention of the tests.  The file sorts last so that a run that stops at the
first failure has already run every other test."""

import ctypes
import math
from ctypes import c_float, c_int, c_void_p

import pytest
import torch

import plain_qwen3 as plain

pytestmark = pytest.mark.gpu

PAGE = 64
WS_FLOATS = 4 * 1024 * 1024      # LLMX_NOALLOC_WS_FLOATS
COUNTERS = 4096                  # LLMX_NOALLOC_COUNTERS
TOO_LARGE = -5                   # LLMX_NOALLOC_TOO_LARGE


def _case(B, H, G, D, lengths, seed):
    """A paged cache with every sequence's keys and values, NaN in every row no sequence owns."""
    g = torch.Generator().manual_seed(seed)
    n_pages = sum((n + PAGE - 1) // PAGE for n in lengths) + 2
    kc = torch.full((n_pages, G, PAGE, D), float("nan"))
    vc = torch.full((n_pages, G, PAGE, D), float("nan"))
    width = max((n + PAGE - 1) // PAGE for n in lengths)
    table = torch.full((B, width), -1, dtype=torch.int32)
    seqs, nxt = [], 1
    for b, n in enumerate(lengths):
        k = torch.randn(n, G, D, generator=g).bfloat16().float()
        v = torch.randn(n, G, D, generator=g).bfloat16().float()
        seqs.append((k, v))
        for lp in range((n + PAGE - 1) // PAGE):
            rows = slice(lp * PAGE, min(n, (lp + 1) * PAGE))
            kc[nxt, :, : rows.stop - rows.start] = k[rows].transpose(0, 1)
            vc[nxt, :, : rows.stop - rows.start] = v[rows].transpose(0, 1)
            table[b, lp] = nxt
            nxt += 1
    q = torch.randn(B, H * D, generator=g).bfloat16()
    past = torch.tensor([n - 1 for n in lengths], dtype=torch.int32)        # the new token's position
    return q, kc.bfloat16().cuda(), vc.bfloat16().cuda(), table.cuda(), past.cuda(), seqs


def _plain(q, seqs, H, G, D, window):
    """The last query of every sequence by the plain implementation."""
    return torch.stack([_last_row(q[b].float().view(H, D), k, v, G, window) for b, (k, v) in enumerate(seqs)])


def _last_row(q_last, k, v, G, window):
    """plain.causal_attention takes whole sequences: the visible keys first..n-1 are made one, the query
    sits at its last position, and that position's row is the answer."""
    n, H, D = k.shape[0], q_last.shape[0], q_last.shape[1]
    first = 0 if window is None else max(0, (n - 1) - (window - 1))
    qs = torch.zeros(n - first, H, D)
    qs[-1] = q_last
    return plain.causal_attention(qs, k[first:], v[first:], G, None)[-1].reshape(-1)


def test_no_alloc_entry_point_matches_the_allocating_one():
    from llmoxide_b200 import kernels
    from llmoxide_b200.csrc.build import load_library

    lib = load_library("attention_decode")
    fn = lib.llmx_attention_decode_noalloc
    fn.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, ctypes.c_longlong, c_void_p, c_int, c_void_p, c_int, c_int,
                   c_int, c_int, c_int, c_float, c_int, c_void_p]
    fn.restype = c_int
    H, G, D = 8, 2, 128
    scale = 1 / math.sqrt(D)
    stream = c_void_p(torch.cuda.current_stream().cuda_stream)

    def call(q, out, kc, vc, table, past, B, window, n_chunks, h=H, g=G):
        return fn(q.data_ptr(), out.data_ptr(), kc.data_ptr(), vc.data_ptr(), kc.shape[0], table.data_ptr(),
                  table.shape[1], past.data_ptr(), B, h, g, D, window, scale, n_chunks, stream)

    # calls in a row on the shared arrays: beyond 8 shares (through the workspace), with and without a
    # window, and up to 8 shares (merged in a cluster, the arrays untouched)
    cases = [([700, 65, 1, 300], 0, 10), ([129, 640, 64, 2], 0, 11), ([500, 90, 333, 64], 100, 12),
             ([700, 65, 1, 300], 0, 4), ([129, 640, 64, 2], 70, 8)]
    for i, (lengths, window, n_chunks) in enumerate(cases):
        B = len(lengths)
        q, kc, vc, table, past, seqs = _case(B, H, G, D, lengths, seed=i)
        qd = q.cuda()
        want = torch.empty_like(qd)
        kernels.attention_decode(qd, want, kc, vc, table, past, H, G, D, window or None, scale, n_chunks=n_chunks)
        got = torch.full_like(qd, float("nan"))
        assert call(qd, got, kc, vc, table, past, B, window, n_chunks) == 0
        torch.cuda.synchronize()
        assert not got.isnan().any()
        assert torch.equal(got, want), (i, "the same kernel with the same shares must give the same bits")
        ref = _plain(q, seqs, H, G, D, window or None)
        err = (got.float().cpu() - ref).abs().max() / ref.abs().max()
        assert err < 6e-3, (i, float(err))     # the kernel tests' tolerance for one bfloat16 rounding
    # beyond 8 shares a request larger than the fixed workspace is refused, and nothing runs
    big_chunks = WS_FLOATS // (B * H * (D + 4)) + 1
    assert big_chunks > 8
    got.fill_(float("nan"))
    assert call(qd, got, kc, vc, table, past, B, 0, big_chunks) == TOO_LARGE
    # so is one with more (sequence, kv head, head group) counters than the library holds
    Bc = COUNTERS // G + 1
    assert call(qd, got, kc, vc, table, past, Bc, 0, 9) == TOO_LARGE
    torch.cuda.synchronize()
    assert got.isnan().all()
    # up to 8 shares no limit applies: sizes that the workspace formula would refuse run (cluster merge)
    many, heads = 64, 64
    assert many * heads * 8 * (D + 4) > WS_FLOATS
    q, kc, vc, table, past, seqs = _case(many, heads, 1, D, [300] * many, seed=9)
    qd = q.cuda()
    got2, want2 = torch.full_like(qd, float("nan")), torch.empty_like(qd)
    kernels.attention_decode(qd, want2, kc, vc, table, past, heads, 1, D, None, scale, n_chunks=8)
    assert call(qd, got2, kc, vc, table, past, many, 0, 8, h=heads, g=1) == 0
    torch.cuda.synchronize()
    assert torch.equal(got2, want2)
    # after the refusals the counters are still zero: a workspace call gives the same bits again
    lengths, window, n_chunks = cases[0]
    q, kc, vc, table, past, seqs = _case(len(lengths), H, G, D, lengths, seed=0)
    qd = q.cuda()
    want, got = torch.empty_like(qd), torch.full_like(qd, float("nan"))
    kernels.attention_decode(qd, want, kc, vc, table, past, H, G, D, None, scale, n_chunks=n_chunks)
    assert call(qd, got, kc, vc, table, past, len(lengths), 0, n_chunks) == 0
    torch.cuda.synchronize()
    assert torch.equal(got, want)
