"""GPU: the decode attention entry point for callers that must not allocate
(a server that gave all device memory to its own pool, a latency-critical loop
that cannot afford cudaMalloc's device-wide synchronisation).  Its workspace
is a fixed array inside the library.  Called here through the exported C
symbol, twice in a row, and compared with the ordinary entry point, whose
workspace the caller allocates.  The file sorts last so that a run that stops
at the first failure has already run every other test."""

import ctypes
import math
from ctypes import c_float, c_int, c_void_p

import pytest
import torch

pytestmark = pytest.mark.gpu

PAGE = 64
WS_FLOATS = 4 * 1024 * 1024      # LLMX_NOALLOC_WS_FLOATS
TOO_LARGE = -5                   # LLMX_NOALLOC_TOO_LARGE


def _case(B, H, G, D, lengths, seed):
    g = torch.Generator().manual_seed(seed)
    n_pages = sum((n + PAGE - 1) // PAGE for n in lengths) + 2
    kc = torch.randn(n_pages, G, PAGE, D, generator=g).bfloat16().cuda()
    vc = torch.randn(n_pages, G, PAGE, D, generator=g).bfloat16().cuda()
    width = max((n + PAGE - 1) // PAGE for n in lengths)
    table = torch.full((B, width), -1, dtype=torch.int32)
    nxt = 1
    for b, n in enumerate(lengths):
        for lp in range((n + PAGE - 1) // PAGE):
            table[b, lp] = nxt
            nxt += 1
    q = torch.randn(B, H * D, generator=g).bfloat16().cuda()
    past = torch.tensor([n - 1 for n in lengths], dtype=torch.int32).cuda()   # the new token's position
    return q, kc, vc, table.cuda(), past


def test_no_alloc_entry_point_matches_the_allocating_one():
    from llmoxide_b200 import kernels
    from llmoxide_b200.csrc.build import load_library

    lib = load_library("attention_decode")
    fn = lib.llmx_attention_decode_noalloc
    fn.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, ctypes.c_longlong, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int,
                   c_int, c_float, c_int, c_void_p]
    fn.restype = c_int
    H, G, D = 8, 2, 128
    scale = 1 / math.sqrt(D)
    stream = c_void_p(torch.cuda.current_stream().cuda_stream)
    for call, lengths in enumerate(([700, 65, 1, 300], [129, 640, 64, 2])):     # two calls in a row
        B = len(lengths)
        q, kc, vc, table, past = _case(B, H, G, D, lengths, seed=call)
        want = torch.empty_like(q)
        n_chunks = 10 + call                # beyond 8 chunks the partials go through the workspace
        kernels.attention_decode(q, want, kc, vc, table, past, H, G, D, None, scale, n_chunks=n_chunks)
        got = torch.full_like(q, float("nan"))
        rc = fn(q.data_ptr(), got.data_ptr(), kc.data_ptr(), vc.data_ptr(), kc.shape[0], table.data_ptr(), table.shape[1],
                past.data_ptr(), B, H, G, D, 0, scale, n_chunks, stream)
        assert rc == 0
        torch.cuda.synchronize()
        assert not got.isnan().any()
        err = (got.float() - want.float()).abs().max() / want.float().abs().max()
        assert err < 6e-3, (call, float(err))      # the kernel tests' tolerance for one bfloat16 rounding
    # a request beyond the fixed workspace is refused, and nothing runs
    big_chunks = WS_FLOATS // (B * H * (D + 4)) + 1
    rc = fn(q.data_ptr(), got.data_ptr(), kc.data_ptr(), vc.data_ptr(), kc.shape[0], table.data_ptr(), table.shape[1],
            past.data_ptr(), B, H, G, D, 0, scale, big_chunks, stream)
    assert rc == TOO_LARGE
