"""Typed Python faces of the ``extern "C"`` kernel launchers.

Each function checks what the kernel cannot check for itself (device, dtype,
contiguity, shapes), passes raw pointers and the current CUDA stream, and
turns a refusal or a launch error into an exception.  Nothing here computes
on the host and nothing falls back to another implementation.
"""

from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_longlong, c_void_p

import torch

from . import guard
from .csrc.build import load_library
from .errors import ExtensionMissing, KernelError, Unsupported

F32, BF16 = 0, 1
PAGE = 64  # tokens per cache page; the same constant as LLMX_PAGE in common.cuh
_DTYPE_TAG = {torch.float32: F32, torch.bfloat16: BF16}

_REFUSALS = {
    1: "a size or stride is out of range",
    2: "unsupported combination of dtypes",
    3: "a size exceeds what this kernel's shared memory or grid allows",
    4: "a required table is missing",
}


def require_gpu() -> None:
    if not torch.cuda.is_available():
        raise ExtensionMissing("no CUDA device is available; llmoxide_b200 has no CPU path")


def _tag(t: torch.Tensor) -> int:
    try:
        return _DTYPE_TAG[t.dtype]
    except KeyError:
        raise Unsupported(f"dtype {t.dtype} is not supported by the kernels (float32 and bfloat16 are)") from None


def _ptr(t):
    """A tensor's address as the plain integer (None for no tensor) that a c_void_p argument converts itself."""
    return None if t is None else t.data_ptr()


# The current stream's handle without building a torch.cuda.Stream object for every launch (a prompt step of a
# few tokens launches some 300 kernels and is bound by the host).
_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_raw_device = getattr(torch._C, "_cuda_getDevice", None)


def _stream():
    if _raw_stream is not None and _raw_device is not None:
        return _raw_stream(_raw_device())
    return torch.cuda.current_stream().cuda_stream


launch_count = 0  # kernels of this package launched (or replayed from a graph) so far


def _check(code: int, what: str) -> None:
    global launch_count
    if code == 0:
        launch_count += 1
        return
    if code < 0:
        raise Unsupported(f"{what}: refused, {_REFUSALS.get(-code, f'code {-code}')}")
    raise KernelError(f"{what}: CUDA error {code} at launch")


def _dev(*tensors):
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise KernelError("a kernel was handed a tensor that is not on the GPU")


def _contig(name, t):
    if not t.is_contiguous():
        raise KernelError(f"{name} must be contiguous")


_fn_cache: dict = {}
_libs_ready: set = set()
_overlap = True


def _library(lib_name: str):
    """The library, loaded onto the GPU while nothing else runs there.  Rule: no CUDA module is loaded in the
    middle of a step, because loading one synchronises with the device while hundreds of launches that overlap
    one another may still be pending.  So the first use of a library waits for the GPU to drain and makes the
    module resident (``llmx_touch``) before anything of it is launched; an engine names its libraries when it
    is built (``preload``), so that no step has to."""
    global launch_count
    lib = load_library(lib_name)
    if lib_name not in _libs_ready:
        if torch.cuda.is_available() and not torch.cuda.is_current_stream_capturing():
            torch.cuda.synchronize()
            touch = getattr(lib, "llmx_touch", None)
            if touch is not None:
                touch.restype = c_int
                _check(touch(), f"loading {lib_name}")
                launch_count -= 1
            torch.cuda.synchronize()
            if lib_name in _STATUS_SLOTS and hasattr(lib, "llmx_set_status_word"):
                lib.llmx_set_status_word.argtypes = [c_void_p]
                lib.llmx_set_status_word.restype = c_int
                _check(lib.llmx_set_status_word(c_void_p(status_word(lib_name).data_ptr())),
                       f"registering the status word of {lib_name}")
                launch_count -= 1
            _libs_ready.add(lib_name)
        if hasattr(lib, "llmx_set_pdl"):
            lib.llmx_set_pdl(int(_overlap))
    return lib


# ---- failure reports -------------------------------------------------------
# One word per library in page-locked host memory that its kernels can write: a bounded wait that ran out,
# or a request a kernel could not serve, leaves a code there.  The host looks at the words whenever it has
# waited for a step anyway (no copy, no extra synchronisation).

_STATUS_SLOTS = {"gemm_tc": 0, "attention_prefill_tc": 1, "attention_decode": 2, "sampling": 3}
_STATUS_MEANING = {
    "gemm_tc": {1: "the producer's wait for a free stage ran out", 2: "the MMA issuer's wait for a stage's data ran out",
                3: "the epilogue's wait for an accumulator ran out", 4: "the MMA issuer's wait for a drained accumulator ran out",
                11: "CTA pair: the producer's wait for a free stage ran out", 12: "CTA pair: the MMA issuer's wait for a stage's data ran out",
                13: "CTA pair: the epilogue's wait for an accumulator ran out",
                14: "CTA pair: the MMA issuer's wait for a drained accumulator ran out"},
    "attention_prefill_tc": {20: "its shared memory is not 1024-byte aligned"},
    "attention_decode": {1: "a copy into shared memory never completed", 2: "its shared memory is not 1024-byte aligned"},
    "sampling": {1: "top_p < 1 over more candidates than the kernel sorts", 2: "top_k beyond what the kernel sorts"},
}
_status_host = None


def status_words() -> torch.Tensor:
    """The page-locked int32 words, one per library that reports (see ``_STATUS_SLOTS``)."""
    global _status_host
    if _status_host is None:
        _status_host = torch.zeros(8, dtype=torch.int32).pin_memory()
    return _status_host


def status_word(lib_name: str) -> torch.Tensor:
    i = _STATUS_SLOTS[lib_name]
    return status_words()[i : i + 1]


def check_status() -> None:
    """Raises ``KernelError`` if a kernel has left a report since the last call, and clears it.  Meaningful
    once the host has waited for the work in question (the words are written as the failure happens)."""
    if _status_host is None:
        return
    words = _status_host.numpy()
    if not words.any():
        return
    found = []
    for name, i in _STATUS_SLOTS.items():
        code = int(words[i])
        if code:
            what = _STATUS_MEANING.get(name, {}).get(code, "a bounded wait ran out")
            found.append(f"{name}: {what} (code {code})")
    words[:] = 0
    raise KernelError("a kernel reported a failure; the step's results are not to be used: " + "; ".join(found))


def test_waits(lib_name: str, cycles: int = 0, withhold: bool = False) -> None:
    """For tests of the failure path: the limit of the library's bounded waits in clock cycles (0: the default
    of about two seconds) and whether one role leaves out one arrival, so that a wait runs out, is reported
    and the kernel winds down through its normal exit."""
    f = _fn(lib_name, "llmx_test_waits", [c_longlong, c_int])
    torch.cuda.synchronize()
    code = f(int(cycles), int(withhold))
    if code:
        raise KernelError(f"{lib_name}: CUDA error {code} setting the wait limit")


def set_overlap(on: bool) -> None:
    """Whether the kernels launched from now on may start while the kernel before them still runs
    (programmatic stream serialization; every kernel waits for its inputs itself).  On for decode steps,
    which are chains of short kernels; the engine switches it off for prompt steps."""
    global _overlap
    if on == _overlap:
        return
    _overlap = on
    for name in _libs_ready:
        lib = load_library(name)
        if hasattr(lib, "llmx_set_pdl"):
            lib.llmx_set_pdl(int(on))


def _fn(lib_name: str, fn_name: str, argtypes):
    key = (lib_name, fn_name)
    f = _fn_cache.get(key)
    if f is None:
        f = getattr(_library(lib_name), fn_name)
        f.argtypes = argtypes
        f.restype = c_int
        _fn_cache[key] = f
    return f


def preload(lib_names) -> None:
    """Makes the named libraries resident now (an engine does this when it is built, so that no step has to)."""
    for name in lib_names:
        _library(name)


# ---------------------------------------------------------------------------


def embed(table: torch.Tensor, tokens: torch.Tensor, out: torch.Tensor, scale: float = 1.0) -> None:
    """out[t,:] = float32(table[tokens[t],:]) * scale.  tokens int32 [T]; out float32 [T,d]."""
    _dev(table, tokens, out)
    _contig("table", table), _contig("out", out)
    assert tokens.dtype == torch.int32 and out.dtype == torch.float32
    f = _fn("elementwise", "llmx_embed",
            [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_void_p])
    _check(f(_ptr(table), _tag(table), _ptr(tokens), _ptr(out), tokens.numel(), table.shape[1],
             table.shape[0], scale, _stream()), "embed")


def softcap(x: torch.Tensor, cap: float) -> None:
    """x = cap * tanh(x / cap) in place; x float32, contiguous."""
    _dev(x)
    _contig("x", x)
    assert x.dtype == torch.float32 and cap > 0
    f = _fn("elementwise", "llmx_softcap", [c_void_p, c_longlong, c_float, c_void_p])
    _check(f(_ptr(x), x.numel(), cap, _stream()), "softcap")


def add_rms_norm(h: torch.Tensor, delta, gain: torch.Tensor, eps: float, out, rows=None,
                 write_h: bool = True) -> None:
    """h float32 [T,d] is the residual stream.  ``delta`` is None or [S,T,d]
    (split partials, summed in order).  v = h + sum(delta); h = v when
    ``write_h``; out[r] = rmsnorm(v[rows[r]]) * gain, or for every row without
    ``rows``.  ``out`` may be None when only the sum is wanted."""
    _dev(h, delta, gain, out, rows)
    assert h.dtype == torch.float32 and gain.dtype == torch.float32
    _contig("h", h)
    d = h.shape[-1]
    n_split, stride, dtag = 1, 0, F32
    if delta is not None:
        _contig("delta", delta)
        if delta.dim() == 2:
            delta = delta.unsqueeze(0)
        assert delta.shape[1:] == h.shape, (delta.shape, h.shape)
        n_split, stride, dtag = delta.shape[0], delta.stride(0), _tag(delta)
    n_rows = h.shape[0] if rows is None else rows.numel()
    if out is not None:
        _contig("out", out)
        assert out.shape[0] >= n_rows and out.shape[-1] == d
    f = _fn("elementwise", "llmx_add_rms_norm",
            [c_void_p, c_void_p, c_int, c_int, c_longlong, c_void_p, c_int, c_void_p, c_float, c_void_p,
             c_int, c_int, c_int, c_void_p])
    _check(f(_ptr(h), _ptr(delta), dtag, n_split, stride, _ptr(rows), n_rows, _ptr(gain), eps, _ptr(out),
             _tag(out) if out is not None else F32, d, int(write_h), _stream()), "add_rms_norm")


ADD_SLICE = 512  # columns per CTA of add_gain_sumsq; the same constant as in elementwise.cu


def add_gain_sumsq(h: torch.Tensor, delta, gain: torch.Tensor, x_out: torch.Tensor, sumsq: torch.Tensor) -> None:
    """The residual add and the first half of an RMSNorm for a step of few tokens: h float32 [T,d] += delta
    (None, [T,d] or split partials [S,T,d], added in order); x_out = bfloat16(h * gain); sumsq[s, t] = the sum
    of squares of h[t] over the s-th slice of ``ADD_SLICE`` columns.  The matrix product that reads ``x_out``
    applies the scale (``gemm_tc(scale=...)``)."""
    _dev(h, delta, gain, x_out, sumsq)
    _contig("h", h), _contig("x_out", x_out)
    T, d = h.shape
    assert h.dtype == torch.float32 and gain.dtype == torch.float32 and gain.shape == (d,)
    assert x_out.shape == (T, d) and x_out.dtype == torch.bfloat16 and d % 4 == 0
    n_slices = (d + ADD_SLICE - 1) // ADD_SLICE
    assert sumsq.dtype == torch.float32 and sumsq.shape[0] >= n_slices and sumsq.stride(0) >= T and sumsq.stride(1) == 1
    n_split, stride, dtag = 1, 0, F32
    if delta is not None:
        _contig("delta", delta)
        if delta.dim() == 2:
            delta = delta.unsqueeze(0)
        assert delta.shape[1:] == h.shape
        n_split, stride, dtag = delta.shape[0], delta.stride(0), _tag(delta)
    f = _fn("elementwise", "llmx_add_gain_sumsq",
            [c_void_p, c_void_p, c_int, c_int, c_longlong, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p])
    _check(f(_ptr(h), _ptr(delta), dtag, n_split, stride, _ptr(gain), _ptr(x_out), _ptr(sumsq), sumsq.stride(0), T, d,
             _stream()), "add_gain_sumsq")


def qk_norm_rope_cache(qkv, q_out, k_cache, v_cache, block_table, token_seq, token_pos, q_gain, k_gain,
                       eps: float, cos, sin, n_rot: int, n_heads: int, n_kv_heads: int, head_dim: int,
                       write_cache: bool = True) -> None:
    """qkv [T,(H+2G)*D], or float32 split partials [S,T,(H+2G)*D] summed in
    order -> q_out [T,H*D] (normed, rotated) and, when ``write_cache``, k
    (normed, rotated) and v into the paged cache entry ``k_cache``/``v_cache``
    [n_pages,G,PAGE,D] at each token's position."""
    _dev(qkv, q_out, k_cache, v_cache, block_table, token_seq, token_pos)
    _contig("qkv", qkv), _contig("q_out", q_out), _contig("block_table", block_table)
    n_split, stride = 1, 0
    if qkv.dim() == 3:
        n_split, stride = qkv.shape[0], qkv.stride(0)
    T = qkv.shape[-2]
    assert qkv.shape[-1] == (n_heads + 2 * n_kv_heads) * head_dim
    assert k_cache.dtype == v_cache.dtype and k_cache.is_contiguous() and v_cache.is_contiguous()
    if head_dim > 256 or head_dim % 2:
        raise Unsupported(f"head_dim {head_dim}: the q/k norm and rotation kernel takes even sizes up to 256")
    f = _fn("elementwise", "llmx_qk_norm_rope_cache",
            [c_void_p, c_int, c_int, c_longlong, c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_int,
             c_void_p, c_void_p, c_void_p, c_void_p, c_float, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
             c_int, c_int, c_void_p])
    _check(f(_ptr(qkv), _tag(qkv), n_split, stride, _ptr(q_out), _tag(q_out), _ptr(k_cache), _ptr(v_cache),
             _tag(k_cache), _ptr(block_table), block_table.shape[1], _ptr(token_seq), _ptr(token_pos),
             _ptr(q_gain), _ptr(k_gain), eps, _ptr(cos), _ptr(sin), n_rot, T, n_heads, n_kv_heads, head_dim,
             int(write_cache), _stream()), "qk_norm_rope_cache")


def silu_gate(gu: torch.Tensor, out: torch.Tensor, block: int = 0) -> None:
    """gu [S,T,2F] or [T,2F] -> out [T,F] = silu(gate) * up.  ``block`` = 0:
    gate columns, then up columns; ``block`` > 0: blocks of that many gate
    columns each followed by the up columns of the same features."""
    _dev(gu, out)
    _contig("gu", gu), _contig("out", out)
    if gu.dim() == 2:
        gu = gu.unsqueeze(0)
    S, T, F2 = gu.shape
    assert out.shape == (T, F2 // 2)
    f = _fn("elementwise", "llmx_silu_gate",
            [c_void_p, c_int, c_int, c_longlong, c_void_p, c_int, c_int, c_int, c_int, c_void_p])
    _check(f(_ptr(gu), _tag(gu), S, gu.stride(0), _ptr(out), _tag(out), T, F2 // 2, block, _stream()), "silu_gate")


def sum_splits(parts: torch.Tensor, out: torch.Tensor) -> None:
    """out = parts.sum(0) with the partials added in order; parts [S, ...]."""
    _dev(parts, out)
    _contig("parts", parts), _contig("out", out)
    assert parts.shape[1:] == out.shape
    f = _fn("elementwise", "llmx_sum_splits",
            [c_void_p, c_int, c_int, c_longlong, c_void_p, c_int, c_longlong, c_void_p])
    _check(f(_ptr(parts), _tag(parts), parts.shape[0], parts.stride(0), _ptr(out), _tag(out), out.numel(),
             _stream()), "sum_splits")


def attention_paged(q, out, k_cache, v_cache, block_table, token_seq, token_pos, n_heads: int,
                    n_kv_heads: int, head_dim: int, window, scale: float) -> None:
    """General attention over the paged cache; q, out [T,H*D]."""
    _dev(q, out, k_cache, v_cache, block_table, token_seq, token_pos)
    _contig("q", q), _contig("out", out), _contig("block_table", block_table)
    if head_dim > 256:
        raise Unsupported(f"head_dim {head_dim}: the general attention kernel takes sizes up to 256")
    if n_heads % n_kv_heads:
        raise Unsupported(f"{n_heads} heads are not a multiple of {n_kv_heads} kv heads")
    f = _fn("attention", "llmx_attention_paged",
            [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p,
             c_int, c_int, c_int, c_int, c_int, c_float, c_void_p])
    _check(f(_ptr(q), _ptr(out), _tag(q), _ptr(k_cache), _ptr(v_cache), _tag(k_cache), _ptr(block_table),
             block_table.shape[1], _ptr(token_seq), _ptr(token_pos), q.shape[0], n_heads, n_kv_heads, head_dim,
             int(window or 0), scale, _stream()), "attention_paged")


def n_sm(device=None) -> int:
    """Streaming multiprocessors of the device (asked once)."""
    from .parts.runtime import kernels_n_sm
    return kernels_n_sm(device if device is not None else "cuda")


def decode_chunks(n_seqs: int, n_kv_heads: int, group: int, n_pages: int, sms: int = 148) -> int:
    """Into how many shares the decode attention kernel cuts every sequence's
    visible keys.  A CTA (two warps) takes one share of one (sequence, kv head,
    8 query heads); two CTAs fit an SM, and the whole grid should be resident
    at once, so the shares are as many as that allows on ``sms`` multiprocessors,
    and never more than would leave a warp without a 32-key tile of a full block
    table.  Up to 8 shares the CTAs of a sequence and kv head merge as one
    thread-block cluster.  Beyond 8 (up to 32) the partials go through a
    workspace, which costs a little more per share; that is taken only where a
    small batch with a long context would otherwise leave most of the GPU idle:
    when 8 shares fill less than half of it and every share still has at least
    8 pages of keys.  It depends on the batch's shape only (not on its lengths),
    so a captured graph stays valid while the shape does; each sequence's own
    length is divided on the device."""
    base = n_seqs * n_kv_heads * ((group + 7) // 8)
    room = 2 * sms // base
    n = max(1, min(room, n_pages, 8))
    if n == 8 and base * 8 <= sms:
        n = max(8, min(3 * sms // (2 * base), n_pages // 8, 32))     # about one and a half CTAs per SM measured best
    return n


_decode_counters: dict = {}


def _counters(device, n: int):
    """Zeroed arrival counters for kernels whose last CTA finishes a reduction;
    every launch leaves them zero, so one buffer per device serves all calls."""
    buf = _decode_counters.get(device)
    if buf is None or buf.numel() < n:
        buf = guard.guarded((max(n, 16384),), torch.int32, device, "decode attention counters", zero=True)
        _decode_counters[device] = buf
    return buf


def attention_decode(q, out, k_cache, v_cache, block_table, seq_past, n_heads: int, n_kv_heads: int,
                     head_dim: int, window, scale: float, n_chunks: int = 0) -> None:
    """One new token per sequence, bfloat16: q, out [B,H*D] in batch order;
    seq_past[b] is the token's position.  Each sequence's keys are split over
    n_chunks CTAs (0: chosen from the batch's shape), which merge inside a
    cluster, or beyond 8 chunks through a float32 workspace."""
    _dev(q, out, k_cache, v_cache, block_table, seq_past)
    _contig("q", q), _contig("out", out), _contig("block_table", block_table)
    assert q.dtype == torch.bfloat16 and k_cache.dtype == torch.bfloat16 and out.dtype == torch.bfloat16
    if head_dim % 16 or head_dim > 256:
        raise Unsupported(f"head_dim {head_dim}: the decode attention kernel takes multiples of 16 up to 256")
    B = q.shape[0]
    n_pages = block_table.shape[1]
    if window:
        n_pages = min(n_pages, (window + PAGE - 2) // PAGE + 1)
    group = n_heads // n_kv_heads
    n_chunks = n_chunks or decode_chunks(B, n_kv_heads, group, n_pages, n_sm(q.device))
    ws = counters = None
    if n_chunks > 8:
        ws = guard.scratch((B * n_heads * n_chunks * (head_dim + 4),), torch.float32, q.device,
                           "decode attention workspace")
        counters = _counters(q.device, B * n_kv_heads * ((group + 7) // 8))
    f = _fn("attention_decode", "llmx_attention_decode",
            [c_void_p, c_void_p, c_void_p, c_void_p, c_longlong, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int,
             c_int, c_int, c_int, c_int, c_float, c_int, c_void_p])
    _check(f(_ptr(q), _ptr(out), _ptr(k_cache), _ptr(v_cache), k_cache.shape[0], _ptr(block_table),
             block_table.shape[1],
             _ptr(seq_past), _ptr(ws), _ptr(counters), B, n_heads, n_kv_heads, head_dim, int(window or 0), scale,
             n_chunks, _stream()), "attention_decode")


def attention_decode_status() -> int:
    """0, or 1 after a decode attention launch whose shared-memory copies never completed."""
    lib = load_library("attention_decode")
    lib.llmx_attention_decode_status.restype = c_int
    return int(lib.llmx_attention_decode_status())


def attention_prefill_supports(q, k_cache, head_dim: int) -> bool:
    return q.dtype == torch.bfloat16 and k_cache.dtype == torch.bfloat16 and head_dim in (64, 128)


def attention_prefill(q, out, k_cache, v_cache, block_table, seq_start, seq_past, n_seqs: int, max_new: int,
                      n_heads: int, n_kv_heads: int, head_dim: int, window, scale: float) -> None:
    """Prompt attention on the tensor cores, bfloat16, head sizes 64 and 128:
    q, out [T,H*D] packed sequence after sequence."""
    _dev(q, out, k_cache, v_cache, block_table, seq_start, seq_past)
    _contig("q", q), _contig("out", out), _contig("block_table", block_table)
    if not attention_prefill_supports(q, k_cache, head_dim):
        raise Unsupported(f"the tiled prompt attention takes bfloat16 and head sizes 64 or 128, not {head_dim}")
    f = _fn("attention_prefill", "llmx_attention_prefill",
            [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int,
             c_int, c_int, c_int, c_float, c_void_p])
    _check(f(_ptr(q), _ptr(out), _ptr(k_cache), _ptr(v_cache), _ptr(block_table), block_table.shape[1],
             _ptr(seq_start), _ptr(seq_past), n_seqs, max_new, n_heads, n_kv_heads, head_dim, int(window or 0),
             scale, _stream()), "attention_prefill")


def attention_prefill_tc(q, out, k_cache, v_cache, block_table, seq_start, seq_past, n_seqs: int, max_new: int,
                         n_heads: int, n_kv_heads: int, head_dim: int, window, scale: float) -> None:
    """Prompt attention on tcgen05, bfloat16, head size 128: q, out [T,H*128]
    packed sequence after sequence; the cache entry is [n_pages,G,64,128]."""
    _dev(q, out, k_cache, v_cache, block_table, seq_start, seq_past)
    _contig("q", q), _contig("out", out), _contig("block_table", block_table)
    assert k_cache.is_contiguous() and v_cache.is_contiguous()
    if head_dim != 128 or q.dtype != torch.bfloat16 or k_cache.dtype != torch.bfloat16:
        raise Unsupported("the tcgen05 prompt attention takes bfloat16 and head size 128")
    f = _fn("attention_prefill_tc", "llmx_attention_prefill_tc",
            [c_void_p, c_void_p, c_void_p, c_void_p, c_longlong, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int,
             c_int, c_int, c_int, c_int, c_int, c_float, c_void_p])
    _check(f(_ptr(q), _ptr(out), _ptr(k_cache), _ptr(v_cache), k_cache.shape[0], _ptr(block_table),
             block_table.shape[1], _ptr(seq_start), _ptr(seq_past), n_seqs, q.shape[0], max_new, n_heads,
             n_kv_heads, head_dim, int(window or 0), scale, _stream()), "attention_prefill_tc")


def attention_prefill_tc_status(reset: bool = True) -> int:
    """0, or which bounded wait of the tcgen05 prompt attention ran out.  Synchronises the device."""
    f = _fn("attention_prefill_tc", "llmx_attention_prefill_tc_status", [c_int])
    return f(int(reset))


def gemm_fma(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> None:
    """out[M,N] = x[M,K] @ w[N,K]^T on the FMA units, float32 accumulation in
    the order k = 0..K-1.  Rows may be strided; the K axis must be dense."""
    _dev(x, w, out)
    M, K = x.shape
    N = w.shape[0]
    assert w.shape[1] == K and out.shape == (M, N)
    assert x.stride(1) == 1 and w.stride(1) == 1 and out.stride(1) == 1
    f = _fn("gemm_fma", "llmx_gemm_fma",
            [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_longlong, c_longlong,
             c_longlong, c_void_p])
    _check(f(_ptr(x), _tag(x), _ptr(w), _tag(w), _ptr(out), _tag(out), M, N, K, x.stride(0), w.stride(0),
             out.stride(0), _stream()), "gemm_fma")


PAIR_MIN_TOKENS = 128      # the CTA-pair kernel (tcgen05 cta_group::2) takes steps of more tokens than this


def gemm_tc_supports(x: torch.Tensor, w: torch.Tensor) -> bool:
    """Shapes the tensor-core kernel takes: bfloat16, dense K axis, K and the
    row strides multiples of 8 elements (TMA wants 16-byte strides and starts)."""
    return (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.stride(1) == 1 and w.stride(1) == 1
            and x.shape[1] % 8 == 0 and x.stride(0) % 8 == 0 and w.stride(0) % 8 == 0
            and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def gemm_tc(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, n_split: int = 1, gated=False,
            pair: bool = False, scale=None, accumulate: bool = False) -> None:
    """bfloat16 x [T,K] times w [N,K]^T on tcgen05.  ``out`` is [T,N] (bfloat16
    or float32), or float32 partials [n_split,T,N] of a split reduction, or,
    with ``gated``, [T,N/2] = silu(gate) * up: ``gated=True`` (or 1) for
    w = [gate rows; up rows], ``gated=2`` for w in blocks of 16 gate rows each
    followed by the 16 up rows of the same features (N/2 a multiple of 16).
    ``pair`` runs the CTA-pair kernel (prompt-sized T > 128; it splits too); with
    ``accumulate`` it adds to a float32 ``out`` instead of overwriting it
    (one float32 addition per element, whatever order the tiles finish in).
    ``scale = (sumsq, parts, eps, d)``, for T <= 64: output row t is multiplied
    by 1/sqrt(sum(sumsq[:parts, t]) / d + eps) before any activation (the
    second half of an RMSNorm whose first half is ``add_gain_sumsq``)."""
    gated = int(gated)
    _dev(x, w, out)
    T, K = x.shape
    N = w.shape[0]
    assert w.shape[1] == K and out.is_contiguous()
    if gated:
        assert n_split == 1 and out.shape == (T, N // 2)
        ldy, stride = N // 2, 0
    elif n_split > 1:
        assert out.shape == (n_split, T, N) and out.dtype == torch.float32
        ldy, stride = N, out.stride(0)
    else:
        assert out.shape == (T, N)
        ldy, stride = N, 0
    assert pair or not accumulate
    if pair:
        assert T > PAIR_MIN_TOKENS and scale is None and not (accumulate and n_split > 1)
        f = _fn("gemm_tc", "llmx_gemm_tc_pair",
                [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_longlong, c_longlong, c_longlong, c_int,
                 c_int, c_int, c_longlong, c_void_p])
        _check(f(_ptr(x), _ptr(w), _ptr(out), _tag(out), T, N, K, x.stride(0), w.stride(0), ldy,
                 gated, int(accumulate), n_split, stride, _stream()), "gemm_tc_pair")
        return
    if scale is None:
        f = _fn("gemm_tc", "llmx_gemm_tc",
                [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_longlong, c_longlong, c_longlong, c_int,
                 c_longlong, c_int, c_void_p])
        _check(f(_ptr(x), _ptr(w), _ptr(out), _tag(out), T, N, K, x.stride(0), w.stride(0), ldy, n_split, stride,
                 gated, _stream()), "gemm_tc")
        return
    sumsq, parts, eps, d = scale
    _dev(sumsq)
    assert T <= 64 and sumsq.dtype == torch.float32 and sumsq.shape[0] >= parts and sumsq.stride(1) == 1
    f = _fn("gemm_tc", "llmx_gemm_tc_scaled",
            [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_longlong, c_longlong, c_longlong, c_int,
             c_longlong, c_int, c_void_p, c_int, c_int, c_float, c_int, c_void_p])
    _check(f(_ptr(x), _ptr(w), _ptr(out), _tag(out), T, N, K, x.stride(0), w.stride(0), ldy, n_split, stride, gated,
             _ptr(sumsq), parts, sumsq.stride(0), eps, d, _stream()), "gemm_tc (row scales)")


def gemm_tc_status(reset: bool = True) -> int:
    """0, or which role of the tensor-core kernel ran out of its bounded wait
    since the last reset.  Synchronises the device."""
    f = _fn("gemm_tc", "llmx_gemm_tc_status", [c_int])
    return f(int(reset))


def fill_normal(out: torch.Tensor, stream: int, quantiles: torch.Tensor, mean: float, std: float,
                storage_dtype: torch.dtype) -> None:
    """out[i] = mean + std * normal(stream, i), rounded to ``storage_dtype`` first: the counter-based
    generator of ``weights.random_init`` (same bits as its host version)."""
    _dev(out, quantiles)
    _contig("out", out)
    assert quantiles.dtype == torch.float32 and quantiles.numel() == 65537 and quantiles.is_contiguous()
    f = _fn("random_init", "llmx_fill_normal",
            [c_void_p, c_int, c_longlong, ctypes.c_ulonglong, c_void_p, c_float, c_float, c_int, c_void_p])
    _check(f(_ptr(out), _tag(out), out.numel(), stream & 0xFFFFFFFFFFFFFFFF, _ptr(quantiles), mean, std,
             _DTYPE_TAG[storage_dtype], _stream()), "fill_normal")


def argmax(logits: torch.Tensor, out_tokens: torch.Tensor) -> None:
    """out_tokens[b] = the last index among the maxima of logits[b,:]."""
    _dev(logits, out_tokens)
    assert logits.dtype == torch.float32 and out_tokens.dtype == torch.int32 and logits.stride(1) == 1
    f = _fn("sampling", "llmx_argmax", [c_void_p, c_longlong, c_int, c_int, c_void_p, c_void_p])
    _check(f(_ptr(logits), logits.stride(0), logits.shape[0], logits.shape[1], _ptr(out_tokens), _stream()),
           "argmax")


def sample(logits, temperature, top_k, top_p, repeat_penalty, recent, uniform, out_tokens, status) -> None:
    """One token per row of float32 ``logits`` [B,V] (changed in place by the
    repetition penalty).  Per-row parameters are device tensors [B]; ``recent``
    is int32 [B,W] with -1 for no token, or None.  ``status`` int32 [1] (on the
    device or page-locked on the host) is set non-zero when a row asked for what
    the kernel cannot do."""
    _dev(logits, temperature, top_k, top_p, repeat_penalty, recent, uniform, out_tokens)
    if not (status.is_cuda or status.is_pinned()):
        raise KernelError("the sampler's status word must be on the GPU or in page-locked host memory")
    assert logits.dtype == torch.float32 and logits.stride(1) == 1
    assert temperature.dtype == torch.float32 and top_p.dtype == torch.float32 and uniform.dtype == torch.float32
    assert top_k.dtype == torch.int32 and out_tokens.dtype == torch.int32 and status.dtype == torch.int32
    f = _fn("sampling", "llmx_sample",
            [c_void_p, c_longlong, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
             c_void_p, c_void_p, c_void_p, c_void_p])
    width = 0 if recent is None else recent.shape[1]
    _check(f(_ptr(logits), logits.stride(0), logits.shape[0], logits.shape[1], _ptr(temperature), _ptr(top_k),
             _ptr(top_p), _ptr(repeat_penalty), _ptr(recent), width, _ptr(uniform), _ptr(out_tokens),
             _ptr(status), _stream()), "sample")
