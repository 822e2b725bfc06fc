"""Plans for the tensor-core matrix product: which launches a weight matrix
takes at a given number of tokens.

Decode is bound by reading the weights once, so a matrix with few 128-row
tiles splits its reduction over K until about one CTA per SM streams; the
float32 partials are summed by the kernel that consumes them (the residual
add + norm, or the gated activation).  A long prompt has tiles enough and does
not split; a short one against a narrow matrix does (``choose_prompt_splits``)."""

from __future__ import annotations

from functools import lru_cache

import torch

from .. import kernels
from ..guard import scratch
from .row_scaled import RowScaled

TILE_ROWS = 128
CTAS_PER_SM = 2               # what the kernel fits per SM at decode tile sizes
MIN_KBLOCKS_PER_SPLIT = 4     # 64-element blocks of K per split, at least
PAIR_MIN_TOKENS = kernels.PAIR_MIN_TOKENS     # above this, CTA pairs (tcgen05 cta_group::2) share each token tile


@lru_cache(maxsize=4096)
def choose_splits(n_rows: int, k: int, n_tokens: int, n_sm: int = 148, max_splits: int = 16) -> int:
    """How many ways to split the reduction over K at ``n_tokens`` tokens, from
    a small time model of the streaming kernel (microseconds): n_sm * CTAS_PER_SM
    CTAs run at once; a CTA streams its share of the weights at
    the HBM rate divided by the CTAs running, but never faster than one CTA
    can pull; every round costs a fixed start and drain; float32 partials are
    written once and read once by the kernel that consumes them."""
    if n_tokens > 64:
        return 1
    tiles = (n_rows + TILE_ROWS - 1) // TILE_ROWS
    k_blocks = (k + 63) // 64
    slots = n_sm * CTAS_PER_SM
    hbm, one_cta, fixed = 6.5e6, 2.5e4, 4.0          # bytes per microsecond; microseconds
    best, best_t = 1, None
    for s in range(1, min(max_splits, max(1, k_blocks // MIN_KBLOCKS_PER_SPLIT)) + 1):
        ctas = tiles * s
        rate = min(hbm / min(ctas, slots), one_cta)
        unit = TILE_ROWS * (k / s) * 2 / rate + fixed
        # persistent CTAs walk their units without waiting for one another: more units than slots cost their
        # share of rounds, plus on average half a unit at the end where the slots run dry unevenly
        t = unit if ctas <= slots else (ctas / slots + 0.5) * unit
        if s > 1:
            t += 2.0 * s * n_tokens * n_rows * 4 / 5.0e6
        if best_t is None or t < best_t - 1e-9:
            best, best_t = s, t
    return best


@lru_cache(maxsize=4096)
def choose_prompt_splits(n_rows: int, k: int, n_tokens: int, n_sm: int = 148, max_splits: int = 8) -> int:
    """The same question for a prompt-sized step (more than 128 tokens), which runs on CTA pairs in units of
    256 rows x 256 tokens.  Whole units are best when there are enough of them to occupy most pairs.  A short
    prompt (or a chunk of one) against a narrow matrix leaves most of the GPU idle (512 tokens x 4096 rows:
    32 units for 74 pairs); then the reduction is split until about one unit per pair runs, each split at
    least 8 blocks of K long.  The float32 partials are summed by the kernel that consumes them."""
    pairs = max(1, n_sm // 2)
    units = -(-n_rows // 256) * -(-n_tokens // 256)
    if units * 5 >= pairs * 4:
        return 1
    return max(1, min(max_splits, pairs // units, ((k + 63) // 64) // 8))


class TensorCoreLinear:
    def __init__(self, weight: torch.Tensor, n_sm: int = 148):
        self.weight, self.n_sm = weight, n_sm
        self.N, self.K = weight.shape

    def adds_to(self, x, residual) -> bool:
        """Whether this product, for these rows, can add its result to ``residual`` itself (prompt-sized steps
        on the CTA-pair kernel: every element of ``residual`` then receives exactly one float32 addition)."""
        return (not isinstance(x, RowScaled) and residual is not None and residual.dtype == torch.float32
                and residual.is_contiguous() and residual.shape == (x.shape[0], self.N) and self.N % 4 == 0
                and x.shape[0] > PAIR_MIN_TOKENS and kernels.gemm_tc_supports(x, self.weight)
                and choose_prompt_splits(self.N, self.K, x.shape[0], self.n_sm) == 1)

    def add_into(self, x, residual) -> None:
        """residual += x W^T."""
        kernels.gemm_tc(x, self.weight, residual, pair=True, accumulate=True)

    def __call__(self, x, out_dtype, splits_ok):
        x, scale = self._unpack(x)
        T = x.shape[0]
        if not kernels.gemm_tc_supports(x, self.weight):
            assert scale is None
            out = torch.empty((T, self.N), dtype=out_dtype, device=x.device)
            kernels.gemm_fma(x, self.weight, out)
            return out
        s = 1
        if splits_ok:
            s = (choose_splits(self.N, self.K, T, self.n_sm) if T <= 64 else
                 choose_prompt_splits(self.N, self.K, T, self.n_sm))
        if s > 1:
            out = scratch((s, T, self.N), torch.float32, x.device, "split partials of a matrix product")
            kernels.gemm_tc(x, self.weight, out, n_split=s, scale=scale, pair=T > PAIR_MIN_TOKENS)
            return out
        out = scratch((T, self.N), out_dtype, x.device, "output of a matrix product")
        kernels.gemm_tc(x, self.weight, out, pair=T > PAIR_MIN_TOKENS, scale=scale)
        return out

    @staticmethod
    def _unpack(x):
        """Plain rows, or rows whose norm's scale is still to be applied (``RowScaled``)."""
        if isinstance(x, RowScaled):
            return x.x, (x.sumsq, x.n_parts, x.eps, x.d)
        return x, None

    def gated(self, x, out_dtype, block: int = 0):
        """silu(gate x) * (up x), [T, N/2]; ``block`` = 0 for weight = [gate rows; up rows], 16 for
        blocks of 16 gate rows each followed by the 16 up rows of the same features."""
        x, scale = self._unpack(x)
        out = scratch((x.shape[0], self.N // 2), out_dtype, x.device, "output of the gated matrix product")
        kernels.gemm_tc(x, self.weight, out, gated=2 if block == 16 else 1, pair=x.shape[0] > PAIR_MIN_TOKENS,
                        scale=scale)
        return out

def plan_for(weight: torch.Tensor, n_sm: int = 148):
    if weight.dtype != torch.bfloat16 or weight.stride(1) != 1 or weight.shape[1] % 8 or weight.stride(0) % 8:
        return None
    return TensorCoreLinear(weight, n_sm)
