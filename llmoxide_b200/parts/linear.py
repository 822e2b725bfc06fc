"""y = x W^T for one weight matrix [out, in] (no bias: the architecture has
none, crates/model/src/qwen35/weights.rs:78-126).  Picks the kernel from the
weight's dtype and the runtime: float32 weights always go through the FMA
kernel in true 32-bit; bfloat16 weights go to the tensor-core kernel when it
takes the shape, else to the FMA kernel."""

from __future__ import annotations

import torch

from .. import kernels
from .row_scaled import RowScaled
from .runtime import Runtime


class Linear:
    def __init__(self, weight: torch.Tensor, rt: Runtime):
        assert weight.dim() == 2 and weight.stride(1) == 1
        self.weight, self.rt = weight, rt
        self.out_features, self.in_features = weight.shape
        self._tc = None
        if rt.tensor_cores and weight.dtype == torch.bfloat16 and rt.dtype == "bfloat16":
            from . import linear_tc
            self._tc = linear_tc.plan_for(weight, rt.n_sm)

    def libraries(self) -> set:
        return {"gemm_tc", "elementwise"} if self._tc is not None else {"gemm_fma"}

    def __call__(self, x, out_dtype=None, splits_ok: bool = False):
        """x [T, in] -> [T, out], or split partials [S, T, out] in float32 when
        ``splits_ok`` and the kernel chose to split the reduction.  ``x`` may be
        ``RowScaled`` (tensor-core path only; see ``parts.row_scaled``)."""
        out_dtype = out_dtype or self.rt.act_dtype
        if self._tc is not None and (isinstance(x, RowScaled) or x.dtype == torch.bfloat16):
            return self._tc(x, out_dtype, splits_ok)
        out = torch.empty((x.shape[0], self.out_features), dtype=out_dtype, device=x.device)
        kernels.gemm_fma(x, self.weight, out)
        return out

    def add_into(self, x, residual) -> bool:
        """residual += x W^T inside the product's kernel, if it can for these rows (then True); else nothing
        happens and the caller takes the product as a tensor and leaves the addition to the norm that follows."""
        if self._tc is None or isinstance(x, RowScaled) or x.dtype != torch.bfloat16 or not self._tc.adds_to(x, residual):
            return False
        self._tc.add_into(x, residual)
        return True

    @property
    def takes_row_scales(self) -> bool:
        return self._tc is not None
