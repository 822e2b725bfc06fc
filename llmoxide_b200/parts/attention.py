"""Grouped-query attention as a mixer: fused q/k/v projection, optional
per-head RMSNorm of q and k, rotation, cache write, attention over the cache
(all keys or a window of them), output projection.

Formulas in the reference's order (crates/model/src/qwen35/cpu.rs:283-368):
q = Wq x, k = Wk x, v = Wv x; per head q <- rope(rms(q) * q_norm), k likewise,
v untouched; k and v of the whole step are stored before any score is taken;
query head hq reads kv head hq // (H/G); scores are scaled by ``scale``; the
query at position p sees keys first..p, first = 0 or p-(w-1) under a window
(crates/model/src/cache.rs:31-37).
"""

from __future__ import annotations

import torch

from .. import kernels
from ..cache import KVNeed
from ..errors import Unsupported
from .linear import Linear
from .registry import register_mixer


@register_mixer("gqa_attention")
class GQAttention:
    def __init__(self, spec, position, weights: dict, rt):
        self.rt = rt
        self.H, self.G, self.D = spec["n_heads"], spec["n_kv_heads"], spec["head_dim"]
        self.scale = float(spec["scale"])
        self.window = spec.get("window")
        self.eps = float(spec.get("qk_norm_eps") or 0.0)
        if self.H % self.G:
            raise Unsupported(f"{self.H} heads are not a multiple of {self.G} kv heads")
        if self.D % 16 or self.D > 256:
            raise Unsupported(f"head_dim {self.D}: the attention kernels take multiples of 16 up to 256")
        t = spec.tensors
        wq, wk, wv = (weights.pop(t[r].name) for r in ("q", "k", "v"))
        if not (wq.dtype == wk.dtype == wv.dtype):
            wq, wk, wv = wq.float(), wk.float(), wv.float()
        # One matrix product for q, k and v: rows of q, then k, then v.
        wqkv = torch.cat([wq, wk, wv], dim=0)
        del wq, wk, wv
        self.qkv = Linear(wqkv, rt)
        self.q_only = Linear(wqkv[: self.H * self.D], rt)
        self.o = Linear(weights.pop(t["o"].name), rt)
        self.q_gain = self.k_gain = None
        if "q_norm" in t:
            self.q_gain = weights.pop(t["q_norm"].name).to(torch.float32).contiguous()
            self.k_gain = weights.pop(t["k_norm"].name).to(torch.float32).contiguous()
        self.position = position

    def cache_need(self):
        return KVNeed(self.G, self.D, self.window), None

    @property
    def takes_row_scales(self) -> bool:
        """Its first products (q|k|v) can apply a norm's row scales in their epilogue."""
        return self.qkv.takes_row_scales and self.q_only.takes_row_scales

    def libraries(self) -> set:
        libs = {"elementwise"} | self.qkv.libraries() | self.o.libraries()
        if self.rt.dtype == "bfloat16" and self.rt.tensor_cores:
            libs |= {"attention_decode",
                     "attention_prefill_tc" if self.D == 128 else "attention_prefill" if self.D == 64 else "attention"}
        else:
            libs.add("attention")
        return libs

    adds_to_residual = True      # forward() takes ``residual`` and may return None: "already added"

    def forward(self, x, ctx, view, writes_cache=True, residual=None):
        H, G, D = self.H, self.G, self.D
        T = x.shape[0]
        dev = x.device
        tables = self.position.rotary_tables() if self.position is not None else None
        cos, sin, n_rot = tables if tables is not None else (None, None, 0)
        block_table = ctx.block_tables[view.group]
        if writes_cache:
            qkv = self.qkv(x, splits_ok=True)
        else:
            # A call that reads another call's cache entry makes only queries.
            q_part = self.q_only(x)
            qkv = torch.empty((T, (H + 2 * G) * D), dtype=q_part.dtype, device=dev)
            qkv[:, : H * D] = q_part
        q = torch.empty((T, H * D), dtype=self.rt.act_dtype, device=dev)
        kernels.qk_norm_rope_cache(qkv, q, view.k, view.v, block_table, ctx.token_seq, ctx.token_pos,
                                   self.q_gain, self.k_gain, self.eps, cos, sin, n_rot, H, G, D, writes_cache)
        out = torch.empty_like(q)
        self.attend(q, out, view, block_table, ctx)
        if residual is not None and self.o.add_into(out, residual):
            return None
        return self.o(out, splits_ok=True)

    def attend(self, q, out, view, block_table, ctx):
        """bfloat16: the split-key kernel when every sequence brings one token;
        for prompts the tcgen05 kernel at head size 128 and the mma.sync tiled
        kernel at head size 64; the general kernel otherwise and always in
        float32."""
        H, G, D = self.H, self.G, self.D
        fast = q.dtype == torch.bfloat16 and view.k.dtype == torch.bfloat16 and self.rt.tensor_cores
        if fast and ctx.is_decode:
            kernels.attention_decode(q, out, view.k, view.v, block_table, ctx.seq_past, H, G, D, self.window,
                                     self.scale)
        elif fast and D == 128:
            kernels.attention_prefill_tc(q, out, view.k, view.v, block_table, ctx.seq_start, ctx.seq_past,
                                         ctx.n_seqs, ctx.max_new, H, G, D, self.window, self.scale)
        elif fast and kernels.attention_prefill_supports(q, view.k, D):
            kernels.attention_prefill(q, out, view.k, view.v, block_table, ctx.seq_start, ctx.seq_past,
                                      ctx.n_seqs, ctx.max_new, H, G, D, self.window, self.scale)
        else:
            kernels.attention_paged(q, out, view.k, view.v, block_table, ctx.token_seq, ctx.token_pos,
                                    H, G, D, self.window, self.scale)
