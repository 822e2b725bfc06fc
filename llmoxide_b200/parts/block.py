"""Arrangements: how one layer's norms, mixer and feed-forward are wired
around the residual stream.  ``pre_norm`` is the reference's block
(crates/model/src/qwen35/cpu.rs:141-146,374-400):
h += mixer(norm(h)); h += feed_forward(norm(h)).

The residual stream stays float32.  Each residual add is fused into the norm
that follows it, so a block hands its last delta on as ``pending`` instead of
adding it itself.  A mixer or feed-forward with ``adds_to_residual`` is given the
stream (``residual=h``) and may add its result there itself, in the kernel of its
last product; it then returns None, and the norm that follows has nothing to add."""

from __future__ import annotations

import torch

from .. import kernels
from .registry import (ARRANGEMENTS, FEED_FORWARDS, MIXERS, NORMS, POSITIONS, lookup, register_arrangement)


def build_part(table, family, spec, *args):
    return lookup(table, family, spec.kind)(spec, *args)


@register_arrangement("pre_norm")
class PreNormBlock:
    def __init__(self, spec, weights: dict, rt):
        position = None
        if spec.position is not None:
            position = rt_shared_position(spec.position, weights, rt)
        self.mixer_norm = build_part(NORMS, "norm", spec.norms["mixer"], weights, rt)
        self.ff_norm = build_part(NORMS, "norm", spec.norms["feed_forward"], weights, rt)
        self.mixer = lookup(MIXERS, "mixer", spec.mixer.kind)(spec.mixer, position, weights, rt)
        self.feed_forward = build_part(FEED_FORWARDS, "feed-forward", spec.feed_forward, weights, rt)

    def cache_need(self):
        return self.mixer.cache_need()

    def libraries(self) -> set:
        libs = set()
        for part in (self.mixer_norm, self.ff_norm, self.mixer, self.feed_forward):
            libs |= getattr(part, "libraries", set)()
        return libs

    def forward(self, h, pending, ctx, view, writes_cache=True):
        probe = getattr(ctx, "probe", None)
        x = _norm(self.mixer_norm, h, pending, self.mixer, plain=probe is not None)
        if probe:
            probe("resid_in", h), probe("attn_norm", x)      # names after crates/model/src/qwen35/cpu.rs:136-401
        if probe is None and getattr(self.mixer, "adds_to_residual", False):
            a = self.mixer.forward(x, ctx, view, writes_cache, residual=h)
        else:
            a = self.mixer.forward(x, ctx, view, writes_cache)
        if probe:
            probe("attn_output", _summed(a))
        x = _norm(self.ff_norm, h, a, self.feed_forward, plain=probe is not None)
        if probe:
            probe("attn_residual", h), probe("attn_post_norm", x)
        if probe is None and getattr(self.feed_forward, "adds_to_residual", False):
            out = self.feed_forward.forward(x, ctx, residual=h)
        else:
            out = self.feed_forward.forward(x, ctx)
        if probe:
            probe("ffn_out", _summed(out))
        return out


def _summed(delta):
    """A delta as one tensor: split partials [S,T,d] are added in order."""
    if delta.dim() == 2:
        return delta
    out = torch.empty(delta.shape[1:], dtype=torch.float32, device=delta.device)
    kernels.sum_splits(delta, out)
    return out


def _norm(norm, h, delta, consumer, plain=False):
    """h += delta; x = norm(h).  Where both sides can, the norm is done in two halves: the norm part leaves the
    scale to the consumer's first products (``takes_row_scales`` on the consumer, ``row_scales_ok`` on the norm);
    not when the step's intermediates are asked for (``plain``), which wants the normalised rows themselves."""
    if not plain and getattr(consumer, "takes_row_scales", False) and getattr(norm, "ROW_SCALE_MAX_TOKENS", 0):
        return norm.add_forward(h, delta, row_scales_ok=True)
    return norm.add_forward(h, delta)


def rt_shared_position(spec, weights, rt):
    """Layers with the same position encoding share one object (and its tables)."""
    key = ("position", spec.kind, tuple(sorted((k, repr(v)) for k, v in spec.params.items())))
    if key not in rt.shared:
        rt.shared[key] = build_part(POSITIONS, "position encoding", spec, weights, rt)
    return rt.shared[key]


def build_block(spec, weights: dict, rt):
    return lookup(ARRANGEMENTS, "block arrangement", spec.arrangement)(spec, weights, rt)
