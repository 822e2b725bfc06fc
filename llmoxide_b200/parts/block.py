"""Arrangements: how one layer's norms, mixer and feed-forward are wired
around the residual stream.  ``pre_norm`` is the reference's block
(crates/model/src/qwen35/cpu.rs:141-146,374-400):
h += mixer(norm(h)); h += feed_forward(norm(h)).

The residual stream stays float32.  Each residual add is fused into the norm
that follows it, so a block hands its last delta on as ``pending`` instead of
adding it itself."""

from __future__ import annotations

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
        x = _norm(self.mixer_norm, h, pending, self.mixer)
        a = self.mixer.forward(x, ctx, view, writes_cache)
        x = _norm(self.ff_norm, h, a, self.feed_forward)
        return self.feed_forward.forward(x, ctx)


def _norm(norm, h, delta, consumer):
    """h += delta; x = norm(h).  Where both sides can, the norm is done in two halves: the norm part leaves the
    scale to the consumer's first products (``takes_row_scales`` on the consumer, ``row_scales_ok`` on the norm)."""
    if getattr(consumer, "takes_row_scales", False) and getattr(norm, "ROW_SCALE_MAX_TOKENS", 0):
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
