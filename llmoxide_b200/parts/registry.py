"""Registries of parts by kind.  A model description names a kind; the builder
looks it up here.  Adding a part is one ``register_*`` call from anywhere (a
test can register a toy part without touching this package).

Interfaces (``rt`` is the ``Runtime``: device, compute dtype, limits):

``Embedding(spec, weights, rt)``
    ``forward(tokens, h)``: writes the float32 residual stream ``h`` [T,d] for
    the int32 token ids [T]; ``table`` is the matrix a tied head may share
    (None if there is none to share).
``Head(spec, weights, rt, embedding)``
    ``forward(x) -> logits``: float32 [n, vocab] for the normalised rows ``x``
    [n,d] in the compute dtype; ``embedding`` is the model's embedding part.
``Norm(spec, weights, rt)``
    ``add_forward(h, delta, rows=None, write_h=True) -> x``: adds ``delta``
    (None, [T,d] or split partials [S,T,d]) to the float32 residual stream
    ``h`` in place and returns the normalised rows in the compute dtype.
``Position(spec, weights, rt)``
    ``rotary_tables() -> (cos, sin, n_rot)`` float32 [positions, n_rot/2], or
    ``None`` when the encoding does not rotate.
``Mixer(spec, position, weights, rt)``
    ``cache_need() -> (KVNeed | None, StateNeed | None)``;
    ``forward(x, ctx, view, writes_cache) -> delta`` with x [T,d] in the
    compute dtype, ``ctx`` the step's ``StepContext``, ``view`` the
    ``CacheEntryView`` of the call's cache entry; returns [T,d] or [S,T,d].
    A part whose forward reads device data on the host sets the class
    attribute ``graph_safe = False``; decode steps then run eagerly.
``FeedForward(spec, weights, rt)``
    ``forward(x, ctx) -> delta``.
``Arrangement(block_spec, weights, rt)``
    ``cache_need()``; ``forward(h, pending, ctx, view, writes_cache) ->
    pending``: runs one layer on the residual stream ``h`` (float32, updated in
    place); ``pending`` is a delta not yet added to ``h``.

Any part may also offer ``libraries() -> set`` with the names of the CUDA
libraries it launches (keys of ``csrc.build.LIBRARIES``); the engine builds and
loads those when it is constructed.  A part that does not say loads its
libraries at their first use, for which the step waits until the GPU is idle.
"""

from __future__ import annotations

from ..errors import ConfigError

EMBEDDINGS: dict = {}
HEADS: dict = {}
MIXERS: dict = {}
FEED_FORWARDS: dict = {}
NORMS: dict = {}
POSITIONS: dict = {}
ARRANGEMENTS: dict = {}


def _register(table, family):
    def deco_factory(kind):
        def deco(cls):
            table[kind] = cls
            return cls
        return deco
    deco_factory.__doc__ = f"Class decorator: registers a {family} under ``kind``."
    return deco_factory


register_embedding = _register(EMBEDDINGS, "embedding")
register_head = _register(HEADS, "head")
register_mixer = _register(MIXERS, "mixer")
register_feed_forward = _register(FEED_FORWARDS, "feed-forward")
register_norm = _register(NORMS, "norm")
register_position = _register(POSITIONS, "position encoding")
register_arrangement = _register(ARRANGEMENTS, "block arrangement")


def lookup(table, family, kind):
    try:
        return table[kind]
    except KeyError:
        raise ConfigError(f"no {family} of kind {kind!r} is registered; known: {sorted(table)}") from None
