"""Architecture-neutral description of a decoder: which parts each layer is
made of, with their sizes and constants, and the order in which layers run.

An architecture's typed configuration (for example ``Qwen3Config``) turns its
own config.json keys into a ``ModelSpec``.  Everything below the spec -- parts,
cache, step function, loader -- reads only the spec, so a part never learns
which model it sits in.  The reference chooses its layer kinds per layer from
the configuration in the same spirit (crates/model/src/qwen35/state.rs:38-57,
crates/model/src/qwen35/cpu.rs:150,266) and lets several layers share one
cache through an index table (crates/model/src/cache.rs:65-123).
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Mapping, Optional, Sequence


@dataclass(frozen=True)
class TensorSpec:
    """One tensor of the checkpoint: its name and the shape it must have."""

    name: str
    shape: tuple
    # "matrix": used by a matrix product (bfloat16 on the fast path);
    # "vector": gains and the like (float32 arithmetic whatever the storage);
    # "table": integer table (kept as int32).
    role: str = "matrix"


@dataclass(frozen=True)
class PartSpec:
    """A part chosen by ``kind`` from the registry of its family, with its
    parameters (sizes, constants) and the checkpoint tensors it owns."""

    kind: str
    params: Mapping[str, Any] = field(default_factory=dict)
    tensors: Mapping[str, TensorSpec] = field(default_factory=dict)  # role in the part -> tensor

    def __getitem__(self, key):
        return self.params[key]

    def get(self, key, default=None):
        return self.params.get(key, default)


@dataclass(frozen=True)
class BlockSpec:
    """One layer: an arrangement (how norms, mixer and feed-forward are wired
    around the residual stream) and the parts it arranges."""

    arrangement: str                      # e.g. "pre_norm"
    mixer: PartSpec
    feed_forward: PartSpec
    norms: Mapping[str, PartSpec]         # role in the arrangement -> norm
    position: Optional[PartSpec] = None   # position encoding handed to the mixer


@dataclass(frozen=True)
class LayerCall:
    """One entry of the run order.  ``layer`` indexes ``ModelSpec.blocks`` (a
    layer may be named twice).  ``cache`` is the cache entry the call uses;
    calls that name the same entry share its keys, values and state, and only
    a call with ``writes_cache`` appends to it."""

    layer: int
    cache: int
    writes_cache: bool = True


@dataclass(frozen=True)
class ModelSpec:
    """``embedding`` and ``head`` are parts like the others (kinds of the embedding and head registries).
    For the common case a bare ``TensorSpec`` may be given for the embedding (a plain gather of that table)
    and a ``TensorSpec`` or ``None`` for the head (a plain matrix product with that matrix, or with the
    embedding's table when None); they are wrapped into the built-in parts."""

    architecture: str
    hidden_size: int
    vocab_size: int
    embedding: Any                        # PartSpec (or a TensorSpec: the table of a plain gather)
    blocks: Sequence[BlockSpec]
    schedule: Sequence[LayerCall]
    final_norm: PartSpec
    head: Any                             # PartSpec (or a TensorSpec / None: a plain product, tied when None)
    max_positions: int
    stop_ids: tuple = ()
    storage_dtype: str = "bfloat16"       # what a random checkpoint is written in
    default_sampling: Mapping[str, Any] = field(default_factory=dict)
    # Tensors a checkpoint may hold beyond the model's own, which are then left alone: exact names, or
    # "*suffix" for every name with that ending (buffers that exporters write beside the weights).
    ignored_tensors: tuple = ()

    def __post_init__(self):
        if isinstance(self.embedding, TensorSpec):
            object.__setattr__(self, "embedding", PartSpec("gather", {}, {"table": self.embedding}))
        if self.head is None:
            object.__setattr__(self, "head", PartSpec("linear", {"tied": True}, {}))
        elif isinstance(self.head, TensorSpec):
            object.__setattr__(self, "head", PartSpec("linear", {}, {"weight": self.head}))

    def is_ignored(self, name: str) -> bool:
        return any(name.endswith(pat[1:]) if pat.startswith("*") else name == pat for pat in self.ignored_tensors)

    def tensors(self) -> list:
        """Every tensor the checkpoint must hold, each once."""
        seen, out = set(), []

        def add(t):
            if t is not None and t.name not in seen:
                seen.add(t.name)
                out.append(t)

        for t in self.embedding.tensors.values():
            add(t)
        for b in self.blocks:
            parts = [b.mixer, b.feed_forward, *b.norms.values()]
            if b.position is not None:
                parts.append(b.position)
            for p in parts:
                for t in p.tensors.values():
                    add(t)
        for t in self.final_norm.tensors.values():
            add(t)
        for t in self.head.tensors.values():
            add(t)
        return out

    def n_cache_entries(self) -> int:
        return 1 + max((c.cache for c in self.schedule), default=-1)


def default_schedule(n_layers: int) -> tuple:
    """Every layer once, in order, each with a cache entry of its own."""
    return tuple(LayerCall(layer=i, cache=i) for i in range(n_layers))
