"""Typed configuration of the dense Qwen3 decoder, read from the keys of its
own config.json, and its description as a ``ModelSpec``.

The reference reads the same quantities from GGUF metadata and refuses
inconsistent ones up front (crates/model/src/qwen35/config.rs:89-177); the
derived sizes follow config.rs:186-208.  Which parts the architecture has and
in what order comes from crates/model/src/qwen35/cpu.rs:138-400: pre-norm
blocks of GQA attention with per-head RMSNorm on q and k and NeoX rotation,
then a SiLU-gated feed-forward; no biases, no embedding scale.
"""

from __future__ import annotations

import json
import math
from dataclasses import dataclass, field
from pathlib import Path
from typing import Optional

from ..errors import ConfigError
from .spec import BlockSpec, ModelSpec, PartSpec, TensorSpec, default_schedule

_REQUIRED = (
    "vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers",
    "num_attention_heads", "rms_norm_eps", "rope_theta", "max_position_embeddings",
)
_DTYPES = {"bfloat16", "float32"}


@dataclass
class Qwen3Config:
    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    rms_norm_eps: float
    rope_theta: float
    max_position_embeddings: int
    tie_word_embeddings: bool = False
    sliding_window: Optional[int] = None
    use_sliding_window: bool = False
    max_window_layers: Optional[int] = None
    layer_types: Optional[list] = None
    torch_dtype: str = "bfloat16"
    eos_token_id: tuple = ()
    bos_token_id: Optional[int] = None
    architectures: tuple = ("Qwen3ForCausalLM",)
    extra: dict = field(default_factory=dict)  # keys carried through untouched
    generation: dict = field(default_factory=dict)  # sampling settings of generation_config.json, if the folder has one

    # ---- reading -----------------------------------------------------------

    @classmethod
    def from_dict(cls, d: dict) -> "Qwen3Config":
        missing = [k for k in _REQUIRED if d.get(k) is None]
        if missing:
            raise ConfigError(f"config.json lacks required key(s): {', '.join(missing)}")
        heads = d["num_attention_heads"]
        # Without their own keys: as many kv heads as heads, and hidden/heads
        # per head (crates/lab/src/engine.rs:70,88).
        kv = d.get("num_key_value_heads") or heads
        head_dim = d.get("head_dim") or (d["hidden_size"] // heads if heads else 0)
        eos = d.get("eos_token_id")
        eos = () if eos is None else tuple(eos) if isinstance(eos, (list, tuple)) else (eos,)
        if d.get("attention_bias"):
            raise ConfigError("attention_bias=true: this decoder has no biases (only .weight tensors exist)")
        act = d.get("hidden_act", "silu")
        if act != "silu":
            raise ConfigError(f"hidden_act={act!r}: the gated feed-forward of this architecture is SiLU")
        if d.get("rope_scaling") not in (None, {}):
            raise ConfigError("rope_scaling is set: only the plain NeoX rotation is built")
        if d.get("num_experts") or d.get("num_local_experts"):
            raise ConfigError("experts are configured: this is the dense architecture")
        dtype = d.get("torch_dtype") or d.get("dtype") or "bfloat16"
        known = {
            *_REQUIRED, "num_key_value_heads", "head_dim", "tie_word_embeddings", "sliding_window",
            "use_sliding_window", "max_window_layers", "layer_types", "torch_dtype", "dtype",
            "eos_token_id", "bos_token_id", "architectures", "attention_bias", "hidden_act",
            "rope_scaling", "num_experts", "num_local_experts",
        }
        cfg = cls(
            vocab_size=d["vocab_size"], hidden_size=d["hidden_size"],
            intermediate_size=d["intermediate_size"], num_hidden_layers=d["num_hidden_layers"],
            num_attention_heads=heads, num_key_value_heads=kv, head_dim=head_dim,
            rms_norm_eps=float(d["rms_norm_eps"]), rope_theta=float(d["rope_theta"]),
            max_position_embeddings=d["max_position_embeddings"],
            tie_word_embeddings=bool(d.get("tie_word_embeddings", False)),
            sliding_window=d.get("sliding_window"),
            use_sliding_window=bool(d.get("use_sliding_window", False)),
            max_window_layers=d.get("max_window_layers"),
            layer_types=list(d["layer_types"]) if d.get("layer_types") is not None else None,
            torch_dtype=dtype, eos_token_id=eos, bos_token_id=d.get("bos_token_id"),
            architectures=tuple(d.get("architectures") or ("Qwen3ForCausalLM",)),
            extra={k: v for k, v in d.items() if k not in known},
        )
        cfg.validate()
        return cfg

    @classmethod
    def from_folder(cls, folder) -> "Qwen3Config":
        return cls.from_dict(json.loads((Path(folder) / "config.json").read_text()))

    def to_dict(self) -> dict:
        d = dict(self.extra)
        d.update(
            architectures=list(self.architectures), model_type="qwen3",
            vocab_size=self.vocab_size, hidden_size=self.hidden_size,
            intermediate_size=self.intermediate_size, num_hidden_layers=self.num_hidden_layers,
            num_attention_heads=self.num_attention_heads, num_key_value_heads=self.num_key_value_heads,
            head_dim=self.head_dim, rms_norm_eps=self.rms_norm_eps, rope_theta=self.rope_theta,
            max_position_embeddings=self.max_position_embeddings,
            tie_word_embeddings=self.tie_word_embeddings, sliding_window=self.sliding_window,
            use_sliding_window=self.use_sliding_window, max_window_layers=self.max_window_layers,
            torch_dtype=self.torch_dtype, hidden_act="silu", attention_bias=False,
            eos_token_id=list(self.eos_token_id) if len(self.eos_token_id) != 1 else self.eos_token_id[0],
            bos_token_id=self.bos_token_id,
        )
        if self.layer_types is not None:
            d["layer_types"] = list(self.layer_types)
        return d

    # ---- checks ------------------------------------------------------------

    def validate(self) -> None:
        def positive(name):
            v = getattr(self, name)
            if not isinstance(v, int) or isinstance(v, bool) or v <= 0:
                raise ConfigError(f"{name} must be a positive integer, got {v!r}")

        for name in ("vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers",
                     "num_attention_heads", "num_key_value_heads", "head_dim", "max_position_embeddings"):
            positive(name)
        if self.num_attention_heads % self.num_key_value_heads:
            raise ConfigError(
                f"num_attention_heads {self.num_attention_heads} is not a multiple of "
                f"num_key_value_heads {self.num_key_value_heads}")
        if self.head_dim % 2:
            raise ConfigError(f"head_dim {self.head_dim} must be even: the rotation pairs dims (i, i + head_dim/2)")
        if not (self.rms_norm_eps > 0 and math.isfinite(self.rms_norm_eps)):
            raise ConfigError(f"rms_norm_eps must be positive, got {self.rms_norm_eps!r}")
        if not (self.rope_theta > 0 and math.isfinite(self.rope_theta)):
            raise ConfigError(f"rope_theta must be positive, got {self.rope_theta!r}")
        if self.torch_dtype not in _DTYPES:
            raise ConfigError(f"torch_dtype {self.torch_dtype!r}: supported are {sorted(_DTYPES)}")
        if self.layer_types is not None:
            if len(self.layer_types) != self.num_hidden_layers:
                raise ConfigError(
                    f"layer_types has {len(self.layer_types)} entries for {self.num_hidden_layers} layers")
            bad = sorted(set(self.layer_types) - {"full_attention", "sliding_attention"})
            if bad:
                raise ConfigError(f"layer_types names unknown kinds: {bad}")
        if any(w is not None for w in self.layer_windows()):
            if not isinstance(self.sliding_window, int) or self.sliding_window <= 0:
                raise ConfigError("a layer uses sliding attention but sliding_window is not a positive integer")

    # ---- derived sizes (crates/model/src/qwen35/config.rs:186-208) ----------

    @property
    def gqa_group(self) -> int:
        return self.num_attention_heads // self.num_key_value_heads

    @property
    def q_dim(self) -> int:
        return self.num_attention_heads * self.head_dim

    @property
    def kv_dim(self) -> int:
        return self.num_key_value_heads * self.head_dim

    @property
    def attn_scale(self) -> float:
        return 1.0 / math.sqrt(self.head_dim)

    def layer_windows(self) -> list:
        """Per layer: None where every earlier key is visible, else the window."""
        n = self.num_hidden_layers
        if self.layer_types is not None:
            return [self.sliding_window if t == "sliding_attention" else None for t in self.layer_types]
        if self.use_sliding_window and self.sliding_window:
            first = n if self.max_window_layers is None else self.max_window_layers
            return [self.sliding_window if i >= first else None for i in range(n)]
        return [None] * n

    def n_params(self) -> int:
        d, f = self.hidden_size, self.intermediate_size
        per_layer = d * (self.q_dim + 2 * self.kv_dim) + self.q_dim * d + 3 * d * f + 2 * d + 2 * self.head_dim
        head = 0 if self.tie_word_embeddings else self.vocab_size * d
        return self.num_hidden_layers * per_layer + self.vocab_size * d + d + head

    def summary(self) -> str:
        """One line, in the manner of crates/model/src/qwen35/config.rs:210-247."""
        windows = [w for w in self.layer_windows() if w is not None]
        return (
            f"qwen3 dense: {self.num_hidden_layers} layers, d {self.hidden_size}, ffn {self.intermediate_size}, "
            f"heads {self.num_attention_heads}/{self.num_key_value_heads} x {self.head_dim}, vocab {self.vocab_size}, "
            f"rope {self.rope_theta:g}, eps {self.rms_norm_eps:g}, "
            f"{'tied' if self.tie_word_embeddings else 'untied'} head, "
            f"{len(windows)} windowed layer(s)" + (f" of {windows[0]}" if windows else "") +
            f", {self.n_params() / 1e6:.1f} M params, {self.torch_dtype}"
        )

    def _default_sampling(self) -> dict:
        out = dict(temperature=0.7, top_k=20, top_p=0.8)
        g = self.generation or {}
        for key in ("temperature", "top_k", "top_p"):
            if g.get(key) is not None:
                out[key] = g[key]
        if g.get("repetition_penalty") is not None:
            out["repeat_penalty"] = g["repetition_penalty"]
        return out

    # ---- description as parts ------------------------------------------------

    def to_spec(self) -> ModelSpec:
        d, f, dh = self.hidden_size, self.intermediate_size, self.head_dim
        eps = self.rms_norm_eps
        position = PartSpec("rope_neox", dict(n_rot=dh, base=self.rope_theta))
        blocks = []
        for i, window in enumerate(self.layer_windows()):
            p = f"model.layers.{i}."
            mixer = PartSpec(
                "gqa_attention",
                dict(hidden_size=d, n_heads=self.num_attention_heads, n_kv_heads=self.num_key_value_heads,
                     head_dim=dh, scale=self.attn_scale, window=window, qk_norm_eps=eps),
                dict(q=TensorSpec(p + "self_attn.q_proj.weight", (self.q_dim, d)),
                     k=TensorSpec(p + "self_attn.k_proj.weight", (self.kv_dim, d)),
                     v=TensorSpec(p + "self_attn.v_proj.weight", (self.kv_dim, d)),
                     o=TensorSpec(p + "self_attn.o_proj.weight", (d, self.q_dim)),
                     q_norm=TensorSpec(p + "self_attn.q_norm.weight", (dh,), "vector"),
                     k_norm=TensorSpec(p + "self_attn.k_norm.weight", (dh,), "vector")),
            )
            ffn = PartSpec(
                "gated_mlp",
                dict(hidden_size=d, intermediate_size=f, activation="silu"),
                dict(gate=TensorSpec(p + "mlp.gate_proj.weight", (f, d)),
                     up=TensorSpec(p + "mlp.up_proj.weight", (f, d)),
                     down=TensorSpec(p + "mlp.down_proj.weight", (d, f))),
            )
            norms = dict(
                mixer=PartSpec("rms_norm", dict(size=d, eps=eps),
                               dict(gain=TensorSpec(p + "input_layernorm.weight", (d,), "vector"))),
                feed_forward=PartSpec("rms_norm", dict(size=d, eps=eps),
                                      dict(gain=TensorSpec(p + "post_attention_layernorm.weight", (d,), "vector"))),
            )
            blocks.append(BlockSpec("pre_norm", mixer, ffn, norms, position))
        return ModelSpec(
            architecture=self.architectures[0],
            hidden_size=d, vocab_size=self.vocab_size,
            # a plain gather (no scale) and a plain product (no cap), tied when the folder has no lm_head
            embedding=PartSpec("gather", dict(scale=None),
                               dict(table=TensorSpec("model.embed_tokens.weight", (self.vocab_size, d)))),
            blocks=tuple(blocks), schedule=default_schedule(self.num_hidden_layers),
            final_norm=PartSpec("rms_norm", dict(size=d, eps=eps),
                                dict(gain=TensorSpec("model.norm.weight", (d,), "vector"))),
            head=(PartSpec("linear", dict(tied=True, softcap=None), {}) if self.tie_word_embeddings else
                  PartSpec("linear", dict(softcap=None), dict(weight=TensorSpec("lm_head.weight", (self.vocab_size, d))))),
            # exporters write the rotation's frequencies beside the weights; a tied model's file may still
            # carry the head (crates/model/src/qwen35/weights.rs:79 decides by presence; here the configuration does)
            ignored_tensors=("*.rotary_emb.inv_freq",) + (("lm_head.weight",) if self.tie_word_embeddings else ()),
            max_positions=self.max_position_embeddings,
            stop_ids=tuple(self.eos_token_id),
            storage_dtype=self.torch_dtype,
            # The folder's own generation_config.json where it has one; else what the model's authors
            # recommend, which the reference falls back to for qwen3 (crates/model/src/sample.rs:43-53).
            default_sampling=self._default_sampling(),
        )
