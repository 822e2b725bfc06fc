"""Tiny configurations of the dense Qwen3 decoder that differ in every size
and option: head counts and groups, head size, widths that are no power of
two, layer count, vocabulary, eps, rotation base, tied or untied head, and
the window."""

import json
from pathlib import Path

TINY_A = dict(
    architectures=["Qwen3ForCausalLM"], model_type="qwen3",
    num_hidden_layers=2, hidden_size=64, num_attention_heads=4, num_key_value_heads=2, head_dim=16,
    intermediate_size=128, vocab_size=256, rope_theta=10000.0, rms_norm_eps=1e-6,
    tie_word_embeddings=True, max_position_embeddings=128, sliding_window=None, use_sliding_window=False,
    torch_dtype="float32", eos_token_id=7,
)
TINY_B = dict(
    architectures=["Qwen3ForCausalLM"], model_type="qwen3",
    num_hidden_layers=3, hidden_size=96, num_attention_heads=6, num_key_value_heads=2, head_dim=32,
    intermediate_size=160, vocab_size=384, rope_theta=1000000.0, rms_norm_eps=1e-5,
    tie_word_embeddings=False, max_position_embeddings=256, use_sliding_window=False,
    torch_dtype="float32", eos_token_id=[11, 12],
)
# Windowed layers between full ones, as many kv heads as heads, odd vocabulary.
TINY_C = dict(
    architectures=["Qwen3ForCausalLM"], model_type="qwen3",
    num_hidden_layers=4, hidden_size=80, num_attention_heads=5, num_key_value_heads=5, head_dim=48,
    intermediate_size=112, vocab_size=307, rope_theta=50000.0, rms_norm_eps=3e-6,
    tie_word_embeddings=False, max_position_embeddings=512, sliding_window=24, use_sliding_window=True,
    layer_types=["full_attention", "sliding_attention", "sliding_attention", "full_attention"],
    torch_dtype="float32", eos_token_id=3,
)
# The head sizes of the tiled tensor-core kernels (128 and 64), q width != hidden width,
# one kv head for four heads, a window shorter than the sequences on one layer.
TINY_D = dict(
    architectures=["Qwen3ForCausalLM"], model_type="qwen3",
    num_hidden_layers=2, hidden_size=192, num_attention_heads=4, num_key_value_heads=1, head_dim=128,
    intermediate_size=320, vocab_size=509, rope_theta=1000000.0, rms_norm_eps=1e-6,
    tie_word_embeddings=True, max_position_embeddings=1024, sliding_window=80, use_sliding_window=True,
    max_window_layers=1, torch_dtype="float32", eos_token_id=[1, 2],
)
TINY_E = dict(
    architectures=["Qwen3ForCausalLM"], model_type="qwen3",
    num_hidden_layers=2, hidden_size=136, num_attention_heads=6, num_key_value_heads=3, head_dim=64,
    intermediate_size=264, vocab_size=300, rope_theta=10000.0, rms_norm_eps=1e-5,
    tie_word_embeddings=False, max_position_embeddings=1024, use_sliding_window=False,
    torch_dtype="float32", eos_token_id=0,
)
# One layer at the layer sizes of Qwen3-8B (hidden 4096, 32 heads, 8 kv heads, head 128, feed-forward
# 12288) with a small vocabulary: the shapes the large kernels are tuned for, at a size the plain
# implementation still walks in seconds.
LAYER_8B = dict(
    architectures=["Qwen3ForCausalLM"], model_type="qwen3",
    num_hidden_layers=1, hidden_size=4096, num_attention_heads=32, num_key_value_heads=8, head_dim=128,
    intermediate_size=12288, vocab_size=1536, rope_theta=1000000.0, rms_norm_eps=1e-6,
    tie_word_embeddings=False, max_position_embeddings=4096, use_sliding_window=False,
    torch_dtype="bfloat16", eos_token_id=0,
)
ALL = {"A": TINY_A, "B": TINY_B, "C": TINY_C, "D": TINY_D, "E": TINY_E}


def make_folder(tmp_path, name: str, dtype: str, seed: int = 1234) -> Path:
    """Writes a model folder with the package's random-weights mode."""
    from llmoxide_b200.config import read_config
    from llmoxide_b200.weights import write_model_folder

    cfg = dict(LAYER_8B if name == "8B" else ALL[name])
    cfg["torch_dtype"] = dtype
    folder = Path(tmp_path) / f"tiny_{name}_{dtype}"
    if not (folder / "model.safetensors").exists():
        write_model_folder(folder, read_config(cfg), seed, dtype)
    return folder


def drawn_config(seed: int) -> dict:
    """A tiny configuration drawn from a seed: every size and option varies, with the awkward values in the
    draw (head sizes in steps of 16 up to 256, widths that are no multiple of 8, a feed-forward width that
    is no multiple of 16, odd vocabularies, windows shorter than a page and longer than one)."""
    import numpy as np

    rng = np.random.default_rng(1000 + seed)
    pick = lambda xs: xs[int(rng.integers(len(xs)))]
    kv = pick([1, 2, 3])
    layers = pick([1, 2, 3])
    window = pick([None, None, 17, 70, 130])
    cfg = dict(
        architectures=["Qwen3ForCausalLM"], model_type="qwen3", num_hidden_layers=layers,
        hidden_size=pick([72, 100, 136, 200, 264]), num_attention_heads=kv * pick([1, 2, 4]),
        num_key_value_heads=kv, head_dim=pick([16, 32, 48, 64, 80, 96, 112, 128, 144, 192, 256]),
        intermediate_size=pick([88, 100, 144, 200, 272]), vocab_size=pick([131, 257, 300, 511]),
        rope_theta=pick([10000.0, 500000.0, 1000000.0]), rms_norm_eps=pick([1e-6, 1e-5, 3e-6]),
        tie_word_embeddings=bool(rng.integers(2)), max_position_embeddings=1024,
        use_sliding_window=window is not None, sliding_window=window, torch_dtype="float32", eos_token_id=1)
    if window is not None:
        cfg["layer_types"] = [pick(["full_attention", "sliding_attention"]) for _ in range(layers)]
    return cfg


def make_folder_of(tmp_path, tag: str, cfg: dict, dtype: str, seed: int = 1234) -> Path:
    """The same for a configuration given as a dictionary."""
    from llmoxide_b200.config import read_config
    from llmoxide_b200.weights import write_model_folder

    cfg = dict(cfg, torch_dtype=dtype)
    folder = Path(tmp_path) / f"tiny_{tag}_{dtype}"
    if not (folder / "model.safetensors").exists():
        write_model_folder(folder, read_config(cfg), seed, dtype)
    return folder


def prompts(vocab: int, lengths, seed: int = 0):
    import numpy as np

    rng = np.random.default_rng(seed)
    return [rng.integers(0, vocab, size=n).tolist() for n in lengths]
