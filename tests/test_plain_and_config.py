"""CPU tests: configuration, registry, weights and their errors, the random-
weights mode, and the plain implementation's own properties (taken from the
reference's unit tests, crates/model/src/ops.rs:213-282,
crates/model/src/sample.rs:194-273)."""

import json
import math

import numpy as np
import pytest
import torch

import plain_qwen3 as plain
from tiny_configs import ALL, TINY_A, TINY_B, TINY_C, TINY_D, make_folder, prompts

from llmoxide_b200.config import Qwen3Config, read_config, register_architecture
from llmoxide_b200.errors import (CheckpointFormatError, ConfigError, UnsupportedArch, WeightsError)
from llmoxide_b200.weights import check_checkpoint, load_checkpoint, open_checkpoint, save_file


# ---- configuration ----------------------------------------------------------

def test_config_reads_every_size_from_its_keys():
    for name, raw in ALL.items():
        cfg = read_config(raw)
        assert isinstance(cfg, Qwen3Config)
        assert cfg.num_hidden_layers == raw["num_hidden_layers"]
        assert cfg.head_dim == raw["head_dim"] and cfg.vocab_size == raw["vocab_size"]
        assert cfg.rms_norm_eps == raw["rms_norm_eps"] and cfg.rope_theta == raw["rope_theta"]
        assert cfg.gqa_group == raw["num_attention_heads"] // raw["num_key_value_heads"]
        assert math.isclose(cfg.attn_scale, 1 / math.sqrt(raw["head_dim"]))
        spec = cfg.to_spec()
        assert len(spec.blocks) == raw["num_hidden_layers"]
        assert bool(spec.head.get("tied")) == raw["tie_word_embeddings"]
        assert ("lm_head.weight" in {t.name for t in spec.tensors()}) != raw["tie_word_embeddings"]
        assert cfg.summary()


def test_config_defaults_and_round_trip():
    raw = dict(TINY_A)
    del raw["head_dim"], raw["num_key_value_heads"]
    cfg = read_config(raw)
    assert cfg.head_dim == 64 // 4 and cfg.num_key_value_heads == 4
    again = read_config(cfg.to_dict())
    assert again.to_spec().tensors() == cfg.to_spec().tensors()
    assert read_config(TINY_B).eos_token_id == (11, 12)


def test_generation_config_sets_the_default_sampling(tmp_path):
    (tmp_path / "config.json").write_text(json.dumps(TINY_A))
    assert read_config(tmp_path).to_spec().default_sampling == dict(temperature=0.7, top_k=20, top_p=0.8)
    (tmp_path / "generation_config.json").write_text(json.dumps(dict(temperature=0.6, top_k=40, repetition_penalty=1.05)))
    assert read_config(tmp_path).to_spec().default_sampling == dict(temperature=0.6, top_k=40, top_p=0.8,
                                                                    repeat_penalty=1.05)


def test_window_layers():
    assert read_config(TINY_C).layer_windows() == [None, 24, 24, None]
    raw = dict(TINY_B, use_sliding_window=True, sliding_window=16, max_window_layers=1)
    assert read_config(raw).layer_windows() == [None, 16, 16]
    assert read_config(TINY_A).layer_windows() == [None, None]
    assert read_config(TINY_D).layer_windows() == [None, 80]


@pytest.mark.parametrize("change, needle", [
    (dict(num_attention_heads=5), "multiple"),
    (dict(head_dim=15), "even"),
    (dict(rms_norm_eps=0.0), "rms_norm_eps"),
    (dict(attention_bias=True), "bias"),
    (dict(hidden_act="gelu"), "hidden_act"),
    (dict(rope_scaling={"type": "yarn"}), "rope_scaling"),
    (dict(layer_types=["full_attention"]), "layer_types"),
    (dict(torch_dtype="float16"), "torch_dtype"),
    (dict(vocab_size=0), "vocab_size"),
])
def test_config_refuses_inconsistent_values(change, needle):
    with pytest.raises(ConfigError, match=needle):
        read_config(dict(TINY_A, **change))


def test_config_missing_keys_and_unknown_architecture():
    raw = dict(TINY_A)
    del raw["rope_theta"], raw["intermediate_size"]
    with pytest.raises(ConfigError, match="intermediate_size.*rope_theta|rope_theta.*intermediate_size"):
        read_config(raw)
    with pytest.raises(UnsupportedArch, match="LlamaForCausalLM"):
        read_config(dict(TINY_A, architectures=["LlamaForCausalLM"]))
    with pytest.raises(ConfigError, match="architectures"):
        read_config({k: v for k, v in TINY_A.items() if k != "architectures"})


def test_another_architecture_registers_without_touching_the_package():
    class Other(Qwen3Config):
        pass

    register_architecture("OtherForCausalLM", Other)
    assert isinstance(read_config(dict(TINY_A, architectures=["OtherForCausalLM"])), Other)


# ---- weights ------------------------------------------------------------------

def test_random_folder_is_seeded_and_loads(tmp_path):
    f1 = make_folder(tmp_path / "x", "A", "float32", seed=5)
    f2 = make_folder(tmp_path / "y", "A", "float32", seed=5)
    f3 = make_folder(tmp_path / "z", "A", "float32", seed=6)
    a, b, c = (plain.read_safetensors(f / "model.safetensors") for f in (f1, f2, f3))
    assert a.keys() == b.keys()
    assert all(torch.equal(a[k], b[k]) for k in a)
    assert not torch.equal(a["model.embed_tokens.weight"], c["model.embed_tokens.weight"])
    assert "lm_head.weight" not in a                      # tied
    m = a["model.layers.0.mlp.up_proj.weight"]
    assert abs(m.std().item() - 0.02) < 2e-3 and abs(m.mean().item()) < 2e-3
    g = a["model.layers.1.input_layernorm.weight"]
    assert abs(g.mean().item() - 1.0) < 2e-2
    spec = read_config(f1).to_spec()
    w = load_checkpoint(f1, spec, "float32", "cpu")
    assert set(w) == {t.name for t in spec.tensors()}
    assert all(torch.equal(w[k], a[k]) for k in w)


def test_precision_policy(tmp_path):
    folder = make_folder(tmp_path, "B", "bfloat16")
    spec = read_config(folder).to_spec()
    # a tensor stored in 32-bit stays so in bfloat16 mode
    entries = open_checkpoint(folder)
    tensors = {n: e.file.tensor(n).clone() for n, e in entries.items()}
    tensors["model.norm.weight"] = tensors["model.norm.weight"].float()
    save_file(tensors, folder / "model.safetensors")
    w16 = load_checkpoint(folder, spec, "bfloat16", "cpu")
    assert w16["model.norm.weight"].dtype == torch.float32
    assert w16["lm_head.weight"].dtype == torch.bfloat16
    w32 = load_checkpoint(folder, spec, "float32", "cpu")
    assert all(t.dtype == torch.float32 for t in w32.values())
    assert torch.equal(w32["lm_head.weight"], w16["lm_head.weight"].float())


def test_one_error_lists_missing_unexpected_and_wrong(tmp_path):
    folder = make_folder(tmp_path, "B", "float32")
    spec = read_config(folder).to_spec()
    entries = open_checkpoint(folder)
    tensors = {n: e.file.tensor(n).clone() for n, e in entries.items()}
    del tensors["model.layers.1.self_attn.k_norm.weight"], tensors["lm_head.weight"]
    tensors["model.layers.9.mlp.up_proj.weight"] = torch.zeros(2, 2)
    tensors["model.layers.0.mlp.down_proj.weight"] = torch.zeros(96, 161)
    tensors["model.norm.weight"] = torch.zeros(96, dtype=torch.int32)
    save_file(tensors, folder / "model.safetensors")
    with pytest.raises(WeightsError) as ei:
        load_checkpoint(folder, spec, "float32", "cpu")
    e = ei.value
    assert e.missing == ["lm_head.weight", "model.layers.1.self_attn.k_norm.weight"]
    assert e.unexpected == ["model.layers.9.mlp.up_proj.weight"]
    assert [n for n, _ in e.wrong] == ["model.layers.0.mlp.down_proj.weight", "model.norm.weight"]
    msg = str(e)
    assert "[96, 161] != expected [96, 160]" in msg and "missing" in msg and "unexpected" in msg


def test_tied_head_in_file_is_ignored_and_truncation_is_caught(tmp_path):
    folder = make_folder(tmp_path, "A", "float32")
    spec = read_config(folder).to_spec()
    entries = open_checkpoint(folder)
    tensors = {n: e.file.tensor(n).clone() for n, e in entries.items()}
    tensors["lm_head.weight"] = tensors["model.embed_tokens.weight"].clone()
    save_file(tensors, folder / "model.safetensors")
    notes = check_checkpoint(spec, open_checkpoint(folder))
    assert len(notes) == 1 and "lm_head" in notes[0]
    path = folder / "model.safetensors"
    data = path.read_bytes()
    path.write_bytes(data[: len(data) - 100])
    with pytest.raises(CheckpointFormatError, match="truncated"):
        open_checkpoint(folder)
    path.write_bytes(b"\x10\x00")
    with pytest.raises(CheckpointFormatError):
        open_checkpoint(folder)


# ---- the plain implementation's own properties --------------------------------

def test_rms_norm_gives_unit_rms():
    x = torch.randn(5, 33)
    y = plain.rms_norm(x, torch.ones(33), 1e-9)
    assert torch.allclose((y * y).mean(-1), torch.ones(5), atol=1e-5)


def test_rope_identity_at_position_zero_and_norm_preserving():
    x = torch.randn(3, 2, 16)
    assert torch.equal(plain.rope_neox(x, [0, 0, 0], 10000.0), x)
    y = plain.rope_neox(x, [5, 77, 1000], 10000.0)
    pair = lambda t: t[..., :8] ** 2 + t[..., 8:] ** 2
    assert torch.allclose(pair(x), pair(y), atol=1e-5)
    # partial rotation leaves the tail alone
    z = plain.rope_neox(x, [5, 6, 7], 10000.0, n_rot=8)
    assert torch.equal(z[..., 8:], x[..., 8:]) and not torch.equal(z[..., :8], x[..., :8])


def test_softmax_sums_to_one_and_attention_is_causal_and_windowed():
    s = plain.softmax_row(torch.tensor([1.0, 2.0, 3.0]))
    assert abs(s.sum().item() - 1) < 1e-6
    q, k, v = torch.randn(6, 4, 8), torch.randn(6, 2, 8), torch.randn(6, 2, 8)
    full = plain.causal_attention(q, k, v, 2)
    assert torch.allclose(full[0, 0], v[0, 0], atol=1e-6)   # position 0 sees only itself
    k2, v2 = k.clone(), v.clone()
    k2[5], v2[5] = 9.0, 9.0                                  # the future does not leak
    assert torch.equal(plain.causal_attention(q, k2, v2, 2)[:5], full[:5])
    win = plain.causal_attention(q, k, v, 2, window=2)
    assert torch.equal(win[:2], full[:2]) and not torch.allclose(win[4], full[4])
    k3, v3 = k.clone(), v.clone()
    k3[:3], v3[:3] = 5.0, 5.0                                # outside the window of query 4 (sees 3, 4)
    assert torch.equal(plain.causal_attention(q, k3, v3, 2, window=2)[4:], win[4:])


def test_plain_forward_prefix_property(tmp_path):
    for name in ("A", "C"):
        folder = make_folder(tmp_path, name, "float32")
        cfg, w = plain.read_model(folder)
        toks = prompts(cfg["vocab_size"], [40])[0]
        whole = plain.forward(cfg, w, toks)
        part = plain.forward(cfg, w, toks[:29])
        assert whole.shape == (40, cfg["vocab_size"])
        assert torch.allclose(whole[:29], part, atol=1e-5)


def test_sampler_properties():
    logits = np.array([0.1, 2.0, -1.0, 2.0, 0.5], dtype=np.float32)
    kw = dict(top_k=64, top_p=1.0, repeat_penalty=1.0, repeat_window=64, u=0.3)
    assert plain.sample(logits, [], temperature=0.0, **kw) == 3          # greedy: last of equal maxima
    assert plain.sample(logits, [], temperature=1.0, **dict(kw, top_k=1)) == 1   # top-k 1 is deterministic
    l2 = logits.copy(); l2[0] = -np.inf
    draws = {plain.sample(l2, [], temperature=1.0, **dict(kw, u=u)) for u in np.linspace(0, 0.999, 50)}
    assert 0 not in draws                                                # -inf is never sampled
    assert plain.sample(logits, [1, 3], temperature=0.0, **dict(kw, repeat_penalty=10.0)) == 4
    draws = {plain.sample(logits, [], temperature=5.0, **dict(kw, top_k=2, u=u)) for u in np.linspace(0, 0.999, 50)}
    assert draws <= {1, 3}                                               # stays inside the top k
    rng = plain.Rng(0)
    xs = [rng.next_f32() for _ in range(4000)]
    assert all(0 <= x < 1 for x in xs) and abs(np.mean(xs) - 0.5) < 0.02


def test_a_checkpoint_split_over_files_with_an_index(tmp_path):
    """model.safetensors.index.json names the file of every tensor; the loaded tensors are the same, and a file the
    index names but the folder lacks is an error of the checkpoint's format."""
    import json

    from llmoxide_b200.errors import CheckpointFormatError

    folder = make_folder(tmp_path, "B", "float32")
    spec = read_config(folder).to_spec()
    whole = load_checkpoint(folder, spec, "float32", "cpu")
    entries = open_checkpoint(folder)
    names = sorted(entries)
    shards = {"model-00001-of-00002.safetensors": names[: len(names) // 2],
              "model-00002-of-00002.safetensors": names[len(names) // 2:]}
    for fname, part in shards.items():
        save_file({n: entries[n].file.tensor(n).clone() for n in part}, folder / fname)
    (folder / "model.safetensors.index.json").write_text(json.dumps(
        {"metadata": {}, "weight_map": {n: fname for fname, part in shards.items() for n in part}}))
    (folder / "model.safetensors").unlink()
    split = load_checkpoint(folder, spec, "float32", "cpu")
    assert set(split) == set(whole) and all(torch.equal(split[k], whole[k]) for k in whole)
    (folder / "model-00002-of-00002.safetensors").unlink()
    with pytest.raises(CheckpointFormatError, match="does not exist"):
        load_checkpoint(folder, spec, "float32", "cpu")
