"""Plain, slow implementation of the dense Qwen3 decoder, for tests only.

It rests on the formulas of bigmah/llmoxide's CPU path (the reference is Rust
over GGUF and cannot be compiled or imported where these tests run, so there is
no bit-level golden output of the reference itself; each function below cites
the lines it restates).  Whole sequences, no cache, one function per part, all
arithmetic in float32 on the CPU (rotation angles in float64, as the reference
does).  It shares no code with ``llmoxide_b200``: it has its own reader for the
model folder, its own configuration handling and its own sampler.
"""

from __future__ import annotations

import json
import math
import struct
from pathlib import Path

import numpy as np
import torch

# --------------------------------------------------------------------------
# Model folder
# --------------------------------------------------------------------------

_ST_DTYPES = {"F32": np.float32, "F16": np.float16, "I32": np.int32, "I64": np.int64}


def read_safetensors(path) -> dict:
    """name -> float32 (or int64) torch tensor.  Format: 8-byte little-endian
    header length, JSON header {name: {dtype, shape, data_offsets}}, payload."""
    raw = Path(path).read_bytes()
    (n,) = struct.unpack("<Q", raw[:8])
    header = json.loads(raw[8 : 8 + n])
    base = 8 + n
    out = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        lo, hi = info["data_offsets"]
        buf = raw[base + lo : base + hi]
        shape = info["shape"]
        if info["dtype"] == "BF16":
            u16 = np.frombuffer(buf, dtype=np.uint16).astype(np.uint32) << 16
            arr = u16.view(np.float32).reshape(shape)
            out[name] = torch.from_numpy(arr.copy())
        else:
            arr = np.frombuffer(buf, dtype=_ST_DTYPES[info["dtype"]]).reshape(shape)
            t = torch.from_numpy(arr.copy())
            out[name] = t.float() if t.is_floating_point() else t.long()
    return out


def read_model(folder):
    folder = Path(folder)
    cfg = json.loads((folder / "config.json").read_text())
    weights = read_safetensors(folder / "model.safetensors")
    return cfg, weights


def layer_windows(cfg) -> list:
    """Per layer: None (every earlier key is visible) or the window width.
    config.json keys of Qwen3: ``layer_types`` names each layer
    "full_attention" or "sliding_attention"; without it, ``use_sliding_window``
    puts the window on layers ``>= max_window_layers``."""
    n = cfg["num_hidden_layers"]
    w = cfg.get("sliding_window")
    types = cfg.get("layer_types")
    if types is not None:
        return [w if t == "sliding_attention" else None for t in types]
    if cfg.get("use_sliding_window") and w:
        first = cfg.get("max_window_layers", n)
        return [w if i >= first else None for i in range(n)]
    return [None] * n


# --------------------------------------------------------------------------
# Parts
# --------------------------------------------------------------------------


def embed(table: torch.Tensor, tokens) -> torch.Tensor:
    """h[t,:] = E[tok_t,:], no scale.  crates/model/src/qwen35/cpu.rs:129-136"""
    return table[torch.as_tensor(tokens, dtype=torch.long)].clone()


def rms_norm(x: torch.Tensor, gain: torch.Tensor, eps: float) -> torch.Tensor:
    """x * 1/sqrt(mean(x^2)+eps), then * gain (a plain multiplier, no +1), over
    the last axis.  crates/model/src/ops.rs:40-59"""
    ms = (x * x).sum(dim=-1, keepdim=True) / x.shape[-1]
    scale = 1.0 / torch.sqrt(ms + np.float32(eps))
    return (x * scale) * gain


def rope_angles(positions, n_rot: int, base: float):
    """cos, sin [T, n_rot/2] as float32.  The angle is a float64 recurrence
    theta_0 = pos, theta_{i+1} = theta_i * base^(-2/n_rot), and only sin/cos
    are rounded to float32.  crates/model/src/ops.rs:142-159"""
    half = n_rot // 2
    theta_scale = float(np.float32(base)) ** (-2.0 / n_rot)
    theta = np.asarray(positions, dtype=np.float64).copy()
    cos = np.empty((len(theta), half), dtype=np.float32)
    sin = np.empty((len(theta), half), dtype=np.float32)
    for i in range(half):
        cos[:, i] = np.cos(theta).astype(np.float32)
        sin[:, i] = np.sin(theta).astype(np.float32)
        theta = theta * theta_scale
    return torch.from_numpy(cos), torch.from_numpy(sin)


def rope_neox(x: torch.Tensor, positions, base: float, n_rot: int | None = None) -> torch.Tensor:
    """x [T, heads, D]; pairs (i, i + n_rot/2) of the first n_rot dims rotate
    by the angle of their position.  crates/model/src/ops.rs:142-159"""
    d = x.shape[-1]
    n_rot = d if n_rot is None else n_rot
    half = n_rot // 2
    cos, sin = rope_angles(positions, n_rot, base)
    cos, sin = cos[:, None, :], sin[:, None, :]
    x0, x1 = x[..., :half], x[..., half:n_rot]
    out = x.clone()
    out[..., :half] = x0 * cos - x1 * sin
    out[..., half:n_rot] = x0 * sin + x1 * cos
    return out


def linear(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """y[t,o] = sum_i W[o,i] x[t,i]; no bias.  crates/model/src/ops.rs:83-101"""
    return x @ w.t()


def softmax_row(s: torch.Tensor) -> torch.Tensor:
    """exp(s - max) * (1 / sum).  crates/model/src/ops.rs:119-135"""
    e = torch.exp(s - s.max())
    return e * (1.0 / e.sum())


def causal_attention(q, k, v, n_kv_heads: int, window=None) -> torch.Tensor:
    """q [T,H,D], k,v [T,G,D] of one whole sequence -> [T,H,D].  Query head hq
    reads kv head hq // (H/G); the query at position p sees keys first..p with
    first = 0, or p-(w-1) under a window; scale 1/sqrt(D).
    crates/model/src/qwen35/cpu.rs:325-355, crates/model/src/cache.rs:31-37"""
    t, n_heads, d = q.shape
    group = n_heads // n_kv_heads
    scale = np.float32(1.0 / math.sqrt(d))
    out = torch.zeros_like(q)
    for i in range(t):
        first = 0 if window is None else max(0, i - (window - 1))
        for hq in range(n_heads):
            g = hq // group
            s = (k[first : i + 1, g, :] @ q[i, hq, :]) * scale
            w = softmax_row(s)
            out[i, hq, :] = w @ v[first : i + 1, g, :]
    return out


def attention_mixer(x, lw, cfg, positions, window):
    """q,k,v projections, per-head RMSNorm of q and k (gain shared by all
    heads, the block norms' eps), rotation of q and k, attention, output
    projection.  v gets no norm and no rotation.
    crates/model/src/qwen35/cpu.rs:283-368"""
    t = x.shape[0]
    h, g = cfg["num_attention_heads"], cfg["num_key_value_heads"]
    d = cfg.get("head_dim") or cfg["hidden_size"] // h
    eps, base = cfg["rms_norm_eps"], cfg["rope_theta"]
    q = linear(x, lw["self_attn.q_proj.weight"]).view(t, h, d)
    k = linear(x, lw["self_attn.k_proj.weight"]).view(t, g, d)
    v = linear(x, lw["self_attn.v_proj.weight"]).view(t, g, d)
    q = rope_neox(rms_norm(q, lw["self_attn.q_norm.weight"], eps), positions, base)
    k = rope_neox(rms_norm(k, lw["self_attn.k_norm.weight"], eps), positions, base)
    a = causal_attention(q, k, v, g, window).reshape(t, h * d)
    return linear(a, lw["self_attn.o_proj.weight"])


def silu(x: torch.Tensor) -> torch.Tensor:
    """x / (1 + exp(-x)).  crates/model/src/ops.rs:176-178"""
    return x / (1.0 + torch.exp(-x))


def swiglu_ffn(x, lw):
    """down(silu(gate x) * (up x)).  crates/model/src/qwen35/cpu.rs:386-395"""
    gate = linear(x, lw["mlp.gate_proj.weight"])
    up = linear(x, lw["mlp.up_proj.weight"])
    return linear(silu(gate) * up, lw["mlp.down_proj.weight"])


def block(h, lw, cfg, positions, window, trace=None, il=0):
    """h += mixer(norm(h)); h += ffn(norm(h)).  ``trace(name, tensor)`` gets the stages under the reference's
    names.  crates/model/src/qwen35/cpu.rs:141-146,374-400 (trace names :147,:369,:377,:384,:396,:401)"""
    eps = cfg["rms_norm_eps"]
    t = trace or (lambda name, x: None)
    x = rms_norm(h, lw["input_layernorm.weight"], eps)
    t(f"attn_norm-{il}", x)
    a = attention_mixer(x, lw, cfg, positions, window)
    t(f"attn_output-{il}", a)
    h = h + a
    t(f"attn_residual-{il}", h)
    x = rms_norm(h, lw["post_attention_layernorm.weight"], eps)
    t(f"attn_post_norm-{il}", x)
    f = swiglu_ffn(x, lw)
    t(f"ffn_out-{il}", f)
    h = h + f
    t(f"l_out-{il}", h)
    return h


def layer_weights(weights: dict, i: int) -> dict:
    prefix = f"model.layers.{i}."
    return {k[len(prefix) :]: v for k, v in weights.items() if k.startswith(prefix)}


def forward(cfg: dict, weights: dict, tokens, trace=None) -> torch.Tensor:
    """Logits [T, V] at every position of one whole sequence that starts at
    position 0.  Final norm, then the head; the head is the embedding table
    when the folder has no lm_head.  crates/model/src/qwen35/cpu.rs:110-417,
    crates/model/src/qwen35/weights.rs:79"""
    positions = list(range(len(tokens)))
    h = embed(weights["model.embed_tokens.weight"], tokens)
    if trace:
        trace("model.input_embed", h)
    windows = layer_windows(cfg)
    for i in range(cfg["num_hidden_layers"]):
        h = block(h, layer_weights(weights, i), cfg, positions, windows[i], trace, i)
    h = rms_norm(h, weights["model.norm.weight"], cfg["rms_norm_eps"])
    if trace:
        trace("result_norm", h)
    head = weights.get("lm_head.weight")
    if head is None:
        head = weights["model.embed_tokens.weight"]
    return linear(h, head)


def greedy_generate(cfg, weights, prompt, n_new: int, stop_ids=()) -> list:
    """Argmax decoding by recomputing the whole sequence every step; a stop
    token is recorded and ends the sequence.  llmoxide/src/session.rs:586-611"""
    ids, out = list(prompt), []
    for _ in range(n_new):
        nxt = argmax(forward(cfg, weights, ids)[-1].numpy())
        out.append(nxt)
        if nxt in stop_ids:
            break
        ids.append(nxt)
    return out


# --------------------------------------------------------------------------
# Sampling
# --------------------------------------------------------------------------

_M64 = (1 << 64) - 1


class Rng:
    """xorshift64*.  crates/model/src/sample.rs:75-92"""

    def __init__(self, seed: int):
        self.s = ((seed * 0x9E3779B97F4A7C15) & _M64) | 1

    def next_f32(self) -> float:
        x = self.s
        x ^= x >> 12
        x ^= (x << 25) & _M64
        x ^= x >> 27
        self.s = x
        return float(np.float32(((x * 0x2545F4914F6CDD1D) & _M64) >> 40) / np.float32(1 << 24))


def argmax(v) -> int:
    """Last index among equal maxima (Rust's max_by keeps the last).
    crates/model/src/sample.rs:186-192"""
    v = np.asarray(v, dtype=np.float32)
    m = v.max()
    return int(np.nonzero(v == m)[0][-1])


def sample(logits, recent, *, temperature, top_k, top_p, repeat_penalty, repeat_window, u) -> int:
    """Penalty on the recent window, then argmax if temperature <= 0, else the
    k largest finite logits sorted downwards, p = exp((l - max)/T), shortest
    prefix with mass >= top_p * sum, and a walk down with r = u * sum.
    ``u`` is the uniform draw.  Ties are ordered by lower token id first (the
    reference's unstable sort leaves that open).
    crates/model/src/sample.rs:116-183"""
    f32 = np.float32
    l = np.array(logits, dtype=np.float32)
    if repeat_penalty != 1.0:
        start = max(0, len(recent) - repeat_window)
        for t in recent[start:]:
            if 0 <= t < len(l):
                l[t] = l[t] / f32(repeat_penalty) if l[t] > 0 else l[t] * f32(repeat_penalty)
    if temperature <= 0:
        return argmax(l)
    finite = [i for i in range(len(l)) if np.isfinite(l[i])]
    if not finite:
        return argmax(l)
    k = min(max(1, top_k if top_k > 0 else len(l)), len(l), len(finite))
    order = sorted(finite, key=lambda i: (-l[i], i))[:k]
    mx = l[order[0]]
    inv_t = f32(1.0) / f32(temperature)
    p = [f32(math.exp(f32((l[i] - mx) * inv_t))) for i in order]
    total = f32(0)
    for x in p:
        total = f32(total + x)
    cutoff = len(order)
    if top_p < 1.0:
        target = f32(top_p) * total
        acc = f32(0)
        for i, x in enumerate(p):
            acc = f32(acc + x)
            if acc >= target:
                cutoff = i + 1
                break
        total = f32(0)
        for x in p[:cutoff]:
            total = f32(total + x)
    r = f32(u) * total
    for i in range(cutoff):
        r = f32(r - p[i])
        if r <= 0:
            return order[i]
    return order[cutoff - 1]
