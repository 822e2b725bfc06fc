"""GPU: each part of a layer alone against the plain implementation, the run
order as data (a layer named twice, a layer that reads another layer's
cache), and parts defined here -- a mixer with state of its own, a
feed-forward, a position encoding -- registered and stepped without any change
to the package."""

import math
from dataclasses import dataclass

import numpy as np
import pytest
import torch

import plain_qwen3 as plain
from tiny_configs import TINY_B, TINY_C, TINY_D

pytestmark = pytest.mark.gpu
DEV = "cuda"


def rel(got, want):
    got, want = got.float().cpu(), want.float().cpu()
    return float((got - want).abs().max() / want.abs().max())


def _rt(dtype="float32", max_positions=256):
    from llmoxide_b200.parts import Runtime
    return Runtime(dtype=dtype, device=torch.device(DEV), max_positions=max_positions)


def _ctx_and_cache(needs, seq_tokens, pasts=None, n_slots=4, max_tokens=1024, dtype=torch.float32, cache=None,
                   slots=None):
    """A StepContext for sequences that bring ``seq_tokens[i]`` tokens."""
    from llmoxide_b200.cache import Cache
    from llmoxide_b200.engine.batch import StepBuffers, build_host_arrays

    if cache is None:
        cache = Cache(needs, n_slots, max_tokens, dtype, torch.device(DEV))
        slots = [cache.acquire() for _ in seq_tokens]
    entries = [(s, [0] * n) for s, n in zip(slots, seq_tokens)]
    lengths = [cache.length(s) for s in slots]
    for s, n in zip(slots, seq_tokens):
        cache.alloc.reserve(s, n)
    n_groups = max(1, cache.n_groups())
    rows = [[cache.alloc.page_row(s, g) for s in slots] for g in range(n_groups)]
    lay, buf, facts = build_host_arrays(entries, [[n - 1] for n in seq_tokens], lengths, rows, n_groups)
    ctx = StepBuffers(torch.device(DEV)).upload(lay, buf, facts)
    return ctx, cache, slots


def _commit(cache, slots, seq_tokens):
    for s, n in zip(slots, seq_tokens):
        cache.alloc.commit(s, n)


def _weights_of(cfg_raw, seed=3):
    from llmoxide_b200.config import read_config
    from llmoxide_b200.weights.random_init import host_tensor

    cfg = read_config(cfg_raw)
    spec = cfg.to_spec()
    w = {t.name: host_tensor(t, seed, torch.float32) for t in spec.tensors()}
    return cfg, spec, w


# ---- parts alone ------------------------------------------------------------------

def test_norm_part():
    from llmoxide_b200.config import PartSpec, TensorSpec
    from llmoxide_b200.parts.registry import NORMS

    d = 200
    gain = 1 + 0.1 * torch.randn(d)
    spec = PartSpec("rms_norm", dict(size=d, eps=3e-6), dict(gain=TensorSpec("g", (d,), "vector")))
    norm = NORMS["rms_norm"](spec, {"g": gain.to(DEV)}, _rt())
    h, delta = torch.randn(9, d), torch.randn(9, d)
    hd = h.to(DEV)
    x = norm.add_forward(hd, delta.to(DEV))
    assert rel(hd, h + delta) < 2e-6 and rel(x, plain.rms_norm(h + delta, gain, 3e-6)) < 2e-6


def test_position_part_tables():
    from llmoxide_b200.config import PartSpec
    from llmoxide_b200.parts.registry import POSITIONS

    for n_rot, base in ((16, 10000.0), (48, 1e6)):
        pos = POSITIONS["rope_neox"](PartSpec("rope_neox", dict(n_rot=n_rot, base=base)), {}, _rt(max_positions=300))
        cos, sin, r = pos.rotary_tables()
        want_c, want_s = plain.rope_angles(list(range(300)), n_rot, base)
        assert r == n_rot and torch.equal(cos.cpu(), want_c) and torch.equal(sin.cpu(), want_s)
    assert POSITIONS["none"](PartSpec("none"), {}, _rt()).rotary_tables() is None


@pytest.mark.parametrize("raw, layer", [(TINY_B, 1), (TINY_C, 1), (TINY_C, 3)])
def test_attention_mixer_part(raw, layer):
    """The mixer alone: two sequences, a prompt step and then single tokens."""
    from llmoxide_b200.parts.block import build_part, rt_shared_position
    from llmoxide_b200.parts.registry import MIXERS

    cfg, spec, w = _weights_of(raw)
    bs = spec.blocks[layer]
    rt = _rt()
    dev_w = {k: v.to(DEV) for k, v in w.items()}
    mixer = MIXERS[bs.mixer.kind](bs.mixer, rt_shared_position(bs.position, dev_w, rt), dev_w, rt)
    d = raw["hidden_size"]
    lens = [70, 29]
    xs = [torch.randn(L, d) for L in lens]
    lw = plain.layer_weights(w, layer)
    window = cfg.layer_windows()[layer]
    want = [plain.attention_mixer(x, lw, raw, list(range(len(x))), window) for x in xs]
    cuts = [40, 29 - 5]
    ctx, cache, slots = _ctx_and_cache([mixer.cache_need()], cuts)
    x0 = torch.cat([x[:c] for x, c in zip(xs, cuts)]).to(DEV)
    out = mixer.forward(x0, ctx, cache.view(0))
    out = out.sum(0) if out.dim() == 3 else out
    assert rel(out, torch.cat([wt[:c] for wt, c in zip(want, cuts)])) < 2e-5
    _commit(cache, slots, cuts)
    done = list(cuts)
    while any(dn < L for dn, L in zip(done, lens)):
        live = [i for i in range(2) if done[i] < lens[i]]
        ctx, _, _ = _ctx_and_cache(None, [1] * len(live), cache=cache, slots=[slots[i] for i in live])
        x1 = torch.stack([xs[i][done[i]] for i in live]).to(DEV)
        out = mixer.forward(x1, ctx, cache.view(0))
        out = out.sum(0) if out.dim() == 3 else out
        assert rel(out, torch.stack([want[i][done[i]] for i in live])) < 2e-5, done
        _commit(cache, [slots[i] for i in live], [1] * len(live))
        for i in live:
            done[i] += 1


def test_feed_forward_part():
    from llmoxide_b200.parts.registry import FEED_FORWARDS

    cfg, spec, w = _weights_of(TINY_B)
    bs = spec.blocks[2]
    ff = FEED_FORWARDS[bs.feed_forward.kind](bs.feed_forward, {k: v.to(DEV) for k, v in w.items()}, _rt())
    x = torch.randn(11, TINY_B["hidden_size"])
    out = ff.forward(x.to(DEV), None)
    out = out.sum(0) if out.dim() == 3 else out
    assert rel(out, plain.swiglu_ffn(x, plain.layer_weights(w, 2))) < 2e-5


def test_feed_forward_adds_to_residual():
    """A prompt-sized bfloat16 step: the feed-forward adds its result to the stream it is given, inside its last
    product, and says so by returning None.  The stream then holds what adding the returned tensor would give,
    up to that tensor's rounding to bfloat16 (the fused sum skips it)."""
    from llmoxide_b200.parts.registry import FEED_FORWARDS

    cfg, spec, w = _weights_of(TINY_D)
    bs = spec.blocks[1]
    ff = FEED_FORWARDS[bs.feed_forward.kind](bs.feed_forward, {k: v.to(DEV).bfloat16() for k, v in w.items()},
                                             _rt("bfloat16"))
    assert ff.adds_to_residual
    g = torch.Generator().manual_seed(1)
    x = torch.randn(300, TINY_D["hidden_size"], generator=g).bfloat16().to(DEV)
    out = ff.forward(x, None)
    assert out is not None and out.dim() == 2
    h0 = torch.randn(300, TINY_D["hidden_size"], generator=g).to(DEV)
    h = h0.clone()
    assert ff.forward(x, None, residual=h) is None
    assert rel(h - h0, out) < 4e-3 and not torch.equal(h, h0)
    few = x[:40]                     # a step of few tokens keeps the addition for the norm that follows
    h = h0[:40].clone()
    assert ff.forward(few, None, residual=h) is not None and torch.equal(h, h0[:40])


def test_block_part():
    from llmoxide_b200.parts import build_block

    cfg, spec, w = _weights_of(TINY_C)
    blk = build_block(spec.blocks[2], {k: v.to(DEV) for k, v in w.items()}, _rt())
    L, d = 90, TINY_C["hidden_size"]
    h = torch.randn(L, d)
    ctx, cache, slots = _ctx_and_cache([blk.cache_need()], [L])
    hd = h.to(DEV)
    pending = blk.forward(hd, None, ctx, cache.view(0))
    pending = pending.sum(0) if pending.dim() == 3 else pending
    want = plain.block(h, plain.layer_weights(w, 2), TINY_C, list(range(L)), cfg.layer_windows()[2])
    assert rel(hd + pending.float(), want) < 2e-5


# ---- the run order is data ------------------------------------------------------------

def test_layer_named_twice_and_shared_cache(tmp_path):
    """Schedule: layer 0, layer 1, layer 0 again (own cache entry), then layer 2
    reading layer 1's keys and values without writing."""
    from dataclasses import replace

    from llmoxide_b200.config import LayerCall, Qwen3Config, register_architecture
    from llmoxide_b200.engine.engine import Engine, LoadOptions
    from llmoxide_b200.weights import write_model_folder

    class Looped(Qwen3Config):
        def to_spec(self):
            spec = super().to_spec()
            sched = (LayerCall(0, 0), LayerCall(1, 1), LayerCall(0, 2), LayerCall(2, 1, writes_cache=False))
            return replace(spec, schedule=sched)

    register_architecture("LoopedTestLM", Looped)
    raw = dict(TINY_B, architectures=["LoopedTestLM"])
    from llmoxide_b200.config import read_config
    folder = write_model_folder(tmp_path / "looped", read_config(raw), 5, "float32")
    cfg, w = plain.read_model(folder)

    def plain_forward(tokens):
        pos = list(range(len(tokens)))
        eps = raw["rms_norm_eps"]
        h = plain.embed(w["model.embed_tokens.weight"], tokens)
        h = plain.block(h, plain.layer_weights(w, 0), raw, pos, None)
        lw1 = plain.layer_weights(w, 1)
        x1 = plain.rms_norm(h, lw1["input_layernorm.weight"], eps)
        h = plain.block(h, lw1, raw, pos, None)
        h = plain.block(h, plain.layer_weights(w, 0), raw, pos, None)
        # layer 2 with layer 1's keys and values
        lw2 = plain.layer_weights(w, 2)
        T, H, G, D = len(tokens), raw["num_attention_heads"], raw["num_key_value_heads"], raw["head_dim"]
        k = plain.rope_neox(plain.rms_norm(plain.linear(x1, lw1["self_attn.k_proj.weight"]).view(T, G, D),
                                           lw1["self_attn.k_norm.weight"], eps), pos, raw["rope_theta"])
        v = plain.linear(x1, lw1["self_attn.v_proj.weight"]).view(T, G, D)
        x2 = plain.rms_norm(h, lw2["input_layernorm.weight"], eps)
        q = plain.rope_neox(plain.rms_norm(plain.linear(x2, lw2["self_attn.q_proj.weight"]).view(T, H, D),
                                           lw2["self_attn.q_norm.weight"], eps), pos, raw["rope_theta"])
        a = plain.causal_attention(q, k, v, G).reshape(T, H * D)
        h = h + plain.linear(a, lw2["self_attn.o_proj.weight"])
        h = h + plain.swiglu_ffn(plain.rms_norm(h, lw2["post_attention_layernorm.weight"], eps), lw2)
        h = plain.rms_norm(h, w["model.norm.weight"], eps)
        return plain.linear(h, w["lm_head.weight"])

    toks = np.random.default_rng(2).integers(0, raw["vocab_size"], 75).tolist()
    want = plain_forward(toks)
    eng = Engine.load(folder, LoadOptions(dtype="float32", max_tokens=256, max_batch=2))
    assert eng.cache.n_groups() == 1 and eng.cache.k_store[0].shape[0] == 3
    slot = eng.acquire()
    got = [eng.step([(slot, toks[:50])], [list(range(50))])]
    got += [eng.step([(slot, [t])]) for t in toks[50:]]
    assert rel(torch.cat(got), want) < 2e-5


# ---- parts of the test's own ------------------------------------------------------------

def _register_toys():
    from llmoxide_b200.cache import KVNeed, StateNeed
    from llmoxide_b200.parts import (register_embedding, register_feed_forward, register_mixer,
                                     register_position)

    @register_embedding("toy_scaled_table")
    class ScaledTable:
        """h = table[token] * scale: an embedding with a scale (the dense Qwen3 decoder has none)."""

        def __init__(self, spec, weights, rt):
            self.table = weights[spec.tensors["table"].name]        # left in: the tied head shares it
            self.scale = float(spec["scale"])

        def forward(self, tokens, h):
            h.copy_(self.table[tokens.long()].float() * self.scale)

    @register_mixer("toy_running_mean")
    class RunningMean:
        """y_t = W * mean(x_0..x_t): its state is the running sum and the count, per sequence, of fixed
        size, kept in the cache's state area.  Everything is computed on the device from the step's own
        index arrays (no host read), so decode steps with this mixer are captured as CUDA graphs."""

        def __init__(self, spec, position, weights, rt):
            self.d = spec["hidden_size"]
            self.w = weights.pop(spec.tensors["w"].name).float()

        def cache_need(self):
            return None, StateNeed((self.d + 1,))

        def forward(self, x, ctx, view, writes_cache=True):
            d, T = self.d, x.shape[0]
            seq = ctx.token_seq.long()                               # token -> sequence of the step
            start = ctx.seq_start.long()
            idx = torch.arange(T, device=x.device)
            # running sums inside each sequence's run of tokens (float64, so that the cut does not show)
            cs = torch.cat([torch.zeros(1, d, dtype=torch.float64, device=x.device), x.double().cumsum(0)])
            within = (cs[idx + 1] - cs[start[seq]]).float()
            n_within = (idx - start[seq] + 1).float()
            state = view.state[ctx.seq_slot.long()[seq]]             # [T, d + 1]: each token's sequence state
            sums, counts = state[:, :d] + within, state[:, d] + n_within
            if writes_cache:
                last = start[1:] - 1                                 # every sequence's last token
                view.state.index_copy_(0, ctx.seq_slot.long(), torch.cat([sums[last], counts[last, None]], dim=1))
            return (sums / counts[:, None]) @ self.w.t()

    @register_mixer("toy_previous_value")
    class PreviousValue:
        """y_t = W v_{t-1} with v_t = the first 8 dims of x_t (zero at a sequence's first position): a mixer that
        keeps values narrower than its keys, in float64 whatever the model's dtype, in the paged cache, and
        finds them through the step's block table.  All on the device."""

        def __init__(self, spec, position, weights, rt):
            self.w = weights.pop(spec.tensors["w"].name).float()          # [d, 8]

        def cache_need(self):
            return KVNeed(n_kv_heads=1, head_dim=16, v_head_dim=8, dtype=torch.float64), None

        def forward(self, x, ctx, view, writes_cache=True):
            assert view.v.shape[-1] == 8 and view.k.shape[-1] == 16 and view.v.dtype == torch.float64
            table = ctx.block_tables[view.group].long()
            seq, pos = ctx.token_seq.long(), ctx.token_pos.long()
            page = table[seq, pos // 64]
            if writes_cache:
                view.v[page, 0, pos % 64] = x[:, :8].double()
            prev = (pos - 1).clamp(min=0)
            v_prev = view.v[table[seq, prev // 64], 0, prev % 64].float() * (pos > 0).float()[:, None]
            return v_prev @ self.w.t()

    @register_feed_forward("toy_routed")
    class Routed:
        """Two experts of one matrix each; a token goes to the expert with the
        larger router logit (float32), so routing is per token and does not
        depend on the batch."""

        def __init__(self, spec, weights, rt):
            self.router = weights.pop(spec.tensors["router"].name).float()
            self.experts = [weights.pop(spec.tensors[f"e{i}"].name).float() for i in range(2)]

        def forward(self, x, ctx):
            x = x.float()
            pick = (x @ self.router.t()).argmax(-1)
            outs = torch.stack([torch.tanh(x @ e.t()) for e in self.experts])
            return outs[pick, torch.arange(len(x), device=x.device)]

    @register_position("toy_half_speed")
    class HalfSpeed:
        """Rotation tables for angle (pos / 2) * base^(-2i/n_rot)."""

        def __init__(self, spec, weights, rt):
            self.n_rot, self.base, self.rt = spec["n_rot"], spec["base"], rt
            half = self.n_rot // 2
            pos = torch.arange(self.rt.max_positions, dtype=torch.float64) / 2
            freq = self.base ** (-2.0 * torch.arange(half, dtype=torch.float64) / self.n_rot)
            ang = pos[:, None] * freq[None, :]
            self.tables = ang.cos().float().to(DEV), ang.sin().float().to(DEV), self.n_rot

        def rotary_tables(self):      # made once: a step, which may be captured as a CUDA graph, only reads them
            return self.tables


def test_toy_parts_register_build_and_step(tmp_path):
    from llmoxide_b200.config import (BlockSpec, ModelSpec, PartSpec, TensorSpec, default_schedule,
                                      register_architecture)
    from llmoxide_b200.engine.engine import Engine, LoadOptions
    from llmoxide_b200.weights import write_model_folder

    _register_toys()
    d, V, H, D = 48, 101, 3, 16

    @dataclass
    class ToyConfig:
        raw: dict

        @classmethod
        def from_dict(cls, raw):
            return cls(raw)

        def to_dict(self):
            return dict(self.raw)

        def to_spec(self):
            norm = lambda n: PartSpec("rms_norm", dict(size=d, eps=1e-5), dict(gain=TensorSpec(n, (d,), "vector")))
            attn = PartSpec("gqa_attention", dict(hidden_size=d, n_heads=H, n_kv_heads=1, head_dim=D,
                                                  scale=1 / math.sqrt(D), window=None, qk_norm_eps=0.0),
                            dict(q=TensorSpec("l1.q", (H * D, d)), k=TensorSpec("l1.k", (D, d)),
                                 v=TensorSpec("l1.v", (D, d)), o=TensorSpec("l1.o", (d, H * D))))
            blocks = (
                BlockSpec("pre_norm", PartSpec("toy_running_mean", dict(hidden_size=d), dict(w=TensorSpec("l0.w", (d, d)))),
                          PartSpec("toy_routed", {}, dict(router=TensorSpec("l0.router", (2, d)),
                                                          e0=TensorSpec("l0.e0", (d, d)), e1=TensorSpec("l0.e1", (d, d)))),
                          dict(mixer=norm("l0.n1"), feed_forward=norm("l0.n2"))),
                BlockSpec("pre_norm", attn,
                          PartSpec("gated_mlp", dict(hidden_size=d, intermediate_size=64, activation="silu"),
                                   dict(gate=TensorSpec("l1.g", (64, d)), up=TensorSpec("l1.u", (64, d)),
                                        down=TensorSpec("l1.d", (d, 64)))),
                          dict(mixer=norm("l1.n1"), feed_forward=norm("l1.n2")),
                          PartSpec("toy_half_speed", dict(n_rot=D, base=100.0))),
            )
            blocks = blocks + (
                BlockSpec("pre_norm", PartSpec("toy_previous_value", {}, dict(w=TensorSpec("l2.w", (d, 8)))),
                          PartSpec("gated_mlp", dict(hidden_size=d, intermediate_size=64, activation="silu"),
                                   dict(gate=TensorSpec("l2.g", (64, d)), up=TensorSpec("l2.u", (64, d)),
                                        down=TensorSpec("l2.d", (d, 64)))),
                          dict(mixer=norm("l2.n1"), feed_forward=norm("l2.n2"))),
            )
            return ModelSpec("ToyLM", d, V,
                             PartSpec("toy_scaled_table", dict(scale=3.0), dict(table=TensorSpec("emb", (V, d)))),
                             blocks, default_schedule(3), norm("final"),
                             PartSpec("linear", dict(tied=True, softcap=5.0), {}),
                             max_positions=512, storage_dtype="float32")

    register_architecture("ToyLM", ToyConfig)
    folder = write_model_folder(tmp_path / "toy", ToyConfig(dict(architectures=["ToyLM"])), 9)
    eng = Engine.load(folder, LoadOptions(dtype="float32", max_tokens=512, max_batch=2))
    assert eng.cache.state_store[0].shape == (2, d + 1) and eng.cache.state_store[1] is None
    assert eng.cache.n_groups() == 2          # the attention layer's keys and values, and the toy's narrower values
    assert eng.cache.v_store[1].shape[-1] == 8 and eng.cache.k_store[1].shape[-1] == 16
    assert eng.model.graph_safe and eng.options.cuda_graphs      # decode steps of this model replay CUDA graphs

    rng = np.random.default_rng(0)
    seqs = [rng.integers(0, V, n).tolist() for n in (37, 80, 5)]

    def whole(toks):
        s = eng.acquire()
        out = eng.step([(s, toks)], [list(range(len(toks)))]).cpu()
        eng.release(s)
        return out

    ref = [whole(t) for t in seqs]
    # cut differently, batched, and in slots whose last owner left state behind
    a, b = eng.acquire(), eng.acquire()
    got_a = [eng.step([(a, seqs[0][:10]), (b, seqs[1][:33])], [list(range(10)), list(range(33))]).cpu()]
    rows_a, rows_b = [got_a[0][:10]], [got_a[0][10:]]
    for i in range(10, 37):
        out = eng.step([(a, [seqs[0][i]]), (b, [seqs[1][23 + i]])]).cpu()
        rows_a.append(out[:1]), rows_b.append(out[1:])
    eng.release(a)
    c = eng.acquire()                                   # takes over a's slot: its state must start at zero
    assert c == a
    rows_c = []
    for i in range(60, 80):
        entries = [(b, [seqs[1][i]])] + ([(c, [seqs[2][i - 60]])] if i - 60 < 5 else [])
        out = eng.step(entries).cpu()
        rows_b.append(out[:1])
        if len(entries) == 2:
            rows_c.append(out[1:])
    assert rel(torch.cat(rows_a), ref[0]) < 1e-5
    assert rel(torch.cat(rows_b), ref[1]) < 1e-5
    assert rel(torch.cat(rows_c), ref[2]) < 1e-5
    assert len(eng._graphs) >= 2 and eng.options.cuda_graphs     # batch shapes of 2 and 1 were captured
    # the parts of the test's own are in the result: the embedding's scale and the head's cap
    assert float(ref[0].abs().max()) <= 5.0
    emb = eng.model.embedding
    assert type(emb).__name__ == "ScaledTable" and eng.model.head.linear.weight.data_ptr() == emb.table.data_ptr()
