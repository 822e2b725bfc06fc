"""Helpers for the replay tests: build traces for the three ways of cutting
the same requests, run them through the engine's replayer (in process) or
through ``bin/trace_run`` (as a user runs it), and compare with the plain
implementation position by position."""

import json
import subprocess
import sys
from pathlib import Path

import numpy as np
import torch

import plain_qwen3 as plain

ROOT = Path(__file__).resolve().parent.parent

# max |delta| / max |expected| over a request's logits.  float32: summation
# order is the only difference.  bfloat16: activations are rounded to 8 bits
# of mantissa between kernels.
TOL = {"float32": 2e-5, "bfloat16": 2e-2}


def trace_whole(requests):
    """Each request alone and whole: one step, every position wanted."""
    steps = []
    for i, (rid, toks) in enumerate(requests.items()):
        steps.append(dict(step=i, entries=[dict(id=rid, tokens=toks, want=list(range(len(toks))))], end=[rid]))
    return steps


def trace_tail_decode(requests, tail=32):
    """The prefix whole, then the last ``tail`` tokens one by one."""
    steps, n = [], 0
    for rid, toks in requests.items():
        cut = max(1, len(toks) - tail)
        steps.append(dict(step=n, entries=[dict(id=rid, tokens=toks[:cut], want=list(range(cut)))],
                          end=[rid] if cut == len(toks) else []))
        n += 1
        for j in range(cut, len(toks)):
            last = j == len(toks) - 1
            steps.append(dict(step=n, entries=[dict(id=rid, tokens=[toks[j]], want=[0])], end=[rid] if last else []))
            n += 1
    return steps


def trace_batches(requests, batch_size, prompt_frac=0.5):
    """Batches of unequal lengths, one after another: a prompt step with every
    request's first part, then one token each; shorter requests end earlier."""
    steps, n = [], 0
    items = list(requests.items())
    for b in range(0, len(items), batch_size):
        group = items[b : b + batch_size]
        cuts = {rid: max(1, int(len(t) * prompt_frac)) for rid, t in group}
        ends = [rid for rid, t in group if cuts[rid] == len(t)]
        steps.append(dict(step=n, entries=[dict(id=rid, tokens=t[: cuts[rid]], want=list(range(cuts[rid])))
                                           for rid, t in group], end=ends))
        n += 1
        live = [(rid, t) for rid, t in group if cuts[rid] < len(t)]
        k = 0
        while live:
            entries = [dict(id=rid, tokens=[t[cuts[rid] + k]], want=[0]) for rid, t in live]
            ends = [rid for rid, t in live if cuts[rid] + k == len(t) - 1]
            steps.append(dict(step=n, entries=entries, end=ends))
            n += 1
            k += 1
            live = [(rid, t) for rid, t in live if cuts[rid] + k < len(t)]
    return steps


def trace_chunks(requests, chunk, batch_size, tail=8, mixed=False):
    """Prompts fed in several multi-token steps (a later chunk of a prompt attends over the cache and the
    chunk itself), several requests per step, then the last ``tail`` tokens one by one.  With ``mixed`` a
    request goes on to single tokens as soon as its own prompt is through, so a step may hold one request's
    chunk beside another's single token; without it, the requests that are through wait for the others."""
    steps, n = [], 0
    items = list(requests.items())
    for b in range(0, len(items), batch_size):
        group = items[b : b + batch_size]
        fed = {rid: 0 for rid, _ in group}
        cut = {rid: max(1, len(t) - tail) for rid, t in group}
        live = list(group)
        while live:
            in_prompt = [rid for rid, _ in live if fed[rid] < cut[rid]]
            entries = []
            for rid, t in live:
                if fed[rid] < cut[rid]:
                    m = min(chunk, cut[rid] - fed[rid])
                elif mixed or not in_prompt:
                    m = 1
                else:
                    continue
                entries.append(dict(id=rid, tokens=t[fed[rid] : fed[rid] + m], want=list(range(m))))
                fed[rid] += m
            ends = [rid for rid, t in live if fed[rid] == len(t)]
            steps.append(dict(step=n, entries=entries, end=ends))
            n += 1
            live = [(rid, t) for rid, t in live if fed[rid] < len(t)]
    return steps


def collect(steps, out_dir, vocab):
    """{request id: [len, vocab] logits} put together from the step files."""
    got = {}
    for st in steps:
        wanted = sum(len(e["want"]) for e in st["entries"])
        if not wanted:
            continue
        arr = np.fromfile(Path(out_dir) / f"{st['step']}.f32", dtype="<f4").reshape(wanted, vocab)
        at = 0
        for e in st["entries"]:
            for _ in e["want"]:
                got.setdefault(e["id"], []).append(arr[at])
                at += 1
    return {rid: np.stack(rows) for rid, rows in got.items()}


def run_in_process(engine, steps, out_dir):
    from llmoxide_b200.engine.replay import Replayer

    rp = Replayer(engine, out_dir)
    for st in steps:
        rp.run_step(st)
    assert not rp.slots, "every request of a trace ends"
    engine.cache.alloc.check_consistent()
    assert engine.cache.alloc.pages_held() == 0


def run_trace_run(folder, dtype, steps, out_dir, max_tokens, env=None, cwd=None, exe=None):
    text = "".join(json.dumps(s) + "\n" for s in steps)
    cmd = [sys.executable, str(exe or ROOT / "bin" / "trace_run"), "--model", str(folder), "--dtype", dtype,
           "--out", str(out_dir), "--max-tokens", str(max_tokens)]
    p = subprocess.run(cmd, input=text, capture_output=True, text=True, env=env, cwd=cwd, timeout=900)
    assert p.returncode == 0, p.stderr[-4000:]
    done = [l for l in p.stdout.splitlines() if l.startswith("done ")]
    assert [int(l.split()[1]) for l in done] == [s["step"] for s in steps]
    return p


def expected_logits(folder, requests):
    cfg, w = plain.read_model(folder)
    return {rid: plain.forward(cfg, w, toks).numpy() for rid, toks in requests.items()}


def rel_err(got, want):
    return float(np.abs(got - want).max() / np.abs(want).max())


def first_bad_position(got, want, tol):
    scale = np.abs(want).max()
    bad = np.nonzero(np.abs(got - want).max(axis=1) > tol * scale)[0]
    return int(bad[0]) if len(bad) else None


def assert_matches(got, want, dtype, what):
    for rid in want:
        assert got[rid].shape == want[rid].shape, (what, rid, got[rid].shape, want[rid].shape)
        err = rel_err(got[rid], want[rid])
        if not err <= TOL[dtype]:
            pos = first_bad_position(got[rid], want[rid], TOL[dtype])
            raise AssertionError(
                f"{what}: request {rid!r} ({len(want[rid])} tokens) differs from the plain implementation, "
                f"rel err {err:.3e} > {TOL[dtype]:.1e}; first wrong position {pos}")
