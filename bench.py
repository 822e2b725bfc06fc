"""Benchmark: decode tokens per second and prefill tokens per second of the
dense Qwen3 decoder at Qwen3-8B layer sizes, bfloat16, random weights, on one
B200.  A "step" is one decode step of a batch of 8 sequences from depth 2048
(context 4096 per sequence).  Prints ONE JSON line.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--layers L] [--impl reference]

``value`` is device-timed (CUDA events around K steps queued back to back);
``e2e`` is the same metric through ``Session.generate`` with host token ids in
and out, every step copying its inputs from pinned host memory and reading
the sampled tokens back.  Weights (16 GB) and cache are far larger than L2,
so nothing is flushed between steps.
"""

from __future__ import annotations

import argparse
import json
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent

# The benchmark's model: Qwen3-8B layer sizes
QWEN3_8B = dict(
    architectures=["Qwen3ForCausalLM"], model_type="qwen3", num_hidden_layers=36, hidden_size=4096,
    num_attention_heads=32, num_key_value_heads=8, head_dim=128, intermediate_size=12288, vocab_size=151936,
    rope_theta=1000000.0, rms_norm_eps=1e-6, tie_word_embeddings=False, max_position_embeddings=40960,
    use_sliding_window=False, sliding_window=None, torch_dtype="bfloat16", eos_token_id=151645,
)
FALLBACK_PEAKS = dict(hbm_gbs=6650.0, bf16_tflops=1590.0, bf16_tflops_sustained=1400.0)


def peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.is_file():
        try:
            raw = json.loads(p.read_text())
            out = dict(FALLBACK_PEAKS)
            out.update({k: float(v) for k, v in raw.items() if k in out and isinstance(v, (int, float))})
            return out, "measured"
        except (ValueError, OSError):
            pass
    return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    """nvidia-smi clocks and throttle reasons during the timed region."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.proc, self.lines = None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "50"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if self.proc is None:
            return dict(sm_mhz=None, sm_max_mhz=None, reasons=["nvidia-smi unavailable"])
        time.sleep(0.25)
        self.proc.terminate()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0])), mx.append(float(parts[1]))
            except ValueError:
                continue
            for n, v in zip(names, parts[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return dict(sm_mhz=statistics.median(sm) if sm else None, sm_max_mhz=max(mx) if mx else None,
                    reasons=sorted(reasons), samples=len(sm))


def model_numbers(cfg, n_layers):
    """Bytes a decode step must read and FLOPs a prompt step must do."""
    d, f, V = cfg.hidden_size, cfg.intermediate_size, cfg.vocab_size
    per_layer = d * (cfg.q_dim + 2 * cfg.kv_dim) + cfg.q_dim * d + 3 * d * f
    weight_bytes = 2 * (n_layers * per_layer + V * d) + 4 * (n_layers * (2 * d + 2 * cfg.head_dim) + d)
    kv_bytes_per_token = n_layers * 2 * cfg.kv_dim * 2

    def prefill_flops(T):
        gemm = 2.0 * T * n_layers * per_layer + 2.0 * V * d           # the head runs on one row
        attn = n_layers * 2.0 * 2.0 * cfg.q_dim * (T * (T + 1) / 2)   # QK^T and PV over the causal half
        return gemm + attn

    return weight_bytes, kv_bytes_per_token, prefill_flops


def timeline(eng, cfg, args, rng) -> int:
    """One replayed decode step seen from inside: every kernel's first thread records when it reached its
    programmatic-launch wait and when the wait returned.  The time from one kernel's return to the next one's is
    that kernel's share of the step's critical path, measured in place (CUDA graph, overlapping launches)."""
    import ctypes
    import re
    from collections import defaultdict

    import torch
    from llmoxide_b200.csrc.build import LIBRARIES, SRC_DIR, load_library

    B, V = args.batch, cfg.vocab_size
    slots = [eng.acquire() for _ in range(B)]
    for s in slots:
        eng.step([(s, rng.integers(0, V, args.depth).tolist())], [[]])

    def step():
        eng.step([(s, [int(rng.integers(0, V))]) for s in slots])

    for _ in range(max(args.warmup, 4)):
        step()
    libs = ("elementwise", "gemm_tc", "attention_decode")

    def kernel_at(lib, line):
        src = (SRC_DIR / LIBRARIES[lib][0][0]).read_text().splitlines()
        for i in range(line - 1, -1, -1):
            m = re.search(r"^\s*(\w+_kernel)\(", src[i]) or re.search(r"__global__.*?(\w+_kernel)\(", src[i])
            if m:
                return m.group(1)
        return f"{lib}:{line}"

    def read_all():
        out = []
        for lib in libs:
            fn = load_library(lib).llmx_timeline_read
            fn.restype = ctypes.c_int
            buf = (ctypes.c_ulonglong * (3 * 65536))()
            n = fn(buf, 65536)
            if n < 0:
                raise RuntimeError(f"timeline of {lib}: CUDA error {-n}")
            out += [(buf[3 * i + 2], buf[3 * i + 1], lib, int(buf[3 * i])) for i in range(n) if buf[3 * i] < 1000000]
        return sorted(out)

    read_all()
    step()
    torch.cuda.synchronize()
    recs = read_all()
    t0 = recs[0][0]
    share = defaultdict(list)
    print(f"{'#':>4} {'kernel':34} {'resident':>10} {'ready':>10} {'to next':>9}   (us)", file=sys.stderr)
    for i, (ready, reached, lib, line) in enumerate(recs):
        name = kernel_at(lib, line)
        nxt = recs[i + 1][0] if i + 1 < len(recs) else ready
        share[name].append((nxt - ready) / 1e3)
        print(f"{i:4d} {name:34} {(reached - t0) / 1e3:10.2f} {(ready - t0) / 1e3:10.2f} {(nxt - ready) / 1e3:9.2f}",
              file=sys.stderr)
    total = (recs[-1][0] - t0) / 1e3
    summary = {k: dict(n=len(v), mean_us=round(sum(v) / len(v), 2), sum_us=round(sum(v), 1)) for k, v in share.items()}
    print(json.dumps(dict(timeline="one decode step", batch=B, depth=args.depth, layers=args.layers,
                          kernels=len(recs), step_us=round(total, 1), per_kernel=summary)))
    return 0


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours")
    ap.add_argument("--layers", type=int, default=QWEN3_8B["num_hidden_layers"],
                    help="fewer layers than the configuration has, for a quick run; reported in config")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=4096)
    ap.add_argument("--depth", type=int, default=2048)
    ap.add_argument("--prefill-tokens", type=int, default=2048)
    ap.add_argument("--no-points", action="store_true", help="skip the batch 1 and batch 64 points")
    ap.add_argument("--no-graphs", action="store_true")
    ap.add_argument("--timeline", action="store_true",
                    help="instead of the benchmark: build the kernels with their in-place timers and print, for "
                         "one replayed decode step, when each kernel's dependency resolved")
    ap.add_argument("--cuda-profiler", choices=["decode", "prefill"], default=None,
                    help="bracket that region with cudaProfilerStart/Stop (for ncu --profile-from-start off)")
    args = ap.parse_args()

    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "bigmah/llmoxide is a Rust workspace over wgpu; no Rust toolchain and no graphics stack "
                          "here, so pip cannot install it and its GPU path cannot run"}))
        return 0
    if args.gpus != 1:
        print(json.dumps({"note": f"this library runs on one GPU; --gpus {args.gpus} is not supported", "n_gpus": args.gpus}))
        return 2

    if args.timeline:
        import os
        os.environ["LLMX_NVCC_EXTRA"] = (os.environ.get("LLMX_NVCC_EXTRA", "") + " -DLLMX_TIMELINE").strip()

    import numpy as np
    import torch

    sys.path.insert(0, str(ROOT))
    from llmoxide_b200 import LoadOptions, Request, Sampling, Session, kernels, read_config

    raw = dict(QWEN3_8B, num_hidden_layers=args.layers)
    cfg = read_config(raw)
    pk, pk_src = peaks()
    B, K, W = args.batch, args.steps, args.warmup
    big_b = 1 if args.no_points else 64
    max_b = max(B, big_b)
    opts = LoadOptions(dtype="bfloat16", max_tokens=max_b * args.context, max_batch=max_b,
                       max_step_tokens=max(args.prefill_tokens, B * args.depth), cuda_graphs=not args.no_graphs)
    t_load = time.time()
    session = Session.random(cfg, seed=0, options=opts)
    eng = session.engine
    torch.cuda.synchronize()
    print(f"[bench] model ready in {time.time() - t_load:.1f} s: {cfg.summary()}", file=sys.stderr)
    weight_bytes, kv_per_token, prefill_flops = model_numbers(cfg, args.layers)
    rng = np.random.default_rng(0)
    V = cfg.vocab_size

    def event_time(fn):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b)

    if args.timeline:
        return timeline(eng, cfg, args, rng)

    # ---- prefill: one prompt of 2,048 tokens ----------------------------------
    T = args.prefill_tokens
    prompt = rng.integers(0, V, T).tolist()

    def one_prefill():
        slot = eng.acquire()
        eng.step([(slot, prompt)])
        eng.release(slot)

    for _ in range(3):
        one_prefill()
    if args.cuda_profiler == "prefill":
        torch.cuda.profiler.start()
        one_prefill()
        torch.cuda.synchronize()
        torch.cuda.profiler.stop()
    prefill_ms = statistics.median(event_time(one_prefill) for _ in range(5))
    prefill = dict(value=T / prefill_ms * 1e3, tokens=T, ms=prefill_ms,
                   frac=prefill_flops(T) / (prefill_ms * 1e-3) / (pk["bf16_tflops"] * 1e12),
                   tflops=prefill_flops(T) / (prefill_ms * 1e-3) / 1e12)
    print(f"[bench] prefill {T} tokens: {prefill_ms:.2f} ms", file=sys.stderr)

    # ---- decode: B sequences at depth, K steps ----------------------------------
    def decode_rate(batch, steps, warmup, sampler=None):
        slots = [eng.acquire() for _ in range(batch)]
        for s in slots:
            eng.step([(s, rng.integers(0, V, args.depth).tolist())], [[]])
        toks = rng.integers(0, V, (warmup + steps, batch)).tolist()
        for i in range(warmup):
            eng.step([(s, [t]) for s, t in zip(slots, toks[i])])
        launches = kernels.launch_count
        if sampler:
            sampler.start()

        def run():
            for i in range(warmup, warmup + steps):
                eng.step([(s, [t]) for s, t in zip(slots, toks[i])])

        if sampler and args.cuda_profiler == "decode":
            torch.cuda.profiler.start()
        ms = event_time(run)
        if sampler and args.cuda_profiler == "decode":
            torch.cuda.profiler.stop()
        clocks = sampler.stop() if sampler else None
        launches = kernels.launch_count - launches
        for s in slots:
            eng.release(s)
        return batch * steps / ms * 1e3, ms / steps, launches, clocks

    value, ms_per_step, launches, clocks = decode_rate(B, K, max(W, 3), ClockSampler())
    mean_depth = args.depth + max(W, 3) + K / 2
    step_bytes = weight_bytes + B * mean_depth * kv_per_token
    achieved = step_bytes / (ms_per_step * 1e-3) / 1e9
    print(f"[bench] decode b{B}: {ms_per_step:.3f} ms/step, {value:.0f} tok/s, {achieved:.0f} GB/s", file=sys.stderr)

    # ---- end to end through the Python entry point --------------------------------
    reqs = [Request(rng.integers(0, V, args.depth).tolist(), max_tokens=K + 1, sampling=Sampling.greedy(),
                    stop_ids=()) for _ in range(B)]
    session.loop.stop_ids = frozenset()
    session.generate([Request(r.prompt[:64], max_tokens=4, sampling=Sampling.greedy()) for r in reqs])  # warm
    t0 = session.timings.decode_seconds, session.timings.decode_tokens
    session.generate(reqs)
    e2e_s = session.timings.decode_seconds - t0[0]
    e2e_tok = session.timings.decode_tokens - t0[1]
    lay_ints = 3 * B + (B + 1) + 2 * B + B + B * max(8, -(-((args.depth + K + 64) // 64) // 8) * 8)
    e2e = dict(value=e2e_tok / e2e_s, unit="tokens/s", h2d_bytes_per_step=4 * lay_ints, d2h_bytes_per_step=4 * B)
    print(f"[bench] e2e decode b{B}: {e2e['value']:.0f} tok/s", file=sys.stderr)

    points = {}
    if not args.no_points:
        points["decode_b1"] = decode_rate(1, max(16, K // 2), 3)[0]
        points["decode_b64"] = decode_rate(64, max(8, K // 4), 3)[0]

    line = dict(
        metric="decode tok/s at batch 8 from depth 2048, Qwen3-8B layer sizes, bf16", value=value, unit="tokens/s",
        n_gpus=1, steps=K, warmup=max(W, 3), ms_per_step=ms_per_step, higher_is_better=True, scaling="weak",
        vs_baseline=None, dtype="bf16", data="synthetic: seeded uniform token ids, random weights N(0,0.02)",
        impl="ours",
        config=dict(model="Qwen3-8B layer sizes", layers=args.layers, layers_of_model=QWEN3_8B["num_hidden_layers"],
                    hidden=cfg.hidden_size, heads=cfg.num_attention_heads, kv_heads=cfg.num_key_value_heads,
                    head_dim=cfg.head_dim, intermediate=cfg.intermediate_size, vocab=cfg.vocab_size,
                    global_batch=B, seq_len=args.context, depth=args.depth, prefill_tokens=T,
                    parallelism="single GPU", l2="weights and cache far larger than L2; no flush",
                    cuda_graphs=not args.no_graphs, peaks=pk_src),
        prefill=prefill,
        roofline=dict(bound="hbm", achieved=achieved, peak=pk["hbm_gbs"], unit="GB/s", frac=achieved / pk["hbm_gbs"]),
        points=points, e2e=e2e, gpu_launches=launches, clocks=clocks,
    )
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
