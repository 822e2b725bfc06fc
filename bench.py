"""Benchmark: decode tokens per second and prefill tokens per second of the
dense Qwen3 decoder at Qwen3-8B layer sizes, bfloat16, random weights, on one
B200.  A "step" is one decode step of a batch of 8 sequences from depth 2048
(context 4096 per sequence).  Prints ONE JSON line.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--layers L] [--impl reference]
    python bench.py --cpu-baseline      # the plain implementation of tests/ on the CPU, tiny configurations

``value`` is device-timed (CUDA events around K steps queued back to back);
``e2e`` is the same metric through ``Session.generate`` with host token ids in
and out, every step copying its inputs from pinned host memory and reading
the sampled tokens back, over at least 256 steps.  ``points`` has the same at
batch 1 and 64 and the prefill rate at other lengths (tokens per second);
``point_details`` has their milliseconds, roofline fractions, end-to-end rates
and the host's microseconds per step.  Weights (16 GB) and cache are far
larger than L2, so nothing is flushed between steps.
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
    ap.add_argument("--cpu-baseline", action="store_true",
                    help="instead of the benchmark: time the plain implementation of tests/ on the CPU (tiny configurations)")
    ap.add_argument("--cuda-profiler", choices=["decode", "prefill"], default=None,
                    help="bracket that region with cudaProfilerStart/Stop (for ncu --profile-from-start off)")
    args = ap.parse_args()

    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "bigmah/llmoxide is a Rust workspace over wgpu; no Rust toolchain and no graphics stack "
                          "here, so pip cannot install it and its GPU path cannot run"}))
        return 0
    if args.cpu_baseline:
        return cpu_baseline()
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
                       max_step_tokens=max(args.prefill_tokens, B * args.depth, 0 if args.no_points else 16 * 2048),
                       cuda_graphs=not args.no_graphs)
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

    def prefill_time(lengths, profile=False):
        """Median milliseconds of one prompt step over sequences of these lengths (slots taken and given back)."""
        prompts = [rng.integers(0, V, n).tolist() for n in lengths]

        def one():
            slots = [eng.acquire() for _ in prompts]
            eng.step(list(zip(slots, prompts)))
            for s in slots:
                eng.release(s)

        for _ in range(3):
            one()
        if profile:
            torch.cuda.profiler.start()
            one()
            torch.cuda.synchronize()
            torch.cuda.profiler.stop()
        return statistics.median(event_time(one) for _ in range(5))

    def prefill_point(lengths, profile=False):
        ms = prefill_time(lengths, profile)
        flops = sum(prefill_flops(n) for n in lengths)
        # (a short prompt step whose shape comes back is replayed as a graph by the engine: say so)
        graph = bool(eng.options.cuda_graphs and sum(lengths) <= eng.options.graph_prompt_tokens)
        return dict(value=sum(lengths) / ms * 1e3, tokens=sum(lengths), ms=ms,
                    frac=flops / (ms * 1e-3) / (pk["bf16_tflops"] * 1e12), tflops=flops / (ms * 1e-3) / 1e12,
                    graph=graph)

    prefill = prefill_point([T], profile=args.cuda_profiler == "prefill")
    print(f"[bench] prefill {T} tokens: {prefill['ms']:.2f} ms", file=sys.stderr)

    # ---- decode: B sequences at depth, K steps ----------------------------------
    def decode_rate(batch, steps, warmup, sampler=None, depth=None):
        depth = depth or args.depth
        slots = [eng.acquire() for _ in range(batch)]
        for s in slots:
            for lo in range(0, depth, 8192):          # deep contexts are fed in chunks
                eng.step([(s, rng.integers(0, V, min(8192, depth - lo)).tolist())], [[]])
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
        mean_depth = depth + warmup + steps / 2
        step_bytes = weight_bytes + batch * mean_depth * kv_per_token
        gbs = step_bytes / (ms / steps * 1e-3) / 1e9
        return dict(value=batch * steps / ms * 1e3, ms_per_step=ms / steps, gb_per_s=gbs, frac=gbs / pk["hbm_gbs"],
                    launches=launches, clocks=clocks)

    main_pt = decode_rate(B, K, max(W, 3), ClockSampler())
    value, ms_per_step, launches, clocks = main_pt["value"], main_pt["ms_per_step"], main_pt["launches"], main_pt["clocks"]
    achieved = main_pt["gb_per_s"]
    print(f"[bench] decode b{B}: {ms_per_step:.3f} ms/step, {value:.0f} tok/s, {achieved:.0f} GB/s", file=sys.stderr)

    # ---- end to end through the Python entry point --------------------------------
    session.loop.stop_ids = frozenset()

    def e2e_rate(batch, steps):
        """Decoded tokens per second through Session.generate (host ids in, host ids out), and the host's own
        time per step.  A short run over the same prompts first, so that the batch's shape has its CUDA graph."""
        prompts = [rng.integers(0, V, args.depth).tolist() for _ in range(batch)]
        session.generate([Request(p, max_tokens=3, sampling=Sampling.greedy(), stop_ids=()) for p in prompts])
        t0 = session.timings.decode_seconds, session.timings.decode_tokens, eng.host_seconds, eng.n_steps
        session.generate([Request(p, max_tokens=steps + 1, sampling=Sampling.greedy(), stop_ids=()) for p in prompts])
        secs = session.timings.decode_seconds - t0[0]
        toks = session.timings.decode_tokens - t0[1]
        host_us = (eng.host_seconds - t0[2]) / max(1, eng.n_steps - t0[3] - 1) * 1e6
        return toks / secs, host_us

    e2e_steps = max(K, 256)
    e2e_value, host_us = e2e_rate(B, e2e_steps)
    lay_ints = 3 * B + (B + 1) + 2 * B + B + B * max(8, -(-((args.depth + e2e_steps + 64) // 64) // 8) * 8)
    e2e = dict(value=e2e_value, unit="tokens/s", steps=e2e_steps, h2d_bytes_per_step=4 * lay_ints,
               d2h_bytes_per_step=4 * B, host_us_per_step=host_us)
    print(f"[bench] e2e decode b{B}: {e2e_value:.0f} tok/s over {e2e_steps} steps, host {host_us:.0f} us/step", file=sys.stderr)

    points, details = {}, {}
    if not args.no_points:
        for batch, steps in ((1, max(16, K // 2)), (64, max(8, K // 4))):
            pt = decode_rate(batch, steps, 3)
            rate, h_us = e2e_rate(batch, 256 if batch == 1 else 96)
            points[f"decode_b{batch}"] = pt["value"]
            details[f"decode_b{batch}"] = dict(ms_per_step=pt["ms_per_step"], gb_per_s=pt["gb_per_s"], frac=pt["frac"],
                                               e2e=rate, e2e_frac_of_device=rate / pt["value"], host_us_per_step=h_us)
        details[f"decode_b{B}"] = dict(ms_per_step=ms_per_step, gb_per_s=achieved, frac=main_pt["frac"], e2e=e2e_value,
                                       e2e_frac_of_device=e2e_value / value, host_us_per_step=host_us)
        for batch, depth in ((8, 8192), (1, 32768)):       # deeper contexts: the cache outweighs the weights
            pt = decode_rate(batch, 16, 3, depth=depth)
            points[f"decode_b{batch}_depth{depth}"] = pt["value"]
            details[f"decode_b{batch}_depth{depth}"] = dict(ms_per_step=pt["ms_per_step"], gb_per_s=pt["gb_per_s"],
                                                            frac=pt["frac"])
        lens16 = rng.integers(64, 2049, 16).tolist()       # an unequal batch: 16 prompts of 64..2048 tokens
        for name, lengths in (("prefill_512", [512]), ("prefill_8192", [8192]), ("prefill_16_unequal", lens16)):
            pp = prefill_point(lengths)
            points[name] = pp["value"]
            details[name] = dict(tokens=pp["tokens"], ms=pp["ms"], frac=pp["frac"], tflops=pp["tflops"],
                                 graph=pp["graph"])

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
        points=points, point_details=details, e2e=e2e, gpu_launches=launches, clocks=clocks,
    )
    print(json.dumps(line))
    return 0


def cpu_baseline() -> int:
    """Tokens per second of the plain implementation (tests/plain_qwen3.py: float32, whole sequences, no cache)
    on this machine's CPU, on the tiny configurations A and B: a prompt step over prompts of 5, 9, 13 (A) and 1, 7, 16, 31 (B) tokens and
    greedy decoding that recomputes the whole sequence for every token.  It is the oracle of the tests, timed
    for orientation; the reference's own CPU path cannot be built here."""
    import tempfile

    sys.path.insert(0, str(ROOT))
    sys.path.insert(0, str(ROOT / "tests"))
    import plain_qwen3 as plain
    from tiny_configs import make_folder, prompts

    out = {}
    with tempfile.TemporaryDirectory() as tmp:
        for name, lengths, n_new in (("A", [5, 9, 13], 8), ("B", [1, 7, 16, 31], 12)):
            cfg, w = plain.read_model(make_folder(tmp, name, "float32"))
            ps = prompts(cfg["vocab_size"], lengths, seed=1)
            t0 = time.perf_counter()
            for p in ps:
                plain.forward(cfg, w, p)
            t_prefill = time.perf_counter() - t0
            t0 = time.perf_counter()
            for p in ps:
                plain.greedy_generate(cfg, w, p, n_new)
            t_decode = time.perf_counter() - t0 - t_prefill
            out[f"tiny_{name}"] = dict(prefill_tokens_per_s=sum(lengths) / t_prefill,
                                       decode_tokens_per_s=len(ps) * n_new / max(t_decode, 1e-9))
    print(json.dumps(dict(impl="plain implementation on the CPU (tests/plain_qwen3.py)", unit="tokens/s", **out)))
    return 0


if __name__ == "__main__":
    sys.exit(main())
