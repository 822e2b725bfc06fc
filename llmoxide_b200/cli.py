"""Command line in the manner of the reference's tool
(llmoxide/src/main.rs:6,19-88):

    llmoxide <model-folder> <prompt> [n] [options]

Greedy by default and template-free: "do the kernels still produce the right
numbers".  There is no tokenizer in this library, so ``<prompt>`` is a list
of token ids ("5,17,3"); several prompts separated by ";" run as one batch.
``n`` is the number of tokens to generate (default 16, main.rs:28).  Like the
reference it reports prefill and decode tokens per second and prints the
generated ids (main.rs:52-57,79-85).  The context is sized as the reference
sizes it: the next power of two above prompt + n + 8, at least 2048
(main.rs:35), or ``LLMOXIDE_CTX`` / ``--ctx`` when given.
"""

from __future__ import annotations

import argparse
import os
import sys
import time


def parse_prompts(text: str) -> list:
    prompts = []
    for part in text.split(";"):
        ids = [int(x) for x in part.replace(",", " ").split()]
        if ids:
            prompts.append(ids)
    if not prompts:
        raise SystemExit("the prompt holds no token ids (expected e.g. \"5,17,3\" or \"5 17 3; 8 9\")")
    return prompts


def next_power_of_two(n: int) -> int:
    return 1 << max(0, (n - 1).bit_length())


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="llmoxide", description=__doc__.split("\n\n")[0],
                                 usage="llmoxide <model-folder> <prompt-ids> [n] [options]")
    ap.add_argument("model", help="folder with config.json and model.safetensors (or a config.json with --random)")
    ap.add_argument("prompt", help='token ids, e.g. "5,17,3"; ";" separates the prompts of a batch')
    ap.add_argument("n", nargs="?", type=int, default=16, help="tokens to generate (default 16)")
    ap.add_argument("--cpu", action="store_true", help="the reference's CPU switch; this library has no CPU path")
    ap.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16")
    ap.add_argument("--random", action="store_true", help="random weights for the configuration at <model>")
    ap.add_argument("--seed", type=int, default=0, help="seed of the sampler (and of --random weights)")
    ap.add_argument("--temperature", type=float, default=0.0, help="<= 0 is greedy (the default)")
    ap.add_argument("--top-k", type=int, default=None)
    ap.add_argument("--top-p", type=float, default=None)
    ap.add_argument("--repeat-penalty", type=float, default=1.0)
    ap.add_argument("--ctx", type=int, default=int(os.environ.get("LLMOXIDE_CTX", 0)),
                    help="positions per sequence (default: as the reference sizes it)")
    ap.add_argument("--ignore-stop", action="store_true", help="do not end at the model's stop tokens")
    args = ap.parse_args(argv)
    if args.cpu:
        print("llmoxide: --cpu: this library has no CPU path; it runs on a CUDA device or not at all",
              file=sys.stderr)
        return 2

    from . import LoadOptions, Request, Sampling, Session

    prompts = parse_prompts(args.prompt)
    longest = max(len(p) for p in prompts)
    n_ctx = args.ctx or max(2048, next_power_of_two(longest + args.n + 8))
    opts = LoadOptions(dtype=args.dtype, max_tokens=n_ctx * len(prompts), max_batch=len(prompts),
                       max_step_tokens=max(sum(len(p) for p in prompts), 1))
    t0 = time.perf_counter()
    if args.random:
        session = Session.random(args.model, args.seed, opts)
    else:
        session = Session.load(args.model, opts)
    info = session.info()
    print(f"{info['architecture']} on {info['device']} ({info['dtype']})", file=sys.stderr)
    print(f"loaded in {time.perf_counter() - t0:.2f}s; prompt {sum(len(p) for p in prompts)} tokens "
          f"in {len(prompts)} sequence(s)", file=sys.stderr)

    base = session.default_sampling
    sampling = Sampling(temperature=args.temperature,
                        top_k=base.top_k if args.top_k is None else args.top_k,
                        top_p=base.top_p if args.top_p is None else args.top_p,
                        repeat_penalty=args.repeat_penalty, seed=args.seed)
    if args.ignore_stop:
        session.loop.stop_ids = frozenset()
    requests = [Request(prompt=p, max_tokens=args.n, sampling=sampling.with_(seed=args.seed + i))
                for i, p in enumerate(prompts)]
    outcomes = session.generate(requests)
    t = session.timings
    print(f"prefill {t.prefill_seconds * 1e3:.1f} ms ({t.prefill_tokens / max(t.prefill_seconds, 1e-9):.1f} tok/s)",
          file=sys.stderr)
    generated = sum(o.generated for o in outcomes)
    print(f"generated {generated} tokens in {t.decode_seconds * 1e3:.1f} ms "
          f"({t.decode_tokens / max(t.decode_seconds, 1e-9):.2f} tok/s)", file=sys.stderr)
    for o in outcomes:
        print(f"ids: {o.tokens}  ({o.reason})")
    return 0


if __name__ == "__main__":
    sys.exit(main())
