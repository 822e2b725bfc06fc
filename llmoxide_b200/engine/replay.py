"""Trace replay: feeds given token ids through the engine step by step and
writes logits.  It samples nothing and owns no model code: it drives the same
``Engine.step``, cache and kernels that generation uses.  The reference has
tools of the same purpose that take explicit token ids and compare logits
(crates/model/src/bin/validate_qwen35.rs:39-48,
crates/gpu/src/bin/bisect_qwen35.rs:16-21,112-130).

Input, one JSON object a line:
    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}
For a step in which something is wanted, ``<out>/<step>.f32`` holds the logits
at the wanted places, in the order of the entries and of ``want``, as
little-endian float32 [wanted, vocab].  After every step ``done <step>`` is
printed and flushed.
"""

from __future__ import annotations

import json
import sys
from pathlib import Path

import numpy as np

from .engine import Engine, LoadOptions


class Replayer:
    def __init__(self, engine: Engine, out_dir, dump: bool = False):
        """With ``dump`` every step also writes its named intermediates, ``<step>.<name>.f32`` as float32
        [tokens of the step, width], for finding the first stage at which two runs part."""
        self.dump = dump
        self.engine, self.out = engine, Path(out_dir)
        self.out.mkdir(parents=True, exist_ok=True)
        self.slots: dict = {}

    def run_step(self, rec: dict) -> None:
        step = rec["step"]
        entries, want = [], []
        for e in rec.get("entries", []):
            rid = e["id"]
            if rid not in self.slots:
                self.slots[rid] = self.engine.acquire()
            entries.append((self.slots[rid], list(e["tokens"])))
            want.append(list(e.get("want", [])))
        if entries:
            probe = None
            if self.dump:
                def probe(name, t, step=step):
                    t.detach().float().cpu().numpy().astype("<f4").tofile(self.out / f"{step}.{name}.f32")
            logits = self.engine.step(entries, want, probe=probe)
            if logits.shape[0] > 0:
                arr = logits.detach().cpu().numpy().astype("<f4", copy=False)
                self.engine.check_status()        # the copy waited for the step: its kernels' reports are in
                tmp = self.out / f".{step}.f32.tmp"
                arr.tofile(tmp)
                tmp.replace(self.out / f"{step}.f32")
        for rid in rec.get("end", []):
            slot = self.slots.pop(rid, None)
            if slot is not None:
                self.engine.release(slot)


def main(argv=None) -> int:
    import argparse

    ap = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    ap.add_argument("--out", required=True, help="folder that receives <step>.f32")
    ap.add_argument("--max-tokens", type=int, required=True,
                    help="most tokens live requests hold at any time, each rounded up to a multiple of 64")
    ap.add_argument("--dump", action="store_true",
                    help="also write every step's named intermediates as <step>.<name>.f32")
    args = ap.parse_args(argv)
    opts = LoadOptions(dtype=args.dtype, max_tokens=args.max_tokens,
                       max_batch=max(1, (args.max_tokens + 63) // 64),
                       max_step_tokens=max(args.max_tokens, 64))
    engine = Engine.load(args.model, opts)
    rp = Replayer(engine, args.out, dump=args.dump)
    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        rec = json.loads(line)
        rp.run_step(rec)
        print(f"done {rec['step']}", flush=True)
    return 0
