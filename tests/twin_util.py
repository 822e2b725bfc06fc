"""Builds and runs the C++ twin of the plain implementation (tests/twin/qwen3_twin.cpp)."""

import shutil
import subprocess
import tempfile
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
_exe = None


def twin_exe() -> Path:
    """The compiled twin (g++, no fused multiply-add, no fast-math), built once per process."""
    global _exe
    if _exe is None:
        gxx = shutil.which("g++") or shutil.which("c++")
        if gxx is None:
            raise RuntimeError("no C++ compiler for the twin")
        out = Path(tempfile.mkdtemp(prefix="qwen3_twin_")) / "qwen3_twin"
        subprocess.run([gxx, "-O2", "-std=c++17", "-ffp-contract=off", "-o", str(out),
                        str(HERE / "twin" / "qwen3_twin.cpp")], check=True)
        _exe = out
    return _exe


def twin_logits(folder, tokens, prefix_len, vocab) -> np.ndarray:
    """[T, vocab] logits: the first ``prefix_len`` tokens in one step, the others one by one."""
    with tempfile.TemporaryDirectory() as tmp:
        out = Path(tmp) / "logits.f32"
        subprocess.run([str(twin_exe()), str(folder), str(out), str(prefix_len), *map(str, tokens)], check=True)
        return np.fromfile(out, dtype="<f4").reshape(len(tokens), vocab)
