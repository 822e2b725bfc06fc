"""Builds and loads the CUDA libraries of this package.

Every ``.cu`` file here becomes one shared library with ``extern "C"``
launchers, compiled by nvcc for sm_100a only and loaded through ctypes.  A
library is built the first time something needs it, so a model compiles just
the kernels it uses; the file name carries a hash of the sources and flags,
so an edited source is rebuilt and a built library is found again.  Libraries
go to ``_build/`` beside the sources when that folder can be written, else to
a per-user folder under the system's temporary directory.  While nvcc runs, a
line is printed to stderr every few seconds.

There is no fallback: without nvcc or without a GPU the engine stops with
``ExtensionMissing``.
"""

from __future__ import annotations

import ctypes
import fcntl
import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import threading
import time
from pathlib import Path

from ..errors import ExtensionMissing

SRC_DIR = Path(__file__).resolve().parent
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC,-fvisibility=hidden", "-shared"]
# library name -> (source files, extra link flags)
LIBRARIES = {
    "elementwise": (["elementwise.cu"], []),
    "attention": (["attention.cu"], []),
    "attention_decode": (["attention_decode.cu"], []),
    "attention_prefill": (["attention_prefill.cu"], []),
    "attention_prefill_tc": (["attention_prefill_tc.cu"], []),
    "gemm_fma": (["gemm_fma.cu"], []),
    "gemm_tc": (["gemm_tc.cu"], []),
    "sampling": (["sampling.cu"], []),
    "random_init": (["random_init.cu"], []),
    # host code only (no CUDA): the cache's bookkeeping and the step plan
    "host_runtime": (["host_runtime.cpp"], []),
}
HEADERS = ["common.cuh", "attention_decode_noalloc.h", "tc_ptx.cuh"]

_loaded: dict = {}
_lock = threading.Lock()


def _say(msg: str) -> None:
    print(f"[llmoxide_b200] {msg}", file=sys.stderr, flush=True)


def find_nvcc() -> str:
    for root in (os.environ.get("CUDA_HOME"), os.environ.get("CUDA_PATH"), "/usr/local/cuda"):
        if root and (Path(root) / "bin" / "nvcc").is_file():
            return str(Path(root) / "bin" / "nvcc")
    found = shutil.which("nvcc")
    if found:
        return found
    raise ExtensionMissing("nvcc was not found (CUDA_HOME, /usr/local/cuda/bin, PATH): the CUDA kernels of "
                           "llmoxide_b200 cannot be built, and there is no other path")


def _host_only(name: str) -> bool:
    return all(src.endswith(".cpp") for src in LIBRARIES[name][0])


def find_cxx() -> str:
    """The C++ compiler for the host-only library."""
    for cand in (os.environ.get("CXX"), "g++", "c++", "clang++"):
        found = shutil.which(cand) if cand else None
        if found:
            return found
    raise ExtensionMissing("no C++ compiler was found (CXX, g++, c++): the host runtime of llmoxide_b200 "
                           "cannot be built, and there is no other path")


def _flags() -> list:
    # LLMX_NVCC_EXTRA: extra nvcc flags (for experiments with -D switches); part of the library's hash
    return list(NVCC_FLAGS) + os.environ.get("LLMX_NVCC_EXTRA", "").split()


def _digest(name: str) -> str:
    sources, extra = LIBRARIES[name]
    h = hashlib.sha256()
    for f in sorted(set(sources) | (set() if _host_only(name) else set(HEADERS))):
        h.update(f.encode())
        h.update((SRC_DIR / f).read_bytes())
    h.update(" ".join(ARCH_FLAGS + _flags() + extra).encode())
    return h.hexdigest()[:16]


def _writable(d: Path) -> bool:
    try:
        d.mkdir(parents=True, exist_ok=True)
        probe = d / f".probe-{os.getpid()}"
        probe.write_bytes(b"")
        probe.unlink()
        return True
    except OSError:
        return False


def build_dirs() -> list:
    """Where a built library is looked for, in order; the first writable one
    receives new builds."""
    dirs = []
    if os.environ.get("LLMOXIDE_B200_BUILD_DIR"):
        dirs.append(Path(os.environ["LLMOXIDE_B200_BUILD_DIR"]))
    dirs.append(SRC_DIR / "_build")
    dirs.append(Path(tempfile.gettempdir()) / f"llmoxide_b200-{os.getuid()}")
    return dirs


def library_path(name: str, must_exist=True):
    fname = f"libllmx_{name}-{_digest(name)}.so"
    for d in build_dirs():
        if (d / fname).is_file():
            return d / fname
    if must_exist:
        return None
    for d in build_dirs():
        if _writable(d):
            return d / fname
    raise ExtensionMissing("no writable folder for the built CUDA libraries: tried "
                           + ", ".join(str(d) for d in build_dirs()))


def compile_library(name: str, verbose=True) -> Path:
    """Compiles one library if it is not there yet; returns its path."""
    have = library_path(name)
    if have is not None:
        return have
    target = library_path(name, must_exist=False)
    nvcc = find_cxx() if _host_only(name) else find_nvcc()
    sources, extra = LIBRARIES[name]
    lock_path = target.with_suffix(".lock")
    with open(lock_path, "w") as lock_file:
        fcntl.flock(lock_file, fcntl.LOCK_EX)
        try:
            if target.is_file():  # another process built it meanwhile
                return target
            tmp = target.with_name(f".{target.name}.{os.getpid()}.tmp")
            if _host_only(name):
                cmd = [nvcc, "-O2", "-std=c++17", "-shared", "-fPIC", "-fvisibility=hidden", *extra,
                       *[str(SRC_DIR / s) for s in sources], "-o", str(tmp)]
            else:
                cmd = [nvcc, *ARCH_FLAGS, *_flags(), *extra, "-I", str(SRC_DIR),
                       *[str(SRC_DIR / s) for s in sources], "-o", str(tmp)]
            if verbose:
                _say(f"compiling {name} ({', '.join(sources)})" + ("" if _host_only(name) else " for sm_100a") + " ...")
            t0 = time.time()
            proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
            done = threading.Event()

            def ticker():
                while not done.wait(10.0):
                    _say(f"  still compiling {name} ({time.time() - t0:.0f} s)")

            th = threading.Thread(target=ticker, daemon=True)
            if verbose:
                th.start()
            out, _ = proc.communicate()
            done.set()
            if proc.returncode != 0:
                tmp.unlink(missing_ok=True)
                raise ExtensionMissing(f"nvcc failed on {name}:\n{' '.join(cmd)}\n{out}")
            os.replace(tmp, target)
            for old in target.parent.glob(f"libllmx_{name}-*.so"):   # earlier versions of this library
                if old != target:
                    old.unlink(missing_ok=True)
            if verbose:
                _say(f"built {target.name} in {time.time() - t0:.1f} s")
            return target
        finally:
            fcntl.flock(lock_file, fcntl.LOCK_UN)
            try:
                lock_path.unlink()
            except OSError:
                pass


def load_library(name: str) -> ctypes.CDLL:
    """The loaded library, built first if needed."""
    with _lock:
        lib = _loaded.get(name)
        if lib is None:
            if name not in LIBRARIES:
                raise ExtensionMissing(f"no CUDA library named {name!r}")
            path = compile_library(name)
            try:
                lib = ctypes.CDLL(str(path))
            except OSError as e:
                raise ExtensionMissing(f"could not load {path}: {e}") from None
            _loaded[name] = lib
        return lib


def build_all(verbose=True) -> list:
    """Compiles every library (the build check; needs nvcc but no GPU)."""
    return [compile_library(name, verbose) for name in LIBRARIES]
