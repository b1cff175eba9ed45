"""Compiles the CUDA sources of ``csrc/`` for sm_100a into shared libraries, at first use.

The libraries export plain C functions (raw pointers and a stream), so they need no Python
or torch headers and a file compiles in seconds.  Each library is built into
``csrc/_build/<name>-<hash of sources and flags>/`` inside the package when that is
writable, else into a per-user folder under the system's temporary directory; nothing is
written under the home directory.  While compiling, a line goes to stderr every few seconds.
"""

from __future__ import annotations

import concurrent.futures
import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import threading
import time
from typing import Dict, List, Sequence

CSRC = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "csrc")

NVCC_FLAGS = [
    "-O3", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden", "--expt-relaxed-constexpr",
]

# library name -> sources.  "core" holds every kernel of the 32-bit path and the generic
# bfloat16 ones; "bf16" holds the tensor-core kernels that only the serving path loads, so a
# 32-bit run compiles (at its first call) only what it needs.
LIBRARIES: Dict[str, List[str]] = {
    "core": ["elementwise.cu", "rope_cache.cu", "attention_generic.cu", "gemm_f32.cu", "sampling.cu"],
    "bf16": ["attention_mma.cu", "attention_tcgen05.cu", "gemm_chain.cu", "gemm_tcgen05.cu"],
}


class BuildError(RuntimeError):
    pass


def find_nvcc() -> str:
    for cand in (os.environ.get("Q25VL_NVCC"),
                 os.path.join(os.environ.get("CUDA_HOME", ""), "bin", "nvcc") if os.environ.get("CUDA_HOME") else None,
                 shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.isfile(cand) and os.access(cand, os.X_OK):
            return cand
    raise BuildError("nvcc not found: set CUDA_HOME or put nvcc on PATH; the CUDA kernels cannot be built")


def _source_hash(sources: Sequence[str]) -> str:
    h = hashlib.sha256()
    h.update(" ".join(NVCC_FLAGS).encode())
    headers = sorted(f for f in os.listdir(CSRC) if f.endswith((".cuh", ".h")))
    for name in list(sources) + headers:
        h.update(name.encode())
        with open(os.path.join(CSRC, name), "rb") as fh:
            h.update(fh.read())
    return h.hexdigest()[:16]


def _build_root() -> str:
    in_tree = os.path.join(CSRC, "_build")
    try:
        os.makedirs(in_tree, exist_ok=True)
        probe = os.path.join(in_tree, f".w{os.getpid()}")
        with open(probe, "w"):
            pass
        os.remove(probe)
        return in_tree
    except OSError:
        root = os.path.join(tempfile.gettempdir(), f"qwen25vl_lite_b200-build-{os.getuid()}")
        os.makedirs(root, exist_ok=True)
        return root


def library_path(name: str) -> str:
    sources = LIBRARIES[name]
    return os.path.join(_build_root(), f"{name}-{_source_hash(sources)}", f"libq25vl_{name}.so")


def build_library(name: str, verbose: bool = True) -> str:
    """Returns the path of the built library, compiling it if it is not there yet."""
    if name not in LIBRARIES:
        raise BuildError(f"unknown kernel library {name!r}; known: {sorted(LIBRARIES)}")
    target = library_path(name)
    if os.path.isfile(target):
        return target
    nvcc = find_nvcc()
    sources = LIBRARIES[name]
    out_dir = os.path.dirname(target)
    os.makedirs(out_dir, exist_ok=True)
    t0 = time.time()
    done = [0]
    stop = threading.Event()

    def progress():
        while not stop.wait(8.0):
            print(f"[qwen25vl-lite] compiling CUDA kernels '{name}' for sm_100a: {done[0]}/{len(sources)} files, "
                  f"{time.time() - t0:.0f}s", file=sys.stderr, flush=True)

    if verbose:
        print(f"[qwen25vl-lite] compiling CUDA kernels '{name}' for sm_100a ({len(sources)} files), first use only",
              file=sys.stderr, flush=True)
        threading.Thread(target=progress, daemon=True).start()

    def compile_one(src: str) -> str:
        obj = os.path.join(out_dir, os.path.splitext(src)[0] + ".o")
        cmd = [nvcc, *NVCC_FLAGS, "-I", CSRC, "-c", os.path.join(CSRC, src), "-o", obj]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise BuildError(f"nvcc failed on {src}:\n{' '.join(cmd)}\n{res.stdout}\n{res.stderr}")
        done[0] += 1
        return obj

    try:
        with concurrent.futures.ThreadPoolExecutor(max_workers=min(len(sources), os.cpu_count() or 4)) as pool:
            objects = list(pool.map(compile_one, sources))
        tmp = target + f".tmp{os.getpid()}"
        cmd = [nvcc, "-shared", "-o", tmp, *objects]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise BuildError(f"linking {name} failed:\n{res.stdout}\n{res.stderr}")
        os.replace(tmp, target)
        for old in os.listdir(os.path.dirname(out_dir)):      # builds of earlier sources are of no use
            if old.startswith(name + "-") and old != os.path.basename(out_dir):
                shutil.rmtree(os.path.join(os.path.dirname(out_dir), old), ignore_errors=True)
    finally:
        stop.set()
    if verbose:
        print(f"[qwen25vl-lite] built {os.path.basename(target)} in {time.time() - t0:.0f}s", file=sys.stderr, flush=True)
    return target


def build_all(verbose: bool = True) -> List[str]:
    return [build_library(name, verbose) for name in LIBRARIES]
