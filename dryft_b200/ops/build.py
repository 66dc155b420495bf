"""Compile the CUDA sources under ``dryft_b200/csrc`` for sm_100a into shared libraries, on demand.

A library is named by its sources, its ``-D`` sizes and a hash of everything that goes into it, so
a stale binary is never loaded and a model only compiles the variants its own sizes need.  The
first call compiles (seconds per file; a progress line is printed now and then), later calls find
the file.  Binaries are kept in ``dryft_b200/csrc/_build`` when that is writable (so they travel
with the tree), else under ``$DRYFT_B200_BUILD_DIR`` or a per-user temporary folder.

hari495/dryft has no native code to build (its GPU code is Triton, compiled at first launch,
``engine/dryft_qwen3/model.py:104-119``); this file is that "compile what this model needs at first
use" step for hand-written CUDA.
"""

from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import time
from typing import Dict, Iterable, Optional, Sequence

CSRC = os.path.normpath(os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", "csrc"))
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "-shared", "--threads", "2"]


class BuildError(RuntimeError):
    pass


def log(msg: str) -> None:
    print(f"[dryft_b200] {msg}", file=sys.stderr, flush=True)


def find_nvcc() -> str:
    cand = [os.environ.get("DRYFT_B200_NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"]
    for c in cand:
        if c and os.path.isfile(c) and os.access(c, os.X_OK):
            return c
    raise BuildError("nvcc not found (looked at $DRYFT_B200_NVCC, PATH and /usr/local/cuda/bin/nvcc); "
                     "the CUDA kernels of dryft_b200 cannot be built and there is no fallback")


def _writable_dir(path: str) -> bool:
    try:
        os.makedirs(path, exist_ok=True)
        probe = os.path.join(path, f".probe_{os.getpid()}")
        with open(probe, "w"):
            pass
        os.remove(probe)
        return True
    except OSError:
        return False


_build_dir_cache: Optional[str] = None


def build_dir() -> str:
    global _build_dir_cache
    if _build_dir_cache is not None:
        return _build_dir_cache
    cands = []
    if os.environ.get("DRYFT_B200_BUILD_DIR"):
        cands.append(os.environ["DRYFT_B200_BUILD_DIR"])
    cands.append(os.path.join(CSRC, "_build"))
    cands.append(os.path.join(tempfile.gettempdir(), f"dryft_b200_build_{os.getuid()}"))
    for c in cands:
        if _writable_dir(c):
            _build_dir_cache = c
            return c
    raise BuildError("no writable folder for compiled kernels; tried: " + ", ".join(cands))


def _digest(sources: Sequence[str], defines: Dict[str, int]) -> str:
    h = hashlib.sha256()
    headers = sorted(f for f in os.listdir(CSRC) if f.endswith((".cuh", ".h")))
    for name in list(sources) + headers:
        with open(os.path.join(CSRC, name), "rb") as f:
            h.update(name.encode())
            h.update(f.read())
    h.update(repr(sorted(defines.items())).encode())
    h.update(" ".join(ARCH_FLAGS + NVCC_FLAGS).encode())
    return h.hexdigest()[:12]


def library_path(name: str, sources: Sequence[str], defines: Optional[Dict[str, int]] = None) -> str:
    defines = defines or {}
    tag = "".join(f"_{k.lower().replace('dryft_', '')}{v}" for k, v in sorted(defines.items()))
    return os.path.join(build_dir(), f"libdryft_{name}{tag}_{_digest(sources, defines)}.so")


def build_library(name: str, sources: Sequence[str], defines: Optional[Dict[str, int]] = None,
                  extra_flags: Iterable[str] = ()) -> str:
    """Path of the shared library, compiling it first if it is not there yet."""
    defines = dict(defines or {})
    out = library_path(name, sources, defines)
    if os.path.isfile(out):
        return out
    nvcc = find_nvcc()
    tmp = f"{out}.tmp{os.getpid()}"
    cmd = [nvcc, *ARCH_FLAGS, *NVCC_FLAGS, *extra_flags, "-I", CSRC]
    cmd += [f"-D{k}={v}" for k, v in sorted(defines.items())]
    cmd += [os.path.join(CSRC, s) for s in sources] + ["-o", tmp]
    what = name + ("" if not defines else " (" + ", ".join(f"{k}={v}" for k, v in sorted(defines.items())) + ")")
    log(f"compiling {what} for sm_100a ...")
    t0 = time.time()
    proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    while True:
        try:
            output, _ = proc.communicate(timeout=10)
            break
        except subprocess.TimeoutExpired:
            log(f"  still compiling {name} ({time.time() - t0:.0f}s)")
    if proc.returncode != 0:
        try:
            os.remove(tmp)
        except OSError:
            pass
        raise BuildError(f"nvcc failed for {what}:\n{' '.join(cmd)}\n{output}")
    os.replace(tmp, out)  # atomic: a concurrent builder of the same library wins or loses whole
    log(f"  built {os.path.basename(out)} in {time.time() - t0:.1f}s")
    return out
