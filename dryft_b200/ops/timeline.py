"""Block timeline of the decode kernels (a development aid).

With ``DRYFT_B200_TRACE=1`` in the environment (set before the first kernel library is built or loaded)
the decode kernels that carry timeline points (``csrc/gemm_decode.cu``, ``csrc/attn_decode.cu``,
``csrc/gemm_stream.cu``) are compiled with them: thread 0 of every block notes the device-wide
nanosecond clock when it starts, when its wait for the launch before it returns, when its prologue is
done and when it ends.  ``collect()`` reads the rings of all loaded libraries; ``launch_table()`` groups
the blocks into launches and prints, for each, the first and the last block's time at every point.  It is
how the overlap of consecutive launches (programmatic dependent launch) was measured.
hari495/dryft has nothing of the kind; it profiles with torch.profiler (``agent/profile.py``).
"""

from __future__ import annotations

import ctypes
import os
from typing import List

import numpy as np

from . import kernels as K

RECORD = np.dtype([("t", np.uint64, 4), ("tag", np.uint32), ("block", np.uint32), ("sm", np.uint32), ("n_blocks", np.uint32)])
CAPACITY = 1 << 17   # DRYFT_TRACE_CAP of csrc/common.cuh
EXPORTS = ("dryft_gemm_decode_trace", "dryft_attn_decode_trace", "dryft_gemm_stream_trace")


def enabled() -> bool:
    return os.environ.get("DRYFT_B200_TRACE") == "1"


def collect() -> np.ndarray:
    """All records held by the loaded kernel libraries (each keeps its last ``CAPACITY`` blocks)."""
    if not enabled():
        raise RuntimeError("set DRYFT_B200_TRACE=1 before the kernels are built and loaded")
    libs = list(K._variants.values()) + [lib for lib in (K._gemm_stream,) if lib is not None]
    out: List[np.ndarray] = []
    for lib in libs:
        for name in EXPORTS:
            fn = getattr(lib, name, None) if hasattr(lib, name) else None
            if fn is None:
                continue
            fn.argtypes = [ctypes.c_void_p, ctypes.c_void_p]
            fn.restype = ctypes.c_int
            buf = np.zeros(CAPACITY, dtype=RECORD)
            count = ctypes.c_uint(0)
            rc = fn(buf.ctypes.data, ctypes.addressof(count))
            if rc != 0:
                raise RuntimeError(f"{name} failed with {rc}")
            out.append(buf[: min(count.value, CAPACITY)] if count.value <= CAPACITY else buf)
    recs = np.concatenate(out) if out else np.zeros(0, dtype=RECORD)
    return recs[recs["t"][:, 3] > 0]


def tag_name(tag: int) -> str:
    if tag == 1:
        return "attn_decode"
    k, mode, norm = tag // 16, (tag % 16) // 2, tag % 2
    return f"gemm K={k} {['store', 'store32', 'residual', 'silu'][mode]}{'+norm' if norm else ''}"


def launch_table(recs: np.ndarray, last_us: float, max_launches: int = 12) -> str:
    """The launches whose blocks ended within the last ``last_us`` microseconds of the records."""
    t = recs["t"].astype(np.int64)
    keep = t[:, 3] > t[:, 3].max() - int(last_us * 1000)
    recs, t = recs[keep], t[keep]
    order = np.argsort(t[:, 1], kind="stable")
    recs, t = recs[order], t[order]
    launches, cur = [], None
    for i in range(len(recs)):
        tag = int(recs["tag"][i])
        if cur is None or cur["tag"] != tag or t[i, 1] - cur["hi"] > 20000:
            cur = {"tag": tag, "rows": [], "hi": t[i, 1]}
            launches.append(cur)
        cur["rows"].append(i)
        cur["hi"] = max(cur["hi"], t[i, 1])
    launches = launches[-max_launches:]
    if not launches:
        return "(no records)"
    base = min(t[np.array(L["rows"]), 0].min() for L in launches)
    lines = ["| launch | blocks | start first..last | wait over first..last | prologue done first..last | end first..last |",
             "|---|---:|---:|---:|---:|---:|"]
    for L in launches:
        tt = (t[np.array(L["rows"])] - base) / 1000.0
        cells = []
        for c in range(4):
            col = tt[:, c][tt[:, c] > -1e6]
            cells.append(f"{col.min():.1f}..{col.max():.1f}" if len(col) else "-")
        lines.append(f"| {tag_name(L['tag'])} | {len(L['rows'])} | " + " | ".join(cells) + " |")
    return "\n".join(lines)
