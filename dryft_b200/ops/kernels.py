"""Python face of the CUDA kernels: loads the compiled libraries with ``ctypes`` and wraps every
launcher in a function that checks devices, dtypes, shapes and contiguity before the launch.

There is no CPU path and no PyTorch stand-in behind these functions: if the library cannot be
built or loaded, or a tensor is not on a CUDA device, they raise.  (The reference degrades to a
PyTorch path when a Triton kernel fails its self-test, ``engine/dryft_qwen3/model.py:104-119``;
this library fails loudly instead.)

All launches go to PyTorch's current CUDA stream, so they order with PyTorch work and are
captured by ``torch.cuda.graph``.
"""

from __future__ import annotations

import ctypes
import threading
from typing import Dict, Optional, Tuple

import torch

from . import build

_i, _f, _p, _ll, _ull = ctypes.c_int, ctypes.c_float, ctypes.c_void_p, ctypes.c_longlong, ctypes.c_ulonglong

CORE_SOURCES = ("elementwise.cu", "rope_kv.cu", "gemm_f32.cu", "sample.cu", "gemm_small_m.cu")
UNSUPPORTED = -2


class KernelError(RuntimeError):
    """A launcher refused its arguments or CUDA reported an error at launch."""


_lock = threading.Lock()
_core: Optional[ctypes.CDLL] = None
_variants: Dict[Tuple, ctypes.CDLL] = {}


def _load(path: str) -> ctypes.CDLL:
    try:
        return ctypes.CDLL(path)
    except OSError as e:  # pragma: no cover - depends on the machine
        raise KernelError(f"cannot load compiled kernels {path}: {e}") from e


def core() -> ctypes.CDLL:
    """The size-independent kernels (metadata, embedding, norms, SiLU*mul, RoPE + cache write,
    32-bit matrix product, small-batch bf16 matrix product, token choice)."""
    global _core
    with _lock:
        if _core is None:
            lib = _load(build.build_library("core", CORE_SOURCES))
            lib.dryft_step_meta.argtypes = [_p, _p, _p, _i, _i, _p, _p, _p]
            lib.dryft_step_advance.argtypes = [_p, _p, _p, _i, _p]
            lib.dryft_tokens_from_state.argtypes = [_p, _p, _p, _i, _p]
            lib.dryft_embed.argtypes = [_i, _p, _p, _p, _i, _i, _i, _p, _p]
            lib.dryft_rmsnorm.argtypes = [_i, _p, _p, _p, _p, _p, _p, _i, _i, _f, _p]
            lib.dryft_residual_add.argtypes = [_i, _p, _p, _ll, _p]
            lib.dryft_silu_mul.argtypes = [_i, _p, _p, _i, _i, _p]
            lib.dryft_qk_norm_rope_store.argtypes = [_i, _p, _i, _p, _p, _p, _p, _p, _p, _p, _p, _p, _p, _i, _i, _i, _i, _i,
                                                     _i, _i, _f, _i, _i, _i, _p]
            lib.dryft_rope_table.argtypes = [_i, _p, _p, _p, _i, _i, _p]
            lib.dryft_gemm_nt_f32.argtypes = [_p, _i, _p, _p, _i, _i, _i, _i, _p]
            lib.dryft_argmax_rows.argtypes = [_p, _i, _i, _ll, _p, _p, _p, _p]
            lib.dryft_sample_rows.argtypes = [_p, _i, _i, _ll, _f, _i, _ull, _p, _p, _i, _p, _p, _p, _p]
            lib.dryft_gemm_small_m.argtypes = [_p, _i, _p, _p, _i, _i, _i, _i, _i, _p, _p, _i, _f, _p, _i, _p]
            lib.dryft_row_sumsq.argtypes = [_p, _i, _i, _p, _p, _p, _p]
            for name in ("dryft_step_meta", "dryft_step_advance", "dryft_tokens_from_state", "dryft_embed",
                         "dryft_rmsnorm", "dryft_residual_add", "dryft_silu_mul", "dryft_qk_norm_rope_store", "dryft_rope_table",
                         "dryft_gemm_nt_f32", "dryft_argmax_rows", "dryft_sample_rows", "dryft_gemm_small_m", "dryft_row_sumsq"):
                getattr(lib, name).restype = _i
            _core = lib
        return _core


def attention_rows_lib(head_dim: int, group: int, page: int) -> ctypes.CDLL:
    """The row-wise (decode / 32-bit) attention kernel compiled for these sizes."""
    if head_dim <= 0 or head_dim % 16:
        raise KernelError(f"attention kernels take head sizes in steps of 16, got head_dim={head_dim}")
    if head_dim > 256:
        raise KernelError(f"attention kernels take head sizes up to 256, got head_dim={head_dim}")
    if group < 1 or group > 16:
        raise KernelError(f"attention kernels take 1..16 query heads per kv head, got {group}")
    key = ("rows", head_dim, group, page)
    with _lock:
        lib = _variants.get(key)
        if lib is None:
            path = build.build_library("attn_rows", ("attn_rows.cu",),
                                       {"DRYFT_HEAD_DIM": head_dim, "DRYFT_GROUP": group, "DRYFT_PAGE": page})
            lib = _load(path)
            lib.dryft_attn_rows.argtypes = [_i, _p, _p, _p, _p, _i, _p, _p, _p, _p, _p, _i, _i, _i, _f, _i, _p]
            lib.dryft_attn_rows.restype = _i
            if (lib.dryft_attn_rows_head_dim(), lib.dryft_attn_rows_group(), lib.dryft_attn_rows_page()) != (head_dim, group, page):
                raise KernelError(f"{path} was compiled for other sizes")
            _variants[key] = lib
        return lib


def gemm_decode_lib(k: int) -> ctypes.CDLL:
    """The decode matrix product compiled for one inner size ``k`` (a multiple of 256)."""
    if k <= 0 or k % 256:
        raise KernelError(f"the specialised decode product takes inner sizes that are multiples of 256, got {k}")
    key = ("gemm_decode", k)
    with _lock:
        lib = _variants.get(key)
        if lib is None:
            lib = _load(build.build_library("gemm_decode", ("gemm_decode.cu",), {"DRYFT_K": k}))
            lib.dryft_gemm_decode.argtypes = [_p, _i, _p, _p, _i, _i, _i, _i, _p, _p, _i, _f, _p, _i, _i, _p, _p, _p]
            lib.dryft_gemm_decode.restype = _i
            if lib.dryft_gemm_decode_k() != k:
                raise KernelError("the compiled decode product is for another inner size")
            _variants[key] = lib
        return lib


_gemm_stream: Optional[ctypes.CDLL] = None


def gemm_stream_lib() -> ctypes.CDLL:
    """The weight-streaming decode product for up to 64 rows on tcgen05 / TMEM / TMA, work cut evenly over the SMs."""
    global _gemm_stream
    with _lock:
        if _gemm_stream is None:
            lib = _load(build.build_library("gemm_stream", ("gemm_stream.cu",)))
            lib.dryft_gemm_stream.argtypes = [_p, _i, _p, _p, _i, _i, _i, _i, _i, _p, _p, _i, _f, _p, _i, _p, _p, _p, _p]
            lib.dryft_gemm_stream.restype = _i
            lib.dryft_gemm_stream_ss_parts.argtypes = [_i, _i]
            lib.dryft_gemm_stream_ss_parts.restype = _i
            lib.dryft_gemm_stream_workspace_floats.restype = _ll
            _gemm_stream = lib
        return _gemm_stream


_stream_scratch: Dict[int, Tuple[torch.Tensor, torch.Tensor]] = {}


def gemm_stream_scratch(device: torch.device) -> Tuple[torch.Tensor, torch.Tensor]:
    """(workspace, tickets) of ``gemm_stream`` on this device: float32 slots for the pieces of tiles that two blocks
    share, and zeroed int32 ticket counters (one per tile; every launch leaves them zero).  One set per device
    serves every launch of a stream, because a launch only touches them after the launch before it has ended."""
    idx = device.index if device.index is not None else torch.cuda.current_device()
    sc = _stream_scratch.get(idx)
    if sc is None:
        dev = torch.device("cuda", idx)
        with torch.cuda.device(dev):
            n = int(gemm_stream_lib().dryft_gemm_stream_workspace_floats())
        sc = (torch.empty(n, dtype=torch.float32, device=dev), torch.zeros(1 << 16, dtype=torch.int32, device=dev))
        _stream_scratch[idx] = sc
    return sc


def attention_decode_supported(head_dim: int, group: int) -> bool:
    """Whether the one-launch decode attention exists for these sizes (the query heads of a kv head
    form one 16-row tensor-core operand)."""
    return head_dim > 0 and head_dim % 16 == 0 and head_dim <= 256 and 1 <= group <= 16


def attention_decode_lib(head_dim: int, group: int, page: int) -> ctypes.CDLL:
    """The fused decode attention (RoPE + cache write + split attention + combine, bfloat16)."""
    if not attention_decode_supported(head_dim, group):
        raise KernelError(f"fused decode attention does not take head_dim={head_dim} with {group} query heads per kv head")
    key = ("decode", head_dim, group, page)
    with _lock:
        lib = _variants.get(key)
        if lib is None:
            path = build.build_library("attn_decode", ("attn_decode.cu",),
                                       {"DRYFT_HEAD_DIM": head_dim, "DRYFT_GROUP": group, "DRYFT_PAGE": page})
            lib = _load(path)
            lib.dryft_attn_decode.argtypes = [_p, _i, _p, _p, _p, _p, _p, _p, _p, _p, _i, _p, _p, _p, _p, _i, _i, _i, _f, _i,
                                              _i, _f, _i, _i, _i, _i, _i, _p]
            lib.dryft_attn_decode.restype = _i
            _variants[key] = lib
        return lib


def attention_prefill_tc_supported(head_dim: int, group: int, page: int) -> bool:
    """Whether the tcgen05 prefill attention exists for these sizes."""
    return head_dim in (64, 128) and page == 64 and group >= 1


def attention_prefill_tc_lib(head_dim: int, group: int, page: int) -> ctypes.CDLL:
    """The tcgen05 / TMEM / TMA prefill attention compiled for these sizes."""
    if not attention_prefill_tc_supported(head_dim, group, page):
        raise KernelError(f"tcgen05 prefill attention takes head sizes 64 and 128 and 64-token pages, got {head_dim}, {page}")
    key = ("prefill_tc", head_dim, group, page)
    with _lock:
        lib = _variants.get(key)
        if lib is None:
            path = build.build_library("attn_prefill_tc", ("attn_prefill_tc.cu",),
                                       {"DRYFT_HEAD_DIM": head_dim, "DRYFT_GROUP": group, "DRYFT_PAGE": page})
            lib = _load(path)
            lib.dryft_attn_prefill_tc.argtypes = [_p, _p, _p, _p, _i, _p, _p, _p, _p, _p, _i, _i, _i, _i, _i, _f, _i, _p, _p]
            lib.dryft_attn_prefill_tc.restype = _i
            _variants[key] = lib
        return lib


_tickets: Dict[int, torch.Tensor] = {}


def tickets(device: torch.device, n: int) -> torch.Tensor:
    """Zeroed int32 counters the decode attention's blocks draw tickets from; every launch leaves
    them zero again, so one buffer per device serves all layers."""
    idx = device.index if device.index is not None else torch.cuda.current_device()
    t = _tickets.get(idx)
    if t is None or t.numel() < n:
        t = torch.zeros(max(n, 1 << 16), dtype=torch.int32, device=torch.device("cuda", idx))
        _tickets[idx] = t
    return t


def attention_prefill_lib(head_dim: int, group: int, page: int) -> ctypes.CDLL:
    """The tensor-core prefill attention kernel (bfloat16) compiled for these sizes."""
    if head_dim <= 0 or head_dim % 16 or head_dim > 256:
        raise KernelError(f"prefill attention takes head sizes 16..256 in steps of 16, got head_dim={head_dim}")
    key = ("prefill", head_dim, group, page)
    with _lock:
        lib = _variants.get(key)
        if lib is None:
            path = build.build_library("attn_prefill", ("attn_prefill.cu",),
                                       {"DRYFT_HEAD_DIM": head_dim, "DRYFT_GROUP": group, "DRYFT_PAGE": page})
            lib = _load(path)
            lib.dryft_attn_prefill.argtypes = [_p, _p, _p, _p, _i, _p, _p, _p, _p, _p, _i, _i, _i, _f, _i, _p]
            lib.dryft_attn_prefill.restype = _i
            _variants[key] = lib
        return lib


# ----------------------------------------------------------------------------- argument checks
_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream() -> ctypes.c_void_p:
    """The current stream's handle (also inside a graph capture).  A prompt step makes hundreds of launches;
    the raw accessor costs a fraction of a microsecond, the Stream object about fifteen."""
    if _raw_stream is not None:
        return ctypes.c_void_p(_raw_stream(torch.cuda.current_device()))
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _ptr(t: Optional[torch.Tensor]) -> ctypes.c_void_p:
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


def _need(t: torch.Tensor, name: str, dtype=None, shape=None) -> torch.Tensor:
    # the common case first (a prompt step makes a thousand of these checks); what fails it is named below
    try:
        if t.is_cuda and t.is_contiguous() and (dtype is None or t.dtype == dtype) and (
                shape is None or (len(shape) == t.dim() and all(s is None or s == d for s, d in zip(shape, t.shape)))):
            return t
    except AttributeError:
        pass
    if not isinstance(t, torch.Tensor):
        raise KernelError(f"{name}: expected a tensor, got {type(t).__name__}")
    if t.device.type != "cuda":
        raise KernelError(f"{name}: is on {t.device}; dryft_b200 kernels run on a CUDA device only")
    if not t.is_contiguous():
        raise KernelError(f"{name}: must be contiguous (shape {tuple(t.shape)}, strides {t.stride()})")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name}: expected {dtype}, got {t.dtype}")
    if shape is not None:
        if len(shape) != t.dim() or any(s is not None and s != d for s, d in zip(shape, t.shape)):
            raise KernelError(f"{name}: expected shape {tuple(shape)}, got {tuple(t.shape)}")
    return t


def _act(t: torch.Tensor, name: str) -> int:
    """1 for bfloat16, 0 for float32; anything else is refused."""
    if t.dtype == torch.bfloat16:
        return 1
    if t.dtype == torch.float32:
        return 0
    raise KernelError(f"{name}: activations are float32 or bfloat16, got {t.dtype}")


launch_count = 0  # kernels of this library launched (or captured into a graph) so far

_error_flags: Dict[int, torch.Tensor] = {}


def error_flag(device: torch.device) -> torch.Tensor:
    """The device int that kernels with bounded waits raise when a wait runs out."""
    idx = device.index if device.index is not None else torch.cuda.current_device()
    if idx not in _error_flags:
        _error_flags[idx] = torch.zeros(1, dtype=torch.int32, device=torch.device("cuda", idx))
    return _error_flags[idx]


_watched: list = []   # (weak reference to a device int32 flag, what a raised flag means)


def watch_flag(flag: torch.Tensor, what: str) -> None:
    """Have ``check_error_flags`` read this device flag too (a part's own error flag, e.g. the embedding's)."""
    import weakref

    _watched.append((weakref.ref(flag), what))


def check_error_flags() -> None:
    """Raise if any kernel gave up a bounded wait, or a part's watched flag was raised, since the last check
    (reads the flags: a sync)."""
    _watched[:] = [(ref, what) for ref, what in _watched if ref() is not None]
    for ref, what in _watched:
        flag = ref()
        if flag is not None and int(flag.item()) != 0:
            flag.zero_()
            raise KernelError(what)
    for idx, flag in _error_flags.items():
        code = int(flag.item())
        if code != 0:
            flag.zero_()
            raise KernelError(f"a kernel on cuda:{idx} gave up waiting for its own copies (bounded wait ran out, "
                              f"place {code}); results since the last check are not valid")


def _ok(rc: int, what: str, n_kernels: int = 1) -> None:
    global launch_count
    if rc == 0:
        launch_count += n_kernels
        return
    if rc == UNSUPPORTED:
        raise KernelError(f"{what}: sizes not supported by this kernel")
    raise KernelError(f"{what}: CUDA error {rc} at launch")


# ----------------------------------------------------------------------------- step metadata
def step_meta(cu_q, seq_slot, seq_len, tok_slot, tok_pos, n_tokens: int, n_seqs: int) -> None:
    for t, n in ((cu_q, "cu_q"), (seq_slot, "seq_slot"), (seq_len, "seq_len"), (tok_slot, "tok_slot"), (tok_pos, "tok_pos")):
        _need(t, n, torch.int32)
    if cu_q.numel() < n_seqs + 1 or seq_slot.numel() < n_seqs or tok_slot.numel() < n_tokens or tok_pos.numel() < n_tokens:
        raise KernelError("step_meta: index arrays shorter than the batch")
    _ok(core().dryft_step_meta(_ptr(cu_q), _ptr(seq_slot), _ptr(seq_len), n_tokens, n_seqs, _ptr(tok_slot), _ptr(tok_pos),
                               _stream()), "step_meta")


def step_advance(cu_q, seq_slot, seq_len, n_seqs: int) -> None:
    for t, n in ((cu_q, "cu_q"), (seq_slot, "seq_slot"), (seq_len, "seq_len")):
        _need(t, n, torch.int32)
    _ok(core().dryft_step_advance(_ptr(cu_q), _ptr(seq_slot), _ptr(seq_len), n_seqs, _stream()), "step_advance")


def tokens_from_state(seq_slot, last_token, tokens, n_seqs: int) -> None:
    for t, n in ((seq_slot, "seq_slot"), (last_token, "last_token"), (tokens, "tokens")):
        _need(t, n, torch.int32)
    _ok(core().dryft_tokens_from_state(_ptr(seq_slot), _ptr(last_token), _ptr(tokens), n_seqs, _stream()), "tokens_from_state")


# ----------------------------------------------------------------------------- elementwise
def embed(tokens, table, out, err=None) -> None:
    _need(tokens, "tokens", torch.int32)
    _need(table, "embedding table")
    n = out.shape[0]
    _need(out, "embedding output", table.dtype, (n, table.shape[1]))
    if tokens.numel() < n:
        raise KernelError("embed: fewer tokens than output rows")
    if err is not None:
        _need(err, "err", torch.int32)
    _ok(core().dryft_embed(_act(table, "embedding table"), _ptr(tokens), _ptr(table), _ptr(out), n, table.shape[1],
                           table.shape[0], _ptr(err), _stream()), "embed")


def rmsnorm(x, weight, eps: float, out, delta=None, rows=None, x_out=None) -> None:
    """``out[r] = norm(x[src] (+ delta[src])) * weight`` with ``src = rows[r]`` if rows is given;
    ``x_out[src]`` receives the summed row when given (may alias ``x``)."""
    hidden = x.shape[-1]
    _need(x, "x")
    _need(weight, "norm weight", torch.float32, (hidden,))
    n_rows = out.shape[0]
    _need(out, "norm output", x.dtype, (n_rows, hidden))
    if delta is not None:
        _need(delta, "delta", x.dtype, tuple(x.shape))
    if rows is not None:
        _need(rows, "rows", torch.int32)
        if rows.numel() < n_rows:
            raise KernelError("rmsnorm: fewer row indices than output rows")
    elif x.shape[0] < n_rows:
        raise KernelError("rmsnorm: input has fewer rows than the output")
    if x_out is not None:
        _need(x_out, "x_out", x.dtype, tuple(x.shape))
    _ok(core().dryft_rmsnorm(_act(x, "x"), _ptr(x), _ptr(delta), _ptr(weight), _ptr(rows), _ptr(x_out), _ptr(out), n_rows,
                             hidden, float(eps), _stream()), f"rmsnorm (width {hidden})")


def residual_add(x, delta) -> None:
    _need(x, "x")
    _need(delta, "delta", x.dtype, tuple(x.shape))
    _ok(core().dryft_residual_add(_act(x, "x"), _ptr(x), _ptr(delta), x.numel(), _stream()), "residual_add")


def silu_mul(gate_up, out) -> None:
    rows, two_i = gate_up.shape
    _need(gate_up, "gate_up")
    if two_i % 2:
        raise KernelError(f"silu_mul: fused gate|up width must be even, got {two_i}")
    _need(out, "silu_mul output", gate_up.dtype, (rows, two_i // 2))
    _ok(core().dryft_silu_mul(_act(gate_up, "gate_up"), _ptr(gate_up), _ptr(out), rows, two_i // 2, _stream()), "silu_mul")


# ----------------------------------------------------------------------------- rope + cache write
def qk_norm_rope_store(qkv, q_norm_w, k_norm_w, inv_freq, tok_slot, tok_pos, q_out, k_pages, v_pages, page_table,
                       n_heads: int, n_kv_heads: int, head_dim: int, rotary_dim: int, eps: float, write_kv: bool = True,
                       cs_table=None, zero_tail: bool = False) -> None:
    """``cs_table`` (from ``rope_table``; optional) holds the step's cos / sin so that layers share them.
    ``zero_tail``: the last token each sequence brings also zeroes the value rows of its page behind its own
    (what the page's last holder left there), for attention kernels that multiply whole pages."""
    n = qkv.shape[0]
    width = (n_heads + (2 * n_kv_heads if write_kv else 0)) * head_dim
    _need(qkv, "qkv", None, (n, width))
    is_bf16 = _act(qkv, "qkv")
    has_norm = q_norm_w is not None
    if has_norm:
        _need(q_norm_w, "q_norm weight", torch.float32, (head_dim,))
        _need(k_norm_w, "k_norm weight", torch.float32, (head_dim,))
    if rotary_dim:
        _need(inv_freq, "inv_freq", torch.float32, (rotary_dim // 2,))
    _need(tok_slot, "tok_slot", torch.int32)
    _need(tok_pos, "tok_pos", torch.int32)
    if tok_slot.numel() < n or tok_pos.numel() < n:
        raise KernelError("qk_norm_rope_store: token index arrays shorter than the batch")
    _need(q_out, "q_out", qkv.dtype, (n, n_heads, head_dim))
    page_size, max_pages = 0, 0
    if write_kv:
        _need(k_pages, "k_pages", qkv.dtype, (None, n_kv_heads, None, head_dim))
        _need(v_pages, "v_pages", qkv.dtype, tuple(k_pages.shape))
        _need(page_table, "page_table", torch.int32)
        page_size, max_pages = k_pages.shape[2], page_table.shape[1]
    if cs_table is not None:
        _need(cs_table, "cs_table", qkv.dtype, (None, 2, rotary_dim // 2))
        if cs_table.shape[0] < n:
            raise KernelError("qk_norm_rope_store: cos/sin table shorter than the batch")
    _ok(core().dryft_qk_norm_rope_store(is_bf16, _ptr(qkv), width, _ptr(q_norm_w), _ptr(k_norm_w), _ptr(inv_freq),
                                        _ptr(cs_table), _ptr(tok_slot), _ptr(tok_pos), _ptr(q_out), _ptr(k_pages if write_kv else None),
                                        _ptr(v_pages if write_kv else None), _ptr(page_table if write_kv else None),
                                        max_pages, n, n_heads, n_kv_heads, head_dim, rotary_dim, page_size, float(eps),
                                        int(has_norm), int(write_kv), int(zero_tail), _stream()), "qk_norm_rope_store")


def rope_table(tok_pos, inv_freq, n_tokens: int, dtype: torch.dtype) -> torch.Tensor:
    """cos | sin of ``pos * inv_freq`` for every token of a step, rounded to ``dtype``: [n_tokens, 2, R/2]."""
    _need(tok_pos, "tok_pos", torch.int32)
    _need(inv_freq, "inv_freq", torch.float32)
    if tok_pos.numel() < n_tokens:
        raise KernelError("rope_table: tok_pos shorter than the batch")
    half = inv_freq.numel()
    table = torch.empty(n_tokens, 2, half, dtype=dtype, device=tok_pos.device)
    is_bf16 = _act(table, "table")
    _ok(core().dryft_rope_table(is_bf16, _ptr(tok_pos), _ptr(inv_freq), _ptr(table), n_tokens, 2 * half, _stream()), "rope_table")
    return table


# ----------------------------------------------------------------------------- attention
def attn_rows(q, k_pages, v_pages, page_table, tok_slot, tok_pos, out, scale: float, window: Optional[int],
              n_splits: int = 1, part_o=None, part_ml=None) -> None:
    n, n_heads, head_dim = q.shape
    is_bf16 = _act(q, "q")
    _need(q, "q")
    n_kv = k_pages.shape[1]
    page = k_pages.shape[2]
    _need(k_pages, "k_pages", q.dtype, (None, n_kv, page, head_dim))
    _need(v_pages, "v_pages", q.dtype, tuple(k_pages.shape))
    _need(page_table, "page_table", torch.int32)
    _need(tok_slot, "tok_slot", torch.int32)
    _need(tok_pos, "tok_pos", torch.int32)
    if tok_slot.numel() < n or tok_pos.numel() < n:
        raise KernelError("attn_rows: token index arrays shorter than the batch")
    _need(out, "attention output", q.dtype, (n, n_heads * head_dim))
    if n_heads % n_kv:
        raise KernelError(f"attn_rows: {n_heads} query heads are not a multiple of {n_kv} kv heads")
    if n_splits > 1:
        _need(part_o, "part_o", torch.float32)
        _need(part_ml, "part_ml", torch.float32)
        if part_o.numel() < n * n_heads * n_splits * head_dim or part_ml.numel() < n * n_heads * n_splits * 2:
            raise KernelError("attn_rows: partial buffers too small for the split count")
    lib = attention_rows_lib(head_dim, n_heads // n_kv, page)
    _ok(lib.dryft_attn_rows(is_bf16, _ptr(q), _ptr(k_pages), _ptr(v_pages), _ptr(page_table), page_table.shape[1],
                            _ptr(tok_slot), _ptr(tok_pos), _ptr(out), _ptr(part_o), _ptr(part_ml), n, n_kv, n_splits,
                            float(scale), int(window or 0), _stream()), f"attn_rows (head_dim {head_dim})",
        n_kernels=2 if n_splits > 1 else 1)


def attn_decode(qkv, q_norm_w, k_norm_w, inv_freq, tok_slot, tok_pos, k_pages, v_pages, page_table, out,
                n_heads: int, n_kv_heads: int, head_dim: int, rotary_dim: int, eps: float, scale: float,
                window: Optional[int], n_splits: int, part_o=None, part_ml=None, write_kv: bool = True, pdl: bool = False,
                shape: int = -1, cluster: bool = True) -> None:
    """One launch for a decode step's attention (bfloat16): per-head q/k norm + RoPE of each row's new
    token, its K/V written into the cache, attention of its query heads over the cache, splits combined.
    ``shape``: warps per block, 0 / 1 / 2 for 8 / 4 / 2; -1 lets the launcher take the widest whose grid is
    resident at once.  ``cluster``: with 2..8 splits the splits of a (row, kv head) run as one thread-block
    cluster and are combined through distributed shared memory (no partial buffers needed); with more
    splits, or ``cluster=False``, they meet in ``part_o`` / ``part_ml`` and the last block to finish combines."""
    n = qkv.shape[0]
    width = (n_heads + (2 * n_kv_heads if write_kv else 0)) * head_dim
    _need(qkv, "qkv", torch.bfloat16, (n, width))
    has_norm = q_norm_w is not None
    if has_norm:
        _need(q_norm_w, "q_norm weight", torch.float32, (head_dim,))
        _need(k_norm_w, "k_norm weight", torch.float32, (head_dim,))
    if rotary_dim:
        _need(inv_freq, "inv_freq", torch.float32, (rotary_dim // 2,))
    page = k_pages.shape[2]
    _need(k_pages, "k_pages", torch.bfloat16, (None, n_kv_heads, page, head_dim))
    _need(v_pages, "v_pages", torch.bfloat16, tuple(k_pages.shape))
    for t, nm in ((page_table, "page_table"), (tok_slot, "tok_slot"), (tok_pos, "tok_pos")):
        _need(t, nm, torch.int32)
    if tok_slot.numel() < n or tok_pos.numel() < n:
        raise KernelError("attn_decode: token index arrays shorter than the batch")
    _need(out, "attention output", torch.bfloat16, (n, n_heads * head_dim))
    if n_heads % n_kv_heads:
        raise KernelError(f"attn_decode: {n_heads} query heads are not a multiple of {n_kv_heads} kv heads")
    tk = None
    use_cluster = bool(cluster) and 2 <= n_splits <= 8
    if n_splits > 1 and not use_cluster:
        _need(part_o, "part_o", torch.float32)
        _need(part_ml, "part_ml", torch.float32)
        if part_o.numel() < n * n_heads * n_splits * head_dim or part_ml.numel() < n * n_heads * n_splits * 2:
            raise KernelError("attn_decode: partial buffers too small for the split count")
        tk = tickets(qkv.device, n * n_kv_heads)
    lib = attention_decode_lib(head_dim, n_heads // n_kv_heads, page)
    _ok(lib.dryft_attn_decode(_ptr(qkv), width, _ptr(q_norm_w), _ptr(k_norm_w), _ptr(inv_freq), _ptr(tok_slot), _ptr(tok_pos),
                              _ptr(k_pages), _ptr(v_pages), _ptr(page_table), page_table.shape[1], _ptr(out), _ptr(part_o),
                              _ptr(part_ml), _ptr(tk), n, n_kv_heads, n_splits, float(scale), int(window or 0),
                              int(rotary_dim), float(eps), int(has_norm), int(write_kv), int(pdl), int(shape), int(use_cluster), _stream()),
        f"attn_decode (head_dim {head_dim})")


def attn_prefill(q, k_pages, v_pages, page_table, tile_tok0, tile_rows, tok_slot, tok_pos, out, n_tiles: int,
                 scale: float, window: Optional[int]) -> None:
    """Causal grouped-query attention of packed prompts over the paged cache (bfloat16, tensor cores).
    Tile ``t`` covers the ``tile_rows[t]`` query tokens from packed index ``tile_tok0[t]`` on, all of one
    sequence; their slot and positions are read from ``tok_slot`` / ``tok_pos``."""
    n, n_heads, head_dim = q.shape
    _need(q, "q", torch.bfloat16)
    n_kv = k_pages.shape[1]
    page = k_pages.shape[2]
    _need(k_pages, "k_pages", torch.bfloat16, (None, n_kv, page, head_dim))
    _need(v_pages, "v_pages", torch.bfloat16, tuple(k_pages.shape))
    for t, nm in ((page_table, "page_table"), (tile_tok0, "tile_tok0"), (tile_rows, "tile_rows"),
                  (tok_slot, "tok_slot"), (tok_pos, "tok_pos")):
        _need(t, nm, torch.int32)
    if tile_tok0.numel() < n_tiles or tile_rows.numel() < n_tiles:
        raise KernelError("attn_prefill: tile arrays shorter than the tile count")
    _need(out, "attention output", torch.bfloat16, (n, n_heads * head_dim))
    if n_heads % n_kv:
        raise KernelError(f"attn_prefill: {n_heads} query heads are not a multiple of {n_kv} kv heads")
    lib = attention_prefill_lib(head_dim, n_heads // n_kv, page)
    _ok(lib.dryft_attn_prefill(_ptr(q), _ptr(k_pages), _ptr(v_pages), _ptr(page_table), page_table.shape[1],
                               _ptr(tile_tok0), _ptr(tile_rows), _ptr(tok_slot), _ptr(tok_pos), _ptr(out), n_tiles,
                               n_heads, n_kv, float(scale), int(window or 0), _stream()),
        f"attn_prefill (head_dim {head_dim})")


def attn_prefill_tc(q, k_pages, v_pages, page_table, tile_tok0, tile_rows, tok_slot, tok_pos, out, n_tiles: int,
                    scale: float, window: Optional[int]) -> None:
    """``attn_prefill`` on the 5th-generation tensor cores (tcgen05.mma, tensor memory, TMA); tiles of up
    to 128 query tokens; head sizes 64 and 128."""
    n, n_heads, head_dim = q.shape
    _need(q, "q", torch.bfloat16)
    n_kv = k_pages.shape[1]
    page = k_pages.shape[2]
    _need(k_pages, "k_pages", torch.bfloat16, (None, n_kv, page, head_dim))
    _need(v_pages, "v_pages", torch.bfloat16, tuple(k_pages.shape))
    for t, nm in ((page_table, "page_table"), (tile_tok0, "tile_tok0"), (tile_rows, "tile_rows"),
                  (tok_slot, "tok_slot"), (tok_pos, "tok_pos")):
        _need(t, nm, torch.int32)
    if tile_tok0.numel() < n_tiles or tile_rows.numel() < n_tiles:
        raise KernelError("attn_prefill_tc: tile arrays shorter than the tile count")
    _need(out, "attention output", torch.bfloat16, (n, n_heads * head_dim))
    if n_heads % n_kv:
        raise KernelError(f"attn_prefill_tc: {n_heads} query heads are not a multiple of {n_kv} kv heads")
    lib = attention_prefill_tc_lib(head_dim, n_heads // n_kv, page)
    _ok(lib.dryft_attn_prefill_tc(_ptr(q), _ptr(k_pages), _ptr(v_pages), _ptr(page_table), page_table.shape[1],
                                  _ptr(tile_tok0), _ptr(tile_rows), _ptr(tok_slot), _ptr(tok_pos), _ptr(out), n_tiles, n,
                                  k_pages.shape[0], n_heads, n_kv, float(scale), int(window or 0),
                                  _ptr(error_flag(q.device)), _stream()),
        f"attn_prefill_tc (head_dim {head_dim})")


# ----------------------------------------------------------------------------- matrix products
def gemm_nt_f32(a, w, out) -> None:
    """``out[M,N] = a[M,K] @ w[N,K].T`` in true 32-bit."""
    m, k = a.shape
    n = w.shape[0]
    _need(a, "a", torch.float32)
    _need(w, "w", torch.float32, (n, k))
    _need(out, "out", torch.float32, (m, n))
    _ok(core().dryft_gemm_nt_f32(_ptr(a), k, _ptr(w), _ptr(out), n, m, n, k, _stream()), "gemm_nt_f32")


SMALL_M_LIMIT = 16  # rows the weight-streaming product takes
SS_STRIDE = 64  # floats per block in the sum-of-squares buffers of the fused decode products


def weighted_ahead_supported(k: int) -> bool:
    """Whether products over ``k`` inputs can take / leave activations weighted ahead (``xw_in`` / ``xw_out``)."""
    return k > 0 and k % 256 == 0


def small_m_ss_parts(n: int, k: int) -> int:
    """Blocks of sums of squares (64 floats each) that ``gemm_small_m(mode="residual")`` leaves for ``n`` outputs over
    ``k`` inputs: one per 16-row tile."""
    return (n + 15) // 16


def gemm_small_m(a, w, out, *, mode: str = "store", norm_w=None, ss_in=None, ss_parts: int = 0, eps: float = 0.0,
                 ss_out=None, pdl: bool = False, xw_in=None, next_w=None, xw_out=None) -> None:
    """``a[M,K] @ w[.,K].T`` for up to 16 rows (decode; K a multiple of 16): bfloat16 operands, 32-bit accumulation,
    every weight byte read once.  ``mode``:

    * ``"store"``: ``out[M,N]`` (bfloat16 or float32) receives the product, ``w`` is ``[N,K]``;
    * ``"residual"``: ``out`` is the residual stream ``x[M,N]``, updated in place ``x += product``; with
      ``ss_out`` ``[small_m_ss_parts(N, K), 64]`` float32 the per-row sums of squares of the new ``x`` are left
      there, one partial per tile of up to 16 columns;
    * ``"silu"``: ``w`` is ``[2N,K]`` (gate rows, then up rows) and ``out[M,N] = silu(gate) * up``.

    With ``norm_w`` ``[K]`` float32 the rows of ``a`` are RMS-normalised on the fly; ``ss_in``
    ``[ss_parts, 64]`` holds their sums of squares as an earlier ``"residual"`` product (or ``row_sumsq``)
    left them.  ``pdl`` launches the kernel as a programmatic dependent of the launch before it: its
    first weight requests overlap that launch's tail.

    The norm split over two launches (inner sizes that are multiples of 256 only, ``weighted_ahead_supported``):
    a ``"residual"`` product given the next norm's weight ``next_w`` ``[N]`` also leaves ``xw_out[M,N] =
    T(x * next_w)``; a product given such ``xw_in`` ``[M,K]`` (with ``ss_in``, ``eps``) multiplies it as plain
    activations and scales its sums by the norm's factor in the epilogue -- no prologue on its critical path."""
    m, k = a.shape
    _need(a, "a", torch.bfloat16)
    if xw_in is not None:
        if not weighted_ahead_supported(k):
            raise KernelError(f"gemm_small_m: activations weighted ahead need an inner size that is a multiple of 256, got {k}")
        _need(xw_in, "xw_in", torch.bfloat16, (m, k))
    if (next_w is None) != (xw_out is None):
        raise KernelError("gemm_small_m: next_w and xw_out go together")
    if xw_out is not None and (mode != "residual" or not weighted_ahead_supported(k)):
        raise KernelError("gemm_small_m: xw_out belongs to mode='residual' with an inner size that is a multiple of 256")
    if mode == "silu":
        n = w.shape[0] // 2
        _need(w, "w", torch.bfloat16, (2 * n, k))
        _need(out, "out", torch.bfloat16, (m, n))
        code = 3
    elif mode == "residual":
        n = w.shape[0]
        _need(w, "w", torch.bfloat16, (n, k))
        _need(out, "residual stream", torch.bfloat16, (m, n))
        code = 2
        if ss_out is not None:
            _need(ss_out, "ss_out", torch.float32)
            if ss_out.numel() < small_m_ss_parts(n, k) * SS_STRIDE:
                raise KernelError("gemm_small_m: ss_out too small (small_m_ss_parts(N, K) blocks of 64 floats are left)")
    elif mode == "store":
        n = w.shape[0]
        _need(w, "w", torch.bfloat16, (n, k))
        _need(out, "out", None, (m, n))
        if out.dtype not in (torch.bfloat16, torch.float32):
            raise KernelError(f"gemm_small_m: output must be bfloat16 or float32, got {out.dtype}")
        code = int(out.dtype == torch.float32)
    else:
        raise KernelError(f"gemm_small_m: unknown mode {mode!r}")
    if mode != "residual" and ss_out is not None:
        raise KernelError("gemm_small_m: ss_out belongs to mode='residual'")
    if norm_w is not None or xw_in is not None:
        if norm_w is not None:
            _need(norm_w, "norm_w", torch.float32, (k,))
        _need(ss_in, "ss_in", torch.float32)
        if ss_parts <= 0 or ss_in.numel() < ss_parts * SS_STRIDE:
            raise KernelError("gemm_small_m: ss_in does not hold ss_parts blocks")
    if xw_out is not None:
        _need(next_w, "next norm weight", torch.float32, (n,))
        _need(xw_out, "xw_out", torch.bfloat16, (m, n))
    if k % 256 == 0:  # the form compiled for this inner size: loops unrolled, offsets immediate
        lib = gemm_decode_lib(k)
        if xw_in is not None:
            rc = lib.dryft_gemm_decode(_ptr(xw_in), k, _ptr(w), _ptr(out), n, code, m, n, None, _ptr(ss_in), int(ss_parts),
                                       float(eps), _ptr(ss_out), int(pdl), 1, _ptr(next_w), _ptr(xw_out), _stream())
            if rc != UNSUPPORTED:
                _ok(rc, f"gemm_decode (M={m}, N={n}, K={k}, mode={mode}, activations weighted ahead)")
                return
            if norm_w is None:  # it refuses what does not fit its shared memory; with norm_w the plain form takes over
                _ok(rc, f"gemm_decode (M={m}, N={n}, K={k}, mode={mode}, activations weighted ahead; give norm_w for the other form)")
        rc = lib.dryft_gemm_decode(_ptr(a), k, _ptr(w), _ptr(out), n, code, m, n, _ptr(norm_w), _ptr(ss_in), int(ss_parts),
                                   float(eps), _ptr(ss_out), int(pdl), 0, _ptr(next_w), _ptr(xw_out), _stream())
        if rc != UNSUPPORTED or xw_out is not None or ss_out is not None:
            # the general form below cannot leave xw_out, and leaves another number of blocks of sums of squares
            _ok(rc, f"gemm_decode (M={m}, N={n}, K={k}, mode={mode})")
            return
    _ok(core().dryft_gemm_small_m(_ptr(a), k, _ptr(w), _ptr(out), n, code, m, n, k, _ptr(norm_w), _ptr(ss_in),
                                  int(ss_parts), float(eps), _ptr(ss_out), int(pdl), _stream()),
        f"gemm_small_m (M={m}, N={n}, K={k}, mode={mode})")


STREAM_M_LIMIT = 64


def gemm_stream_supported(m: int, k: int) -> bool:
    return 0 < m <= STREAM_M_LIMIT and k > 0 and k % 64 == 0


def gemm_stream_ss_parts(n_out: int, k_in: int) -> int:
    """Blocks of sums of squares that ``gemm_stream(mode="residual")`` leaves in ``ss_out``."""
    return int(gemm_stream_lib().dryft_gemm_stream_ss_parts(int(n_out), int(k_in)))


def gemm_stream(a, w, out, *, mode: str = "store", norm_w=None, ss_in=None, ss_parts: int = 0, eps: float = 0.0,
                ss_out=None, pdl: bool = False) -> None:
    """``gemm_small_m``'s contract for up to 64 rows, on tcgen05 with the weights streamed by TMA through a
    shared-memory ring, the work cut evenly over the SMs and tiles that two blocks share summed in block order.
    ``ss_out`` must hold ``gemm_stream_ss_parts(N, K)`` blocks of 64 floats."""
    m, k = a.shape
    _need(a, "a", torch.bfloat16)
    if not gemm_stream_supported(m, k):
        raise KernelError(f"gemm_stream takes 1..{STREAM_M_LIMIT} rows and inner sizes that are multiples of 64, got M={m}, K={k}")
    code = {"store": 1 if out.dtype == torch.float32 else 0, "residual": 2, "silu": 3}.get(mode)
    if code is None:
        raise KernelError(f"gemm_stream: unknown mode {mode!r}")
    rows = w.shape[0]
    n = rows // 2 if mode == "silu" else rows
    _need(w, "w", torch.bfloat16, (2 * n if mode == "silu" else n, k))
    _need(out, "out", torch.float32 if code == 1 else torch.bfloat16, (m, n))
    if n > (1 << 16) * 64:
        raise KernelError(f"gemm_stream: {n} outputs are more than its ticket counters cover")
    if norm_w is not None:
        if mode == "residual":
            raise KernelError("gemm_stream: a residual product takes plain activations")
        _need(norm_w, "norm weight", torch.float32, (k,))
        _need(ss_in, "ss_in", torch.float32)
        if ss_parts <= 0 or ss_in.numel() < ss_parts * SS_STRIDE:
            raise KernelError("gemm_stream: ss_in does not hold ss_parts blocks")
    if ss_out is not None:
        if mode != "residual":
            raise KernelError("gemm_stream: ss_out belongs to mode='residual'")
        _need(ss_out, "ss_out", torch.float32)
        if ss_out.numel() < gemm_stream_ss_parts(n, k) * SS_STRIDE:
            raise KernelError("gemm_stream: ss_out too small")
    ws, tk = gemm_stream_scratch(a.device)
    _ok(gemm_stream_lib().dryft_gemm_stream(_ptr(a), k, _ptr(w), _ptr(out), n, code, m, n, k, _ptr(norm_w), _ptr(ss_in),
                                            int(ss_parts), float(eps), _ptr(ss_out), int(pdl), _ptr(error_flag(a.device)),
                                            _ptr(ws), _ptr(tk), _stream()),
        f"gemm_stream (M={m}, N={n}, K={k}, mode={mode})")


SMALL_M_CUT_BYTES = 100 * 1024  # the shared-memory cut that csrc/gemm_decode.cu asks for (CARVEOUT_BYTES)


def small_m_staged_bytes(m: int, k: int) -> int:
    """Shared memory of one block of the per-size decode product with the norm on the way in (csrc/gemm_decode.cu,
    ``launch3``): two groups' partial sums or the norm's weight, 64 factors, the ``m`` rows and a row of zeros, one
    reserved KB."""
    mp = 8 if m <= 8 else 16
    head = (max(2 * 8 * 16 * (mp + 1) * 4, k * 2) + 15) // 16 * 16   # two groups' partial sums
    rows = m + 1 if m < mp else mp
    return head + 256 + rows * (k + 32) * 2 + 1024


def fused_rows_supported(m: int, k: int, small_m_max: int, stream_m_max: int, normed: bool = False) -> bool:
    """Whether ``fused_product`` takes ``m`` rows over ``k`` inputs: the register-streaming product up to
    ``small_m_max`` rows, the tcgen05 one up to ``stream_m_max``.  ``normed``: the product has the norm on its way
    in, so its rows stay in shared memory; above 8 rows that is taken only for widths whose 16 staged rows keep
    a block under the cut that leaves L1 large enough for the weights in flight.  Measured at 9 to 16 rows:
    width 2,560: 2.38-2.40 ms a step against 2.74-2.77 ms with the library's products; width 4,096 (ten rows
    fit): 4.18 against 3.86 ms; width 5,120: 16.4 against 13.2 ms."""
    if m <= min(small_m_max, SMALL_M_LIMIT):
        if m > 8 and normed and k % 256 == 0 and small_m_staged_bytes(16, k) > SMALL_M_CUT_BYTES:
            return False
        return k % 16 == 0
    return m <= min(stream_m_max, STREAM_M_LIMIT) and gemm_stream_supported(m, k)


def fused_ss_parts(m: int, n: int, k: int, small_m_max: int) -> int:
    """Blocks of sums of squares that ``fused_product(mode="residual")`` of these sizes leaves in ``ss_out``."""
    if m <= min(small_m_max, SMALL_M_LIMIT):
        return small_m_ss_parts(n, k)
    return gemm_stream_ss_parts(n, k)


def fused_product(a, w, out, *, small_m_max: int, **kw) -> None:
    """A decode product with its norm / residual / SiLU*mul fused in, by the kernel that suits the row count:
    ``gemm_small_m`` (weights streamed through registers into mma.sync) up to ``small_m_max`` rows, ``gemm_stream``
    (TMA ring, tcgen05, even cut over the SMs) above.  Activations weighted ahead (``xw_in`` / ``xw_out``) belong
    to the former only."""
    if a.shape[0] <= min(small_m_max, SMALL_M_LIMIT):
        gemm_small_m(a, w, out, **kw)
        return
    if kw.get("xw_in") is not None or kw.get("xw_out") is not None:
        raise KernelError("fused_product: activations weighted ahead are not taken above small_m_max rows")
    kw = {k_: v for k_, v in kw.items() if k_ not in ("xw_in", "xw_out", "next_w")}
    gemm_stream(a, w, out, **kw)


def row_sumsq(x, ss, norm_w=None, xw_out=None) -> None:
    """``ss[m] = sum(x[m]^2)`` for up to 64 rows of bfloat16 ``x``: one block of sums of squares.  With a norm
    weight it also leaves ``xw_out = T(x * norm_w)`` for a product that takes activations weighted ahead."""
    rows, hidden = x.shape
    _need(x, "x", torch.bfloat16)
    _need(ss, "ss", torch.float32)
    if ss.numel() < SS_STRIDE:
        raise KernelError("row_sumsq: ss holds fewer than 64 floats")
    if (norm_w is None) != (xw_out is None):
        raise KernelError("row_sumsq: norm_w and xw_out go together")
    if xw_out is not None:
        _need(norm_w, "norm weight", torch.float32, (hidden,))
        _need(xw_out, "xw_out", torch.bfloat16, (rows, hidden))
    _ok(core().dryft_row_sumsq(_ptr(x), rows, hidden, _ptr(ss), _ptr(norm_w), _ptr(xw_out), _stream()), "row_sumsq")


# ----------------------------------------------------------------------------- token choice
def argmax_rows(logits, out, row_slot=None, last_token=None) -> None:
    rows, vocab = logits.shape
    _need(logits, "logits", torch.float32)
    _need(out, "chosen tokens", torch.int32)
    if out.numel() < rows:
        raise KernelError("argmax_rows: output shorter than the rows")
    if row_slot is not None:
        _need(row_slot, "row_slot", torch.int32)
        _need(last_token, "last_token", torch.int32)
    _ok(core().dryft_argmax_rows(_ptr(logits), rows, vocab, vocab, _ptr(out), _ptr(row_slot), _ptr(last_token), _stream()),
        "argmax_rows")


def sample_rows(logits, temperature: float, top_k: int, seed: int, row_seq, row_step, out, row_slot=None, last_token=None,
                step_base: int = 0) -> None:
    """Row r draws with uniform(seed, row_seq[r] (or r), step_base + row_step[r] (or 0))."""
    rows, vocab = logits.shape
    _need(logits, "logits", torch.float32)
    _need(out, "chosen tokens", torch.int32)
    if not temperature > 0.0:
        raise KernelError("sample_rows: temperature must be positive (use argmax_rows for greedy)")
    for t, nm in ((row_seq, "row_seq"), (row_step, "row_step")):
        if t is None:
            continue
        _need(t, nm, torch.int32)
        if t.numel() < rows:
            raise KernelError(f"sample_rows: {nm} shorter than the rows")
    if row_slot is not None:
        _need(row_slot, "row_slot", torch.int32)
        _need(last_token, "last_token", torch.int32)
    _ok(core().dryft_sample_rows(_ptr(logits), rows, vocab, vocab, float(temperature), int(top_k), int(seed) & (2**64 - 1),
                                 _ptr(row_seq), _ptr(row_step), int(step_base), _ptr(out), _ptr(row_slot), _ptr(last_token),
                                 _stream()), "sample_rows")
