"""The allocation-free attention entry point, called through its exported C symbol.

``dryft_attn_rows_static_scratch`` is for hosts of the library that cannot allocate device memory
themselves (a fixed start-up budget, an application that owns the allocator, a stream capture in
progress): its split partials live in a device array built into the library.  The test calls the
symbol directly with ctypes, twice in a row with different inputs (the array keeps the first call's
contents, which must not matter), and checks each result against the ordinary entry point, which is
handed scratch buffers; sizes beyond the built-in array must be refused, not truncated.

This file sorts last on purpose: if it fails, a run that stops at the first failure has already run
every other test."""

import ctypes
import math

import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda"
SCRATCH_TOO_SMALL = -3


def _ptr(t):
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


def _case(dtype, seed, n_heads, n_kv, d, page=64):
    g = torch.Generator().manual_seed(seed)
    lens = [1, 64, 130, 300]
    n_pages, max_pages = 12, 5
    kc = torch.randn(n_pages, n_kv, page, d, generator=g).to(dtype).to(DEV)
    vc = torch.randn(n_pages, n_kv, page, d, generator=g).to(dtype).to(DEV)
    perm = torch.randperm(n_pages, generator=g).tolist()
    pt = torch.zeros(len(lens), max_pages, dtype=torch.int32)
    for s, L in enumerate(lens):
        for lp in range((L + page - 1) // page):
            pt[s, lp] = perm.pop()
    rows = [(0, 0), (1, 63), (2, 129), (3, 299), (3, 100), (-1, 0)]
    q = torch.randn(len(rows), n_heads, d, generator=g).to(dtype).to(DEV)
    slot = torch.tensor([r[0] for r in rows], dtype=torch.int32, device=DEV)
    pos = torch.tensor([r[1] for r in rows], dtype=torch.int32, device=DEV)
    return q, kc, vc, pt.to(DEV), slot, pos


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_static_scratch_entry_point_matches_the_ordinary_one(dtype):
    from dryft_b200.ops import kernels as K

    n_heads, n_kv, d, splits = 8, 2, 128, 4
    lib = K.attention_rows_lib(d, n_heads // n_kv, 64)
    fn = lib.dryft_attn_rows_static_scratch
    fn.restype = ctypes.c_int
    i, f, p = ctypes.c_int, ctypes.c_float, ctypes.c_void_p
    fn.argtypes = [i, p, p, p, p, i, p, p, p, i, i, i, f, i, p]
    lib.dryft_attn_rows_static_scratch_floats.restype = ctypes.c_longlong
    capacity = lib.dryft_attn_rows_static_scratch_floats()
    assert capacity == 1 << 20
    scale = 1.0 / math.sqrt(d)
    tol = 2e-2 if dtype == torch.bfloat16 else 2e-5
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    for call, (seed, window) in enumerate([(1, 0), (2, 70)]):  # two calls in a row, other inputs, shared scratch
        q, kc, vc, pt, slot, pos = _case(dtype, seed, n_heads, n_kv, d)
        n = q.shape[0]
        out = torch.full((n, n_heads * d), 7.0, device=DEV).to(dtype)
        rc = fn(int(dtype == torch.bfloat16), _ptr(q), _ptr(kc), _ptr(vc), _ptr(pt), pt.shape[1], _ptr(slot), _ptr(pos),
                _ptr(out), n, n_kv, splits, scale, window, stream)
        assert rc == 0, f"call {call}: return code {rc}"
        ref = torch.empty_like(out)
        part_o = torch.empty(n, n_heads, splits, d, device=DEV)
        part_ml = torch.empty(n, n_heads, splits, 2, device=DEV)
        K.attn_rows(q, kc, vc, pt, slot, pos, ref, scale, window or None, splits, part_o, part_ml)
        torch.cuda.synchronize()
        assert torch.isfinite(out.float()).all()
        torch.testing.assert_close(out.float(), ref.float(), rtol=tol, atol=tol)
    # a request beyond the built-in scratch is refused and launches nothing
    big_rows = capacity // (n_heads * splits * (d + 2)) + 1
    untouched = torch.full((1,), 3.0, device=DEV).to(dtype)
    rc = fn(int(dtype == torch.bfloat16), _ptr(q), _ptr(kc), _ptr(vc), _ptr(pt), pt.shape[1], _ptr(slot), _ptr(pos),
            _ptr(untouched), big_rows, n_kv, splits, scale, 0, stream)
    assert rc == SCRATCH_TOO_SMALL
    # counts whose product would wrap around 64 bits are refused too (the check divides, it does not multiply)
    rc = fn(int(dtype == torch.bfloat16), _ptr(q), _ptr(kc), _ptr(vc), _ptr(pt), pt.shape[1], _ptr(slot), _ptr(pos),
            _ptr(untouched), 2**31 - 1, 65535, 65535, scale, 0, stream)
    assert rc == SCRATCH_TOO_SMALL
    torch.cuda.synchronize()
    assert float(untouched[0]) == 3.0
