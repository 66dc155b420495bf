"""Kernel microbenchmarks on Qwen3-4B shapes: ``python -m dryft_b200.ops.microbench <what>``.

``attn-prefill``   causal prompt attention of one sequence: mma.sync kernel against the tcgen05 kernel
``decode-chain``   a layer's four decode products as a chain of programmatic launches in a CUDA graph,
                   36 layers with weights of their own: gemm_small_m / gemm_decode against gemm_stream
``decode-products``  each of a layer's four products alone (36 weights of its own, in a CUDA graph), 8 / 16 / 64 rows:
                   gemm_small_m, gemm_stream (with its fusions, and as a plain store) and the library's torch.mm

The functions take the sizes as arguments (``layers``, ``rows``, ``tokens``) so that a test can run them small.

Timed with CUDA events after warm-ups; inputs of a chain are larger than L2.  The numbers quoted under
``profiles/`` come from here.  hari495/dryft times whole generations only (``agent/bench.py``).
"""

from __future__ import annotations

import sys

import torch

from . import kernels as K

DEV = "cuda"
BF = torch.bfloat16


def _time(fn, iters: int) -> float:
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(iters):
        fn()
    e.record()
    torch.cuda.synchronize()
    return s.elapsed_time(e) * 1000.0 / iters   # microseconds


def attn_prefill(token_counts=(2048, 8192)) -> None:
    n_heads, n_kv, d, page = 32, 8, 128, 64
    for tokens in token_counts:
        n_pages = (tokens + page - 1) // page + 1
        kc = torch.randn(n_pages, n_kv, page, d, device=DEV).to(BF)
        vc = torch.randn_like(kc)
        pt = torch.arange(n_pages, dtype=torch.int32, device=DEV).view(1, n_pages).contiguous()
        q = torch.randn(tokens, n_heads, d, device=DEV).to(BF)
        slot = torch.zeros(tokens, dtype=torch.int32, device=DEV)
        pos = torch.arange(tokens, dtype=torch.int32, device=DEV)
        out = torch.empty(tokens, n_heads * d, device=DEV, dtype=BF)
        flops = 4 * n_heads * d * tokens * (tokens + 1) / 2
        for name, fn, tile in (("mma.sync", K.attn_prefill, 64), ("tcgen05", K.attn_prefill_tc, 128)):
            nt = (tokens + tile - 1) // tile
            t0 = torch.arange(nt - 1, -1, -1, dtype=torch.int32, device=DEV) * tile   # longest tiles first
            rows = torch.minimum(torch.full_like(t0, tile), tokens - t0).to(torch.int32)
            us = _time(lambda: fn(q, kc, vc, pt, t0, rows, slot, pos, out, nt, 0.088, None), 20)
            print(f"attention, {tokens} tokens, {name:8s} ({tile}-row tiles): {us:8.1f} us  {flops / us / 1e6:6.0f} TFLOP/s", flush=True)
    K.check_error_flags()


def decode_chain(layers: int = 36, small_rows=(1, 8, 16), stream_rows=(32, 64)) -> None:
    hidden, q_dim, inter = 2560, 4096, 9728
    w_qkv = (torch.randn(layers, 6144, hidden, device=DEV) * 0.02).to(BF)
    w_o = (torch.randn(layers, hidden, q_dim, device=DEV) * 0.02).to(BF)
    w_gu = (torch.randn(layers, 2 * inter, hidden, device=DEV) * 0.02).to(BF)
    w_d = (torch.randn(layers, hidden, inter, device=DEV) * 0.02).to(BF)
    nw = torch.ones(hidden, device=DEV)
    weight_bytes = (6144 * hidden + hidden * q_dim + 2 * inter * hidden + hidden * inter) * 2

    def run(which: str, m: int) -> None:
        x = torch.randn(m, hidden, device=DEV).to(BF)
        qkv = torch.empty(m, 6144, device=DEV, dtype=BF)
        act = torch.empty(m, inter, device=DEV, dtype=BF)
        o = torch.randn(m, q_dim, device=DEV).to(BF)
        if which == "gemm_stream":
            f, p1, p2 = K.gemm_stream, K.gemm_stream_ss_parts(hidden, q_dim), K.gemm_stream_ss_parts(hidden, inter)
        else:
            f, p1, p2 = K.gemm_small_m, K.small_m_ss_parts(hidden, q_dim), K.small_m_ss_parts(hidden, inter)
        ss0 = torch.zeros(64, device=DEV)
        K.row_sumsq(x, ss0)
        ss1, ss2 = torch.zeros(p1 * 64, device=DEV), torch.zeros(p2 * 64, device=DEV)

        def layer(i: int) -> None:
            first = i == 0
            f(x, w_qkv[i], qkv, norm_w=nw, ss_in=ss0 if first else ss2, ss_parts=1 if first else p2, eps=1e-6, pdl=True)
            f(o, w_o[i], x, mode="residual", ss_out=ss1, pdl=True)
            f(x, w_gu[i], act, mode="silu", norm_w=nw, ss_in=ss1, ss_parts=p1, eps=1e-6, pdl=True)
            f(act, w_d[i], x, mode="residual", ss_out=ss2, pdl=True)

        for i in range(layers):
            layer(i)
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for i in range(layers):
                layer(i)
        us = _time(g.replay, 5) / layers
        print(f"{which:12s} M={m:2d}: {us:7.2f} us/layer  {weight_bytes / us / 1e6:5.2f} TB/s", flush=True)

    for m in small_rows:
        run("gemm_small_m", m)
        run("gemm_stream", m)
    for m in stream_rows:
        run("gemm_stream", m)
    K.check_error_flags()


def decode_products(layers: int = 36, rows=(8, 16, 64)) -> None:
    """Microseconds per product, each product alone (its ``layers`` weights one after the other in a CUDA graph)."""
    shapes = {"qkv": (6144, 2560, "store", True), "o_proj": (2560, 4096, "residual", False),
              "gate|up": (9728, 2560, "silu", True), "down": (2560, 9728, "residual", False)}

    def graph_us(fn) -> float:
        fn()
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            fn()
        return _time(g.replay, 5) / layers

    for m in rows:
        for name, (n, k, mode, norm) in shapes.items():
            n_rows = 2 * n if mode == "silu" else n
            ws = [(torch.randn(n_rows, k, device=DEV) * 0.02).to(BF) for _ in range(layers)]
            x = torch.randn(m, k, device=DEV).to(BF)
            nw = torch.ones(k, device=DEV)
            ss = torch.zeros(64, device=DEV)
            K.row_sumsq(x, ss)
            out = torch.zeros(m, n, device=DEV, dtype=BF)
            ss_stream = torch.zeros(K.gemm_stream_ss_parts(n, k) * 64, device=DEV)
            ss_small = torch.zeros(K.small_m_ss_parts(n, k) * 64, device=DEV)

            def fused(f, ss_out):
                for w in ws:
                    if norm:
                        f(x, w, out, mode=mode, norm_w=nw, ss_in=ss, ss_parts=1, eps=1e-6, pdl=True)
                    else:
                        f(x, w, out, mode=mode, ss_out=ss_out, pdl=True)

            res = {"gemm_stream": graph_us(lambda: fused(K.gemm_stream, ss_stream)),
                   "gemm_stream, plain store": graph_us(lambda: [K.gemm_stream(x, w[:n], out, pdl=True) for w in ws]),
                   "torch.mm": graph_us(lambda: [torch.mm(x, w.t()) for w in ws])}
            if m <= K.SMALL_M_LIMIT:
                res["gemm_small_m"] = graph_us(lambda: fused(K.gemm_small_m, ss_small))
            mb = n_rows * k * 2 / 1e6
            print(f"M={m:3d} {name:8s} {mb:6.1f} MB | " + " | ".join(f"{a} {b:6.1f} us" for a, b in res.items()), flush=True)
            del ws
    K.check_error_flags()


def main(argv) -> int:
    what = {"attn-prefill": attn_prefill, "decode-chain": decode_chain, "decode-products": decode_products}
    if len(argv) != 2 or argv[1] not in what:
        print("usage: python -m dryft_b200.ops.microbench " + "|".join(what), file=sys.stderr)
        return 2
    with torch.no_grad():
        what[argv[1]]()
    return 0


if __name__ == "__main__":
    sys.exit(main(sys.argv))
