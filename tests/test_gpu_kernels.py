"""Each CUDA kernel alone against a plain PyTorch 32-bit reference of the same operation, at sizes
other than the tiny models': widths that are no power of two, odd row counts, head sizes 16..256,
several group sizes, vocabularies that are prime.  Outputs are surrounded by canary values where a
kernel could write out of its place (the reference's own self-tests check "nothing else in the cache
was touched", ``engine/dryft_qwen3/kernels/rope_qknorm.py:199-202,225-227``)."""

import math

import pytest
import torch

import plain_qwen3 as P

pytestmark = pytest.mark.gpu

DEV = "cuda"


def K():
    from dryft_b200.ops import kernels

    return kernels


def _r(x, dtype):
    return x.to(dtype).to(torch.float32)


def _tol(dtype):
    # one bf16 rounding of the result (2^-8 relative) plus accumulation-order noise; fp32: a few ulps
    return (2e-2, 2e-2) if dtype == torch.bfloat16 else (2e-5, 2e-5)


# bfloat16 attention outputs: two bfloat16 ulps of the result (its own rounding, and the rounding of P before
# the second product, kernels/attn_decode.py:12-14,89) plus an absolute term for outputs near zero: a constant
# here, the analytic bound of P's rounding (`_assert_bf16_attention`) where a test has hundreds of thousands of
# outputs and the tail of that rounding (3.1e-3 to 3.5e-3 in 4 of 300 draws) would cross a constant 3e-3.  One key dropped among a hundred moves
# an output by about 1e-2: outside.  (tests/test_gpu_attention_keys.py has the tests no single key can pass.)
ATTN_BF16_TOL = dict(rtol=2.0 ** -7, atol=3e-3)


# ------------------------------------------------------------------------------------ metadata
def test_step_meta_and_advance():
    k = K()
    cu = torch.tensor([0, 3, 4, 9], dtype=torch.int32, device=DEV)
    slot = torch.tensor([5, -1, 2], dtype=torch.int32, device=DEV)
    seq_len = torch.tensor([0, 0, 7, 0, 0, 100, 0, 0], dtype=torch.int32, device=DEV)
    n = 12  # 3 padding tokens beyond cu[-1]
    ts = torch.full((n,), 77, dtype=torch.int32, device=DEV)
    tp = torch.full((n,), 77, dtype=torch.int32, device=DEV)
    k.step_meta(cu, slot, seq_len, ts, tp, n, 3)
    assert ts.tolist() == [5, 5, 5, -1, 2, 2, 2, 2, 2, -1, -1, -1]
    assert tp.tolist() == [100, 101, 102, 0, 7, 8, 9, 10, 11, 0, 0, 0]
    k.step_advance(cu, slot, seq_len, 3)
    assert seq_len.tolist() == [0, 0, 12, 0, 0, 103, 0, 0]


# ------------------------------------------------------------------------------------ embedding
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("hidden", [80, 2560, 36])
def test_embed(dtype, hidden):
    k = K()
    vocab = 331
    table = torch.randn(vocab, hidden, device=DEV).to(dtype)
    toks = torch.tensor([0, 330, 17, 17, 5], dtype=torch.int32, device=DEV)
    out = torch.full((5, hidden), 9.0, device=DEV).to(dtype)
    err = torch.zeros(1, dtype=torch.int32, device=DEV)
    k.embed(toks, table, out, err)
    assert torch.equal(out, table[toks.long()])
    assert err.item() == 0
    bad = torch.tensor([3, vocab, -1], dtype=torch.int32, device=DEV)
    out3 = torch.full((3, hidden), 9.0, device=DEV).to(dtype)
    k.embed(bad, table, out3, err)
    assert err.item() == 1 and torch.equal(out3[0], table[3]) and out3[1:].abs().max().item() == 0


# ------------------------------------------------------------------------------------ norms
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rows,hidden,eps", [(1, 80, 1e-5), (7, 2560, 1e-6), (33, 200, 3e-6), (3, 13000, 1e-6),
                                             (300, 2560, 1e-6), (257, 72, 1e-5), (260, 5128, 1e-6)])
def test_rmsnorm_plain_add_gather(dtype, rows, hidden, eps):
    k = K()
    x = (torch.randn(rows, hidden, device=DEV) * 3).to(dtype)
    d = torch.randn(rows, hidden, device=DEV).to(dtype)
    w = (1 + 0.1 * torch.randn(hidden, device=DEV)).to(dtype).float()
    rt, at = _tol(dtype)
    # plain
    out = torch.empty_like(x)
    k.rmsnorm(x, w, eps, out)
    ref = P.rmsnorm(x.cpu(), w.cpu(), eps)
    torch.testing.assert_close(out.cpu().float(), ref.float(), rtol=rt, atol=at)
    # fused residual add: x updated in place, exactly the rounded 32-bit sum
    x2 = x.clone()
    k.rmsnorm(x2, w, eps, out, delta=d, x_out=x2)
    s = P.residual_add(x.cpu(), d.cpu())
    assert torch.equal(x2.cpu(), s)
    torch.testing.assert_close(out.cpu().float(), P.rmsnorm(s, w.cpu(), eps).float(), rtol=rt, atol=at)
    # gathered rows, input untouched
    idx = torch.tensor([rows - 1, 0, rows // 2], dtype=torch.int32, device=DEV)
    x3 = x.clone()
    outg = torch.empty(3, hidden, device=DEV, dtype=dtype)
    k.rmsnorm(x3, w, eps, outg, delta=d, rows=idx)
    assert torch.equal(x3, x)
    torch.testing.assert_close(outg.cpu().float(), P.rmsnorm(s[idx.cpu().long()], w.cpu(), eps).float(), rtol=rt, atol=at)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rows,inter", [(1, 224), (5, 9728), (19, 177)])
def test_silu_mul(dtype, rows, inter):
    k = K()
    gu = (torch.randn(rows, 2 * inter, device=DEV) * 4).to(dtype)
    out = torch.empty(rows, inter, device=DEV, dtype=dtype)
    k.silu_mul(gu, out)
    ref = P.silu_mul(gu[:, :inter].cpu(), gu[:, inter:].cpu())
    rt, at = _tol(dtype)
    torch.testing.assert_close(out.cpu().float(), ref.float(), rtol=rt, atol=at)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_residual_add(dtype):
    k = K()
    x = torch.randn(7, 333, device=DEV).to(dtype)
    d = torch.randn(7, 333, device=DEV).to(dtype)
    ref = P.residual_add(x.cpu(), d.cpu())
    k.residual_add(x, d)
    assert torch.equal(x.cpu(), ref)


# ------------------------------------------------------------------------------------ matrix products
@pytest.mark.parametrize("m,n,k_", [(1, 1, 1), (5, 67, 33), (64, 64, 16), (130, 257, 100), (3, 384, 80)])
def test_gemm_f32(m, n, k_):
    k = K()
    a = torch.randn(m, k_, device=DEV)
    w = torch.randn(n, k_, device=DEV)
    out = torch.full((m, n), 7.0, device=DEV)
    k.gemm_nt_f32(a, w, out)
    ref = (a.double() @ w.double().T).float()
    torch.testing.assert_close(out, ref, rtol=1e-5, atol=1e-5 * math.sqrt(k_))
    # a row's result does not depend on the other rows in the batch: bit-identical
    out1 = torch.empty(1, n, device=DEV)
    k.gemm_nt_f32(a[m - 1:m].contiguous(), w, out1)
    assert torch.equal(out1[0], out[m - 1])


@pytest.mark.parametrize("m", [1, 3, 8, 9, 16])
@pytest.mark.parametrize("n,k_", [(2560, 2560), (331, 96), (19, 4096), (6144, 1008), (48, 16), (160, 9728), (100, 256), (333, 1024),
                                  (4750, 4096)])   # the last: tiles for every SM twice over, so 16 warps share a tile
@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
def test_gemm_small_m(m, n, k_, out_dtype):
    k = K()
    a = torch.randn(m, k_, device=DEV).to(torch.bfloat16)
    w = (torch.randn(n, k_, device=DEV) / math.sqrt(k_)).to(torch.bfloat16)
    out = torch.full((m, n), 5.0, device=DEV, dtype=out_dtype)
    k.gemm_small_m(a, w, out)
    ref = a.double() @ w.double().T
    tol = 1e-2 if out_dtype == torch.bfloat16 else 1e-4
    torch.testing.assert_close(out.double(), ref, rtol=tol, atol=tol)
    # independent of the batch: row 0 alone gives the same bits
    out1 = torch.empty(1, n, device=DEV, dtype=out_dtype)
    k.gemm_small_m(a[:1].contiguous(), w, out1)
    assert torch.equal(out1[0], out[0])


@pytest.mark.parametrize("m", [1, 5, 8, 13, 16])   # 5 and 13: a row of zeros stands for the rest of the 8 / 16-row operand
@pytest.mark.parametrize("n,k_", [(2560, 2560), (96, 176), (200, 1008), (4096, 1024), (208, 256), (1000, 512), (320, 5120), (4736, 4096)])   # 5,120: one block an SM; 4,736 x 4,096: 16 warps a tile
def test_gemm_small_m_fused_norm_residual_silu(m, n, k_):
    """The fused forms of the decode product against the plain parts: RMSNorm of the input from
    sums of squares left by an earlier product, residual add with new sums of squares, SiLU*mul."""
    k = K()
    bf = torch.bfloat16
    eps = 1e-5
    x = (torch.randn(m, k_, device=DEV) * 2).to(bf)
    nw = (1 + 0.1 * torch.randn(k_, device=DEV)).to(bf).float()
    w = (torch.randn(n, k_, device=DEV) / math.sqrt(k_)).to(bf)
    ss = torch.zeros(64, device=DEV)
    k.row_sumsq(x, ss)
    torch.testing.assert_close(ss[:m].cpu(), x.float().pow(2).sum(-1).cpu(), rtol=1e-5, atol=1e-5)
    h_ref = P.rmsnorm(x.cpu(), nw.cpu(), eps)
    # norm prologue + plain store
    out = torch.empty(m, n, device=DEV, dtype=bf)
    k.gemm_small_m(x, w, out, norm_w=nw, ss_in=ss, ss_parts=1, eps=eps)
    ref = h_ref.double() @ w.cpu().double().T
    torch.testing.assert_close(out.cpu().double(), ref, rtol=2e-2, atol=2e-2)
    # a row's bits do not depend on how many rows there are, up to 8 and from 9 to 16 (the kernel's form is
    # chosen by the sizes of the product and by that class, never by M)
    if m in (8, 16):
        sub = 1 if m == 8 else 9
        ss_sub = torch.zeros(64, device=DEV)
        k.row_sumsq(x[:sub].contiguous(), ss_sub)
        out_sub = torch.empty(sub, n, device=DEV, dtype=bf)
        k.gemm_small_m(x[:sub].contiguous(), w, out_sub, norm_w=nw, ss_in=ss_sub, ss_parts=1, eps=eps)
        assert torch.equal(out_sub, out[:sub])
    # residual epilogue with sums of squares for the next norm
    res = torch.randn(m, n, device=DEV).to(bf)
    res0 = res.clone()
    parts = k.small_m_ss_parts(n, k_)
    ss_out = torch.full((parts * 64,), -1.0, device=DEV)
    k.gemm_small_m(x, w, res, mode="residual", ss_out=ss_out)
    prod = P.matmul_nt(x.cpu(), w.cpu(), bf)
    want = P.residual_add(res0.cpu(), prod)
    torch.testing.assert_close(res.cpu().float(), want.float(), rtol=2e-2, atol=2e-2)
    got_ss = ss_out.view(parts, 64)[:, :m].sum(0).cpu()
    torch.testing.assert_close(got_ss, res.float().pow(2).sum(-1).cpu(), rtol=1e-4, atol=1e-4)
    # the sums chain: a second product normalises the new stream from them
    if n % 16 == 0:
        w2 = (torch.randn(48, n, device=DEV) / math.sqrt(n)).to(bf)
        nw2 = (1 + 0.1 * torch.randn(n, device=DEV)).to(bf).float()
        out2 = torch.empty(m, 48, device=DEV, dtype=torch.float32)
        k.gemm_small_m(res, w2, out2, norm_w=nw2, ss_in=ss_out, ss_parts=parts, eps=eps)
        ref2 = P.rmsnorm(res.cpu(), nw2.cpu(), eps).double() @ w2.cpu().double().T
        torch.testing.assert_close(out2.cpu().double(), ref2, rtol=2e-2, atol=2e-2)
    # the norm split over two launches: the residual product leaves the new stream weighted for the next
    # norm, and a second product scales its sums by the norm's factor instead of normalising its input
    if k.weighted_ahead_supported(k_) and k.weighted_ahead_supported(n):
        res3 = res0.clone()
        nw2 = (1 + 0.1 * torch.randn(n, device=DEV)).to(bf).float()
        xw = torch.full((m, n), 7.0, device=DEV, dtype=bf)
        ss3 = torch.full((parts * 64,), -1.0, device=DEV)
        k.gemm_small_m(x, w, res3, mode="residual", ss_out=ss3, next_w=nw2, xw_out=xw)
        assert torch.equal(res3, res)
        assert torch.equal(xw.cpu(), (res.float().cpu() * nw2.cpu()).to(bf))
        w2 = (torch.randn(48, n, device=DEV) / math.sqrt(n)).to(bf)
        out3 = torch.empty(m, 48, device=DEV, dtype=torch.float32)
        k.gemm_small_m(res, w2, out3, xw_in=xw, norm_w=nw2, ss_in=ss3, ss_parts=parts, eps=eps)   # norm_w: for sizes the split form refuses
        ref3 = P.rmsnorm(res.cpu(), nw2.cpu(), eps).double() @ w2.cpu().double().T
        torch.testing.assert_close(out3.cpu().double(), ref3, rtol=2e-2, atol=2e-2)
        act3 = torch.empty(m, 24, device=DEV, dtype=bf)
        k.gemm_small_m(res, w2, act3, mode="silu", xw_in=xw, norm_w=nw2, ss_in=ss3, ss_parts=parts, eps=eps)
        gu3 = P.matmul_nt(P.rmsnorm(res.cpu(), nw2.cpu(), eps), w2.cpu(), bf)
        torch.testing.assert_close(act3.cpu().float(), P.silu_mul(gu3[:, :24], gu3[:, 24:]).float(), rtol=3e-2, atol=3e-2)
    # SiLU*mul epilogue over gate rows then up rows
    inter = n // 2
    act = torch.empty(m, inter, device=DEV, dtype=bf)
    k.gemm_small_m(x, w[: 2 * inter], act, mode="silu")
    gu = P.matmul_nt(x.cpu(), w[: 2 * inter].cpu(), bf)
    want = P.silu_mul(gu[:, :inter], gu[:, inter:])
    torch.testing.assert_close(act.cpu().float(), want.float(), rtol=3e-2, atol=3e-2)


@pytest.mark.parametrize("m", [1, 8, 13, 40, 64])
@pytest.mark.parametrize("n,k_", [(2560, 2560), (6144, 2560), (2560, 9728), (1000, 192), (200, 128), (19456, 256)])
def test_gemm_stream(m, n, k_):
    """The weight-streaming decode product (tcgen05, a TMA ring, the work cut evenly over the SMs, shared tiles
    summed in block order through tickets) against the plain parts, in every form: store (bfloat16 and 32-bit),
    norm on the way in from sums of squares, residual add leaving new sums of squares that a second product
    normalises from, SiLU*mul with and without a norm; 1..64 rows; output counts that are no multiple of the
    128-row tile; few tiles cut into many pieces (2,560 outputs over 9,728 inputs) and many tiles with few
    pieces.  Launches repeat bit for bit and leave the ticket counters at zero."""
    k = K()
    bf = torch.bfloat16
    eps = 1e-5
    x = (torch.randn(m, k_, device=DEV) * 2).to(bf)
    nw = (1 + 0.1 * torch.randn(k_, device=DEV)).to(bf).float()
    w = (torch.randn(n, k_, device=DEV) / math.sqrt(k_)).to(bf)
    # plain store, both output types; a row's result does not depend on the other rows
    out = torch.empty(m, n, device=DEV, dtype=bf)
    k.gemm_stream(x, w, out)
    ref = x.cpu().double() @ w.cpu().double().T
    torch.testing.assert_close(out.cpu().double(), ref, rtol=2e-2, atol=2e-2)
    out32 = torch.empty(m, n, device=DEV, dtype=torch.float32)
    k.gemm_stream(x, w, out32)
    torch.testing.assert_close(out32.cpu().double(), ref, rtol=1e-3, atol=1e-3)
    one = torch.empty(1, n, device=DEV, dtype=torch.float32)
    k.gemm_stream(x[m - 1:].contiguous(), w, one)
    assert torch.equal(one[0], out32[m - 1])
    # norm prologue
    ss = torch.zeros(64, device=DEV)
    k.row_sumsq(x, ss)
    h_ref = P.rmsnorm(x.cpu(), nw.cpu(), eps)
    k.gemm_stream(x, w, out, norm_w=nw, ss_in=ss, ss_parts=1, eps=eps)
    torch.testing.assert_close(out.cpu().double(), h_ref.double() @ w.cpu().double().T, rtol=2e-2, atol=2e-2)
    # residual epilogue with sums of squares, chained into a second normalised product
    res = torch.randn(m, n, device=DEV).to(bf)
    res0 = res.clone()
    parts = k.gemm_stream_ss_parts(n, k_)
    ss_out = torch.full((parts * 64,), -1.0, device=DEV)
    k.gemm_stream(x, w, res, mode="residual", ss_out=ss_out)
    want = P.residual_add(res0.cpu(), P.matmul_nt(x.cpu(), w.cpu(), bf))
    torch.testing.assert_close(res.cpu().float(), want.float(), rtol=2e-2, atol=2e-2)
    got_ss = ss_out.view(parts, 64)[:, :m].sum(0).cpu()
    torch.testing.assert_close(got_ss, res.float().pow(2).sum(-1).cpu(), rtol=1e-4, atol=1e-4)
    if n % 64 == 0:
        w2 = (torch.randn(48, n, device=DEV) / math.sqrt(n)).to(bf)
        nw2 = (1 + 0.1 * torch.randn(n, device=DEV)).to(bf).float()
        out2 = torch.empty(m, 48, device=DEV, dtype=torch.float32)
        k.gemm_stream(res, w2, out2, norm_w=nw2, ss_in=ss_out, ss_parts=parts, eps=eps)
        ref2 = P.rmsnorm(res.cpu(), nw2.cpu(), eps).double() @ w2.cpu().double().T
        torch.testing.assert_close(out2.cpu().double(), ref2, rtol=2e-2, atol=2e-2)
    # SiLU*mul over gate rows then up rows, plain and with the norm on the way in
    inter = n // 2
    act = torch.empty(m, inter, device=DEV, dtype=bf)
    k.gemm_stream(x, w[: 2 * inter], act, mode="silu")
    gu = P.matmul_nt(x.cpu(), w[: 2 * inter].cpu(), bf)
    torch.testing.assert_close(act.cpu().float(), P.silu_mul(gu[:, :inter], gu[:, inter:]).float(), rtol=3e-2, atol=3e-2)
    act_n = torch.empty(m, inter, device=DEV, dtype=bf)
    k.gemm_stream(x, w[: 2 * inter], act_n, mode="silu", norm_w=nw, ss_in=ss, ss_parts=1, eps=eps)
    gu = P.matmul_nt(h_ref, w[: 2 * inter].cpu(), bf)
    torch.testing.assert_close(act_n.cpu().float(), P.silu_mul(gu[:, :inter], gu[:, inter:]).float(), rtol=3e-2, atol=3e-2)
    # the same launches again: the same bits (pieces are added in block order, whoever finishes last), tickets at zero
    again = torch.empty_like(out32)
    k.gemm_stream(x, w, again)
    assert torch.equal(again, out32)
    res2 = res0.clone()
    ss2 = torch.full((parts * 64,), -1.0, device=DEV)
    k.gemm_stream(x, w, res2, mode="residual", ss_out=ss2)
    assert torch.equal(res2, res) and torch.equal(ss2.view(parts, 64)[:, :m], ss_out.view(parts, 64)[:, :m])
    torch.cuda.synchronize()
    assert int(k.gemm_stream_scratch(torch.device(DEV, 0))[1].abs().sum()) == 0
    k.check_error_flags()


def test_gemm_small_m_refuses_odd_k():
    k = K()
    a = torch.zeros(2, 12, device=DEV, dtype=torch.bfloat16)
    w = torch.zeros(4, 12, device=DEV, dtype=torch.bfloat16)
    with pytest.raises(k.KernelError):
        k.gemm_small_m(a, w, torch.empty(2, 4, device=DEV, dtype=torch.bfloat16))
    a = torch.zeros(17, 32, device=DEV, dtype=torch.bfloat16)  # more rows than the kernel takes
    w = torch.zeros(4, 32, device=DEV, dtype=torch.bfloat16)
    with pytest.raises(k.KernelError):
        k.gemm_small_m(a, w, torch.empty(17, 4, device=DEV, dtype=torch.bfloat16))
    k.check_error_flags()


# ------------------------------------------------------------------------------------ rope + cache write
def _paged_cache(n_pages, n_kv, page, d, dtype, fill=0.0):
    kc = torch.full((n_pages, n_kv, page, d), fill, device=DEV).to(dtype)
    return kc, kc.clone()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("with_table", [False, True])
@pytest.mark.parametrize("n_heads,n_kv,d,rot,theta,eps", [(4, 2, 16, 16, 1e4, 1e-6), (6, 2, 48, 48, 5e5, 1e-5),
                                                            (8, 8, 128, 128, 5e6, 1e-6), (3, 1, 64, 32, 1e4, 1e-6),
                                                            (2, 1, 24, 18, 1e4, 1e-6), (3, 1, 256, 256, 1e6, 1e-6),
                                                            (6, 3, 32, 32, 1e6, 1e-5), (5, 1, 64, 64, 1e4, 1e-6),
                                                            (32, 8, 128, 128, 5e6, 1e-6)])
def test_qk_norm_rope_store(dtype, with_table, n_heads, n_kv, d, rot, theta, eps):
    """With the step's cos / sin table and with angles evaluated in the kernel: same result."""
    k = K()
    page, n_pages, max_pages, slots = 64, 9, 4, 3
    # tokens of two sequences at scattered positions (page boundaries 63/64, a far position)
    tok_slot = torch.tensor([2, 2, 2, 0, 0, -1], dtype=torch.int32, device=DEV)
    tok_pos = torch.tensor([62, 63, 64, 0, 200, 0], dtype=torch.int32, device=DEV)
    n = 6
    pt = torch.zeros(slots, max_pages, dtype=torch.int32, device=DEV)
    pt[2, 0], pt[2, 1], pt[0, 0], pt[0, 3] = 7, 3, 5, 1
    width = (n_heads + 2 * n_kv) * d
    qkv = (torch.randn(n, width, device=DEV) * 2).to(dtype)
    wq = (1 + 0.1 * torch.randn(d, device=DEV)).to(dtype).float()
    wk = (1 + 0.1 * torch.randn(d, device=DEV)).to(dtype).float()
    inv_freq = (1.0 / (theta ** (torch.arange(0, rot, 2, dtype=torch.int64).float() / rot))).to(DEV)
    canary = 123.0
    kc, vc = _paged_cache(n_pages, n_kv, page, d, dtype, canary)
    q_out = torch.full((n, n_heads, d), canary, device=DEV).to(dtype)
    table = k.rope_table(tok_pos, inv_freq, n, dtype) if with_table else None
    k.qk_norm_rope_store(qkv, wq, wk, inv_freq, tok_slot, tok_pos, q_out, kc, vc, pt, n_heads, n_kv, d, rot, eps,
                         cs_table=table)

    # plain reference
    qc = qkv.cpu()
    q = qc[:, :n_heads * d].view(n, n_heads, d)
    kk = qc[:, n_heads * d:(n_heads + n_kv) * d].view(n, n_kv, d)
    vv = qc[:, (n_heads + n_kv) * d:].view(n, n_kv, d)
    qn = P.rmsnorm(q, wq.cpu(), eps)
    kn = P.rmsnorm(kk, wk.cpu(), eps)
    cos, sin = P.rope_cos_sin(tok_pos.cpu(), rot, theta, dtype)

    def rot_part(x):
        return torch.cat((P.apply_rope(x[..., :rot], cos, sin), x[..., rot:]), dim=-1)

    q_ref, k_ref = rot_part(qn), rot_part(kn)
    rt, at = _tol(dtype)
    live = [0, 1, 2, 3, 4]
    torch.testing.assert_close(q_out[live].cpu().float(), q_ref[live].float(), rtol=rt, atol=at)
    assert q_out[5].abs().max().item() == 0  # padding token: zero query
    touched = torch.zeros(n_pages, n_kv, page, dtype=torch.bool)
    for i in live:
        s, p = int(tok_slot[i]), int(tok_pos[i])
        pg = int(pt[s, p // page])
        torch.testing.assert_close(kc[pg, :, p % page].cpu().float(), k_ref[i].float(), rtol=rt, atol=at)
        assert torch.equal(vc[pg, :, p % page].cpu(), vv[i])
        touched[pg, :, p % page] = True
    # nothing else in the cache was written
    assert (kc.cpu().float()[~touched] == canary).all() and (vc.cpu().float()[~touched] == canary).all()


# ------------------------------------------------------------------------------------ attention
def _fill_cache(seqs, n_kv, d, page, dtype, n_pages, max_pages, slots, scatter_seed=0):
    """Put each sequence's keys/values into randomly chosen pages; returns caches, page table."""
    g = torch.Generator().manual_seed(scatter_seed)
    perm = torch.randperm(n_pages, generator=g).tolist()
    kc, vc = _paged_cache(n_pages, n_kv, page, d, dtype, 0.0)
    pt = torch.zeros(slots, max_pages, dtype=torch.int32, device=DEV)
    for slot, (kseq, vseq) in seqs.items():
        L = kseq.shape[0]
        for lp in range((L + page - 1) // page):
            pp = perm.pop()
            pt[slot, lp] = pp
            n = min(page, L - lp * page)
            kc[pp, :, :n] = kseq[lp * page:lp * page + n].transpose(0, 1).to(DEV)
            vc[pp, :, :n] = vseq[lp * page:lp * page + n].transpose(0, 1).to(DEV)
    return kc, vc, pt


def _attn_ref(q, kseq, vseq, pos, scale, window, p_round=None):
    """q [nH, D] at position pos over keys 0..pos of one sequence (32-bit).  ``p_round``: the probabilities go
    into the second product rounded to this type, as the bfloat16 kernels round them (relative to the row's
    maximum, before the division by the 32-bit sum; kernels/attn_decode.py:12-14,89).  Where a row's keys fit one
    block of the kernel the roundings then coincide; a 32-bit P would differ from the kernel by up to
    2^-9 * sum(p |v|), about 3e-3 for a row of three keys with values near 3."""
    nH, D = q.shape
    nKV = kseq.shape[1]
    G = nH // nKV
    lo = max(0, pos + 1 - window) if window else 0
    kf = kseq[lo:pos + 1].float()
    vf = vseq[lo:pos + 1].float()
    qf = q.float().view(nKV, G, D)
    sc = torch.einsum("hgd,nhd->hgn", qf, kf) * scale
    if p_round is None:
        p = torch.softmax(sc, dim=-1)
        return torch.einsum("hgn,nhd->hgd", p, vf).reshape(nH * D)
    e = torch.exp(sc - sc.max(dim=-1, keepdim=True).values)
    num = torch.einsum("hgn,nhd->hgd", e.to(p_round).float(), vf)
    return (num / e.sum(dim=-1, keepdim=True)).reshape(nH * D)


def _p_rounding_bound(q, kseq, vseq, pos, scale, window):
    """sum_i p_i |v_i| per output: a probability rounded to bfloat16 is off by at most 2^-9 of itself, so this
    times 2^-9 bounds what that rounding moves an output by -- twice that between two evaluations that round at
    different maxima (a kernel that walks the keys in blocks, and the reference above)."""
    nH, D = q.shape
    nKV = kseq.shape[1]
    G = nH // nKV
    lo = max(0, pos + 1 - window) if window else 0
    sc = torch.einsum("hgd,nhd->hgn", q.float().view(nKV, G, D), kseq[lo:pos + 1].float()) * scale
    return torch.einsum("hgn,nhd->hgd", torch.softmax(sc, dim=-1), vseq[lo:pos + 1].float().abs()).reshape(nH * D)


def _assert_bf16_attention(out, ref, bound, what=""):
    """Two bfloat16 ulps of the result (its own rounding and accumulation order) plus the bound of P's rounding."""
    err = (out - ref).abs()
    allowed = ATTN_BF16_TOL["rtol"] * ref.abs() + 2.0 ** -8 * bound + 5e-4
    worst = (err - allowed).max()
    assert worst <= 0, f"{what}: off by {float(err.flatten()[(err - allowed).argmax()]):.3g} where {float(allowed.flatten()[(err - allowed).argmax()]):.3g} is allowed"


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("n_heads,n_kv,d", [(4, 2, 16), (6, 2, 48), (8, 2, 128), (5, 5, 64), (16, 1, 32), (2, 1, 256)])
@pytest.mark.parametrize("window", [None, 70])
def test_attn_rows(dtype, n_heads, n_kv, d, window):
    k = K()
    page = 64
    lens = {0: 1, 1: 63, 2: 64, 3: 65, 4: 300}
    seqs = {s: ((torch.randn(L, n_kv, d)).to(dtype), torch.randn(L, n_kv, d).to(dtype)) for s, L in lens.items()}
    kc, vc, pt = _fill_cache(seqs, n_kv, d, page, dtype, n_pages=16, max_pages=6, slots=6)
    # rows: the last position of every sequence, a middle position, and a padding row
    rows = [(0, 0), (1, 62), (2, 63), (3, 64), (4, 299), (4, 150), (-1, 0), (4, 64)]
    tok_slot = torch.tensor([r[0] for r in rows], dtype=torch.int32, device=DEV)
    tok_pos = torch.tensor([r[1] for r in rows], dtype=torch.int32, device=DEV)
    n = len(rows)
    q = torch.randn(n, n_heads, d).to(dtype)
    scale = 1.0 / math.sqrt(d)
    ref = torch.stack([
        _attn_ref(q[i], seqs[s][0], seqs[s][1], p, scale, window) if s >= 0 else torch.zeros(n_heads * d)
        for i, (s, p) in enumerate(rows)])
    rt, at = (ATTN_BF16_TOL["rtol"], ATTN_BF16_TOL["atol"]) if dtype == torch.bfloat16 else _tol(dtype)
    for splits in (1, 3, 8):
        out = torch.full((n, n_heads * d), 9.0, device=DEV).to(dtype)
        part_o = torch.empty(n, n_heads, splits, d, device=DEV) if splits > 1 else None
        part_ml = torch.empty(n, n_heads, splits, 2, device=DEV) if splits > 1 else None
        k.attn_rows(q.to(DEV), kc, vc, pt, tok_slot, tok_pos, out, scale, window, splits, part_o, part_ml)
        assert torch.isfinite(out.float()).all()
        torch.testing.assert_close(out.cpu().float(), ref, rtol=rt, atol=at)


@pytest.mark.parametrize("n_heads,n_kv,d,rot", [(4, 2, 16, 16), (6, 2, 48, 48), (8, 2, 128, 128), (5, 5, 64, 32), (16, 1, 32, 32),
                                                 (4, 2, 256, 256)])
@pytest.mark.parametrize("window", [None, 70])
def test_attn_decode_fused(n_heads, n_kv, d, rot, window):
    """The one-launch decode attention against the plain parts: q/k norm + RoPE of the new token, its
    K/V written into the cache (and nothing else), attention over old keys plus the new one, for
    every split count and every block shape (8, 4, 2 warps, and the launcher's own choice); tickets are
    left at zero."""
    k = K()
    dtype = torch.bfloat16
    page, theta, eps = 64, 1e4, 1e-5
    scale = 1.0 / math.sqrt(d)
    lens = {0: 0, 1: 63, 2: 64, 3: 200, 4: 129}  # tokens already cached; the new token goes at this position
    seqs = {s: (torch.randn(L + 1, n_kv, d).to(dtype), torch.randn(L + 1, n_kv, d).to(dtype)) for s, L in lens.items()}
    rows = [(0, 0), (1, 63), (-1, 0), (2, 64), (3, 200), (4, 129)]
    n = len(rows)
    width = (n_heads + 2 * n_kv) * d
    qkv = (torch.randn(n, width) * 2).to(dtype)
    wq = (1 + 0.1 * torch.randn(d)).to(dtype).float()
    wk = (1 + 0.1 * torch.randn(d)).to(dtype).float()
    inv_freq = 1.0 / (theta ** (torch.arange(0, rot, 2, dtype=torch.int64).float() / rot))
    # plain: rotate q and the new k, put new k/v at the row's position, attend
    pos_t = torch.tensor([r[1] for r in rows])
    cos, sin = P.rope_cos_sin(pos_t, rot, theta, dtype)
    q = qkv[:, :n_heads * d].view(n, n_heads, d)
    kn = qkv[:, n_heads * d:(n_heads + n_kv) * d].view(n, n_kv, d)
    vn = qkv[:, (n_heads + n_kv) * d:].view(n, n_kv, d)
    rot_part = lambda x: torch.cat((P.apply_rope(x[..., :rot], cos, sin), x[..., rot:]), dim=-1)
    q_r = rot_part(P.rmsnorm(q, wq, eps))
    k_r = rot_part(P.rmsnorm(kn, wk, eps))
    refs = []
    for i, (s, pos) in enumerate(rows):
        if s < 0:
            refs.append(torch.zeros(n_heads * d))
            continue
        kseq, vseq = seqs[s][0].clone(), seqs[s][1].clone()
        kseq[pos], vseq[pos] = k_r[i], vn[i]
        refs.append(_attn_ref(q_r[i], kseq, vseq, pos, scale, window, p_round=torch.bfloat16))
    ref = torch.stack(refs)
    # (splits, block shape, splits combined inside a thread-block cluster or through memory)
    for splits, shape, cluster in ((1, -1, True), (2, 0, True), (7, 1, True), (1, 2, True), (3, 2, False), (5, -1, True),
                                   (8, 2, True), (7, 0, False), (12, 1, True)):
        old = {s: (kv[0][:lens[s]], kv[1][:lens[s]]) for s, kv in seqs.items()}
        # pages for L+1 tokens, only L filled; the rest is a canary the kernel must not touch
        kc, vc, pt = _fill_cache({s: (torch.cat([kv[0], torch.full((1, n_kv, d), 55.0).to(dtype)]),
                                      torch.cat([kv[1], torch.full((1, n_kv, d), 55.0).to(dtype)])) for s, kv in old.items()},
                                 n_kv, d, page, dtype, n_pages=16, max_pages=5, slots=6, scatter_seed=splits + shape + 2 * cluster)
        kc0, vc0 = kc.clone(), vc.clone()
        out = torch.full((n, n_heads * d), 9.0, device=DEV, dtype=dtype)
        po = torch.empty(n, n_heads, splits, d, device=DEV) if splits > 1 else None
        pm = torch.empty(n, n_heads, splits, 2, device=DEV) if splits > 1 else None
        i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
        run = lambda: k.attn_decode(qkv.to(DEV), wq.to(DEV), wk.to(DEV), inv_freq.to(DEV), i32([r[0] for r in rows]),
                                    i32([r[1] for r in rows]), kc, vc, pt, out, n_heads, n_kv, d, rot, eps, scale, window,
                                    splits, po, pm, shape=shape, cluster=cluster)
        if d == 256 and shape == 0:
            with pytest.raises(k.KernelError):   # eight warps' rings of 256-wide rows do not fit an SM: refused, not wrong
                run()
            continue
        run()
        assert torch.isfinite(out.float()).all()
        torch.testing.assert_close(out.cpu().float(), ref, **ATTN_BF16_TOL)
        changed_k = (kc != kc0).any(dim=-1)
        changed_v = (vc != vc0).any(dim=-1)
        assert int(changed_k.sum()) == 5 * n_kv and int(changed_v.sum()) == 5 * n_kv  # one row per live token and kv head
        for i, (s, pos) in enumerate(rows):
            if s < 0:
                continue
            pg = int(pt[s, pos // page])
            torch.testing.assert_close(kc[pg, :, pos % page].cpu().float(), k_r[i].float(), rtol=2e-2, atol=2e-2)
            assert torch.equal(vc[pg, :, pos % page].cpu(), vn[i])
        if splits > 1:
            assert int(k.tickets(torch.device(DEV, 0), 1).abs().sum()) == 0


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_attn_rows_far_key_stands_out(dtype):
    """One key among hundreds is made to dominate (query and that key scaled so its score stands out);
    the output must be that key's value, wherever in the cache the key lies — first page, a page
    boundary, the last position — and whatever the split count."""
    k = K()
    n_heads, n_kv, d, page, L = 4, 2, 32, 64, 700
    scale = 1.0 / math.sqrt(d)
    for target in (0, 63, 64, 333, 639, 640, 699):
        kseq = torch.randn(L, n_kv, d) * 0.1
        vseq = torch.randn(L, n_kv, d)
        q = torch.randn(1, n_heads, d) * 0.1
        direction = torch.randn(d)
        direction /= direction.norm()
        kseq[target] = direction * 30.0
        q[0] = direction * 30.0
        seqs = {1: (kseq.to(dtype), vseq.to(dtype))}
        kc, vc, pt = _fill_cache(seqs, n_kv, d, page, dtype, n_pages=13, max_pages=12, slots=2, scatter_seed=target)
        tok_slot = torch.tensor([1], dtype=torch.int32, device=DEV)
        tok_pos = torch.tensor([L - 1], dtype=torch.int32, device=DEV)
        for splits in (1, 5):
            out = torch.empty(1, n_heads * d, device=DEV, dtype=dtype)
            po = torch.empty(1, n_heads, splits, d, device=DEV) if splits > 1 else None
            pm = torch.empty(1, n_heads, splits, 2, device=DEV) if splits > 1 else None
            k.attn_rows(q.to(dtype).to(DEV), kc, vc, pt, tok_slot, tok_pos, out, scale, None, splits, po, pm)
            want = seqs[1][1][target].float().repeat_interleave(n_heads // n_kv, dim=0).reshape(-1)
            torch.testing.assert_close(out[0].cpu().float(), want, rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("n_heads,n_kv,d", [(4, 2, 16), (6, 2, 48), (8, 2, 128), (3, 3, 64), (2, 1, 256)])
@pytest.mark.parametrize("window", [None, 40])
def test_attn_prefill(n_heads, n_kv, d, window):
    """Packed prompts of unequal lengths, some continuing an earlier chunk, against plain attention."""
    k = K()
    dtype = torch.bfloat16
    page, tile = 64, 64
    scale = 1.0 / math.sqrt(d)
    # (slot, tokens already cached, new tokens of this step)
    plan = [(3, 0, 1), (0, 0, 130), (5, 100, 77), (1, 64, 64), (2, 0, 63)]
    seqs = {}
    for slot, old, new in plan:
        L = old + new
        seqs[slot] = (torch.randn(L, n_kv, d).to(dtype), torch.randn(L, n_kv, d).to(dtype))
    kc, vc, pt = _fill_cache(seqs, n_kv, d, page, dtype, n_pages=20, max_pages=4, slots=6, scatter_seed=3)
    tok_slot, tok_pos, tiles0, tilesn, qs, refs, bounds = [], [], [], [], [], [], []
    base = 0
    for slot, old, new in plan:
        q = torch.randn(new, n_heads, d).to(dtype)
        qs.append(q)
        for i in range(new):
            tok_slot.append(slot)
            tok_pos.append(old + i)
            refs.append(_attn_ref(q[i], seqs[slot][0], seqs[slot][1], old + i, scale, window, p_round=torch.bfloat16))
            bounds.append(_p_rounding_bound(q[i], seqs[slot][0], seqs[slot][1], old + i, scale, window))
        for q0 in range(0, new, tile):
            tiles0.append(base + q0)
            tilesn.append(min(tile, new - q0))
        base += new
    n = base
    q_all = torch.cat(qs).to(DEV)
    out = torch.full((n, n_heads * d), 9.0, device=DEV, dtype=dtype)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    k.attn_prefill(q_all, kc, vc, pt, i32(tiles0), i32(tilesn), i32(tok_slot), i32(tok_pos), out, len(tiles0), scale, window)
    ref = torch.stack(refs)
    assert torch.isfinite(out.float()).all()
    _assert_bf16_attention(out.cpu().float(), ref, torch.stack(bounds), "attn_prefill")


@pytest.mark.parametrize("n_heads,n_kv,d", [(8, 2, 128), (3, 3, 64), (4, 1, 128)])
@pytest.mark.parametrize("window", [None, 40])
def test_attn_prefill_tc(n_heads, n_kv, d, window):
    """The tcgen05 prefill attention against plain attention: packed prompts of unequal lengths, tiles
    of up to 128 tokens, some continuing an earlier chunk."""
    k = K()
    dtype = torch.bfloat16
    page, tile = 64, 128
    scale = 1.0 / math.sqrt(d)
    plan = [(3, 0, 1), (0, 0, 300), (5, 100, 77), (1, 64, 128), (2, 0, 129)]  # (slot, cached, new)
    seqs = {}
    for slot, old, new in plan:
        L = old + new
        seqs[slot] = (torch.randn(L, n_kv, d).to(dtype), torch.randn(L, n_kv, d).to(dtype))
    kc, vc, pt = _fill_cache(seqs, n_kv, d, page, dtype, n_pages=24, max_pages=6, slots=6, scatter_seed=5)
    tok_slot, tok_pos, tiles0, tilesn, qs, refs, bounds = [], [], [], [], [], [], []
    base = 0
    for slot, old, new in plan:
        q = torch.randn(new, n_heads, d).to(dtype)
        qs.append(q)
        for i in range(new):
            tok_slot.append(slot)
            tok_pos.append(old + i)
            refs.append(_attn_ref(q[i], seqs[slot][0], seqs[slot][1], old + i, scale, window, p_round=torch.bfloat16))
            bounds.append(_p_rounding_bound(q[i], seqs[slot][0], seqs[slot][1], old + i, scale, window))
        for q0 in range(0, new, tile):
            tiles0.append(base + q0)
            tilesn.append(min(tile, new - q0))
        base += new
    n = base
    out = torch.full((n, n_heads * d), 9.0, device=DEV, dtype=dtype)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    k.attn_prefill_tc(torch.cat(qs).to(DEV), kc, vc, pt, i32(tiles0), i32(tilesn), i32(tok_slot), i32(tok_pos), out,
                      len(tiles0), scale, window)
    torch.cuda.synchronize()
    k.check_error_flags()
    assert torch.isfinite(out.float()).all()
    _assert_bf16_attention(out.cpu().float(), torch.stack(refs), torch.stack(bounds), "attn_prefill_tc")


@pytest.mark.parametrize("where", ["early", "late", "steps"])
def test_attn_prefill_tc_running_maximum(where):
    """The tcgen05 kernel keeps a running maximum that moves only on large growth and rescales O in tensor
    memory then.  One key that stands out early (no later growth), one that stands out late (O is
    rescaled after hundreds of keys), and key sizes that rise in steps (growth below and above the
    threshold, tile after tile) must all give plain attention's result."""
    k = K()
    dtype = torch.bfloat16
    n_heads, n_kv, d, page, tile = 4, 2, 128, 64, 128
    L = 450
    scale = 1.0 / math.sqrt(d)
    g = torch.Generator().manual_seed(11)
    keys = torch.randn(L, n_kv, d, generator=g)
    vals = torch.randn(L, n_kv, d, generator=g)
    q = torch.randn(L, n_heads, d, generator=g)
    if where == "steps":
        keys *= (0.25 * (1 + torch.arange(L) // 64)).view(L, 1, 1) * 2.0
    else:
        at = 3 if where == "early" else 389
        keys[at] = 0
        keys[at, :, 0] = 24.0
        q[:, :, 0] = 20.0   # score 480 * scale = 42 above the rest at that key
        vals[at] = 5.0
    seqs = {1: (keys.to(dtype), vals.to(dtype))}
    kc, vc, pt = _fill_cache(seqs, n_kv, d, page, dtype, n_pages=12, max_pages=8, slots=2, scatter_seed=3)
    qb = q.to(dtype)
    refs = [_attn_ref(qb[i], seqs[1][0], seqs[1][1], i, scale, None) for i in range(L)]
    tiles0 = list(range(0, L, tile))
    tilesn = [min(tile, L - t) for t in tiles0]
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    out = torch.full((L, n_heads * d), 9.0, device=DEV, dtype=dtype)
    k.attn_prefill_tc(qb.to(DEV), kc, vc, pt, i32(tiles0), i32(tilesn), i32([1] * L), i32(list(range(L))), out,
                      len(tiles0), scale, None)
    torch.cuda.synchronize()
    k.check_error_flags()
    ref = torch.stack(refs)
    if where != "steps":
        at = 3 if where == "early" else 389
        assert (ref[at + 5:, :] - 5.0).abs().max() < 0.05   # the marked key takes all the weight after it
    torch.testing.assert_close(out.cpu().float(), ref, rtol=2e-2, atol=2e-2)


def test_attn_prefill_tc_is_the_same_every_time():
    """Many blocks, many launches, one input, L2 flushed every other launch so that K and V arrive late:
    every launch must give the same bits.  (A block once read its accumulator after a wait that one parity
    bit could not decide -- the P V product of the tile before the last still running -- about one prompt
    step in forty; nothing in the kernel may depend on when its copies and products finish.)"""
    k = K()
    dtype = torch.bfloat16
    n_heads, n_kv, d, page, tile = 16, 4, 128, 64, 128
    scale = 1.0 / math.sqrt(d)
    lens = [70, 250, 129, 5, 200, 128, 33, 90, 64, 17, 31, 3]
    seqs = {i: (torch.randn(L, n_kv, d).to(dtype), torch.randn(L, n_kv, d).to(dtype)) for i, L in enumerate(lens)}
    kc, vc, pt = _fill_cache(seqs, n_kv, d, page, dtype, n_pages=40, max_pages=4, slots=len(lens), scatter_seed=9)
    tok_slot, tok_pos, tiles0, tilesn = [], [], [], []
    base = 0
    for i, L in enumerate(lens):
        tok_slot += [i] * L
        tok_pos += list(range(L))
        for q0 in range(0, L, tile):
            tiles0.append(base + q0)
            tilesn.append(min(tile, L - q0))
        base += L
    q = torch.randn(base, n_heads, d, device=DEV).to(dtype)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    args = (q, kc, vc, pt, i32(tiles0), i32(tilesn), i32(tok_slot), i32(tok_pos))
    first = torch.empty(base, n_heads * d, device=DEV, dtype=dtype)
    k.attn_prefill_tc(*args, first, len(tiles0), scale, None)
    out = torch.empty_like(first)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=DEV)   # larger than L2: the next launch's K and V come late
    for it in range(120):
        if it % 2:
            flush.fill_(it & 255)
        k.attn_prefill_tc(*args, out, len(tiles0), scale, None)
        assert torch.equal(out, first), f"launch {it} differs"
    torch.cuda.synchronize()
    k.check_error_flags()


# ------------------------------------------------------------------------------------ token choice
def test_argmax_rows_ties_and_state():
    k = K()
    vocab = 1543
    lg = torch.randn(5, vocab, device=DEV)
    lg[0, 700] = lg[0, 33] = 50.0  # tie: the lower index wins
    lg[1, vocab - 1] = 60.0
    lg[2, 0] = 60.0
    lg[3] = -3.0  # all equal
    out = torch.empty(5, dtype=torch.int32, device=DEV)
    slots = torch.tensor([4, -1, 0, 2, 1], dtype=torch.int32, device=DEV)
    last = torch.full((6,), -7, dtype=torch.int32, device=DEV)
    k.argmax_rows(lg, out, slots, last)
    want = [33, vocab - 1, 0, 0, int(lg[4].argmax())]
    assert out.tolist() == want
    assert last.tolist() == [0, want[4], 0, -7, 33, -7]


@pytest.mark.parametrize("vocab", [331, 1024, 151936])
@pytest.mark.parametrize("temperature,top_k", [(0.7, 20), (1.0, 0), (1.3, 1), (0.5, 5000)])
def test_sample_rows_matches_plain(vocab, temperature, top_k):
    k = K()
    rows = 6
    g = torch.Generator().manual_seed(vocab + top_k)
    lg = (torch.randn(rows, vocab, generator=g) * 3).float()
    lg[1, 5] = lg[1, 100] = lg[1, 300] = lg[1].max() + 1.0  # ties at the top
    lg[2, : min(50, vocab)] = 2.5                                # ties straddling the top-k boundary
    seqs = torch.tensor([0, 1, 2, 3, 10, 999], dtype=torch.int32)
    out = torch.empty(rows, dtype=torch.int32, device=DEV)
    for step in (0, 1, 7):
        k.sample_rows(lg.to(DEV), temperature, top_k, 1234, seqs.to(DEV), None, out, step_base=step)
        got = out.tolist()
        want = [P.choose_token(lg[r], temperature, top_k, P.uniform_draw(1234, int(seqs[r]), step)) for r in range(rows)]
        assert got == want, (step, got, want)


# ------------------------------------------------------------------------------------ the timing tool
def test_microbench_runs_small(capsys):
    """``python -m dryft_b200.ops.microbench``'s functions at sizes a test can afford: every line they print carries
    a positive time (the numbers under ``profiles/`` come from the same functions at full size)."""
    from dryft_b200.ops import microbench

    with torch.no_grad():
        microbench.attn_prefill(token_counts=(256,))
        microbench.decode_chain(layers=1, small_rows=(8,), stream_rows=(16,))
        microbench.decode_products(layers=1, rows=(8, 64))
    lines = [ln for ln in capsys.readouterr().out.splitlines() if ln.strip()]
    assert len(lines) == 2 + 3 + 8
    import re

    for ln in lines:
        times = [float(t) for t in re.findall(r"([0-9.]+) us", ln)]
        assert times and all(t > 0 for t in times), ln
    assert microbench.main(["microbench", "no-such-thing"]) == 2
