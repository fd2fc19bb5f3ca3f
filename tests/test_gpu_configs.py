"""The benchmark configurations at their FULL sizes.  Two kinds of check: size-independent
properties (a fused or strided kernel must agree with the same computation spelled as a chain of
the primitive operators that the small-case tests have already pinned to the reference), and the
CPU oracle itself on SAMPLES of the full-size result — rows, columns and windows that include the
first and last tiles, the last split and the highest indices, so that an index error that only
shows beyond 2^31 bytes or in the last row cannot pass on both sides."""
import numpy as np
import pytest
import torch

import oracle_lib as ol
from oracle_lib import HostView
from gpu_util import assert_bits_equal, assert_close

pytestmark = pytest.mark.gpu
RTOL = 1e-5


def _bits_equal(a, b):
    return torch.equal(a.view(torch.int32), b.view(torch.int32))


def _max_rel(a, b):
    d = (a.double() - b.double()).abs()
    return float((d / b.double().abs().clamp_min(1e-30)).max())


def test_config3_reductions_full_size(ct):
    """X[8192,16384] ~ N(0,1), seed 2: sum/mean/var/max/argmax over dim 0 and dim 1."""
    g = torch.Generator(device="cuda")
    g.manual_seed(2)
    X = torch.randn(8192, 16384, device="cuda", generator=g)
    for dim, n in ((0, 8192), (1, 16384)):
        s = ct.reduce(ct.SUM, X, dim)
        # mean == mul_scalar(sum, 1/N), bit for bit (the reference's definition)
        assert _bits_equal(ct.reduce(ct.MEAN, X, dim), ct.unary(ct.MUL_S, s, 1.0 / n))
        # var == the chain mean -> sub -> mul -> mean of the reference's BatchNorm recipe
        keep = (1, 16384) if dim == 0 else (8192, 1)
        mu = ct.reduce(ct.MEAN, X, dim).view(keep)
        d = ct.binary(ct.SUB, X, mu)
        chain = ct.reduce(ct.MEAN, ct.binary(ct.MUL, d, d), dim)
        assert _max_rel(ct.reduce(ct.VAR, X, dim), chain) < RTOL
        # max/argmax: argmax indexes the maximum; max of the other-dim maxima is the global one
        mx = ct.reduce(ct.MAX, X, dim)
        am = ct.reduce(ct.ARGMAX, X, dim).long()
        picked = X.gather(dim, am.unsqueeze(dim)).squeeze(dim)          # torch only indexes the check
        assert _bits_equal(picked, mx)
        assert ct.reduce(ct.MAX, mx, -1).item() == ct.reduce(ct.MAX, X, -1).item()
        # sums agree with a transposed layout (other kernel shape), fp64 accumulation on both
        st = ct.reduce(ct.SUM, ct.contiguous(ct.DView.of(X).permute([1, 0])), 1 - dim)
        assert _max_rel(st, s) < 1e-6 or float((st - s).abs().max()) < 1e-3
    del X


def test_config3_reductions_full_size_against_the_oracle(ct, oracle):
    """The oracle on 192 columns (dim 0) and 192 rows (dim 1) of the full-size X: the first and
    last column tile / row, the rows of the last split, and a stretch in the middle."""
    g = torch.Generator(device="cuda")
    g.manual_seed(2)
    X = torch.randn(8192, 16384, device="cuda", generator=g)
    X[8191, 16383] = 0.0
    X[0, 16383] = -0.0
    host = X.cpu().numpy()
    whole = HostView.contig(host)
    for dim, extent in ((0, 16384), (1, 8192)):
        starts = (0, extent // 2 - 37, extent - 64)
        for op in (ol.SUM, ol.MEAN, ol.VAR, ol.MAX, ol.MIN, ol.ARGMAX):
            got = ct.reduce(op, X, dim).cpu().numpy()
            for lo in starts:
                ref = oracle.reduce(op, whole.narrow(1 - dim, lo, 64), dim)
                if op in (ol.MAX, ol.MIN, ol.ARGMAX):
                    assert_bits_equal(got[lo:lo + 64], ref, f"op {op} dim {dim} at {lo}")
                else:
                    assert_close(got[lo:lo + 64], ref, RTOL, f"op {op} dim {dim} at {lo}")
    del X


def test_config4_permuted_softmax_chain_full_size(ct, oracle):
    """S = permute(0,2,1,3) of a [32,1024,12,1024] buffer, M[1,12,1,1024]: S+M, then the chain
    max -> sub -> exp -> sum -> div along the last dim, fused and unfused."""
    g = torch.Generator(device="cuda")
    g.manual_seed(4)
    buf = torch.randn(32, 1024, 12, 1024, device="cuda", generator=g)
    g.manual_seed(5)
    M = -torch.rand(1, 12, 1, 1024, device="cuda", generator=g)
    S = ct.DView.of(buf).permute([0, 2, 1, 3])
    t = ct.binary(ct.ADD, S, M)                                 # strided in, contiguous out
    # same values as packing first, then a contiguous broadcast add
    t2 = ct.binary(ct.ADD, ct.contiguous(S), M)
    assert _bits_equal(t, t2)
    del t2
    m = ct.reduce(ct.MAX, t, 3).view(32, 12, 1024, 1)
    e = ct.unary(ct.EXP, ct.binary(ct.SUB, t, m))
    del t
    z = ct.reduce(ct.SUM, e, 3).view(32, 12, 1024, 1)
    chain = ct.binary(ct.DIV, e, z)
    del e
    fused = ct.softmax(S, M)
    assert _max_rel(fused, chain) < RTOL
    differing = (fused.view(torch.int32) != chain.view(torch.int32)).float().mean().item()
    assert differing < 1e-3                                     # the two differ only in rare last bits
    rows = ct.reduce(ct.SUM, fused, 3)
    assert float((rows - 1).abs().max()) < 1e-5
    # the oracle on sampled rows [b, h, q, :] of S + M and of softmax(S + M), the last batch,
    # head and row (the highest addresses of the 1.5 GiB buffer) among them
    t = ct.binary(ct.ADD, S, M)
    picks = [(0, 0, 0), (0, 11, 1023), (13, 5, 511), (31, 0, 0), (31, 11, 1022), (31, 11, 1023)]
    x_rows = np.stack([buf[b, q, h, :].cpu().numpy() for b, h, q in picks])       # S[b,h,q,:] = buf[b,q,h,:]
    m_rows = np.stack([M[0, h, 0, :].cpu().numpy() for b, h, q in picks])
    hx, hm = HostView.contig(x_rows), HostView.contig(m_rows)
    assert_bits_equal(np.stack([t[b, h, q].cpu().numpy() for b, h, q in picks]), oracle.binary(ol.ADD, hx, hm), "S+M rows")
    assert_close(np.stack([fused[b, h, q].cpu().numpy() for b, h, q in picks]), oracle.softmax(hx, hm), RTOL,
                 "softmax(S+M) rows")
    assert_close(np.stack([chain[b, h, q].cpu().numpy() for b, h, q in picks]), oracle.softmax(hx, hm), RTOL,
                 "unfused chain rows")


def test_config5_gpt2_rows_full_size(ct, oracle):
    """GPT-2 small non-GEMM ops on [8,1024,768] / [8,1024,3072] / [8,12,1024,1024]."""
    g = torch.Generator(device="cuda")
    g.manual_seed(6)
    x = torch.randn(8, 1024, 768, device="cuda", generator=g)
    r = torch.randn(8, 1024, 768, device="cuda", generator=g)
    gamma = 1 + 0.02 * torch.randn(768, device="cuda", generator=g)
    beta = 0.02 * torch.randn(768, device="cuda", generator=g)
    h = ct.binary(ct.ADD, x, r)                                 # residual add
    # LayerNorm: fused vs the chain of the reference's BatchNorm recipe applied per row
    mu = ct.reduce(ct.MEAN, h, 2).view(8, 1024, 1)
    d = ct.binary(ct.SUB, h, mu)
    v = ct.reduce(ct.MEAN, ct.binary(ct.MUL, d, d), 2).view(8, 1024, 1)
    rstd = ct.unary(ct.POW_S, ct.unary(ct.ADD_S, v, 1e-5), -0.5)
    chain = ct.binary(ct.ADD, ct.binary(ct.MUL, ct.binary(ct.MUL, d, rstd), gamma), beta)
    fused = ct.layernorm(h, gamma, beta, 1e-5)
    assert float((fused - chain).abs().max()) < 1e-5
    # tanh-GELU on [8,1024,3072]: fused functor vs the chain of primitives, bit for bit
    a = torch.randn(8, 1024, 3072, device="cuda", generator=g)
    u = ct.binary(ct.MUL, ct.binary(ct.MUL, a, a), a)
    u = ct.unary(ct.MUL_S, ct.binary(ct.ADD, a, ct.unary(ct.MUL_S, u, 0.044715)), 0.7978845608028654)
    gchain = ct.binary(ct.MUL, ct.unary(ct.MUL_S, a, 0.5), ct.unary(ct.ADD_S, ct.unary(ct.TANH, u), 1.0))
    assert _bits_equal(ct.unary(ct.GELU_TANH, a), gchain)
    # causal attention softmax on [8,12,1024,1024]: flag == explicit -1e9 mask tensor
    s = torch.randn(8, 12, 1024, 1024, device="cuda", generator=g)
    i = torch.arange(1024, device="cuda")
    mask = torch.where(i[None, :] > i[:, None], -1e9, 0.0).float().view(1, 1, 1024, 1024)
    by_flag = ct.softmax(s, None, causal=True)
    by_mask = ct.softmax(s, mask)
    assert _bits_equal(by_flag, by_mask)
    assert float(by_flag[0, 0, 0, 1:].abs().max()) == 0.0
    # the oracle on samples of every op: first / middle / last rows, windows and attention matrices
    for lo in (0, 4000, 8 * 1024 - 16):
        rows_h = HostView.contig(h.view(-1, 768)[lo:lo + 16].cpu().numpy())
        xs = HostView.contig(x.view(-1, 768)[lo:lo + 16].cpu().numpy())
        rs = HostView.contig(r.view(-1, 768)[lo:lo + 16].cpu().numpy())
        assert_bits_equal(rows_h.numpy(), oracle.binary(ol.ADD, xs, rs), "residual add rows")
        want = oracle.layernorm(rows_h, HostView.contig(gamma.cpu().numpy()), HostView.contig(beta.cpu().numpy()), 1e-5)
        assert_close(fused.view(-1, 768)[lo:lo + 16].cpu().numpy(), want, RTOL, "layernorm rows")
    ga = ct.unary(ct.GELU_TANH, a).view(-1)
    for lo in (0, a.numel() // 2 - 777, a.numel() - (1 << 16)):
        win = HostView.contig(a.view(-1)[lo:lo + (1 << 16)].cpu().numpy())
        assert_bits_equal(ga[lo:lo + (1 << 16)].cpu().numpy(), oracle.unary(ol.GELU_TANH, win), "gelu window")
    for b, hd in ((0, 0), (7, 11)):
        mat = HostView.contig(s[b, hd].cpu().numpy().reshape(1, 1, 1024, 1024))
        assert_close(by_flag[b, hd].cpu().numpy().reshape(1, 1, 1024, 1024), oracle.softmax(mat, None, causal=True), RTOL,
                     "causal softmax matrix")


def test_config2_sweep_full_size_against_the_oracle(ct, oracle):
    """add, mul, exp, relu, gelu on 2^30-element tensors: three 2^20-element windows of every result
    (start, an odd offset in the middle, the end) against the oracle, and the ragged tail of a
    tensor of 2^30 + 5 elements."""
    n = 1 << 30
    g = torch.Generator(device="cuda")
    g.manual_seed(1)
    x = torch.randn(n + 5, device="cuda", generator=g)
    y = torch.randn(n + 5, device="cuda", generator=g)
    w = 1 << 20
    starts = (0, n // 2 - 12345, n - w)

    def windows(t, lows):
        return [HostView.contig(t[lo:lo + w].cpu().numpy()) for lo in lows]

    for ragged in (False, True):
        xs, ys = (x, y) if ragged else (x[:n], y[:n])
        lows = (n + 5 - w,) if ragged else starts
        xw, yw = windows(xs, lows), windows(ys, lows)
        for op in (ol.ADD, ol.MUL):
            out = ct.binary(op, xs, ys)
            for lo, hx, hy in zip(lows, xw, yw):
                assert_bits_equal(out[lo:lo + w].cpu().numpy(), oracle.binary(op, hx, hy), f"binary {op} at {lo}")
            del out
        for op in (ol.EXP, ol.RELU, ol.GELU_TANH):
            out = ct.unary(op, xs)
            for lo, hx in zip(lows, xw):
                assert_bits_equal(out[lo:lo + w].cpu().numpy(), oracle.unary(op, hx), f"unary {op} at {lo}")
            del out


def test_dense_bit_pattern_blocks_fp32_unary(ct, oracle):
    """exp, gelu, tanh, log and sigmoid on 2^30 consecutive-bit-pattern inputs each (four blocks of
    2^28 patterns spread over the fp32 range: small/large, both signs, NaN/inf) against the
    oracle; NaN results compare equal whatever their payload."""
    import oracle_lib as ol
    for op in (ol.EXP, ol.GELU_TANH, ol.TANH, ol.LOG, ol.SIGMOID):
        for chunk in range(0, 16, 5):                           # 4 of the 16 chunks per op: 2^30 patterns
            start = chunk << 28
            xin, ref = oracle.sweep(op, start, 1, 1 << 28)
            got = ct.unary(op, torch.from_numpy(xin).cuda()).cpu().numpy()
            nan = np.isnan(ref)
            assert np.array_equal(np.isnan(got), nan), (op, chunk)
            assert np.array_equal(got.view(np.uint32)[~nan], ref.view(np.uint32)[~nan]), (op, chunk)
