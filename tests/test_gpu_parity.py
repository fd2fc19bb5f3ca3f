"""GPU parity tests: every case goes through the C ABI on cuda:0 and is compared with the
plain-C oracle and with the golden vectors of the real reference.  Bit-exact for elementwise,
integer, max/min, argmax and copy cases; sums/means/variances and the fused rows to 1e-5
relative (the tolerance the operator path states for fp32)."""
import numpy as np
import pytest
import torch

import cases as C
import oracle_lib as ol
from oracle_lib import HostView
from gpu_util import to_device, assert_bits_equal, assert_close

pytestmark = pytest.mark.gpu

CASES = C.all_cases()
GOLDEN = C.load_golden()
RTOL = 1e-5


def run_gpu(ct, case):
    k = case["kind"]
    dv = [to_device(v) for v in case["views"]]
    if k == "binary":
        return ct.binary(case["op"], dv[0], dv[1])
    if k == "unary":
        return ct.unary(case["op"], dv[0], case["scalar"])
    if k == "copy":
        return ct.contiguous(dv[0])
    if k == "reduce":
        return ct.reduce(case["op"], dv[0], case["dim"])
    if k == "softmax":
        out = ct.softmax(dv[0], dv[1] if len(dv) > 1 else None, case["causal"])
        return out
    if k == "layernorm":
        return ct.layernorm(dv[0], dv[1], dv[2], case["scalar"])
    if k == "log_softmax":
        return ct.log_softmax(dv[0], dv[1] if len(dv) > 1 else None)
    if k == "gather":
        return ct.gather(dv[0], case["dim"], dv[1])
    if k == "accgrad":
        grad = torch.from_numpy(case["views"][0].numpy()).cuda()
        return ct.accumulate_grad(grad, dv[1])
    if k == "matmul":
        return ct.matmul(dv[0], dv[1])
    if k == "bn_moments":
        return ct.channel_moments(dv[0])[case["op"]]
    if k == "bn_apply":
        p = dv[1:] + [None] * (5 - len(dv))
        return ct.batchnorm_apply(dv[0], p[0], p[1], p[2], p[3], case["scalar"])
    if k == "cat":
        return ct.cat(dv, case["dim"])
    if k == "div_bwd":
        return ct.div_backward(dv[0], dv[1], dv[2], want_a=case["op"] == 0, want_b=case["op"] == 1)[case["op"]]
    if k == "tanh_bwd":
        return ct.tanh_backward(dv[0], dv[1])
    if k == "ce":
        return ct.cross_entropy(dv[0], dv[1], bool(case["op"]))
    if k == "ce_bwd":
        batch = case["views"][0].shape[0]
        return ct.cross_entropy_backward(dv[0], dv[1], case["scalar"] / (batch if case["op"] else 1))
    if k == "optim":
        p = torch.from_numpy(case["views"][0].numpy()).cuda()
        g = torch.from_numpy(case["views"][1].numpy()).cuda()
        m, v = torch.zeros_like(p), torch.zeros_like(p)
        for t in range(1, case["dim"] + 1):
            if case["op"] == 0:
                ct.sgd_step(p, g, case["scalar"])
            elif case["op"] <= 2:
                ct.adam_step(p, g, m, v, case["scalar"], t, weight_decay=0.01 if case["op"] == 2 else None)
            else:       # RMSprop's alpha travels in beta2, as in the golden generator
                ct.optimizer_step(case["op"], p, g, m, v, t, case["scalar"], weight_decay=0.01, alpha=0.999)
        return p
    raise ValueError(k)


def expected_shape(case, ref):
    return ref.shape


@pytest.mark.parametrize("case", CASES, ids=[c["name"] for c in CASES])
def test_case_vs_oracle_and_golden(ct, oracle, case):
    got = run_gpu(ct, case).cpu().numpy()
    ref = C.run_case(oracle, case)
    got = got.reshape(ref.shape)
    gold = GOLDEN[case["name"]]
    if case["exact"]:
        assert_bits_equal(got, ref, case["name"])
        assert C.digest(got) == gold["digest"], f"{case['name']}: differs from the reference's golden output"
    else:
        # softmax(x) - 1 at the label cancels: an absolute floor of a few fp32 ulps of 1.0 for that kind
        atol = 3e-7 * abs(case["scalar"]) if case["kind"] == "ce_bwd" else 0.0
        assert_close(got, ref, RTOL, case["name"], atol)
        assert_close(got, gold["out"], RTOL, case["name"] + " (golden)", atol)


def test_causal_flag(ct, oracle):
    x = HostView.contig(np.random.default_rng(5).standard_normal((2, 3, 40, 40)).astype(np.float32))
    got = ct.softmax(to_device(x), None, causal=True).cpu().numpy()
    ref = oracle.softmax(x, None, causal=True)
    assert_close(got, ref, RTOL, "causal softmax")
    assert np.all(got[..., 0, 1:] == 0.0)          # masked entries underflow to exactly 0


# ---- the CPU-runnable configuration: A[1024,1024], B[1,1024] ~ U(-1,1), seed 0 -------------------------
def test_config_cpu_runnable(ct, oracle):
    rng = np.random.default_rng(0)
    A = rng.uniform(-1, 1, (1024, 1024)).astype(np.float32)
    B = rng.uniform(-1, 1, (1, 1024)).astype(np.float32)
    hA, hB = HostView.contig(A), HostView.contig(B)
    dA, dB = to_device(hA), to_device(hB)
    assert_bits_equal(ct.binary(ct.ADD, dA, dB), oracle.binary(ol.ADD, hA, hB), "A+B")
    assert_bits_equal(ct.binary(ct.MUL, dA, dB), oracle.binary(ol.MUL, hA, hB), "A*B")
    den_ref = oracle.unary(ol.ADD_S, HostView.contig(oracle.unary(ol.ABS, hB)), 1.0)
    den = ct.unary(ct.ADD_S, ct.unary(ct.ABS, dB), 1.0)
    assert_bits_equal(den, den_ref, "|B|+1")
    assert_bits_equal(ct.binary(ct.DIV, dA, den), oracle.binary(ol.DIV, hA, HostView.contig(den_ref)), "A/(|B|+1)")
    assert_bits_equal(ct.unary(ct.RELU, dA), oracle.unary(ol.RELU, hA), "relu(A)")
    for dim in (1, -1):
        assert_bits_equal(ct.reduce(ct.MAX, dA, dim), oracle.reduce(ol.MAX, hA, dim), f"max {dim}")
        assert_close(ct.reduce(ct.SUM, dA, dim), oracle.reduce(ol.SUM, hA, dim), RTOL, f"sum {dim}")
        assert_close(ct.reduce(ct.MEAN, dA, dim), oracle.reduce(ol.MEAN, hA, dim), RTOL, f"mean {dim}")


# ---- mid-size cases that exercise every kernel shape (oracle still finishes in seconds) --------------------
@pytest.mark.parametrize("n", [1, 3, 17, 1025, 4096, 4097, (1 << 20) + 5, 1 << 22])
@pytest.mark.parametrize("op", [ol.ADD, ol.MUL, ol.DIV])
def test_flat_binary_sizes(ct, oracle, n, op):
    rng = np.random.default_rng(n)
    a = HostView.contig(rng.standard_normal(n).astype(np.float32))
    b = HostView.contig(rng.standard_normal(n).astype(np.float32))
    assert_bits_equal(ct.binary(op, to_device(a), to_device(b)), oracle.binary(op, a, b), f"n={n}")


@pytest.mark.parametrize("n", [1, 5, 1023, (1 << 20) + 3, 1 << 22])
@pytest.mark.parametrize("op", [ol.EXP, ol.RELU, ol.GELU_TANH, ol.TANH, ol.LOG, ol.SIGMOID, ol.MUL_S])
def test_flat_unary_sizes(ct, oracle, n, op):
    x = np.random.default_rng(n + 1).standard_normal(n).astype(np.float32)
    if op == ol.LOG:
        x = np.abs(x) + np.float32(1e-6)
    h = HostView.contig(x)
    assert_bits_equal(ct.unary(op, to_device(h), 0.3), oracle.unary(op, h, 0.3), f"n={n}")


@pytest.mark.parametrize("op", [ol.EXP, ol.LOG, ol.TANH, ol.SIGMOID, ol.GELU_TANH, ol.SQRT, ol.RELU, ol.ABS])
def test_bit_pattern_sweep(ct, oracle, op):
    """Every 521st fp32 bit pattern (8.2 M inputs: NaN, inf, denormals, both signs)."""
    count = (1 << 32) // 521
    xin, ref = oracle.sweep(op, 7, 521, count)
    got = ct.unary(op, torch.from_numpy(xin).cuda())
    assert_bits_equal(got, ref, ol.UNARY_NAMES[op])


@pytest.mark.parametrize("op", [ol.EXP, ol.LOG, ol.TANH, ol.SIGMOID, ol.GELU_TANH])
def test_packed_functions_equal_the_scalar_ones_on_every_fp32_pattern(ct, op):
    """The contiguous kernel evaluates exp/log/tanh/sigmoid/gelu two lanes per instruction
    (packed fp32x2 arithmetic); the strided kernels use the one-lane functions that
    test_bit_pattern_sweep pins against the oracle.  Both must give the same bits for ALL 2^32
    inputs: 32 blocks of 2^27 consecutive bit patterns, each once through a contiguous view and
    once through a stride-2 view."""
    m = 1 << 27
    wide = torch.empty(2 * m, dtype=torch.float32, device="cuda")
    for block in range(32):
        lo = -(1 << 31) + block * m
        x = torch.arange(lo, lo + m, dtype=torch.int64, device="cuda").to(torch.int32).view(torch.float32)
        wide[::2] = x
        packed = ct.unary(op, x)
        scalar = ct.unary(op, ct.DView.of(wide[::2]))
        same = torch.equal(packed.view(torch.int32), scalar.view(torch.int32))
        if not same:
            bad = (packed.view(torch.int32) != scalar.view(torch.int32)).nonzero()[:4].flatten().tolist()
            raise AssertionError(f"{ol.UNARY_NAMES[op]}: block {block}, first differing patterns "
                                 f"{[hex((lo + i) & 0xFFFFFFFF) for i in bad]}")
        del packed, scalar, x


@pytest.mark.parametrize("shape,dim", [((2048, 4096), 0), ((2048, 4096), 1), ((4099, 1031), 0), ((4099, 1031), 1),
                                       ((8, 300000), 1), ((300000, 8), 0), ((3, 700, 1100), 1), ((1 << 22,), 0)])
@pytest.mark.parametrize("op", [ol.SUM, ol.MEAN, ol.MAX, ol.MIN, ol.VAR, ol.ARGMAX])
def test_reduce_shapes(ct, oracle, shape, dim, op):
    x = HostView.contig(np.random.default_rng(sum(shape) + dim).standard_normal(shape).astype(np.float32))
    got = ct.reduce(op, to_device(x), dim)
    ref = oracle.reduce(op, x, dim)
    if op in (ol.MAX, ol.MIN, ol.ARGMAX):
        assert_bits_equal(got, ref, f"{shape} dim {dim}")
    else:
        assert_close(got, ref, RTOL, f"{shape} dim {dim}")


@pytest.mark.parametrize("op", [ol.SUM, ol.MEAN, ol.MAX, ol.MIN, ol.VAR])
def test_reduce_full_sizes(ct, oracle, op):
    for n in (1, 7, 65536, (1 << 22) + 3):
        x = HostView.contig((np.random.default_rng(n).standard_normal(n) + 0.25).astype(np.float32))
        got = ct.reduce(op, to_device(x), -1)
        ref = oracle.reduce(op, x, -1)
        if op in (ol.MAX, ol.MIN):
            assert_bits_equal(got, ref, f"full n={n}")
        else:
            assert_close(got, ref, RTOL, f"full n={n}")


def _zeros_mix(seed, shape, sign, dtype=np.float32):
    """Zeros of both signs among values on one side of zero: max (sign=+1) / min (sign=-1) is a zero
    and its sign is the sign of the first zero of the line."""
    pick = (np.array([-0.0, 0.0, -1.5, -3.0]) * sign).astype(dtype)
    return pick[np.random.default_rng(seed).integers(0, 4, shape)]


@pytest.mark.parametrize("shape,dim", [((2048, 4096), 0), ((2048, 4096), 1), ((4099, 1031), 0), ((4099, 1031), 1),
                                       ((8, 300000), 1), ((300000, 8), 0), ((64, 20000), 1), ((3, 700, 1100), 1),
                                       ((1 << 22,), 0), (((1 << 22) + 3,), -1), ((1500, 1500), -1)])
@pytest.mark.parametrize("op", [ol.MAX, ol.MIN])
def test_minmax_signed_zero_is_the_first_in_index_order(ct, oracle, shape, dim, op):
    """Every reduction kernel shape on data whose extreme is a zero of either sign."""
    x = HostView.contig(_zeros_mix(sum(shape), shape, 1.0 if op == ol.MAX else -1.0))
    assert_bits_equal(ct.reduce(op, to_device(x), dim), oracle.reduce(op, x, dim), f"{shape} dim {dim}")
    if len(shape) == 2:          # the transposed view: strided lines (generic kernels), permuted full reduction
        t = x.permute([1, 0])
        assert_bits_equal(ct.reduce(op, to_device(t), dim if dim < 0 else 1 - dim),
                          oracle.reduce(op, t, dim if dim < 0 else 1 - dim), f"{shape}^T")


@pytest.mark.parametrize("dtype", [np.float64, np.int32])
@pytest.mark.parametrize("shape,dim", [(((1 << 22) + 5,), -1), ((1 << 20, 8), 0), ((8, 1 << 20), 1), ((3000, 700), 0),
                                       ((3000, 700), 1), ((64, 50000), 1), ((70, 4, 30000), 2)])
@pytest.mark.parametrize("op", [ol.SUM, ol.MEAN, ol.MAX, ol.MIN, ol.VAR, ol.ARGMAX])
def test_reduce_other_dtypes_and_strided_shapes(ct, oracle, dtype, shape, dim, op):
    """Float64 / Int32 tensors (and Float32 shapes outside the fast paths, below) go through the
    generic kernels: a thread, a warp or a CTA chunk per line — a full reduction is one long line."""
    if (op == ol.VAR and dtype == np.int32) or (op == ol.ARGMAX and dim < 0):
        pytest.skip("not defined")
    rng = np.random.default_rng(len(shape) * 7 + abs(dim))
    raw = rng.standard_normal(shape) * 50
    x = HostView.contig(raw.astype(dtype))
    got = ct.reduce(op, to_device(x), dim)
    ref = oracle.reduce(op, x, dim)
    if op in (ol.MAX, ol.MIN, ol.ARGMAX) or dtype == np.int32 and op == ol.SUM:
        assert_bits_equal(got, ref, f"{dtype.__name__} {shape} dim {dim}")
    elif dtype == np.int32:      # mean of integers truncates: a last-bit difference of the fp64 sum can flip it
        assert np.max(np.abs(got.cpu().numpy().astype(np.int64) - ref.astype(np.int64))) <= 1
    else:
        assert_close(got, ref, RTOL, f"{dtype.__name__} {shape} dim {dim}")


@pytest.mark.parametrize("shape,dim", [((1 << 20, 8), 0), ((5000, 24), 0), ((40, 70001), 1)])
@pytest.mark.parametrize("op", [ol.SUM, ol.MAX, ol.VAR, ol.ARGMAX])
def test_reduce_f32_outside_the_fast_paths(ct, oracle, shape, dim, op):
    """Fewer than 32 columns, or a strided reduce dim: Float32 lines the row / column kernels do not take."""
    x = HostView.contig(np.random.default_rng(shape[1]).standard_normal(shape).astype(np.float32))
    views = [x] if shape[1] < 32 else [HostView(x.buf, (shape[0], shape[1] // 2), (shape[1], 2), 1)]
    for v in views:
        got, ref = ct.reduce(op, to_device(v), dim), oracle.reduce(op, v, dim)
        if op in (ol.MAX, ol.ARGMAX):
            assert_bits_equal(got, ref, f"{shape} dim {dim}")
        else:
            assert_close(got, ref, RTOL, f"{shape} dim {dim}")


def test_first_scratch_use_on_a_side_stream(ct, oracle):
    """A reduction that makes the library (re)allocate its workspace, issued on a non-blocking side
    stream: the clearing of the fresh workspace must be ordered before the kernel on THAT stream."""
    buf = np.random.default_rng(77).standard_normal(1 << 27).astype(np.float32)
    x = HostView(buf, (1 << 13, 1 << 13), (1 << 14, 2), 0)    # every other element: packed into the workspace first
    d = to_device(x)
    assert ct.reduce_workspace_bytes(d, -1) > (128 << 20)      # larger than any workspace an earlier test grew
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        got = ct.reduce(ct.SUM, d, -1)
        again = ct.reduce(ct.SUM, d, -1)
        cols = ct.reduce(ct.SUM, d, 0)                          # the ticket kernels on the same fresh workspace
    side.synchronize()
    assert_close(got, oracle.reduce(ol.SUM, x, -1), RTOL)
    assert_bits_equal(again, got.cpu().numpy())
    assert_close(cols, oracle.reduce(ol.SUM, x, 0), RTOL)


def test_output_overlapping_an_input_is_refused(ct):
    a = torch.zeros(64, 64, device="cuda")
    b = torch.ones(64, 64, device="cuda")
    for call in (lambda: ct.binary(ct.ADD, a, b, out=a), lambda: ct.unary(ct.EXP, a, out=a),
                 lambda: ct.reduce(ct.SUM, a, 0, out=a.view(-1)[:64]), lambda: ct.softmax(a, out=a),
                 lambda: ct.binary(ct.ADD, a, b, out=b.view(-1)[: 64 * 64].view(64, 64))):
        with pytest.raises(ct.CtbError) as e:
            call()
        assert e.value.code == 5 and "overlaps an input" in e.value.message
    # neighbours in one allocation do not overlap
    buf = torch.zeros(2, 64, 64, device="cuda")
    ct.binary(ct.ADD, buf[0], b, out=buf[1])
    assert torch.all(buf[1] == 1)


def test_backward_chains_accumulate_into_gradient_buffers(ct, oracle):
    """accumulate = 1: the chain's result is added into an existing gradient buffer, NaN / infinite
    contributions skipped (accumulate_grad's rule); strided buffers and 1 GiB operands included."""
    rng = np.random.default_rng(21)
    g = HostView.contig(rng.standard_normal((300, 257)).astype(np.float32))
    a = HostView.contig(rng.standard_normal((300, 257)).astype(np.float32))
    bnp = rng.standard_normal((300, 257)).astype(np.float32)
    bnp[5, 7] = 0.0                                     # g / 0 -> inf: skipped
    b = HostView.contig(bnp)
    start_a = rng.standard_normal((300, 257)).astype(np.float32)
    start_b = rng.standard_normal((300, 257)).astype(np.float32)
    da, db = oracle.div_backward(g, a, b)
    want_a = oracle.accumulate_grad(start_a, HostView.contig(da))
    want_b = oracle.accumulate_grad(start_b, HostView.contig(db))
    buf_a, buf_b = torch.from_numpy(start_a).cuda(), torch.from_numpy(start_b).cuda()
    ct.div_backward(to_device(g), to_device(a), to_device(b), out_a=buf_a, out_b=buf_b, accumulate=True)
    assert_bits_equal(buf_a, want_a, "grad_a += g / b")
    assert_bits_equal(buf_b, want_b, "grad_b += chain")
    assert buf_a[5, 7].item() == start_a[5, 7]
    # a transposed gradient buffer (strided kernel)
    tbuf = torch.from_numpy(np.ascontiguousarray(start_a.T)).cuda()
    ct.tanh_backward(to_device(g), to_device(a), out=ct.DView.of(tbuf).permute([1, 0]), accumulate=True)
    want_t = oracle.accumulate_grad(start_a, HostView.contig(oracle.tanh_backward(g, a)))
    assert_close(tbuf.cpu().numpy().T, want_t, RTOL, "tanh backward into a transposed buffer", atol=1e-6)
    # cross-entropy gradient added to an existing buffer
    logits = HostView.contig(rng.standard_normal((64, 1500)).astype(np.float32) * 4)
    labels = HostView.contig(rng.integers(0, 1500, (64, 1)).astype(np.int32))
    start = rng.standard_normal((64, 1500)).astype(np.float32)
    buf = torch.from_numpy(start).cuda()
    ct.cross_entropy_backward(to_device(logits), to_device(labels), 1.0 / 64, out=buf, accumulate=True)
    want = start + oracle.cross_entropy_backward(logits, labels, True, 1.0)
    assert_close(buf, want, RTOL, "ce backward accumulate", atol=1e-6)
    # a label outside the row raises the flag instead of a device-side error
    bad = torch.zeros(1, dtype=torch.int32, device="cuda")
    lab_bad = labels.numpy().copy()
    lab_bad[3, 0] = 1500
    ct.cross_entropy(to_device(logits), to_device(HostView.contig(lab_bad)), True, bad=bad)
    assert bad.item() == 1
    ct.cross_entropy(to_device(logits), to_device(labels), True, bad=bad)
    assert bad.item() == 0


@pytest.mark.parametrize("rows,classes", [(4096, 1000), (512, 50257), (65536, 10), (300, 16384), (200, 32768), (64, 20000),
                                          (2048, 2048), (1000, 1028), (777, 1536), (500, 2044), (300, 4096), (300, 8192)])
def test_cross_entropy_sizes(ct, oracle, rows, classes):
    rng = np.random.default_rng(rows + classes)
    logits = HostView.contig((rng.standard_normal((rows, classes)) * 3).astype(np.float32))
    labels = HostView.contig(rng.integers(0, classes, (rows, 1)).astype(np.int32))
    got = ct.cross_entropy(to_device(logits), to_device(labels), True)
    assert_close(got, oracle.cross_entropy(logits, labels, True), RTOL, "loss")
    grad = ct.cross_entropy_backward(to_device(logits), to_device(labels), 1.0 / rows)
    # The reference accumulates the row's sum of exponentials in fp32, class after class: once the
    # running sum is large, terms below half its ulp are lost, and over 50257 classes the sum itself
    # is only good to ~1e-4 (the kernel's fp64 sum is the more accurate one).  The comparison allows
    # for that: 4e-9 * classes relative, and the same fraction of the largest possible entry absolute.
    rtol = max(RTOL, 4e-9 * classes)
    assert_close(grad, oracle.cross_entropy_backward(logits, labels, True, 1.0), rtol, "gradient", atol=max(3e-7, rtol) / rows)


@pytest.mark.parametrize("classes,pad", [(40001, 3), (50257, 0), (9000, 5), (12288, 4), (33000, 1)])
def test_cross_entropy_long_and_strided_rows(ct, classes, pad):
    """Rows beyond the register kernels (one sweep with a running maximum), rows that start at every
    4-byte phase (a slice of a wider buffer), and the gradient added into an existing buffer — against
    the definition evaluated in float64."""
    rows = 37
    rng = np.random.default_rng(classes + pad)
    wide = (rng.standard_normal((rows, classes + pad)) * 4).astype(np.float32)
    labels = rng.integers(0, classes, (rows, 1)).astype(np.int32)
    labels[1, 0] = -1                                  # counts from the end
    dwide = torch.from_numpy(wide).cuda()
    x = dwide[:, pad // 2: pad // 2 + classes] if pad else dwide
    xs = wide[:, pad // 2: pad // 2 + classes].astype(np.float64) if pad else wide.astype(np.float64)
    lab = np.where(labels[:, 0] < 0, labels[:, 0] + classes, labels[:, 0])
    sh = xs - xs.max(1, keepdims=True)
    logz = np.log(np.exp(sh).sum(1))
    want_loss = float(np.mean(-(sh[np.arange(rows), lab] - logz)))
    got = ct.cross_entropy(ct.DView.of(x), torch.from_numpy(labels).cuda(), True)
    assert abs(float(got) - want_loss) <= 1e-5 * abs(want_loss)
    soft = np.exp(sh - logz[:, None])
    soft[np.arange(rows), lab] -= 1.0
    want = soft / rows
    grad = ct.cross_entropy_backward(ct.DView.of(x), torch.from_numpy(labels).cuda(), 1.0 / rows)
    np.testing.assert_allclose(grad.cpu().numpy(), want, rtol=2e-5, atol=1e-9)
    start = rng.standard_normal((rows, classes)).astype(np.float32)
    buf = torch.from_numpy(start).cuda()
    ct.cross_entropy_backward(ct.DView.of(x), torch.from_numpy(labels).cuda(), 1.0 / rows, out=buf, accumulate=True)
    np.testing.assert_allclose(buf.cpu().numpy(), start + want, rtol=2e-5, atol=2e-7)


def test_argmax_ties_prefer_first_index(ct, oracle):
    x = np.zeros((64, 5000), np.float32)
    x[:, 1234] = 3.0
    x[:, 4321] = 3.0
    x[:, 77] = 3.0
    h = HostView.contig(x)
    got = ct.reduce(ct.ARGMAX, to_device(h), 1).cpu().numpy()
    assert np.all(got == 77)
    assert_bits_equal(ct.reduce(ct.ARGMAX, to_device(h.permute([1, 0])), 0), oracle.reduce(ol.ARGMAX, h.permute([1, 0]), 0))


def test_reductions_are_deterministic(ct):
    x = torch.randn(1 << 24, device="cuda")
    m = x.view(4096, 4096)
    for args in ((ct.SUM, x, -1), (ct.SUM, m, 0), (ct.SUM, m, 1), (ct.VAR, m, 0)):
        a = ct.reduce(*args).cpu().numpy()
        for _ in range(3):
            assert np.array_equal(a.view(np.uint32), ct.reduce(*args).cpu().numpy().view(np.uint32))


def test_caller_workspace(ct, oracle):
    x = HostView.contig(np.random.default_rng(3).standard_normal((4096, 512)).astype(np.float32))
    d = to_device(x)
    need = ct.reduce_workspace_bytes(d, 0)
    assert need > 0
    ws = torch.zeros(need // 4 + 64, dtype=torch.int32, device="cuda")
    got = ct.reduce(ct.SUM, d, 0, workspace=ws)
    assert_close(got, oracle.reduce(ol.SUM, x, 0), RTOL)
    with pytest.raises(ct.CtbError) as e:
        ct.reduce(ct.SUM, d, 0, workspace=ws[:16])
    assert e.value.code == 7


def test_full_reduce_partials_for_sharding(ct, oracle):
    """Two shards' fp64 partials summed on the host and finalised == the unsharded result."""
    x = np.random.default_rng(9).standard_normal(1 << 21).astype(np.float32)
    d = torch.from_numpy(x).cuda()
    p0 = ct.reduce_full_partial(ct.SUM, d[: 1 << 20])
    p1 = ct.reduce_full_partial(ct.SUM, d[1 << 20:])
    tot = p0 + p1                                   # stands in for the all-reduce
    for op in (ct.SUM, ct.MEAN):
        got = ct.finalize_full(op, tot, x.size)
        assert_close(got, oracle.reduce(op, HostView.contig(x), -1), RTOL)
    m0 = ct.reduce_full_partial(ct.MAX, d[: 1 << 20])
    m1 = ct.reduce_full_partial(ct.MAX, d[1 << 20:])
    got = ct.finalize_full(ct.MAX, torch.maximum(m0, m1), x.size)
    assert_bits_equal(got, oracle.reduce(ol.MAX, HostView.contig(x), -1))


@pytest.mark.parametrize("cols", [1, 3, 32, 768, 1024, 1000, 3072, 8192, 10000])
def test_fused_rows_widths(ct, oracle, cols):
    rows = 37
    rng = np.random.default_rng(cols)
    x = HostView.contig(rng.standard_normal((rows, cols)).astype(np.float32))
    g = HostView.contig(rng.normal(1, 0.02, cols).astype(np.float32))
    b = HostView.contig(rng.normal(0, 0.02, cols).astype(np.float32))
    assert_close(ct.softmax(to_device(x)), oracle.softmax(x), RTOL, f"softmax cols={cols}")
    if cols > 1:
        assert_close(ct.layernorm(to_device(x), to_device(g), to_device(b)), oracle.layernorm(x, g, b), RTOL,
                     f"layernorm cols={cols}")


def test_softmax_chain_equals_unfused_chain(ct):
    """The fused kernel against the same chain run op by op through the C ABI."""
    x = torch.randn(64, 12, 1024, device="cuda")
    m = ct.reduce(ct.MAX, x, 2).view(64, 12, 1)
    s = ct.binary(ct.SUB, x, m)
    e = ct.unary(ct.EXP, s)
    z = ct.reduce(ct.SUM, e, 2).view(64, 12, 1)
    chain = ct.binary(ct.DIV, e, z)
    fused = ct.softmax(x)
    assert_close(fused, chain.cpu().numpy(), RTOL)
    assert (fused.cpu().numpy().view(np.uint32) != chain.cpu().numpy().view(np.uint32)).mean() < 1e-3


# ---- host-buffer entry points ---------------------------------------------------------------------------------
def test_host_entry_points(ct, oracle):
    n = (1 << 25) + 12345                       # > one pipeline chunk, ragged
    rng = np.random.default_rng(1)
    a = torch.from_numpy(rng.standard_normal(n).astype(np.float32)).pin_memory()
    b = torch.from_numpy(rng.standard_normal(n).astype(np.float32)).pin_memory()
    out = torch.empty(n, dtype=torch.float32).pin_memory()
    ct.binary_host(ct.ADD, a, b, out)
    ha, hb = HostView.contig(a.numpy()), HostView.contig(b.numpy())
    assert_bits_equal(out.numpy(), oracle.binary(ol.ADD, ha, hb), "host add")
    ct.unary_host(ct.GELU_TANH, a, out)
    assert_bits_equal(out.numpy(), oracle.unary(ol.GELU_TANH, ha), "host gelu")
    A = torch.from_numpy(rng.standard_normal((512, 300)).astype(np.float32))
    B = torch.from_numpy(rng.standard_normal((1, 300)).astype(np.float32))
    o2 = torch.empty(512, 300)
    ct.binary_host(ct.MUL, A, B, o2)
    assert_bits_equal(o2.numpy(), oracle.binary(ol.MUL, HostView.contig(A.numpy()), HostView.contig(B.numpy())))
    r = torch.empty(300)
    ct.reduce_host(ct.SUM, A, 0, r)
    assert_close(r.numpy(), oracle.reduce(ol.SUM, HostView.contig(A.numpy()), 0), RTOL)


# ---- size-independent properties at benchmark scale -----------------------------------------------------------------
def test_large_properties(ct):
    n = 1 << 28                                   # 1 GiB per tensor
    x = torch.randn(n, device="cuda")
    y = torch.randn(n, device="cuda")
    s = ct.binary(ct.ADD, x, y)
    back = ct.binary(ct.SUB, s, y)                # (x + y) - y == x up to one rounding of x+y
    err = ct.reduce(ct.MAX, ct.unary(ct.ABS, ct.binary(ct.SUB, back, x)), -1).item()
    assert err < 1e-5
    del back
    # commutativity is exact
    s2 = ct.binary(ct.ADD, y, x)
    assert ct.reduce(ct.SUM, ct.binary(ct.NE, s, s2), -1).item() == 0.0
    del s2
    # relu is idempotent and equals max(x, 0) expressed through compare+mul
    r = ct.unary(ct.RELU, x)
    assert ct.reduce(ct.SUM, ct.binary(ct.NE, ct.unary(ct.RELU, r), r), -1).item() == 0.0
    assert ct.reduce(ct.MIN, r, -1).item() == 0.0
    # checksum of checksums: full sum == sum of row sums == sum of column sums (fp64 accumulation)
    m = x.view(1 << 14, 1 << 14)
    full = ct.reduce(ct.SUM, x, -1).item()
    rows = ct.reduce(ct.SUM, ct.reduce(ct.SUM, m, 1), -1).item()
    cols = ct.reduce(ct.SUM, ct.reduce(ct.SUM, m, 0), -1).item()
    scale = abs(full) + n ** 0.5
    assert abs(full - rows) < 1e-5 * scale and abs(full - cols) < 1e-5 * scale
    # max over everything == max of row maxima == max of column maxima, exactly
    mx = ct.reduce(ct.MAX, x, -1).item()
    assert mx == ct.reduce(ct.MAX, ct.reduce(ct.MAX, m, 1), -1).item() == ct.reduce(ct.MAX, ct.reduce(ct.MAX, m, 0), -1).item()
    # argmax points at the maximum
    am = ct.reduce(ct.ARGMAX, m, 1)
    picked = m.gather(1, am.long().view(-1, 1)).view(-1)          # torch used only to index the check
    assert torch.equal(picked, ct.reduce(ct.MAX, m, 1))


def test_errors_on_device(ct):
    a = torch.zeros(4, 3, device="cuda")
    b = torch.zeros(4, 2, device="cuda")
    with pytest.raises(ct.CtbError) as e:
        ct.binary(ct.ADD, a, b, out=torch.zeros(4, 3, device="cuda"))
    assert e.value.code == 2 and e.value.message == "Shape mismatch in binary op"
    with pytest.raises(ct.CtbError) as e:
        ct.reduce(ct.ARGMAX, a, 2)
    assert e.value.code == 4
    with pytest.raises(ct.CtbError) as e:
        ct.unary(ct.EXP, torch.zeros(4, dtype=torch.int32, device="cuda"))
    assert e.value.code == 3
    empty = ct.binary(ct.ADD, torch.zeros(0, 3, device="cuda"), torch.zeros(1, 3, device="cuda"))
    assert empty.shape == (0, 3)
