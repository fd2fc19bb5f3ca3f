"""GPU tests of the entry points that serve the callers either side of the operator path:
log-softmax rows (Loss::CrossEntropy), gather (Tensor::gather) and accumulate_grad (autograd).
The catalogue cases of these kinds run in test_gpu_parity.py; here are the shapes and edge
cases the catalogue does not hold."""
import numpy as np
import pytest
import torch

import oracle_lib as ol
from oracle_lib import HostView
from gpu_util import to_device, assert_bits_equal, assert_close

pytestmark = pytest.mark.gpu
RTOL = 1e-5


@pytest.mark.parametrize("cols", [1, 7, 128, 1000, 1024, 4096, 5000, 40000])
def test_log_softmax_widths(ct, oracle, cols):
    rows = 37 if cols < 10000 else 3
    x = HostView.contig((np.random.default_rng(cols).standard_normal((rows, cols)) * 4).astype(np.float32))
    got = ct.log_softmax(to_device(x)).cpu().numpy()
    ref = oracle.log_softmax(x)
    np.testing.assert_allclose(got, ref, rtol=RTOL, atol=1e-6)


def test_log_softmax_is_log_of_softmax(ct):
    x = torch.randn(64, 50257 // 8, device="cuda") * 3
    ls = ct.log_softmax(x)
    sm = ct.softmax(x)
    assert torch.allclose(ls.exp(), sm, rtol=1e-5, atol=1e-9)
    assert torch.allclose(ls.exp().sum(-1), torch.ones(64, device="cuda"), rtol=1e-5)


def test_log_softmax_rejects_what_softmax_rejects(ct):
    with pytest.raises(ct.CtbError):
        ct.log_softmax(torch.zeros(4, 4, dtype=torch.float64, device="cuda"))


def test_cross_entropy_chain(ct, oracle):
    """Loss::CrossEntropy (src/neuralnet/loss.cpp:90-118): log-softmax, gather the target's
    log-probability, negate, mean."""
    rng = np.random.default_rng(3)
    logits = HostView.contig((rng.standard_normal((256, 1000)) * 2).astype(np.float32))
    target = HostView.contig(rng.integers(0, 1000, (256, 1)).astype(np.int32))
    lp = ct.log_softmax(to_device(logits))
    picked = ct.gather(lp, 1, to_device(target))
    nll = ct.unary(ct.MUL_S, picked, -1.0)
    loss = ct.reduce(ct.MEAN, nll, ct.DIM_FULL).cpu().numpy()
    ref_lp = oracle.log_softmax(logits)
    ref_pick = oracle.gather(HostView.contig(ref_lp), 1, target)
    ref = oracle.reduce(ol.MEAN, HostView.contig(oracle.unary(ol.MUL_S, HostView.contig(ref_pick), -1.0)), -1)
    np.testing.assert_allclose(loss, ref, rtol=RTOL)


def test_gather_out_of_bounds_is_reported(ct):
    x = torch.arange(12, dtype=torch.float32, device="cuda").reshape(3, 4)
    idx = torch.tensor([[0], [4], [1]], dtype=torch.int32, device="cuda")
    with pytest.raises(ct.CtbError) as e:
        ct.gather(x, 1, idx)
    assert e.value.code == 4 and "Gather index out of bounds" in e.value.message
    idx = torch.tensor([[0], [-5], [1]], dtype=torch.int32, device="cuda")
    with pytest.raises(ct.CtbError):
        ct.gather(x, 1, idx)
    # the reference's argument checks
    with pytest.raises(ct.CtbError) as e:
        ct.gather(x, 2, idx)
    assert e.value.code == 4
    with pytest.raises(ct.CtbError) as e:
        ct.gather(x, 1, idx.float())
    assert "Index tensor must be integer type" in e.value.message
    with pytest.raises(ct.CtbError) as e:
        ct.gather(x, 1, torch.zeros(5, 1, dtype=torch.int32, device="cuda"))
    assert "Index shape dimension mismatch" in e.value.message


@pytest.mark.parametrize("index_dtype", ["int64", "int16", "uint8", "int8"])
@pytest.mark.parametrize("x_dtype", ["float32", "float64", "int16", "uint8", "int64"])
def test_gather_any_integer_index_and_element_size(ct, index_dtype, x_dtype):
    """The reference reads indices through double from any integer dtype (src/core/tensor.cpp:385-386) and
    moves elements of any size."""
    torch.manual_seed(11)
    x = (torch.randn(64, 100, device="cuda") * 50).to(getattr(torch, x_dtype))
    idx = torch.randint(0, 100, (64, 37), device="cuda").to(getattr(torch, index_dtype))
    got = ct.gather(x.t(), 0, idx.t().contiguous())          # a strided source as well
    assert torch.equal(got, torch.gather(x.t(), 0, idx.t().long()))
    assert torch.equal(ct.gather(x, 1, idx), torch.gather(x, 1, idx.long()))


def test_gather_large_matches_torch(ct):
    x = torch.randn(4096, 512, device="cuda")
    idx = torch.randint(0, 512, (4096, 64), device="cuda", dtype=torch.int32)
    got = ct.gather(x, 1, idx)
    assert torch.equal(got, torch.gather(x, 1, idx.long()))


@pytest.mark.parametrize("tshape,sshape", [
    ((16,), (5, 7, 16)),             # two leading dims fold together (contiguous source)
    ((7, 1), (5, 7, 16)),            # folds on both sides of a kept dim
    ((1, 7, 16), (5, 7, 16)),
    ((5, 1, 16), (5, 7, 16)),
    ((1, 1, 1), (5, 7, 16)),
    ((1,), (33,)),
    ((5, 7, 16), (7, 16)),           # the source broadcasts into the target
    ((3, 5), (1, 5)),
])
def test_accumulate_grad_folds(ct, oracle, tshape, sshape):
    rng = np.random.default_rng(len(tshape) * 100 + len(sshape))
    g0 = rng.standard_normal(tshape).astype(np.float32)
    src = HostView.contig(rng.standard_normal(sshape).astype(np.float32))
    grad = torch.from_numpy(g0.copy()).cuda()
    ct.accumulate_grad(grad, to_device(src))
    ref = oracle.accumulate_grad(g0, src)
    np.testing.assert_allclose(grad.cpu().numpy(), ref, rtol=RTOL, atol=1e-6)


def test_accumulate_grad_strided_buffers(ct, oracle):
    """A gradient buffer that is a view (transposed / sliced) and a permuted source."""
    rng = np.random.default_rng(9)
    g0 = rng.standard_normal((48, 64)).astype(np.float32)
    src = HostView.contig(rng.standard_normal((64, 48)).astype(np.float32))
    store = torch.from_numpy(g0.copy()).cuda()
    grad_t = store.t()                                   # [64, 48] view with strides (1, 64)
    ct.accumulate_grad(ct.DView.of(grad_t), to_device(src))
    ref = oracle.accumulate_grad(np.ascontiguousarray(g0.T), src)
    assert_bits_equal(grad_t.contiguous(), ref, "transposed gradient buffer")
    # bias gradient into a sliced (non-contiguous) buffer
    wide = torch.zeros(48, 2, device="cuda")
    col = wide[:, 0]
    ct.accumulate_grad(ct.DView.of(col), to_device(src))
    ref = oracle.accumulate_grad(np.zeros(48, np.float32), src)
    np.testing.assert_allclose(col.cpu().numpy(), ref, rtol=RTOL, atol=1e-6)
    assert torch.all(wide[:, 1] == 0)


def test_accumulate_grad_twice_and_large(ct):
    g = torch.randn(8192, 4096, device="cuda")
    bias = torch.zeros(4096, device="cuda")
    ct.accumulate_grad(bias, g)
    ct.accumulate_grad(bias, g)
    want = 2 * g.double().sum(0)
    assert torch.allclose(bias.double(), want, rtol=1e-5, atol=1e-3)
    w = torch.zeros(8192, 4096, device="cuda")
    ct.accumulate_grad(w, g)
    assert torch.equal(w, g)


def test_accumulate_grad_shape_mismatch(ct):
    with pytest.raises(ct.CtbError) as e:
        ct.accumulate_grad(torch.zeros(3, 4, device="cuda"), torch.zeros(3, 5, device="cuda"))
    assert e.value.code == 2


def test_sgd_large_and_other_dtypes(ct, oracle):
    p = torch.randn(1 << 24, device="cuda")
    g = torch.randn(1 << 24, device="cuda")
    want = p - g * torch.tensor(0.05, dtype=torch.float32, device="cuda")     # two fp32 roundings, as the reference
    ct.sgd_step(p, g, 0.05)
    assert torch.equal(p, want)
    # odd length and a misaligned start (scalar path)
    base = torch.randn(1001 + 1, device="cuda")
    gb = torch.randn(1001 + 1, device="cuda")
    pv, gv = base[1:], gb[1:]
    want = pv - gv * torch.tensor(0.5, dtype=torch.float32, device="cuda")
    ct.sgd_step(ct.DView.of(pv), ct.DView.of(gv), 0.5)
    assert torch.equal(pv, want)
    for dt, npdt in ((torch.float64, np.float64), (torch.int32, np.int32)):
        p0 = (np.random.default_rng(1).standard_normal(77) * 10).astype(npdt)
        g0 = (np.random.default_rng(2).standard_normal(77) * 10).astype(npdt)
        pd, gd = torch.from_numpy(p0.copy()).cuda(), torch.from_numpy(g0).cuda()
        ct.sgd_step(pd, gd, 0.3)
        assert_bits_equal(pd, oracle.optimizer_steps(0, p0, g0, 1, 0.3), f"sgd {dt}")


def test_adam_trajectory_large(ct, oracle):
    rng = np.random.default_rng(4)
    p0 = rng.standard_normal(100003).astype(np.float32)
    g0 = (rng.standard_normal(100003) * 3).astype(np.float32)
    for kind, wd in ((1, None), (2, 0.05)):
        p, g = torch.from_numpy(p0.copy()).cuda(), torch.from_numpy(g0).cuda()
        m, v = torch.zeros_like(p), torch.zeros_like(p)
        for t in range(1, 6):
            ct.adam_step(p, g, m, v, 1e-3, t, weight_decay=wd)
        ref = oracle.optimizer_steps(kind, p0, g0, 5, 1e-3, weight_decay=0.05)
        assert_bits_equal(p, ref, f"adam kind {kind}")


def test_optimizer_argument_checks(ct):
    p = torch.zeros(8, device="cuda")
    with pytest.raises(ct.CtbError) as e:
        ct.sgd_step(p, torch.zeros(9, device="cuda"), 0.1)
    assert e.value.code == 2
    with pytest.raises(ct.CtbError) as e:
        ct.sgd_step(ct.DView.of(torch.zeros(8, 2, device="cuda")[:, 0]), p, 0.1)
    assert "contiguous" in e.value.message
    with pytest.raises(ct.CtbError) as e:
        ct.adam_step(p.double(), p.double(), p, p, 0.1, 1)
    assert e.value.code == 3
    with pytest.raises(ct.CtbError) as e:
        ct.adam_step(p, p, p, p, 0.1, 0)
    assert e.value.code == 5


def test_cat_matches_torch_and_copy_into_slices(ct):
    a = torch.randn(300, 257, device="cuda")
    b = torch.randn(300, 1023, device="cuda")
    c = torch.randn(300, 4, device="cuda")
    assert torch.equal(ct.cat([a, b, c], 1), torch.cat([a, b, c], 1))
    assert torch.equal(ct.cat([a, a.flip(0).contiguous()], 0), torch.cat([a, a.flip(0)], 0))
    big = torch.randn(8, 1024, 3072, device="cuda")
    assert torch.equal(ct.cat([big, big], 2), torch.cat([big, big], 2))
    p = torch.randn(16, 64, 12, 32, device="cuda").permute(0, 2, 1, 3)
    assert torch.equal(ct.cat([p, p], 1), torch.cat([p, p], 1))
    # copy_into: a strided destination, a broadcast source
    dst = torch.zeros(64, 96, device="cuda")
    ct.copy_into(torch.arange(32, dtype=torch.float32, device="cuda").reshape(1, 32), ct.DView.of(dst[:, 32:64]))
    assert torch.equal(dst[:, 32:64], torch.arange(32, dtype=torch.float32, device="cuda").expand(64, 32))
    assert float(dst[:, :32].abs().sum()) == 0 and float(dst[:, 64:].abs().sum()) == 0
    ct.copy_into(a.t(), ct.DView.of(torch.empty(257, 300, device="cuda")))


def test_cat_errors(ct):
    a = torch.zeros(2, 3, device="cuda")
    for bad, code, text in (([a, torch.zeros(2, 3, 1, device="cuda")], 2, "cat_mp: ndim mismatch"),
                            ([a, torch.zeros(3, 4, device="cuda")], 2, "cat_mp: shape mismatch outside cat dim"),
                            ([a, a.double()], 3, "cat_mp: dtype mismatch")):
        with pytest.raises(ct.CtbError) as e:
            ct.cat(bad, 0)
        assert e.value.code == code and text in e.value.message
    with pytest.raises(ct.CtbError) as e:
        ct.cat([a], 2)
    assert e.value.code == 4


@pytest.mark.parametrize("shape", [(64, 256, 28, 28), (32, 64, 7, 7), (16, 3, 33, 65), (4096, 512), (1000, 37),
                                   (8, 20000, 16), (3, 5, 2, 2, 6), (5, 7, 24), (3, 50, 8, 33)])
def test_batchnorm_forward_shapes(ct, shape):
    torch.manual_seed(len(shape) * 7 + shape[1])
    x = torch.randn(*shape, device="cuda") * 1.5 + 0.5
    c = shape[1]
    dims = [d for d in range(len(shape)) if d != 1]
    mean, var = ct.channel_moments(x)
    xd = x.double()
    assert torch.allclose(mean.double(), xd.mean(dims), rtol=1e-5, atol=1e-6)
    assert torch.allclose(var.double(), xd.var(dims, unbiased=False), rtol=1e-5, atol=1e-7)
    gamma = 1 + 0.1 * torch.randn(c, device="cuda")
    beta = 0.1 * torch.randn(c, device="cuda")
    y = ct.batchnorm_apply(x, mean, var, gamma, beta, 1e-5)
    bshape = [1, c] + [1] * (len(shape) - 2)
    want = (xd - mean.double().view(bshape)) / torch.sqrt(var.double().view(bshape) + 1e-5) * gamma.double().view(bshape) + beta.double().view(bshape)
    assert torch.allclose(y.double(), want, rtol=2e-5, atol=2e-6)
    # parameters given as [1, C, 1, ...] views, no affine part
    y2 = ct.batchnorm_apply(x, mean.view(bshape), var.view(bshape), None, None, 1e-5)
    want2 = (xd - mean.double().view(bshape)) / torch.sqrt(var.double().view(bshape) + 1e-5)
    assert torch.allclose(y2.double(), want2, rtol=2e-5, atol=2e-6)


def test_batchnorm_matches_oracle_bitwise_on_apply(ct, oracle):
    rng = np.random.default_rng(12)
    x = rng.standard_normal((9, 6, 10, 12)).astype(np.float32)
    mean = rng.standard_normal(6).astype(np.float32)
    var = (np.abs(rng.standard_normal(6)) + 0.2).astype(np.float32)
    g = rng.standard_normal(6).astype(np.float32)
    b = rng.standard_normal(6).astype(np.float32)
    got = ct.batchnorm_apply(*(torch.from_numpy(a).cuda() for a in (x, mean, var, g, b)), 1e-5)
    ref = oracle.batchnorm_apply(x, mean, var, g, b, 1e-5)
    np.testing.assert_allclose(got.cpu().numpy(), ref, rtol=1e-6, atol=0)      # pow() may differ in the last bit


def test_batchnorm_argument_checks(ct):
    x = torch.zeros(4, 3, 5, device="cuda")
    with pytest.raises(ct.CtbError) as e:
        ct.channel_moments(x.permute(0, 2, 1))
    assert "contiguous" in e.value.message
    with pytest.raises(ct.CtbError) as e:
        ct.batchnorm_apply(x, torch.zeros(4, device="cuda"), torch.zeros(3, device="cuda"))
    assert e.value.code == 2
    with pytest.raises(ct.CtbError) as e:
        ct.channel_moments(torch.zeros(4, device="cuda"))
    assert e.value.code == 2


def test_matmul_large_is_bit_identical_to_the_scalar_reference_order(ct, oracle):
    rng = np.random.default_rng(21)
    a = HostView.contig(rng.standard_normal((257, 770)).astype(np.float32))
    b = HostView.contig(rng.standard_normal((770, 515)).astype(np.float32))
    got = ct.matmul(to_device(a), to_device(b))
    assert_bits_equal(got, oracle.matmul(a, b), "matmul 257x770x515")
    # batched, the right operand shared and transposed
    a3 = HostView.contig(rng.standard_normal((6, 100, 64)).astype(np.float32))
    bt = HostView.contig(rng.standard_normal((48, 64)).astype(np.float32)).permute([1, 0])
    assert_bits_equal(ct.matmul(to_device(a3), to_device(bt)), oracle.matmul(a3, bt), "batched matmul")


def test_matmul_errors(ct):
    x = torch.zeros(4, 5, device="cuda")
    with pytest.raises(ct.CtbError) as e:
        ct.matmul(x, x)
    assert "matmul_mp shape mismatch" in e.value.message
    with pytest.raises(ct.CtbError) as e:
        ct.matmul(torch.zeros(5, device="cuda"), x, out=torch.zeros(4, device="cuda"))
    assert "requires at least 2D" in e.value.message


def test_mlp_forward_loss_and_sgd_step_end_to_end(ct, oracle):
    """The reference's MNIST recipe (test/train_mnist.cpp: Linear -> ReLU -> Linear ->
    CrossEntropy, SGD) with every tensor operation on the device, against the same chain of
    oracle calls: forward activations and the loss, then the gradient of the last layer
    (softmax - onehot, bias gradient through accumulate_grad) and one SGD step."""
    rng = np.random.default_rng(33)
    B, D, H, C = 64, 784, 128, 10
    x = HostView.contig(rng.uniform(0, 1, (B, D)).astype(np.float32))
    w1 = HostView.contig((rng.standard_normal((D, H)) * 0.05).astype(np.float32))
    b1 = HostView.contig(np.zeros((1, H), np.float32))
    w2 = HostView.contig((rng.standard_normal((H, C)) * 0.05).astype(np.float32))
    b2 = HostView.contig((rng.standard_normal((1, C)) * 0.01).astype(np.float32))
    y = HostView.contig(rng.integers(0, C, (B, 1)).astype(np.int32))
    hv = lambda a: HostView.contig(a)

    # device
    dx, dw1, db1, dw2, db2, dy = (to_device(v) for v in (x, w1, b1, w2, b2, y))
    h = ct.unary(ct.RELU, ct.binary(ct.ADD, ct.matmul(dx, dw1), db1))
    logits = ct.binary(ct.ADD, ct.matmul(h, dw2), db2)
    logp = ct.log_softmax(logits)
    loss = ct.reduce(ct.MEAN, ct.unary(ct.MUL_S, ct.gather(logp, 1, dy), -1.0), ct.DIM_FULL)
    # oracle
    oh = oracle.unary(ol.RELU, hv(oracle.binary(ol.ADD, hv(oracle.matmul(x, w1)), b1)))
    ologits = oracle.binary(ol.ADD, hv(oracle.matmul(hv(oh), w2)), b2)
    ologp = oracle.log_softmax(hv(ologits))
    oloss = oracle.reduce(ol.MEAN, hv(oracle.unary(ol.MUL_S, hv(oracle.gather(hv(ologp), 1, y)), -1.0)), -1)
    assert_bits_equal(h, oh, "hidden activations")
    assert_bits_equal(logits, ologits, "logits")
    assert_close(logp, ologp, RTOL, "log-probabilities")
    assert_close(loss, oloss, RTOL, "loss")

    # d loss / d logits = (softmax - onehot) / B ; bias gradient = its column sums ; SGD step on b2
    onehot = torch.zeros(B, C, device="cuda")
    onehot.scatter_(1, torch.from_numpy(y.numpy()).cuda().long(), 1.0)
    dlogits = ct.unary(ct.MUL_S, ct.binary(ct.SUB, ct.softmax(logits), onehot), 1.0 / B)
    gb2 = torch.zeros(1, C, device="cuda")
    ct.accumulate_grad(gb2, dlogits)
    new_b2 = torch.from_numpy(b2.numpy()).cuda()
    ct.sgd_step(new_b2, gb2, 0.1)
    od = oracle.unary(ol.MUL_S, hv(oracle.binary(ol.SUB, hv(oracle.softmax(hv(ologits))), hv(onehot.cpu().numpy()))), 1.0 / B)
    ogb2 = oracle.accumulate_grad(np.zeros((1, C), np.float32), hv(od))
    onew = oracle.optimizer_steps(0, b2.numpy(), ogb2, 1, 0.1)
    np.testing.assert_allclose(gb2.cpu().numpy(), ogb2, rtol=1e-4, atol=1e-7)
    np.testing.assert_allclose(new_b2.cpu().numpy(), onew, rtol=1e-5, atol=1e-7)


@pytest.mark.parametrize("cols", [8196, 12289, 16384, 30001, 50257, 65536, 100003, 250000])
def test_softmax_long_rows_cluster_kernel(ct, oracle, cols):
    """Rows beyond the register kernels, aligned and unaligned row starts: plain rows through the
    three-sweep kernels (512 threads, 1024 beyond 57344 columns), masked and causal ones staged in the
    shared memory of a thread-block cluster; softmax of 98305 .. 204800 columns on the clusters too."""
    rng = np.random.default_rng(cols)
    x = HostView.contig((rng.standard_normal((5, cols)) * 3).astype(np.float32))
    np.testing.assert_allclose(ct.softmax(to_device(x)).cpu().numpy(), oracle.softmax(x), rtol=RTOL, atol=1e-12)
    np.testing.assert_allclose(ct.log_softmax(to_device(x)).cpu().numpy(), oracle.log_softmax(x), rtol=RTOL, atol=1e-6)
    if cols <= 30001:
        m = HostView.contig(-rng.random((1, cols)).astype(np.float32))
        np.testing.assert_allclose(ct.softmax(to_device(x), to_device(m)).cpu().numpy(), oracle.softmax(x, m), rtol=RTOL, atol=1e-12)
        sq = HostView.contig(rng.standard_normal((2, 3, 8, cols)).astype(np.float32)[:, :, :, :])
        got = ct.softmax(to_device(sq), None, causal=True).cpu().numpy()
        ref = oracle.softmax(sq, None, causal=True)
        np.testing.assert_allclose(got, ref, rtol=RTOL, atol=1e-12)


@pytest.mark.parametrize("cols", [8196, 12288, 16384, 16388, 30000, 32768, 32772, 40001, 50257, 131075])
def test_layernorm_long_rows(ct, oracle, cols):
    """LayerNorm rows beyond the register kernels: the three-sweep kernel, aligned and unaligned rows."""
    rng = np.random.default_rng(cols)
    x = HostView.contig((rng.standard_normal((7, cols)) * 2 + 0.3).astype(np.float32))
    g = HostView.contig((1 + 0.02 * rng.standard_normal(cols)).astype(np.float32))
    b = HostView.contig((0.02 * rng.standard_normal(cols)).astype(np.float32))
    got = ct.layernorm(to_device(x), to_device(g), to_device(b), 1e-5).cpu().numpy()
    np.testing.assert_allclose(got, oracle.layernorm(x, g, b, 1e-5), rtol=RTOL, atol=1e-6)
    got = ct.layernorm(to_device(x), None, None, 1e-5).cpu().numpy()
    np.testing.assert_allclose(got, oracle.layernorm(x, None, None, 1e-5), rtol=RTOL, atol=1e-6)


def test_empty_and_degenerate_inputs(ct):
    """Zero-sized tensors and extents of one go through the caller-side entry points without a
    launch error and give the obvious results."""
    dev = "cuda"
    z = torch.zeros(0, 5, device=dev)
    assert ct.log_softmax(z).shape == (0, 5)
    assert ct.softmax(z).shape == (0, 5)
    assert ct.cat([z, torch.ones(2, 5, device=dev)], 0).shape == (2, 5)
    assert ct.cat([torch.ones(3, 0, device=dev), torch.ones(3, 2, device=dev)], 1).shape == (3, 2)
    assert ct.gather(torch.ones(4, 3, device=dev), 1, torch.zeros(4, 0, dtype=torch.int32, device=dev)).shape == (4, 0)
    g = torch.ones(5, device=dev)
    ct.accumulate_grad(g, torch.zeros(0, 5, device=dev))            # nothing to add
    assert torch.equal(g, torch.ones(5, device=dev))
    k0 = ct.matmul(torch.ones(3, 0, device=dev), torch.ones(0, 4, device=dev))
    assert k0.shape == (3, 4) and float(k0.abs().sum()) == 0.0      # empty sums are zero
    one = torch.full((1, 1), 3.0, device=dev)
    assert float(ct.softmax(one)) == 1.0 and float(ct.log_softmax(one)) == 0.0
    assert float(ct.matmul(one, one)) == 9.0
    p = torch.zeros(0, device=dev)
    ct.sgd_step(p, p, 0.1)
    ct.adam_step(p, p, p, p, 0.1, 1)
    m, v = ct.channel_moments(torch.full((2, 3, 1), 5.0, device=dev))
    assert torch.equal(m, torch.full((3,), 5.0, device=dev)) and float(v.abs().sum()) == 0.0
    torch.cuda.synchronize()


# ---- matmul on the tensor cores (tcgen05, TF32 products) ---------------------------------------------------
@pytest.mark.parametrize("m,n,k,b_is_transposed_view", [
    (128, 128, 32, True), (128, 128, 128, False), (256, 384, 64, True), (300, 200, 100, False), (300, 200, 100, True),
    (1000, 1000, 1000, True), (77, 129, 513, False), (1, 130, 40, True), (4096, 512, 2048, True), (64, 64, 1, False),
    # enough tiles for the 256-wide tile to be chosen, ragged in every dim; several tiles per CTA (both
    # accumulators reused, the load ring running across tile boundaries) for either tile width
    (1300, 1800, 100, True), (1300, 1801, 72, False), (2048, 2048, 256, True), (4096, 4096, 96, True),
    (80000, 100, 40, True), (5000, 129, 33, False)])
def test_matmul_tensor_cores_within_the_tf32_tolerance(ct, oracle, m, n, k, b_is_transposed_view):
    """|out - exact| <= 2^-9 * sum_k |a_ik b_kj|: every product is formed from the operands' upper 19 bits.
    The exact value is the fp64 product; the reference's own fp32 GEMMs lie within 1e-6 of it."""
    rng = np.random.default_rng(m * 7 + n * 3 + k)
    a = rng.standard_normal((m, k)).astype(np.float32)
    if b_is_transposed_view:                       # b = W^T for a weight matrix W[n, k]: what Linear::forward passes
        w = rng.standard_normal((n, k)).astype(np.float32)
        b_host = w.T
        db = ct.DView.of(torch.from_numpy(w).cuda()).permute([1, 0])
    else:
        b_host = rng.standard_normal((k, n)).astype(np.float32)
        db = torch.from_numpy(b_host).cuda()
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    got = ct.matmul_tc(torch.from_numpy(a).cuda(), db, status=status).cpu().numpy()
    assert status.item() == 0, f"a wait inside the kernel gave up (code {status.item()})"
    exact = a.astype(np.float64) @ b_host.astype(np.float64)
    bound = 2.0 ** -9 * (np.abs(a).astype(np.float64) @ np.abs(b_host).astype(np.float64)) + 1e-30
    assert got.shape == (m, n)
    assert np.all(np.abs(got - exact) <= bound), float(np.max(np.abs(got - exact) / bound))
    # and against the bit-exact CUDA-core entry point (== matmul_mp of the reference)
    plain = ct.matmul(torch.from_numpy(a).cuda(), db).cpu().numpy()
    assert np.all(np.abs(got - plain) <= bound + 1e-5 * np.abs(plain))


def test_matmul_tensor_cores_batched_and_empty_k(ct):
    rng = np.random.default_rng(3)
    a = rng.standard_normal((3, 130, 72)).astype(np.float32)
    b = rng.standard_normal((72, 50)).astype(np.float32)              # shared by every batch entry
    got = ct.matmul_tc(torch.from_numpy(a).cuda(), torch.from_numpy(b).cuda()).cpu().numpy()
    exact = a.astype(np.float64) @ b.astype(np.float64)
    bound = 2.0 ** -9 * (np.abs(a).astype(np.float64) @ np.abs(b).astype(np.float64))
    assert np.all(np.abs(got - exact) <= bound)
    z = ct.matmul_tc(torch.zeros(5, 0, device="cuda"), torch.zeros(0, 7, device="cuda"))
    assert z.shape == (5, 7) and float(z.abs().max()) == 0.0
    with pytest.raises(ct.CtbError) as e:
        ct.matmul_tc(torch.zeros(4, 5, device="cuda"), torch.zeros(6, 7, device="cuda"))
    assert e.value.message == "matmul_mp shape mismatch"


@pytest.mark.parametrize("cols", [1000, 2048, 12288, 20000, 50257])
def test_rows_with_special_values_follow_the_reference_chain(ct, oracle, cols):
    """+inf, -inf, NaN and huge entries inside rows, for every row-kernel family (warp rows, thread
    groups, the three-sweep kernels): what the reference's chain of operators gives (max ignores a
    NaN, inf - inf is NaN, the exponential clamps its argument), element for element."""
    rng = np.random.default_rng(cols)
    x = (rng.standard_normal((8, cols)) * 3).astype(np.float32)
    x[1, cols // 3] = np.inf
    x[2, 5::7] = -np.inf
    x[3, cols // 2] = np.nan
    x[4, :] = 1e30
    x[5, :] = -np.inf
    x[6, 0] = np.inf
    x[6, cols - 1] = np.inf
    x[7, ::2] = 3e38
    hx = HostView.contig(x)
    with np.errstate(all="ignore"):
        want_sm, want_lsm = oracle.softmax(hx), oracle.log_softmax(hx)
    got_sm = ct.softmax(to_device(hx)).cpu().numpy()
    got_lsm = ct.log_softmax(to_device(hx)).cpu().numpy()
    np.testing.assert_allclose(got_sm, want_sm, rtol=RTOL, atol=1e-12, equal_nan=True)
    np.testing.assert_allclose(got_lsm, want_lsm, rtol=RTOL, atol=1e-6, equal_nan=True)
    # the masked kernels (thread-block clusters for the long rows) on the same rows
    m = HostView.contig(-rng.random((1, cols)).astype(np.float32))
    with np.errstate(all="ignore"):
        want_masked = oracle.softmax(hx, m)
    np.testing.assert_allclose(ct.softmax(to_device(hx), to_device(m)).cpu().numpy(), want_masked, rtol=RTOL, atol=1e-12, equal_nan=True)


@pytest.mark.parametrize("cols", [1000, 2048, 12288, 20000, 50257])
def test_layernorm_and_cross_entropy_rows_with_special_values(ct, oracle, cols):
    """The same kinds of rows through LayerNorm and the cross-entropy kernels (register rows, the
    one-sweep loss, the three-sweep gradient)."""
    rng = np.random.default_rng(cols + 1)
    x = (rng.standard_normal((6, cols)) * 3).astype(np.float32)
    x[1, cols // 3] = np.inf
    x[2, 5::7] = -np.inf
    x[3, cols // 2] = np.nan
    x[4, :] = 1e30
    x[5, ::2] = 3e38
    hx = HostView.contig(x)
    g = HostView.contig((1 + 0.02 * rng.standard_normal(cols)).astype(np.float32))
    b = HostView.contig((0.02 * rng.standard_normal(cols)).astype(np.float32))
    with np.errstate(all="ignore"):
        want = oracle.layernorm(hx, g, b, 1e-5)
    got = ct.layernorm(to_device(hx), to_device(g), to_device(b), 1e-5).cpu().numpy()
    np.testing.assert_allclose(got, want, rtol=RTOL, atol=1e-6, equal_nan=True)
    labels = rng.integers(0, cols, (6, 1)).astype(np.int32)
    for row in range(6):                     # row by row: a NaN loss of one row would hide the others in the mean
        hr = HostView.contig(np.ascontiguousarray(x[row:row + 1]))
        hl = HostView.contig(np.ascontiguousarray(labels[row:row + 1]))
        with np.errstate(all="ignore"):
            want_loss = oracle.cross_entropy(hr, hl, True)
            want_grad = oracle.cross_entropy_backward(hr, hl, True, 1.0)
        got_loss = ct.cross_entropy(to_device(hr), to_device(hl), True).cpu().numpy()
        got_grad = ct.cross_entropy_backward(to_device(hr), to_device(hl), 1.0).cpu().numpy()
        np.testing.assert_allclose(got_loss, want_loss, rtol=RTOL, atol=1e-6, equal_nan=True, err_msg=f"loss of row {row}")
        np.testing.assert_allclose(got_grad, want_grad, rtol=max(RTOL, 4e-9 * cols), atol=1e-6, equal_nan=True, err_msg=f"gradient of row {row}")


@pytest.mark.parametrize("cols,pad,shift", [(20000, 3, 1), (50257, 0, 0), (50257, 5, 2), (17000, 4, 0), (70001, 1, 1), (33000, 2, 1)])
def test_long_rows_of_a_wider_buffer(ct, cols, pad, shift):
    """The three-sweep kernels on rows cut out of a wider buffer: input rows start at every 4-byte phase,
    and at a 16-byte phase that differs from the output row's (walked element by element) — softmax,
    log-softmax and LayerNorm against the definitions evaluated in float64."""
    rows = 11
    rng = np.random.default_rng(cols + pad + shift)
    wide = (rng.standard_normal((rows, cols + pad)) * 3 + 0.5).astype(np.float32)
    x = torch.from_numpy(wide).cuda()[:, shift:shift + cols]
    xs = wide[:, shift:shift + cols].astype(np.float64)
    sh = xs - xs.max(1, keepdims=True)
    logz = np.log(np.exp(sh).sum(1, keepdims=True))
    np.testing.assert_allclose(ct.softmax(ct.DView.of(x)).cpu().numpy(), np.exp(sh - logz), rtol=2e-5, atol=1e-12)
    np.testing.assert_allclose(ct.log_softmax(ct.DView.of(x)).cpu().numpy(), sh - logz, rtol=2e-5, atol=2e-6)
    gamma = (1 + 0.02 * rng.standard_normal(cols)).astype(np.float32)
    beta = (0.02 * rng.standard_normal(cols)).astype(np.float32)
    mu = xs.mean(1, keepdims=True)
    var = ((xs - mu) ** 2).mean(1, keepdims=True)
    want = (xs - mu) / np.sqrt(var + 1e-5) * gamma + beta
    got = ct.layernorm(ct.DView.of(x), torch.from_numpy(gamma).cuda(), torch.from_numpy(beta).cuda(), 1e-5)
    np.testing.assert_allclose(got.cpu().numpy(), want, rtol=2e-5, atol=2e-6)
    got = ct.layernorm(ct.DView.of(x), None, None, 1e-5)
    np.testing.assert_allclose(got.cpu().numpy(), (xs - mu) / np.sqrt(var + 1e-5), rtol=2e-5, atol=2e-6)


def test_batchnorm_with_special_values_follows_the_reference_chain(ct, oracle):
    """Channels that hold +inf, -inf, NaN or huge values: moments and normalised output as the
    reference's operator chain gives them (NaN and inf propagate through the sums; the other channels
    are untouched)."""
    rng = np.random.default_rng(77)
    x = rng.standard_normal((6, 7, 5, 8)).astype(np.float32)
    x[1, 1, 2, 3] = np.inf
    x[2, 2, 0, 0] = -np.inf
    x[3, 3, 4, 7] = np.nan
    x[:, 4] = 1e30
    x[0, 5, 1, 1] = 3e38
    x[5, 5, 1, 1] = 3e38
    with np.errstate(all="ignore"):
        want_mean, want_var = oracle.channel_moments(x)
    mean, var = ct.channel_moments(torch.from_numpy(x).cuda())
    np.testing.assert_allclose(mean.cpu().numpy().ravel(), np.asarray(want_mean).ravel(), rtol=RTOL, atol=1e-6, equal_nan=True)
    np.testing.assert_allclose(var.cpu().numpy().ravel(), np.asarray(want_var).ravel(), rtol=RTOL, atol=1e-6, equal_nan=True)
    g = rng.standard_normal(7).astype(np.float32)
    b = rng.standard_normal(7).astype(np.float32)
    m_in, v_in = np.asarray(want_mean, np.float32).ravel(), np.asarray(want_var, np.float32).ravel()
    with np.errstate(all="ignore"):
        want = oracle.batchnorm_apply(x, m_in, v_in, g, b, 1e-5)
    got = ct.batchnorm_apply(*(torch.from_numpy(a).cuda() for a in (x, m_in, v_in, g, b)), 1e-5)
    np.testing.assert_allclose(got.cpu().numpy(), want, rtol=1e-6, atol=0, equal_nan=True)
