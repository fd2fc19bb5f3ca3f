// Tests of the C++ host layer, written the way the reference's own unit tests are
// (test/test_ops.cpp and test/test.cpp there: plain main(), known answers), against the same
// operator names.  Needs a CUDA device; prints "ALL PASSED" and exits 0 on success.
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <stdexcept>
#include <string>

#include "ctb_host.h"
#include "../../include/ctb200.h"
#include "ops_dispatch.h"
#include "opsmp.h"

static int g_checks = 0;
#define CHECK(cond)                                                                  \
    do {                                                                             \
        ++g_checks;                                                                  \
        if (!(cond)) { std::fprintf(stderr, "FAILED %s:%d: %s\n", __FILE__, __LINE__, #cond); std::exit(1); } \
    } while (0)
#define CHECK_NEAR(a, b, eps) CHECK(std::fabs(double(a) - double(b)) <= (eps))
#define CHECK_THROWS(expr, type, text)                                               \
    do {                                                                             \
        bool ok = false;                                                             \
        try { (void)(expr); } catch (const type& e) { ok = std::string(e.what()) == (text); } \
        CHECK(ok);                                                                   \
    } while (0)

struct GradFn { std::string op; size_t n_inputs; double scalar; };   // a stand-in autograd node

int main() {
    // factories and shapes (reference test/test_ops.cpp:41-61)
    Tensor ones = Tensor::ones({2, 3});
    CHECK(ones.numel() == 6);
    CHECK_NEAR(ones[0][0], 1.0, 1e-5);
    CHECK_NEAR(ones[1][2], 1.0, 1e-5);
    Tensor f = Tensor::full({2, 2}, 3.14);
    CHECK_NEAR(f[1][1], 3.14, 1e-5);
    Tensor r = Tensor::arange(0, 5, 1, DType::Float32);
    CHECK(r.numel() == 5);
    CHECK_NEAR(r[4], 4.0, 1e-5);

    // arithmetic (test/test_ops.cpp:63-85)
    Tensor a = Tensor::full({2, 2}, 2.0), b = Tensor::full({2, 2}, 3.0);
    CHECK_NEAR((a + b)[0][0], 5.0, 1e-5);
    CHECK_NEAR((b - a)[1][1], 1.0, 1e-5);
    CHECK_NEAR((a * b)[0][1], 6.0, 1e-5);
    CHECK_NEAR((a / b)[1][0], 2.0 / 3.0, 1e-5);
    CHECK_NEAR(div_scalar(a, 4.0)[0][0], 0.5, 1e-6);
    CHECK_NEAR((a / 4.0)[0][0], 2.0 - 4.0, 1e-6);          // Tensor / double is sub_scalar, as in the reference's header (ops_dispatch.h:84)
    CHECK_NEAR((1.0 - a)[0][0], -1.0, 1e-6);

    // reductions (test/test_ops.cpp:113-128): dim = -1 reduces everything to shape {1}
    Tensor t = Tensor::from_vector({1, 2, 3, 4}, {2, 2});
    CHECK(sum(t).numel() == 1);
    CHECK_NEAR(sum(t).item<double>(), 10.0, 1e-5);
    CHECK_NEAR(mean(t).item<double>(), 2.5, 1e-5);
    CHECK_NEAR(max(t).item<double>(), 4.0, 1e-5);
    CHECK_NEAR(min(t).item<double>(), 1.0, 1e-5);
    Tensor s1 = sum(t, 1);
    CHECK(s1.shape() == std::vector<size_t>({2}));
    CHECK_NEAR(s1[0], 3.0, 1e-6);
    CHECK_NEAR(s1[1], 7.0, 1e-6);
    CHECK_NEAR(sum_mp(t)[1], 7.0, 1e-6);                 // *_mp: -1 means the last dim
    CHECK_NEAR(var(t, 0)[0], 1.0, 1e-6);
    Tensor am = argmax(Tensor::from_vector({5, 7, 7, 1}, {1, 4}), 1);
    CHECK(am._dtype() == DType::Int32 && (int)double(am[0]) == 1);
    CHECK((int)double(argmax(t, -1)[0]) == 1);           // negative dim wraps

    // broadcasting (test/test_ops.cpp:130-149)
    Tensor br = Tensor::ones({2, 2}) + Tensor::full({1, 2}, 2.0);
    CHECK(br.shape() == std::vector<size_t>({2, 2}));
    CHECK_NEAR(br[1][1], 3.0, 1e-6);
    CHECK((Tensor::full({1, 1}, 2.0) + Tensor::full({1}, 1.0)).shape() == std::vector<size_t>({1}));

    // views (test/test_ops.cpp:151-173, test/test.cpp:54-115)
    Tensor m = Tensor::from_vector({0, 1, 2, 3, 4, 5}, {2, 3});
    Tensor p = m.permute({1, 0});
    CHECK(p.shape() == std::vector<size_t>({3, 2}) && !p.is_contiguous());
    CHECK_NEAR(p[2][1], 5.0, 1e-6);
    CHECK(p.impl->data.get() == m.impl->data.get());     // a view: same storage
    Tensor pc = p.contiguous();
    CHECK(pc.is_contiguous());
    CHECK_NEAR(pc[1][0], 1.0, 1e-6);
    CHECK_NEAR(pc[1][1], 4.0, 1e-6);
    CHECK_NEAR(p.reshape({6})[3], 4.0, 1e-6);            // reshape of a permuted view repacks
    CHECK_NEAR(m.flatten()[5], 5.0, 1e-6);
    CHECK_NEAR((p + Tensor::full({3, 2}, 1.0))[2][0], 3.0, 1e-6);   // strided operand through the GPU
    CHECK_NEAR(sum(p, 0)[1], 12.0, 1e-6);
    CHECK_NEAR(m.select(0, 1)[2], 5.0, 1e-6);
    CHECK(m.unsqueeze(0).shape() == std::vector<size_t>({1, 2, 3}));
    CHECK(m.unsqueeze(0).squeeze().shape() == std::vector<size_t>({2, 3}));
    m[0][0] = 9.0;
    CHECK_NEAR(p[0][0], 9.0, 1e-6);                      // writes through the proxy hit shared storage

    // unary flavours and edge values
    Tensor x = Tensor::from_vector({-1.0, 0.0, 0.5, 100.0}, {4});
    CHECK_NEAR(relu(x)[0], 0.0, 0.0);
    CHECK_NEAR(exp(x)[2], std::exp(0.5), 1e-6);
    CHECK(double(exp(x)[3]) > 2.4e38 && double(exp(x)[3]) < 2.41e38);   // the Cephes clamp, not inf
    CHECK_NEAR(tanh(x)[0], std::tanh(-1.0), 1e-6);
    CHECK_NEAR(ln(Tensor::full({1}, 1.5))[0], 0.405465, 1e-6);
    CHECK_NEAR(gelu(x)[2], 0.345714, 1e-5);
    CHECK_NEAR((x > 0.25)[2], 1.0, 0.0);
    CHECK((x > 0.25)._dtype() == DType::Float32);        // comparisons answer in the input dtype

    // the *_mp names of src/core/opsmp.h
    CHECK_NEAR(add_mp(a, b)[0][0], 5.0, 1e-6);
    CHECK_NEAR(diff_mp(b, a)[0][0], 1.0, 1e-6);
    CHECK_NEAR(mult_mp(a, b)[1][1], 6.0, 1e-6);
    CHECK_NEAR(Relu_mp(x)[0], 0.0, 0.0);
    CHECK_NEAR(exp_mp(x)[1], 1.0, 0.0);
    CHECK_NEAR(mult_scalar_mp(a, 1.5)[0][0], 3.0, 1e-6);

    // integer semantics (test/test_ops.cpp:203-213): truncation
    Tensor i3 = Tensor::from_vector({3, 5}, {2}, DType::Int32);
    CHECK((int)double(div_scalar(i3, 2.0)[0]) == 1 && (int)double(div_scalar(i3, 2.0)[1]) == 2);
    CHECK((int)double(Tensor::from_vector({1.5, 2.5}, {2}).astype(DType::Int32)[1]) == 2);

    // element types of the reference's scalar back-end: served under the *_mp names (through double,
    // stored like x86's static_cast), refused under the dispatcher's names like the reference does
    Tensor u8a = Tensor::from_vector({200, 100, 7, 0}, {2, 2}, DType::UInt8);
    Tensor u8b = Tensor::from_vector({100, 100, 2, 0}, {2, 2}, DType::UInt8);
    Tensor u8s = add_mp(u8a, u8b);
    CHECK(u8s._dtype() == DType::UInt8 && (int)double(u8s[0][0]) == 44 && (int)double(u8s[0][1]) == 200);   // 300 -> 44
    CHECK((int)double(div_mp(u8a, Tensor::from_vector({3, 3, 3, 3}, {2, 2}, DType::UInt8))[1][0]) == 2);
    Tensor i64 = Tensor::from_vector({1e12, -3.0}, {2}, DType::Int64);
    CHECK(double(mult_scalar_mp(i64, 2.0)[0]) == 2e12 && double(abs_mp(i64)[1]) == 3.0);
    CHECK((int)double(sum_mp(Tensor::from_vector({1, 2, 3, 4, 5, 6}, {2, 3}, DType::Int16), 1)[1]) == 15);
    CHECK(double(u8a.permute({1, 0}).contiguous()[0][1]) == 7.0);
    CHECK_THROWS(add(u8a, u8b), std::runtime_error, "add: unsupported dtype or op not registered");
    CHECK_THROWS(add_mp(Tensor::from_vector({1, 2}, {2}, DType::UInt16), Tensor::from_vector({1, 2}, {2}, DType::UInt16)),
                 std::runtime_error, "add: unsupported dtype or op not registered");

    // fused rows
    Tensor sm = softmax(Tensor::from_vector({1, 2, 3, 1, 1, 1}, {2, 3}));
    CHECK_NEAR(double(sm[0][0]) + double(sm[0][1]) + double(sm[0][2]), 1.0, 1e-6);
    CHECK_NEAR(sm[1][2], 1.0 / 3.0, 1e-6);
    Tensor cs = causal_softmax(Tensor::ones({2, 2}));
    CHECK_NEAR(cs[0][0], 1.0, 0.0);
    CHECK_NEAR(cs[0][1], 0.0, 0.0);
    CHECK_NEAR(cs[1][1], 0.5, 1e-6);
    Tensor ln_ = layer_norm(Tensor::from_vector({1, 2, 3, 4}, {1, 4}), Tensor::ones({4}), Tensor::zeros({4}));
    CHECK_NEAR(ln_[0][3], 1.5 / std::sqrt(1.25 + 1e-5), 1e-5);

    // the callers' side: CrossEntropy's chain (src/neuralnet/loss.cpp:97-110), gather, accumulate_grad
    Tensor logits = Tensor::from_vector({1, 2, 3, 1, 1, 1}, {2, 3});
    Tensor lsm = log_softmax(logits);
    CHECK_NEAR(lsm[1][0], std::log(1.0 / 3.0), 1e-6);
    CHECK_NEAR(std::exp(double(lsm[0][0])) + std::exp(double(lsm[0][1])) + std::exp(double(lsm[0][2])), 1.0, 1e-6);
    Tensor tgt = Tensor::from_vector({2, 0}, {2, 1}, DType::Int32);
    Tensor picked = lsm.gather(tgt, 1);
    CHECK(picked.numel() == 2);
    CHECK_NEAR(picked[0][0], double(lsm[0][2]), 0.0);
    CHECK_NEAR(picked[1][0], double(lsm[1][0]), 0.0);
    CHECK_NEAR(mean(picked * -1.0).item<double>(), -(double(lsm[0][2]) + double(lsm[1][0])) / 2, 1e-6);
    CHECK_NEAR(lsm.gather(Tensor::from_vector({2, 0}, {2, 1}, DType::Int64), 1)[0][0], double(lsm[0][2]), 0.0);     // any integer index dtype
    CHECK_NEAR(lsm.gather(Tensor::from_vector({1, 2}, {2, 1}, DType::UInt8), 1)[1][0], double(lsm[1][2]), 0.0);
    CHECK_THROWS(lsm.gather(Tensor::from_vector({3, 0}, {2, 1}, DType::Int32), 1), std::out_of_range, "Gather index out of bounds");
    CHECK_THROWS(lsm.gather(tgt, 2), std::out_of_range, "Gather dimension out of range");
    CHECK_THROWS(lsm.gather(Tensor::from_vector({0, 0}, {2, 1}), 1), std::runtime_error, "Index tensor must be integer type");
    Tensor bias_grad = Tensor::zeros({3});
    ctb_host::accumulate_grad(bias_grad, logits);            // [2,3] folds into [3]
    CHECK_NEAR(bias_grad[0], 2.0, 0.0);
    CHECK_NEAR(bias_grad[2], 4.0, 0.0);
    ctb_host::accumulate_grad(bias_grad, Tensor::full({3}, std::nan("")));   // NaN contributions are skipped
    CHECK_NEAR(bias_grad[1], 3.0, 0.0);

    Tensor c01 = cat({Tensor::from_vector({1, 2, 3, 4}, {2, 2}), Tensor::from_vector({5, 6}, {1, 2})}, 0);
    CHECK(c01.shape()[0] == 3 && c01.shape()[1] == 2);
    CHECK_NEAR(c01[2][1], 6.0, 0.0);
    Tensor c1 = cat_mp({Tensor::from_vector({1, 2, 3, 4}, {2, 2}), Tensor::from_vector({5, 6}, {2, 1})}, 1);
    CHECK(c1.shape()[1] == 3);
    CHECK_NEAR(c1[0][2], 5.0, 0.0);
    CHECK_NEAR(c1[1][0], 3.0, 0.0);
    CHECK_THROWS(cat({Tensor::ones({2, 2}), Tensor::ones({3, 3})}, 0), std::runtime_error, "cat_mp: shape mismatch outside cat dim");
    CHECK_THROWS(cat({}, 0), std::runtime_error, "cat_mp: empty list");

    // Linear::forward (src/neuralnet/layer.cpp:32-37): matmul + bias
    Tensor mx = Tensor::from_vector({1, 2, 3, 4, 5, 6}, {2, 3});
    Tensor mw = Tensor::from_vector({1, 0, 0, 1, 1, 1}, {3, 2});
    Tensor my = matmul_mp(mx, mw) + Tensor::from_vector({10, 20}, {1, 2});
    CHECK_NEAR(my[0][0], 14.0, 0.0);
    CHECK_NEAR(my[0][1], 25.0, 0.0);
    CHECK_NEAR(my[1][0], 20.0, 0.0);
    CHECK_NEAR(my[1][1], 31.0, 0.0);
    CHECK_THROWS(matmul(mx, mx), std::runtime_error, "matmul_mp shape mismatch");
    CHECK_NEAR(matmul_mp(mx, mw)[1][1], 11.0, 0.0);

    // BatchNorm forward pieces: x[N=2, C=2, S=2]
    Tensor bx = Tensor::from_vector({1, 3, 10, 30, 5, 7, 50, 70}, {2, 2, 2});
    Tensor bm, bv;
    channel_moments(bx, bm, bv);
    CHECK_NEAR(bm[0], 4.0, 1e-6);
    CHECK_NEAR(bm[1], 40.0, 1e-5);
    CHECK_NEAR(bv[0], 5.0, 1e-5);
    CHECK_NEAR(bv[1], 500.0, 1e-3);
    Tensor by = batch_norm_apply(bx, bm, bv, Tensor::full({2}, 2.0), Tensor::full({2}, 1.0), 0.0);
    CHECK_NEAR(by[0][0][0], 2.0 * (1.0 - 4.0) / std::sqrt(5.0) + 1.0, 1e-5);
    CHECK_NEAR(by[1][1][1], 2.0 * (70.0 - 40.0) / std::sqrt(500.0) + 1.0, 1e-5);

    // errors: the reference's exception types and texts
    CHECK_THROWS(Tensor::ones({2, 3}) + Tensor::ones({2, 2}), std::runtime_error, "Shape mismatch in binary op");
    CHECK_THROWS(add(Tensor(), a), std::runtime_error, "binary_op: null input");
    CHECK_THROWS(relu(Tensor()), std::runtime_error, "unary_op: null input");
    CHECK_THROWS(argmax(t, 5), std::out_of_range, "argmax: dim out of range");
    CHECK_THROWS(t.reshape({5}), std::runtime_error, "Reshape size mismatch");
    CHECK_THROWS(t[2], std::out_of_range, "Index out of bounds");

    // autograd hook: requires_grad propagates and the registered factory builds the node
    ctb_host::set_grad_factory([](const std::string& op, const std::vector<Tensor>& in, double s) {
        return std::make_shared<GradFn>(GradFn{op, in.size(), s});
    });
    Tensor w = Tensor::full({2, 2}, 3.0, DType::Float32, true);
    Tensor y = mul(w, a);
    CHECK(y.requires_grad() && y.impl->grad_fn && y.impl->grad_fn->op == "mul" && y.impl->grad_fn->n_inputs == 2);
    Tensor z = mul_scalar(y, 2.0);
    CHECK(z.impl->grad_fn->op == "mul_scalar" && z.impl->grad_fn->scalar == 2.0);
    CHECK(!add(a, b).requires_grad() && !max(w).requires_grad());

    // Device tags (src/core/device.h:5-25): a tensor lives on the GPU its tag names, results stay there
    CHECK(a.device() == Device(DeviceType::CUDA, ctb_host::device()));
    CHECK((a + b).device() == a.device());
    CHECK(a.to(Device(DeviceType::CUDA, ctb_host::device())).impl == a.impl);        // already there: no copy
    if (ctb_device_count() >= 2) {
        Tensor far = a.to(Device(DeviceType::CUDA, 1));
        CHECK(far.device() == Device(DeviceType::CUDA, 1));
        Tensor far_sum = far + b.to(Device(DeviceType::CUDA, 1));
        CHECK(far_sum.device() == Device(DeviceType::CUDA, 1));
        CHECK_NEAR(far_sum[1][1], 5.0, 1e-6);
        CHECK_NEAR(sum(far).item<double>(), 8.0, 1e-6);
        CHECK_THROWS(far + b, std::runtime_error, "add: tensors must be on same device");
    } else {
        CHECK_THROWS(a.to(Device(DeviceType::CUDA, 1)), std::runtime_error, "Tensor::to: no such CUDA device");
    }
    // operator results come from the pool: once a result of this size has been freed, further ones
    // cost no driver allocation (hits grow, misses do not)
    { Tensor warm = a + b; }
    ctb_pool_info before, after;
    CHECK(ctb_pool_stats(ctb_host::device(), &before) == 0);
    for (int i = 0; i < 5; ++i) { Tensor tmp = a + b; }
    CHECK(ctb_pool_stats(ctb_host::device(), &after) == 0);
    CHECK(after.misses == before.misses && after.hits >= before.hits + 5);
    // a mean that carries a gradient is the reference's two operators (sum, mul_scalar)
    Tensor mean_w = mean(w, 1);
    CHECK(mean_w.impl->grad_fn && mean_w.impl->grad_fn->op == "mul_scalar" && mean_w.impl->grad_fn->scalar == 0.5);
    CHECK_NEAR(mean_w[0], 3.0, 1e-6);
    CHECK(sum(t, -2).numel() == 2);                       // negative dims other than -1 wrap
    CHECK_THROWS(sum(t, -5), std::out_of_range, "reduction: dim out of range");

    // the fused bodies for the loss and autograd libraries: one kernel each, same numbers as the chains
    {
        Tensor logits = Tensor::from_vector({1.0, 2.0, 0.5, -1.0, 0.0, 3.0}, {2, 3});
        Tensor labels = Tensor::from_vector({1, 2}, {2, 1}, DType::Int32);
        const double l0 = -(2.0 - std::log(std::exp(1.0) + std::exp(2.0) + std::exp(0.5)));
        const double l1 = -(3.0 - std::log(std::exp(-1.0) + std::exp(0.0) + std::exp(3.0)));
        CHECK_NEAR(ctb_host::cross_entropy(logits, labels, true)[0], (l0 + l1) / 2, 1e-6);
        CHECK_NEAR(ctb_host::cross_entropy(logits, labels, false)[0], l0 + l1, 1e-6);
        Tensor g = ctb_host::cross_entropy_backward(logits, labels, 0.5);
        const double z0 = std::exp(1.0) + std::exp(2.0) + std::exp(0.5);
        CHECK(g.shape() == logits.shape());
        CHECK_NEAR(g[0][0], 0.5 * std::exp(1.0) / z0, 1e-6);
        CHECK_NEAR(g[0][1], 0.5 * (std::exp(2.0) / z0 - 1.0), 1e-6);
        CHECK_NEAR(double(g[1][0]) + double(g[1][1]) + double(g[1][2]), 0.0, 1e-6);
        Tensor wrong = Tensor::from_vector({1, 3}, {2, 1}, DType::Int32);
        CHECK_THROWS(ctb_host::cross_entropy(logits, wrong, true), std::out_of_range, "Gather index out of bounds");

        Tensor up = Tensor::from_vector({1.0, 2.0, 3.0, 4.0}, {2, 2}), num = Tensor::from_vector({2.0, 4.0, 6.0, 8.0}, {2, 2});
        Tensor den = Tensor::from_vector({2.0, 4.0}, {1, 2});                     // broadcast over the rows
        Tensor ga, gb;
        ctb_host::div_backward(up, num, den, &ga, &gb);
        CHECK(ga.shape() == std::vector<size_t>({2, 2}) && gb.shape() == std::vector<size_t>({2, 2}));
        CHECK_NEAR(ga[1][1], 4.0 / 4.0, 1e-6);                                      // grad / b
        CHECK_NEAR(gb[1][0], -3.0 * 6.0 / 4.0, 1e-6);                              // -grad * a / b^2
        ctb_host::div_backward(up, num, den, nullptr, &gb);                        // either side alone
        CHECK_NEAR(gb[0][1], -2.0 * 4.0 / 16.0, 1e-6);
        Tensor th = ctb_host::tanh_backward(up, num);
        CHECK_NEAR(th[0][0], 1.0 * (1.0 - std::tanh(2.0) * std::tanh(2.0)), 1e-6);
    }
    // matmul on the tensor cores when asked for: TF32 products, the same shapes and the same backward node
    {
        const size_t M = 96, K = 200, N = 72;
        std::vector<double> av(M * K), bv(N * K);
        for (size_t i = 0; i < av.size(); ++i) av[i] = double((i * 37) % 101) / 64.0 - 0.75;
        for (size_t i = 0; i < bv.size(); ++i) bv[i] = double((i * 53) % 89) / 32.0 - 1.25;
        Tensor ma = Tensor::from_vector(av, {M, K}), mb = Tensor::from_vector(bv, {N, K}, DType::Float32, true);
        Tensor exact = matmul(ma, mb.permute({1, 0}));
        ctb_host::set_matmul_tensor_cores(true);
        Tensor fast = matmul(ma, mb.permute({1, 0}));
        ctb_host::set_matmul_tensor_cores(false);
        CHECK(fast.shape() == exact.shape() && fast.requires_grad() && fast.impl->grad_fn && fast.impl->grad_fn->op == "matmul");
        double worst = 0.0, bound = 0.0;
        for (size_t i : {size_t(0), M / 2, M - 1})
            for (size_t j : {size_t(0), N / 3, N - 1}) {
                double mag = 0.0;
                for (size_t k = 0; k < K; ++k) mag += std::fabs(av[i * K + k] * bv[j * K + k]);
                worst = std::fmax(worst, std::fabs(double(fast[i][j]) - double(exact[i][j])));
                bound = std::fmax(bound, mag / 512.0);
            }
        CHECK(worst <= bound);
        Tensor again = matmul(ma, mb.permute({1, 0}));                                       // switched off again: the exact kernel
        CHECK(double(again[M - 1][N - 1]) == double(exact[M - 1][N - 1]));
    }

    std::printf("ALL PASSED (%d checks)\n", g_checks);
    return 0;
}
