// One program, four builds: the reference's own callers of the operator path — autograd.cpp,
// layer.cpp, loss.cpp, unchanged — driven through a Linear layer, two losses and a chain of
// elementwise operators, forward and backward, and — with the optimizer classes of train_utils.h —
// through three training steps per optimizer; plus the reference's BatchNorm and activation modules
// and its Dropout module (batchnorm.cpp, Relu.cpp, dropout.cpp), unchanged as well; in the second
// generation also its norm functions and its metrics (dropout.cpp, norm.cpp, metrics.h through the umbrella headers
// core.h and neuralnet.h).
//
//   build                      tensor/operator layer                     callers
//   callers_gen2_ref           the reference's src/core (CPU)            the reference's, unchanged
//   callers_gen2_ref_scalar    the same, feature probes answering "no"   the reference's, unchanged
//   callers_gen2_b200          ctensor_b200/host (GPU)                   the reference's, unchanged
//   callers_gen1_ref           the reference's tensor1/opsmp (CPU)       the reference's, unchanged
//   callers_gen1_b200          ctensor_b200/host/gen1 (GPU)              the reference's, unchanged
//
// It prints one "name count v0 v1 ..." line per result (loss values and every gradient).  The
// tests compare the lines of a *_b200 build with those of the *_ref build.  A section that
// throws prints "name unavailable <reason>".
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <exception>
#include <iomanip>          // the reference's train_utils.h uses std::setprecision without including it
#include <iostream>
#include <limits>
#include <string>
#include <unordered_map>
#include <vector>

#ifdef CTB_GEN1
#include "tensor1.h"
#include "opsmp.h"
#include "autograd.h"
#include "layer.h"
#include "loss.h"
#include "train_utils.h"
#include "batchnorm.h"
#include "Relu.h"
#include "dropout.h"
#define CTB_HAVE_BATCHNORM 1
#define DATA(t) ((t).impl->storage->data.get())
#define GRAD(t) ((t).impl->storage->grad.get())
#define F_EXP exp_mp
#define F_LN ln_mp
#define F_TANH tanh_mp
#define F_RELU Relu_mp
#define F_MEAN_ROWS(t) mean_mp((t), 1)
// every dim folded in turn (flatten() would cut the graph: it attaches no backward node here)
static Tensor sum_all(Tensor t) {
    while (t.impl->ndim > 1) t = sum_mp(t, (int)t.impl->ndim - 1);
    return sum_mp(t, 0);
}
#define F_SUM_ALL(t) sum_all(t)
#else
#include "core/tensor.h"
#include "core/ops_dispatch.h"
#include "core/autograd.h"
#include "neuralnet/layer.h"
#include "neuralnet/loss.h"
#include "neuralnet/train_utils.h"
#include "neuralnet/batchnorm/batchnorm.h"
#include "neuralnet/Relu.h"
#include "neuralnet/dropout/dropout.h"
#include "neuralnet/norm/norm.h"          // includes core.h: every header of src/core
#include "neuralnet/metrics.h"            // includes neuralnet.h: every header of src/neuralnet
#define CTB_HAVE_BATCHNORM 1
#define DATA(t) ((t).impl->data->data.get())
#define GRAD(t) ((t).impl->grad ? (t).impl->grad->data->data.get() : nullptr)
#define F_EXP exp
#define F_LN ln
#define F_TANH tanh
#define F_RELU relu
#define F_MEAN_ROWS(t) mean((t), 1)
// Everything summed as reshape-to-1-d + sum over dim 0: sum(t, -1) means "everything" on the
// reference's SIMD back-ends and "the last dim" on its scalar one (src/core/opsmp.cpp:598), and a
// dim-wise sum of a 2-d tensor cannot sit in a graph here — GradSum::backward
// (src/core/autograd.cpp:369-373) hands the reduced gradient to accumulate_grad without
// re-inserting the folded dim, which then reads past its end.
#define F_SUM_ALL(t) sum((t).reshape({(t).numel()}), 0)
#define CTB_NO_DIMWISE_SUM_BACKWARD 1
#endif

namespace {

// a small deterministic generator (the same numbers in every build)
struct Lcg {
    uint64_t s;
    explicit Lcg(uint64_t seed) : s(seed * 6364136223846793005ull + 1442695040888963407ull) {}
    double next() {       // uniform in (-1, 1)
        s = s * 6364136223846793005ull + 1442695040888963407ull;
        return ((double)((s >> 11) & ((1ull << 53) - 1)) / (double)(1ull << 52)) - 1.0;
    }
};

Tensor filled(const std::vector<size_t>& shape, uint64_t seed, double scale, bool requires_grad, double shift = 0.0) {
    Tensor t(shape, DType::Float32, requires_grad);
    Lcg g(seed);
    const size_t n = t.numel();
    for (size_t i = 0; i < n; ++i) write_scalar_at(DATA(t), i, DType::Float32, g.next() * scale + shift);
    return t;
}

void print_values(const char* name, const void* p, size_t n) {
    std::printf("%s %zu", name, n);
    for (size_t i = 0; i < n; ++i) std::printf(" %.9g", read_scalar_at(p, i, DType::Float32));
    std::printf("\n");
}
void print_data(const char* name, const Tensor& t) { print_values(name, DATA(t), t.numel()); }
void print_grad(const char* name, const Tensor& t) {
    const void* g = GRAD(t);
    if (!g) { std::printf("%s unavailable no gradient buffer\n", name); return; }
    print_values(name, g, t.numel());
}

void print_number(const char* name, double v) { std::printf("%s 1 %.9g\n", name, v); }

template <typename F> void section(const char* name, F body) {
    try {
        body();
    } catch (const std::exception& e) {
        std::printf("%s unavailable %s\n", name, e.what());
    }
}

}  // namespace

int main() {
    std::setvbuf(stdout, nullptr, _IOLBF, 1 << 16);      // a crash inside a caller loses no finished line
    const size_t batch = 12, in_f = 16, out_f = 10;

    // Linear -> MSE (layer.cpp: matmul + broadcast add; loss.cpp: sub, pow_scalar, full sum).
    // The backward pass runs through the same loss spelled with operators: the reference's own
    // GradMSE::backward writes numel(pred) values into the one-element gradient of the loss
    // (loss.cpp, GradMSE::backward) and cannot be run for more than one element.
    section("mse", [&] {
        Linear lin((int)in_f, (int)out_f, true, DType::Float32);
        lin.weight = filled({out_f, in_f}, 1, 0.5, true);
        lin.bias = filled({out_f}, 2, 0.1, true);
        Tensor x = filled({batch, in_f}, 3, 1.0, true);
        Tensor target = filled({batch, out_f}, 4, 1.0, false);
        Tensor y = lin.forward(x);
        print_data("mse.forward", y);
        print_data("mse.loss", Loss::MSE(y, target));
        Tensor d = y - target;
        Tensor loss = F_SUM_ALL(d * d) * (1.0 / (double)(batch * out_f));
        print_data("mse.loss_from_operators", loss);
        loss.backward();
        print_grad("mse.grad_weight", lin.weight);
        print_grad("mse.grad_bias", lin.bias);
        print_grad("mse.grad_input", x);
    });

    // Linear -> CrossEntropy -> backward (loss.cpp: row max, sub, exp, row sum, ln, gather, mean)
    section("ce", [&] {
        Linear lin((int)in_f, (int)out_f, true, DType::Float32);
        lin.weight = filled({out_f, in_f}, 5, 0.5, true);
        lin.bias = filled({out_f}, 6, 0.1, true);
        Tensor x = filled({batch, in_f}, 7, 1.0, true);
        Tensor labels({batch, 1}, DType::Int32, false);
        for (size_t i = 0; i < batch; ++i) write_scalar_at(DATA(labels), i, DType::Int32, (double)((i * 7 + 3) % out_f));
        Tensor logits = lin.forward(x);
        Tensor loss = Loss::CrossEntropy(logits, labels, "mean");
        print_data("ce.loss", loss);
        loss.backward();
        print_grad("ce.grad_weight", lin.weight);
        print_grad("ce.grad_bias", lin.bias);
        print_grad("ce.grad_input", x);
    });

    // elementwise chain with broadcasting, through the autograd nodes of add/sub/mul/div,
    // scalar ops, exp/ln/tanh/relu and a full sum: accumulate_grad folds the broadcast dims
    section("chain", [&] {
        Tensor a = filled({6, 8}, 8, 1.0, true);
        Tensor b = filled({1, 8}, 9, 0.5, true, 1.5);          // in (1, 2): safe divisor, ln argument
        Tensor c = filled({6, 1}, 10, 1.0, true);
        Tensor u = (a * b + c) / b - a * 0.25;
        Tensor v = F_TANH(u) + F_RELU(a) * F_EXP(c * 0.5) - F_LN(b);
        Tensor total = F_SUM_ALL(v);
        print_data("chain.value", total);
        total.backward();
        print_grad("chain.grad_a", a);
        print_grad("chain.grad_b", b);
        print_grad("chain.grad_c", c);
    });

    // the same kind of chain on same-shape operands (no broadcast folds, no ln): the part the
    // reference's SIMD back-ends can run as well
    section("plain", [&] {
        Tensor a = filled({6, 8}, 12, 1.0, true);
        Tensor b = filled({6, 8}, 13, 0.5, true, 1.5);
        Tensor w = F_TANH(a * b + a / b) * F_RELU(a) + F_EXP(b * 0.5) - a * 0.125;
        Tensor total = F_SUM_ALL(w);
        print_data("plain.value", total);
        total.backward();
        print_grad("plain.grad_a", a);
        print_grad("plain.grad_b", b);
    });

    // dim-wise mean through the graph (sum + mul_scalar nodes), then a full sum
    section("rowmean", [&] {
        Tensor a = filled({5, 7}, 11, 2.0, true);
        Tensor m = F_MEAN_ROWS(a * a);
        Tensor total = F_SUM_ALL(m);
        print_data("rowmean.value", total);
#ifndef CTB_NO_DIMWISE_SUM_BACKWARD
        total.backward();
        print_grad("rowmean.grad_a", a);
#endif
    });
#ifdef CTB_HAVE_BATCHNORM
    // BatchNorm (src/neuralnet/batchnorm/batchnorm.cpp, unchanged): training-mode forward over
    // x[N, C, H, W] (permute, reshape, mean, sub, mul, pow_scalar, broadcasts), its backward node,
    // the running statistics, and the inference-mode forward
    section("bn", [&] {
        BatchNorm bn(3);
        bn.gamma = filled({3}, 31, 0.5, true, 1.0);
        bn.beta = filled({3}, 32, 0.1, true);
        Tensor x = filled({4, 3, 5, 5}, 33, 1.0, true);
        Tensor y = bn.forward(x);
        print_data("bn.forward", y);
        print_data("bn.running_mean", bn.running_mean);
        print_data("bn.running_var", bn.running_var);
        Tensor total = F_SUM_ALL(y * y);
        print_data("bn.value", total);
        total.backward();
        print_grad("bn.grad_x", x);
        print_grad("bn.grad_gamma", bn.gamma);
        print_grad("bn.grad_beta", bn.beta);
        bn.eval();
        print_data("bn.eval_forward", bn.forward(x));
    });
#endif

    // The activation modules of Relu.cpp (unchanged): Relu, LeakyRelu and PRelu with their own
    // backward nodes (host loops over the storage the operators produced)
    section("act", [&] {
        Tensor x = filled({6, 8}, 41, 2.0, true);
        Relu relu_module;
        print_data("act.relu", relu_module.forward(x));
        Tensor leaky = LeakyRelu(x, 0.1);
        print_data("act.leaky", leaky);
        Tensor total = F_SUM_ALL(leaky * leaky);
        total.backward();
        print_grad("act.leaky_grad_x", x);
        Tensor z = filled({6, 8}, 42, 2.0, true);
        PRelu prelu(1, 0.25);
        Tensor pz = prelu.forward(z);
        print_data("act.prelu", pz);
        Tensor total2 = F_SUM_ALL(pz * pz);
        total2.backward();
        print_grad("act.prelu_grad_x", z);
        print_grad("act.prelu_grad_weight", prelu.weight);
    });

    // Dropout (src/neuralnet/dropout/dropout.cpp, root dropout.cpp, unchanged): the mask is drawn on the host from a
    // generator with a fixed seed, so every build draws the same one; forward = input * mask * scale
    // through the operators, GradDropout::backward the same on the gradient; identity after eval()
    section("dropout", [&] {
        Dropout drop(0.3);
        Tensor x = filled({6, 8}, 51, 1.0, true);
        Tensor y = drop.forward(x);
        print_data("dropout.forward", y);
        Tensor total = F_SUM_ALL(y * y);
        print_data("dropout.value", total);
        total.backward();
        print_grad("dropout.grad_x", x);
        drop.eval();
        print_data("dropout.eval_forward", drop.forward(x));
    });

#ifndef CTB_GEN1
    // The norm functions (src/neuralnet/norm/norm.cpp, unchanged): abs, pow_scalar, sum / max / min
    // over a dim, sqrt, the comparison against zero, unsqueeze for keepdim, and the global forms
    section("norm", [&] {
        Tensor x = filled({5, 7}, 52, 2.0, false);
        for (size_t i = 0; i < x.numel(); i += 4) write_scalar_at(DATA(x), i, DType::Float32, 0.0);   // zeros for the count
        const double inf = std::numeric_limits<double>::infinity();
        print_data("norm.l1_rows", norm(x, 1.0, 1));
        print_data("norm.l2_cols", norm(x, 2.0, 0));
        print_data("norm.max_rows", norm(x, inf, 1));
        print_data("norm.min_cols", norm(x, -inf, 0));
        print_data("norm.count_rows", norm(x, 0.0, 1));
        print_data("norm.l3_rows_keepdim", norm(x, 3.0, 1, true));
        print_data("norm.l2_negative_dim", norm(x, 2.0, -2));         // wraps to dim 0
        print_data("norm.l2_global", norm(x, 2.0));
        print_data("norm.l1_global", norm(x, 1.0));
        print_data("norm.l3_global", norm(x, 3.0));
        print_data("norm.infinity_global", infinity_norm(x));
        print_data("norm.zero_cols", zero_norm(x, 0));
    });

    // The metrics of src/neuralnet/metrics.h (header-only, unchanged): argmax, comparisons, astype,
    // full sums and means, item<float>()
    section("metrics", [&] {
        Tensor logits = filled({12, 10}, 53, 1.0, false);
        Tensor labels({12, 1}, DType::Int32, false);
        for (size_t i = 0; i < 12; ++i) {       // half of the labels are the row's argmax, half are not
            size_t best = 0;
            for (size_t c = 1; c < 10; ++c)
                if (read_scalar_at(DATA(logits), i * 10 + c, DType::Float32) > read_scalar_at(DATA(logits), i * 10 + best, DType::Float32)) best = c;
            write_scalar_at(DATA(labels), i, DType::Int32, (double)(i % 2 ? best : (best + 3) % 10));
        }
        print_number("metrics.accuracy", (double)torch::metrics::accuracy(logits, labels));
        print_number("metrics.accuracy_score", torch::metrics::accuracy_score(logits, labels));
        Tensor scores = filled({16, 1}, 54, 0.5, false, 0.5);
        Tensor truth({16, 1}, DType::Float32, false);
        for (size_t i = 0; i < 16; ++i) write_scalar_at(DATA(truth), i, DType::Float32, (double)((i * 5 + 1) % 3 == 0));
        print_number("metrics.binary_accuracy", torch::metrics::binary_accuracy(scores, truth));
        print_number("metrics.precision", torch::metrics::precision_score(scores, truth));
        print_number("metrics.recall", torch::metrics::recall_score(scores, truth));
        print_number("metrics.f1", torch::metrics::f1_score(scores, truth, 0.4f));
        Tensor predicted = filled({24}, 55, 1.0, false), wanted = filled({24}, 56, 1.0, false);
        print_number("metrics.mse", torch::metrics::mean_squared_error(predicted, wanted));
        print_number("metrics.mae", torch::metrics::mean_absolute_error(predicted, wanted));
        print_number("metrics.r2", torch::metrics::r2_score(predicted, wanted));
    });
#endif

    // Three training steps of Linear -> CrossEntropy with each optimizer class of train_utils.h:
    // zero_grad, forward, backward, step — the loop a user of the reference writes.  In the *_b200
    // builds the classes are the host layer's (one fused kernel per parameter and step).
    auto train = [&](const char* name, auto make_optimizer) {
        section(name, [&] {
            Linear lin((int)in_f, (int)out_f, true, DType::Float32);
            lin.weight = filled({out_f, in_f}, 21, 0.5, true);
            lin.bias = filled({out_f}, 22, 0.1, true);
            Tensor x = filled({batch, in_f}, 23, 1.0, false);
            Tensor labels({batch, 1}, DType::Int32, false);
            for (size_t i = 0; i < batch; ++i) write_scalar_at(DATA(labels), i, DType::Int32, (double)((i * 3 + 1) % out_f));
            std::vector<Tensor*> params = {&lin.weight, &lin.bias};
            auto opt = make_optimizer(params);
            std::string tag(name);
            for (int it = 0; it < 3; ++it) {
                opt.zero_grad();
                Tensor loss = Loss::CrossEntropy(lin.forward(x), labels, "mean");
                if (it == 2) print_data((tag + ".loss").c_str(), loss);
                loss.backward();
                opt.step();
            }
            print_data((tag + ".weight").c_str(), lin.weight);
            print_data((tag + ".bias").c_str(), lin.bias);
        });
    };
    train("optim_sgd", [](std::vector<Tensor*>& p) { return SGD(p, 0.1); });
    train("optim_adam", [](std::vector<Tensor*>& p) { return Adam(p, 0.01); });
    train("optim_adamw", [](std::vector<Tensor*>& p) { return AdamW(p, 0.01, 0.9, 0.999, 1e-8, 0.05); });
    train("optim_adamax", [](std::vector<Tensor*>& p) { return Adamax(p, 0.01); });
    train("optim_nadam", [](std::vector<Tensor*>& p) { return NAdam(p, 0.01); });
    train("optim_radam", [](std::vector<Tensor*>& p) { return RAdam(p, 0.01); });
    train("optim_rmsprop", [](std::vector<Tensor*>& p) { return RMSprop(p, 0.01); });
    train("optim_adagrad", [](std::vector<Tensor*>& p) { return Adagrad(p, 0.05); });
    train("optim_lion", [](std::vector<Tensor*>& p) { return Lion(p, 0.01, 0.9, 0.99, 0.05); });
    return 0;
}
