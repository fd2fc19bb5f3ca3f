// A training step as a user of the reference writes it — two Linear layers with a relu between
// them, Loss::CrossEntropy, backward(), an SGD optimizer from train_utils.h — timed.  Built twice
// (tests/cpp/build_callers.sh, oracle/build_callers_ref.sh): over the B200 host layer with the
// reference's autograd.cpp / layer.cpp / loss.cpp unchanged, and against the reference itself
// (scalar back-end, the one on which its backward passes run on an AVX-512 host).
//
//   train_step_program [batch] [features] [hidden] [classes] [steps]
//
// Prints one JSON object: milliseconds per step (after two warm-up steps), first and last loss.
#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <exception>
#include <iomanip>
#include <iostream>
#include <string>
#include <unordered_map>
#include <vector>

#include "core/tensor.h"
#include "core/ops_dispatch.h"
#include "core/autograd.h"
#include "neuralnet/layer.h"
#include "neuralnet/loss.h"
#include "neuralnet/train_utils.h"

namespace {

Tensor filled(const std::vector<size_t>& shape, uint64_t seed, double scale, bool requires_grad) {
    Tensor t(shape, DType::Float32, requires_grad);
    float* p = (float*)t.impl->data->data.get();
    uint64_t s = seed * 6364136223846793005ull + 1442695040888963407ull;
    for (size_t i = 0, n = t.numel(); i < n; ++i) {
        s = s * 6364136223846793005ull + 1442695040888963407ull;
        p[i] = (float)((((double)((s >> 11) & ((1ull << 53) - 1)) / (double)(1ull << 52)) - 1.0) * scale);
    }
    return t;
}

double first_value(const Tensor& t) { return read_scalar_at(t.impl->data->data.get(), 0, DType::Float32); }

}  // namespace

int main(int argc, char** argv) {
    const size_t batch = argc > 1 ? std::atoi(argv[1]) : 512, features = argc > 2 ? std::atoi(argv[2]) : 1024;
    const size_t hidden = argc > 3 ? std::atoi(argv[3]) : 1024, classes = argc > 4 ? std::atoi(argv[4]) : 16;
    const int steps = argc > 5 ? std::atoi(argv[5]) : 5;
    try {
        Linear l1((int)features, (int)hidden, true, DType::Float32), l2((int)hidden, (int)classes, true, DType::Float32);
        l1.weight = filled({hidden, features}, 1, 0.05, true);
        l1.bias = filled({hidden}, 2, 0.01, true);
        l2.weight = filled({classes, hidden}, 3, 0.05, true);
        l2.bias = filled({classes}, 4, 0.01, true);
        Tensor x = filled({batch, features}, 5, 1.0, false);
        Tensor labels({batch, 1}, DType::Int32, false);
        for (size_t i = 0; i < batch; ++i) write_scalar_at(labels.impl->data->data.get(), i, DType::Int32, (double)((i * 5 + 1) % classes));
        std::vector<Tensor*> params = {&l1.weight, &l1.bias, &l2.weight, &l2.bias};
        SGD opt(params, 0.05);
        double first = 0.0, last = 0.0;
        double phase_ms[4] = {0, 0, 0, 0};          // forward, loss, backward, zero_grad + step
        auto now = [] { return std::chrono::steady_clock::now(); };
        auto lap = [&](int i, std::chrono::steady_clock::time_point t0) {
            phase_ms[i] += std::chrono::duration<double, std::milli>(now() - t0).count();
        };
        auto step = [&] {
            auto t0 = now();
            opt.zero_grad();
            lap(3, t0);
            t0 = now();
            Tensor logits = l2.forward(relu(l1.forward(x)));
            lap(0, t0);
            t0 = now();
            Tensor loss = Loss::CrossEntropy(logits, labels, "mean");
            last = first_value(loss);
            lap(1, t0);
            t0 = now();
            loss.backward();
            lap(2, t0);
            t0 = now();
            opt.step();
            lap(3, t0);
        };
        step();
        first = last;
        step();
        for (double& p : phase_ms) p = 0.0;
        const auto t0 = std::chrono::steady_clock::now();
        for (int i = 0; i < steps; ++i) step();
        const double ms = std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - t0).count() / steps;
        std::printf("{\"batch\": %zu, \"features\": %zu, \"hidden\": %zu, \"classes\": %zu, \"steps\": %d, \"ms_per_step\": %.3f, "
                    "\"forward_ms\": %.3f, \"loss_ms\": %.3f, \"backward_ms\": %.3f, \"optimizer_ms\": %.3f, "
                    "\"loss_first\": %.9g, \"loss_last\": %.9g}\n", batch, features, hidden, classes, steps, ms,
                    phase_ms[0] / steps, phase_ms[1] / steps, phase_ms[2] / steps, phase_ms[3] / steps, first, last);
    } catch (const std::exception& e) {
        std::printf("{\"error\": \"%s\"}\n", e.what());
        return 1;
    }
    return 0;
}
