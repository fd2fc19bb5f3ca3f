// Timing of the C++ host layer itself — the drop-in path a caller of the reference uses:
// Tensor operands in pooled managed memory, `a + b`, relu(a) and sum(a, 1) through the operator
// API of ops_dispatch.h, every call waiting for its kernel as the callers expect.
//
//   bench_host_layer [log2 sizes...]      default: 20 24 28
//
// Prints one JSON object: per size the microseconds per call and the GB/s (algorithmic bytes:
// 12 B/element for add, 8 for relu, 4 (+ the row results) for sum), with output allocation from
// the pool inside the timed call, as it is for a caller.
#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <string>
#include <vector>

#include "ctb_host.h"
#include "ops_dispatch.h"
#include "../../include/ctb200.h"

namespace {

double seconds_per_call(int reps, const std::function<void()>& f) {
    for (int i = 0; i < 3; ++i) f();
    ctb_host::sync_for_host_access();
    const auto t0 = std::chrono::steady_clock::now();
    for (int i = 0; i < reps; ++i) f();
    ctb_host::sync_for_host_access();
    return std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count() / reps;
}

Tensor filled(size_t rows, size_t cols, float value) {
    Tensor t({rows, cols}, DType::Float32, false);
    float* p = (float*)t.impl->data->data.get();
    for (size_t i = 0, n = rows * cols; i < n; ++i) p[i] = value + (float)(i % 7);
    // the host wrote the pages: move them to the GPU before timing, as a training loop's tensors are
    ctb_prefetch_managed(p, rows * cols * sizeof(float), ctb_host::device(), nullptr);
    return t;
}

}  // namespace

int main(int argc, char** argv) {
    std::vector<int> sizes;
    for (int i = 1; i < argc; ++i) sizes.push_back(std::atoi(argv[i]));
    if (sizes.empty()) sizes = {20, 24, 28};
    try {
        std::string out = "{";
        for (size_t k = 0; k < sizes.size(); ++k) {
            const int lg = sizes[k];
            const size_t n = size_t(1) << lg, cols = 1024, rows = n / cols;
            Tensor a = filled(rows, cols, 1.0f), b = filled(rows, cols, 2.0f);
            const int reps = lg >= 28 ? 10 : lg >= 24 ? 50 : 200;
            const double t_add = seconds_per_call(reps, [&] { Tensor c = a + b; });
            const double t_relu = seconds_per_call(reps, [&] { Tensor c = relu(a); });
            const double t_sum = seconds_per_call(reps, [&] { Tensor c = sum(a, 1); });
            char buf[512];
            std::snprintf(buf, sizeof buf,
                          "%s\"2^%d\": {\"add_us\": %.1f, \"add_GBs\": %.1f, \"relu_us\": %.1f, \"relu_GBs\": %.1f, "
                          "\"sum_dim1_us\": %.1f, \"sum_dim1_GBs\": %.1f}",
                          k ? ", " : "", lg, t_add * 1e6, 12.0 * n / t_add / 1e9, t_relu * 1e6, 8.0 * n / t_relu / 1e9,
                          t_sum * 1e6, (4.0 * n + 4.0 * rows) / t_sum / 1e9);
            out += buf;
        }
        ctb_pool_info info;
        ctb_pool_stats(ctb_host::device(), &info);
        char tail[256];
        std::snprintf(tail, sizeof tail, ", \"pool\": {\"hits\": %llu, \"misses\": %llu}}", (unsigned long long)info.hits,
                      (unsigned long long)info.misses);
        out += tail;
        std::printf("%s\n", out.c_str());
    } catch (const std::exception& e) {
        std::printf("{\"error\": \"%s\"}\n", e.what());
        return 1;
    }
    return 0;
}
