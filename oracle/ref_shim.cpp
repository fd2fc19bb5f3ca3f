// TEST INFRASTRUCTURE — not part of the product.
//
// extern "C" driver around the UNMODIFIED reference implementation (CTensor "src tree":
// src/core/{tensor,opsmp,ops_dispatch,autograd}.cpp, src/cpu/AVX2/*, src/cpu/AVX512/*).
// It is compiled together with the reference's own sources by oracle/build_ref.sh into
// oracle/_ref/libctensor_ref.so and is used (a) to pin the plain-C restatement in
// oracle/ctb_oracle.c, (b) to generate the golden fixtures under tests/golden/, and
// (c) as the timed "reference" CPU baseline of bench.py.
//
// The driver wraps caller-owned host memory in a reference `Tensor` view (shape, strides in
// elements, offset), calls the named reference function and copies the result bytes out.
// Which reference function each entry calls is stated next to it (file:line in the reference).
#include <cstdint>
#include <cstring>
#include <memory>
#include <stdexcept>
#include <string>
#include <vector>
#include <omp.h>
#include <chrono>

#include "tensor.h"
#include "opsmp.h"
#include "ops_dispatch.h"
#include "ops_avx2_f32.h"
#include "ops_avx512_f32.h"
#include "autograd.h"
#include "neuralnet/loss.h"          // declares Loss, which train_utils.h uses without including it
#include "neuralnet/train_utils.h"   // header-only optimizers (SGD, Adam, AdamW)

namespace {

thread_local std::string g_err;

struct RefView {          // mirrors struct ctb_view of include/ctb200.h (host pointers here)
    void*   base;
    int64_t offset;
    int32_t dtype;        // reference DType numbering: 0 Float32, 1 Int32, 2 Double64
    int32_t ndim;
    int64_t shape[8];
    int64_t stride[8];
};

// Wrap caller memory in a reference Tensor without copying (no-op deleter).
Tensor wrap(const RefView* v) {
    SmallVector<size_t, 5> shape, strides;
    size_t span = (size_t)v->offset + 1;
    for (int i = 0; i < v->ndim; ++i) {
        shape.push_back((size_t)v->shape[i]);
        strides.push_back((size_t)v->stride[i]);
        if (v->shape[i] > 0) span += (size_t)(v->shape[i] - 1) * (size_t)v->stride[i];
    }
    auto st = std::make_shared<Storage>();
    st->size = span;
    st->device = Device(DeviceType::CPU);
    st->data = std::shared_ptr<void>(v->base, [](void*) {});
    Tensor t;
    t.impl = intrusive_ptr<Tensorimpl>(new Tensorimpl(st, (size_t)v->offset, shape, strides,
                                                      (DType)v->dtype, false));
    return t;
}

// Copy a (contiguous, freshly allocated) reference result into caller memory.
int64_t emit(const Tensor& r, void* out, int64_t out_capacity_bytes) {
    if (!r.impl) throw std::runtime_error("reference returned an empty tensor");
    if (!r.is_contiguous()) throw std::runtime_error("reference result not contiguous");
    size_t bytes = r.numel() * dtype_size(r.impl->dtype);
    if ((int64_t)bytes > out_capacity_bytes) throw std::runtime_error("output buffer too small");
    std::memcpy(out, (const char*)r.impl->data->data.get() + r.impl->offset * dtype_size(r.impl->dtype), bytes);
    return (int64_t)r.numel();
}

enum Path { PATH_MP = 0, PATH_AVX2 = 1, PATH_AVX512 = 2, PATH_DISPATCH = 3 };

// Operator codes shared with include/ctb200.h.
enum BinOp { B_ADD = 0, B_SUB, B_MUL, B_DIV, B_LT, B_LE, B_GT, B_GE, B_EQ, B_NE, B_POW };
enum UnOp {
    U_ADD_S = 0, U_SUB_S, U_RSUB_S, U_MUL_S, U_DIV_S, U_RDIV_S, U_POW_S, U_RPOW_S,
    U_LT_S, U_LE_S, U_GT_S, U_GE_S, U_EQ_S, U_NE_S,
    U_ABS, U_RELU, U_EXP, U_LOG, U_TANH, U_SIGMOID, U_SQRT, U_GELU_TANH,
    U_SIN, U_COS, U_TAN, U_ASIN, U_ACOS, U_ATAN, U_SINH, U_COSH, U_SOFTPLUS
};
enum RedOp { R_SUM = 0, R_MEAN, R_MAX, R_MIN, R_VAR, R_ARGMAX };

Tensor do_binary(int path, int op, const Tensor& a, const Tensor& b) {
    switch (path) {
    case PATH_MP:       // src/core/opsmp.cpp:391-409,708-713
        switch (op) {
        case B_ADD: return add_mp(a, b);   case B_SUB: return diff_mp(a, b);
        case B_MUL: return mult_mp(a, b);  case B_DIV: return div_mp(a, b);
        case B_LT: return lt_mp(a, b);     case B_LE: return le_mp(a, b);
        case B_GT: return gt_mp(a, b);     case B_GE: return ge_mp(a, b);
        case B_EQ: return eq_mp(a, b);     case B_NE: return ne_mp(a, b);
        case B_POW: return pow_mp(a, b);
        } break;
    case PATH_AVX2:     // src/cpu/AVX2/ops_avx2_f32.cpp:574-604
        switch (op) {
        case B_ADD: return add_avx2_f32(a, b); case B_SUB: return sub_avx2_f32(a, b);
        case B_MUL: return mul_avx2_f32(a, b); case B_DIV: return div_avx2_f32(a, b);
        } break;
    case PATH_AVX512:   // src/cpu/AVX512/ops_avx512_f32.cpp:370-381
        switch (op) {
        case B_ADD: return add_avx512_f32(a, b); case B_SUB: return sub_avx512_f32(a, b);
        case B_MUL: return mul_avx512_f32(a, b); case B_DIV: return div_avx512_f32(a, b);
        } break;
    case PATH_DISPATCH: // src/core/ops_dispatch.cpp:219-233,342-347
        switch (op) {
        case B_ADD: return add(a, b); case B_SUB: return sub(a, b);
        case B_MUL: return mul(a, b); case B_DIV: return div(a, b);
        case B_LT: return lt(a, b);   case B_LE: return le(a, b);
        case B_GT: return gt(a, b);   case B_GE: return ge(a, b);
        case B_EQ: return eq(a, b);   case B_NE: return ne(a, b);
        } break;
    }
    throw std::runtime_error("ref_binary: op not available on this path");
}

// GELU (tanh form) as a chain of reference primitives, each step rounded to fp32.
// tanh flavour = the reference's SIMD Cephes tanh (src/cpu/AVX512/ops_avx512_f32.cpp:187-193).
Tensor gelu_chain(const Tensor& x, int tanh_path) {
    Tensor u = mult_mp(x, x);
    u = mult_mp(u, x);
    u = mult_scalar_mp(u, 0.044715);
    u = add_mp(x, u);
    u = mult_scalar_mp(u, 0.7978845608028654);
    Tensor t = (tanh_path == PATH_AVX2) ? tanh_avx2_f32(u) : tanh_avx512_f32(u);
    t = add_scalar_mp(t, 1.0);
    Tensor h = mult_scalar_mp(x, 0.5);
    return mult_mp(h, t);
}

Tensor do_unary(int path, int op, const Tensor& a, double s) {
    // Scalar ops and scalar comparisons exist only as *_mp (src/core/opsmp.cpp:418-456,701-706).
    switch (op) {
    case U_ADD_S:  return add_scalar_mp(a, s);
    case U_SUB_S:  return sub_scalar_mp(a, s);
    case U_RSUB_S: return sub_afterscalar_mp(s, a);
    case U_MUL_S:  return mult_scalar_mp(a, s);
    case U_DIV_S:  return div_scalar_mp(a, s);
    case U_RDIV_S: return scalar_div_mp(s, a);
    case U_POW_S:  return pow_scalar_mp(a, s);
    case U_RPOW_S: return scalar_pow_mp(s, a);
    case U_LT_S: return lt_mp(a, s); case U_LE_S: return le_mp(a, s);
    case U_GT_S: return gt_mp(a, s); case U_GE_S: return ge_mp(a, s);
    case U_EQ_S: return eq_mp(a, s); case U_NE_S: return neq_mp(a, s);
    default: break;
    }
    if (op == U_GELU_TANH) return gelu_chain(a, path == PATH_AVX2 ? PATH_AVX2 : PATH_AVX512);
    switch (path) {
    case PATH_MP:       // src/core/opsmp.cpp:562-589
        switch (op) {
        case U_ABS: return abs_mp(a);   case U_RELU: return Relu_mp(a);
        case U_EXP: return exp_mp(a);   case U_LOG: return ln_mp(a);
        case U_TANH: return tanh_mp(a); case U_SIGMOID: return sigmoid_mp(a);
        case U_SQRT: return sqrt_mp(a);
        case U_SIN: return sin_mp(a);   case U_COS: return cos_mp(a);   case U_TAN: return tan_mp(a);
        case U_ASIN: return asin_mp(a); case U_ACOS: return acos_mp(a); case U_ATAN: return atan_mp(a);
        case U_SINH: return sinh_mp(a); case U_COSH: return cosh_mp(a); case U_SOFTPLUS: return softplus_mp(a);
        } break;
    case PATH_AVX2:     // src/cpu/AVX2/ops_avx2_f32.cpp:606-641
        switch (op) {
        case U_ABS: return abs_avx2_f32(a);   case U_RELU: return relu_avx2_f32(a);
        case U_EXP: return exp_avx2_f32(a);   case U_LOG: return ln_avx2_f32(a);
        case U_TANH: return tanh_avx2_f32(a); case U_SIGMOID: return sigmoid_avx2_f32(a);
        case U_SQRT: return sqrt_avx2_f32(a);
        } break;
    case PATH_AVX512:   // src/cpu/AVX512/ops_avx512_f32.cpp:444-457
        switch (op) {
        case U_ABS: return abs_avx512_f32(a);   case U_RELU: return relu_avx512_f32(a);
        case U_EXP: return exp_avx512_f32(a);   case U_LOG: return ln_avx512_f32(a);
        case U_TANH: return tanh_avx512_f32(a); case U_SIGMOID: return sigmoid_avx512_f32(a);
        case U_SQRT: return sqrt_avx512_f32(a);
        } break;
    case PATH_DISPATCH: // src/core/ops_dispatch.cpp:319-335
        switch (op) {
        case U_ABS: return abs(a);   case U_RELU: return relu(a);
        case U_EXP: return exp(a);   case U_LOG: return ln(a);
        case U_TANH: return tanh(a); case U_SIGMOID: return sigmoid(a);
        case U_SQRT: return sqrt(a);
        } break;
    }
    throw std::runtime_error("ref_unary: op not available on this path");
}

std::vector<size_t> keepdim_shape(const Tensor& a, int dim) {
    std::vector<size_t> s = a.shape();
    s[dim] = 1;
    return s;
}

// Biased variance along `dim`, the recipe of src/neuralnet/batchnorm/batchnorm.cpp:54-61:
// mean -> reshape(keepdim) -> broadcast sub -> mul -> mean.
Tensor var_chain(const Tensor& x, int dim) {
    Tensor mu = mean_mp(x, dim).reshape(keepdim_shape(x, dim));
    Tensor d = diff_mp(x, mu);
    return mean_mp(mult_mp(d, d), dim);
}

Tensor do_reduce(int path, int op, const Tensor& a, int dim) {
    int nd = (int)a.impl->ndim;
    if (dim >= nd || dim < -1) throw std::out_of_range("ref_reduce: dim out of range");
    if (op == R_ARGMAX) {           // src/core/ops_dispatch.cpp:427-526 (dim is mandatory there)
        if (dim < 0) throw std::out_of_range("ref_reduce: argmax needs dim >= 0");
        return argmax(a, dim);
    }
    if (dim == -1) {
        // "reduce everything": the *_mp kernels treat -1 as "last dim" (src/core/opsmp.cpp:598),
        // so the full reduction through the scalar path is sum_mp over the flattened tensor.
        if (path == PATH_MP) {
            Tensor f = a.flatten();
            switch (op) {
            case R_SUM: return sum_mp(f, 0);
            case R_MEAN: return mean_mp(f, 0);
            case R_MAX: return max_mp(f, 0);
            case R_MIN: return min_mp(f, 0);
            case R_VAR: return var_chain(f, 0);
            }
        } else if (path == PATH_AVX2) {       // src/cpu/AVX2/ops_avx2_f32.cpp:778-966
            switch (op) {
            case R_SUM: return sum_avx2_f32(a, -1);
            case R_MEAN: return mean_avx2_f32(a, -1);
            case R_MAX: return max_avx2_f32(a, -1);
            case R_MIN: return min_avx2_f32(a, -1);
            }
        } else if (path == PATH_AVX512) {     // src/cpu/AVX512/ops_avx512_f32.cpp:480-566
            switch (op) {
            case R_SUM: return sum_avx512_f32(a, -1);
            case R_MEAN: return mean_avx512_f32(a, -1);
            case R_MAX: return max_avx512_f32(a, -1);
            case R_MIN: return min_avx512_f32(a, -1);
            }
        } else {                              // src/core/ops_dispatch.cpp:360-424
            switch (op) {
            case R_SUM: return sum(a, -1);
            case R_MEAN: return mean(a, -1);
            case R_MAX: return max(a, -1);
            case R_MIN: return min(a, -1);
            }
        }
        throw std::runtime_error("ref_reduce: op not available on this path");
    }
    if (path == PATH_DISPATCH) {
        switch (op) {
        case R_SUM: return sum(a, dim);
        case R_MEAN: return mean(a, dim);
        case R_MAX: return max(a, dim);
        case R_MIN: return min(a, dim);
        }
    }
    // Dim-wise reductions only exist in the scalar path (src/core/opsmp.cpp:672-697).
    switch (op) {
    case R_SUM: return sum_mp(a, dim);
    case R_MEAN: return mean_mp(a, dim);
    case R_MAX: return max_mp(a, dim);
    case R_MIN: return min_mp(a, dim);
    case R_VAR: return var_chain(a, dim);
    }
    throw std::runtime_error("ref_reduce: unknown op");
}

template <typename F>
int64_t guarded(F&& f) {
    try {
        g_err.clear();
        return f();
    } catch (const std::exception& e) {
        g_err = e.what();
        return -1;
    } catch (...) {
        g_err = "unknown exception";
        return -1;
    }
}

}  // namespace

extern "C" {

const char* ref_last_error() { return g_err.c_str(); }

// bit 0: avx2, bit 1: avx512f (what the reference's dispatcher probes,
// src/core/ops_dispatch.cpp:23-36)
int ref_cpu_features() {
    int f = 0;
    if (__builtin_cpu_supports("avx2")) f |= 1;
    if (__builtin_cpu_supports("avx512f")) f |= 2;
    return f;
}

void ref_set_threads(int n) { if (n > 0) omp_set_num_threads(n); }
int ref_max_threads() { return omp_get_max_threads(); }

// All entries return the number of output elements, or -1 (message in ref_last_error()).
int64_t ref_binary(int path, int op, const RefView* a, const RefView* b, void* out, int64_t cap) {
    return guarded([&] { return emit(do_binary(path, op, wrap(a), wrap(b)), out, cap); });
}

int64_t ref_unary(int path, int op, const RefView* a, double scalar, void* out, int64_t cap) {
    return guarded([&] { return emit(do_unary(path, op, wrap(a), scalar), out, cap); });
}

int64_t ref_reduce(int path, int op, const RefView* a, int dim, void* out, int64_t cap) {
    return guarded([&] { return emit(do_reduce(path, op, wrap(a), dim), out, cap); });
}

// Tensor::contiguous()/clone() strided gather (src/core/tensor.cpp:60-116,233-236).
int64_t ref_contiguous(const RefView* a, void* out, int64_t cap) {
    return guarded([&] { return emit(wrap(a).clone(), out, cap); });
}

// Softmax over the last dim, the log-softmax recipe of src/neuralnet/loss.cpp:97-101 without
// the final log: max -> reshape -> sub -> exp -> sum -> reshape -> div.  `mask` (may be NULL)
// is added first with broadcasting (the additive causal/bias mask of the benchmark configs).
int64_t ref_softmax_lastdim(int exp_path, const RefView* x, const RefView* mask, void* out, int64_t cap) {
    return guarded([&] {
        Tensor t = wrap(x);
        if (mask) t = add_mp(t, wrap(mask));
        int last = (int)t.impl->ndim - 1;
        std::vector<size_t> keep = keepdim_shape(t, last);
        Tensor m = max_mp(t, last).reshape(keep);
        Tensor s = diff_mp(t, m);
        Tensor e = (exp_path == PATH_AVX2) ? exp_avx2_f32(s) : exp_avx512_f32(s);
        Tensor z = sum_mp(e, last).reshape(keep);
        return emit(div_mp(e, z), out, cap);
    });
}

// LayerNorm over the last dim, the BatchNorm recipe of
// src/neuralnet/batchnorm/batchnorm.cpp:103-113 applied row-wise.
int64_t ref_layernorm_lastdim(const RefView* x, const RefView* gamma, const RefView* beta,
                              double eps, void* out, int64_t cap) {
    return guarded([&] {
        Tensor t = wrap(x);
        int last = (int)t.impl->ndim - 1;
        std::vector<size_t> keep = keepdim_shape(t, last);
        Tensor mu = mean_mp(t, last).reshape(keep);
        Tensor d = diff_mp(t, mu);
        Tensor v = mean_mp(mult_mp(d, d), last).reshape(keep);
        Tensor r = pow_scalar_mp(add_scalar_mp(v, eps), -0.5);
        Tensor y = mult_mp(d, r);
        if (gamma) y = mult_mp(y, wrap(gamma));
        if (beta) y = add_mp(y, wrap(beta));
        return emit(y, out, cap);
    });
}

// Log-softmax over the last dim, the recipe of Loss::CrossEntropy (src/neuralnet/loss.cpp:97-104):
// max -> reshape -> sub -> exp -> sum -> reshape -> ln -> sub, with the SIMD exp flavour named by
// exp_path and the AVX2 ln (the flavour the product pins; the AVX-512 ln is numerically wrong).
int64_t ref_log_softmax_lastdim(int exp_path, const RefView* x, const RefView* mask, void* out, int64_t cap) {
    return guarded([&] {
        Tensor t = wrap(x);
        if (mask) t = add_mp(t, wrap(mask));
        int last = (int)t.impl->ndim - 1;
        std::vector<size_t> keep = keepdim_shape(t, last);
        Tensor m = max_mp(t, last).reshape(keep);
        Tensor s = diff_mp(t, m);
        Tensor e = (exp_path == PATH_AVX2) ? exp_avx2_f32(s) : exp_avx512_f32(s);
        Tensor z = sum_mp(e, last).reshape(keep);
        Tensor l = ln_avx2_f32(z);
        return emit(diff_mp(s, l), out, cap);
    });
}

// Tensor::gather (src/core/tensor.cpp:344-428).
int64_t ref_gather(const RefView* x, int dim, const RefView* index, void* out, int64_t cap) {
    return guarded([&] { return emit(wrap(x).gather(wrap(index), (size_t)dim), out, cap); });
}

// accumulate_grad (src/core/autograd.cpp:63-156).  `target` gives the parameter's shape; its
// gradient buffer is created by the reference (ensure_grad_buffer: contiguous, zeroed), seeded
// with `grad_init` (contiguous, target's numel), accumulated into, and copied out.
// The reference folds the broadcast axes with sum(g, axis) through its dispatcher, which throws
// on AVX-512 hosts ("sum_avx512: only dim=-1").  The folds are therefore done here with sum_mp,
// the function that dispatcher picks on every other host, keeping the folded dim as size 1;
// the reference's accumulate_grad then performs the accumulation step (incl. its NaN/Inf rule).
int64_t ref_accumulate_grad(const RefView* target, const void* grad_init, const RefView* src, void* out, int64_t cap) {
    return guarded([&] {
        Tensor t = wrap(target);
        ensure_grad_buffer(t, true);
        Tensorimpl* gi = t.impl->grad.get();
        if (!gi) throw std::runtime_error("reference created no gradient buffer");
        const size_t bytes = t.numel() * dtype_size(t.impl->dtype);
        std::memcpy((char*)gi->data->data.get() + gi->offset * dtype_size(gi->dtype), grad_init, bytes);
        Tensor g = wrap(src);
        const size_t td = t.impl->ndim, gd = g.impl->ndim, nd = td > gd ? td : gd;
        for (int i = (int)nd - 1; i >= 0; --i) {                    // autograd.cpp:72-82, last axis first
            const size_t tsz = (size_t)i < nd - td ? 1 : t.impl->shape[i - (nd - td)];
            if ((size_t)i < nd - gd) continue;
            const int ax = i - (int)(nd - gd);
            if (tsz == 1 && g.impl->shape[ax] > 1) g = sum_mp(g, ax).reshape(keepdim_shape(g, ax));
        }
        if (gd > td) {      // leading dims the target lacks are all 1 now: drop them, as sum() does
            std::vector<size_t> sh(g.impl->shape.begin() + (gd - td), g.impl->shape.end());
            if (sh.empty()) sh.push_back(1);
            g = g.reshape(sh);
        }
        accumulate_grad(t, g);
        if ((int64_t)bytes > cap) throw std::runtime_error("output buffer too small");
        std::memcpy(out, (const char*)gi->data->data.get() + gi->offset * dtype_size(gi->dtype), bytes);
        return (int64_t)t.numel();
    });
}

// BatchNorm forward statistics and normalisation with the reference's own operator sequence
// (src/neuralnet/batchnorm/batchnorm.cpp:40-61 and :103-113; the sums go through mean_mp, the
// function the dispatcher picks on hosts without AVX-512 — its AVX-512 path throws for dim-wise
// reductions).  x: contiguous [N, C, ...]; out_mean/out_var: C floats.
int64_t ref_channel_moments(const RefView* x, float* out_mean, float* out_var) {
    return guarded([&] {
        Tensor input = wrap(x);
        const size_t ndim = input.impl->ndim;
        std::vector<size_t> perm(ndim);
        perm[0] = 1;
        perm[1] = 0;
        for (size_t i = 2; i < ndim; ++i) perm[i] = i;
        const size_t C = input.impl->shape[1], rest = input.numel() / C;
        Tensor flat = input.permute(perm).reshape({C, rest});
        Tensor mean_val = mean_mp(flat, 1);
        Tensor diff = diff_mp(flat, mean_val.reshape({C, 1}));
        Tensor var_val = mean_mp(mult_mp(diff, diff), 1);
        std::memcpy(out_mean, mean_val.impl->data->data.get(), C * 4);
        std::memcpy(out_var, var_val.impl->data->data.get(), C * 4);
        return (int64_t)C;
    });
}

int64_t ref_batchnorm_apply(const RefView* x, const RefView* mean, const RefView* var, const RefView* gamma,
                            const RefView* beta, double eps, void* out, int64_t cap) {
    return guarded([&] {
        Tensor input = wrap(x);
        std::vector<size_t> bshape(input.impl->ndim, 1);
        bshape[1] = input.impl->shape[1];
        Tensor x_centered = diff_mp(input, wrap(mean).reshape(bshape));
        Tensor inv_std = pow_scalar_mp(add_scalar_mp(wrap(var).reshape(bshape), eps), -0.5);
        Tensor y = mult_mp(x_centered, inv_std);
        if (gamma) y = mult_mp(y, wrap(gamma).reshape(bshape));
        if (beta) y = add_mp(y, wrap(beta).reshape(bshape));
        return emit(y, out, cap);
    });
}

// matmul_mp (src/core/opsmp.cpp:460-558), the scalar back-end.
int64_t ref_matmul(const RefView* a, const RefView* b, void* out, int64_t cap) {
    return guarded([&] { return emit(matmul_mp(wrap(a), wrap(b)), out, cap); });
}

// cat_mp (src/core/opsmp.cpp:717-804).
int64_t ref_cat(const RefView* const* in, int count, int dim, void* out, int64_t cap) {
    return guarded([&] {
        std::vector<Tensor> ts;
        for (int i = 0; i < count; ++i) ts.push_back(wrap(in[i]));
        return emit(cat_mp(ts, (size_t)dim), out, cap);
    });
}

// Optimizer steps, src/neuralnet/train_utils.h:50-188 (SGD, Adam, AdamW): `steps` calls of
// step() on one fp32 parameter whose gradient buffer holds `grad` (the same gradient every
// step).  The updated parameter is copied to `param_out`; Adam's moment vectors are private to
// the reference's classes and are pinned through the parameter trajectory.
// kind: 0 SGD, 1 Adam, 2 AdamW, 3 Adamax, 4 NAdam, 5 RAdam, 6 RMSprop (beta2 carries alpha),
// 7 Adagrad, 8 Lion.
int64_t ref_optimizer_steps(int kind, const float* param, const float* grad, int64_t n, int steps,
                            double lr, double beta1, double beta2, double eps, double weight_decay,
                            float* param_out) {
    return guarded([&] {
        Tensor p({(size_t)n}, DType::Float32, true);
        std::memcpy(p.impl->data->data.get(), param, (size_t)n * 4);
        ensure_grad_buffer(p, true);
        std::memcpy(p.impl->grad->data->data.get(), grad, (size_t)n * 4);
        std::vector<Tensor*> params{&p};
        std::unique_ptr<Optimizer> opt;
        if (kind == 0) opt.reset(new SGD(params, lr));
        else if (kind == 1) opt.reset(new Adam(params, lr, beta1, beta2, eps));
        else if (kind == 2) opt.reset(new AdamW(params, lr, beta1, beta2, eps, weight_decay));
        else if (kind == 3) opt.reset(new Adamax(params, lr, beta1, beta2, eps));
        else if (kind == 4) opt.reset(new NAdam(params, lr, beta1, beta2, eps));
        else if (kind == 5) opt.reset(new RAdam(params, lr, beta1, beta2, eps));
        else if (kind == 6) opt.reset(new RMSprop(params, lr, beta2 /* alpha */, eps));
        else if (kind == 7) opt.reset(new Adagrad(params, lr, eps));
        else if (kind == 8) opt.reset(new Lion(params, lr, beta1, beta2, weight_decay));
        else throw std::runtime_error("ref_optimizer_steps: unknown kind");
        for (int s = 0; s < steps; ++s) opt->step();
        std::memcpy(param_out, p.impl->data->data.get(), (size_t)n * 4);
        return n;
    });
}

// The reference's own backward nodes on same-shape operands (no broadcast fold, so that
// accumulate_grad needs no dim-wise sum, which the dispatcher cannot do on AVX-512 hosts).
// Each entry builds the node, gives the result tensor a gradient buffer holding `g`, calls the
// node's backward and copies the operands' accumulated gradients out (they start at zero).
namespace {
Tensor owned_copy(const RefView* v, bool requires_grad) {
    Tensor src = wrap(v);
    Tensor t = src.contiguous().clone();
    t.requires_grad_(requires_grad);
    return t;
}
Tensor result_with_grad(const Tensor& like, const RefView* g) {
    Tensor self(like.shape(), like._dtype(), true);
    ensure_grad_buffer(self, true);
    Tensor gv = wrap(g).contiguous();
    std::memcpy(self.impl->grad->data->data.get(),
                (const char*)gv.impl->data->data.get() + gv.impl->offset * dtype_size(gv._dtype()),
                self.numel() * dtype_size(self._dtype()));
    return self;
}
int64_t emit_grad(const Tensor& t, void* out, int64_t cap) {
    if (!t.impl->grad) throw std::runtime_error("reference produced no gradient");
    Tensor g;
    g.impl = t.impl->grad;
    return emit(g, out, cap);
}
}  // namespace

// GradDiv::backward, src/core/autograd.cpp:188-202
int64_t ref_div_backward(const RefView* g, const RefView* a, const RefView* b, void* out_a, void* out_b, int64_t cap) {
    return guarded([&] {
        Tensor ta = owned_copy(a, true), tb = owned_copy(b, true);
        GradDiv node(ta, tb);
        Tensor self = result_with_grad(ta, g);
        node.backward(self);
        emit_grad(ta, out_a, cap);
        return emit_grad(tb, out_b, cap);
    });
}

// GradTanh::backward, src/core/autograd.cpp:434-438
int64_t ref_tanh_backward(const RefView* g, const RefView* t, void* out, int64_t cap) {
    return guarded([&] {
        Tensor tt = owned_copy(t, true);
        GradTanh node(tt);
        Tensor self = result_with_grad(tt, g);
        node.backward(self);
        return emit_grad(tt, out, cap);
    });
}

// GradCrossEntropy::backward, src/neuralnet/loss.cpp:319-370.  `grad_out` is the loss's incoming
// gradient (the node divides it by the batch size itself for reduction == "mean").
int64_t ref_cross_entropy_backward(const RefView* logits, const RefView* labels, int mean, double grad_out, void* out,
                                   int64_t cap) {
    return guarded([&] {
        Tensor pred = owned_copy(logits, true), target = owned_copy(labels, false);
        GradCrossEntropy node(pred, target, mean ? "mean" : "sum");
        Tensor self({1}, DType::Float32, true);
        ensure_grad_buffer(self, true);
        write_scalar_at(self.impl->grad->data->data.get(), 0, DType::Float32, grad_out);
        node.backward(self);
        return emit_grad(pred, out, cap);
    });
}

// Wall time (seconds, std::chrono like the reference's own test/time_avx.cpp:11-24) of one
// benchmark step on contiguous 1-d inputs of n elements: add, mul, exp, relu and the GELU
// chain, each through the named back-end, results dropped as soon as they exist (the output
// allocation every reference op performs is inside the time; no copy-out is).
double ref_bench_step(int path, const float* x, const float* y, int64_t n) {
    RefView vx{}, vy{};
    vx.base = (void*)x; vx.dtype = 0; vx.ndim = 1; vx.shape[0] = n; vx.stride[0] = 1;
    vy = vx; vy.base = (void*)y;
    try {
        g_err.clear();
        Tensor a = wrap(&vx), b = wrap(&vy);
        const int tanh_path = (path == PATH_AVX2) ? PATH_AVX2 : PATH_AVX512;
        auto t0 = std::chrono::high_resolution_clock::now();
        { Tensor r = do_binary(path, B_ADD, a, b); }
        { Tensor r = do_binary(path, B_MUL, a, b); }
        { Tensor r = do_unary(path, U_EXP, a, 0.0); }
        { Tensor r = do_unary(path, U_RELU, a, 0.0); }
        { Tensor r = gelu_chain(a, tanh_path); }
        auto t1 = std::chrono::high_resolution_clock::now();
        return std::chrono::duration<double>(t1 - t0).count();
    } catch (const std::exception& e) {
        g_err = e.what();
        return -1.0;
    }
}

// The same five operators timed one by one: seconds[0..4] = add, mul, exp, relu, GELU chain.
int ref_bench_ops(int path, const float* x, const float* y, int64_t n, double* seconds) {
    RefView vx{}, vy{};
    vx.base = (void*)x; vx.dtype = 0; vx.ndim = 1; vx.shape[0] = n; vx.stride[0] = 1;
    vy = vx; vy.base = (void*)y;
    try {
        g_err.clear();
        Tensor a = wrap(&vx), b = wrap(&vy);
        const int tanh_path = (path == PATH_AVX2) ? PATH_AVX2 : PATH_AVX512;
        using clk = std::chrono::high_resolution_clock;
        auto lap = [&](int i, clk::time_point t0) { seconds[i] = std::chrono::duration<double>(clk::now() - t0).count(); };
        { auto t0 = clk::now(); { Tensor r = do_binary(path, B_ADD, a, b); } lap(0, t0); }
        { auto t0 = clk::now(); { Tensor r = do_binary(path, B_MUL, a, b); } lap(1, t0); }
        { auto t0 = clk::now(); { Tensor r = do_unary(path, U_EXP, a, 0.0); } lap(2, t0); }
        { auto t0 = clk::now(); { Tensor r = do_unary(path, U_RELU, a, 0.0); } lap(3, t0); }
        { auto t0 = clk::now(); { Tensor r = gelu_chain(a, tanh_path); } lap(4, t0); }
        return 0;
    } catch (const std::exception& e) {
        g_err = e.what();
        return -1;
    }
}

}  // extern "C"
