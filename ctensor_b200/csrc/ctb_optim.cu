// Optimizer steps as fused in-place element-wise kernels: SGD, Adam and AdamW of the reference's
// src/neuralnet/train_utils.h:50-188 (fp32 fast paths; SGD also its double-precision fallback
// for the other dtypes).  Each step reads and writes every operand once: 12 B/element for SGD,
// 28 B/element for Adam (param, grad, m, v in; param, m, v out).
// The arithmetic follows the reference's expressions operation by operation in fp32 (the
// reference's shipped flags do not contract them), so results are bit-identical.
#include "ctb_common.cuh"
#include "ctb_math.cuh"

namespace ctb {

namespace {

constexpr int kOptThreads = 256;
constexpr int kOptVec = 4;

struct AdamArgs {
    float b1, one_minus_b1, b2, one_minus_b2, lr_t, eps;
    double lr_wd;            // lr * weight_decay (AdamW)
    int decoupled_decay;
};

// p[i] -= (float)lr * g[i]                                     (train_utils.h:66-68)
__device__ __forceinline__ float sgd_update(float p, float g, float lr) {
    return __fsub_rn(p, __fmul_rn(lr, g));
}

// theta -= (float)(lr*wd*theta);  m = b1*m + (1-b1)*g;  v = b2*v + (1-b2)*g*g;
// theta -= lr_t*m / (sqrt(v) + eps)                            (train_utils.h:121-126,178-183)
__device__ __forceinline__ void adam_update(float& p, float g, float& m, float& v, const AdamArgs& a) {
    if (a.decoupled_decay) p = __fsub_rn(p, __double2float_rn(__dmul_rn(a.lr_wd, (double)p)));
    m = __fadd_rn(__fmul_rn(a.b1, m), __fmul_rn(a.one_minus_b1, g));
    v = __fadd_rn(__fmul_rn(a.b2, v), __fmul_rn(__fmul_rn(a.one_minus_b2, g), g));
    p = __fsub_rn(p, __fdiv_rn(__fmul_rn(a.lr_t, m), __fadd_rn(__fsqrt_rn(v), a.eps)));
}

template <bool VECTOR>
__global__ void __launch_bounds__(kOptThreads)
sgd_f32_kernel(float* __restrict__ p, const float* __restrict__ g, int64_t n, float lr) {
    using V = Vec<float, kOptVec>;
    const int64_t i = ((int64_t)blockIdx.x * kOptThreads + threadIdx.x) * (VECTOR ? kOptVec : 1);
    if (VECTOR) {
        if (i + kOptVec <= n) {
            V vp = ldg_stream(reinterpret_cast<const V*>(p + i));
            const V vg = ldg_stream(reinterpret_cast<const V*>(g + i));
#pragma unroll
            for (int k = 0; k < kOptVec; ++k) vp.v[k] = sgd_update(vp.v[k], vg.v[k], lr);
            stg_stream(reinterpret_cast<V*>(p + i), vp);
        } else {
            for (int64_t j = i; j < n; ++j) p[j] = sgd_update(p[j], g[j], lr);
        }
    } else if (i < n) {
        p[i] = sgd_update(p[i], g[i], lr);
    }
}

// Fallback of the reference for the other dtypes: (T)(p - lr*g) in double (train_utils.h:72-76).
template <typename T>
__global__ void __launch_bounds__(kOptThreads)
sgd_generic_kernel(T* __restrict__ p, const T* __restrict__ g, int64_t n, double lr) {
    const int64_t i = (int64_t)blockIdx.x * kOptThreads + threadIdx.x;
    if (i < n) p[i] = from_double<T>(__dsub_rn(to_double(p[i]), __dmul_rn(lr, to_double(g[i]))));
}

template <bool VECTOR>
__global__ void __launch_bounds__(kOptThreads)
adam_f32_kernel(float* __restrict__ p, const float* __restrict__ g, float* __restrict__ m,
                float* __restrict__ v, int64_t n, AdamArgs a) {
    using V = Vec<float, kOptVec>;
    const int64_t i = ((int64_t)blockIdx.x * kOptThreads + threadIdx.x) * (VECTOR ? kOptVec : 1);
    if (VECTOR) {
        if (i + kOptVec <= n) {
            V vp = ldg_stream(reinterpret_cast<const V*>(p + i));
            const V vg = ldg_stream(reinterpret_cast<const V*>(g + i));
            V vm = ldg_stream(reinterpret_cast<const V*>(m + i));
            V vv = ldg_stream(reinterpret_cast<const V*>(v + i));
#pragma unroll
            for (int k = 0; k < kOptVec; ++k) adam_update(vp.v[k], vg.v[k], vm.v[k], vv.v[k], a);
            stg_stream(reinterpret_cast<V*>(p + i), vp);
            stg_stream(reinterpret_cast<V*>(m + i), vm);
            stg_stream(reinterpret_cast<V*>(v + i), vv);
        } else {
            for (int64_t j = i; j < n; ++j) adam_update(p[j], g[j], m[j], v[j], a);
        }
    } else if (i < n) {
        adam_update(p[i], g[i], m[i], v[i], a);
    }
}

// ---- the other optimizers of train_utils.h: Adamax :190-239, NAdam :241-291, RAdam :293-355,
// RMSprop :357-396, Adagrad :398-437, Lion :439-494 (fp32 fast paths) ------------------------------------
struct OptArgs {
    float b1, one_minus_b1, b2, one_minus_b2, step_size, eps, lr, lr_decay, rect, inv_bc1, inv_bc2;
    int rectified;      // RAdam: rho_t > 4
    int decay;          // Lion: weight_decay > 0
};

template <int KIND>
__device__ __forceinline__ void opt_update(float& p, float g, float& s1, float& s2, const OptArgs& a) {
    if (KIND == CTB_OPT_ADAMAX) {          // s1 = m, s2 = u
        s1 = __fadd_rn(__fmul_rn(a.b1, s1), __fmul_rn(a.one_minus_b1, g));
        const float x = __fmul_rn(a.b2, s2), y = fabsf(g);
        s2 = (x < y) ? y : x;              // std::max(x, y)
        p = __fsub_rn(p, __fdiv_rn(__fmul_rn(a.step_size, s1), __fadd_rn(s2, a.eps)));
    } else if (KIND == CTB_OPT_NADAM) {    // s1 = m, s2 = v
        s1 = __fadd_rn(__fmul_rn(a.b1, s1), __fmul_rn(a.one_minus_b1, g));
        s2 = __fadd_rn(__fmul_rn(a.b2, s2), __fmul_rn(__fmul_rn(a.one_minus_b2, g), g));
        const float mn = __fadd_rn(__fmul_rn(a.b1, s1), __fmul_rn(a.one_minus_b1, g));
        p = __fsub_rn(p, __fdiv_rn(__fmul_rn(a.step_size, mn), __fadd_rn(__fsqrt_rn(s2), a.eps)));
    } else if (KIND == CTB_OPT_RADAM) {    // s1 = m, s2 = v; inv_bc* hold (float)bias_correction*
        s1 = __fadd_rn(__fmul_rn(a.b1, s1), __fmul_rn(a.one_minus_b1, g));
        s2 = __fadd_rn(__fmul_rn(a.b2, s2), __fmul_rn(__fmul_rn(a.one_minus_b2, g), g));
        const float m_hat = __fdiv_rn(s1, a.inv_bc1);
        if (a.rectified) {
            const float v_hat = __fadd_rn(__fsqrt_rn(__fdiv_rn(s2, a.inv_bc2)), a.eps);
            p = __fsub_rn(p, __fdiv_rn(__fmul_rn(__fmul_rn(a.lr, a.rect), m_hat), v_hat));
        } else {
            p = __fsub_rn(p, __fmul_rn(a.lr, m_hat));
        }
    } else if (KIND == CTB_OPT_RMSPROP) {  // s1 = v; b2 holds alpha
        s1 = __fadd_rn(__fmul_rn(a.b2, s1), __fmul_rn(__fmul_rn(a.one_minus_b2, g), g));
        p = __fsub_rn(p, __fdiv_rn(__fmul_rn(a.lr, g), __fadd_rn(__fsqrt_rn(s1), a.eps)));
    } else if (KIND == CTB_OPT_ADAGRAD) {  // s1 = sum of squares
        s1 = __fadd_rn(s1, __fmul_rn(g, g));
        p = __fsub_rn(p, __fdiv_rn(__fmul_rn(a.lr, g), __fadd_rn(__fsqrt_rn(s1), a.eps)));
    } else {                               // Lion: s1 = m
        const float m_t = s1;
        if (a.decay) p = __fsub_rn(p, __fmul_rn(a.lr_decay, p));
        const float c = __fadd_rn(__fmul_rn(a.b1, m_t), __fmul_rn(a.one_minus_b1, g));
        const float sign = (c > 0.0f) ? 1.0f : ((c < 0.0f) ? -1.0f : 0.0f);
        p = __fsub_rn(p, __fmul_rn(a.lr, sign));
        s1 = __fadd_rn(__fmul_rn(a.b2, m_t), __fmul_rn(a.one_minus_b2, g));
    }
}

template <int KIND, bool TWO_STATES, bool VECTOR>
__global__ void __launch_bounds__(kOptThreads)
opt_f32_kernel(float* __restrict__ p, const float* __restrict__ g, float* __restrict__ s1, float* __restrict__ s2,
               int64_t n, OptArgs a) {
    using V = Vec<float, kOptVec>;
    const int64_t i = ((int64_t)blockIdx.x * kOptThreads + threadIdx.x) * (VECTOR ? kOptVec : 1);
    if (VECTOR && i + kOptVec <= n) {
        V vp = ldg_stream(reinterpret_cast<const V*>(p + i));
        const V vg = ldg_stream(reinterpret_cast<const V*>(g + i));
        V v1 = ldg_stream(reinterpret_cast<const V*>(s1 + i)), v2;
        if (TWO_STATES) v2 = ldg_stream(reinterpret_cast<const V*>(s2 + i));
#pragma unroll
        for (int k = 0; k < kOptVec; ++k) {
            float dummy = 0.0f;
            opt_update<KIND>(vp.v[k], vg.v[k], v1.v[k], TWO_STATES ? v2.v[k] : dummy, a);
        }
        stg_stream(reinterpret_cast<V*>(p + i), vp);
        stg_stream(reinterpret_cast<V*>(s1 + i), v1);
        if (TWO_STATES) stg_stream(reinterpret_cast<V*>(s2 + i), v2);
    } else {
        const int64_t end = VECTOR ? n : (i + 1 < n ? i + 1 : n);
        for (int64_t j = i; j < end; ++j) {
            float dummy = 0.0f;
            opt_update<KIND>(p[j], g[j], s1[j], TWO_STATES ? s2[j] : dummy, a);
        }
    }
}

template <int KIND, bool TWO_STATES>
void opt_launch(float* p, const float* g, float* s1, float* s2, int64_t n, const OptArgs& a, cudaStream_t st) {
    const bool vec = is_aligned(p, 16) && is_aligned(g, 16) && is_aligned(s1, 16) && (!TWO_STATES || is_aligned(s2, 16));
    if (vec) opt_f32_kernel<KIND, TWO_STATES, true><<<(unsigned)ceil_div(n, (int64_t)kOptThreads * kOptVec), kOptThreads, 0, st>>>(p, g, s1, s2, n, a);
    else opt_f32_kernel<KIND, TWO_STATES, false><<<(unsigned)ceil_div(n, (int64_t)kOptThreads), kOptThreads, 0, st>>>(p, g, s1, s2, n, a);
}

unsigned opt_grid(int64_t n, int per_thread) {
    return (unsigned)ceil_div(n, (int64_t)kOptThreads * per_thread);
}

}  // namespace

int launch_sgd(int dtype, void* p, const void* g, int64_t n, double lr, cudaStream_t st) {
    if (n == 0) return CTB_OK;
    if (n > (int64_t)0x7FFFFFFF * kOptThreads) return set_error(CTB_ERR_LIMIT, "optimizer step: tensor too large for one launch");
    switch (dtype) {
    case CTB_F32:
        if (is_aligned(p, 16) && is_aligned(g, 16))
            sgd_f32_kernel<true><<<opt_grid(n, kOptVec), kOptThreads, 0, st>>>((float*)p, (const float*)g, n, (float)lr);
        else
            sgd_f32_kernel<false><<<opt_grid(n, 1), kOptThreads, 0, st>>>((float*)p, (const float*)g, n, (float)lr);
        break;
    case CTB_I32: sgd_generic_kernel<int32_t><<<opt_grid(n, 1), kOptThreads, 0, st>>>((int32_t*)p, (const int32_t*)g, n, lr); break;
    case CTB_F64: sgd_generic_kernel<double><<<opt_grid(n, 1), kOptThreads, 0, st>>>((double*)p, (const double*)g, n, lr); break;
    default: return set_error(CTB_ERR_DTYPE, "sgd_step: unsupported dtype");
    }
    return cuda_error(cudaGetLastError(), "sgd launch");
}

int launch_adam(float* p, const float* g, float* m, float* v, int64_t n, double lr, double beta1, double beta2,
                double eps, int step, double weight_decay, int decoupled_decay, cudaStream_t st) {
    if (n == 0) return CTB_OK;
    if (n > (int64_t)0x7FFFFFFF * kOptThreads) return set_error(CTB_ERR_LIMIT, "optimizer step: tensor too large for one launch");
    AdamArgs a;
    a.b1 = (float)beta1;
    a.one_minus_b1 = 1.0f - (float)beta1;
    a.b2 = (float)beta2;
    a.one_minus_b2 = 1.0f - (float)beta2;
    const double bc1 = 1.0 - pow(beta1, step), bc2 = 1.0 - pow(beta2, step);    // train_utils.h:115-118
    a.lr_t = (float)(lr * sqrt(bc2) / bc1);
    a.eps = (float)eps;
    a.lr_wd = lr * weight_decay;
    a.decoupled_decay = decoupled_decay;
    if (is_aligned(p, 16) && is_aligned(g, 16) && is_aligned(m, 16) && is_aligned(v, 16))
        adam_f32_kernel<true><<<opt_grid(n, kOptVec), kOptThreads, 0, st>>>(p, g, m, v, n, a);
    else
        adam_f32_kernel<false><<<opt_grid(n, 1), kOptThreads, 0, st>>>(p, g, m, v, n, a);
    return cuda_error(cudaGetLastError(), "adam launch");
}

int launch_optimizer(int kind, float* p, const float* g, float* s1, float* s2, int64_t n,
                     const ctb_optimizer_hyper& h, int step, cudaStream_t st) {
    if (n == 0) return CTB_OK;
    if (n > (int64_t)0x7FFFFFFF * kOptThreads) return set_error(CTB_ERR_LIMIT, "optimizer step: tensor too large for one launch");
    OptArgs a{};
    a.b1 = (float)h.beta1;
    a.one_minus_b1 = 1.0f - (float)h.beta1;
    a.b2 = (float)h.beta2;
    a.one_minus_b2 = 1.0f - (float)h.beta2;
    a.eps = (float)h.eps;
    a.lr = (float)h.lr;
    const double bc1 = 1.0 - pow(h.beta1, step), bc2 = 1.0 - pow(h.beta2, step);
    switch (kind) {
    case CTB_OPT_ADAMAX:
        a.step_size = (float)(h.lr / bc1);
        opt_launch<CTB_OPT_ADAMAX, true>(p, g, s1, s2, n, a, st);
        break;
    case CTB_OPT_NADAM:
        a.step_size = (float)(h.lr * sqrt(bc2) / bc1);
        opt_launch<CTB_OPT_NADAM, true>(p, g, s1, s2, n, a, st);
        break;
    case CTB_OPT_RADAM: {
        // the reference's mixed float/double expressions, type for type (train_utils.h:303,328,341-343)
        const float rho_inf = 2.0f / (1.0f - (float)h.beta2) - 1.0f;
        const float rho_t = (float)(rho_inf - 2.0f * step * pow(h.beta2, step) / (1.0f - pow(h.beta2, step)));
        a.inv_bc1 = (float)bc1;
        a.inv_bc2 = (float)bc2;
        a.rectified = rho_t > 4.0f;
        if (a.rectified)
            a.rect = sqrtf(((rho_t - 4.0f) * (rho_t - 2.0f) * rho_inf) / ((rho_inf - 4.0f) * (rho_inf - 2.0f) * rho_t));
        opt_launch<CTB_OPT_RADAM, true>(p, g, s1, s2, n, a, st);
        break;
    }
    case CTB_OPT_RMSPROP:
        a.b2 = (float)h.alpha;
        a.one_minus_b2 = 1.0f - (float)h.alpha;
        opt_launch<CTB_OPT_RMSPROP, false>(p, g, s1, s2, n, a, st);
        break;
    case CTB_OPT_ADAGRAD:
        opt_launch<CTB_OPT_ADAGRAD, false>(p, g, s1, s2, n, a, st);
        break;
    case CTB_OPT_LION:
        a.lr_decay = (float)(h.lr * h.weight_decay);
        a.decay = h.weight_decay > 0;
        opt_launch<CTB_OPT_LION, false>(p, g, s1, s2, n, a, st);
        break;
    default:
        return set_error(CTB_ERR_ARG, "optimizer step: unknown optimizer %d", kind);
    }
    return cuda_error(cudaGetLastError(), "optimizer launch");
}

}  // namespace ctb
