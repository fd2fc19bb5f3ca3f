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

}  // namespace ctb
