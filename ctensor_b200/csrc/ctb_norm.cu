// BatchNorm forward as two kernels: per-channel moments and the normalisation, for x[N, C, S]
// (S = product of the trailing dims, 1 for a 2-d input).  They replace the chain of primitive
// operators in BatchNorm::forward of the reference (src/neuralnet/batchnorm/batchnorm.cpp:40-61
// statistics, :103-113 normalisation), which materialises a permuted copy of the input and six
// temporaries of the input's size.
#include "ctb_reduce.cuh"
#include "ctb_math.cuh"

namespace ctb {

namespace {

constexpr int kNormThreads = 256;
constexpr int kNormUnroll = 8;

struct Moments { double s1, s2; };          // sums of d and d*d, d = x - shift

__device__ __forceinline__ Moments moments_add(Moments a, const Moments& b) {
    a.s1 = __dadd_rn(a.s1, b.s1);
    a.s2 = __dadd_rn(a.s2, b.s2);
    return a;
}
__device__ __forceinline__ void moments_push(Moments& a, float x, double shift) {
    const double d = __dsub_rn((double)x, shift);
    a.s1 = __dadd_rn(a.s1, d);
    a.s2 = fma(d, d, a.s2);
}

// CTA-wide sum of Moments; result valid in thread 0.
__device__ __forceinline__ Moments moments_cta_sum(Moments m, Moments* smem) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
        m.s1 = __dadd_rn(m.s1, __shfl_down_sync(0xffffffffu, m.s1, off));
        m.s2 = __dadd_rn(m.s2, __shfl_down_sync(0xffffffffu, m.s2, off));
    }
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    __syncthreads();
    if (lane == 0) smem[w] = m;
    __syncthreads();
    if (w == 0) {
        m = lane < kNormThreads / 32 ? smem[lane] : Moments{0.0, 0.0};
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) {
            m.s1 = __dadd_rn(m.s1, __shfl_down_sync(0xffffffffu, m.s1, off));
            m.s2 = __dadd_rn(m.s2, __shfl_down_sync(0xffffffffu, m.s2, off));
        }
    }
    return m;
}

// mean = mul_scalar(sum, 1/count) as the reference's mean() does it: the fp64 sum rounded to
// fp32, times 1.0/count in double, rounded again (src/core/ops_dispatch.cpp:385-390).
// var  = biased variance from the shifted moments.
__device__ __forceinline__ void moments_finish(const Moments& m, double shift, double count, float* mean, float* var) {
    const float sum = __double2float_rn(fma(shift, count, m.s1));
    *mean = __double2float_rn(__dmul_rn((double)sum, 1.0 / count));
    double v = (m.s2 - m.s1 * m.s1 / count) / count;
    if (v < 0.0) v = 0.0;
    *var = __double2float_rn(v);
}

// grid = (C, splits).  CTA (c, g) folds the flattened (n, s) range [g*chunk, (g+1)*chunk) of
// channel c: element f lives at ((f / S) * C + c) * S + f % S.  VEC = 4 needs S % 4 == 0 (a vector
// never straddles two lines).  Partials are combined in split order by the CTA that draws the
// channel's last ticket.
template <int VEC>
__global__ void __launch_bounds__(kNormThreads)
channel_moments_kernel(const float* __restrict__ x, float* __restrict__ mean, float* __restrict__ var,
                       int64_t C, int64_t S, int64_t F, FastDiv divS, int64_t chunk,
                       uint32_t* tickets, Moments* partials) {
    using V = Vec<float, VEC>;
    __shared__ Moments smem[kNormThreads / 32];
    __shared__ bool is_last;
    const int64_t c = blockIdx.x;
    const int splits = gridDim.y;
    const double shift = (double)x[c * S];                       // x[0, c, 0]
    const int64_t lo = (int64_t)blockIdx.y * chunk;
    int64_t hi = lo + chunk;
    if (hi > F) hi = F;
    const int64_t line_step = C * S;
    Moments acc{0.0, 0.0};
    const int64_t stride = (int64_t)kNormThreads * VEC;
    int64_t f = lo + (int64_t)threadIdx.x * VEC;
    auto address = [&](int64_t ff) {
        const uint32_t n = fast_div((uint32_t)ff, divS);
        return x + (int64_t)n * line_step + c * S + (ff - (int64_t)n * S);
    };
    for (; f + (kNormUnroll - 1) * stride < hi; f += kNormUnroll * stride) {
        V v[kNormUnroll];
#pragma unroll
        for (int u = 0; u < kNormUnroll; ++u) v[u] = ldg_stream(reinterpret_cast<const V*>(address(f + u * stride)));
#pragma unroll
        for (int u = 0; u < kNormUnroll; ++u)
#pragma unroll
            for (int k = 0; k < VEC; ++k) moments_push(acc, v[u].v[k], shift);
    }
    for (; f < hi; f += stride) {
        const V v = ldg_stream(reinterpret_cast<const V*>(address(f)));
#pragma unroll
        for (int k = 0; k < VEC; ++k) moments_push(acc, v.v[k], shift);
    }
    acc = moments_cta_sum(acc, smem);
    if (splits == 1) {
        if (threadIdx.x == 0) moments_finish(acc, shift, (double)F, mean + c, var + c);
        return;
    }
    if (threadIdx.x == 0) {
        partials[c * splits + blockIdx.y] = acc;
        __threadfence();
        const uint32_t t = atomicAdd(&tickets[c], 1u);
        is_last = (t == (uint32_t)splits - 1);
        if (is_last) tickets[c] = 0;
    }
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    if (threadIdx.x == 0) {
        Moments total{0.0, 0.0};
        for (int s = 0; s < splits; ++s) {
            const ulonglong2 raw = __ldcg(reinterpret_cast<const ulonglong2*>(partials + c * splits + s));
            Moments p;
            p.s1 = __longlong_as_double((long long)raw.x);
            p.s2 = __longlong_as_double((long long)raw.y);
            total = moments_add(total, p);
        }
        moments_finish(total, shift, (double)F, mean + c, var + c);
    }
}

// rstd[c] = pow_scalar(add_scalar(var, eps), -0.5): both steps in double, each rounded to fp32
// (src/core/opsmp.cpp:418-451).
__global__ void rstd_kernel(const float* __restrict__ var, int64_t vstride, float* __restrict__ rstd, int64_t C, double eps) {
    const int64_t c = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (c < C) {
        const float ve = __double2float_rn(__dadd_rn((double)var[c * vstride], eps));
        rstd[c] = __double2float_rn(pow((double)ve, -0.5));
    }
}

// y = ((x - mean[c]) * rstd[c]) * gamma[c] + beta[c], every step rounded to fp32
// (batchnorm.cpp:103-113).  One vector of VEC elements per thread; with VEC = 4 either the four
// elements share a channel (S % 4 == 0) or they are four consecutive channels (S == 1, C % 4 == 0).
struct NormParams {
    const float* mean; int64_t mstride;
    const float* rstd;
    const float* gamma; int64_t gstride;     // may be null
    const float* beta; int64_t bstride;      // may be null
};

// PARAMS: 0 = the VEC elements share one channel (S % VEC == 0), 1 = consecutive channels with
// strided parameter views (S == 1), 2 = consecutive channels, all parameters contiguous and
// 16-byte aligned (vector loads).
template <int VEC, int PARAMS>
__global__ void __launch_bounds__(kNormThreads)
batchnorm_apply_kernel(const float* __restrict__ x, float* __restrict__ out, NormParams p, int64_t numel,
                       FastDiv divS, FastDiv divC) {
    using V = Vec<float, VEC>;
    const int64_t i = ((int64_t)blockIdx.x * kNormThreads + threadIdx.x) * VEC;
    if (i >= numel) return;
    V v = ldg_stream(reinterpret_cast<const V*>(x + i));
    const uint32_t line = fast_div((uint32_t)i, divS);                 // n * C + c  (i itself when S == 1)
    const uint32_t c0 = line - fast_div(line, divC) * divC.d;
    if constexpr (PARAMS == 2) {
        const V m = *reinterpret_cast<const V*>(p.mean + c0), r = *reinterpret_cast<const V*>(p.rstd + c0);
        V g, b;
        if (p.gamma) g = *reinterpret_cast<const V*>(p.gamma + c0);
        if (p.beta) b = *reinterpret_cast<const V*>(p.beta + c0);
#pragma unroll
        for (int k = 0; k < VEC; ++k) {
            float y = __fmul_rn(__fsub_rn(v.v[k], m.v[k]), r.v[k]);
            if (p.gamma) y = __fmul_rn(y, g.v[k]);
            if (p.beta) y = __fadd_rn(y, b.v[k]);
            v.v[k] = y;
        }
    } else {
#pragma unroll
        for (int k = 0; k < VEC; ++k) {
            const int64_t c = PARAMS == 1 ? c0 + k : c0;
            float y = __fmul_rn(__fsub_rn(v.v[k], p.mean[c * p.mstride]), p.rstd[c]);
            if (p.gamma) y = __fmul_rn(y, p.gamma[c * p.gstride]);
            if (p.beta) y = __fadd_rn(y, p.beta[c * p.bstride]);
            v.v[k] = y;
        }
    }
    stg_stream(reinterpret_cast<V*>(out + i), v);
}

// The shared-channel case (S % 8 == 0, 32-byte aligned tensors) with the tile shape of the
// contiguous elementwise kernels: one tile of 256 threads x 2 x 256-bit vectors per CTA, both loads
// issued before the first use ([128,256,64,128]: 6.37 TB/s with one 128-bit vector per thread).
__global__ void __launch_bounds__(kNormThreads)
batchnorm_apply_wide_kernel(const float* __restrict__ x, float* __restrict__ out, NormParams p, int64_t numel,
                            FastDiv divS, FastDiv divC) {
    using V = Vec<float, 8>;
    constexpr int U = 2;
    const int64_t base = (int64_t)blockIdx.x * (kNormThreads * 8 * U) + (int64_t)threadIdx.x * 8;
    V v[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
        const int64_t i = base + (int64_t)u * kNormThreads * 8;
        if (i < numel) v[u] = ldg_stream(reinterpret_cast<const V*>(x + i));
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
        const int64_t i = base + (int64_t)u * kNormThreads * 8;
        if (i >= numel) break;
        const uint32_t line = fast_div((uint32_t)i, divS);
        const uint32_t c = line - fast_div(line, divC) * divC.d;
        const float m = p.mean[c * p.mstride], r = p.rstd[c];
        const float g = p.gamma ? p.gamma[c * p.gstride] : 0.0f, b = p.beta ? p.beta[c * p.bstride] : 0.0f;
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            float y = __fmul_rn(__fsub_rn(v[u].v[k], m), r);
            if (p.gamma) y = __fmul_rn(y, g);
            if (p.beta) y = __fadd_rn(y, b);
            v[u].v[k] = y;
        }
        stg_stream(reinterpret_cast<V*>(out + i), v[u]);
    }
}

}  // namespace

size_t channel_moments_workspace_bytes(int64_t C, int sm_count) {
    // tickets, then up to one wave of partials (sm_count * 8 CTAs), never fewer than one per channel
    const int64_t ctas = (int64_t)sm_count * 8 > C ? (int64_t)sm_count * 8 : C;
    return kTicketBytes + (size_t)(ctas + C) * sizeof(Moments);
}

int launch_channel_moments(const float* x, float* mean, float* var, int64_t N, int64_t C, int64_t S,
                           void* ws, size_t ws_bytes, cudaStream_t st) {
    if (C == 0) return CTB_OK;
    const int64_t F = N * S;
    if (F == 0) return set_error(CTB_ERR_SHAPE, "batchnorm: empty batch");
    if (F >= 0x7FFFFFFFll || C > 65535 * 32ll) return set_error(CTB_ERR_LIMIT, "batchnorm: more than 2^31 elements per channel");
    DeviceInfo di;
    int rc = current_device_info(&di);
    if (rc) return rc;
    const bool vec4 = S % 4 == 0 && is_aligned(x, 16);
    const int64_t gran = (int64_t)kNormThreads * 4 * kNormUnroll;
    int64_t splits = ((int64_t)di.sm_count * 6) / C;                   // about one resident wave
    if (splits > F / gran) splits = F / gran;
    if (splits > 1 && C > kTicketSlots) splits = 1;
    if (splits < 1) splits = 1;
    int64_t chunk = ceil_div(ceil_div(F, splits), gran) * gran;
    splits = ceil_div(F, chunk);
    const size_t need = splits > 1 ? kTicketBytes + (size_t)C * splits * sizeof(Moments) : 0;
    if (need > ws_bytes || (need && !ws)) return set_error(CTB_ERR_WORKSPACE, "batchnorm: workspace of %zu bytes needed, %zu given", need, ws_bytes);
    uint32_t* tickets = (uint32_t*)ws;
    Moments* partials = (Moments*)((char*)ws + kTicketBytes);
    const FastDiv divS = make_fastdiv((uint32_t)S);
    dim3 grid((unsigned)C, (unsigned)splits);
    if (vec4) channel_moments_kernel<4><<<grid, kNormThreads, 0, st>>>(x, mean, var, C, S, F, divS, chunk, tickets, partials);
    else channel_moments_kernel<1><<<grid, kNormThreads, 0, st>>>(x, mean, var, C, S, F, divS, chunk, tickets, partials);
    return cuda_error(cudaGetLastError(), "channel moments launch");
}

int launch_batchnorm_apply(const float* x, const float* mean, int64_t mstride, const float* var, int64_t vstride,
                           const float* gamma, int64_t gstride, const float* beta, int64_t bstride, double eps,
                           float* rstd_scratch, float* out, int64_t N, int64_t C, int64_t S, cudaStream_t st) {
    const int64_t numel = N * C * S;
    if (numel == 0) return CTB_OK;
    if (numel >= 0x7FFFFFFFll) return set_error(CTB_ERR_LIMIT, "batchnorm: tensor too large for one launch");
    rstd_kernel<<<(unsigned)ceil_div(C, 256), 256, 0, st>>>(var, vstride, rstd_scratch, C, eps);
    NormParams p{mean, mstride, rstd_scratch, gamma, gstride, beta, bstride};
    const FastDiv divS = make_fastdiv((uint32_t)S), divC = make_fastdiv((uint32_t)C);
    const bool aligned = is_aligned(x, 16) && is_aligned(out, 16);
    const bool params_vec = mstride == 1 && is_aligned(mean, 16) && is_aligned(rstd_scratch, 16) &&
                            (!gamma || (gstride == 1 && is_aligned(gamma, 16))) &&
                            (!beta || (bstride == 1 && is_aligned(beta, 16)));
    const unsigned grid4 = (unsigned)ceil_div(numel, kNormThreads * 4);
    if (S % 8 == 0 && is_aligned(x, 32) && is_aligned(out, 32))
        batchnorm_apply_wide_kernel<<<(unsigned)ceil_div(numel, kNormThreads * 16), kNormThreads, 0, st>>>(x, out, p, numel, divS, divC);
    else if (aligned && S % 4 == 0)
        batchnorm_apply_kernel<4, 0><<<grid4, kNormThreads, 0, st>>>(x, out, p, numel, divS, divC);
    else if (aligned && S == 1 && C % 4 == 0 && params_vec)
        batchnorm_apply_kernel<4, 2><<<grid4, kNormThreads, 0, st>>>(x, out, p, numel, divS, divC);
    else if (aligned && S == 1 && C % 4 == 0)
        batchnorm_apply_kernel<4, 1><<<grid4, kNormThreads, 0, st>>>(x, out, p, numel, divS, divC);
    else
        batchnorm_apply_kernel<1, 0><<<(unsigned)ceil_div(numel, kNormThreads), kNormThreads, 0, st>>>(x, out, p, numel, divS, divC);
    return cuda_error(cudaGetLastError(), "batchnorm apply launch");
}

}  // namespace ctb
