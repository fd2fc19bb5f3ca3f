// Fused row kernels: softmax and LayerNorm over the last dim, one pass over HBM.
//
// The reference has no such operators; its modules build them from primitive ops that each
// materialise a tensor (log-softmax inside Loss::CrossEntropy, src/neuralnet/loss.cpp:97-104;
// BatchNorm forward, src/neuralnet/batchnorm/batchnorm.cpp:103-113).  These kernels compute
// the same chains with the same fp32 rounding after every step, but keep the row in
// registers: x (and the mask) are read once and the result is written once.
//
// A row is owned by a group of GROUP threads (a warp for short rows, a CTA otherwise); each
// thread keeps NV vectors of VEC floats.  Rows longer than GROUP*NV*VEC fall back to a
// re-reading kernel.
#include "ctb_reduce.cuh"
#include "ctb_math.cuh"

namespace ctb {

namespace {

struct RowIdx {
    DimSet dims;
    int64_t stride[2][CTB_MAX_DIMS];      // [0] = x, [1] = mask
};

// Offsets of a row's first element in x and in the mask.
__device__ __forceinline__ void row_offsets(const RowIdx& o, int64_t row, int64_t* xo, int64_t* mo) {
    int64_t off[2] = {0, 0};
    dimset_offsets<2>(o.dims, row, o.stride, off);
    *xo = off[0];
    *mo = off[1];
}

// max with the reference's NaN rule: std::max(acc, v) keeps acc unless acc < v.
__device__ __forceinline__ float max_ref(float acc, float v) { return (acc < v) ? v : acc; }

// Group-wide reductions whose result is the same bit pattern in every thread of the group.
template <int GROUP>
__device__ __forceinline__ float group_max(float v, float* smem) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) v = max_ref(v, __shfl_xor_sync(0xffffffffu, v, off));
    if (GROUP == 32) return v;
    const int w = threadIdx.x >> 5;
    __syncthreads();
    if ((threadIdx.x & 31) == 0) smem[w] = v;
    __syncthreads();
    float r = smem[0];
#pragma unroll
    for (int i = 1; i < GROUP / 32; ++i) r = max_ref(r, smem[i]);
    return r;
}

template <int GROUP>
__device__ __forceinline__ double group_sum(double v, double* smem) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) v = __dadd_rn(v, __shfl_xor_sync(0xffffffffu, v, off));
    if (GROUP == 32) return v;
    const int w = threadIdx.x >> 5;
    __syncthreads();
    if ((threadIdx.x & 31) == 0) smem[w] = v;
    __syncthreads();
    double r = smem[0];
#pragma unroll
    for (int i = 1; i < GROUP / 32; ++i) r = __dadd_rn(r, smem[i]);
    return r;
}

template <int VEC>
__device__ __forceinline__ void load_vec(float* dst, const float* src, int64_t col, int64_t cols) {
    if (VEC == 4) {
        Vec<float, 4> v = ldg_stream(reinterpret_cast<const Vec<float, 4>*>(src + col));
#pragma unroll
        for (int k = 0; k < 4; ++k) dst[k] = v.v[k];
    } else {
        dst[0] = src[col];
    }
}
template <int VEC>
__device__ __forceinline__ void store_vec(float* dst, int64_t col, const float* src) {
    if (VEC == 4) {
        Vec<float, 4> v;
#pragma unroll
        for (int k = 0; k < 4; ++k) v.v[k] = src[k];
        stg_stream(reinterpret_cast<Vec<float, 4>*>(dst + col), v);
    } else {
        dst[col] = src[0];
    }
}

// ---- softmax ---------------------------------------------------------------------------------------------
// t = x (+ mask); m = max(t); e = exp(t - m); z = (float)sum_fp64(e); out = e / z.
//
// `causal`: column j of row q (q = index within the second-to-last dim) is excluded when j > q.
// This equals adding a -1e9 mask tensor: the masked exponentials are exactly 0 (the exponent
// clamp of exp_cephes), so they change neither the maximum nor the sum for finite inputs, and
// their outputs are +0.  Fully masked vectors are therefore neither read nor evaluated.
//
// The division uses one reciprocal per row: r ~ 1/z (estimate + Newton step), then per element
// q = e*r, rem = fma(-z, q, e), out = fma(rem, r, q) — the remainder-corrected quotient, which
// equals IEEE e/z except in rare last-bit cases; quotients that may be subnormal take the IEEE
// division.  (The chain's stated tolerance for this step is 1e-5 relative.)
__device__ __forceinline__ float row_reciprocal(float z) {
    float r;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(z));
    const float err = fmaf(-z, r, 1.0f);
    return fmaf(r, err, r);
}
__device__ __forceinline__ float div_by_row(float e, float z, float r) {
    const float q = __fmul_rn(e, r);
    const float rem = fmaf(-z, q, e);
    float out = fmaf(rem, r, q);
    if (e < 1e-30f) out = (e == 0.0f) ? 0.0f : __fdiv_rn(e, z);    // rare: quotient may be subnormal
    return out;
}

template <int GROUP, int VEC, int NV>
__global__ void __launch_bounds__(GROUP == 32 ? 256 : GROUP)
softmax_rows_kernel(const float* __restrict__ x, const float* __restrict__ mask, float* __restrict__ out,
                    RowIdx o, int64_t rows, int64_t cols64, int64_t qlen, int m_inner, int has_mask, int causal) {
    __shared__ float smax[8];
    __shared__ double ssum[8];
    constexpr int GROUPS_PER_CTA = (GROUP == 32) ? 8 : 1;
    const int tid = (GROUP == 32) ? (threadIdx.x & 31) : threadIdx.x;
    const int cols = (int)cols64;                       // rows handled here have < 2^31 columns
    const int64_t g0 = (int64_t)blockIdx.x * GROUPS_PER_CTA + ((GROUP == 32) ? (threadIdx.x >> 5) : 0);
    const int64_t gstep = (int64_t)gridDim.x * GROUPS_PER_CTA;
    for (int64_t row = g0; row < rows; row += gstep) {
        int64_t xo, mo;
        row_offsets(o, row, &xo, &mo);
        const float* xr = x + xo;
        const float* mr = has_mask ? mask + mo : nullptr;
        int live = cols;                                // columns [0, live) take part
        if (causal) {
            int q = 0;
            if ((threadIdx.x & 31) == 0) q = (int)(row % qlen);
            q = __shfl_sync(0xffffffffu, q, 0);
            live = min(cols, q + 1);
        }
        float t[NV][VEC];
        float m = -INFINITY;
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            const int col = (i * GROUP + tid) * VEC;
            if (col < live) {
                load_vec<VEC>(t[i], xr, col, cols);
                if (has_mask) {
                    float mv[VEC];
                    if (m_inner) load_vec<VEC>(mv, mr, col, cols);
                    else {
#pragma unroll
                        for (int k = 0; k < VEC; ++k) mv[k] = mr[0];
                    }
#pragma unroll
                    for (int k = 0; k < VEC; ++k) t[i][k] = __fadd_rn(t[i][k], mv[k]);
                }
                if (causal && col + VEC > live) {        // partly live vector: drop the masked lanes
#pragma unroll
                    for (int k = 0; k < VEC; ++k)
                        if (col + k >= live) t[i][k] = -INFINITY;
                }
#pragma unroll
                for (int k = 0; k < VEC; ++k) m = fmaxf(m, t[i][k]);   // == std::max(acc, v): NaN v ignored
            }
        }
        m = group_max<GROUP>(m, smax);
        double z = 0.0;
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            const int col = (i * GROUP + tid) * VEC;
            if (col < live) {
                if constexpr (VEC % 2 == 0) {
#pragma unroll
                    for (int k = 0; k < VEC; k += 2) {
                        const float2 e = exp_cephes2(__fadd2_rn(make_float2(t[i][k], t[i][k + 1]), splat2(-m)));
                        t[i][k] = e.x;
                        t[i][k + 1] = e.y;
                    }
                } else {
#pragma unroll
                    for (int k = 0; k < VEC; ++k) t[i][k] = exp_cephes(__fsub_rn(t[i][k], m));
                }
#pragma unroll
                for (int k = 0; k < VEC; ++k) z = __dadd_rn(z, (double)t[i][k]);
            }
        }
        z = group_sum<GROUP>(z, ssum);
        const float zf = __double2float_rn(z);
        const float rz = row_reciprocal(zf);
        float* orow = out + row * cols64;
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            const int col = (i * GROUP + tid) * VEC;
            if (col < cols) {
                float r[VEC];
                if (col < live) {
#pragma unroll
                    for (int k = 0; k < VEC; ++k) r[k] = div_by_row(t[i][k], zf, rz);
                } else {
#pragma unroll
                    for (int k = 0; k < VEC; ++k) r[k] = 0.0f;
                }
                store_vec<VEC>(orow, col, r);
            }
        }
    }
}

// Long rows: one CTA per row, three passes over global memory (the row is re-read from L2).
__global__ void __launch_bounds__(256)
softmax_rows_long_kernel(const float* __restrict__ x, const float* __restrict__ mask, float* __restrict__ out,
                         RowIdx o, int64_t rows, int64_t cols, int64_t qlen, int m_inner, int has_mask, int causal) {
    __shared__ float smax[8];
    __shared__ double ssum[8];
    for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
        int64_t xo, mo;
        row_offsets(o, row, &xo, &mo);
        const float* xr = x + xo;
        const float* mr = has_mask ? mask + mo : nullptr;
        const int64_t live = causal ? min(cols, row % qlen + 1) : cols;
        auto tval = [&](int64_t c) {
            float v = xr[c];
            if (has_mask) v = __fadd_rn(v, mr[m_inner ? c : 0]);
            return v;
        };
        float m = -INFINITY;
        for (int64_t c = threadIdx.x; c < live; c += 256) m = max_ref(m, tval(c));
        m = group_max<256>(m, smax);
        double z = 0.0;
        float* orow = out + row * cols;
        for (int64_t c = threadIdx.x; c < live; c += 256) {
            float e = exp_cephes(__fsub_rn(tval(c), m));
            orow[c] = e;
            z = __dadd_rn(z, (double)e);
        }
        z = group_sum<256>(z, ssum);
        const float zf = __double2float_rn(z);
        const float rz = row_reciprocal(zf);
        for (int64_t c = threadIdx.x; c < cols; c += 256) orow[c] = (c < live) ? div_by_row(orow[c], zf, rz) : 0.0f;
    }
}

// ---- layernorm -------------------------------------------------------------------------------------------
// mu = mean(x); d = x - mu; v = mean(d*d); r = (v + eps)^-0.5; y = d*r*gamma + beta, with
// mean(.) = (float)((double)(float)sum_fp64 * (1.0/cols)) and the scalar steps in double,
// as mul_scalar / add_scalar / pow_scalar do (src/core/opsmp.cpp:297,418-451).
template <int GROUP, int VEC, int NV>
__global__ void __launch_bounds__(GROUP == 32 ? 256 : GROUP)
layernorm_rows_kernel(const float* __restrict__ x, const float* __restrict__ gamma, int64_t gstride,
                      const float* __restrict__ beta, int64_t bstride, float* __restrict__ out,
                      RowIdx o, int64_t rows, int64_t cols64, double inv_cols, double eps) {
    __shared__ double ssum[8];
    constexpr int GROUPS_PER_CTA = (GROUP == 32) ? 8 : 1;
    const int tid = (GROUP == 32) ? (threadIdx.x & 31) : threadIdx.x;
    const int cols = (int)cols64;
    const int64_t g0 = (int64_t)blockIdx.x * GROUPS_PER_CTA + ((GROUP == 32) ? (threadIdx.x >> 5) : 0);
    const int64_t gstep = (int64_t)gridDim.x * GROUPS_PER_CTA;
    for (int64_t row = g0; row < rows; row += gstep) {
        int64_t xo, mo;
        row_offsets(o, row, &xo, &mo);
        const float* xr = x + xo;
        float t[NV][VEC];
        double s = 0.0;
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            const int col = (i * GROUP + tid) * VEC;
            if (col < cols) {
                load_vec<VEC>(t[i], xr, col, cols);
#pragma unroll
                for (int k = 0; k < VEC; ++k) s = __dadd_rn(s, (double)t[i][k]);
            }
        }
        s = group_sum<GROUP>(s, ssum);
        const float mu = __double2float_rn(__dmul_rn((double)__double2float_rn(s), inv_cols));
        double s2 = 0.0;
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            const int col = (i * GROUP + tid) * VEC;
            if (col < cols) {
#pragma unroll
                for (int k = 0; k < VEC; ++k) {
                    t[i][k] = __fsub_rn(t[i][k], mu);
                    s2 = __dadd_rn(s2, (double)__fmul_rn(t[i][k], t[i][k]));
                }
            }
        }
        s2 = group_sum<GROUP>(s2, ssum);
        const float v = __double2float_rn(__dmul_rn((double)__double2float_rn(s2), inv_cols));
        const float ve = __double2float_rn(__dadd_rn((double)v, eps));
        const float rstd = __double2float_rn(__ddiv_rn(1.0, __dsqrt_rn((double)ve)));
        float* orow = out + row * cols64;
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            const int col = (i * GROUP + tid) * VEC;
            if (col < cols) {
                float r[VEC];
#pragma unroll
                for (int k = 0; k < VEC; ++k) {
                    float y = __fmul_rn(t[i][k], rstd);
                    if (gamma) y = __fmul_rn(y, gamma[(col + k) * gstride]);
                    if (beta) y = __fadd_rn(y, beta[(col + k) * bstride]);
                    r[k] = y;
                }
                store_vec<VEC>(orow, col, r);
            }
        }
    }
}

__global__ void __launch_bounds__(256)
layernorm_rows_long_kernel(const float* __restrict__ x, const float* __restrict__ gamma, int64_t gstride,
                           const float* __restrict__ beta, int64_t bstride, float* __restrict__ out,
                           RowIdx o, int64_t rows, int64_t cols, double inv_cols, double eps) {
    __shared__ double ssum[8];
    for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
        int64_t xo, mo;
        row_offsets(o, row, &xo, &mo);
        const float* xr = x + xo;
        double s = 0.0;
        for (int64_t c = threadIdx.x; c < cols; c += 256) s = __dadd_rn(s, (double)xr[c]);
        s = group_sum<256>(s, ssum);
        const float mu = __double2float_rn(__dmul_rn((double)__double2float_rn(s), inv_cols));
        double s2 = 0.0;
        float* orow = out + row * cols;
        for (int64_t c = threadIdx.x; c < cols; c += 256) {
            float d = __fsub_rn(xr[c], mu);
            orow[c] = d;
            s2 = __dadd_rn(s2, (double)__fmul_rn(d, d));
        }
        s2 = group_sum<256>(s2, ssum);
        const float v = __double2float_rn(__dmul_rn((double)__double2float_rn(s2), inv_cols));
        const float ve = __double2float_rn(__dadd_rn((double)v, eps));
        const float rstd = __double2float_rn(__ddiv_rn(1.0, __dsqrt_rn((double)ve)));
        for (int64_t c = threadIdx.x; c < cols; c += 256) {
            float y = __fmul_rn(orow[c], rstd);
            if (gamma) y = __fmul_rn(y, gamma[c * gstride]);
            if (beta) y = __fadd_rn(y, beta[c * bstride]);
            orow[c] = y;
        }
    }
}

RowIdx row_idx(const RowsGeom& g) {
    RowIdx o{};
    dimset_init(&o.dims, g.nouter, g.oshape);
    for (int d = 0; d < g.nouter; ++d) {
        o.stride[0][d] = g.xstride[d];
        o.stride[1][d] = g.mstride[d];
    }
    return o;
}

bool rows_vec4(const RowsGeom& g, const float* x, const float* m, const float* out) {
    if (g.cols % 4) return false;
    if (!is_aligned(x, 16) || !is_aligned(out, 16)) return false;
    for (int d = 0; d < g.nouter; ++d) if (g.xstride[d] % 4) return false;
    if (g.has_mask && g.m_inner) {
        if (!is_aligned(m, 16)) return false;
        for (int d = 0; d < g.nouter; ++d) if (g.mstride[d] % 4) return false;
    }
    return true;
}

// One pass per CTA (a grid of short-lived CTAs measured faster than a persistent one here).
int rows_grid(int64_t rows, int groups_per_cta, int /*sm_count*/, int /*ctas_per_sm*/) {
    int64_t blocks = ceil_div(rows, groups_per_cta);
    if (blocks > 0x7FFFFFFFll) blocks = 0x7FFFFFFFll;
    return (int)(blocks < 1 ? 1 : blocks);
}

}  // namespace

// Dispatch over (GROUP, VEC, NV): the smallest per-thread footprint that covers the row.
#define CTB_ROWS_DISPATCH(KERNEL, ARGS)                                                        \
    do {                                                                                       \
        const int64_t per_v = vec4 ? 4 : 1;                                                    \
        const int64_t nv_warp = ceil_div(g.cols, 32 * per_v);                                  \
        const int64_t nv_128 = ceil_div(g.cols, 128 * per_v);                                  \
        const int64_t nv_cta = ceil_div(g.cols, 256 * per_v);                                  \
        const int gw = rows_grid(g.rows, 8, di.sm_count, 8);                                   \
        const int gc = rows_grid(g.rows, 1, di.sm_count, 8);                                   \
        if (vec4) {                                                                            \
            if (nv_warp <= 1) KERNEL<32, 4, 1><<<gw, 256, 0, st>>> ARGS;                       \
            else if (nv_warp <= 2) KERNEL<32, 4, 2><<<gw, 256, 0, st>>> ARGS;                  \
            else if (nv_128 <= 1) KERNEL<128, 4, 1><<<gc, 128, 0, st>>> ARGS;                  \
            else if (nv_128 <= 2) KERNEL<128, 4, 2><<<gc, 128, 0, st>>> ARGS;                  \
            else if (nv_128 <= 4) KERNEL<128, 4, 4><<<gc, 128, 0, st>>> ARGS;                  \
            else if (nv_cta <= 4) KERNEL<256, 4, 4><<<gc, 256, 0, st>>> ARGS;                  \
            else if (nv_cta <= 8) KERNEL<256, 4, 8><<<gc, 256, 0, st>>> ARGS;                  \
            else launched = false;                                                             \
        } else {                                                                               \
            if (nv_warp <= 4) KERNEL<32, 1, 4><<<gw, 256, 0, st>>> ARGS;                       \
            else if (nv_128 <= 8) KERNEL<128, 1, 8><<<gc, 128, 0, st>>> ARGS;                  \
            else if (nv_cta <= 16) KERNEL<256, 1, 16><<<gc, 256, 0, st>>> ARGS;                \
            else if (nv_cta <= 32) KERNEL<256, 1, 32><<<gc, 256, 0, st>>> ARGS;                \
            else launched = false;                                                             \
        }                                                                                      \
    } while (0)

int launch_softmax(const RowsGeom& g, const float* x, const float* mask, int causal, float* out,
                   cudaStream_t st) {
    if (g.rows == 0 || g.cols == 0) return CTB_OK;
    DeviceInfo di;
    int rc = current_device_info(&di);
    if (rc) return rc;
    const RowIdx o = row_idx(g);
    const bool vec4 = rows_vec4(g, x, mask, out);
    bool launched = true;
    CTB_ROWS_DISPATCH(softmax_rows_kernel, (x, mask, out, o, g.rows, g.cols, g.qlen, g.m_inner, g.has_mask, causal));
    if (!launched) {
        const int grid = rows_grid(g.rows, 1, di.sm_count, 8);
        softmax_rows_long_kernel<<<grid, 256, 0, st>>>(x, mask, out, o, g.rows, g.cols, g.qlen, g.m_inner, g.has_mask, causal);
    }
    return cuda_error(cudaGetLastError(), "softmax launch");
}

int launch_layernorm(const RowsGeom& g, const float* x, const float* gamma, int64_t gstride,
                     const float* beta, int64_t bstride, double eps, float* out, cudaStream_t st) {
    if (g.rows == 0 || g.cols == 0) return CTB_OK;
    DeviceInfo di;
    int rc = current_device_info(&di);
    if (rc) return rc;
    const RowIdx o = row_idx(g);
    const bool vec4 = rows_vec4(g, x, nullptr, out);
    const double inv = 1.0 / (double)g.cols;
    bool launched = true;
    CTB_ROWS_DISPATCH(layernorm_rows_kernel, (x, gamma, gstride, beta, bstride, out, o, g.rows, g.cols, inv, eps));
    if (!launched) {
        const int grid = rows_grid(g.rows, 1, di.sm_count, 8);
        layernorm_rows_long_kernel<<<grid, 256, 0, st>>>(x, gamma, gstride, beta, bstride, out, o, g.rows, g.cols, inv, eps);
    }
    return cuda_error(cudaGetLastError(), "layernorm launch");
}

}  // namespace ctb
