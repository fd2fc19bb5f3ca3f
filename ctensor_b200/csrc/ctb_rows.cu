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
#include "ctb_sweep.cuh"
#include "ctb_backward.cuh"

namespace ctb {

namespace {

struct RowIdx {
    DimSet dims;                          // outer dims in ENUMERATION order (x's memory order)
    int64_t stride[3][CTB_MAX_DIMS];      // [0] = x, [1] = mask (elements), [2] = output row number
};

// For enumeration index `i`: offsets of the row's first element in x and in the mask, and the
// row's number in the (row-major) output.  Rows are walked in the order x lies in memory, so a
// permuted input is read sequentially and the output is written as a few sequential streams.
__device__ __forceinline__ void row_offsets(const RowIdx& o, int64_t i, int64_t* xo, int64_t* mo, int64_t* orow) {
    int64_t off[3] = {0, 0, 0};
    dimset_offsets<3>(o.dims, i, o.stride, off);
    *xo = off[0];
    *mo = off[1];
    *orow = off[2];
}

// Row maxima use fmaxf: like std::max(acc, v) of the reference it ignores a NaN v.

// Group-wide reductions whose result is the same bit pattern in every thread of the group.
// A CTA holds several groups (one row each); groups wider than a warp synchronise on their own
// named barrier (ids 1..15; id 0 is the CTA barrier), so a group at the ragged end of the grid
// can leave without stalling its neighbours.
template <int GROUP>
__device__ __forceinline__ void group_barrier() {
    if (GROUP > 32) asm volatile("bar.sync %0, %1;" ::"r"(1 + (int)threadIdx.x / GROUP), "r"(GROUP) : "memory");
}

template <int GROUP>
__device__ __forceinline__ float group_max(float v, float* smem) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, off));
    if (GROUP == 32) return v;
    float* s = smem + (threadIdx.x / GROUP) * (GROUP / 32);
    group_barrier<GROUP>();                 // the slots may still be read from the previous use
    if ((threadIdx.x & 31) == 0) s[(threadIdx.x % GROUP) >> 5] = v;
    group_barrier<GROUP>();
    float r = s[0];
#pragma unroll
    for (int i = 1; i < GROUP / 32; ++i) r = fmaxf(r, s[i]);
    return r;
}

template <int GROUP>
__device__ __forceinline__ double group_sum(double v, double* smem) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) v = __dadd_rn(v, __shfl_xor_sync(0xffffffffu, v, off));
    if (GROUP == 32) return v;
    double* s = smem + (threadIdx.x / GROUP) * (GROUP / 32);
    group_barrier<GROUP>();
    if ((threadIdx.x & 31) == 0) s[(threadIdx.x % GROUP) >> 5] = v;
    group_barrier<GROUP>();
    double r = s[0];
#pragma unroll
    for (int i = 1; i < GROUP / 32; ++i) r = __dadd_rn(r, s[i]);
    return r;
}

// CTA-wide variants for the long-row kernels (every thread of the CTA takes part).
__device__ __forceinline__ float cta_max256(float v, float* smem) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, off));
    __syncthreads();
    if ((threadIdx.x & 31) == 0) smem[threadIdx.x >> 5] = v;
    __syncthreads();
    float r = smem[0];
#pragma unroll
    for (int i = 1; i < 8; ++i) r = fmaxf(r, smem[i]);
    return r;
}
__device__ __forceinline__ double cta_sum256(double v, double* smem) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) v = __dadd_rn(v, __shfl_xor_sync(0xffffffffu, v, off));
    __syncthreads();
    if ((threadIdx.x & 31) == 0) smem[threadIdx.x >> 5] = v;
    __syncthreads();
    double r = smem[0];
#pragma unroll
    for (int i = 1; i < 8; ++i) r = __dadd_rn(r, smem[i]);
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
// r = row_reciprocal(z) is a usable reciprocal only for a normal z below 2^126: beyond that (a row
// whose exponentials hit the clamp, e.g. inf - inf = NaN arguments: each term 2.4e38), for an
// infinite or NaN sum and for a subnormal one the estimate is 0, NaN or infinite, and the row is
// divided by IEEE division — e / inf = 0, e / NaN = NaN, as the reference's div gives.
__device__ __forceinline__ bool reciprocal_usable(float r) { return r > 0.0f && r < INFINITY; }
__device__ __forceinline__ float div_by_row(float e, float z, float r) {
    if (!reciprocal_usable(r)) return __fdiv_rn(e, z);
    const float q = __fmul_rn(e, r);
    const float rem = fmaf(-z, q, e);
    float out = fmaf(rem, r, q);
    if (e < 1e-30f) out = (e == 0.0f) ? 0.0f : __fdiv_rn(e, z);    // rare: quotient may be subnormal
    return out;
}

// Threads per CTA: 8 warp-rows; for row groups of 128/256 threads, 512 threads while a thread
// holds at most 4 vectors and 256 threads when it holds more (measured: 2048 columns 6.1 against
// 5.8 TB/s with 512, 4096 columns 6.7 against 6.3 and 8192 columns 6.4 against 5.2 with 256).
// (CTAs that hold a single 4 KiB row each measured 2.4x slower than 8 rows per CTA: the kernel
// becomes bound by CTA launch rate.)
template <int GROUP, int NV> struct RowCta {
    static constexpr int kThreads = GROUP == 32 ? 256 : (GROUP > 256 ? GROUP : (NV <= 4 ? 512 : 256));
};

// MODE bits (compile time, so the unrolled load loop has no run-time branch and all loads of a
// row are in flight together): 1 = additive mask, 2 = the mask's last dim is contiguous
// (else one value per row), 4 = causal, 8 = log-softmax: out = (t - m) - log((float)sum), the
// chain of Loss::CrossEntropy (src/neuralnet/loss.cpp:97-104); not combined with causal.
template <int GROUP, int VEC, int NV, int MODE>
__global__ void __launch_bounds__(RowCta<GROUP, NV>::kThreads)
softmax_rows_kernel(const float* __restrict__ x, const float* __restrict__ mask, float* __restrict__ out,
                    RowIdx o, int64_t rows, int cols, int64_t qlen) {
    constexpr int THREADS = RowCta<GROUP, NV>::kThreads;
    constexpr int GPC = THREADS / GROUP;                // rows per CTA
    constexpr bool has_mask = (MODE & 1) != 0, m_inner = (MODE & 2) != 0, causal = (MODE & 4) != 0;
    constexpr bool log_out = (MODE & 8) != 0;
    __shared__ float smax[THREADS / 32];
    __shared__ double ssum[THREADS / 32];
    const int tid = threadIdx.x % GROUP;
    const int64_t ridx = (int64_t)blockIdx.x * GPC + threadIdx.x / GROUP;
    if (ridx >= rows) return;                           // whole groups leave together
    int64_t xo, mo, row;
    row_offsets(o, ridx, &xo, &mo, &row);
    const float* xr = x + xo;
    int live = cols;                                    // columns [0, live) take part
    if (causal) live = min(cols, (int)(row % qlen) + 1);
    float t[NV][VEC];
    float m = -INFINITY;
    // Pass A issues every load of the row back to back (nothing else in the loop body, so all
    // of them are in flight together); pass B applies mask / causal cut-off and takes the max.
    float m0 = 0.0f;
    if (has_mask && !m_inner) m0 = mask[mo];
    // (Which loop shape keeps all loads of the row in flight is decided by the instruction
    // scheduler; measured on B200: one loop for the plain case, two passes as soon as a mask or
    // the causal cut-off adds work between the loads.)
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int col = (i * GROUP + tid) * VEC;
        if (col < live) {
            load_vec<VEC>(t[i], xr, col, cols);
            if ((MODE & 7) == 0) {             // no mask, not causal (log-softmax included): one loop
#pragma unroll
                for (int k = 0; k < VEC; ++k) m = fmaxf(m, t[i][k]);
            }
        }
    }
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int col = (i * GROUP + tid) * VEC;
        if ((MODE & 7) != 0 && col < live) {
            if (has_mask) {
                float mv[VEC];
                if (m_inner) load_vec<VEC>(mv, mask + mo, col, cols);     // L1/L2 resident: short latency
                else {
#pragma unroll
                    for (int k = 0; k < VEC; ++k) mv[k] = m0;
                }
#pragma unroll
                for (int k = 0; k < VEC; ++k) t[i][k] = __fadd_rn(t[i][k], mv[k]);
            }
            if (causal) {                               // partly live vector: drop the masked lanes
#pragma unroll
                for (int k = 0; k < VEC; ++k)
                    if (col + k >= live) t[i][k] = -INFINITY;
            }
#pragma unroll
            for (int k = 0; k < VEC; ++k) m = fmaxf(m, t[i][k]);
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
                    const float2 sh = __fadd2_rn(make_float2(t[i][k], t[i][k + 1]), splat2(-m));
                    const float2 e = exp_cephes2(sh);
                    t[i][k] = log_out ? sh.x : e.x;           // log-softmax keeps the shifted input
                    t[i][k + 1] = log_out ? sh.y : e.y;
                    z = __dadd_rn(__dadd_rn(z, (double)e.x), (double)e.y);
                }
            } else {
#pragma unroll
                for (int k = 0; k < VEC; ++k) {
                    const float sh = __fsub_rn(t[i][k], m);
                    const float e = exp_cephes(sh);
                    t[i][k] = log_out ? sh : e;
                    z = __dadd_rn(z, (double)e);
                }
            }
        }
    }
    z = group_sum<GROUP>(z, ssum);
    const float zf = __double2float_rn(z);
    float* orow = out + row * (int64_t)cols;
    if constexpr (log_out) {
        const float lz = log_cephes(zf);
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            const int col = (i * GROUP + tid) * VEC;
            if (col < cols) {
                float r[VEC];
#pragma unroll
                for (int k = 0; k < VEC; ++k) r[k] = __fsub_rn(t[i][k], lz);
                store_vec<VEC>(orow, col, r);
            }
        }
        return;
    }
    const float rz = row_reciprocal(zf);
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int col = (i * GROUP + tid) * VEC;
        if (col < cols) {
            float r[VEC];
            if (col < live) {
                if constexpr (VEC % 2 == 0) {
                    float smallest = t[i][0];
#pragma unroll
                    for (int k = 0; k < VEC; k += 2) {
                        const float2 e = make_float2(t[i][k], t[i][k + 1]);
                        const float2 q = __fmul2_rn(e, splat2(rz));
                        const float2 rem = __ffma2_rn(splat2(-zf), q, e);
                        const float2 res = __ffma2_rn(rem, splat2(rz), q);
                        r[k] = res.x;
                        r[k + 1] = res.y;
                        smallest = fminf(smallest, fminf(e.x, e.y));
                    }
                    if (!reciprocal_usable(rz)) {       // the row's sum is huge, infinite, NaN or subnormal
#pragma unroll
                        for (int k = 0; k < VEC; ++k) r[k] = __fdiv_rn(t[i][k], zf);
                    } else if (smallest < 1e-30f) {     // rare: a quotient may be subnormal (or e == 0)
#pragma unroll
                        for (int k = 0; k < VEC; ++k)
                            if (t[i][k] < 1e-30f) r[k] = (t[i][k] == 0.0f) ? 0.0f : __fdiv_rn(t[i][k], zf);
                    }
                } else {
#pragma unroll
                    for (int k = 0; k < VEC; ++k) r[k] = div_by_row(t[i][k], zf, rz);
                }
            } else {
#pragma unroll
                for (int k = 0; k < VEC; ++k) r[k] = 0.0f;
            }
            store_vec<VEC>(orow, col, r);
        }
    }
}

// ---- cross-entropy rows ------------------------------------------------------------------------------------
// Loss::CrossEntropy (src/neuralnet/loss.cpp:90-118) and GradCrossEntropy::backward (:319-370) on
// the same row-in-registers scheme: the logits are read once, and either one value per row is
// written (MODE 0: nll = -((x[label] - max) - ln((float)sum exp(x - max)))) or the gradient row
// (MODE 1: dx = (exp(x - max) * (1 / sum) - [c == label]) * scale; MODE 2: the same added into dx,
// NaN / infinite values skipped, which is accumulate_grad's rule, src/core/autograd.cpp:139-151).
// Labels are one Int32 per row, negative values counting from the end like Tensor::gather's; a
// label outside the row sets *bad and the row contributes 0 / no one-hot term.
__device__ __forceinline__ int64_t ce_label(int32_t label, int64_t classes, int32_t* bad) {
    int64_t l = label;
    if (l < 0) l += classes;
    if (l < 0 || l >= classes) {
        if (bad) *bad = 1;
        return -1;
    }
    return l;
}

#ifndef CTB_CE_LOSS_F32_PARTIALS
#define CTB_CE_LOSS_F32_PARTIALS 1
#endif

template <int GROUP, int VEC, int NV, int MODE>
__global__ void __launch_bounds__(RowCta<GROUP, NV>::kThreads)
ce_rows_kernel(const float* __restrict__ x, int64_t row_stride, const int32_t* __restrict__ labels, int64_t label_stride,
               int64_t rows, int cols, float scale, float* __restrict__ out, int64_t out_stride, int32_t* bad) {
    constexpr int THREADS = RowCta<GROUP, NV>::kThreads;
    constexpr int GPC = THREADS / GROUP;
    __shared__ float smax[THREADS / 32];
    __shared__ double ssum[THREADS / 32];
    const int tid = threadIdx.x % GROUP;
    const int64_t row = (int64_t)blockIdx.x * GPC + threadIdx.x / GROUP;
    if (row >= rows) return;                            // whole groups leave together
    const float* xr = x + row * row_stride;
    float t[NV][VEC];
    // the backward pass starts its maximum at the reference's value (loss.cpp:345)
    float m = MODE == 0 ? -INFINITY : -1e9f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int col = (i * GROUP + tid) * VEC;
        if (col < cols) {
            load_vec<VEC>(t[i], xr, col, cols);
#pragma unroll
            for (int k = 0; k < VEC; ++k) m = fmaxf(m, t[i][k]);
        }
    }
    m = group_max<GROUP>(m, smax);
    double z = 0.0;
    // The loss pass is bound by instruction issue (one exponential per 4 bytes read): a thread's own
    // terms (at most NV * VEC of them, each in (0, 1]) are summed in two fp32 lanes and widened once;
    // the gradient pass keeps the fp64 sum per term.
    constexpr bool kF32Partials = CTB_CE_LOSS_F32_PARTIALS && MODE == 0 && VEC % 2 == 0;
    float2 zz = make_float2(0.0f, 0.0f);
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int col = (i * GROUP + tid) * VEC;
        if (col < cols) {
            if constexpr (VEC % 2 == 0) {
#pragma unroll
                for (int k = 0; k < VEC; k += 2) {
                    const float2 sh = __fadd2_rn(make_float2(t[i][k], t[i][k + 1]), splat2(-m));
                    const float2 e = MODE == 0 ? exp_cephes2(sh) : exp_nan_through2(sh);
                    t[i][k] = e.x;
                    t[i][k + 1] = e.y;
                    if constexpr (kF32Partials) zz = __fadd2_rn(zz, e);
                    else z = __dadd_rn(__dadd_rn(z, (double)e.x), (double)e.y);
                }
            } else {
#pragma unroll
                for (int k = 0; k < VEC; ++k) {
                    t[i][k] = MODE == 0 ? exp_cephes(__fsub_rn(t[i][k], m)) : exp_nan_through(__fsub_rn(t[i][k], m));
                    z = __dadd_rn(z, (double)t[i][k]);
                }
            }
        }
    }
    if constexpr (kF32Partials) z = __dadd_rn((double)zz.x, (double)zz.y);
    z = group_sum<GROUP>(z, ssum);
    const float zf = __double2float_rn(z);
    const int64_t l = ce_label(labels[row * label_stride], cols, tid == 0 ? bad : nullptr);
    if constexpr (MODE == 0) {
        if (tid == 0) {
            float nll = 0.0f;
            if (l >= 0) {
                const float picked = __fsub_rn(__fsub_rn(xr[l], m), log_cephes(zf));
                nll = __double2float_rn(__dmul_rn((double)picked, -1.0));
            }
            out[row] = nll;
        }
        return;
    }
    const float inv = zf > 1e-12f ? __fdiv_rn(1.0f, zf) : 0.0f;
    float* orow = out + row * out_stride;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int col = (i * GROUP + tid) * VEC;
        if (col < cols) {
            float r[VEC];
#pragma unroll
            for (int k = 0; k < VEC; ++k) {
                float p = __fmul_rn(t[i][k], inv);
                if (col + k == l) p = __fsub_rn(p, 1.0f);
                r[k] = __fmul_rn(p, scale);
            }
            if constexpr (MODE == 2) {
                float old[VEC];
                load_vec<VEC>(old, orow, col, cols);
#pragma unroll
                for (int k = 0; k < VEC; ++k) r[k] = BinaryFn<kOpAddFinite, float>::apply(old[k], r[k]);
            }
            store_vec<VEC>(orow, col, r);
        }
    }
}

// CTA-wide reductions for the long-row kernels (any block size).
__device__ __forceinline__ float cta_max_any(float v, float* smem) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, off));
    const int nw = blockDim.x >> 5;
    __syncthreads();
    if ((threadIdx.x & 31) == 0) smem[threadIdx.x >> 5] = v;
    __syncthreads();
    float r = smem[0];
    for (int i = 1; i < nw; ++i) r = fmaxf(r, smem[i]);
    return r;
}
__device__ __forceinline__ double cta_sum_any(double v, double* smem) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) v = __dadd_rn(v, __shfl_xor_sync(0xffffffffu, v, off));
    const int nw = blockDim.x >> 5;
    __syncthreads();
    if ((threadIdx.x & 31) == 0) smem[threadIdx.x >> 5] = v;
    __syncthreads();
    double r = smem[0];
    for (int i = 1; i < nw; ++i) r = __dadd_rn(r, smem[i]);
    return r;
}

// Rows too long for one CTA's registers, spread over a thread-block cluster: each of the CS CTAs
// of a cluster stages cols/CS columns of the row in its shared memory (so several rows' CTAs share
// an SM and their load / compute / store phases overlap), and the row maximum and the row sum are
// exchanged through distributed shared memory.  x is read once, the result is written once.
// Every CTA of a cluster reaches every cluster barrier (no early exit), so the barriers cannot
// block.  Global accesses are 128-bit where the address allows it: the first elements of a
// CTA's range are handled one by one until the address is 16-byte aligned (row starts of a
// 50257-column matrix are not).
constexpr int kClusterRowThreads = 256;

__device__ __forceinline__ unsigned cluster_rank() {
    unsigned r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_barrier() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Value of the same shared-memory variable in CTA `rank` of the cluster.
template <typename T>
__device__ __forceinline__ T cluster_peer_load(const T* local, unsigned rank);
template <>
__device__ __forceinline__ float cluster_peer_load<float>(const float* local, unsigned rank) {
    unsigned a = (unsigned)__cvta_generic_to_shared(local), ra;
    float v;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(ra) : "r"(a), "r"(rank));
    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(ra) : "memory");
    return v;
}
template <>
__device__ __forceinline__ double cluster_peer_load<double>(const double* local, unsigned rank) {
    unsigned a = (unsigned)__cvta_generic_to_shared(local), ra;
    double v;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(ra) : "r"(a), "r"(rank));
    asm volatile("ld.shared::cluster.f64 %0, [%1];" : "=d"(v) : "r"(ra) : "memory");
    return v;
}

// Register variant of the cluster kernel for rows whose starts are 16-byte aligned and that carry
// no mask: every CTA of the cluster keeps 256 x NV x 4 columns of the row in registers (the same
// body as softmax_rows_kernel: packed exponentials, ~30 instructions per element) and only the two
// row-wide reductions cross CTAs through distributed shared memory.  LOG: log-softmax.
template <int CS, int NV, bool LOG>
__global__ void __launch_bounds__(kClusterRowThreads)
softmax_rows_cluster_reg_kernel(const float* __restrict__ x, float* __restrict__ out, RowIdx o, int64_t rows, int cols) {
    __shared__ float smax[kClusterRowThreads / 32];
    __shared__ double ssum[kClusterRowThreads / 32];
    __shared__ float cta_max;
    __shared__ double cta_sum;
    constexpr int T = kClusterRowThreads;
    const int tid = threadIdx.x;
    const unsigned rank = cluster_rank();
    const int64_t ridx = blockIdx.x / CS;
    int64_t xo, mo, row;
    row_offsets(o, ridx, &xo, &mo, &row);
    const int c_lo = (int)rank * (T * NV * 4);
    const float* xr = x + xo + c_lo;
    const int live = cols - c_lo;                       // columns of this CTA's range that exist (may be <= 0)
    float t[NV][4];
    float m = -INFINITY;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int col = (i * T + tid) * 4;
        if (col < live) {
            load_vec<4>(t[i], xr, col, cols);
#pragma unroll
            for (int k = 0; k < 4; ++k) m = fmaxf(m, t[i][k]);
        }
    }
    m = cta_max_any(m, smax);
    if (tid == 0) cta_max = m;
    cluster_barrier();
#pragma unroll
    for (unsigned r = 0; r < CS; ++r) m = fmaxf(m, cluster_peer_load(&cta_max, r));
    double z = 0.0;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int col = (i * T + tid) * 4;
        if (col < live) {
#pragma unroll
            for (int k = 0; k < 4; k += 2) {
                const float2 sh = __fadd2_rn(make_float2(t[i][k], t[i][k + 1]), splat2(-m));
                const float2 e = exp_cephes2(sh);
                t[i][k] = LOG ? sh.x : e.x;
                t[i][k + 1] = LOG ? sh.y : e.y;
                z = __dadd_rn(__dadd_rn(z, (double)e.x), (double)e.y);
            }
        }
    }
    z = cta_sum_any(z, ssum);
    if (tid == 0) cta_sum = z;
    cluster_barrier();
    z = 0.0;
#pragma unroll
    for (unsigned r = 0; r < CS; ++r) z = __dadd_rn(z, cluster_peer_load(&cta_sum, r));   // rank order: deterministic
    const float zf = __double2float_rn(z);
    const float rz = row_reciprocal(zf);
    const float lz = LOG ? log_cephes(zf) : 0.0f;
    float* orow = out + row * (int64_t)cols + c_lo;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int col = (i * T + tid) * 4;
        if (col < live) {
            float r[4];
            if (LOG) {
#pragma unroll
                for (int k = 0; k < 4; ++k) r[k] = __fsub_rn(t[i][k], lz);
            } else {
                float smallest = t[i][0];
#pragma unroll
                for (int k = 0; k < 4; k += 2) {
                    const float2 e = make_float2(t[i][k], t[i][k + 1]);
                    const float2 q = __fmul2_rn(e, splat2(rz));
                    const float2 rem = __ffma2_rn(splat2(-zf), q, e);
                    const float2 res = __ffma2_rn(rem, splat2(rz), q);
                    r[k] = res.x;
                    r[k + 1] = res.y;
                    smallest = fminf(smallest, fminf(e.x, e.y));
                }
                if (!reciprocal_usable(rz)) {           // the row's sum is huge, infinite, NaN or subnormal
#pragma unroll
                    for (int k = 0; k < 4; ++k) r[k] = __fdiv_rn(t[i][k], zf);
                } else if (smallest < 1e-30f) {         // rare: a quotient may be subnormal (or e == 0)
#pragma unroll
                    for (int k = 0; k < 4; ++k)
                        if (t[i][k] < 1e-30f) r[k] = (t[i][k] == 0.0f) ? 0.0f : __fdiv_rn(t[i][k], zf);
                }
            }
            store_vec<4>(orow, col, r);
        }
    }
    cluster_barrier();                                    // peers may still be reading cta_sum
}

// MODE (compile time): bit 0 = mask / causal handling compiled in (run-time flags decide),
// bit 3 (8) = log-softmax.  The plain modes (0 and 8) are what vocabulary logits use.
// Shared-memory layout: element i of this CTA's range sits at srow[i + a], a = (address of the
// range's first input element / 4) mod 4, so that 128-bit global loads land on 128-bit shared
// stores; the output range usually has the same alignment (b == a) and pass 3 is vector too.
template <int CS, int MODE>
__global__ void __launch_bounds__(kClusterRowThreads)
softmax_rows_cluster_kernel(const float* __restrict__ x, const float* __restrict__ mask, float* __restrict__ out,
                            RowIdx o, int64_t rows, int cols, int chunk, int64_t qlen, int m_inner, int has_mask_rt,
                            int causal_rt) {
    extern __shared__ __align__(16) float srow[];
    __shared__ float smax[kClusterRowThreads / 32];
    __shared__ double ssum[kClusterRowThreads / 32];
    __shared__ float cta_max;
    __shared__ double cta_sum;
    constexpr int T = kClusterRowThreads;
    constexpr bool general = (MODE & 1) != 0, log_out = (MODE & 8) != 0;
    using V4 = Vec<float, 4>;
    const bool has_mask = general && has_mask_rt, causal = general && causal_rt;
    const int tid = threadIdx.x;
    const unsigned rank = cluster_rank();
    const int64_t ridx = blockIdx.x / CS;                 // one row per cluster; the grid is rows * CS
    int64_t xo, mo, row;
    row_offsets(o, ridx, &xo, &mo, &row);
    const float* xr = x + xo;
    const float* mr = has_mask ? mask + mo : nullptr;
    const float m0 = (has_mask && !m_inner) ? mr[0] : 0.0f;
    const int live = causal ? (int)min((int64_t)cols, row % qlen + 1) : cols;
    const int c_lo = (int)rank * chunk;
    const int c_hi = min(c_lo + chunk, cols);             // this CTA's columns [c_lo, c_hi)
    const int n = c_hi - c_lo;                            // >= 1
    const int nl = max(0, min(c_hi, live) - c_lo);        // of which the first nl take part
    const int a = (int)((reinterpret_cast<uintptr_t>(xr + c_lo) >> 2) & 3);
    float* sr = srow + a;                                 // sr[i] = element i; sr + i is 16-byte aligned iff (i + a) % 4 == 0

    auto masked = [&](float t, int i) {
        if (has_mask) t = __fadd_rn(t, m_inner ? mr[c_lo + i] : m0);
        return t;
    };
    // vector body [v_lo, v_hi) of the live part in element indices (multiples of 4 after the shift)
    const int v_lo = min(nl, (4 - a) & 3);
    const int nvec = (nl - v_lo) >> 2;
    const int v_hi = v_lo + 4 * nvec;

    // pass 1: HBM -> shared memory, running maximum
    float m = -INFINITY;
    if (tid < v_lo) { const float t = masked(xr[c_lo + tid], tid); sr[tid] = t; m = fmaxf(m, t); }
    if (tid < nl - v_hi) { const int i = v_hi + tid; const float t = masked(xr[c_lo + i], i); sr[i] = t; m = fmaxf(m, t); }
    {
        const V4* xv = reinterpret_cast<const V4*>(xr + c_lo + v_lo);
        V4* sv = reinterpret_cast<V4*>(sr + v_lo);
        int j = tid;
        for (; j + 3 * T < nvec; j += 4 * T) {
            V4 v[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) v[u] = ldg_stream(xv + j + u * T);
#pragma unroll
            for (int u = 0; u < 4; ++u) {
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    if (general) v[u].v[k] = masked(v[u].v[k], v_lo + 4 * (j + u * T) + k);
                    m = fmaxf(m, v[u].v[k]);
                }
                sv[j + u * T] = v[u];
            }
        }
        for (; j < nvec; j += T) {
            V4 v = ldg_stream(xv + j);
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                if (general) v.v[k] = masked(v.v[k], v_lo + 4 * j + k);
                m = fmaxf(m, v.v[k]);
            }
            sv[j] = v;
        }
    }
    m = cta_max_any(m, smax);
    if (tid == 0) cta_max = m;
    cluster_barrier();
#pragma unroll
    for (unsigned r = 0; r < CS; ++r) m = fmaxf(m, cluster_peer_load(&cta_max, r));

    // pass 2: exponentials in place (log-softmax keeps the shifted input), fp64 partial sum
    double z = 0.0;
    auto expo = [&](int i) {
        const float sh = __fsub_rn(sr[i], m);
        const float e = exp_cephes(sh);
        sr[i] = log_out ? sh : e;
        z = __dadd_rn(z, (double)e);
    };
    if (tid < v_lo) expo(tid);
    if (tid < nl - v_hi) expo(v_hi + tid);
    {
        V4* sv = reinterpret_cast<V4*>(sr + v_lo);
        for (int j = tid; j < nvec; j += T) {
            V4 v = sv[j];
            const float2 s0 = __fadd2_rn(make_float2(v.v[0], v.v[1]), splat2(-m));
            const float2 s1 = __fadd2_rn(make_float2(v.v[2], v.v[3]), splat2(-m));
            const float2 e0 = exp_cephes2(s0), e1 = exp_cephes2(s1);
            z = __dadd_rn(__dadd_rn(__dadd_rn(__dadd_rn(z, (double)e0.x), (double)e0.y), (double)e1.x), (double)e1.y);
            if (log_out) { v.v[0] = s0.x; v.v[1] = s0.y; v.v[2] = s1.x; v.v[3] = s1.y; }
            else { v.v[0] = e0.x; v.v[1] = e0.y; v.v[2] = e1.x; v.v[3] = e1.y; }
            sv[j] = v;
        }
    }
    z = cta_sum_any(z, ssum);
    if (tid == 0) cta_sum = z;
    cluster_barrier();
    z = 0.0;
#pragma unroll
    for (unsigned r = 0; r < CS; ++r) z = __dadd_rn(z, cluster_peer_load(&cta_sum, r));   // rank order: deterministic
    const float zf = __double2float_rn(z);
    const float rz = row_reciprocal(zf);
    const float lz = log_out ? log_cephes(zf) : 0.0f;

    // pass 3: shared memory -> HBM
    {
        float* orow = out + row * (int64_t)cols + c_lo;
        auto result = [&](int i) {
            if (general && i >= nl) return 0.0f;
            return log_out ? __fsub_rn(sr[i], lz) : div_by_row(sr[i], zf, rz);
        };
        const int b = (int)((reinterpret_cast<uintptr_t>(orow) >> 2) & 3);
        const int o_lo = min(n, (4 - b) & 3);
        const int onvec = (n - o_lo) >> 2;
        const int o_hi = o_lo + 4 * onvec;
        if (tid < o_lo) orow[tid] = result(tid);
        if (tid < n - o_hi) orow[o_hi + tid] = result(o_hi + tid);
        V4* ov = reinterpret_cast<V4*>(orow + o_lo);
        if (b == a) {                                     // shared and global vectors line up
            const V4* sv = reinterpret_cast<const V4*>(sr + o_lo);
            for (int j = tid; j < onvec; j += T) {
                V4 v = sv[j], r;
                if (log_out) {
                    const float2 r0 = __fadd2_rn(make_float2(v.v[0], v.v[1]), splat2(-lz));
                    const float2 r1 = __fadd2_rn(make_float2(v.v[2], v.v[3]), splat2(-lz));
                    r.v[0] = r0.x; r.v[1] = r0.y; r.v[2] = r1.x; r.v[3] = r1.y;
                } else {
                    // packed remainder-corrected quotient; IEEE division where a quotient may be subnormal
                    float smallest = v.v[0];
#pragma unroll
                    for (int k = 0; k < 4; k += 2) {
                        const float2 e = make_float2(v.v[k], v.v[k + 1]);
                        const float2 q = __fmul2_rn(e, splat2(rz));
                        const float2 rem = __ffma2_rn(splat2(-zf), q, e);
                        const float2 res = __ffma2_rn(rem, splat2(rz), q);
                        r.v[k] = res.x;
                        r.v[k + 1] = res.y;
                        smallest = fminf(smallest, fminf(e.x, e.y));
                    }
                    if (!reciprocal_usable(rz)) {
#pragma unroll
                        for (int k = 0; k < 4; ++k) r.v[k] = __fdiv_rn(v.v[k], zf);
                    } else if (smallest < 1e-30f) {
#pragma unroll
                        for (int k = 0; k < 4; ++k)
                            if (v.v[k] < 1e-30f) r.v[k] = (v.v[k] == 0.0f) ? 0.0f : __fdiv_rn(v.v[k], zf);
                    }
                }
                if (general) {
#pragma unroll
                    for (int k = 0; k < 4; ++k)
                        if (o_lo + 4 * j + k >= nl) r.v[k] = 0.0f;
                }
                stg_stream(ov + j, r);
            }
        } else {
            for (int j = tid; j < onvec; j += T) {
                V4 r;
#pragma unroll
                for (int k = 0; k < 4; ++k) r.v[k] = result(o_lo + 4 * j + k);
                stg_stream(ov + j, r);
            }
        }
    }
    cluster_barrier();                                    // peers may still be reading cta_sum
}

// Long rows: one CTA per row, three passes over global memory (the row is re-read from L2).
__global__ void __launch_bounds__(256)
softmax_rows_long_kernel(const float* __restrict__ x, const float* __restrict__ mask, float* __restrict__ out,
                         RowIdx o, int64_t rows, int64_t cols, int64_t qlen, int m_inner, int has_mask, int causal,
                         int log_out) {
    __shared__ float smax[8];
    __shared__ double ssum[8];
    for (int64_t ridx = blockIdx.x; ridx < rows; ridx += gridDim.x) {
        int64_t xo, mo, row;
        row_offsets(o, ridx, &xo, &mo, &row);
        const float* xr = x + xo;
        const float* mr = has_mask ? mask + mo : nullptr;
        const int64_t live = causal ? min(cols, row % qlen + 1) : cols;
        auto tval = [&](int64_t c) {
            float v = xr[c];
            if (has_mask) v = __fadd_rn(v, mr[m_inner ? c : 0]);
            return v;
        };
        float m = -INFINITY;
        for (int64_t c = threadIdx.x; c < live; c += 256) m = fmaxf(m, tval(c));
        m = cta_max256(m, smax);
        double z = 0.0;
        float* orow = out + row * cols;
        for (int64_t c = threadIdx.x; c < live; c += 256) {
            const float sh = __fsub_rn(tval(c), m);
            const float e = exp_cephes(sh);
            orow[c] = log_out ? sh : e;
            z = __dadd_rn(z, (double)e);
        }
        z = cta_sum256(z, ssum);
        const float zf = __double2float_rn(z);
        if (log_out) {
            const float lz = log_cephes(zf);
            for (int64_t c = threadIdx.x; c < cols; c += 256) orow[c] = __fsub_rn(orow[c], lz);
            continue;
        }
        const float rz = row_reciprocal(zf);
        for (int64_t c = threadIdx.x; c < cols; c += 256) orow[c] = (c < live) ? div_by_row(orow[c], zf, rz) : 0.0f;
    }
}

// Long rows without a mask, vectorised: one 512-thread CTA per row sweeps the row three times —
// maximum; exponentials (each computed once, written unnormalised, summed); division — with the
// second and third sweep served by L2 (a row of 50257 floats is 200 KB; two CTAs per SM keep 60 MB
// in flight).  Log-softmax writes nothing in the second sweep and reads x a third time.  The
// kernels that keep the row on chip across a cluster serialise load, reductions and store per row
// with two resident CTAs per SM; here every sweep is a plain stream with four vectors in flight.
// Rows whose start is not 16-byte aligned are peeled (at most three elements at either end); a row
// whose input and output start at different 16-byte phases is walked element by element.
#ifndef CTB_SOFTMAX_SWEEP
#define CTB_SOFTMAX_SWEEP 1
#endif
// vectors in flight per thread in the first sweep, the one that comes from HBM (8 against 4: +1 .. 5 %)
#ifndef CTB_SWEEP1_LOADS
#define CTB_SWEEP1_LOADS 8
#endif
#ifndef CTB_SOFTMAX_COLS_1024
#define CTB_SOFTMAX_COLS_1024 0
#endif
#ifndef CTB_CE_GRAD_COLS_1024
#define CTB_CE_GRAD_COLS_1024 0
#endif
#ifndef CTB_SOFTMAX_SWEEP_WIDE_COLS
#define CTB_SOFTMAX_SWEEP_WIDE_COLS 57344
#endif

// T = 512 (two CTAs per SM) or 1024 (one: half as many rows in flight, for rows so long that the
// rows of 296 CTAs, input and output, no longer fit in L2 together).
// (Issuing the next step's loads before consuming the current step's vectors — sweep_vectors'
// PIPELINED — measured within noise here, unlike in the cross-entropy gradient; the plain form is used.)
template <bool LOG, int T>
__global__ void __launch_bounds__(T, 1024 / T)
softmax_rows_sweep_kernel(const float* __restrict__ x, float* out, RowIdx o, int64_t rows, int64_t cols) {
    __shared__ float smax[T / 32];
    __shared__ double ssum[T / 32];
    using V4 = Vec<float, 4>;
    const int tid = threadIdx.x;
    for (int64_t ridx = blockIdx.x; ridx < rows; ridx += gridDim.x) {
        int64_t xo, mo, row;
        row_offsets(o, ridx, &xo, &mo, &row);
        const float* xr = x + xo;
        float* orow = out + row * cols;
        const bool same_phase = ((reinterpret_cast<uintptr_t>(xr) ^ reinterpret_cast<uintptr_t>(orow)) & 15) == 0;
        const int64_t head = same_phase ? min(cols, (int64_t)((4 - ((reinterpret_cast<uintptr_t>(xr) >> 2) & 3)) & 3)) : cols;
        const int64_t nvec = (cols - head) >> 2;
        const int64_t tail = head + 4 * nvec;                   // [0, head) and [tail, cols): element by element
        const V4* xv = reinterpret_cast<const V4*>(xr + head);
        V4* ov = reinterpret_cast<V4*>(orow + head);
        // ---- sweep 1: the maximum -------------------------------------------------------------------
        float m = -INFINITY;
        for (int64_t c = tid; c < head; c += T) m = fmaxf(m, xr[c]);
        for (int64_t c = tail + tid; c < cols; c += T) m = fmaxf(m, xr[c]);
        auto load_x = [&](int64_t k) { return ldg_stream(xv + k); };
        sweep_vectors<T, false, CTB_SWEEP1_LOADS>(nvec, tid, load_x, [&](const V4& v, int64_t) {
            m = fmaxf(fmaxf(m, fmaxf(v.v[0], v.v[1])), fmaxf(v.v[2], v.v[3]));
        });
        m = cta_max_any(m, smax);
        // ---- sweep 2: exponentials and their sum (from L2) ------------------------------------------------
        double z = 0.0;
        auto scalar_exp = [&](int64_t c) {
            const float e = exp_cephes(__fsub_rn(xr[c], m));
            if (!LOG) orow[c] = e;
            z = __dadd_rn(z, (double)e);
        };
        for (int64_t c = tid; c < head; c += T) scalar_exp(c);
        for (int64_t c = tail + tid; c < cols; c += T) scalar_exp(c);
        auto vector_exp = [&](const V4& v, int64_t k) {
            const float2 e0 = exp_cephes2(__fadd2_rn(make_float2(v.v[0], v.v[1]), splat2(-m)));
            const float2 e1 = exp_cephes2(__fadd2_rn(make_float2(v.v[2], v.v[3]), splat2(-m)));
            if (!LOG) {
                V4 e;
                e.v[0] = e0.x, e.v[1] = e0.y, e.v[2] = e1.x, e.v[3] = e1.y;
                stg_stream(ov + k, e);
            }
            const float2 s = __fadd2_rn(e0, e1);               // four terms in (0, 1] meet in fp32: one widening per vector
            z = __dadd_rn(z, (double)__fadd_rn(s.x, s.y));
        };
        sweep_vectors<T, false>(nvec, tid, load_x, vector_exp);
        z = cta_sum_any(z, ssum);
        const float zf = __double2float_rn(z);
        // ---- sweep 3: the result (every thread re-reads what it wrote itself) ------------------------------
        if constexpr (LOG) {
            const float lz = log_cephes(zf);
            auto fin = [&](float v) { return __fsub_rn(__fsub_rn(v, m), lz); };
            for (int64_t c = tid; c < head; c += T) orow[c] = fin(xr[c]);
            for (int64_t c = tail + tid; c < cols; c += T) orow[c] = fin(xr[c]);
            sweep_vectors<T, false>(nvec, tid, load_x, [&](V4 v, int64_t k) {
#pragma unroll
                for (int q = 0; q < 4; ++q) v.v[q] = fin(v.v[q]);
                stg_stream(ov + k, v);
            });
        } else {
            const float rz = row_reciprocal(zf);
            for (int64_t c = tid; c < head; c += T) orow[c] = div_by_row(orow[c], zf, rz);
            for (int64_t c = tail + tid; c < cols; c += T) orow[c] = div_by_row(orow[c], zf, rz);
            sweep_vectors<T, false>(nvec, tid, [&](int64_t k) { return ldg_stream(ov + k); }, [&](V4 v, int64_t k) {
#pragma unroll
                for (int q = 0; q < 4; ++q) v.v[q] = div_by_row(v.v[q], zf, rz);
                stg_stream(ov + k, v);
            });
        }
    }
}

// ---- layernorm -------------------------------------------------------------------------------------------
// mu = mean(x); d = x - mu; v = mean(d*d); r = (v + eps)^-0.5; y = d*r*gamma + beta, with
// mean(.) = (float)((double)(float)sum_fp64 * (1.0/cols)) and the scalar steps in double,
// as mul_scalar / add_scalar / pow_scalar do (src/core/opsmp.cpp:297,418-451).
// MODE (compile time): 0 = no scale/shift, 1 = gamma and beta are contiguous rows (vector
// loads), 2 = general (either may be absent or strided).
template <int GROUP, int VEC, int NV, int MODE>
__global__ void __launch_bounds__(RowCta<GROUP, NV>::kThreads)
layernorm_rows_kernel(const float* __restrict__ x, const float* __restrict__ gamma, int64_t gstride,
                      const float* __restrict__ beta, int64_t bstride, float* __restrict__ out,
                      RowIdx o, int64_t rows, int cols, double inv_cols, double eps) {
    constexpr int THREADS = RowCta<GROUP, NV>::kThreads;
    constexpr int GPC = THREADS / GROUP;
    __shared__ double ssum[THREADS / 32];
    const int tid = threadIdx.x % GROUP;
    const int64_t ridx = (int64_t)blockIdx.x * GPC + threadIdx.x / GROUP;
    if (ridx >= rows) return;
    int64_t xo, mo, row;
    row_offsets(o, ridx, &xo, &mo, &row);
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
    float* orow = out + row * (int64_t)cols;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int col = (i * GROUP + tid) * VEC;
        if (col < cols) {
            float r[VEC];
            if (MODE == 1) {
                float gv[VEC], bv[VEC];
                load_vec<VEC>(gv, gamma, col, cols);
                load_vec<VEC>(bv, beta, col, cols);
#pragma unroll
                for (int k = 0; k < VEC; ++k)
                    r[k] = __fadd_rn(__fmul_rn(__fmul_rn(t[i][k], rstd), gv[k]), bv[k]);
            } else {
#pragma unroll
                for (int k = 0; k < VEC; ++k) {
                    float y = __fmul_rn(t[i][k], rstd);
                    if (MODE == 2) {
                        if (gamma) y = __fmul_rn(y, gamma[(int64_t)(col + k) * gstride]);
                        if (beta) y = __fadd_rn(y, beta[(int64_t)(col + k) * bstride]);
                    }
                    r[k] = y;
                }
            }
            store_vec<VEC>(orow, col, r);
        }
    }
}

// Rows beyond the register kernels: one 512-thread CTA per row sweeps x three times — sum; squared
// deviations; result — the second and third sweep served by L2, the output written once (the
// arithmetic of layernorm_rows_kernel; rows are peeled to 16-byte alignment like the softmax
// sweeps).  Measured against the cluster-of-CTAs kernel it replaced (TB/s): [8192,32768] 4.2 -> 4.9;
// rows that kernel could not take went through a scalar loop: [5341,50257] 1.3 -> 3.7,
// [1000,262145] 1.0 -> 2.5; against the 1024-thread register CTA: [13000,20000] 3.4 -> 4.2.
// (Two sweeps — both moments about the row's first element in fp64, then the result — measured
// slower up to 65536 columns, 3.3 against 3.7 TB/s at 50257: four fp64 operations per element cost
// more than the sweep through L2 they save.)
#ifndef CTB_LAYERNORM_COLS_1024
#define CTB_LAYERNORM_COLS_1024 0
#endif
__global__ void __launch_bounds__(512, 2)
layernorm_rows_sweep_kernel(const float* __restrict__ x, const float* __restrict__ gamma, int64_t gstride,
                            const float* __restrict__ beta, int64_t bstride, float* __restrict__ out,
                            RowIdx o, int64_t rows, int64_t cols, double inv_cols, double eps) {
    __shared__ double ssum[16];
    using V4 = Vec<float, 4>;
    constexpr int T = 512;
    const int tid = threadIdx.x;
    for (int64_t ridx = blockIdx.x; ridx < rows; ridx += gridDim.x) {
        int64_t xo, mo, row;
        row_offsets(o, ridx, &xo, &mo, &row);
        const float* xr = x + xo;
        float* orow = out + row * cols;
        const bool same_phase = ((reinterpret_cast<uintptr_t>(xr) ^ reinterpret_cast<uintptr_t>(orow)) & 15) == 0;
        const int64_t head = same_phase ? min(cols, (int64_t)((4 - ((reinterpret_cast<uintptr_t>(xr) >> 2) & 3)) & 3)) : cols;
        const int64_t nvec = (cols - head) >> 2;
        const int64_t tail = head + 4 * nvec;
        const V4* xv = reinterpret_cast<const V4*>(xr + head);
        V4* ov = reinterpret_cast<V4*>(orow + head);
        // ---- sweep 1: the mean (four independent fp64 chains per thread, one per vector lane) ------------------
        auto load_x = [&](int64_t k) { return ldg_stream(xv + k); };
        double sl[4] = {0.0, 0.0, 0.0, 0.0};
        for (int64_t c = tid; c < head; c += T) sl[0] = __dadd_rn(sl[0], (double)xr[c]);
        for (int64_t c = tail + tid; c < cols; c += T) sl[1] = __dadd_rn(sl[1], (double)xr[c]);
        sweep_vectors<T, false, CTB_SWEEP1_LOADS>(nvec, tid, load_x, [&](const V4& v, int64_t) {
#pragma unroll
            for (int q = 0; q < 4; ++q) sl[q] = __dadd_rn(sl[q], (double)v.v[q]);
        });
        const double s = cta_sum_any(__dadd_rn(__dadd_rn(sl[0], sl[1]), __dadd_rn(sl[2], sl[3])), ssum);
        const float mu = __double2float_rn(__dmul_rn((double)__double2float_rn(s), inv_cols));
        // ---- sweep 2: the variance (from L2) -------------------------------------------------------------
        double vl[4] = {0.0, 0.0, 0.0, 0.0};
        auto dev2 = [&](float v, int lane) {
            const float d = __fsub_rn(v, mu);
            vl[lane] = __dadd_rn(vl[lane], (double)__fmul_rn(d, d));
        };
        for (int64_t c = tid; c < head; c += T) dev2(xr[c], 0);
        for (int64_t c = tail + tid; c < cols; c += T) dev2(xr[c], 1);
        sweep_vectors<T, false>(nvec, tid, load_x, [&](const V4& v, int64_t) {
#pragma unroll
            for (int q = 0; q < 4; ++q) dev2(v.v[q], q);
        });
        double s2 = __dadd_rn(__dadd_rn(vl[0], vl[1]), __dadd_rn(vl[2], vl[3]));
        s2 = cta_sum_any(s2, ssum);
        const float var = __double2float_rn(__dmul_rn((double)__double2float_rn(s2), inv_cols));
        const float ve = __double2float_rn(__dadd_rn((double)var, eps));
        const float rstd = __double2float_rn(__ddiv_rn(1.0, __dsqrt_rn((double)ve)));
        // ---- sweep 3: the result ---------------------------------------------------------------------------
        auto fin = [&](float v, int64_t c) {
            float y = __fmul_rn(__fsub_rn(v, mu), rstd);
            if (gamma) y = __fmul_rn(y, gamma[c * gstride]);
            if (beta) y = __fadd_rn(y, beta[c * bstride]);
            return y;
        };
        for (int64_t c = tid; c < head; c += T) orow[c] = fin(xr[c], c);
        for (int64_t c = tail + tid; c < cols; c += T) orow[c] = fin(xr[c], c);
        const bool gvec = (!gamma || (gstride == 1 && (reinterpret_cast<uintptr_t>(gamma + head) & 15) == 0)) &&
                          (!beta || (bstride == 1 && (reinterpret_cast<uintptr_t>(beta + head) & 15) == 0));
        auto vector_fin = [&](V4 v, int64_t k) {
            const int64_t c0 = head + 4 * k;
            if (gvec) {
                V4 gv, bv;
                if (gamma) gv = *reinterpret_cast<const V4*>(gamma + c0);
                if (beta) bv = *reinterpret_cast<const V4*>(beta + c0);
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    float y = __fmul_rn(__fsub_rn(v.v[q], mu), rstd);
                    if (gamma) y = __fmul_rn(y, gv.v[q]);
                    if (beta) y = __fadd_rn(y, bv.v[q]);
                    v.v[q] = y;
                }
            } else {
#pragma unroll
                for (int q = 0; q < 4; ++q) v.v[q] = fin(v.v[q], c0 + q);
            }
            stg_stream(ov + k, v);
        };
        sweep_vectors<T, false>(nvec, tid, load_x, vector_fin);
    }
}

RowIdx row_idx(const RowsGeom& g) {
    RowIdx o{};
    int order[CTB_MAX_DIMS];
    for (int d = 0; d < g.nouter; ++d) order[d] = d;
    for (int i = 1; i < g.nouter; ++i)          // by decreasing x stride; ties keep the logical order
        for (int j = i; j > 0 && g.xstride[order[j]] > g.xstride[order[j - 1]]; --j) {
            const int t = order[j]; order[j] = order[j - 1]; order[j - 1] = t;
        }
    int64_t out_stride[CTB_MAX_DIMS];
    int64_t run = 1;
    for (int d = g.nouter - 1; d >= 0; --d) { out_stride[d] = run; run *= g.oshape[d]; }
    int64_t shape[CTB_MAX_DIMS];
    for (int k = 0; k < g.nouter; ++k) {
        const int d = order[k];
        shape[k] = g.oshape[d];
        o.stride[0][k] = g.xstride[d];
        o.stride[1][k] = g.mstride[d];
        o.stride[2][k] = out_stride[d];
    }
    dimset_init(&o.dims, g.nouter, shape);
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

// One row per group, GPC groups per CTA, one pass per CTA.
int rows_grid(int64_t rows, int groups_per_cta) {
    int64_t blocks = ceil_div(rows, groups_per_cta);
    if (blocks > 0x7FFFFFFFll) blocks = 0x7FFFFFFFll;
    return (int)(blocks < 1 ? 1 : blocks);
}

}  // namespace

// Dispatch over (GROUP, VEC, NV): a warp per row up to 8 vectors per lane (1024 floats), then
// 128-, 256- and 512-thread groups (up to 16384 columns), and a 1024-thread CTA per row up to the
// caller's `cols_1024` columns (at most 32768; 0: never); MASKED is a compile-time switch so the
// plain case carries no mask/causal code.  Measured against the cluster kernels they replace
// (softmax / log-softmax / LayerNorm, TB/s): [16384,16384] 5.1 / 5.3 / 4.6 -> 5.2 / 5.7 / 5.8;
// [20000,12288] 4.1 / 4.2 / 3.6 -> 5.4 / 5.2 / 5.7.  The 1024-thread CTA ([10000,20000]: 3.7 / 3.7 /
// 3.3) lost to the three-sweep kernels (4.2 / 4.6 / 4.2) and now serves masked and causal rows and
// the accumulating cross-entropy gradient only.
#define CTB_MODES_SOFTMAX(KERNEL, G, V, N, ARGS)                                               \
    switch (mode) {                                                                            \
    case 0: KERNEL<G, V, N, 0><<<grid, thr, 0, st>>> ARGS; break;                              \
    case 1: KERNEL<G, V, N, 1><<<grid, thr, 0, st>>> ARGS; break;                              \
    case 3: KERNEL<G, V, N, 3><<<grid, thr, 0, st>>> ARGS; break;                              \
    case 4: KERNEL<G, V, N, 4><<<grid, thr, 0, st>>> ARGS; break;                              \
    case 5: KERNEL<G, V, N, 5><<<grid, thr, 0, st>>> ARGS; break;                              \
    case 7: KERNEL<G, V, N, 7><<<grid, thr, 0, st>>> ARGS; break;                              \
    case 8: KERNEL<G, V, N, 8><<<grid, thr, 0, st>>> ARGS; break;                              \
    case 9: KERNEL<G, V, N, 9><<<grid, thr, 0, st>>> ARGS; break;                              \
    default: KERNEL<G, V, N, 11><<<grid, thr, 0, st>>> ARGS; break;                            \
    }
#define CTB_MODES_LAYERNORM(KERNEL, G, V, N, ARGS)                                             \
    switch (mode) {                                                                            \
    case 0: KERNEL<G, V, N, 0><<<grid, thr, 0, st>>> ARGS; break;                              \
    case 1: KERNEL<G, V, N, 1><<<grid, thr, 0, st>>> ARGS; break;                              \
    default: KERNEL<G, V, N, 2><<<grid, thr, 0, st>>> ARGS; break;                             \
    }
#define CTB_MODES_CE(KERNEL, G, V, N, ARGS)                                                    \
    switch (mode) {                                                                            \
    case 0: KERNEL<G, V, N, 0><<<grid, thr, 0, st>>> ARGS; break;                              \
    case 1: KERNEL<G, V, N, 1><<<grid, thr, 0, st>>> ARGS; break;                              \
    default: KERNEL<G, V, N, 2><<<grid, thr, 0, st>>> ARGS; break;                             \
    }
#define CTB_ROWS_LAUNCH(MODES, KERNEL, G, V, N, ARGS)                                          \
    do {                                                                                       \
        const int grid = rows_grid(g.rows, RowCta<G, N>::kThreads / G);                        \
        const int thr = RowCta<G, N>::kThreads;                                                \
        MODES(KERNEL, G, V, N, ARGS)                                                           \
    } while (0)

// W16: CTB_ROWS_W16_ON keeps rows of 1025 .. 2048 columns with one warp per row (16 vectors per lane),
// CTB_ROWS_W16_OFF hands them to the 128-thread groups (and instantiates nothing).
#define CTB_ROWS_W16_ON(MODES, KERNEL, ARGS) else if (nv_warp <= 16) CTB_ROWS_LAUNCH(MODES, KERNEL, 32, 4, 16, ARGS);
#define CTB_ROWS_W16_OFF(MODES, KERNEL, ARGS)
#define CTB_ROWS_DISPATCH(MODES, KERNEL, ARGS, W16)                                                        \
    do {                                                                                       \
        const int64_t per_v = vec4 ? 4 : 1;                                                    \
        const int64_t nv_warp = ceil_div(g.cols, 32 * per_v);                                  \
        const int64_t nv_128 = ceil_div(g.cols, 128 * per_v);                                  \
        const int64_t nv_256 = ceil_div(g.cols, 256 * per_v);                                  \
        if (vec4) {                                                                            \
            if (nv_warp <= 1) CTB_ROWS_LAUNCH(MODES, KERNEL, 32, 4, 1, ARGS);                         \
            else if (nv_warp <= 2) CTB_ROWS_LAUNCH(MODES, KERNEL, 32, 4, 2, ARGS);                    \
            else if (nv_warp <= 4) CTB_ROWS_LAUNCH(MODES, KERNEL, 32, 4, 4, ARGS);                    \
            else if (nv_warp <= 8) CTB_ROWS_LAUNCH(MODES, KERNEL, 32, 4, 8, ARGS);                    \
            W16(MODES, KERNEL, ARGS)                                                           \
            else if (nv_128 <= 4) CTB_ROWS_LAUNCH(MODES, KERNEL, 128, 4, 4, ARGS);                    \
            else if (nv_128 <= 8) CTB_ROWS_LAUNCH(MODES, KERNEL, 128, 4, 8, ARGS);                    \
            else if (nv_256 <= 8) CTB_ROWS_LAUNCH(MODES, KERNEL, 256, 4, 8, ARGS);                    \
            else if (nv_256 <= 16) CTB_ROWS_LAUNCH(MODES, KERNEL, 512, 4, 8, ARGS);                   \
            else if (g.cols <= cols_1024) CTB_ROWS_LAUNCH(MODES, KERNEL, 1024, 4, 8, ARGS);           \
            else launched = false;                                                             \
        } else {                                                                               \
            if (nv_warp <= 4) CTB_ROWS_LAUNCH(MODES, KERNEL, 32, 1, 4, ARGS);                         \
            else if (nv_warp <= 16) CTB_ROWS_LAUNCH(MODES, KERNEL, 32, 1, 16, ARGS);                  \
            else if (nv_128 <= 16) CTB_ROWS_LAUNCH(MODES, KERNEL, 128, 1, 16, ARGS);                  \
            else if (nv_256 <= 32) CTB_ROWS_LAUNCH(MODES, KERNEL, 256, 1, 32, ARGS);                  \
            else launched = false;                                                             \
        }                                                                                      \
    } while (0)

namespace {

template <int CS, int MODE>
int launch_softmax_cluster_mode(int chunk, const RowsGeom& g, const float* x, const float* mask, int causal,
                                float* out, const RowIdx& o, cudaStream_t st) {
    const size_t smem = ((size_t)chunk + 4) * sizeof(float);         // + the alignment shift
    auto kernel = softmax_rows_cluster_kernel<CS, MODE>;
    CTB_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(g.rows * CS));
    cfg.blockDim = dim3(kClusterRowThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = CS;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    CTB_CUDA_TRY(cudaLaunchKernelEx(&cfg, kernel, x, mask, out, o, g.rows, (int)g.cols, chunk, g.qlen,
                                    (int)g.m_inner, (int)g.has_mask, causal));
    return CTB_OK;
}

template <int CS, int NV, bool LOG>
int launch_softmax_cluster_reg(const RowsGeom& g, const float* x, float* out, const RowIdx& o, cudaStream_t st) {
    auto kernel = softmax_rows_cluster_reg_kernel<CS, NV, LOG>;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(g.rows * CS));
    cfg.blockDim = dim3(kClusterRowThreads);
    cfg.dynamicSmemBytes = 0;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = CS;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    CTB_CUDA_TRY(cudaLaunchKernelEx(&cfg, kernel, x, out, o, g.rows, (int)g.cols));
    return CTB_OK;
}

// Aligned, unmasked rows of up to 4 x 8192 columns: the register variant.  Returns false when
// the shape is not covered.
bool try_softmax_cluster_reg(const RowsGeom& g, const float* x, int log_out, float* out, const RowIdx& o,
                             cudaStream_t st, int* rc) {
    constexpr int64_t per_cta = (int64_t)kClusterRowThreads * 8 * 4;       // NV = 8
    const int64_t need = ceil_div(g.cols, per_cta);
    // beyond 4 CTAs per row the shared-memory variant with its evenly cut ranges measured faster
    // ([5336,50304]: 3.8 against 3.6 TB/s)
    if (need > 4 || g.rows * 4 >= 0x7FFFFFFFll) return false;
#define CTB_REG_CLUSTER(CS)                                                                          \
    *rc = log_out ? launch_softmax_cluster_reg<CS, 8, true>(g, x, out, o, st)                        \
                  : launch_softmax_cluster_reg<CS, 8, false>(g, x, out, o, st)
    if (need <= 2) { CTB_REG_CLUSTER(2); }
    else { CTB_REG_CLUSTER(4); }
#undef CTB_REG_CLUSTER
    return true;
}

template <int CS>
int launch_softmax_cluster_cs(int chunk, const RowsGeom& g, const float* x, const float* mask, int causal,
                              int log_out, float* out, const RowIdx& o, cudaStream_t st) {
    const bool general = g.has_mask || causal;
    if (general) {
        if (log_out) return launch_softmax_cluster_mode<CS, 9>(chunk, g, x, mask, causal, out, o, st);
        return launch_softmax_cluster_mode<CS, 1>(chunk, g, x, mask, causal, out, o, st);
    }
    if (log_out) return launch_softmax_cluster_mode<CS, 8>(chunk, g, x, mask, causal, out, o, st);
    return launch_softmax_cluster_mode<CS, 0>(chunk, g, x, mask, causal, out, o, st);
}

int launch_softmax_cluster(int cs, int chunk, const RowsGeom& g, const float* x, const float* mask, int causal,
                           int log_out, float* out, const RowIdx& o, cudaStream_t st) {
    if (cs == 2) return launch_softmax_cluster_cs<2>(chunk, g, x, mask, causal, log_out, out, o, st);
    if (cs == 4) return launch_softmax_cluster_cs<4>(chunk, g, x, mask, causal, log_out, out, o, st);
    return launch_softmax_cluster_cs<8>(chunk, g, x, mask, causal, log_out, out, o, st);
}

}  // namespace

int launch_softmax(const RowsGeom& g, const float* x, const float* mask, int causal, int log_out, float* out,
                   cudaStream_t st) {
    if (g.rows == 0 || g.cols == 0) return CTB_OK;
    DeviceInfo di;
    int rc = current_device_info(&di);
    if (rc) return rc;
    const RowIdx o = row_idx(g);
    const bool vec4 = rows_vec4(g, x, mask, out);
    // mode 2 and 6 (contiguous flag without a mask) do not occur
    if (log_out && causal) return set_error(CTB_ERR_ARG, "log_softmax: no causal variant");
    const int mode = (g.has_mask ? 1 : 0) | (g.has_mask && g.m_inner ? 2 : 0) | (causal ? 4 : 0) | (log_out ? 8 : 0);
    bool launched = g.cols < 0x7FFFFFFFll && g.rows < 0x7FFFFFFFll;   // else: the grid-stride long-row kernel
    const int64_t cols_1024 = (g.has_mask || causal) ? 24576 : CTB_SOFTMAX_COLS_1024;       // plain rows: the sweeps
    if (launched)
        CTB_ROWS_DISPATCH(CTB_MODES_SOFTMAX, softmax_rows_kernel, (x, mask, out, o, g.rows, (int)g.cols, g.qlen), CTB_ROWS_W16_OFF);
    if (!launched) {
        const int grid = rows_grid(g.rows, 1);
        // clusters of 2 / 4 / 8 CTAs: about 8K - 12.5K columns (32 - 50 KiB of shared memory) per CTA
        // measured best ([5341,50257]: 3.1 / 3.7 / 3.2 TB/s with 2 / 4 / 8 CTAs)
        const int cs = g.cols <= 25600 ? 2 : (g.cols <= 51200 ? 4 : 8);
        const int64_t chunk = ceil_div(ceil_div(g.cols, cs), 4) * 4;
        // measured, [rows, cols] of 1 GiB, softmax / log-softmax in TB/s, sweeps against the cluster kernels:
        // 25000: 4.4 / 4.9 against 3.8 / 3.7; 32768: 4.9 / 5.2 against 4.7 / 4.7; 50257: 4.2 / 4.4 against
        // 3.6 / 3.7; 65536: 4.0 / 4.0 against 3.9 / 3.9; 131072: 3.1 / 3.6 against 3.5 / 3.5; 262145 (beyond
        // the clusters' reach): 2.5 / 3.1 against 0.8 / 1.1
        const bool cluster_reach = chunk * 4 <= 100 * 1024;
        if (CTB_SOFTMAX_SWEEP && !g.has_mask && !causal && (log_out || g.cols <= 98304 || !cluster_reach)) {
            if (g.cols <= CTB_SOFTMAX_SWEEP_WIDE_COLS) {
                if (log_out) softmax_rows_sweep_kernel<true, 512><<<grid, 512, 0, st>>>(x, out, o, g.rows, g.cols);
                else softmax_rows_sweep_kernel<false, 512><<<grid, 512, 0, st>>>(x, out, o, g.rows, g.cols);
            } else {
                if (log_out) softmax_rows_sweep_kernel<true, 1024><<<grid, 1024, 0, st>>>(x, out, o, g.rows, g.cols);
                else softmax_rows_sweep_kernel<false, 1024><<<grid, 1024, 0, st>>>(x, out, o, g.rows, g.cols);
            }
        } else if (vec4 && !g.has_mask && !causal && try_softmax_cluster_reg(g, x, log_out, out, o, st, &rc)) {
            if (rc) return rc;
        } else if (g.cols < 0x7FFFFFFFll && chunk * 4 <= 100 * 1024 && g.rows * cs < 0x7FFFFFFFll) {
            rc = launch_softmax_cluster(cs, (int)chunk, g, x, mask, causal, log_out, out, o, st);
            if (rc) return rc;
        } else {
            softmax_rows_long_kernel<<<grid, 256, 0, st>>>(x, mask, out, o, g.rows, g.cols, g.qlen, g.m_inner, g.has_mask, causal, log_out);
        }
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
    int mode = 2;
    if (!gamma && !beta) mode = 0;
    else if (gamma && beta && gstride == 1 && bstride == 1 && vec4 && is_aligned(gamma, 16) && is_aligned(beta, 16)) mode = 1;
    bool launched = g.cols < 0x7FFFFFFFll && g.rows < 0x7FFFFFFFll;   // else: the grid-stride long-row kernel
    const int64_t cols_1024 = CTB_LAYERNORM_COLS_1024;
    if (launched)
        CTB_ROWS_DISPATCH(CTB_MODES_LAYERNORM, layernorm_rows_kernel, (x, gamma, gstride, beta, bstride, out, o, g.rows, (int)g.cols, inv, eps), CTB_ROWS_W16_OFF);
    if (!launched) {
        const int grid = rows_grid(g.rows, 1);
        layernorm_rows_sweep_kernel<<<grid, 512, 0, st>>>(x, gamma, gstride, beta, bstride, out, o, g.rows, g.cols, inv, eps);
    }
    return cuda_error(cudaGetLastError(), "layernorm launch");
}

// Cross-entropy rows that fit the register scheme (up to 16384 classes; the gradient up to 32768).  mode 0: out = nll[rows];
// 1: out = dx; 2: out += dx.  Returns false, having launched nothing, for longer rows.
bool launch_ce_rows_registers(int mode, const float* x, int64_t row_stride, const int32_t* labels, int64_t label_stride,
                              int64_t rows, int64_t classes, float scale, float* out, int64_t out_stride, int32_t* bad,
                              cudaStream_t st) {
    struct { int64_t rows, cols; } g{rows, classes};
    bool vec4 = classes % 4 == 0 && is_aligned(x, 16) && row_stride % 4 == 0;
    if (mode != 0) vec4 = vec4 && is_aligned(out, 16) && out_stride % 4 == 0;
    bool launched = classes < 0x7FFFFFFFll && rows < 0x7FFFFFFFll;
    // a 1024-thread CTA per row beats the two-sweep kernel for the accumulating gradient (3.1 -> 4.3
    // TB/s at 32768 classes) but neither the three-sweep one of the plain gradient (4.7) nor the
    // loss pass, which writes nothing
    const int64_t cols_1024 = mode == 0 ? 0 : (mode == 1 ? CTB_CE_GRAD_COLS_1024 : 32768);
    // Rows of 1025 .. 2048 classes stay with one warp per row (16 vectors per lane) instead of 128
    // threads: the loss pass, bound by instruction issue, pays for a group's barriers by the element
    // (3.8 -> 5.4 TB/s at 2048 classes), and the gradient gains 7-10 %; softmax and LayerNorm
    // measured slower that way at 1280 .. 2048 columns and keep the 128-thread groups.
    if (launched)
        CTB_ROWS_DISPATCH(CTB_MODES_CE, ce_rows_kernel,
                          (x, row_stride, labels, label_stride, rows, (int)classes, scale, out, out_stride, bad), CTB_ROWS_W16_ON);
    return launched;
}

}  // namespace ctb
