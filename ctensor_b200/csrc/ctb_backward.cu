// Backward bodies the reference spells as chains of elementwise operators, and the
// cross-entropy rows of its loss module, each as one pass:
//
//   GradDiv::backward   src/core/autograd.cpp:188-202   da = g / b
//                                                       db = -((g * a) / ((b * b) + 1e-6))
//   GradTanh::backward  src/core/autograd.cpp:434-438   dt = g * (1 / (cosh t * cosh t))
//   Loss::CrossEntropy  src/neuralnet/loss.cpp:90-118   loss = mean|sum over rows of
//                                                       -(log_softmax(x)[row, label[row]])
//   GradCrossEntropy    src/neuralnet/loss.cpp:319-370  dx = (softmax(x) - onehot(label)) * scale
//
// The elementwise chains keep the reference's rounding points: every operator result is rounded
// to the tensor's dtype before the next one uses it, scalar steps are done in double and rounded
// once.  On the CPU each of those steps is a pass over a fresh temporary (six operators and five
// temporaries for db); here the operands are read once and the result is written — or added into
// an existing gradient buffer, skipping NaN / infinite values as accumulate_grad does
// (src/core/autograd.cpp:139-151) — once.
#include "ctb_common.cuh"
#include "ctb_math.cuh"
#include "ctb_sweep.cuh"
#include "ctb_backward.cuh"

namespace ctb {
namespace {

// ---- the three chains ------------------------------------------------------------------------------
template <int KIND, typename T> struct BwdFn;
template <typename T> struct BwdFn<kBwdDivA, T> {
    __device__ __forceinline__ static T apply(T g, T, T b) { return BinaryFn<CTB_DIV, T>::apply(g, b); }
};
template <typename T> struct BwdFn<kBwdDivB, T> {
    __device__ __forceinline__ static T apply(T g, T a, T b) {
        const T num = BinaryFn<CTB_MUL, T>::apply(g, a);
        const T den = BinaryFn<CTB_MUL, T>::apply(b, b);
        const T den_safe = from_double<T>(__dadd_rn(to_double(den), 1e-6));      // add_scalar
        const T res = BinaryFn<CTB_DIV, T>::apply(num, den_safe);
        return from_double<T>(__dmul_rn(to_double(res), -1.0));                  // mul_scalar
    }
};
// cosh: for Float32 the single-precision libm function — what the reference's SIMD back-ends call
// (std::cosh on a float, src/cpu/AVX512/ops_avx512_f32.cpp:459-477); the double-precision one for
// Double64.  Both are within a few ulp of the reference's result, far inside the 1e-5 contract.
template <typename T> __device__ __forceinline__ T cosh_of(T t) { return from_double<T>(cosh(to_double(t))); }
template <> __device__ __forceinline__ float cosh_of<float>(float t) { return coshf(t); }

template <typename T> struct BwdFn<kBwdTanh, T> {
    __device__ __forceinline__ static T apply(T g, T t, T) {
        const T c = cosh_of<T>(t);
        const T c2 = BinaryFn<CTB_MUL, T>::apply(c, c);
        const T inv = from_double<T>(__ddiv_rn(1.0, to_double(c2)));             // div_scalar_rev
        return BinaryFn<CTB_MUL, T>::apply(g, inv);
    }
};

template <typename T, bool ACC> __device__ __forceinline__ T finish(T old, T v) {
    return ACC ? BinaryFn<kOpAddFinite, T>::apply(old, v) : v;
}

// Every operand contiguous and of the result's shape: 128-bit accesses, one tile of
// 256 threads x 2 vectors per CTA, all loads issued before the first use.
template <int KIND, typename T, bool ACC, int VEC>
__global__ void __launch_bounds__(256)
bwd_flat_kernel(const T* __restrict__ g, const T* __restrict__ x, const T* __restrict__ y, T* __restrict__ out, int64_t n) {
    using V = Vec<T, VEC>;
    constexpr int U = 2;
    constexpr int64_t TILE = 256 * VEC * U;
    const int64_t base = (int64_t)blockIdx.x * TILE + (int64_t)threadIdx.x * VEC;
    constexpr bool NEED_Y = KIND != kBwdTanh;
    if ((int64_t)(blockIdx.x + 1) * TILE <= n) {
        V vg[U], vx[U], vy[U], vo[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int64_t at = base + (int64_t)u * 256 * VEC;
            vg[u] = ldg_stream(reinterpret_cast<const V*>(g + at));
            if (KIND != kBwdDivA) vx[u] = ldg_stream(reinterpret_cast<const V*>(x + at));
            if (NEED_Y) vy[u] = ldg_stream(reinterpret_cast<const V*>(y + at));
            if (ACC) vo[u] = ldg_stream(reinterpret_cast<const V*>(out + at));
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            V r;
#pragma unroll
            for (int k = 0; k < VEC; ++k)
                r.v[k] = finish<T, ACC>(ACC ? vo[u].v[k] : T(0),
                                        BwdFn<KIND, T>::apply(vg[u].v[k], KIND != kBwdDivA ? vx[u].v[k] : T(0), NEED_Y ? vy[u].v[k] : T(0)));
            stg_stream(reinterpret_cast<V*>(out + base + (int64_t)u * 256 * VEC), r);
        }
    } else {
        for (int64_t i = (int64_t)blockIdx.x * TILE + threadIdx.x; i < n; i += 256)
            out[i] = finish<T, ACC>(ACC ? out[i] : T(0),
                                    BwdFn<KIND, T>::apply(g[i], KIND != kBwdDivA ? x[i] : T(0), NEED_Y ? y[i] : T(0)));
    }
}

// Both gradients of a division in one pass over (g, a, b) when everything is contiguous: 20 bytes per
// element instead of the 28 of two separate passes.
template <typename T, bool ACC, int VEC>
__global__ void __launch_bounds__(256)
div_both_flat_kernel(const T* __restrict__ g, const T* __restrict__ a, const T* __restrict__ b, T* __restrict__ da,
                     T* __restrict__ db, int64_t n) {
    using V = Vec<T, VEC>;
    constexpr int64_t TILE = 256 * VEC;
    const int64_t base = (int64_t)blockIdx.x * TILE + (int64_t)threadIdx.x * VEC;
    if ((int64_t)(blockIdx.x + 1) * TILE <= n) {
        const V vg = ldg_stream(reinterpret_cast<const V*>(g + base));
        const V va = ldg_stream(reinterpret_cast<const V*>(a + base));
        const V vb = ldg_stream(reinterpret_cast<const V*>(b + base));
        V oa, ob;
        if (ACC) {
            oa = ldg_stream(reinterpret_cast<const V*>(da + base));
            ob = ldg_stream(reinterpret_cast<const V*>(db + base));
        }
        V ra, rb;
#pragma unroll
        for (int k = 0; k < VEC; ++k) {
            ra.v[k] = finish<T, ACC>(ACC ? oa.v[k] : T(0), BwdFn<kBwdDivA, T>::apply(vg.v[k], T(0), vb.v[k]));
            rb.v[k] = finish<T, ACC>(ACC ? ob.v[k] : T(0), BwdFn<kBwdDivB, T>::apply(vg.v[k], va.v[k], vb.v[k]));
        }
        stg_stream(reinterpret_cast<V*>(da + base), ra);
        stg_stream(reinterpret_cast<V*>(db + base), rb);
    } else {
        for (int64_t i = (int64_t)blockIdx.x * TILE + threadIdx.x; i < n; i += 256) {
            da[i] = finish<T, ACC>(ACC ? da[i] : T(0), BwdFn<kBwdDivA, T>::apply(g[i], T(0), b[i]));
            db[i] = finish<T, ACC>(ACC ? db[i] : T(0), BwdFn<kBwdDivB, T>::apply(g[i], a[i], b[i]));
        }
    }
}

// Any strides / broadcasting: one multiplier-division chain per element.
struct BwdIdx {
    DimSet dims;
    int64_t stride[4][CTB_MAX_DIMS];      // g, x, y, out
    int64_t numel;
};
template <int KIND, typename T, bool ACC>
__global__ void __launch_bounds__(256)
bwd_strided_kernel(const T* __restrict__ g, const T* __restrict__ x, const T* __restrict__ y, T* __restrict__ out, BwdIdx ix) {
    const int64_t step = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < ix.numel; i += step) {
        int64_t off[4] = {0, 0, 0, 0};
        dimset_offsets<4>(ix.dims, i, ix.stride, off);
        const T v = BwdFn<KIND, T>::apply(g[off[0]], x ? x[off[1]] : T(0), y ? y[off[2]] : T(0));
        out[off[3]] = finish<T, ACC>(ACC ? out[off[3]] : T(0), v);
    }
}

template <int KIND, typename T>
int launch_kind(const BwdPlan& p, const T* g, const T* x, const T* y, T* out, int accumulate, cudaStream_t st) {
    if (p.numel == 0) return CTB_OK;
    if (p.flat) {
        constexpr int VEC = 16 / sizeof(T);
        const bool aligned = is_aligned(g, 16) && is_aligned(out, 16) && (!x || is_aligned(x, 16)) && (!y || is_aligned(y, 16));
        const int64_t tile = 256 * 2 * (aligned ? VEC : 1);
        const unsigned grid = (unsigned)ceil_div(p.numel, tile);
        if (aligned) {
            if (accumulate) bwd_flat_kernel<KIND, T, true, VEC><<<grid, 256, 0, st>>>(g, x, y, out, p.numel);
            else bwd_flat_kernel<KIND, T, false, VEC><<<grid, 256, 0, st>>>(g, x, y, out, p.numel);
        } else {
            if (accumulate) bwd_flat_kernel<KIND, T, true, 1><<<grid, 256, 0, st>>>(g, x, y, out, p.numel);
            else bwd_flat_kernel<KIND, T, false, 1><<<grid, 256, 0, st>>>(g, x, y, out, p.numel);
        }
        return cuda_error(cudaGetLastError(), "backward chain launch");
    }
    BwdIdx ix{};
    dimset_init(&ix.dims, p.ndim, p.shape);
    ix.numel = p.numel;
    for (int k = 0; k < 4; ++k)
        for (int d = 0; d < p.ndim; ++d) ix.stride[k][d] = p.stride[k][d];
    int64_t blocks = ceil_div(p.numel, 256);
    if (blocks > 0x7FFFFFFFll) blocks = 0x7FFFFFFFll;
    if (accumulate) bwd_strided_kernel<KIND, T, true><<<(unsigned)blocks, 256, 0, st>>>(g, x, y, out, ix);
    else bwd_strided_kernel<KIND, T, false><<<(unsigned)blocks, 256, 0, st>>>(g, x, y, out, ix);
    return cuda_error(cudaGetLastError(), "backward chain launch");
}

template <typename T>
int launch_typed(int kind, const BwdPlan& p, const void* g, const void* x, const void* y, void* out, int accumulate,
                 cudaStream_t st) {
    switch (kind) {
    case kBwdDivA: return launch_kind<kBwdDivA, T>(p, (const T*)g, (const T*)nullptr, (const T*)y, (T*)out, accumulate, st);
    case kBwdDivB: return launch_kind<kBwdDivB, T>(p, (const T*)g, (const T*)x, (const T*)y, (T*)out, accumulate, st);
    case kBwdTanh: return launch_kind<kBwdTanh, T>(p, (const T*)g, (const T*)x, (const T*)nullptr, (T*)out, accumulate, st);
    }
    return set_error(CTB_ERR_ARG, "backward chain: unknown kind %d", kind);
}

// ---- cross-entropy rows ---------------------------------------------------------------------------------
// Rows of up to 16384 classes (32768 for the gradient) are served by the register-row kernel of
// ctb_rows.cu (one read of the logits).  The kernel here takes the longer rows (vocabulary-sized
// logits), one 512-thread CTA per row:
//   pass 1  one sweep over the row that keeps, per thread, a running maximum m and the sum
//           z = sum exp(x - m), rescaling z by exp(m_old - m_new) whenever the maximum moves (rare
//           after the first few elements); the CTA then folds the (m, z) pairs: M = max m,
//           Z = sum z * exp(m - M).  This equals max -> sub -> exp -> sum of Loss::CrossEntropy
//           (src/neuralnet/loss.cpp:97-101) up to the rounding of the rescaling factors (~1e-7
//           relative, inside the loss's 1e-5 contract) and reads the row ONCE.
//   pass 2  (gradient only) re-reads the row — with two CTAs per SM about 60 MB of rows are in
//           flight, which the 126 MB L2 holds — and writes (exp(x - M) / Z - onehot) * scale.
// 128-bit accesses after a scalar head that brings the row to 16-byte alignment (rows of 50257
// floats start at every 4-byte phase).
#ifndef CTB_CE_SWEEP1_LOADS
#define CTB_CE_SWEEP1_LOADS 8
#endif
constexpr int kCeLongThreads = 512;       // two CTAs of 64 registers per SM

__device__ __forceinline__ float cta_max_long(float v, float* smem) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, off));
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    __syncthreads();
    if (lane == 0) smem[w] = v;
    __syncthreads();
    float r = lane < kCeLongThreads / 32 ? smem[lane] : -INFINITY;   // one warp folds the warps' values
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) r = fmaxf(r, __shfl_xor_sync(0xffffffffu, r, off));
    return r;
}
__device__ __forceinline__ double cta_sum_long(double v, double* smem) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) v = __dadd_rn(v, __shfl_xor_sync(0xffffffffu, v, off));
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    __syncthreads();
    if (lane == 0) smem[w] = v;
    __syncthreads();
    double r = lane < kCeLongThreads / 32 ? smem[lane] : 0.0;
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) r = __dadd_rn(r, __shfl_xor_sync(0xffffffffu, r, off));
    return r;                                     // xor tree: the same bits in every thread
}

__device__ __forceinline__ int64_t resolve_label(int32_t label, int64_t classes, int32_t* bad) {
    int64_t l = label;
    if (l < 0) l += classes;                       // negative indices count from the end, as Tensor::gather's
    if (l < 0 || l >= classes) {
        if (bad) *bad = 1;
        return -1;
    }
    return l;
}

// running (m, z) of one thread.  GRAD: the exponential lets a NaN argument through
// (exp_nan_through).  Otherwise (the loss, which follows the operator chain max -> sub -> exp ->
// sum): a NaN logit is ignored by the maximum and its term is the clamped exponential of NaN,
// whatever the maximum — such terms are counted apart (`nan_terms`), outside the rescaling.
template <bool GRAD>
struct OnlineSum {
    float m;
    double z;
    int nan_terms;
    __device__ __forceinline__ void raise(float vm) {          // the maximum moves to vm > m
        z = __dmul_rn(z, (double)exp_cephes(__fsub_rn(m, vm)));   // exp(-inf) = 0 on the first element (z is 0 then)
        m = vm;
    }
    __device__ __forceinline__ void push(float v) {
        if (!GRAD && v != v) {
            ++nan_terms;
            return;
        }
        if (v > m) raise(v);
        const float d = __fsub_rn(v, m);
        z = __dadd_rn(z, (double)(GRAD ? exp_nan_through(d) : exp_cephes(d)));
    }
    __device__ __forceinline__ void push4(const Vec<float, 4>& v) {
        if (!GRAD) {
            const float probe = __fadd_rn(__fadd_rn(v.v[0], v.v[1]), __fadd_rn(v.v[2], v.v[3]));
            if (probe != probe) {                               // rare: a NaN among the four (or inf - inf)
#pragma unroll
                for (int q = 0; q < 4; ++q) push(v.v[q]);
                return;
            }
        }
        const float vm = fmaxf(fmaxf(v.v[0], v.v[1]), fmaxf(v.v[2], v.v[3]));
        if (vm > m) raise(vm);
        const float2 d0 = __fadd2_rn(make_float2(v.v[0], v.v[1]), splat2(-m));
        const float2 d1 = __fadd2_rn(make_float2(v.v[2], v.v[3]), splat2(-m));
        const float2 e0 = GRAD ? exp_nan_through2(d0) : exp_cephes2(d0);
        const float2 e1 = GRAD ? exp_nan_through2(d1) : exp_cephes2(d1);
        // the four terms of a vector (each in (0, 1]) meet in fp32 first: one widening per vector
        const float2 s = __fadd2_rn(e0, e1);
        z = __dadd_rn(z, (double)__fadd_rn(s.x, s.y));
    }
    // this thread's share of the row sum under the row maximum M
    __device__ __forceinline__ double under(float M) const {
        double r = __dmul_rn(z, (double)exp_cephes(__fsub_rn(m, M)));
        if (!GRAD && nan_terms) r = __dadd_rn(r, __dmul_rn((double)nan_terms, (double)exp_cephes(__int_as_float(0x7fc00000))));
        return r;
    }
};

// MODE 0: out[row] = nll; 2: out[row, :] += gradient (finite values only), two sweeps;
// 3: out[row, :] = gradient, in three sweeps that use the output row as scratch
template <int MODE>
__global__ void __launch_bounds__(kCeLongThreads, 2)
ce_long_rows_kernel(const float* __restrict__ x, int64_t row_stride, const int32_t* __restrict__ labels, int64_t label_stride,
                    int64_t rows, int64_t classes, float scale, float* __restrict__ out, int64_t out_stride, int32_t* bad) {
    __shared__ float smax[32];
    __shared__ double ssum[32];
    using V4 = Vec<float, 4>;
    constexpr int T = kCeLongThreads;
    const int tid = threadIdx.x;
    for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
        const float* line = x + row * row_stride;
        const int64_t head = min(classes, (int64_t)((4 - ((reinterpret_cast<uintptr_t>(line) >> 2) & 3)) & 3));
        const int64_t nvec = (classes - head) >> 2;
        const int64_t tail = head + 4 * nvec;                   // [tail, classes): at most 3 elements
        const V4* lv = reinterpret_cast<const V4*>(line + head);
        if constexpr (MODE == 3) {
            // Gradient into a fresh buffer, three sweeps with each exponential computed once: maximum;
            // e = exp(x - M) written into the output row and summed; (e / Z - onehot) * scale over the
            // output row.  Sweeps two and three are served by L2.  (The two-sweep form above computes
            // every exponential twice and is bound by instruction issue: 3.5 against 4.3 TB/s at 50257
            // classes.)
            float* orow = out + row * out_stride;
            const bool out_vec = ((reinterpret_cast<uintptr_t>(orow + head) & 15) == 0);
            V4* ov = reinterpret_cast<V4*>(orow + head);
            float mx = -1e9f;                                   // the reference's starting value (loss.cpp:345)
            if (tid < head) mx = fmaxf(mx, line[tid]);
            if (tid < classes - tail) mx = fmaxf(mx, line[tail + tid]);
            auto load_x = [&](int64_t k) { return ldg_stream(lv + k); };
            sweep_vectors<T, false, CTB_CE_SWEEP1_LOADS>(nvec, tid, load_x, [&](const V4& v, int64_t) {
                mx = fmaxf(fmaxf(mx, fmaxf(v.v[0], v.v[1])), fmaxf(v.v[2], v.v[3]));
            });
            const float M = cta_max_long(mx, smax);
            double z = 0.0;
            auto scalar_exp = [&](int64_t c) {
                const float e = exp_nan_through(__fsub_rn(line[c], M));
                orow[c] = e;
                z = __dadd_rn(z, (double)e);
            };
            if (tid < head) scalar_exp(tid);
            if (tid < classes - tail) scalar_exp(tail + tid);
            auto vector_exp = [&](const V4& v, int64_t k) {
                const float2 e0 = exp_nan_through2(__fadd2_rn(make_float2(v.v[0], v.v[1]), splat2(-M)));
                const float2 e1 = exp_nan_through2(__fadd2_rn(make_float2(v.v[2], v.v[3]), splat2(-M)));
                if (out_vec) {
                    V4 e;
                    e.v[0] = e0.x, e.v[1] = e0.y, e.v[2] = e1.x, e.v[3] = e1.y;
                    stg_stream(ov + k, e);
                } else {
                    float* q = orow + head + 4 * k;
                    q[0] = e0.x, q[1] = e0.y, q[2] = e1.x, q[3] = e1.y;
                }
                const float2 s2 = __fadd2_rn(e0, e1);
                z = __dadd_rn(z, (double)__fadd_rn(s2.x, s2.y));
            };
            sweep_vectors<T>(nvec, tid, load_x, vector_exp);
            const float zf = __double2float_rn(cta_sum_long(z, ssum));
            const int64_t l = resolve_label(labels[row * label_stride], classes, tid == 0 ? bad : nullptr);
            const float inv = zf > 1e-12f ? __fdiv_rn(1.0f, zf) : 0.0f;
            auto fin = [&](float e, int64_t c) {
                float p = __fmul_rn(e, inv);
                if (c == l) p = __fsub_rn(p, 1.0f);
                return __fmul_rn(p, scale);
            };
            if (tid < head) orow[tid] = fin(orow[tid], tid);
            if (tid < classes - tail) orow[tail + tid] = fin(orow[tail + tid], tail + tid);
            if (out_vec) {
                sweep_vectors<T>(nvec, tid, [&](int64_t k) { return ldg_stream(ov + k); }, [&](V4 v, int64_t k) {
                    const int64_t c0 = head + 4 * k;
#pragma unroll
                    for (int q = 0; q < 4; ++q) v.v[q] = fin(v.v[q], c0 + q);
                    stg_stream(ov + k, v);
                });
            } else {
                for (int64_t k = tid; k < nvec; k += T) {
                    const int64_t c0 = head + 4 * k;
#pragma unroll
                    for (int q = 0; q < 4; ++q) orow[c0 + q] = fin(orow[c0 + q], c0 + q);
                }
            }
            continue;
        }
        // ---- pass 1 ------------------------------------------------------------------------------------
        OnlineSum<MODE != 0> acc{MODE == 0 ? -INFINITY : -1e9f, 0.0, 0};       // the gradient starts at the reference's -1e9 (loss.cpp:345)
        if (tid < head) acc.push(line[tid]);
        if (tid < classes - tail) acc.push(line[tail + tid]);
        int64_t j = tid;
        for (; j + 3 * T < nvec; j += 4 * T) {                   // four loads in flight
            V4 v[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) v[u] = ldg_stream(lv + j + u * T);
#pragma unroll
            for (int u = 0; u < 4; ++u) acc.push4(v[u]);
        }
        for (; j < nvec; j += T) acc.push4(ldg_stream(lv + j));
        const float M = cta_max_long(acc.m, smax);
        const double Z = cta_sum_long(acc.under(M), ssum);
        const float zf = __double2float_rn(Z);
        const int64_t l = resolve_label(labels[row * label_stride], classes, tid == 0 ? bad : nullptr);
        if constexpr (MODE == 0) {
            if (tid == 0) {
                float nll = 0.0f;
                if (l >= 0) {
                    const float picked = __fsub_rn(__fsub_rn(line[l], M), log_cephes(zf));
                    nll = __double2float_rn(__dmul_rn((double)picked, -1.0));
                }
                out[row] = nll;
            }
        } else {
            // ---- pass 2 --------------------------------------------------------------------------------
            const float inv = zf > 1e-12f ? __fdiv_rn(1.0f, zf) : 0.0f;
            float* orow = out + row * out_stride;
            auto grad = [&](float v, int64_t c, float old) {
                float p = __fmul_rn(exp_nan_through(__fsub_rn(v, M)), inv);
                if (c == l) p = __fsub_rn(p, 1.0f);
                const float g = __fmul_rn(p, scale);
                return MODE == 2 ? BinaryFn<kOpAddFinite, float>::apply(old, g) : g;
            };
            if (tid < head) orow[tid] = grad(line[tid], tid, MODE == 2 ? orow[tid] : 0.0f);
            if (tid < classes - tail) orow[tail + tid] = grad(line[tail + tid], tail + tid, MODE == 2 ? orow[tail + tid] : 0.0f);
            const bool out_vec = ((reinterpret_cast<uintptr_t>(orow + head) & 15) == 0);
            for (int64_t k = tid; k < nvec; k += T) {
                const V4 v = ldg_stream(lv + k);                 // L2
                const int64_t c0 = head + 4 * k;
                V4 r;
                if (out_vec) {
                    V4 old;
                    if (MODE == 2) old = *reinterpret_cast<const V4*>(orow + c0);
                    const float2 e0 = exp_nan_through2(__fadd2_rn(make_float2(v.v[0], v.v[1]), splat2(-M)));
                    const float2 e1 = exp_nan_through2(__fadd2_rn(make_float2(v.v[2], v.v[3]), splat2(-M)));
                    const float e[4] = {e0.x, e0.y, e1.x, e1.y};
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        float p = __fmul_rn(e[q], inv);
                        if (c0 + q == l) p = __fsub_rn(p, 1.0f);
                        const float g = __fmul_rn(p, scale);
                        r.v[q] = MODE == 2 ? BinaryFn<kOpAddFinite, float>::apply(old.v[q], g) : g;
                    }
                    stg_stream(reinterpret_cast<V4*>(orow + c0), r);
                } else {
#pragma unroll
                    for (int q = 0; q < 4; ++q) orow[c0 + q] = grad(v.v[q], c0 + q, MODE == 2 ? orow[c0 + q] : 0.0f);
                }
            }
        }
    }
}

}  // namespace

int launch_backward_chain(int kind, int dtype, const BwdPlan& p, const void* g, const void* x, const void* y, void* out,
                          int accumulate, cudaStream_t st) {
    switch (dtype) {
    case CTB_F32: return launch_typed<float>(kind, p, g, x, y, out, accumulate, st);
    case CTB_F64: return launch_typed<double>(kind, p, g, x, y, out, accumulate, st);
    }
    return set_error(CTB_ERR_DTYPE, "backward chain: only Float32 and Double64 gradients are supported");
}

template <typename T>
static int launch_div_both_t(int64_t n, const T* g, const T* a, const T* b, T* da, T* db, int accumulate, cudaStream_t st) {
    constexpr int VEC = 16 / sizeof(T);
    const bool aligned = is_aligned(g, 16) && is_aligned(a, 16) && is_aligned(b, 16) && is_aligned(da, 16) && is_aligned(db, 16);
    const unsigned grid = (unsigned)ceil_div(n, 256 * (aligned ? VEC : 1));
    if (aligned) {
        if (accumulate) div_both_flat_kernel<T, true, VEC><<<grid, 256, 0, st>>>(g, a, b, da, db, n);
        else div_both_flat_kernel<T, false, VEC><<<grid, 256, 0, st>>>(g, a, b, da, db, n);
    } else {
        if (accumulate) div_both_flat_kernel<T, true, 1><<<grid, 256, 0, st>>>(g, a, b, da, db, n);
        else div_both_flat_kernel<T, false, 1><<<grid, 256, 0, st>>>(g, a, b, da, db, n);
    }
    return cuda_error(cudaGetLastError(), "div backward launch");
}

int launch_div_backward_both(int dtype, int64_t n, const void* g, const void* a, const void* b, void* da, void* db,
                             int accumulate, cudaStream_t st) {
    if (n == 0) return CTB_OK;
    if (dtype == CTB_F32) return launch_div_both_t<float>(n, (const float*)g, (const float*)a, (const float*)b, (float*)da, (float*)db, accumulate, st);
    if (dtype == CTB_F64) return launch_div_both_t<double>(n, (const double*)g, (const double*)a, (const double*)b, (double*)da, (double*)db, accumulate, st);
    return set_error(CTB_ERR_DTYPE, "backward chain: only Float32 and Double64 gradients are supported");
}

int launch_ce_forward_rows(const float* x, int64_t row_stride, const int32_t* labels, int64_t label_stride, int64_t rows,
                           int64_t classes, float* nll, int32_t* bad, cudaStream_t st) {
    if (rows == 0) return CTB_OK;
    if (!launch_ce_rows_registers(0, x, row_stride, labels, label_stride, rows, classes, 0.0f, nll, 0, bad, st)) {
        const unsigned grid = (unsigned)(rows < 0x7FFFFFFFll ? rows : 0x7FFFFFFFll);
        ce_long_rows_kernel<0><<<grid, kCeLongThreads, 0, st>>>(x, row_stride, labels, label_stride, rows, classes, 0.0f, nll, 0, bad);
    }
    return cuda_error(cudaGetLastError(), "cross-entropy rows launch");
}

int launch_ce_backward_rows(const float* x, int64_t row_stride, const int32_t* labels, int64_t label_stride, int64_t rows,
                            int64_t classes, float scale, float* dx, int64_t dx_stride, int accumulate, int32_t* bad,
                            cudaStream_t st) {
    if (rows == 0) return CTB_OK;
    if (!launch_ce_rows_registers(accumulate ? 2 : 1, x, row_stride, labels, label_stride, rows, classes, scale, dx, dx_stride, bad, st)) {
        const unsigned grid = (unsigned)(rows < 0x7FFFFFFFll ? rows : 0x7FFFFFFFll);
        if (accumulate) ce_long_rows_kernel<2><<<grid, kCeLongThreads, 0, st>>>(x, row_stride, labels, label_stride, rows, classes, scale, dx, dx_stride, bad);
        else ce_long_rows_kernel<3><<<grid, kCeLongThreads, 0, st>>>(x, row_stride, labels, label_stride, rows, classes, scale, dx, dx_stride, bad);
    }
    return cuda_error(cudaGetLastError(), "cross-entropy backward launch");
}

}  // namespace ctb
