// Reduction kernels of the operator path: sum / mean / max / min / var / argmax along one dim
// or over the whole tensor.  They replace reduction_op_impl (src/core/opsmp.cpp:593-697 of the
// reference), the SIMD full reductions (src/cpu/AVX2/ops_avx2_f32.cpp:778-966,
// src/cpu/AVX512/ops_avx512_f32.cpp:480-566) and argmax (src/core/ops_dispatch.cpp:427-526).
//
// Kernel shapes (picked on the host from the geometry):
//   rows_warp  : reduce dim contiguous, short lines -> one warp per output, shuffle tree.
//   rows_block : reduce dim contiguous, long lines  -> one CTA per output, shuffle + smem tree.
//   rows_split : few, very long contiguous lines (full-tensor reductions) -> each line is cut
//                into `splits` chunks, one CTA per chunk writes an fp64 partial to scratch;
//                the CTA that takes the last ticket combines the partials IN INDEX ORDER.
//   cols       : an outer dim is contiguous (e.g. dim 0 of a row-major matrix) -> threads are
//                coalesced along that dim and walk the reduce dim; row chunks are split over
//                CTAs and combined by the same ticket scheme.
//   generic    : any other geometry or dtype: a thread, a warp or a CTA chunk per output line,
//                picked from the number and length of the lines.
// Sums accumulate in fp64.  Every combine order is fixed by the launch geometry alone, so
// results are identical from run to run.  No kernel waits on another block: the ticket is an
// atomic counter that is read once, and the block that sees the last value does the combine.
#include "ctb_reduce.cuh"
#include "ctb_math.cuh"
#include <cstring>
#include <mutex>
#include <type_traits>

namespace ctb {

#ifndef CTB_RED_THREADS
#define CTB_RED_THREADS 256
#endif
#ifndef CTB_RED_UNROLL
#define CTB_RED_UNROLL 8
#endif
#ifndef CTB_RED_SPLIT_UNROLL
#define CTB_RED_SPLIT_UNROLL 16            // full-tensor reductions: 16 x 16 B in flight per thread
#endif
#ifndef CTB_RED_SPLIT_CTAS_PER_SM
#define CTB_RED_SPLIT_CTAS_PER_SM 4
#endif
#ifndef CTB_RED_BLOCK_THREADS
#define CTB_RED_BLOCK_THREADS 512          // one CTA per long row: 512 threads measured best on B200
#endif
#ifndef CTB_RED_BLOCK_UNROLL
#define CTB_RED_BLOCK_UNROLL CTB_RED_UNROLL    // loads in flight per thread of the CTA-per-row kernel
#endif
#ifndef CTB_RED_BLOCK_THREADS_MINMAX
#define CTB_RED_BLOCK_THREADS_MINMAX CTB_RED_BLOCK_THREADS
#endif
#ifndef CTB_RED_BLOCK_PERSIST
#define CTB_RED_BLOCK_PERSIST 0                // CTA-per-row kernel: CTAs per SM of a persistent grid (0: one CTA per row)
#endif
#ifndef CTB_RED_COLS_UNROLL
#define CTB_RED_COLS_UNROLL 16             // row loads in flight per thread of the column kernel
#endif
#ifndef CTB_RED_BLOCK_THREADS_SHIFT
#define CTB_RED_BLOCK_THREADS_SHIFT 256    // the same for variance (with per-lane accumulators: 6.04 / 6.60 / 6.77 TB/s at 16384 / 32768 / 65536 columns)
#endif
#ifndef CTB_RED_SHIFT_WARP_ROWS
#define CTB_RED_SHIFT_WARP_ROWS 64         // variance: warp per line from this many lines per SM (32 and 16 measured slower)
#endif
#ifndef CTB_RED_COLS_CTAS_PER_SM
#define CTB_RED_COLS_CTAS_PER_SM 3         // register budget of the column kernel: at least this many CTAs per SM
#endif

constexpr int64_t kRowsWarpSmall = 2048;
constexpr int64_t kRowsWarpMax = 8192;
constexpr int kCounterSlots = kTicketSlots;           // uint32 tickets at the start of scratch
constexpr size_t kCounterBytes = kTicketBytes;

// ---- accumulation policies ------------------------------------------------------------------------
// VT is the element type as the policy sees it (float on the fast paths, double on the generic
// path).  add() receives the element's index along the reduced dim and the line's shift value.
template <typename VT> struct SumPol {
    struct Acc { double s; };
    __device__ __forceinline__ static Acc init() { return {0.0}; }
    __device__ __forceinline__ static void add(Acc& a, VT x, int64_t, double) { a.s = __dadd_rn(a.s, (double)x); }
    __device__ __forceinline__ static Acc combine(const Acc& a, const Acc& b) { return {__dadd_rn(a.s, b.s)}; }
    __device__ __forceinline__ static Acc shfl_down(const Acc& a, int off) { return {__shfl_down_sync(0xffffffffu, a.s, off)}; }
};

// std::max(acc, val) == (acc < val) ? val : acc — a NaN val never replaces acc
// (src/core/opsmp.cpp:679-691).  The reference walks the line in index order, so when the
// extreme value is a zero and zeros of both signs are present it returns the FIRST zero of the
// line (+0 and -0 compare equal, the earlier one stays).  A tree cannot know which zero came
// first from the values alone, so the accumulator also carries z = 2*index + signbit of the
// earliest zero seen (kNoZero when none); the finaliser takes the sign from z when m == 0.
// The hot loops pay one test per batch of loads for it: a thread walks its elements in index
// order, so only the batch in which its running extreme BECOMES zero can hold the zero that
// matters (m == 0 with z still unset); that batch is then re-read out of line (note_zeros_strided).
// KEY: int64_t in general; int32_t where the reduced dim is shorter than 2^30 (the Float32 kernels pick
// it at launch): the accumulator is then 8 bytes, like the arg-reduction's.
template <typename VT, bool IS_MAX, typename KEY = int64_t> struct MinMaxPol {
    struct Acc { VT m; KEY z; };
    static constexpr KEY kNoZero = sizeof(KEY) == 8 ? (KEY)0x7FFFFFFFFFFFFFFFll : (KEY)0x7FFFFFFF;
    // One min/max instruction: it returns the operand that is not NaN (acc never is: it starts at
    // an infinity), like the compare-and-keep above; which zero it returns for +0 against -0 does not
    // matter, value() takes the sign of a zero result from z.
    __device__ __forceinline__ static VT pick(VT acc, VT v) {
        if (sizeof(VT) == 4) return IS_MAX ? (VT)fmaxf((float)acc, (float)v) : (VT)fminf((float)acc, (float)v);
        return IS_MAX ? (VT)fmax((double)acc, (double)v) : (VT)fmin((double)acc, (double)v);
    }
    __device__ __forceinline__ static Acc init() {
        return {IS_MAX ? -(VT)INFINITY : (VT)INFINITY, kNoZero};
    }
    __device__ __forceinline__ static void add(Acc& a, VT x, int64_t, double) { a.m = pick(a.m, x); }
    // the running extreme is a zero and no zero has been noted yet
    __device__ __forceinline__ static bool became_zero(const Acc& a) { return a.m == (VT)0 && a.z == kNoZero; }
    __device__ __forceinline__ static void note_zero(Acc& a, VT x, int64_t idx) {
        if (x == (VT)0) {
            const KEY key = (KEY)(2 * idx + (signbit(x) ? 1 : 0));
            if (key < a.z) a.z = key;
        }
    }
    __device__ __forceinline__ static Acc combine(const Acc& a, const Acc& b) {
        return {pick(a.m, b.m), a.z < b.z ? a.z : b.z};
    }
    __device__ __forceinline__ static Acc shfl_down(const Acc& a, int off) {
        return {__shfl_down_sync(0xffffffffu, a.m, off), __shfl_down_sync(0xffffffffu, a.z, off)};
    }
    // the extreme with the reference's sign rule for zeros applied
    __device__ __forceinline__ static VT value(const Acc& a) {
        if (a.m == (VT)0 && a.z != kNoZero) return (a.z & 1) ? -(VT)0 : (VT)0;
        return a.m;
    }
};

// Biased variance from two shifted moments in fp64: with d = x - shift (shift = first element of
// the line), var = (sum d^2 - (sum d)^2 / n) / n.
template <typename VT> struct VarPol {
    struct Acc { double s1, s2; };
    __device__ __forceinline__ static Acc init() { return {0.0, 0.0}; }
    __device__ __forceinline__ static void add(Acc& a, VT x, int64_t, double shift) {
        // Float32 elements: the difference in the element's own precision (exact when x is within a
        // factor 2 of the shift, else rounded to 2^-24 relative: far inside the 1e-5 contract).  One
        // fp64 operation fewer per element: [8192,16384] over dim 1 5.52 -> 5.72 TB/s, 2^28 elements 6.46 -> 6.66.
        const double d = sizeof(VT) == 4 ? (double)__fsub_rn((float)x, (float)shift) : __dsub_rn((double)x, shift);
        a.s1 = __dadd_rn(a.s1, d);
        a.s2 = fma(d, d, a.s2);
    }
    // Two neighbouring Float32 elements at once: their differences, the sum of the two and the sum of
    // their squares in fp32 (each rounded to 2^-24 relative), then ONE widening and ONE fp64 addition
    // per moment for the pair.  With s2 = sum d^2 the result's error is below 3e-7 * s2 / n, i.e.
    // 3e-7 relative unless the line's first element lies many standard deviations from its mean.
    __device__ __forceinline__ static void add2(Acc& a, float x0, float x1, double shift) {
        const float sf = (float)shift;
        const float d0 = __fsub_rn(x0, sf), d1 = __fsub_rn(x1, sf);
        a.s1 = __dadd_rn(a.s1, (double)__fadd_rn(d0, d1));
        a.s2 = __dadd_rn(a.s2, (double)__fmaf_rn(d1, d1, __fmul_rn(d0, d0)));
    }
    __device__ __forceinline__ static Acc combine(const Acc& a, const Acc& b) {
        return {__dadd_rn(a.s1, b.s1), __dadd_rn(a.s2, b.s2)};
    }
    __device__ __forceinline__ static Acc shfl_down(const Acc& a, int off) {
        return {__shfl_down_sync(0xffffffffu, a.s1, off), __shfl_down_sync(0xffffffffu, a.s2, off)};
    }
};

// First index of the maximum; strict '>' against a running maximum that starts at -1e18
// (src/core/ops_dispatch.cpp:460-472,511-521): NaN and values <= -1e18 never win, an all-
// losing line yields index 0.  For fp32 the start value is the largest float <= -1e18, which
// makes the fp32 compare equivalent to the reference's compare in double.
template <typename VT> struct ArgmaxPol {
    struct Acc { VT v; int32_t i; };
    __device__ __forceinline__ static VT floor_value() {
        if (sizeof(VT) == 4) return (VT)__uint_as_float(0xDD5E0B6Cu);   // -1.00000005e18f
        return (VT)-1e18;
    }
    __device__ __forceinline__ static Acc init() { return {floor_value(), 0}; }
    __device__ __forceinline__ static void add(Acc& a, VT x, int64_t idx, double) {
        if (x > a.v) { a.v = x; a.i = (int32_t)idx; }
    }
    __device__ __forceinline__ static Acc combine(const Acc& a, const Acc& b) {
        if (b.v > a.v || (b.v == a.v && b.i < a.i)) return b;
        return a;
    }
    __device__ __forceinline__ static Acc shfl_down(const Acc& a, int off) {
        return {__shfl_down_sync(0xffffffffu, a.v, off), __shfl_down_sync(0xffffffffu, a.i, off)};
    }
};

// ---- finalisation ------------------------------------------------------------------------------------
// sum: (T)acc.  mean: the sum is rounded to T first, then multiplied by 1.0/n in double and
// rounded again (mean = mul_scalar(sum, 1.0/N), src/core/ops_dispatch.cpp:385-390).
template <typename T, typename Acc>
__device__ __forceinline__ void finalize_store(int op, const Acc& a, int64_t n, void* out, int64_t oi,
                                               double* partial_out);

template <typename T> struct Finalize {
    template <typename VT>
    __device__ __forceinline__ static void run(int op, const typename SumPol<VT>::Acc& a, int64_t n, void* out, int64_t oi, double* po) {
        if (po) { po[oi] = a.s; return; }
        T s = from_double<T>(a.s);
        if (op == kOpSumAccumulate) {
            if (isfinite(to_double(s))) ((T*)out)[oi] = from_double<T>(__dadd_rn(to_double(((T*)out)[oi]), to_double(s)));
            return;
        }
        if (op == CTB_MEAN) s = from_double<T>(__dmul_rn(to_double(s), 1.0 / (double)n));
        ((T*)out)[oi] = s;
    }
    template <typename VT, bool IS_MAX, typename KEY>
    __device__ __forceinline__ static void run_mm(const typename MinMaxPol<VT, IS_MAX, KEY>::Acc& a, void* out, int64_t oi, double* po) {
        const VT m = MinMaxPol<VT, IS_MAX, KEY>::value(a);
        if (po) { po[oi] = (double)m; return; }
        ((T*)out)[oi] = from_double<T>((double)m);
    }
    template <typename VT>
    __device__ __forceinline__ static void run_var(const typename VarPol<VT>::Acc& a, int64_t n, void* out, int64_t oi) {
        double dn = (double)n;
        double v = (a.s2 - a.s1 * a.s1 / dn) / dn;
        if (v < 0.0) v = 0.0;
        ((T*)out)[oi] = from_double<T>(v);
    }
};

template <typename T, typename Pol> struct Fin;
template <typename T, typename VT> struct Fin<T, SumPol<VT>> {
    __device__ __forceinline__ static void run(int op, const typename SumPol<VT>::Acc& a, int64_t n, void* out, int64_t oi, double* po) {
        Finalize<T>::template run<VT>(op, a, n, out, oi, po);
    }
};
template <typename T, typename VT, bool M, typename KEY> struct Fin<T, MinMaxPol<VT, M, KEY>> {
    __device__ __forceinline__ static void run(int, const typename MinMaxPol<VT, M, KEY>::Acc& a, int64_t, void* out, int64_t oi, double* po) {
        Finalize<T>::template run_mm<VT, M, KEY>(a, out, oi, po);
    }
};
template <typename T, typename VT> struct Fin<T, VarPol<VT>> {
    __device__ __forceinline__ static void run(int, const typename VarPol<VT>::Acc& a, int64_t n, void* out, int64_t oi, double*) {
        Finalize<T>::template run_var<VT>(a, n, out, oi);
    }
};
template <typename T, typename VT> struct Fin<T, ArgmaxPol<VT>> {
    __device__ __forceinline__ static void run(int, const typename ArgmaxPol<VT>::Acc& a, int64_t, void* out, int64_t oi, double*) {
        ((int32_t*)out)[oi] = a.i;
    }
};

// Row loads kept in flight per thread by the column kernel: 16 measured best where the
// per-element work is heavier (fp64 sums, variance, arg-reduction), 8 for plain max/min.
template <typename Pol> struct ColsUnroll { static constexpr int value = CTB_RED_COLS_UNROLL; };
#ifndef CTB_RED_COLS_UNROLL_MINMAX
#define CTB_RED_COLS_UNROLL_MINMAX 8
#endif
template <typename VT, bool M, typename KEY> struct ColsUnroll<MinMaxPol<VT, M, KEY>> { static constexpr int value = CTB_RED_COLS_UNROLL_MINMAX; };

template <typename Pol> struct NeedsShift { static constexpr bool value = false; };
template <typename VT> struct NeedsShift<VarPol<VT>> { static constexpr bool value = true; };

// Policies that take two neighbouring fp32 elements in one step (add2).
template <typename Pol> struct TakesPairs { static constexpr bool value = false; };
#ifdef CTB_VAR_PAIRS
template <> struct TakesPairs<VarPol<float>> { static constexpr bool value = true; };
#endif

// Policies whose batches accumulate per vector lane (see accumulate_batch).
template <typename Pol> struct LaneAccs { static constexpr bool value = false; };
// variance: 4 independent fp64 chains per thread ([8192,16384] over dim 1: 5.71 -> 6.04 TB/s with 256-thread CTAs)
template <> struct LaneAccs<VarPol<float>> { static constexpr bool value = true; };
#ifdef CTB_LANE_ACCS_SUM
template <> struct LaneAccs<SumPol<float>> { static constexpr bool value = true; };
#endif

// Policies that must know where the zeros of a line are (max/min, see MinMaxPol).
template <typename Pol> struct TracksZero { static constexpr bool value = false; };
template <typename VT, bool M, typename KEY> struct TracksZero<MinMaxPol<VT, M, KEY>> { static constexpr bool value = true; };

// The rare batch that holds a zero: re-read it (it is in L1) and note the zeros, out of line, so
// that the hot loop keeps its register budget (inlined and unrolled, this path cost the split
// kernel 38 registers and the column kernel spills).
template <typename Pol>
__device__ __noinline__ void note_zeros_strided(typename Pol::Acc* acc, const float* p, int64_t idx0, int64_t idx_step,
                                                int64_t ptr_step, int batches, int vec, int acc_per_lane) {
    for (int u = 0; u < batches; ++u)
        for (int k = 0; k < vec; ++k)
            Pol::note_zero(acc[acc_per_lane ? k : 0], p[u * ptr_step + k], idx0 + u * idx_step + (acc_per_lane ? 0 : k));
}

// One element through a policy on the scalar paths (ragged ends, the generic kernels).
template <typename Pol, typename VT>
__device__ __forceinline__ void add_element(typename Pol::Acc& acc, VT x, int64_t idx, double shift) {
    Pol::add(acc, x, idx, shift);
    if constexpr (TracksZero<Pol>::value) {
        if (Pol::became_zero(acc)) Pol::note_zero(acc, x, idx);
    }
}

// ---- helpers -----------------------------------------------------------------------------------------
struct OuterIdx {
    DimSet dims;
    int64_t stride[1][CTB_MAX_DIMS];
};

__device__ __forceinline__ int64_t outer_offset(const OuterIdx& o, int64_t i) {
    int64_t off[1] = {0};
    dimset_offsets<1>(o.dims, i, o.stride, off);
    return off[0];
}

// L2-coherent load of a scratch accumulator written by another CTA.
template <typename A>
__device__ __forceinline__ A load_cg(const A* p) {
    A r;
    if constexpr (sizeof(A) == 4) {
        unsigned u = __ldcg(reinterpret_cast<const unsigned*>(p));
        memcpy(&r, &u, 4);
    } else if constexpr (sizeof(A) == 8) {
        unsigned long long u = __ldcg(reinterpret_cast<const unsigned long long*>(p));
        memcpy(&r, &u, 8);
    } else {
        static_assert(sizeof(A) == 16, "unexpected accumulator size");
        ulonglong2 u = __ldcg(reinterpret_cast<const ulonglong2*>(p));
        memcpy(&r, &u, 16);
    }
    return r;
}

template <typename Pol>
__device__ __forceinline__ typename Pol::Acc warp_reduce(typename Pol::Acc a) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) a = Pol::combine(a, Pol::shfl_down(a, off));
    return a;   // valid in lane 0
}

// CTA-wide reduce; result valid in thread 0.  smem must hold THREADS/32 accumulators.  The warp
// results are folded by a second shuffle tree in warp 0 (a serial loop in thread 0 kept the whole
// CTA resident for THREADS/32 dependent fp64 additions).
template <typename Pol, int THREADS>
__device__ __forceinline__ typename Pol::Acc block_reduce(typename Pol::Acc a, typename Pol::Acc* smem) {
    constexpr int NW = THREADS / 32;
    static_assert(NW <= 32, "one warp folds the warp results");
    a = warp_reduce<Pol>(a);
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    __syncthreads();                       // smem may still be read from a previous use
    if (lane == 0) smem[w] = a;
    __syncthreads();
    if (w == 0) {
        a = lane < NW ? smem[lane] : Pol::init();
        a = warp_reduce<Pol>(a);
    }
    return a;
}

// Accumulate elements [lo, hi) of one contiguous line; `nthr` cooperating threads, this one
// has rank `tid`.  Vector loads when VEC > 1 (caller guarantees alignment of line + lo).
// U vector loads issued back to back, then consumed.
template <typename Pol, int VEC, int U, bool LANES = false>
__device__ __forceinline__ void accumulate_batch(typename Pol::Acc& acc, const float* __restrict__ line,
                                                 int64_t j, int64_t stride, float shift_f) {
    using V = Vec<float, VEC>;
    V v[U];
#pragma unroll
    for (int u = 0; u < U; ++u) v[u] = ldg_stream(reinterpret_cast<const V*>(line + j + u * stride));
    // The line's shift value comes from a load of its own.  The empty volatile asm pins every use
    // of it (starting with the conversion to double) behind the vector loads above; without it
    // the conversion was scheduled first and each line waited for that one load before issuing
    // the rest ([8192,16384] fp32 variance: over dim 0 6.33 -> 6.59 TB/s, over dim 1 5.40 -> 5.52).
    float sf = shift_f;
    if (NeedsShift<Pol>::value) asm volatile("" : "+f"(sf));
    const double shift = (double)sf;
    if constexpr (TakesPairs<Pol>::value && VEC % 2 == 0) {
#pragma unroll
        for (int u = 0; u < U; ++u)
#pragma unroll
            for (int k = 0; k < VEC; k += 2) Pol::add2(acc, v[u].v[k], v[u].v[k + 1], shift);
    } else if constexpr (LANES && LaneAccs<Pol>::value && VEC > 1 && U > 1) {
        // one accumulator per vector lane inside the batch: VEC independent fp64 dependency chains of
        // length U instead of one of length U * VEC, folded in lane order at the end of the batch
        typename Pol::Acc part[VEC];
#pragma unroll
        for (int k = 0; k < VEC; ++k) part[k] = Pol::init();
#pragma unroll
        for (int u = 0; u < U; ++u)
#pragma unroll
            for (int k = 0; k < VEC; ++k) Pol::add(part[k], v[u].v[k], j + u * stride + k, shift);
#pragma unroll
        for (int k = 0; k < VEC; ++k) acc = Pol::combine(acc, part[k]);
    } else {
#pragma unroll
        for (int u = 0; u < U; ++u)
#pragma unroll
            for (int k = 0; k < VEC; ++k) Pol::add(acc, v[u].v[k], j + u * stride + k, shift);
    }
    if constexpr (TracksZero<Pol>::value) {
        if (Pol::became_zero(acc)) note_zeros_strided<Pol>(&acc, line + j, j, stride, stride, U, VEC, 0);
    }
}

template <typename Pol, int VEC, int UNROLL, bool LANES = false>
__device__ __forceinline__ void accumulate_line(typename Pol::Acc& acc, const float* __restrict__ line,
                                                int64_t lo, int64_t hi, int tid, int nthr, float shift) {
    const int64_t stride = (int64_t)nthr * VEC;
    int64_t j = lo + (int64_t)tid * VEC;
    // main loop: UNROLL loads in flight; the remainder keeps as many in flight as it has
    // (UNROLL/2, UNROLL/4, ... 1) instead of degrading to one load at a time
    for (; j + (UNROLL - 1) * stride + VEC <= hi; j += UNROLL * stride)
        accumulate_batch<Pol, VEC, UNROLL, LANES>(acc, line, j, stride, shift);
    if constexpr (UNROLL >= 16) {
        if (j + 7 * stride + VEC <= hi) { accumulate_batch<Pol, VEC, 8, LANES>(acc, line, j, stride, shift); j += 8 * stride; }
    }
    if constexpr (UNROLL >= 8) {
        if (j + 3 * stride + VEC <= hi) { accumulate_batch<Pol, VEC, 4, LANES>(acc, line, j, stride, shift); j += 4 * stride; }
    }
    if constexpr (UNROLL >= 4) {
        if (j + 1 * stride + VEC <= hi) { accumulate_batch<Pol, VEC, 2, LANES>(acc, line, j, stride, shift); j += 2 * stride; }
    }
    for (; j + VEC <= hi; j += stride) accumulate_batch<Pol, VEC, 1>(acc, line, j, stride, shift);
    if (VEC > 1) {   // ragged end of the line
        for (int k = 0; k < VEC; ++k)
            if (j + k < hi) add_element<Pol>(acc, line[j + k], j + k, (double)shift);
    }
}

// ---- rows_warp ------------------------------------------------------------------------------------------
template <typename Pol, int VEC, int THREADS>
__global__ void __launch_bounds__(THREADS)
reduce_rows_warp_kernel(const float* __restrict__ a, void* out, OuterIdx o, int64_t nout, int64_t rlen, int op) {
    const int lane = threadIdx.x & 31;
    const int64_t warps = (int64_t)gridDim.x * (THREADS / 32);
    for (int64_t row = (int64_t)blockIdx.x * (THREADS / 32) + (threadIdx.x >> 5); row < nout; row += warps) {
        const float* line = a + outer_offset(o, row);
        const float shift = NeedsShift<Pol>::value ? line[0] : 0.0f;
        typename Pol::Acc acc = Pol::init();
        accumulate_line<Pol, VEC, CTB_RED_UNROLL>(acc, line, 0, rlen, lane, 32, shift);
        acc = warp_reduce<Pol>(acc);
        if (lane == 0) Fin<float, Pol>::run(op, acc, rlen, out, row, nullptr);
    }
}

// ---- rows_block -----------------------------------------------------------------------------------------
// Loads in flight per thread and resident CTAs per SM the CTA-per-row kernel is compiled for.
// Variance: 4 loads in flight and a register budget that lets 5 CTAs of 256 threads share an SM
// measured best ([8192,16384] over dim 1, same run: 5.19 TB/s with 8 loads and no budget, 6.04 with
// 4 loads and no budget, 6.40 with 4 loads and 5 CTAs, 5.76 with 6 CTAs; rows of 32768 / 65536
// elements 6.08 -> 6.78 / 6.36 -> 6.78): the heavier per-element work wants more rows in flight
// per SM rather than more loads per thread.
#ifndef CTB_RED_VAR_UNROLL
#define CTB_RED_VAR_UNROLL 4
#endif
#ifndef CTB_RED_VAR_MINB
#define CTB_RED_VAR_MINB 5
#endif
#ifndef CTB_RED_BLOCK_MINB
#define CTB_RED_BLOCK_MINB 0                  // 0: no occupancy request, the compiler's own register choice
#endif
template <typename Pol> struct BlockShape { static constexpr int unroll = CTB_RED_BLOCK_UNROLL, min_ctas = CTB_RED_BLOCK_MINB; };
template <typename VT> struct BlockShape<VarPol<VT>> { static constexpr int unroll = CTB_RED_VAR_UNROLL, min_ctas = CTB_RED_VAR_MINB; };
// max/min: one CTA per SM requested, i.e. no register ceiling below the hardware's — the compiler then
// keeps all 8 loads of a batch in flight in 56 registers instead of 40 (same run, TB/s: [8192,16384]
// 6.47 -> 6.82, rows of 32768 / 65536 elements 6.83 -> 7.14 / 6.57 -> 6.94).
#ifndef CTB_RED_MINMAX_MINB
#define CTB_RED_MINMAX_MINB 1
#endif
template <typename VT, bool M, typename KEY> struct BlockShape<MinMaxPol<VT, M, KEY>> { static constexpr int unroll = CTB_RED_BLOCK_UNROLL, min_ctas = CTB_RED_MINMAX_MINB; };

template <typename Pol, int VEC, int THREADS>
__global__ void __launch_bounds__(THREADS, BlockShape<Pol>::min_ctas)
reduce_rows_block_kernel(const float* __restrict__ a, void* out, OuterIdx o, int64_t nout, int64_t rlen, int op) {
    __shared__ typename Pol::Acc smem[THREADS / 32];
    for (int64_t row = blockIdx.x; row < nout; row += gridDim.x) {
        const float* line = a + outer_offset(o, row);
        const float shift = NeedsShift<Pol>::value ? line[0] : 0.0f;
        typename Pol::Acc acc = Pol::init();
        accumulate_line<Pol, VEC, BlockShape<Pol>::unroll, true>(acc, line, 0, rlen, threadIdx.x, THREADS, shift);
        acc = block_reduce<Pol, THREADS>(acc, smem);
        if (threadIdx.x == 0) Fin<float, Pol>::run(op, acc, rlen, out, row, nullptr);
    }
}

// Loads in flight per thread of the full-tensor kernel, and whether a batch accumulates per vector
// lane.  Variance of 2^28 elements: 6.59 TB/s with 16 loads and one accumulator chain, 6.75 with 8
// loads and per-lane accumulators, 6.78 with 4 (5.59 with 16: registers).
#ifndef CTB_RED_SPLIT_VAR_UNROLL
#define CTB_RED_SPLIT_VAR_UNROLL 4
#endif
#ifndef CTB_RED_SPLIT_VAR_LANES
#define CTB_RED_SPLIT_VAR_LANES 1
#endif
#ifndef CTB_RED_SPLIT_MINMAX_MINB
#define CTB_RED_SPLIT_MINMAX_MINB 0
#endif
#ifndef CTB_RED_SPLIT_MINMAX_UNROLL
#define CTB_RED_SPLIT_MINMAX_UNROLL CTB_RED_SPLIT_UNROLL
#endif
template <typename Pol> struct SplitShape { static constexpr int unroll = CTB_RED_SPLIT_UNROLL, min_ctas = 0; static constexpr bool lanes = false; };
template <typename VT, bool M, typename KEY> struct SplitShape<MinMaxPol<VT, M, KEY>> { static constexpr int unroll = CTB_RED_SPLIT_MINMAX_UNROLL, min_ctas = CTB_RED_SPLIT_MINMAX_MINB; static constexpr bool lanes = false; };
template <typename VT> struct SplitShape<VarPol<VT>> { static constexpr int unroll = CTB_RED_SPLIT_VAR_UNROLL, min_ctas = 0; static constexpr bool lanes = CTB_RED_SPLIT_VAR_LANES != 0; };

// ---- rows_split -----------------------------------------------------------------------------------------
// grid = (splits, nout).  Scratch: tickets[nout] (uint32, zero before and after), then
// partials[nout][splits].
template <typename Pol, int VEC, int THREADS>
__global__ void __launch_bounds__(THREADS, SplitShape<Pol>::min_ctas)
reduce_rows_split_kernel(const float* __restrict__ a, void* out, double* partial_out, OuterIdx o,
                         int64_t rlen, int64_t chunk, int op, uint32_t* tickets,
                         typename Pol::Acc* partials) {
    __shared__ typename Pol::Acc smem[THREADS / 32];
    __shared__ bool is_last;
    const int64_t row = blockIdx.y;
    const int splits = gridDim.x;
    const float* line = a + outer_offset(o, row);
    const float shift = NeedsShift<Pol>::value ? line[0] : 0.0f;
    const int64_t lo = (int64_t)blockIdx.x * chunk;
    int64_t hi = lo + chunk;
    if (hi > rlen) hi = rlen;
    typename Pol::Acc acc = Pol::init();
    if (lo < hi) accumulate_line<Pol, VEC, SplitShape<Pol>::unroll, SplitShape<Pol>::lanes>(acc, line, lo, hi, threadIdx.x, THREADS, shift);
    acc = block_reduce<Pol, THREADS>(acc, smem);
    if (threadIdx.x == 0) {
        partials[row * splits + blockIdx.x] = acc;
        __threadfence();
        const uint32_t t = atomicAdd(&tickets[row], 1u);
        is_last = (t == (uint32_t)splits - 1);
    }
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    // fixed-order combine: thread t folds partials t, t+THREADS, ... then the CTA tree
    typename Pol::Acc c = Pol::init();
    const typename Pol::Acc* p = partials + row * splits;
    for (int i = threadIdx.x; i < splits; i += THREADS) c = Pol::combine(c, load_cg(p + i));
    c = block_reduce<Pol, THREADS>(c, smem);
    if (threadIdx.x == 0) {
        Fin<float, Pol>::run(op, c, rlen, out, row, partial_out);
        tickets[row] = 0;
    }
}

// ---- cols -----------------------------------------------------------------------------------------------
// Outer dims = [batch..., C] with the last one contiguous.  CTA = 32 x 8 threads: x walks
// columns (VEC each), y walks rows.  grid = (column tiles, row splits, batch).
template <typename Pol, int VEC, int U>
__device__ __forceinline__ void cols_batch(typename Pol::Acc (&acc)[VEC], const float* __restrict__ q,
                                           int64_t step, int64_t r, const float (&shift_f)[VEC]) {
    using V = Vec<float, VEC>;
    V v[U];
#pragma unroll
    for (int u = 0; u < U; ++u) v[u] = ldg_stream(reinterpret_cast<const V*>(q + u * step));
    double shift[VEC];                   // uses pinned behind the loads, as in accumulate_batch
#pragma unroll
    for (int k = 0; k < VEC; ++k) {
        float sf = shift_f[k];
        if (NeedsShift<Pol>::value) asm volatile("" : "+f"(sf));
        shift[k] = (double)sf;
    }
#pragma unroll
    for (int u = 0; u < U; ++u)
#pragma unroll
        for (int k = 0; k < VEC; ++k) Pol::add(acc[k], v[u].v[k], r + 8 * u, shift[k]);
    if constexpr (TracksZero<Pol>::value) {
        bool became = false;
#pragma unroll
        for (int k = 0; k < VEC; ++k) became |= Pol::became_zero(acc[k]);
        if (became) note_zeros_strided<Pol>(acc, q, r, 8, step, U, VEC, 1);
    }
}

#ifndef CTB_RED_COLS_MINMAX_CTAS
#define CTB_RED_COLS_MINMAX_CTAS CTB_RED_COLS_CTAS_PER_SM
#endif
template <typename Pol> struct ColsCtas { static constexpr int value = CTB_RED_COLS_CTAS_PER_SM; };
template <typename VT, bool M, typename KEY> struct ColsCtas<MinMaxPol<VT, M, KEY>> { static constexpr int value = CTB_RED_COLS_MINMAX_CTAS; };

template <typename Pol, int VEC>
__global__ void __launch_bounds__(256, ColsCtas<Pol>::value)
reduce_cols_kernel(const float* __restrict__ a, void* out, OuterIdx batch, int64_t ncols, int64_t rlen,
                   int64_t rstride, int64_t rows_per_split, int op, uint32_t* tickets,
                   typename Pol::Acc* partials) {
    using V = Vec<float, VEC>;
    using Acc = typename Pol::Acc;
    __shared__ Acc smem[8][32 * VEC + 1];
    __shared__ bool is_last;
    const int x = threadIdx.x & 31, y = threadIdx.x >> 5;
    const int64_t col = ((int64_t)blockIdx.x * 32 + x) * VEC;
    const int64_t b = blockIdx.z;
    const float* base = a + outer_offset(batch, b);
    const int splits = gridDim.y;
    const int64_t r0 = (int64_t)blockIdx.y * rows_per_split;
    int64_t r1 = r0 + rows_per_split;
    if (r1 > rlen) r1 = rlen;

    Acc acc[VEC];
    float shift[VEC];
#pragma unroll
    for (int k = 0; k < VEC; ++k) { acc[k] = Pol::init(); shift[k] = 0.0f; }
    const bool active = col < ncols;     // ncols % VEC == 0 when VEC > 1
    if (active) {
        if (NeedsShift<Pol>::value) {
#pragma unroll
            for (int k = 0; k < VEC; ++k) shift[k] = base[col + k];
        }
        // CU row loads in flight; the remainder keeps as many in flight as it has (CU/2, ... 1)
        constexpr int CU = ColsUnroll<Pol>::value;
        const int64_t step = 8 * rstride;
        int64_t r = r0 + y;
        const float* q = base + col + r * rstride;
        for (; r + 8 * (CU - 1) < r1; r += 8 * CU, q += CU * step) cols_batch<Pol, VEC, CU>(acc, q, step, r, shift);
        if constexpr (CU >= 16) {
            if (r + 8 * 7 < r1) { cols_batch<Pol, VEC, 8>(acc, q, step, r, shift); r += 64; q += 8 * step; }
        }
        if constexpr (CU >= 8) {
            if (r + 8 * 3 < r1) { cols_batch<Pol, VEC, 4>(acc, q, step, r, shift); r += 32; q += 4 * step; }
        }
        if (r + 8 < r1) { cols_batch<Pol, VEC, 2>(acc, q, step, r, shift); r += 16; q += 2 * step; }
        if (r < r1) cols_batch<Pol, VEC, 1>(acc, q, step, r, shift);
    }
#pragma unroll
    for (int k = 0; k < VEC; ++k) smem[y][x * VEC + k] = acc[k];
    __syncthreads();
    // 32*VEC columns, one thread each (threads 0..32*VEC-1), rows y = 0..7 in order
    const int ct = threadIdx.x;
    const int64_t ccol = (int64_t)blockIdx.x * 32 * VEC + ct;
    const bool cact = ct < 32 * VEC && ccol < ncols;
    Acc c = Pol::init();
    if (cact) {
        c = smem[0][ct];
#pragma unroll
        for (int yy = 1; yy < 8; ++yy) c = Pol::combine(c, smem[yy][ct]);
    }
    if (splits == 1) {
        if (cact) Fin<float, Pol>::run(op, c, rlen, out, b * ncols + ccol, nullptr);
        return;
    }
    Acc* part = partials + (b * splits) * ncols;
    if (cact) part[(int64_t)blockIdx.y * ncols + ccol] = c;
    __syncthreads();                          // the CTA's partials are ordered before thread 0's fence
    if (threadIdx.x == 0) {
        __threadfence();                      // cumulative: publishes them device-wide before the ticket
        const uint32_t slot = (uint32_t)(b * gridDim.x + blockIdx.x);
        const uint32_t t = atomicAdd(&tickets[slot], 1u);
        is_last = (t == (uint32_t)splits - 1);
        if (is_last) tickets[slot] = 0;
    }
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    if (cact) {
        Acc f = load_cg(part + ccol);
        for (int s = 1; s < splits; ++s) f = Pol::combine(f, load_cg(part + (int64_t)s * ncols + ccol));
        Fin<float, Pol>::run(op, f, rlen, out, b * ncols + ccol, nullptr);
    }
}

// ---- generic --------------------------------------------------------------------------------------------
template <typename Pol, typename T>
__global__ void __launch_bounds__(256)
reduce_generic_kernel(const T* __restrict__ a, void* out, OuterIdx o, int64_t nout, int64_t rlen,
                      int64_t rstride, int op) {
    const int64_t step = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < nout; i += step) {
        const T* line = a + outer_offset(o, i);
        const double shift = NeedsShift<Pol>::value && rlen > 0 ? to_double(line[0]) : 0.0;
        typename Pol::Acc acc = Pol::init();
        for (int64_t k = 0; k < rlen; ++k) add_element<Pol>(acc, to_double(line[k * rstride]), k, shift);
        Fin<T, Pol>::run(op, acc, rlen, out, i, nullptr);
    }
}

// Generic lines, a warp per line: lanes stride over the line (coalesced when rstride == 1).
template <typename Pol, typename T>
__global__ void __launch_bounds__(256)
reduce_generic_warp_kernel(const T* __restrict__ a, void* out, OuterIdx o, int64_t nout, int64_t rlen,
                           int64_t rstride, int op) {
    const int lane = threadIdx.x & 31;
    const int64_t warps = (int64_t)gridDim.x * 8;
    for (int64_t i = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5); i < nout; i += warps) {
        const T* line = a + outer_offset(o, i);
        const double shift = NeedsShift<Pol>::value ? to_double(line[0]) : 0.0;
        typename Pol::Acc acc = Pol::init();
        for (int64_t k = lane; k < rlen; k += 32) add_element<Pol>(acc, to_double(line[k * rstride]), k, shift);
        acc = warp_reduce<Pol>(acc);
        if (lane == 0) Fin<T, Pol>::run(op, acc, rlen, out, i, nullptr);
    }
}

// Generic lines, few and long: grid = (splits, lines); a CTA folds elements [lo, hi) of its line,
// four loads in flight per thread; with more than one split the partials are combined in index
// order by the CTA that draws the line's last ticket (as in reduce_rows_split_kernel).
template <typename Pol, typename T, int THREADS>
__global__ void __launch_bounds__(THREADS)
reduce_generic_split_kernel(const T* __restrict__ a, void* out, OuterIdx o, int64_t nout, int64_t rlen,
                            int64_t rstride, int64_t chunk, int op, uint32_t* tickets,
                            typename Pol::Acc* partials) {
    __shared__ typename Pol::Acc smem[THREADS / 32];
    __shared__ bool is_last;
    const int splits = gridDim.x;
    for (int64_t row = blockIdx.y; row < nout; row += gridDim.y) {
        const T* line = a + outer_offset(o, row);
        const double shift = NeedsShift<Pol>::value ? to_double(line[0]) : 0.0;
        const int64_t lo = (int64_t)blockIdx.x * chunk;
        int64_t hi = lo + chunk;
        if (hi > rlen) hi = rlen;
        typename Pol::Acc acc = Pol::init();
        int64_t k = lo + threadIdx.x;
        for (; k + 3 * THREADS < hi; k += 4 * THREADS) {
            T v[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) v[u] = line[(k + u * THREADS) * rstride];
#pragma unroll
            for (int u = 0; u < 4; ++u) add_element<Pol>(acc, to_double(v[u]), k + u * THREADS, shift);
        }
        for (; k < hi; k += THREADS) add_element<Pol>(acc, to_double(line[k * rstride]), k, shift);
        acc = block_reduce<Pol, THREADS>(acc, smem);
        if (splits == 1) {
            if (threadIdx.x == 0) Fin<T, Pol>::run(op, acc, rlen, out, row, nullptr);
            continue;
        }
        if (threadIdx.x == 0) {
            partials[row * splits + blockIdx.x] = acc;
            __threadfence();
            const uint32_t t = atomicAdd(&tickets[row], 1u);
            is_last = (t == (uint32_t)splits - 1);
        }
        __syncthreads();
        if (is_last) {          // uniform across the CTA
            __threadfence();
            typename Pol::Acc c = Pol::init();
            const typename Pol::Acc* p = partials + row * splits;
            for (int i = threadIdx.x; i < splits; i += THREADS) c = Pol::combine(c, load_cg(p + i));
            c = block_reduce<Pol, THREADS>(c, smem);
            if (threadIdx.x == 0) {
                Fin<T, Pol>::run(op, c, rlen, out, row, nullptr);
                tickets[row] = 0;
            }
        }
        __syncthreads();        // is_last and smem are reused by the next line
    }
}

// ---- multi-GPU finalisation ---------------------------------------------------------------------------
template <typename T>
__global__ void finalize_full_kernel(int op, const double* partial, int64_t total, T* out) {
    if (threadIdx.x != 0 || blockIdx.x != 0) return;
    T s = from_double<T>(partial[0]);
    if (op == CTB_MEAN) s = from_double<T>(__dmul_rn(to_double(s), 1.0 / (double)total));
    out[0] = s;
}

// ---- host side --------------------------------------------------------------------------------------------
namespace {

enum Shape { SH_ROWS_WARP, SH_ROWS_BLOCK, SH_ROWS_SPLIT, SH_COLS, SH_GENERIC, SH_GENERIC_WARP, SH_GENERIC_SPLIT };

struct Choice {
    Shape shape;
    int vec;             // 4 or 1
    int splits;          // rows_split / cols
    int64_t chunk;       // rows_split: elements per split; cols: rows per split
    int64_t coltiles;    // cols
    int64_t batch;       // cols
    int splits_bound;    // cols: most splits any operator's kernel may use (sizes the scratch)
    size_t acc_bytes_max = 16;
};

bool all_multiple(const int64_t* v, int n, int64_t m) {
    for (int i = 0; i < n; ++i) if (v[i] % m) return false;
    return true;
}

// Row splits of the column kernel for a grid of `tiles` CTAs per split when `slots` CTAs can be
// resident at once.  Up to one wave: as many splits as fit in it (a second, partly filled wave
// measured 25 % slower than a single one that is 86 % full).  More tiles than slots: enough
// splits for about four waves of small CTAs, so that the last wave's tail stays short.
int cols_splits(int64_t tiles, int64_t slots, int64_t rlen) {
    int64_t want = tiles <= slots ? slots / tiles : ceil_div(4 * slots, tiles);
    const int64_t max_splits = rlen / 64;
    if (want > max_splits) want = max_splits;
    if (want > 64) want = 64;
    if (want > 1 && tiles > kCounterSlots) want = 1;
    return want < 1 ? 1 : (int)want;
}

// Upper bound over every occupancy a column kernel can have (1..8 CTAs of 256 threads per SM):
// the workspace size must not depend on the operator.
int cols_splits_bound(int64_t tiles, int sm_count, int64_t rlen) {
    int s = 1;
    for (int occ = 1; occ <= 8; ++occ) {
        const int v = cols_splits(tiles, (int64_t)sm_count * occ, rlen);
        if (v > s) s = v;
    }
    return s;
}

// Any dtype and geometry the Float32 fast paths do not take.  A thread per line when the lines
// are short or plentiful enough to fill the machine that way; a CTA per line chunk when there are
// few long lines (a full reduction of a Float64 or Int32 tensor is ONE line: a thread per line
// would fold the whole tensor serially); a warp per line in between.
constexpr int kGenericThreads = 256;
void choose_generic(const ReduceGeom& g, int sm_count, Choice* c) {
    c->shape = SH_GENERIC;
    c->vec = 1;
    c->splits = 1;
    c->chunk = g.rlen;
    if (g.nout == 0 || g.rlen < 64) return;
    const int64_t resident_threads = (int64_t)sm_count * 2048;
    if (g.nout >= resident_threads) return;
    if (g.nout * 32 >= resident_threads || g.rlen < 4096) { c->shape = SH_GENERIC_WARP; return; }
    c->shape = SH_GENERIC_SPLIT;
    int64_t want = ceil_div((int64_t)sm_count * 8, g.nout);          // about 8 CTAs per SM in all
    const int64_t max_splits = g.rlen / (4 * kGenericThreads);       // at least one unrolled pass each
    if (want > max_splits) want = max_splits;
    if (want > 4096) want = 4096;
    if (want < 1 || g.nout > kCounterSlots) want = 1;
    c->chunk = ceil_div(g.rlen, want);
    c->splits = (int)ceil_div(g.rlen, c->chunk);
}

Choice choose(const ReduceGeom& g, int dtype, const void* a, int sm_count) {
    Choice c{};
    choose_generic(g, sm_count, &c);
    if (dtype != CTB_F32 || g.nout == 0 || g.rlen == 0) return c;
    const bool base16 = a == nullptr || is_aligned(a, 16);
    if (g.rstride == 1 || g.rlen == 1) {
        c.vec = (base16 && all_multiple(g.ostride, g.nouter, 4) && g.rlen % 4 == 0) ? 4 : 1;
        if (g.nout <= 2 * (int64_t)sm_count && g.rlen >= 65536 && g.nout <= 65535 && g.nout <= kCounterSlots) {
            c.shape = SH_ROWS_SPLIT;
            int64_t want = (int64_t)sm_count * CTB_RED_SPLIT_CTAS_PER_SM / g.nout;
            if (want < 1) want = 1;
            const int64_t gran = (int64_t)CTB_RED_THREADS * 4 * CTB_RED_SPLIT_UNROLL;   // whole unrolled passes, vector-aligned
            int64_t chunk = ceil_div(ceil_div(g.rlen, want), gran) * gran;
            c.chunk = chunk;
            c.splits = (int)ceil_div(g.rlen, chunk);
            return c;
        }
        // A warp per line (no CTA barrier per line) when the lines are short, or when there are
        // enough of them to fill the machine with warps and a 512-thread CTA would fit badly:
        // lines up to 8192 elements (a CTA per 4096-element line measured 3.7 TB/s against the
        // warp's 6.6) and longer lines that are not a whole number of CTA-wide batches
        // ([40000,10000]: 7.1 against 5.1 TB/s).  A CTA per line otherwise.
        const int64_t cta_batch = (int64_t)CTB_RED_BLOCK_THREADS * 4 * CTB_RED_BLOCK_UNROLL;
        const bool many_lines = g.nout >= (int64_t)sm_count * 32;
        const bool warp = g.rlen <= kRowsWarpSmall ||
                          (many_lines && (g.rlen <= kRowsWarpMax || g.rlen % cta_batch != 0));
        c.shape = warp ? SH_ROWS_WARP : SH_ROWS_BLOCK;
        return c;
    }
    // column case: innermost outer dim contiguous
    if (g.nouter >= 1 && g.ostride[g.nouter - 1] == 1) {
        const int64_t ncols = g.oshape[g.nouter - 1];
        int64_t batch = 1;
        for (int d = 0; d < g.nouter - 1; ++d) batch *= g.oshape[d];
        if (batch <= 65535 && ncols >= 32) {
            c.vec = (base16 && ncols % 4 == 0 && g.rstride % 4 == 0 && all_multiple(g.ostride, g.nouter - 1, 4)) ? 4 : 1;
            c.coltiles = ceil_div(ncols, 32 * c.vec);
            c.batch = batch;
            // splits and rows per split depend on the kernel's occupancy: set at launch (cols_splits)
            c.splits = 0;
            c.chunk = 0;
            c.splits_bound = cols_splits_bound(c.coltiles * batch, sm_count, g.rlen);
            c.shape = SH_COLS;
            return c;
        }
    }
    return c;
}

size_t scratch_bytes(const ReduceGeom& g, const Choice& c) {
    if (c.shape == SH_ROWS_SPLIT) return kCounterBytes + (size_t)g.nout * c.splits * 16;
    if (c.shape == SH_COLS && c.splits_bound > 1) return kCounterBytes + (size_t)c.batch * c.splits_bound * g.oshape[g.nouter - 1] * 16;
    if (c.shape == SH_GENERIC_SPLIT && c.splits > 1) return kCounterBytes + (size_t)g.nout * c.splits * 16;
    return 0;
}

OuterIdx outer_of(const ReduceGeom& g, int n) {
    OuterIdx o{};
    dimset_init(&o.dims, n, g.oshape);
    for (int d = 0; d < n; ++d) o.stride[0][d] = g.ostride[d];
    return o;
}

// Resident CTAs per SM of a kernel (1..8); 4 if the runtime cannot say.
int kernel_occupancy(const void* kernel, int threads) {
    int n = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, kernel, threads, 0) != cudaSuccess) { cudaGetLastError(); n = 0; }
    if (n < 1) n = 4;
    return n > 8 ? 8 : n;
}

template <typename Pol>
int launch_fast(const Choice& c, const ReduceGeom& g, const float* a, void* out, double* partial_out,
                void* ws, int op, int sm_count, cudaStream_t st) {
    constexpr int T = CTB_RED_THREADS;
    uint32_t* tickets = (uint32_t*)ws;
    typename Pol::Acc* partials = (typename Pol::Acc*)((char*)ws + kCounterBytes);
    static_assert(sizeof(typename Pol::Acc) <= 16, "accumulator larger than the scratch slot");
    Shape shape = c.shape;
    // variance does three fp64 operations per element after the loads of a CTA-wide batch have
    // landed; with a CTA per line that phase is not covered by loads, with a warp per line other
    // warps' loads cover it ([16384,16384]: 6.1 against 5.4 TB/s) — if there are lines enough
    if (shape == SH_ROWS_BLOCK && NeedsShift<Pol>::value && g.nout >= (int64_t)sm_count * CTB_RED_SHIFT_WARP_ROWS) shape = SH_ROWS_WARP;
    switch (shape) {
    case SH_ROWS_WARP: {
        // one warp per row, one pass per CTA (a persistent grid measured slower)
        int64_t blocks = ceil_div(g.nout, T / 32);
        if (blocks > 0x7FFFFFFFll) blocks = 0x7FFFFFFFll;
        const unsigned grid = (unsigned)blocks;
        if (c.vec == 4) reduce_rows_warp_kernel<Pol, 4, T><<<grid, T, 0, st>>>(a, out, outer_of(g, g.nouter), g.nout, g.rlen, op);
        else reduce_rows_warp_kernel<Pol, 1, T><<<grid, T, 0, st>>>(a, out, outer_of(g, g.nouter), g.nout, g.rlen, op);
        break;
    }
    case SH_ROWS_BLOCK: {
        int64_t blocks = g.nout < 0x7FFFFFFFll ? g.nout : 0x7FFFFFFFll;
        if (CTB_RED_BLOCK_PERSIST > 0 && blocks > (int64_t)sm_count * CTB_RED_BLOCK_PERSIST) blocks = (int64_t)sm_count * CTB_RED_BLOCK_PERSIST;
        const unsigned grid = (unsigned)blocks;
        auto launch = [&](auto tb) {
            constexpr int TB = decltype(tb)::value;
            if (c.vec == 4) reduce_rows_block_kernel<Pol, 4, TB><<<grid, TB, 0, st>>>(a, out, outer_of(g, g.nouter), g.nout, g.rlen, op);
            else reduce_rows_block_kernel<Pol, 1, TB><<<grid, TB, 0, st>>>(a, out, outer_of(g, g.nouter), g.nout, g.rlen, op);
        };
        if constexpr (NeedsShift<Pol>::value) {
            launch(std::integral_constant<int, CTB_RED_BLOCK_THREADS_SHIFT>());
        } else if constexpr (TracksZero<Pol>::value) {
            // max / min: lines of up to two 256-thread batches run best with 256 threads ([8192,16384]:
            // 6.62 against 6.27 TB/s), longer ones with 512 ([8192,32768]: 6.95 against 6.61)
            if (g.rlen <= (int64_t)2 * 256 * 4 * CTB_RED_BLOCK_UNROLL) launch(std::integral_constant<int, 256>());
            else launch(std::integral_constant<int, CTB_RED_BLOCK_THREADS_MINMAX>());
        } else {
            launch(std::integral_constant<int, CTB_RED_BLOCK_THREADS>());
        }
        break;
    }
    case SH_ROWS_SPLIT: {
        dim3 grid(c.splits, (unsigned)g.nout);
        if (c.vec == 4) reduce_rows_split_kernel<Pol, 4, T><<<grid, T, 0, st>>>(a, out, partial_out, outer_of(g, g.nouter), g.rlen, c.chunk, op, tickets, partials);
        else reduce_rows_split_kernel<Pol, 1, T><<<grid, T, 0, st>>>(a, out, partial_out, outer_of(g, g.nouter), g.rlen, c.chunk, op, tickets, partials);
        break;
    }
    case SH_COLS: {
        // resident CTAs per SM of this instantiation, asked once per process
        static const int occ4 = kernel_occupancy((const void*)reduce_cols_kernel<Pol, 4>, 256);
        static const int occ1 = kernel_occupancy((const void*)reduce_cols_kernel<Pol, 1>, 256);
        const int occ = c.vec == 4 ? occ4 : occ1;
        const int splits = cols_splits(c.coltiles * c.batch, (int64_t)sm_count * occ, g.rlen);
        const int64_t chunk = ceil_div(ceil_div(g.rlen, (int64_t)splits), 8) * 8;
        dim3 grid((unsigned)c.coltiles, (unsigned)ceil_div(g.rlen, chunk), (unsigned)c.batch);
        const int64_t ncols = g.oshape[g.nouter - 1];
        if (c.vec == 4) reduce_cols_kernel<Pol, 4><<<grid, 256, 0, st>>>(a, out, outer_of(g, g.nouter - 1), ncols, g.rlen, g.rstride, chunk, op, tickets, partials);
        else reduce_cols_kernel<Pol, 1><<<grid, 256, 0, st>>>(a, out, outer_of(g, g.nouter - 1), ncols, g.rlen, g.rstride, chunk, op, tickets, partials);
        break;
    }
    default: return set_error(CTB_ERR_ARG, "reduce: internal shape error");
    }
    return cuda_error(cudaGetLastError(), "reduce launch");
}

template <typename Pol, typename T>
int launch_generic_pol(const Choice& c, int op, const ReduceGeom& g, const T* a, void* out, void* ws, int sm_count,
                       cudaStream_t st) {
    static_assert(sizeof(typename Pol::Acc) <= 16, "accumulator larger than the scratch slot");
    OuterIdx o = outer_of(g, g.nouter);
    const int64_t cap = (int64_t)sm_count * 8;
    if (c.shape == SH_GENERIC_SPLIT) {
        uint32_t* tickets = (uint32_t*)ws;
        typename Pol::Acc* partials = (typename Pol::Acc*)((char*)ws + kCounterBytes);
        dim3 grid((unsigned)c.splits, (unsigned)(g.nout < 65535 ? g.nout : 65535));
        reduce_generic_split_kernel<Pol, T, kGenericThreads><<<grid, kGenericThreads, 0, st>>>(
            a, out, o, g.nout, g.rlen, g.rstride, c.chunk, op, tickets, partials);
    } else if (c.shape == SH_GENERIC_WARP) {
        int64_t blocks = ceil_div(g.nout, 8);
        if (blocks > cap * 4) blocks = cap * 4;
        reduce_generic_warp_kernel<Pol, T><<<(unsigned)blocks, 256, 0, st>>>(a, out, o, g.nout, g.rlen, g.rstride, op);
    } else {
        int64_t blocks = ceil_div(g.nout, 256);
        if (blocks > cap) blocks = cap;
        if (blocks < 1) blocks = 1;
        reduce_generic_kernel<Pol, T><<<(unsigned)blocks, 256, 0, st>>>(a, out, o, g.nout, g.rlen, g.rstride, op);
    }
    return cuda_error(cudaGetLastError(), "reduce_generic launch");
}

template <typename T>
int launch_generic_t(const Choice& c, int op, const ReduceGeom& g, const T* a, void* out, void* ws, int sm_count,
                     cudaStream_t st) {
    switch (op) {
    case CTB_SUM: case CTB_MEAN: case kOpSumAccumulate:
        return launch_generic_pol<SumPol<double>, T>(c, op, g, a, out, ws, sm_count, st);
    case CTB_MAX: return launch_generic_pol<MinMaxPol<double, true>, T>(c, op, g, a, out, ws, sm_count, st);
    case CTB_MIN: return launch_generic_pol<MinMaxPol<double, false>, T>(c, op, g, a, out, ws, sm_count, st);
    case CTB_VAR: return launch_generic_pol<VarPol<double>, T>(c, op, g, a, out, ws, sm_count, st);
    case CTB_ARGMAX: return launch_generic_pol<ArgmaxPol<double>, T>(c, op, g, a, out, ws, sm_count, st);
    }
    return set_error(CTB_ERR_ARG, "reduce: unknown operator code %d", op);
}

}  // namespace

size_t reduce_workspace_bytes(const ReduceGeom& g, int dtype) {
    DeviceInfo di;
    if (current_device_info(&di) != CTB_OK) di.sm_count = 148;
    // the base address is not known here: take the larger of the aligned (vector) and the
    // unaligned (scalar) layout
    const size_t vec_need = scratch_bytes(g, choose(g, dtype, nullptr, di.sm_count));
    const size_t scalar_need = scratch_bytes(g, choose(g, dtype, reinterpret_cast<const void*>(4), di.sm_count));
    return vec_need > scalar_need ? vec_need : scalar_need;
}

int launch_reduce(int op, int dtype, const ReduceGeom& g, const void* a, void* out,
                  double* partial_out, void* ws, size_t ws_bytes, cudaStream_t st) {
    if (op < 0 || op > kOpSumAccumulate) return set_error(CTB_ERR_ARG, "reduce: unknown operator code %d", op);
    DeviceInfo di;
    int rc = current_device_info(&di);
    if (rc) return rc;
    if (g.nout == 0) return CTB_OK;
    Choice c = choose(g, dtype, a, di.sm_count);
    if (partial_out && c.shape != SH_ROWS_SPLIT) {
        // the fp64 partial is only produced by the split kernel; force it (splits may be 1)
        if (dtype != CTB_F32 || g.rstride != 1 || g.nout != 1)
            return set_error(CTB_ERR_ARG, "reduce: fp64 partials need a dense Float32 input");
        c.shape = SH_ROWS_SPLIT;
        c.vec = (is_aligned(a, 16) && g.rlen % 4 == 0) ? 4 : 1;
        c.chunk = ceil_div(g.rlen > 0 ? g.rlen : 1, (int64_t)CTB_RED_THREADS * 4 * CTB_RED_SPLIT_UNROLL) * CTB_RED_THREADS * 4 * CTB_RED_SPLIT_UNROLL;
        c.splits = 1;
    }
    const size_t need = scratch_bytes(g, c);
    if (need > ws_bytes || (need && !ws)) return set_error(CTB_ERR_WORKSPACE, "reduce: workspace of %zu bytes needed, %zu given", need, ws_bytes);
    if (need && !is_aligned(ws, 256)) return set_error(CTB_ERR_WORKSPACE, "reduce: workspace must be 256-byte aligned");

    if (c.shape == SH_GENERIC || c.shape == SH_GENERIC_WARP || c.shape == SH_GENERIC_SPLIT) {
        switch (dtype) {
        case CTB_F32: return launch_generic_t<float>(c, op, g, (const float*)a, out, ws, di.sm_count, st);
        case CTB_I32: return launch_generic_t<int32_t>(c, op, g, (const int32_t*)a, out, ws, di.sm_count, st);
        case CTB_F64: return launch_generic_t<double>(c, op, g, (const double*)a, out, ws, di.sm_count, st);
        // the element types the reference reduces through double on its scalar back-end only
        case CTB_U8: return launch_generic_t<uint8_t>(c, op, g, (const uint8_t*)a, out, ws, di.sm_count, st);
        case CTB_I8: return launch_generic_t<int8_t>(c, op, g, (const int8_t*)a, out, ws, di.sm_count, st);
        case CTB_I16: return launch_generic_t<int16_t>(c, op, g, (const int16_t*)a, out, ws, di.sm_count, st);
        case CTB_I64: return launch_generic_t<int64_t>(c, op, g, (const int64_t*)a, out, ws, di.sm_count, st);
        case CTB_BOOL: return launch_generic_t<bool>(c, op, g, (const bool*)a, out, ws, di.sm_count, st);
        }
        return set_error(CTB_ERR_DTYPE, "reduce: unsupported dtype");
    }
    const float* fa = (const float*)a;
    switch (op) {
    case CTB_SUM: case CTB_MEAN: case kOpSumAccumulate: return launch_fast<SumPol<float>>(c, g, fa, out, partial_out, ws, op, di.sm_count, st);
    case CTB_MAX:
        if (g.rlen < (int64_t(1) << 30)) return launch_fast<MinMaxPol<float, true, int32_t>>(c, g, fa, out, partial_out, ws, op, di.sm_count, st);
        return launch_fast<MinMaxPol<float, true>>(c, g, fa, out, partial_out, ws, op, di.sm_count, st);
    case CTB_MIN:
        if (g.rlen < (int64_t(1) << 30)) return launch_fast<MinMaxPol<float, false, int32_t>>(c, g, fa, out, partial_out, ws, op, di.sm_count, st);
        return launch_fast<MinMaxPol<float, false>>(c, g, fa, out, partial_out, ws, op, di.sm_count, st);
    case CTB_VAR: return launch_fast<VarPol<float>>(c, g, fa, out, nullptr, ws, op, di.sm_count, st);
    case CTB_ARGMAX: return launch_fast<ArgmaxPol<float>>(c, g, fa, out, nullptr, ws, op, di.sm_count, st);
    }
    return set_error(CTB_ERR_ARG, "reduce: unknown operator code %d", op);
}

// ---- scratch that needs no allocation ---------------------------------------------------------------
// Part of the library's device image: present on every GPU that loads it, for the life of the
// process.  In host code this name is only a handle; the device address comes from
// cudaGetSymbolAddress, looked up once per device with that device current.
static __device__ __align__(256) unsigned char g_static_scratch[CTB_NOALLOC_SCRATCH_BYTES];

namespace {
std::mutex g_static_mu;
void* g_static_addr[64] = {};

int static_scratch_address(void** ptr) {
    int dev = -1;
    CTB_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return set_error(CTB_ERR_CUDA, "device index %d out of range", dev);
    std::lock_guard<std::mutex> lk(g_static_mu);
    if (!g_static_addr[dev]) {
        void* p = nullptr;
        CTB_CUDA_TRY(cudaGetSymbolAddress(&p, g_static_scratch));
        if (!p) return set_error(CTB_ERR_CUDA, "static scratch has no device address");
        g_static_addr[dev] = p;
    }
    *ptr = g_static_addr[dev];
    return CTB_OK;
}
}  // namespace

int launch_reduce_static_scratch(int op, int dtype, const ReduceGeom& g, const void* a, void* out,
                                 cudaStream_t st) {
    const size_t need = reduce_workspace_bytes(g, dtype);
    if (need > CTB_NOALLOC_SCRATCH_BYTES)
        return set_error(CTB_ERR_LIMIT,
                         "reduction without allocation: this shape needs %zu bytes of scratch, the fixed buffer holds %u",
                         need, (unsigned)CTB_NOALLOC_SCRATCH_BYTES);
    void* ws = nullptr;
    if (need) {
        int rc = static_scratch_address(&ws);
        if (rc) return rc;
        // the array keeps the previous call's contents; the tickets must start at zero
        CTB_CUDA_TRY(cudaMemsetAsync(ws, 0, kTicketBytes, st));
    }
    return launch_reduce(op, dtype, g, a, out, nullptr, ws, need ? CTB_NOALLOC_SCRATCH_BYTES : 0, st);
}

int launch_finalize_full(int op, int dtype, const double* partial, int64_t total, void* out, cudaStream_t st) {
    switch (dtype) {
    case CTB_F32: finalize_full_kernel<float><<<1, 32, 0, st>>>(op, partial, total, (float*)out); break;
    case CTB_I32: finalize_full_kernel<int32_t><<<1, 32, 0, st>>>(op, partial, total, (int32_t*)out); break;
    case CTB_F64: finalize_full_kernel<double><<<1, 32, 0, st>>>(op, partial, total, (double*)out); break;
    case CTB_U8: finalize_full_kernel<uint8_t><<<1, 32, 0, st>>>(op, partial, total, (uint8_t*)out); break;
    case CTB_I8: finalize_full_kernel<int8_t><<<1, 32, 0, st>>>(op, partial, total, (int8_t*)out); break;
    case CTB_I16: finalize_full_kernel<int16_t><<<1, 32, 0, st>>>(op, partial, total, (int16_t*)out); break;
    case CTB_I64: finalize_full_kernel<int64_t><<<1, 32, 0, st>>>(op, partial, total, (int64_t*)out); break;
    case CTB_BOOL: finalize_full_kernel<bool><<<1, 32, 0, st>>>(op, partial, total, (bool*)out); break;
    default: return set_error(CTB_ERR_DTYPE, "finalize: unsupported dtype");
    }
    return cuda_error(cudaGetLastError(), "finalize launch");
}

}  // namespace ctb
