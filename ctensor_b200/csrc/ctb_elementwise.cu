// Elementwise kernels of the operator path (binary broadcast ops, unary ops, strided copy).
//
// Three kernel shapes, picked by the host from the collapsed iteration plan:
//   ew_flat  : every operand is contiguous (or a single broadcast element) -> one flat index
//              space, 128/256-bit streaming loads and stores, several loads in flight per thread.
//   ew_rows  : [outer dims..., inner] where every operand's inner stride is 0 or 1
//              (row broadcast [R,C]o[1,C], column broadcast [R,C]o[R,1], permuted views whose
//              innermost dim is contiguous, bias adds).  Offsets are computed once per
//              (row, column-chunk) tile, the inner dim is accessed with vector loads when the
//              alignment allows it.
//   ew_gather: anything else — one div/mod chain per element (the "strided-gather" path).
//
// These replace binary_op_impl / unary_op_impl (src/core/opsmp.cpp:136-385 of the reference),
// the AVX2 contiguous/general paths (src/cpu/AVX2/ops_avx2_f32.cpp:357-568) and
// Tensor::clone's odometer copy (src/core/tensor.cpp:84-113).
#include "ctb_common.cuh"
#include "ctb_math.cuh"

namespace ctb {

// Tunables (overridable at build time for sweeps).
#ifndef CTB_EW_THREADS
#define CTB_EW_THREADS 256
#endif
#ifndef CTB_EW_VEC_BYTES
#define CTB_EW_VEC_BYTES 32
#endif
#ifndef CTB_EW_UNROLL
#define CTB_EW_UNROLL 2
#endif
#ifndef CTB_ROWS_VEC_BYTES
#define CTB_ROWS_VEC_BYTES 16
#endif
#ifndef CTB_ROWS_UNROLL
#define CTB_ROWS_UNROLL 4
#endif

// ---- functor adapters ----------------------------------------------------------------------------
template <int OP, typename T> struct BinAdapter {
    static constexpr bool kHasPair = false;
    __device__ __forceinline__ static T apply2(T x, T y) { return BinaryFn<OP, T>::apply(x, y); }
    __device__ __forceinline__ static T apply1(T x, double) { return x; }
};
template <int OP, typename T> struct UnAdapter {
    static constexpr bool kHasPair = false;
    __device__ __forceinline__ static T apply2(T x, T) { return x; }
    __device__ __forceinline__ static T apply1(T x, double s) { return UnaryFn<OP, T>::apply(x, s); }
};
template <int OP> struct UnAdapter<OP, float> {
    static constexpr bool kHasPair = UnaryFn<OP, float>::kHasPair;
    __device__ __forceinline__ static float apply2(float x, float) { return x; }
    __device__ __forceinline__ static float apply1(float x, double s) { return UnaryFn<OP, float>::apply(x, s); }
    __device__ __forceinline__ static float2 apply_pair(float2 x, double s) { return UnaryFn<OP, float>::apply_pair(x, s); }
};
template <typename T> struct CopyAdapter {
    static constexpr bool kHasPair = false;
    __device__ __forceinline__ static T apply2(T x, T) { return x; }
    __device__ __forceinline__ static T apply1(T x, double) { return x; }
};

// r = f(va [, vb]) over one vector; unary functors with a packed form process two lanes at a time.
template <typename F, typename T, int NIN, int VEC>
__device__ __forceinline__ void apply_vec(Vec<T, VEC>& r, const Vec<T, VEC>& va, const Vec<T, VEC>& vb, double scalar) {
    if constexpr (NIN == 1 && F::kHasPair && VEC % 2 == 0) {
#pragma unroll
        for (int k = 0; k < VEC; k += 2) {
            const float2 t = F::apply_pair(make_float2(va.v[k], va.v[k + 1]), scalar);
            r.v[k] = t.x;
            r.v[k + 1] = t.y;
        }
    } else {
#pragma unroll
        for (int k = 0; k < VEC; ++k) {
            if (NIN == 2) r.v[k] = F::apply2(va.v[k], vb.v[k]);
            else r.v[k] = F::apply1(va.v[k], scalar);
        }
    }
}

// ------------------------------------------------------------------------------------------------
// ew_flat: out[i] = f(a[i * sa], b[i * sb]) with sa, sb in {0, 1}.
// One CTA per tile of THREADS*VEC*UNROLL consecutive elements (no grid-stride loop: on B200 a
// grid of one-tile CTAs measured ~10 % faster than a persistent grid for these streaming
// kernels).  Pass u of thread t touches vector (u*THREADS + t), so every warp-level access is
// one fully coalesced request, and all UNROLL*NIN loads are issued before the first use.
// The CTA after the last full tile handles the ragged tail with scalar accesses.
// ------------------------------------------------------------------------------------------------
template <typename F, typename T, int NIN, int VEC, int UNROLL, int THREADS>
__global__ void __launch_bounds__(THREADS)
ew_flat_kernel(const T* __restrict__ a, const T* __restrict__ b, T* __restrict__ out,
               int64_t n, int a_bcast, int b_bcast, double scalar) {
    using V = Vec<T, VEC>;
    constexpr int64_t TILE = (int64_t)THREADS * VEC * UNROLL;
    const int64_t full_tiles = n / TILE;
    const int64_t tile = blockIdx.x;
    T a0 = a_bcast ? a[0] : T(0);
    T b0 = (NIN == 2 && b_bcast) ? b[0] : T(0);

    if (tile < full_tiles) {
        const int64_t base = tile * TILE + (int64_t)threadIdx.x * VEC;
        V va[UNROLL], vb[UNROLL];
        if (!a_bcast) {
#pragma unroll
            for (int u = 0; u < UNROLL; ++u)
                va[u] = ldg_stream(reinterpret_cast<const V*>(a + base + (int64_t)u * THREADS * VEC));
        }
        if (NIN == 2 && !b_bcast) {
#pragma unroll
            for (int u = 0; u < UNROLL; ++u)
                vb[u] = ldg_stream(reinterpret_cast<const V*>(b + base + (int64_t)u * THREADS * VEC));
        }
        if (a_bcast) {
#pragma unroll
            for (int u = 0; u < UNROLL; ++u)
#pragma unroll
                for (int k = 0; k < VEC; ++k) va[u].v[k] = a0;
        }
        if (NIN == 2 && b_bcast) {
#pragma unroll
            for (int u = 0; u < UNROLL; ++u)
#pragma unroll
                for (int k = 0; k < VEC; ++k) vb[u].v[k] = b0;
        }
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            V r;
            apply_vec<F, T, NIN, VEC>(r, va[u], vb[u], scalar);
            stg_stream(reinterpret_cast<V*>(out + base + (int64_t)u * THREADS * VEC), r);
        }
    } else {
        for (int64_t i = full_tiles * TILE + threadIdx.x; i < n; i += THREADS) {
            T x = a_bcast ? a0 : a[i];
            if (NIN == 2) {
                T y = b_bcast ? b0 : b[i];
                out[i] = F::apply2(x, y);
            } else {
                out[i] = F::apply1(x, scalar);
            }
        }
    }
}

// ------------------------------------------------------------------------------------------------
// ew_rows: plan dims = [outer..., inner]; inner strides are 0/1 for every input.
// A tile is VEC*THREADS consecutive inner elements of one row.  tile -> (row, chunk) by one
// 32-bit div, row -> per-operand offsets by ndim-1 div/mods, both once per thread per tile.
// Rows are enumerated in the order the host chose (oshape/ostride* are listed in that order):
// for a permuted input it follows the INPUT's memory order, so reads stream sequentially and
// the writes form a few sequential streams, instead of reads hopping between distant 4 KiB runs.
// ------------------------------------------------------------------------------------------------
struct RowsArgs {
    DimSet outer;                           // outer dims in enumeration order (all < 2^31)
    int64_t stride[3][CTB_MAX_DIMS];        // [0], [1] = inputs, [2] = output, per outer dim
    int32_t istride[2];                     // inner stride per input: 0 or 1
    uint32_t inner;                         // inner length
    FastDiv tiles_per_row;
    uint32_t ntiles;                        // rows * tiles_per_row (< 2^31)
};

// MODE picks the body at compile time, because run-time tests on the operands' inner strides and
// on the tile's raggedness inside the unrolled load loop made the scheduler wait for each load
// before issuing the next one:
//   ROWS_GENERAL     any inner strides 0/1, any alignment, ragged rows: element-wise accesses.
//   ROWS_VEC         everything 16-byte aligned, inner % VEC == 0, first input inner-contiguous,
//                    second input (if any) inner-contiguous: unconditional vector loads.
//   ROWS_VEC_BSCALAR same, but the second input has inner stride 0 (one value per row).
// In the two vector modes a thread without work loads from a valid dummy address (the row
// start) instead of branching around the load, and only its store is predicated.
enum { ROWS_GENERAL = 0, ROWS_VEC = 1, ROWS_VEC_BSCALAR = 2 };

template <typename F, typename T, int NIN, int VEC, int UNROLL, int THREADS, int MODE>
__global__ void __launch_bounds__(THREADS)
ew_rows_kernel(const T* __restrict__ a, const T* __restrict__ b, T* __restrict__ out,
               RowsArgs g, double scalar) {
    using V = Vec<T, VEC>;
    constexpr uint32_t TILE = THREADS * VEC;
    constexpr bool ALIGNED = false;                     // the general body works element by element
    // Per-tile offsets are computed by one thread each and shared through smem: the div/mod
    // chain would otherwise be repeated by all THREADS threads and dominate the kernel.
    __shared__ int64_t s_oa[UNROLL], s_ob[UNROLL], s_oo[UNROLL];
    __shared__ uint32_t s_col[UNROLL];
    for (uint32_t t0 = blockIdx.x * UNROLL; t0 < g.ntiles; t0 += gridDim.x * UNROLL) {
        if (threadIdx.x < UNROLL) {
            const uint32_t t = t0 + threadIdx.x;
            uint32_t col0 = 0xFFFFFFFFu;                // "no tile"
            int64_t oa = 0, ob = 0, oout = 0;
            if (t < g.ntiles) {
                const uint32_t row = fast_div(t, g.tiles_per_row);
                col0 = (t - row * g.tiles_per_row.d) * TILE;
                int64_t off[3] = {0, 0, 0};
                dimset_offsets<3>(g.outer, row, g.stride, off);
                oa = off[0];
                ob = off[1];
                oout = off[2];
            }
            s_oa[threadIdx.x] = oa;
            s_ob[threadIdx.x] = ob;
            s_oo[threadIdx.x] = oout;
            s_col[threadIdx.x] = col0;
        }
        __syncthreads();
        if constexpr (MODE != ROWS_GENERAL) {
            V va[UNROLL], vb[UNROLL];
            int64_t oo[UNROLL];
            bool act[UNROLL];
#pragma unroll
            for (int u = 0; u < UNROLL; ++u) {
                const uint32_t col0 = s_col[u];
                const uint32_t col = col0 + threadIdx.x * VEC;          // wraps for "no tile": then >= inner or caught by col0
                act[u] = col0 != 0xFFFFFFFFu && col < g.inner;
                const uint32_t c = act[u] ? col : 0u;
                oo[u] = s_oo[u] + c;
                va[u] = ldg_stream(reinterpret_cast<const V*>(a + s_oa[u] + c));
                if constexpr (NIN == 2) {
                    if constexpr (MODE == ROWS_VEC) {
                        vb[u] = ldg_stream(reinterpret_cast<const V*>(b + s_ob[u] + c));
                    } else {
                        const T sb = b[s_ob[u]];
#pragma unroll
                        for (int k = 0; k < VEC; ++k) vb[u].v[k] = sb;
                    }
                }
            }
#pragma unroll
            for (int u = 0; u < UNROLL; ++u) {
                V r;
                apply_vec<F, T, NIN, VEC>(r, va[u], vb[u], scalar);
                if (act[u]) stg_stream(reinterpret_cast<V*>(out + oo[u]), r);
            }
        } else {
        V va[UNROLL], vb[UNROLL];
        int64_t oo[UNROLL];
        uint32_t cnt[UNROLL];
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            cnt[u] = 0;
            const uint32_t col0 = s_col[u];
            if (col0 == 0xFFFFFFFFu) continue;
            const uint32_t col = col0 + threadIdx.x * VEC;
            if (col >= g.inner) continue;
            oo[u] = s_oo[u] + col;
            const uint32_t left = g.inner - col;
            cnt[u] = left < (uint32_t)VEC ? left : (uint32_t)VEC;
            const T* pa = a + s_oa[u] + (g.istride[0] ? col : 0);
            const T* pb = (NIN == 2) ? b + s_ob[u] + (g.istride[1] ? col : 0) : nullptr;
            if (ALIGNED && cnt[u] == VEC) {
                if (g.istride[0]) va[u] = ldg_stream(reinterpret_cast<const V*>(pa));
                else {
                    const T s = *pa;
#pragma unroll
                    for (int k = 0; k < VEC; ++k) va[u].v[k] = s;
                }
                if (NIN == 2) {
                    if (g.istride[1]) vb[u] = ldg_stream(reinterpret_cast<const V*>(pb));
                    else {
                        const T s = *pb;
#pragma unroll
                        for (int k = 0; k < VEC; ++k) vb[u].v[k] = s;
                    }
                }
            } else {
#pragma unroll
                for (int k = 0; k < VEC; ++k) {
                    if ((uint32_t)k < cnt[u]) {
                        va[u].v[k] = pa[g.istride[0] ? k : 0];
                        if (NIN == 2) vb[u].v[k] = pb[g.istride[1] ? k : 0];
                    }
                }
            }
        }
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            if (cnt[u] == 0) continue;
            V r;
            apply_vec<F, T, NIN, VEC>(r, va[u], vb[u], scalar);
            if (ALIGNED && cnt[u] == VEC) {
                stg_stream(reinterpret_cast<V*>(out + oo[u]), r);
            } else {
#pragma unroll
                for (int k = 0; k < VEC; ++k)
                    if ((uint32_t)k < cnt[u]) out[oo[u] + k] = r.v[k];
            }
        }
        }
        __syncthreads();      // smem is rewritten by the next pass
    }
}

// ------------------------------------------------------------------------------------------------
// ew_gather: fully general strided operands; one output element per thread per step.
// ------------------------------------------------------------------------------------------------
struct GatherArgs {
    DimSet dims;
    int64_t stride[3][CTB_MAX_DIMS];       // [0], [1] = inputs, [2] = output (OUT_STRIDED only)
    int64_t numel;
};

template <typename F, typename T, int NIN, bool OUT_STRIDED>
__global__ void __launch_bounds__(256)
ew_gather_kernel(const T* __restrict__ a, const T* __restrict__ b, T* __restrict__ out,
                 GatherArgs g, double scalar) {
    const int64_t step = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < g.numel; i += step) {
        int64_t off[3] = {0, 0, 0};
        if (OUT_STRIDED) dimset_offsets<3>(g.dims, i, g.stride, off);
        else dimset_offsets<2>(g.dims, i, g.stride, off);
        const int64_t o = OUT_STRIDED ? off[2] : i;
        if (NIN == 2) out[o] = F::apply2(a[off[0]], b[off[1]]);
        else out[o] = F::apply1(a[off[0]], scalar);
    }
}

// ---- host-side shape classification and launch ----------------------------------------------------
namespace {

bool plan_is_flat(const Plan& p) {
    if (p.ndim != 1) return false;
    if (p.out_strided && p.ostride[0] != 1 && p.shape[0] > 1) return false;
    for (int i = 0; i < p.nin; ++i)
        if (p.stride[i][0] != 0 && p.stride[i][0] != 1) return false;
    return true;
}

bool plan_is_rows(const Plan& p) {
    if (p.ndim < 2) return false;
    if (p.out_strided && p.ostride[p.ndim - 1] != 1) return false;
    for (int i = 0; i < p.nin; ++i) {
        int64_t s = p.stride[i][p.ndim - 1];
        if (s != 0 && s != 1) return false;
    }
    if (p.shape[p.ndim - 1] < 32) return false;              // tiny rows: gather is as good
    if (p.shape[p.ndim - 1] > 0xFFFFFFFFll) return false;
    for (int d = 0; d < p.ndim - 1; ++d) if (p.shape[d] > 0xFFFFFFFFll) return false;
    return true;
}

// The general strided kernel alone: what the element types outside Float32 / Int32 / Double64 use
// (the reference serves them through its type-erased scalar loop as well).
template <typename F, typename T, int NIN>
int launch_gather_shape(const Plan& p, const T* a, const T* b, T* out, double scalar, cudaStream_t st) {
    GatherArgs ga{};
    dimset_init(&ga.dims, p.ndim, p.shape);
    for (int d = 0; d < p.ndim; ++d)
        for (int i = 0; i < NIN; ++i) ga.stride[i][d] = p.stride[i][d];
    ga.numel = p.numel;
    int64_t blocks = ceil_div(p.numel, 256);
    if (blocks > 0x7FFFFFFFll) blocks = 0x7FFFFFFFll;
    if (p.out_strided) {
        for (int d = 0; d < p.ndim; ++d) ga.stride[2][d] = p.ostride[d];
        ew_gather_kernel<F, T, NIN, true><<<(unsigned)blocks, 256, 0, st>>>(a, b, out, ga, scalar);
    } else {
        ew_gather_kernel<F, T, NIN, false><<<(unsigned)blocks, 256, 0, st>>>(a, b, out, ga, scalar);
    }
    return cuda_error(cudaGetLastError(), "ew_gather launch");
}

template <typename F, typename T, int NIN>
int launch_shapes(const Plan& p, const T* a, const T* b, T* out, double scalar, cudaStream_t st) {
    constexpr int THREADS = CTB_EW_THREADS;
    constexpr int VEC = CTB_EW_VEC_BYTES / (int)sizeof(T);
    constexpr int UNROLL = CTB_EW_UNROLL;
    if (p.numel == 0) return CTB_OK;

    if (plan_is_flat(p)) {
        const int a_b = p.stride[0][0] == 0 && p.numel > 1;
        const int b_b = NIN == 2 && p.stride[1][0] == 0 && p.numel > 1;
        const bool aligned = is_aligned(out, CTB_EW_VEC_BYTES) && (a_b || is_aligned(a, CTB_EW_VEC_BYTES)) &&
                             (NIN == 1 || b_b || is_aligned(b, CTB_EW_VEC_BYTES));
        if (aligned) {
            constexpr int64_t TILE = (int64_t)THREADS * VEC * UNROLL;
            const int64_t grid = p.numel / TILE + (p.numel % TILE ? 1 : 0);
            if (grid > 0x7FFFFFFFll) return set_error(CTB_ERR_LIMIT, "elementwise: tensor too large for one launch");
            ew_flat_kernel<F, T, NIN, VEC, UNROLL, THREADS><<<(unsigned)grid, THREADS, 0, st>>>(a, b, out, p.numel, a_b, b_b, scalar);
        } else {
            // misaligned base (an odd view offset): scalar accesses, still coalesced
            constexpr int64_t TILE = (int64_t)THREADS * UNROLL * 4;
            const int64_t grid = p.numel / TILE + (p.numel % TILE ? 1 : 0);
            if (grid > 0x7FFFFFFFll) return set_error(CTB_ERR_LIMIT, "elementwise: tensor too large for one launch");
            ew_flat_kernel<F, T, NIN, 1, UNROLL * 4, THREADS><<<(unsigned)grid, THREADS, 0, st>>>(a, b, out, p.numel, a_b, b_b, scalar);
        }
        return cuda_error(cudaGetLastError(), "ew_flat launch");
    }

    if (plan_is_rows(p)) {
        constexpr int RVEC = CTB_ROWS_VEC_BYTES / (int)sizeof(T);
        constexpr int RUNROLL = CTB_ROWS_UNROLL;
        RowsArgs g{};
        const int nd = p.ndim;
        // Enumeration order of the outer dims: by decreasing stride of the first full-size
        // (non-broadcast) input, i.e. that input's memory order; ties keep the output order.
        int order[CTB_MAX_DIMS];
        for (int d = 0; d < nd - 1; ++d) order[d] = d;
        int lead = 0;
        for (int i = 0; i < NIN; ++i) {
            bool full = true;
            for (int d = 0; d < nd - 1; ++d) if (p.stride[i][d] == 0) full = false;
            if (full) { lead = i; break; }
        }
        for (int i = 1; i < nd - 1; ++i)
            for (int j = i; j > 0 && p.stride[lead][order[j]] > p.stride[lead][order[j - 1]]; --j) {
                const int t = order[j]; order[j] = order[j - 1]; order[j - 1] = t;
            }
        int64_t out_stride[CTB_MAX_DIMS];
        if (p.out_strided) {
            for (int d = 0; d < nd - 1; ++d) out_stride[d] = p.ostride[d];
        } else {
            int64_t st = p.shape[nd - 1];
            for (int d = nd - 2; d >= 0; --d) { out_stride[d] = st; st *= p.shape[d]; }
        }
        int64_t rows = 1;
        // vector accesses need every operand that is read or written as vectors (inner stride 1)
        // to start on a vector boundary in every row
        const T* in_ptr[2] = {a, b};
        bool aligned = is_aligned(out, CTB_ROWS_VEC_BYTES) && (p.shape[nd - 1] % RVEC == 0);
        for (int i = 0; i < NIN; ++i)
            if (p.stride[i][nd - 1] == 1 && !is_aligned(in_ptr[i], CTB_ROWS_VEC_BYTES)) aligned = false;
        int64_t oshape[CTB_MAX_DIMS];
        for (int k = 0; k < nd - 1; ++k) {
            const int d = order[k];
            oshape[k] = p.shape[d];
            g.stride[2][k] = out_stride[d];
            if (out_stride[d] % RVEC != 0) aligned = false;
            rows *= p.shape[d];
            for (int i = 0; i < NIN; ++i) {
                g.stride[i][k] = p.stride[i][d];
                if (p.stride[i][nd - 1] == 1 && p.stride[i][d] % RVEC != 0) aligned = false;
            }
        }
        dimset_init(&g.outer, nd - 1, oshape);
        for (int i = 0; i < NIN; ++i) g.istride[i] = (int32_t)p.stride[i][nd - 1];
        g.inner = (uint32_t)p.shape[nd - 1];
        constexpr int64_t TILE = (int64_t)THREADS * RVEC;
        const int64_t tpr = ceil_div(p.shape[nd - 1], TILE);
        const int64_t ntiles = rows * tpr;
        if (ntiles < 0x7FFFFFFFll - 4096 && g.outer.fast) {
            g.tiles_per_row = make_fastdiv((uint32_t)tpr);
            g.ntiles = (uint32_t)ntiles;
            const unsigned grid = (unsigned)ceil_div(ntiles, RUNROLL);      // one pass per CTA
            const bool vec_ok = aligned && g.istride[0] == 1;
            if (vec_ok && (NIN == 1 || g.istride[1] == 1))
                ew_rows_kernel<F, T, NIN, RVEC, RUNROLL, THREADS, ROWS_VEC><<<grid, THREADS, 0, st>>>(a, b, out, g, scalar);
            else if (NIN == 2 && vec_ok)
                ew_rows_kernel<F, T, NIN, RVEC, RUNROLL, THREADS, (NIN == 2 ? ROWS_VEC_BSCALAR : ROWS_VEC)><<<grid, THREADS, 0, st>>>(a, b, out, g, scalar);
            else
                ew_rows_kernel<F, T, NIN, RVEC, RUNROLL, THREADS, ROWS_GENERAL><<<grid, THREADS, 0, st>>>(a, b, out, g, scalar);
            return cuda_error(cudaGetLastError(), "ew_rows launch");
        }
    }

    return launch_gather_shape<F, T, NIN>(p, a, b, out, scalar, st);
}

template <int OP>
int launch_binary_dt(int dtype, const Plan& p, const void* a, const void* b, void* out, cudaStream_t st) {
    switch (dtype) {
    case CTB_F32: return launch_shapes<BinAdapter<OP, float>, float, 2>(p, (const float*)a, (const float*)b, (float*)out, 0.0, st);
    case CTB_I32: return launch_shapes<BinAdapter<OP, int32_t>, int32_t, 2>(p, (const int32_t*)a, (const int32_t*)b, (int32_t*)out, 0.0, st);
    case CTB_F64: return launch_shapes<BinAdapter<OP, double>, double, 2>(p, (const double*)a, (const double*)b, (double*)out, 0.0, st);
#define CTB_NARROW(CODE, T) case CODE: return launch_gather_shape<BinAdapter<OP, T>, T, 2>(p, (const T*)a, (const T*)b, (T*)out, 0.0, st);
    CTB_NARROW(CTB_U8, uint8_t) CTB_NARROW(CTB_I8, int8_t) CTB_NARROW(CTB_I16, int16_t) CTB_NARROW(CTB_I64, int64_t) CTB_NARROW(CTB_BOOL, bool)
#undef CTB_NARROW
    }
    return set_error(CTB_ERR_DTYPE, "binary op: unsupported dtype or op not registered");
}

template <int OP>
int launch_unary_dt(int dtype, const Plan& p, const void* a, double s, void* out, cudaStream_t st) {
    switch (dtype) {
    case CTB_F32: return launch_shapes<UnAdapter<OP, float>, float, 1>(p, (const float*)a, nullptr, (float*)out, s, st);
    case CTB_I32: return launch_shapes<UnAdapter<OP, int32_t>, int32_t, 1>(p, (const int32_t*)a, nullptr, (int32_t*)out, s, st);
    case CTB_F64: return launch_shapes<UnAdapter<OP, double>, double, 1>(p, (const double*)a, nullptr, (double*)out, s, st);
#define CTB_NARROW(CODE, T) case CODE: return launch_gather_shape<UnAdapter<OP, T>, T, 1>(p, (const T*)a, nullptr, (T*)out, s, st);
    CTB_NARROW(CTB_U8, uint8_t) CTB_NARROW(CTB_I8, int8_t) CTB_NARROW(CTB_I16, int16_t) CTB_NARROW(CTB_I64, int64_t) CTB_NARROW(CTB_BOOL, bool)
#undef CTB_NARROW
    }
    return set_error(CTB_ERR_DTYPE, "unary op: unsupported dtype");
}

}  // namespace

int launch_binary(int op, int dtype, const Plan& p, const void* a, const void* b, void* out, cudaStream_t st) {
    switch (op) {
#define CASE(OP) case OP: return launch_binary_dt<OP>(dtype, p, a, b, out, st);
    CASE(CTB_ADD) CASE(CTB_SUB) CASE(CTB_MUL) CASE(CTB_DIV)
    CASE(CTB_LT) CASE(CTB_LE) CASE(CTB_GT) CASE(CTB_GE) CASE(CTB_EQ) CASE(CTB_NE) CASE(CTB_POW)
    CASE(kOpAddFinite)
#undef CASE
    }
    return set_error(CTB_ERR_ARG, "binary op: unknown operator code %d", op);
}

int launch_unary(int op, int dtype, const Plan& p, const void* a, double s, void* out, cudaStream_t st) {
    if (unary_is_f32_only(op) && dtype != CTB_F32)
        return set_error(CTB_ERR_DTYPE, "unary op %d: only Float32 has a pinned flavour", op);
    switch (op) {
#define CASE(OP) case OP: return launch_unary_dt<OP>(dtype, p, a, s, out, st);
    CASE(CTB_ADD_S) CASE(CTB_SUB_S) CASE(CTB_RSUB_S) CASE(CTB_MUL_S) CASE(CTB_DIV_S) CASE(CTB_RDIV_S)
    CASE(CTB_POW_S) CASE(CTB_RPOW_S)
    CASE(CTB_LT_S) CASE(CTB_LE_S) CASE(CTB_GT_S) CASE(CTB_GE_S) CASE(CTB_EQ_S) CASE(CTB_NE_S)
    CASE(CTB_ABS) CASE(CTB_RELU) CASE(CTB_SQRT)
    CASE(CTB_SIN) CASE(CTB_COS) CASE(CTB_TAN) CASE(CTB_ASIN) CASE(CTB_ACOS) CASE(CTB_ATAN)
    CASE(CTB_SINH) CASE(CTB_COSH) CASE(CTB_SOFTPLUS)
#undef CASE
    // fp32-only flavours: instantiate for float alone
#define CASEF(OP) case OP: return launch_shapes<UnAdapter<OP, float>, float, 1>(p, (const float*)a, nullptr, (float*)out, s, st);
    CASEF(CTB_EXP) CASEF(CTB_LOG) CASEF(CTB_TANH) CASEF(CTB_SIGMOID) CASEF(CTB_GELU_TANH)
#undef CASEF
    }
    return set_error(CTB_ERR_ARG, "unary op: unknown operator code %d", op);
}

int launch_copy(int elem_bytes, const Plan& p, const void* a, void* out, cudaStream_t st) {
    if (elem_bytes == 4)
        return launch_shapes<CopyAdapter<uint32_t>, uint32_t, 1>(p, (const uint32_t*)a, nullptr, (uint32_t*)out, 0.0, st);
    if (elem_bytes == 8)
        return launch_shapes<CopyAdapter<uint64_t>, uint64_t, 1>(p, (const uint64_t*)a, nullptr, (uint64_t*)out, 0.0, st);
    if (elem_bytes == 1)
        return launch_gather_shape<CopyAdapter<uint8_t>, uint8_t, 1>(p, (const uint8_t*)a, nullptr, (uint8_t*)out, 0.0, st);
    if (elem_bytes == 2)
        return launch_gather_shape<CopyAdapter<uint16_t>, uint16_t, 1>(p, (const uint16_t*)a, nullptr, (uint16_t*)out, 0.0, st);
    return set_error(CTB_ERR_DTYPE, "copy: unsupported element size %d", elem_bytes);
}

}  // namespace ctb
