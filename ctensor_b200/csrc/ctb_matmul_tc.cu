// Tensor-core matrix product for sm_100a: out = a x b on the 5th-generation tensor cores
// (tcgen05.mma, kind::tf32, accumulators in tensor memory), operands brought into shared memory by
// TMA (cp.async.bulk.tensor, 128-byte swizzle).  A persistent kernel: one CTA per SM walks over
// output tiles of 128 x TILE_N (TILE_N = 256 or 128) and overlaps the read-back of one tile's
// accumulator with the products of the next.
//
// This is the second matmul entry point.  ctb_matmul (ctb_matmul.cu) reproduces matmul_mp
// (src/core/opsmp.cpp:460-558 of the reference) bit for bit on the CUDA cores; this one follows the
// reference's SIMD GEMMs (src/cpu/AVX2/ops_avx2_f32.cpp:650-775), which already differ from
// matmul_mp in summation order and fused multiply-adds, under a stated tolerance: the products
// are formed from the operands' upper 19 bits (TF32: 10 mantissa bits) and accumulated in fp32.
//
// Layout of one CTA (192 threads, 6 warps):
//   warp 0, one elected lane : TMA producer — per k-block (32 columns of fp32 = 128 bytes per row)
//                              one A box [128 rows x 128 B] and one B box [TILE_N rows x 128 B] into
//                              a ring of kStages shared-memory stages; completion on mbarrier
//                              full[s].  The ring runs on across tile boundaries.
//   warp 1, one elected lane : MMA issuer — waits full[s], issues 4 tcgen05.mma (K = 8 each) per
//                              stage into one of TWO 128 x TILE_N fp32 accumulators in tensor
//                              memory, then tcgen05.commit -> mbarrier empty[s]; after a tile's
//                              last k-block a commit -> mbarrier acc_full[buffer]
//   warps 2..5               : epilogue — wait acc_full[buffer], tcgen05.ld (32 lanes x 32 columns
//                              per instruction; a warp reaches the accumulator rows 32 (w mod 4) ..
//                              + 31), store, arrive on mbarrier acc_empty[buffer]
// Both operands are K-major in global memory: A[M, K] with unit stride along K, and B given as
// B^T[N, K] with unit stride along K (the host passes a transposed copy when b is not laid out
// like that; for the reference's Linear layer, which multiplies by weight.permute({1, 0}), b
// already is).  TMA fills everything outside the matrices with zeros, so M, N and K need no
// padding; the epilogue bounds its stores.  Tiles are visited in bands of 16 tile rows, column by
// column inside a band, so that the CTAs of one wave share A and B panels in L2.
//
// No wait in this kernel is unbounded: every mbarrier wait gives up after kSpinLimit polls, raises
// the error word in global memory and sets the CTA's abort flag, which every other wait loop
// checks; the CTA then drains what it issued, frees its tensor memory and returns.
#include <cuda.h>

#include <cstdlib>

#include "ctb_common.cuh"

namespace ctb {
namespace {

constexpr int kTileM = 128, kTileK = 32;                    // kTileK fp32 = one 128-byte swizzle row
constexpr int kUmmaK = 8;                                    // K of one tcgen05.mma, kind::tf32
constexpr int kThreads = 192;                                // producer warp, MMA warp, 4 epilogue warps
constexpr int kGroupM = 16;                                  // tile rows per band of the visiting order
constexpr uint32_t kSpinLimit = 1u << 20;
constexpr double kWideTileGain = 1.5;                        // measured mainloop efficiency of the 256-wide tile over the 128-wide one

template <int TILE_N> struct Cfg {
    // the ring is as deep as shared memory allows: what hides the load latency is bytes in flight
    static constexpr int kStages = TILE_N == 256 ? 4 : 6;
    static constexpr uint32_t kStageBytesA = kTileM * kTileK * 4, kStageBytesB = TILE_N * kTileK * 4;
    static constexpr uint32_t kTmemCols = 2 * TILE_N;       // two fp32 accumulators (a power of two >= 32)
    static constexpr size_t kSmemBytes = 1024 + (size_t)kStages * (kStageBytesA + kStageBytesB) + 256;
    // instruction descriptor: D = F32, A = B = TF32, both K-major, N = TILE_N, M = 128
    static constexpr uint32_t kIdesc = (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(TILE_N >> 3) << 17) | ((uint32_t)(kTileM >> 4) << 24);
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.b32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return ok != 0;
}
// Bounded wait: false when the limit ran out or another thread of the CTA gave up.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile uint32_t* abort_flag, int* error,
                                          int where) {
    for (uint32_t it = 0; it < kSpinLimit; ++it) {
        if (mbar_try_wait(bar, parity)) return true;
        if (*abort_flag) return false;
    }
    *abort_flag = 1;
    if (error) atomicCAS(error, 0, where);
    return false;
}

// 64-bit shared-memory matrix descriptor: K-major tile, 128-byte swizzle, 8-row groups 1024 B apart
__device__ __forceinline__ uint64_t umma_desc(uint32_t smem_addr) {
    const uint32_t lo = ((smem_addr & 0x3FFFFu) >> 4) | (1u << 16);          // start address, LBO field = 1 (unused when swizzled)
    const uint32_t hi = (1024u >> 4) | (1u << 14) | (2u << 29);              // SBO = 1024 B, descriptor version 1, SWIZZLE_128B
    return ((uint64_t)hi << 32) | lo;
}

__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 ::"r"(smem_u32(dst)), "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// Tile `t` of the visiting order -> (tile row, tile column): bands of kGroupM tile rows, inside a
// band column by column, so that consecutive tiles (which run at the same time on neighbouring
// SMs) share one B panel and kGroupM A panels.
__device__ __forceinline__ void tile_coords(int64_t t, int tiles_m, int tiles_n, int& tm, int& tn) {
    const int64_t band_tiles = (int64_t)kGroupM * tiles_n;
    const int band = (int)(t / band_tiles);
    const int first = band * kGroupM;
    const int rows = min(kGroupM, tiles_m - first);
    const int64_t in_band = t - (int64_t)band * band_tiles;
    tm = first + (int)(in_band % rows);
    tn = (int)(in_band / rows);
}

template <int TILE_N>
__global__ void __launch_bounds__(kThreads, 1)
matmul_tf32_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, float* __restrict__ c,
                   int64_t M, int64_t N, int64_t K, int64_t ldc, int tiles_m, int tiles_n, int* error) {
    using C = Cfg<TILE_N>;
    constexpr int kStages = C::kStages;
    extern __shared__ uint8_t smem_raw[];
    // 1024-byte alignment of the tiles (the swizzle pattern repeats every 1024 bytes)
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* tiles_a = smem;
    uint8_t* tiles_b = smem + kStages * C::kStageBytesA;
    uint64_t* full = (uint64_t*)(smem + kStages * (C::kStageBytesA + C::kStageBytesB));
    uint64_t* empty = full + kStages;
    uint64_t* acc_full = empty + kStages;          // [2]: the MMAs of a tile have finished
    uint64_t* acc_empty = acc_full + 2;            // [2]: the epilogue has read the accumulator back
    uint32_t* tmem_slot = (uint32_t*)(acc_empty + 2);
    volatile uint32_t* abort_flag = tmem_slot + 1;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int num_kb = (int)((K + kTileK - 1) / kTileK);
    const int64_t num_tiles = (int64_t)tiles_m * tiles_n;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&acc_full[b], 1);
            mbar_init(&acc_empty[b], 4);           // one arrival per epilogue warp
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {                      // the whole warp allocates the accumulators' tensor-memory columns
        __syncwarp();                     // .sync.aligned: lane 0 comes back from the barrier set-up first
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(C::kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;

    int64_t issued = 0;                   // k-blocks whose loads the producer has issued (all tiles)
    if (warp == 0) {
        if (lane == 0 && num_kb > 0) {
            // ---- TMA producer -----------------------------------------------------------------------
            int64_t it = 0;
            bool ok = true;
            for (int64_t t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
                int tm, tn;
                tile_coords(t, tiles_m, tiles_n, tm, tn);
                for (int kb = 0; kb < num_kb; ++kb, ++it) {
                    const int s = (int)(it % kStages);
                    if (it >= kStages && !mbar_wait(&empty[s], (uint32_t)((it / kStages) - 1) & 1, abort_flag, error, 1)) { ok = false; break; }
                    mbar_expect_tx(&full[s], C::kStageBytesA + C::kStageBytesB);
                    tma_load_2d(tiles_a + s * C::kStageBytesA, &map_a, kb * kTileK, tm * kTileM, &full[s]);
                    tma_load_2d(tiles_b + s * C::kStageBytesB, &map_b, kb * kTileK, tn * TILE_N, &full[s]);
                    issued = it + 1;
                }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        if (lane == 0 && num_kb > 0) {
            // ---- MMA issuer -------------------------------------------------------------------------
            int64_t it = 0;
            int local = 0;                // tiles this CTA has started
            bool ok = true;
            for (int64_t t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, ++local) {
                const int buf = local & 1;
                // the epilogue must have read this accumulator's previous tile back
                if (local >= 2 && !mbar_wait(&acc_empty[buf], (uint32_t)((local >> 1) - 1) & 1, abort_flag, error, 4)) { ok = false; break; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t acc = tmem_base + (uint32_t)(buf * TILE_N);
                for (int kb = 0; kb < num_kb; ++kb, ++it) {
                    const int s = (int)(it % kStages);
                    if (!mbar_wait(&full[s], (uint32_t)(it / kStages) & 1, abort_flag, error, 2)) { ok = false; break; }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint64_t desc_a = umma_desc(smem_u32(tiles_a + s * C::kStageBytesA));
                    const uint64_t desc_b = umma_desc(smem_u32(tiles_b + s * C::kStageBytesB));
#pragma unroll
                    for (int k = 0; k < kTileK / kUmmaK; ++k) {
                        // the next 8 columns of the swizzled row: 32 bytes further, i.e. +2 in the address field
                        const uint64_t da = desc_a + (uint64_t)(k * kUmmaK * 4 >> 4);
                        const uint64_t db = desc_b + (uint64_t)(k * kUmmaK * 4 >> 4);
                        const uint32_t accumulate = (kb > 0 || k > 0) ? 1u : 0u;
                        asm volatile(
                            "{\n\t.reg .pred p;\n\t"
                            "setp.ne.b32 p, %4, 0;\n\t"
                            "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
                            ::"r"(acc), "l"(da), "l"(db), "r"(C::kIdesc), "r"(accumulate) : "memory");
                    }
                    // the stage is free again once these MMAs have read it
                    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(&empty[s])) : "memory");
                }
                // the accumulator is complete when everything issued above has finished (also on an
                // early exit, so that the epilogue's wait ends)
                asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(&acc_full[buf])) : "memory");
            }
        }
        __syncwarp();
    } else {
        // ---- epilogue: tensor memory -> registers -> global --------------------------------------------
        const int quarter = warp & 3;         // the tensor-memory lanes a warp may read: 32 (warp mod 4) ..
        int local = 0;
        bool ok = true;
        for (int64_t t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, ++local) {
            int tm, tn;
            tile_coords(t, tiles_m, tiles_n, tm, tn);
            const int buf = local & 1;
            // warp-uniform: the tensor-memory loads below are .sync.aligned and must see the whole warp
            const bool have = num_kb > 0 &&
                              __all_sync(0xffffffffu, mbar_wait(&acc_full[buf], (uint32_t)(local >> 1) & 1, abort_flag, error, 3) && !*abort_flag);
            if (num_kb > 0 && !have) { ok = false; break; }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const int64_t row = (int64_t)tm * kTileM + quarter * 32 + lane;
#pragma unroll 1
            for (int chunk = 0; chunk < TILE_N / 32; ++chunk) {
                uint32_t v[32];
                if (have) {
                    const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(buf * TILE_N + chunk * 32);
                    asm volatile(
                        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
                        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
                        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
                          "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
                          "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
                          "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
                        : "r"(taddr) : "memory");
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                } else {
#pragma unroll
                    for (int i = 0; i < 32; ++i) v[i] = 0u;                           // K == 0: an empty sum
                }
                const int64_t col0 = (int64_t)tn * TILE_N + chunk * 32;
                if (row < M && col0 < N) {
                    float* dst = c + row * ldc + col0;
                    if (col0 + 32 <= N && (((uintptr_t)dst) & 15) == 0) {
#pragma unroll
                        for (int i = 0; i < 32; i += 4)
                            *reinterpret_cast<float4*>(dst + i) = make_float4(__uint_as_float(v[i]), __uint_as_float(v[i + 1]),
                                                                              __uint_as_float(v[i + 2]), __uint_as_float(v[i + 3]));
                    } else {
#pragma unroll
                        for (int i = 0; i < 32; ++i)
                            if (col0 + i < N) dst[i] = __uint_as_float(v[i]);
                    }
                }
            }
            if (have) {
                // this warp is done with the accumulator: the MMA warp may overwrite it
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                __syncwarp();
                if (lane == 0) mbar_arrive(&acc_empty[buf]);
            }
        }
        __syncwarp();
    }

    // ---- orderly exit ----------------------------------------------------------------------------------
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (*abort_flag && warp == 0 && lane == 0) {
        // loads that were issued but never consumed still write into this CTA's shared memory: give
        // each of them a bounded wait before the CTA goes away
        for (int64_t it = issued > kStages ? issued - kStages : 0; it < issued; ++it)
            for (uint32_t n = 0; n < kSpinLimit && !mbar_try_wait(&full[it % kStages], (uint32_t)(it / kStages) & 1); ++n) {}
    }
    __syncthreads();
    __syncwarp();
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(C::kTmemCols) : "memory");
}

// ---- host side ----------------------------------------------------------------------------------------
using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                   const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess) {
            cudaGetLastError();
            p = nullptr;
        }
        return (EncodeTiledFn)p;
    }();
    return fn;
}

// A [rows, K] fp32 matrix with unit stride along K and `ld` elements between rows, as a 2-d tensor map
// with boxes of kTileK x box_rows elements and the 128-byte swizzle.
int make_map(CUtensorMap* map, const float* base, int64_t rows, int64_t K, int64_t ld, int box_rows) {
    EncodeTiledFn enc = encode_fn();
    if (!enc) return set_error(CTB_ERR_CUDA, "matmul_tc: the driver offers no cuTensorMapEncodeTiled");
    const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)ld * sizeof(float)};
    const cuuint32_t box[2] = {(cuuint32_t)kTileK, (cuuint32_t)box_rows};
    const cuuint32_t elem[2] = {1, 1};
    const CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, (void*)base, dims, strides, box, elem,
                           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return set_error(CTB_ERR_CUDA, "matmul_tc: cuTensorMapEncodeTiled failed (%d)", (int)r);
    return CTB_OK;
}

template <int TILE_N>
int launch_tile(const float* a, int64_t lda, const float* bt, int64_t ldb, float* c, int64_t ldc, int64_t M, int64_t N,
                int64_t K, int* error, int sm_count, cudaStream_t st) {
    using C = Cfg<TILE_N>;
    // the attribute is per device and the call is cheap and idempotent
    CTB_CUDA_TRY(cudaFuncSetAttribute(matmul_tf32_kernel<TILE_N>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)C::kSmemBytes));
    CUtensorMap map_a, map_b;
    int rc;
    // K == 0: the maps cannot describe an empty dim; the kernel then writes zeros without touching them
    const int64_t k_for_map = K > 0 ? K : 1;
    if ((rc = make_map(&map_a, a, M, k_for_map, lda, kTileM))) return rc;
    if ((rc = make_map(&map_b, bt, N, k_for_map, ldb, TILE_N))) return rc;
    const int64_t tiles_m = ceil_div(M, (int64_t)kTileM), tiles_n = ceil_div(N, (int64_t)TILE_N);
    if (tiles_m > INT32_MAX / 2 || tiles_n > INT32_MAX / 2) return set_error(CTB_ERR_LIMIT, "matmul_tc: matrix too large");
    const int64_t tiles = tiles_m * tiles_n;
    const unsigned grid = (unsigned)(tiles < sm_count ? tiles : sm_count);      // one persistent CTA per SM
    matmul_tf32_kernel<TILE_N><<<grid, kThreads, C::kSmemBytes, st>>>(map_a, map_b, c, M, N, K, ldc, (int)tiles_m, (int)tiles_n, error);
    return cuda_error(cudaGetLastError(), "matmul_tc launch");
}

// Tile width for a problem.  A 256-wide tile moves 1.5 instead of 2 operand bytes per 128 x 128 x 32
// block of products and gives the load ring twice the time per stage, but it quantises the work
// into half as many, twice as long pieces: take it unless that costs more rounds of the machine
// than it saves.  The environment variable CTB_MATMUL_TC_TILE_N (128 | 256) overrides the choice.
int choose_tile_n(int64_t M, int64_t N, int sm_count) {
    static const int forced = [] {
        const char* e = getenv("CTB_MATMUL_TC_TILE_N");
        return e ? atoi(e) : 0;
    }();
    if (forced == 128 || forced == 256) return forced;
    if (N <= 128) return 128;
    const int64_t tm = ceil_div(M, (int64_t)kTileM);
    const int64_t rounds128 = ceil_div(tm * ceil_div(N, (int64_t)128), (int64_t)sm_count);
    const int64_t rounds256 = ceil_div(tm * ceil_div(N, (int64_t)256), (int64_t)sm_count);
    // cost in units of one 128-wide tile's mainloop; the wide tile's mainloop runs ~1.5x as efficiently
    return (double)rounds256 * 2.0 / kWideTileGain <= (double)rounds128 ? 256 : 128;
}

}  // namespace

// c[M, N] (row stride ldc) = a[M, K] (row stride lda, unit stride along K) x bt[N, K]^T (row stride ldb).
// a and bt must be 16-byte aligned with row strides that are multiples of 4 elements (TMA's rules).
// `error`: one int in device memory, 0 before the call; non-zero afterwards if a wait inside the
// kernel gave up (1 producer, 2 MMA issuer on a stage, 3 epilogue, 4 MMA issuer on an accumulator).
int launch_matmul_tf32(const float* a, int64_t lda, const float* bt, int64_t ldb, float* c, int64_t ldc, int64_t M,
                       int64_t N, int64_t K, int* error, cudaStream_t st) {
    if (M == 0 || N == 0) return CTB_OK;
    DeviceInfo di;
    int rc;
    if ((rc = current_device_info(&di))) return rc;
    if (choose_tile_n(M, N, di.sm_count) == 256) return launch_tile<256>(a, lda, bt, ldb, c, ldc, M, N, K, error, di.sm_count, st);
    return launch_tile<128>(a, lda, bt, ldb, c, ldc, M, N, K, error, di.sm_count, st);
}

}  // namespace ctb
