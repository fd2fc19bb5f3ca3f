// Tensor-core matrix product for sm_100a: out = a x b on the 5th-generation tensor cores
// (tcgen05.mma, kind::tf32, accumulators in tensor memory), operands brought into shared memory by
// TMA (cp.async.bulk.tensor, 128-byte swizzle), one 128 x 128 output tile per CTA.
//
// This is the second matmul entry point.  ctb_matmul (ctb_matmul.cu) reproduces matmul_mp
// (src/core/opsmp.cpp:460-558 of the reference) bit for bit on the CUDA cores; this one follows the
// reference's SIMD GEMMs (src/cpu/AVX2/ops_avx2_f32.cpp:650-775), which already differ from
// matmul_mp in summation order and fused multiply-adds, under a stated tolerance: the products
// are formed from the operands' upper 19 bits (TF32: 10 mantissa bits) and accumulated in fp32.
//
// Layout of one CTA (128 threads, 4 warps):
//   warp 0, one elected lane : TMA producer — per k-block (32 columns of fp32 = 128 bytes per row)
//                              one A box [128 rows x 128 B] and one B box [128 rows x 128 B] into a
//                              ring of kStages shared-memory stages; completion on mbarrier full[s]
//   warp 1, one elected lane : MMA issuer — waits full[s], issues 4 tcgen05.mma (K = 8 each) per
//                              stage into the 128 x 128 fp32 accumulator in tensor memory, then
//                              tcgen05.commit -> mbarrier empty[s]; after the last k-block a commit
//                              -> mbarrier accum
//   all 4 warps              : epilogue — wait accum, tcgen05.ld (32 lanes x 32 columns per
//                              instruction, warp w owns accumulator rows 32w .. 32w+31), store
// Both operands are K-major in global memory: A[M, K] with unit stride along K, and B given as
// B^T[N, K] with unit stride along K (the host passes a transposed copy when b is not laid out
// like that; for the reference's Linear layer, which multiplies by weight.permute({1, 0}), b
// already is).  TMA fills everything outside the matrices with zeros, so M, N and K need no
// padding; the epilogue bounds its stores.
//
// No wait in this kernel is unbounded: every mbarrier wait gives up after kSpinLimit polls, raises
// the error word in global memory and sets the CTA's abort flag, which every other wait loop
// checks; the CTA then drains what it issued, frees its tensor memory and returns.
#include <cuda.h>

#include <mutex>

#include "ctb_common.cuh"

namespace ctb {
namespace {

constexpr int kTileM = 128, kTileN = 128, kTileK = 32;      // kTileK fp32 = one 128-byte swizzle row
constexpr int kStages = 4;
constexpr int kUmmaK = 8;                                    // K of one tcgen05.mma, kind::tf32
constexpr uint32_t kStageBytesA = kTileM * kTileK * 4, kStageBytesB = kTileN * kTileK * 4;
constexpr uint32_t kTmemCols = 128;                          // fp32 accumulator columns (power of two >= 32)
constexpr uint32_t kSpinLimit = 1u << 20;
constexpr size_t kSmemBytes = 1024 + (size_t)kStages * (kStageBytesA + kStageBytesB) + 256;

// instruction descriptor: D = F32, A = B = TF32, both K-major, N = 128, M = 128
constexpr uint32_t kIdesc = (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(kTileN >> 3) << 17) | ((uint32_t)(kTileM >> 4) << 24);

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

__global__ void __launch_bounds__(128, 1)
matmul_tf32_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, float* __restrict__ c,
                   int64_t M, int64_t N, int64_t K, int64_t ldc, int* error) {
    extern __shared__ uint8_t smem_raw[];
    // 1024-byte alignment of the tiles (the swizzle pattern repeats every 1024 bytes)
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* tiles_a = smem;
    uint8_t* tiles_b = smem + kStages * kStageBytesA;
    uint64_t* full = (uint64_t*)(smem + kStages * (kStageBytesA + kStageBytesB));
    uint64_t* empty = full + kStages;
    uint64_t* accum = empty + kStages;
    uint32_t* tmem_slot = (uint32_t*)(accum + 1);
    volatile uint32_t* abort_flag = tmem_slot + 1;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int num_kb = (int)((K + kTileK - 1) / kTileK);
    const int tile_n = blockIdx.x, tile_m = blockIdx.y;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        mbar_init(accum, 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {                      // the whole warp allocates the accumulator's tensor-memory columns
        __syncwarp();                     // .sync.aligned: lane 0 comes back from the barrier set-up first
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;

    int issued = 0;                       // k-blocks whose loads the producer has issued
    if (warp == 0 && lane == 0) {
        // ---- TMA producer -------------------------------------------------------------------------
        for (int kb = 0; kb < num_kb; ++kb) {
            const int s = kb % kStages;
            if (kb >= kStages && !mbar_wait(&empty[s], ((kb / kStages) - 1) & 1, abort_flag, error, 1)) break;
            mbar_expect_tx(&full[s], kStageBytesA + kStageBytesB);
            tma_load_2d(tiles_a + s * kStageBytesA, &map_a, kb * kTileK, tile_m * kTileM, &full[s]);
            tma_load_2d(tiles_b + s * kStageBytesB, &map_b, kb * kTileK, tile_n * kTileN, &full[s]);
            issued = kb + 1;
        }
    } else if (warp == 1 && lane == 0) {
        // ---- MMA issuer ---------------------------------------------------------------------------
        bool ok = true;
        for (int kb = 0; kb < num_kb && ok; ++kb) {
            const int s = kb % kStages;
            ok = mbar_wait(&full[s], (kb / kStages) & 1, abort_flag, error, 2);
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint64_t desc_a = umma_desc(smem_u32(tiles_a + s * kStageBytesA));
            const uint64_t desc_b = umma_desc(smem_u32(tiles_b + s * kStageBytesB));
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
                    ::"r"(tmem_base), "l"(da), "l"(db), "r"(kIdesc), "r"(accumulate) : "memory");
            }
            // the stage is free again once these MMAs have read it
            asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(&empty[s])) : "memory");
        }
        // the accumulator is complete when everything issued above has finished (also on an early exit,
        // so that the epilogue's wait ends)
        asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(accum)) : "memory");
    }
    __syncwarp();

    // ---- epilogue: tensor memory -> registers -> global ---------------------------------------------
    // warp-uniform: the tensor-memory loads below are .sync.aligned and must see the whole warp
    const bool have = __all_sync(0xffffffffu, num_kb > 0 && mbar_wait(accum, 0, abort_flag, error, 3) && !*abort_flag);
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const int64_t row = (int64_t)tile_m * kTileM + warp * 32 + lane;         // warp w reads accumulator lanes 32w..32w+31
#pragma unroll 1
    for (int chunk = 0; chunk < kTileN / 32; ++chunk) {
        uint32_t v[32];
        if (have) {
            const uint32_t taddr = tmem_base + ((uint32_t)(warp * 32) << 16) + (uint32_t)(chunk * 32);
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
            for (int i = 0; i < 32; ++i) v[i] = 0u;                               // K == 0: an empty sum
        }
        const int64_t col0 = (int64_t)tile_n * kTileN + chunk * 32;
        if (row < M && (have || num_kb == 0)) {
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

    // ---- orderly exit ----------------------------------------------------------------------------------
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (*abort_flag && warp == 0 && lane == 0) {
        // loads that were issued but never consumed still write into this CTA's shared memory: give
        // each of them a bounded wait before the CTA goes away
        for (int kb = issued > kStages ? issued - kStages : 0; kb < issued; ++kb)
            for (uint32_t it = 0; it < kSpinLimit && !mbar_try_wait(&full[kb % kStages], (kb / kStages) & 1); ++it) {}
    }
    __syncthreads();
    __syncwarp();
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
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

}  // namespace

// c[M, N] (row stride ldc) = a[M, K] (row stride lda, unit stride along K) x bt[N, K]^T (row stride ldb).
// a and bt must be 16-byte aligned with row strides that are multiples of 4 elements (TMA's rules).
// `error`: one int in device memory, 0 before the call; non-zero afterwards if a wait inside the
// kernel gave up (1 producer, 2 MMA issuer, 3 epilogue).
int launch_matmul_tf32(const float* a, int64_t lda, const float* bt, int64_t ldb, float* c, int64_t ldc, int64_t M,
                       int64_t N, int64_t K, int* error, cudaStream_t st) {
    if (M == 0 || N == 0) return CTB_OK;
    static std::once_flag once;
    static cudaError_t attr_rc = cudaSuccess;
    std::call_once(once, [] {
        attr_rc = cudaFuncSetAttribute(matmul_tf32_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytes);
    });
    // the attribute is per device: set it again when the current device never saw it (cheap, idempotent)
    CTB_CUDA_TRY(cudaFuncSetAttribute(matmul_tf32_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytes));
    if (attr_rc != cudaSuccess) return cuda_error(attr_rc, "matmul_tc shared-memory opt-in");
    CUtensorMap map_a, map_b;
    int rc;
    // K == 0: the maps cannot describe an empty dim; the kernel then writes zeros without touching them
    const int64_t k_for_map = K > 0 ? K : 1;
    if ((rc = make_map(&map_a, a, M, k_for_map, lda, kTileM))) return rc;
    if ((rc = make_map(&map_b, bt, N, k_for_map, ldb, kTileN))) return rc;
    const dim3 grid((unsigned)ceil_div(N, kTileN), (unsigned)ceil_div(M, kTileM));
    matmul_tf32_kernel<<<grid, 128, kSmemBytes, st>>>(map_a, map_b, c, M, N, K, ldc, error);
    return cuda_error(cudaGetLastError(), "matmul_tc launch");
}

}  // namespace ctb
