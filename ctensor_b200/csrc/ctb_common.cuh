// Shared declarations of the sm_100a operator library: status/error plumbing, the collapsed
// iteration plan handed to kernels, launch geometry constants and vector load/store helpers.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include <stddef.h>
#include "../../include/ctb200.h"

namespace ctb {

// ---- error plumbing (host) -------------------------------------------------------------------
int set_error(int code, const char* fmt, ...);
int cuda_error(cudaError_t e, const char* what);
#define CTB_CUDA_TRY(expr)                                         \
    do {                                                           \
        cudaError_t _e = (expr);                                   \
        if (_e != cudaSuccess) return ::ctb::cuda_error(_e, #expr); \
    } while (0)

// ---- device properties ----------------------------------------------------------------------
struct DeviceInfo {
    int device;
    int sm_count;        // 148 on B200
};
int current_device_info(DeviceInfo* info);

// ---- iteration plan -------------------------------------------------------------------------
// The host collapses (out, a, b) into at most CTB_MAX_DIMS joint dims (size-1 dims dropped,
// adjacent dims merged when every operand allows it — the same folding idea as the reference's
// TensorIterator, src/core/opsmp.cpp:76-126).  dims are ordered outer -> inner; the output is
// always contiguous so its strides are implied.
constexpr int kMaxOperands = 3;
struct Plan {
    int32_t ndim;                       // >= 1
    int32_t nin;                        // number of inputs (1 or 2; up to 3 for fused rows)
    int64_t numel;                      // output elements
    int64_t shape[CTB_MAX_DIMS];
    int64_t stride[kMaxOperands][CTB_MAX_DIMS];   // per input, elements, 0 = broadcast
};

// ---- vector access ----------------------------------------------------------------------------
// 128-bit and 256-bit global accesses (sm_100 has 256-bit ld/st.global).  Plain loads and stores:
// on B200 the default cache policy measured faster than .nc, L1::no_allocate or .cs hints for
// these read-once / write-once streams.
template <typename T, int N> struct alignas(sizeof(T) * N) Vec { T v[N]; };

__device__ __forceinline__ Vec<float, 4> ldg_stream(const Vec<float, 4>* p) {
    Vec<float, 4> r;
    asm volatile("ld.global.v4.f32 {%0,%1,%2,%3}, [%4];"
                 : "=f"(r.v[0]), "=f"(r.v[1]), "=f"(r.v[2]), "=f"(r.v[3]) : "l"(p));
    return r;
}
__device__ __forceinline__ Vec<float, 8> ldg_stream(const Vec<float, 8>* p) {
    Vec<float, 8> r;
    asm volatile("ld.global.v8.f32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=f"(r.v[0]), "=f"(r.v[1]), "=f"(r.v[2]), "=f"(r.v[3]),
                   "=f"(r.v[4]), "=f"(r.v[5]), "=f"(r.v[6]), "=f"(r.v[7]) : "l"(p));
    return r;
}
__device__ __forceinline__ void stg_stream(Vec<float, 4>* p, const Vec<float, 4>& r) {
    asm volatile("st.global.v4.f32 [%0], {%1,%2,%3,%4};"
                 :: "l"(p), "f"(r.v[0]), "f"(r.v[1]), "f"(r.v[2]), "f"(r.v[3]) : "memory");
}
__device__ __forceinline__ void stg_stream(Vec<float, 8>* p, const Vec<float, 8>& r) {
    asm volatile("st.global.v8.f32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};"
                 :: "l"(p), "f"(r.v[0]), "f"(r.v[1]), "f"(r.v[2]), "f"(r.v[3]),
                    "f"(r.v[4]), "f"(r.v[5]), "f"(r.v[6]), "f"(r.v[7]) : "memory");
}
// Generic (any 4/8-byte T) fallbacks through plain C++ vector copies.
template <typename T, int N>
__device__ __forceinline__ Vec<T, N> ldg_stream(const Vec<T, N>* p) { return *p; }
template <typename T, int N>
__device__ __forceinline__ void stg_stream(Vec<T, N>* p, const Vec<T, N>& r) { *p = r; }

__host__ __device__ __forceinline__ bool is_aligned(const void* p, size_t bytes) {
    return (reinterpret_cast<uintptr_t>(p) % bytes) == 0;
}

inline int64_t ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }

// Broadcast lane 0's 64-bit value to the whole warp (index arithmetic with divisions is done
// by one lane and shared, not repeated by all 32).
__device__ __forceinline__ int64_t warp_bcast64(int64_t v) {
    int lo = __shfl_sync(0xffffffffu, (int)(v & 0xffffffffll), 0);
    int hi = __shfl_sync(0xffffffffu, (int)(v >> 32), 0);
    return ((int64_t)hi << 32) | (uint32_t)lo;
}

// ---- launchers implemented in the .cu files ---------------------------------------------------
// All return a ctb_status and never synchronise.
int launch_binary(int op, int dtype, const Plan& plan, const void* a, const void* b, void* out,
                  cudaStream_t stream);
int launch_unary(int op, int dtype, const Plan& plan, const void* a, double scalar, void* out,
                 cudaStream_t stream);
int launch_copy(int elem_bytes, const Plan& plan, const void* a, void* out, cudaStream_t stream);

struct ReducePlan;   // ctb_reduce.cuh
}  // namespace ctb
