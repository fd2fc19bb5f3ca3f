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
// TensorIterator, src/core/opsmp.cpp:76-126).  dims are ordered outer -> inner.  Operator results
// are fresh contiguous tensors, so the output's strides are normally implied by the shape; a copy
// into a slice of an existing tensor (cat) sets `out_strided` and gives them in `ostride`.
constexpr int kMaxOperands = 3;
struct Plan {
    int32_t ndim;                       // >= 1
    int32_t nin;                        // number of inputs (1 or 2; up to 3 for fused rows)
    int64_t numel;                      // output elements
    int64_t shape[CTB_MAX_DIMS];
    int64_t stride[kMaxOperands][CTB_MAX_DIMS];   // per input, elements, 0 = broadcast
    int32_t out_strided;                // 0: the output is contiguous
    int64_t ostride[CTB_MAX_DIMS];      // output strides when out_strided
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

// ---- index decomposition --------------------------------------------------------------------------
// Division by a run-time constant through a precomputed multiplier (Granlund-Montgomery):
// q = (umulhi(n, mul) + n) >> shr, exact for 0 <= n < 2^31 and 1 <= d < 2^31.  A 32-bit
// hardware-emulated division costs ~20 issue slots and a 64-bit one ~70; this costs 3.
struct FastDiv {
    uint32_t d, mul, shr;
};
inline FastDiv make_fastdiv(uint32_t d) {
    FastDiv f;
    f.d = d ? d : 1;
    uint32_t s = 0;
    while (s < 32 && (1ull << s) < f.d) ++s;
    f.shr = s;
    f.mul = (uint32_t)((((uint64_t)1 << 32) * (((uint64_t)1 << s) - f.d)) / f.d + 1);
    return f;
}
__device__ __forceinline__ uint32_t fast_div(uint32_t n, const FastDiv& f) {
    return (__umulhi(n, f.mul) + n) >> f.shr;
}

// Mixed-radix decomposition of a linear index over up to CTB_MAX_DIMS dims (outer -> inner)
// into a weighted sum with per-dim strides.  `fast` says every dim and the index fit 31 bits.
struct DimSet {
    int32_t n;
    int32_t fast;
    int64_t shape[CTB_MAX_DIMS];
    FastDiv fd[CTB_MAX_DIMS];
};
inline void dimset_init(DimSet* s, int n, const int64_t* shape) {
    s->n = n;
    int64_t total = 1;
    bool fast = true;
    for (int d = 0; d < n; ++d) {
        s->shape[d] = shape[d];
        total *= shape[d] > 0 ? shape[d] : 1;
        if (shape[d] >= 0x7FFFFFFFll || total >= 0x7FFFFFFFll) fast = false;
    }
    s->fast = fast;
    for (int d = 0; d < n; ++d) s->fd[d] = make_fastdiv(fast ? (uint32_t)shape[d] : 1u);
}
// off_k += coord_d * stride_k[d] for NS stride sets at once.
template <int NS>
__device__ __forceinline__ void dimset_offsets(const DimSet& s, int64_t i, const int64_t (*stride)[CTB_MAX_DIMS],
                                               int64_t* off) {
    if (s.fast) {
        uint32_t t = (uint32_t)i;
        for (int d = s.n - 1; d >= 0; --d) {
            const uint32_t q = fast_div(t, s.fd[d]);
            const uint32_t c = t - q * s.fd[d].d;
            t = q;
#pragma unroll
            for (int k = 0; k < NS; ++k) off[k] += (int64_t)c * stride[k][d];
        }
    } else {
        for (int d = s.n - 1; d >= 0; --d) {
            const int64_t q = i / s.shape[d];
            const int64_t c = i - q * s.shape[d];
            i = q;
#pragma unroll
            for (int k = 0; k < NS; ++k) off[k] += c * stride[k][d];
        }
    }
}

// ---- launchers implemented in the .cu files ---------------------------------------------------
// All return a ctb_status and never synchronise.
int launch_binary(int op, int dtype, const Plan& plan, const void* a, const void* b, void* out,
                  cudaStream_t stream);
int launch_unary(int op, int dtype, const Plan& plan, const void* a, double scalar, void* out,
                 cudaStream_t stream);
int launch_copy(int elem_bytes, const Plan& plan, const void* a, void* out, cudaStream_t stream);
// out[i] = x[i with coordinate `dim` replaced by index[i]]; shapes/strides have `ndim` entries.
int launch_gather(int elem_bytes, int ndim, const int64_t* ishape, const int64_t* xstride, const int64_t* istride,
                  int dim, int64_t gsize, const void* x, const void* index, int index_dtype, void* out, int32_t* bad,
                  cudaStream_t st);
// grad[...] += src[...] (finite values only) over `shape`, any strides.
int launch_accumulate_strided(int dtype, int ndim, const int64_t* shape, const int64_t* gstride,
                              const int64_t* sstride, void* grad, const void* src, cudaStream_t stream);

// In-place optimizer steps on contiguous buffers of n elements.
int launch_sgd(int dtype, void* param, const void* grad, int64_t n, double lr, cudaStream_t stream);
int launch_adam(float* param, const float* grad, float* m, float* v, int64_t n, double lr, double beta1,
                double beta2, double eps, int step, double weight_decay, int decoupled_decay,
                cudaStream_t stream);

// c[batch][M][N] (contiguous) = a x b with the given element strides; a batch stride of 0 repeats
// that operand for every batch entry.
int launch_matmul(int dtype, const void* a, const void* b, void* c, int64_t batch, int64_t M, int64_t N, int64_t K,
                  int64_t a_m, int64_t a_k, int64_t a_batch, int64_t b_k, int64_t b_n, int64_t b_batch,
                  cudaStream_t stream);

// Tensor-core product (ctb_matmul_tc.cu): c[M, N] = a[M, K] x bt[N, K]^T, fp32 in and out, TF32 products.
int launch_matmul_tf32(const float* a, int64_t lda, const float* bt, int64_t ldb, float* c, int64_t ldc, int64_t M,
                       int64_t N, int64_t K, int* error, cudaStream_t stream);

int launch_optimizer(int kind, float* param, const float* grad, float* state1, float* state2, int64_t n,
                     const ctb_optimizer_hyper& hyper, int step, cudaStream_t stream);

struct ReducePlan;   // ctb_reduce.cuh
}  // namespace ctb
