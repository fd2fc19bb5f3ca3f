// Plain (non-tensor-core) batched matrix product, so that callers of the operator path that
// also multiply matrices (Linear::forward, src/neuralnet/layer.cpp:32) run on the device.
// Numerics are those of matmul_mp (src/core/opsmp.cpp:460-558), the reference's scalar back-end:
//   Float32: c = 0; for k in order: c = fl(c + fl(a[m,k] * b[k,n]))   (fp32, unfused, k ascending;
//            the reference's 64-wide k blocks store and reload the fp32 partial, which is the same)
//   other dtypes: products and sum in double, one cast at the end.
// Every output element is accumulated by one thread with k ascending, so results are bit-identical
// to matmul_mp.  This is a correctness-first kernel (shared-memory tiles, fp32 FMA pipe unused by
// design: the contract forbids fused multiply-adds); a tensor-core GEMM would be a different
// numerical contract and is out of scope here.
#include "ctb_common.cuh"
#include "ctb_math.cuh"

namespace ctb {

namespace {

struct MatmulArgs {
    int64_t M, N, K;
    int64_t a_m, a_k, a_batch;       // element strides
    int64_t b_k, b_n, b_batch;
};

constexpr int kTile = 64;            // output tile edge
constexpr int kTileK = 16;
constexpr int kMicro = 4;            // each of 16 x 16 threads owns a 4 x 4 block of the tile

__global__ void __launch_bounds__(256)
matmul_f32_kernel(const float* __restrict__ a, const float* __restrict__ b, float* __restrict__ c, MatmulArgs g) {
    __shared__ float sa[kTileK][kTile + 1];      // sa[k][m]
    __shared__ float sb[kTileK][kTile + 1];      // sb[k][n]
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    const int64_t m0 = (int64_t)blockIdx.y * kTile, n0 = (int64_t)blockIdx.x * kTile;
    const float* ab = a + (int64_t)blockIdx.z * g.a_batch;
    const float* bb = b + (int64_t)blockIdx.z * g.b_batch;
    float* cb = c + (int64_t)blockIdx.z * g.M * g.N;
    float acc[kMicro][kMicro];
#pragma unroll
    for (int i = 0; i < kMicro; ++i)
#pragma unroll
        for (int j = 0; j < kMicro; ++j) acc[i][j] = 0.0f;
    const bool a_walks_m = g.a_k != 1 && g.a_m == 1, b_walks_k = g.b_n != 1 && g.b_k == 1;
    for (int64_t k0 = 0; k0 < g.K; k0 += kTileK) {
        // 64 x 16 elements of A and 16 x 64 of B, four per thread each; zero beyond the edges
        // (the zero products leave the in-range sums unchanged)
        // Consecutive threads walk the operand's contiguous dim, whichever it is: k for a row-major
        // A, m for a transposed view of one (what the backward pass of a product multiplies by);
        // n for a row-major B, k for a transposed view (the weight of a Linear layer).  The order
        // of the sum over k does not depend on it.
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            const int e = threadIdx.x + r * 256;
            const int am = a_walks_m ? (e & 63) : (e >> 4), ak = a_walks_m ? (e >> 6) : (e & 15);
            const int64_t m = m0 + am, k = k0 + ak;
            sa[ak][am] = (m < g.M && k < g.K) ? ab[m * g.a_m + k * g.a_k] : 0.0f;
            const int bk = b_walks_k ? (e & 15) : (e >> 6), bn = b_walks_k ? (e >> 4) : (e & 63);
            const int64_t kk = k0 + bk, n = n0 + bn;
            sb[bk][bn] = (kk < g.K && n < g.N) ? bb[kk * g.b_k + n * g.b_n] : 0.0f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < kTileK; ++kk) {
            float av[kMicro], bv[kMicro];
#pragma unroll
            for (int i = 0; i < kMicro; ++i) av[i] = sa[kk][ty * kMicro + i];
#pragma unroll
            for (int j = 0; j < kMicro; ++j) bv[j] = sb[kk][tx * kMicro + j];
#pragma unroll
            for (int i = 0; i < kMicro; ++i)
#pragma unroll
                for (int j = 0; j < kMicro; ++j) acc[i][j] = __fadd_rn(acc[i][j], __fmul_rn(av[i], bv[j]));
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < kMicro; ++i) {
        const int64_t m = m0 + ty * kMicro + i;
        if (m >= g.M) continue;
#pragma unroll
        for (int j = 0; j < kMicro; ++j) {
            const int64_t n = n0 + tx * kMicro + j;
            if (n < g.N) cb[m * g.N + n] = acc[i][j];
        }
    }
}

// The generic fallback of matmul_mp (:536-554): double products, double sum, one cast.
template <typename T>
__global__ void __launch_bounds__(256)
matmul_generic_kernel(const T* __restrict__ a, const T* __restrict__ b, T* __restrict__ c, MatmulArgs g, int64_t batch) {
    const int64_t total = batch * g.M * g.N;
    const int64_t step = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += step) {
        const int64_t bi = i / (g.M * g.N), r = i - bi * g.M * g.N;
        const int64_t m = r / g.N, n = r - m * g.N;
        const T* pa = a + bi * g.a_batch + m * g.a_m;
        const T* pb = b + bi * g.b_batch + n * g.b_n;
        double sum = 0.0;
        for (int64_t k = 0; k < g.K; ++k)
            sum = __dadd_rn(sum, __dmul_rn(to_double(pa[k * g.a_k]), to_double(pb[k * g.b_k])));
        c[i] = from_double<T>(sum);
    }
}

}  // namespace

int launch_matmul(int dtype, const void* a, const void* b, void* c, int64_t batch, int64_t M, int64_t N, int64_t K,
                  int64_t a_m, int64_t a_k, int64_t a_batch, int64_t b_k, int64_t b_n, int64_t b_batch,
                  cudaStream_t st) {
    if (batch * M * N == 0) return CTB_OK;
    MatmulArgs g{M, N, K, a_m, a_k, a_batch, b_k, b_n, b_batch};
    if (dtype == CTB_F32) {
        const int64_t gx = ceil_div(N, kTile), gy = ceil_div(M, kTile);
        if (gx > 0x7FFFFFFFll || gy > 65535 || batch > 65535)
            return set_error(CTB_ERR_LIMIT, "matmul: shape too large for one launch");
        dim3 grid((unsigned)gx, (unsigned)gy, (unsigned)batch);
        matmul_f32_kernel<<<grid, 256, 0, st>>>((const float*)a, (const float*)b, (float*)c, g);
    } else {
        int64_t blocks = ceil_div(batch * M * N, 256);
        if (blocks > 0x7FFFFFFFll) blocks = 0x7FFFFFFFll;
        if (dtype == CTB_F64)
            matmul_generic_kernel<double><<<(unsigned)blocks, 256, 0, st>>>((const double*)a, (const double*)b, (double*)c, g, batch);
        else if (dtype == CTB_I32)
            matmul_generic_kernel<int32_t><<<(unsigned)blocks, 256, 0, st>>>((const int32_t*)a, (const int32_t*)b, (int32_t*)c, g, batch);
        else
            return set_error(CTB_ERR_DTYPE, "matmul: unsupported dtype");
    }
    return cuda_error(cudaGetLastError(), "matmul launch");
}

}  // namespace ctb
