// Index-driven kernels next to the operator path: gather along a dim (Tensor::gather,
// src/core/tensor.cpp:344-428 of the reference) and the strided in-place accumulation that
// accumulate_grad ends with (src/core/autograd.cpp:116-155).
#include "ctb_common.cuh"
#include "ctb_math.cuh"

namespace ctb {

namespace {

struct GatherIdx {
    DimSet dims;                          // the index tensor's shape (= the output's)
    int64_t stride[2][CTB_MAX_DIMS];      // [0] = x (0 at the gather dim), [1] = index tensor
    int64_t numel;
    int64_t gstride;                      // x's stride along the gather dim
    int64_t gsize;                        // x's extent along the gather dim
};

// The index tensor may hold any dtype: the reference reads it through double and truncates
// (src/core/tensor.cpp:385-386; first generation: tensor1.cpp:548-549).
__device__ __forceinline__ int64_t load_index(const void* p, int64_t off, int dtype) {
    switch (dtype) {
    case CTB_I32: return ((const int32_t*)p)[off];
    case CTB_I64: return ((const int64_t*)p)[off];
    case CTB_F32: return (int64_t)((const float*)p)[off];
    case CTB_F64: return (int64_t)((const double*)p)[off];
    case CTB_U8: case CTB_BOOL: return ((const uint8_t*)p)[off];
    case CTB_I8: return ((const int8_t*)p)[off];
    case CTB_U16: return ((const uint16_t*)p)[off];
    case CTB_I16: return ((const int16_t*)p)[off];
    case CTB_U32: return ((const uint32_t*)p)[off];
    default: return (int64_t)((const unsigned long long*)p)[off];          // CTB_U64
    }
}

// One output element per thread.  T is an unsigned integer of the element's size: the value is
// moved, not converted (the reference's read_scalar_at/write_scalar_at round trip through
// double is the identity for every dtype it stores).
template <typename T>
__global__ void __launch_bounds__(256)
gather_kernel(const T* __restrict__ x, const void* __restrict__ index, int index_dtype, T* __restrict__ out, GatherIdx g,
              int32_t* bad) {
    const int64_t step = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < g.numel; i += step) {
        int64_t off[2] = {0, 0};
        dimset_offsets<2>(g.dims, i, g.stride, off);
        int64_t idx = load_index(index, off[1], index_dtype);
        if (idx < 0) idx += g.gsize;                        // Python-style negative index
        T v = 0;
        if (idx < 0 || idx >= g.gsize) {
            if (bad) *bad = 1;                              // every writer stores the same value
        } else {
            v = x[off[0] + idx * g.gstride];
        }
        out[i] = v;
    }
}

struct AccIdx {
    DimSet dims;                          // the target's shape
    int64_t stride[2][CTB_MAX_DIMS];      // [0] = grad buffer, [1] = source (0 where it broadcasts)
    int64_t numel;
};

// grad[i] = (T)((double)grad[i] + (double)src[i]) unless src[i] is NaN or infinite
// (src/core/autograd.cpp:139-151), for any strides on either side.
template <typename T>
__global__ void __launch_bounds__(256)
accumulate_strided_kernel(T* __restrict__ grad, const T* __restrict__ src, AccIdx g) {
    const int64_t step = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < g.numel; i += step) {
        int64_t off[2] = {0, 0};
        dimset_offsets<2>(g.dims, i, g.stride, off);
        grad[off[0]] = BinaryFn<kOpAddFinite, T>::apply(grad[off[0]], src[off[1]]);
    }
}

unsigned grid_for(int64_t n) {
    int64_t blocks = ceil_div(n, 256);
    if (blocks > 0x7FFFFFFFll) blocks = 0x7FFFFFFFll;
    return (unsigned)(blocks < 1 ? 1 : blocks);
}

}  // namespace

int launch_gather(int elem_bytes, int ndim, const int64_t* ishape, const int64_t* xstride, const int64_t* istride,
                  int dim, int64_t gsize, const void* x, const void* index, int index_dtype, void* out, int32_t* bad,
                  cudaStream_t st) {
    GatherIdx g{};
    dimset_init(&g.dims, ndim, ishape);
    g.numel = 1;
    for (int d = 0; d < ndim; ++d) {
        g.numel *= ishape[d];
        g.stride[0][d] = d == dim ? 0 : xstride[d];
        g.stride[1][d] = istride[d];
    }
    g.gstride = xstride[dim];
    g.gsize = gsize;
    if (g.numel == 0) return CTB_OK;
    const unsigned grid = grid_for(g.numel);
    switch (elem_bytes) {
    case 8: gather_kernel<unsigned long long><<<grid, 256, 0, st>>>((const unsigned long long*)x, index, index_dtype, (unsigned long long*)out, g, bad); break;
    case 4: gather_kernel<uint32_t><<<grid, 256, 0, st>>>((const uint32_t*)x, index, index_dtype, (uint32_t*)out, g, bad); break;
    case 2: gather_kernel<uint16_t><<<grid, 256, 0, st>>>((const uint16_t*)x, index, index_dtype, (uint16_t*)out, g, bad); break;
    case 1: gather_kernel<uint8_t><<<grid, 256, 0, st>>>((const uint8_t*)x, index, index_dtype, (uint8_t*)out, g, bad); break;
    default: return set_error(CTB_ERR_DTYPE, "gather: unsupported element size");
    }
    return cuda_error(cudaGetLastError(), "gather launch");
}

int launch_accumulate_strided(int dtype, int ndim, const int64_t* shape, const int64_t* gstride,
                              const int64_t* sstride, void* grad, const void* src, cudaStream_t st) {
    AccIdx g{};
    dimset_init(&g.dims, ndim, shape);
    g.numel = 1;
    for (int d = 0; d < ndim; ++d) {
        g.numel *= shape[d];
        g.stride[0][d] = gstride[d];
        g.stride[1][d] = sstride[d];
    }
    if (g.numel == 0) return CTB_OK;
    switch (dtype) {
    case CTB_F32: accumulate_strided_kernel<float><<<grid_for(g.numel), 256, 0, st>>>((float*)grad, (const float*)src, g); break;
    case CTB_I32: accumulate_strided_kernel<int32_t><<<grid_for(g.numel), 256, 0, st>>>((int32_t*)grad, (const int32_t*)src, g); break;
    case CTB_F64: accumulate_strided_kernel<double><<<grid_for(g.numel), 256, 0, st>>>((double*)grad, (const double*)src, g); break;
    default: return set_error(CTB_ERR_DTYPE, "accumulate_grad: unsupported dtype");
    }
    return cuda_error(cudaGetLastError(), "accumulate launch");
}

}  // namespace ctb
