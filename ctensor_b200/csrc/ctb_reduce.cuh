// Host-visible interface of the reduction and fused-row kernels (ctb_reduce.cu, ctb_rows.cu).
#pragma once
#include "ctb_common.cuh"

namespace ctb {

// A strided input seen by a reduction: `outer` dims index the outputs, one `reduce` dim
// (length rlen, stride rstride) is folded.  A full reduction of a dense buffer is planned as
// outer = {}, rlen = numel, rstride = 1.
struct ReduceGeom {
    int32_t nouter;
    int64_t oshape[CTB_MAX_DIMS];
    int64_t ostride[CTB_MAX_DIMS];
    int64_t nout;        // product of oshape (1 when nouter == 0)
    int64_t rlen;
    int64_t rstride;
    int64_t total;       // element count that "mean"/"var" divide by (== rlen)
};

// Split reductions keep their tickets (uint32 counters, zero between launches) in the first
// kTicketBytes of the scratch buffer; nothing else may be written there.
// Internal reduction operator (not part of the public enum): out[i] += (T)sum unless the sum is
// NaN or infinite — reduction and accumulation of accumulate_grad (src/core/autograd.cpp:84-151)
// in one kernel.
constexpr int kOpSumAccumulate = CTB_REDUCE_OP_COUNT;

constexpr int kTicketSlots = 16384;
constexpr size_t kTicketBytes = kTicketSlots * sizeof(uint32_t);

// Bytes of scratch the chosen kernel shape needs for this geometry (0 when none).
size_t reduce_workspace_bytes(const ReduceGeom& g, int dtype);

// Launch the reduction.  `out` is T (or int32 for argmax); `partial_out` (may be null) asks for
// the raw fp64 accumulator instead of the finalised T (full reductions only, used by the
// multi-GPU path).  `ws` must hold reduce_workspace_bytes() bytes, zero-initialised once at
// allocation (the kernels leave their tickets at zero again).
int launch_reduce(int op, int dtype, const ReduceGeom& g, const void* a, void* out,
                  double* partial_out, void* ws, size_t ws_bytes, cudaStream_t stream);

// The same launch with scratch taken from the library's fixed device array (no allocation).
// Fails with CTB_ERR_LIMIT when the geometry needs more than CTB_NOALLOC_SCRATCH_BYTES.
int launch_reduce_static_scratch(int op, int dtype, const ReduceGeom& g, const void* a, void* out,
                                 cudaStream_t stream);

int launch_finalize_full(int op, int dtype, const double* partial, int64_t total, void* out,
                         cudaStream_t stream);

// Fused rows (fp32).  x: [outer..., cols] with inner stride 1; mask (optional): same outer dims
// with broadcast strides, inner stride 0 or 1.
struct RowsGeom {
    int32_t nouter;
    int64_t oshape[CTB_MAX_DIMS];
    int64_t xstride[CTB_MAX_DIMS];
    int64_t mstride[CTB_MAX_DIMS];
    int64_t rows;
    int64_t cols;
    int64_t qlen;        // size of the second-to-last dim (row index within it drives `causal`)
    int32_t m_inner;     // mask inner stride (0 or 1)
    int32_t has_mask;
};
int launch_softmax(const RowsGeom& g, const float* x, const float* mask, int causal, int log_out, float* out,
                   cudaStream_t stream);
int launch_layernorm(const RowsGeom& g, const float* x, const float* gamma, int64_t gstride,
                     const float* beta, int64_t bstride, double eps, float* out,
                     cudaStream_t stream);

// BatchNorm forward pieces for a contiguous fp32 x[N, C, S] (ctb_norm.cu).
size_t channel_moments_workspace_bytes(int64_t C, int sm_count);
int launch_channel_moments(const float* x, float* mean, float* var, int64_t N, int64_t C, int64_t S,
                           void* ws, size_t ws_bytes, cudaStream_t stream);
int launch_batchnorm_apply(const float* x, const float* mean, int64_t mstride, const float* var, int64_t vstride,
                           const float* gamma, int64_t gstride, const float* beta, int64_t bstride, double eps,
                           float* rstd_scratch, float* out, int64_t N, int64_t C, int64_t S, cudaStream_t stream);

}  // namespace ctb
