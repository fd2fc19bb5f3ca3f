// Host-visible interface of the backward-body and cross-entropy kernels (ctb_backward.cu).
#pragma once
#include "ctb_common.cuh"

namespace ctb {

enum { kBwdDivA = 0, kBwdDivB = 1, kBwdTanh = 2 };

// Iteration space of a backward chain: the (collapsed) shape of the result with element strides
// for the incoming gradient, the two forward operands and the output.  `flat` = every operand
// present is contiguous over that shape.
struct BwdPlan {
    int32_t ndim;
    int32_t flat;
    int64_t numel;
    int64_t shape[CTB_MAX_DIMS];
    int64_t stride[4][CTB_MAX_DIMS];      // g, x, y, out
};

// out = chain(g, x, y), or out += chain(...) (finite values only) when `accumulate`.
// kBwdDivA uses (g, y = b); kBwdDivB (g, x = a, y = b); kBwdTanh (g, x = t).
int launch_backward_chain(int kind, int dtype, const BwdPlan& p, const void* g, const void* x, const void* y,
                          void* out, int accumulate, cudaStream_t stream);

// Both outputs of the division's backward step for contiguous same-shape operands of n elements.
int launch_div_backward_both(int dtype, int64_t n, const void* g, const void* a, const void* b, void* da, void* db,
                             int accumulate, cudaStream_t stream);

// nll[row] for x[rows, classes] (row stride in elements, classes contiguous), labels[row * label_stride].
int launch_ce_forward_rows(const float* x, int64_t row_stride, const int32_t* labels, int64_t label_stride,
                           int64_t rows, int64_t classes, float* nll, int32_t* bad, cudaStream_t stream);
int launch_ce_backward_rows(const float* x, int64_t row_stride, const int32_t* labels, int64_t label_stride,
                            int64_t rows, int64_t classes, float scale, float* dx, int64_t dx_stride,
                            int accumulate, int32_t* bad, cudaStream_t stream);

// The same two passes with the row held in registers (ctb_rows.cu), for rows of up to 16384 classes (gradient: 32768):
// mode 0 writes nll[rows] to `out`, 1 writes the gradient rows, 2 adds them into `out`.  False:
// nothing was launched (the row is too long).
bool launch_ce_rows_registers(int mode, const float* x, int64_t row_stride, const int32_t* labels, int64_t label_stride,
                              int64_t rows, int64_t classes, float scale, float* out, int64_t out_stride, int32_t* bad,
                              cudaStream_t stream);

}  // namespace ctb
