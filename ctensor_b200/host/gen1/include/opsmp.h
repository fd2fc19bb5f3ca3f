// First-generation operator names of the reference (root opsmp.h:30-127): the `*_mp` functions
// and the operators its callers use (autograd.cpp: sum_mp, exp_mp, tanh_mp, gt_mp ...;
// loss.cpp: sum_mp, ln_mp, exp_mp, max_mp ...; layer.cpp: matmul_mp, operator+).  Same names,
// argument meaning, result shapes and error texts; every function runs a kernel of the B200
// operator library (include/ctb200.h) — none computes on the host.
//
// Semantics kept from the reference's opsmp.cpp: results are fresh contiguous tensors with the
// dtype of the first operand; requires_grad propagates and the result gets the backward node the
// reference would attach (through ctb_gen1::set_grad_factory); reductions read dim = -1 as the
// LAST dim and drop the reduced dim; mean_mp is sum_mp followed by mult_scalar_mp (two nodes);
// max_mp / min_mp / comparisons attach no node.
#pragma once
#include <vector>
#include "tensor1.h"

// The names are kept in lists (one list per signature) that expand to the declarations and, further
// down, to the operator overloads that forward to them.

// Tensor f(const Tensor&, const Tensor&)
#define CTB_GEN1_TENSOR_TENSOR(X) \
    X(add_mp) X(diff_mp) X(mult_mp) X(div_mp) X(pow_mp) X(matmul_mp) \
    X(lt_mp) X(le_mp) X(gt_mp) X(ge_mp) X(eq_mp) X(ne_mp)
// Tensor f(const Tensor&, double)
#define CTB_GEN1_TENSOR_SCALAR(X) \
    X(add_scalar_mp) X(sub_scalar_mp) X(mult_scalar_mp) X(div_scalar_mp) X(pow_scalar_mp) \
    X(lt_mp) X(le_mp) X(gt_mp) X(ge_mp) X(eq_mp) X(neq_mp)
// Tensor f(double, const Tensor&)
#define CTB_GEN1_SCALAR_TENSOR(X) X(sub_afterscalar_mp) X(scalar_div_mp) X(scalar_pow_mp)
// Tensor f(const Tensor&)
#define CTB_GEN1_UNARY(X) \
    X(abs_mp) X(ln_mp) X(exp_mp) X(sqrt_mp) X(sin_mp) X(asin_mp) X(cos_mp) X(acos_mp) X(tan_mp) X(atan_mp) \
    X(tanh_mp) X(sinh_mp) X(cosh_mp) X(sigmoid_mp) X(Relu_mp) X(softplus_mp)
// Tensor f(const Tensor&, int dim = -1): -1 is the last dim
#define CTB_GEN1_REDUCTIONS(X) X(sum_mp) X(mean_mp) X(max_mp) X(min_mp)

#define CTB_X(name) Tensor name(const Tensor& a, const Tensor& b);
CTB_GEN1_TENSOR_TENSOR(CTB_X)
#undef CTB_X
#define CTB_X(name) Tensor name(const Tensor& a, double scalar);
CTB_GEN1_TENSOR_SCALAR(CTB_X)
#undef CTB_X
#define CTB_X(name) Tensor name(double scalar, const Tensor& a);
CTB_GEN1_SCALAR_TENSOR(CTB_X)
#undef CTB_X
#define CTB_X(name) Tensor name(const Tensor& a);
CTB_GEN1_UNARY(CTB_X)
#undef CTB_X
#define CTB_X(name) Tensor name(const Tensor& t, int dim = -1);
CTB_GEN1_REDUCTIONS(CTB_X)
#undef CTB_X
Tensor cat_mp(const std::vector<Tensor>& tensors, size_t dim);

// ---- operators: symbol, tensor-tensor function, tensor-scalar function, scalar-tensor function -------------
#define CTB_GEN1_ARITHMETIC(X)                                          \
    X(+, add_mp, add_scalar_mp(a, s), add_scalar_mp(a, s))               \
    X(-, diff_mp, sub_scalar_mp(a, s), sub_afterscalar_mp(s, a))         \
    X(*, mult_mp, mult_scalar_mp(a, s), mult_scalar_mp(a, s))            \
    X(/, div_mp, div_scalar_mp(a, s), scalar_div_mp(s, a))               \
    X(^, pow_mp, pow_scalar_mp(a, s), scalar_pow_mp(s, a))
#define CTB_X(op, tt, ts, st)                                                                     \
    inline Tensor operator op(const Tensor& a, const Tensor& b) { return tt(a, b); }               \
    inline Tensor operator op(const Tensor& a, double s) { return ts; }                            \
    inline Tensor operator op(double s, const Tensor& a) { return st; }                            \
    inline Tensor& operator op##=(Tensor& a, const Tensor& b) { a = tt(a, b); return a; }          \
    inline Tensor& operator op##=(Tensor& a, double s) { a = ts; return a; }
CTB_GEN1_ARITHMETIC(CTB_X)
#undef CTB_X
inline Tensor operator-(const Tensor& a) { return mult_scalar_mp(a, -1.0); }

// comparisons: symbol, tensor-tensor function, tensor-scalar function
#define CTB_GEN1_COMPARISONS(X) X(<, lt_mp, lt_mp) X(<=, le_mp, le_mp) X(>, gt_mp, gt_mp) X(>=, ge_mp, ge_mp) X(==, eq_mp, eq_mp) X(!=, ne_mp, neq_mp)
#define CTB_X(op, tt, ts)                                                                          \
    inline Tensor operator op(const Tensor& a, const Tensor& b) { return tt(a, b); }               \
    inline Tensor operator op(const Tensor& a, double b) { return ts(a, b); }
CTB_GEN1_COMPARISONS(CTB_X)
#undef CTB_X
