// Operator API of the B200 library: the free functions callers of the reference use
// (src/core/ops_dispatch.h:10-104 there), same names, argument meaning, result shapes and
// error texts.  Every function forwards to the C ABI (include/ctb200.h); none computes on the
// host.  Results are fresh contiguous tensors; `requires_grad` propagates and a grad node is
// attached through ctb_host::set_grad_factory (ctb_host.h) when the caller's autograd library
// registered one.
#pragma once
#include <vector>
#include "tensor.h"

// binary, NumPy-style broadcasting
Tensor add(const Tensor& a, const Tensor& b);
Tensor sub(const Tensor& a, const Tensor& b);
Tensor mul(const Tensor& a, const Tensor& b);
Tensor div(const Tensor& a, const Tensor& b);
Tensor pow(const Tensor& a, const Tensor& b);

// tensor (op) scalar: evaluated in double, rounded once to the tensor's dtype
Tensor add_scalar(const Tensor& a, double scalar);
Tensor sub_scalar(const Tensor& a, double scalar);
Tensor sub_scalar_rev(double scalar, const Tensor& a);
Tensor mul_scalar(const Tensor& a, double scalar);
Tensor div_scalar(const Tensor& a, double scalar);
Tensor div_scalar_rev(double scalar, const Tensor& a);
Tensor pow_scalar(const Tensor& a, double scalar);
Tensor pow_scalar_rev(double scalar, const Tensor& a);

// comparisons: 1/0 in the dtype of `a`
Tensor lt(const Tensor& a, const Tensor& b);
Tensor le(const Tensor& a, const Tensor& b);
Tensor gt(const Tensor& a, const Tensor& b);
Tensor ge(const Tensor& a, const Tensor& b);
Tensor eq(const Tensor& a, const Tensor& b);
Tensor ne(const Tensor& a, const Tensor& b);
Tensor lt(const Tensor& a, double b);
Tensor le(const Tensor& a, double b);
Tensor gt(const Tensor& a, double b);
Tensor ge(const Tensor& a, double b);
Tensor eq(const Tensor& a, double b);
Tensor ne(const Tensor& a, double b);

// unary
Tensor abs(const Tensor& a);
Tensor log(const Tensor& a);
Tensor ln(const Tensor& a);
Tensor exp(const Tensor& a);
Tensor sqrt(const Tensor& a);
Tensor sin(const Tensor& a);
Tensor cos(const Tensor& a);
Tensor tan(const Tensor& a);
Tensor asin(const Tensor& a);
Tensor acos(const Tensor& a);
Tensor atan(const Tensor& a);
Tensor sinh(const Tensor& a);
Tensor cosh(const Tensor& a);
Tensor softplus(const Tensor& a);
Tensor tanh(const Tensor& a);
Tensor sigmoid(const Tensor& a);
Tensor relu(const Tensor& a);
Tensor gelu(const Tensor& a);                       // tanh form; not in the reference

// reductions; dim = -1 reduces everything to shape {1}
Tensor sum(const Tensor& a, int dim = -1);
Tensor mean(const Tensor& a, int dim = -1);
Tensor max(const Tensor& a, int dim = -1);
Tensor min(const Tensor& a, int dim = -1);
Tensor var(const Tensor& a, int dim = -1);          // biased; not in the reference
Tensor argmax(const Tensor& a, int dim);

// fused rows over the last dim (not in the reference; the chains its modules spell out)
Tensor softmax(const Tensor& a);
Tensor softmax(const Tensor& a, const Tensor& additive_mask);
Tensor causal_softmax(const Tensor& a);
Tensor log_softmax(const Tensor& a);                 // the chain inside Loss::CrossEntropy

Tensor cat(const std::vector<Tensor>& tensors, size_t dim);
Tensor matmul(const Tensor& a, const Tensor& b);     // the arithmetic of matmul_mp (fp32, k ascending)

// BatchNorm::forward of the reference in two calls (its statistics block and its normalisation
// block): x is a contiguous Float32 [N, C, ...]; mean/var/gamma/beta hold C elements.
void channel_moments(const Tensor& x, Tensor& mean, Tensor& var);
Tensor batch_norm_apply(const Tensor& x, const Tensor& mean, const Tensor& var, const Tensor& gamma,
                        const Tensor& beta, double eps = 1e-5);
Tensor layer_norm(const Tensor& a, const Tensor& gamma, const Tensor& beta, double eps = 1e-5);

// operators
inline Tensor operator+(const Tensor& a, const Tensor& b) { return add(a, b); }
inline Tensor operator+(const Tensor& a, double s) { return add_scalar(a, s); }
inline Tensor operator+(double s, const Tensor& a) { return add_scalar(a, s); }
inline Tensor operator-(const Tensor& a, const Tensor& b) { return sub(a, b); }
inline Tensor operator-(const Tensor& a, double s) { return sub_scalar(a, s); }
inline Tensor operator-(double s, const Tensor& a) { return sub_scalar_rev(s, a); }
inline Tensor operator-(const Tensor& a) { return mul_scalar(a, -1.0); }
inline Tensor operator*(const Tensor& a, const Tensor& b) { return mul(a, b); }
inline Tensor operator*(const Tensor& a, double s) { return mul_scalar(a, s); }
inline Tensor operator*(double s, const Tensor& a) { return mul_scalar(a, s); }
inline Tensor operator/(const Tensor& a, const Tensor& b) { return div(a, b); }
// The reference's header routes Tensor / double to sub_scalar (src/core/ops_dispatch.h:84, a typo
// there) and callers are compiled against it: the input gradient of its BatchNorm
// (src/neuralnet/batchnorm/batchnorm.cpp:186, `inv_std / M`) is what that typo makes of it.  A
// drop-in gives the callers the numbers they get from the reference, so the operator does the same
// here; define CTB_SCALAR_DIVISION_DIVIDES to get a division (div_scalar is the named function
// for it either way).
#ifdef CTB_SCALAR_DIVISION_DIVIDES
inline Tensor operator/(const Tensor& a, double s) { return div_scalar(a, s); }
#else
inline Tensor operator/(const Tensor& a, double s) { return sub_scalar(a, s); }
#endif
inline Tensor operator/(double s, const Tensor& a) { return div_scalar_rev(s, a); }
inline Tensor operator^(const Tensor& a, const Tensor& b) { return pow(a, b); }
inline Tensor operator^(const Tensor& a, double s) { return pow_scalar(a, s); }
inline Tensor operator^(double s, const Tensor& a) { return pow_scalar_rev(s, a); }

inline Tensor& operator+=(Tensor& a, const Tensor& b) { a = add(a, b); return a; }
inline Tensor& operator+=(Tensor& a, double s) { a = add_scalar(a, s); return a; }
inline Tensor& operator-=(Tensor& a, const Tensor& b) { a = sub(a, b); return a; }
inline Tensor& operator-=(Tensor& a, double s) { a = sub_scalar(a, s); return a; }
inline Tensor& operator*=(Tensor& a, const Tensor& b) { a = mul(a, b); return a; }
inline Tensor& operator*=(Tensor& a, double s) { a = mul_scalar(a, s); return a; }
inline Tensor& operator/=(Tensor& a, const Tensor& b) { a = div(a, b); return a; }
inline Tensor& operator/=(Tensor& a, double s) { a = div_scalar(a, s); return a; }

inline Tensor operator<(const Tensor& a, double b) { return lt(a, b); }
inline Tensor operator<=(const Tensor& a, double b) { return le(a, b); }
inline Tensor operator>(const Tensor& a, double b) { return gt(a, b); }
inline Tensor operator>=(const Tensor& a, double b) { return ge(a, b); }
inline Tensor operator==(const Tensor& a, double b) { return eq(a, b); }
inline Tensor operator!=(const Tensor& a, double b) { return ne(a, b); }
inline Tensor operator<(const Tensor& a, const Tensor& b) { return lt(a, b); }
inline Tensor operator<=(const Tensor& a, const Tensor& b) { return le(a, b); }
inline Tensor operator>(const Tensor& a, const Tensor& b) { return gt(a, b); }
inline Tensor operator>=(const Tensor& a, const Tensor& b) { return ge(a, b); }
inline Tensor operator==(const Tensor& a, const Tensor& b) { return eq(a, b); }
inline Tensor operator!=(const Tensor& a, const Tensor& b) { return ne(a, b); }
