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

Tensor add_mp(const Tensor& a, const Tensor& b);
Tensor diff_mp(const Tensor& a, const Tensor& b);
Tensor mult_mp(const Tensor& a, const Tensor& b);
Tensor div_mp(const Tensor& a, const Tensor& b);
Tensor pow_mp(const Tensor& a, const Tensor& b);
Tensor matmul_mp(const Tensor& A, const Tensor& B);

Tensor add_scalar_mp(const Tensor& a, double scalar);
Tensor sub_scalar_mp(const Tensor& a, double scalar);
Tensor sub_afterscalar_mp(double scalar, const Tensor& a);
Tensor mult_scalar_mp(const Tensor& a, double scalar);
Tensor div_scalar_mp(const Tensor& a, double scalar);
Tensor scalar_div_mp(double scalar, const Tensor& a);
Tensor pow_scalar_mp(const Tensor& a, double scalar);
Tensor scalar_pow_mp(double scalar, const Tensor& a);

Tensor abs_mp(const Tensor& a);
Tensor ln_mp(const Tensor& a);
Tensor exp_mp(const Tensor& a);
Tensor sqrt_mp(const Tensor& a);
Tensor sin_mp(const Tensor& a);
Tensor asin_mp(const Tensor& a);
Tensor cos_mp(const Tensor& a);
Tensor acos_mp(const Tensor& a);
Tensor tan_mp(const Tensor& a);
Tensor atan_mp(const Tensor& a);
Tensor tanh_mp(const Tensor& a);
Tensor sinh_mp(const Tensor& a);
Tensor cosh_mp(const Tensor& a);
Tensor sigmoid_mp(const Tensor& a);
Tensor Relu_mp(const Tensor& a);
Tensor softplus_mp(const Tensor& a);

Tensor sum_mp(const Tensor& t, int dim = -1);
Tensor mean_mp(const Tensor& t, int dim = -1);
Tensor max_mp(const Tensor& t, int dim = -1);
Tensor min_mp(const Tensor& t, int dim = -1);

Tensor lt_mp(const Tensor& a, double b);
Tensor le_mp(const Tensor& a, double b);
Tensor gt_mp(const Tensor& a, double b);
Tensor ge_mp(const Tensor& a, double b);
Tensor eq_mp(const Tensor& a, double b);
Tensor neq_mp(const Tensor& a, double b);
Tensor lt_mp(const Tensor& a, const Tensor& b);
Tensor le_mp(const Tensor& a, const Tensor& b);
Tensor gt_mp(const Tensor& a, const Tensor& b);
Tensor ge_mp(const Tensor& a, const Tensor& b);
Tensor eq_mp(const Tensor& a, const Tensor& b);
Tensor ne_mp(const Tensor& a, const Tensor& b);

Tensor cat_mp(const std::vector<Tensor>& tensors, size_t dim);

inline Tensor operator+(const Tensor& a, const Tensor& b) { return add_mp(a, b); }
inline Tensor operator+(const Tensor& a, double s) { return add_scalar_mp(a, s); }
inline Tensor operator+(double s, const Tensor& a) { return add_scalar_mp(a, s); }
inline Tensor operator-(const Tensor& a, const Tensor& b) { return diff_mp(a, b); }
inline Tensor operator-(const Tensor& a, double s) { return sub_scalar_mp(a, s); }
inline Tensor operator-(double s, const Tensor& a) { return sub_afterscalar_mp(s, a); }
inline Tensor operator-(const Tensor& a) { return mult_scalar_mp(a, -1.0); }
inline Tensor operator*(const Tensor& a, const Tensor& b) { return mult_mp(a, b); }
inline Tensor operator*(const Tensor& a, double s) { return mult_scalar_mp(a, s); }
inline Tensor operator*(double s, const Tensor& a) { return mult_scalar_mp(a, s); }
inline Tensor operator/(const Tensor& a, const Tensor& b) { return div_mp(a, b); }
inline Tensor operator/(const Tensor& a, double s) { return div_scalar_mp(a, s); }
inline Tensor operator/(double s, const Tensor& a) { return scalar_div_mp(s, a); }
inline Tensor operator^(const Tensor& a, const Tensor& b) { return pow_mp(a, b); }
inline Tensor operator^(const Tensor& a, double s) { return pow_scalar_mp(a, s); }
inline Tensor operator^(double s, const Tensor& a) { return scalar_pow_mp(s, a); }

inline Tensor& operator+=(Tensor& a, const Tensor& b) { a = add_mp(a, b); return a; }
inline Tensor& operator+=(Tensor& a, double s) { a = add_scalar_mp(a, s); return a; }
inline Tensor& operator-=(Tensor& a, const Tensor& b) { a = diff_mp(a, b); return a; }
inline Tensor& operator-=(Tensor& a, double s) { a = sub_scalar_mp(a, s); return a; }
inline Tensor& operator*=(Tensor& a, const Tensor& b) { a = mult_mp(a, b); return a; }
inline Tensor& operator*=(Tensor& a, double s) { a = mult_scalar_mp(a, s); return a; }
inline Tensor& operator/=(Tensor& a, const Tensor& b) { a = div_mp(a, b); return a; }
inline Tensor& operator/=(Tensor& a, double s) { a = div_scalar_mp(a, s); return a; }
inline Tensor& operator^=(Tensor& a, const Tensor& b) { a = pow_mp(a, b); return a; }
inline Tensor& operator^=(Tensor& a, double s) { a = pow_scalar_mp(a, s); return a; }

inline Tensor operator<(const Tensor& a, double b) { return lt_mp(a, b); }
inline Tensor operator<=(const Tensor& a, double b) { return le_mp(a, b); }
inline Tensor operator>(const Tensor& a, double b) { return gt_mp(a, b); }
inline Tensor operator>=(const Tensor& a, double b) { return ge_mp(a, b); }
inline Tensor operator==(const Tensor& a, double b) { return eq_mp(a, b); }
inline Tensor operator!=(const Tensor& a, double b) { return neq_mp(a, b); }
inline Tensor operator<(const Tensor& a, const Tensor& b) { return lt_mp(a, b); }
inline Tensor operator<=(const Tensor& a, const Tensor& b) { return le_mp(a, b); }
inline Tensor operator>(const Tensor& a, const Tensor& b) { return gt_mp(a, b); }
inline Tensor operator>=(const Tensor& a, const Tensor& b) { return ge_mp(a, b); }
inline Tensor operator==(const Tensor& a, const Tensor& b) { return eq_mp(a, b); }
inline Tensor operator!=(const Tensor& a, const Tensor& b) { return ne_mp(a, b); }
