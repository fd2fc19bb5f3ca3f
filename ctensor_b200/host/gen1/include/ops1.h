// The sequential operator names of the reference's first generation (root ops1.h:29-85):
// add_, diff_, mult_, div_, Relu_, exp_, ln_, tanh_, sum, mean, max, min ...  On the GPU there is
// one implementation per operator, so these are the `*_mp` operators under their other names.
// As in the reference, include either this header's operators or opsmp.h's in one translation
// unit, not both: the operator overloads live in opsmp.h only.
#pragma once
#include "opsmp.h"

inline Tensor add_(const Tensor& a, const Tensor& b) { return add_mp(a, b); }
inline Tensor add(const Tensor& a, const Tensor& b) { return add_mp(a, b); }
inline Tensor diff_(const Tensor& a, const Tensor& b) { return diff_mp(a, b); }
inline Tensor mult_(const Tensor& a, const Tensor& b) { return mult_mp(a, b); }
inline Tensor div_(const Tensor& a, const Tensor& b) { return div_mp(a, b); }
inline Tensor pow_(const Tensor& a, const Tensor& b) { return pow_mp(a, b); }
inline Tensor matmul_(const Tensor& a, const Tensor& b) { return matmul_mp(a, b); }
inline Tensor add_scalar(const Tensor& a, double s) { return add_scalar_mp(a, s); }
inline Tensor sub_scalar(const Tensor& a, double s) { return sub_scalar_mp(a, s); }
inline Tensor sub_afterscalar(double s, const Tensor& a) { return sub_afterscalar_mp(s, a); }
inline Tensor mult_scalar(const Tensor& a, double s) { return mult_scalar_mp(a, s); }
inline Tensor div_scalar(const Tensor& a, double s) { return div_scalar_mp(a, s); }
inline Tensor scalar_div(double s, const Tensor& a) { return scalar_div_mp(s, a); }
inline Tensor pow_scalar(const Tensor& a, double s) { return pow_scalar_mp(a, s); }
inline Tensor scalar_pow(double s, const Tensor& a) { return scalar_pow_mp(s, a); }
inline Tensor abs_(const Tensor& a) { return abs_mp(a); }
inline Tensor ln_(const Tensor& a) { return ln_mp(a); }
inline Tensor exp_(const Tensor& a) { return exp_mp(a); }
inline Tensor sqrt_(const Tensor& a) { return sqrt_mp(a); }
inline Tensor sin_(const Tensor& a) { return sin_mp(a); }
inline Tensor asin_(const Tensor& a) { return asin_mp(a); }
inline Tensor sinh_(const Tensor& a) { return sinh_mp(a); }
inline Tensor cos_(const Tensor& a) { return cos_mp(a); }
inline Tensor acos_(const Tensor& a) { return acos_mp(a); }
inline Tensor cosh_(const Tensor& a) { return cosh_mp(a); }
inline Tensor tan_(const Tensor& a) { return tan_mp(a); }
inline Tensor atan_(const Tensor& a) { return atan_mp(a); }
inline Tensor tanh_(const Tensor& a) { return tanh_mp(a); }
inline Tensor sigmoid_(const Tensor& a) { return sigmoid_mp(a); }
inline Tensor Relu_(const Tensor& a) { return Relu_mp(a); }
inline Tensor softplus_(const Tensor& a) { return softplus_mp(a); }
inline Tensor sum(const Tensor& t, int dim = -1) { return sum_mp(t, dim); }
inline Tensor mean(const Tensor& t, int dim = -1) { return mean_mp(t, dim); }
inline Tensor max(const Tensor& t, int dim = -1) { return max_mp(t, dim); }
inline Tensor min(const Tensor& t, int dim = -1) { return min_mp(t, dim); }
inline Tensor lt(const Tensor& a, double b) { return lt_mp(a, b); }
inline Tensor le(const Tensor& a, double b) { return le_mp(a, b); }
inline Tensor gt(const Tensor& a, double b) { return gt_mp(a, b); }
inline Tensor ge(const Tensor& a, double b) { return ge_mp(a, b); }
inline Tensor eq(const Tensor& a, double b) { return eq_mp(a, b); }
inline Tensor neq(const Tensor& a, double b) { return neq_mp(a, b); }
inline Tensor lt(const Tensor& a, const Tensor& b) { return lt_mp(a, b); }
inline Tensor le(const Tensor& a, const Tensor& b) { return le_mp(a, b); }
inline Tensor gt(const Tensor& a, const Tensor& b) { return gt_mp(a, b); }
inline Tensor ge(const Tensor& a, const Tensor& b) { return ge_mp(a, b); }
inline Tensor eq(const Tensor& a, const Tensor& b) { return eq_mp(a, b); }
inline Tensor ne(const Tensor& a, const Tensor& b) { return ne_mp(a, b); }
inline Tensor cat(const std::vector<Tensor>& tensors, size_t dim) { return cat_mp(tensors, dim); }
