// The `*_mp` operator names (src/core/opsmp.h:30-88 of the reference; its legacy tree spells
// the same set in opsmp.h:30-111 and ops1.h:29-85).  Callers such as the legacy autograd.cpp,
// layer.cpp and loss.cpp use these names directly; here they are the same GPU operators as
// ops_dispatch.h.  One semantic difference is kept from the reference: the *_mp reductions
// read dim = -1 as "the last dim" (src/core/opsmp.cpp:598), while sum()/mean()/max()/min() of
// ops_dispatch.h read it as "everything".
#pragma once
#include "ops_dispatch.h"

inline Tensor add_mp(const Tensor& a, const Tensor& b) { return add(a, b); }
inline Tensor diff_mp(const Tensor& a, const Tensor& b) { return sub(a, b); }
inline Tensor mult_mp(const Tensor& a, const Tensor& b) { return mul(a, b); }
inline Tensor div_mp(const Tensor& a, const Tensor& b) { return div(a, b); }
inline Tensor pow_mp(const Tensor& a, const Tensor& b) { return pow(a, b); }

inline Tensor add_scalar_mp(const Tensor& a, double s) { return add_scalar(a, s); }
inline Tensor sub_scalar_mp(const Tensor& a, double s) { return sub_scalar(a, s); }
inline Tensor sub_afterscalar_mp(double s, const Tensor& a) { return sub_scalar_rev(s, a); }
inline Tensor mult_scalar_mp(const Tensor& a, double s) { return mul_scalar(a, s); }
inline Tensor div_scalar_mp(const Tensor& a, double s) { return div_scalar(a, s); }
inline Tensor scalar_div_mp(double s, const Tensor& a) { return div_scalar_rev(s, a); }
inline Tensor pow_scalar_mp(const Tensor& a, double s) { return pow_scalar(a, s); }
inline Tensor scalar_pow_mp(double s, const Tensor& a) { return pow_scalar_rev(s, a); }

inline Tensor abs_mp(const Tensor& a) { return abs(a); }
inline Tensor ln_mp(const Tensor& a) { return ln(a); }
inline Tensor exp_mp(const Tensor& a) { return exp(a); }
inline Tensor sqrt_mp(const Tensor& a) { return sqrt(a); }
inline Tensor sin_mp(const Tensor& a) { return sin(a); }
inline Tensor asin_mp(const Tensor& a) { return asin(a); }
inline Tensor cos_mp(const Tensor& a) { return cos(a); }
inline Tensor acos_mp(const Tensor& a) { return acos(a); }
inline Tensor tan_mp(const Tensor& a) { return tan(a); }
inline Tensor atan_mp(const Tensor& a) { return atan(a); }
inline Tensor sinh_mp(const Tensor& a) { return sinh(a); }
inline Tensor cosh_mp(const Tensor& a) { return cosh(a); }
inline Tensor softplus_mp(const Tensor& a) { return softplus(a); }
inline Tensor tanh_mp(const Tensor& a) { return tanh(a); }
inline Tensor sigmoid_mp(const Tensor& a) { return sigmoid(a); }
inline Tensor Relu_mp(const Tensor& a) { return relu(a); }
inline Tensor matmul_mp(const Tensor& a, const Tensor& b) { return matmul(a, b); }
inline Tensor cat_mp(const std::vector<Tensor>& tensors, size_t dim) { return cat(tensors, dim); }

namespace ctb_host { int last_dim_if_negative(const Tensor& t, int dim); }
inline Tensor sum_mp(const Tensor& t, int dim = -1) { return sum(t, ctb_host::last_dim_if_negative(t, dim)); }
inline Tensor mean_mp(const Tensor& t, int dim = -1) { return mean(t, ctb_host::last_dim_if_negative(t, dim)); }
inline Tensor max_mp(const Tensor& t, int dim = -1) { return max(t, ctb_host::last_dim_if_negative(t, dim)); }
inline Tensor min_mp(const Tensor& t, int dim = -1) { return min(t, ctb_host::last_dim_if_negative(t, dim)); }

inline Tensor lt_mp(const Tensor& a, double b) { return lt(a, b); }
inline Tensor le_mp(const Tensor& a, double b) { return le(a, b); }
inline Tensor gt_mp(const Tensor& a, double b) { return gt(a, b); }
inline Tensor ge_mp(const Tensor& a, double b) { return ge(a, b); }
inline Tensor eq_mp(const Tensor& a, double b) { return eq(a, b); }
inline Tensor neq_mp(const Tensor& a, double b) { return ne(a, b); }
inline Tensor lt_mp(const Tensor& a, const Tensor& b) { return lt(a, b); }
inline Tensor le_mp(const Tensor& a, const Tensor& b) { return le(a, b); }
inline Tensor gt_mp(const Tensor& a, const Tensor& b) { return gt(a, b); }
inline Tensor ge_mp(const Tensor& a, const Tensor& b) { return ge(a, b); }
inline Tensor eq_mp(const Tensor& a, const Tensor& b) { return eq(a, b); }
inline Tensor ne_mp(const Tensor& a, const Tensor& b) { return ne(a, b); }
