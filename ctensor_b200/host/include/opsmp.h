// The `*_mp` operator names (src/core/opsmp.h:30-88 of the reference; its legacy tree spells
// the same set in opsmp.h:30-111 and ops1.h:29-85).  Callers such as the legacy autograd.cpp,
// layer.cpp and loss.cpp use these names directly; here they are the same GPU operators as
// ops_dispatch.h.  One semantic difference is kept from the reference: the *_mp reductions
// read dim = -1 as "the last dim" (src/core/opsmp.cpp:598), while sum()/mean()/max()/min() of
// ops_dispatch.h read it as "everything".
// A second one: the *_mp names accept the element types that only the reference's scalar back-end
// serves (UInt8, Int8, Int16, Int64, Bool: read_scalar_at / write_scalar_at, src/core/tensor.h:54-86),
// while the ops_dispatch.h names refuse them like the reference's dispatcher
// ("unsupported dtype or op not registered", src/core/ops_dispatch.cpp:206-209).
#pragma once
#include "ops_dispatch.h"

namespace ctb_host {
// While one of these lives, operators of this thread accept the scalar back-end's element types.
struct ScalarBackEndScope {
    ScalarBackEndScope();
    ~ScalarBackEndScope();
    ScalarBackEndScope(const ScalarBackEndScope&) = delete;
    ScalarBackEndScope& operator=(const ScalarBackEndScope&) = delete;
private:
    bool prev_;
};
}  // namespace ctb_host

inline Tensor add_mp(const Tensor& a, const Tensor& b) { ctb_host::ScalarBackEndScope scope; return add(a, b); }
inline Tensor diff_mp(const Tensor& a, const Tensor& b) { ctb_host::ScalarBackEndScope scope; return sub(a, b); }
inline Tensor mult_mp(const Tensor& a, const Tensor& b) { ctb_host::ScalarBackEndScope scope; return mul(a, b); }
inline Tensor div_mp(const Tensor& a, const Tensor& b) { ctb_host::ScalarBackEndScope scope; return div(a, b); }
inline Tensor pow_mp(const Tensor& a, const Tensor& b) { ctb_host::ScalarBackEndScope scope; return pow(a, b); }

inline Tensor add_scalar_mp(const Tensor& a, double s) { ctb_host::ScalarBackEndScope scope; return add_scalar(a, s); }
inline Tensor sub_scalar_mp(const Tensor& a, double s) { ctb_host::ScalarBackEndScope scope; return sub_scalar(a, s); }
inline Tensor sub_afterscalar_mp(double s, const Tensor& a) { ctb_host::ScalarBackEndScope scope; return sub_scalar_rev(s, a); }
inline Tensor mult_scalar_mp(const Tensor& a, double s) { ctb_host::ScalarBackEndScope scope; return mul_scalar(a, s); }
inline Tensor div_scalar_mp(const Tensor& a, double s) { ctb_host::ScalarBackEndScope scope; return div_scalar(a, s); }
inline Tensor scalar_div_mp(double s, const Tensor& a) { ctb_host::ScalarBackEndScope scope; return div_scalar_rev(s, a); }
inline Tensor pow_scalar_mp(const Tensor& a, double s) { ctb_host::ScalarBackEndScope scope; return pow_scalar(a, s); }
inline Tensor scalar_pow_mp(double s, const Tensor& a) { ctb_host::ScalarBackEndScope scope; return pow_scalar_rev(s, a); }

inline Tensor abs_mp(const Tensor& a) { ctb_host::ScalarBackEndScope scope; return abs(a); }
inline Tensor ln_mp(const Tensor& a) { ctb_host::ScalarBackEndScope scope; return ln(a); }
inline Tensor exp_mp(const Tensor& a) { ctb_host::ScalarBackEndScope scope; return exp(a); }
inline Tensor sqrt_mp(const Tensor& a) { ctb_host::ScalarBackEndScope scope; return sqrt(a); }
inline Tensor sin_mp(const Tensor& a) { ctb_host::ScalarBackEndScope scope; return sin(a); }
inline Tensor asin_mp(const Tensor& a) { ctb_host::ScalarBackEndScope scope; return asin(a); }
inline Tensor cos_mp(const Tensor& a) { ctb_host::ScalarBackEndScope scope; return cos(a); }
inline Tensor acos_mp(const Tensor& a) { ctb_host::ScalarBackEndScope scope; return acos(a); }
inline Tensor tan_mp(const Tensor& a) { ctb_host::ScalarBackEndScope scope; return tan(a); }
inline Tensor atan_mp(const Tensor& a) { ctb_host::ScalarBackEndScope scope; return atan(a); }
inline Tensor sinh_mp(const Tensor& a) { ctb_host::ScalarBackEndScope scope; return sinh(a); }
inline Tensor cosh_mp(const Tensor& a) { ctb_host::ScalarBackEndScope scope; return cosh(a); }
inline Tensor softplus_mp(const Tensor& a) { ctb_host::ScalarBackEndScope scope; return softplus(a); }
inline Tensor tanh_mp(const Tensor& a) { ctb_host::ScalarBackEndScope scope; return tanh(a); }
inline Tensor sigmoid_mp(const Tensor& a) { ctb_host::ScalarBackEndScope scope; return sigmoid(a); }
inline Tensor Relu_mp(const Tensor& a) { ctb_host::ScalarBackEndScope scope; return relu(a); }
inline Tensor matmul_mp(const Tensor& a, const Tensor& b) { ctb_host::ScalarBackEndScope scope; return matmul(a, b); }
inline Tensor cat_mp(const std::vector<Tensor>& tensors, size_t dim) { ctb_host::ScalarBackEndScope scope; return cat(tensors, dim); }

namespace ctb_host { int last_dim_if_negative(const Tensor& t, int dim); }
inline Tensor sum_mp(const Tensor& t, int dim = -1) { ctb_host::ScalarBackEndScope scope; return sum(t, ctb_host::last_dim_if_negative(t, dim)); }
inline Tensor mean_mp(const Tensor& t, int dim = -1) { ctb_host::ScalarBackEndScope scope; return mean(t, ctb_host::last_dim_if_negative(t, dim)); }
inline Tensor max_mp(const Tensor& t, int dim = -1) { ctb_host::ScalarBackEndScope scope; return max(t, ctb_host::last_dim_if_negative(t, dim)); }
inline Tensor min_mp(const Tensor& t, int dim = -1) { ctb_host::ScalarBackEndScope scope; return min(t, ctb_host::last_dim_if_negative(t, dim)); }

inline Tensor lt_mp(const Tensor& a, double b) { ctb_host::ScalarBackEndScope scope; return lt(a, b); }
inline Tensor le_mp(const Tensor& a, double b) { ctb_host::ScalarBackEndScope scope; return le(a, b); }
inline Tensor gt_mp(const Tensor& a, double b) { ctb_host::ScalarBackEndScope scope; return gt(a, b); }
inline Tensor ge_mp(const Tensor& a, double b) { ctb_host::ScalarBackEndScope scope; return ge(a, b); }
inline Tensor eq_mp(const Tensor& a, double b) { ctb_host::ScalarBackEndScope scope; return eq(a, b); }
inline Tensor neq_mp(const Tensor& a, double b) { ctb_host::ScalarBackEndScope scope; return ne(a, b); }
inline Tensor lt_mp(const Tensor& a, const Tensor& b) { ctb_host::ScalarBackEndScope scope; return lt(a, b); }
inline Tensor le_mp(const Tensor& a, const Tensor& b) { ctb_host::ScalarBackEndScope scope; return le(a, b); }
inline Tensor gt_mp(const Tensor& a, const Tensor& b) { ctb_host::ScalarBackEndScope scope; return gt(a, b); }
inline Tensor ge_mp(const Tensor& a, const Tensor& b) { ctb_host::ScalarBackEndScope scope; return ge(a, b); }
inline Tensor eq_mp(const Tensor& a, const Tensor& b) { ctb_host::ScalarBackEndScope scope; return eq(a, b); }
inline Tensor ne_mp(const Tensor& a, const Tensor& b) { ctb_host::ScalarBackEndScope scope; return ne(a, b); }
