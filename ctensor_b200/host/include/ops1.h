// The legacy sequential operator names (ops1.h:29-85 of the reference's root tree: add_, diff_,
// mult_, div_, Relu_, exp_, ln_, tanh_, ...).  In the reference they are single-threaded
// double-precision loops; here they are the same GPU operators as ops_dispatch.h, so a legacy
// caller keeps compiling.  Do not include together with opsmp.h's operator overloads in a
// translation unit that also defines its own (the reference has the same restriction).
#pragma once
#include "ops_dispatch.h"

inline Tensor add_(const Tensor& a, const Tensor& b) { return add(a, b); }
inline Tensor diff_(const Tensor& a, const Tensor& b) { return sub(a, b); }
inline Tensor mult_(const Tensor& a, const Tensor& b) { return mul(a, b); }
inline Tensor div_(const Tensor& a, const Tensor& b) { return div(a, b); }
inline Tensor matmul_(const Tensor& a, const Tensor& b) { return matmul(a, b); }
inline Tensor sub_afterscalar(double s, const Tensor& a) { return sub_scalar_rev(s, a); }
inline Tensor mult_scalar(const Tensor& a, double s) { return mul_scalar(a, s); }
inline Tensor scalar_div(double s, const Tensor& a) { return div_scalar_rev(s, a); }
inline Tensor scalar_pow(double s, const Tensor& a) { return pow_scalar_rev(s, a); }

inline Tensor abs_(const Tensor& a) { return abs(a); }
inline Tensor ln_(const Tensor& a) { return ln(a); }
inline Tensor exp_(const Tensor& a) { return exp(a); }
inline Tensor sqrt_(const Tensor& a) { return sqrt(a); }
inline Tensor pow_(const Tensor& a, const Tensor& b) { return pow(a, b); }
inline Tensor sin_(const Tensor& a) { return sin(a); }
inline Tensor asin_(const Tensor& a) { return asin(a); }
inline Tensor sinh_(const Tensor& a) { return sinh(a); }
inline Tensor cos_(const Tensor& a) { return cos(a); }
inline Tensor acos_(const Tensor& a) { return acos(a); }
inline Tensor cosh_(const Tensor& a) { return cosh(a); }
inline Tensor tan_(const Tensor& a) { return tan(a); }
inline Tensor atan_(const Tensor& a) { return atan(a); }
inline Tensor softplus_(const Tensor& a) { return softplus(a); }
inline Tensor tanh_(const Tensor& a) { return tanh(a); }
inline Tensor sigmoid_(const Tensor& a) { return sigmoid(a); }
inline Tensor Relu_(const Tensor& a) { return relu(a); }

inline Tensor neq(const Tensor& a, double b) { return ne(a, b); }
