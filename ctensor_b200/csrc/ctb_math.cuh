// Device-side arithmetic of the operator path.  Every function states the reference code whose
// results it reproduces bit-for-bit (paths relative to the reference repository).  The library
// is compiled with -fmad=false -prec-div=true -prec-sqrt=true -ftz=false; fused multiply-adds
// below are explicit (fmaf) and unfused operations use the _rn intrinsics so that no compiler
// setting can change a rounding point.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include <math.h>
#include "../../include/ctb200.h"

namespace ctb {

// ---- fp32 transcendental flavours -------------------------------------------------------------
// exp512_ps, src/cpu/AVX512/ops_avx512_f32.cpp:63-92 (== exp256_ps, src/cpu/AVX2/
// ops_avx2_f32.cpp:58-100, as GCC contracts it under the shipped -O3 -mfma flags).
// SSE min/max return the second operand on an unordered compare: min_ps(x, HI) gives HI for NaN,
// as fminf does.
constexpr float kExpHi = 88.3762626647949f;

// Clamp, fx = x*log2(e) + 0.5 and floor(fx) for exp_cephes.  |fx| <= 129, so adding 1.5*2^23
// with rounding toward minus infinity gives floor(fx) + 1.5*2^23 exactly: no conversion, no
// compare.  Returns -floor(fx) and the bit pattern of 2^floor(fx); x is clamped in place.
__device__ __forceinline__ void exp_cephes_front(float& x, float& neg_fx, int32_t& pow2n_bits,
                                                 float hi = kExpHi) {
    x = fminf(x, hi);
    x = fmaxf(x, -kExpHi);
    const float fx = fmaf(x, 1.44269504088896341f, 0.5f);
    const float MAGIC = 12582912.0f;                // 0x4B400000, ulp 1
    const float r = __fadd_rd(fx, MAGIC);
    pow2n_bits = (__float_as_int(r) - (0x4B400000 - 127)) << 23;
    neg_fx = __fsub_rn(MAGIC, r);
}

__device__ __forceinline__ float exp_cephes(float x) {
    float neg_fx;
    int32_t pbits;
    exp_cephes_front(x, neg_fx, pbits);
    x = fmaf(neg_fx, 0.693359375f, x);
    x = fmaf(neg_fx, -2.12194440e-4f, x);
    float z = __fmul_rn(x, x);
    float y = 1.9875691500E-4f;
    y = fmaf(y, x, 1.3981999507E-3f);
    y = fmaf(y, x, 8.3334519073E-3f);
    y = fmaf(y, x, 4.1665795894E-2f);
    y = fmaf(y, x, 1.6666665459E-1f);
    y = fmaf(y, x, 0.5f);
    y = fmaf(y, z, x);
    y = __fadd_rn(y, 1.0f);
    return __fmul_rn(y, __int_as_float(pbits));
}

// log256_ps, src/cpu/AVX2/ops_avx2_f32.cpp:103-158 as compiled with the shipped flags:
// the y*z product is fused into the following add, e*Q1 is rounded on its own.
__device__ __forceinline__ float log_cephes(float x) {
    bool invalid = (x <= 0.0f);
    x = (x > 1.17549435e-38f) ? x : 1.17549435e-38f;
    uint32_t bits = __float_as_uint(x);
    int32_t emm0 = (int32_t)(bits >> 23) - 127;
    x = __uint_as_float((bits & 0x7fffffu) | 0x3f000000u);
    float e = __fadd_rn(__int2float_rn(emm0), 1.0f);
    bool m = (x < 0.707106781186547524f);
    float tmp = m ? x : 0.0f;
    x = __fsub_rn(x, 1.0f);
    e = __fsub_rn(e, m ? 1.0f : 0.0f);
    x = __fadd_rn(x, tmp);
    float z = __fmul_rn(x, x);
    float y = 7.0376836292E-2f;
    y = fmaf(y, x, -1.1514610310E-1f);
    y = fmaf(y, x, 1.1676998740E-1f);
    y = fmaf(y, x, -1.2420140846E-1f);
    y = fmaf(y, x, 1.4249322787E-1f);
    y = fmaf(y, x, -1.6668057665E-1f);
    y = fmaf(y, x, 2.0000714765E-1f);
    y = fmaf(y, x, -2.4999993993E-1f);
    y = fmaf(y, x, 3.3333331174E-1f);
    y = __fmul_rn(y, x);
    float t = __fmul_rn(e, -2.12194440e-4f);
    y = fmaf(y, z, t);
    y = fmaf(-z, 0.5f, y);
    x = __fadd_rn(x, y);
    x = fmaf(e, 0.693359375f, x);
    return invalid ? __uint_as_float(0xFFFFFFFFu) : x;
}

// tanh512_ps, src/cpu/AVX512/ops_avx512_f32.cpp:187-193
__device__ __forceinline__ float tanh_cephes(float x) {
    float e = exp_cephes(__fmul_rn(x, 2.0f));
    return __fdiv_rn(__fsub_rn(e, 1.0f), __fadd_rn(e, 1.0f));
}

// sigmoid512_ps, src/cpu/AVX512/ops_avx512_f32.cpp:195-201
__device__ __forceinline__ float sigmoid_cephes(float x) {
    float e = exp_cephes(__uint_as_float(__float_as_uint(x) ^ 0x80000000u));
    return __fdiv_rn(1.0f, __fadd_rn(1.0f, e));
}

// (float)((double)x * s): mult_scalar_mp, src/core/opsmp.cpp:297,433-436
__device__ __forceinline__ float mul_scalar_f32(float x, double s) {
    return __double2float_rn(__dmul_rn((double)x, s));
}

// Tanh-form GELU as the chain mul, mul, mul_scalar(0.044715), add, mul_scalar(sqrt(2/pi)),
// tanh, add_scalar(1), mul_scalar(x, 0.5), mul with fp32 rounding after every step.
// (double)t + 1.0 and (double)x * 0.5 rounded to fp32 equal the fp32 operations: a double
// holds any fp32 sum/product to more than 2*24+2 bits, so the second rounding is innocuous.
__device__ __forceinline__ float gelu_tanh_chain(float x) {
    float u = __fmul_rn(x, x);
    u = __fmul_rn(u, x);
    u = mul_scalar_f32(u, 0.044715);
    u = __fadd_rn(x, u);
    u = mul_scalar_f32(u, 0.7978845608028654);
    float t = tanh_cephes(u);
    t = __fadd_rn(t, 1.0f);
    float h = __fmul_rn(x, 0.5f);
    return __fmul_rn(h, t);
}

// ---- packed (two lanes per instruction) variants ------------------------------------------------
// sm_100 has packed fp32 instructions (fma/add/mul.rn.f32x2): one issue slot does two IEEE
// operations, and exp/tanh/sigmoid/GELU are bound by issue slots, not by HBM.  Each lane computes
// exactly the scalar sequence above, so results are bit-identical to the scalar functions (each
// pair function was compared with its scalar twin over all 2^32 inputs on a B200).
__device__ __forceinline__ float2 splat2(float a) { return make_float2(a, a); }

// exp_cephes for two lanes: clamp, fx and floor per lane; range reduction and polynomial packed.
// `hi` may lower the upper clamp for callers that saturate earlier (tanh).
__device__ __forceinline__ float2 exp_cephes2(float2 v, float hi = kExpHi) {
    // the front end of exp_cephes_front, lane for lane, with the three arithmetic steps packed:
    // fx, the round-down add that takes floor(fx), and MAGIC - r (as fma(r, -1, MAGIC): the same
    // single rounding of the same exact value)
    const float x0 = fmaxf(fminf(v.x, hi), -kExpHi), x1 = fmaxf(fminf(v.y, hi), -kExpHi);
    const float MAGIC = 12582912.0f;
    const float2 fx = __ffma2_rn(make_float2(x0, x1), splat2(1.44269504088896341f), splat2(0.5f));
    const float2 r = __fadd2_rd(fx, splat2(MAGIC));
    const int32_t p0 = (__float_as_int(r.x) - (0x4B400000 - 127)) << 23;
    const int32_t p1 = (__float_as_int(r.y) - (0x4B400000 - 127)) << 23;
    const float2 nfx = __ffma2_rn(r, splat2(-1.0f), splat2(MAGIC));
    float2 x = make_float2(x0, x1);
    x = __ffma2_rn(nfx, splat2(0.693359375f), x);
    x = __ffma2_rn(nfx, splat2(-2.12194440e-4f), x);
    const float2 z = __fmul2_rn(x, x);
    float2 y = splat2(1.9875691500E-4f);
    y = __ffma2_rn(y, x, splat2(1.3981999507E-3f));
    y = __ffma2_rn(y, x, splat2(8.3334519073E-3f));
    y = __ffma2_rn(y, x, splat2(4.1665795894E-2f));
    y = __ffma2_rn(y, x, splat2(1.6666665459E-1f));
    y = __ffma2_rn(y, x, splat2(0.5f));
    y = __ffma2_rn(y, z, x);
    y = __fadd2_rn(y, splat2(1.0f));
    return __fmul2_rn(y, make_float2(__int_as_float(p0), __int_as_float(p1)));
}

// The exponential as GradCrossEntropy::backward takes it (std::exp, src/neuralnet/loss.cpp:351): a
// NaN argument — a NaN logit, or inf - inf under an infinite row maximum — gives NaN, where the
// operator exp above clamps it to its upper bound.  Arguments there are <= 0 otherwise.
__device__ __forceinline__ float exp_nan_through(float d) {
    const float e = exp_cephes(d);
    return d != d ? d : e;
}
__device__ __forceinline__ float2 exp_nan_through2(float2 d) {
    float2 e = exp_cephes2(d);
    e.x = d.x != d.x ? d.x : e.x;
    e.y = d.y != d.y ? d.y : e.y;
    return e;
}

// Reciprocal estimate refined by one Newton step, for b in [1, 2^26].
__device__ __forceinline__ float2 rcp_newton2(float2 b, float2 nb) {
    float2 r;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r.x) : "f"(b.x));
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r.y) : "f"(b.y));
    const float2 err = __ffma2_rn(nb, r, splat2(1.0f));
    return __ffma2_rn(r, err, r);
}

// tanh_cephes for two lanes.  (e-1)/(e+1) equals 1 for every e >= 2^25 (both e-1 and e+1 round
// to e), so the argument of exp is clamped at 17.4 (exp_cephes(17.4) > 2^25) instead of 88.38;
// that keeps the denominator in the range where reciprocal + Newton + one remainder correction
// equals IEEE division.
constexpr float kTanhExpHi = 17.4f;
__device__ __forceinline__ float2 tanh_cephes2(float2 x) {
    const float2 e = exp_cephes2(__fmul2_rn(x, splat2(2.0f)), kTanhExpHi);
    const float2 a = __fadd2_rn(e, splat2(-1.0f));
    const float2 b = __fadd2_rn(e, splat2(1.0f));
    const float2 nb = make_float2(-b.x, -b.y);
    const float2 r = rcp_newton2(b, nb);
    const float2 q = __fmul2_rn(a, r);
    const float2 rem = __ffma2_rn(nb, q, a);
    return __ffma2_rn(rem, r, q);
}

// log_cephes for two lanes: mantissa/exponent split per lane, polynomial packed.  The exponent
// (+1, -1 when the mantissa is below sqrt(1/2)) becomes a float through the 1.5*2^23 bit
// pattern, which is exact for these small integers and needs no conversion instruction.
__device__ __forceinline__ void log_cephes_front(float x, float& mant_m1, float& e, bool& invalid) {
    invalid = (x <= 0.0f);
    x = fmaxf(x, 1.17549435e-38f);                  // max_ps(x, FLT_MIN): NaN -> FLT_MIN, as fmaxf does
    const uint32_t bits = __float_as_uint(x);
    const float m = __uint_as_float((bits & 0x7fffffu) | 0x3f000000u);
    const bool lo = (m < 0.707106781186547524f);
    const int32_t ei = (int32_t)(bits >> 23) + (0x4B400000 - 126) - (lo ? 1 : 0);
    e = __fsub_rn(__int_as_float(ei), 12582912.0f);
    mant_m1 = __fadd_rn(__fsub_rn(m, 1.0f), lo ? m : 0.0f);
}
__device__ __forceinline__ float2 log_cephes2(float2 v) {
    float x0, x1, e0, e1;
    bool i0, i1;
    log_cephes_front(v.x, x0, e0, i0);
    log_cephes_front(v.y, x1, e1, i1);
    const float2 x = make_float2(x0, x1), e = make_float2(e0, e1);
    const float2 z = __fmul2_rn(x, x);
    float2 y = splat2(7.0376836292E-2f);
    y = __ffma2_rn(y, x, splat2(-1.1514610310E-1f));
    y = __ffma2_rn(y, x, splat2(1.1676998740E-1f));
    y = __ffma2_rn(y, x, splat2(-1.2420140846E-1f));
    y = __ffma2_rn(y, x, splat2(1.4249322787E-1f));
    y = __ffma2_rn(y, x, splat2(-1.6668057665E-1f));
    y = __ffma2_rn(y, x, splat2(2.0000714765E-1f));
    y = __ffma2_rn(y, x, splat2(-2.4999993993E-1f));
    y = __ffma2_rn(y, x, splat2(3.3333331174E-1f));
    y = __fmul2_rn(y, x);
    const float2 t = __fmul2_rn(e, splat2(-2.12194440e-4f));
    y = __ffma2_rn(y, z, t);
    y = __ffma2_rn(z, splat2(-0.5f), y);
    float2 r = __fadd2_rn(x, y);
    r = __ffma2_rn(e, splat2(0.693359375f), r);
    if (i0) r.x = __uint_as_float(0xFFFFFFFFu);
    if (i1) r.y = __uint_as_float(0xFFFFFFFFu);
    return r;
}

// sigmoid_cephes for two lanes: 1/(1+e) through the corrected reciprocal; IEEE division where
// the quotient can be subnormal (e beyond 1e18; never reached for x > -41).
__device__ __forceinline__ float2 sigmoid_cephes2(float2 x) {
    const float2 e = exp_cephes2(make_float2(-x.x, -x.y));
    const float2 b = __fadd2_rn(e, splat2(1.0f));
    const float2 nb = make_float2(-b.x, -b.y);
    const float2 r = rcp_newton2(b, nb);
    const float2 rem = __ffma2_rn(nb, r, splat2(1.0f));
    float2 t = __ffma2_rn(rem, r, r);
    if (e.x > 1.0e18f) t.x = __fdiv_rn(1.0f, b.x);
    if (e.y > 1.0e18f) t.y = __fdiv_rn(1.0f, b.y);
    return t;
}

// ---- exact formulations of the GELU chain -----------------------------------------------------------
// The chain has two scalar multiplies that the reference evaluates in double,
// (float)((double)x * s).  Done with conversion instructions they cost four operations per element
// on the conversion / special-function (XU) pipe, which — with the reciprocal of tanh — is the pipe
// that bounds the kernel.  Build-time choice (-DCTB_GELU_VARIANT=n); every variant gives the same
// bits for every one of the 2^32 inputs:
//   0: conversion instructions (5 XU operations per element, 28.4 instructions)
//   1: the fp32 -> fp64 widenings done with integer instructions (3 XU, 36 instructions): no faster
//   2: the division of tanh from an integer first guess and three Newton steps instead of the
//      reciprocal unit (4 XU, 30 instructions): no faster
//   3: variant 1 on magnitudes — every step up to the argument of tanh is odd in x and rounds
//      symmetrically, so the widenings need no sign handling (two integer instructions each) and
//      the sign is put back once (3 XU, ~33 instructions): 3-6 % faster than 0, the more so when the
//      SM clock is held down by the power cap.  This is what ships.
//   4: 3 and 2 together (2 XU operations per element)
#ifndef CTB_GELU_VARIANT
#define CTB_GELU_VARIANT 3
#endif
// (float)((double)x * s) with the widening done by integer instructions.  Exact for normal x; zero,
// denormal, infinite and NaN inputs give other doubles, which the GELU chain does not notice.
__device__ __forceinline__ float mul_scalar_int_widen(float x, double s) {
    const uint32_t b = __float_as_uint(x);
    const uint32_t hi = (b & 0x80000000u) | (((b & 0x7fffffffu) >> 3) + 0x38000000u);
    const uint32_t lo = b << 29;
    return __double2float_rn(__dmul_rn(__hiloint2double((int)hi, (int)lo), s));
}
// The same for x >= 0 (no sign to carry) in two integer instructions: the bits of x shifted into a
// double's layout WITHOUT re-biasing the exponent are the double x * 2^-896 — exactly, for zero and
// denormal x too (m * 2^-149 becomes the denormal double m * 2^-1045) — and the scalar carries the
// factor 2^896 instead (an exact scaling of both operands: the product and its rounding are those
// of (double)x * s).  Infinite and NaN inputs give finite values, which the GELU chain does not notice.
__device__ __forceinline__ float mul_scalar_int_widen_pos(float x, double s) {
    const uint32_t b = __float_as_uint(x);
    return __double2float_rn(__dmul_rn(__hiloint2double((int)(b >> 3), (int)(b << 29)), s * 0x1p896));
}
// tanh_cephes2 with the reciprocal of (e + 1) from an integer first guess and three Newton steps
__device__ __forceinline__ float2 tanh_cephes2_no_rcp_unit(float2 x) {
    const float2 e = exp_cephes2(__fmul2_rn(x, splat2(2.0f)), kTanhExpHi);
    const float2 a = __fadd2_rn(e, splat2(-1.0f));
    const float2 b = __fadd2_rn(e, splat2(1.0f));
    const float2 nb = make_float2(-b.x, -b.y);
    float2 r = make_float2(__uint_as_float(0x7EF311C7u - __float_as_uint(b.x)), __uint_as_float(0x7EF311C7u - __float_as_uint(b.y)));
#pragma unroll
    for (int i = 0; i < 3; ++i) {
        const float2 err = __ffma2_rn(nb, r, splat2(1.0f));
        r = __ffma2_rn(r, err, r);
    }
    const float2 q = __fmul2_rn(a, r);
    const float2 rem = __ffma2_rn(nb, q, a);
    return __ffma2_rn(rem, r, q);
}

// The two scalar multiplies stay double-precision multiplies: an fp32 two-product emulation with a
// near-tie check was bit-exact too but slower (more fp32 instructions than it saves elsewhere).
__device__ __forceinline__ float2 gelu_tanh_chain2(float2 x) {
#if CTB_GELU_VARIANT == 1
    float2 u = __fmul2_rn(x, x);
    u = __fmul2_rn(u, x);
    u.x = mul_scalar_int_widen(u.x, 0.044715);
    u.y = mul_scalar_int_widen(u.y, 0.044715);
    u = __fadd2_rn(x, u);
    u.x = mul_scalar_int_widen(u.x, 0.7978845608028654);
    u.y = mul_scalar_int_widen(u.y, 0.7978845608028654);
    float2 tv = tanh_cephes2(u);
    tv = __fadd2_rn(tv, splat2(1.0f));
    return __fmul2_rn(__fmul2_rn(x, splat2(0.5f)), tv);
#elif CTB_GELU_VARIANT == 3 || CTB_GELU_VARIANT == 4
    const float2 ax = make_float2(fabsf(x.x), fabsf(x.y));
    float2 u = __fmul2_rn(__fmul2_rn(x, x), ax);
    u.x = mul_scalar_int_widen_pos(u.x, 0.044715);
    u.y = mul_scalar_int_widen_pos(u.y, 0.044715);
    u = __fadd2_rn(ax, u);
    u.x = __uint_as_float(__float_as_uint(mul_scalar_int_widen_pos(u.x, 0.7978845608028654)) | (__float_as_uint(x.x) & 0x80000000u));
    u.y = __uint_as_float(__float_as_uint(mul_scalar_int_widen_pos(u.y, 0.7978845608028654)) | (__float_as_uint(x.y) & 0x80000000u));
#if CTB_GELU_VARIANT == 4
    float2 tv = tanh_cephes2_no_rcp_unit(u);
#else
    float2 tv = tanh_cephes2(u);
#endif
    tv = __fadd2_rn(tv, splat2(1.0f));
    return __fmul2_rn(__fmul2_rn(x, splat2(0.5f)), tv);
#elif CTB_GELU_VARIANT == 2
    float2 u = __fmul2_rn(x, x);
    u = __fmul2_rn(u, x);
    u.x = mul_scalar_f32(u.x, 0.044715);
    u.y = mul_scalar_f32(u.y, 0.044715);
    u = __fadd2_rn(x, u);
    u.x = mul_scalar_f32(u.x, 0.7978845608028654);
    u.y = mul_scalar_f32(u.y, 0.7978845608028654);
    float2 tv = tanh_cephes2_no_rcp_unit(u);
    tv = __fadd2_rn(tv, splat2(1.0f));
    return __fmul2_rn(__fmul2_rn(x, splat2(0.5f)), tv);
#else
    float2 u = __fmul2_rn(x, x);
    u = __fmul2_rn(u, x);
    u.x = mul_scalar_f32(u.x, 0.044715);
    u.y = mul_scalar_f32(u.y, 0.044715);
    u = __fadd2_rn(x, u);
    u.x = mul_scalar_f32(u.x, 0.7978845608028654);
    u.y = mul_scalar_f32(u.y, 0.7978845608028654);
    float2 t = tanh_cephes2(u);
    t = __fadd2_rn(t, splat2(1.0f));
    const float2 h = __fmul2_rn(x, splat2(0.5f));
    return __fmul2_rn(h, t);
#endif
}

// static_cast<int32_t>(double) as x86 cvttsd2si does it (write_scalar_at,
// src/core/tensor.h:77): truncation, INT32_MIN for NaN / out of range.
__device__ __forceinline__ int32_t d2i_x86(double v) {
    return (v > -2147483649.0 && v < 2147483648.0) ? __double2int_rz(v) : INT32_MIN;
}

// ---- typed load/convert -----------------------------------------------------------------------
template <typename T> __device__ __forceinline__ double to_double(T v) { return (double)v; }
template <typename T> __device__ __forceinline__ T from_double(double v);
template <> __device__ __forceinline__ float from_double<float>(double v) { return __double2float_rn(v); }
template <> __device__ __forceinline__ double from_double<double>(double v) { return v; }
template <> __device__ __forceinline__ int32_t from_double<int32_t>(double v) { return d2i_x86(v); }
// The narrow integer types as x86 compiles static_cast<T>(double) (write_scalar_at,
// src/core/tensor.h:79-83): a 32-bit truncating conversion whose low bits are stored; Int64 through
// the 64-bit conversion (INT64_MIN for NaN / out of range); Bool is value != 0.
template <> __device__ __forceinline__ uint8_t from_double<uint8_t>(double v) { return (uint8_t)d2i_x86(v); }
template <> __device__ __forceinline__ int8_t from_double<int8_t>(double v) { return (int8_t)d2i_x86(v); }
template <> __device__ __forceinline__ int16_t from_double<int16_t>(double v) { return (int16_t)d2i_x86(v); }
template <> __device__ __forceinline__ int64_t from_double<int64_t>(double v) {
    return (v >= -9223372036854775808.0 && v < 9223372036854775808.0) ? __double2ll_rz(v) : INT64_MIN;
}
template <> __device__ __forceinline__ bool from_double<bool>(double v) { return v != 0.0; }

// ---- binary functors: out = (T) op((double)a, (double)b), src/core/opsmp.cpp:198,249-252 --------
// For fp32 the four arithmetic ops are evaluated directly in fp32: the double-precision result
// rounded to fp32 equals the IEEE fp32 operation (double rounding is innocuous for + - * /).
// Internal operator (not part of the public enum): a + b, or a unchanged when b is NaN or
// infinite — the accumulation step of accumulate_grad, src/core/autograd.cpp:139-151.
constexpr int kOpAddFinite = CTB_BINARY_OP_COUNT;

template <int OP, typename T> struct BinaryFn {
    __device__ __forceinline__ static T apply(T a, T b) {
        double x = to_double(a), y = to_double(b), r;
        if (OP == kOpAddFinite) return isfinite(y) ? from_double<T>(__dadd_rn(x, y)) : a;
        if (OP == CTB_ADD) r = __dadd_rn(x, y);
        else if (OP == CTB_SUB) r = __dsub_rn(x, y);
        else if (OP == CTB_MUL) r = __dmul_rn(x, y);
        else if (OP == CTB_DIV) r = __ddiv_rn(x, y);
        else if (OP == CTB_LT) r = x < y ? 1.0 : 0.0;
        else if (OP == CTB_LE) r = x <= y ? 1.0 : 0.0;
        else if (OP == CTB_GT) r = x > y ? 1.0 : 0.0;
        else if (OP == CTB_GE) r = x >= y ? 1.0 : 0.0;
        else if (OP == CTB_EQ) r = x == y ? 1.0 : 0.0;
        else if (OP == CTB_POW) r = pow(x, y);
        else r = x != y ? 1.0 : 0.0;
        return from_double<T>(r);
    }
};
template <int OP> struct BinaryFn<OP, float> {
    __device__ __forceinline__ static float apply(float a, float b) {
        if (OP == kOpAddFinite) return isfinite(b) ? __fadd_rn(a, b) : a;
        if (OP == CTB_ADD) return __fadd_rn(a, b);
        if (OP == CTB_SUB) return __fsub_rn(a, b);
        if (OP == CTB_MUL) return __fmul_rn(a, b);
        if (OP == CTB_DIV) return __fdiv_rn(a, b);
        if (OP == CTB_LT) return a < b ? 1.0f : 0.0f;
        if (OP == CTB_LE) return a <= b ? 1.0f : 0.0f;
        if (OP == CTB_GT) return a > b ? 1.0f : 0.0f;
        if (OP == CTB_GE) return a >= b ? 1.0f : 0.0f;
        if (OP == CTB_EQ) return a == b ? 1.0f : 0.0f;
        if (OP == CTB_POW) return __double2float_rn(pow((double)a, (double)b));
        return a != b ? 1.0f : 0.0f;
    }
};

// ---- unary functors -----------------------------------------------------------------------------
// Scalar ops: (T) op((double)x, s), src/core/opsmp.cpp:418-456; scalar comparisons :701-706;
// abs/sqrt/relu :562,565,581-584.
template <int OP> __device__ __forceinline__ double unary_double(double x, double s) {
    if (OP == CTB_ADD_S) return __dadd_rn(x, s);
    if (OP == CTB_SUB_S) return __dsub_rn(x, s);
    if (OP == CTB_RSUB_S) return __dsub_rn(s, x);
    if (OP == CTB_MUL_S) return __dmul_rn(x, s);
    if (OP == CTB_DIV_S) return __ddiv_rn(x, s);
    if (OP == CTB_RDIV_S) return __ddiv_rn(s, x);
    if (OP == CTB_POW_S) return pow(x, s);
    if (OP == CTB_RPOW_S) return pow(s, x);
    if (OP == CTB_LT_S) return x < s ? 1.0 : 0.0;
    if (OP == CTB_LE_S) return x <= s ? 1.0 : 0.0;
    if (OP == CTB_GT_S) return x > s ? 1.0 : 0.0;
    if (OP == CTB_GE_S) return x >= s ? 1.0 : 0.0;
    if (OP == CTB_EQ_S) return x == s ? 1.0 : 0.0;
    if (OP == CTB_NE_S) return x != s ? 1.0 : 0.0;
    if (OP == CTB_ABS) return fabs(x);
    if (OP == CTB_RELU) return x > 0 ? x : 0.0;
    if (OP == CTB_SQRT) return __dsqrt_rn(x);
    if (OP == CTB_SIN) return sin(x);
    if (OP == CTB_COS) return cos(x);
    if (OP == CTB_TAN) return tan(x);
    if (OP == CTB_ASIN) return asin(x);
    if (OP == CTB_ACOS) return acos(x);
    if (OP == CTB_ATAN) return atan(x);
    if (OP == CTB_SINH) return sinh(x);
    if (OP == CTB_COSH) return cosh(x);
    if (OP == CTB_SOFTPLUS) return log(1.0 + exp(x));
    return x;
}

template <int OP, typename T> struct UnaryFn {
    __device__ __forceinline__ static T apply(T x, double s) {
        return from_double<T>(unary_double<OP>(to_double(x), s));
    }
};
template <int OP> struct UnaryFn<OP, float> {
    __device__ __forceinline__ static float apply(float x, double s) {
        if (OP == CTB_ABS) return fabsf(x);
        if (OP == CTB_RELU) return x > 0.0f ? x : 0.0f;       // NaN -> 0, -0 -> +0
        if (OP == CTB_SQRT) return __fsqrt_rn(x);             // == (float)sqrt((double)x)
        if (OP == CTB_EXP) return exp_cephes(x);
        if (OP == CTB_LOG) return log_cephes(x);
        if (OP == CTB_TANH) return tanh_cephes(x);
        if (OP == CTB_SIGMOID) return sigmoid_cephes(x);
        if (OP == CTB_GELU_TANH) return gelu_tanh_chain(x);
        return __double2float_rn(unary_double<OP>((double)x, s));
    }
    // Two lanes at once where a packed implementation exists (same bits as apply()).
    static constexpr bool kHasPair = (OP == CTB_GELU_TANH || OP == CTB_TANH || OP == CTB_SIGMOID ||
                                      OP == CTB_LOG || OP == CTB_EXP);
    __device__ __forceinline__ static float2 apply_pair(float2 x, double s) {
        if (OP == CTB_GELU_TANH) return gelu_tanh_chain2(x);
        if (OP == CTB_TANH) return tanh_cephes2(x);
        if (OP == CTB_SIGMOID) return sigmoid_cephes2(x);
        if (OP == CTB_LOG) return log_cephes2(x);
        if (OP == CTB_EXP) return exp_cephes2(x);
        return make_float2(apply(x.x, s), apply(x.y, s));
    }
};

__host__ __device__ inline bool unary_is_f32_only(int op) {
    return op == CTB_EXP || op == CTB_LOG || op == CTB_TANH || op == CTB_SIGMOID ||
           op == CTB_GELU_TANH;
}

}  // namespace ctb
