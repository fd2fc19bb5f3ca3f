/*
 * ctb_oracle.c — TEST INFRASTRUCTURE, not part of the product.
 *
 * A plain-C, CPU restatement of the reference's (ZYROS-OFFICIEL/CTensor) elementwise,
 * broadcast and reduction operators, used only as the checker of the CUDA path (tests,
 * the smoke run and the cpu_baseline leg of the benchmark).  Nothing that ships may call it.
 *
 * Pinning: every function here is compared bit-for-bit (sums/means/variances: to 1e-6
 * relative) with the reference's own compiled code (oracle/_ref/libctensor_ref.so, built
 * by oracle/build_ref.sh from the reference sources) by tests/test_oracle.py,
 * and with the committed golden vectors under tests/golden/ that the same reference
 * build generated (tests/golden/make_golden.py).
 *
 * Build: gcc -O2 -ffp-contract=off -fopenmp -fPIC -shared  (contraction OFF: every fused
 * multiply-add below is written explicitly as fmaf, the unfused ones must stay unfused).
 *
 * Each function cites the reference file:line it follows (paths relative to the reference).
 */
#include <math.h>
#include <stdint.h>
#include <string.h>
#include <stdlib.h>
#include <float.h>

#define ORC_MAX_DIMS 8

typedef struct orc_view {       /* same layout as struct ctb_view (include/ctb200.h) */
    void*   base;
    int64_t offset;
    int32_t dtype;              /* the reference's DType numbering: 0 f32, 1 i32, 2 f64, 3 u8, 4 u16, 5 u32, 6 u64, 7 i8, 8 i16, 9 i64, 10 bool */
    int32_t ndim;
    int64_t shape[ORC_MAX_DIMS];
    int64_t stride[ORC_MAX_DIMS];
} orc_view;

enum { ORC_F32 = 0, ORC_I32 = 1, ORC_F64 = 2 };
enum { B_ADD = 0, B_SUB, B_MUL, B_DIV, B_LT, B_LE, B_GT, B_GE, B_EQ, B_NE, B_POW };
enum {
    U_ADD_S = 0, U_SUB_S, U_RSUB_S, U_MUL_S, U_DIV_S, U_RDIV_S, U_POW_S, U_RPOW_S,
    U_LT_S, U_LE_S, U_GT_S, U_GE_S, U_EQ_S, U_NE_S,
    U_ABS, U_RELU, U_EXP, U_LOG, U_TANH, U_SIGMOID, U_SQRT, U_GELU_TANH,
    U_SIN, U_COS, U_TAN, U_ASIN, U_ACOS, U_ATAN, U_SINH, U_COSH, U_SOFTPLUS
};
enum { R_SUM = 0, R_MEAN, R_MAX, R_MIN, R_VAR, R_ARGMAX };

static inline uint32_t f2u(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }
static inline float u2f(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }

/* ------------------------------------------------------------------------------------------
 * Typed element access through double: read_scalar_at / write_scalar_at,
 * src/core/tensor.h:54-86.  The int32 store is `static_cast<int32_t>(double)`, i.e. x86
 * cvttsd2si: truncation toward zero, and the "integer indefinite" value INT32_MIN for NaN
 * and out-of-range inputs.
 * ---------------------------------------------------------------------------------------- */
static inline int32_t d2i_x86(double v) {
    if (!(v > -2147483649.0 && v < 2147483648.0)) return INT32_MIN;
    return (int32_t)v;
}
/* Element sizes, type-erased loads and stores: dtype_size / read_scalar_at / write_scalar_at,
 * src/core/tensor.h:30-86.  The stores are x86's static_cast<T>(double): the narrow integer types
 * take the low bits of the 32-bit truncating conversion, Int64 the 64-bit one (INT64_MIN outside
 * its range), Bool is value != 0; UInt16 / UInt32 / UInt64 have no store in the reference (a
 * result of such a type keeps the zeros it was allocated with). */
enum { ORC_U8 = 3, ORC_U16 = 4, ORC_U32 = 5, ORC_U64 = 6, ORC_I8 = 7, ORC_I16 = 8, ORC_I64 = 9, ORC_BOOL = 10 };
static inline size_t esize(int dt) {
    switch (dt) {
    case ORC_F64: case ORC_U64: case ORC_I64: return 8;
    case ORC_U16: case ORC_I16: return 2;
    case ORC_U8: case ORC_I8: case ORC_BOOL: return 1;
    default: return 4;
    }
}
static inline int64_t d2ll_x86(double v) {
    return (v >= -9223372036854775808.0 && v < 9223372036854775808.0) ? (int64_t)v : INT64_MIN;
}
static inline double rd(const void* p, int64_t i, int dt) {
    switch (dt) {
    case ORC_F32: return (double)((const float*)p)[i];
    case ORC_I32: return (double)((const int32_t*)p)[i];
    case ORC_U8:  return (double)((const uint8_t*)p)[i];
    case ORC_U16: return (double)((const uint16_t*)p)[i];
    case ORC_U32: return (double)((const uint32_t*)p)[i];
    case ORC_U64: return (double)((const uint64_t*)p)[i];
    case ORC_I8:  return (double)((const int8_t*)p)[i];
    case ORC_I16: return (double)((const int16_t*)p)[i];
    case ORC_I64: return (double)((const int64_t*)p)[i];
    case ORC_BOOL: return ((const uint8_t*)p)[i] ? 1.0 : 0.0;
    default:      return ((const double*)p)[i];
    }
}
static inline void wr(void* p, int64_t i, int dt, double v) {
    switch (dt) {
    case ORC_F32: ((float*)p)[i] = (float)v; break;
    case ORC_I32: ((int32_t*)p)[i] = d2i_x86(v); break;
    case ORC_U8:  ((uint8_t*)p)[i] = (uint8_t)d2i_x86(v); break;
    case ORC_I8:  ((int8_t*)p)[i] = (int8_t)d2i_x86(v); break;
    case ORC_I16: ((int16_t*)p)[i] = (int16_t)d2i_x86(v); break;
    case ORC_I64: ((int64_t*)p)[i] = d2ll_x86(v); break;
    case ORC_BOOL: ((uint8_t*)p)[i] = v != 0.0; break;
    case ORC_U16: case ORC_U32: case ORC_U64: break;
    default:      ((double*)p)[i] = v; break;
    }
}

static int64_t numel(const orc_view* v) {
    int64_t n = 1;
    for (int i = 0; i < v->ndim; ++i) n *= v->shape[i];
    return n;
}

/* ------------------------------------------------------------------------------------------
 * Cephes-style fp32 transcendental flavours, exactly as the reference's SIMD back-ends
 * compute them under their shipped flags (-O3 -mavx2 -mfma / -O3 -mavx512f -mavx512dq, GCC
 * contraction on).  SSE min/max semantics: the SECOND operand is returned when the compare
 * is unordered.
 * ---------------------------------------------------------------------------------------- */

/* exp512_ps src/cpu/AVX512/ops_avx512_f32.cpp:63-92 == exp256_ps
 * src/cpu/AVX2/ops_avx2_f32.cpp:58-100 after contraction. */
float orc_exp_f32(float x) {
    const float HI = 88.3762626647949f, LO = -88.3762626647949f;
    x = (x < HI) ? x : HI;                       /* min_ps(x, HI): NaN -> HI */
    x = (x > LO) ? x : LO;                       /* max_ps(x, LO)            */
    float fx = fmaf(x, 1.44269504088896341f, 0.5f);
    fx = floorf(fx);
    x = fmaf(-fx, 0.693359375f, x);
    x = fmaf(-fx, -2.12194440e-4f, x);
    float z = x * x;
    float y = 1.9875691500E-4f;
    y = fmaf(y, x, 1.3981999507E-3f);
    y = fmaf(y, x, 8.3334519073E-3f);
    y = fmaf(y, x, 4.1665795894E-2f);
    y = fmaf(y, x, 1.6666665459E-1f);
    y = fmaf(y, x, 0.5f);
    y = fmaf(y, z, x);
    y = y + 1.0f;
    int32_t n = (int32_t)fx;                     /* cvttps: fx is integral here */
    float pow2n = u2f((uint32_t)(n + 127) << 23);
    return y * pow2n;
}

/* log256_ps src/cpu/AVX2/ops_avx2_f32.cpp:103-158 (the AVX-512 twin at
 * src/cpu/AVX512/ops_avx512_f32.cpp:95-140 is numerically wrong for mantissas >= 1/sqrt2 and
 * is not followed). */
float orc_log_f32(float x) {
    int invalid = (x <= 0.0f);                   /* _CMP_LE_OQ: false for NaN */
    x = (x > 1.17549435e-38f) ? x : 1.17549435e-38f;   /* max_ps(x, FLT_MIN): NaN -> FLT_MIN */
    uint32_t bits = f2u(x);
    int32_t emm0 = (int32_t)(bits >> 23);
    x = u2f((bits & 0x7fffffu) | f2u(0.5f));
    emm0 -= 127;
    float e = (float)emm0;
    e = e + 1.0f;
    int m = (x < 0.707106781186547524f);
    float tmp = m ? x : 0.0f;
    x = x - 1.0f;
    e = e - (m ? 1.0f : 0.0f);
    x = x + tmp;
    float z = x * x;
    float y = 7.0376836292E-2f;
    y = fmaf(y, x, -1.1514610310E-1f);
    y = fmaf(y, x, 1.1676998740E-1f);
    y = fmaf(y, x, -1.2420140846E-1f);
    y = fmaf(y, x, 1.4249322787E-1f);
    y = fmaf(y, x, -1.6668057665E-1f);
    y = fmaf(y, x, 2.0000714765E-1f);
    y = fmaf(y, x, -2.4999993993E-1f);
    y = fmaf(y, x, 3.3333331174E-1f);
    y = y * x;
    float t = e * -2.12194440e-4f;               /* rounded product ...           */
    y = fmaf(y, z, t);                           /* ... the y*z product is fused  */
    y = fmaf(-z, 0.5f, y);
    x = x + y;
    x = fmaf(e, 0.693359375f, x);
    if (invalid) return u2f(0xFFFFFFFFu);        /* or_ps with an all-ones mask   */
    return x;
}

/* tanh512_ps src/cpu/AVX512/ops_avx512_f32.cpp:187-193 */
float orc_tanh_f32(float x) {
    float e = orc_exp_f32(x * 2.0f);
    return (e - 1.0f) / (e + 1.0f);
}

/* sigmoid512_ps src/cpu/AVX512/ops_avx512_f32.cpp:195-201 (sign flipped by XOR) */
float orc_sigmoid_f32(float x) {
    float e = orc_exp_f32(u2f(f2u(x) ^ 0x80000000u));
    return 1.0f / (1.0f + e);
}

/* GELU, tanh form, as a chain of reference primitives with every step rounded to fp32:
 * mul, mul, mul_scalar(0.044715), add, mul_scalar(sqrt(2/pi)), tanh, add_scalar(1),
 * mul_scalar(x, 0.5), mul.  Scalar steps are done in double and rounded once
 * (src/core/opsmp.cpp:297). */
float orc_gelu_tanh_f32(float x) {
    float u = x * x;
    u = u * x;
    u = (float)((double)u * 0.044715);
    u = x + u;
    u = (float)((double)u * 0.7978845608028654);
    float t = orc_tanh_f32(u);
    t = (float)((double)t + 1.0);
    float h = (float)((double)x * 0.5);
    return h * t;
}

/* ------------------------------------------------------------------------------------------
 * Binary operators with right-aligned broadcasting: binary_op_impl + TensorIterator,
 * src/core/opsmp.cpp:46-129,136-269.  Result: contiguous, broadcast shape, dtype of a,
 * out[i] = (T) op((double)a, (double)b).
 * ---------------------------------------------------------------------------------------- */
static inline double bin_apply(int op, double x, double y) {
    switch (op) {
    case B_ADD: return x + y;
    case B_SUB: return x - y;
    case B_MUL: return x * y;
    case B_DIV: return x / y;
    case B_LT: return x < y ? 1.0 : 0.0;
    case B_LE: return x <= y ? 1.0 : 0.0;
    case B_GT: return x > y ? 1.0 : 0.0;
    case B_GE: return x >= y ? 1.0 : 0.0;
    case B_EQ: return x == y ? 1.0 : 0.0;
    case B_POW: return pow(x, y);                 /* pow_mp, src/core/opsmp.cpp:411-414 */
    default:   return x != y ? 1.0 : 0.0;
    }
}

/* Broadcast shape (src/core/opsmp.cpp:19-40).  Returns ndim or -1 if not broadcastable. */
int orc_broadcast_shape(const orc_view* a, const orc_view* b, int64_t* shape) {
    int nd = a->ndim > b->ndim ? a->ndim : b->ndim;
    for (int i = 0; i < nd; ++i) {
        int64_t da = (i < nd - a->ndim) ? 1 : a->shape[i - (nd - a->ndim)];
        int64_t db = (i < nd - b->ndim) ? 1 : b->shape[i - (nd - b->ndim)];
        if (da != db && da != 1 && db != 1) return -1;
        shape[i] = da > db ? da : db;
    }
    return nd;
}

int64_t orc_binary(int op, const orc_view* a, const orc_view* b, void* out) {
    int64_t shape[ORC_MAX_DIMS], sa[ORC_MAX_DIMS], sb[ORC_MAX_DIMS];
    int nd = orc_broadcast_shape(a, b, shape);
    if (nd < 0) return -1;
    int64_t n = 1;
    for (int i = 0; i < nd; ++i) {
        int ia = i - (nd - a->ndim), ib = i - (nd - b->ndim);
        sa[i] = (ia < 0 || a->shape[ia] == 1) ? 0 : a->stride[ia];
        sb[i] = (ib < 0 || b->shape[ib] == 1) ? 0 : b->stride[ib];
        n *= shape[i];
    }
    int dt = a->dtype;
    #pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; ++i) {
        int64_t t = i, ia = a->offset, ib = b->offset;
        for (int d = nd - 1; d >= 0; --d) {
            int64_t c = t % shape[d];
            t /= shape[d];
            ia += c * sa[d];
            ib += c * sb[d];
        }
        wr(out, i, dt, bin_apply(op, rd(a->base, ia, dt), rd(b->base, ib, dt)));
    }
    return n;
}

/* ------------------------------------------------------------------------------------------
 * Unary operators: unary_op_impl src/core/opsmp.cpp:272-385 with the functors of
 * :418-456 (scalar ops), :701-706 (scalar comparisons), :562-589 (abs, sqrt, relu); the
 * fp32 exp/log/tanh/sigmoid flavours above.
 * ---------------------------------------------------------------------------------------- */
static int unary_needs_f32(int op) {
    return op == U_EXP || op == U_LOG || op == U_TANH || op == U_SIGMOID || op == U_GELU_TANH;
}

static inline double un_apply(int op, double x, double s) {
    switch (op) {
    case U_ADD_S:  return x + s;
    case U_SUB_S:  return x - s;
    case U_RSUB_S: return s - x;
    case U_MUL_S:  return x * s;
    case U_DIV_S:  return x / s;
    case U_RDIV_S: return s / x;
    case U_POW_S:  return pow(x, s);
    case U_RPOW_S: return pow(s, x);
    case U_LT_S: return x < s ? 1.0 : 0.0;
    case U_LE_S: return x <= s ? 1.0 : 0.0;
    case U_GT_S: return x > s ? 1.0 : 0.0;
    case U_GE_S: return x >= s ? 1.0 : 0.0;
    case U_EQ_S: return x == s ? 1.0 : 0.0;
    case U_NE_S: return x != s ? 1.0 : 0.0;
    case U_ABS:  return fabs(x);
    case U_RELU: return x > 0 ? x : 0.0;
    case U_SQRT: return sqrt(x);
    /* libm in double, src/core/opsmp.cpp:566-574,586-589 */
    case U_SIN:  return sin(x);
    case U_COS:  return cos(x);
    case U_TAN:  return tan(x);
    case U_ASIN: return asin(x);
    case U_ACOS: return acos(x);
    case U_ATAN: return atan(x);
    case U_SINH: return sinh(x);
    case U_COSH: return cosh(x);
    case U_SOFTPLUS: return log(1.0 + exp(x));
    default:     return x;
    }
}

float orc_unary_f32_scalar(int op, float x, double s) {
    switch (op) {
    case U_EXP: return orc_exp_f32(x);
    case U_LOG: return orc_log_f32(x);
    case U_TANH: return orc_tanh_f32(x);
    case U_SIGMOID: return orc_sigmoid_f32(x);
    case U_GELU_TANH: return orc_gelu_tanh_f32(x);
    default: return (float)un_apply(op, (double)x, s);
    }
}

int64_t orc_unary(int op, const orc_view* a, double s, void* out) {
    int dt = a->dtype;
    if (unary_needs_f32(op) && dt != ORC_F32) return -1;
    int64_t n = numel(a);
    int nd = a->ndim;
    #pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; ++i) {
        int64_t t = i, ia = a->offset;
        for (int d = nd - 1; d >= 0; --d) {
            int64_t c = t % a->shape[d];
            t /= a->shape[d];
            ia += c * a->stride[d];
        }
        if (dt == ORC_F32) ((float*)out)[i] = orc_unary_f32_scalar(op, ((const float*)a->base)[ia], s);
        else wr(out, i, dt, un_apply(op, rd(a->base, ia, dt), s));
    }
    return n;
}

/* Evaluate a unary fp32 op on `count` bit patterns start, start+step, ... (for exhaustive or
 * sampled sweeps against the compiled reference). */
void orc_unary_sweep_f32(int op, uint32_t start, uint32_t step, int64_t count, double s,
                         float* in, float* out) {
    #pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < count; ++i) {
        float x = u2f(start + (uint32_t)i * step);
        if (in) in[i] = x;
        out[i] = orc_unary_f32_scalar(op, x, s);
    }
}

/* ------------------------------------------------------------------------------------------
 * Strided gather into contiguous storage: Tensor::clone, src/core/tensor.cpp:60-116.
 * ---------------------------------------------------------------------------------------- */
int64_t orc_contiguous(const orc_view* a, void* out) {
    int64_t n = numel(a);
    int nd = a->ndim;
    size_t es = esize(a->dtype);
    #pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; ++i) {
        int64_t t = i, ia = a->offset;
        for (int d = nd - 1; d >= 0; --d) {
            int64_t c = t % a->shape[d];
            t /= a->shape[d];
            ia += c * a->stride[d];
        }
        memcpy((char*)out + (size_t)i * es, (const char*)a->base + (size_t)ia * es, es);
    }
    return n;
}

/* ------------------------------------------------------------------------------------------
 * Reductions.
 *  - sum/max/min along a dim: reduction_op_impl, src/core/opsmp.cpp:593-670 — fp64
 *    accumulator, elements visited in index order, acc initialised to 0 / -inf / +inf,
 *    std::max(acc,val) = (acc < val) ? val : acc (a NaN val is ignored), result cast to the
 *    input dtype; the reduced dim is removed (1-d input -> shape {1}).
 *  - mean = mult_scalar_mp(sum, 1.0/count): the sum is ROUNDED to the dtype first, then
 *    multiplied in double and rounded again (src/core/opsmp.cpp:693-697).
 *  - var  = mean((x - mean(x))^2) with every intermediate rounded to the dtype
 *    (src/neuralnet/batchnorm/batchnorm.cpp:54-61).
 *  - argmax: first index of the maximum, strict `>`, running maximum initialised to -1e18,
 *    int32 result (src/core/ops_dispatch.cpp:427-526).
 *  - dim == -1: everything is reduced ("full"), i.e. the same rules on the flattened tensor.
 * ---------------------------------------------------------------------------------------- */
static inline double round_dt(double v, int dt) {
    if (dt == ORC_F32) return (double)(float)v;
    if (dt == ORC_I32) return (double)d2i_x86(v);
    if (dt == ORC_F64) return v;
    uint64_t slot = 0;                    /* the other types: through their own store and load */
    wr(&slot, 0, dt, v);
    return rd(&slot, 0, dt);
}

/* element offset of flattened logical index i (used by the full reductions) */
static inline int64_t lin_off(const orc_view* a, int64_t i) {
    int64_t off = a->offset;
    for (int d = a->ndim - 1; d >= 0; --d) {
        int64_t c = i % a->shape[d];
        i /= a->shape[d];
        off += c * a->stride[d];
    }
    return off;
}

static void reduce_line(int op, const orc_view* a, int64_t base, int64_t len, int64_t stride,
                        int full, void* out, int64_t oi) {
    int dt = a->dtype;
    const void* p = a->base;
#define AT(k) (full ? lin_off(a, (k)) : base + (k) * stride)
    if (op == R_ARGMAX) {
        double best = -1e18;
        int32_t bi = 0;
        for (int64_t k = 0; k < len; ++k) {
            double v = rd(p, AT(k), dt);
            if (v > best) { best = v; bi = (int32_t)k; }
        }
        ((int32_t*)out)[oi] = bi;
        return;
    }
    if (op == R_MAX || op == R_MIN) {
        double acc = (op == R_MAX) ? -INFINITY : INFINITY;
        for (int64_t k = 0; k < len; ++k) {
            double v = rd(p, AT(k), dt);
            if (op == R_MAX) acc = (acc < v) ? v : acc;
            else             acc = (v < acc) ? v : acc;
        }
        wr(out, oi, dt, acc);
        return;
    }
    double acc = 0.0;
    for (int64_t k = 0; k < len; ++k) acc += rd(p, AT(k), dt);
    if (op == R_SUM) { wr(out, oi, dt, acc); return; }
    double inv = 1.0 / (double)len;
    double mean = round_dt(round_dt(acc, dt) * inv, dt);
    if (op == R_MEAN) { wr(out, oi, dt, mean); return; }
    /* R_VAR */
    double acc2 = 0.0;
    for (int64_t k = 0; k < len; ++k) {
        double d = round_dt(rd(p, AT(k), dt) - mean, dt);
        acc2 += round_dt(d * d, dt);
    }
    wr(out, oi, dt, round_dt(acc2, dt) * inv);
#undef AT
}

int64_t orc_reduce(int op, const orc_view* a, int dim, void* out) {
    int nd = a->ndim;
    if (dim < -1 || dim >= nd) return -1;
    if (op == R_ARGMAX && dim < 0) return -1;
    if (dim == -1) {
        reduce_line(op, a, 0, numel(a), 0, 1, out, 0);
        return 1;
    }
    int64_t oshape[ORC_MAX_DIMS], ostride[ORC_MAX_DIMS];
    int ond = 0;
    int64_t on = 1;
    for (int d = 0; d < nd; ++d) if (d != dim) { oshape[ond] = a->shape[d]; ostride[ond] = a->stride[d]; on *= a->shape[d]; ++ond; }
    int64_t len = a->shape[dim], rs = a->stride[dim];
    #pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < on; ++i) {
        int64_t t = i, base = a->offset;
        for (int d = ond - 1; d >= 0; --d) {
            int64_t c = t % oshape[d];
            t /= oshape[d];
            base += c * ostride[d];
        }
        reduce_line(op, a, base, len, rs, 0, out, i);
    }
    return on;
}

/* ------------------------------------------------------------------------------------------
 * Softmax over the last dim: the chain of src/neuralnet/loss.cpp:97-101 (max, sub, exp, sum,
 * div; no final log), after an optional broadcast add of `mask` and an optional causal mask
 * (-1e9 where column > row of the last two dims, added as an fp32 tensor would be).
 * Output contiguous fp32 with the broadcast shape of (x, mask).
 * ---------------------------------------------------------------------------------------- */
int64_t orc_softmax_lastdim(const orc_view* x, const orc_view* mask, int causal, void* out) {
    if (x->dtype != ORC_F32 || x->ndim < 1) return -1;
    orc_view xv = *x;
    float* tmp = NULL;
    int64_t n = numel(x);
    if (mask) {
        int64_t shape[ORC_MAX_DIMS];
        int nd = orc_broadcast_shape(x, mask, shape);
        if (nd < 0) return -1;
        n = 1;
        for (int i = 0; i < nd; ++i) n *= shape[i];
        tmp = (float*)malloc((size_t)n * 4);
        if (orc_binary(B_ADD, x, mask, tmp) < 0) { free(tmp); return -1; }
        xv.base = tmp; xv.offset = 0; xv.ndim = nd;
        int64_t st = 1;
        for (int i = nd - 1; i >= 0; --i) { xv.shape[i] = shape[i]; xv.stride[i] = st; st *= shape[i]; }
    }
    int nd = xv.ndim;
    int64_t cols = xv.shape[nd - 1], cs = xv.stride[nd - 1];
    int64_t rows = n / (cols ? cols : 1);
    int64_t qlen = nd >= 2 ? xv.shape[nd - 2] : 1;
    float* o = (float*)out;
    #pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < rows; ++r) {
        int64_t t = r, base = xv.offset;
        for (int d = nd - 2; d >= 0; --d) {
            int64_t c = t % xv.shape[d];
            t /= xv.shape[d];
            base += c * xv.stride[d];
        }
        int64_t q = r % qlen;
        const float* px = (const float*)xv.base;
        float* row = o + r * cols;
        double m = -INFINITY;
        for (int64_t j = 0; j < cols; ++j) {
            float v = px[base + j * cs];
            if (causal) v = v + ((j > q) ? -1e9f : 0.0f);
            row[j] = v;
            m = (m < (double)v) ? (double)v : m;
        }
        float mf = (float)m;
        double z = 0.0;
        for (int64_t j = 0; j < cols; ++j) {
            float e = orc_exp_f32(row[j] - mf);
            row[j] = e;
            z += (double)e;
        }
        float zf = (float)z;
        for (int64_t j = 0; j < cols; ++j) row[j] = row[j] / zf;
    }
    free(tmp);
    return n;
}

/* ------------------------------------------------------------------------------------------
 * LayerNorm over the last dim: the chain of src/neuralnet/batchnorm/batchnorm.cpp:103-113
 * per row: mu = mean(x); d = x - mu; v = mean(d*d); r = pow_scalar(add_scalar(v, eps), -0.5);
 * y = d*r; y = y*gamma; y = y+beta — every step rounded to fp32, scalar steps in double.
 * ---------------------------------------------------------------------------------------- */
int64_t orc_layernorm_lastdim(const orc_view* x, const orc_view* gamma, const orc_view* beta,
                              double eps, void* out) {
    if (x->dtype != ORC_F32 || x->ndim < 1) return -1;
    int nd = x->ndim;
    int64_t n = numel(x), cols = x->shape[nd - 1], cs = x->stride[nd - 1];
    int64_t rows = n / (cols ? cols : 1);
    float* o = (float*)out;
    const float* px = (const float*)x->base;
    const float* pg = gamma ? (const float*)gamma->base + gamma->offset : NULL;
    const float* pb = beta ? (const float*)beta->base + beta->offset : NULL;
    int64_t gs = gamma ? gamma->stride[gamma->ndim - 1] : 0;
    int64_t bs = beta ? beta->stride[beta->ndim - 1] : 0;
    double inv = 1.0 / (double)cols;
    #pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < rows; ++r) {
        int64_t t = r, base = x->offset;
        for (int d = nd - 2; d >= 0; --d) {
            int64_t c = t % x->shape[d];
            t /= x->shape[d];
            base += c * x->stride[d];
        }
        float* row = o + r * cols;
        double acc = 0.0;
        for (int64_t j = 0; j < cols; ++j) acc += (double)px[base + j * cs];
        float mu = (float)((double)(float)acc * inv);
        double acc2 = 0.0;
        for (int64_t j = 0; j < cols; ++j) {
            float d = px[base + j * cs] - mu;
            row[j] = d;
            acc2 += (double)(d * d);
        }
        float v = (float)((double)(float)acc2 * inv);
        float ve = (float)((double)v + eps);
        float rstd = (float)pow((double)ve, -0.5);
        for (int64_t j = 0; j < cols; ++j) {
            float y = row[j] * rstd;
            if (pg) y = y * pg[j * gs];
            if (pb) y = y + pb[j * bs];
            row[j] = y;
        }
    }
    return n;
}

/* ------------------------------------------------------------------------------------------
 * Log-softmax over the last dim: the chain of Loss::CrossEntropy, src/neuralnet/loss.cpp:97-104
 * (max -> sub -> exp -> sum -> ln -> sub), after an optional broadcast add of `mask`.
 * Output contiguous fp32 with the broadcast shape of (x, mask).
 * ---------------------------------------------------------------------------------------- */
int64_t orc_log_softmax_lastdim(const orc_view* x, const orc_view* mask, void* out) {
    if (x->dtype != ORC_F32 || x->ndim < 1) return -1;
    orc_view xv = *x;
    float* tmp = NULL;
    int64_t n = numel(x);
    if (mask) {
        int64_t shape[ORC_MAX_DIMS];
        int nd = orc_broadcast_shape(x, mask, shape);
        if (nd < 0) return -1;
        n = 1;
        for (int i = 0; i < nd; ++i) n *= shape[i];
        tmp = (float*)malloc((size_t)n * 4);
        if (orc_binary(B_ADD, x, mask, tmp) < 0) { free(tmp); return -1; }
        xv.base = tmp; xv.offset = 0; xv.ndim = nd;
        int64_t st = 1;
        for (int i = nd - 1; i >= 0; --i) { xv.shape[i] = shape[i]; xv.stride[i] = st; st *= shape[i]; }
    }
    int nd = xv.ndim;
    int64_t cols = xv.shape[nd - 1], cs = xv.stride[nd - 1];
    int64_t rows = n / (cols ? cols : 1);
    float* o = (float*)out;
    #pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < rows; ++r) {
        int64_t t = r, base = xv.offset;
        for (int d = nd - 2; d >= 0; --d) {
            int64_t c = t % xv.shape[d];
            t /= xv.shape[d];
            base += c * xv.stride[d];
        }
        const float* px = (const float*)xv.base;
        float* row = o + r * cols;
        double m = -INFINITY;
        for (int64_t j = 0; j < cols; ++j) {
            float v = px[base + j * cs];
            m = (m < (double)v) ? (double)v : m;
        }
        float mf = (float)m;
        double z = 0.0;
        for (int64_t j = 0; j < cols; ++j) {
            float sh = px[base + j * cs] - mf;
            row[j] = sh;
            z += (double)orc_exp_f32(sh);
        }
        float lz = orc_log_f32((float)z);
        for (int64_t j = 0; j < cols; ++j) row[j] = row[j] - lz;
    }
    free(tmp);
    return n;
}

/* ------------------------------------------------------------------------------------------
 * Tensor::gather, src/core/tensor.cpp:344-428: out[i] = x[coords(i) with coordinate `dim`
 * replaced by index[i]]; negative indices count from the end.  Returns the element count,
 * -1 for a malformed call, -2 for an index out of bounds (the reference throws).
 * ---------------------------------------------------------------------------------------- */
int64_t orc_gather(const orc_view* x, int dim, const orc_view* index, void* out) {
    if (dim < 0 || dim >= x->ndim || x->ndim != index->ndim || index->dtype != ORC_I32) return -1;
    int nd = x->ndim;
    for (int d = 0; d < nd; ++d)
        if (d != dim && index->shape[d] > x->shape[d]) return -1;
    int64_t n = numel(index);
    const int32_t* pi = (const int32_t*)index->base;
    for (int64_t i = 0; i < n; ++i) {
        int64_t t = i, xoff = x->offset, ioff = index->offset;
        for (int d = nd - 1; d >= 0; --d) {
            int64_t c = t % index->shape[d];
            t /= index->shape[d];
            ioff += c * index->stride[d];
            if (d != dim) xoff += c * x->stride[d];
        }
        int64_t idx = pi[ioff];
        if (idx < 0) idx += x->shape[dim];
        if (idx < 0 || idx >= x->shape[dim]) return -2;
        xoff += idx * x->stride[dim];
        memcpy((char*)out + (size_t)i * esize(x->dtype), (const char*)x->base + (size_t)xoff * esize(x->dtype), esize(x->dtype));
    }
    return n;
}

/* ------------------------------------------------------------------------------------------
 * accumulate_grad, src/core/autograd.cpp:63-156: the dims in which the target has extent 1
 * (or which it lacks) and the source has more are summed (sum() per axis: fp64 accumulation,
 * rounded to the dtype after every axis), then grad[i] = (T)((double)grad[i] + (double)g[i])
 * for every finite g[i].  `grad` is the target's gradient buffer, contiguous, updated in
 * place; tshape/tnd give the target's shape.  (The reference folds the axes in increasing
 * order with indices that are only right for a single folded axis; here every flagged axis is
 * folded, last axis first.)
 * ---------------------------------------------------------------------------------------- */
int64_t orc_accumulate_grad(void* grad, const int64_t* tshape, int tnd, const orc_view* src) {
    int nd = tnd > src->ndim ? tnd : src->ndim;
    int dt = src->dtype;
    int64_t ts[ORC_MAX_DIMS], ss[ORC_MAX_DIMS];
    for (int d = 0; d < nd; ++d) {
        int jt = d - (nd - tnd), js = d - (nd - src->ndim);
        ts[d] = jt < 0 ? 1 : tshape[jt];
        ss[d] = js < 0 ? 1 : src->shape[js];
        if (ts[d] != ss[d] && ts[d] != 1 && ss[d] != 1) return -1;
    }
    /* contiguous working copy of the source */
    int64_t n = numel(src);
    size_t es = esize(dt);
    void* cur = malloc((size_t)(n ? n : 1) * es);
    if (orc_contiguous(src, cur) < 0) { free(cur); return -1; }
    int64_t cs[ORC_MAX_DIMS];
    for (int d = 0; d < nd; ++d) cs[d] = ss[d];
    for (int ax = nd - 1; ax >= 0; --ax) {
        if (!(ts[ax] == 1 && cs[ax] > 1)) continue;
        int64_t outer = 1, inner = 1, len = cs[ax];
        for (int d = 0; d < ax; ++d) outer *= cs[d];
        for (int d = ax + 1; d < nd; ++d) inner *= cs[d];
        int64_t on = outer * inner;
        void* nxt = malloc((size_t)(on > 0 ? on : 1) * es);
        for (int64_t o = 0; o < outer; ++o)
            for (int64_t i = 0; i < inner; ++i) {
                double acc = 0.0;
                for (int64_t k = 0; k < len; ++k) acc += rd(cur, (o * len + k) * inner + i, dt);
                wr(nxt, o * inner + i, dt, acc);
            }
        free(cur);
        cur = nxt;
        cs[ax] = 1;
    }
    /* element-wise accumulation with broadcasting of the (reduced) source */
    int64_t tn = 1;
    for (int d = 0; d < nd; ++d) tn *= ts[d];
    for (int64_t i = 0; i < tn; ++i) {
        int64_t t = i, soff = 0, run = 1;
        int64_t sstr[ORC_MAX_DIMS];
        for (int d = nd - 1; d >= 0; --d) { sstr[d] = cs[d] == 1 ? 0 : run; run *= cs[d]; }
        for (int d = nd - 1; d >= 0; --d) {
            int64_t c = t % ts[d];
            t /= ts[d];
            soff += c * sstr[d];
        }
        double g = rd(cur, soff, dt);
        if (!isfinite(g)) continue;
        wr(grad, i, dt, rd(grad, i, dt) + g);
    }
    free(cur);
    return tn;
}

/* ------------------------------------------------------------------------------------------
 * Optimizer steps, src/neuralnet/train_utils.h:50-188, in place on contiguous buffers.
 * SGD: fp32 fast path p -= (float)lr*g (:66-68), other dtypes through double (:72-76).
 * Adam / AdamW (fp32): :113-127 / :176-184.  `step` is the 1-based step count.
 * ---------------------------------------------------------------------------------------- */
void orc_sgd_step(int dtype, void* p, const void* g, int64_t n, double lr) {
    if (dtype == ORC_F32) {
        float* pp = (float*)p;
        const float* gg = (const float*)g;
        for (int64_t i = 0; i < n; ++i) pp[i] -= (float)lr * gg[i];
    } else {
        for (int64_t i = 0; i < n; ++i) wr(p, i, dtype, rd(p, i, dtype) - lr * rd(g, i, dtype));
    }
}

void orc_adam_step(float* theta, const float* grad, float* m, float* v, int64_t n, double lr,
                   double beta1, double beta2, double eps, int step, double weight_decay,
                   int decoupled_decay) {
    double bc1 = 1.0 - pow(beta1, step), bc2 = 1.0 - pow(beta2, step);
    float lr_t = (float)(lr * sqrt(bc2) / bc1);
    for (int64_t i = 0; i < n; ++i) {
        float g = grad[i];
        if (decoupled_decay) theta[i] -= (float)(lr * weight_decay * theta[i]);
        m[i] = (float)beta1 * m[i] + (1.0f - (float)beta1) * g;
        v[i] = (float)beta2 * v[i] + (1.0f - (float)beta2) * g * g;
        theta[i] -= lr_t * m[i] / (sqrtf(v[i]) + (float)eps);
    }
}

/* ------------------------------------------------------------------------------------------
 * cat_mp, src/core/opsmp.cpp:717-804 (its element-wise path, which also covers what the
 * contiguous fast path does): out is contiguous with the inputs' shape and the extents along
 * `dim` added up.  Returns the output element count, -1 for a malformed call.
 * ---------------------------------------------------------------------------------------- */
int64_t orc_cat(const orc_view* const* in, int count, int dim, void* out) {
    if (count <= 0) return -1;
    int nd = in[0]->ndim, dt = in[0]->dtype;
    if (dim < 0 || dim >= nd) return -1;
    int64_t oshape[ORC_MAX_DIMS], ostride[ORC_MAX_DIMS], total = 0;
    for (int i = 0; i < count; ++i) {
        if (in[i]->ndim != nd || in[i]->dtype != dt) return -1;
        for (int d = 0; d < nd; ++d)
            if (d != dim && in[i]->shape[d] != in[0]->shape[d]) return -1;
        total += in[i]->shape[dim];
    }
    for (int d = 0; d < nd; ++d) oshape[d] = d == dim ? total : in[0]->shape[d];
    int64_t run = 1;
    for (int d = nd - 1; d >= 0; --d) { ostride[d] = run; run *= oshape[d]; }
    int64_t at = 0;
    for (int i = 0; i < count; ++i) {
        int64_t n = numel(in[i]);
        for (int64_t j = 0; j < n; ++j) {
            int64_t t = j, src = in[i]->offset, dst = 0;
            for (int d = nd - 1; d >= 0; --d) {
                int64_t c = t % in[i]->shape[d];
                t /= in[i]->shape[d];
                src += c * in[i]->stride[d];
                dst += (c + (d == dim ? at : 0)) * ostride[d];
            }
            memcpy((char*)out + (size_t)dst * esize(dt), (const char*)in[i]->base + (size_t)src * esize(dt), esize(dt));
        }
        at += in[i]->shape[dim];
    }
    return run;
}

/* ------------------------------------------------------------------------------------------
 * BatchNorm forward for a contiguous fp32 x[N, C, S], src/neuralnet/batchnorm/batchnorm.cpp.
 * Statistics (:46-61): mean = mean(x over n, s); var = mean((x - mean)^2), both with the
 * reference's mean = (float)((double)(float)sum * (1.0/count)) and fp32 element-wise steps.
 * Normalisation (:103-113): y = ((x - mean) * pow_scalar(add_scalar(var, eps), -0.5)) * gamma + beta.
 * ---------------------------------------------------------------------------------------- */
void orc_channel_moments(const float* x, int64_t N, int64_t C, int64_t S, float* mean, float* var) {
    double count = (double)(N * S), inv = 1.0 / count;
    #pragma omp parallel for schedule(static)
    for (int64_t c = 0; c < C; ++c) {
        double acc = 0.0;
        for (int64_t n = 0; n < N; ++n)
            for (int64_t s = 0; s < S; ++s) acc += (double)x[(n * C + c) * S + s];
        float mu = (float)((double)(float)acc * inv);
        double acc2 = 0.0;
        for (int64_t n = 0; n < N; ++n)
            for (int64_t s = 0; s < S; ++s) {
                float d = x[(n * C + c) * S + s] - mu;
                acc2 += (double)(d * d);
            }
        mean[c] = mu;
        var[c] = (float)((double)(float)acc2 * inv);
    }
}

void orc_batchnorm_apply(const float* x, int64_t N, int64_t C, int64_t S, const float* mean, const float* var,
                         const float* gamma, const float* beta, double eps, float* out) {
    #pragma omp parallel for schedule(static)
    for (int64_t line = 0; line < N * C; ++line) {
        int64_t c = line % C;
        float ve = (float)((double)var[c] + eps);
        float rstd = (float)pow((double)ve, -0.5);
        for (int64_t s = 0; s < S; ++s) {
            float y = (x[line * S + s] - mean[c]) * rstd;
            if (gamma) y = y * gamma[c];
            if (beta) y = y + beta[c];
            out[line * S + s] = y;
        }
    }
}

/* ------------------------------------------------------------------------------------------
 * matmul_mp, src/core/opsmp.cpp:460-558: 2-d operands or 3-d with one leading batch dim.
 * Float32: fp32 accumulation, k ascending, unfused (the reference's k blocks of 64 store and
 * reload the fp32 partial sum: the same sequence).  Other dtypes: double products and sum.
 * out: contiguous [batch, M, N].  Returns the element count or -1.
 * ---------------------------------------------------------------------------------------- */
int64_t orc_matmul(const orc_view* a, const orc_view* b, void* out) {
    if (a->ndim < 2 || b->ndim < 2 || a->ndim > 3 || b->ndim > 3 || a->dtype != b->dtype) return -1;
    int64_t K = a->shape[a->ndim - 1], M = a->shape[a->ndim - 2], N = b->shape[b->ndim - 1];
    if (b->shape[b->ndim - 2] != K) return -1;
    int64_t ba = a->ndim == 3 ? a->shape[0] : 1, bb = b->ndim == 3 ? b->shape[0] : 1;
    int64_t batch = ba > bb ? ba : bb;
    if ((ba != batch && ba != 1) || (bb != batch && bb != 1)) return -1;
    int64_t sa = (a->ndim == 3 && ba > 1) ? a->stride[0] : 0, sb = (b->ndim == 3 && bb > 1) ? b->stride[0] : 0;
    int64_t am = a->stride[a->ndim - 2], ak = a->stride[a->ndim - 1];
    int64_t bk = b->stride[b->ndim - 2], bn = b->stride[b->ndim - 1];
    int dt = a->dtype;
    #pragma omp parallel for collapse(2) schedule(static)
    for (int64_t bi = 0; bi < batch; ++bi)
        for (int64_t m = 0; m < M; ++m)
            for (int64_t n = 0; n < N; ++n) {
                int64_t ia = a->offset + bi * sa + m * am, ib = b->offset + bi * sb + n * bn;
                if (dt == ORC_F32) {
                    const float* pa = (const float*)a->base;
                    const float* pb = (const float*)b->base;
                    float sum = 0.0f;
                    for (int64_t k = 0; k < K; ++k) sum += pa[ia + k * ak] * pb[ib + k * bk];
                    ((float*)out)[(bi * M + m) * N + n] = sum;
                } else {
                    double sum = 0.0;
                    for (int64_t k = 0; k < K; ++k) sum += rd(a->base, ia + k * ak, dt) * rd(b->base, ib + k * bk, dt);
                    wr(out, (bi * M + m) * N + n, dt, sum);
                }
            }
    return batch * M * N;
}

/* The other optimizers of src/neuralnet/train_utils.h (fp32): kind 3 Adamax :190-239, 4 NAdam
 * :241-291, 5 RAdam :293-355, 6 RMSprop :357-396, 7 Adagrad :398-437, 8 Lion :439-494.
 * s1/s2 are the state vectors (m/u, m/v, m/v, v, sum_sq, m). */
void orc_optimizer_step(int kind, float* theta, const float* grad, float* s1, float* s2, int64_t n,
                        double lr, double beta1, double beta2, double eps, double weight_decay,
                        double alpha, int t) {
    double bc1 = 1.0 - pow(beta1, t), bc2 = 1.0 - pow(beta2, t);
    if (kind == 3) {
        float step_size = (float)(lr / bc1);
        for (int64_t i = 0; i < n; ++i) {
            float g = grad[i];
            s1[i] = (float)beta1 * s1[i] + (1.0f - (float)beta1) * g;
            float x = (float)beta2 * s2[i], y = fabsf(g);
            s2[i] = (x < y) ? y : x;
            theta[i] -= step_size * s1[i] / (s2[i] + (float)eps);
        }
    } else if (kind == 4) {
        float step_size = (float)(lr * sqrt(bc2) / bc1);
        for (int64_t i = 0; i < n; ++i) {
            float g = grad[i];
            s1[i] = (float)beta1 * s1[i] + (1.0f - (float)beta1) * g;
            s2[i] = (float)beta2 * s2[i] + (1.0f - (float)beta2) * g * g;
            float mn = (float)beta1 * s1[i] + (1.0f - (float)beta1) * g;
            theta[i] -= step_size * mn / (sqrtf(s2[i]) + (float)eps);
        }
    } else if (kind == 5) {
        float rho_inf = 2.0f / (1.0f - (float)beta2) - 1.0f;
        float rho_t = rho_inf - 2.0f * t * pow(beta2, t) / (1.0f - pow(beta2, t));
        for (int64_t i = 0; i < n; ++i) {
            float g = grad[i];
            s1[i] = (float)beta1 * s1[i] + (1.0f - (float)beta1) * g;
            s2[i] = (float)beta2 * s2[i] + (1.0f - (float)beta2) * g * g;
            float m_hat = s1[i] / (float)bc1;
            if (rho_t > 4.0f) {
                float v_hat = sqrtf(s2[i] / (float)bc2) + (float)eps;
                float rect = sqrtf(((rho_t - 4.0f) * (rho_t - 2.0f) * rho_inf) / ((rho_inf - 4.0f) * (rho_inf - 2.0f) * rho_t));
                theta[i] -= (float)lr * rect * m_hat / v_hat;
            } else {
                theta[i] -= (float)lr * m_hat;
            }
        }
    } else if (kind == 6) {
        for (int64_t i = 0; i < n; ++i) {
            float g = grad[i];
            s1[i] = (float)alpha * s1[i] + (1.0f - (float)alpha) * g * g;
            theta[i] -= (float)lr * g / (sqrtf(s1[i]) + (float)eps);
        }
    } else if (kind == 7) {
        for (int64_t i = 0; i < n; ++i) {
            float g = grad[i];
            s1[i] += g * g;
            theta[i] -= (float)lr * g / (sqrtf(s1[i]) + (float)eps);
        }
    } else if (kind == 8) {
        float b1 = (float)beta1, b2 = (float)beta2, lr_decay = (float)(lr * weight_decay), lr_f = (float)lr;
        for (int64_t i = 0; i < n; ++i) {
            float g = grad[i], m_t = s1[i];
            if (weight_decay > 0) theta[i] -= lr_decay * theta[i];
            float c_t = b1 * m_t + (1.0f - b1) * g;
            float sign_ct = (c_t > 0.0f) ? 1.0f : ((c_t < 0.0f) ? -1.0f : 0.0f);
            theta[i] -= lr_f * sign_ct;
            s1[i] = b2 * m_t + (1.0f - b2) * g;
        }
    }
}

/* ------------------------------------------------------------------------------------------
 * GradCrossEntropy::backward, src/neuralnet/loss.cpp:319-370, restated loop for loop:
 * out[b, c] = (exp(x[b,c] - max_b) / sum_b - (c == label[b])) * scale, with the row maximum
 * started at -1e9f, libm's single-precision exp, the row sum accumulated in fp32 in class order,
 * one reciprocal per row (0 when the sum is <= 1e-12) and `scale` = grad_out (/ batch for the
 * mean reduction) rounded to fp32.  x: contiguous fp32 [batch, classes]; labels: int32[batch].
 * ---------------------------------------------------------------------------------------- */
void orc_cross_entropy_backward(const float* x, const int32_t* labels, int64_t batch, int64_t classes, int mean,
                                double grad_out, float* out) {
    if (mean) grad_out /= (double)batch;
    const float scale = (float)grad_out;
#pragma omp parallel for
    for (int64_t b = 0; b < batch; ++b) {
        const float* row = x + b * classes;
        float* g = out + b * classes;
        float max_val = -1e9f;
        for (int64_t c = 0; c < classes; ++c)
            if (row[c] > max_val) max_val = row[c];
        float sum_exp = 0.0f;
        for (int64_t c = 0; c < classes; ++c) {
            const float v = expf(row[c] - max_val);
            g[c] = v;
            sum_exp += v;
        }
        const int label = labels[b];
        const float inv_sum = (sum_exp > 1e-12f) ? (1.0f / sum_exp) : 0.0f;
        for (int64_t c = 0; c < classes; ++c) {
            float prob = g[c] * inv_sum;
            if ((int)c == label) prob -= 1.0f;
            g[c] = prob * scale;
        }
    }
}
