/*
 * ctb200.h — C ABI of the B200 (sm_100a) elementwise / broadcast / reduction operator path.
 *
 * This is the boundary a maintainer of the reference (ZYROS-OFFICIEL/CTensor) binds at the
 * place the reference already left a hook: the `device().is_cpu()` test followed by
 * `throw "...: unsupported device"` in src/core/ops_dispatch.cpp:206-212,295-311,362-376.
 * Every entry point takes plain pointers, sizes and a CUDA stream handle; no C++ or torch
 * type crosses it.  All pointers inside a `ctb_view` are DEVICE pointers unless the entry
 * point's name ends in `_host`.
 *
 * Conventions
 *  - Return value: 0 (CTB_OK) or a ctb_status code; ctb_last_error() gives the message of the
 *    last failing call on this host thread.  The messages equal the reference's exception
 *    texts ("binary_op: null input", "Shape mismatch in binary op", ...), so a C++ shim can
 *    re-throw them unchanged.  Nothing in device code aborts, traps or waits on another block.
 *  - Calls are asynchronous on `stream` (a cudaStream_t passed as void*; NULL = the legacy
 *    default stream).  The caller synchronises.  The `_host` entry points are synchronous.
 *  - Shapes and strides are in ELEMENTS, strides are non-negative, at most CTB_MAX_DIMS dims —
 *    the layout of the reference's Tensorimpl (src/core/tensor.h:322-358).
 *  - `out` views must be contiguous row-major (every reference op writes a fresh contiguous
 *    tensor: src/core/opsmp.cpp:148,277,607) and must not overlap an input: such a call is
 *    refused with CTB_ERR_ARG (in-place entry points say so explicitly).
 *  - There is no CPU fallback: without a CUDA device every compute entry point fails with
 *    CTB_ERR_CUDA.
 */
#ifndef CTB200_H
#define CTB200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define CTB_MAX_DIMS 8
#define CTB_ABI_VERSION 1

/* Element types; numbering follows the reference's DType enum (src/core/tensor.h:23-25).
 * Float32, Int32 and Double64 run on every kernel shape.  The other integer types and Bool are
 * what the reference's scalar back-end handles through double (read_scalar_at / write_scalar_at,
 * src/core/tensor.h:54-86; its dispatcher refuses them, src/core/ops_dispatch.cpp:206-209):
 * ctb_binary, ctb_unary (the operators evaluated in double), ctb_reduce and the copies accept
 * UInt8, Int8, Int16, Int64 and Bool on the general strided kernels, with the stores of x86
 * static_cast (8- and 16-bit types: the low bits of the truncated 32-bit integer; Int64:
 * INT64_MIN outside its range; Bool: value != 0).  UInt16, UInt32 and UInt64 can only be copied:
 * the reference itself cannot store them (write_scalar_at has no case for them). */
enum ctb_dtype {
    CTB_F32 = 0, CTB_I32 = 1, CTB_F64 = 2, CTB_U8 = 3, CTB_U16 = 4, CTB_U32 = 5, CTB_U64 = 6,
    CTB_I8 = 7, CTB_I16 = 8, CTB_I64 = 9, CTB_BOOL = 10
};

enum ctb_status {
    CTB_OK = 0,
    CTB_ERR_NULL = 1,      /* null view / null base pointer            */
    CTB_ERR_SHAPE = 2,     /* shapes not broadcastable / out mismatch  */
    CTB_ERR_DTYPE = 3,     /* unsupported dtype for this op            */
    CTB_ERR_DIM = 4,       /* reduction dim out of range               */
    CTB_ERR_ARG = 5,       /* bad op code, ndim, negative stride, ...  */
    CTB_ERR_CUDA = 6,      /* CUDA runtime error (no device, launch)   */
    CTB_ERR_WORKSPACE = 7, /* caller workspace too small / misaligned  */
    CTB_ERR_LIMIT = 8      /* size beyond a documented fixed maximum   */
};

/* A strided N-d view: replaces (Tensorimpl::data, offset, shape, strides, dtype),
 * src/core/tensor.h:322-337; Gen-1 twin tensor1.h:77-189. */
typedef struct ctb_view {
    void*   base;                   /* start of the storage buffer                     */
    int64_t offset;                 /* element offset of the view's first element      */
    int32_t dtype;                  /* enum ctb_dtype                                   */
    int32_t ndim;                   /* 0..CTB_MAX_DIMS (0 = one element)               */
    int64_t shape[CTB_MAX_DIMS];
    int64_t stride[CTB_MAX_DIMS];   /* elements; 0 allowed (broadcast)                 */
} ctb_view;

/* Binary operators: add/sub/mul/div — src/core/ops_dispatch.cpp:219-233 -> add_mp..div_mp
 * src/core/opsmp.cpp:391-409 (Gen 1: add_/diff_/mult_/div_ ops1.cpp:149-444, *_mp root
 * opsmp.cpp:178-196); comparisons — src/core/ops_dispatch.cpp:342-347, opsmp.cpp:708-713
 * (result 1.0/0.0 in the dtype of `a`). */
enum ctb_binary_op {
    CTB_ADD = 0, CTB_SUB = 1, CTB_MUL = 2, CTB_DIV = 3,
    CTB_LT = 4, CTB_LE = 5, CTB_GT = 6, CTB_GE = 7, CTB_EQ = 8, CTB_NE = 9,
    CTB_POW = 10,          /* pow_mp, src/core/opsmp.cpp:411-414: std::pow in double, rounded once */
    CTB_BINARY_OP_COUNT
};

/* Unary operators.  *_S take the `scalar` argument (a double, applied in double precision
 * and rounded once: src/core/opsmp.cpp:297,418-456); comparisons with a scalar
 * src/core/opsmp.cpp:701-706; math ops src/core/ops_dispatch.cpp:319-335.
 * For CTB_F32 the transcendental flavours are the reference's SIMD Cephes polynomials as its
 * shipped flags compile them: exp/tanh/sigmoid src/cpu/AVX512/ops_avx512_f32.cpp:63-92,
 * 187-201; log src/cpu/AVX2/ops_avx2_f32.cpp:103-158.  CTB_GELU_TANH is the tanh-form GELU
 * written as a chain of those primitives with every step rounded to fp32. */
enum ctb_unary_op {
    CTB_ADD_S = 0, CTB_SUB_S = 1, CTB_RSUB_S = 2, CTB_MUL_S = 3, CTB_DIV_S = 4, CTB_RDIV_S = 5,
    CTB_POW_S = 6, CTB_RPOW_S = 7,
    CTB_LT_S = 8, CTB_LE_S = 9, CTB_GT_S = 10, CTB_GE_S = 11, CTB_EQ_S = 12, CTB_NE_S = 13,
    CTB_ABS = 14, CTB_RELU = 15, CTB_EXP = 16, CTB_LOG = 17, CTB_TANH = 18, CTB_SIGMOID = 19,
    CTB_SQRT = 20, CTB_GELU_TANH = 21,
    /* The remaining unary set of the reference (src/core/opsmp.cpp:566-589): evaluated like its
     * scalar path, i.e. the double-precision libm function of (double)x rounded once to the
     * tensor's dtype.  CUDA's and glibc's libm can differ in the last bit of a double, so these
     * agree with the reference to ~1e-7 relative rather than bit for bit.  (The reference's SIMD
     * sin/cos polynomials, src/cpu/AVX512/ops_avx512_f32.cpp:143-185, compute x*cos(x)-like
     * values and are not followed.) */
    CTB_SIN = 22, CTB_COS = 23, CTB_TAN = 24, CTB_ASIN = 25, CTB_ACOS = 26, CTB_ATAN = 27,
    CTB_SINH = 28, CTB_COSH = 29, CTB_SOFTPLUS = 30,
    CTB_UNARY_OP_COUNT
};

/* Reductions: sum/mean src/core/ops_dispatch.cpp:360-390, opsmp.cpp:672-677,693-697;
 * max/min :392-424, opsmp.cpp:679-691; argmax :427-526 (int32 out, first maximum);
 * var = biased variance, the recipe of src/neuralnet/batchnorm/batchnorm.cpp:54-61. */
enum ctb_reduce_op {
    CTB_SUM = 0, CTB_MEAN = 1, CTB_MAX = 2, CTB_MIN = 3, CTB_VAR = 4, CTB_ARGMAX = 5,
    CTB_REDUCE_OP_COUNT
};

#define CTB_DIM_FULL (-1)   /* "reduce everything" (the reference's API-level dim = -1) */

/* ---- library ---------------------------------------------------------------------------- */
int         ctb_abi_version(void);
const char* ctb_last_error(void);
/* Number of CUDA devices visible to the library (0 when there is none). */
int         ctb_device_count(void);

/* ---- memory: replaces Storage::allocate, src/core/tensor.cpp:18-39 (calloc) --------------- */
/* Stream-ordered allocation from the device's memory pool; `zero` != 0 clears the buffer
 * (the reference's calloc promise for Tensor::zeros / fresh tensors). */
int ctb_alloc(void** ptr, size_t bytes, int zero, void* stream);
int ctb_free(void* ptr, void* stream);
int ctb_sync(void* stream);
/* Host-dereferenceable storage for callers that read tensor memory on the CPU between
 * operators (the reference's own unfinished CUDA allocator chose cudaMallocManaged too:
 * src/core/tensor.h:274).  Synchronous; `zero` != 0 clears the buffer. */
int ctb_alloc_managed(void** ptr, size_t bytes, int zero);
int ctb_free_managed(void* ptr);
/* The pooled form of the above: what Storage::allocate should call for every operator result.
 * The reference sketches it (a size-bucketed pool of managed blocks rounded to 512 bytes,
 * src/core/tensor.h:253-289, behind Storage::allocate, src/core/tensor.cpp:18-39) but never
 * finishes it.  ctb_pool_alloc_managed returns a block of at least `bytes` bytes of managed
 * memory whose preferred location is `device`: a cached block of the same rounded size when one
 * is free (no driver call, pages already resident in HBM), a new cudaMallocManaged block
 * otherwise.  `zero` != 0 clears it on `stream` (only Tensor::zeros / fresh tensors promise
 * zeros; operator outputs are overwritten anyway and skip the extra pass).
 * ctb_pool_free_managed returns a block to its device's free list; it never waits for the
 * device, so the caller's next use of the memory must be ordered after the last kernel that
 * touched it (one stream per device gives that).  ctb_pool_trim frees the cached blocks of one
 * device (-1: all); ctb_pool_set_limit bounds the idle bytes a device keeps (default 64 GiB). */
typedef struct ctb_pool_info {
    size_t   live_bytes;      /* handed out and not yet returned            */
    size_t   cached_bytes;    /* idle in the free lists                     */
    size_t   cached_blocks;
    uint64_t hits, misses;    /* allocations served from / past the cache   */
    uint64_t trims;           /* cached blocks given back to the driver     */
} ctb_pool_info;
int ctb_pool_alloc_managed(void** ptr, size_t bytes, int zero, int device, void* stream);
int ctb_pool_free_managed(void* ptr);
int ctb_pool_trim(int device);
int ctb_pool_set_limit(int device, size_t cached_bytes);
int ctb_pool_stats(int device, ctb_pool_info* info);
/* Ask for the pages of a managed range to be moved to `device` ahead of the first kernel
 * (advisory; a no-op where the platform cannot prefetch managed memory). */
int ctb_prefetch_managed(void* ptr, size_t bytes, int device, void* stream);
/* Select the CUDA device of the calling host thread / wait for all work on it. */
int ctb_set_device(int index);
int ctb_device_sync(void);

/* ---- elementwise -------------------------------------------------------------------------- */
/* out = a (op) b with NumPy-style right-aligned broadcasting (src/core/opsmp.cpp:19-40);
 * `out` has the broadcast shape and the dtype of `a`; `b` must have the dtype of `a`. */
int ctb_binary(int op, const ctb_view* a, const ctb_view* b, const ctb_view* out, void* stream);

/* out[i] = f(a[i], scalar); `out` has the shape and dtype of `a`. */
int ctb_unary(int op, const ctb_view* a, double scalar, const ctb_view* out, void* stream);

/* Strided gather into contiguous storage: Tensor::contiguous()/clone(),
 * src/core/tensor.cpp:60-116,233-236 (Gen 1 tensor1.cpp:120-178).  Bit copy, any dtype. */
int ctb_copy_strided(const ctb_view* src, const ctb_view* out, void* stream);

/* ---- reductions --------------------------------------------------------------------------- */
/* dim >= 0: reduce that dim, `out` has the input shape without it (no keepdim; a 1-d input
 * gives shape {1}).  dim == CTB_DIM_FULL: reduce everything to one element.  `out` has the
 * dtype of `a`, except CTB_ARGMAX which writes CTB_I32 and needs dim >= 0.
 * Accumulation is fp64 with a fixed combine order, so results are run-to-run identical.
 * max/min return the zero the reference returns when the extreme is a zero of which both signs
 * occur (the first in index order).  Scratch memory for split reductions comes from a
 * per-device workspace the library allocates on first use (cudaMalloc) and keeps — a fresh
 * workspace is cleared on `stream`; calls on one device that share it must be stream-ordered
 * with respect to each other. */
int ctb_reduce(int op, const ctb_view* a, int dim, const ctb_view* out, void* stream);

/* Same, with caller-provided scratch (256-byte aligned device memory of at least
 * ctb_reduce_workspace_bytes(a, dim) bytes; may be NULL when that is 0). */
size_t ctb_reduce_workspace_bytes(const ctb_view* a, int dim);
int ctb_reduce_ws(int op, const ctb_view* a, int dim, const ctb_view* out,
                  void* workspace, size_t workspace_bytes, void* stream);

/* Dim-wise reduction for callers that must not allocate device memory.
 * (No counterpart in the reference, which has no GPU path and therefore no scratch memory.)
 *
 * Who needs it: code that runs where cudaMalloc is off limits — inside a memory-pool or
 * allocator callback, in a real-time or pre-provisioned process whose device memory is fully
 * budgeted at start-up, or in a host that forbids the library's lazily grown workspace
 * because an allocation may synchronise the device or fail late.  ctb_reduce() grows a
 * per-device workspace with cudaMalloc on first use; ctb_reduce_ws() avoids that only if the
 * caller can provide scratch, which such callers cannot.
 *
 * Same semantics and results as ctb_reduce(op, a, dim, out, stream) for dim >= 0.  The scratch
 * of the split reduction kernels (tickets + fp64 partials) lives in a fixed array inside the
 * library's device image, CTB_NOALLOC_SCRATCH_BYTES large; every GPU that loads the library
 * holds that much until the process exits.  A reduction that needs more scratch (a column
 * reduction of more than about 2^18 / splits columns) is refused with CTB_ERR_LIMIT and a
 * message that states both sizes.  Full reductions (CTB_DIM_FULL) are not offered here.
 *
 * The call performs no cudaMalloc/cudaFree and calls no allocating library routine.  The
 * first call on a device looks up the array's device address (cudaGetSymbolAddress); make
 * that first call outside any stream capture.  All calls on a device share the one array and
 * it keeps whatever the previous call left: the part that must start at zero (the tickets) is
 * cleared on `stream` before every launch, and two calls that overlap on the GPU (different
 * streams without an ordering between them) race on it — order them. */
#define CTB_NOALLOC_SCRATCH_BYTES (4u * 1024u * 1024u + 64u * 1024u)
int ctb_reduce_dim_noalloc(int op, const ctb_view* a, int dim, const ctb_view* out, void* stream);

/* Multi-GPU full reductions: the local shard's fp64 partial (sum for CTB_SUM/MEAN, max/min as
 * double for CTB_MAX/MIN) is written to `partial` (one double in device memory).  The caller
 * all-reduces the partials (sum / max / min) across ranks and calls ctb_finalize_full, which
 * applies the reference's rounding: out = (T)partial, and for CTB_MEAN
 * out = (T)((double)(T)partial * (1.0 / total_count)) (src/core/ops_dispatch.cpp:385-390). */
int ctb_reduce_full_partial(int op, const ctb_view* a, double* partial, void* stream);
int ctb_finalize_full(int op, const double* partial, int64_t total_count,
                      const ctb_view* out, void* stream);

/* ---- several GPUs in one process -----------------------------------------------------------
 * (No counterpart in the reference, which is CPU-only; its Device type, src/core/device.h:5-25,
 * names a GPU by index and that is what the `devices` lists here hold.)
 * The path shards along the leading dim: ctb_shard_range gives shard `index` of `parts` of a dim
 * of `total` elements ([lo, hi), sizes differing by at most one).  Elementwise, broadcast and
 * row-wise operators then run per shard with no communication.  ctb_comm_init_all builds one
 * NCCL communicator over `ndev` GPUs (devices == NULL: GPUs 0..ndev-1; ndev <= 0: all visible)
 * with one stream per GPU; NCCL is loaded at that moment (libnccl.so.2, or the library named by
 * the environment variable CTB_NCCL_LIBRARY).  One communicator per process; calling it again
 * replaces the communicator.
 * ctb_allreduce: in-place all-reduce (op = CTB_SUM / CTB_MAX / CTB_MIN) of `count` elements at
 * buffers[r] on the GPU of rank r, queued on the communicator's streams (ctb_comm_stream(r) lets
 * the caller order its own kernels before it; ctb_comm_sync waits for all of them).
 * ctb_full_reduce_sharded: shards[r] (on the GPU of rank r) are the leading-dim shards of one
 * tensor; every GPU reduces its shard to an fp64 partial, ONE all-reduce of a double combines
 * them, every GPU writes the result (outs[r], one element) with the reference's rounding —
 * `total_count` is the element count mean divides by.  Returns when all GPUs are done. */
int   ctb_shard_range(int64_t total, int parts, int index, int64_t* lo, int64_t* hi);
int   ctb_comm_init_all(int ndev, const int* devices);
int   ctb_comm_size(void);
int   ctb_comm_device(int rank);
void* ctb_comm_stream(int rank);
int   ctb_comm_sync(void);
int   ctb_comm_destroy(void);
int   ctb_allreduce(void* const* buffers, size_t count, int dtype, int op);
int   ctb_full_reduce_sharded(int op, const ctb_view* const* shards, int64_t total_count,
                              const ctb_view* const* outs);

/* ---- fused rows ----------------------------------------------------------------------------
 * Softmax over the last dim = the chain max -> sub -> exp -> sum -> div of
 * src/neuralnet/loss.cpp:97-101 in one pass over the rows.  `mask` (may be NULL) is first added
 * with broadcasting (additive bias / mask tensor).  `causal` != 0 additionally adds -1e9 to
 * every element whose last-dim index exceeds its second-to-last-dim index.  fp32 only. */
int ctb_softmax_lastdim(const ctb_view* x, const ctb_view* mask, int causal,
                        const ctb_view* out, void* stream);

/* Log-softmax over the last dim = the chain max -> sub -> exp -> sum -> ln -> sub that
 * Loss::CrossEntropy builds from primitive ops (src/neuralnet/loss.cpp:97-104), one pass over the
 * rows: out = (t - max t) - ln((float)sum exp(t - max t)), t = x (+ mask).  fp32 only. */
int ctb_log_softmax_lastdim(const ctb_view* x, const ctb_view* mask, const ctb_view* out, void* stream);

/* LayerNorm over the last dim = the chain of src/neuralnet/batchnorm/batchnorm.cpp:103-113
 * applied per row: mean, centre, biased variance, (var+eps)^-0.5, scale, shift.
 * gamma/beta: 1-d views of the row length, or NULL.  fp32 only. */
int ctb_layernorm_lastdim(const ctb_view* x, const ctb_view* gamma, const ctb_view* beta,
                          double eps, const ctb_view* out, void* stream);

/* BatchNorm forward, src/neuralnet/batchnorm/batchnorm.cpp:40-113, for a contiguous fp32
 * x[N, C, ...].  ctb_channel_moments: per-channel mean and biased variance over every dim but
 * dim 1 (:46-61; the reference permutes, copies and runs mean / sub / mul / mean).
 * ctb_batchnorm_apply: y = ((x - mean[c]) * (var[c] + eps)^-0.5) * gamma[c] + beta[c] with every
 * step rounded to fp32 and the scalar steps in double (:103-113); mean/var/gamma/beta hold C
 * elements (any view whose other dims are 1, e.g. [C] or [1,C,1,1]); gamma/beta may be NULL.
 * The running-statistics update (:63-86) is C scalar operations and stays with the caller. */
int ctb_channel_moments(const ctb_view* x, const ctb_view* mean, const ctb_view* var, void* stream);
int ctb_batchnorm_apply(const ctb_view* x, const ctb_view* mean, const ctb_view* var,
                        const ctb_view* gamma, const ctb_view* beta, double eps,
                        const ctb_view* out, void* stream);

/* ---- callers either side of the path --------------------------------------------------------
 * Tensor::gather, src/core/tensor.cpp:344-428: out[i] = x[i with coordinate `dim` replaced by
 * index[i]].  `index` has x's number of dims and extents no larger than x's outside `dim`; it may
 * hold any dtype — the reference reads an index through double and truncates it (:385-386; it
 * refuses the floating types at :352-356, the first generation's tensor1.cpp:548-549 takes them
 * too; that check is the caller's).  `out` is contiguous with index's shape and x's dtype, any of
 * the eleven.  Negative indices count from the end.  The reference throws "Gather index out of bounds"; a kernel cannot, so such an element
 * is written as 0 and *bad (one int32 in device memory, may be NULL; cleared on `stream` first)
 * is set to 1 for the caller to test after synchronising. */
int ctb_gather(const ctb_view* x, int dim, const ctb_view* index, const ctb_view* out,
               int32_t* bad, void* stream);

/* accumulate_grad, src/core/autograd.cpp:63-156: grad += src, where every dim in which `grad`
 * has extent 1 (or which it lacks) and `src` has more is summed first (the backward rule of
 * broadcasting), and a NaN or infinite contribution is skipped.  `grad` (in-out) may have any
 * strides; the shapes must be broadcast-compatible.  The folds run as sum reductions (fp64
 * accumulation, rounded to the dtype like the reference's sum()); when `grad` is contiguous the
 * last fold adds into it directly, so a bias gradient is one kernel.  Neighbouring folded dims
 * the source is contiguous across are folded together (the reference folds one axis per pass).
 * Intermediate sums live in the library's per-device workspace (see ctb_reduce). */
int ctb_accumulate_grad(const ctb_view* grad, const ctb_view* src, void* stream);

/* Backward bodies the reference spells as operator chains, one pass each.
 * GradDiv::backward, src/core/autograd.cpp:188-202, for out = a / b with incoming gradient `grad`:
 *   grad_a = grad / b                                   (div)
 *   grad_b = -((grad * a) / ((b * b) + 1e-6))           (mul, mul, add_scalar, div, mul_scalar)
 * GradTanh::backward, src/core/autograd.cpp:434-438, for out = tanh(t):
 *   grad_t = grad * (1 / (cosh t * cosh t))             (cosh, mul, div_scalar_rev, mul)
 * with the chain's rounding points kept (every operator result rounded to the dtype; cosh is the
 * double-precision libm function rounded once, so tanh_backward agrees to ~1e-7).  a, b, t and
 * grad broadcast against the output's shape; either of grad_a / grad_b may be NULL.
 * accumulate == 0: the outputs are fresh contiguous tensors of the broadcast shape (feed them to
 * ctb_accumulate_grad when a broadcast dim has to be folded).  accumulate != 0: the outputs are
 * existing gradient buffers of that shape (any strides) and the result is ADDED into them, NaN /
 * infinite values skipped, which is accumulate_grad's rule (src/core/autograd.cpp:139-151) —
 * the whole backward step of a same-shape division is then two kernels.  Float32 / Double64. */
int ctb_div_backward(const ctb_view* grad, const ctb_view* a, const ctb_view* b, const ctb_view* grad_a,
                     const ctb_view* grad_b, int accumulate, void* stream);
int ctb_tanh_backward(const ctb_view* grad, const ctb_view* t, const ctb_view* grad_t, int accumulate,
                      void* stream);

/* Loss::CrossEntropy, src/neuralnet/loss.cpp:90-118: logits [Batch, Classes] (Float32, classes
 * contiguous), labels: one Int32 class index per row in a [Batch] or [Batch, 1] view (negative
 * values count from the end, like Tensor::gather's indices).  loss (one Float32 element) =
 * mean (mean != 0) or sum over the rows of -(log_softmax(logits)[row, label]) — the chain
 * max -> sub -> exp -> sum -> ln -> sub -> gather -> mul_scalar(-1) -> mean in one pass over the
 * logits plus a reduction of Batch values.  A label outside the row sets *bad (one int32 in device
 * memory, may be NULL; cleared on `stream` first) and contributes 0; the reference throws there.
 * GradCrossEntropy::backward, src/neuralnet/loss.cpp:319-370:
 *   grad_logits[row, c] = (softmax(logits)[row, c] - (c == label[row])) * grad_scale
 * where grad_scale is the loss's incoming gradient, already divided by Batch for the mean
 * reduction (the reference does that division on the host, :337-340).  accumulate as above.
 * Uses the library's per-device workspace (see ctb_reduce). */
int ctb_cross_entropy(const ctb_view* logits, const ctb_view* labels, int mean, const ctb_view* loss,
                      int32_t* bad, void* stream);
int ctb_cross_entropy_backward(const ctb_view* logits, const ctb_view* labels, double grad_scale,
                               const ctb_view* grad_logits, int accumulate, int32_t* bad, void* stream);

/* matmul_mp, src/core/opsmp.cpp:460-558 (the reference's scalar back-end): out = a x b for 2-d
 * operands or 3-d operands with one leading batch dim (an operand without it, or with batch
 * extent 1, is reused for every batch entry); any strides; `out` contiguous [batch, M, N] (or
 * [M, N]).  Float32 accumulates in fp32 with k ascending and no fused multiply-add — bit-identical
 * to matmul_mp; other dtypes accumulate in double.  A plain shared-memory kernel: it exists so
 * that callers of the operator path which also multiply matrices run on the device, not as a
 * tuned GEMM (tensor cores would change the arithmetic). */
int ctb_matmul(const ctb_view* a, const ctb_view* b, const ctb_view* out, void* stream);

/* The same product on the tensor cores (tcgen05.mma, TF32 products, fp32 accumulation in tensor
 * memory, operands staged by TMA): what the reference's SIMD GEMMs are to its scalar one
 * (src/cpu/AVX2/ops_avx2_f32.cpp:650-775 against src/core/opsmp.cpp:460-558) — another summation
 * order and rounding, many times the speed.  Float32 only; same shape rules as ctb_matmul.
 * Tolerance: each product uses the upper 19 bits of its operands (10 mantissa bits), so
 * |out - exact| <= 2^-9 * sum_k |a_ik * b_kj|.  Operands that TMA can read as they lie (unit
 * stride along K — for b that means a transposed view of an [N, K] matrix, which is what
 * Linear::forward passes — 16-byte aligned rows) are used in place; others are packed into the
 * library's workspace first.  `status` (one int32 in device memory, may be NULL; cleared on
 * `stream` first): non-zero afterwards if a bounded wait inside the kernel gave up, in which case
 * `out` is not valid.  sm_100a only; one GPU. */
int ctb_matmul_tc(const ctb_view* a, const ctb_view* b, const ctb_view* out, int32_t* status, void* stream);

/* Copy `src` into the existing (possibly strided) view `dst` of the same shape and dtype; `src`
 * may broadcast.  The building block of cat and of writes into slices. */
int ctb_copy_into(const ctb_view* src, const ctb_view* dst, void* stream);

/* cat_mp, src/core/opsmp.cpp:717-804: concatenate `count` views along `dim` into `out`
 * (contiguous, the inputs' shape with the extents along `dim` added up).  All inputs have the
 * same number of dims, dtype and extents outside `dim`; any strides.  One strided copy per input. */
int ctb_cat(const ctb_view* const* inputs, int count, int dim, const ctb_view* out, void* stream);

/* Optimizer steps, src/neuralnet/train_utils.h:50-188, in place on contiguous buffers.
 * ctb_sgd_step: param -= (float)lr * grad for CTB_F32 (:66-68); (T)(param - lr*grad) in double
 * for the other dtypes (:72-76).
 * ctb_adam_step (CTB_F32 only, like the reference, which skips other dtypes): the update of
 * Adam (:113-127) or, with decoupled_decay != 0, of AdamW (:176-184, which first does
 * param -= (float)(lr*weight_decay*param)).  `m`, `v`: the moment vectors (device memory,
 * param's element count, zero before the first step); `step` is the 1-based step count t. */
int ctb_sgd_step(const ctb_view* param, const ctb_view* grad, double lr, void* stream);
int ctb_adam_step(const ctb_view* param, const ctb_view* grad, float* m, float* v, double lr,
                  double beta1, double beta2, double eps, int step, double weight_decay,
                  int decoupled_decay, void* stream);

/* The other optimizers of src/neuralnet/train_utils.h (fp32 parameters, contiguous, in place):
 * Adamax :190-239 (state1 = m, state2 = u), NAdam :241-291 (m, v), RAdam :293-355 (m, v),
 * RMSprop :357-396 (state1 = v; hyper.alpha), Adagrad :398-437 (state1 = sum of squares),
 * Lion :439-494 (state1 = m; hyper.weight_decay).  state buffers: device memory, param's element
 * count, zero before the first step; state2 may be NULL where unused.  CTB_OPT_SGD / ADAM / ADAMW
 * are routed to ctb_sgd_step / ctb_adam_step.  `step` is the 1-based step count. */
enum ctb_optimizer {
    CTB_OPT_SGD = 0, CTB_OPT_ADAM = 1, CTB_OPT_ADAMW = 2, CTB_OPT_ADAMAX = 3, CTB_OPT_NADAM = 4,
    CTB_OPT_RADAM = 5, CTB_OPT_RMSPROP = 6, CTB_OPT_ADAGRAD = 7, CTB_OPT_LION = 8,
    CTB_OPTIMIZER_COUNT
};
typedef struct ctb_optimizer_hyper {
    double lr, beta1, beta2, eps, weight_decay, alpha;
} ctb_optimizer_hyper;
int ctb_optimizer_step(int kind, const ctb_view* param, const ctb_view* grad, float* state1,
                       float* state2, const ctb_optimizer_hyper* hyper, int step, void* stream);

/* ---- host-buffer entry points ---------------------------------------------------------------
 * Same semantics as ctb_binary / ctb_unary / ctb_reduce, but every view points to HOST memory
 * (pinned memory gives full PCIe speed).  Inputs are staged to `device`, the kernel runs there
 * and the result is copied back before the call returns.  Contiguous same-shape inputs are
 * processed in chunks so that upload, kernel and download overlap.  The calls of one device
 * share its staging buffer and streams: they are serialised inside the library (a second host
 * thread waits), and no copy is left in flight when a call returns, also when it fails. */
int ctb_binary_host(int op, const ctb_view* a, const ctb_view* b, const ctb_view* out, int device);
int ctb_unary_host(int op, const ctb_view* a, double scalar, const ctb_view* out, int device);
int ctb_reduce_host(int op, const ctb_view* a, int dim, const ctb_view* out, int device);

#ifdef __cplusplus
}
#endif
#endif /* CTB200_H */
