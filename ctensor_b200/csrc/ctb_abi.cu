// C ABI of the operator library (declared in include/ctb200.h): argument validation, broadcast
// and collapse planning on the host, dispatch to the kernels, per-device scratch, and the
// host-buffer entry points.  Error texts equal the reference's exception messages
// (src/core/opsmp.cpp:138,144,274,595; src/core/ops_dispatch.cpp:428,433) so a C++ shim can
// re-throw them unchanged.
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <string>
#include <vector>

#include "ctb_common.cuh"
#include "ctb_math.cuh"
#include "ctb_reduce.cuh"
#include "ctb_backward.cuh"

namespace ctb {

// ---- errors ------------------------------------------------------------------------------------
static thread_local std::string g_last_error;

int set_error(int code, const char* fmt, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof buf, fmt, ap);
    va_end(ap);
    g_last_error = buf;
    return code;
}

int cuda_error(cudaError_t e, const char* what) {
    if (e == cudaSuccess) return CTB_OK;
    return set_error(CTB_ERR_CUDA, "CUDA error in %s: %s", what, cudaGetErrorString(e));
}

// ---- per-device state ----------------------------------------------------------------------------
namespace {
constexpr int kMaxDevices = 64;
struct DeviceState {
    bool known = false;
    int sm_count = 0;
    void* ws = nullptr;          // reduction scratch
    size_t ws_bytes = 0;
    void* stage = nullptr;       // staging for the host-buffer entry points
    size_t stage_bytes = 0;
    cudaStream_t streams[3] = {nullptr, nullptr, nullptr};
};
DeviceState g_dev[kMaxDevices];
std::mutex g_mu;
// The host-buffer entry points of one device share its staging buffer and its three streams:
// one such call at a time per device (others wait here).
std::mutex g_host_mu[kMaxDevices];
}  // namespace

int current_device_info(DeviceInfo* info) {
    int dev = -1;
    CTB_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= kMaxDevices) return set_error(CTB_ERR_CUDA, "device index %d out of range", dev);
    std::lock_guard<std::mutex> lk(g_mu);
    DeviceState& s = g_dev[dev];
    if (!s.known) {
        CTB_CUDA_TRY(cudaDeviceGetAttribute(&s.sm_count, cudaDevAttrMultiProcessorCount, dev));
        s.known = true;
    }
    info->device = dev;
    info->sm_count = s.sm_count;
    return CTB_OK;
}

namespace {

// Scratch that grows on demand.  The split kernels need the ticket region at its start to be
// zero; a fresh allocation is cleared ON THE CALLER'S STREAM, so the clear is ordered before the
// kernel that follows whatever kind of stream that is (a clear on the legacy default stream is
// not ordered against non-blocking streams).  Growing frees the old buffer, which waits for
// the device: work of other streams that still used it has finished by then.
int ensure_workspace(size_t bytes, void** out, cudaStream_t st) {
    *out = nullptr;
    if (bytes == 0) return CTB_OK;
    DeviceInfo di;
    int rc = current_device_info(&di);
    if (rc) return rc;
    std::lock_guard<std::mutex> lk(g_mu);
    DeviceState& s = g_dev[di.device];
    if (s.ws_bytes < bytes) {
        size_t want = bytes < (size_t(8) << 20) ? (size_t(8) << 20) : bytes;
        if (s.ws) CTB_CUDA_TRY(cudaFree(s.ws));
        s.ws = nullptr;
        s.ws_bytes = 0;
        CTB_CUDA_TRY(cudaMalloc(&s.ws, want));
        CTB_CUDA_TRY(cudaMemsetAsync(s.ws, 0, kTicketBytes, st));
        s.ws_bytes = want;
    }
    *out = s.ws;
    return CTB_OK;
}

size_t dtype_bytes(int dt) {
    switch (dt) {
    case CTB_F64: case CTB_U64: case CTB_I64: return 8;
    case CTB_U16: case CTB_I16: return 2;
    case CTB_U8: case CTB_I8: case CTB_BOOL: return 1;
    }
    return 4;
}
// A dtype the library knows; what a given operator accepts is decided where it is launched.
bool dtype_ok(int dt) { return dt >= CTB_F32 && dt <= CTB_BOOL; }

int64_t view_numel(const ctb_view* v) {
    int64_t n = 1;
    for (int i = 0; i < v->ndim; ++i) n *= v->shape[i];
    return n;
}

// Largest element index the view can touch + 1, counted from `base` (0 for an empty view).
int64_t view_span(const ctb_view* v) {
    int64_t hi = v->offset;
    for (int i = 0; i < v->ndim; ++i) {
        if (v->shape[i] == 0) return 0;
        hi += (v->shape[i] - 1) * v->stride[i];
    }
    return hi + 1;
}

int check_view(const ctb_view* v, const char* null_msg, const char* who) {
    if (!v) return set_error(CTB_ERR_NULL, "%s", null_msg);
    if (v->ndim < 0 || v->ndim > CTB_MAX_DIMS) return set_error(CTB_ERR_ARG, "%s: ndim %d not in 0..%d", who, v->ndim, CTB_MAX_DIMS);
    if (!v->base) {       // an empty tensor may have no storage at all
        bool empty = false;
        for (int i = 0; i < v->ndim; ++i) if (v->shape[i] == 0) empty = true;
        if (!empty) return set_error(CTB_ERR_NULL, "%s", null_msg);
    }
    if (!dtype_ok(v->dtype)) return set_error(CTB_ERR_DTYPE, "%s: unsupported dtype", who);
    if (v->offset < 0) return set_error(CTB_ERR_ARG, "%s: negative offset", who);
    for (int i = 0; i < v->ndim; ++i)
        if (v->shape[i] < 0 || v->stride[i] < 0) return set_error(CTB_ERR_ARG, "%s: negative shape or stride", who);
    return CTB_OK;
}

// Same rule as Tensor::is_contiguous (src/core/tensor.cpp:244-254): size-1 dims are ignored.
bool view_contiguous(const ctb_view* v) {
    int64_t expect = 1;
    for (int i = v->ndim - 1; i >= 0; --i) {
        if (v->shape[i] > 1) {
            if (v->stride[i] != expect) return false;
            expect *= v->shape[i];
        }
    }
    return true;
}

int check_out(const ctb_view* out, int64_t numel, int dtype, const char* who) {
    int rc = check_view(out, "output: null view", who);
    if (rc) return rc;
    if (out->dtype != dtype) return set_error(CTB_ERR_DTYPE, "%s: output dtype mismatch", who);
    if (view_numel(out) != numel) return set_error(CTB_ERR_SHAPE, "%s: output has %lld elements, expected %lld", who, (long long)view_numel(out), (long long)numel);
    if (!view_contiguous(out)) return set_error(CTB_ERR_SHAPE, "%s: output must be contiguous", who);
    return CTB_OK;
}

// The byte range of storage a view can touch: [lo, hi).
void view_bytes(const ctb_view* v, const char** lo, const char** hi) {
    const size_t es = dtype_bytes(v->dtype);
    const int64_t span = view_span(v);
    *lo = (const char*)v->base + (size_t)v->offset * es;
    *hi = span > v->offset ? (const char*)v->base + (size_t)span * es : *lo;
}

// Every operator writes a FRESH tensor (src/core/opsmp.cpp:148,277,607); the kernels read inputs
// through non-coherent loads and in another order than they write, so an output that overlaps an
// input is refused instead of computed wrongly.
int check_no_alias(const ctb_view* out, const ctb_view* const* in, int nin, const char* who) {
    const char *olo, *ohi;
    view_bytes(out, &olo, &ohi);
    if (olo == ohi) return CTB_OK;
    for (int i = 0; i < nin; ++i) {
        if (!in[i] || !in[i]->base) continue;
        const char *lo, *hi;
        view_bytes(in[i], &lo, &hi);
        if (lo < ohi && olo < hi) return set_error(CTB_ERR_ARG, "%s: the output overlaps an input", who);
    }
    return CTB_OK;
}

inline const void* elem_ptr(const ctb_view* v) {
    return (const char*)v->base + (size_t)v->offset * dtype_bytes(v->dtype);
}
inline void* elem_ptr_mut(const ctb_view* v) {
    return (char*)v->base + (size_t)v->offset * dtype_bytes(v->dtype);
}

// Right-aligned broadcast of up to kMaxOperands inputs, then collapse.
// Returns CTB_ERR_SHAPE if the shapes are not broadcastable (src/core/opsmp.cpp:19-28).
// `dst` (optional): the output is this strided view instead of a fresh contiguous buffer; it must
// have the broadcast shape, and its strides take part in the collapse.
int build_plan(const ctb_view* const* in, int nin, Plan* plan, const ctb_view* dst = nullptr) {
    int nd = 0;
    for (int i = 0; i < nin; ++i) nd = in[i]->ndim > nd ? in[i]->ndim : nd;
    if (dst && dst->ndim > nd) nd = dst->ndim;
    int64_t shape[CTB_MAX_DIMS], stride[kMaxOperands][CTB_MAX_DIMS], ostride[CTB_MAX_DIMS];
    for (int d = 0; d < nd; ++d) {
        int64_t s = 1;
        for (int i = 0; i < nin; ++i) {
            int j = d - (nd - in[i]->ndim);
            int64_t di = j < 0 ? 1 : in[i]->shape[j];
            if (di != 1) {
                if (s != 1 && s != di) return set_error(CTB_ERR_SHAPE, "Shape mismatch in binary op");
                s = di;
            }
        }
        if (dst) {      // the destination fixes the extent; inputs may only broadcast into it
            const int jd = d - (nd - dst->ndim);
            const int64_t dd = jd < 0 ? 1 : dst->shape[jd];
            if (s != 1 && s != dd) return set_error(CTB_ERR_SHAPE, "Shape mismatch in binary op");
            s = dd;
        }
        shape[d] = s;
        for (int i = 0; i < nin; ++i) {
            int j = d - (nd - in[i]->ndim);
            stride[i][d] = (j < 0 || in[i]->shape[j] == 1) ? 0 : in[i]->stride[j];
        }
    }
    // a zero-sized dim anywhere makes the result empty
    int64_t numel = 1;
    for (int d = 0; d < nd; ++d) {
        // broadcasting a size-0 dim against size-1 gives 0
        for (int i = 0; i < nin; ++i) {
            int j = d - (nd - in[i]->ndim);
            if (j >= 0 && in[i]->shape[j] == 0) shape[d] = 0;
        }
        numel *= shape[d];
    }
    if (dst) {
        for (int d = 0; d < nd; ++d) {
            const int j = d - (nd - dst->ndim);
            const int64_t dd = j < 0 ? 1 : dst->shape[j];
            if (dd != shape[d]) return set_error(CTB_ERR_SHAPE, "Shape mismatch in binary op");
            ostride[d] = (j < 0 || dd == 1) ? 0 : dst->stride[j];
        }
    }
    plan->nin = nin;
    plan->numel = numel;
    plan->out_strided = dst ? 1 : 0;
    // drop size-1 dims, merge neighbours
    int k = 0;
    for (int d = 0; d < nd; ++d) {
        if (shape[d] == 1) continue;
        if (k > 0) {
            bool merge = true;
            for (int i = 0; i < nin; ++i)
                if (plan->stride[i][k - 1] != stride[i][d] * shape[d]) merge = false;
            if (dst && plan->ostride[k - 1] != ostride[d] * shape[d]) merge = false;
            if (merge) {
                plan->shape[k - 1] *= shape[d];
                for (int i = 0; i < nin; ++i) plan->stride[i][k - 1] = stride[i][d];
                if (dst) plan->ostride[k - 1] = ostride[d];
                continue;
            }
        }
        plan->shape[k] = shape[d];
        for (int i = 0; i < nin; ++i) plan->stride[i][k] = stride[i][d];
        if (dst) plan->ostride[k] = ostride[d];
        ++k;
    }
    if (k == 0) {
        plan->shape[0] = 1;
        for (int i = 0; i < nin; ++i) plan->stride[i][0] = 0;
        if (dst) plan->ostride[0] = 0;
        k = 1;
    }
    plan->ndim = k;
    return CTB_OK;
}

// Geometry of a reduction over `dim` (>= 0): outer dims in output order, merged where the
// input is contiguous across them.
void reduce_geom_dim(const ctb_view* a, int dim, ReduceGeom* g) {
    memset(g, 0, sizeof *g);
    int k = 0;
    int64_t nout = 1;
    for (int d = 0; d < a->ndim; ++d) {
        if (d == dim) continue;
        nout *= a->shape[d];
        if (a->shape[d] == 1) continue;
        if (k > 0 && g->ostride[k - 1] == a->stride[d] * a->shape[d]) {
            g->oshape[k - 1] *= a->shape[d];
            g->ostride[k - 1] = a->stride[d];
            continue;
        }
        g->oshape[k] = a->shape[d];
        g->ostride[k] = a->stride[d];
        ++k;
    }
    g->nouter = k;
    g->nout = nout;
    g->rlen = a->shape[dim];
    g->rstride = a->shape[dim] == 1 ? 1 : a->stride[dim];
    g->total = g->rlen;
}

// A view is "dense" when it is some permutation of a gap-free block of memory; a full
// reduction of it may then run in memory order (sum/mean/var are order-insensitive at the
// stated tolerance, max/min exactly).
bool view_dense(const ctb_view* a) {
    int idx[CTB_MAX_DIMS], k = 0;
    for (int d = 0; d < a->ndim; ++d) if (a->shape[d] != 1) idx[k++] = d;
    for (int i = 1; i < k; ++i)
        for (int j = i; j > 0 && a->stride[idx[j]] > a->stride[idx[j - 1]]; --j) {
            int t = idx[j]; idx[j] = idx[j - 1]; idx[j - 1] = t;
        }
    int64_t expect = 1;
    for (int i = k - 1; i >= 0; --i) {
        if (a->stride[idx[i]] != expect) return false;
        expect *= a->shape[idx[i]];
    }
    return true;
}

void reduce_geom_full_dense(const ctb_view* a, ReduceGeom* g) {
    memset(g, 0, sizeof *g);
    g->nouter = 0;
    g->nout = 1;
    g->rlen = view_numel(a);
    g->rstride = 1;
    g->total = g->rlen;
}

int reduce_out_check(int op, const ctb_view* a, int dim, const ctb_view* out) {
    int64_t nout = 1;
    if (dim != CTB_DIM_FULL)
        for (int d = 0; d < a->ndim; ++d) if (d != dim) nout *= a->shape[d];
    int rc = check_out(out, nout, op == CTB_ARGMAX ? CTB_I32 : a->dtype, "reduction");
    if (rc) return rc;
    const ctb_view* in[1] = {a};
    return check_no_alias(out, in, 1, "reduction");
}

int reduce_arg_check(int op, const ctb_view* a, int dim) {
    int rc = check_view(a, "reduction: null input", "reduction");
    if (rc) return rc;
    if (op < 0 || op >= CTB_REDUCE_OP_COUNT) return set_error(CTB_ERR_ARG, "reduction: unknown operator code %d", op);
    if (op == CTB_VAR && a->dtype != CTB_F32 && a->dtype != CTB_F64)
        return set_error(CTB_ERR_DTYPE, "var: not defined for integer tensors");
    if (op == CTB_ARGMAX) {
        if (dim < 0 || dim >= a->ndim) return set_error(CTB_ERR_DIM, "argmax: dim out of range");
    } else if (dim != CTB_DIM_FULL && (dim < 0 || dim >= a->ndim)) {
        return set_error(CTB_ERR_DIM, "reduction: dim out of range");
    }
    return CTB_OK;
}

// Scratch needed by ctb_reduce for (a, dim): kernel scratch, plus a packed copy of the input
// when a full reduction is asked of a non-dense view.
// `op` < 0 = not known (the size query): the larger answer.  A dense but permuted view is
// folded in memory order for sum/mean/var; max/min must see the elements in the view's own
// order (which zero comes first decides the sign of a zero result), so they pack it first.
size_t reduce_ws_need(int op, const ctb_view* a, int dim, size_t* copy_bytes, bool want_partial = false) {
    ReduceGeom g;
    *copy_bytes = 0;
    if (dim == CTB_DIM_FULL) {
        const bool order_matters = op < 0 || op == CTB_MAX || op == CTB_MIN;
        if (!view_dense(a) || (order_matters && !view_contiguous(a))) *copy_bytes = (((size_t)view_numel(a) * dtype_bytes(a->dtype)) + 255) / 256 * 256;
        reduce_geom_full_dense(a, &g);
    } else {
        reduce_geom_dim(a, dim, &g);
    }
    size_t kernel_ws = reduce_workspace_bytes(g, a->dtype);
    // the packed copy must never overlap the ticket region at the start of the scratch
    if (*copy_bytes && kernel_ws < kTicketBytes) kernel_ws = kTicketBytes;
    // fp64 partials always come from the split kernel, even for inputs it would not pick itself
    if (want_partial && kernel_ws < kTicketBytes + 256) kernel_ws = kTicketBytes + 256;
    return *copy_bytes + kernel_ws;
}

int do_reduce(int op, const ctb_view* a, int dim, const ctb_view* out, double* partial,
              void* ws, size_t ws_bytes, cudaStream_t st) {
    ReduceGeom g;
    const void* src = elem_ptr(a);
    size_t copy_bytes = 0;
    const size_t need = reduce_ws_need(op, a, dim, &copy_bytes, partial != nullptr);
    if (need > ws_bytes || (need && !ws)) return set_error(CTB_ERR_WORKSPACE, "reduction: workspace of %zu bytes needed, %zu given", need, ws_bytes);
    if (need && !is_aligned(ws, 256)) return set_error(CTB_ERR_WORKSPACE, "reduction: workspace must be 256-byte aligned");
    if (dim == CTB_DIM_FULL) {
        if (copy_bytes) {
            // pack the view first (what the reference does: contiguous() before a full reduction,
            // src/cpu/AVX2/ops_avx2_f32.cpp:782)
            const ctb_view* in[1] = {a};
            Plan p;
            int rc = build_plan(in, 1, &p);
            if (rc) return rc;
            void* packed = (char*)ws + (need - copy_bytes);
            rc = launch_copy((int)dtype_bytes(a->dtype), p, src, packed, st);
            if (rc) return rc;
            src = packed;
        }
        reduce_geom_full_dense(a, &g);
    } else {
        reduce_geom_dim(a, dim, &g);
    }
    void* o = out ? elem_ptr_mut(out) : nullptr;
    return launch_reduce(op, a->dtype, g, src, o, partial, ws, need - copy_bytes, st);
}

int rows_geom(const ctb_view* x, const ctb_view* mask, RowsGeom* g, const char* who) {
    memset(g, 0, sizeof *g);
    if (x->dtype != CTB_F32) return set_error(CTB_ERR_DTYPE, "%s: only Float32 is supported", who);
    if (x->ndim < 1) return set_error(CTB_ERR_SHAPE, "%s: needs at least one dim", who);
    const int nd = x->ndim;
    if (x->shape[nd - 1] > 1 && x->stride[nd - 1] != 1) return set_error(CTB_ERR_SHAPE, "%s: the last dim must be contiguous", who);
    g->cols = x->shape[nd - 1];
    g->qlen = nd >= 2 ? x->shape[nd - 2] : 1;
    if (g->qlen == 0) g->qlen = 1;
    g->rows = 1;
    g->nouter = nd - 1;
    for (int d = 0; d < nd - 1; ++d) {
        g->oshape[d] = x->shape[d];
        g->xstride[d] = x->shape[d] == 1 ? 0 : x->stride[d];
        g->rows *= x->shape[d];
    }
    if (mask) {
        if (mask->dtype != CTB_F32) return set_error(CTB_ERR_DTYPE, "%s: mask must be Float32", who);
        if (mask->ndim > nd) return set_error(CTB_ERR_SHAPE, "Shape mismatch in binary op");
        g->has_mask = 1;
        const int pad = nd - mask->ndim;
        for (int d = 0; d < nd; ++d) {
            const int j = d - pad;
            const int64_t ms = j < 0 ? 1 : mask->shape[j];
            if (ms != 1 && ms != x->shape[d]) return set_error(CTB_ERR_SHAPE, "Shape mismatch in binary op");
            const int64_t st = (j < 0 || ms == 1) ? 0 : mask->stride[j];
            if (d == nd - 1) {
                if (st != 0 && st != 1) return set_error(CTB_ERR_SHAPE, "%s: the mask's last dim must be contiguous or broadcast", who);
                g->m_inner = (int32_t)st;
            } else {
                g->mstride[d] = st;
            }
        }
    }
    return CTB_OK;
}

// ---- host-buffer helpers ----------------------------------------------------------------------------
int ensure_stage(int device, size_t bytes, void** out, cudaStream_t** streams) {
    std::lock_guard<std::mutex> lk(g_mu);
    DeviceState& s = g_dev[device];
    for (int i = 0; i < 3; ++i)
        if (!s.streams[i]) CTB_CUDA_TRY(cudaStreamCreateWithFlags(&s.streams[i], cudaStreamNonBlocking));
    if (s.stage_bytes < bytes) {
        if (s.stage) CTB_CUDA_TRY(cudaFree(s.stage));
        s.stage = nullptr;
        s.stage_bytes = 0;
        CTB_CUDA_TRY(cudaMalloc(&s.stage, bytes));
        s.stage_bytes = bytes;
    }
    *out = s.stage;
    *streams = s.streams;
    return CTB_OK;
}

struct DeviceGuard {
    int prev = -1;
    bool ok = false;
    explicit DeviceGuard(int device) {
        if (cudaGetDevice(&prev) != cudaSuccess) return;
        ok = cudaSetDevice(device) == cudaSuccess;
    }
    ~DeviceGuard() { if (prev >= 0) cudaSetDevice(prev); }
};

size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

// Upload the storage span a host view touches; returns the device view in *dv.
int upload_view(const ctb_view* hv, char* dbuf, size_t* used, ctb_view* dv, cudaStream_t st) {
    const size_t es = dtype_bytes(hv->dtype);
    const int64_t span = view_span(hv);
    *dv = *hv;
    dv->base = dbuf + *used;
    dv->offset = 0;
    if (span > hv->offset) {
        const size_t bytes = (size_t)(span - hv->offset) * es;
        CTB_CUDA_TRY(cudaMemcpyAsync(dv->base, (const char*)hv->base + (size_t)hv->offset * es, bytes, cudaMemcpyHostToDevice, st));
        *used += align_up(bytes, 256);
    }
    return CTB_OK;
}

size_t span_bytes(const ctb_view* v) {
    const int64_t span = view_span(v);
    return span > v->offset ? align_up((size_t)(span - v->offset) * dtype_bytes(v->dtype), 256) : 0;
}

constexpr int64_t kHostChunkElems = int64_t(1) << 24;     // 64 MiB of fp32 per pipelined chunk

}  // namespace
}  // namespace ctb

// ====================================================================================================
//                                              C ABI
// ====================================================================================================
using namespace ctb;

extern "C" {

int ctb_abi_version(void) { return CTB_ABI_VERSION; }

const char* ctb_last_error(void) { return g_last_error.c_str(); }

int ctb_device_count(void) {
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess) { cudaGetLastError(); return 0; }
    return n;
}

int ctb_alloc(void** ptr, size_t bytes, int zero, void* stream) {
    if (!ptr) return set_error(CTB_ERR_NULL, "ctb_alloc: null result pointer");
    *ptr = nullptr;
    if (bytes == 0) bytes = 1;
    cudaStream_t st = (cudaStream_t)stream;
    CTB_CUDA_TRY(cudaMallocAsync(ptr, bytes, st));
    if (zero) CTB_CUDA_TRY(cudaMemsetAsync(*ptr, 0, bytes, st));
    return CTB_OK;
}

int ctb_free(void* ptr, void* stream) {
    if (!ptr) return CTB_OK;
    CTB_CUDA_TRY(cudaFreeAsync(ptr, (cudaStream_t)stream));
    return CTB_OK;
}

int ctb_sync(void* stream) {
    CTB_CUDA_TRY(cudaStreamSynchronize((cudaStream_t)stream));
    return CTB_OK;
}

int ctb_alloc_managed(void** ptr, size_t bytes, int zero) {
    if (!ptr) return set_error(CTB_ERR_NULL, "ctb_alloc_managed: null result pointer");
    *ptr = nullptr;
    if (bytes == 0) bytes = 1;
    CTB_CUDA_TRY(cudaMallocManaged(ptr, bytes, cudaMemAttachGlobal));
    if (zero) CTB_CUDA_TRY(cudaMemset(*ptr, 0, bytes));
    return CTB_OK;
}

int ctb_free_managed(void* ptr) {
    if (!ptr) return CTB_OK;
    CTB_CUDA_TRY(cudaFree(ptr));
    return CTB_OK;
}

int ctb_set_device(int index) {
    CTB_CUDA_TRY(cudaSetDevice(index));
    return CTB_OK;
}

int ctb_device_sync(void) {
    CTB_CUDA_TRY(cudaDeviceSynchronize());
    return CTB_OK;
}

int ctb_binary(int op, const ctb_view* a, const ctb_view* b, const ctb_view* out, void* stream) {
    int rc;
    if ((rc = check_view(a, "binary_op: null input", "binary_op"))) return rc;
    if ((rc = check_view(b, "binary_op: null input", "binary_op"))) return rc;
    if (op < 0 || op >= CTB_BINARY_OP_COUNT) return set_error(CTB_ERR_ARG, "binary_op: unknown operator code %d", op);
    if (a->dtype != b->dtype) return set_error(CTB_ERR_DTYPE, "binary_op: operands must have the same dtype");
    const ctb_view* in[2] = {a, b};
    Plan p;
    if ((rc = build_plan(in, 2, &p))) return rc;
    if ((rc = check_out(out, p.numel, a->dtype, "binary_op"))) return rc;
    if ((rc = check_no_alias(out, in, 2, "binary_op"))) return rc;
    return launch_binary(op, a->dtype, p, elem_ptr(a), elem_ptr(b), elem_ptr_mut(out), (cudaStream_t)stream);
}

int ctb_unary(int op, const ctb_view* a, double scalar, const ctb_view* out, void* stream) {
    int rc;
    if ((rc = check_view(a, "unary_op: null input", "unary_op"))) return rc;
    if (op < 0 || op >= CTB_UNARY_OP_COUNT) return set_error(CTB_ERR_ARG, "unary_op: unknown operator code %d", op);
    const ctb_view* in[1] = {a};
    Plan p;
    if ((rc = build_plan(in, 1, &p))) return rc;
    if ((rc = check_out(out, p.numel, a->dtype, "unary_op"))) return rc;
    if ((rc = check_no_alias(out, in, 1, "unary_op"))) return rc;
    return launch_unary(op, a->dtype, p, elem_ptr(a), scalar, elem_ptr_mut(out), (cudaStream_t)stream);
}

int ctb_copy_strided(const ctb_view* src, const ctb_view* out, void* stream) {
    int rc;
    if ((rc = check_view(src, "copy: null input", "copy"))) return rc;
    const ctb_view* in[1] = {src};
    Plan p;
    if ((rc = build_plan(in, 1, &p))) return rc;
    if ((rc = check_out(out, p.numel, src->dtype, "copy"))) return rc;
    if ((rc = check_no_alias(out, in, 1, "copy"))) return rc;
    return launch_copy((int)dtype_bytes(src->dtype), p, elem_ptr(src), elem_ptr_mut(out), (cudaStream_t)stream);
}

size_t ctb_reduce_workspace_bytes(const ctb_view* a, int dim) {
    if (check_view(a, "reduction: null input", "reduction")) return 0;
    if (dim != CTB_DIM_FULL && (dim < 0 || dim >= a->ndim)) return 0;
    size_t copy_bytes;
    return reduce_ws_need(-1, a, dim, &copy_bytes);
}

int ctb_reduce_ws(int op, const ctb_view* a, int dim, const ctb_view* out, void* workspace,
                  size_t workspace_bytes, void* stream) {
    int rc;
    if ((rc = reduce_arg_check(op, a, dim))) return rc;
    if ((rc = reduce_out_check(op, a, dim, out))) return rc;
    // a caller's buffer has unknown contents: clear the ticket region the split kernels rely on
    if (workspace && workspace_bytes >= kTicketBytes && ctb_reduce_workspace_bytes(a, dim) > 0)
        CTB_CUDA_TRY(cudaMemsetAsync(workspace, 0, kTicketBytes, (cudaStream_t)stream));
    return do_reduce(op, a, dim, out, nullptr, workspace, workspace_bytes, (cudaStream_t)stream);
}

int ctb_reduce(int op, const ctb_view* a, int dim, const ctb_view* out, void* stream) {
    int rc;
    if ((rc = reduce_arg_check(op, a, dim))) return rc;
    if ((rc = reduce_out_check(op, a, dim, out))) return rc;
    size_t copy_bytes;
    const size_t need = reduce_ws_need(op, a, dim, &copy_bytes);
    void* ws = nullptr;
    if ((rc = ensure_workspace(need, &ws, (cudaStream_t)stream))) return rc;
    return do_reduce(op, a, dim, out, nullptr, ws, need, (cudaStream_t)stream);
}

int ctb_reduce_dim_noalloc(int op, const ctb_view* a, int dim, const ctb_view* out, void* stream) {
    int rc;
    if ((rc = reduce_arg_check(op, a, dim))) return rc;
    if (dim == CTB_DIM_FULL)
        return set_error(CTB_ERR_DIM, "reduction without allocation: a dim >= 0 is required");
    if ((rc = reduce_out_check(op, a, dim, out))) return rc;
    ReduceGeom g;
    reduce_geom_dim(a, dim, &g);
    return launch_reduce_static_scratch(op, a->dtype, g, elem_ptr(a), elem_ptr_mut(out), (cudaStream_t)stream);
}

int ctb_reduce_full_partial(int op, const ctb_view* a, double* partial, void* stream) {
    int rc;
    if ((rc = reduce_arg_check(op, a, CTB_DIM_FULL))) return rc;
    if (!partial) return set_error(CTB_ERR_NULL, "reduction: null partial pointer");
    if (op != CTB_SUM && op != CTB_MEAN && op != CTB_MAX && op != CTB_MIN)
        return set_error(CTB_ERR_ARG, "reduction: fp64 partials exist for sum/mean/max/min only");
    if (a->dtype != CTB_F32) return set_error(CTB_ERR_DTYPE, "reduction: fp64 partials need a Float32 input");
    size_t copy_bytes;
    const size_t need = reduce_ws_need(op, a, CTB_DIM_FULL, &copy_bytes, true);
    void* ws = nullptr;
    if ((rc = ensure_workspace(need, &ws, (cudaStream_t)stream))) return rc;
    return do_reduce(op, a, CTB_DIM_FULL, nullptr, partial, ws, need, (cudaStream_t)stream);
}

int ctb_finalize_full(int op, const double* partial, int64_t total_count, const ctb_view* out, void* stream) {
    int rc;
    if (!partial) return set_error(CTB_ERR_NULL, "reduction: null partial pointer");
    if ((rc = check_view(out, "output: null view", "finalize"))) return rc;
    if (view_numel(out) != 1) return set_error(CTB_ERR_SHAPE, "finalize: output must hold one element");
    return launch_finalize_full(op, out->dtype, partial, total_count, elem_ptr_mut(out), (cudaStream_t)stream);
}

static int softmax_entry(const ctb_view* x, const ctb_view* mask, int causal, int log_out, const ctb_view* out,
                         void* stream, const char* who) {
    int rc;
    if ((rc = check_view(x, "softmax: null input", who))) return rc;
    if (mask && (rc = check_view(mask, "softmax: null mask", who))) return rc;
    RowsGeom g;
    if ((rc = rows_geom(x, mask, &g, who))) return rc;
    if ((rc = check_out(out, g.rows * g.cols, CTB_F32, who))) return rc;
    const ctb_view* ins[2] = {x, mask};
    if ((rc = check_no_alias(out, ins, 2, who))) return rc;
    return launch_softmax(g, (const float*)elem_ptr(x), mask ? (const float*)elem_ptr(mask) : nullptr,
                          causal, log_out, (float*)elem_ptr_mut(out), (cudaStream_t)stream);
}

int ctb_softmax_lastdim(const ctb_view* x, const ctb_view* mask, int causal, const ctb_view* out, void* stream) {
    return softmax_entry(x, mask, causal, 0, out, stream, "softmax");
}

int ctb_log_softmax_lastdim(const ctb_view* x, const ctb_view* mask, const ctb_view* out, void* stream) {
    return softmax_entry(x, mask, 0, 1, out, stream, "log_softmax");
}

int ctb_layernorm_lastdim(const ctb_view* x, const ctb_view* gamma, const ctb_view* beta, double eps,
                          const ctb_view* out, void* stream) {
    int rc;
    if ((rc = check_view(x, "layernorm: null input", "layernorm"))) return rc;
    RowsGeom g;
    if ((rc = rows_geom(x, nullptr, &g, "layernorm"))) return rc;
    const ctb_view* gb[2] = {gamma, beta};
    int64_t st[2] = {0, 0};
    for (int i = 0; i < 2; ++i) {
        if (!gb[i]) continue;
        if ((rc = check_view(gb[i], "layernorm: null scale/shift", "layernorm"))) return rc;
        if (gb[i]->dtype != CTB_F32) return set_error(CTB_ERR_DTYPE, "layernorm: scale/shift must be Float32");
        if (view_numel(gb[i]) != g.cols || gb[i]->ndim < 1 || gb[i]->shape[gb[i]->ndim - 1] != g.cols)
            return set_error(CTB_ERR_SHAPE, "Shape mismatch in binary op");
        st[i] = gb[i]->stride[gb[i]->ndim - 1];
    }
    if ((rc = check_out(out, g.rows * g.cols, CTB_F32, "layernorm"))) return rc;
    const ctb_view* ins[3] = {x, gamma, beta};
    if ((rc = check_no_alias(out, ins, 3, "layernorm"))) return rc;
    return launch_layernorm(g, (const float*)elem_ptr(x), gamma ? (const float*)elem_ptr(gamma) : nullptr, st[0],
                            beta ? (const float*)elem_ptr(beta) : nullptr, st[1], eps,
                            (float*)elem_ptr_mut(out), (cudaStream_t)stream);
}

// ---- gather ------------------------------------------------------------------------------------------
int ctb_gather(const ctb_view* x, int dim, const ctb_view* index, const ctb_view* out, int32_t* bad, void* stream) {
    int rc;
    if ((rc = check_view(x, "Gather on empty tensor", "gather"))) return rc;
    if ((rc = check_view(index, "Gather with empty index", "gather"))) return rc;
    if (dim < 0 || dim >= x->ndim) return set_error(CTB_ERR_DIM, "Gather dimension out of range");
    if (x->ndim != index->ndim) return set_error(CTB_ERR_SHAPE, "Input and index must have same number of dimensions");
    if (!dtype_ok(index->dtype)) return set_error(CTB_ERR_DTYPE, "gather: unsupported index dtype");
    for (int d = 0; d < x->ndim; ++d)
        if (d != dim && index->shape[d] > x->shape[d])
            return set_error(CTB_ERR_SHAPE, "Index shape dimension mismatch with input");
    if ((rc = check_out(out, view_numel(index), x->dtype, "gather"))) return rc;
    if (bad) CTB_CUDA_TRY(cudaMemsetAsync(bad, 0, sizeof(int32_t), (cudaStream_t)stream));
    if (view_numel(index) == 0) return CTB_OK;
    return launch_gather((int)dtype_bytes(x->dtype), x->ndim, index->shape, x->stride, index->stride, dim,
                         x->shape[dim], elem_ptr(x), elem_ptr(index), index->dtype, elem_ptr_mut(out), bad,
                         (cudaStream_t)stream);
}

// ---- accumulate_grad ---------------------------------------------------------------------------------
namespace {

// Dense row-major strides of `shape` with 0 for size-1 dims.
void dense_strides(int nd, const int64_t* shape, int64_t* stride) {
    int64_t run = 1;
    for (int d = nd - 1; d >= 0; --d) {
        stride[d] = shape[d] == 1 ? 0 : run;
        run *= shape[d];
    }
}

// `v` with dims [lo, hi] (contiguous across each other) merged into one; returns its index.
int merge_dims(const ctb_view& v, int lo, int hi, ctb_view* m) {
    *m = v;
    int64_t len = 1;
    for (int d = lo; d <= hi; ++d) len *= v.shape[d];
    int k = 0;
    for (int d = 0; d < v.ndim; ++d) {
        if (d > lo && d <= hi) continue;
        m->shape[k] = d == lo ? len : v.shape[d];
        m->stride[k] = d == lo ? v.stride[hi] : v.stride[d];
        ++k;
    }
    m->ndim = k;
    return lo;
}

}  // namespace

int ctb_accumulate_grad(const ctb_view* grad, const ctb_view* src, void* stream) {
    int rc;
    if ((rc = check_view(grad, "accumulate_grad: null gradient buffer", "accumulate_grad"))) return rc;
    if ((rc = check_view(src, "accumulate_grad: null source", "accumulate_grad"))) return rc;
    if (grad->dtype != src->dtype) return set_error(CTB_ERR_DTYPE, "accumulate_grad: dtype mismatch");
    cudaStream_t st = (cudaStream_t)stream;
    const int nd = grad->ndim > src->ndim ? grad->ndim : src->ndim;
    if (nd == 0) {
        const int64_t one = 1, zero = 0;
        return launch_accumulate_strided(grad->dtype, 1, &one, &zero, &zero, elem_ptr_mut(grad), elem_ptr(src), st);
    }
    // right-aligned shapes; which source dims fold (target 1, source > 1)
    int64_t tshape[CTB_MAX_DIMS], tstride[CTB_MAX_DIMS];
    bool fold[CTB_MAX_DIMS], src_bcast = false;
    ctb_view cur = *src;
    cur.ndim = nd;
    int nfold = 0;
    for (int d = 0; d < nd; ++d) {
        const int jt = d - (nd - grad->ndim), js = d - (nd - src->ndim);
        tshape[d] = jt < 0 ? 1 : grad->shape[jt];
        tstride[d] = (jt < 0 || grad->shape[jt] == 1) ? 0 : grad->stride[jt];
        cur.shape[d] = js < 0 ? 1 : src->shape[js];
        cur.stride[d] = (js < 0 || src->shape[js] == 1) ? 0 : src->stride[js];
        if (tshape[d] != cur.shape[d] && tshape[d] != 1 && cur.shape[d] != 1)
            return set_error(CTB_ERR_SHAPE, "Shape mismatch in binary op");
        fold[d] = tshape[d] == 1 && cur.shape[d] > 1;
        if (fold[d]) ++nfold;
        if (cur.shape[d] == 1 && tshape[d] > 1) src_bcast = true;
    }
    int64_t tnumel = 1, snumel = 1;
    for (int d = 0; d < nd; ++d) { tnumel *= tshape[d]; snumel *= cur.shape[d]; }
    if (tnumel == 0 || snumel == 0) return CTB_OK;

    // groups of neighbouring folded dims the source is contiguous across, last group first
    struct Group { int lo, hi; };
    Group groups[CTB_MAX_DIMS];
    int ngroups = 0;
    for (int d = nd - 1; d >= 0; --d) {
        if (!fold[d]) continue;
        int lo = d;
        while (lo > 0 && fold[lo - 1] && cur.stride[lo - 1] == cur.stride[lo] * cur.shape[lo]) --lo;
        groups[ngroups++] = {lo, d};
        d = lo;
    }
    // scratch: kernel scratch of the largest step, then two buffers for intermediate sums
    const size_t eb = dtype_bytes(src->dtype);
    size_t kernel_ws = 0, tmp_elems = 0;
    {
        ctb_view sim = cur;
        for (int gi = 0; gi < ngroups; ++gi) {
            ctb_view m;
            const int rd = merge_dims(sim, groups[gi].lo, groups[gi].hi, &m);
            ReduceGeom g;
            reduce_geom_dim(&m, rd, &g);
            const size_t need = reduce_workspace_bytes(g, src->dtype);
            if (need > kernel_ws) kernel_ws = need;
            for (int d = groups[gi].lo; d <= groups[gi].hi; ++d) sim.shape[d] = 1;
            dense_strides(nd, sim.shape, sim.stride);
            int64_t n = 1;
            for (int d = 0; d < nd; ++d) n *= sim.shape[d];
            if ((size_t)n > tmp_elems) tmp_elems = (size_t)n;
        }
    }
    // the ticket region at the start of the shared workspace must stay zero between calls:
    // intermediate sums never go there, even when no step of this call needs kernel scratch
    if (kernel_ws < kTicketBytes) kernel_ws = kTicketBytes;
    kernel_ws = (kernel_ws + 255) / 256 * 256;
    const size_t tmp_bytes = (tmp_elems * eb + 255) / 256 * 256;
    void* ws = nullptr;
    if (ngroups > 0 && (rc = ensure_workspace(kernel_ws + 2 * tmp_bytes, &ws, st))) return rc;

    const bool grad_dense = view_contiguous(grad);
    for (int gi = 0; gi < ngroups; ++gi) {
        ctb_view m;
        const int rd = merge_dims(cur, groups[gi].lo, groups[gi].hi, &m);
        ReduceGeom g;
        reduce_geom_dim(&m, rd, &g);
        const bool last = gi == ngroups - 1;
        if (last && grad_dense && !src_bcast) {
            // the last fold adds straight into the gradient buffer: out[i] += (T)sum
            return launch_reduce(kOpSumAccumulate, src->dtype, g, elem_ptr(&m), elem_ptr_mut(grad), nullptr, ws, kernel_ws, st);
        }
        void* tmp = (char*)ws + kernel_ws + (gi % 2) * tmp_bytes;
        if ((rc = launch_reduce(CTB_SUM, src->dtype, g, elem_ptr(&m), tmp, nullptr, ws, kernel_ws, st))) return rc;
        for (int d = groups[gi].lo; d <= groups[gi].hi; ++d) cur.shape[d] = 1;
        dense_strides(nd, cur.shape, cur.stride);
        cur.base = tmp;
        cur.offset = 0;
    }
    // element-wise accumulation of `cur` (possibly broadcast) into the gradient buffer
    if (grad_dense) {
        ctb_view t = *grad;
        t.ndim = nd;
        for (int d = 0; d < nd; ++d) t.shape[d] = tshape[d];
        dense_strides(nd, t.shape, t.stride);
        const ctb_view* in[2] = {&t, &cur};
        Plan p;
        if ((rc = build_plan(in, 2, &p))) return rc;
        return launch_binary(kOpAddFinite, grad->dtype, p, elem_ptr(grad), elem_ptr(&cur), elem_ptr_mut(grad), st);
    }
    return launch_accumulate_strided(grad->dtype, nd, tshape, tstride, cur.stride, elem_ptr_mut(grad), elem_ptr(&cur), st);
}

// ---- BatchNorm forward ---------------------------------------------------------------------------------
namespace {

// x[N, C, trailing...] contiguous fp32 -> (N, C, S)
int batchnorm_geom(const ctb_view* x, int64_t* N, int64_t* C, int64_t* S, const char* who) {
    int rc;
    if ((rc = check_view(x, "batchnorm: null input", who))) return rc;
    if (x->dtype != CTB_F32) return set_error(CTB_ERR_DTYPE, "%s: only Float32 is supported", who);
    if (x->ndim < 2) return set_error(CTB_ERR_SHAPE, "%s: input needs [batch, channels, ...]", who);
    if (!view_contiguous(x)) return set_error(CTB_ERR_SHAPE, "%s: input must be contiguous", who);
    *N = x->shape[0];
    *C = x->shape[1];
    *S = 1;
    for (int d = 2; d < x->ndim; ++d) *S *= x->shape[d];
    return CTB_OK;
}

// A per-channel parameter: C elements in any view whose other dims have extent 1.
int channel_param(const ctb_view* v, int64_t C, const char* who, const float** ptr, int64_t* stride) {
    int rc;
    if ((rc = check_view(v, "batchnorm: null parameter", who))) return rc;
    if (v->dtype != CTB_F32) return set_error(CTB_ERR_DTYPE, "%s: parameters must be Float32", who);
    if (view_numel(v) != C) return set_error(CTB_ERR_SHAPE, "Shape mismatch in binary op");
    *stride = 0;
    for (int d = 0; d < v->ndim; ++d) if (v->shape[d] == C && C > 1) *stride = v->stride[d];
    *ptr = (const float*)elem_ptr(v);
    return CTB_OK;
}

}  // namespace

int ctb_channel_moments(const ctb_view* x, const ctb_view* mean, const ctb_view* var, void* stream) {
    int rc;
    int64_t N, C, S;
    if ((rc = batchnorm_geom(x, &N, &C, &S, "channel_moments"))) return rc;
    if ((rc = check_out(mean, C, CTB_F32, "channel_moments"))) return rc;
    if ((rc = check_out(var, C, CTB_F32, "channel_moments"))) return rc;
    if (N * S == 0) return set_error(CTB_ERR_SHAPE, "channel_moments: empty batch");
    if (S == 1) {
        // [N, C]: the statistics are column reductions; the column kernel reads whole rows
        ctb_view x2 = *x;
        x2.ndim = 2;
        x2.shape[0] = N; x2.shape[1] = C;
        x2.stride[0] = C; x2.stride[1] = 1;
        if ((rc = ctb_reduce(CTB_MEAN, &x2, 0, mean, stream))) return rc;
        return ctb_reduce(CTB_VAR, &x2, 0, var, stream);
    }
    DeviceInfo di;
    if ((rc = current_device_info(&di))) return rc;
    const size_t need = channel_moments_workspace_bytes(C, di.sm_count);
    void* ws = nullptr;
    if ((rc = ensure_workspace(need, &ws, (cudaStream_t)stream))) return rc;
    return launch_channel_moments((const float*)elem_ptr(x), (float*)elem_ptr_mut(mean), (float*)elem_ptr_mut(var),
                                  N, C, S, ws, need, (cudaStream_t)stream);
}

int ctb_batchnorm_apply(const ctb_view* x, const ctb_view* mean, const ctb_view* var, const ctb_view* gamma,
                        const ctb_view* beta, double eps, const ctb_view* out, void* stream) {
    int rc;
    int64_t N, C, S;
    if ((rc = batchnorm_geom(x, &N, &C, &S, "batchnorm"))) return rc;
    const float *pm, *pv, *pg = nullptr, *pb = nullptr;
    int64_t sm, sv, sg = 0, sb = 0;
    if ((rc = channel_param(mean, C, "batchnorm", &pm, &sm))) return rc;
    if ((rc = channel_param(var, C, "batchnorm", &pv, &sv))) return rc;
    if (gamma && (rc = channel_param(gamma, C, "batchnorm", &pg, &sg))) return rc;
    if (beta && (rc = channel_param(beta, C, "batchnorm", &pb, &sb))) return rc;
    if ((rc = check_out(out, N * C * S, CTB_F32, "batchnorm"))) return rc;
    if (N * C * S == 0) return CTB_OK;
    // 1/sqrt(var + eps) per channel lives behind the workspace's ticket region
    void* ws = nullptr;
    if ((rc = ensure_workspace(kTicketBytes + (size_t)C * sizeof(float), &ws, (cudaStream_t)stream))) return rc;
    return launch_batchnorm_apply((const float*)elem_ptr(x), pm, sm, pv, sv, pg, sg, pb, sb, eps,
                                  (float*)((char*)ws + kTicketBytes), (float*)elem_ptr_mut(out), N, C, S,
                                  (cudaStream_t)stream);
}

// ---- backward bodies, cross-entropy rows -----------------------------------------------------------------
namespace {

// Broadcast `ops` (null entries allowed) against the shape of `out`, which fixes every extent,
// and collapse.  stride row k of the plan belongs to ops[k]; row 3 to `out`.
int build_bwd_plan(const ctb_view* const* ops, const ctb_view* out, BwdPlan* plan) {
    const int nd = out->ndim;
    int64_t shape[CTB_MAX_DIMS], stride[4][CTB_MAX_DIMS];
    for (int k = 0; k < 3; ++k)
        if (ops[k] && ops[k]->ndim > nd) return set_error(CTB_ERR_SHAPE, "Shape mismatch in binary op");
    for (int d = 0; d < nd; ++d) {
        shape[d] = out->shape[d];
        stride[3][d] = out->shape[d] == 1 ? 0 : out->stride[d];
        for (int k = 0; k < 3; ++k) {
            stride[k][d] = 0;
            if (!ops[k]) continue;
            const int j = d - (nd - ops[k]->ndim);
            const int64_t e = j < 0 ? 1 : ops[k]->shape[j];
            if (e != 1 && e != shape[d]) return set_error(CTB_ERR_SHAPE, "Shape mismatch in binary op");
            stride[k][d] = (j < 0 || e == 1) ? 0 : ops[k]->stride[j];
        }
    }
    plan->numel = 1;
    int k = 0;
    for (int d = 0; d < nd; ++d) {
        plan->numel *= shape[d];
        if (shape[d] == 1) continue;
        bool merge = k > 0;
        for (int q = 0; q < 4 && merge; ++q)
            if (plan->stride[q][k - 1] != stride[q][d] * shape[d]) merge = false;
        if (merge) {
            plan->shape[k - 1] *= shape[d];
            for (int q = 0; q < 4; ++q) plan->stride[q][k - 1] = stride[q][d];
            continue;
        }
        plan->shape[k] = shape[d];
        for (int q = 0; q < 4; ++q) plan->stride[q][k] = stride[q][d];
        ++k;
    }
    if (k == 0) {
        plan->shape[0] = 1;
        for (int q = 0; q < 4; ++q) plan->stride[q][0] = 0;
        k = 1;
    }
    plan->ndim = k;
    plan->flat = k == 1 && plan->stride[3][0] == 1;
    for (int q = 0; q < 3; ++q)
        if (ops[q] && plan->stride[q][0] != 1) plan->flat = 0;
    if (plan->numel == 1) plan->flat = 0;       // all strides collapse to 0: the strided kernel handles it
    return CTB_OK;
}

int backward_chain_entry(int kind, const char* who, const ctb_view* grad, const ctb_view* x, const ctb_view* y,
                         const ctb_view* out, int accumulate, void* stream) {
    int rc;
    if ((rc = check_view(grad, "backward: null gradient", who))) return rc;
    if (x && (rc = check_view(x, "backward: null operand", who))) return rc;
    if (y && (rc = check_view(y, "backward: null operand", who))) return rc;
    if ((rc = check_view(out, "output: null view", who))) return rc;
    const ctb_view* ops[3] = {grad, x, y};
    for (int k = 0; k < 3; ++k)
        if (ops[k] && ops[k]->dtype != out->dtype) return set_error(CTB_ERR_DTYPE, "%s: operands must have the same dtype", who);
    if (!accumulate) {
        if (!view_contiguous(out)) return set_error(CTB_ERR_SHAPE, "%s: output must be contiguous", who);
        if ((rc = check_no_alias(out, ops, 3, who))) return rc;
    }
    BwdPlan plan;
    if ((rc = build_bwd_plan(ops, out, &plan))) return rc;
    return launch_backward_chain(kind, out->dtype, plan, elem_ptr(grad), x ? elem_ptr(x) : nullptr,
                                 y ? elem_ptr(y) : nullptr, elem_ptr_mut(out), accumulate, (cudaStream_t)stream);
}

// logits [rows, classes] (classes contiguous), labels: `rows` Int32 values in a [rows] or [rows, 1] view
int ce_geometry(const ctb_view* logits, const ctb_view* labels, const char* who, int64_t* rows, int64_t* classes,
                int64_t* row_stride, int64_t* label_stride) {
    int rc;
    if ((rc = check_view(logits, "Loss::CrossEntropy: null tensor", who))) return rc;
    if ((rc = check_view(labels, "Loss::CrossEntropy: null tensor", who))) return rc;
    if (logits->ndim != 2) return set_error(CTB_ERR_SHAPE, "CrossEntropy: Pred must be 2D [Batch, Classes]");
    if (logits->dtype != CTB_F32) return set_error(CTB_ERR_DTYPE, "%s: only Float32 logits are supported", who);
    if (labels->dtype != CTB_I32) return set_error(CTB_ERR_DTYPE, "Index tensor must be integer type");
    *rows = logits->shape[0];
    *classes = logits->shape[1];
    if (*classes > 1 && logits->stride[1] != 1) return set_error(CTB_ERR_SHAPE, "%s: the class dim must be contiguous", who);
    *row_stride = *rows > 1 ? logits->stride[0] : 0;
    if (view_numel(labels) != *rows) return set_error(CTB_ERR_SHAPE, "%s: one label per row is expected", who);
    *label_stride = 0;
    for (int d = 0; d < labels->ndim; ++d)
        if (labels->shape[d] == *rows && *rows > 1) *label_stride = labels->stride[d];
    return CTB_OK;
}

}  // namespace

int ctb_div_backward(const ctb_view* grad, const ctb_view* a, const ctb_view* b, const ctb_view* grad_a,
                     const ctb_view* grad_b, int accumulate, void* stream) {
    int rc;
    if (!grad_a && !grad_b) return set_error(CTB_ERR_NULL, "div_backward: no output requested");
    if (!b) return set_error(CTB_ERR_NULL, "backward: null operand");
    if (grad_a && grad_b && a && grad && !check_view(grad, "", "") && !check_view(a, "", "") && !check_view(b, "", "") &&
        !check_view(grad_a, "", "") && !check_view(grad_b, "", "") && grad_a->dtype == grad_b->dtype) {
        // every operand contiguous and of one shape: both gradients in a single pass
        const ctb_view* opsa[3] = {grad, nullptr, b};
        const ctb_view* opsb[3] = {grad, a, b};
        BwdPlan pa, pb;
        bool same = grad->dtype == grad_a->dtype && a->dtype == grad_a->dtype && b->dtype == grad_a->dtype;
        if (same && !build_bwd_plan(opsa, grad_a, &pa) && !build_bwd_plan(opsb, grad_b, &pb) && pa.flat && pb.flat &&
            pa.numel == pb.numel && (accumulate || (!check_no_alias(grad_a, opsb, 3, "div_backward") &&
                                                    !check_no_alias(grad_b, opsb, 3, "div_backward")))) {
            const ctb_view* outs[1] = {grad_a};
            if (!check_no_alias(grad_b, outs, 1, "div_backward"))
                return launch_div_backward_both(grad_a->dtype, pa.numel, elem_ptr(grad), elem_ptr(a), elem_ptr(b),
                                                elem_ptr_mut(grad_a), elem_ptr_mut(grad_b), accumulate, (cudaStream_t)stream);
        }
    }
    if (grad_a && (rc = backward_chain_entry(kBwdDivA, "div_backward", grad, nullptr, b, grad_a, accumulate, stream))) return rc;
    if (grad_b) {
        if (!a) return set_error(CTB_ERR_NULL, "backward: null operand");
        if ((rc = backward_chain_entry(kBwdDivB, "div_backward", grad, a, b, grad_b, accumulate, stream))) return rc;
    }
    return CTB_OK;
}

int ctb_tanh_backward(const ctb_view* grad, const ctb_view* t, const ctb_view* grad_t, int accumulate, void* stream) {
    if (!t) return set_error(CTB_ERR_NULL, "backward: null operand");
    return backward_chain_entry(kBwdTanh, "tanh_backward", grad, t, nullptr, grad_t, accumulate, stream);
}

int ctb_cross_entropy(const ctb_view* logits, const ctb_view* labels, int mean, const ctb_view* loss, int32_t* bad,
                      void* stream) {
    int rc;
    int64_t rows, classes, row_stride, label_stride;
    if ((rc = ce_geometry(logits, labels, "cross_entropy", &rows, &classes, &row_stride, &label_stride))) return rc;
    if ((rc = check_out(loss, 1, CTB_F32, "cross_entropy"))) return rc;
    if (rows == 0 || classes == 0) return set_error(CTB_ERR_SHAPE, "cross_entropy: empty batch");
    cudaStream_t st = (cudaStream_t)stream;
    if (bad) CTB_CUDA_TRY(cudaMemsetAsync(bad, 0, sizeof(int32_t), st));
    // scratch: [tickets | kernel scratch of the reduction | nll[rows]]
    ctb_view nll;
    memset(&nll, 0, sizeof nll);
    nll.dtype = CTB_F32;
    nll.ndim = 1;
    nll.shape[0] = rows;
    nll.stride[0] = 1;
    ReduceGeom g;
    reduce_geom_full_dense(&nll, &g);
    size_t kernel_ws = reduce_workspace_bytes(g, CTB_F32);
    if (kernel_ws < kTicketBytes) kernel_ws = kTicketBytes;
    kernel_ws = (kernel_ws + 255) / 256 * 256;
    void* ws = nullptr;
    if ((rc = ensure_workspace(kernel_ws + (size_t)rows * sizeof(float), &ws, st))) return rc;
    float* nll_buf = (float*)((char*)ws + kernel_ws);
    if ((rc = launch_ce_forward_rows((const float*)elem_ptr(logits), row_stride, (const int32_t*)elem_ptr(labels),
                                     label_stride, rows, classes, nll_buf, bad, st))) return rc;
    // mean(nll) / sum(nll) as the reduction operators compute them (fp64 accumulation, sum rounded
    // to fp32, then times 1/rows in double and rounded: src/core/ops_dispatch.cpp:385-390)
    return launch_reduce(mean ? CTB_MEAN : CTB_SUM, CTB_F32, g, nll_buf, elem_ptr_mut(loss), nullptr, ws, kernel_ws, st);
}

int ctb_cross_entropy_backward(const ctb_view* logits, const ctb_view* labels, double grad_scale,
                               const ctb_view* grad_logits, int accumulate, int32_t* bad, void* stream) {
    int rc;
    int64_t rows, classes, row_stride, label_stride;
    if ((rc = ce_geometry(logits, labels, "cross_entropy_backward", &rows, &classes, &row_stride, &label_stride))) return rc;
    if ((rc = check_view(grad_logits, "output: null view", "cross_entropy_backward"))) return rc;
    if (grad_logits->dtype != CTB_F32 || grad_logits->ndim != 2 || grad_logits->shape[0] != rows || grad_logits->shape[1] != classes)
        return set_error(CTB_ERR_SHAPE, "cross_entropy_backward: the gradient must be Float32 [Batch, Classes]");
    if (classes > 1 && grad_logits->stride[1] != 1) return set_error(CTB_ERR_SHAPE, "cross_entropy_backward: the class dim must be contiguous");
    const ctb_view* ins[2] = {logits, labels};
    if ((rc = check_no_alias(grad_logits, ins, 2, "cross_entropy_backward"))) return rc;
    cudaStream_t st = (cudaStream_t)stream;
    if (bad) CTB_CUDA_TRY(cudaMemsetAsync(bad, 0, sizeof(int32_t), st));
    if (rows == 0 || classes == 0) return CTB_OK;
    return launch_ce_backward_rows((const float*)elem_ptr(logits), row_stride, (const int32_t*)elem_ptr(labels), label_stride,
                                   rows, classes, (float)grad_scale, (float*)elem_ptr_mut(grad_logits),
                                   rows > 1 ? grad_logits->stride[0] : 0, accumulate, bad, st);
}

// ---- matmul ------------------------------------------------------------------------------------------
int ctb_matmul(const ctb_view* a, const ctb_view* b, const ctb_view* out, void* stream) {
    int rc;
    if ((rc = check_view(a, "matmul: null input", "matmul"))) return rc;
    if ((rc = check_view(b, "matmul: null input", "matmul"))) return rc;
    if (a->ndim < 2 || b->ndim < 2) return set_error(CTB_ERR_SHAPE, "matmul_mp requires at least 2D tensors");
    if (a->ndim > 3 || b->ndim > 3) return set_error(CTB_ERR_SHAPE, "matmul: at most one batch dim is supported");
    if (a->dtype != b->dtype) return set_error(CTB_ERR_DTYPE, "matmul: operands must have the same dtype");
    const int64_t K = a->shape[a->ndim - 1], M = a->shape[a->ndim - 2], N = b->shape[b->ndim - 1];
    if (b->shape[b->ndim - 2] != K) return set_error(CTB_ERR_SHAPE, "matmul_mp shape mismatch");
    const int64_t batch_a = a->ndim == 3 ? a->shape[0] : 1, batch_b = b->ndim == 3 ? b->shape[0] : 1;
    const int64_t batch = batch_a > batch_b ? batch_a : batch_b;
    if ((batch_a != batch && batch_a != 1) || (batch_b != batch && batch_b != 1))
        return set_error(CTB_ERR_SHAPE, "matmul_mp shape mismatch");
    if ((rc = check_out(out, batch * M * N, a->dtype, "matmul"))) return rc;
    const int64_t sa = (a->ndim == 3 && batch_a > 1) ? a->stride[0] : 0;
    const int64_t sb = (b->ndim == 3 && batch_b > 1) ? b->stride[0] : 0;
    return launch_matmul(a->dtype, elem_ptr(a), elem_ptr(b), elem_ptr_mut(out), batch, M, N, K,
                         a->stride[a->ndim - 2], a->stride[a->ndim - 1], sa,
                         b->stride[b->ndim - 2], b->stride[b->ndim - 1], sb, (cudaStream_t)stream);
}

// Tensor-core matmul: operands are brought to the layout the kernel's TMA loads need (unit stride
// along K, rows 16-byte aligned) — directly when the views already have it, through a packed copy in
// the library's workspace otherwise.
int ctb_matmul_tc(const ctb_view* a, const ctb_view* b, const ctb_view* out, int32_t* status, void* stream) {
    int rc;
    if ((rc = check_view(a, "matmul: null input", "matmul_tc"))) return rc;
    if ((rc = check_view(b, "matmul: null input", "matmul_tc"))) return rc;
    if (a->ndim < 2 || b->ndim < 2) return set_error(CTB_ERR_SHAPE, "matmul_mp requires at least 2D tensors");
    if (a->ndim > 3 || b->ndim > 3) return set_error(CTB_ERR_SHAPE, "matmul: at most one batch dim is supported");
    if (a->dtype != CTB_F32 || b->dtype != CTB_F32) return set_error(CTB_ERR_DTYPE, "matmul_tc: only Float32 tensors are supported");
    const int64_t K = a->shape[a->ndim - 1], M = a->shape[a->ndim - 2], N = b->shape[b->ndim - 1];
    if (b->shape[b->ndim - 2] != K) return set_error(CTB_ERR_SHAPE, "matmul_mp shape mismatch");
    const int64_t batch_a = a->ndim == 3 ? a->shape[0] : 1, batch_b = b->ndim == 3 ? b->shape[0] : 1;
    const int64_t batch = batch_a > batch_b ? batch_a : batch_b;
    if ((batch_a != batch && batch_a != 1) || (batch_b != batch && batch_b != 1))
        return set_error(CTB_ERR_SHAPE, "matmul_mp shape mismatch");
    if ((rc = check_out(out, batch * M * N, CTB_F32, "matmul_tc"))) return rc;
    const ctb_view* ins[2] = {a, b};
    if ((rc = check_no_alias(out, ins, 2, "matmul_tc"))) return rc;
    cudaStream_t st = (cudaStream_t)stream;
    if (batch * M * N == 0) return CTB_OK;
    if (M >= (int64_t(1) << 31) || N >= (int64_t(1) << 31) || K >= (int64_t(1) << 31))
        return set_error(CTB_ERR_LIMIT, "matmul_tc: extents must be below 2^31");

    // which operands can be used where they lie
    const int64_t Kp = (K + 3) / 4 * 4;
    auto usable = [&](const ctb_view* v, int row_dim, int k_dim, int64_t rows) {
        const bool k_unit = K <= 1 || v->stride[k_dim] == 1;
        const int64_t ld = v->stride[row_dim];
        const bool ld_ok = rows <= 1 || (ld % 4 == 0 && ld >= K);
        const bool batch_ok = v->ndim < 3 || v->shape[0] == 1 || v->stride[0] % 4 == 0;
        return k_unit && ld_ok && batch_ok && is_aligned(elem_ptr(v), 16);
    };
    const bool a_direct = usable(a, a->ndim - 2, a->ndim - 1, M);
    const bool b_direct = usable(b, b->ndim - 1, b->ndim - 2, N);      // b[K, N] seen as bt[N, K]: rows = N, k = dim -2
    const size_t a_bytes = a_direct ? 0 : align_up((size_t)batch_a * M * Kp * 4, 256);
    const size_t b_bytes = b_direct ? 0 : align_up((size_t)batch_b * N * Kp * 4, 256);
    void* ws = nullptr;
    if ((rc = ensure_workspace(kTicketBytes + 256 + a_bytes + b_bytes, &ws, st))) return rc;
    int* err_word = (int*)((char*)ws + kTicketBytes);
    float* a_pack = (float*)((char*)ws + kTicketBytes + 256);
    float* b_pack = (float*)((char*)a_pack + a_bytes);
    int* err = status ? status : err_word;
    CTB_CUDA_TRY(cudaMemsetAsync(err, 0, sizeof(int), st));

    // packed copies: [batch, rows, Kp] with the pad columns zeroed (zeros add nothing to the products)
    auto pack = [&](const ctb_view* v, bool transpose, int64_t nb, int64_t rows, float* dst) -> int {
        if (Kp != K) CTB_CUDA_TRY(cudaMemsetAsync(dst, 0, (size_t)nb * rows * Kp * 4, st));
        ctb_view src = *v;                       // as [nb, rows, K]
        const int nd = v->ndim;
        const int rd = transpose ? nd - 1 : nd - 2, kd = transpose ? nd - 2 : nd - 1;
        src.ndim = 3;
        src.shape[0] = nb;            src.stride[0] = (nd == 3 && v->shape[0] > 1) ? v->stride[0] : 0;
        src.shape[1] = rows;          src.stride[1] = v->stride[rd];
        src.shape[2] = K;             src.stride[2] = v->stride[kd];
        ctb_view d = src;
        d.base = dst;
        d.offset = 0;
        d.stride[0] = rows * Kp; d.stride[1] = Kp; d.stride[2] = 1;
        if (K == 0) return CTB_OK;
        return ctb_copy_into(&src, &d, stream);
    };
    if (!a_direct && (rc = pack(a, false, batch_a, M, a_pack))) return rc;
    if (!b_direct && (rc = pack(b, true, batch_b, N, b_pack))) return rc;

    for (int64_t i = 0; i < batch; ++i) {
        const float* pa;
        const float* pb;
        int64_t lda, ldb;
        if (a_direct) {
            pa = (const float*)elem_ptr(a) + ((a->ndim == 3 && batch_a > 1) ? i * a->stride[0] : 0);
            lda = M > 1 ? a->stride[a->ndim - 2] : Kp;
        } else {
            pa = a_pack + (batch_a > 1 ? i : 0) * M * Kp;
            lda = Kp;
        }
        if (b_direct) {
            pb = (const float*)elem_ptr(b) + ((b->ndim == 3 && batch_b > 1) ? i * b->stride[0] : 0);
            ldb = N > 1 ? b->stride[b->ndim - 1] : Kp;
        } else {
            pb = b_pack + (batch_b > 1 ? i : 0) * N * Kp;
            ldb = Kp;
        }
        float* pc = (float*)elem_ptr_mut(out) + i * M * N;
        if ((rc = launch_matmul_tf32(pa, lda, pb, ldb, pc, N, M, N, K, err, st))) return rc;
    }
    return CTB_OK;
}

// ---- copies into existing tensors: copy_into, cat ----------------------------------------------------------
int ctb_copy_into(const ctb_view* src, const ctb_view* dst, void* stream) {
    int rc;
    if ((rc = check_view(src, "copy: null input", "copy"))) return rc;
    if ((rc = check_view(dst, "output: null view", "copy"))) return rc;
    if (src->dtype != dst->dtype) return set_error(CTB_ERR_DTYPE, "copy: output dtype mismatch");
    const ctb_view* in[1] = {src};
    Plan p;
    if ((rc = build_plan(in, 1, &p, dst))) return rc;
    return launch_copy((int)dtype_bytes(src->dtype), p, elem_ptr(src), elem_ptr_mut(dst), (cudaStream_t)stream);
}

int ctb_cat(const ctb_view* const* inputs, int count, int dim, const ctb_view* out, void* stream) {
    int rc;
    if (!inputs || count <= 0) return set_error(CTB_ERR_ARG, "cat_mp: empty list");
    for (int i = 0; i < count; ++i)
        if ((rc = check_view(inputs[i], "cat_mp: null tensor", "cat_mp"))) return rc;
    const int nd = inputs[0]->ndim;
    if (dim < 0 || dim >= nd) return set_error(CTB_ERR_DIM, "cat_mp: dim out of range");
    int64_t total = 0;
    for (int i = 0; i < count; ++i) {
        if (inputs[i]->ndim != nd) return set_error(CTB_ERR_SHAPE, "cat_mp: ndim mismatch");
        if (inputs[i]->dtype != inputs[0]->dtype) return set_error(CTB_ERR_DTYPE, "cat_mp: dtype mismatch");
        for (int d = 0; d < nd; ++d)
            if (d != dim && inputs[i]->shape[d] != inputs[0]->shape[d])
                return set_error(CTB_ERR_SHAPE, "cat_mp: shape mismatch outside cat dim");
        total += inputs[i]->shape[dim];
    }
    int64_t numel = total;
    for (int d = 0; d < nd; ++d) if (d != dim) numel *= inputs[0]->shape[d];
    if ((rc = check_out(out, numel, inputs[0]->dtype, "cat_mp"))) return rc;
    if (out->ndim != nd) return set_error(CTB_ERR_SHAPE, "cat_mp: output has the wrong number of dims");
    for (int d = 0; d < nd; ++d)
        if (out->shape[d] != (d == dim ? total : inputs[0]->shape[d]))
            return set_error(CTB_ERR_SHAPE, "cat_mp: output has the wrong shape");
    // row-major strides of the output; each input lands in its slice along `dim`
    int64_t ostride[CTB_MAX_DIMS], run = 1;
    for (int d = nd - 1; d >= 0; --d) { ostride[d] = run; run *= out->shape[d]; }
    int64_t at = 0;
    for (int i = 0; i < count; ++i) {
        ctb_view slice = *out;
        for (int d = 0; d < nd; ++d) { slice.stride[d] = ostride[d]; slice.shape[d] = inputs[i]->shape[d]; }
        slice.offset = out->offset + at * ostride[dim];
        at += inputs[i]->shape[dim];
        if (inputs[i]->shape[dim] == 0) continue;
        if ((rc = ctb_copy_into(inputs[i], &slice, stream))) return rc;
    }
    return CTB_OK;
}

// ---- optimizer steps ---------------------------------------------------------------------------------
static int optimizer_operands(const ctb_view* param, const ctb_view* grad, const char* who) {
    int rc;
    if ((rc = check_view(param, "optimizer step: null parameter", who))) return rc;
    if ((rc = check_view(grad, "optimizer step: null gradient", who))) return rc;
    if (param->dtype != grad->dtype) return set_error(CTB_ERR_DTYPE, "%s: parameter and gradient dtypes differ", who);
    if (view_numel(param) != view_numel(grad)) return set_error(CTB_ERR_SHAPE, "%s: parameter and gradient sizes differ", who);
    // the reference walks raw storage linearly (train_utils.h:62-68): only contiguous buffers mean the same here
    if (!view_contiguous(param) || !view_contiguous(grad)) return set_error(CTB_ERR_SHAPE, "%s: parameter and gradient must be contiguous", who);
    return CTB_OK;
}

int ctb_sgd_step(const ctb_view* param, const ctb_view* grad, double lr, void* stream) {
    int rc;
    if ((rc = optimizer_operands(param, grad, "sgd_step"))) return rc;
    return launch_sgd(param->dtype, elem_ptr_mut(param), elem_ptr(grad), view_numel(param), lr, (cudaStream_t)stream);
}

int ctb_adam_step(const ctb_view* param, const ctb_view* grad, float* m, float* v, double lr, double beta1,
                  double beta2, double eps, int step, double weight_decay, int decoupled_decay, void* stream) {
    int rc;
    if ((rc = optimizer_operands(param, grad, "adam_step"))) return rc;
    if (param->dtype != CTB_F32) return set_error(CTB_ERR_DTYPE, "adam_step: only Float32 parameters are updated");
    if (view_numel(param) == 0) return CTB_OK;
    if (!m || !v) return set_error(CTB_ERR_NULL, "adam_step: null moment buffer");
    if (step < 1) return set_error(CTB_ERR_ARG, "adam_step: the step count starts at 1");
    return launch_adam((float*)elem_ptr_mut(param), (const float*)elem_ptr(grad), m, v, view_numel(param), lr, beta1,
                       beta2, eps, step, weight_decay, decoupled_decay, (cudaStream_t)stream);
}

int ctb_optimizer_step(int kind, const ctb_view* param, const ctb_view* grad, float* state1, float* state2,
                       const ctb_optimizer_hyper* hyper, int step, void* stream) {
    if (!hyper) return set_error(CTB_ERR_NULL, "optimizer step: null hyper-parameters");
    if (kind == CTB_OPT_SGD) return ctb_sgd_step(param, grad, hyper->lr, stream);
    if (kind == CTB_OPT_ADAM || kind == CTB_OPT_ADAMW)
        return ctb_adam_step(param, grad, state1, state2, hyper->lr, hyper->beta1, hyper->beta2, hyper->eps, step,
                             hyper->weight_decay, kind == CTB_OPT_ADAMW, stream);
    if (kind < 0 || kind >= CTB_OPTIMIZER_COUNT) return set_error(CTB_ERR_ARG, "optimizer step: unknown optimizer %d", kind);
    int rc;
    if ((rc = optimizer_operands(param, grad, "optimizer_step"))) return rc;
    if (param->dtype != CTB_F32) return set_error(CTB_ERR_DTYPE, "optimizer_step: only Float32 parameters are updated");
    const bool two = kind == CTB_OPT_ADAMAX || kind == CTB_OPT_NADAM || kind == CTB_OPT_RADAM;
    if (view_numel(param) == 0) return CTB_OK;
    if (!state1 || (two && !state2)) return set_error(CTB_ERR_NULL, "optimizer_step: null state buffer");
    if (step < 1) return set_error(CTB_ERR_ARG, "optimizer_step: the step count starts at 1");
    return launch_optimizer(kind, (float*)elem_ptr_mut(param), (const float*)elem_ptr(grad), state1, state2,
                            view_numel(param), *hyper, step, (cudaStream_t)stream);
}

// ---- host-buffer entry points --------------------------------------------------------------------------
static int host_elementwise(int nin, int op, const ctb_view* a, const ctb_view* b, double scalar,
                            const ctb_view* out, int device) {
    int rc;
    const char* who = nin == 2 ? "binary_op" : "unary_op";
    if ((rc = check_view(a, nin == 2 ? "binary_op: null input" : "unary_op: null input", who))) return rc;
    if (nin == 2 && (rc = check_view(b, "binary_op: null input", who))) return rc;
    if (nin == 2 && a->dtype != b->dtype) return set_error(CTB_ERR_DTYPE, "binary_op: operands must have the same dtype");
    const ctb_view* in[2] = {a, b};
    Plan p;
    if ((rc = build_plan(in, nin, &p))) return rc;
    if ((rc = check_out(out, p.numel, a->dtype, who))) return rc;
    if (p.numel == 0) return CTB_OK;
    if (device < 0 || device >= kMaxDevices) return set_error(CTB_ERR_CUDA, "cannot select CUDA device %d", device);
    std::lock_guard<std::mutex> host_lock(g_host_mu[device]);
    DeviceGuard guard(device);
    if (!guard.ok) return set_error(CTB_ERR_CUDA, "cannot select CUDA device %d", device);
    const size_t es = dtype_bytes(a->dtype);
    char* stage;
    cudaStream_t* streams;

    bool flat = p.ndim == 1;
    for (int i = 0; i < nin; ++i) if (p.stride[i][0] != 1) flat = false;
    if (flat && p.numel > kHostChunkElems) {
        // pipelined: chunk c uses stage slot c % 3 on stream c % 3 (upload -> kernel -> download)
        const int64_t chunk = kHostChunkElems;
        const size_t slot = align_up((size_t)chunk * es, 256) * (nin + 1);
        if ((rc = ensure_stage(device, slot * 3, (void**)&stage, &streams))) return rc;
        const char* ha = (const char*)elem_ptr(a);
        const char* hb = nin == 2 ? (const char*)elem_ptr(b) : nullptr;
        char* ho = (char*)elem_ptr_mut(out);
        int64_t c = 0;
        // one chunk: upload -> kernel -> download on its stream
        auto run_chunk = [&](int64_t lo, int64_t c) -> int {
            const int64_t n = p.numel - lo < chunk ? p.numel - lo : chunk;
            cudaStream_t st = streams[c % 3];
            char* base = stage + slot * (c % 3);
            char* da = base;
            char* db = base + align_up((size_t)chunk * es, 256);
            char* dout = base + align_up((size_t)chunk * es, 256) * nin;
            CTB_CUDA_TRY(cudaMemcpyAsync(da, ha + (size_t)lo * es, (size_t)n * es, cudaMemcpyHostToDevice, st));
            if (nin == 2) CTB_CUDA_TRY(cudaMemcpyAsync(db, hb + (size_t)lo * es, (size_t)n * es, cudaMemcpyHostToDevice, st));
            Plan cp = p;
            cp.numel = n;
            cp.shape[0] = n;
            int r = nin == 2 ? launch_binary(op, a->dtype, cp, da, db, dout, st)
                             : launch_unary(op, a->dtype, cp, da, scalar, dout, st);
            if (r) return r;
            CTB_CUDA_TRY(cudaMemcpyAsync(ho + (size_t)lo * es, dout, (size_t)n * es, cudaMemcpyDeviceToHost, st));
            return CTB_OK;
        };
        for (int64_t lo = 0; lo < p.numel && !rc; lo += chunk, ++c) rc = run_chunk(lo, c);
        // also on failure: no copy may still read or write the caller's buffers after the return
        for (int i = 0; i < 3; ++i) {
            const cudaError_t e = cudaStreamSynchronize(streams[i]);
            if (e != cudaSuccess && !rc) rc = cuda_error(e, "host-buffer pipeline");
        }
        return rc;
    }
    // general case: upload the touched storage spans, run once, download
    const size_t out_bytes = align_up((size_t)p.numel * es, 256);
    const size_t total = span_bytes(a) + (nin == 2 ? span_bytes(b) : 0) + out_bytes;
    if ((rc = ensure_stage(device, total, (void**)&stage, &streams))) return rc;
    cudaStream_t st = streams[0];
    size_t used = 0;
    ctb_view da, db, dout = *out;
    if ((rc = upload_view(a, stage, &used, &da, st))) return rc;
    if (nin == 2 && (rc = upload_view(b, stage, &used, &db, st))) return rc;
    dout.base = stage + used;
    dout.offset = 0;
    rc = nin == 2 ? ctb_binary(op, &da, &db, &dout, st) : ctb_unary(op, &da, scalar, &dout, st);
    if (rc) { cudaStreamSynchronize(st); return rc; }    // the uploads still read the caller's buffers
    CTB_CUDA_TRY(cudaMemcpyAsync(elem_ptr_mut(out), dout.base, (size_t)p.numel * es, cudaMemcpyDeviceToHost, st));
    CTB_CUDA_TRY(cudaStreamSynchronize(st));
    return CTB_OK;
}

int ctb_binary_host(int op, const ctb_view* a, const ctb_view* b, const ctb_view* out, int device) {
    if (op < 0 || op >= CTB_BINARY_OP_COUNT) return set_error(CTB_ERR_ARG, "binary_op: unknown operator code %d", op);
    return host_elementwise(2, op, a, b, 0.0, out, device);
}

int ctb_unary_host(int op, const ctb_view* a, double scalar, const ctb_view* out, int device) {
    if (op < 0 || op >= CTB_UNARY_OP_COUNT) return set_error(CTB_ERR_ARG, "unary_op: unknown operator code %d", op);
    return host_elementwise(1, op, a, nullptr, scalar, out, device);
}

int ctb_reduce_host(int op, const ctb_view* a, int dim, const ctb_view* out, int device) {
    int rc;
    if ((rc = reduce_arg_check(op, a, dim))) return rc;
    if ((rc = reduce_out_check(op, a, dim, out))) return rc;
    if (device < 0 || device >= kMaxDevices) return set_error(CTB_ERR_CUDA, "cannot select CUDA device %d", device);
    std::lock_guard<std::mutex> host_lock(g_host_mu[device]);
    DeviceGuard guard(device);
    if (!guard.ok) return set_error(CTB_ERR_CUDA, "cannot select CUDA device %d", device);
    const size_t oes = dtype_bytes(out->dtype);
    const int64_t nout = view_numel(out);
    char* stage;
    cudaStream_t* streams;
    const size_t total = span_bytes(a) + align_up((size_t)nout * oes, 256);
    if ((rc = ensure_stage(device, total, (void**)&stage, &streams))) return rc;
    cudaStream_t st = streams[0];
    size_t used = 0;
    ctb_view da, dout = *out;
    if ((rc = upload_view(a, stage, &used, &da, st))) return rc;
    dout.base = stage + used;
    dout.offset = 0;
    if ((rc = ctb_reduce(op, &da, dim, &dout, st))) { cudaStreamSynchronize(st); return rc; }
    CTB_CUDA_TRY(cudaMemcpyAsync(elem_ptr_mut(out), dout.base, (size_t)nout * oes, cudaMemcpyDeviceToHost, st));
    CTB_CUDA_TRY(cudaStreamSynchronize(st));
    return CTB_OK;
}

}  // extern "C"
