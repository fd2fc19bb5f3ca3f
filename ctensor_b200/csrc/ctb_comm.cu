// Multi-GPU side of the operator path, single process: one communicator over the GPUs of the box,
// one stream per GPU, and the one collective the path has — the all-reduce that combines the
// per-GPU partials of a full-tensor reduction.
//
// How the path shards (nothing of this exists in the reference, which is CPU-only):
//   * elementwise / broadcast / row-wise operators: the leading dim is cut into equal contiguous
//     ranges (ctb_shard_range), one per GPU; no communication.
//   * full-tensor sum / mean / max / min: every GPU reduces its shard to one fp64 partial
//     (ctb_reduce_full_partial), ONE ncclAllReduce of a double (sum / max / min) combines them,
//     every GPU applies the reference's rounding (ctb_finalize_full).
//   * a reduction over the leading dim of row shards: per-GPU fp64 partial rows, one all-reduce
//     of them (ctb_allreduce on Double64 buffers), rounding by the caller.
// No GPU reads another GPU's memory in a kernel of this library; NCCL moves the bytes.
//
// NCCL is loaded when ctb_comm_init_all is first called (dlopen of libnccl.so.2, or of the
// library named by CTB_NCCL_LIBRARY), so the operator library itself has no link-time
// dependency on it and a process that already carries an NCCL (a Python process with torch, for
// one) shares that copy.
#include <dlfcn.h>
#include <nccl.h>

#include <cstdlib>
#include <cstring>
#include <mutex>
#include <string>
#include <vector>

#include "ctb_common.cuh"

namespace ctb {
namespace {

struct NcclApi {
    void* handle = nullptr;
    ncclResult_t (*CommInitAll)(ncclComm_t*, int, const int*) = nullptr;
    ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
    ncclResult_t (*AllReduce)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*GroupStart)() = nullptr;
    ncclResult_t (*GroupEnd)() = nullptr;
    const char* (*GetErrorString)(ncclResult_t) = nullptr;
};

struct Comm {
    int n = 0;
    std::vector<int> devices;
    std::vector<ncclComm_t> comms;
    std::vector<cudaStream_t> streams;
    std::vector<double*> partial;         // one fp64 slot per device for the full reductions
};

std::mutex g_comm_mu;
NcclApi g_nccl;
Comm g_comm;

int load_nccl() {
    if (g_nccl.handle) return CTB_OK;
    const char* name = std::getenv("CTB_NCCL_LIBRARY");
    if (!name || !*name) name = "libnccl.so.2";
    void* h = dlopen(name, RTLD_NOW | RTLD_LOCAL);
    if (!h) return set_error(CTB_ERR_CUDA, "cannot load NCCL (%s): %s", name, dlerror());
    NcclApi api;
    api.handle = h;
    api.CommInitAll = (decltype(api.CommInitAll))dlsym(h, "ncclCommInitAll");
    api.CommDestroy = (decltype(api.CommDestroy))dlsym(h, "ncclCommDestroy");
    api.AllReduce = (decltype(api.AllReduce))dlsym(h, "ncclAllReduce");
    api.GroupStart = (decltype(api.GroupStart))dlsym(h, "ncclGroupStart");
    api.GroupEnd = (decltype(api.GroupEnd))dlsym(h, "ncclGroupEnd");
    api.GetErrorString = (decltype(api.GetErrorString))dlsym(h, "ncclGetErrorString");
    if (!api.CommInitAll || !api.CommDestroy || !api.AllReduce || !api.GroupStart || !api.GroupEnd || !api.GetErrorString) {
        dlclose(h);
        return set_error(CTB_ERR_CUDA, "%s lacks a required NCCL entry point", name);
    }
    g_nccl = api;
    return CTB_OK;
}

int nccl_error(ncclResult_t r, const char* what) {
    if (r == ncclSuccess) return CTB_OK;
    return set_error(CTB_ERR_CUDA, "NCCL error in %s: %s", what, g_nccl.GetErrorString ? g_nccl.GetErrorString(r) : "?");
}

struct DeviceRestore {
    int prev = -1;
    DeviceRestore() { if (cudaGetDevice(&prev) != cudaSuccess) { cudaGetLastError(); prev = -1; } }
    ~DeviceRestore() { if (prev >= 0) cudaSetDevice(prev); }
};

void destroy_locked() {
    for (int i = 0; i < g_comm.n; ++i) {
        if (cudaSetDevice(g_comm.devices[i]) != cudaSuccess) { cudaGetLastError(); continue; }
        if (g_comm.streams[i]) cudaStreamSynchronize(g_comm.streams[i]);
        if (g_comm.comms[i]) g_nccl.CommDestroy(g_comm.comms[i]);
        if (g_comm.streams[i]) cudaStreamDestroy(g_comm.streams[i]);
        if (g_comm.partial[i]) cudaFree(g_comm.partial[i]);
    }
    g_comm = Comm();
}

bool nccl_type(int dtype, ncclDataType_t* t, size_t* bytes) {
    switch (dtype) {
    case CTB_F32: *t = ncclFloat32; *bytes = 4; return true;
    case CTB_I32: *t = ncclInt32; *bytes = 4; return true;
    case CTB_F64: *t = ncclFloat64; *bytes = 8; return true;
    }
    return false;
}

bool nccl_op(int op, ncclRedOp_t* r) {
    switch (op) {
    case CTB_SUM: case CTB_MEAN: *r = ncclSum; return true;
    case CTB_MAX: *r = ncclMax; return true;
    case CTB_MIN: *r = ncclMin; return true;
    }
    return false;
}

// In-place all-reduce of buffers[i] (on device i) on the communicator's streams; no waiting.
int allreduce_locked(void* const* buffers, size_t count, ncclDataType_t t, ncclRedOp_t op) {
    int rc = nccl_error(g_nccl.GroupStart(), "ncclGroupStart");
    if (rc) return rc;
    for (int i = 0; i < g_comm.n && !rc; ++i)
        rc = nccl_error(g_nccl.AllReduce(buffers[i], buffers[i], count, t, op, g_comm.comms[i], g_comm.streams[i]), "ncclAllReduce");
    const int rc_end = nccl_error(g_nccl.GroupEnd(), "ncclGroupEnd");     // always closes the group
    return rc ? rc : rc_end;
}

int sync_all_locked() {
    int rc = CTB_OK;
    for (int i = 0; i < g_comm.n; ++i) {
        cudaError_t e = cudaSetDevice(g_comm.devices[i]);
        if (e == cudaSuccess) e = cudaStreamSynchronize(g_comm.streams[i]);
        if (e != cudaSuccess && !rc) rc = cuda_error(e, "communicator stream");
    }
    return rc;
}

}  // namespace
}  // namespace ctb

using namespace ctb;

extern "C" {

int ctb_shard_range(int64_t total, int parts, int index, int64_t* lo, int64_t* hi) {
    if (!lo || !hi) return set_error(CTB_ERR_NULL, "ctb_shard_range: null result pointer");
    if (total < 0 || parts <= 0 || index < 0 || index >= parts) return set_error(CTB_ERR_ARG, "ctb_shard_range: bad arguments");
    // the first (total % parts) shards get one more element: sizes differ by at most one
    const int64_t base = total / parts, extra = total % parts;
    *lo = index * base + (index < extra ? index : extra);
    *hi = *lo + base + (index < extra ? 1 : 0);
    return CTB_OK;
}

int ctb_comm_init_all(int ndev, const int* devices) {
    std::lock_guard<std::mutex> lk(g_comm_mu);
    int visible = 0;
    if (cudaGetDeviceCount(&visible) != cudaSuccess) { cudaGetLastError(); visible = 0; }
    if (visible <= 0) return set_error(CTB_ERR_CUDA, "no CUDA device (this library has no CPU fallback)");
    if (ndev <= 0) ndev = visible;
    if (ndev > visible) return set_error(CTB_ERR_ARG, "ctb_comm_init_all: %d devices asked for, %d visible", ndev, visible);
    int rc = load_nccl();
    if (rc) return rc;
    if (g_comm.n) destroy_locked();
    DeviceRestore restore;
    Comm c;
    c.n = ndev;
    c.devices.resize(ndev);
    c.comms.assign(ndev, nullptr);
    c.streams.assign(ndev, nullptr);
    c.partial.assign(ndev, nullptr);
    for (int i = 0; i < ndev; ++i) {
        c.devices[i] = devices ? devices[i] : i;
        if (c.devices[i] < 0 || c.devices[i] >= visible) return set_error(CTB_ERR_ARG, "ctb_comm_init_all: no device %d", c.devices[i]);
        for (int j = 0; j < i; ++j)
            if (c.devices[j] == c.devices[i]) return set_error(CTB_ERR_ARG, "ctb_comm_init_all: device %d listed twice", c.devices[i]);
    }
    g_comm = c;
    if ((rc = nccl_error(g_nccl.CommInitAll(g_comm.comms.data(), ndev, g_comm.devices.data()), "ncclCommInitAll"))) {
        g_comm = Comm();
        return rc;
    }
    for (int i = 0; i < ndev; ++i) {
        cudaError_t e = cudaSetDevice(g_comm.devices[i]);
        if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&g_comm.streams[i], cudaStreamNonBlocking);
        if (e == cudaSuccess) e = cudaMalloc((void**)&g_comm.partial[i], 256);
        if (e != cudaSuccess) {
            rc = cuda_error(e, "communicator set-up");
            destroy_locked();
            return rc;
        }
    }
    return CTB_OK;
}

int ctb_comm_size(void) {
    std::lock_guard<std::mutex> lk(g_comm_mu);
    return g_comm.n;
}

int ctb_comm_device(int rank) {
    std::lock_guard<std::mutex> lk(g_comm_mu);
    return (rank >= 0 && rank < g_comm.n) ? g_comm.devices[rank] : -1;
}

void* ctb_comm_stream(int rank) {
    std::lock_guard<std::mutex> lk(g_comm_mu);
    return (rank >= 0 && rank < g_comm.n) ? (void*)g_comm.streams[rank] : nullptr;
}

int ctb_comm_sync(void) {
    std::lock_guard<std::mutex> lk(g_comm_mu);
    if (!g_comm.n) return set_error(CTB_ERR_ARG, "no communicator (call ctb_comm_init_all first)");
    DeviceRestore restore;
    return sync_all_locked();
}

int ctb_comm_destroy(void) {
    std::lock_guard<std::mutex> lk(g_comm_mu);
    if (!g_comm.n) return CTB_OK;
    DeviceRestore restore;
    destroy_locked();
    return CTB_OK;
}

int ctb_allreduce(void* const* buffers, size_t count, int dtype, int op) {
    std::lock_guard<std::mutex> lk(g_comm_mu);
    if (!g_comm.n) return set_error(CTB_ERR_ARG, "no communicator (call ctb_comm_init_all first)");
    if (!buffers) return set_error(CTB_ERR_NULL, "ctb_allreduce: null buffer list");
    for (int i = 0; i < g_comm.n; ++i)
        if (!buffers[i] && count) return set_error(CTB_ERR_NULL, "ctb_allreduce: null buffer for rank %d", i);
    ncclDataType_t t;
    ncclRedOp_t r;
    size_t bytes;
    if (!nccl_type(dtype, &t, &bytes)) return set_error(CTB_ERR_DTYPE, "ctb_allreduce: unsupported dtype");
    if (!nccl_op(op, &r)) return set_error(CTB_ERR_ARG, "ctb_allreduce: the operator must be sum, max or min");
    if (count == 0) return CTB_OK;
    return allreduce_locked(buffers, count, t, r);
}

int ctb_full_reduce_sharded(int op, const ctb_view* const* shards, int64_t total_count, const ctb_view* const* outs) {
    std::lock_guard<std::mutex> lk(g_comm_mu);
    if (!g_comm.n) return set_error(CTB_ERR_ARG, "no communicator (call ctb_comm_init_all first)");
    if (!shards || !outs) return set_error(CTB_ERR_NULL, "reduction: null input");
    ncclRedOp_t r;
    if (!nccl_op(op, &r)) return set_error(CTB_ERR_ARG, "reduction: sharded full reductions exist for sum/mean/max/min");
    DeviceRestore restore;
    for (int i = 0; i < g_comm.n; ++i)
        if (!shards[i] || !outs[i]) return set_error(CTB_ERR_NULL, "reduction: null input");
    // an error after the first launch waits for what was queued before it returns: the caller's
    // buffers are then no longer in use (the error text of the failing call is kept)
    auto fail = [&](int code) {
        const std::string text = ctb_last_error();
        sync_all_locked();
        return set_error(code, "%s", text.c_str());
    };
    int rc;
    // 1. every GPU folds its shard to one fp64 partial, on its communicator stream
    for (int i = 0; i < g_comm.n; ++i) {
        const cudaError_t e = cudaSetDevice(g_comm.devices[i]);
        if (e != cudaSuccess) return fail(cuda_error(e, "cudaSetDevice"));
        if ((rc = ctb_reduce_full_partial(op, shards[i], g_comm.partial[i], g_comm.streams[i]))) return fail(rc);
    }
    // 2. one all-reduce of a double
    std::vector<void*> bufs(g_comm.partial.begin(), g_comm.partial.end());
    if ((rc = allreduce_locked(bufs.data(), 1, ncclFloat64, r))) return fail(rc);
    // 3. the reference's rounding on every GPU
    for (int i = 0; i < g_comm.n; ++i) {
        const cudaError_t e = cudaSetDevice(g_comm.devices[i]);
        if (e != cudaSuccess) return fail(cuda_error(e, "cudaSetDevice"));
        if ((rc = ctb_finalize_full(op, g_comm.partial[i], total_count, outs[i], g_comm.streams[i]))) return fail(rc);
    }
    return sync_all_locked();
}

}  // extern "C"
