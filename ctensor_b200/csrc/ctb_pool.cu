// Pooled host-dereferenceable (CUDA managed) storage: the device allocator behind the host
// layer's Storage::allocate.
//
// The reference sketches the same thing and never finishes it: a size-bucketed pool of
// cudaMallocManaged blocks rounded to 512 bytes (src/core/tensor.h:253-289) behind
// Storage::allocate (src/core/tensor.cpp:18-39).  Every operator of the reference returns a fresh
// tensor, so a training step allocates and frees the same few sizes over and over; cudaMallocManaged
// and cudaFree cost tens of microseconds to milliseconds each and cudaFree waits for the device.
// Here a freed block goes onto a per-device free list keyed by its rounded size and is handed out
// again without touching the driver; its pages are already resident in HBM, so the next kernel
// that writes it takes no page faults.
//
// Ordering rule: a block may be reused while earlier kernels that read it are still queued only
// if the next user is ordered after them.  The host layer issues everything on one stream per
// device, which gives exactly that; a caller that uses several streams synchronises before it
// frees.
#include <cstring>
#include <map>
#include <mutex>
#include <unordered_map>
#include <vector>

#include "ctb_common.cuh"

namespace ctb {
namespace {

constexpr int kMaxPoolDevices = 64;
constexpr size_t kRound = 512;                       // the reference's rounding (tensor.h:262)
constexpr size_t kLargeRound = size_t(2) << 20;      // blocks of 1 MiB and more: whole 2 MiB pages

struct DevicePool {
    std::multimap<size_t, void*> free_blocks;        // rounded size -> cached block
    size_t cached_bytes = 0;
    size_t live_bytes = 0;
    size_t limit_bytes = size_t(64) << 30;           // cached (idle) bytes kept at most
    uint64_t hits = 0, misses = 0, trims = 0;
};

struct BlockInfo {
    size_t bytes;
    int device;
};

std::mutex g_pool_mu;
DevicePool g_pool[kMaxPoolDevices];
std::unordered_map<void*, BlockInfo> g_blocks;       // every block handed out or cached

size_t round_size(size_t bytes) {
    if (bytes == 0) bytes = 1;
    const size_t r = bytes >= (size_t(1) << 20) ? kLargeRound : kRound;
    return (bytes + r - 1) / r * r;
}

// Free cached blocks, largest first, until at most `keep` cached bytes remain.  Caller holds the lock.
void trim_locked(DevicePool& p, size_t keep) {
    while (p.cached_bytes > keep && !p.free_blocks.empty()) {
        auto it = std::prev(p.free_blocks.end());
        cudaFree(it->second);
        g_blocks.erase(it->second);
        p.cached_bytes -= it->first;
        p.free_blocks.erase(it);
        ++p.trims;
    }
}

}  // namespace
}  // namespace ctb

using namespace ctb;

extern "C" {

int ctb_pool_alloc_managed(void** ptr, size_t bytes, int zero, int device, void* stream) {
    if (!ptr) return set_error(CTB_ERR_NULL, "ctb_pool_alloc_managed: null result pointer");
    *ptr = nullptr;
    if (device < 0 || device >= kMaxPoolDevices) return set_error(CTB_ERR_ARG, "ctb_pool_alloc_managed: device %d out of range", device);
    const size_t rounded = round_size(bytes);
    void* p = nullptr;
    {
        std::lock_guard<std::mutex> lk(g_pool_mu);
        DevicePool& pool = g_pool[device];
        auto it = pool.free_blocks.find(rounded);
        if (it != pool.free_blocks.end()) {
            p = it->second;
            pool.free_blocks.erase(it);
            pool.cached_bytes -= rounded;
            pool.live_bytes += rounded;
            ++pool.hits;
        } else {
            ++pool.misses;
        }
    }
    if (!p) {
        cudaError_t e = cudaMallocManaged(&p, rounded, cudaMemAttachGlobal);
        if (e != cudaSuccess) {
            // out of memory with idle blocks cached: give them back and try once more
            cudaGetLastError();
            {
                std::lock_guard<std::mutex> lk(g_pool_mu);
                for (int d = 0; d < kMaxPoolDevices; ++d) trim_locked(g_pool[d], 0);
            }
            e = cudaMallocManaged(&p, rounded, cudaMemAttachGlobal);
        }
        if (e != cudaSuccess) return cuda_error(e, "cudaMallocManaged");
        // pages live in this device's HBM unless the host touches them; the hint is advisory
        // (platforms without concurrent managed access reject it) and failure is not an error
        if (cudaMemAdvise(p, rounded, cudaMemAdviseSetPreferredLocation, device) != cudaSuccess) cudaGetLastError();
        std::lock_guard<std::mutex> lk(g_pool_mu);
        g_blocks[p] = {rounded, device};
        g_pool[device].live_bytes += rounded;
    }
    if (zero) {
        const cudaError_t e = cudaMemsetAsync(p, 0, bytes ? bytes : 1, (cudaStream_t)stream);
        if (e != cudaSuccess) {
            ctb_pool_free_managed(p);         // the block stays accounted for: back onto its free list
            return cuda_error(e, "cudaMemsetAsync");
        }
    }
    *ptr = p;
    return CTB_OK;
}

int ctb_pool_free_managed(void* ptr) {
    if (!ptr) return CTB_OK;
    std::lock_guard<std::mutex> lk(g_pool_mu);
    auto it = g_blocks.find(ptr);
    if (it == g_blocks.end()) return set_error(CTB_ERR_ARG, "ctb_pool_free_managed: not a block of this pool");
    DevicePool& pool = g_pool[it->second.device];
    const size_t bytes = it->second.bytes;
    pool.live_bytes -= bytes;
    pool.free_blocks.emplace(bytes, ptr);
    pool.cached_bytes += bytes;
    if (pool.cached_bytes > pool.limit_bytes) trim_locked(pool, pool.limit_bytes);
    return CTB_OK;
}

int ctb_pool_trim(int device) {
    std::lock_guard<std::mutex> lk(g_pool_mu);
    for (int d = 0; d < kMaxPoolDevices; ++d)
        if (device < 0 || d == device) trim_locked(g_pool[d], 0);
    return CTB_OK;
}

int ctb_pool_set_limit(int device, size_t cached_bytes) {
    if (device < 0 || device >= kMaxPoolDevices) return set_error(CTB_ERR_ARG, "ctb_pool_set_limit: device %d out of range", device);
    std::lock_guard<std::mutex> lk(g_pool_mu);
    g_pool[device].limit_bytes = cached_bytes;
    trim_locked(g_pool[device], cached_bytes);
    return CTB_OK;
}

int ctb_pool_stats(int device, ctb_pool_info* info) {
    if (!info) return set_error(CTB_ERR_NULL, "ctb_pool_stats: null result pointer");
    if (device < 0 || device >= kMaxPoolDevices) return set_error(CTB_ERR_ARG, "ctb_pool_stats: device %d out of range", device);
    std::lock_guard<std::mutex> lk(g_pool_mu);
    const DevicePool& p = g_pool[device];
    info->live_bytes = p.live_bytes;
    info->cached_bytes = p.cached_bytes;
    info->cached_blocks = p.free_blocks.size();
    info->hits = p.hits;
    info->misses = p.misses;
    info->trims = p.trims;
    return CTB_OK;
}

int ctb_prefetch_managed(void* ptr, size_t bytes, int device, void* stream) {
    if (!ptr || bytes == 0) return CTB_OK;
    // advisory: where managed memory cannot be prefetched the first kernel migrates the pages itself
    if (cudaMemPrefetchAsync(ptr, bytes, device, (cudaStream_t)stream) != cudaSuccess) cudaGetLastError();
    return CTB_OK;
}

}  // extern "C"
