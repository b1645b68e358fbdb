// VRAM slab allocator on CUDA virtual memory management: address space is reserved once per slab,
// physical memory is mapped region by region on demand and unmapped again under a byte ceiling.
//
// B200-side equivalent of the reference's stagehand-vmm crate (vmm_src/allocator.rs, slab.rs,
// eviction.rs, handle.rs): same verbs and the same policy -- a region is evictable when nobody holds
// it (refcount 0) and its release event has completed; victims go lowest slab priority first, least
// recently used first (vmm_src/eviction.rs:15-144).  Differences: one mutex instead of the lock-free
// fast path, and every wait is bounded.  sh_vmm_prefetch_async hands the mapping to one worker thread, as
// the reference's prefetch does (vmm_src/prefetch.rs); sh_vmm_ensure_resident with hold = 0 still maps in
// the calling thread.
//
// The driver entry points are resolved at run time (cudaGetDriverEntryPoint), so the library still
// loads on a host that has no GPU driver.
#include "../../include/stagehand_b200.h"

#include <cuda.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <chrono>
#include <cstdarg>
#include <cstdio>
#include <condition_variable>
#include <cstring>
#include <deque>
#include <map>
#include <mutex>
#include <thread>
#include <vector>

namespace {

thread_local char g_vmm_err[384] = "";

int vfail(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_vmm_err, sizeof(g_vmm_err), fmt, ap);
    va_end(ap);
    return code;
}

struct Driver {
    CUresult (*GetGranularity)(size_t*, const CUmemAllocationProp*, CUmemAllocationGranularity_flags) = nullptr;
    CUresult (*AddressReserve)(CUdeviceptr*, size_t, size_t, CUdeviceptr, unsigned long long) = nullptr;
    CUresult (*AddressFree)(CUdeviceptr, size_t) = nullptr;
    CUresult (*Create)(CUmemGenericAllocationHandle*, size_t, const CUmemAllocationProp*, unsigned long long) = nullptr;
    CUresult (*Map)(CUdeviceptr, size_t, size_t, CUmemGenericAllocationHandle, unsigned long long) = nullptr;
    CUresult (*SetAccess)(CUdeviceptr, size_t, const CUmemAccessDesc*, size_t) = nullptr;
    CUresult (*Unmap)(CUdeviceptr, size_t) = nullptr;
    CUresult (*Release)(CUmemGenericAllocationHandle) = nullptr;
    bool ok = false;
};

template <typename F>
bool resolve(const char* name, F* out) {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult status;
    if (cudaGetDriverEntryPoint(name, &fn, cudaEnableDefault, &status) != cudaSuccess || fn == nullptr ||
        status != cudaDriverEntryPointSuccess) {
        (void)cudaGetLastError();
        return false;
    }
    *out = reinterpret_cast<F>(fn);
    return true;
}

Driver& driver() {
    static Driver d;
    static std::once_flag once;
    std::call_once(once, [] {
        d.ok = resolve("cuMemGetAllocationGranularity", &d.GetGranularity) &&
               resolve("cuMemAddressReserve", &d.AddressReserve) && resolve("cuMemAddressFree", &d.AddressFree) &&
               resolve("cuMemCreate", &d.Create) && resolve("cuMemMap", &d.Map) &&
               resolve("cuMemSetAccess", &d.SetAccess) && resolve("cuMemUnmap", &d.Unmap) &&
               resolve("cuMemRelease", &d.Release);
    });
    return d;
}

struct Region {
    size_t offset = 0, size = 0;          // granularity-rounded, inside the slab's reservation
    bool mapped = false;
    CUmemGenericAllocationHandle handle = 0;
    int refcount = 0;
    uint64_t last_access = 0;
    cudaEvent_t released = nullptr;       // recorded on the user's stream at release
    bool event_pending = false;
};

struct Slab {
    CUdeviceptr base = 0;
    size_t size = 0;
    uint32_t priority = 0;
    std::vector<Region> regions;
};

struct Allocator {
    int device = 0;
    size_t granularity = 0;
    size_t ceiling = 0;
    size_t mapped = 0;
    uint64_t clock = 0;
    int64_t evictions = 0;
    int next_slab = 1;
    std::map<int, Slab> slabs;
    std::mutex mu;
    CUmemAllocationProp prop{};
    // background prefetch: (slab, region) requests served by one worker thread under `mu`
    std::deque<std::pair<int, int>> requests;
    std::condition_variable wake, idle;
    std::thread worker;
    bool worker_started = false, worker_busy = false, stopping = false;
    int64_t prefetch_failures = 0;
};

size_t round_up(size_t v, size_t g) { return (v + g - 1) / g * g; }

bool event_done(Region& r, int timeout_ms) {
    if (!r.event_pending) return true;
    const auto deadline = std::chrono::steady_clock::now() + std::chrono::milliseconds(timeout_ms);
    for (;;) {
        const cudaError_t q = cudaEventQuery(r.released);
        if (q == cudaSuccess) {
            r.event_pending = false;
            return true;
        }
        if (q != cudaErrorNotReady) {
            (void)cudaGetLastError();
            return false;
        }
        if (std::chrono::steady_clock::now() >= deadline) return false;
        std::this_thread::sleep_for(std::chrono::microseconds(50));
    }
}

int unmap_region(Allocator& a, Slab& s, Region& r) {
    Driver& d = driver();
    if (!r.mapped) return SH_OK;
    CUresult e = d.Unmap(s.base + r.offset, r.size);
    if (e != CUDA_SUCCESS) return vfail(SH_ERR_CUDA, "cuMemUnmap failed (%d)", static_cast<int>(e));
    e = d.Release(r.handle);
    if (e != CUDA_SUCCESS) return vfail(SH_ERR_CUDA, "cuMemRelease failed (%d)", static_cast<int>(e));
    r.mapped = false;
    r.handle = 0;
    a.mapped -= r.size;
    return SH_OK;
}

// Unmap unreferenced regions (lowest slab priority, then least recently used) until `need` more bytes fit.
int make_room(Allocator& a, size_t need, int skip_slab, int skip_region) {
    while (a.mapped + need > a.ceiling) {
        Slab* vs = nullptr;
        Region* vr = nullptr;
        for (auto& [sid, s] : a.slabs) {
            for (size_t i = 0; i < s.regions.size(); ++i) {
                Region& r = s.regions[i];
                if (!r.mapped || r.refcount > 0 || (sid == skip_slab && static_cast<int>(i) == skip_region)) continue;
                if (vr == nullptr || s.priority < vs->priority ||
                    (s.priority == vs->priority && r.last_access < vr->last_access)) {
                    vs = &s;
                    vr = &r;
                }
            }
        }
        if (vr == nullptr)
            return vfail(SH_ERR_OOM, "VRAM ceiling of %zu bytes reached and no region is evictable (mapped %zu, need %zu)",
                         a.ceiling, a.mapped, need);
        if (!event_done(*vr, 10000)) return vfail(SH_ERR_TIMEOUT, "released region is still in use on the GPU after 10 s");
        const int rc = unmap_region(a, *vs, *vr);
        if (rc != SH_OK) return rc;
        a.evictions += 1;
    }
    return SH_OK;
}

int map_region(Allocator& a, int slab_id, Slab& s, int region_id, Region& r) {
    Driver& d = driver();
    if (r.size > a.ceiling) return vfail(SH_ERR_OOM, "region of %zu bytes exceeds the VRAM ceiling of %zu", r.size, a.ceiling);
    int rc = make_room(a, r.size, slab_id, region_id);
    if (rc != SH_OK) return rc;
    CUresult e = d.Create(&r.handle, r.size, &a.prop, 0);
    if (e == CUDA_ERROR_OUT_OF_MEMORY) return vfail(SH_ERR_OOM, "cuMemCreate: out of device memory (%zu bytes)", r.size);
    if (e != CUDA_SUCCESS) return vfail(SH_ERR_CUDA, "cuMemCreate failed (%d)", static_cast<int>(e));
    e = d.Map(s.base + r.offset, r.size, 0, r.handle, 0);
    if (e != CUDA_SUCCESS) {
        d.Release(r.handle);
        return vfail(SH_ERR_CUDA, "cuMemMap failed (%d)", static_cast<int>(e));
    }
    CUmemAccessDesc access{};
    access.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
    access.location.id = a.device;
    access.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
    e = d.SetAccess(s.base + r.offset, r.size, &access, 1);
    if (e != CUDA_SUCCESS) {
        d.Unmap(s.base + r.offset, r.size);
        d.Release(r.handle);
        return vfail(SH_ERR_CUDA, "cuMemSetAccess failed (%d)", static_cast<int>(e));
    }
    r.mapped = true;
    a.mapped += r.size;
    return SH_OK;
}

Allocator* as_alloc(uint64_t h) { return reinterpret_cast<Allocator*>(static_cast<uintptr_t>(h)); }

int find(Allocator& a, int slab, int region, Slab** s_out, Region** r_out) {
    auto it = a.slabs.find(slab);
    if (it == a.slabs.end()) return vfail(SH_ERR_INVALID_ARG, "unknown slab %d", slab);
    *s_out = &it->second;
    if (r_out != nullptr) {
        if (region < 0 || region >= static_cast<int>(it->second.regions.size()))
            return vfail(SH_ERR_INVALID_ARG, "unknown region %d of slab %d", region, slab);
        *r_out = &it->second.regions[static_cast<size_t>(region)];
    }
    return SH_OK;
}

}  // namespace

extern "C" {

int32_t sh_vmm_last_error(char* buf, int32_t buf_len) {
    const int32_t n = static_cast<int32_t>(strlen(g_vmm_err));
    if (buf != nullptr && buf_len > 0) {
        const int32_t c = std::min(n, buf_len - 1);
        memcpy(buf, g_vmm_err, static_cast<size_t>(c));
        buf[c] = '\0';
    }
    return n;
}

int32_t sh_vmm_create(int32_t device, uint64_t ceiling_bytes, uint64_t* allocator_out) {
    if (allocator_out == nullptr) return vfail(SH_ERR_INVALID_ARG, "null allocator_out");
    if (cudaSetDevice(device) != cudaSuccess) {
        (void)cudaGetLastError();
        return vfail(SH_ERR_CUDA, "cudaSetDevice(%d) failed", device);
    }
    (void)cudaFree(nullptr);   // make sure the primary context exists before driver calls
    if (!driver().ok) return vfail(SH_ERR_UNSUPPORTED, "CUDA virtual memory management entry points are not available");
    auto* a = new Allocator();
    a->device = device;
    a->prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
    a->prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
    a->prop.location.id = device;
    if (driver().GetGranularity(&a->granularity, &a->prop, CU_MEM_ALLOC_GRANULARITY_MINIMUM) != CUDA_SUCCESS ||
        a->granularity == 0) {
        delete a;
        return vfail(SH_ERR_CUDA, "cuMemGetAllocationGranularity failed");
    }
    size_t free_b = 0, total_b = 0;
    cudaMemGetInfo(&free_b, &total_b);
    a->ceiling = ceiling_bytes != 0 ? static_cast<size_t>(ceiling_bytes) : total_b / 10 * 9;
    *allocator_out = static_cast<uint64_t>(reinterpret_cast<uintptr_t>(a));
    return SH_OK;
}

int32_t sh_vmm_destroy(uint64_t allocator) {
    Allocator* a = as_alloc(allocator);
    if (a == nullptr) return SH_OK;
    if (a->worker_started) {
        {
            std::lock_guard<std::mutex> lk(a->mu);
            a->stopping = true;
            a->requests.clear();
        }
        a->wake.notify_all();
        a->worker.join();
    }
    {
        std::lock_guard<std::mutex> lk(a->mu);
        for (auto& [sid, s] : a->slabs) {
            for (auto& r : s.regions) {
                (void)event_done(r, 10000);
                (void)unmap_region(*a, s, r);
                if (r.released != nullptr) cudaEventDestroy(r.released);
            }
            driver().AddressFree(s.base, s.size);
        }
        a->slabs.clear();
    }
    delete a;
    return SH_OK;
}

int32_t sh_vmm_create_slab(uint64_t allocator, uint64_t total_bytes, int32_t* slab_out) {
    Allocator* a = as_alloc(allocator);
    if (a == nullptr || slab_out == nullptr || total_bytes == 0) return vfail(SH_ERR_INVALID_ARG, "bad create_slab arguments");
    std::lock_guard<std::mutex> lk(a->mu);
    Slab s;
    s.size = round_up(static_cast<size_t>(total_bytes), a->granularity);
    const CUresult e = driver().AddressReserve(&s.base, s.size, a->granularity, 0, 0);
    if (e != CUDA_SUCCESS) return vfail(SH_ERR_CUDA, "cuMemAddressReserve(%zu) failed (%d)", s.size, static_cast<int>(e));
    const int id = a->next_slab++;
    a->slabs.emplace(id, std::move(s));
    *slab_out = id;
    return SH_OK;
}

int32_t sh_vmm_define_region(uint64_t allocator, int32_t slab, uint64_t offset, uint64_t size, int32_t* region_out) {
    Allocator* a = as_alloc(allocator);
    if (a == nullptr || region_out == nullptr || size == 0) return vfail(SH_ERR_INVALID_ARG, "bad define_region arguments");
    std::lock_guard<std::mutex> lk(a->mu);
    Slab* s = nullptr;
    const int rc = find(*a, slab, -1, &s, nullptr);
    if (rc != SH_OK) return rc;
    Region r;
    r.offset = static_cast<size_t>(offset) / a->granularity * a->granularity;
    r.size = round_up(static_cast<size_t>(offset + size) - r.offset, a->granularity);
    if (r.offset + r.size > s->size) return vfail(SH_ERR_INVALID_ARG, "region [%llu, +%llu) does not fit slab %d (%zu bytes)",
                                                   static_cast<unsigned long long>(offset),
                                                   static_cast<unsigned long long>(size), slab, s->size);
    for (const Region& other : s->regions)
        if (r.offset < other.offset + other.size && other.offset < r.offset + r.size)
            return vfail(SH_ERR_INVALID_ARG, "region overlaps another region of slab %d after rounding to %zu bytes", slab,
                         a->granularity);
    s->regions.push_back(r);
    *region_out = static_cast<int32_t>(s->regions.size() - 1);
    return SH_OK;
}

static void prefetch_loop(Allocator* a) {
    (void)cudaSetDevice(a->device);
    (void)cudaFree(nullptr);                       // the primary context becomes current on this thread
    std::unique_lock<std::mutex> lk(a->mu);
    for (;;) {
        a->wake.wait(lk, [a] { return a->stopping || !a->requests.empty(); });
        if (a->stopping) break;
        const std::pair<int, int> req = a->requests.front();
        a->requests.pop_front();
        a->worker_busy = true;
        Slab* s = nullptr;
        Region* r = nullptr;
        // best effort: a request for something destroyed meanwhile, or one that finds no room, is dropped
        if (find(*a, req.first, req.second, &s, &r) == SH_OK && !r->mapped) {
            if (map_region(*a, req.first, *s, req.second, *r) != SH_OK) a->prefetch_failures += 1;
            else r->last_access = ++a->clock;
        }
        a->worker_busy = false;
        if (a->requests.empty()) a->idle.notify_all();
    }
}

int32_t sh_vmm_prefetch_async(uint64_t allocator, int32_t slab, int32_t region) {
    Allocator* a = as_alloc(allocator);
    if (a == nullptr) return vfail(SH_ERR_INVALID_ARG, "null allocator");
    std::lock_guard<std::mutex> lk(a->mu);
    Slab* s = nullptr;
    Region* r = nullptr;
    const int rc = find(*a, slab, region, &s, &r);
    if (rc != SH_OK) return rc;
    if (r->mapped) return SH_OK;
    if (!a->worker_started) {
        a->worker = std::thread(prefetch_loop, a);
        a->worker_started = true;
    }
    a->requests.emplace_back(slab, region);
    a->wake.notify_one();
    return SH_OK;
}

int32_t sh_vmm_prefetch_wait(uint64_t allocator, int32_t timeout_ms) {
    Allocator* a = as_alloc(allocator);
    if (a == nullptr) return vfail(SH_ERR_INVALID_ARG, "null allocator");
    std::unique_lock<std::mutex> lk(a->mu);
    const bool done = a->idle.wait_for(lk, std::chrono::milliseconds(timeout_ms < 0 ? 0 : timeout_ms),
                                       [a] { return a->requests.empty() && !a->worker_busy; });
    return done ? SH_OK : vfail(SH_ERR_TIMEOUT, "prefetch requests still pending after %d ms", timeout_ms);
}

int32_t sh_vmm_ensure_resident(uint64_t allocator, int32_t slab, int32_t region, int32_t hold, void** dev_ptr_out) {
    Allocator* a = as_alloc(allocator);
    if (a == nullptr) return vfail(SH_ERR_INVALID_ARG, "null allocator");
    std::lock_guard<std::mutex> lk(a->mu);
    Slab* s = nullptr;
    Region* r = nullptr;
    int rc = find(*a, slab, region, &s, &r);
    if (rc != SH_OK) return rc;
    if (!r->mapped) {
        rc = map_region(*a, slab, *s, region, *r);
        if (rc != SH_OK) return rc;
    }
    r->last_access = ++a->clock;
    if (hold) r->refcount += 1;
    if (dev_ptr_out != nullptr) *dev_ptr_out = reinterpret_cast<void*>(s->base + r->offset);
    return SH_OK;
}

int32_t sh_vmm_release(uint64_t allocator, int32_t slab, int32_t region, uint64_t stream) {
    Allocator* a = as_alloc(allocator);
    if (a == nullptr) return vfail(SH_ERR_INVALID_ARG, "null allocator");
    std::lock_guard<std::mutex> lk(a->mu);
    Slab* s = nullptr;
    Region* r = nullptr;
    const int rc = find(*a, slab, region, &s, &r);
    if (rc != SH_OK) return rc;
    if (r->refcount <= 0) return vfail(SH_ERR_INVALID_ARG, "region %d of slab %d is not held", region, slab);
    r->refcount -= 1;
    if (r->released == nullptr && cudaEventCreateWithFlags(&r->released, cudaEventDisableTiming) != cudaSuccess) {
        (void)cudaGetLastError();
        return vfail(SH_ERR_CUDA, "cudaEventCreate failed");
    }
    if (cudaEventRecord(r->released, reinterpret_cast<cudaStream_t>(static_cast<uintptr_t>(stream))) != cudaSuccess) {
        (void)cudaGetLastError();
        return vfail(SH_ERR_CUDA, "cudaEventRecord failed");
    }
    r->event_pending = true;
    return SH_OK;
}

int32_t sh_vmm_set_priority(uint64_t allocator, int32_t slab, uint32_t priority) {
    Allocator* a = as_alloc(allocator);
    if (a == nullptr) return vfail(SH_ERR_INVALID_ARG, "null allocator");
    std::lock_guard<std::mutex> lk(a->mu);
    Slab* s = nullptr;
    const int rc = find(*a, slab, -1, &s, nullptr);
    if (rc != SH_OK) return rc;
    s->priority = priority;
    return SH_OK;
}

int32_t sh_vmm_set_ceiling(uint64_t allocator, uint64_t ceiling_bytes) {
    Allocator* a = as_alloc(allocator);
    if (a == nullptr || ceiling_bytes == 0) return vfail(SH_ERR_INVALID_ARG, "bad ceiling");
    std::lock_guard<std::mutex> lk(a->mu);
    a->ceiling = static_cast<size_t>(ceiling_bytes);
    return make_room(*a, 0, -1, -1);
}

int32_t sh_vmm_destroy_slab(uint64_t allocator, int32_t slab) {
    Allocator* a = as_alloc(allocator);
    if (a == nullptr) return vfail(SH_ERR_INVALID_ARG, "null allocator");
    std::lock_guard<std::mutex> lk(a->mu);
    Slab* s = nullptr;
    int rc = find(*a, slab, -1, &s, nullptr);
    if (rc != SH_OK) return rc;
    for (const Region& r : s->regions)
        if (r.refcount > 0) return vfail(SH_ERR_BUSY, "slab %d still has held regions", slab);
    for (Region& r : s->regions) {
        if (!event_done(r, 10000)) return vfail(SH_ERR_TIMEOUT, "a region of slab %d is still in use on the GPU", slab);
        rc = unmap_region(*a, *s, r);
        if (rc != SH_OK) return rc;
        if (r.released != nullptr) cudaEventDestroy(r.released);
    }
    driver().AddressFree(s->base, s->size);
    a->slabs.erase(slab);
    return SH_OK;
}

int32_t sh_vmm_stats(uint64_t allocator, ShVmmStats* out) {
    Allocator* a = as_alloc(allocator);
    if (a == nullptr || out == nullptr) return vfail(SH_ERR_INVALID_ARG, "bad stats arguments");
    std::lock_guard<std::mutex> lk(a->mu);
    out->total_slabs = static_cast<int64_t>(a->slabs.size());
    out->total_regions = 0;
    out->mapped_regions = 0;
    for (auto& [sid, s] : a->slabs) {
        out->total_regions += static_cast<int64_t>(s.regions.size());
        for (auto& r : s.regions) out->mapped_regions += r.mapped ? 1 : 0;
    }
    out->mapped_bytes = static_cast<int64_t>(a->mapped);
    out->vram_ceiling = static_cast<int64_t>(a->ceiling);
    out->granularity = static_cast<int64_t>(a->granularity);
    out->evictions = a->evictions;
    return SH_OK;
}

}  // extern "C"
