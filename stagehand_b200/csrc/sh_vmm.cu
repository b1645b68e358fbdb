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
    // One event per release whose work may still be running: every holder records its own, on its own
    // stream, so a second release never hides what the first stream still has queued.  Completed events
    // stay in the list and are recorded again by later releases.
    struct Release {
        cudaEvent_t event = nullptr;
        bool pending = false;
    };
    std::vector<Release> releases;
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

// Non-blocking: true when every release event of the region has completed (or none is pending).
// A query that fails for any other reason than "not ready" counts as not idle.
bool region_idle(Region& r) {
    for (auto& rel : r.releases) {
        if (!rel.pending) continue;
        const cudaError_t q = cudaEventQuery(rel.event);
        if (q == cudaSuccess) {
            rel.pending = false;
            continue;
        }
        if (q != cudaErrorNotReady) (void)cudaGetLastError();
        return false;
    }
    return true;
}

void destroy_release_events(Region& r) {
    for (auto& rel : r.releases)
        if (rel.event != nullptr) cudaEventDestroy(rel.event);
    r.releases.clear();
}

constexpr int kReleaseWaitMs = 10000;

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

// Unmap unreferenced regions until `need` more bytes fit.  A region is a victim only when nobody holds
// it AND the work queued before its releases has finished; among those, lowest slab priority first, then
// least recently used.  Released regions whose work is still running are never waited for while an idle
// one exists.  When every candidate is still busy, the allocator's mutex is dropped while this thread
// polls (other callers keep going), for at most kReleaseWaitMs in total; only then SH_ERR_TIMEOUT.
// `lk` must hold a.mu on entry and holds it on return.  Pointers into a.slabs taken by the caller before
// the call may be stale afterwards when `*waited` comes back true.
int make_room(Allocator& a, std::unique_lock<std::mutex>& lk, size_t need, int skip_slab, int skip_region, bool* waited) {
    const auto deadline = std::chrono::steady_clock::now() + std::chrono::milliseconds(kReleaseWaitMs);
    while (a.mapped + need > a.ceiling) {
        Slab* vs = nullptr;
        Region* vr = nullptr;
        bool busy_candidates = false;
        for (auto& [sid, s] : a.slabs) {
            for (size_t i = 0; i < s.regions.size(); ++i) {
                Region& r = s.regions[i];
                if (!r.mapped || r.refcount > 0 || (sid == skip_slab && static_cast<int>(i) == skip_region)) continue;
                if (!region_idle(r)) {
                    busy_candidates = true;
                    continue;
                }
                if (vr == nullptr || s.priority < vs->priority ||
                    (s.priority == vs->priority && r.last_access < vr->last_access)) {
                    vs = &s;
                    vr = &r;
                }
            }
        }
        if (vr != nullptr) {
            const int rc = unmap_region(a, *vs, *vr);
            if (rc != SH_OK) return rc;
            a.evictions += 1;
            continue;
        }
        if (!busy_candidates)
            return vfail(SH_ERR_OOM, "VRAM ceiling of %zu bytes reached and no region is evictable (mapped %zu, need %zu)",
                         a.ceiling, a.mapped, need);
        if (std::chrono::steady_clock::now() >= deadline)
            return vfail(SH_ERR_TIMEOUT, "every released region is still in use on the GPU after %d ms", kReleaseWaitMs);
        if (waited != nullptr) *waited = true;
        lk.unlock();
        std::this_thread::sleep_for(std::chrono::microseconds(100));
        lk.lock();
    }
    return SH_OK;
}

int find(Allocator& a, int slab, int region, Slab** s_out, Region** r_out);

// Maps (slab_id, region_id).  `lk` holds a.mu; it may be dropped and retaken while room is made, so the
// region is looked up again afterwards (it may have been destroyed, or mapped by another thread).
int map_region(Allocator& a, std::unique_lock<std::mutex>& lk, int slab_id, int region_id) {
    Driver& d = driver();
    Slab* sp = nullptr;
    Region* rp = nullptr;
    int rc = find(a, slab_id, region_id, &sp, &rp);
    if (rc != SH_OK) return rc;
    if (rp->size > a.ceiling)
        return vfail(SH_ERR_OOM, "region of %zu bytes exceeds the VRAM ceiling of %zu", rp->size, a.ceiling);
    bool waited = false;
    rc = make_room(a, lk, rp->size, slab_id, region_id, &waited);
    if (rc != SH_OK) return rc;
    if (waited) {
        rc = find(a, slab_id, region_id, &sp, &rp);
        if (rc != SH_OK) return rc;
        if (rp->mapped) return SH_OK;
    }
    Slab& s = *sp;
    Region& r = *rp;
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
                const auto deadline = std::chrono::steady_clock::now() + std::chrono::milliseconds(kReleaseWaitMs);
                while (!region_idle(r) && std::chrono::steady_clock::now() < deadline)
                    std::this_thread::sleep_for(std::chrono::microseconds(100));
                (void)unmap_region(*a, s, r);
                destroy_release_events(r);
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
            if (map_region(*a, lk, req.first, req.second) != SH_OK) a->prefetch_failures += 1;
            else if (find(*a, req.first, req.second, &s, &r) == SH_OK) r->last_access = ++a->clock;
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
    std::unique_lock<std::mutex> lk(a->mu);
    Slab* s = nullptr;
    Region* r = nullptr;
    int rc = find(*a, slab, region, &s, &r);
    if (rc != SH_OK) return rc;
    if (!r->mapped) {
        rc = map_region(*a, lk, slab, region);
        if (rc != SH_OK) return rc;
        rc = find(*a, slab, region, &s, &r);       // the lock may have been dropped while room was made
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
    (void)region_idle(*r);                          // retire completed events so one of them can be reused
    Region::Release* slot = nullptr;
    for (auto& rel : r->releases)
        if (!rel.pending) { slot = &rel; break; }
    if (slot == nullptr) {
        Region::Release fresh;
        if (cudaEventCreateWithFlags(&fresh.event, cudaEventDisableTiming) != cudaSuccess) {
            (void)cudaGetLastError();
            return vfail(SH_ERR_CUDA, "cudaEventCreate failed");
        }
        r->releases.push_back(fresh);
        slot = &r->releases.back();
    }
    if (cudaEventRecord(slot->event, reinterpret_cast<cudaStream_t>(static_cast<uintptr_t>(stream))) != cudaSuccess) {
        (void)cudaGetLastError();
        return vfail(SH_ERR_CUDA, "cudaEventRecord failed");
    }
    slot->pending = true;
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
    std::unique_lock<std::mutex> lk(a->mu);
    a->ceiling = static_cast<size_t>(ceiling_bytes);
    return make_room(*a, lk, 0, -1, -1, nullptr);
}

int32_t sh_vmm_destroy_slab(uint64_t allocator, int32_t slab) {
    Allocator* a = as_alloc(allocator);
    if (a == nullptr) return vfail(SH_ERR_INVALID_ARG, "null allocator");
    std::unique_lock<std::mutex> lk(a->mu);
    const auto deadline = std::chrono::steady_clock::now() + std::chrono::milliseconds(kReleaseWaitMs);
    Slab* s = nullptr;
    // First make sure nothing holds or still uses any region; nothing is torn down before that, so a
    // BUSY or TIMEOUT answer leaves the slab exactly as it was.  The mutex is dropped between polls.
    for (;;) {
        const int rc = find(*a, slab, -1, &s, nullptr);
        if (rc != SH_OK) return rc;
        bool idle = true;
        for (Region& r : s->regions) {
            if (r.refcount > 0) return vfail(SH_ERR_BUSY, "slab %d still has held regions", slab);
            idle = region_idle(r) && idle;
        }
        if (idle) break;
        if (std::chrono::steady_clock::now() >= deadline)
            return vfail(SH_ERR_TIMEOUT, "a region of slab %d is still in use on the GPU", slab);
        lk.unlock();
        std::this_thread::sleep_for(std::chrono::microseconds(100));
        lk.lock();
    }
    int first_error = SH_OK;
    for (Region& r : s->regions) {
        const int rc = unmap_region(*a, *s, r);
        if (rc != SH_OK && first_error == SH_OK) first_error = rc;
        destroy_release_events(r);
    }
    if (first_error != SH_OK) return first_error;     // regions that did unmap stay unmapped; events are gone and forgotten
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
