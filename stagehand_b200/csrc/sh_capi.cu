// C ABI of the SquareQ streaming path (declarations and reference citations:
// include/stagehand_b200.h).  Thin, non-blocking wrappers over the CUDA runtime
// plus the launcher of the block kernel.  No torch types, no interpreter calls.
#include "sh_common.h"

#include <algorithm>
#include <atomic>
#include <chrono>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <map>
#include <mutex>
#include <thread>
#include <vector>

namespace shc {

thread_local char g_err[512] = "";

int fail(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
    return code;
}

int cuda_fail(cudaError_t e, const char* what) {
    const int code = (e == cudaErrorMemoryAllocation) ? SH_ERR_OOM : SH_ERR_CUDA;
    return fail(code, "%s: %s (%d)", what, cudaGetErrorString(e), static_cast<int>(e));
}

Counters g_ctr;

// per-launch timing records
struct ProfRecord {
    cudaEvent_t start, stop;
    int64_t elements, bytes;
    int kind;                       // 0 = block-kernel launch(es) of one block, 1 = the copies of one block load
};
std::mutex g_prof_mu;
std::vector<ProfRecord> g_prof_pending;
std::vector<cudaEvent_t> g_prof_free;
std::atomic<int> g_prof_on{0};

// call with g_prof_mu held
cudaEvent_t prof_event() {
    if (!g_prof_free.empty()) {
        cudaEvent_t e = g_prof_free.back();
        g_prof_free.pop_back();
        return e;
    }
    cudaEvent_t e = nullptr;
    if (cudaEventCreate(&e) != cudaSuccess) return nullptr;
    return e;
}

int wait_event_bounded(cudaEvent_t ev, int timeout_ms) {
    const auto deadline = std::chrono::steady_clock::now() + std::chrono::milliseconds(timeout_ms < 0 ? 0 : timeout_ms);
    int spins = 0;
    for (;;) {
        const cudaError_t q = cudaEventQuery(ev);
        if (q == cudaSuccess) return SH_OK;
        if (q != cudaErrorNotReady) return cuda_fail(q, "cudaEventQuery");
        if (std::chrono::steady_clock::now() >= deadline) return fail(SH_ERR_TIMEOUT, "event not complete after %d ms", timeout_ms);
        if (++spins > 200) std::this_thread::sleep_for(std::chrono::microseconds(50));
    }
}

int launch_plans(const sq::BlockPlan* plans, int n_plans, int64_t elements, int64_t traffic, int out_dtype,
                 cudaStream_t stream, int32_t* status_dev) {
    ProfRecord rec{nullptr, nullptr, elements, traffic, 0};
    const bool prof = g_prof_on.load(std::memory_order_relaxed) != 0;
    if (prof) {
        std::lock_guard<std::mutex> lk(g_prof_mu);
        rec.start = prof_event();
        rec.stop = prof_event();
        if (rec.start == nullptr || rec.stop == nullptr) {       // only one could be had: give it back, time nothing
            if (rec.start != nullptr) g_prof_free.push_back(rec.start);
            if (rec.stop != nullptr) g_prof_free.push_back(rec.stop);
            rec.start = rec.stop = nullptr;
        }
    }
    if (rec.start) cudaEventRecord(rec.start, stream);
    for (int p = 0; p < n_plans; ++p) {
        const cudaError_t e = sq::launch_plan(plans[p], out_dtype, stream, status_dev);
        if (e != cudaSuccess) {
            if (rec.start) {
                std::lock_guard<std::mutex> lk(g_prof_mu);
                g_prof_free.push_back(rec.start);
                g_prof_free.push_back(rec.stop);
            }
            return cuda_fail(e, "block kernel launch");
        }
        g_ctr.launches.fetch_add(1, std::memory_order_relaxed);
    }
    if (rec.stop) {
        cudaEventRecord(rec.stop, stream);
        std::lock_guard<std::mutex> lk(g_prof_mu);
        g_prof_pending.push_back(rec);
    }
    g_ctr.elements.fetch_add(elements, std::memory_order_relaxed);
    return SH_OK;
}

bool copy_timing_begin(cudaStream_t stream, cudaEvent_t* start_out, cudaEvent_t* stop_out) {
    if (g_prof_on.load(std::memory_order_relaxed) == 0) return false;
    {
        std::lock_guard<std::mutex> lk(g_prof_mu);
        *start_out = prof_event();
        *stop_out = prof_event();
        if (*start_out == nullptr || *stop_out == nullptr) {
            if (*start_out != nullptr) g_prof_free.push_back(*start_out);
            if (*stop_out != nullptr) g_prof_free.push_back(*stop_out);
            return false;
        }
    }
    cudaEventRecord(*start_out, stream);
    return true;
}

void copy_timing_end(cudaStream_t stream, cudaEvent_t start, cudaEvent_t stop, int64_t bytes) {
    cudaEventRecord(stop, stream);
    std::lock_guard<std::mutex> lk(g_prof_mu);
    g_prof_pending.push_back(ProfRecord{start, stop, 0, bytes, 1});
}

void copy_timing_abandon(cudaEvent_t start, cudaEvent_t stop) {
    std::lock_guard<std::mutex> lk(g_prof_mu);
    g_prof_free.push_back(start);
    g_prof_free.push_back(stop);
}

}  // namespace shc

namespace {

using namespace shc;

int launch_block(const ShParamDesc* descs, int32_t n, const void* packed, size_t packed_bytes, void* out,
                 size_t out_bytes, int32_t out_dtype, cudaStream_t stream, int32_t* status_dev) {
    if (n < 0 || (n > 0 && descs == nullptr)) return fail(SH_ERR_INVALID_ARG, "null descriptor array");
    if (n == 0) return SH_OK;
    if (out == nullptr) return fail(SH_ERR_INVALID_ARG, "null output slab");
    const int max_plans = (n + sq::kMaxDescs - 1) / sq::kMaxDescs;
    std::vector<sq::BlockPlan> plans(static_cast<size_t>(max_plans));
    int n_plans = 0;
    int64_t elements = 0, traffic = 0;
    char err[256];
    const int rc = sq::build_plans(descs, n, packed, packed_bytes, out, out_bytes, out_dtype, plans.data(), &n_plans,
                                   &elements, &traffic, err, sizeof(err));
    if (rc != SH_OK) return fail(rc, "%s", err);
    return launch_plans(plans.data(), n_plans, elements, traffic, out_dtype, stream, status_dev);
}

// Read-back state of one device status word (sh_status_poll).
struct StatusWatch {
    int32_t* host = nullptr;        // page-locked landing word
    cudaEvent_t landed = nullptr;
    bool pending = false;
    int32_t sticky = 0;             // every bit ever seen
};
std::mutex g_status_mu;
std::map<int32_t*, StatusWatch> g_status;

}  // namespace

using namespace shc;

extern "C" {

int32_t sh_abi_version(void) { return SH_ABI_VERSION; }

int32_t sh_last_error(char* buf, int32_t buf_len) {
    const int32_t n = static_cast<int32_t>(strlen(g_err));
    if (buf != nullptr && buf_len > 0) {
        const int32_t c = std::min(n, buf_len - 1);
        memcpy(buf, g_err, static_cast<size_t>(c));
        buf[c] = '\0';
    }
    return n;
}

int32_t sh_init(int32_t device) {
    int count = 0;
    SH_CUDA(cudaGetDeviceCount(&count), "cudaGetDeviceCount");
    if (device < 0 || device >= count) return fail(SH_ERR_INVALID_ARG, "device %d out of range (0..%d)", device, count - 1);
    SH_CUDA(cudaSetDevice(device), "cudaSetDevice");
    cudaDeviceProp prop;
    SH_CUDA(cudaGetDeviceProperties(&prop, device), "cudaGetDeviceProperties");
    if (prop.major != 10)
        return fail(SH_ERR_UNSUPPORTED, "device %d is sm_%d%d; this library carries sm_100a code only", device, prop.major,
                    prop.minor);
    // Load the library's device image on this GPU now -- with it the fixed staging array of
    // sh_dequant_from_host_noalloc -- so that its memory is paid for here, not at that entry point's first call.
    // Best effort: if the array cannot be had (no memory left), only that entry point is affected and it
    // reports the failure itself when called.
    char why[200];
    (void)noalloc_prepare_current_device(why, sizeof(why));
    (void)cudaGetLastError();
    return SH_OK;
}

int32_t sh_shutdown(void) {
    std::lock_guard<std::mutex> lk(g_prof_mu);
    for (auto& r : g_prof_pending) {
        cudaEventDestroy(r.start);
        cudaEventDestroy(r.stop);
    }
    g_prof_pending.clear();
    for (auto e : g_prof_free) cudaEventDestroy(e);
    g_prof_free.clear();
    std::lock_guard<std::mutex> lk2(g_status_mu);
    for (auto& [dev, w] : g_status) {
        if (w.landed != nullptr) cudaEventDestroy(w.landed);
        if (w.host != nullptr) cudaFreeHost(w.host);
    }
    g_status.clear();
    return SH_OK;
}

int32_t sh_device_info(int32_t device, ShDeviceInfo* out) {
    if (out == nullptr) return fail(SH_ERR_INVALID_ARG, "null out");
    cudaDeviceProp prop;
    SH_CUDA(cudaGetDeviceProperties(&prop, device), "cudaGetDeviceProperties");
    out->device = device;
    out->cc_major = prop.major;
    out->cc_minor = prop.minor;
    out->sm_count = prop.multiProcessorCount;
    out->total_mem_bytes = static_cast<int64_t>(prop.totalGlobalMem);
    out->l2_bytes = static_cast<int64_t>(prop.l2CacheSize);
    return SH_OK;
}

int32_t sh_stats(ShStats* out) {
    if (out == nullptr) return fail(SH_ERR_INVALID_ARG, "null out");
    out->kernel_launches = g_ctr.launches.load();
    out->elements_dequantised = g_ctr.elements.load();
    out->h2d_copies = g_ctr.h2d_copies.load();
    out->h2d_bytes = g_ctr.h2d_bytes.load();
    out->peer_copies = g_ctr.peer_copies.load();
    out->peer_bytes = g_ctr.peer_bytes.load();
    out->kernel_status_errors = g_ctr.status_errors.load();
    return SH_OK;
}

int32_t sh_stats_reset(void) {
    g_ctr.launches = 0; g_ctr.elements = 0; g_ctr.h2d_copies = 0; g_ctr.h2d_bytes = 0;
    g_ctr.peer_copies = 0; g_ctr.peer_bytes = 0; g_ctr.status_errors = 0;
    return SH_OK;
}

// ── streams and events ──────────────────────────────────────────────────

int32_t sh_stream_create(int32_t priority, uint64_t* stream_out) {
    if (stream_out == nullptr) return fail(SH_ERR_INVALID_ARG, "null stream_out");
    int lo = 0, hi = 0;
    SH_CUDA(cudaDeviceGetStreamPriorityRange(&lo, &hi), "cudaDeviceGetStreamPriorityRange");
    const int prio = std::max(hi, std::min(lo, static_cast<int>(priority)));   // hi is the numerically smallest
    cudaStream_t s = nullptr;
    SH_CUDA(cudaStreamCreateWithPriority(&s, cudaStreamNonBlocking, prio), "cudaStreamCreateWithPriority");
    *stream_out = static_cast<uint64_t>(reinterpret_cast<uintptr_t>(s));
    return SH_OK;
}

int32_t sh_stream_destroy(uint64_t stream) {
    SH_CUDA(cudaStreamDestroy(as_stream(stream)), "cudaStreamDestroy");
    return SH_OK;
}

int32_t sh_stream_synchronize(uint64_t stream, int32_t timeout_ms) {
    cudaEvent_t ev = nullptr;
    SH_CUDA(cudaEventCreateWithFlags(&ev, cudaEventDisableTiming), "cudaEventCreate");
    cudaError_t e = cudaEventRecord(ev, as_stream(stream));
    if (e != cudaSuccess) {
        cudaEventDestroy(ev);
        return cuda_fail(e, "cudaEventRecord");
    }
    const int rc = wait_event_bounded(ev, timeout_ms);
    cudaEventDestroy(ev);
    return rc;
}

int32_t sh_stream_wait_event(uint64_t stream, uint64_t event) {
    SH_CUDA(cudaStreamWaitEvent(as_stream(stream), as_event(event), 0), "cudaStreamWaitEvent");
    return SH_OK;
}

int32_t sh_event_create(int32_t enable_timing, uint64_t* event_out) {
    if (event_out == nullptr) return fail(SH_ERR_INVALID_ARG, "null event_out");
    cudaEvent_t ev = nullptr;
    SH_CUDA(cudaEventCreateWithFlags(&ev, enable_timing ? cudaEventDefault : cudaEventDisableTiming), "cudaEventCreate");
    *event_out = static_cast<uint64_t>(reinterpret_cast<uintptr_t>(ev));
    return SH_OK;
}

int32_t sh_event_destroy(uint64_t event) {
    SH_CUDA(cudaEventDestroy(as_event(event)), "cudaEventDestroy");
    return SH_OK;
}

int32_t sh_event_record(uint64_t event, uint64_t stream) {
    SH_CUDA(cudaEventRecord(as_event(event), as_stream(stream)), "cudaEventRecord");
    return SH_OK;
}

int32_t sh_event_query(uint64_t event) {
    const cudaError_t q = cudaEventQuery(as_event(event));
    if (q == cudaSuccess) return SH_OK;
    if (q == cudaErrorNotReady) return SH_ERR_BUSY;
    return cuda_fail(q, "cudaEventQuery");
}

int32_t sh_event_wait(uint64_t event, int32_t timeout_ms) { return wait_event_bounded(as_event(event), timeout_ms); }

int32_t sh_event_elapsed_ms(uint64_t start, uint64_t stop, float* ms_out) {
    if (ms_out == nullptr) return fail(SH_ERR_INVALID_ARG, "null ms_out");
    SH_CUDA(cudaEventElapsedTime(ms_out, as_event(start), as_event(stop)), "cudaEventElapsedTime");
    return SH_OK;
}

// ── memory ──────────────────────────────────────────────────────────────

int32_t sh_host_alloc(size_t bytes, void** ptr_out) {
    if (ptr_out == nullptr || bytes == 0) return fail(SH_ERR_INVALID_ARG, "bad host allocation request");
    SH_CUDA(cudaHostAlloc(ptr_out, bytes, cudaHostAllocPortable), "cudaHostAlloc");
    return SH_OK;
}

int32_t sh_host_free(void* ptr) {
    if (ptr == nullptr) return SH_OK;
    SH_CUDA(cudaFreeHost(ptr), "cudaFreeHost");
    return SH_OK;
}

int32_t sh_host_register(void* ptr, size_t bytes) {
    if (ptr == nullptr || bytes == 0) return fail(SH_ERR_INVALID_ARG, "bad host registration request");
    SH_CUDA(cudaHostRegister(ptr, bytes, cudaHostRegisterPortable), "cudaHostRegister");
    return SH_OK;
}

int32_t sh_host_unregister(void* ptr) {
    SH_CUDA(cudaHostUnregister(ptr), "cudaHostUnregister");
    return SH_OK;
}

int32_t sh_device_alloc(size_t bytes, void** ptr_out) {
    if (ptr_out == nullptr || bytes == 0) return fail(SH_ERR_INVALID_ARG, "bad device allocation request");
    SH_CUDA(cudaMalloc(ptr_out, bytes), "cudaMalloc");
    return SH_OK;
}

int32_t sh_device_free(void* ptr) {
    if (ptr == nullptr) return SH_OK;
    SH_CUDA(cudaFree(ptr), "cudaFree");
    return SH_OK;
}

int32_t sh_pack_rows(void* dst, int64_t dst_ld, const void* src, int64_t src_ld, int64_t rows, int64_t row_bytes,
                     int32_t n_threads) {
    if (dst == nullptr || src == nullptr || rows < 0 || row_bytes < 0 || dst_ld < row_bytes || src_ld < row_bytes)
        return fail(SH_ERR_INVALID_ARG, "bad pack_rows arguments");
    if (rows == 0 || row_bytes == 0) return SH_OK;
    auto work = [=](int64_t r0, int64_t r1) {
        uint8_t* d = static_cast<uint8_t*>(dst);
        const uint8_t* s = static_cast<const uint8_t*>(src);
        if (dst_ld == row_bytes && src_ld == row_bytes) {
            memcpy(d + r0 * row_bytes, s + r0 * row_bytes, static_cast<size_t>((r1 - r0) * row_bytes));
            return;
        }
        for (int64_t r = r0; r < r1; ++r) memcpy(d + r * dst_ld, s + r * src_ld, static_cast<size_t>(row_bytes));
    };
    const int64_t total = rows * row_bytes;
    int threads = std::max(1, static_cast<int>(n_threads));
    threads = static_cast<int>(std::min<int64_t>(threads, std::max<int64_t>(1, total / (4 << 20))));
    threads = static_cast<int>(std::min<int64_t>(threads, rows));
    if (threads <= 1) {
        work(0, rows);
        return SH_OK;
    }
    std::vector<std::thread> pool;
    pool.reserve(static_cast<size_t>(threads));
    const int64_t chunk = (rows + threads - 1) / threads;
    for (int t = 0; t < threads; ++t) {
        const int64_t r0 = t * chunk, r1 = std::min(rows, r0 + chunk);
        if (r0 >= r1) break;
        pool.emplace_back(work, r0, r1);
    }
    for (auto& th : pool) th.join();
    return SH_OK;
}

int32_t sh_sync_bytes(void* dst, const void* src, size_t bytes, int32_t* changed_out) {
    if (bytes != 0 && (dst == nullptr || src == nullptr)) return fail(SH_ERR_INVALID_ARG, "null sync pointer");
    const bool differs = bytes != 0 && memcmp(dst, src, bytes) != 0;
    if (differs) memcpy(dst, src, bytes);
    if (changed_out != nullptr) *changed_out = differs ? 1 : 0;
    return SH_OK;
}

// ── data movement ───────────────────────────────────────────────────────

int32_t sh_copy_h2d_async(void* dst_dev, const void* src_host, size_t bytes, uint64_t stream) {
    if (bytes == 0) return SH_OK;
    if (dst_dev == nullptr || src_host == nullptr) return fail(SH_ERR_INVALID_ARG, "null copy pointer");
    SH_CUDA(cudaMemcpyAsync(dst_dev, src_host, bytes, cudaMemcpyHostToDevice, as_stream(stream)), "cudaMemcpyAsync H2D");
    g_ctr.h2d_copies.fetch_add(1, std::memory_order_relaxed);
    g_ctr.h2d_bytes.fetch_add(static_cast<int64_t>(bytes), std::memory_order_relaxed);
    return SH_OK;
}

int32_t sh_pull_block_async(void* dst_local, const void* src_dev, size_t bytes, uint64_t stream) {
    if (bytes == 0) return SH_OK;
    if (dst_local == nullptr || src_dev == nullptr) return fail(SH_ERR_INVALID_ARG, "null copy pointer");
    SH_CUDA(cudaMemcpyAsync(dst_local, src_dev, bytes, cudaMemcpyDeviceToDevice, as_stream(stream)),
            "cudaMemcpyAsync D2D");
    g_ctr.peer_copies.fetch_add(1, std::memory_order_relaxed);
    g_ctr.peer_bytes.fetch_add(static_cast<int64_t>(bytes), std::memory_order_relaxed);
    return SH_OK;
}

int32_t sh_peer_enable(int32_t peer_device) {
    int cur = 0;
    SH_CUDA(cudaGetDevice(&cur), "cudaGetDevice");
    if (cur == peer_device) return SH_OK;
    int can = 0;
    SH_CUDA(cudaDeviceCanAccessPeer(&can, cur, peer_device), "cudaDeviceCanAccessPeer");
    if (!can) return fail(SH_ERR_UNSUPPORTED, "device %d cannot access device %d", cur, peer_device);
    const cudaError_t e = cudaDeviceEnablePeerAccess(peer_device, 0);
    if (e == cudaErrorPeerAccessAlreadyEnabled) {
        (void)cudaGetLastError();
        return SH_OK;
    }
    if (e != cudaSuccess) return cuda_fail(e, "cudaDeviceEnablePeerAccess");
    return SH_OK;
}

int32_t sh_ipc_export(void* dev_ptr, uint8_t handle_out[64]) {
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
    if (dev_ptr == nullptr || handle_out == nullptr) return fail(SH_ERR_INVALID_ARG, "null ipc argument");
    cudaIpcMemHandle_t h;
    SH_CUDA(cudaIpcGetMemHandle(&h, dev_ptr), "cudaIpcGetMemHandle");
    memcpy(handle_out, &h, 64);
    return SH_OK;
}

int32_t sh_ipc_open(const uint8_t handle[64], void** dev_ptr_out) {
    if (handle == nullptr || dev_ptr_out == nullptr) return fail(SH_ERR_INVALID_ARG, "null ipc argument");
    cudaIpcMemHandle_t h;
    memcpy(&h, handle, 64);
    SH_CUDA(cudaIpcOpenMemHandle(dev_ptr_out, h, cudaIpcMemLazyEnablePeerAccess), "cudaIpcOpenMemHandle");
    return SH_OK;
}

int32_t sh_ipc_close(void* dev_ptr) {
    if (dev_ptr == nullptr) return SH_OK;
    SH_CUDA(cudaIpcCloseMemHandle(dev_ptr), "cudaIpcCloseMemHandle");
    return SH_OK;
}

// ── the block kernel ────────────────────────────────────────────────────

int32_t sh_dequant_block_async(const ShParamDesc* descs, int32_t n_descs, const void* packed_dev, size_t packed_bytes,
                               void* out_dev, size_t out_bytes, int32_t out_dtype, uint64_t stream,
                               int32_t* status_dev) {
    return launch_block(descs, n_descs, packed_dev, packed_bytes, out_dev, out_bytes, out_dtype, as_stream(stream),
                        status_dev);
}

int32_t sh_stream_block_async(const ShParamDesc* descs, int32_t n_descs, const void* packed_host, size_t packed_bytes,
                              void* staging_dev, void* out_dev, size_t out_bytes, int32_t out_dtype,
                              uint64_t copy_stream, uint64_t dequant_stream, uint64_t ev_copied, uint64_t ev_ready,
                              int32_t* status_dev) {
    if (packed_host == nullptr || staging_dev == nullptr) return fail(SH_ERR_INVALID_ARG, "null image pointer");
    if (copy_stream != dequant_stream && ev_copied == 0)
        return fail(SH_ERR_INVALID_ARG, "two streams need ev_copied to order the kernel after the copy");
    // validate before anything is enqueued so a bad descriptor leaves both streams untouched; the plans
    // built for the check are the ones launched
    if (n_descs < 0 || (n_descs > 0 && descs == nullptr)) return fail(SH_ERR_INVALID_ARG, "null descriptor array");
    if (n_descs > 0 && out_dev == nullptr) return fail(SH_ERR_INVALID_ARG, "null output slab");
    const int max_plans = (std::max(n_descs, 1) + sq::kMaxDescs - 1) / sq::kMaxDescs;
    std::vector<sq::BlockPlan> plans(static_cast<size_t>(max_plans));
    int n_plans = 0;
    int64_t elements = 0, traffic = 0;
    char err[256];
    int rc = sq::build_plans(descs, n_descs, staging_dev, packed_bytes, out_dev, out_bytes, out_dtype, plans.data(),
                             &n_plans, &elements, &traffic, err, sizeof(err));
    if (rc != SH_OK) return fail(rc, "%s", err);
    rc = sh_copy_h2d_async(staging_dev, packed_host, packed_bytes, copy_stream);
    if (rc != SH_OK) return rc;
    if (ev_copied != 0) {
        SH_CUDA(cudaEventRecord(as_event(ev_copied), as_stream(copy_stream)), "cudaEventRecord");
        if (copy_stream != dequant_stream)
            SH_CUDA(cudaStreamWaitEvent(as_stream(dequant_stream), as_event(ev_copied), 0), "cudaStreamWaitEvent");
    }
    rc = launch_plans(plans.data(), n_plans, elements, traffic, out_dtype, as_stream(dequant_stream), status_dev);
    if (rc != SH_OK) return rc;
    if (ev_ready != 0) SH_CUDA(cudaEventRecord(as_event(ev_ready), as_stream(dequant_stream)), "cudaEventRecord");
    return SH_OK;
}

int32_t sh_status_poll(int32_t* status_dev, uint64_t stream, int32_t* bits_out) {
    if (status_dev == nullptr) return fail(SH_ERR_INVALID_ARG, "null status word");
    std::lock_guard<std::mutex> lk(g_status_mu);
    StatusWatch& w = g_status[status_dev];
    if (w.host == nullptr) {
        SH_CUDA(cudaHostAlloc(reinterpret_cast<void**>(&w.host), sizeof(int32_t), cudaHostAllocPortable), "cudaHostAlloc");
        *w.host = 0;
        SH_CUDA(cudaEventCreateWithFlags(&w.landed, cudaEventDisableTiming), "cudaEventCreate");
    }
    if (w.pending) {
        const cudaError_t q = cudaEventQuery(w.landed);
        if (q == cudaErrorNotReady) {                       // the previous read-back has not landed: nothing new to say
            if (bits_out != nullptr) *bits_out = w.sticky;
            return SH_OK;
        }
        if (q != cudaSuccess) return cuda_fail(q, "cudaEventQuery");
        w.pending = false;
        if (*w.host != 0) {
            w.sticky |= *w.host;
            g_ctr.status_errors.fetch_add(1, std::memory_order_relaxed);
        }
    }
    // next read-back, ordered on `stream` behind the launches queued so far; the word is cleared behind it,
    // so bits set by later launches on that stream are seen by the next poll and none is lost
    SH_CUDA(cudaMemcpyAsync(w.host, status_dev, sizeof(int32_t), cudaMemcpyDeviceToHost, as_stream(stream)),
            "cudaMemcpyAsync D2H");
    SH_CUDA(cudaMemsetAsync(status_dev, 0, sizeof(int32_t), as_stream(stream)), "cudaMemsetAsync");
    SH_CUDA(cudaEventRecord(w.landed, as_stream(stream)), "cudaEventRecord");
    w.pending = true;
    if (bits_out != nullptr) *bits_out = w.sticky;
    return SH_OK;
}

int32_t sh_status_forget(int32_t* status_dev) {
    std::lock_guard<std::mutex> lk(g_status_mu);
    auto it = g_status.find(status_dev);
    if (it == g_status.end()) return SH_OK;
    if (it->second.pending) (void)wait_event_bounded(it->second.landed, 10000);
    if (it->second.landed != nullptr) cudaEventDestroy(it->second.landed);
    if (it->second.host != nullptr) cudaFreeHost(it->second.host);
    g_status.erase(it);
    return SH_OK;
}

int32_t sh_set_peer_ctas_per_sm(int32_t ctas_per_sm) {
    sq::set_peer_ctas_per_sm(ctas_per_sm);
    return SH_OK;
}

int32_t sh_set_peer_deep_loads(int32_t on) {
    sq::set_peer_deep_loads(on != 0);
    return SH_OK;
}

int32_t sh_set_peer_bulk_loads(int32_t on) {
    sq::set_peer_bulk_loads(on != 0);
    return SH_OK;
}

int32_t sh_profile_enable(int32_t on) {
    g_prof_on.store(on ? 1 : 0);
    return SH_OK;
}

int32_t sh_profile_collect(double* kernel_ms_out, int64_t* launches_out, int64_t* elements_out, int64_t* bytes_out,
                           int32_t timeout_ms) {
    std::vector<ProfRecord> recs;
    {
        std::lock_guard<std::mutex> lk(g_prof_mu);
        recs.swap(g_prof_pending);
    }
    double ms = 0.0;
    int64_t elements = 0, bytes = 0, n = 0;
    int rc = SH_OK;
    for (auto& r : recs) {
        if (rc == SH_OK) rc = wait_event_bounded(r.stop, timeout_ms);
        if (rc == SH_OK && r.kind == 0) {
            float t = 0.f;
            if (cudaEventElapsedTime(&t, r.start, r.stop) == cudaSuccess) {
                ms += t;
                elements += r.elements;
                bytes += r.bytes;
                ++n;
            }
        }
    }
    {
        std::lock_guard<std::mutex> lk(g_prof_mu);
        for (auto& r : recs) {
            g_prof_free.push_back(r.start);
            g_prof_free.push_back(r.stop);
        }
    }
    if (kernel_ms_out) *kernel_ms_out = ms;
    if (launches_out) *launches_out = n;
    if (elements_out) *elements_out = elements;
    if (bytes_out) *bytes_out = bytes;
    return rc;
}

int32_t sh_profile_poll(ShProfileSums* out) {
    if (out == nullptr) return fail(SH_ERR_INVALID_ARG, "null out");
    memset(out, 0, sizeof(*out));
    std::lock_guard<std::mutex> lk(g_prof_mu);
    size_t kept = 0;
    for (size_t i = 0; i < g_prof_pending.size(); ++i) {
        ProfRecord& r = g_prof_pending[i];
        const cudaError_t q = cudaEventQuery(r.stop);
        if (q == cudaErrorNotReady) {                  // still running: stays for a later poll
            g_prof_pending[kept++] = r;
            continue;
        }
        float t = 0.f;
        if (q == cudaSuccess && cudaEventElapsedTime(&t, r.start, r.stop) == cudaSuccess) {
            if (r.kind == 0) {
                out->kernel_ms += t;
                out->kernel_blocks += 1;
                out->elements += r.elements;
                out->kernel_bytes += r.bytes;
            } else {
                out->copy_ms += t;
                out->copies += 1;
                out->copy_bytes += r.bytes;
            }
        } else {
            (void)cudaGetLastError();
        }
        g_prof_free.push_back(r.start);
        g_prof_free.push_back(r.stop);
    }
    g_prof_pending.resize(kept);
    out->pending = static_cast<int64_t>(kept);
    return SH_OK;
}

}  // extern "C"
