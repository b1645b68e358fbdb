// Slot-rotation transfer engine: every block lives in page-locked host memory, a small window of GPU
// slots (whose memory the caller owns) holds the blocks around the one that is computing.
//
// B200-side equivalent of the reference's stagehand-turbo crate (turbo_src/engine.rs): same verbs,
// same step() policy -- make the current block resident, write the previous one back asynchronously,
// start copying the next one (engine.rs:304-341).  Differences: one page-locked allocation per block
// instead of one per parameter, one event per block instead of one shared prefetch event, and every
// wait carries a deadline instead of cudaEventSynchronize / cudaStreamSynchronize without bound.
#include "../../include/stagehand_b200.h"

#include <cuda_runtime.h>

#include <algorithm>
#include <chrono>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <thread>
#include <vector>

namespace {

thread_local char g_turbo_err[256] = "";

int tfail(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_turbo_err, sizeof(g_turbo_err), fmt, ap);
    va_end(ap);
    return code;
}

enum Location : int { kCpu = 0, kGpu = 1, kH2D = 2, kD2H = 3 };

struct Block {
    std::vector<size_t> sizes, offsets;     // per parameter, offsets into `host`
    size_t total = 0;
    uint8_t* host = nullptr;                // one page-locked allocation
    Location location = kCpu;
    int slot = -1;
    cudaEvent_t moved = nullptr;            // last H2D or D2H of this block
    // INT8 block: `host` holds the packed image (packed_bytes); on the GPU it occupies parameter position 0
    // of its slot (out_bytes, the expanded slab) and is never written back -- the image is the source.
    bool int8 = false;
    std::vector<ShParamDesc> descs;
    size_t packed_bytes = 0, out_bytes = 0;
    int out_dtype = 0;
};

struct Slot {
    std::vector<void*> ptrs;                // GPU pointers supplied by the caller (set_slot_gpu_ptrs)
    std::vector<size_t> sizes;              // capacity per parameter position
    int block = -1;
};

struct Engine {
    std::vector<Block> blocks;
    std::vector<Slot> slots;
    std::vector<int> free_slots;
    cudaStream_t prefetch = nullptr, evict = nullptr;
    cudaEvent_t fence = nullptr;            // orders the evict stream after the caller's work
    std::vector<void*> staging;             // per slot: where a packed INT8 image lands before it is expanded
    size_t staging_bytes = 0;
    int device = 0;
    bool initialized = false;
};

Engine* as_engine(uint64_t h) { return reinterpret_cast<Engine*>(static_cast<uintptr_t>(h)); }

int cuda_check(cudaError_t e, const char* what) {
    if (e == cudaSuccess) return SH_OK;
    (void)cudaGetLastError();
    return tfail(e == cudaErrorMemoryAllocation ? SH_ERR_OOM : SH_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e));
}

int wait_event(cudaEvent_t ev, int timeout_ms) {
    const auto deadline = std::chrono::steady_clock::now() + std::chrono::milliseconds(timeout_ms < 0 ? 0 : timeout_ms);
    for (int spins = 0;; ++spins) {
        const cudaError_t q = cudaEventQuery(ev);
        if (q == cudaSuccess) return SH_OK;
        if (q != cudaErrorNotReady) return cuda_check(q, "cudaEventQuery");
        if (std::chrono::steady_clock::now() >= deadline) return tfail(SH_ERR_TIMEOUT, "transfer not complete after %d ms", timeout_ms);
        if (spins > 200) std::this_thread::sleep_for(std::chrono::microseconds(50));
    }
}

void release_slot(Engine& e, int block) {
    Block& b = e.blocks[static_cast<size_t>(block)];
    if (b.slot >= 0) {
        e.slots[static_cast<size_t>(b.slot)].block = -1;
        e.free_slots.push_back(b.slot);
        b.slot = -1;
    }
}

// Blocks whose write-back has finished become CPU-resident and give their slot back.
int finish_evictions(Engine& e, int timeout_ms) {
    for (size_t i = 0; i < e.blocks.size(); ++i) {
        Block& b = e.blocks[i];
        if (b.location != kD2H) continue;
        const int rc = wait_event(b.moved, timeout_ms);
        if (rc != SH_OK) return rc;
        b.location = kCpu;
        release_slot(e, static_cast<int>(i));
    }
    return SH_OK;
}

int async_prefetch(Engine& e, int block, int timeout_ms) {
    if (block < 0 || block >= static_cast<int>(e.blocks.size())) return SH_OK;
    Block& b = e.blocks[static_cast<size_t>(block)];
    if (b.location == kGpu || b.location == kH2D) return SH_OK;
    if (b.location == kD2H) {
        const int rc = wait_event(b.moved, timeout_ms);
        if (rc != SH_OK) return rc;
        b.location = kCpu;
        release_slot(e, block);
    }
    if (b.slot < 0) {
        if (e.free_slots.empty()) return tfail(SH_ERR_BUSY, "no free GPU slot: raise the window or evict a block");
        b.slot = e.free_slots.back();
        e.free_slots.pop_back();
        e.slots[static_cast<size_t>(b.slot)].block = block;
    }
    Slot& s = e.slots[static_cast<size_t>(b.slot)];
    if (b.int8) {
        // packed image over the link (1 byte per weight), then the block kernel expands it into the slot
        if (s.ptrs[0] == nullptr) return tfail(SH_ERR_INVALID_ARG, "slot %d has no GPU pointer for parameter 0", b.slot);
        void* stage = e.staging[static_cast<size_t>(b.slot)];
        int rc = cuda_check(cudaMemcpyAsync(stage, b.host, b.packed_bytes, cudaMemcpyHostToDevice, e.prefetch),
                            "cudaMemcpyAsync H2D");
        if (rc != SH_OK) return rc;
        rc = sh_dequant_block_async(b.descs.data(), static_cast<int32_t>(b.descs.size()), stage, b.packed_bytes, s.ptrs[0],
                                    b.out_bytes, b.out_dtype, static_cast<uint64_t>(reinterpret_cast<uintptr_t>(e.prefetch)),
                                    nullptr);
        if (rc != SH_OK) {
            char why[200];
            sh_last_error(why, sizeof(why));
            return tfail(rc, "block kernel: %s", why);
        }
    }
    for (size_t i = 0; i < b.sizes.size() && !b.int8; ++i) {
        if (b.sizes[i] == 0) continue;
        if (s.ptrs[i] == nullptr) return tfail(SH_ERR_INVALID_ARG, "slot %d has no GPU pointer for parameter %zu", b.slot, i);
        const int rc = cuda_check(cudaMemcpyAsync(s.ptrs[i], b.host + b.offsets[i], b.sizes[i], cudaMemcpyHostToDevice, e.prefetch),
                                  "cudaMemcpyAsync H2D");
        if (rc != SH_OK) return rc;
    }
    const int rc = cuda_check(cudaEventRecord(b.moved, e.prefetch), "cudaEventRecord");
    if (rc != SH_OK) return rc;
    b.location = kH2D;
    return SH_OK;
}

int async_evict(Engine& e, int block, uint64_t caller_stream) {
    if (block < 0 || block >= static_cast<int>(e.blocks.size())) return SH_OK;
    Block& b = e.blocks[static_cast<size_t>(block)];
    if (b.location == kCpu || b.location == kD2H || b.slot < 0) return SH_OK;
    Slot& s = e.slots[static_cast<size_t>(b.slot)];
    if (b.int8) {
        // nothing to write back: the slot is free once everything the caller has queued so far has run
        cudaStream_t caller = reinterpret_cast<cudaStream_t>(static_cast<uintptr_t>(caller_stream));
        int rc = SH_OK;
        if (b.location == kH2D && (rc = cuda_check(cudaStreamWaitEvent(caller, b.moved, 0), "cudaStreamWaitEvent")) != SH_OK)
            return rc;
        if ((rc = cuda_check(cudaEventRecord(b.moved, caller), "cudaEventRecord")) != SH_OK) return rc;
        b.location = kD2H;
        return SH_OK;
    }
    // the write-back starts only after everything the caller has queued so far (its use of the block)
    int rc = cuda_check(cudaEventRecord(e.fence, reinterpret_cast<cudaStream_t>(static_cast<uintptr_t>(caller_stream))),
                        "cudaEventRecord");
    if (rc != SH_OK) return rc;
    rc = cuda_check(cudaStreamWaitEvent(e.evict, e.fence, 0), "cudaStreamWaitEvent");
    if (rc != SH_OK) return rc;
    if (b.location == kH2D) {
        rc = cuda_check(cudaStreamWaitEvent(e.evict, b.moved, 0), "cudaStreamWaitEvent");
        if (rc != SH_OK) return rc;
    }
    for (size_t i = 0; i < b.sizes.size(); ++i) {
        if (b.sizes[i] == 0) continue;
        rc = cuda_check(cudaMemcpyAsync(b.host + b.offsets[i], s.ptrs[i], b.sizes[i], cudaMemcpyDeviceToHost, e.evict),
                        "cudaMemcpyAsync D2H");
        if (rc != SH_OK) return rc;
    }
    rc = cuda_check(cudaEventRecord(b.moved, e.evict), "cudaEventRecord");
    if (rc != SH_OK) return rc;
    b.location = kD2H;
    return SH_OK;
}

int sync_prefetch(Engine& e, int block, uint64_t caller_stream, int timeout_ms) {
    Block& b = e.blocks[static_cast<size_t>(block)];
    if (b.location == kGpu) return SH_OK;
    if (b.location != kH2D) {
        const int rc = async_prefetch(e, block, timeout_ms);
        if (rc != SH_OK) return rc;
    }
    // device-side ordering for the caller's stream; the host only waits up to the deadline
    int rc = cuda_check(cudaStreamWaitEvent(reinterpret_cast<cudaStream_t>(static_cast<uintptr_t>(caller_stream)), b.moved, 0),
                        "cudaStreamWaitEvent");
    if (rc != SH_OK) return rc;
    rc = wait_event(b.moved, timeout_ms);
    if (rc != SH_OK) return rc;
    b.location = kGpu;
    return SH_OK;
}

}  // namespace

extern "C" {

int32_t sh_turbo_last_error(char* buf, int32_t buf_len) {
    const int32_t n = static_cast<int32_t>(strlen(g_turbo_err));
    if (buf != nullptr && buf_len > 0) {
        const int32_t c = n < buf_len - 1 ? n : buf_len - 1;
        memcpy(buf, g_turbo_err, static_cast<size_t>(c));
        buf[c] = '\0';
    }
    return n;
}

int32_t sh_turbo_create(uint64_t* engine_out) {
    if (engine_out == nullptr) return tfail(SH_ERR_INVALID_ARG, "null engine_out");
    *engine_out = static_cast<uint64_t>(reinterpret_cast<uintptr_t>(new Engine()));
    return SH_OK;
}

int32_t sh_turbo_destroy(uint64_t engine) {
    Engine* e = as_engine(engine);
    if (e == nullptr) return SH_OK;
    // Everything that exists is released, whether or not initialize() ran to its end: a failure half-way
    // (out of page-locked or device memory) leaves streams, events and some buffers behind.
    if (e->prefetch != nullptr) cudaStreamSynchronize(e->prefetch);     // shutdown only: the caller has drained already
    if (e->evict != nullptr) cudaStreamSynchronize(e->evict);
    for (Block& b : e->blocks) {
        if (b.host != nullptr) cudaFreeHost(b.host);
        if (b.moved != nullptr) cudaEventDestroy(b.moved);
    }
    for (void* p : e->staging)
        if (p != nullptr) cudaFree(p);
    if (e->fence != nullptr) cudaEventDestroy(e->fence);
    if (e->prefetch != nullptr) cudaStreamDestroy(e->prefetch);
    if (e->evict != nullptr) cudaStreamDestroy(e->evict);
    delete e;                                    // GPU slot memory belongs to the caller and is not freed here
    return SH_OK;
}

int32_t sh_turbo_register_block(uint64_t engine, const uint64_t* param_sizes, int32_t n_params, int32_t* block_out) {
    Engine* e = as_engine(engine);
    if (e == nullptr || block_out == nullptr || n_params < 0 || (n_params > 0 && param_sizes == nullptr))
        return tfail(SH_ERR_INVALID_ARG, "bad register_block arguments");
    if (e->initialized) return tfail(SH_ERR_INVALID_ARG, "blocks must be registered before initialize");
    Block b;
    for (int i = 0; i < n_params; ++i) {
        b.offsets.push_back(b.total);
        b.sizes.push_back(static_cast<size_t>(param_sizes[i]));
        b.total += (static_cast<size_t>(param_sizes[i]) + 255) / 256 * 256;
    }
    e->blocks.push_back(std::move(b));
    *block_out = static_cast<int32_t>(e->blocks.size() - 1);
    return SH_OK;
}

int32_t sh_turbo_register_int8_block(uint64_t engine, const ShParamDesc* descs, int32_t n_descs, uint64_t packed_bytes,
                                     uint64_t out_bytes, int32_t out_dtype, int32_t* block_out) {
    Engine* e = as_engine(engine);
    if (e == nullptr || block_out == nullptr || descs == nullptr || n_descs < 1 || packed_bytes == 0 || out_bytes == 0)
        return tfail(SH_ERR_INVALID_ARG, "bad register_int8_block arguments");
    if (out_dtype != SH_DT_BF16 && out_dtype != SH_DT_F16 && out_dtype != SH_DT_F32)
        return tfail(SH_ERR_INVALID_ARG, "unknown out_dtype %d", out_dtype);
    if (e->initialized) return tfail(SH_ERR_INVALID_ARG, "blocks must be registered before initialize");
    Block b;
    b.int8 = true;
    b.descs.assign(descs, descs + n_descs);
    b.packed_bytes = static_cast<size_t>(packed_bytes);
    b.out_bytes = static_cast<size_t>(out_bytes);
    b.out_dtype = out_dtype;
    b.offsets.push_back(0);
    b.sizes.push_back(b.out_bytes);                       // what it needs of a slot
    b.total = (b.packed_bytes + 255) / 256 * 256;         // what it needs of page-locked host memory
    e->blocks.push_back(std::move(b));
    *block_out = static_cast<int32_t>(e->blocks.size() - 1);
    return SH_OK;
}

int32_t sh_turbo_initialize(uint64_t engine, int32_t device, int32_t window_size) {
    Engine* e = as_engine(engine);
    if (e == nullptr) return tfail(SH_ERR_INVALID_ARG, "null engine");
    if (e->initialized) return tfail(SH_ERR_INVALID_ARG, "Already initialized");
    if (e->prefetch != nullptr || e->evict != nullptr)
        return tfail(SH_ERR_INVALID_ARG, "an earlier initialize failed part-way; destroy this engine and create a new one");
    if (e->blocks.empty()) return tfail(SH_ERR_INVALID_ARG, "No blocks registered");
    if (window_size < 1) return tfail(SH_ERR_INVALID_ARG, "window_size must be at least 1");
    int rc = cuda_check(cudaSetDevice(device), "cudaSetDevice");
    if (rc != SH_OK) return rc;
    e->device = device;
    size_t max_params = 0;
    for (const Block& b : e->blocks) max_params = std::max(max_params, b.sizes.size());
    std::vector<size_t> capacity(max_params, 0);
    for (const Block& b : e->blocks)
        for (size_t i = 0; i < b.sizes.size(); ++i) capacity[i] = std::max(capacity[i], b.sizes[i]);
    if ((rc = cuda_check(cudaStreamCreateWithFlags(&e->prefetch, cudaStreamNonBlocking), "cudaStreamCreate")) != SH_OK) return rc;
    if ((rc = cuda_check(cudaStreamCreateWithFlags(&e->evict, cudaStreamNonBlocking), "cudaStreamCreate")) != SH_OK) return rc;
    if ((rc = cuda_check(cudaEventCreateWithFlags(&e->fence, cudaEventDisableTiming), "cudaEventCreate")) != SH_OK) return rc;
    for (Block& b : e->blocks) {
        if ((rc = cuda_check(cudaEventCreateWithFlags(&b.moved, cudaEventDisableTiming), "cudaEventCreate")) != SH_OK) return rc;
        if (b.total == 0) continue;
        if ((rc = cuda_check(cudaHostAlloc(reinterpret_cast<void**>(&b.host), b.total, cudaHostAllocPortable), "cudaHostAlloc")) != SH_OK)
            return rc;
    }
    const int window = std::min<int>(window_size, static_cast<int>(e->blocks.size()));
    for (const Block& b : e->blocks)
        if (b.int8) e->staging_bytes = std::max(e->staging_bytes, b.total);
    for (int s = 0; s < window; ++s) {
        void* stage = nullptr;
        if (e->staging_bytes != 0 && (rc = cuda_check(cudaMalloc(&stage, e->staging_bytes), "cudaMalloc")) != SH_OK) return rc;
        e->staging.push_back(stage);
        Slot slot;
        slot.ptrs.assign(max_params, nullptr);
        slot.sizes = capacity;
        e->free_slots.push_back(static_cast<int>(e->slots.size()));
        e->slots.push_back(std::move(slot));
    }
    e->initialized = true;
    return SH_OK;
}

int32_t sh_turbo_stage_block(uint64_t engine, int32_t block, const uint64_t* src_ptrs, int32_t n_ptrs) {
    Engine* e = as_engine(engine);
    if (e == nullptr || !e->initialized || block < 0 || block >= static_cast<int>(e->blocks.size()))
        return tfail(SH_ERR_INVALID_ARG, "bad stage_block arguments");
    Block& b = e->blocks[static_cast<size_t>(block)];
    if (n_ptrs != static_cast<int>(b.sizes.size())) return tfail(SH_ERR_INVALID_ARG, "Expected %zu ptrs, got %d", b.sizes.size(), n_ptrs);
    if (b.int8) {                                          // the one pointer is the packed image
        memcpy(b.host, reinterpret_cast<const void*>(static_cast<uintptr_t>(src_ptrs[0])), b.packed_bytes);
        return SH_OK;
    }
    for (size_t i = 0; i < b.sizes.size(); ++i)
        if (b.sizes[i] != 0) memcpy(b.host + b.offsets[i], reinterpret_cast<const void*>(static_cast<uintptr_t>(src_ptrs[i])), b.sizes[i]);
    return SH_OK;
}

int32_t sh_turbo_set_slot_gpu_ptrs(uint64_t engine, int32_t slot, const uint64_t* ptrs, int32_t n_ptrs) {
    Engine* e = as_engine(engine);
    if (e == nullptr || !e->initialized || slot < 0 || slot >= static_cast<int>(e->slots.size()))
        return tfail(SH_ERR_INVALID_ARG, "Slot %d out of range", slot);
    Slot& s = e->slots[static_cast<size_t>(slot)];
    if (n_ptrs != static_cast<int>(s.ptrs.size())) return tfail(SH_ERR_INVALID_ARG, "Expected %zu ptrs, got %d", s.ptrs.size(), n_ptrs);
    for (size_t i = 0; i < s.ptrs.size(); ++i) s.ptrs[i] = reinterpret_cast<void*>(static_cast<uintptr_t>(ptrs[i]));
    return SH_OK;
}

int32_t sh_turbo_step(uint64_t engine, int32_t block, int32_t backward, uint64_t caller_stream, int32_t timeout_ms) {
    Engine* e = as_engine(engine);
    if (e == nullptr || !e->initialized) return tfail(SH_ERR_INVALID_ARG, "engine not initialized");
    const int n = static_cast<int>(e->blocks.size());
    if (block < 0 || block >= n) return tfail(SH_ERR_INVALID_ARG, "block_idx %d >= %d", block, n);
    int rc = sync_prefetch(*e, block, caller_stream, timeout_ms);
    if (rc != SH_OK) return rc;
    const int evict = backward ? (block + 1 < n ? block + 1 : -1) : (block > 0 ? block - 1 : -1);
    const int next = backward ? (block > 0 ? block - 1 : -1) : (block + 1 < n ? block + 1 : -1);
    if (evict >= 0) {
        if ((rc = finish_evictions(*e, timeout_ms)) != SH_OK) return rc;
        if ((rc = async_evict(*e, evict, caller_stream)) != SH_OK) return rc;
    }
    if (next >= 0) {
        if (e->free_slots.empty() && e->blocks[static_cast<size_t>(next)].slot < 0)
            if ((rc = finish_evictions(*e, timeout_ms)) != SH_OK) return rc;
        rc = async_prefetch(*e, next, timeout_ms);
        if (rc != SH_OK && rc != SH_ERR_BUSY) return rc;     // no slot yet is fine: the block is fetched when it is needed
    }
    return SH_OK;
}

int32_t sh_turbo_evict_sync(uint64_t engine, int32_t block, uint64_t caller_stream, int32_t timeout_ms) {
    Engine* e = as_engine(engine);
    if (e == nullptr || !e->initialized) return tfail(SH_ERR_INVALID_ARG, "engine not initialized");
    const int rc = async_evict(*e, block, caller_stream);
    return rc != SH_OK ? rc : finish_evictions(*e, timeout_ms);
}

int32_t sh_turbo_ptr(uint64_t engine, int32_t block, int32_t param, int32_t on_gpu, uint64_t* ptr_out) {
    Engine* e = as_engine(engine);
    if (e == nullptr || ptr_out == nullptr || block < 0 || block >= static_cast<int>(e->blocks.size()))
        return tfail(SH_ERR_INVALID_ARG, "bad pointer query");
    Block& b = e->blocks[static_cast<size_t>(block)];
    if (param < 0 || param >= static_cast<int>(b.sizes.size())) return tfail(SH_ERR_INVALID_ARG, "parameter %d out of range", param);
    if (!on_gpu) {
        *ptr_out = static_cast<uint64_t>(reinterpret_cast<uintptr_t>(b.host + b.offsets[static_cast<size_t>(param)]));
        return SH_OK;
    }
    if (b.slot < 0) return tfail(SH_ERR_INVALID_ARG, "Block %d not on GPU", block);
    *ptr_out = static_cast<uint64_t>(reinterpret_cast<uintptr_t>(e->slots[static_cast<size_t>(b.slot)].ptrs[static_cast<size_t>(param)]));
    return SH_OK;
}

int32_t sh_turbo_block_state(uint64_t engine, int32_t block, int32_t* location_out, int32_t* slot_out) {
    Engine* e = as_engine(engine);
    if (e == nullptr || block < 0 || block >= static_cast<int>(e->blocks.size())) return tfail(SH_ERR_INVALID_ARG, "Block %d out of range", block);
    if (location_out != nullptr) *location_out = static_cast<int32_t>(e->blocks[static_cast<size_t>(block)].location);
    if (slot_out != nullptr) *slot_out = e->blocks[static_cast<size_t>(block)].slot;
    return SH_OK;
}

int32_t sh_turbo_counts(uint64_t engine, int32_t* blocks_out, int32_t* slots_out, int32_t* free_out) {
    Engine* e = as_engine(engine);
    if (e == nullptr) return tfail(SH_ERR_INVALID_ARG, "null engine");
    if (blocks_out != nullptr) *blocks_out = static_cast<int32_t>(e->blocks.size());
    if (slots_out != nullptr) *slots_out = static_cast<int32_t>(e->slots.size());
    if (free_out != nullptr) *free_out = static_cast<int32_t>(e->free_slots.size());
    return SH_OK;
}

int32_t sh_turbo_drain(uint64_t engine, int32_t timeout_ms) {
    Engine* e = as_engine(engine);
    if (e == nullptr || !e->initialized) return SH_OK;
    int rc = finish_evictions(*e, timeout_ms);
    if (rc != SH_OK) return rc;
    for (Block& b : e->blocks)
        if (b.location == kH2D) {
            if ((rc = wait_event(b.moved, timeout_ms)) != SH_OK) return rc;
            b.location = kGpu;
        }
    return SH_OK;
}

}  // extern "C"
