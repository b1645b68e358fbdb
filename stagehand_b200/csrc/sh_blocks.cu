// Registered blocks and the VRAM slab pool of the C ABI.
//
// sh_block_register validates a block's descriptors and builds its launch plans ONCE; sh_block_load is
// then the whole per-load work of the streaming path in one call that never blocks: order the copy
// stream(s) after the staging slab's previous reader, move the packed image (host link, or copy-engine
// pulls from the arenas of several GPUs), order the dequant stream after the copies and after the output
// slab's previous readers, launch the block kernel, record the caller's events.
//
// The slab pool keeps the bookkeeping of the output slabs (which slab is free, which block sits where,
// which event guards a slab's reuse) on this side of the ABI; the memory itself is handed in by the
// caller, as the reference's engine takes its slot pointers from torch (turbo_src/engine.rs:361-372).
#include "sh_common.h"

#include <cstdio>
#include <cstring>
#include <map>
#include <mutex>
#include <string>
#include <vector>

namespace {

using namespace shc;

struct Block {
    std::vector<sq::BlockPlan> plans;     // built against sq::kPlanStandInBase
    int64_t elements = 0, traffic = 0;
    size_t packed_bytes = 0, out_bytes = 0;
    int out_dtype = 0;
    std::vector<ShGatherPiece> pieces;
    cudaEvent_t joined = nullptr;         // copy stream -> dequant stream
    cudaEvent_t joined2 = nullptr;        // second copy stream -> first
};

Block* as_block(uint64_t h) { return reinterpret_cast<Block*>(static_cast<uintptr_t>(h)); }

bool aligned256(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 255u) == 0; }

// ── slab pool ────────────────────────────────────────────────────────────

struct PoolSlab {
    void* ptr = nullptr;
    size_t bytes = 0;
    bool in_use = false;
    std::string block;                    // holder while in use
    cudaEvent_t released = nullptr;       // recorded at release; the next writer's stream waits for it
    bool has_release = false;
};

struct Pool {
    std::mutex mu;
    std::vector<PoolSlab> slabs;
    std::map<std::string, int> where;     // block id -> slot while held
    int64_t acquires = 0, reuses = 0;
};

Pool* as_pool(uint64_t h) { return reinterpret_cast<Pool*>(static_cast<uintptr_t>(h)); }

}  // namespace

extern "C" {

// ── registered blocks ────────────────────────────────────────────────────

int32_t sh_block_register(const ShParamDesc* descs, int32_t n_descs, size_t packed_bytes, size_t out_bytes,
                          int32_t out_dtype, uint64_t* block_out) {
    if (block_out == nullptr) return fail(SH_ERR_INVALID_ARG, "null block_out");
    if (n_descs < 1 || descs == nullptr) return fail(SH_ERR_INVALID_ARG, "a block needs at least one descriptor");
    auto* b = new Block();
    b->plans.resize(static_cast<size_t>((n_descs + sq::kMaxDescs - 1) / sq::kMaxDescs));
    int n_plans = 0;
    char err[256];
    const int rc = sq::build_plans(descs, n_descs, sq::kPlanStandInBase, packed_bytes, sq::kPlanStandInBase, out_bytes,
                                   out_dtype, b->plans.data(), &n_plans, &b->elements, &b->traffic, err, sizeof(err));
    if (rc != SH_OK) {
        delete b;
        return fail(rc, "%s", err);
    }
    b->plans.resize(static_cast<size_t>(n_plans));
    b->packed_bytes = packed_bytes;
    b->out_bytes = out_bytes;
    b->out_dtype = out_dtype;
    for (cudaEvent_t* ev : {&b->joined, &b->joined2}) {
        const cudaError_t e = cudaEventCreateWithFlags(ev, cudaEventDisableTiming);
        if (e != cudaSuccess) {
            for (cudaEvent_t made : {b->joined, b->joined2})
                if (made != nullptr) cudaEventDestroy(made);
            delete b;
            return cuda_fail(e, "cudaEventCreate");
        }
    }
    *block_out = static_cast<uint64_t>(reinterpret_cast<uintptr_t>(b));
    return SH_OK;
}

int32_t sh_block_set_gather(uint64_t block, const ShGatherPiece* pieces, int32_t n_pieces) {
    Block* b = as_block(block);
    if (b == nullptr || n_pieces < 0 || (n_pieces > 0 && pieces == nullptr))
        return fail(SH_ERR_INVALID_ARG, "bad gather arguments");
    for (int i = 0; i < n_pieces; ++i) {
        const ShGatherPiece& p = pieces[i];
        if (p.src_dev == 0 || p.bytes == 0) return fail(SH_ERR_INVALID_ARG, "gather piece %d: null source or zero size", i);
        if (p.staging_off > b->packed_bytes || p.bytes > b->packed_bytes - p.staging_off)
            return fail(SH_ERR_INVALID_ARG, "gather piece %d: [%llu, +%llu) lies outside the %zu-byte image", i,
                        static_cast<unsigned long long>(p.staging_off), static_cast<unsigned long long>(p.bytes),
                        b->packed_bytes);
    }
    b->pieces.assign(pieces, pieces + n_pieces);
    return SH_OK;
}

int32_t sh_block_unregister(uint64_t block) {
    Block* b = as_block(block);
    if (b == nullptr) return SH_OK;
    for (cudaEvent_t ev : {b->joined, b->joined2})
        if (ev != nullptr) cudaEventDestroy(ev);
    delete b;
    return SH_OK;
}

int32_t sh_block_load(uint64_t block, const ShBlockLoad* a) {
    Block* b = as_block(block);
    if (b == nullptr || a == nullptr) return fail(SH_ERR_INVALID_ARG, "null block or arguments");
    if (a->out_dev == nullptr || !aligned256(a->out_dev))
        return fail(SH_ERR_INVALID_ARG, "the output slab must be non-null and 256-byte aligned");
    cudaStream_t copy = as_stream(a->copy_stream), copy2 = as_stream(a->copy_stream2), dq = as_stream(a->dequant_stream);
    const void* packed_base = nullptr;
    bool copied = false;
    CopyTiming timing;
    int64_t copy_bytes = 0;

    switch (a->src_kind) {
        case SH_SRC_HOST: {
            if (a->src == nullptr || a->staging_dev == nullptr || !aligned256(a->staging_dev))
                return fail(SH_ERR_INVALID_ARG, "host source: the image and a 256-byte aligned staging slab are required");
            if (a->ev_staging_free != 0)
                SH_CUDA(cudaStreamWaitEvent(copy, as_event(a->ev_staging_free), 0), "cudaStreamWaitEvent");
            timing.begin(copy);
            copy_bytes = static_cast<int64_t>(b->packed_bytes);
            SH_CUDA(cudaMemcpyAsync(a->staging_dev, a->src, b->packed_bytes, cudaMemcpyHostToDevice, copy), "cudaMemcpyAsync H2D");
            g_ctr.h2d_copies.fetch_add(1, std::memory_order_relaxed);
            g_ctr.h2d_bytes.fetch_add(static_cast<int64_t>(b->packed_bytes), std::memory_order_relaxed);
            packed_base = a->staging_dev;
            copied = true;
            break;
        }
        case SH_SRC_DEVICE: {
            if (a->src == nullptr || !aligned256(a->src))
                return fail(SH_ERR_INVALID_ARG, "device source: a 256-byte aligned image address is required");
            packed_base = a->src;
            break;
        }
        case SH_SRC_GATHER: {
            if (a->staging_dev == nullptr || !aligned256(a->staging_dev))
                return fail(SH_ERR_INVALID_ARG, "gather: a 256-byte aligned staging slab is required");
            if (b->pieces.empty()) return fail(SH_ERR_INVALID_ARG, "gather: no pieces were registered for this block");
            const bool two = copy2 != nullptr && copy2 != copy && b->pieces.size() > 1;
            if (a->ev_staging_free != 0) {
                SH_CUDA(cudaStreamWaitEvent(copy, as_event(a->ev_staging_free), 0), "cudaStreamWaitEvent");
                if (two) SH_CUDA(cudaStreamWaitEvent(copy2, as_event(a->ev_staging_free), 0), "cudaStreamWaitEvent");
            }
            timing.begin(copy);
            uint8_t* staging = static_cast<uint8_t*>(a->staging_dev);
            int64_t bytes = 0;
            for (size_t i = 0; i < b->pieces.size(); ++i) {
                const ShGatherPiece& p = b->pieces[i];
                SH_CUDA(cudaMemcpyAsync(staging + p.staging_off, reinterpret_cast<const void*>(static_cast<uintptr_t>(p.src_dev)),
                                        p.bytes, cudaMemcpyDeviceToDevice, (two && (i & 1)) ? copy2 : copy),
                        "cudaMemcpyAsync D2D");
                bytes += static_cast<int64_t>(p.bytes);
            }
            if (two) {     // fold the second copy stream back into the first: "copied" means every piece has landed
                SH_CUDA(cudaEventRecord(b->joined2, copy2), "cudaEventRecord");
                SH_CUDA(cudaStreamWaitEvent(copy, b->joined2, 0), "cudaStreamWaitEvent");
            }
            g_ctr.peer_copies.fetch_add(static_cast<int64_t>(b->pieces.size()), std::memory_order_relaxed);
            g_ctr.peer_bytes.fetch_add(bytes, std::memory_order_relaxed);
            copy_bytes = bytes;
            packed_base = a->staging_dev;
            copied = true;
            break;
        }
        default:
            return fail(SH_ERR_INVALID_ARG, "unknown source kind %d", a->src_kind);
    }

    if (copied) {
        timing.end(copy_bytes);
        for (uint64_t ev : {a->ev_copied, a->ev_copied2})
            if (ev != 0) SH_CUDA(cudaEventRecord(as_event(ev), copy), "cudaEventRecord");
        if (copy != dq) {
            SH_CUDA(cudaEventRecord(b->joined, copy), "cudaEventRecord");
            SH_CUDA(cudaStreamWaitEvent(dq, b->joined, 0), "cudaStreamWaitEvent");
        }
    }
    if (a->ev_out_free != 0) SH_CUDA(cudaStreamWaitEvent(dq, as_event(a->ev_out_free), 0), "cudaStreamWaitEvent");
    if (a->ev_src_ready != 0) SH_CUDA(cudaStreamWaitEvent(dq, as_event(a->ev_src_ready), 0), "cudaStreamWaitEvent");

    // the plans are moved to this load's buffers on a private copy (the registered ones stay as built)
    sq::BlockPlan local[2];
    std::vector<sq::BlockPlan> many;
    sq::BlockPlan* plans = local;
    if (b->plans.size() > 2) {
        many = b->plans;
        plans = many.data();
    } else {
        for (size_t i = 0; i < b->plans.size(); ++i) local[i] = b->plans[i];
    }
    for (size_t i = 0; i < b->plans.size(); ++i) sq::rebase_plan(plans[i], packed_base, a->out_dev);
    const int rc = launch_plans(plans, static_cast<int>(b->plans.size()), b->elements, b->traffic, b->out_dtype, dq,
                                a->status_dev);
    if (rc != SH_OK) return rc;
    for (uint64_t ev : {a->ev_ready, a->ev_ready2, a->ev_ready3})
        if (ev != 0) SH_CUDA(cudaEventRecord(as_event(ev), dq), "cudaEventRecord");
    return SH_OK;
}

// ── VRAM slab pool ───────────────────────────────────────────────────────

int32_t sh_vram_pool_create(int32_t n_slabs, const uint64_t* base_ptrs, const uint64_t* slab_bytes, uint64_t* pool_out) {
    if (pool_out == nullptr || n_slabs < 0 || (n_slabs > 0 && (base_ptrs == nullptr || slab_bytes == nullptr)))
        return fail(SH_ERR_INVALID_ARG, "bad pool arguments");
    auto* p = new Pool();
    *pool_out = static_cast<uint64_t>(reinterpret_cast<uintptr_t>(p));
    for (int i = 0; i < n_slabs; ++i) {
        int32_t slot = -1;
        const int rc = sh_vram_pool_add_slab(*pool_out, base_ptrs[i], slab_bytes[i], &slot);
        if (rc != SH_OK) {
            sh_vram_pool_destroy(*pool_out);
            *pool_out = 0;
            return rc;
        }
    }
    return SH_OK;
}

int32_t sh_vram_pool_add_slab(uint64_t pool, uint64_t base_ptr, uint64_t bytes, int32_t* slot_out) {
    Pool* p = as_pool(pool);
    if (p == nullptr || base_ptr == 0 || bytes == 0) return fail(SH_ERR_INVALID_ARG, "bad slab");
    if ((base_ptr & 255u) != 0) return fail(SH_ERR_INVALID_ARG, "slab memory must be 256-byte aligned");
    PoolSlab s;
    s.ptr = reinterpret_cast<void*>(static_cast<uintptr_t>(base_ptr));
    s.bytes = static_cast<size_t>(bytes);
    SH_CUDA(cudaEventCreateWithFlags(&s.released, cudaEventDisableTiming), "cudaEventCreate");
    std::lock_guard<std::mutex> lk(p->mu);
    p->slabs.push_back(s);
    if (slot_out != nullptr) *slot_out = static_cast<int32_t>(p->slabs.size() - 1);
    return SH_OK;
}

int32_t sh_slab_acquire(uint64_t pool, const char* block_id, uint64_t bytes, uint64_t max_bytes, uint64_t writer_stream,
                        int32_t* slot_out, uint64_t* ptr_out) {
    Pool* p = as_pool(pool);
    if (p == nullptr || block_id == nullptr || slot_out == nullptr) return fail(SH_ERR_INVALID_ARG, "bad acquire arguments");
    std::lock_guard<std::mutex> lk(p->mu);
    if (p->where.count(block_id) != 0) return fail(SH_ERR_INVALID_ARG, "block %s already holds slot %d", block_id, p->where[block_id]);
    // smallest free slab that fits (and is not larger than the caller allows)
    int best = -1;
    for (size_t i = 0; i < p->slabs.size(); ++i) {
        const PoolSlab& s = p->slabs[i];
        if (s.in_use || s.ptr == nullptr || s.bytes < bytes || (max_bytes != 0 && s.bytes > max_bytes)) continue;
        if (best < 0 || s.bytes < p->slabs[static_cast<size_t>(best)].bytes) best = static_cast<int>(i);
    }
    if (best < 0) return SH_ERR_BUSY;              // nothing free of that size: the caller adds a slab or evicts
    PoolSlab& s = p->slabs[static_cast<size_t>(best)];
    if (s.has_release) {
        // device-side ordering only: the writer's stream starts after the work queued before the release
        SH_CUDA(cudaStreamWaitEvent(as_stream(writer_stream), s.released, 0), "cudaStreamWaitEvent");
        p->reuses += 1;
    }
    s.in_use = true;
    s.block = block_id;
    p->where[s.block] = best;
    p->acquires += 1;
    *slot_out = best;
    if (ptr_out != nullptr) *ptr_out = static_cast<uint64_t>(reinterpret_cast<uintptr_t>(s.ptr));
    return SH_OK;
}

int32_t sh_slab_release(uint64_t pool, int32_t slot, uint64_t reader_stream) {
    Pool* p = as_pool(pool);
    if (p == nullptr) return fail(SH_ERR_INVALID_ARG, "null pool");
    std::lock_guard<std::mutex> lk(p->mu);
    if (slot < 0 || slot >= static_cast<int>(p->slabs.size()) || !p->slabs[static_cast<size_t>(slot)].in_use)
        return fail(SH_ERR_INVALID_ARG, "slot %d is not held", slot);
    PoolSlab& s = p->slabs[static_cast<size_t>(slot)];
    SH_CUDA(cudaEventRecord(s.released, as_stream(reader_stream)), "cudaEventRecord");
    s.has_release = true;
    s.in_use = false;
    p->where.erase(s.block);
    s.block.clear();
    return SH_OK;
}

int32_t sh_vram_pool_remove_slab(uint64_t pool, int32_t slot, int32_t timeout_ms) {
    Pool* p = as_pool(pool);
    if (p == nullptr) return fail(SH_ERR_INVALID_ARG, "null pool");
    std::lock_guard<std::mutex> lk(p->mu);
    if (slot < 0 || slot >= static_cast<int>(p->slabs.size())) return fail(SH_ERR_INVALID_ARG, "unknown slot %d", slot);
    PoolSlab& s = p->slabs[static_cast<size_t>(slot)];
    if (s.ptr == nullptr) return SH_OK;
    if (s.in_use) return fail(SH_ERR_BUSY, "slot %d is held by block %s", slot, s.block.c_str());
    if (s.has_release && timeout_ms >= 0) {
        const int rc = wait_event_bounded(s.released, timeout_ms);   // its last readers must be done before the memory goes
        if (rc != SH_OK) return rc;
    }
    cudaEventDestroy(s.released);
    s = PoolSlab();                                 // the slot number is retired, never reused
    return SH_OK;
}

int32_t sh_block_location(uint64_t pool, const char* block_id, int32_t* slot_out) {
    Pool* p = as_pool(pool);
    if (p == nullptr || block_id == nullptr || slot_out == nullptr) return fail(SH_ERR_INVALID_ARG, "bad location arguments");
    std::lock_guard<std::mutex> lk(p->mu);
    auto it = p->where.find(block_id);
    *slot_out = it == p->where.end() ? -1 : it->second;
    return SH_OK;
}

int32_t sh_vram_pool_stats(uint64_t pool, ShPoolStats* out) {
    Pool* p = as_pool(pool);
    if (p == nullptr || out == nullptr) return fail(SH_ERR_INVALID_ARG, "bad stats arguments");
    std::lock_guard<std::mutex> lk(p->mu);
    memset(out, 0, sizeof(*out));
    for (const PoolSlab& s : p->slabs) {
        if (s.ptr == nullptr) continue;
        out->slabs += 1;
        out->total_bytes += static_cast<int64_t>(s.bytes);
        if (s.in_use) out->held_slabs += 1;
        else out->free_bytes += static_cast<int64_t>(s.bytes);
    }
    out->acquires = p->acquires;
    out->reuses = p->reuses;
    return SH_OK;
}

int32_t sh_vram_pool_destroy(uint64_t pool) {
    Pool* p = as_pool(pool);
    if (p == nullptr) return SH_OK;
    for (PoolSlab& s : p->slabs)
        if (s.released != nullptr) cudaEventDestroy(s.released);
    delete p;                                       // slab memory belongs to the caller and is not freed here
    return SH_OK;
}

}  // extern "C"
