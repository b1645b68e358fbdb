/*
 * stagehand_b200 -- C ABI of the B200-native SquareQ weight-streaming path.
 *
 * Plain C types only: pointers, sizes, integer handles.  Streams and events
 * cross the boundary as uint64_t holding a cudaStream_t / cudaEvent_t, the same
 * convention the reference's native crates use for streams coming from
 * torch.cuda.Stream.cuda_stream (vmm_src/python.rs:64-73).
 *
 * Every function returns an int32 status: 0 = ok, negative = SH_ERR_*.  The
 * text of the last failure on the calling thread is read with sh_last_error().
 * No function calls back into the host language, takes its interpreter lock,
 * or blocks -- except the explicit *_wait / *_synchronize calls, which take a
 * deadline in milliseconds and return SH_ERR_TIMEOUT when it passes.
 *
 * Each declaration names the reference interface it replaces (paths relative
 * to the reference project).
 */
#ifndef STAGEHAND_B200_H
#define STAGEHAND_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define SH_ABI_VERSION 2

/* status codes */
#define SH_OK                 0
#define SH_ERR_INVALID_ARG   -1
#define SH_ERR_OOM           -2
#define SH_ERR_CUDA          -3
#define SH_ERR_TIMEOUT       -4
#define SH_ERR_BUSY          -5   /* "not ready yet" from the query calls */
#define SH_ERR_UNSUPPORTED   -6

/* what a descriptor asks the block kernel to produce */
#define SH_KIND_DEQUANT_I8    0   /* int8 rows * fp32 row scale (- fp32 row zero point) -> out dtype */
#define SH_KIND_CAST_F32      1   /* fp32 vector -> out dtype (bias, norm weights)                  */
#define SH_KIND_COPY          2   /* raw bytes (already in the out dtype)                           */
#define SH_KIND_ZERO          3   /* zero fill                                                      */

/* runtime dtype of the block's VRAM slab */
#define SH_DT_BF16            0
#define SH_DT_F16             1
#define SH_DT_F32             2

/* descriptor flags */
#define SH_DESC_PEER_SOURCE   1u  /* source bytes live in another GPU's memory: plain loads only */
#define SH_DESC_ABSOLUTE      2u  /* src_off / scale_off / zp_off are absolute device addresses (a stripe of the
                                     matrix resident in some GPU's arena), not offsets into the packed image; the
                                     caller vouches for their extent -- only alignment is checked */

/*
 * One parameter of a block.  All *_off fields are byte offsets: sources from
 * the start of the packed image, dst_off from the start of the output slab.
 *
 *   DEQUANT_I8: rows x cols int8 at src_off with row stride ld bytes; rows fp32
 *               scales at scale_off; rows fp32 zero points at zp_off, or
 *               zp_off = -1 when every zero point is zero.  Output is dense
 *               [rows, cols] in the out dtype at dst_off.
 *   CAST_F32:   cols fp32 values at src_off -> cols out-dtype values at dst_off.
 *   COPY:       cols bytes from src_off to dst_off.
 *   ZERO:       cols bytes of zero at dst_off.
 *
 * Replaces, per parameter, one iteration of the layout loop in
 * src/stagehand/scheduler.py:263-325.
 */
typedef struct ShParamDesc {
    int32_t  kind;
    uint32_t flags;
    int64_t  src_off;
    int64_t  scale_off;
    int64_t  zp_off;
    int64_t  dst_off;
    int64_t  rows;
    int64_t  cols;
    int64_t  ld;
} ShParamDesc;

typedef struct ShDeviceInfo {
    int32_t device;
    int32_t cc_major;
    int32_t cc_minor;
    int32_t sm_count;
    int64_t total_mem_bytes;
    int64_t l2_bytes;
} ShDeviceInfo;

typedef struct ShStats {
    int64_t kernel_launches;      /* block-kernel launches since sh_init / sh_stats_reset   */
    int64_t elements_dequantised; /* int8 weights converted                                   */
    int64_t h2d_copies;           /* host-to-device copies issued                             */
    int64_t h2d_bytes;
    int64_t peer_copies;          /* device-to-device copies issued (local or peer source)    */
    int64_t peer_bytes;
    int64_t kernel_status_errors; /* status-word read-backs (sh_status_poll) that came back non-zero */
} ShStats;

/* ── library ─────────────────────────────────────────────────────────── */

/* ABI version of the loaded library (SH_ABI_VERSION it was built with). */
int32_t sh_abi_version(void);

/* Copies the last error text of the calling thread into buf (NUL-terminated). Returns its length. */
int32_t sh_last_error(char* buf, int32_t buf_len);

/*
 * Selects the device for the calling thread and checks that it can run the
 * sm_100a kernels.  Replaces TransferEngine::initialize's cudaSetDevice
 * (turbo_src/engine.rs:102-126) and SlabAllocator::new(device) (vmm_src/allocator.rs:80-137).
 */
int32_t sh_init(int32_t device);
int32_t sh_shutdown(void);
int32_t sh_device_info(int32_t device, ShDeviceInfo* out);
int32_t sh_stats(ShStats* out);
int32_t sh_stats_reset(void);

/* ── streams and events ──────────────────────────────────────────────── */

/*
 * Non-blocking stream with a priority (negative = higher), as the reference's
 * copy stream (src/stagehand/__init__.py:159-161; turbo_src/engine.rs:127-130).
 */
int32_t sh_stream_create(int32_t priority, uint64_t* stream_out);
int32_t sh_stream_destroy(uint64_t stream);
int32_t sh_stream_synchronize(uint64_t stream, int32_t timeout_ms);
int32_t sh_stream_wait_event(uint64_t stream, uint64_t event);

/*
 * Events: record / query / bounded wait.  Replace torch.cuda.Event use in
 * src/stagehand/transfer.py:129-135,:188,:203 and cudaEvent* in turbo_src/cuda_ffi.rs:49-54.
 * sh_event_query returns SH_OK when complete and SH_ERR_BUSY when not.
 * sh_event_wait polls until the deadline instead of blocking without bound.
 */
int32_t sh_event_create(int32_t enable_timing, uint64_t* event_out);
int32_t sh_event_destroy(uint64_t event);
int32_t sh_event_record(uint64_t event, uint64_t stream);
int32_t sh_event_query(uint64_t event);
int32_t sh_event_wait(uint64_t event, int32_t timeout_ms);
int32_t sh_event_elapsed_ms(uint64_t start, uint64_t stop, float* ms_out);

/* ── memory ──────────────────────────────────────────────────────────── */

/*
 * Page-locked host memory for packed block images.  Replaces cudaMallocHost /
 * cudaFreeHost in turbo_src/engine.rs:132-138,:396-415 and the pin_memory slabs
 * of src/stagehand/pool.py:86-101.
 */
int32_t sh_host_alloc(size_t bytes, void** ptr_out);
int32_t sh_host_free(void* ptr);
/* Page-lock / unlock memory the caller already owns (e.g. a torch CPU tensor). */
int32_t sh_host_register(void* ptr, size_t bytes);
int32_t sh_host_unregister(void* ptr);

/*
 * Device memory outside any caching allocator, for INT8 images that stay
 * resident in HBM (one GPU's share of a sharded model).  Exportable with
 * sh_ipc_export.  No reference counterpart beyond cudaMalloc in turbo_src/cuda_ffi.rs:31.
 */
int32_t sh_device_alloc(size_t bytes, void** ptr_out);
int32_t sh_device_free(void* ptr);

/*
 * Row-strided host copy on several threads: rows x row_bytes from src (stride
 * src_ld) to dst (stride dst_ld).  Builds a packed image from slab tensors
 * whose rows are padded.  Replaces the per-parameter host copies of
 * TransferEngine::stage_block_to_pinned (turbo_src/engine.rs:159-176).
 */
int32_t sh_pack_rows(void* dst, int64_t dst_ld, const void* src, int64_t src_ld,
                     int64_t rows, int64_t row_bytes, int32_t n_threads);

/*
 * Host memory: make dst[0, bytes) equal src[0, bytes), writing only when they differ; *changed_out says
 * whether they did.  Keeps the small module-owned parameters (norm weights, biases) of a packed image
 * current without touching it when nothing changed -- the reference restages them at every load
 * (src/stagehand/scheduler.py:310-322).
 */
int32_t sh_sync_bytes(void* dst, const void* src, size_t bytes, int32_t* changed_out);

/* ── data movement ───────────────────────────────────────────────────── */

/*
 * Asynchronous host-to-device copy of a packed image on `stream`.  Replaces
 * gpu_dest.copy_(src, non_blocking=True) in src/stagehand/transfer.py:132-133 and
 * cudaMemcpyAsync in turbo_src/engine.rs:202-231.
 */
int32_t sh_copy_h2d_async(void* dst_dev, const void* src_host, size_t bytes, uint64_t stream);

/*
 * Asynchronous device-to-device copy of a packed image into a local staging
 * slab; src may be a peer GPU's memory opened with sh_ipc_open (copy engines,
 * no SM use).  The reference is single-GPU: no counterpart.
 */
int32_t sh_pull_block_async(void* dst_local, const void* src_dev, size_t bytes, uint64_t stream);

/* Enable direct access from the current device to `peer_device` (idempotent). */
int32_t sh_peer_enable(int32_t peer_device);

/* 64-byte inter-process handle of a sh_device_alloc allocation, and its peer-side mapping. */
int32_t sh_ipc_export(void* dev_ptr, uint8_t handle_out[64]);
int32_t sh_ipc_open(const uint8_t handle[64], void** dev_ptr_out);
int32_t sh_ipc_close(void* dev_ptr);

/* ── the block kernel ────────────────────────────────────────────────── */

/*
 * Launches the sm_100a block kernel on `stream`: for every descriptor, reads
 * its source inside packed_dev[0, packed_bytes) and writes its destination
 * inside out_dev[0, out_bytes) in `out_dtype`.  Descriptors are validated on the
 * host first (bounds, alignment of the element size); an invalid one fails the
 * call with SH_ERR_INVALID_ARG and nothing is launched.  `status_dev` is either
 * NULL or a device int32 the kernel ORs error bits into (it never faults on a
 * bad descriptor or a scale fetch that does not complete: it records and skips).
 *
 * `descs` is host memory and is consumed before the call returns.
 *
 * Replaces the SquareQ host dequant _copy_squareq_backed_params_into_buffer
 * (src/stagehand/scheduler.py:243-325) -- the output bytes are what that
 * function writes into the pinned slab, produced directly in VRAM.
 */
int32_t sh_dequant_block_async(const ShParamDesc* descs, int32_t n_descs,
                               const void* packed_dev, size_t packed_bytes,
                               void* out_dev, size_t out_bytes, int32_t out_dtype,
                               uint64_t stream, int32_t* status_dev);

/*
 * One block from HOST memory to runtime-dtype weights in VRAM:
 *   copy_stream:    H2D copy of the packed image into staging_dev, record ev_copied
 *   dequant_stream: wait ev_copied, run the block kernel into out_dev, record ev_ready
 * ev_copied / ev_ready may be 0 (then no event is recorded; with ev_copied = 0 and
 * two different streams the call fails, because the kernel could not be ordered
 * after the copy).  The caller makes its compute stream wait on ev_ready.
 *
 * Replaces _stage_block_to_host + submit_h2d for a SquareQ block
 * (src/stagehand/scheduler.py:953-987, src/stagehand/transfer.py:108-143).
 */
int32_t sh_stream_block_async(const ShParamDesc* descs, int32_t n_descs,
                              const void* packed_host, size_t packed_bytes,
                              void* staging_dev, void* out_dev, size_t out_bytes, int32_t out_dtype,
                              uint64_t copy_stream, uint64_t dequant_stream,
                              uint64_t ev_copied, uint64_t ev_ready, int32_t* status_dev);

/*
 * Non-blocking watch on a device status word (the `status_dev` handed to the block-kernel calls).  Each call
 * looks at the previous read-back if it has landed -- a non-zero word is ORed into the sticky bits returned
 * in *bits_out and counted in ShStats.kernel_status_errors -- and queues the next one on `stream`: a
 * device-to-host copy of the word followed by clearing it, so bits set by later launches on that stream are
 * seen by a later poll.  Bits: 1 = a scale fetch timed out and plain loads were used (results correct),
 * 2 = a descriptor with an unknown path was skipped (its destination bytes are stale).  Meant to be called
 * once per step; sh_status_forget drops the watch (before the word's memory is freed).  The reference has
 * no device code and therefore no counterpart.
 */
int32_t sh_status_poll(int32_t* status_dev, uint64_t stream, int32_t* bits_out);
int32_t sh_status_forget(int32_t* status_dev);

/* ── registered blocks: validate and plan once, load with one call ───── */

/* where sh_block_load takes the packed image from */
#define SH_SRC_HOST    0   /* src = page-locked host image: one copy over the host link into staging_dev  */
#define SH_SRC_DEVICE  1   /* src = the image in device memory (this GPU's, or a peer's with               */
                           /* SH_DESC_PEER_SOURCE descriptors): the kernel reads it in place, no staging    */
#define SH_SRC_GATHER  2   /* the pieces given to sh_block_set_gather are pulled into staging_dev by copy   */
                           /* engines (one cudaMemcpyAsync each); src is unused                             */

/* `bytes` at device address `src_dev` (this GPU's memory or a peer's mapped arena) land at staging_dev + staging_off */
typedef struct ShGatherPiece {
    uint64_t src_dev;
    uint64_t staging_off;
    uint64_t bytes;
} ShGatherPiece;

/*
 * Arguments of one load.  Streams and events are raw handles; an event field of 0 means "none".
 *   ev_staging_free  the copy stream(s) wait for it before overwriting staging_dev (the kernel that last read it)
 *   ev_out_free      the dequant stream waits for it before writing out_dev (the slab's previous readers)
 *   ev_src_ready     the dequant stream waits for it before the kernel (e.g. a side copy the absolute
 *                    descriptors read from)
 *   ev_copied/2      recorded on copy_stream once every copy of this load has been queued behind it
 *   ev_ready/2/3     recorded on dequant_stream after the block kernel (one for the consumer, one for the
 *                    staging slab's next writer, one for whatever else the kernel read)
 * copy_stream2 (0 = none) takes every second piece of a gather so that two copy engines run side by side.
 * staging_dev and out_dev (and src for SH_SRC_DEVICE) must be 256-byte aligned.
 */
typedef struct ShBlockLoad {
    const void* src;
    void*       staging_dev;
    void*       out_dev;
    int32_t*    status_dev;
    uint64_t    copy_stream;
    uint64_t    copy_stream2;
    uint64_t    dequant_stream;
    uint64_t    ev_staging_free;
    uint64_t    ev_out_free;
    uint64_t    ev_src_ready;
    uint64_t    ev_copied;
    uint64_t    ev_copied2;
    uint64_t    ev_ready;
    uint64_t    ev_ready2;
    uint64_t    ev_ready3;
    int32_t     src_kind;
    int32_t     reserved;
} ShBlockLoad;

/*
 * sh_block_register checks a block's descriptors (as sh_dequant_block_async does) against an image of
 * packed_bytes and a slab of out_bytes and builds its launch plans once; the handle is then loaded any number
 * of times with sh_block_load, which does no validation beyond its pointers and never blocks:
 *   copy stream(s):  wait ev_staging_free; host copy or gather copies into staging_dev; record ev_copied
 *   dequant stream:  wait for the copies, ev_out_free and ev_src_ready; block kernel; record ev_ready
 * Descriptors flagged SH_DESC_ABSOLUTE keep their addresses; the others are offsets into whatever image the
 * load names (staging_dev, or src for SH_SRC_DEVICE).  A failed call may have queued its copies already; it
 * never launches a kernel on bad arguments.  Handles are independent of one another and of the calling thread,
 * but one handle is not synchronised internally: do not call sh_block_set_gather or sh_block_unregister on it
 * while another thread is inside sh_block_load for the same handle.  Unregistering a block whose loads are
 * still running on the GPU is fine (everything a launch needs was handed over when it was queued).
 *
 * Replaces, per block load, _stage_block_to_host + submit_h2d (src/stagehand/scheduler.py:953-987,
 * src/stagehand/transfer.py:108-143); registration replaces TransferEngine::register_block
 * (turbo_src/engine.rs:82-100) for packed INT8 blocks.
 */
int32_t sh_block_register(const ShParamDesc* descs, int32_t n_descs, size_t packed_bytes, size_t out_bytes,
                          int32_t out_dtype, uint64_t* block_out);
int32_t sh_block_set_gather(uint64_t block, const ShGatherPiece* pieces, int32_t n_pieces);
int32_t sh_block_load(uint64_t block, const ShBlockLoad* args);
int32_t sh_block_unregister(uint64_t block);

/* ── VRAM slab pool ──────────────────────────────────────────────────── */

typedef struct ShPoolStats {
    int64_t slabs;
    int64_t held_slabs;
    int64_t total_bytes;
    int64_t free_bytes;
    int64_t acquires;
    int64_t reuses;       /* acquires that found a slab released earlier (and ordered the writer after its readers) */
} ShPoolStats;

/*
 * Output slabs of the streaming path.  The memory is the caller's (torch allocations, so that the
 * watermarks of the budget manager see it -- as the reference's engine takes slot pointers from torch,
 * turbo_src/engine.rs:361-372); the pool keeps which slab is free, which block holds which slot and the
 * event that guards a slab's reuse.
 *   sh_vram_pool_create     n_slabs may be 0; slabs can be added later     engine.rs:140-152 (slot table)
 *   sh_vram_pool_add_slab   a new slab, free                              set_slot_gpu_ptrs, engine.rs:361-372
 *   sh_slab_acquire         smallest free slab of `bytes` .. `max_bytes` (max_bytes = bytes: exact size; 0: no
 *                           upper limit) for block_id; writer_stream is ordered (on the device) after the
 *                           slab's release event; SH_ERR_BUSY when none is free
 *   sh_slab_release         records the release event on reader_stream and frees the slot
 *   sh_vram_pool_remove_slab  forgets a free slab so its memory can go: waits (bounded) for its release event,
 *                           or not at all with timeout_ms < 0 when the memory's next user is ordered behind
 *                           the releasing stream anyway (a stream-ordered allocator)
 *   sh_block_location       slot held by block_id, or -1                  block_slot, engine.rs:375-394
 */
int32_t sh_vram_pool_create(int32_t n_slabs, const uint64_t* base_ptrs, const uint64_t* slab_bytes, uint64_t* pool_out);
int32_t sh_vram_pool_add_slab(uint64_t pool, uint64_t base_ptr, uint64_t bytes, int32_t* slot_out);
int32_t sh_slab_acquire(uint64_t pool, const char* block_id, uint64_t bytes, uint64_t max_bytes, uint64_t writer_stream,
                        int32_t* slot_out, uint64_t* ptr_out);
int32_t sh_slab_release(uint64_t pool, int32_t slot, uint64_t reader_stream);
int32_t sh_vram_pool_remove_slab(uint64_t pool, int32_t slot, int32_t timeout_ms);
int32_t sh_block_location(uint64_t pool, const char* block_id, int32_t* slot_out);
int32_t sh_vram_pool_stats(uint64_t pool, ShPoolStats* out);
int32_t sh_vram_pool_destroy(uint64_t pool);

/*
 * Cap, in CTAs per SM, on block-kernel launches that read another GPU's memory
 * (descriptors flagged SH_DESC_PEER_SOURCE); 0 lifts it (the default).  Such a
 * launch runs at the pace of its NVLink reads; capped, it leaves most of every
 * SM to the kernels of the model running beside it and walks its tiles
 * grid-stride.  Results are identical either way.  No counterpart in the
 * reference, which has no multi-GPU path.  Negative values are treated as 0.
 */
int32_t sh_set_peer_ctas_per_sm(int32_t ctas_per_sm);

/*
 * Variant of the block kernel for blocks that read another GPU's memory: 8 instead of 4 sixteen-byte loads in
 * flight per thread and at most 4 instead of 16 CTAs resident per SM, so the NVLink latency is covered by
 * bytes in flight per thread rather than by the number of waiting threads.  Applies to plans built (or blocks
 * registered) after the call; off by default; results are identical either way.  No counterpart in the
 * reference.
 */
int32_t sh_set_peer_deep_loads(int32_t on);

/*
 * Another variant for blocks that read another GPU's memory: every 8 KiB tile that lies in a peer's arena is
 * fetched with ONE bulk asynchronous copy (cp.async.bulk, the SM's TMA engine; never multicast) into shared
 * memory, completion counted on an mbarrier and waited for with a bound -- on a time-out the tile is read with
 * plain loads instead and a status bit is set.  Applies to plans built (or blocks registered) after the call;
 * off by default; results are identical either way.  No counterpart in the reference.
 */
int32_t sh_set_peer_bulk_loads(int32_t on);

/*
 * Per-launch device timing of the block kernel (CUDA events on the launching
 * stream).  While enabled every launch is bracketed by a pair of timing events;
 * sh_profile_collect waits for them (bounded) and returns the sums since the
 * last collect.  Replaces nothing in the reference (its telemetry has a
 * copy_time_ms field that is never filled, src/stagehand/telemetry.py:31).
 */
int32_t sh_profile_enable(int32_t on);
int32_t sh_profile_collect(double* kernel_ms_out, int64_t* launches_out, int64_t* elements_out,
                           int64_t* bytes_out, int32_t timeout_ms);

/*
 * The same records without waiting: sh_profile_poll sums the ones whose GPU work has finished -- block-kernel
 * time per block, and (for sh_block_load) the time its copies took on the copy stream -- and leaves the rest
 * for a later poll.  This is what fills copy_time_ms / dequant_time_ms of the runtime's per-step telemetry
 * (the reference declares copy_time_ms and never fills it, src/stagehand/telemetry.py:31).
 */
typedef struct ShProfileSums {
    double  kernel_ms;
    double  copy_ms;
    int64_t kernel_blocks;     /* blocks whose kernel time is in kernel_ms        */
    int64_t copies;            /* block loads whose copy time is in copy_ms       */
    int64_t elements;          /* int8 weights expanded by those kernels          */
    int64_t kernel_bytes;      /* their algorithmic HBM bytes                     */
    int64_t copy_bytes;        /* bytes moved by those copies                     */
    int64_t pending;           /* records still running, left for the next poll   */
} ShProfileSums;
int32_t sh_profile_poll(ShProfileSums* out);

/* ── slot-rotation transfer engine ───────────────────────────────────── */

/*
 * Every registered block is kept in page-locked host memory; a window of GPU slots (memory owned by
 * the caller, handed in with sh_turbo_set_slot_gpu_ptrs) holds the blocks around the one computing.
 * sh_turbo_step(block, direction) = make `block` resident (the caller's stream is ordered after its
 * copy), write the previous block back asynchronously, start copying the next one.  All waits are
 * bounded by timeout_ms.  Failure text: sh_turbo_last_error.  Locations: 0 cpu, 1 gpu, 2 h2d, 3 d2h.
 *
 * Replaces the reference's TransferEngine (turbo_src/lib.rs:19-119, turbo_src/engine.rs:67-415):
 *   sh_turbo_create / destroy     TransferEngine::new / Drop          engine.rs:67-80, :396-415
 *   sh_turbo_register_block       register_block(param_sizes)         engine.rs:82-100
 *   sh_turbo_initialize           initialize(device, window_size)     engine.rs:102-157
 *   sh_turbo_stage_block          stage_block(idx, src_ptrs)          engine.rs:159-176
 *   sh_turbo_set_slot_gpu_ptrs    set_slot_gpu_ptrs(slot, ptrs)       engine.rs:361-373
 *   sh_turbo_step                 step(idx, "forward"|"backward")     engine.rs:304-341 (backward = 1)
 *   sh_turbo_evict_sync           evict_sync(idx)                     engine.rs:298-302
 *   sh_turbo_ptr                  gpu_ptr / cpu_ptr(block, param)     engine.rs:344-359 (on_gpu = 1 / 0)
 *   sh_turbo_block_state          block_location / block_slot         engine.rs:375-394 (slot -1 = none)
 *   sh_turbo_counts               num_blocks / num_gpu_slots / num_free_slots   engine.rs:380-382
 *   sh_turbo_drain                drain()                             lib.rs:107-118
 *
 * sh_turbo_register_int8_block has no counterpart there (the reference's engine moves bf16 bytes only):
 * it registers a block as a packed SquareQ INT8 image (*packed_bytes*, what sh_pack_rows and the Python
 * planner produce) with the descriptors that expand it.  Such a block occupies parameter position 0 of
 * its slot (*out_bytes* of the runtime dtype); sh_turbo_stage_block takes one pointer, the image; a
 * step copies the image over the link into a staging buffer the engine owns (one per slot) and runs the
 * block kernel into the slot; eviction copies nothing back.  sh_turbo_ptr(block, 0, on_gpu = 0) is the
 * host image.
 */
int32_t sh_turbo_create(uint64_t* engine_out);
int32_t sh_turbo_destroy(uint64_t engine);
int32_t sh_turbo_register_block(uint64_t engine, const uint64_t* param_sizes, int32_t n_params, int32_t* block_out);
int32_t sh_turbo_register_int8_block(uint64_t engine, const ShParamDesc* descs, int32_t n_descs, uint64_t packed_bytes,
                                     uint64_t out_bytes, int32_t out_dtype, int32_t* block_out);
int32_t sh_turbo_initialize(uint64_t engine, int32_t device, int32_t window_size);
int32_t sh_turbo_stage_block(uint64_t engine, int32_t block, const uint64_t* src_ptrs, int32_t n_ptrs);
int32_t sh_turbo_set_slot_gpu_ptrs(uint64_t engine, int32_t slot, const uint64_t* ptrs, int32_t n_ptrs);
int32_t sh_turbo_step(uint64_t engine, int32_t block, int32_t backward, uint64_t caller_stream, int32_t timeout_ms);
int32_t sh_turbo_evict_sync(uint64_t engine, int32_t block, uint64_t caller_stream, int32_t timeout_ms);
int32_t sh_turbo_ptr(uint64_t engine, int32_t block, int32_t param, int32_t on_gpu, uint64_t* ptr_out);
int32_t sh_turbo_block_state(uint64_t engine, int32_t block, int32_t* location_out, int32_t* slot_out);
int32_t sh_turbo_counts(uint64_t engine, int32_t* blocks_out, int32_t* slots_out, int32_t* free_out);
int32_t sh_turbo_drain(uint64_t engine, int32_t timeout_ms);
int32_t sh_turbo_last_error(char* buf, int32_t buf_len);

/* ── VRAM slab allocator on CUDA virtual memory management ───────────── */

typedef struct ShVmmStats {
    int64_t total_slabs;
    int64_t total_regions;
    int64_t mapped_regions;
    int64_t mapped_bytes;
    int64_t vram_ceiling;
    int64_t granularity;
    int64_t evictions;
} ShVmmStats;

/*
 * Address space is reserved once per slab; physical memory is mapped per region on demand and
 * unmapped again (lowest slab priority first, then least recently used, never a held region, never
 * before the region's release event has completed) to stay under a byte ceiling.  A request that does
 * not fit and finds nothing evictable fails with SH_ERR_OOM; waits are bounded (SH_ERR_TIMEOUT).
 * Failure text: sh_vmm_last_error.
 *
 * Replaces the reference's SlabAllocator (vmm_src/python.rs:44-135, vmm_src/allocator.rs:80-533):
 *   sh_vmm_create           SlabAllocator(device, ceiling_mb)      python.rs:44-52  (ceiling 0 = 90 % of the device)
 *   sh_vmm_create_slab      create_slab(total_size)                python.rs:54-56
 *   sh_vmm_define_region    define_region(slab, offset, size)      python.rs:58-64
 *   sh_vmm_ensure_resident  ensure_resident(slab, region, stream)  python.rs:66-80  (hold = 1)
 *                           prefetch(slab, region)                 python.rs:82-85  (hold = 0: map, do not hold)
 *   sh_vmm_release          ResidentHandle.release / drop          vmm_src/handle.rs:65-110 (records an event on `stream`)
 *   sh_vmm_set_priority     set_priority(slab, priority)           python.rs:87-89
 *   sh_vmm_set_ceiling      set_vram_ceiling(bytes)                python.rs:91-94
 *   sh_vmm_destroy_slab     destroy_slab(slab)                     python.rs:96-98 (SH_ERR_BUSY while a region is held)
 *   sh_vmm_stats            stats()                                python.rs:100-121
 */
int32_t sh_vmm_create(int32_t device, uint64_t ceiling_bytes, uint64_t* allocator_out);
int32_t sh_vmm_destroy(uint64_t allocator);
int32_t sh_vmm_create_slab(uint64_t allocator, uint64_t total_bytes, int32_t* slab_out);
int32_t sh_vmm_define_region(uint64_t allocator, int32_t slab, uint64_t offset, uint64_t size, int32_t* region_out);
int32_t sh_vmm_ensure_resident(uint64_t allocator, int32_t slab, int32_t region, int32_t hold, void** dev_ptr_out);
int32_t sh_vmm_release(uint64_t allocator, int32_t slab, int32_t region, uint64_t stream);
/* Background prefetch (reference: vmm_src/prefetch.rs, python.rs:82-85): the request is queued and one worker
 * thread maps the region; best effort, a request that finds no room is dropped.  sh_vmm_prefetch_wait returns
 * when the queue is empty and the worker idle (SH_ERR_TIMEOUT after timeout_ms). */
int32_t sh_vmm_prefetch_async(uint64_t allocator, int32_t slab, int32_t region);
int32_t sh_vmm_prefetch_wait(uint64_t allocator, int32_t timeout_ms);
int32_t sh_vmm_set_priority(uint64_t allocator, int32_t slab, uint32_t priority);
int32_t sh_vmm_set_ceiling(uint64_t allocator, uint64_t ceiling_bytes);
int32_t sh_vmm_destroy_slab(uint64_t allocator, int32_t slab);
int32_t sh_vmm_stats(uint64_t allocator, ShVmmStats* out);
int32_t sh_vmm_last_error(char* buf, int32_t buf_len);

/*
 * Host image -> runtime-dtype weights in VRAM for callers that cannot allocate device memory on this
 * path (a process whose GPU memory was handed to another allocator at start-up, a plug-in that must
 * not grow its footprint, a loop where an allocation would stall the device).  It is
 * sh_stream_block_async on ONE stream with the staging slab replaced by a fixed array inside the
 * library's device image: SH_NOALLOC_MAX_BYTES per GPU that loads the library, held until exit.
 * Once set up it calls no cudaMalloc / cudaFree and no allocating library routine; the caller passes
 * the host image and the output slab as usual.
 *
 *   - packed_bytes above SH_NOALLOC_MAX_BYTES (or more than 128 descriptors) fails with
 *     SH_ERR_INVALID_ARG and a message; nothing is enqueued.
 *   - The array's device address is resolved (cudaGetSymbolAddress) once per device, with that device
 *     current: by sh_init(device), or else by the first call of this entry point on the device.  That
 *     is also the moment CUDA loads this part of the library onto the GPU and the array's memory is
 *     taken -- so call sh_init (or make one warm-up call) on every device BEFORE handing the device's
 *     memory to another allocator, and before any stream capture begins.  A process that skips both
 *     can see this entry point's first call fail for lack of memory.
 *   - Every call shares the one array, which keeps the previous call's bytes.  Nothing in it has to
 *     start at zero -- each call overwrites every byte its kernel reads -- but two calls whose GPU
 *     work overlaps (different streams, no ordering between them) race on it: serialise them.
 *   - Failure text: sh_noalloc_last_error (this entry point keeps its own per-thread message).
 *
 * This entry point has no counterpart in the reference.
 */
#define SH_NOALLOC_MAX_BYTES (32 * 1024 * 1024)
int32_t sh_dequant_from_host_noalloc(const ShParamDesc* descs, int32_t n_descs,
                                     const void* packed_host, size_t packed_bytes,
                                     void* out_dev, size_t out_bytes, int32_t out_dtype,
                                     uint64_t stream, int32_t* status_dev);
int32_t sh_noalloc_last_error(char* buf, int32_t buf_len);

#ifdef __cplusplus
}
#endif
#endif /* STAGEHAND_B200_H */
