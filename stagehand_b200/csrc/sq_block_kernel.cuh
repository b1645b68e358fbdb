// Block kernel of the SquareQ streaming path: plan structures shared by the
// launcher (sq_block_kernel.cu) and the C ABI (sh_capi.cu).
//
// One launch produces every parameter of one block in its VRAM slab.  Work is
// cut into fixed-size tiles, one CTA per tile, so the hardware scheduler keeps
// all 148 SMs busy whatever the mix of parameter shapes in the block.
#pragma once

#include <cstddef>
#include <cstdint>
#include <cuda_runtime.h>

#include "../../include/stagehand_b200.h"

namespace sq {

constexpr int kMaxDescs       = 128;   // descriptors per launch (more -> several launches); ~10 KiB of kernel parameters
// Tuning knobs (measured on B200): 128 threads x 4 vector loads with the register budget capped so that 16 CTAs
// (2048 threads) are resident per SM.  Full occupancy is what keeps enough bytes in flight: the same kernel at
// 10 CTAs per SM reaches 5.5 TB/s where this configuration reaches 6.5 TB/s on a 604 M-weight matrix.
#ifndef SQ_THREADS
#define SQ_THREADS 128
#endif
#ifndef SQ_SEGS_PER_THREAD
#define SQ_SEGS_PER_THREAD 4
#endif
#ifndef SQ_MIN_CTAS_PER_SM
#define SQ_MIN_CTAS_PER_SM 16
#endif
constexpr int kThreads        = SQ_THREADS;   // threads per CTA
constexpr int kSegBytes       = 16;    // one int8 vector load = 16 weights
constexpr int kSegsPerThread  = SQ_SEGS_PER_THREAD;     // vector loads in flight per thread
constexpr int kTileSegs       = kThreads * kSegsPerThread;   // 512 vectors = 8 KiB int8 -> 16 KiB bf16 per tile
constexpr int kTileItems      = kThreads * 16;               // items per tile on the element-wise paths
constexpr int kSmemRows       = kTileSegs + 8;               // scale rows staged per tile (worst case 1 row / vector)
// The "deep" variant for launches that read another GPU's memory: twice the loads in flight per thread, a
// quarter of the resident threads (4 CTAs per SM).  NVLink latency is covered by bytes in flight per thread
// instead of by thread count, so the launch leaves most of every SM's thread slots to other kernels.
constexpr int kDeepSegsPerThread = 8;
constexpr int kDeepMinCtasPerSm  = 4;

// how a descriptor is executed
enum Path : int32_t {
    kPathDequantVec    = 0,  // 16-byte loads, 16-byte stores, scales staged in shared memory
    kPathDequantScalar = 1,  // any alignment, any cols
    kPathCastVec       = 2,  // 4 fp32 per item
    kPathCastScalar    = 3,
    kPathCopyVec       = 4,  // 16 bytes per item
    kPathCopyScalar    = 5,
    kPathZeroVec       = 6,
    kPathZeroScalar    = 7,
};

constexpr int kStageMinRows    = 32;    // tiles spanning fewer scale rows read them with plain cached loads
constexpr uint32_t kFlagDense      = 0x400u;   // source rows are contiguous (ld == cols): vector i of the matrix is at src + 16 i
constexpr uint32_t kFlagStore32    = 0x200u;   // every 16-weight output vector starts on a 32-byte boundary
constexpr uint32_t kFlagRelative   = 0x800u;   // host side only: src / scale / zp were derived from the packed base (rebase_plan moves them)
constexpr uint32_t kFlagBulkScales = 0x100u;   // (bit 0 is SH_DESC_PEER_SOURCE) scale (and zero-point) rows may be fetched with a bulk async copy

struct DescDev {
    const uint8_t* src;
    const float*   scale;
    const float*   zp;        // nullptr: all zero points are zero
    uint8_t*       dst;
    int64_t        rows;
    int64_t        cols;      // dequant: weights per row; cast: elements; copy/zero: bytes
    int64_t        ld;        // dequant: source row stride in bytes
    int32_t        path;
    uint32_t       flags;
    int32_t        segs_per_row;
    int32_t        pad_;
    uint64_t       row_magic;  // floor(2^32 / segs_per_row) + 1: (t * row_magic) >> 32 == t / segs_per_row for every
                               // in-tile index t; 0 when segs_per_row is so large that the quotient is 0 or 1
};

struct BlockPlan {
    int32_t  n_desc;
    int32_t  total_tiles;
    uint32_t tile_stride;                 // CTA b works on tile (b * tile_stride) mod total_tiles; 1 = in order.
    uint32_t segs_per_thread;             // vector loads per thread of the dequant tiles (kSegsPerThread or kDeepSegsPerThread)
    uint32_t bulk_peer;                   // 1: tiles read from a peer GPU arrive by one bulk asynchronous copy each
    uint32_t pad2_;
                                          // A stride coprime with total_tiles scatters neighbouring CTAs over the
                                          // whole launch, so a launch that reads from several GPUs pulls from all
                                          // of them at once instead of one stripe (one peer) at a time.
    uint32_t tile_begin[kMaxDescs + 1];   // first tile of each descriptor; [n_desc] = total
    DescDev  d[kMaxDescs];
};

// device status bits (ORed into the caller's status word)
constexpr int32_t kStatusBulkTimeout = 1;   // a scale fetch did not complete in time; plain loads were used instead
constexpr int32_t kStatusBadPath     = 2;   // a descriptor carried an unknown path and was skipped

// Builds launch plans from user descriptors.  Returns SH_OK or SH_ERR_INVALID_ARG with `err` filled.
// `plans_out` must hold ceil(n / kMaxDescs) entries.
int build_plans(const ShParamDesc* descs, int n, const void* packed, size_t packed_bytes,
                void* out, size_t out_bytes, int out_dtype, BlockPlan* plans_out, int* n_plans_out,
                int64_t* elements_out, int64_t* traffic_bytes_out, char* err, size_t err_len);

// Plans can be built once against a stand-in base and moved to the real buffers at every launch: build with
// packed = out = kPlanStandInBase, then rebase_plan(copy, real_packed, real_out).  Both real bases must be
// 256-byte aligned, so that every alignment decision taken at build time still holds.
static void* const kPlanStandInBase = reinterpret_cast<void*>(uintptr_t(1) << 20);
void rebase_plan(BlockPlan& plan, const void* packed_base, void* out_base);

// Launches one plan on `stream`.
cudaError_t launch_plan(const BlockPlan& plan, int out_dtype, cudaStream_t stream, int32_t* status_dev);

// Cap, in CTAs per SM, on launches that read another GPU's memory (0 = none).
void set_peer_ctas_per_sm(int n);
int peer_ctas_per_sm();

// Whether plans that read another GPU's memory are built for the deep variant (off by default).
void set_peer_deep_loads(bool on);
bool peer_deep_loads();

// Whether tiles read from another GPU's memory are fetched with one bulk asynchronous copy (TMA engine, no
// multicast, bounded wait) into shared memory instead of per-thread 16-byte loads (off by default).
void set_peer_bulk_loads(bool on);
bool peer_bulk_loads();

}  // namespace sq
