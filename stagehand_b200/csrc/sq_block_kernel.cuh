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

constexpr int kMaxDescs       = 32;    // descriptors per launch (more -> several launches)
constexpr int kThreads        = 256;   // threads per CTA
constexpr int kSegBytes       = 16;    // one int8 vector load = 16 weights
constexpr int kSegsPerThread  = 4;     // vector loads in flight per thread
constexpr int kTileSegs       = kThreads * kSegsPerThread;   // 1024 vectors = 16 KiB int8 per tile
constexpr int kTileItems      = kThreads * 16;               // items per tile on the element-wise paths
constexpr int kSmemRows       = kTileSegs + 8;               // scale rows staged per tile (worst case 1 row / vector)

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
};

struct BlockPlan {
    int32_t  n_desc;
    int32_t  total_tiles;
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

// Launches one plan on `stream`.
cudaError_t launch_plan(const BlockPlan& plan, int out_dtype, cudaStream_t stream, int32_t* status_dev);

}  // namespace sq
