// sm_100a block kernel: packed INT8 image (+ fp32 row scales) -> runtime-dtype
// weights written straight into the block's VRAM slab.
//
// Arithmetic per weight (bit-exact with the reference's host dequant,
// src/stagehand/scheduler.py:290-300):
//     x = (float) q            exact
//     y = x - zero_point[row]  one fp32 rounding (skipped when all zero points are 0: identical bits)
//     w = y * scale[row]       one fp32 rounding (never contracted into an FMA)
//     out = round-to-nearest-even(w) in bf16 / fp16, or w itself for fp32
// Subnormals are kept (no flush-to-zero), overflow rounds to +-Inf.
//
// The kernel is bound by HBM: 1 byte read + 2 bytes written per weight.  Its
// fast path issues one 16-byte coalesced load per lane (16 weights), stages the
// tile's scale rows in shared memory with a bulk asynchronous copy (TMA engine,
// completion on an mbarrier with a bounded wait) while those loads are in
// flight (only for tiles that span many rows; long rows read their few scales with cached loads),
// and writes one 32-byte store per load (two 16-byte stores when the destination is not 32-byte aligned).
#include "sq_block_kernel.cuh"

#include <atomic>

#include <cstdio>
#include <cstring>
#include <cuda_bf16.h>
#include <cuda_fp16.h>

namespace sq {

// ── small PTX wrappers ───────────────────────────────────────────────────

__device__ __forceinline__ uint32_t smem_addr(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t arrivals) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(bar)), "r"(arrivals) : "memory");
}

// makes the initialised barrier visible to the asynchronous (bulk-copy) proxy
__device__ __forceinline__ void mbar_init_fence() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_addr(bar)), "r"(bytes)
                 : "memory");
}

// global -> this CTA's shared memory, completion counted in bytes on `bar`.
// Source and destination must be 16-byte aligned and `bytes` a multiple of 16.
__device__ __forceinline__ void bulk_copy_g2s(void* dst_smem, const void* src_gmem, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cta.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     smem_addr(dst_smem)),
                 "l"(src_gmem), "r"(bytes), "r"(smem_addr(bar))
                 : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(smem_addr(bar)), "r"(parity)
        : "memory");
    return done != 0;
}

// Bounded wait: gives up after kBulkWaitSpins polls (each poll already blocks
// for a hardware-defined slice) so a copy that never lands cannot hang the GPU.
constexpr int kBulkWaitSpins = 1 << 16;
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity) {
    for (int i = 0; i < kBulkWaitSpins; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
    }
    return false;
}

// 16-byte read-only load that does not allocate in L1 (each weight is read once).
__device__ __forceinline__ int4 load_stream16(const void* p) {
    int4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.s32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

// Plain 16-byte load (used when the source is a peer GPU's memory).
__device__ __forceinline__ int4 load_plain16(const void* p) {
    int4 v;
    asm volatile("ld.global.v4.s32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

__device__ __forceinline__ void store16(void* p, const uint4& v) {
    asm volatile("st.global.v4.b32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
                 : "memory");
}

// One 32-byte store (sm_100: 256-bit global stores); `p` must be 32-byte aligned.
__device__ __forceinline__ void store32(void* p, const uint4& a, const uint4& b) {
    asm volatile("st.global.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(p), "r"(a.x), "r"(a.y), "r"(a.z),
                 "r"(a.w), "r"(b.x), "r"(b.y), "r"(b.z), "r"(b.w)
                 : "memory");
}

// ── conversion ───────────────────────────────────────────────────────────

// Byte k of `w` (a signed int8) as an exact fp32: bias the byte to unsigned,
// drop it into the mantissa of 2^23, subtract 2^23 + 128.
template <int K>
__device__ __forceinline__ float int8_lane_to_float(uint32_t w_biased) {
    const uint32_t bits = __byte_perm(w_biased, 0x4B000000u, 0x7440u | K);
    return __fsub_rn(__uint_as_float(bits), 8388736.0f);
}

template <bool HasZp>
__device__ __forceinline__ float dequant_one(float x, float scale, float zp) {
    if (HasZp) x = __fsub_rn(x, zp);
    return __fmul_rn(x, scale);
}

template <typename OutT>
struct Pack;

template <>
struct Pack<__nv_bfloat16> {
    static __device__ __forceinline__ uint32_t two(float a, float b) {
        __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
        return *reinterpret_cast<uint32_t*>(&h);
    }
    static __device__ __forceinline__ void one(void* dst, float a) {
        *reinterpret_cast<__nv_bfloat16*>(dst) = __float2bfloat16_rn(a);
    }
};

template <>
struct Pack<__half> {
    static __device__ __forceinline__ uint32_t two(float a, float b) {
        __half2 h = __floats2half2_rn(a, b);
        return *reinterpret_cast<uint32_t*>(&h);
    }
    static __device__ __forceinline__ void one(void* dst, float a) {
        *reinterpret_cast<__half*>(dst) = __float2half_rn(a);
    }
};

template <>
struct Pack<float> {
    static __device__ __forceinline__ void one(void* dst, float a) { *reinterpret_cast<float*>(dst) = a; }
};

// 16 int8 (one int4) -> 16 outputs at dst (16-byte aligned).
template <typename OutT, bool HasZp>
__device__ __forceinline__ void convert_store16(const int4& q, float scale, float zp, uint8_t* dst, bool wide) {
    const uint32_t w[4] = {static_cast<uint32_t>(q.x) ^ 0x80808080u, static_cast<uint32_t>(q.y) ^ 0x80808080u,
                           static_cast<uint32_t>(q.z) ^ 0x80808080u, static_cast<uint32_t>(q.w) ^ 0x80808080u};
    float f[16];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        f[4 * i + 0] = dequant_one<HasZp>(int8_lane_to_float<0>(w[i]), scale, zp);
        f[4 * i + 1] = dequant_one<HasZp>(int8_lane_to_float<1>(w[i]), scale, zp);
        f[4 * i + 2] = dequant_one<HasZp>(int8_lane_to_float<2>(w[i]), scale, zp);
        f[4 * i + 3] = dequant_one<HasZp>(int8_lane_to_float<3>(w[i]), scale, zp);
    }
    if constexpr (sizeof(OutT) == 2) {
        uint4 lo, hi;
        lo.x = Pack<OutT>::two(f[0], f[1]);
        lo.y = Pack<OutT>::two(f[2], f[3]);
        lo.z = Pack<OutT>::two(f[4], f[5]);
        lo.w = Pack<OutT>::two(f[6], f[7]);
        hi.x = Pack<OutT>::two(f[8], f[9]);
        hi.y = Pack<OutT>::two(f[10], f[11]);
        hi.z = Pack<OutT>::two(f[12], f[13]);
        hi.w = Pack<OutT>::two(f[14], f[15]);
        if (wide) {
            store32(dst, lo, hi);
        } else {
            store16(dst, lo);
            store16(dst + 16, hi);
        }
    } else {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            uint4 v;
            v.x = __float_as_uint(f[4 * i + 0]);
            v.y = __float_as_uint(f[4 * i + 1]);
            v.z = __float_as_uint(f[4 * i + 2]);
            v.w = __float_as_uint(f[4 * i + 3]);
            store16(dst + 16 * i, v);
        }
    }
}

// ── tile bodies ──────────────────────────────────────────────────────────

// row offset (within the tile's first row) of in-tile vector index t: t / segs_per_row without a division
__device__ __forceinline__ uint32_t tile_row_of(uint32_t t, uint32_t spr, uint64_t magic) {
    if (magic != 0) return static_cast<uint32_t>((static_cast<uint64_t>(t) * magic) >> 32);
    return t >= spr ? 1u : 0u;
}

template <typename OutT, bool HasZp, bool Dense, int kSegsPerThread, bool Bulk = false>
__device__ __forceinline__ void dequant_vec_tile(const DescDev& D, int64_t local_tile, float* s_scale, float* s_zp,
                                                 uint64_t* s_bar, int32_t* status, bool may_stage, int4* s_tile = nullptr) {
    constexpr int kTileSegs = kThreads * kSegsPerThread;       // shadows the namespace constants: this variant's tile
    const uint32_t spr = static_cast<uint32_t>(D.segs_per_row);
    const uint64_t magic = D.row_magic;
    const int64_t total_segs = D.rows * static_cast<int64_t>(spr);
    const int64_t seg0 = local_tile * kTileSegs;
    const int64_t remaining = total_segs - seg0;
    const uint32_t n_segs = remaining < kTileSegs ? static_cast<uint32_t>(remaining) : kTileSegs;
    const bool peer = (D.flags & SH_DESC_PEER_SOURCE) != 0;
    const bool wide = (D.flags & kFlagStore32) != 0;

    int4 q[kSegsPerThread];
    uint32_t row_off[kSegsPerThread];
    uint32_t cseg[kSegsPerThread];
    int64_t row_first;
    uint32_t cseg_first;

    bool bulk_timed_out = false;
    if (Dense) {
        // Contiguous rows: the address of a vector does not depend on its row, so every load is
        // issued before any index arithmetic; rows are only needed to pick the scale.
        const uint8_t* base = D.src + seg0 * kSegBytes;
        bool from_smem = false;
        if (Bulk && peer) {
            // The whole tile (contiguous in the peer's memory) in one bulk asynchronous copy into shared memory:
            // the copy engine of the SM issues the NVLink reads instead of 128 threads' worth of 16-byte loads.
            // No multicast; completion is counted on the CTA's mbarrier and waited for with a bound.
            if (threadIdx.x == 0) {
                mbar_init(s_bar, 1);
                mbar_init_fence();
                mbar_arrive_expect_tx(s_bar, n_segs * kSegBytes);
                bulk_copy_g2s(s_tile, base, n_segs * kSegBytes, s_bar);
            }
            __syncthreads();   // barrier initialised before anyone polls it
            from_smem = mbar_wait_bounded(s_bar, 0);
            if (!from_smem) {
                bulk_timed_out = true;      // fall back to plain loads below; the result stays correct
                if (status != nullptr) atomicOr(status, kStatusBulkTimeout);
            }
        }
#pragma unroll
        for (int i = 0; i < kSegsPerThread; ++i) {
            const uint32_t o = threadIdx.x + i * kThreads;
            if (o < n_segs) {
                const uint8_t* p = base + static_cast<uint32_t>(o * kSegBytes);
                q[i] = from_smem ? s_tile[o] : (peer ? load_plain16(p) : load_stream16(p));
            } else {
                q[i] = make_int4(0, 0, 0, 0);
            }
        }
        row_first = seg0 / spr;
        cseg_first = static_cast<uint32_t>(seg0 - row_first * spr);
#pragma unroll
        for (int i = 0; i < kSegsPerThread; ++i) row_off[i] = tile_row_of(cseg_first + threadIdx.x + i * kThreads, spr, magic);
    } else {
        row_first = seg0 / spr;
        cseg_first = static_cast<uint32_t>(seg0 - row_first * spr);
#pragma unroll
        for (int i = 0; i < kSegsPerThread; ++i) {
            const uint32_t o = threadIdx.x + i * kThreads;
            const uint32_t t = cseg_first + o;
            row_off[i] = tile_row_of(t, spr, magic);
            cseg[i] = t - row_off[i] * spr;
            if (o < n_segs) {
                const uint8_t* p = D.src + (row_first + row_off[i]) * D.ld + static_cast<int64_t>(cseg[i]) * kSegBytes;
                q[i] = peer ? load_plain16(p) : load_stream16(p);
            } else {
                q[i] = make_int4(0, 0, 0, 0);
            }
        }
    }

    const uint32_t rows_in_tile = (cseg_first + n_segs - 1) / spr + 1;
    // rows staged in shared memory: [r_lo, r_lo + n_stage), r_lo aligned down to 4 rows (16 bytes)
    const int64_t r_lo = row_first & ~int64_t(3);
    const uint32_t lead = static_cast<uint32_t>(row_first - r_lo);
    const uint32_t n_stage = (lead + rows_in_tile + 3u) & ~3u;
    // Staging pays when a tile spans many scale rows (short rows); with long rows a tile needs a
    // handful of scales and plain cached loads are cheaper than a barrier round trip.
    bool staged = may_stage && (D.flags & kFlagBulkScales) != 0 && rows_in_tile >= kStageMinRows &&
                  n_stage <= static_cast<uint32_t>(kSmemRows);
    if (staged) {
        if (threadIdx.x == 0) {
            mbar_init(s_bar, 1);
            mbar_init_fence();
            const uint32_t bytes = n_stage * 4u;
            mbar_arrive_expect_tx(s_bar, HasZp ? 2u * bytes : bytes);
            bulk_copy_g2s(s_scale, D.scale + r_lo, bytes, s_bar);
            if (HasZp) bulk_copy_g2s(s_zp, D.zp + r_lo, bytes, s_bar);
        }
        __syncthreads();   // barrier initialised before anyone polls it
    }

    bool timed_out = false;
    if (staged && !mbar_wait_bounded(s_bar, 0)) {
        staged = false;   // fall back to plain loads for this thread; the result stays correct
        timed_out = true;
        if (status != nullptr) atomicOr(status, kStatusBulkTimeout);
    }

    // the destination is dense in every case: output vector i of the matrix is at dst + i * 16 * sizeof(OutT)
    uint8_t* out_base = D.dst + seg0 * (kSegBytes * sizeof(OutT));
#pragma unroll
    for (int i = 0; i < kSegsPerThread; ++i) {
        const uint32_t o = threadIdx.x + i * kThreads;
        if (o >= n_segs) continue;
        float s, z = 0.0f;
        if (staged) {
            s = s_scale[lead + row_off[i]];
            if (HasZp) z = s_zp[lead + row_off[i]];
        } else {
            const int64_t row = row_first + row_off[i];
            s = peer ? D.scale[row] : __ldg(D.scale + row);
            if (HasZp) z = peer ? D.zp[row] : __ldg(D.zp + row);
        }
        convert_store16<OutT, HasZp>(q[i], s, z, out_base + static_cast<size_t>(o) * (kSegBytes * sizeof(OutT)), wide);
    }
    // A copy that was still in flight when the wait gave up targets this CTA's shared
    // memory: give it one more bounded chance to land before the CTA retires.
    if (timed_out || bulk_timed_out) (void)mbar_wait_bounded(s_bar, 0);
}

template <typename OutT>
__device__ __forceinline__ void dequant_scalar_tile(const DescDev& D, int64_t local_tile) {
    const int64_t total = D.rows * D.cols;
    const int64_t e0 = local_tile * kTileItems;
    const bool has_zp = D.zp != nullptr;
#pragma unroll 4
    for (int i = 0; i < kTileItems / kThreads; ++i) {
        const int64_t e = e0 + threadIdx.x + static_cast<int64_t>(i) * kThreads;
        if (e >= total) break;
        const int64_t row = e / D.cols;
        const int64_t col = e - row * D.cols;
        const float x = static_cast<float>(static_cast<int>(*reinterpret_cast<const int8_t*>(D.src + row * D.ld + col)));
        float y = x;
        if (has_zp) y = __fsub_rn(x, D.zp[row]);
        Pack<OutT>::one(D.dst + e * sizeof(OutT), __fmul_rn(y, D.scale[row]));
    }
}

template <typename OutT>
__device__ __forceinline__ void cast_tile(const DescDev& D, int64_t local_tile, bool vec) {
    const float* src = reinterpret_cast<const float*>(D.src);
    if (vec) {
        const int64_t items = D.cols / 4;
        const int64_t i0 = local_tile * kTileItems;
        for (int k = 0; k < kTileItems / kThreads; ++k) {
            const int64_t it = i0 + threadIdx.x + static_cast<int64_t>(k) * kThreads;
            if (it >= items) break;
            const float4 v = *reinterpret_cast<const float4*>(src + it * 4);
            uint8_t* dst = D.dst + it * 4 * sizeof(OutT);
            if constexpr (sizeof(OutT) == 2) {
                uint2 o;
                o.x = Pack<OutT>::two(v.x, v.y);
                o.y = Pack<OutT>::two(v.z, v.w);
                *reinterpret_cast<uint2*>(dst) = o;
            } else {
                *reinterpret_cast<float4*>(dst) = v;
            }
        }
    } else {
        const int64_t i0 = local_tile * kTileItems;
        for (int k = 0; k < kTileItems / kThreads; ++k) {
            const int64_t it = i0 + threadIdx.x + static_cast<int64_t>(k) * kThreads;
            if (it >= D.cols) break;
            Pack<OutT>::one(D.dst + it * sizeof(OutT), src[it]);
        }
    }
}

__device__ __forceinline__ void copy_zero_tile(const DescDev& D, int64_t local_tile, bool vec, bool zero) {
    const int64_t i0 = local_tile * kTileItems;
    if (vec) {
        const int64_t items = D.cols / 16;
        for (int k = 0; k < kTileItems / kThreads; ++k) {
            const int64_t it = i0 + threadIdx.x + static_cast<int64_t>(k) * kThreads;
            if (it >= items) break;
            uint4 v = make_uint4(0, 0, 0, 0);
            if (!zero) v = *reinterpret_cast<const uint4*>(D.src + it * 16);
            store16(D.dst + it * 16, v);
        }
    } else {
        for (int k = 0; k < kTileItems / kThreads; ++k) {
            const int64_t it = i0 + threadIdx.x + static_cast<int64_t>(k) * kThreads;
            if (it >= D.cols) break;
            D.dst[it] = zero ? uint8_t(0) : D.src[it];
        }
    }
}

// ── the kernel ───────────────────────────────────────────────────────────

template <typename OutT, bool GridStride, int Segs, bool Bulk = false>
__global__ void __launch_bounds__(kThreads, (GridStride || Segs != kSegsPerThread) ? kDeepMinCtasPerSm : SQ_MIN_CTAS_PER_SM)
sq_block_kernel(const __grid_constant__ BlockPlan plan, int32_t* status) {
    __shared__ alignas(16) float s_scale[kSmemRows];
    __shared__ alignas(16) float s_zp[kSmemRows];
    __shared__ alignas(8) uint64_t s_bar;
    // landing area of a tile fetched from a peer GPU with one bulk copy (the Bulk instantiation only)
    __shared__ alignas(128) int4 s_tile[Bulk ? kThreads * Segs : 1];

    // One tile per CTA when the grid covers the launch; a capped grid (launches that read a peer GPU's
    // memory, see launch_plan) walks the tiles grid-stride.  Only a CTA with a single tile stages scales
    // through shared memory: the barrier is initialised once per CTA.
    const uint32_t total = static_cast<uint32_t>(plan.total_tiles);
    constexpr bool single = !GridStride;
    for (uint32_t work = blockIdx.x; work < total; work += GridStride ? gridDim.x : total) {
    const uint32_t tile = plan.tile_stride == 1u
                              ? work
                              : static_cast<uint32_t>((static_cast<uint64_t>(work) * plan.tile_stride) % total);
    // descriptor of this tile: the last d with tile_begin[d] <= tile (binary search, uniform across the CTA)
    int d = 0;
    for (int hi = plan.n_desc; hi - d > 1;) {
        const int mid = (d + hi) >> 1;
        if (tile >= plan.tile_begin[mid]) d = mid; else hi = mid;
    }
    const DescDev& D = plan.d[d];
    const int64_t local_tile = static_cast<int64_t>(tile - plan.tile_begin[d]);

    switch (D.path) {
        case kPathDequantVec:
            if (D.flags & kFlagDense) {
                if (D.zp != nullptr) dequant_vec_tile<OutT, true, true, Segs, Bulk>(D, local_tile, s_scale, s_zp, &s_bar, status, single, s_tile);
                else                 dequant_vec_tile<OutT, false, true, Segs, Bulk>(D, local_tile, s_scale, s_zp, &s_bar, status, single, s_tile);
            } else {
                if (D.zp != nullptr) dequant_vec_tile<OutT, true, false, Segs>(D, local_tile, s_scale, s_zp, &s_bar, status, single);
                else                 dequant_vec_tile<OutT, false, false, Segs>(D, local_tile, s_scale, s_zp, &s_bar, status, single);
            }
            break;
        case kPathDequantScalar: dequant_scalar_tile<OutT>(D, local_tile); break;
        case kPathCastVec:       cast_tile<OutT>(D, local_tile, true); break;
        case kPathCastScalar:    cast_tile<OutT>(D, local_tile, false); break;
        case kPathCopyVec:       copy_zero_tile(D, local_tile, true, false); break;
        case kPathCopyScalar:    copy_zero_tile(D, local_tile, false, false); break;
        case kPathZeroVec:       copy_zero_tile(D, local_tile, true, true); break;
        case kPathZeroScalar:    copy_zero_tile(D, local_tile, false, true); break;
        default:
            if (threadIdx.x == 0 && status != nullptr) atomicOr(status, kStatusBadPath);
            break;
    }
    }
}

// CTAs per SM a launch that reads another GPU's memory may occupy (0 = no cap).  Such a launch runs at the
// pace of the NVLink reads, several times longer than a local one; left uncapped it holds every thread slot
// of every SM for that time and the model's own kernels queue behind it.
static std::atomic<int> g_peer_ctas_per_sm{0};
static std::atomic<int> g_sm_count{0};
static std::atomic<bool> g_peer_deep{false};
static std::atomic<bool> g_peer_bulk{false};

void set_peer_bulk_loads(bool on) { g_peer_bulk.store(on); }
bool peer_bulk_loads() { return g_peer_bulk.load(); }

void set_peer_deep_loads(bool on) { g_peer_deep.store(on); }
bool peer_deep_loads() { return g_peer_deep.load(); }

void set_peer_ctas_per_sm(int n) { g_peer_ctas_per_sm.store(n < 0 ? 0 : n); }
int peer_ctas_per_sm() { return g_peer_ctas_per_sm.load(); }

static int sm_count() {
    int n = g_sm_count.load();
    if (n == 0) {
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
            n = 148;
        g_sm_count.store(n);
    }
    return n;
}

cudaError_t launch_plan(const BlockPlan& plan, int out_dtype, cudaStream_t stream, int32_t* status_dev) {
    if (plan.total_tiles <= 0) return cudaSuccess;
    unsigned ctas = static_cast<unsigned>(plan.total_tiles);
    const int cap = g_peer_ctas_per_sm.load();
    if (cap > 0 && plan.tile_stride != 1u) {     // a scattered launch is one that reads peer memory
        const unsigned limit = static_cast<unsigned>(cap) * static_cast<unsigned>(sm_count());
        if (ctas > limit) ctas = limit;
    }
    const dim3 grid(ctas), block(kThreads);
    const bool stride = ctas < static_cast<unsigned>(plan.total_tiles);
    const bool deep = plan.segs_per_thread == static_cast<uint32_t>(kDeepSegsPerThread);
    const bool bulk = plan.bulk_peer != 0 && !deep && !stride;
#define SQ_LAUNCH(T)                                                                                              \
    do {                                                                                                          \
        if (bulk)            sq_block_kernel<T, false, kSegsPerThread, true><<<grid, block, 0, stream>>>(plan, status_dev); \
        else if (deep && stride)  sq_block_kernel<T, true, kDeepSegsPerThread><<<grid, block, 0, stream>>>(plan, status_dev);   \
        else if (deep)       sq_block_kernel<T, false, kDeepSegsPerThread><<<grid, block, 0, stream>>>(plan, status_dev);  \
        else if (stride)     sq_block_kernel<T, true, kSegsPerThread><<<grid, block, 0, stream>>>(plan, status_dev);       \
        else                 sq_block_kernel<T, false, kSegsPerThread><<<grid, block, 0, stream>>>(plan, status_dev);      \
    } while (0)
    switch (out_dtype) {
        case SH_DT_BF16: SQ_LAUNCH(__nv_bfloat16); break;
        case SH_DT_F16:  SQ_LAUNCH(__half); break;
        case SH_DT_F32:  SQ_LAUNCH(float); break;
        default: return cudaErrorInvalidValue;
    }
#undef SQ_LAUNCH
    return cudaGetLastError();
}

// ── host-side plan builder ───────────────────────────────────────────────

static inline bool aligned(const void* p, uintptr_t a) { return (reinterpret_cast<uintptr_t>(p) % a) == 0; }

static inline int64_t ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }

// [off, off + len) lies inside [0, total): written so that no sum can overflow, whatever the caller passes
static inline bool in_range(int64_t off, int64_t len, int64_t total) {
    return off >= 0 && len >= 0 && off <= total && len <= total - off;
}

constexpr int64_t kMaxCount = int64_t(1) << 40;     // rows x cols, row strides and vector lengths stay below this

static uint32_t gcd_u32(uint32_t a, uint32_t b) {
    while (b != 0) {
        const uint32_t t = a % b;
        a = b;
        b = t;
    }
    return a;
}

// Finishes a plan: total tile count and the CTA -> tile stride.  Launches that read another GPU's memory
// use a stride near total / golden ratio (coprime with total, so the mapping is a permutation).
static void close_plan(BlockPlan& plan, uint32_t tiles) {
    plan.tile_begin[plan.n_desc] = tiles;
    plan.total_tiles = static_cast<int32_t>(tiles);
    plan.tile_stride = 1;
    bool remote = false;
    for (int i = 0; i < plan.n_desc; ++i) remote = remote || (plan.d[i].flags & SH_DESC_PEER_SOURCE) != 0;
    if (remote && tiles > 64) {
        uint32_t stride = static_cast<uint32_t>(static_cast<double>(tiles) * 0.6180339887);
        while (stride > 1 && gcd_u32(stride, tiles) != 1) --stride;
        plan.tile_stride = stride > 1 ? stride : 1;
    }
}

void rebase_plan(BlockPlan& plan, const void* packed_base, void* out_base) {
    const ptrdiff_t dp = static_cast<const uint8_t*>(packed_base) - static_cast<const uint8_t*>(kPlanStandInBase);
    const ptrdiff_t dq = static_cast<uint8_t*>(out_base) - static_cast<uint8_t*>(kPlanStandInBase);
    for (int i = 0; i < plan.n_desc; ++i) {
        DescDev& D = plan.d[i];
        if (D.flags & kFlagRelative) {
            if (D.src != nullptr) D.src += dp;
            if (D.scale != nullptr) D.scale = reinterpret_cast<const float*>(reinterpret_cast<const uint8_t*>(D.scale) + dp);
            if (D.zp != nullptr) D.zp = reinterpret_cast<const float*>(reinterpret_cast<const uint8_t*>(D.zp) + dp);
        }
        D.dst += dq;
    }
}

int build_plans(const ShParamDesc* descs, int n, const void* packed, size_t packed_bytes, void* out,
                size_t out_bytes, int out_dtype, BlockPlan* plans_out, int* n_plans_out, int64_t* elements_out,
                int64_t* traffic_bytes_out, char* err, size_t err_len) {
    const int64_t osz = out_dtype == SH_DT_F32 ? 4 : 2;
    if (out_dtype != SH_DT_BF16 && out_dtype != SH_DT_F16 && out_dtype != SH_DT_F32) {
        snprintf(err, err_len, "unknown out_dtype %d", out_dtype);
        return SH_ERR_INVALID_ARG;
    }
    const uint8_t* pbase = static_cast<const uint8_t*>(packed);
    uint8_t* obase = static_cast<uint8_t*>(out);
    const int64_t pbytes = static_cast<int64_t>(packed_bytes);
    const int64_t obytes = static_cast<int64_t>(out_bytes);
    int64_t elements = 0, traffic = 0;
    int n_plans = 0;
    BlockPlan* plan = nullptr;
    uint32_t tiles = 0;
    // every plan of one call uses one tile size: the deep variant when it is switched on and the block reads peer memory
    bool reads_peer = false;
    for (int i = 0; i < n; ++i) reads_peer = reads_peer || (descs[i].flags & SH_DESC_PEER_SOURCE) != 0;
    const int segs = (reads_peer && peer_deep_loads()) ? kDeepSegsPerThread : kSegsPerThread;
    const int64_t tile_segs = static_cast<int64_t>(kThreads) * segs;

    for (int i = 0; i < n; ++i) {
        const ShParamDesc& u = descs[i];
        if (plan == nullptr || plan->n_desc == kMaxDescs) {
            if (plan != nullptr) close_plan(*plan, tiles);
            plan = &plans_out[n_plans++];
            memset(plan, 0, sizeof(BlockPlan));
            plan->segs_per_thread = static_cast<uint32_t>(segs);
            plan->bulk_peer = (reads_peer && peer_bulk_loads() && segs == kSegsPerThread) ? 1u : 0u;
            tiles = 0;
        }
        DescDev D;
        memset(&D, 0, sizeof(D));
        D.flags = u.flags & SH_DESC_PEER_SOURCE;
        const bool absolute = (u.flags & SH_DESC_ABSOLUTE) != 0;
        if (!absolute && u.kind != SH_KIND_ZERO) D.flags |= kFlagRelative;
        int64_t dst_bytes = 0, n_tiles = 0;
#define SQ_FAIL(...)                                      \
    do {                                                  \
        snprintf(err, err_len, __VA_ARGS__);              \
        return SH_ERR_INVALID_ARG;                        \
    } while (0)
        if (u.dst_off < 0 || u.dst_off > obytes) SQ_FAIL("descriptor %d: dst_off negative or beyond the output slab", i);
        switch (u.kind) {
            case SH_KIND_DEQUANT_I8: {
                if (u.rows <= 0 || u.cols <= 0 || u.ld < u.cols) SQ_FAIL("descriptor %d: bad rows/cols/ld", i);
                if (u.rows > kMaxCount / u.cols || u.ld > kMaxCount / u.rows) SQ_FAIL("descriptor %d: matrix too large", i);
                if (absolute) {
                    if (u.src_off <= 0 || u.scale_off <= 0 || u.zp_off == 0)
                        SQ_FAIL("descriptor %d: null absolute source address", i);
                    D.src = reinterpret_cast<const uint8_t*>(static_cast<uintptr_t>(u.src_off));
                    D.scale = reinterpret_cast<const float*>(static_cast<uintptr_t>(u.scale_off));
                    D.zp = u.zp_off > 0 ? reinterpret_cast<const float*>(static_cast<uintptr_t>(u.zp_off)) : nullptr;
                } else {
                    if (!in_range(u.src_off, (u.rows - 1) * u.ld + u.cols, pbytes))
                        SQ_FAIL("descriptor %d: int8 rows outside the packed image", i);
                    if (u.scale_off % 4 != 0 || !in_range(u.scale_off, u.rows * 4, pbytes))
                        SQ_FAIL("descriptor %d: scales outside the packed image or not 4-byte aligned", i);
                    if (u.zp_off >= 0 && (u.zp_off % 4 != 0 || !in_range(u.zp_off, u.rows * 4, pbytes)))
                        SQ_FAIL("descriptor %d: zero points outside the packed image or not 4-byte aligned", i);
                    D.src = pbase + u.src_off;
                    D.scale = reinterpret_cast<const float*>(pbase + u.scale_off);
                    D.zp = u.zp_off >= 0 ? reinterpret_cast<const float*>(pbase + u.zp_off) : nullptr;
                }
                dst_bytes = u.rows * u.cols * osz;
                if (!aligned(D.scale, 4) || (D.zp && !aligned(D.zp, 4)))
                    SQ_FAIL("descriptor %d: scale pointer not 4-byte aligned", i);
                D.rows = u.rows; D.cols = u.cols; D.ld = u.ld;
                const bool vec = (u.cols % kSegBytes == 0) && (u.ld % kSegBytes == 0) && aligned(D.src, 16) &&
                                 aligned(obase + u.dst_off, 16) && (u.cols / kSegBytes) < (int64_t(1) << 30);
                if (vec) {
                    D.path = kPathDequantVec;
                    D.segs_per_row = static_cast<int32_t>(u.cols / kSegBytes);
                    n_tiles = ceil_div(u.rows * D.segs_per_row, tile_segs);
                    // bulk scale fetch: 16-byte aligned arrays whose 4-row padding stays inside the image
                    const int64_t rows4 = (u.rows + 3) & ~int64_t(3);
                    const bool bulk_ok = !absolute && !(D.flags & SH_DESC_PEER_SOURCE) && aligned(D.scale, 16) &&
                                         in_range(u.scale_off, rows4 * 4, pbytes) &&
                                         (D.zp == nullptr || (aligned(D.zp, 16) && in_range(u.zp_off, rows4 * 4, pbytes)));
                    if (bulk_ok) D.flags |= kFlagBulkScales;
                    if (osz == 2 && aligned(obase + u.dst_off, 32)) D.flags |= kFlagStore32;
                    if (u.ld == u.cols) D.flags |= kFlagDense;
                    const uint64_t spr64 = static_cast<uint64_t>(D.segs_per_row);
                    // valid for every in-tile index of the larger (deep) tile, hence of both
                    D.row_magic = ((spr64 + kThreads * kDeepSegsPerThread) * spr64 < (uint64_t(1) << 32))
                                      ? ((uint64_t(1) << 32) / spr64 + 1) : 0;
                } else {
                    D.path = kPathDequantScalar;
                    n_tiles = ceil_div(u.rows * u.cols, kTileItems);
                }
                elements += u.rows * u.cols;
                traffic += u.rows * u.cols * (1 + osz) + u.rows * (D.zp ? 8 : 4);
                break;
            }
            case SH_KIND_CAST_F32: {
                if (u.cols < 0 || u.cols > kMaxCount) SQ_FAIL("descriptor %d: negative or oversized count", i);
                if (!absolute && (u.src_off % 4 != 0 || !in_range(u.src_off, u.cols * 4, pbytes)))
                    SQ_FAIL("descriptor %d: fp32 source outside the packed image or not 4-byte aligned", i);
                if (absolute && u.src_off <= 0) SQ_FAIL("descriptor %d: null absolute source address", i);
                dst_bytes = u.cols * osz;
                D.src = absolute ? reinterpret_cast<const uint8_t*>(static_cast<uintptr_t>(u.src_off)) : pbase + u.src_off;
                if (!aligned(D.src, 4)) SQ_FAIL("descriptor %d: fp32 source pointer not 4-byte aligned", i);
                D.rows = 1; D.cols = u.cols;
                const bool vec = (u.cols % 4 == 0) && aligned(D.src, 16) && aligned(obase + u.dst_off, 4 * osz);
                D.path = vec ? kPathCastVec : kPathCastScalar;
                n_tiles = ceil_div(vec ? u.cols / 4 : u.cols, kTileItems);
                traffic += u.cols * (4 + osz);
                break;
            }
            case SH_KIND_COPY:
            case SH_KIND_ZERO: {
                if (u.cols < 0 || u.cols > kMaxCount) SQ_FAIL("descriptor %d: negative or oversized byte count", i);
                const bool zero = u.kind == SH_KIND_ZERO;
                if (!zero && !absolute && !in_range(u.src_off, u.cols, pbytes))
                    SQ_FAIL("descriptor %d: copy source outside the packed image", i);
                if (!zero && absolute && u.src_off <= 0) SQ_FAIL("descriptor %d: null absolute source address", i);
                dst_bytes = u.cols;
                D.src = zero ? nullptr
                             : (absolute ? reinterpret_cast<const uint8_t*>(static_cast<uintptr_t>(u.src_off)) : pbase + u.src_off);
                D.rows = 1; D.cols = u.cols;
                const bool vec = (u.cols % 16 == 0) && aligned(obase + u.dst_off, 16) && (zero || aligned(D.src, 16));
                D.path = zero ? (vec ? kPathZeroVec : kPathZeroScalar) : (vec ? kPathCopyVec : kPathCopyScalar);
                n_tiles = ceil_div(vec ? u.cols / 16 : u.cols, kTileItems);
                traffic += u.cols * (zero ? 1 : 2);
                break;
            }
            default:
                SQ_FAIL("descriptor %d: unknown kind %d", i, u.kind);
        }
        if (u.kind != SH_KIND_COPY && u.kind != SH_KIND_ZERO && !aligned(obase + u.dst_off, osz))
            SQ_FAIL("descriptor %d: destination not aligned to the element size", i);
        if (!in_range(u.dst_off, dst_bytes, obytes)) SQ_FAIL("descriptor %d: destination outside the output slab", i);
        if (tiles + static_cast<uint64_t>(n_tiles) > 0x7FFFFFFFull) SQ_FAIL("descriptor %d: too many tiles", i);
#undef SQ_FAIL
        D.dst = obase + u.dst_off;
        plan->tile_begin[plan->n_desc] = tiles;
        plan->d[plan->n_desc] = D;
        plan->n_desc += 1;
        tiles += static_cast<uint32_t>(n_tiles);
    }
    if (plan != nullptr) close_plan(*plan, tiles);
    *n_plans_out = n_plans;
    if (elements_out) *elements_out = elements;
    if (traffic_bytes_out) *traffic_bytes_out = traffic;
    return SH_OK;
}

}  // namespace sq
