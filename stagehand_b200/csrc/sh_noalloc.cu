// sh_dequant_from_host_noalloc: the host-image entry point for callers that must not allocate.
//
// Some hosts of this library cannot call cudaMalloc on the path that delivers weights: code that
// runs after the process has handed all device memory to another allocator (an inference server
// that pre-reserves the whole GPU at start-up), code inside a latency-critical loop where an
// allocation would synchronise the device, or a plug-in that is forbidden to grow the process's
// footprint after initialisation.  sh_stream_block_async needs a device staging slab that somebody
// allocated; this variant brings its own: a fixed array in the library's device image.  Every GPU
// that loads the library holds SH_NOALLOC_MAX_BYTES of it until the process exits.
//
// When is that memory taken?  CUDA loads a library's device image on a GPU the first time something in it
// is used there, and the array comes with the image.  sh_init() resolves the array's address, so a process
// that calls sh_init on each device before it gives its VRAM away has paid for the array by then; a process
// that skips sh_init pays at this entry point's first call on the device, which can fail for lack of memory.
#include "sh_common.h"

#include <cstdio>
#include <cstring>
#include <mutex>

namespace {

// The scratch: where the packed image lands before the block kernel expands it.
static __device__ __align__(256) unsigned char g_noalloc_staging[SH_NOALLOC_MAX_BYTES];

constexpr int kMaxDevices = 64;
constexpr int kMaxPlans = 1;                 // one launch plan (128 descriptors) per call, on the stack
std::mutex g_setup_mu;
void* g_staging_ptr[kMaxDevices] = {nullptr};

thread_local char g_noalloc_err[256] = "";

// Device address of the array on the current device.  In host code the array's name is only a
// stand-in for the symbol, not a device address, so it is resolved once per device.
int staging_address(void** out) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
        snprintf(g_noalloc_err, sizeof(g_noalloc_err), "cudaGetDevice failed or device index out of range (%d)", dev);
        return SH_ERR_CUDA;
    }
    std::lock_guard<std::mutex> lk(g_setup_mu);
    if (g_staging_ptr[dev] == nullptr) {
        void* ptr = nullptr;
        e = cudaGetSymbolAddress(&ptr, g_noalloc_staging);
        if (e != cudaSuccess || ptr == nullptr) {
            snprintf(g_noalloc_err, sizeof(g_noalloc_err), "cudaGetSymbolAddress: %s", cudaGetErrorString(e));
            return SH_ERR_CUDA;
        }
        g_staging_ptr[dev] = ptr;
    }
    *out = g_staging_ptr[dev];
    return SH_OK;
}

}  // namespace

int shc::noalloc_prepare_current_device(char* err, size_t err_len) {
    void* ptr = nullptr;
    const int rc = staging_address(&ptr);
    if (rc != SH_OK && err != nullptr && err_len > 0) snprintf(err, err_len, "%s", g_noalloc_err);
    return rc;
}

extern "C" {

int32_t sh_noalloc_last_error(char* buf, int32_t buf_len) {
    const int32_t n = static_cast<int32_t>(strlen(g_noalloc_err));
    if (buf != nullptr && buf_len > 0) {
        const int32_t c = n < buf_len - 1 ? n : buf_len - 1;
        memcpy(buf, g_noalloc_err, static_cast<size_t>(c));
        buf[c] = '\0';
    }
    return n;
}

int32_t sh_dequant_from_host_noalloc(const ShParamDesc* descs, int32_t n_descs, const void* packed_host,
                                     size_t packed_bytes, void* out_dev, size_t out_bytes, int32_t out_dtype,
                                     uint64_t stream, int32_t* status_dev) {
    g_noalloc_err[0] = '\0';
    if (n_descs < 0 || (n_descs > 0 && descs == nullptr) || packed_host == nullptr || out_dev == nullptr) {
        snprintf(g_noalloc_err, sizeof(g_noalloc_err), "null argument");
        return SH_ERR_INVALID_ARG;
    }
    if (packed_bytes > static_cast<size_t>(SH_NOALLOC_MAX_BYTES)) {
        snprintf(g_noalloc_err, sizeof(g_noalloc_err),
                 "packed image of %zu bytes exceeds the built-in staging area of %d bytes (SH_NOALLOC_MAX_BYTES); "
                 "use sh_stream_block_async with a staging slab of your own",
                 packed_bytes, SH_NOALLOC_MAX_BYTES);
        return SH_ERR_INVALID_ARG;
    }
    if (n_descs > kMaxPlans * sq::kMaxDescs) {
        snprintf(g_noalloc_err, sizeof(g_noalloc_err), "%d descriptors exceed the limit of %d for this entry point",
                 n_descs, kMaxPlans * sq::kMaxDescs);
        return SH_ERR_INVALID_ARG;
    }
    if (n_descs == 0) return SH_OK;

    void* staging = nullptr;
    int rc = staging_address(&staging);
    if (rc != SH_OK) return rc;

    sq::BlockPlan plans[kMaxPlans];
    int n_plans = 0;
    int64_t elements = 0;
    rc = sq::build_plans(descs, n_descs, staging, packed_bytes, out_dev, out_bytes, out_dtype, plans, &n_plans, &elements,
                         nullptr, g_noalloc_err, sizeof(g_noalloc_err));
    if (rc != SH_OK) return rc;

    cudaStream_t s = reinterpret_cast<cudaStream_t>(static_cast<uintptr_t>(stream));
    cudaError_t e = cudaMemcpyAsync(staging, packed_host, packed_bytes, cudaMemcpyHostToDevice, s);
    if (e != cudaSuccess) {
        snprintf(g_noalloc_err, sizeof(g_noalloc_err), "cudaMemcpyAsync: %s", cudaGetErrorString(e));
        return SH_ERR_CUDA;
    }
    for (int p = 0; p < n_plans; ++p) {
        e = sq::launch_plan(plans[p], out_dtype, s, status_dev);   // the plans carry the staging address to the kernel
        if (e != cudaSuccess) {
            snprintf(g_noalloc_err, sizeof(g_noalloc_err), "block kernel launch: %s", cudaGetErrorString(e));
            return SH_ERR_CUDA;
        }
        shc::g_ctr.launches.fetch_add(1, std::memory_order_relaxed);
    }
    shc::g_ctr.elements.fetch_add(elements, std::memory_order_relaxed);
    shc::g_ctr.h2d_copies.fetch_add(1, std::memory_order_relaxed);
    shc::g_ctr.h2d_bytes.fetch_add(static_cast<int64_t>(packed_bytes), std::memory_order_relaxed);
    return SH_OK;
}

}  // extern "C"
