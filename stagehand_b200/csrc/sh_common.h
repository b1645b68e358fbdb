// Pieces shared by the translation units of the C ABI: the per-thread error text, the counters behind
// sh_stats, the launcher that brackets block-kernel launches with profiling events, and the hook that
// makes the allocation-free entry point's device array resident at sh_init.
#pragma once

#include <atomic>
#include <cstdint>
#include <cuda_runtime.h>

#include "../../include/stagehand_b200.h"
#include "sq_block_kernel.cuh"

namespace shc {

// Sets the calling thread's error text (read back with sh_last_error) and returns `code`.
int fail(int code, const char* fmt, ...);
int cuda_fail(cudaError_t e, const char* what);

#define SH_CUDA(call, what)                                        \
    do {                                                           \
        cudaError_t e__ = (call);                                  \
        if (e__ != cudaSuccess) return ::shc::cuda_fail(e__, what); \
    } while (0)

inline cudaStream_t as_stream(uint64_t s) { return reinterpret_cast<cudaStream_t>(static_cast<uintptr_t>(s)); }
inline cudaEvent_t as_event(uint64_t e) { return reinterpret_cast<cudaEvent_t>(static_cast<uintptr_t>(e)); }

struct Counters {
    std::atomic<int64_t> launches{0}, elements{0}, h2d_copies{0}, h2d_bytes{0}, peer_copies{0}, peer_bytes{0},
        status_errors{0};
};
extern Counters g_ctr;

// Launches `n_plans` plans of one block on `stream` (counted in sh_stats; bracketed by timing events while
// sh_profile_enable is on).  `elements` / `traffic` describe the whole block.
int launch_plans(const sq::BlockPlan* plans, int n_plans, int64_t elements, int64_t traffic, int out_dtype,
                 cudaStream_t stream, int32_t* status_dev);

// While sh_profile_enable is on: brackets the copies of one block load with timing events on `stream`.
// copy_timing_begin returns false (and sets nothing) when profiling is off.
bool copy_timing_begin(cudaStream_t stream, cudaEvent_t* start_out, cudaEvent_t* stop_out);
void copy_timing_end(cudaStream_t stream, cudaEvent_t start, cudaEvent_t stop, int64_t bytes);
void copy_timing_abandon(cudaEvent_t start, cudaEvent_t stop);      // the load failed: the events go back unused

// Brackets the copies of one sh_block_load; whatever path the function leaves by, the events are accounted for.
struct CopyTiming {
    cudaStream_t stream = nullptr;
    cudaEvent_t start = nullptr, stop = nullptr;
    bool open = false;
    void begin(cudaStream_t s) { stream = s; open = copy_timing_begin(s, &start, &stop); }
    void end(int64_t bytes) { if (open) { copy_timing_end(stream, start, stop, bytes); open = false; } }
    ~CopyTiming() { if (open) copy_timing_abandon(start, stop); }
};

// Polls an event until done or until the deadline; never blocks without bound.
int wait_event_bounded(cudaEvent_t ev, int timeout_ms);

// sh_noalloc.cu: resolves the device address of the built-in staging array on the current device, which
// also makes the CUDA module that holds it resident.  Returns SH_OK or SH_ERR_CUDA (text in `err`).
int noalloc_prepare_current_device(char* err, size_t err_len);

}  // namespace shc
