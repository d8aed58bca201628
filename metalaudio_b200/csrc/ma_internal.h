// Internal host-side declarations shared by the translation units of the library.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>

#include "../../include/metalaudio_cuda.h"

constexpr int kAuxStreams = 3;

struct ma_context {
    int device = 0;
    int sm_count = 0;
    cudaStream_t stream = nullptr;
    cudaStream_t copy_stream = nullptr;   // host -> device leg of the pipelined *_host calls
    cudaStream_t d2h_stream = nullptr;    // device -> host leg
    // Further lanes of the large transforms: chunks of a batch rotate over `stream` and these, forked
    // from and joined back to `stream` inside each call.
    cudaStream_t aux_stream[kAuxStreams] = {};
    cudaEvent_t ev_fork = nullptr, ev_join[kAuxStreams] = {};
    // Device workspace of the *_host calls: two lanes of ws_lane_bytes each, allocated once
    // (ma_context_reserve_workspace or the first *_host call) and grown only when a single row
    // does not fit.  Lane events: input copied, kernels done, output copied.
    char* ws = nullptr;
    size_t ws_lane_bytes = 0;
    cudaEvent_t ev_in[2] = {nullptr, nullptr}, ev_k[2] = {nullptr, nullptr}, ev_out[2] = {nullptr, nullptr};
    void* pinned = nullptr;       // staging buffer, used as two halves
    size_t pinned_bytes = 0;
    cudaEvent_t ev_half[2] = {nullptr, nullptr};
    cudaEvent_t ev_begin = nullptr, ev_end = nullptr, ev_sync = nullptr;
    bool timing_open = false;
    bool lost = false;
    int fault_site = -1;          // host-side fault injection: next call reaching the site fails
    int fault_error = 0;
    char name[256] = {0};
    int32_t* d_error_flag = nullptr;  // set by a kernel whose bounded wait ran out
    int32_t* h_error_flag = nullptr;  // pinned mirror read at synchronisation
    // Output rows of the latest convolution streaming step on this context (any object): the next
    // step's first kernel may overlap that step's last one unless it reads these rows.
    const float* step_out = nullptr;
    const float* step_out_end = nullptr;
    // Kernels this context has queued, and the count right after the latest streaming step's last
    // kernel: equal when nothing else of the library was queued on the stream since that step.
    uint64_t launch_seq = 0;
    uint64_t step_end_seq = UINT64_MAX;
};

namespace ma {

extern std::atomic<uint64_t> g_launch_count;
extern thread_local int32_t t_last_cuda_error;

// Records a CUDA error for ma_last_cuda_error and maps it to a status.
ma_status cuda_fail(cudaError_t e);
// Returns MA_OK, MA_ERR_DEVICE_LOST, or an injected fault for `site`; makes the
// context's device current.
ma_status enter(ma_context* ctx, int site);
// Checks the launch error of the kernel just queued and counts it.
ma_status after_launch(ma_context* ctx);

// Host <-> device copies through the context (direct for pinned memory, staged
// through the pinned buffer otherwise).  Synchronous with respect to the host buffer.
ma_status copy_h2d(ma_context* ctx, void* dptr, const void* host, size_t bytes);
ma_status copy_d2h(ma_context* ctx, void* host, const void* dptr, size_t bytes);

// True when the pointer is page-locked host memory the runtime knows (cudaHostAlloc / registered).
bool is_pinned(const void* p);
// Makes sure the context's two workspace lanes hold at least `min_lane_bytes` each (grow-only; a
// growth waits for all queued work first).  Returns the lanes.
ma_status workspace_lanes(ma_context* ctx, size_t min_lane_bytes, char** lane0, char** lane1, size_t* lane_bytes);

// Stream-ordered temporary device memory for the *_host entry points.
ma_status temp_alloc(ma_context* ctx, size_t bytes, void** dptr);
void temp_free(ma_context* ctx, void* dptr);

}  // namespace ma

#define MA_CUDA(expr)                                         \
    do {                                                      \
        cudaError_t _e = (expr);                              \
        if (_e != cudaSuccess) return ::ma::cuda_fail(_e);    \
    } while (0)

#define MA_TRY(expr)                         \
    do {                                     \
        ma_status _s = (expr);               \
        if (_s != MA_OK) return _s;          \
    } while (0)
