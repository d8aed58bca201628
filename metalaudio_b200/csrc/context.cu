// CUDA device / stream context, buffers, staging copies, timing and host-side fault
// injection: the slice of AudioDevice / ComputeContext / Tensor the DSP hot path needs.
#include <chrono>
#include <cstring>
#include <new>
#include <thread>

#include "bulk_copy.cuh"
#include "ma_internal.h"

namespace ma {

std::atomic<uint64_t> g_launch_count{0};
thread_local int32_t t_last_cuda_error = 0;

ma_status cuda_fail(cudaError_t e) {
    t_last_cuda_error = (int32_t)e;
    (void)cudaGetLastError();  // clear the sticky-less error state
    if (e == cudaErrorMemoryAllocation) return MA_ERR_ALLOC;
    if (e == cudaErrorNoDevice || e == cudaErrorInvalidDevice || e == cudaErrorInsufficientDriver)
        return MA_ERR_DEVICE_LOST;
    return MA_ERR_CUDA;
}

static ma_status injected(ma_context* ctx) {
    const int err = ctx->fault_error;
    const int site = ctx->fault_site;
    ctx->fault_site = -1;
    ctx->fault_error = 0;
    if (site == MA_FAULT_DEVICE_LOST) {
        ctx->lost = true;
        return MA_ERR_DEVICE_LOST;
    }
    return cuda_fail((cudaError_t)err);
}

ma_status enter(ma_context* ctx, int site) {
    if (ctx == nullptr) return MA_ERR_INVALID_ARGUMENT;
    if (ctx->lost) return MA_ERR_DEVICE_LOST;
    if (ctx->fault_site >= 0 && (ctx->fault_site == site || ctx->fault_site == MA_FAULT_DEVICE_LOST))
        return injected(ctx);
    MA_CUDA(cudaSetDevice(ctx->device));
    return MA_OK;
}

ma_status after_launch(ma_context* ctx) {
    if (ctx != nullptr) ++ctx->launch_seq;
    g_launch_count.fetch_add(1, std::memory_order_relaxed);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return cuda_fail(e);
    return MA_OK;
}

bool is_pinned(const void* p) {
    cudaPointerAttributes a;
    cudaError_t e = cudaPointerGetAttributes(&a, p);
    if (e != cudaSuccess) {
        (void)cudaGetLastError();
        return false;
    }
    return a.type == cudaMemoryTypeHost;
}

ma_status copy_h2d(ma_context* ctx, void* dptr, const void* host, size_t bytes) {
    if (bytes == 0) return MA_OK;
    if (is_pinned(host)) {
        MA_CUDA(cudaMemcpyAsync(dptr, host, bytes, cudaMemcpyHostToDevice, ctx->stream));
        MA_CUDA(cudaStreamSynchronize(ctx->stream));
        return MA_OK;
    }
    const size_t half = ctx->pinned_bytes / 2;
    size_t off = 0;
    int h = 0;
    while (off < bytes) {
        const size_t n = bytes - off < half ? bytes - off : half;
        char* stage = (char*)ctx->pinned + (size_t)h * half;
        MA_CUDA(cudaEventSynchronize(ctx->ev_half[h]));
        std::memcpy(stage, (const char*)host + off, n);
        MA_CUDA(cudaMemcpyAsync((char*)dptr + off, stage, n, cudaMemcpyHostToDevice, ctx->stream));
        MA_CUDA(cudaEventRecord(ctx->ev_half[h], ctx->stream));
        off += n;
        h ^= 1;
    }
    MA_CUDA(cudaStreamSynchronize(ctx->stream));
    return MA_OK;
}

ma_status copy_d2h(ma_context* ctx, void* host, const void* dptr, size_t bytes) {
    if (bytes == 0) return MA_OK;
    if (is_pinned(host)) {
        MA_CUDA(cudaMemcpyAsync(host, dptr, bytes, cudaMemcpyDeviceToHost, ctx->stream));
        MA_CUDA(cudaStreamSynchronize(ctx->stream));
        return MA_OK;
    }
    const size_t half = ctx->pinned_bytes / 2;
    size_t off = 0, prev_off = 0, prev_n = 0;
    int h = 0;
    bool have_prev = false;
    while (off < bytes || have_prev) {
        size_t n = 0;
        if (off < bytes) {
            n = bytes - off < half ? bytes - off : half;
            char* stage = (char*)ctx->pinned + (size_t)h * half;
            MA_CUDA(cudaMemcpyAsync(stage, (const char*)dptr + off, n, cudaMemcpyDeviceToHost, ctx->stream));
            MA_CUDA(cudaEventRecord(ctx->ev_half[h], ctx->stream));
        }
        if (have_prev) {  // drain the other half while this one is in flight
            MA_CUDA(cudaEventSynchronize(ctx->ev_half[h ^ 1]));
            std::memcpy((char*)host + prev_off, (char*)ctx->pinned + (size_t)(h ^ 1) * half, prev_n);
            have_prev = false;
        }
        if (n > 0) {
            prev_off = off;
            prev_n = n;
            have_prev = true;
            off += n;
            h ^= 1;
        }
    }
    return MA_OK;
}

ma_status workspace_lanes(ma_context* ctx, size_t min_lane_bytes, char** lane0, char** lane1, size_t* lane_bytes) {
    constexpr size_t kDefaultLane = (size_t)256 << 20;
    if (ctx->ws == nullptr || ctx->ws_lane_bytes < min_lane_bytes) {
        if (ctx->fault_site == MA_FAULT_ALLOC) return injected(ctx);
        size_t want = ctx->ws == nullptr && min_lane_bytes < kDefaultLane ? kDefaultLane : min_lane_bytes;
        want = (want + 255) & ~(size_t)255;
        if (ctx->ws != nullptr) {
            MA_CUDA(cudaDeviceSynchronize());
            (void)cudaFree(ctx->ws);
            ctx->ws = nullptr;
            ctx->ws_lane_bytes = 0;
        }
        MA_CUDA(cudaMalloc((void**)&ctx->ws, 2 * want));
        ctx->ws_lane_bytes = want;
    }
    *lane0 = ctx->ws;
    *lane1 = ctx->ws + ctx->ws_lane_bytes;
    *lane_bytes = ctx->ws_lane_bytes;
    return MA_OK;
}

ma_status temp_alloc(ma_context* ctx, size_t bytes, void** dptr) {
    *dptr = nullptr;
    if (bytes == 0) bytes = 16;
    if (ctx->fault_site == MA_FAULT_ALLOC) return injected(ctx);
    MA_CUDA(cudaMallocAsync(dptr, bytes, ctx->stream));
    return MA_OK;
}

void temp_free(ma_context* ctx, void* dptr) {
    if (dptr != nullptr) (void)cudaFreeAsync(dptr, ctx->stream);
}

// One thread waits, with the kernels' bounded wait, on a barrier that no copy will ever complete,
// gives up after `polls` polls and raises the context's error flag - the path a transform kernel
// takes when a staged copy does not arrive.  Nothing faults and nothing hangs.
__global__ void bounded_wait_probe_kernel(int32_t* error_flag, int polls) {
    __shared__ uint64_t bar;
    bulk_barrier_init(&bar);
    if (!bulk_barrier_wait(&bar, 0, polls)) *error_flag = 1;
}

}  // namespace ma

using namespace ma;

extern "C" {

const char* ma_status_string(ma_status s) {
    switch (s) {
        case MA_OK: return "ok";
        case MA_ERR_INVALID_ARGUMENT: return "invalid argument";
        case MA_ERR_SIZE_NOT_POW2: return "FFT size must be a power of 2";
        case MA_ERR_SIZE_TOO_LARGE: return "FFT size exceeds the maximum of 2^24";
        case MA_ERR_INVALID_HOP: return "hop size must satisfy 0 < hop <= FFT size";
        case MA_ERR_INPUT_TOO_SHORT: return "input shorter than required";
        case MA_ERR_BATCH_OVERFLOW: return "batch size overflows the buffer size computation";
        case MA_ERR_ISTFT_OVERFLOW: return "iSTFT output length overflows";
        case MA_ERR_EMPTY_KERNEL: return "kernel must not be empty";
        case MA_ERR_KERNEL_NOT_CONFIGURED: return "convolution kernel not configured";
        case MA_ERR_INVALID_PARTITION_STATE: return "invalid partition state";
        case MA_ERR_OUTPUT_OVERFLOW: return "convolution output size overflows";
        case MA_ERR_ALLOC: return "buffer allocation failed";
        case MA_ERR_TIMEOUT: return "GPU operation timed out";
        case MA_ERR_DEVICE_LOST: return "no usable CUDA device (device lost or not found)";
        case MA_ERR_CUDA: return "CUDA execution error";
        case MA_ERR_UNSUPPORTED: return "unsupported configuration";
        case MA_ERR_SCRATCH_LIMIT: return "transform needs more scratch than the built-in static buffer holds";
        case MA_ERR_INPUT_SIZE_MISMATCH: return "convolution input exceeds the expected size (circular wrap-around)";
        default: return "unknown status";
    }
}

int32_t ma_last_cuda_error(void) { return t_last_cuda_error; }

uint64_t ma_kernel_launch_count(void) { return g_launch_count.load(std::memory_order_relaxed); }

int32_t ma_device_count(void) {
    int n = 0;
    cudaError_t e = cudaGetDeviceCount(&n);
    if (e != cudaSuccess) {
        (void)cudaGetLastError();
        t_last_cuda_error = (int32_t)e;
        return 0;
    }
    return n;
}

ma_status ma_context_create(int32_t device_index, size_t pinned_bytes, ma_context** out) {
    if (out == nullptr) return MA_ERR_INVALID_ARGUMENT;
    *out = nullptr;
    int n = ma_device_count();
    if (n <= 0 || device_index < 0 || device_index >= n) return MA_ERR_DEVICE_LOST;
    MA_CUDA(cudaSetDevice(device_index));
    ma_context* ctx = new (std::nothrow) ma_context();
    if (ctx == nullptr) return MA_ERR_ALLOC;
    ctx->device = device_index;
    cudaDeviceProp prop;
    cudaError_t e = cudaGetDeviceProperties(&prop, device_index);
    if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&ctx->stream, cudaStreamNonBlocking);
    if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&ctx->copy_stream, cudaStreamNonBlocking);
    if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&ctx->d2h_stream, cudaStreamNonBlocking);
    for (int i = 0; i < kAuxStreams && e == cudaSuccess; ++i) {
        e = cudaStreamCreateWithFlags(&ctx->aux_stream[i], cudaStreamNonBlocking);
        if (e == cudaSuccess) e = cudaEventCreateWithFlags(&ctx->ev_join[i], cudaEventDisableTiming);
    }
    if (e == cudaSuccess) e = cudaEventCreateWithFlags(&ctx->ev_fork, cudaEventDisableTiming);
    for (int i = 0; i < 2 && e == cudaSuccess; ++i) {
        e = cudaEventCreateWithFlags(&ctx->ev_in[i], cudaEventDisableTiming);
        if (e == cudaSuccess) e = cudaEventCreateWithFlags(&ctx->ev_k[i], cudaEventDisableTiming);
        if (e == cudaSuccess) e = cudaEventCreateWithFlags(&ctx->ev_out[i], cudaEventDisableTiming);
    }
    if (e == cudaSuccess) {
        ctx->sm_count = prop.multiProcessorCount;
        std::strncpy(ctx->name, prop.name, sizeof(ctx->name) - 1);
        ctx->pinned_bytes = pinned_bytes ? pinned_bytes : ((size_t)64 << 20);
        ctx->pinned_bytes &= ~(size_t)255;
        if (ctx->pinned_bytes < 512) ctx->pinned_bytes = 512;
        e = cudaHostAlloc(&ctx->pinned, ctx->pinned_bytes, cudaHostAllocDefault);
    }
    for (int i = 0; i < 2 && e == cudaSuccess; ++i)
        e = cudaEventCreateWithFlags(&ctx->ev_half[i], cudaEventDisableTiming);
    if (e == cudaSuccess) e = cudaEventCreate(&ctx->ev_begin);
    if (e == cudaSuccess) e = cudaEventCreate(&ctx->ev_end);
    if (e == cudaSuccess) e = cudaEventCreateWithFlags(&ctx->ev_sync, cudaEventDisableTiming);
    if (e == cudaSuccess) e = cudaMalloc((void**)&ctx->d_error_flag, sizeof(int32_t));
    if (e == cudaSuccess) e = cudaMemsetAsync(ctx->d_error_flag, 0, sizeof(int32_t), ctx->stream);  // ordered before every kernel of the context
    if (e == cudaSuccess) e = cudaHostAlloc((void**)&ctx->h_error_flag, sizeof(int32_t), cudaHostAllocDefault);
    if (e == cudaSuccess) *ctx->h_error_flag = 0;
    if (e == cudaSuccess) {
        // Keep freed stream-ordered temporaries cached instead of returning them to the OS.
        cudaMemPool_t pool;
        if (cudaDeviceGetDefaultMemPool(&pool, device_index) == cudaSuccess) {
            uint64_t thresh = UINT64_MAX;
            (void)cudaMemPoolSetAttribute(pool, cudaMemPoolAttrReleaseThreshold, &thresh);
        }
        (void)cudaGetLastError();
    }
    if (e != cudaSuccess) {
        ma_status s = cuda_fail(e);
        ma_context_destroy(ctx);
        return s;
    }
    *out = ctx;
    return MA_OK;
}

ma_status ma_context_destroy(ma_context* ctx) {
    if (ctx == nullptr) return MA_OK;
    (void)cudaSetDevice(ctx->device);
    if (ctx->stream) (void)cudaStreamSynchronize(ctx->stream);
    for (int i = 0; i < 2; ++i)
        if (ctx->ev_half[i]) (void)cudaEventDestroy(ctx->ev_half[i]);
    if (ctx->ev_begin) (void)cudaEventDestroy(ctx->ev_begin);
    if (ctx->ev_end) (void)cudaEventDestroy(ctx->ev_end);
    if (ctx->ev_sync) (void)cudaEventDestroy(ctx->ev_sync);
    if (ctx->pinned) (void)cudaFreeHost(ctx->pinned);
    if (ctx->d_error_flag) (void)cudaFree(ctx->d_error_flag);
    if (ctx->h_error_flag) (void)cudaFreeHost(ctx->h_error_flag);
    for (int i = 0; i < 2; ++i) {
        if (ctx->ev_in[i]) (void)cudaEventDestroy(ctx->ev_in[i]);
        if (ctx->ev_k[i]) (void)cudaEventDestroy(ctx->ev_k[i]);
        if (ctx->ev_out[i]) (void)cudaEventDestroy(ctx->ev_out[i]);
    }
    if (ctx->ws) (void)cudaFree(ctx->ws);
    if (ctx->copy_stream) (void)cudaStreamDestroy(ctx->copy_stream);
    if (ctx->d2h_stream) (void)cudaStreamDestroy(ctx->d2h_stream);
    for (int i = 0; i < kAuxStreams; ++i) {
        if (ctx->aux_stream[i]) (void)cudaStreamDestroy(ctx->aux_stream[i]);
        if (ctx->ev_join[i]) (void)cudaEventDestroy(ctx->ev_join[i]);
    }
    if (ctx->ev_fork) (void)cudaEventDestroy(ctx->ev_fork);
    if (ctx->stream) (void)cudaStreamDestroy(ctx->stream);
    (void)cudaGetLastError();
    delete ctx;
    return MA_OK;
}

ma_status ma_context_sync(ma_context* ctx, double timeout_s) {
    MA_TRY(enter(ctx, MA_FAULT_SYNC));
    if (timeout_s <= 0.0) timeout_s = 2.0;
    // A kernel whose bounded wait ran out leaves a flag; fetch it behind the queued work.
    MA_CUDA(cudaMemcpyAsync(ctx->h_error_flag, ctx->d_error_flag, sizeof(int32_t), cudaMemcpyDeviceToHost, ctx->stream));
    MA_CUDA(cudaEventRecord(ctx->ev_sync, ctx->stream));
    const auto t0 = std::chrono::steady_clock::now();
    for (;;) {
        cudaError_t e = cudaEventQuery(ctx->ev_sync);
        if (e == cudaSuccess) {
            if (*ctx->h_error_flag != 0) {
                *ctx->h_error_flag = 0;
                (void)cudaMemsetAsync(ctx->d_error_flag, 0, sizeof(int32_t), ctx->stream);
                return MA_ERR_TIMEOUT;
            }
            return MA_OK;
        }
        if (e != cudaErrorNotReady) return cuda_fail(e);
        const double dt = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
        if (dt > timeout_s) return MA_ERR_TIMEOUT;
        if (dt > 0.0005) std::this_thread::sleep_for(std::chrono::microseconds(50));
    }
}

ma_status ma_context_device_name(ma_context* ctx, char* buf, size_t buf_len) {
    if (ctx == nullptr || buf == nullptr || buf_len == 0) return MA_ERR_INVALID_ARGUMENT;
    std::strncpy(buf, ctx->name, buf_len - 1);
    buf[buf_len - 1] = 0;
    return MA_OK;
}

void* ma_context_stream(ma_context* ctx) { return ctx ? (void*)ctx->stream : nullptr; }

ma_status ma_context_mark_lost(ma_context* ctx) {
    if (ctx == nullptr) return MA_ERR_INVALID_ARGUMENT;
    ctx->lost = true;
    return MA_OK;
}

ma_status ma_context_is_available(ma_context* ctx, int32_t* available) {
    if (ctx == nullptr || available == nullptr) return MA_ERR_INVALID_ARGUMENT;
    *available = ctx->lost ? 0 : 1;
    return MA_OK;
}

ma_status ma_timing_begin(ma_context* ctx) {
    MA_TRY(enter(ctx, MA_FAULT_LAUNCH));
    MA_CUDA(cudaEventRecord(ctx->ev_begin, ctx->stream));
    ctx->timing_open = true;
    return MA_OK;
}

ma_status ma_timing_end(ma_context* ctx, float* milliseconds) {
    MA_TRY(enter(ctx, MA_FAULT_SYNC));
    if (!ctx->timing_open || milliseconds == nullptr) return MA_ERR_INVALID_ARGUMENT;
    MA_CUDA(cudaEventRecord(ctx->ev_end, ctx->stream));
    MA_CUDA(cudaEventSynchronize(ctx->ev_end));
    MA_CUDA(cudaEventElapsedTime(milliseconds, ctx->ev_begin, ctx->ev_end));
    ctx->timing_open = false;
    return MA_OK;
}

ma_status ma_test_inject_fault(ma_context* ctx, int32_t site, int32_t cuda_error) {
    if (ctx == nullptr || site < MA_FAULT_ALLOC || site > MA_FAULT_DEVICE_LOST) return MA_ERR_INVALID_ARGUMENT;
    ctx->fault_site = site;
    ctx->fault_error = cuda_error;
    return MA_OK;
}

ma_status ma_test_bounded_wait(ma_context* ctx, int32_t polls) {
    MA_TRY(enter(ctx, MA_FAULT_LAUNCH));
    if (polls < 1 || polls > (1 << 16)) return MA_ERR_INVALID_ARGUMENT;
    bounded_wait_probe_kernel<<<1, 1, 0, ctx->stream>>>(ctx->d_error_flag, polls);
    return after_launch(ctx);
}

ma_status ma_context_reserve_workspace(ma_context* ctx, size_t bytes) {
    MA_TRY(enter(ctx, MA_FAULT_ALLOC));
    char *a, *b;
    size_t lane;
    return workspace_lanes(ctx, (bytes + 1) / 2, &a, &b, &lane);
}

ma_status ma_buffer_alloc(ma_context* ctx, size_t bytes, void** dptr) {
    if (dptr == nullptr) return MA_ERR_INVALID_ARGUMENT;
    *dptr = nullptr;
    MA_TRY(enter(ctx, MA_FAULT_ALLOC));
    MA_CUDA(cudaMalloc(dptr, bytes ? bytes : 16));
    return MA_OK;
}

ma_status ma_buffer_free(ma_context* ctx, void* dptr) {
    if (ctx == nullptr) return MA_ERR_INVALID_ARGUMENT;
    if (dptr == nullptr) return MA_OK;
    (void)cudaSetDevice(ctx->device);
    MA_CUDA(cudaStreamSynchronize(ctx->stream));
    MA_CUDA(cudaFree(dptr));
    return MA_OK;
}

ma_status ma_buffer_zero(ma_context* ctx, void* dptr, size_t bytes) {
    MA_TRY(enter(ctx, MA_FAULT_LAUNCH));
    MA_CUDA(cudaMemsetAsync(dptr, 0, bytes, ctx->stream));
    return MA_OK;
}

ma_status ma_memcpy_h2d(ma_context* ctx, void* dptr, const void* host, size_t bytes) {
    MA_TRY(enter(ctx, MA_FAULT_LAUNCH));
    if ((dptr == nullptr || host == nullptr) && bytes) return MA_ERR_INVALID_ARGUMENT;
    return copy_h2d(ctx, dptr, host, bytes);
}

ma_status ma_memcpy_d2h(ma_context* ctx, void* host, const void* dptr, size_t bytes) {
    MA_TRY(enter(ctx, MA_FAULT_LAUNCH));
    if ((dptr == nullptr || host == nullptr) && bytes) return MA_ERR_INVALID_ARGUMENT;
    return copy_d2h(ctx, host, dptr, bytes);
}

ma_status ma_memcpy_h2d_async(ma_context* ctx, void* dptr, const void* host, size_t bytes) {
    MA_TRY(enter(ctx, MA_FAULT_LAUNCH));
    MA_CUDA(cudaMemcpyAsync(dptr, host, bytes, cudaMemcpyHostToDevice, ctx->stream));
    return MA_OK;
}

ma_status ma_memcpy_d2h_async(ma_context* ctx, void* host, const void* dptr, size_t bytes) {
    MA_TRY(enter(ctx, MA_FAULT_LAUNCH));
    MA_CUDA(cudaMemcpyAsync(host, dptr, bytes, cudaMemcpyDeviceToHost, ctx->stream));
    return MA_OK;
}

ma_status ma_host_alloc(ma_context* ctx, size_t bytes, void** hptr) {
    if (hptr == nullptr) return MA_ERR_INVALID_ARGUMENT;
    *hptr = nullptr;
    MA_TRY(enter(ctx, MA_FAULT_ALLOC));
    MA_CUDA(cudaHostAlloc(hptr, bytes ? bytes : 16, cudaHostAllocDefault));
    return MA_OK;
}

ma_status ma_host_free(ma_context* ctx, void* hptr) {
    if (ctx == nullptr) return MA_ERR_INVALID_ARGUMENT;
    if (hptr == nullptr) return MA_OK;
    MA_CUDA(cudaFreeHost(hptr));
    return MA_OK;
}

}  // extern "C"
