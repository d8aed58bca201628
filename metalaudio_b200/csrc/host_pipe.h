// Three-stage host pipeline shared by the *_host entry points that move whole arrays.
//
// Those calls cut their rows (signals, channels) into chunks that fit one lane of the context's device
// workspace and run the chunks through a three-stage pipeline when the host memory is pinned:
// host -> device copies on one stream, the transform on the context's stream, device -> host
// copies on a third, chained by events, two lanes deep - chunk c's results travel back while chunk
// c+1 is transformed and chunk c+2 is on its way in (PCIe is full duplex).  Nothing is allocated
// per call once the workspace exists, and the host waits once, at the end.  Pageable host memory
// takes the same chunks one after the other through the staging buffer.
#pragma once
#include "ma_internal.h"

namespace ma {


inline size_t round256(size_t b) { return (b + 255) & ~(size_t)255; }

struct Pipe {
    ma_context* ctx;
    bool pinned;
    int64_t chunk;  // signals per chunk
    char* lane[2];
    ma_status st = MA_OK;

    void before_copy_in(int64_t c) {
        const int l = (int)(c & 1);
        if (pinned && c >= 2 && st == MA_OK) fail(cudaStreamWaitEvent(ctx->copy_stream, ctx->ev_k[l], 0));
    }
    void before_kernels(int64_t c) {
        const int l = (int)(c & 1);
        if (!pinned || st != MA_OK) return;
        fail(cudaEventRecord(ctx->ev_in[l], ctx->copy_stream));
        fail(cudaStreamWaitEvent(ctx->stream, ctx->ev_in[l], 0));
        if (c >= 2) fail(cudaStreamWaitEvent(ctx->stream, ctx->ev_out[l], 0));
    }
    void before_copy_out(int64_t c) {
        const int l = (int)(c & 1);
        if (!pinned || st != MA_OK) return;
        fail(cudaEventRecord(ctx->ev_k[l], ctx->stream));
        fail(cudaStreamWaitEvent(ctx->d2h_stream, ctx->ev_k[l], 0));
    }
    void after_copy_out(int64_t c) {
        const int l = (int)(c & 1);
        if (pinned && st == MA_OK) fail(cudaEventRecord(ctx->ev_out[l], ctx->d2h_stream));
    }
    // rows x width floats between a strided host array and a dense-strided device array
    void in2d(void* d, size_t dpitch, const void* h, size_t hpitch, size_t width, size_t rows) {
        if (st != MA_OK || rows == 0) return;
        if (pinned) {
            fail(cudaMemcpy2DAsync(d, dpitch, h, hpitch, width, rows, cudaMemcpyHostToDevice, ctx->copy_stream));
        } else if (dpitch == width && hpitch == width) {
            st = copy_h2d(ctx, d, h, width * rows);
        } else {
            for (size_t r = 0; r < rows && st == MA_OK; ++r)
                st = copy_h2d(ctx, (char*)d + r * dpitch, (const char*)h + r * hpitch, width);
        }
    }
    void out2d(void* h, size_t hpitch, const void* d, size_t dpitch, size_t width, size_t rows) {
        if (st != MA_OK || rows == 0) return;
        if (pinned) {
            fail(cudaMemcpy2DAsync(h, hpitch, d, dpitch, width, rows, cudaMemcpyDeviceToHost, ctx->d2h_stream));
        } else if (dpitch == width && hpitch == width) {
            st = copy_d2h(ctx, h, d, width * rows);
        } else {
            for (size_t r = 0; r < rows && st == MA_OK; ++r)
                st = copy_d2h(ctx, (char*)h + r * hpitch, (const char*)d + r * dpitch, width);
        }
    }
    // waits for everything the call queued, also after a failure half-way
    ma_status finish() {
        cudaError_t e = cudaStreamSynchronize(ctx->copy_stream);
        cudaError_t e2 = cudaStreamSynchronize(ctx->stream);
        cudaError_t e3 = cudaStreamSynchronize(ctx->d2h_stream);
        if (st == MA_OK) {
            if (e != cudaSuccess) st = cuda_fail(e);
            else if (e2 != cudaSuccess) st = cuda_fail(e2);
            else if (e3 != cudaSuccess) st = cuda_fail(e3);
        }
        return st;
    }
    void fail(cudaError_t e) {
        if (e != cudaSuccess && st == MA_OK) st = cuda_fail(e);
    }
};

// Chunk size and lanes for rows that need `row_bytes` of workspace each (sub-buffers included).
inline ma_status pipe_open(Pipe& p, ma_context* ctx, bool pinned, int64_t rows, size_t row_bytes, size_t fixed_bytes) {
    size_t lane_bytes = 0;
    MA_TRY(workspace_lanes(ctx, row_bytes + fixed_bytes, &p.lane[0], &p.lane[1], &lane_bytes));
    int64_t chunk = (int64_t)((lane_bytes - fixed_bytes) / row_bytes);
    if (chunk < 1) chunk = 1;
    // at least four chunks when there are rows enough, so that the three stages overlap
    if (pinned && rows >= 4 && chunk > (rows + 3) / 4) chunk = (rows + 3) / 4;
    if (chunk > rows) chunk = rows;
    p.ctx = ctx;
    p.pinned = pinned;
    p.chunk = chunk;
    return MA_OK;
}


}  // namespace ma
