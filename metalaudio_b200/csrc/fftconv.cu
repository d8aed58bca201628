// One-shot FFT convolution (the reference's Convolution `.fft` mode,
// Sources/MetalDSP/Convolution.swift:210-248 set-up, :437-493 process):
//
//   fft_size = next power of two >= expected_input + taps - 1
//   y = IFFT( FFT(zero-padded x) * FFT(zero-padded h) ),  fft_size samples per signal
//
// Built on the library's real-input transforms.  Up to 8192 points one kernel transforms the input
// rows to half spectra (zero padding applied by its loader) and a second one transforms back with
// the bin-by-bin product by the kernel's half spectrum fused into its loads (both are spectra of
// real signals, so the product's upper half is the conjugate mirror and never has to exist) and
// the 1/N scale.  Above 8192 points the
// two-pass transforms are fused around the product: columns forward (zero padding applied by the
// loader), then one kernel that runs the row transform, the product and the inverse row transform
// in place on the L2-resident pass data, then columns inverse; HBM sees the input and the output
// only.  All work buffers are sized at creation; the process calls allocate nothing.
#include <new>

#include "fft_plan.h"
#include "ma_internal.h"

struct ma_fftconv {
    ma_context* ctx = nullptr;
    ma_fft_plan* plan = nullptr;
    int64_t taps = 0, expected = 0, n = 0;
    int32_t max_signals = 0;
    float* d_padded = nullptr;   // [n]: the zero-padded kernel, small plans only
    float2* d_spec = nullptr;    // [max_signals][n/2+1]
    float2* d_kernel = nullptr;  // [n/2+1], or for large plans the spectrum in pass-2 row order
    bool large = false;
};

namespace ma {

// dst[s][0..n) = src[s][0..len) followed by zeros.
__global__ void __launch_bounds__(256) fftconv_pad_kernel(const float* __restrict__ src, int64_t len, int64_t stride,
                                                          float* __restrict__ dst, int64_t n, int64_t total) {
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t s = i / n, j = i - s * n;
        dst[i] = j < len ? __ldg(src + s * stride + j) : 0.f;
    }
}

static int grid_for(ma_context* ctx, int64_t total) {
    const int64_t want = (total + 255) / 256, cap = (int64_t)ctx->sm_count * 8;
    return (int)(want < cap ? (want > 0 ? want : 1) : cap);
}

static ma_status fftconv_run(ma_fftconv* fc, const float* d_in, int64_t len, int64_t in_stride, int32_t n_signals,
                             float* d_out) {
    ma_context* ctx = fc->ctx;
    const int64_t n = fc->n, bins = n / 2 + 1;
    if (fc->large) return launch_conv_large(fc->plan, d_in, len, in_stride, fc->d_kernel, d_out, n_signals);
    // forward transforms with the zero padding applied by the loader, straight from the caller's rows
    R2CParams f{};
    f.in = d_in;
    f.signal_stride = in_stride;
    f.frames_per_signal = 1;
    f.total_frames = n_signals;
    f.signal_len = len;
    f.hop = (int32_t)n;
    f.frame_valid = (int32_t)(len < n ? len : n);
    f.out_a = reinterpret_cast<float*>(fc->d_spec);
    f.out_signal_stride = bins;
    f.out_frame_stride = 0;
    f.layout = LAYOUT_HALF_INTERLEAVED;
    f.mag_kind = MAG_NONE;
    MA_TRY(launch_r2c_small(fc->plan, f));
    // inverse transforms with the product by the kernel spectrum fused into their loads
    C2RParams c{};
    c.in_a = reinterpret_cast<const float*>(fc->d_spec);
    c.in_frame_stride = bins;
    c.in_signal_stride = 0;
    c.frames_per_signal = n_signals;
    c.n_signals = 1;
    c.layout = LAYOUT_HALF_INTERLEAVED;
    c.hop = (int32_t)n;
    c.out = d_out;
    c.out_signal_stride = 0;
    c.mul = fc->d_kernel;
    return launch_c2r_small(fc->plan, c);
}

}  // namespace ma

using namespace ma;

extern "C" {

ma_status ma_fftconv_create(ma_context* ctx, const float* kernel, int64_t taps, int64_t expected_input,
                            int32_t max_signals, ma_fftconv** out) {
    if (out == nullptr) return MA_ERR_INVALID_ARGUMENT;
    *out = nullptr;
    if (ctx == nullptr || max_signals <= 0 || expected_input <= 0) return MA_ERR_INVALID_ARGUMENT;
    if (kernel == nullptr || taps <= 0) return MA_ERR_EMPTY_KERNEL;
    if (expected_input > INT64_MAX - taps) return MA_ERR_OUTPUT_OVERFLOW;
    const int64_t min_size = expected_input + taps - 1;
    if (min_size > ((int64_t)1 << 24)) return MA_ERR_SIZE_TOO_LARGE;
    int64_t n = 2;  // the transforms start at two points
    while (n < min_size) n <<= 1;
    MA_TRY(enter(ctx, MA_FAULT_ALLOC));
    ma_fftconv* fc = new (std::nothrow) ma_fftconv();
    if (fc == nullptr) return MA_ERR_ALLOC;
    fc->ctx = ctx;
    fc->taps = taps;
    fc->expected = expected_input;
    fc->n = n;
    fc->max_signals = max_signals;
    const int64_t bins = n / 2 + 1;
    ma_status st = ma_fft_plan_create(ctx, (int32_t)n, nullptr, (int32_t)n, &fc->plan);
    fc->large = st == MA_OK && fc->plan->large;
    // large plans keep the kernel spectrum in pass-2 row order: (N2/2+1) rows of N1 values
    const int64_t kernel_elems = fc->large ? (int64_t)(fc->plan->n2 / 2 + 1) * fc->plan->n1 : bins;
    if (st == MA_OK) {
        cudaError_t e = cudaMalloc((void**)&fc->d_kernel, sizeof(float2) * (size_t)kernel_elems);
        if (e == cudaSuccess && !fc->large) {
            e = cudaMalloc((void**)&fc->d_padded, sizeof(float) * (size_t)n);
            if (e == cudaSuccess) e = cudaMalloc((void**)&fc->d_spec, sizeof(float2) * (size_t)bins * max_signals);
        }
        if (e != cudaSuccess) st = cuda_fail(e);
    }
    float* d_taps = nullptr;
    if (st == MA_OK) {
        cudaError_t e = cudaMalloc((void**)&d_taps, sizeof(float) * (size_t)taps);
        if (e != cudaSuccess) st = cuda_fail(e);
    }
    if (st == MA_OK) st = copy_h2d(ctx, d_taps, kernel, sizeof(float) * (size_t)taps);
    if (st == MA_OK && fc->large) st = launch_spec_rows_large(fc->plan, d_taps, taps, fc->d_kernel);
    if (st == MA_OK && !fc->large) {
        fftconv_pad_kernel<<<grid_for(ctx, n), 256, 0, ctx->stream>>>(d_taps, taps, taps, fc->d_padded, n, n);
        st = after_launch(ctx);
        if (st == MA_OK)
            st = ma_fft_forward_dev(fc->plan, fc->d_padded, reinterpret_cast<float*>(fc->d_kernel), nullptr, nullptr, 0,
                                    1.f, 1, MA_LAYOUT_HALF_INTERLEAVED);
    }
    if (st == MA_OK) st = ma_context_sync(ctx, 30.0);
    if (d_taps != nullptr) (void)cudaFree(d_taps);
    if (st != MA_OK) {
        ma_fftconv_destroy(fc);
        return st;
    }
    *out = fc;
    return MA_OK;
}

ma_status ma_fftconv_destroy(ma_fftconv* fc) {
    if (fc == nullptr) return MA_OK;
    if (fc->plan) (void)ma_fft_plan_destroy(fc->plan);
    if (fc->d_padded) (void)cudaFree(fc->d_padded);
    if (fc->d_spec) (void)cudaFree(fc->d_spec);
    if (fc->d_kernel) (void)cudaFree(fc->d_kernel);
    delete fc;
    return MA_OK;
}

ma_status ma_fftconv_fft_size(ma_fftconv* fc, int64_t* fft_size) {
    if (fc == nullptr || fft_size == nullptr) return MA_ERR_INVALID_ARGUMENT;
    *fft_size = fc->n;
    return MA_OK;
}

static ma_status fftconv_check(ma_fftconv* fc, const void* in, int64_t len, int64_t in_stride, int32_t n_signals,
                               const void* out) {
    if (fc == nullptr) return MA_ERR_KERNEL_NOT_CONFIGURED;
    if (in == nullptr || out == nullptr || len <= 0 || n_signals <= 0 || in_stride < len) return MA_ERR_INVALID_ARGUMENT;
    if (n_signals > fc->max_signals) return MA_ERR_BATCH_OVERFLOW;
    if (len > fc->expected) return MA_ERR_INPUT_SIZE_MISMATCH;  // would wrap around (Convolution.swift:461-467)
    return MA_OK;
}

ma_status ma_fftconv_process_dev(ma_fftconv* fc, const float* in, int64_t len, int64_t in_stride, int32_t n_signals,
                                 float* out) {
    MA_TRY(fftconv_check(fc, in, len, in_stride, n_signals, out));
    MA_TRY(enter(fc->ctx, MA_FAULT_LAUNCH));
    return fftconv_run(fc, in, len, in_stride, n_signals, out);
}

ma_status ma_fftconv_process_host(ma_fftconv* fc, const float* in, int64_t len, int64_t in_stride, int32_t n_signals,
                                  float* out) {
    MA_TRY(fftconv_check(fc, in, len, in_stride, n_signals, out));
    ma_context* ctx = fc->ctx;
    MA_TRY(enter(ctx, MA_FAULT_LAUNCH));
    void *d_in = nullptr, *d_out = nullptr;
    const size_t in_bytes = sizeof(float) * (size_t)len * n_signals, out_bytes = sizeof(float) * (size_t)fc->n * n_signals;
    MA_TRY(temp_alloc(ctx, in_bytes, &d_in));
    ma_status st = temp_alloc(ctx, out_bytes, &d_out);
    for (int32_t s = 0; st == MA_OK && s < n_signals; ++s)  // rows may be strided on the host
        st = copy_h2d(ctx, (float*)d_in + (size_t)s * len, in + (size_t)s * in_stride, sizeof(float) * (size_t)len);
    if (st == MA_OK) st = fftconv_run(fc, (const float*)d_in, len, len, n_signals, (float*)d_out);
    if (st == MA_OK) st = copy_d2h(ctx, out, d_out, out_bytes);
    temp_free(ctx, d_in);
    if (d_out != nullptr) temp_free(ctx, d_out);
    return st;
}

}  // extern "C"
