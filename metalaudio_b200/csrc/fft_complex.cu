// Complex-input transforms on interleaved (re, im) data: the explicit-backend calls
// forwardGPU / inverseGPU of the reference (FFT.swift:945-1107, :1176-1315), for every plan size.
//
// A complex sequence z = a + i b is carried by the real-input machinery the rest of the library is
// built around: FFT(z) = FFT(a) + i FFT(b) with both real transforms Hermitian, so
//   Z[k]     = A[k] + i B[k]                  0 <= k <= N/2
//   Z[N - k] = conj(A[k]) + i conj(B[k])      0 <  k <  N/2
// Three launches per chunk: split (a and b into two real rows), the batched real forward
// transform of 2 rows per sequence (small or multi-pass path, whatever the plan is), combine.
// The inverse uses IFFT(Z) = conj(FFT(conj Z)) / N: the split negates the imaginary row and the
// combine conjugates and scales.  Intermediate rows and half spectra live in a plan-owned work
// buffer that is allocated on the first such call.
#include <new>

#include "fft_plan.h"

namespace ma {

__global__ void __launch_bounds__(256) complex_split_kernel(const float2* __restrict__ in, float* __restrict__ rows,
                                                            int64_t n, int64_t batch, float im_sign) {
    const int64_t total = n * batch;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t b = i / n, k = i - b * n;
        const float2 z = __ldcs(in + i);
        rows[(2 * b) * n + k] = z.x;
        rows[(2 * b + 1) * n + k] = im_sign * z.y;
    }
}

__global__ void __launch_bounds__(256) complex_combine_kernel(const float2* __restrict__ spec, float2* __restrict__ out,
                                                              int64_t n, int64_t batch, float conj_sign, float scale) {
    const int64_t total = n * batch, kh = n / 2 + 1;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t b = i / n, k = i - b * n;
        const bool upper = k > n / 2;
        const int64_t kk = upper ? n - k : k;
        const float2 A = __ldg(spec + (2 * b) * kh + kk);
        const float2 B = __ldg(spec + (2 * b + 1) * kh + kk);
        // lower half: A + iB; upper half: conj(A) + i conj(B)
        const float re = upper ? A.x + B.y : A.x - B.y;
        const float im = upper ? B.x - A.y : A.y + B.x;
        out[i] = make_float2(re * scale, conj_sign * im * scale);
    }
}

static int grid_for(ma_context* ctx, int64_t total) {
    const int64_t want = (total + 255) / 256, cap = (int64_t)ctx->sm_count * 8;
    return (int)(want < cap ? (want > 0 ? want : 1) : cap);
}

// Sequences per chunk and the work buffer (rows, then half spectra) sized for it.
static ma_status complex_workspace(ma_fft_plan* plan, int64_t* chunk, float** rows, float2** spec) {
    const int64_t n = plan->n, kh = n / 2 + 1;
    int64_t cb = ((int64_t)64 << 20) / (8 * n);  // about 64 MiB of real rows per chunk
    if (cb < 1) cb = 1;
    const size_t rows_bytes = (size_t)(2 * cb * n) * sizeof(float);
    const size_t spec_bytes = (size_t)(2 * cb * kh) * sizeof(float2);
    if (plan->d_cwork == nullptr)  // first complex transform through this plan
        MA_CUDA(cudaMalloc((void**)&plan->d_cwork, rows_bytes + spec_bytes));
    *chunk = cb;
    *rows = plan->d_cwork;
    *spec = reinterpret_cast<float2*>(reinterpret_cast<char*>(plan->d_cwork) + rows_bytes);
    return MA_OK;
}

}  // namespace ma

using namespace ma;

extern "C" {

ma_status ma_fft_complex_dev(ma_fft_plan* plan, const float* in, float* out, int64_t batch, int32_t inverse) {
    if (plan == nullptr) return MA_ERR_INVALID_ARGUMENT;
    ma_context* ctx = plan->ctx;
    MA_TRY(enter(ctx, MA_FAULT_LAUNCH));
    if (batch == 0) return MA_OK;
    if (batch < 0 || in == nullptr || out == nullptr) return MA_ERR_INVALID_ARGUMENT;
    int64_t total;
    if (__builtin_mul_overflow(batch, 2 * (int64_t)plan->n, &total)) return MA_ERR_BATCH_OVERFLOW;
    if ((reinterpret_cast<uintptr_t>(in) | reinterpret_cast<uintptr_t>(out)) & 7) return MA_ERR_INVALID_ARGUMENT;
    int64_t chunk = 0;
    float* rows = nullptr;
    float2* spec = nullptr;
    MA_TRY(complex_workspace(plan, &chunk, &rows, &spec));
    const int64_t n = plan->n;
    const float sign = inverse ? -1.0f : 1.0f;
    const float scale = inverse ? 1.0f / (float)n : 1.0f;
    for (int64_t done = 0; done < batch; done += chunk) {
        const int64_t cb = batch - done < chunk ? batch - done : chunk;
        complex_split_kernel<<<grid_for(ctx, cb * n), 256, 0, ctx->stream>>>(
            reinterpret_cast<const float2*>(in) + done * n, rows, n, cb, sign);
        MA_TRY(after_launch(ctx));
        MA_TRY(ma_fft_forward_dev(plan, rows, reinterpret_cast<float*>(spec), nullptr, nullptr, 0, 1.0f, 2 * cb,
                                  MA_LAYOUT_HALF_INTERLEAVED));
        complex_combine_kernel<<<grid_for(ctx, cb * n), 256, 0, ctx->stream>>>(
            spec, reinterpret_cast<float2*>(out) + done * n, n, cb, sign, scale);
        MA_TRY(after_launch(ctx));
    }
    return MA_OK;
}

ma_status ma_fft_complex_host(ma_fft_plan* plan, const float* in, float* out, int64_t batch, int32_t inverse) {
    if (plan == nullptr) return MA_ERR_INVALID_ARGUMENT;
    ma_context* ctx = plan->ctx;
    MA_TRY(enter(ctx, MA_FAULT_LAUNCH));
    if (batch == 0) return MA_OK;
    if (batch < 0 || in == nullptr || out == nullptr) return MA_ERR_INVALID_ARGUMENT;
    int64_t total;
    if (__builtin_mul_overflow(batch, 2 * (int64_t)plan->n, &total) || total > (INT64_MAX / 16)) return MA_ERR_BATCH_OVERFLOW;
    const size_t bytes = (size_t)total * sizeof(float);
    float *d_in = nullptr, *d_out = nullptr;
    ma_status st = temp_alloc(ctx, bytes, (void**)&d_in);
    if (st == MA_OK) st = temp_alloc(ctx, bytes, (void**)&d_out);
    if (st == MA_OK) st = copy_h2d(ctx, d_in, in, bytes);
    if (st == MA_OK) st = ma_fft_complex_dev(plan, d_in, d_out, batch, inverse);
    if (st == MA_OK) st = copy_d2h(ctx, out, d_out, bytes);
    temp_free(ctx, d_in);
    temp_free(ctx, d_out);
    return st;
}

}  // extern "C"
