// Elementwise steps on either side of the transforms, as the reference's shader library holds them
// (Sources/MetalDSP/Shaders/DSP.metal): compute_magnitude + compute_phase (:784-813) as one pass
// over interleaved complex bins, polar_to_complex (:821-834), to_decibels (:861-881).
// Pure streaming kernels: every element is read once and written once.
#include "ma_internal.h"

namespace ma {

__global__ void __launch_bounds__(256) to_polar_kernel(const float2* __restrict__ spec, float* __restrict__ mag,
                                                       float* __restrict__ phase, int64_t count) {
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < count; i += (int64_t)gridDim.x * blockDim.x) {
        const float2 c = __ldcs(spec + i);
        if (mag != nullptr) __stcs(mag + i, sqrtf(c.x * c.x + c.y * c.y));
        if (phase != nullptr) __stcs(phase + i, atan2f(c.y, c.x));
    }
}

__global__ void __launch_bounds__(256) from_polar_kernel(const float* __restrict__ mag, const float* __restrict__ phase,
                                                         float2* __restrict__ spec, int64_t count) {
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < count; i += (int64_t)gridDim.x * blockDim.x) {
        float s, c;
        sincosf(__ldcs(phase + i), &s, &c);
        const float m = __ldcs(mag + i);
        __stcs(spec + i, make_float2(m * c, m * s));
    }
}

// 20*log10(max(x/reference, 1e-10)) clamped below at min_db; reference <= 0 writes min_db.
__global__ void __launch_bounds__(256) decibels_kernel(float* __restrict__ data, int64_t count, float reference,
                                                       float min_db) {
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < count; i += (int64_t)gridDim.x * blockDim.x) {
        if (reference <= 0.f) {
            data[i] = min_db;
            continue;
        }
        const float ratio = fmaxf(data[i] / reference, 1e-10f);
        data[i] = fmaxf(20.f * log10f(ratio), min_db);
    }
}

static int stream_grid(ma_context* ctx, int64_t count) {
    const int64_t want = (count + 255) / 256, cap = (int64_t)ctx->sm_count * 8;
    return (int)(want < cap ? want : cap);
}

}  // namespace ma

using namespace ma;

extern "C" {

ma_status ma_spectrum_to_polar_dev(ma_context* ctx, const float* spectrum, float* magnitude, float* phase,
                                   int64_t count) {
    if (ctx == nullptr || count < 0 || (count > 0 && (spectrum == nullptr || (magnitude == nullptr && phase == nullptr))))
        return MA_ERR_INVALID_ARGUMENT;
    MA_TRY(enter(ctx, MA_FAULT_LAUNCH));
    if (count == 0) return MA_OK;
    to_polar_kernel<<<stream_grid(ctx, count), 256, 0, ctx->stream>>>(reinterpret_cast<const float2*>(spectrum), magnitude,
                                                                      phase, count);
    return after_launch(ctx);
}

ma_status ma_polar_to_spectrum_dev(ma_context* ctx, const float* magnitude, const float* phase, float* spectrum,
                                   int64_t count) {
    if (ctx == nullptr || count < 0 || (count > 0 && (spectrum == nullptr || magnitude == nullptr || phase == nullptr)))
        return MA_ERR_INVALID_ARGUMENT;
    MA_TRY(enter(ctx, MA_FAULT_LAUNCH));
    if (count == 0) return MA_OK;
    from_polar_kernel<<<stream_grid(ctx, count), 256, 0, ctx->stream>>>(magnitude, phase, reinterpret_cast<float2*>(spectrum),
                                                                        count);
    return after_launch(ctx);
}

ma_status ma_to_decibels_dev(ma_context* ctx, float* data, int64_t count, float reference, float min_db) {
    if (ctx == nullptr || count < 0 || (count > 0 && data == nullptr)) return MA_ERR_INVALID_ARGUMENT;
    MA_TRY(enter(ctx, MA_FAULT_LAUNCH));
    if (count == 0) return MA_OK;
    decibels_kernel<<<stream_grid(ctx, count), 256, 0, ctx->stream>>>(data, count, reference, min_db);
    return after_launch(ctx);
}

}  // extern "C"
