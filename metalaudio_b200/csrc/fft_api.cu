// C ABI: FFT plan, forward / inverse / magnitude, STFT / iSTFT.
#include <limits>
#include <new>

#include "fft_plan.h"
#include "host_pipe.h"
#include "host_tables.h"

namespace ma {
ma_status launch_magnitude(ma_fft_plan* plan, const float* re, const float* im, float* out, int64_t batch,
                           int kind, float db_scale);
}
using namespace ma;

static bool mul_overflow(int64_t a, int64_t b, int64_t* r) { return __builtin_mul_overflow(a, b, r); }
static bool add_overflow(int64_t a, int64_t b, int64_t* r) { return __builtin_add_overflow(a, b, r); }

static ma_status upload(ma_context* ctx, const void* host, size_t bytes, void** dptr) {
    MA_CUDA(cudaMalloc(dptr, bytes));
    return copy_h2d(ctx, *dptr, host, bytes);
}

static bool valid_layout(int layout) {
    return layout == MA_LAYOUT_HALF_INTERLEAVED || layout == MA_LAYOUT_FULL_SPLIT || layout == MA_LAYOUT_HALF_PACKED ||
           layout == MA_LAYOUT_HALF_POLAR;
}
// Layouts that use the second array.
// The plain transforms' host forms go through the pipeline from this many bytes per call (pinned arrays,
// at least four transforms); smaller calls copy, transform and copy back on the context's stream.
constexpr size_t kPipelineFromBytes = (size_t)16 << 20;

static bool two_arrays(int layout) { return layout == MA_LAYOUT_FULL_SPLIT || layout == MA_LAYOUT_HALF_POLAR; }

// Output floats per frame in array a / b for a layout.
static int64_t floats_a(int n, int layout) {
    if (layout == MA_LAYOUT_FULL_SPLIT) return n;
    if (layout == MA_LAYOUT_HALF_PACKED) return n;  // N/2 complex
    if (layout == MA_LAYOUT_HALF_POLAR) return n / 2 + 1;
    return 2 * (int64_t)(n / 2 + 1);
}
static int64_t complex_per_frame(int n, int layout) {
    return layout == MA_LAYOUT_HALF_PACKED ? n / 2 : n / 2 + 1;
}

namespace ma {
ma_status check_forward_args(ma_fft_plan* plan, const float* in, const float* out_a, const float* out_b,
                             const float* mag, int mag_kind, int64_t batch, int layout) {
    if (batch < 0 || !valid_layout(layout) || in == nullptr || out_a == nullptr) return MA_ERR_INVALID_ARGUMENT;
    if (two_arrays(layout) && out_b == nullptr) return MA_ERR_INVALID_ARGUMENT;
    if (mag != nullptr && (mag_kind < MA_MAG_MAGNITUDE || mag_kind > MA_MAG_DB)) return MA_ERR_INVALID_ARGUMENT;
    int64_t total;
    if (mul_overflow(batch, plan->n, &total)) return MA_ERR_BATCH_OVERFLOW;
    if (plan->large && layout == MA_LAYOUT_HALF_POLAR) return MA_ERR_UNSUPPORTED;
    return MA_OK;
}
}  // namespace ma

extern "C" {

ma_status ma_fft_plan_create(ma_context* ctx, int32_t n, const float* window, int32_t hop, ma_fft_plan** out) {
    if (out == nullptr) return MA_ERR_INVALID_ARGUMENT;
    *out = nullptr;
    // Validation order of FFT.init (FFT.swift:443-455).
    if (n < 2 || (n & (n - 1)) != 0) return MA_ERR_SIZE_NOT_POW2;
    if (n > (1 << 24)) return MA_ERR_SIZE_TOO_LARGE;
    if (hop <= 0 || hop > n) return MA_ERR_INVALID_HOP;
    MA_TRY(enter(ctx, MA_FAULT_ALLOC));
    ma_fft_plan* p = new (std::nothrow) ma_fft_plan();
    if (p == nullptr) return MA_ERR_ALLOC;
    p->ctx = ctx;
    p->n = n;
    p->m = n / 2;
    p->hop = hop;
    p->large = n > kMaxSmallN;
    ma_status st = MA_OK;
    if (window != nullptr) {
        p->h_window.assign(window, window + n);
        st = upload(ctx, window, sizeof(float) * (size_t)n, (void**)&p->d_window);
    }
    if (st == MA_OK && !p->large && window != nullptr) {
        const std::vector<float> syn = make_synthesis_table(window, p->m);
        if (!syn.empty()) st = upload(ctx, syn.data(), syn.size() * sizeof(float), (void**)&p->d_window_syn);
    }
    if (st == MA_OK && !p->large) {
        cudaError_t e = cudaMalloc((void**)&p->d_norm, 2 * sizeof(float) * (size_t)hop);
        if (e != cudaSuccess) st = cuda_fail(e);
    }
    if (st == MA_OK && !p->large) {
        auto twM = make_stage_tables_for(p->m, false);
        auto twI = make_stage_tables_for(p->m, plan_pairable_rt(p->m));
        auto twN = make_hermitian_table(p->m);
        st = upload(ctx, twM.data(), twM.size() * sizeof(float2), (void**)&p->d_twM);
        if (st == MA_OK) st = upload(ctx, twI.data(), twI.size() * sizeof(float2), (void**)&p->d_twInv);
        if (st == MA_OK) st = upload(ctx, twN.data(), twN.size() * sizeof(float2), (void**)&p->d_twN);
    }
    if (st == MA_OK && p->large) st = large_plan_init(p);
    if (st != MA_OK) {
        ma_fft_plan_destroy(p);
        return st;
    }
    *out = p;
    return MA_OK;
}

ma_status ma_fft_plan_destroy(ma_fft_plan* plan) {
    if (plan == nullptr) return MA_OK;
    if (plan->ctx) {
        (void)cudaSetDevice(plan->ctx->device);
        (void)cudaStreamSynchronize(plan->ctx->stream);
    }
    large_plan_destroy(plan);
    if (plan->d_window) (void)cudaFree(plan->d_window);
    if (plan->d_window_syn) (void)cudaFree(plan->d_window_syn);
    if (plan->d_twM) (void)cudaFree(plan->d_twM);
    if (plan->d_twInv) (void)cudaFree(plan->d_twInv);
    if (plan->d_twN) (void)cudaFree(plan->d_twN);
    if (plan->d_norm) (void)cudaFree(plan->d_norm);
    if (plan->d_cwork) (void)cudaFree(plan->d_cwork);
    (void)cudaGetLastError();
    delete plan;
    return MA_OK;
}

ma_status ma_fft_plan_scratch_bytes(ma_fft_plan* plan, size_t* bytes) {
    if (plan == nullptr || bytes == nullptr) return MA_ERR_INVALID_ARGUMENT;
    *bytes = plan->large ? (size_t)plan->scratch_batch * (size_t)plan->scratch_lanes * (size_t)(plan->n2 / 2 + 1) * plan->n1 * sizeof(float2) : 0;
    return MA_OK;
}

ma_status ma_fft_forward_dev(ma_fft_plan* plan, const float* in, float* out_a, float* out_b, float* mag,
                             int32_t mag_kind, float db_reference, int64_t batch, int32_t layout) {
    if (plan == nullptr) return MA_ERR_INVALID_ARGUMENT;
    MA_TRY(enter(plan->ctx, MA_FAULT_LAUNCH));
    if (batch == 0) return MA_OK;  // empty batch is a no-op (STFT.swift:99-100)
    MA_TRY(check_forward_args(plan, in, out_a, out_b, mag, mag_kind, batch, layout));
    const int64_t total = batch * plan->n;
    const float db_scale = 1.0f / db_reference;
    if (plan->large) return launch_r2c_large(plan, in, out_a, out_b, mag, mag_kind, db_scale, batch, layout);
    R2CParams p{};
    p.in = in;
    p.signal_stride = 0;
    p.frames_per_signal = batch;
    p.total_frames = batch;
    p.signal_len = total;
    p.hop = plan->n;
    p.frame_valid = plan->n;
    p.window = nullptr;
    p.out_a = out_a;
    p.out_b = out_b;
    p.mag = mag;
    p.out_signal_stride = 0;
    p.out_frame_stride = complex_per_frame(plan->n, layout);
    p.layout = layout;
    p.mag_kind = mag_kind;
    p.db_scale = db_scale;
    return launch_r2c_small(plan, p);
}

ma_status ma_fft_inverse_dev(ma_fft_plan* plan, const float* in_a, const float* in_b, float* out, int64_t batch,
                             int32_t layout) {
    if (plan == nullptr) return MA_ERR_INVALID_ARGUMENT;
    MA_TRY(enter(plan->ctx, MA_FAULT_LAUNCH));
    if (batch == 0) return MA_OK;
    if (batch < 0 || !valid_layout(layout) || in_a == nullptr || out == nullptr) return MA_ERR_INVALID_ARGUMENT;
    if (two_arrays(layout) && in_b == nullptr) return MA_ERR_INVALID_ARGUMENT;
    int64_t total;
    if (mul_overflow(batch, plan->n, &total)) return MA_ERR_BATCH_OVERFLOW;
    if (plan->large && layout == MA_LAYOUT_HALF_POLAR) return MA_ERR_UNSUPPORTED;
    if (plan->large) return launch_c2r_large(plan, in_a, in_b, out, batch, layout);
    C2RParams p{};
    p.in_a = in_a;
    p.in_b = in_b;
    p.in_signal_stride = 0;
    p.in_frame_stride = complex_per_frame(plan->n, layout);
    p.frames_per_signal = batch;
    p.n_signals = 1;
    p.layout = layout;
    p.out = out;
    return launch_c2r_small(plan, p);
}

ma_status ma_fft_magnitude_dev(ma_fft_plan* plan, const float* re, const float* im, float* out, int64_t batch,
                               int32_t kind, float db_reference) {
    if (plan == nullptr) return MA_ERR_INVALID_ARGUMENT;
    MA_TRY(enter(plan->ctx, MA_FAULT_LAUNCH));
    if (batch == 0) return MA_OK;
    if (batch < 0 || re == nullptr || im == nullptr || out == nullptr || kind < MA_MAG_MAGNITUDE || kind > MA_MAG_DB)
        return MA_ERR_INVALID_ARGUMENT;
    return launch_magnitude(plan, re, im, out, batch, kind, 1.0f / db_reference);
}

ma_status ma_stft_frame_count(ma_fft_plan* plan, int64_t length, int64_t* frames) {
    if (plan == nullptr || frames == nullptr) return MA_ERR_INVALID_ARGUMENT;
    *frames = 0;
    if (length < plan->n) return MA_ERR_INPUT_TOO_SHORT;
    *frames = (length - plan->n) / plan->hop + 1;
    return MA_OK;
}

ma_status ma_istft_output_length(ma_fft_plan* plan, int64_t frames, int64_t* length) {
    if (plan == nullptr || length == nullptr) return MA_ERR_INVALID_ARGUMENT;
    *length = 0;
    if (frames <= 0) return MA_OK;
    int64_t a, b;
    if (mul_overflow(frames - 1, plan->hop, &a) || add_overflow(a, plan->n, &b)) return MA_ERR_ISTFT_OVERFLOW;
    *length = b;
    return MA_OK;
}

ma_status ma_stft_dev(ma_fft_plan* plan, const float* signals, int64_t length, int64_t signal_stride,
                      int64_t n_signals, float* out_a, float* out_b, float* mag, int32_t mag_kind,
                      float db_reference, int32_t layout) {
    if (plan == nullptr) return MA_ERR_INVALID_ARGUMENT;
    MA_TRY(enter(plan->ctx, MA_FAULT_LAUNCH));
    if (n_signals == 0) return MA_OK;
    if (n_signals < 0 || !valid_layout(layout) || signals == nullptr || out_a == nullptr) return MA_ERR_INVALID_ARGUMENT;
    if (two_arrays(layout) && out_b == nullptr) return MA_ERR_INVALID_ARGUMENT;
    if (mag != nullptr && (mag_kind < MA_MAG_MAGNITUDE || mag_kind > MA_MAG_DB)) return MA_ERR_INVALID_ARGUMENT;
    int64_t frames;
    MA_TRY(ma_stft_frame_count(plan, length, &frames));
    if (n_signals > 1 && signal_stride < length) return MA_ERR_INVALID_ARGUMENT;
    int64_t total, total_out;
    if (mul_overflow(frames, n_signals, &total) || mul_overflow(total, plan->n, &total_out))
        return MA_ERR_BATCH_OVERFLOW;
    if (plan->large) {
        if (layout == MA_LAYOUT_HALF_POLAR) return MA_ERR_UNSUPPORTED;
        return launch_stft_large(plan, signals, signal_stride, frames, n_signals, out_a, out_b, mag, mag_kind,
                                 1.0f / db_reference, layout);
    }
    R2CParams p{};
    p.in = signals;
    p.signal_stride = signal_stride;
    p.frames_per_signal = frames;
    p.total_frames = total;
    p.signal_len = length;
    p.hop = plan->hop;
    p.frame_valid = plan->n;
    p.window = plan->d_window;
    p.out_a = out_a;
    p.out_b = out_b;
    p.mag = mag;
    p.out_frame_stride = complex_per_frame(plan->n, layout);
    p.out_signal_stride = frames * p.out_frame_stride;
    p.layout = layout;
    p.mag_kind = mag_kind;
    p.db_scale = 1.0f / db_reference;
    return launch_r2c_small(plan, p);
}

ma_status ma_istft_dev(ma_fft_plan* plan, const float* in_a, const float* in_b, int64_t frames,
                       int64_t n_signals, float* out, int64_t out_stride, float floor, int32_t layout) {
    if (plan == nullptr) return MA_ERR_INVALID_ARGUMENT;
    MA_TRY(enter(plan->ctx, MA_FAULT_LAUNCH));
    if (frames == 0 || n_signals == 0) return MA_OK;  // frameCount == 0 -> empty output (STFT.swift:389)
    if (frames < 0 || n_signals < 0 || !valid_layout(layout) || in_a == nullptr || out == nullptr)
        return MA_ERR_INVALID_ARGUMENT;
    if (two_arrays(layout) && in_b == nullptr) return MA_ERR_INVALID_ARGUMENT;
    if (!(floor > 0.f)) return MA_ERR_INVALID_ARGUMENT;
    int64_t out_len;
    MA_TRY(ma_istft_output_length(plan, frames, &out_len));
    if (n_signals > 1 && out_stride < out_len) return MA_ERR_INVALID_ARGUMENT;
    int64_t total, total_in;
    if (mul_overflow(frames, n_signals, &total) || mul_overflow(total, plan->n, &total_in))
        return MA_ERR_BATCH_OVERFLOW;
    if (plan->large) {
        if (layout == MA_LAYOUT_HALF_POLAR) return MA_ERR_UNSUPPORTED;
        return launch_istft_large(plan, in_a, in_b, frames, n_signals, out, out_stride, out_len, floor, layout);
    }
    C2RParams p{};
    p.in_a = in_a;
    p.in_b = in_b;
    p.in_frame_stride = complex_per_frame(plan->n, layout);
    p.in_signal_stride = frames * p.in_frame_stride;
    p.frames_per_signal = frames;
    p.n_signals = n_signals;
    p.layout = layout;
    p.hop = plan->hop;
    p.window = plan->d_window;
    p.out = out;
    p.out_signal_stride = out_stride;
    p.out_len = out_len;
    p.floor = floor;
    return launch_istft_small(plan, p);
}

// ------------------------------------------------------------------ host-pointer forms

ma_status ma_fft_forward_host(ma_fft_plan* plan, const float* in, float* out_a, float* out_b, float* mag,
                              int32_t mag_kind, float db_reference, int64_t batch, int32_t layout) {
    if (plan == nullptr) return MA_ERR_INVALID_ARGUMENT;
    ma_context* ctx = plan->ctx;
    MA_TRY(enter(ctx, MA_FAULT_LAUNCH));
    if (batch == 0) return MA_OK;
    if (batch < 0 || !valid_layout(layout) || in == nullptr || out_a == nullptr) return MA_ERR_INVALID_ARGUMENT;
    if (two_arrays(layout) && out_b == nullptr) return MA_ERR_INVALID_ARGUMENT;
    int64_t total;
    if (mul_overflow(batch, plan->n, &total) || total > (int64_t)(std::numeric_limits<int64_t>::max() / 16))
        return MA_ERR_BATCH_OVERFLOW;
    const size_t in_b_ = (size_t)total * sizeof(float);
    const size_t a_b = (size_t)(batch * floats_a(plan->n, layout)) * sizeof(float);
    const size_t b_b = two_arrays(layout) ? a_b : 0;
    const size_t m_b = mag ? (size_t)(batch * (plan->n / 2 + 1)) * sizeof(float) : 0;
    if (batch >= 4 && in_b_ + a_b + b_b + m_b >= kPipelineFromBytes && is_pinned(in) && is_pinned(out_a) &&
        (!b_b || is_pinned(out_b)) && (!m_b || is_pinned(mag))) {
        // Large batches between pinned arrays: chunks of transforms through the three-stage pipeline.
        const int64_t fa = floats_a(plan->n, layout), fm = mag ? plan->n / 2 + 1 : 0;
        const bool two = b_b != 0;
        Pipe pp;
        MA_TRY(pipe_open(pp, ctx, true, batch, sizeof(float) * (size_t)(plan->n + fa + (two ? fa : 0) + fm), 4 * 256));
        for (int64_t b0 = 0, c = 0; b0 < batch && pp.st == MA_OK; b0 += pp.chunk, ++c) {
            const int64_t cb = batch - b0 < pp.chunk ? batch - b0 : pp.chunk;
            char* base = pp.lane[c & 1];
            float* c_in = reinterpret_cast<float*>(base);
            float* c_a = reinterpret_cast<float*>(base + round256(sizeof(float) * (size_t)(pp.chunk * plan->n)));
            float* c_b = two ? c_a + ((pp.chunk * fa + 63) & ~(int64_t)63) : nullptr;
            float* c_m = mag ? (two ? c_b : c_a) + ((pp.chunk * fa + 63) & ~(int64_t)63) : nullptr;
            pp.before_copy_in(c);
            const size_t wi = sizeof(float) * (size_t)(cb * plan->n), wa = sizeof(float) * (size_t)(cb * fa);
            pp.in2d(c_in, wi, in + b0 * plan->n, wi, wi, 1);
            pp.before_kernels(c);
            if (pp.st == MA_OK) pp.st = ma_fft_forward_dev(plan, c_in, c_a, c_b, c_m, mag_kind, db_reference, cb, layout);
            pp.before_copy_out(c);
            pp.out2d(out_a + b0 * fa, wa, c_a, wa, wa, 1);
            if (two) pp.out2d(out_b + b0 * fa, wa, c_b, wa, wa, 1);
            if (mag) pp.out2d(mag + b0 * fm, sizeof(float) * (size_t)(cb * fm), c_m, sizeof(float) * (size_t)(cb * fm),
                              sizeof(float) * (size_t)(cb * fm), 1);
            pp.after_copy_out(c);
        }
        return pp.finish();
    }
    float *d_in = nullptr, *d_a = nullptr, *d_b = nullptr, *d_m = nullptr;
    ma_status st = temp_alloc(ctx, in_b_, (void**)&d_in);
    if (st == MA_OK) st = temp_alloc(ctx, a_b, (void**)&d_a);
    if (st == MA_OK && b_b) st = temp_alloc(ctx, b_b, (void**)&d_b);
    if (st == MA_OK && m_b) st = temp_alloc(ctx, m_b, (void**)&d_m);
    if (st == MA_OK) st = copy_h2d(ctx, d_in, in, in_b_);
    if (st == MA_OK) st = ma_fft_forward_dev(plan, d_in, d_a, d_b, d_m, mag_kind, db_reference, batch, layout);
    if (st == MA_OK) st = copy_d2h(ctx, out_a, d_a, a_b);
    if (st == MA_OK && b_b) st = copy_d2h(ctx, out_b, d_b, b_b);
    if (st == MA_OK && m_b) st = copy_d2h(ctx, mag, d_m, m_b);
    temp_free(ctx, d_in);
    temp_free(ctx, d_a);
    temp_free(ctx, d_b);
    temp_free(ctx, d_m);
    return st;
}

ma_status ma_fft_inverse_host(ma_fft_plan* plan, const float* in_a, const float* in_b, float* out, int64_t batch,
                              int32_t layout) {
    if (plan == nullptr) return MA_ERR_INVALID_ARGUMENT;
    ma_context* ctx = plan->ctx;
    MA_TRY(enter(ctx, MA_FAULT_LAUNCH));
    if (batch == 0) return MA_OK;
    if (batch < 0 || !valid_layout(layout) || in_a == nullptr || out == nullptr) return MA_ERR_INVALID_ARGUMENT;
    if (two_arrays(layout) && in_b == nullptr) return MA_ERR_INVALID_ARGUMENT;
    int64_t total;
    if (mul_overflow(batch, plan->n, &total) || total > (int64_t)(std::numeric_limits<int64_t>::max() / 16))
        return MA_ERR_BATCH_OVERFLOW;
    const size_t a_b = (size_t)(batch * floats_a(plan->n, layout)) * sizeof(float);
    const size_t b_b = two_arrays(layout) ? a_b : 0;
    const size_t o_b = (size_t)total * sizeof(float);
    if (batch >= 4 && a_b + b_b + o_b >= kPipelineFromBytes && is_pinned(in_a) && (!b_b || is_pinned(in_b)) &&
        is_pinned(out)) {
        const int64_t fa = floats_a(plan->n, layout);
        const bool two = b_b != 0;
        Pipe pp;
        MA_TRY(pipe_open(pp, ctx, true, batch, sizeof(float) * (size_t)(fa + (two ? fa : 0) + plan->n), 4 * 256));
        for (int64_t b0 = 0, c = 0; b0 < batch && pp.st == MA_OK; b0 += pp.chunk, ++c) {
            const int64_t cb = batch - b0 < pp.chunk ? batch - b0 : pp.chunk;
            char* base = pp.lane[c & 1];
            float* c_a = reinterpret_cast<float*>(base);
            float* c_b = two ? c_a + ((pp.chunk * fa + 63) & ~(int64_t)63) : nullptr;
            float* c_o = (two ? c_b : c_a) + ((pp.chunk * fa + 63) & ~(int64_t)63);
            pp.before_copy_in(c);
            const size_t wa = sizeof(float) * (size_t)(cb * fa), wo = sizeof(float) * (size_t)(cb * plan->n);
            pp.in2d(c_a, wa, in_a + b0 * fa, wa, wa, 1);
            if (two) pp.in2d(c_b, wa, in_b + b0 * fa, wa, wa, 1);
            pp.before_kernels(c);
            if (pp.st == MA_OK) pp.st = ma_fft_inverse_dev(plan, c_a, c_b, c_o, cb, layout);
            pp.before_copy_out(c);
            pp.out2d(out + b0 * plan->n, wo, c_o, wo, wo, 1);
            pp.after_copy_out(c);
        }
        return pp.finish();
    }
    float *d_a = nullptr, *d_b = nullptr, *d_o = nullptr;
    ma_status st = temp_alloc(ctx, a_b, (void**)&d_a);
    if (st == MA_OK && b_b) st = temp_alloc(ctx, b_b, (void**)&d_b);
    if (st == MA_OK) st = temp_alloc(ctx, o_b, (void**)&d_o);
    if (st == MA_OK) st = copy_h2d(ctx, d_a, in_a, a_b);
    if (st == MA_OK && b_b) st = copy_h2d(ctx, d_b, in_b, b_b);
    if (st == MA_OK) st = ma_fft_inverse_dev(plan, d_a, d_b, d_o, batch, layout);
    if (st == MA_OK) st = copy_d2h(ctx, out, d_o, o_b);
    temp_free(ctx, d_a);
    temp_free(ctx, d_b);
    temp_free(ctx, d_o);
    return st;
}

ma_status ma_fft_magnitude_host(ma_fft_plan* plan, const float* re, const float* im, float* out, int64_t batch,
                                int32_t kind, float db_reference) {
    if (plan == nullptr) return MA_ERR_INVALID_ARGUMENT;
    ma_context* ctx = plan->ctx;
    MA_TRY(enter(ctx, MA_FAULT_LAUNCH));
    if (batch == 0) return MA_OK;
    if (batch < 0 || re == nullptr || im == nullptr || out == nullptr) return MA_ERR_INVALID_ARGUMENT;
    // The reference reads only bins 0..N/2 of each array (FFT.swift:1785-1790); a single
    // frame may therefore be passed with just N/2+1 valid elements.
    const int kh = plan->n / 2 + 1;
    const size_t row = (size_t)plan->n * sizeof(float);
    const size_t in_bytes = batch == 1 ? (size_t)kh * sizeof(float) : (size_t)batch * row;
    const size_t o_b = (size_t)batch * kh * sizeof(float);
    float *d_re = nullptr, *d_im = nullptr, *d_o = nullptr;
    ma_status st = temp_alloc(ctx, (size_t)batch * row, (void**)&d_re);
    if (st == MA_OK) st = temp_alloc(ctx, (size_t)batch * row, (void**)&d_im);
    if (st == MA_OK) st = temp_alloc(ctx, o_b, (void**)&d_o);
    if (st == MA_OK) st = copy_h2d(ctx, d_re, re, in_bytes);
    if (st == MA_OK) st = copy_h2d(ctx, d_im, im, in_bytes);
    if (st == MA_OK) st = ma_fft_magnitude_dev(plan, d_re, d_im, d_o, batch, kind, db_reference);
    if (st == MA_OK) st = copy_d2h(ctx, out, d_o, o_b);
    temp_free(ctx, d_re);
    temp_free(ctx, d_im);
    temp_free(ctx, d_o);
    return st;
}

ma_status ma_stft_host(ma_fft_plan* plan, const float* signals, int64_t length, int64_t signal_stride,
                       int64_t n_signals, float* out_a, float* out_b, float* mag, int32_t mag_kind,
                       float db_reference, int32_t layout) {
    if (plan == nullptr) return MA_ERR_INVALID_ARGUMENT;
    ma_context* ctx = plan->ctx;
    MA_TRY(enter(ctx, MA_FAULT_LAUNCH));
    if (n_signals == 0) return MA_OK;
    if (n_signals < 0 || !valid_layout(layout) || signals == nullptr || out_a == nullptr) return MA_ERR_INVALID_ARGUMENT;
    if (two_arrays(layout) && out_b == nullptr) return MA_ERR_INVALID_ARGUMENT;
    int64_t frames;
    MA_TRY(ma_stft_frame_count(plan, length, &frames));
    if (n_signals > 1 && signal_stride < length) return MA_ERR_INVALID_ARGUMENT;
    int64_t total, total_out;
    if (mul_overflow(frames, n_signals, &total) || mul_overflow(total, 4 * (int64_t)plan->n, &total_out))
        return MA_ERR_BATCH_OVERFLOW;
    // Device copy of a chunk's signals is dense: signal s at s*dlen, dlen a multiple of 4 floats so
    // every row keeps the 16-byte alignment the bulk-staged kernels want.
    const int64_t dlen = (length + 3) & ~(int64_t)3;
    const int64_t fa = frames * floats_a(plan->n, layout);         // floats per signal in array a (and b)
    const int64_t fm = mag ? frames * (plan->n / 2 + 1) : 0;
    const bool two = two_arrays(layout);
    const size_t row_bytes = sizeof(float) * (size_t)(dlen + fa + (two ? fa : 0) + fm);
    const bool pinned = is_pinned(signals) && is_pinned(out_a) && (!two || is_pinned(out_b)) && (!mag || is_pinned(mag));
    Pipe pp;
    MA_TRY(pipe_open(pp, ctx, pinned, n_signals, row_bytes, 4 * 256));
    for (int64_t s0 = 0, c = 0; s0 < n_signals && pp.st == MA_OK; s0 += pp.chunk, ++c) {
        const int64_t cs = n_signals - s0 < pp.chunk ? n_signals - s0 : pp.chunk;
        char* base = pp.lane[c & 1];
        float* d_in = reinterpret_cast<float*>(base);
        float* d_a = reinterpret_cast<float*>(base + round256(sizeof(float) * (size_t)(pp.chunk * dlen)));
        float* d_b = two ? d_a + ((pp.chunk * fa + 63) & ~(int64_t)63) : nullptr;
        float* d_m = mag ? (two ? d_b : d_a) + ((pp.chunk * fa + 63) & ~(int64_t)63) : nullptr;
        pp.before_copy_in(c);
        pp.in2d(d_in, sizeof(float) * (size_t)dlen, signals + s0 * signal_stride, sizeof(float) * (size_t)signal_stride,
                sizeof(float) * (size_t)length, (size_t)cs);
        pp.before_kernels(c);
        if (pp.st == MA_OK)
            pp.st = ma_stft_dev(plan, d_in, length, dlen, cs, d_a, d_b, d_m, mag_kind, db_reference, layout);
        pp.before_copy_out(c);
        const size_t wa = sizeof(float) * (size_t)(cs * fa);
        pp.out2d(out_a + s0 * fa, wa, d_a, wa, wa, 1);
        if (two) pp.out2d(out_b + s0 * fa, wa, d_b, wa, wa, 1);
        if (mag) pp.out2d(mag + s0 * fm, sizeof(float) * (size_t)(cs * fm), d_m, sizeof(float) * (size_t)(cs * fm),
                          sizeof(float) * (size_t)(cs * fm), 1);
        pp.after_copy_out(c);
    }
    return pp.finish();
}

ma_status ma_istft_host(ma_fft_plan* plan, const float* in_a, const float* in_b, int64_t frames,
                        int64_t n_signals, float* out, int64_t out_stride, float floor, int32_t layout) {
    if (plan == nullptr) return MA_ERR_INVALID_ARGUMENT;
    ma_context* ctx = plan->ctx;
    MA_TRY(enter(ctx, MA_FAULT_LAUNCH));
    if (frames == 0 || n_signals == 0) return MA_OK;
    if (frames < 0 || n_signals < 0 || !valid_layout(layout) || in_a == nullptr || out == nullptr)
        return MA_ERR_INVALID_ARGUMENT;
    if (two_arrays(layout) && in_b == nullptr) return MA_ERR_INVALID_ARGUMENT;
    int64_t out_len;
    MA_TRY(ma_istft_output_length(plan, frames, &out_len));
    if (n_signals > 1 && out_stride < out_len) return MA_ERR_INVALID_ARGUMENT;
    int64_t total, total_in;
    if (mul_overflow(frames, n_signals, &total) || mul_overflow(total, 4 * (int64_t)plan->n, &total_in))
        return MA_ERR_BATCH_OVERFLOW;
    const int64_t fa = frames * floats_a(plan->n, layout);
    const bool two = two_arrays(layout);
    const int64_t dol = (out_len + 3) & ~(int64_t)3;  // device row stride of the output
    const size_t row_bytes = sizeof(float) * (size_t)(fa + (two ? fa : 0) + dol);
    const bool pinned = is_pinned(in_a) && (!two || is_pinned(in_b)) && is_pinned(out);
    if (n_signals == 1) out_stride = out_len;
    Pipe pp;
    MA_TRY(pipe_open(pp, ctx, pinned, n_signals, row_bytes, 4 * 256));
    for (int64_t s0 = 0, c = 0; s0 < n_signals && pp.st == MA_OK; s0 += pp.chunk, ++c) {
        const int64_t cs = n_signals - s0 < pp.chunk ? n_signals - s0 : pp.chunk;
        char* base = pp.lane[c & 1];
        float* d_a = reinterpret_cast<float*>(base);
        float* d_b = two ? d_a + ((pp.chunk * fa + 63) & ~(int64_t)63) : nullptr;
        float* d_o = (two ? d_b : d_a) + ((pp.chunk * fa + 63) & ~(int64_t)63);
        pp.before_copy_in(c);
        const size_t wa = sizeof(float) * (size_t)(cs * fa);
        pp.in2d(d_a, wa, in_a + s0 * fa, wa, wa, 1);
        if (two) pp.in2d(d_b, wa, in_b + s0 * fa, wa, wa, 1);
        pp.before_kernels(c);
        if (pp.st == MA_OK) pp.st = ma_istft_dev(plan, d_a, d_b, frames, cs, d_o, dol, floor, layout);
        pp.before_copy_out(c);
        pp.out2d(out + s0 * out_stride, sizeof(float) * (size_t)out_stride, d_o, sizeof(float) * (size_t)dol,
                 sizeof(float) * (size_t)out_len, (size_t)cs);
        pp.after_copy_out(c);
    }
    return pp.finish();
}

}  // extern "C"
