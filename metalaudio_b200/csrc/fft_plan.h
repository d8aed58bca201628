// FFT plan object and the internal launch entry points other translation units use.
#pragma once
#include <vector>

#include "fft_kernels.cuh"
#include "ma_internal.h"

struct ma_fft_plan {
    ma_context* ctx = nullptr;
    int n = 0;        // real transform size N
    int m = 0;        // complex length N/2
    int hop = 0;
    bool large = false;         // N > 8192: multi-pass path
    float* d_window = nullptr;  // N floats or nullptr
    float* d_window_syn = nullptr;  // the same window in the register-ring iSTFT's thread order, times 1/N (paired plans)
    float2* d_twM = nullptr;    // stage twiddle tables, forward radix order (fft_core.cuh layout)
    float2* d_twInv = nullptr;  // stage tables the inverse kernels use (reversed order when pairable)
    float2* d_twN = nullptr;    // small path: exp(-2 pi i k/N), k <= M/2
    std::vector<float> h_window;  // host copy of the window (empty: none)
    float* d_norm = nullptr;    // iSTFT interior normaliser, hop floats (see launch_istft_small)
    float norm_floor = -1.0f;   // floor the table was built for
    // large path (N = n1 * n2): see fft_large.cu
    int n1 = 0, n2 = 0;
    ma_fft_plan* sub_cols = nullptr;  // tables for the n2-point real transforms
    float2* d_tw1 = nullptr;          // exp(-2 pi i j/n1), j < n1
    float2* d_twc = nullptr;          // pass twiddles in the column pass's layout
    float2* d_twr = nullptr;          // pass twiddles in the row passes' layout, then their steps
    float2* d_scratch = nullptr;      // (n2/2+1) x n1 complex per transform in a pass
    int64_t scratch_batch = 0;        // transforms one lane of the scratch holds
    int scratch_lanes = 1;            // lanes (chunks in flight on separate streams)
    float* d_frames = nullptr;        // iSTFT above 8192 points: scratch_batch inverse frames (allocated on first use)
    float* d_cwork = nullptr;         // complex-input transforms: real rows + half spectra of one chunk (allocated on first use)
};

namespace ma {

constexpr int kMaxSmallN = 8192;

// Queue the forward / inverse / iSTFT kernels for N <= 8192.  Parameters carry device
// pointers; tables are filled in from the plan.
ma_status launch_r2c_small(ma_fft_plan* plan, R2CParams p);
ma_status launch_c2r_small(ma_fft_plan* plan, C2RParams p);
ma_status launch_istft_small(ma_fft_plan* plan, C2RParams p);

// Large path (N > 8192), contiguous frames only.
ma_status large_plan_init(ma_fft_plan* plan);
void large_plan_destroy(ma_fft_plan* plan);
// `scratch` != nullptr: pass data goes through that buffer, `scratch_batch` transforms at a time,
// instead of the plan's own allocation.
ma_status launch_r2c_large(ma_fft_plan* plan, const float* in, float* out_a, float* out_b, float* mag,
                           int mag_kind, float db_scale, int64_t batch, int layout, float2* scratch = nullptr,
                           int64_t scratch_batch = 0);
// Argument checks of the batched forward transform (batch > 0), shared by every entry point that
// runs it: pointers, layout, magnitude kind, batch * N overflow, layouts the large path lacks.
ma_status check_forward_args(ma_fft_plan* plan, const float* in, const float* out_a, const float* out_b,
                             const float* mag, int mag_kind, int64_t batch, int layout);
ma_status launch_c2r_large(ma_fft_plan* plan, const float* in_a, const float* in_b, float* out,
                           int64_t batch, int layout);
// STFT / iSTFT above 8192 points (fft_large.cu): frames are read straight from the signal with
// the window applied by the loader; inverse frames pass through d_frames and are overlap-added in
// frame order, then normalised.
ma_status launch_stft_large(ma_fft_plan* plan, const float* signals, int64_t signal_stride, int64_t frames,
                            int64_t n_signals, float* out_a, float* out_b, float* mag, int mag_kind,
                            float db_scale, int layout);
ma_status launch_istft_large(ma_fft_plan* plan, const float* in_a, const float* in_b, int64_t frames,
                             int64_t n_signals, float* out, int64_t out_stride, int64_t out_len, float floor,
                             int layout);
// Convolution through a large plan with the spectrum kept on chip (fft_large.cu).
ma_status launch_spec_rows_large(ma_fft_plan* plan, const float* in, int64_t valid, float2* spec_rows);
ma_status launch_conv_large(ma_fft_plan* plan, const float* in, int64_t valid, int64_t in_stride,
                            const float2* spec_rows, float* out, int64_t batch);

}  // namespace ma
