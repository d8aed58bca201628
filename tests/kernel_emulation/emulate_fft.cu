// CPU execution of the small-FFT kernel bodies through the thread-block emulator.
// TEST INFRASTRUCTURE ONLY (built by tests/test_kernel_emulation.py into a private .so).
#include <cstdint>
#include <cstring>
#include <vector>

#include "../../metalaudio_b200/csrc/fft_kernels.cuh"
#include "../../metalaudio_b200/csrc/host_tables.h"
#include "../../metalaudio_b200/csrc/pconv_tiling.h"
#include "host_cta.h"

using namespace ma;

extern "C" {

// Forward R2C of total_frames frames; returns 0 on success, -1 for an unsupported size.
int emul_r2c(int n, int aligned, const float* in, long long signal_stride, long long frames_per_signal,
             long long total_frames, long long signal_len, int hop, int frame_valid,
             const float* window, float* out_a, float* out_b, float* mag, long long out_signal_stride,
             long long out_frame_stride, int layout, int mag_kind, float db_scale, int nblocks) {
    const int M = n / 2;
    auto twM = make_stage_tables_for(M, false);
    auto twN = make_hermitian_table(M);
    R2CParams p{};
    p.in = in; p.signal_stride = signal_stride; p.frames_per_signal = frames_per_signal;
    p.total_frames = total_frames; p.signal_len = signal_len; p.hop = hop; p.frame_valid = frame_valid;
    p.window = window; p.out_a = out_a; p.out_b = out_b; p.mag = mag;
    p.out_signal_stride = out_signal_stride; p.out_frame_stride = out_frame_stride;
    p.layout = layout; p.mag_kind = mag_kind; p.db_scale = db_scale;
    p.twM = twM.data(); p.twN = twN.data();
    p.bulk_ok = (aligned && hop % 4 == 0 && signal_stride % 4 == 0 && n % 4 == 0) ? 1 : 0;
    int rc = -1;
#define RUN(MM)                                                                              \
    {                                                                                        \
        using S = CtaShape<MM>;                                                              \
        run_grid(nblocks, S::THREADS, S::SMEM_BYTES_PREFETCH, [&](HostCta& cta, void* sm) {  \
            if (aligned && layout == 0 && mag_kind == 0 && mag != nullptr)                   \
                r2c_body<MM, true, 0, 0, HostCta>(p, cta, (float2*)sm);                      \
            else if (aligned) r2c_body<MM, true, -1, -2, HostCta>(p, cta, (float2*)sm);      \
            else r2c_body<MM, false, -1, -2, HostCta>(p, cta, (float2*)sm);                  \
        });                                                                                  \
        rc = 0;                                                                              \
    }
    MA_DISPATCH_M(M, RUN)
#undef RUN
    return rc;
}

int emul_c2r(int n, const float* in_a, const float* in_b, long long in_signal_stride,
             long long in_frame_stride, long long frames_per_signal, long long n_signals, int layout,
             float* out, int nblocks) {
    const int M = n / 2;
    auto twM = make_stage_tables_for(M, plan_pairable_rt(M));
    auto twN = make_hermitian_table(M);
    C2RParams p{};
    p.in_a = in_a; p.in_b = in_b; p.in_signal_stride = in_signal_stride; p.in_frame_stride = in_frame_stride;
    p.frames_per_signal = frames_per_signal; p.n_signals = n_signals; p.layout = layout; p.out = out;
    p.twM = twM.data(); p.twN = twN.data();
    int rc = -1;
#define RUN(MM)                                                                              \
    {                                                                                        \
        using S = CtaShape<MM>;                                                              \
        run_grid(nblocks, S::THREADS, S::SMEM_BYTES_STAGED, [&](HostCta& cta, void* sm) {    \
            if (layout == 0) c2r_body<MM, 0, HostCta>(p, cta, (float2*)sm);                  \
            else c2r_body<MM, -1, HostCta>(p, cta, (float2*)sm);                             \
        });                                                                                  \
        rc = 0;                                                                              \
    }
    MA_DISPATCH_M(M, RUN)
#undef RUN
    return rc;
}

int emul_istft(int n, int hop, const float* in_a, const float* in_b, long long in_signal_stride,
               long long in_frame_stride, long long frames, long long n_signals, int layout,
               const float* window, float floor, float* out, long long out_signal_stride,
               long long out_len, int chunks_per_signal, int nblocks) {
    const int M = n / 2;
    auto twM = make_stage_tables_for(M, plan_pairable_rt(M));
    auto twN = make_hermitian_table(M);
    C2RParams p{};
    p.in_a = in_a; p.in_b = in_b; p.in_signal_stride = in_signal_stride; p.in_frame_stride = in_frame_stride;
    p.frames_per_signal = frames; p.n_signals = n_signals; p.layout = layout; p.hop = hop;
    p.window = window; p.out = out; p.out_signal_stride = out_signal_stride; p.out_len = out_len;
    p.floor = floor; p.chunks_per_signal = chunks_per_signal;
    auto norm = make_norm_table(window, n, hop, floor);
    norm.resize(2 * (size_t)hop);
    for (int r = 0; r < hop; ++r) norm[(size_t)(hop + r)] = 1.0f / norm[(size_t)r];
    p.norm_mid = norm.data();
    p.norm_mid_inv = norm.data() + hop;
    auto syn = make_synthesis_table(window, M);
    p.window_syn = (window != nullptr && !syn.empty()) ? reinterpret_cast<const float4*>(syn.data()) : nullptr;
    p.twM = twM.data(); p.twN = twN.data();
    int rc = -1;
    int used_fast = 0;
#define RUN(MM)                                                                                  \
    {                                                                                            \
        constexpr int ELEMS = smem_elems_per_fft<MM, 1>();                                       \
        const bool fast = istft_fast_ok<MM>(p);                                                  \
        const size_t smem = fast ? (size_t)(2 * MM / hop == 4 ? IstftFastShape<MM, 4>::SMEM_BYTES : IstftFastShape<MM, 0>::SMEM_BYTES) \
                                 : 2 * ELEMS * sizeof(float2) + (size_t)n * sizeof(float);       \
        used_fast = fast ? 1 : 0;                                                                \
        run_grid(nblocks, FftPlan<MM>::T, smem, [&](HostCta& cta, void* sm) {                    \
            if constexpr (plan_pairable<MM>()) {                                                 \
                if (fast && 2 * MM / hop == 4) { istft_fast_body<MM, 0, 4, HostCta>(p, cta, (float2*)sm); return; } \
                if (fast) { istft_fast_body<MM, 0, 0, HostCta>(p, cta, (float2*)sm); return; }   \
            }                                                                                    \
            istft_body<MM, HostCta>(p, cta, (float2*)sm);                                        \
        });                                                                                      \
        rc = 0;                                                                                  \
    }
    MA_DISPATCH_M(M, RUN)
#undef RUN
    return rc == 0 ? used_fast : rc;
}

// Walks the staging schedule of the time-tiled multiply-accumulate for P partitions and t_total
// output blocks (timeline of P - 1 + t_total rows) exactly as the kernel issues it, and counts
//   out_of_bounds: fetches whose source row is outside [0, tl_len),
//   stale:         ring reads that feed a stored output (t < t_total, p < P) but find another
//                  row, or a clamped one, in the slot.
// Returns out_of_bounds + stale (0 = sound); the two counts are written to counts[0..1].
long long emul_tiled_rows(int P, long long t_total, long long* counts) {
    constexpr int TT = 16;
    using TL = MacTiling<TT>;
    const long long tl_len = (long long)P - 1 + t_total;
    long long oob = 0, stale = 0;
    const long long t_ctas = (t_total + TL::kWarps * TT - 1) / (TL::kWarps * TT);
    for (long long y = 0; y < t_ctas; ++y) {
        const long long t0_cta = y * TL::kWarps * TT;
        std::vector<long long> want(TL::kRing, INT64_MIN), got(TL::kRing, INT64_MIN);
        auto stage = [&](long long first, int count) {
            for (int r = 0; r < count; ++r) {
                const long long row = first + r;
                const long long src = TL::fetch_row(row, tl_len);
                if (src < 0 || src >= tl_len) ++oob;
                want[row & (TL::kRing - 1)] = row;
                got[row & (TL::kRing - 1)] = src;
            }
        };
        // a ring read of `row` that feeds output block t at partition p
        auto read = [&](long long row, long long t, long long p) {
            if (t >= t_total || p >= P || p < 0) return;  // never stored / never consumed
            const int slot = (int)(row & (TL::kRing - 1));
            if (want[slot] != row || got[slot] != row) ++stale;
        };
        stage(TL::chunk0_first(P, t0_cta), TL::kChunk0Rows);
        for (int warp = 0; warp < TL::kWarps; ++warp) {
            const long long base = TL::base0(P, t0_cta) + warp * TT, t0 = t0_cta + warp * TT;
            for (int i = 0; i < TT; ++i) read(base + i, t0 + i, 0);  // the initial window
        }
        for (int p0 = 0; p0 < P; p0 += TT) {
            // the kernel issues the look-ahead copies first, but they land in slots the current
            // chunk does not read (checked here by staging them before the reads)
            if (p0 + TT < P) stage(TL::lookahead_first(P, t0_cta, p0), TT);
            for (int warp = 0; warp < TL::kWarps; ++warp) {
                const long long base = TL::base0(P, t0_cta) + warp * TT, t0 = t0_cta + warp * TT;
                for (int j = 0; j < TT; ++j) {
                    const int p = p0 + j;
                    if (p >= P || p == 0) continue;
                    // row base - p enters the window and serves output i at partition p + i
                    for (int i = 0; i < TT; ++i)
                        if (p + i < P && t0 + i < t_total) {
                            read(base - p, t0 + i, p + i);
                            break;  // one genuine consumer is enough to require the row
                        }
                }
            }
        }
    }
    counts[0] = oob;
    counts[1] = stale;
    return oob + stale;
}

}  // extern "C"
