// Host-side table generation shared by the library and the CPU emulator.
// Twiddles are evaluated in float64 and rounded once to float32, as the reference does
// for its twiddle LUT (Sources/MetalDSP/FFT.swift:651-665).
#pragma once
#include <cmath>
#include <vector>

#include <cuda_runtime.h>

#include "fft_core.cuh"

// Compile-time dispatch over the supported in-shared-memory complex lengths.
#define MA_DISPATCH_M(M_VALUE, MACRO)   \
    switch (M_VALUE) {                  \
        case 1: MACRO(1); break;        \
        case 2: MACRO(2); break;        \
        case 4: MACRO(4); break;        \
        case 8: MACRO(8); break;        \
        case 16: MACRO(16); break;      \
        case 32: MACRO(32); break;      \
        case 64: MACRO(64); break;      \
        case 128: MACRO(128); break;    \
        case 256: MACRO(256); break;    \
        case 512: MACRO(512); break;    \
        case 1024: MACRO(1024); break;  \
        case 2048: MACRO(2048); break;  \
        case 4096: MACRO(4096); break;  \
        default: break;                 \
    }

namespace ma {

// exp(-2*pi*i*j/len) for j in [0, count)
inline std::vector<float2> make_twiddles(int64_t len, int64_t count) {
    std::vector<float2> tw((size_t)count);
    const double step = -2.0 * M_PI / (double)len;
    for (int64_t j = 0; j < count; ++j) {
        const double a = step * (double)j;
        tw[(size_t)j] = make_float2((float)std::cos(a), (float)std::sin(a));
    }
    return tw;
}

// Stage twiddle table of plan P in the layout fft_core.cuh documents.
template <class P>
inline std::vector<float2> make_stage_tables() {
    std::vector<float2> tw((size_t)(stage_tw_total<P>() > 0 ? stage_tw_total<P>() : 1), make_float2(1.f, 0.f));
    for (int s = 1; s < P::NS; ++s) {
        const int r = P::radix(s), ns = P::ns_before(s), off = stage_tw_offset<P>(s);
        for (int k = 1; k < r; ++k)
            for (int j = 0; j < ns; ++j) {
                const double a = -2.0 * M_PI * (double)j * (double)k / ((double)ns * (double)r);
                tw[(size_t)(off + (k - 1) * ns + j)] = make_float2((float)std::cos(a), (float)std::sin(a));
            }
    }
    return tw;
}

// Stage tables for complex length m: forward radix order (rev = false) or reversed.
inline std::vector<float2> make_stage_tables_for(int m, bool rev) {
    std::vector<float2> out;
#define MA_TW_CASE(MM) out = rev ? make_stage_tables<FftPlanRev<MM>>() : make_stage_tables<FftPlan<MM>>();
    switch (m) {
        case 1: MA_TW_CASE(1) break;
        case 2: MA_TW_CASE(2) break;
        case 4: MA_TW_CASE(4) break;
        case 8: MA_TW_CASE(8) break;
        case 16: MA_TW_CASE(16) break;
        case 32: MA_TW_CASE(32) break;
        case 64: MA_TW_CASE(64) break;
        case 128: MA_TW_CASE(128) break;
        case 256: MA_TW_CASE(256) break;
        case 512: MA_TW_CASE(512) break;
        case 1024: MA_TW_CASE(1024) break;
        case 2048: MA_TW_CASE(2048) break;
        case 4096: MA_TW_CASE(4096) break;
        default: break;
    }
#undef MA_TW_CASE
    return out;
}

// Twiddles of the Hermitian pre/post-process, exp(-2 pi i idx / (2m)).  Pairable plans index
// them [k][j] -> idx = j + k*NL with NL = m / (last forward radix), j <= NL/2, so that the lanes
// of a warp (consecutive j) load contiguously; other plans use idx = k, k <= m/2.
template <int MM>
inline std::vector<float2> make_hermitian_table_t() {
    const double step = -2.0 * M_PI / (2.0 * (double)MM);
    std::vector<float2> tw;
    if constexpr (plan_pairable<MM>()) {
        constexpr int rl = FftPlan<MM>::radix(FftPlan<MM>::NS - 1), NL = MM / rl;
        tw.resize((size_t)rl * (NL / 2 + 1));
        for (int k = 0; k < rl; ++k)
            for (int j = 0; j <= NL / 2; ++j) {
                const double a = step * (double)(j + k * NL);
                tw[(size_t)(k * (NL / 2 + 1) + j)] = make_float2((float)std::cos(a), (float)std::sin(a));
            }
    } else {
        tw.resize((size_t)(MM / 2 + 1));
        for (int k = 0; k <= MM / 2; ++k)
            tw[(size_t)k] = make_float2((float)std::cos(step * k), (float)std::sin(step * k));
    }
    return tw;
}

inline std::vector<float2> make_hermitian_table(int m) {
    std::vector<float2> out;
    switch (m) {
        case 1: out = make_hermitian_table_t<1>(); break;
        case 2: out = make_hermitian_table_t<2>(); break;
        case 4: out = make_hermitian_table_t<4>(); break;
        case 8: out = make_hermitian_table_t<8>(); break;
        case 16: out = make_hermitian_table_t<16>(); break;
        case 32: out = make_hermitian_table_t<32>(); break;
        case 64: out = make_hermitian_table_t<64>(); break;
        case 128: out = make_hermitian_table_t<128>(); break;
        case 256: out = make_hermitian_table_t<256>(); break;
        case 512: out = make_hermitian_table_t<512>(); break;
        case 1024: out = make_hermitian_table_t<1024>(); break;
        case 2048: out = make_hermitian_table_t<2048>(); break;
        case 4096: out = make_hermitian_table_t<4096>(); break;
        default: break;
    }
    return out;
}

// Runtime form of plan_pairable<M>().
inline bool plan_pairable_rt(int m) {
    switch (m) {
        case 32: return plan_pairable<32>();
        case 64: return plan_pairable<64>();
        case 128: return plan_pairable<128>();
        case 256: return plan_pairable<256>();
        case 512: return plan_pairable<512>();
        case 1024: return plan_pairable<1024>();
        case 2048: return plan_pairable<2048>();
        case 4096: return plan_pairable<4096>();
        default: return false;
    }
}

// Synthesis-window table of the register-ring iSTFT (istft_fast_body with a compile-time overlap
// count): thread t of a frame reads, for q2 < R/2, one 16-byte entry [q2*T + t] =
// (w[2n0+1], w[2n0], w[2n1+1], w[2n1]) / N with n0 = t + 2*q2*T, n1 = n0 + T - the pair order the
// inverse transform leaves its samples in, and the 1/N scale folded in.  2M floats; empty when the
// complex length has no paired plan.  window == nullptr means all ones.
inline std::vector<float> make_synthesis_table(const float* window, int m) {
    std::vector<float> tab;
    int R = 0, T = 0;
#define MA_RT_CASE(MM)                  \
    if (plan_pairable<MM>()) {          \
        R = FftPlan<MM>::R;             \
        T = FftPlan<MM>::T;             \
    }
    MA_DISPATCH_M(m, MA_RT_CASE)
#undef MA_RT_CASE
    if (R < 2) return tab;
    const float scale = 1.0f / (float)(2 * m);
    tab.resize((size_t)(2 * m));
    for (int q2 = 0; q2 < R / 2; ++q2)
        for (int t = 0; t < T; ++t)
            for (int e = 0; e < 2; ++e) {
                const int n = t + (2 * q2 + e) * T;
                float* dst = &tab[(size_t)(4 * (q2 * T + t) + 2 * e)];
                dst[0] = (window ? window[2 * n + 1] : 1.0f) * scale;
                dst[1] = (window ? window[2 * n] : 1.0f) * scale;
            }
    return tab;
}

// Interior window-sum table of the iSTFT normaliser: for an output position with every
// overlapping frame present the sum of squared window depends only on the position modulo
// hop.  Accumulated in float32 in increasing frame order (largest window offset first), as the
// reference's sequential loop adds them, denormal sums zeroed, floor applied
// (Sources/MetalDSP/STFT.swift:474-479, :513-520).  window == nullptr means all ones.
inline std::vector<float> make_norm_table(const float* window, int n, int hop, float floor) {
    std::vector<float> tab((size_t)hop);
    for (int r = 0; r < hop; ++r) {
        float acc = 0.f;
        const int top = r + ((n - 1 - r) / hop) * hop;
        for (int off = top; off >= 0; off -= hop) {
            const float w = window ? window[off] : 1.0f;
            acc += w * w;
        }
        if (acc < 1.17549435e-38f) acc = 0.f;
        tab[(size_t)r] = acc > floor ? acc : floor;
    }
    return tab;
}

}  // namespace ma
