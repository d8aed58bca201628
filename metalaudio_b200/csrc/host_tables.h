// Host-side table generation shared by the library and the CPU emulator.
// Twiddles are evaluated in float64 and rounded once to float32, as the reference does
// for its twiddle LUT (Sources/MetalDSP/FFT.swift:651-665).
#pragma once
#include <cmath>
#include <vector>

#include <cuda_runtime.h>

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
