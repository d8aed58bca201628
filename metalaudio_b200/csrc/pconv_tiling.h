// Row arithmetic of the time-tiled multiply-accumulate (pconv_mac_tiled_kernel), kept apart from
// the kernel so the test-suite can walk exactly the same index computations on the CPU.
//
// The timeline of a channel holds tl_len = P - 1 + T rows: P - 1 rows of history, then the T block
// spectra of the call.  Output block t, partition p reads timeline row (P - 1) + t - p.  A CTA
// covers kWarps*TT consecutive outputs starting at t0_cta; it stages timeline rows in a ring of
// kRing rows, a chunk of TT partitions ahead of their use.
#pragma once
#include <stdint.h>

#include "fft_core.cuh"

namespace ma {

template <int TT>
struct MacTiling {
    static constexpr int kWarps = 4;
    static constexpr int kRing = 128;
    static constexpr int kChunk0Rows = kWarps * TT - 1 + TT;  // rows staged before the first chunk
    static_assert(kWarps * TT - 1 + 2 * TT <= kRing, "timeline ring too small");

    // Timeline row of the CTA's first output at partition 0.
    static MA_HD int64_t base0(int P, int64_t t0_cta) { return (int64_t)(P - 1) + t0_cta; }
    // First row of the kChunk0Rows rows staged up front: chunk 0 consumes [base0-TT+1, base0+kWarps*TT-1].
    static MA_HD int64_t chunk0_first(int P, int64_t t0_cta) { return base0(P, t0_cta) - TT + 1; }
    // First of the TT rows staged while chunk p0 is consumed (they serve chunk p0 + TT).
    static MA_HD int64_t lookahead_first(int P, int64_t t0_cta, int p0) { return base0(P, t0_cta) - p0 - 2 * TT + 1; }
    // Row actually fetched for staged row `row`.  Rows past the end feed outputs that are never
    // stored; rows before the start belong to partitions >= P that are never consumed: both are
    // clamped into the channel's own timeline, so no fetch leaves [0, tl_len).
    static MA_HD int64_t fetch_row(int64_t row, int64_t tl_len) {
        if (row > tl_len - 1) row = tl_len - 1;
        if (row < 0) row = 0;
        return row;
    }
};

}  // namespace ma
