// Multichannel biquad cascades (Direct Form II Transposed), parallel in time.
//
// Replaces the reference's biquad_filter_multichannel shader (Sources/MetalDSP/Shaders/DSP.metal:
// 709-744; one thread walks a whole channel sample by sample) and the per-filter loops of
// BiquadFilter.process / FilterBank.processSeries / processParallel
// (Sources/MetalDSP/Filters.swift:515-660, :845-868).  Same recurrence per section,
//     y = b0*x + z1;   z1 = b1*x - a1*y + z2;   z2 = b2*x - a2*y,
// same [channel][sample] layout and per-channel (z1, z2) state that survives between calls.
//
// The recurrence is linear in (state, input): the state after a block of samples is
//     s_end = A^len * s_init + e0,     A = [[-a1, 1], [-a2, 0]] (zero-input state transition),
// e0 being the end state reached from a zero state.  One CTA of 256 threads owns a channel and
// walks it in tiles of 8192 samples; every thread first runs its 32 consecutive samples from a
// zero state to get e0, the end states are combined by a warp scan (powers of A^32 from a
// host-built table) and a short serial pass over the 8 warps, which gives every thread the true
// state in front of its samples; it then runs the recurrence again from that state and keeps the
// outputs.  States and recurrences are double precision (see biquad_kernel), data is float32.
// Cascaded sections run back to back on the registers.  Cascades of three and more sections use a
// variant with 16 samples per thread that keeps the data in double precision from one section to
// the next (the float <-> double conversions, 16 per clock and SM, otherwise cost more than the
// recurrences themselves).  Loads and stores of a tile are contiguous;
// the tile is re-indexed through swizzled shared memory, and the next tile is fetched
// asynchronously while the current one is filtered.
#include <cuda_pipeline.h>

#include <cmath>
#include <new>
#include <type_traits>
#include <vector>

#include "ma_internal.h"

namespace ma {

constexpr int kBqThreads = 256, kBqWarps = kBqThreads / 32;
// samples per thread: 32 for short cascades (data exchanged between sections as float32, like the
// reference's arrays), 16 for cascades kept in double precision (the doubles need the registers)
constexpr int kBqPerShort = 32, kBqPerLong = 16, kBqLongFrom = 3;
constexpr int kBqMaxSections = 32;
// Table of one (coefficient set, section), doubles:
//   [0..4]     b0 b1 b2 a1 a2 (the float32 coefficients, widened)
//   [5..6]     c1 = b1 - a1*b0, c2 = b2 - a2*b0 (the state update with the output substituted)
//   [8..135]   A^(PER*l) row-major 2x2, l < 32 (PER: samples per thread)
//   [136..139] A^(PER*32)
//   [140..171] A^(PER*32*w), w < 8: a warp's worth of samples, w times over
constexpr int kBqCoef = 0, kBqPl = 8, kBqPw = 136, kBqPx = 140, kBqTable = 172;

struct BiquadLaunch {
    const float* in;
    float* out;
    int64_t in_stride, out_stride, samples;
    const double* tables;         // [n_sets][n_sections][kBqTable]
    const int32_t* channel_to_set;
    float2* state;                // [n_channels][n_sections]
    int32_t n_sections;
};

__device__ __forceinline__ double2 mat_vec(const double* m, double2 v) {
    return make_double2(fma(m[0], v.x, m[1] * v.y), fma(m[2], v.x, m[3] * v.y));
}

// Tile layout in shared memory: 16-byte chunks of four samples; chunk c of row r (a row is 32
// consecutive samples: one thread's, or two threads' in the 16-sample variant) sits at column c ^ (r & 7).  Both access patterns are then conflict-free
// with 16-byte accesses: a thread walking its own row, and consecutive threads touching
// consecutive chunks of the signal.
__device__ __forceinline__ int swizzled(int i) {
    const int g = i >> 2, r = g >> 3;
    return (((r << 3) | ((g & 7) ^ (r & 7))) << 2) | (i & 3);
}

// Why double precision inside: a thread restarts the recurrence every 32 samples.  In float32 the
// rounding drift of one block and the freshly computed state of the next do not line up, which
// leaves a small step at every block boundary; a later section that rejects the band the signal
// lives in (high-pass after low-pass) passes those steps unattenuated, and the result ends up an
// order of magnitude further from the exact filter than the serial float32 walk.  With the state
// in double the steps vanish and every section's output is the exact filter's, rounded once to
// float32 (the precision sections exchange data in, as the reference's float arrays do).
template <int kBqPer, bool DBL>
__global__ void __launch_bounds__(kBqThreads, 2) biquad_kernel(const BiquadLaunch p) {
    constexpr int kBqTile = kBqThreads * kBqPer;
    using X = typename std::conditional<DBL, double, float>::type;  // how a thread holds its samples between sections
    extern __shared__ __align__(16) double bq_smem[];
    double* tab = bq_smem;                                              // n_sections * kBqTable
    double2* warp_end = reinterpret_cast<double2*>(tab + p.n_sections * kBqTable);  // [2][kBqWarps]
    double2* carry = warp_end + 2 * kBqWarps;                           // [2][n_sections]: read one, write the other
    float* tiles = reinterpret_cast<float*>(carry + 2 * p.n_sections);  // two tiles: one in use, one being filled
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int64_t ch = blockIdx.x;
    const int set = p.channel_to_set != nullptr ? p.channel_to_set[ch] : 0;
    const double* gtab = p.tables + (int64_t)set * p.n_sections * kBqTable;
    for (int i = tid; i < p.n_sections * kBqTable; i += kBqThreads) tab[i] = __ldg(gtab + i);
    for (int s = tid; s < p.n_sections; s += kBqThreads) {
        const float2 z = p.state[ch * p.n_sections + s];
        carry[s] = make_double2((double)z.x, (double)z.y);
    }
    const float* in = p.in + ch * p.in_stride;
    float* out = p.out + ch * p.out_stride;
    const bool vec_in = (reinterpret_cast<uintptr_t>(in) & 15) == 0;
    const bool vec_out = (reinterpret_cast<uintptr_t>(out) & 15) == 0;
    __syncthreads();

    constexpr int kTileFloats = kBqTile;
    // Full, 16-byte aligned tiles are fetched one iteration ahead with asynchronous 16-byte copies
    // (global -> shared without passing through registers), so the load latency of tile i+1 is
    // spent while tile i is filtered.
    auto prefetch = [&](int64_t base, float* dst) {
#pragma unroll
        for (int k = 0; k < kBqPer / 4; ++k) {
            const int i = 4 * (tid + k * kBqThreads);
            __pipeline_memcpy_async(dst + swizzled(i), in + base + i, 16);
        }
        __pipeline_commit();
    };
    auto full_tile = [&](int64_t base) { return vec_in && base + kBqTile <= p.samples; };
    bool fetched = false;
    if (p.samples > 0 && full_tile(0)) {
        prefetch(0, tiles);
        fetched = true;
    }
    int par = 0;
    for (int64_t base = 0; base < p.samples; base += kBqTile, par ^= 1) {
        float* tile = tiles + par * kTileFloats;
        const double2* carry_in = carry + par * p.n_sections;
        double2* carry_out = carry + (par ^ 1) * p.n_sections;
        const int64_t left = p.samples - base;
        const int valid = left < kBqTile ? (int)left : kBqTile;
        // ---- this tile: already on its way, or loaded here (ragged / unaligned: zeros beyond the end)
        if (fetched) {
            __pipeline_wait_prior(0);
        } else {
#pragma unroll 4
            for (int k = 0; k < kBqPer; ++k) {
                const int i = tid + k * kBqThreads;
                tile[swizzled(i)] = i < valid ? __ldcs(in + base + i) : 0.f;
            }
        }
        // ---- next tile: start it now (its buffer was last read two iterations ago, before the barriers since)
        fetched = false;
        if (base + kBqTile < p.samples && full_tile(base + kBqTile)) {
            prefetch(base + kBqTile, tiles + (par ^ 1) * kTileFloats);
            fetched = true;
        }
        __syncthreads();
        X x[kBqPer];
#pragma unroll
        for (int k = 0; k < kBqPer / 4; ++k) {
            const int g = tid * (kBqPer / 4) + k, r = g >> 3;  // 16-byte chunk g of the tile: row r, column g & 7
            const float4 v = reinterpret_cast<const float4*>(tile)[(r << 3) | ((g & 7) ^ (r & 7))];
            x[4 * k] = (X)v.x; x[4 * k + 1] = (X)v.y; x[4 * k + 2] = (X)v.z; x[4 * k + 3] = (X)v.w;
        }
        const bool last_tile = left <= kBqTile;
        const int last_local = valid - 1 - tid * kBqPer;  // index of the signal's last sample in this thread
        const bool owns_last = last_tile && last_local >= 0 && last_local < kBqPer;

        for (int s = 0; s < p.n_sections; ++s) {
            const double* T = tab + s * kBqTable;
            // With y = b0*x + z1 substituted, the state update is
            //     z1' = -a1*z1 + (z2 + c1*x),   z2' = -a2*z1 + c2*x,
            // one dependent multiply-add per sample instead of two (the output is off the chain).
            // In double precision the rearrangement changes nothing at float32 output level.
            const double b0 = T[0], a1 = T[3], a2 = T[4], c1 = T[5], c2 = T[6];
            // ---- zero-state pass over this thread's samples: only its end state is kept
            double z1 = 0.0, z2 = 0.0;
#pragma unroll
            for (int j = 0; j < kBqPer; ++j) {
                const double xv = (double)x[j];
                const double z1n = fma(-a1, z1, fma(c1, xv, z2));
                z2 = fma(-a2, z1, c2 * xv);
                z1 = z1n;
            }
            // ---- inclusive scan of the end states across the warp: E_l = P*E_{l-1} + e_l, P = A^32
            double2 e = make_double2(z1, z2);
#pragma unroll
            for (int d = 0; d < 5; ++d) {
                const double2 up = make_double2(__shfl_up_sync(0xffffffffu, e.x, 1 << d),
                                                __shfl_up_sync(0xffffffffu, e.y, 1 << d));
                if (lane >= (1 << d)) {
                    const double2 m = mat_vec(T + kBqPl + 4 * (1 << d), up);
                    e.x += m.x;
                    e.y += m.y;
                }
            }
            double2* wend = warp_end + (s & 1) * kBqWarps;
            if (lane == 31) wend[warp] = e;
            __syncthreads();
            // ---- carry into this warp.  32-sample variant: every warp does the same work (a serial walk
            // over the warps before it made the last warp the one all others wait for at the next barrier):
            // lane v < 8 takes warp v's end state, an inclusive scan over those lanes with A^(W*2^d), W a
            // warp's worth of samples, and the tile's incoming state advanced by A^(W*warp).  Measured 5 %
            // faster with one section; the 16-sample variant (whose sections are short) measured 12 %
            // slower that way and keeps the serial walk.
            static_assert(kBqWarps == 8, "the cross-warp scan below covers eight warps");
            double2 c;
            if constexpr (!DBL) {
                double2 ev = lane < kBqWarps ? wend[lane] : make_double2(0.0, 0.0);
#pragma unroll
                for (int d = 0; d < 3; ++d) {
                    const double2 up = make_double2(__shfl_up_sync(0xffffffffu, ev.x, 1 << d),
                                                    __shfl_up_sync(0xffffffffu, ev.y, 1 << d));
                    if (lane >= (1 << d) && lane < kBqWarps) {
                        const double2 m = mat_vec(T + kBqPx + 4 * (1 << d), up);
                        ev.x += m.x;
                        ev.y += m.y;
                    }
                }
                const int src = warp > 0 ? warp - 1 : 0;
                c = make_double2(__shfl_sync(0xffffffffu, ev.x, src), __shfl_sync(0xffffffffu, ev.y, src));
                if (warp == 0) c = make_double2(0.0, 0.0);
                const double2 m = mat_vec(T + kBqPx + 4 * warp, carry_in[s]);
                c.x += m.x;
                c.y += m.y;
            } else {
                c = carry_in[s];
                for (int w = 0; w < warp; ++w) {
                    const double2 m = mat_vec(T + kBqPw, c);
                    c = make_double2(m.x + wend[w].x, m.y + wend[w].y);
                }
            }
            double2 prev = make_double2(__shfl_up_sync(0xffffffffu, e.x, 1), __shfl_up_sync(0xffffffffu, e.y, 1));
            if (lane == 0) prev = make_double2(0.0, 0.0);
            const double2 pc = mat_vec(T + kBqPl + 4 * lane, c);
            // ---- second pass from the true state in front of this thread's samples; the thread
            // that holds the signal's last sample also records the state after it
            double s1 = prev.x + pc.x, s2 = prev.y + pc.y;
            double f1 = 0.0, f2 = 0.0;
            // CAPTURE (the signal's last tile only): remember the state right after sample last_local
            auto second_pass = [&](auto capture) {
                constexpr bool CAPTURE = decltype(capture)::value;
#pragma unroll
                for (int j = 0; j < kBqPer; ++j) {
                    const double xv = (double)x[j];
                    const double yv = fma(b0, xv, s1);
                    const double s1n = fma(-a1, s1, fma(c1, xv, s2));
                    s2 = fma(-a2, s1, c2 * xv);
                    s1 = s1n;
                    x[j] = (X)yv;  // input of the next section
                    if (CAPTURE && j == last_local) {
                        f1 = s1;
                        f2 = s2;
                    }
                }
            };
            if (last_tile) second_pass(std::true_type{});
            else second_pass(std::false_type{});
            if (owns_last) {
                // results below the smallest normal are stored as zero (DSP.metal:736-740)
                float g1 = (float)f1, g2 = (float)f2;
                if (fabsf(g1) < 1.17549435e-38f) g1 = 0.f;
                if (fabsf(g2) < 1.17549435e-38f) g2 = 0.f;
                p.state[ch * p.n_sections + s] = make_float2(g1, g2);
            }
            // carry for the next tile: the state the last thread ends in
            if (!last_tile && tid == kBqThreads - 1) carry_out[s] = make_double2(s1, s2);
        }
        // ---- contiguous store through the same tile
#pragma unroll
        for (int k = 0; k < kBqPer / 4; ++k) {
            const int g = tid * (kBqPer / 4) + k, r = g >> 3;
            reinterpret_cast<float4*>(tile)[(r << 3) | ((g & 7) ^ (r & 7))] =
                make_float4((float)x[4 * k], (float)x[4 * k + 1], (float)x[4 * k + 2], (float)x[4 * k + 3]);
        }
        __syncthreads();
        if (vec_out && valid == kBqTile) {
#pragma unroll
            for (int k = 0; k < kBqPer / 4; ++k) {
                const int i = 4 * (tid + k * kBqThreads);
                __stcs(reinterpret_cast<float4*>(out + base + i), *reinterpret_cast<const float4*>(tile + swizzled(i)));
            }
        } else {
#pragma unroll 4
            for (int k = 0; k < kBqPer; ++k) {
                const int i = tid + k * kBqThreads;
                if (i < valid) __stcs(out + base + i, tile[swizzled(i)]);
            }
        }
        __syncthreads();  // the tile and the carries are reused by the next iteration
    }
}

// out[n] = (sum over channels, in channel order) * scale: FilterBank.processParallel's mix.
__global__ void __launch_bounds__(256) channel_mix_kernel(const float* __restrict__ in, int32_t n_channels, int64_t stride,
                                                          int64_t samples, float scale, float* __restrict__ out) {
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < samples; i += (int64_t)gridDim.x * blockDim.x) {
        float acc = 0.f;
        for (int32_t c = 0; c < n_channels; ++c) acc += in[c * stride + i];
        out[i] = acc * scale;
    }
}

// Builds the table of one section in double precision from float32 coefficients.
static void build_table(const float* c, double* t, int per) {
    for (int i = 0; i < kBqTable; ++i) t[i] = 0.0;
    for (int i = 0; i < 5; ++i) t[kBqCoef + i] = (double)c[i];
    const double a1 = c[3], a2 = c[4];
    t[5] = (double)c[1] - a1 * (double)c[0];
    t[6] = (double)c[2] - a2 * (double)c[0];
    auto mul = [](const double* a, const double* b, double* r) {
        const double r0 = a[0] * b[0] + a[1] * b[2], r1 = a[0] * b[1] + a[1] * b[3];
        const double r2 = a[2] * b[0] + a[3] * b[2], r3 = a[2] * b[1] + a[3] * b[3];
        r[0] = r0; r[1] = r1; r[2] = r2; r[3] = r3;
    };
    const double A[4] = {-a1, 1.0, -a2, 0.0};
    double P[4] = {1.0, 0.0, 0.0, 1.0};
    for (int n = 0; n < per; ++n) mul(A, P, P);  // A^per
    double pl[4] = {1.0, 0.0, 0.0, 1.0};
    for (int l = 0; l < 32; ++l) {
        for (int i = 0; i < 4; ++i) t[kBqPl + 4 * l + i] = pl[i];
        mul(P, pl, pl);
    }
    for (int i = 0; i < 4; ++i) t[kBqPw + i] = pl[i];  // A^(32*per)
    double px[4] = {1.0, 0.0, 0.0, 1.0};
    for (int w = 0; w < kBqWarps; ++w) {
        for (int i = 0; i < 4; ++i) t[kBqPx + 4 * w + i] = px[i];
        mul(pl, px, px);
    }
}

}  // namespace ma

using namespace ma;

struct ma_biquad {
    ma_context* ctx = nullptr;
    int32_t channels = 0, sections = 0, sets = 0;
    double* d_tables = nullptr;
    int32_t* d_map = nullptr;
    float2* d_state = nullptr;
    bool smem_raised = false;
    int per = kBqPerShort;  // samples per thread: the kernel variant, fixed by the section count
};

static size_t biquad_smem(int sections, int per) {
    return sizeof(float) * (size_t)(2 * kBqThreads * per) + sizeof(double) * (size_t)(sections * kBqTable) +
           sizeof(double2) * (size_t)(2 * kBqWarps + 2 * sections);
}

extern "C" {

ma_status ma_biquad_create(ma_context* ctx, int32_t n_channels, int32_t n_sections, ma_biquad** out) {
    if (out == nullptr) return MA_ERR_INVALID_ARGUMENT;
    *out = nullptr;
    if (ctx == nullptr || n_channels <= 0 || n_sections <= 0 || n_sections > kBqMaxSections) return MA_ERR_INVALID_ARGUMENT;
    MA_TRY(enter(ctx, MA_FAULT_ALLOC));
    ma_biquad* bq = new (std::nothrow) ma_biquad();
    if (bq == nullptr) return MA_ERR_ALLOC;
    bq->ctx = ctx;
    bq->channels = n_channels;
    bq->sections = n_sections;
    bq->per = n_sections >= kBqLongFrom ? kBqPerLong : kBqPerShort;
    cudaError_t e = cudaMalloc((void**)&bq->d_state, sizeof(float2) * (size_t)n_channels * n_sections);
    if (e == cudaSuccess) e = cudaMemsetAsync(bq->d_state, 0, sizeof(float2) * (size_t)n_channels * n_sections, ctx->stream);  // ordered before the first kernel of the context
    if (e != cudaSuccess) {
        ma_biquad_destroy(bq);
        return cuda_fail(e);
    }
    *out = bq;
    return MA_OK;
}

ma_status ma_biquad_destroy(ma_biquad* bq) {
    if (bq == nullptr) return MA_OK;
    if (bq->d_tables) (void)cudaFree(bq->d_tables);
    if (bq->d_map) (void)cudaFree(bq->d_map);
    if (bq->d_state) (void)cudaFree(bq->d_state);
    delete bq;
    return MA_OK;
}

ma_status ma_biquad_set_coefficients(ma_biquad* bq, const float* coeffs, int32_t n_sets, const int32_t* channel_to_set) {
    if (bq == nullptr || coeffs == nullptr || n_sets <= 0) return MA_ERR_INVALID_ARGUMENT;
    if (channel_to_set == nullptr && n_sets != 1) return MA_ERR_INVALID_ARGUMENT;
    ma_context* ctx = bq->ctx;
    MA_TRY(enter(ctx, MA_FAULT_ALLOC));
    for (int64_t i = 0; i < (int64_t)n_sets * bq->sections * 5; ++i)
        if (!std::isfinite(coeffs[i])) return MA_ERR_INVALID_ARGUMENT;
    if (channel_to_set != nullptr)
        for (int32_t c = 0; c < bq->channels; ++c)
            if (channel_to_set[c] < 0 || channel_to_set[c] >= n_sets) return MA_ERR_INVALID_ARGUMENT;
    std::vector<double> tables((size_t)n_sets * bq->sections * kBqTable);
    for (int64_t i = 0; i < (int64_t)n_sets * bq->sections; ++i) build_table(coeffs + 5 * i, tables.data() + kBqTable * i, bq->per);
    MA_TRY(ma_context_sync(ctx, 30.0));  // nothing in flight may still read the old tables
    if (bq->d_tables) (void)cudaFree(bq->d_tables);
    if (bq->d_map) (void)cudaFree(bq->d_map);
    bq->d_tables = nullptr;
    bq->d_map = nullptr;
    MA_CUDA(cudaMalloc((void**)&bq->d_tables, tables.size() * sizeof(double)));
    MA_TRY(copy_h2d(ctx, bq->d_tables, tables.data(), tables.size() * sizeof(double)));
    if (channel_to_set != nullptr) {
        MA_CUDA(cudaMalloc((void**)&bq->d_map, sizeof(int32_t) * (size_t)bq->channels));
        MA_TRY(copy_h2d(ctx, bq->d_map, channel_to_set, sizeof(int32_t) * (size_t)bq->channels));
    }
    bq->sets = n_sets;
    return ma_context_sync(ctx, 30.0);
}

ma_status ma_biquad_process_dev(ma_biquad* bq, const float* in, int64_t in_stride, float* out, int64_t out_stride,
                                int64_t samples) {
    if (bq == nullptr) return MA_ERR_INVALID_ARGUMENT;
    ma_context* ctx = bq->ctx;
    MA_TRY(enter(ctx, MA_FAULT_LAUNCH));
    if (bq->d_tables == nullptr) return MA_ERR_KERNEL_NOT_CONFIGURED;
    if (samples == 0) return MA_OK;
    if (samples < 0 || in == nullptr || out == nullptr || in_stride < 0) return MA_ERR_INVALID_ARGUMENT;
    if (bq->channels > 1 && out_stride < samples) return MA_ERR_INVALID_ARGUMENT;
    if (in_stride != 0 && bq->channels > 1 && in_stride < samples) return MA_ERR_INVALID_ARGUMENT;
    const size_t smem = biquad_smem(bq->sections, bq->per);
    const bool long_cascade = bq->per == kBqPerLong;
    if (!bq->smem_raised) {
        if (long_cascade)
            MA_CUDA(cudaFuncSetAttribute(biquad_kernel<kBqPerLong, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)biquad_smem(kBqMaxSections, kBqPerLong)));
        else
            MA_CUDA(cudaFuncSetAttribute(biquad_kernel<kBqPerShort, false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)biquad_smem(kBqMaxSections, kBqPerShort)));
        bq->smem_raised = true;
    }
    BiquadLaunch p{};
    p.in = in;
    p.out = out;
    p.in_stride = in_stride;
    p.out_stride = out_stride;
    p.samples = samples;
    p.tables = bq->d_tables;
    p.channel_to_set = bq->d_map;
    p.state = bq->d_state;
    p.n_sections = bq->sections;
    if (long_cascade) biquad_kernel<kBqPerLong, true><<<(unsigned)bq->channels, kBqThreads, smem, ctx->stream>>>(p);
    else biquad_kernel<kBqPerShort, false><<<(unsigned)bq->channels, kBqThreads, smem, ctx->stream>>>(p);
    return after_launch(ctx);
}

ma_status ma_biquad_process_host(ma_biquad* bq, const float* in, int64_t in_stride, float* out, int64_t out_stride,
                                 int64_t samples) {
    if (bq == nullptr) return MA_ERR_INVALID_ARGUMENT;
    ma_context* ctx = bq->ctx;
    MA_TRY(enter(ctx, MA_FAULT_LAUNCH));
    if (bq->d_tables == nullptr) return MA_ERR_KERNEL_NOT_CONFIGURED;
    if (samples == 0) return MA_OK;
    if (samples < 0 || in == nullptr || out == nullptr || in_stride < 0) return MA_ERR_INVALID_ARGUMENT;
    const int C = bq->channels;
    if (C > 1 && (out_stride < samples || (in_stride != 0 && in_stride < samples))) return MA_ERR_INVALID_ARGUMENT;
    const int in_rows = in_stride == 0 ? 1 : C;
    float *d_in = nullptr, *d_out = nullptr;
    ma_status st = temp_alloc(ctx, sizeof(float) * (size_t)samples * in_rows, (void**)&d_in);
    if (st == MA_OK) st = temp_alloc(ctx, sizeof(float) * (size_t)samples * C, (void**)&d_out);
    for (int c = 0; c < in_rows && st == MA_OK; ++c)
        st = copy_h2d(ctx, d_in + (int64_t)c * samples, in + (int64_t)c * in_stride, sizeof(float) * (size_t)samples);
    if (st == MA_OK) st = ma_biquad_process_dev(bq, d_in, in_stride == 0 ? 0 : samples, d_out, samples, samples);
    for (int c = 0; c < C && st == MA_OK; ++c)
        st = copy_d2h(ctx, out + (int64_t)c * out_stride, d_out + (int64_t)c * samples, sizeof(float) * (size_t)samples);
    temp_free(ctx, d_in);
    temp_free(ctx, d_out);
    return st;
}

ma_status ma_biquad_reset(ma_biquad* bq) {
    if (bq == nullptr) return MA_ERR_INVALID_ARGUMENT;
    MA_TRY(enter(bq->ctx, MA_FAULT_LAUNCH));
    MA_CUDA(cudaMemsetAsync(bq->d_state, 0, sizeof(float2) * (size_t)bq->channels * bq->sections, bq->ctx->stream));
    return MA_OK;
}

ma_status ma_biquad_get_state(ma_biquad* bq, float* state) {
    if (bq == nullptr || state == nullptr) return MA_ERR_INVALID_ARGUMENT;
    MA_TRY(enter(bq->ctx, MA_FAULT_LAUNCH));
    return copy_d2h(bq->ctx, state, bq->d_state, sizeof(float2) * (size_t)bq->channels * bq->sections);
}

ma_status ma_biquad_set_state(ma_biquad* bq, const float* state) {
    if (bq == nullptr || state == nullptr) return MA_ERR_INVALID_ARGUMENT;
    MA_TRY(enter(bq->ctx, MA_FAULT_LAUNCH));
    return copy_h2d(bq->ctx, bq->d_state, state, sizeof(float2) * (size_t)bq->channels * bq->sections);
}

ma_status ma_channel_mix_dev(ma_context* ctx, const float* in, int32_t n_channels, int64_t stride, int64_t samples,
                             float scale, float* out) {
    if (ctx == nullptr || n_channels <= 0 || samples < 0 || (samples > 0 && (in == nullptr || out == nullptr)))
        return MA_ERR_INVALID_ARGUMENT;
    MA_TRY(enter(ctx, MA_FAULT_LAUNCH));
    if (samples == 0) return MA_OK;
    const int64_t want = (samples + 255) / 256, cap = (int64_t)ctx->sm_count * 8;
    channel_mix_kernel<<<(int)(want < cap ? want : cap), 256, 0, ctx->stream>>>(in, n_channels, stride, samples, scale, out);
    return after_launch(ctx);
}

}  // extern "C"
