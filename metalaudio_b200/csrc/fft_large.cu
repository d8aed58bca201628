// Real-input transforms above 8192 points (up to 2^24): two passes through an L2-sized
// scratch buffer.  N = N1 * N2, sample n = n1 + N1*n2, bin k = k1*N2 + k2.
//
//   forward  pass 1 (cols_r2c):  for W1 adjacent n1 at a time, the N2-point real transform over
//                                n2 of x[n1 + N1*n2], times exp(-2 pi i n1 k2 / N)
//                                -> C[k2][n1], k2 = 0..N2/2            (lanes run along n1)
//            pass 2 (rows_fwd):  for W2 adjacent k2 at a time, the N1-point complex transform
//                                over n1 -> X[k1*N2 + k2]; bins above N/2 come from the
//                                conjugate mirror; the store is transposed in shared memory so
//                                that W2 adjacent bins leave together
//   inverse  pass A (rows_inv):  gather X[k1*N2 + k2] (mirror above N/2), inverse N1-point
//                                transform over k1, times exp(+2 pi i n1 k2 / N) -> D[k2][n1]
//            pass B (cols_c2r):  N2-point real inverse over k2 -> x[n1 + N1*n2] / N
//
// A batch is cut into chunks of about 96 MB of pass data (about 4*N bytes per transform); consecutive
// chunks alternate between two lanes (streams, each with its own scratch), so that one chunk's
// launch gaps and last wave are filled by the other's kernels.
// The forward row pass stages its tile (W2 consecutive scratch rows: one contiguous block) with a
// single bulk asynchronous copy of the TMA unit into its idle exchange buffer; the strided tiles of
// the other passes use plain coalesced loads and stores.  No multicast anywhere.
#include <cuda.h>
#include <cuda_pipeline.h>

#include <atomic>
#include <cmath>
#include <new>
#include <vector>

#include "bulk_copy.cuh"
#include "fft_plan.h"
#include "host_tables.h"

namespace ma {

struct LargeParams {
    const float* in;     // forward: real input; inverse: layout array a
    const float* in_b;   // inverse FULL_SPLIT imag
    float* out_a;
    float* out_b;
    float* mag;
    float2* scratch;
    int64_t batch;       // transforms in this chunk
    int n, n1, n2;
    int layout, mag_kind;
    float db_scale;
    const float2* twM2;  // stage twiddle tables of FftPlan<M2>
    const float2* twN2;  // exp(-2 pi i k/N2), k <= M2/2
    const float2* tw1;   // stage twiddle tables of FftPlan<N1>
    // Pass twiddles exp(-2 pi i n1 k2 / N) as geometric sequences in k2 (column pass) or n1 (row passes),
    // laid out so that a warp's loads are contiguous:
    const float2* twc;       // [T(M2) + 2][N1]: rows t < T: n1*t; row T: the step n1*T; row T+1: n1*M2
    const float2* twr;       // [N2/2 + 1][T(N1)]: k2*t for t < T
    const float2* twr_step;  // [N2/2 + 1]: the step k2*T
    int64_t in_stride;   // forward pass 1: floats between consecutive transforms' inputs
    int64_t valid;       // forward pass 1: samples present per transform, the rest reads as zero
    float2* spec_rows;   // convolution: kernel spectrum in pass-2 row order [N2/2+1][N1]
    const float* window; // forward pass 1: analysis window applied by the loader (STFT), or nullptr
    int32_t* error_flag; // set to 1 when a bounded wait for a staged tile ran out
};

// w[q] = base * step^q for q < n (n <= 17), products of depth <= 3 from step, step^4, step^8, step^12, step^16.
template <int n>
__device__ __forceinline__ void geometric_twiddles(float2* w, float2 base, float2 step) {
    const float2 s2 = cmul(step, step), s3 = cmul(s2, step), s4 = cmul(s2, s2);
    const float2 s8 = cmul(s4, s4), s12 = cmul(s8, s4), s16 = cmul(s8, s8);
#pragma unroll
    for (int q = 0; q < n; ++q) {
        const int lo = q & 3, hi = q >> 2;
        float2 v = base;
        if (lo == 1) v = cmul(v, step);
        else if (lo == 2) v = cmul(v, s2);
        else if (lo == 3) v = cmul(v, s3);
        if (hi == 1) v = cmul(v, s4);
        else if (hi == 2) v = cmul(v, s8);
        else if (hi == 3) v = cmul(v, s12);
        else if (hi == 4) v = cmul(v, s16);
        w[q] = v;
    }
}

struct DevCtaL {
    __device__ __forceinline__ void sync() { __syncthreads(); }
};

extern __shared__ __align__(128) float4 ma_large_smem[];

// Every pass runs its transforms through ONE exchange buffer (a barrier in front of each exchange
// write keeps it behind the previous exchange's reads): half the shared memory of two buffers, which
// is what lets a fourth 256-thread CTA, or a second 512-thread CTA, onto an SM.
// Resident CTAs per SM asked of the compiler.  256 threads: the inverse column pass fits 64 registers;
// the forward one with plain loads would spill 196 bytes there and measured slower than at 3, while its
// tensor-map staged form needs no registers for the tile and fits 64 without spills.  512 threads
// (transforms of 131072 points and more): 2, i.e. 64 registers with at most 300 bytes of spills -
// measured 12 to 26 % faster per forward + inverse pair from 2^17 to 2^22 points than one CTA with 128
// registers.
constexpr int kColsR2cCtas = 3, kColsR2cTmaCtas = 4, kColsC2rCtas = 4, kBigCtas = 2;
// The fused row pass of the convolution (two transforms and a product on the registers) spills 200-300 bytes
// at 64 registers: its 512-thread plans stay at one CTA per SM (2^20-point convolution of 256 signals:
// 1.82 ms against 1.96 ms at two).
constexpr int kRowsMulBigCtas = 1;

// ---------------------------------------------------------------- forward pass 1
template <int M2, int W1>
__global__ void __launch_bounds__(W1* FftPlan<M2>::T, (W1 * FftPlan<M2>::T) <= 256 ? kColsR2cCtas : kBigCtas) cols_r2c_kernel(const LargeParams p) {
    using P = FftPlan<M2>;
    constexpr int R = P::R, T = P::T;
    float2* smem = reinterpret_cast<float2*>(ma_large_smem);
    const int i = threadIdx.x % W1;
    const int t = threadIdx.x / W1;
    const int tiles = p.n1 / W1;
    DevCtaL cta;
    for (int64_t blk = blockIdx.x; blk < p.batch * tiles; blk += gridDim.x) {
        const int64_t b = blk / tiles;
        const int n1 = (int)(blk - b * tiles) * W1 + i;
        const float* x = p.in + b * p.in_stride + n1;
        float2 v[R];
        if (p.valid >= p.n) {
#pragma unroll
            for (int q = 0; q < R; ++q) {
                const int64_t j = t + q * T;
                v[q] = make_float2(__ldcs(x + (2 * j) * p.n1), __ldcs(x + (2 * j + 1) * p.n1));
            }
        } else {  // zero-padded input (the convolution's transforms): samples at and beyond `valid` read as 0
#pragma unroll
            for (int q = 0; q < R; ++q) {
                const int64_t j = t + q * T;
                const int64_t i0 = (2 * j) * p.n1, i1 = (2 * j + 1) * p.n1;
                v[q] = make_float2(n1 + i0 < p.valid ? __ldcs(x + i0) : 0.f, n1 + i1 < p.valid ? __ldcs(x + i1) : 0.f);
            }
        }
        if (p.window != nullptr) {  // STFT: frames overlap in the signal, the window table stays in L2
            const float* w = p.window + n1;
#pragma unroll
            for (int q = 0; q < R; ++q) {
                const int64_t j = t + q * T;
                v[q].x *= __ldg(w + (2 * j) * p.n1);
                v[q].y *= __ldg(w + (2 * j + 1) * p.n1);
            }
        }
        int parity = 0;
        float2* sbuf0 = smem + i;
        fft_forward_regs<M2, W1, DevCtaL, true>(v, t, sbuf0, 0, parity, p.twM2, cta);
        float2* sb = sbuf0;
        cta.sync();  // the exchange's reads are done before the buffer is rewritten
#pragma unroll
        for (int q = 0; q < R; ++q) sb[saddr<W1>(t + q * T)] = v[q];
        cta.sync();
        float2* c = p.scratch + b * (int64_t)(M2 + 1) * p.n1 + n1;
        // pass twiddles exp(-2 pi i n1 k / N) for k = t + q*T as a geometric sequence from two table
        // values (lanes run along n1, so each load is one contiguous row segment; a gather from a
        // single N/2-entry table cost up to an L1 wavefront per lane)
        const float2* tc = p.twc + n1;
        float2 wk[R / 2 + 1];
        geometric_twiddles<R / 2 + 1>(wk, __ldg(tc + t * p.n1), __ldg(tc + T * p.n1));
        const float2 wm2 = __ldg(tc + (T + 1) * p.n1);  // exp(-2 pi i n1 M2 / N)
#pragma unroll
        for (int q = 0; q <= R / 2; ++q) {
            const int k = t + q * T;
            if (k > M2 / 2) continue;
            const float2 a = sb[saddr<W1>(k)];
            const float2 bb = sb[saddr<W1>((M2 - k) & (M2 - 1))];
            float2 xk, xm;
            herm_post(a, bb, __ldg(p.twN2 + k), xk, xm);
            const int km = M2 - k;
            c[(int64_t)k * p.n1] = cmul(xk, wk[q]);
            c[(int64_t)km * p.n1] = cmul(xm, cmul(wm2, cconj(wk[q])));
        }
        cta.sync();  // the exchange buffers are reused by the next tile
    }
}

// The same pass with its tile staged by the copy unit through a tensor map (cp.async.bulk.tensor): for
// 16-byte aligned inputs without window and tiles of 16 or 32 columns.  Launched with
// one CTA per tile (the grid-stride loop runs once).
template <int M2, int W1>
__global__ void __launch_bounds__(W1* FftPlan<M2>::T, (W1 * FftPlan<M2>::T) <= 256 ? kColsR2cTmaCtas : kBigCtas) cols_r2c_tma_kernel(const LargeParams p, const __grid_constant__ CUtensorMap in_map) {
    using P = FftPlan<M2>;
    constexpr int R = P::R, T = P::T;
    float2* smem = reinterpret_cast<float2*>(ma_large_smem);
    const int i = threadIdx.x % W1;
    const int t = threadIdx.x / W1;
    const int tiles = p.n1 / W1;
    DevCtaL cta;
    {
        const int64_t blk = blockIdx.x;  // one tile per CTA
        if (blk >= p.batch * tiles) return;
        const int64_t b = blk / tiles;
        const int n1 = (int)(blk - b * tiles) * W1 + i;
        // The tile - W1 adjacent samples of every one of the N2 rows of this transform's N2 x N1 view - is
        // one box (two for 512 rows) of the input's tensor map: the copy unit gathers the strided row
        // segments into the exchange buffer, which is idle until the first exchange, and every thread
        // picks its points from there.  One tile per CTA, so the barrier sees a single phase.
        constexpr int ROWS = 2 * M2, BOX_ROWS = ROWS < 256 ? ROWS : 256;
        float* land = reinterpret_cast<float*>(smem);
        uint64_t* bar = reinterpret_cast<uint64_t*>(smem + M2 * W1);
        if (threadIdx.x == 0) {
            bulk_barrier_init(bar);
            bulk_barrier_expect(bar, (uint32_t)(ROWS * W1 * sizeof(float)));
#pragma unroll
            for (int r0 = 0; r0 < ROWS; r0 += BOX_ROWS)
                bulk_tensor_load_3d(land + r0 * W1, &in_map, n1 - i, r0, (int)b, bar);
        }
        __syncthreads();  // the barrier is initialised before anyone polls it
        if (!bulk_barrier_wait(bar, 0) && p.error_flag != nullptr) *p.error_flag = 1;
        float2 v[R];
#pragma unroll
        for (int q = 0; q < R; ++q) {
            const int j = t + q * T;
            v[q] = make_float2(land[(2 * j) * W1 + i], land[(2 * j + 1) * W1 + i]);
        }
        if (p.valid < p.n) {
            // zero-padded input: rows beyond the tensor's extent arrived as zeros; the row that holds sample
            // `valid` is only partly the transform's own
#pragma unroll
            for (int q = 0; q < R; ++q) {
                const int64_t j = t + q * T;
                if (n1 + (2 * j) * p.n1 >= p.valid) v[q].x = 0.f;
                if (n1 + (2 * j + 1) * p.n1 >= p.valid) v[q].y = 0.f;
            }
        }
        int parity = 0;
        float2* sbuf0 = smem + i;
        fft_forward_regs<M2, W1, DevCtaL, true>(v, t, sbuf0, 0, parity, p.twM2, cta);
        float2* sb = sbuf0;
        cta.sync();  // the exchange's reads are done before the buffer is rewritten
#pragma unroll
        for (int q = 0; q < R; ++q) sb[saddr<W1>(t + q * T)] = v[q];
        cta.sync();
        float2* c = p.scratch + b * (int64_t)(M2 + 1) * p.n1 + n1;
        // pass twiddles exp(-2 pi i n1 k / N) for k = t + q*T as a geometric sequence from two table
        // values (lanes run along n1, so each load is one contiguous row segment; a gather from a
        // single N/2-entry table cost up to an L1 wavefront per lane)
        const float2* tc = p.twc + n1;
        float2 wk[R / 2 + 1];
        geometric_twiddles<R / 2 + 1>(wk, __ldg(tc + t * p.n1), __ldg(tc + T * p.n1));
        const float2 wm2 = __ldg(tc + (T + 1) * p.n1);  // exp(-2 pi i n1 M2 / N)
#pragma unroll
        for (int q = 0; q <= R / 2; ++q) {
            const int k = t + q * T;
            if (k > M2 / 2) continue;
            const float2 a = sb[saddr<W1>(k)];
            const float2 bb = sb[saddr<W1>((M2 - k) & (M2 - 1))];
            float2 xk, xm;
            herm_post(a, bb, __ldg(p.twN2 + k), xk, xm);
            const int km = M2 - k;
            c[(int64_t)k * p.n1] = cmul(xk, wk[q]);
            c[(int64_t)km * p.n1] = cmul(xm, cmul(wm2, cconj(wk[q])));
        }
    }
}

// Writes bin k (value v) and, where asked, its conjugate mirror, in the requested layout.
__device__ __forceinline__ void store_bin(const LargeParams& p, int64_t b, int64_t k, int k2, float2 v) {
    const int64_t n = p.n, half = n / 2;
    const bool interior = k2 > 0 && k2 < p.n2 / 2;
    if (p.layout == LAYOUT_FULL_SPLIT) {
        float* re = p.out_a + b * n;
        float* im = p.out_b + b * n;
        re[k] = v.x;
        im[k] = v.y;
        if (interior) {
            re[n - k] = v.x;
            im[n - k] = -v.y;
        }
    } else {
        int64_t idx = k;
        float2 val = v;
        if (k > half) {
            if (!interior) return;
            idx = n - k;
            val.y = -v.y;
        }
        if (p.layout == LAYOUT_HALF_PACKED) {
            float2* o = reinterpret_cast<float2*>(p.out_a) + b * half;
            if (idx == 0) o[0].x = val.x;
            else if (idx == half) o[0].y = val.x;
            else o[idx] = val;
        } else {
            float2* o = reinterpret_cast<float2*>(p.out_a) + b * (half + 1);
            o[idx] = val;
        }
        if (p.mag != nullptr) p.mag[b * (half + 1) + idx] = mag_value(val, p.mag_kind, p.db_scale);
        return;
    }
    if (p.mag != nullptr && k <= half) p.mag[b * (half + 1) + k] = mag_value(v, p.mag_kind, p.db_scale);
    if (p.mag != nullptr && interior && n - k <= half) p.mag[b * (half + 1) + (n - k)] = mag_value(v, p.mag_kind, p.db_scale);
}

// Stores a transposed tile (rows r0 .. r0+W2-1 of the second pass, all N1 columns) into a half
// spectrum.  Bin k = k1*n2 + kk2 lies in the lower half for k1 < N1/2 and is stored as is; for
// k1 >= N1/2 its conjugate is bin n-k of the lower half (stored for interior rows only, the edge
// rows' mirrors being produced directly).  Which case applies is known per unrolled iteration.
// A tile is W2 consecutive rows of the chunk's global row list (row g = transform * (N2/2+1) + k2),
// so it may span the end of one transform and the start of the next: every thread derives the
// transform and the row of its own column.
template <int N1, int W2, int THREADS, bool PACKED>
__device__ __forceinline__ void store_half_tile(const LargeParams& p, int64_t g0, int64_t rows_total, const float2* tile) {
    static_assert(THREADS % W2 == 0 && (N1 * W2) % THREADS == 0, "tile shape");
    constexpr int ITER = N1 * W2 / THREADS, KSTEP = THREADS / W2;
    static_assert(ITER % 2 == 0 && (N1 / 2) % KSTEP == 0, "the halves must split between iterations");
    const int s = threadIdx.x % W2;
    const int k1base = threadIdx.x / W2;
    const int m2 = p.n2 / 2;
    const int64_t g = g0 + s;
    if (g >= rows_total) return;
    const int64_t b = g / (m2 + 1);
    const int kk2 = (int)(g - b * (m2 + 1));
    const int n = (int)p.n, half = n / 2;
    const bool interior = kk2 > 0 && kk2 < m2;
    float2* o = reinterpret_cast<float2*>(p.out_a) + b * (int64_t)(PACKED ? half : half + 1);
    float* mg = p.mag != nullptr ? p.mag + b * (int64_t)(half + 1) : nullptr;
#pragma unroll
    for (int it = 0; it < ITER / 2; ++it) {
        const int k1 = k1base + it * KSTEP;
        const int k = k1 * p.n2 + kk2;
        const float2 v = tile[k1 * (W2 + 1) + s];
        if (PACKED && k == 0) o[0].x = v.x;
        else o[k] = v;
        if (mg != nullptr) mg[k] = mag_value(v, p.mag_kind, p.db_scale);
    }
#pragma unroll
    for (int it = ITER / 2; it < ITER; ++it) {
        const int k1 = k1base + it * KSTEP;
        const int k = k1 * p.n2 + kk2;
        float2 v = tile[k1 * (W2 + 1) + s];
        if (k == half) {
            if (PACKED) o[0].y = v.x;
            else o[half] = v;
            if (mg != nullptr) mg[half] = mag_value(v, p.mag_kind, p.db_scale);
        } else if (interior) {
            v.y = -v.y;
            o[n - k] = v;
            if (mg != nullptr) mg[n - k] = mag_value(v, p.mag_kind, p.db_scale);
        }
    }
}

// Shared memory of a row-pass CTA: its exchange buffer, and room for the transposed tile
// [N1][W2+1] the passes build in the same place.
template <int N1, int W2>
constexpr __host__ __device__ size_t rows_smem_bytes() {
    size_t x = (size_t)smem_elems_per_fft<N1, 1>() * W2 * sizeof(float2);
    size_t tile = (size_t)N1 * (W2 + 1) * sizeof(float2);
    size_t b = x > tile ? x : tile;
    return (b + 15) & ~(size_t)15;
}

// ---------------------------------------------------------------- forward pass 2
template <int N1, int W2>
__global__ void __launch_bounds__(W2* FftPlan<N1>::T, (W2 * FftPlan<N1>::T) <= 256 ? 4 : kBigCtas) rows_fwd_kernel(const LargeParams p) {
    using P = FftPlan<N1>;
    constexpr int R = P::R, T = P::T;
    constexpr int ELEMS = smem_elems_per_fft<N1, 1>();
    constexpr int BUF = ELEMS * W2;
    constexpr int THREADS = W2 * T;
    float2* smem = reinterpret_cast<float2*>(ma_large_smem);
    const int slot = threadIdx.x / T;
    const int t = threadIdx.x % T;
    const int m2 = p.n2 / 2;
    // Tiles run over the chunk's global row list (row g = transform * (m2+1) + k2, which is also the
    // scratch's row order), so only the chunk's last tile can be ragged.
    const int64_t rows_total = p.batch * (int64_t)(m2 + 1);
    const int64_t tiles = (rows_total + W2 - 1) / W2;
    DevCtaL cta;
    // The tile - W2 consecutive scratch rows, one contiguous block - is staged by ONE bulk asynchronous
    // copy (the TMA unit's untiled form) into the exchange buffer, which is idle until the first
    // exchange; every thread then picks its points from shared memory.
    uint64_t* bar = reinterpret_cast<uint64_t*>(reinterpret_cast<char*>(smem) + rows_smem_bytes<N1, W2>());
    uint32_t phase = 0;
    if (threadIdx.x == 0) bulk_barrier_init(bar);
    __syncthreads();
    for (int64_t blk = blockIdx.x; blk < tiles; blk += gridDim.x) {
        const int64_t g0 = blk * W2;
        const int64_t g = g0 + slot;
        const bool active = g < rows_total;
        if (threadIdx.x == 0) {
            const int64_t rows_here = rows_total - g0 < W2 ? rows_total - g0 : W2;
            bulk_copy_g2s(smem, p.scratch + g0 * N1, (uint32_t)(rows_here * N1 * sizeof(float2)), bar);
        }
        if (!bulk_barrier_wait(bar, phase) && p.error_flag != nullptr) *p.error_flag = 1;
        phase ^= 1;
        float2 v[R];
#pragma unroll
        for (int q = 0; q < R; ++q) v[q] = active ? smem[slot * N1 + t + q * T] : make_float2(0.f, 0.f);
        cta.sync();  // every thread has its points: the exchange buffer may be written
        int parity = 0;
        fft_forward_regs<N1, 1, DevCtaL, true>(v, t, smem + slot * ELEMS, BUF, parity, p.tw1, cta);
        cta.sync();  // everyone is done with the exchange buffers: reuse them as the tile
        float2* tile = smem;  // [k1][W2+1]
#pragma unroll
        for (int q = 0; q < R; ++q) tile[(t + q * T) * (W2 + 1) + slot] = v[q];
        cta.sync();
        if (p.layout == LAYOUT_FULL_SPLIT) {
            for (int idx = threadIdx.x; idx < N1 * W2; idx += THREADS) {
                const int s = idx % W2;
                const int k1 = idx / W2;
                const int64_t gs = g0 + s;
                if (gs >= rows_total) continue;
                const int64_t b = gs / (m2 + 1);
                const int kk2 = (int)(gs - b * (m2 + 1));
                store_bin(p, b, (int64_t)k1 * p.n2 + kk2, kk2, tile[k1 * (W2 + 1) + s]);
            }
        } else if (p.layout == LAYOUT_HALF_PACKED) {
            store_half_tile<N1, W2, THREADS, true>(p, g0, rows_total, tile);
        } else {
            store_half_tile<N1, W2, THREADS, false>(p, g0, rows_total, tile);
        }
        cta.sync();
    }
}

// Spectrum bin k of transform b for the inverse, from any layout (Hermitian input assumed).
__device__ __forceinline__ float2 load_bin(const LargeParams& p, int64_t b, int64_t k) {
    const int64_t n = p.n, half = n / 2;
    if (p.layout == LAYOUT_FULL_SPLIT) {
        float2 v = make_float2(__ldg(p.in + b * n + k), __ldg(p.in_b + b * n + k));
        if (k == 0 || k == half) v.y = 0.f;
        return v;
    }
    const bool mirror = k > half;
    const int64_t idx = mirror ? n - k : k;
    float2 v;
    if (p.layout == LAYOUT_HALF_PACKED) {
        const float2* x = reinterpret_cast<const float2*>(p.in) + b * half;
        if (idx == 0) v = make_float2(__ldg(x).x, 0.f);
        else if (idx == half) v = make_float2(__ldg(x).y, 0.f);
        else v = __ldg(x + idx);
    } else {
        const float2* x = reinterpret_cast<const float2*>(p.in) + b * (half + 1);
        v = __ldg(x + idx);
        if (idx == 0 || idx == half) v.y = 0.f;
    }
    if (mirror) v.y = -v.y;
    return v;
}

// ---------------------------------------------------------------- inverse pass A
template <int N1, int W2>
__global__ void __launch_bounds__(W2* FftPlan<N1>::T, (W2 * FftPlan<N1>::T) <= 256 ? 4 : kBigCtas) rows_inv_kernel(const LargeParams p) {
    using P = FftPlan<N1>;
    constexpr int R = P::R, T = P::T;
    constexpr int ELEMS = smem_elems_per_fft<N1, 1>();
    constexpr int BUF = ELEMS * W2;
    constexpr int THREADS = W2 * T;
    float2* smem = reinterpret_cast<float2*>(ma_large_smem);
    const int slot = threadIdx.x / T;
    const int t = threadIdx.x % T;
    const int m2 = p.n2 / 2;
    // tiles over the chunk's global row list (row g = transform * (m2+1) + k2), as in rows_fwd_kernel
    const int64_t rows_total = p.batch * (int64_t)(m2 + 1);
    const int64_t tiles = (rows_total + W2 - 1) / W2;
    DevCtaL cta;
    for (int64_t blk = blockIdx.x; blk < tiles; blk += gridDim.x) {
        const int64_t g0 = blk * W2;
        float2* tile = smem;
        // The gather goes from global to shared memory by asynchronous 4- and 8-byte copies (no registers
        // hold it, which is what lets a fourth CTA onto an SM); the conjugation of the mirrored half, the
        // two real bins and the real / imaginary swap (the inverse runs as a forward transform of the
        // swapped spectrum) are applied when a thread picks up its points.
        const bool full_split = p.layout == LAYOUT_FULL_SPLIT;
        const bool packed = p.layout == LAYOUT_HALF_PACKED;
        {
            static_assert(THREADS % W2 == 0 && (N1 * W2) % THREADS == 0, "tile load shape");
            constexpr int ITER = N1 * W2 / THREADS, KSTEP = THREADS / W2;
            static_assert(ITER % 2 == 0 && (N1 / 2) % KSTEP == 0, "the halves must split between iterations");
            const int s = threadIdx.x % W2;
            const int k1base = threadIdx.x / W2;
            const int64_t gs = g0 + s;
            const bool live = gs < rows_total;
            const int64_t b = live ? gs / (m2 + 1) : 0;
            const int kk2 = live ? (int)(gs - b * (m2 + 1)) : 0;
            const int64_t n = p.n, half = n / 2;
            if (!live) {
#pragma unroll
                for (int it = 0; it < ITER; ++it) tile[(k1base + it * KSTEP) * (W2 + 1) + s] = make_float2(0.f, 0.f);
            } else if (full_split) {
                const float* re = p.in + b * n;
                const float* im = p.in_b + b * n;
#pragma unroll
                for (int it = 0; it < ITER; ++it) {
                    const int64_t k = (int64_t)(k1base + it * KSTEP) * p.n2 + kk2;
                    float* dst = reinterpret_cast<float*>(tile + (k1base + it * KSTEP) * (W2 + 1) + s);
                    __pipeline_memcpy_async(dst, re + k, 4);
                    __pipeline_memcpy_async(dst + 1, im + k, 4);
                }
            } else {
                const float2* src = reinterpret_cast<const float2*>(p.in) + b * (packed ? half : half + 1);
                const int nn = (int)n, hh = (int)half;
                // lower half (k1 < N1/2): bin k itself; upper half: bin n-k (conjugated on pick-up)
#pragma unroll
                for (int it = 0; it < ITER; ++it) {
                    const int k = (k1base + it * KSTEP) * p.n2 + kk2;
                    int idx = it < ITER / 2 ? k : nn - k;
                    if (packed && idx == hh) idx = 0;
                    __pipeline_memcpy_async(tile + (k1base + it * KSTEP) * (W2 + 1) + s, src + idx, 8);
                }
            }
            __pipeline_commit();
            __pipeline_wait_prior(0);
        }
        cta.sync();
        float2 v[R];
        {
            const int64_t gr = g0 + slot;
            // the row's two real bins (k = 0 and k = N/2) sit in thread 0's points 0 and R/2 when k2 = 0
            const bool real_bins = t == 0 && gr < rows_total && gr % (m2 + 1) == 0;
#pragma unroll
            for (int q = 0; q < R; ++q) {
                float2 val = tile[(t + q * T) * (W2 + 1) + slot];
                if (q == 0 && real_bins) val.y = 0.f;
                if (q == R / 2 && real_bins) val = make_float2(packed ? val.y : val.x, 0.f);
                if (q >= R / 2 && !full_split) val.y = -val.y;  // k1 >= N1/2: the conjugate mirror
                v[q] = make_float2(val.y, val.x);
            }
        }
        cta.sync();
        int parity = 0;
        fft_forward_regs<N1, 1, DevCtaL, true>(v, t, smem + slot * ELEMS, BUF, parity, p.tw1, cta);
        const int64_t g = g0 + slot;
        if (g < rows_total) {
            const int k2 = (int)(g % (m2 + 1));
            float2* row = p.scratch + g * N1;
            float2 wq[R];
            geometric_twiddles<R>(wq, __ldg(p.twr + k2 * T + t), __ldg(p.twr_step + k2));
#pragma unroll
            for (int q = 0; q < R; ++q) {
                const int n1 = t + q * T;
                row[n1] = cmul(make_float2(v[q].y, v[q].x), cconj(wq[q]));
            }
        }
        cta.sync();
    }
}

// ---------------------------------------------------------------- convolution pass 2
// Both row passes of a transform pair with the bin-by-bin product in between, on the scratch rows
// in place: C[k2][.] -> forward N1-point transform -> times the kernel spectrum's row k2 ->
// inverse transform -> times exp(+2 pi i n1 k2 / N) -> D[k2][.].  The spectrum of the signal
// never leaves the registers.  STORE_SPECTRUM: stop after the forward transform and write the row
// to p.spec_rows (how the kernel's own spectrum is prepared).
template <int N1, int W2, bool STORE_SPECTRUM>
__global__ void __launch_bounds__(W2* FftPlan<N1>::T, (W2 * FftPlan<N1>::T) <= 256 ? 3 : kRowsMulBigCtas) rows_mul_kernel(const LargeParams p) {
    using P = FftPlan<N1>;
    constexpr int R = P::R, T = P::T;
    constexpr int ELEMS = smem_elems_per_fft<N1, 1>();
    constexpr int BUF = ELEMS * W2;
    float2* smem = reinterpret_cast<float2*>(ma_large_smem);
    const int slot = threadIdx.x / T;
    const int t = threadIdx.x % T;
    const int m2 = p.n2 / 2;
    // tiles over the chunk's global row list (row g = transform * (m2+1) + k2), as in rows_fwd_kernel
    const int64_t rows_total = p.batch * (int64_t)(m2 + 1);
    const int64_t tiles = (rows_total + W2 - 1) / W2;
    DevCtaL cta;
    for (int64_t blk = blockIdx.x; blk < tiles; blk += gridDim.x) {
        const int64_t g = blk * W2 + slot;
        const bool active = g < rows_total;
        const int k2 = active ? (int)(g % (m2 + 1)) : 0;
        float2* row = p.scratch + (active ? g : 0) * N1;
        const float2* hrow = p.spec_rows + (int64_t)(active ? k2 : 0) * N1;
        float2 v[R], h[R];
#pragma unroll
        for (int q = 0; q < R; ++q) v[q] = active ? row[t + q * T] : make_float2(0.f, 0.f);
        if constexpr (!STORE_SPECTRUM) {
#pragma unroll
            for (int q = 0; q < R; ++q) h[q] = __ldg(hrow + t + q * T);
        }
        int parity = 0;
        fft_forward_regs<N1, 1, DevCtaL, true>(v, t, smem + slot * ELEMS, BUF, parity, p.tw1, cta);
        if constexpr (STORE_SPECTRUM) {
            if (active) {
#pragma unroll
                for (int q = 0; q < R; ++q) p.spec_rows[(int64_t)k2 * N1 + t + q * T] = v[q];
            }
        } else {
#pragma unroll
            for (int q = 0; q < R; ++q) {
                const float2 y = cmul(v[q], h[q]);
                v[q] = make_float2(y.y, y.x);  // swapped: the inverse runs as a forward transform
            }
            cta.sync();  // the first transform's exchange reads are done before the buffers are rewritten
            fft_forward_regs<N1, 1, DevCtaL, true>(v, t, smem + slot * ELEMS, BUF, parity, p.tw1, cta);
            if (active) {
                float2 wq[R];
                geometric_twiddles<R>(wq, __ldg(p.twr + k2 * T + t), __ldg(p.twr_step + k2));
#pragma unroll
                for (int q = 0; q < R; ++q) row[t + q * T] = cmul(make_float2(v[q].y, v[q].x), cconj(wq[q]));
            }
        }
        cta.sync();
    }
}

// ---------------------------------------------------------------- inverse pass B
template <int M2, int W1>
__global__ void __launch_bounds__(W1* FftPlan<M2>::T, (W1 * FftPlan<M2>::T) <= 256 ? kColsC2rCtas : kBigCtas) cols_c2r_kernel(const LargeParams p) {
    using P = FftPlan<M2>;
    constexpr int R = P::R, T = P::T;
    float2* smem = reinterpret_cast<float2*>(ma_large_smem);
    const int i = threadIdx.x % W1;
    const int t = threadIdx.x / W1;
    const int tiles = p.n1 / W1;
    const float scale = 1.0f / (float)p.n;
    DevCtaL cta;
    for (int64_t blk = blockIdx.x; blk < p.batch * tiles; blk += gridDim.x) {
        const int64_t b = blk / tiles;
        const int n1 = (int)(blk - b * tiles) * W1 + i;
        const float2* d = p.scratch + b * (int64_t)(M2 + 1) * p.n1 + n1;
        int parity = 0;
        float2* sbuf0 = smem + i;
        float2* sb = sbuf0;
        float2 ra[R / 2 + 1], rb[R / 2 + 1];
#pragma unroll
        for (int q = 0; q <= R / 2; ++q) {  // every load in flight before the first use
            const int k = t + q * T;
            const int kc = k > M2 / 2 ? M2 / 2 : k;
            ra[q] = d[(int64_t)kc * p.n1];
            rb[q] = d[(int64_t)(M2 - kc) * p.n1];
        }
#pragma unroll
        for (int q = 0; q <= R / 2; ++q) {
            const int k = t + q * T;
            if (k > M2 / 2) continue;
            float2 a = ra[q];
            float2 bb = rb[q];
            if (k == 0) {
                a.y = 0.f;
                bb.y = 0.f;
            }
            float2 zk, zm;
            herm_pre(a, bb, __ldg(p.twN2 + k), zk, zm);
            sb[saddr<W1>(k)] = make_float2(zk.y, zk.x);
            if (k > 0) sb[saddr<W1>(M2 - k)] = make_float2(zm.y, zm.x);
        }
        cta.sync();
        float2 v[R];
#pragma unroll
        for (int q = 0; q < R; ++q) v[q] = sb[saddr<W1>(t + q * T)];
        fft_forward_regs<M2, W1, DevCtaL, true>(v, t, sbuf0, 0, parity, p.twM2, cta);
        float* x = p.out_a + b * (int64_t)p.n + n1;
#pragma unroll
        for (int q = 0; q < R; ++q) {
            const int64_t j = t + q * T;
            __stcs(x + (2 * j) * p.n1, v[q].y * scale);
            __stcs(x + (2 * j + 1) * p.n1, v[q].x * scale);
        }
        cta.sync();
    }
}

// The same pass with both of its strided tiles moved by the copy unit through tensor maps: the scratch
// rows k2 < M2 of W1 columns land in the exchange buffer as one box (the row k2 = M2 as a plain bulk copy
// behind it), the Hermitian step rewrites that buffer in place (each (k, M2-k) pair of a column belongs to
// one thread), and the real output tile - N2 rows of W1 samples - is assembled in the same buffer and
// stored as boxes.  For 16-byte aligned dense outputs and tiles of 32 columns; one tile per CTA.
template <int M2, int W1>
__global__ void __launch_bounds__(W1* FftPlan<M2>::T, (W1 * FftPlan<M2>::T) <= 256 ? kColsC2rCtas : kBigCtas)
    cols_c2r_tma_kernel(const LargeParams p, const __grid_constant__ CUtensorMap scratch_map,
                        const __grid_constant__ CUtensorMap out_map) {
    using P = FftPlan<M2>;
    constexpr int R = P::R, T = P::T;
    constexpr int ROWS = 2 * M2, BOX_ROWS = ROWS < 256 ? ROWS : 256;
    float2* smem = reinterpret_cast<float2*>(ma_large_smem);
    float2* last_row = smem + M2 * W1;  // scratch row k2 = M2
    uint64_t* bar = reinterpret_cast<uint64_t*>(last_row + W1);
    const int i = threadIdx.x % W1;
    const int t = threadIdx.x / W1;
    const int tiles = p.n1 / W1;
    const float scale = 1.0f / (float)p.n;
    DevCtaL cta;
    const int64_t blk = blockIdx.x;  // one tile per CTA
    if (blk >= p.batch * tiles) return;
    const int64_t b = blk / tiles;
    const int n1_0 = (int)(blk - b * tiles) * W1;
    if (threadIdx.x == 0) {
        bulk_barrier_init(bar);
        bulk_barrier_expect(bar, (uint32_t)((M2 + 1) * W1 * sizeof(float2)));
        bulk_tensor_load_3d(smem, &scratch_map, 2 * n1_0, 0, (int)b, bar);
        bulk_copy_part(last_row, p.scratch + (b * (int64_t)(M2 + 1) + M2) * p.n1 + n1_0, (uint32_t)(W1 * sizeof(float2)), bar);
    }
    __syncthreads();  // the barrier is initialised before anyone polls it
    if (!bulk_barrier_wait(bar, 0) && p.error_flag != nullptr) *p.error_flag = 1;
    int parity = 0;
    float2* sbuf0 = smem + i;
#pragma unroll
    for (int q = 0; q <= R / 2; ++q) {
        const int k = t + q * T;
        if (k > M2 / 2) continue;
        float2 a = sbuf0[k * W1];
        float2 bb = k == 0 ? last_row[i] : sbuf0[(M2 - k) * W1];
        if (k == 0) {
            a.y = 0.f;
            bb.y = 0.f;
        }
        float2 zk, zm;
        herm_pre(a, bb, __ldg(p.twN2 + k), zk, zm);
        sbuf0[saddr<W1>(k)] = make_float2(zk.y, zk.x);
        if (k > 0) sbuf0[saddr<W1>(M2 - k)] = make_float2(zm.y, zm.x);
    }
    cta.sync();
    float2 v[R];
#pragma unroll
    for (int q = 0; q < R; ++q) v[q] = sbuf0[saddr<W1>(t + q * T)];
    fft_forward_regs<M2, W1, DevCtaL, true>(v, t, sbuf0, 0, parity, p.twM2, cta);
    cta.sync();  // the last exchange's reads are done: the buffer becomes the output tile [N2][W1]
    float* tile = reinterpret_cast<float*>(smem);
#pragma unroll
    for (int q = 0; q < R; ++q) {
        const int j = t + q * T;
        tile[(2 * j) * W1 + i] = v[q].y * scale;
        tile[(2 * j + 1) * W1 + i] = v[q].x * scale;
    }
    bulk_proxy_fence();
    cta.sync();
    if (threadIdx.x == 0) {
#pragma unroll
        for (int r0 = 0; r0 < ROWS; r0 += BOX_ROWS) bulk_tensor_store_3d(&out_map, n1_0, r0, (int)b, tile + r0 * W1);
        bulk_store_commit_and_wait_read();
    }
}

// ---------------------------------------------------------------- host side
struct LargeShape {
    int n1, m2;  // the tile widths of the passes are chosen per size in dispatch_cols / dispatch_rows
};

static bool large_shape(int n, LargeShape* s) {
    int lg = 0;
    while ((1 << lg) < n) ++lg;
    if (lg < 14 || lg > 24) return false;
    const int lg2 = (lg + 1) / 2;  // N2 >= N1
    const int n2 = 1 << lg2;
    s->n1 = n >> lg2;
    s->m2 = n2 / 2;
    return true;
}

// cuTensorMapEncodeTiled through the runtime's driver entry point lookup (no link against the driver
// library); nullptr when the driver does not offer it.
using TensorMapEncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                       const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                       CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static TensorMapEncodeFn tensor_map_encoder() {
    static std::atomic<void*> cached{nullptr};
    static std::atomic<bool> looked{false};
    if (!looked.load(std::memory_order_acquire)) {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess)
            fn = nullptr;
        (void)cudaGetLastError();
        cached.store(fn, std::memory_order_release);
        looked.store(true, std::memory_order_release);
    }
    return reinterpret_cast<TensorMapEncodeFn>(cached.load(std::memory_order_acquire));
}

// Tensor map of `batch` dense [rows][row_floats] float arrays `batch_stride` floats apart, with boxes of
// box_rows x box_floats; false when the array does not qualify (alignment, stride) or the driver cannot
// encode it.
static bool tile_tensor_map(const float* base, int64_t row_floats, int64_t rows, int64_t batch, int64_t batch_stride,
                            int box_floats, int box_rows, CUtensorMap* map) {
    if ((reinterpret_cast<uintptr_t>(base) & 15) != 0 || (batch_stride & 3) != 0 || (row_floats & 3) != 0 ||
        batch_stride < rows * row_floats || batch > (int64_t)1 << 30)
        return false;
    TensorMapEncodeFn enc = tensor_map_encoder();
    if (enc == nullptr) return false;
    const cuuint64_t dims[3] = {(cuuint64_t)row_floats, (cuuint64_t)rows, (cuuint64_t)batch};
    const cuuint64_t strides[2] = {(cuuint64_t)row_floats * sizeof(float), (cuuint64_t)batch_stride * sizeof(float)};
    const cuuint32_t box[3] = {(cuuint32_t)box_floats, (cuuint32_t)box_rows, 1u};
    const cuuint32_t estr[3] = {1u, 1u, 1u};
    return enc(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<float*>(base), dims, strides, box, estr,
               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// The forward pass's real input seen as [batch][rows][N1] floats (no window).  Zero-padded inputs get
// only the rows that hold samples: boxes reaching beyond them are filled with zeros by the copy unit.
static bool input_tensor_map(const LargeParams& p, int box_floats, int box_rows, CUtensorMap* map) {
    if (p.window != nullptr || p.valid <= 0) return false;
    const int64_t rows = p.valid >= p.n ? p.n2 : (p.valid + p.n1 - 1) / p.n1;
    // the last transform's last row must still lie inside the caller's array
    if (p.valid < p.n && rows * p.n1 > p.valid && p.in_stride < rows * p.n1) return false;
    return tile_tensor_map(p.in, p.n1, rows, p.batch, p.in_stride, box_floats, box_rows, map);
}

template <int M2, int W1>
static ma_status run_cols(ma_fft_plan* plan, const LargeParams& p, bool inverse, cudaStream_t st) {
    constexpr int threads = W1 * FftPlan<M2>::T;
    constexpr size_t smem = (size_t)M2 * W1 * sizeof(float2);
    ma_context* ctx = plan->ctx;
    auto kf = cols_r2c_kernel<M2, W1>;
    auto ki = cols_c2r_kernel<M2, W1>;
    static int occ_f[64] = {0}, occ_i[64] = {0};
    int& occ = inverse ? occ_i[ctx->device & 63] : occ_f[ctx->device & 63];
    if (occ == 0) {
        int n = 0;
        if (inverse) {
            MA_CUDA(cudaFuncSetAttribute(ki, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
            MA_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, ki, threads, smem));
            if constexpr (W1 == 32 && M2 <= 128)
                MA_CUDA(cudaFuncSetAttribute(cols_c2r_tma_kernel<M2, W1>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             (int)(smem + W1 * sizeof(float2) + 16)));
        } else {
            MA_CUDA(cudaFuncSetAttribute(kf, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
            MA_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, kf, threads, smem));
            if constexpr (W1 >= 16)
                MA_CUDA(cudaFuncSetAttribute(cols_r2c_tma_kernel<M2, W1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem + 16));
        }
        occ = n > 0 ? n : 1;
    }
    const int64_t work = p.batch * (p.n1 / W1);
    const int64_t cap = (int64_t)ctx->sm_count * occ;
    // forward passes: one CTA per tile (measured 5 % faster than persistent CTAs); inverse passes: persistent
    const int grid = !inverse ? (int)work : (int)(work < cap ? work : cap);
    if (inverse) {
        CUtensorMap smap, omap;
        bool staged = false;
        if constexpr (W1 == 32 && M2 <= 128) {  // the 512-thread plans measured 2 % slower staged
            const int64_t per = (int64_t)(M2 + 1) * p.n1 * 2;  // floats of scratch per transform
            staged = tile_tensor_map(reinterpret_cast<const float*>(p.scratch), 2 * (int64_t)p.n1, M2 + 1, p.batch, per, 2 * W1, M2, &smap) &&
                     tile_tensor_map(p.out_a, p.n1, p.n2, p.batch, p.n, W1, 2 * M2 < 256 ? 2 * M2 : 256, &omap);
            if (staged)
                cols_c2r_tma_kernel<M2, W1><<<(int)work, threads, smem + W1 * sizeof(float2) + 16, st>>>(p, smap, omap);
        }
        if (!staged) ki<<<grid, threads, smem, st>>>(p);
    } else {
        CUtensorMap map;
        bool staged = false;
        if constexpr (W1 >= 16) staged = input_tensor_map(p, W1, 2 * M2 < 256 ? 2 * M2 : 256, &map);
        if constexpr (W1 >= 16) {
            if (staged) cols_r2c_tma_kernel<M2, W1><<<grid, threads, smem + 16, st>>>(p, map);
        }
        if (!staged) kf<<<grid, threads, smem, st>>>(p);
    }
    return after_launch(ctx);
}

template <int N1, int W2>
static ma_status run_rows(ma_fft_plan* plan, const LargeParams& p, bool inverse, cudaStream_t st) {
    constexpr int threads = W2 * FftPlan<N1>::T;
    // the exchange buffer plus 16 bytes for the staging barrier of the forward pass
    constexpr size_t smem = rows_smem_bytes<N1, W2>() + 16;
    ma_context* ctx = plan->ctx;
    auto kf = rows_fwd_kernel<N1, W2>;
    auto ki = rows_inv_kernel<N1, W2>;
    static int occ_f[64] = {0}, occ_i[64] = {0};
    int& occ = inverse ? occ_i[ctx->device & 63] : occ_f[ctx->device & 63];
    if (occ == 0) {
        int n = 0;
        if (inverse) {
            MA_CUDA(cudaFuncSetAttribute(ki, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
            MA_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, ki, threads, smem));
        } else {
            MA_CUDA(cudaFuncSetAttribute(kf, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
            MA_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, kf, threads, smem));
        }
        occ = n > 0 ? n : 1;
    }
    const int m2 = p.n2 / 2;
    const int64_t work = (p.batch * (int64_t)(m2 + 1) + W2 - 1) / W2;  // tiles over the chunk's global row list
    const int64_t cap = (int64_t)ctx->sm_count * occ;
    // one CTA per tile (measured 3-5 % faster than persistent CTAs), except the inverse pass of the
    // 512-thread plans (1 % slower that way): persistent
    const int grid = (!inverse || threads <= 256) ? (int)work : (int)(work < cap ? work : cap);
    if (inverse) ki<<<grid, threads, smem, st>>>(p);
    else kf<<<grid, threads, smem, st>>>(p);
    return after_launch(ctx);
}

// Raises a kernel's dynamic shared-memory limit and returns its resident CTAs per SM (cached in occ).
template <typename K>
static ma_status kernel_occupancy(K kernel, int threads, size_t smem, int* occ) {
    if (*occ == 0) {
        int n = 0;
        MA_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        MA_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, kernel, threads, smem));
        *occ = n > 0 ? n : 1;
    }
    return MA_OK;
}

template <int N1, int W2>
static ma_status run_rows_mul(ma_fft_plan* plan, const LargeParams& p, bool store_spectrum, cudaStream_t st) {
    constexpr int threads = W2 * FftPlan<N1>::T;
    constexpr size_t smem = rows_smem_bytes<N1, W2>();
    ma_context* ctx = plan->ctx;
    static int occ[2][64] = {};
    int* o = &occ[store_spectrum ? 1 : 0][ctx->device & 63];
    if (store_spectrum) MA_TRY(kernel_occupancy(rows_mul_kernel<N1, W2, true>, threads, smem, o));
    else MA_TRY(kernel_occupancy(rows_mul_kernel<N1, W2, false>, threads, smem, o));
    const int m2 = p.n2 / 2;
    const int64_t work = (p.batch * (int64_t)(m2 + 1) + W2 - 1) / W2;  // tiles over the chunk's global row list
    const int64_t cap = (int64_t)ctx->sm_count * *o;
    const int grid = (int)(work < cap ? work : cap);
    if (store_spectrum) rows_mul_kernel<N1, W2, true><<<grid, threads, smem, st>>>(p);
    else rows_mul_kernel<N1, W2, false><<<grid, threads, smem, st>>>(p);
    return after_launch(ctx);
}

static ma_status dispatch_rows_mul(ma_fft_plan* plan, const LargeParams& p, bool store_spectrum, cudaStream_t st) {
    switch (p.n1) {
        case 128: return run_rows_mul<128, 32>(plan, p, store_spectrum, st);
        case 256: return run_rows_mul<256, 16>(plan, p, store_spectrum, st);
        case 512: return run_rows_mul<512, 16>(plan, p, store_spectrum, st);
        case 1024: return run_rows_mul<1024, 8>(plan, p, store_spectrum, st);
        case 2048: return run_rows_mul<2048, 4>(plan, p, store_spectrum, st);
        case 4096: return run_rows_mul<4096, 2>(plan, p, store_spectrum, st);
        default: return MA_ERR_UNSUPPORTED;
    }
}

static ma_status dispatch_cols(ma_fft_plan* plan, const LargeParams& p, bool inverse, cudaStream_t st) {
    switch (p.n2 / 2) {
        case 64: return run_cols<64, 32>(plan, p, inverse, st);
        case 128: return run_cols<128, 32>(plan, p, inverse, st);
        case 256: return run_cols<256, 32>(plan, p, inverse, st);
        case 512: return run_cols<512, 16>(plan, p, inverse, st);
        case 1024: return run_cols<1024, 8>(plan, p, inverse, st);
        case 2048: return run_cols<2048, 4>(plan, p, inverse, st);
        default: return MA_ERR_UNSUPPORTED;
    }
}

static ma_status dispatch_rows(ma_fft_plan* plan, const LargeParams& p, bool inverse, cudaStream_t st) {
    switch (p.n1) {
        case 128: return run_rows<128, 32>(plan, p, inverse, st);
        case 256: return run_rows<256, 16>(plan, p, inverse, st);
        case 512: return run_rows<512, 16>(plan, p, inverse, st);
        case 1024: return run_rows<1024, 8>(plan, p, inverse, st);
        case 2048: return run_rows<2048, 4>(plan, p, inverse, st);
        case 4096: return run_rows<4096, 2>(plan, p, inverse, st);
        default: return MA_ERR_UNSUPPORTED;
    }
}

static ma_status upload_tw(ma_context* ctx, int64_t len, int64_t count, float2** dptr) {
    auto tw = make_twiddles(len, count);
    MA_CUDA(cudaMalloc((void**)dptr, tw.size() * sizeof(float2)));
    return copy_h2d(ctx, *dptr, tw.data(), tw.size() * sizeof(float2));
}

ma_status large_plan_init(ma_fft_plan* plan) {
    LargeShape s;
    if (!large_shape(plan->n, &s)) return MA_ERR_UNSUPPORTED;
    ma_context* ctx = plan->ctx;
    plan->n1 = s.n1;
    plan->n2 = 2 * s.m2;
    {
        auto tw = make_stage_tables_for(s.m2, false);  // column stage twiddles
        MA_CUDA(cudaMalloc((void**)&plan->d_twM, tw.size() * sizeof(float2)));
        MA_TRY(copy_h2d(ctx, plan->d_twM, tw.data(), tw.size() * sizeof(float2)));
        auto t1 = make_stage_tables_for(s.n1, false);  // row stage twiddles
        MA_CUDA(cudaMalloc((void**)&plan->d_tw1, t1.size() * sizeof(float2)));
        MA_TRY(copy_h2d(ctx, plan->d_tw1, t1.data(), t1.size() * sizeof(float2)));
    }
    MA_TRY(upload_tw(ctx, 2 * s.m2, s.m2 / 2 + 1, &plan->d_twN)); // column Hermitian twiddles
    {
        // pass twiddles in the layouts the kernels load them in (see LargeParams); angles reduced in
        // integers, values rounded once from double precision
        const int64_t n = plan->n;
        const int t1 = fft_plan_threads(s.m2), t2 = fft_plan_threads(s.n1);
        auto w = [n](int64_t j) {
            const double a = -2.0 * 3.14159265358979323846 * (double)(j % n) / (double)n;
            return make_float2((float)std::cos(a), (float)std::sin(a));
        };
        std::vector<float2> twc((size_t)(t1 + 2) * s.n1), twr((size_t)(s.m2 + 1) * t2), step((size_t)s.m2 + 1);
        for (int64_t n1 = 0; n1 < s.n1; ++n1) {
            for (int t = 0; t <= t1; ++t) twc[(size_t)t * s.n1 + n1] = w(n1 * t);
            twc[(size_t)(t1 + 1) * s.n1 + n1] = w(n1 * s.m2);
        }
        for (int64_t k2 = 0; k2 <= s.m2; ++k2) {
            for (int t = 0; t < t2; ++t) twr[(size_t)k2 * t2 + t] = w(k2 * t);
            step[(size_t)k2] = w(k2 * t2);
        }
        MA_CUDA(cudaMalloc((void**)&plan->d_twc, twc.size() * sizeof(float2)));
        MA_TRY(copy_h2d(ctx, plan->d_twc, twc.data(), twc.size() * sizeof(float2)));
        MA_CUDA(cudaMalloc((void**)&plan->d_twr, (twr.size() + step.size()) * sizeof(float2)));
        MA_TRY(copy_h2d(ctx, plan->d_twr, twr.data(), twr.size() * sizeof(float2)));
        MA_TRY(copy_h2d(ctx, plan->d_twr + twr.size(), step.data(), step.size() * sizeof(float2)));
    }
    // Two lanes of about 96 MB of pass data each.  The passes are bound by latency and instruction
    // issue, not by HBM, so whether the scratch stays in the 126 MB L2 matters little (measured for
    // 4096 transforms of 65536 points: one lane of 192 MB 1.79 ms per forward + inverse pair, of 48 MB
    // 2.06 ms, of 16 MB 2.90 ms: every extra launch costs about 5 us of ramp-up and drain).  A second
    // lane on its own stream fills those gaps with the other chunk's kernels: 1.62 ms, flat from
    // 24 to 192 MB per lane and from two to four lanes.
    const size_t per = (size_t)(s.m2 + 1) * s.n1 * sizeof(float2);
    const size_t chunk_mb = 96;
    plan->scratch_lanes = 2;
    int64_t chunk = (int64_t)((chunk_mb << 20) / per);
    if (chunk < 1) chunk = 1;
    plan->scratch_batch = chunk;
    MA_CUDA(cudaMalloc((void**)&plan->d_scratch, per * (size_t)chunk * (size_t)plan->scratch_lanes));
    return MA_OK;
}

void large_plan_destroy(ma_fft_plan* plan) {
    if (plan->d_tw1) (void)cudaFree(plan->d_tw1);
    if (plan->d_twc) (void)cudaFree(plan->d_twc);
    if (plan->d_twr) (void)cudaFree(plan->d_twr);
    if (plan->d_frames) (void)cudaFree(plan->d_frames);
    plan->d_frames = nullptr;
    if (plan->d_scratch) (void)cudaFree(plan->d_scratch);
    plan->d_tw1 = nullptr;
    plan->d_twc = nullptr;
    plan->d_twr = nullptr;
    plan->d_scratch = nullptr;
}

// Cuts a batch into chunks of `chunk` transforms and runs body(first, count, scratch, stream) on each.
// With several lanes (the plan's own scratch), consecutive chunks rotate over the context's stream
// and its auxiliary streams, each lane with its own part of the scratch: one chunk's launch gaps and
// last, partly filled wave are covered by the other lanes' kernels.  The auxiliary streams start
// behind everything queued on the context's stream and are joined back before returning - also when
// a launch failed - so callers see one stream.
template <class Body>
static ma_status for_chunks(ma_fft_plan* plan, int64_t batch, float2* scratch, int64_t chunk, int lanes, Body&& body) {
    ma_context* ctx = plan->ctx;
    if (lanes > 1 + kAuxStreams) lanes = 1 + kAuxStreams;
    const int64_t chunks = (batch + chunk - 1) / chunk;
    const int used = chunks < lanes ? (int)chunks : lanes;  // lanes that get work
    if (used > 1) {
        MA_CUDA(cudaEventRecord(ctx->ev_fork, ctx->stream));
        for (int l = 1; l < used; ++l) MA_CUDA(cudaStreamWaitEvent(ctx->aux_stream[l - 1], ctx->ev_fork, 0));
    }
    const int64_t lane_elems = chunk * (int64_t)(plan->n2 / 2 + 1) * plan->n1;
    ma_status st = MA_OK;
    int lane = 0;
    for (int64_t done = 0; done < batch && st == MA_OK; done += chunk, lane = (lane + 1) % used) {
        const int64_t count = batch - done < chunk ? batch - done : chunk;
        st = body(done, count, scratch + lane * lane_elems, lane == 0 ? ctx->stream : ctx->aux_stream[lane - 1]);
    }
    for (int l = 1; l < used; ++l) {
        MA_CUDA(cudaEventRecord(ctx->ev_join[l - 1], ctx->aux_stream[l - 1]));
        MA_CUDA(cudaStreamWaitEvent(ctx->stream, ctx->ev_join[l - 1], 0));
    }
    return st;
}

static void fill_tables(ma_fft_plan* plan, LargeParams& p) {
    p.n = plan->n;
    p.n1 = plan->n1;
    p.n2 = plan->n2;
    p.scratch = plan->d_scratch;
    p.twM2 = plan->d_twM;
    p.twN2 = plan->d_twN;
    p.tw1 = plan->d_tw1;
    p.twc = plan->d_twc;
    p.twr = plan->d_twr;
    p.twr_step = plan->d_twr + (size_t)(plan->n2 / 2 + 1) * fft_plan_threads(plan->n1);
    p.in_stride = plan->n;
    p.valid = plan->n;
    p.error_flag = plan->ctx->d_error_flag;
}

ma_status launch_r2c_large(ma_fft_plan* plan, const float* in, float* out_a, float* out_b, float* mag,
                           int mag_kind, float db_scale, int64_t batch, int layout, float2* scratch,
                           int64_t scratch_batch) {
    const int64_t n = plan->n, half = n / 2;
    const bool own = scratch == nullptr;  // a caller-provided pass buffer is used as one lane
    return for_chunks(plan, batch, own ? plan->d_scratch : scratch, own ? plan->scratch_batch : scratch_batch,
                      own ? plan->scratch_lanes : 1, [&](int64_t done, int64_t count, float2* lane_scratch, cudaStream_t st) {
        LargeParams p{};
        fill_tables(plan, p);
        p.scratch = lane_scratch;
        p.batch = count;
        p.in = in + done * n;
        p.layout = layout;
        p.mag_kind = mag_kind;
        p.db_scale = db_scale;
        if (layout == LAYOUT_FULL_SPLIT) {
            p.out_a = out_a + done * n;
            p.out_b = out_b + done * n;
        } else {
            p.out_a = out_a + done * 2 * (layout == LAYOUT_HALF_PACKED ? half : half + 1);
        }
        p.mag = mag ? mag + done * (half + 1) : nullptr;
        MA_TRY(dispatch_cols(plan, p, false, st));
        return dispatch_rows(plan, p, false, st);
    });
}

ma_status launch_c2r_large(ma_fft_plan* plan, const float* in_a, const float* in_b, float* out, int64_t batch,
                           int layout) {
    const int64_t n = plan->n, half = n / 2;
    return for_chunks(plan, batch, plan->d_scratch, plan->scratch_batch, plan->scratch_lanes,
                      [&](int64_t done, int64_t count, float2* lane_scratch, cudaStream_t st) {
        LargeParams p{};
        fill_tables(plan, p);
        p.scratch = lane_scratch;
        p.batch = count;
        p.layout = layout;
        if (layout == LAYOUT_FULL_SPLIT) {
            p.in = in_a + done * n;
            p.in_b = in_b + done * n;
        } else {
            p.in = in_a + done * 2 * (layout == LAYOUT_HALF_PACKED ? half : half + 1);
        }
        p.out_a = out + done * n;
        MA_TRY(dispatch_rows(plan, p, true, st));
        return dispatch_cols(plan, p, true, st);
    });
}

// Overlap-add of `count` inverse frames (frame f0 + i at frames[i*n]) into one signal's output:
// out[o] += sum over those frames covering o of frame[o - f*hop] * window[o - f*hop], frames taken
// in increasing order (the reference's loop order).  One thread per output sample of the span.
__global__ void __launch_bounds__(256) ola_add_kernel(const float* __restrict__ frames, int64_t count, int64_t f0, int n,
                                                      int hop, const float* __restrict__ window, float* __restrict__ out) {
    const int64_t span = (count - 1) * hop + n;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < span; i += (int64_t)gridDim.x * blockDim.x) {
        int64_t lo = i >= n ? (i - n) / hop + 1 : 0;
        int64_t hi = i / hop;
        if (hi > count - 1) hi = count - 1;
        float acc = 0.f;
        for (int64_t f = lo; f <= hi; ++f) {
            const int64_t k = i - f * hop;
            const float v = __ldcs(frames + f * n + k);
            acc += window != nullptr ? v * __ldg(window + k) : v;
        }
        out[f0 * hop + i] += acc;
    }
}

// out[o] /= max(sum of window^2 over the frames covering o, floor)   (STFT.swift:491-522)
__global__ void __launch_bounds__(256) ola_normalise_kernel(float* __restrict__ out, int64_t out_len, const float* __restrict__ window,
                                                            int n, int hop, int64_t frames, float floor) {
    for (int64_t o = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; o < out_len; o += (int64_t)gridDim.x * blockDim.x)
        out[o] = out[o] / window_sum_at(window, o, n, hop, frames, floor);
}

static int stream_grid(ma_context* ctx, int64_t total) {
    const int64_t want = (total + 255) / 256, cap = (int64_t)ctx->sm_count * 8;
    return (int)(want < cap ? (want > 0 ? want : 1) : cap);
}

ma_status launch_stft_large(ma_fft_plan* plan, const float* signals, int64_t signal_stride, int64_t frames,
                            int64_t n_signals, float* out_a, float* out_b, float* mag, int mag_kind,
                            float db_scale, int layout) {
    const int64_t n = plan->n, half = n / 2;
    for (int64_t s = 0; s < n_signals; ++s) {
        MA_TRY(for_chunks(plan, frames, plan->d_scratch, plan->scratch_batch, plan->scratch_lanes,
                          [&](int64_t f0, int64_t count, float2* lane_scratch, cudaStream_t st) {
            const int64_t g = s * frames + f0;  // global frame index of the chunk's first frame
            LargeParams p{};
            fill_tables(plan, p);
            p.scratch = lane_scratch;
            p.batch = count;
            p.in = signals + s * signal_stride + f0 * plan->hop;
            p.in_stride = plan->hop;
            p.window = plan->d_window;
            p.layout = layout;
            p.mag_kind = mag_kind;
            p.db_scale = db_scale;
            if (layout == LAYOUT_FULL_SPLIT) {
                p.out_a = out_a + g * n;
                p.out_b = out_b + g * n;
            } else {
                p.out_a = out_a + g * 2 * (layout == LAYOUT_HALF_PACKED ? half : half + 1);
            }
            p.mag = mag ? mag + g * (half + 1) : nullptr;
            MA_TRY(dispatch_cols(plan, p, false, st));
            return dispatch_rows(plan, p, false, st);
        }));
    }
    return MA_OK;
}

ma_status launch_istft_large(ma_fft_plan* plan, const float* in_a, const float* in_b, int64_t frames,
                             int64_t n_signals, float* out, int64_t out_stride, int64_t out_len, float floor,
                             int layout) {
    ma_context* ctx = plan->ctx;
    const int64_t n = plan->n, half = n / 2;
    const int64_t step = plan->scratch_batch * plan->scratch_lanes;  // inverse frames per round: every lane's chunk
    if (plan->d_frames == nullptr)  // first overlap-add through this plan
        MA_CUDA(cudaMalloc((void**)&plan->d_frames, sizeof(float) * (size_t)n * (size_t)step));
    const int64_t per_frame = layout == LAYOUT_FULL_SPLIT ? n : 2 * (layout == LAYOUT_HALF_PACKED ? half : half + 1);
    for (int64_t s = 0; s < n_signals; ++s) {
        float* row = out + s * out_stride;
        MA_CUDA(cudaMemsetAsync(row, 0, sizeof(float) * (size_t)out_len, ctx->stream));
        for (int64_t f0 = 0; f0 < frames; f0 += step) {
            const int64_t count = frames - f0 < step ? frames - f0 : step;
            const int64_t g = s * frames + f0;
            MA_TRY(launch_c2r_large(plan, in_a + g * per_frame, in_b ? in_b + g * per_frame : nullptr, plan->d_frames,
                                    count, layout));
            ola_add_kernel<<<stream_grid(ctx, (count - 1) * plan->hop + n), 256, 0, ctx->stream>>>(
                plan->d_frames, count, f0, (int)n, plan->hop, plan->d_window, row);
            MA_TRY(after_launch(ctx));
        }
        ola_normalise_kernel<<<stream_grid(ctx, out_len), 256, 0, ctx->stream>>>(row, out_len, plan->d_window, (int)n,
                                                                                 plan->hop, frames, floor);
        MA_TRY(after_launch(ctx));
    }
    return MA_OK;
}

// Spectrum of one real signal of `valid` samples (zero-padded to N) in pass-2 row order, for
// launch_conv_large.  spec_rows holds (N2/2+1) * N1 complex values.
ma_status launch_spec_rows_large(ma_fft_plan* plan, const float* in, int64_t valid, float2* spec_rows) {
    LargeParams p{};
    fill_tables(plan, p);
    p.batch = 1;
    p.in = in;
    p.valid = valid;
    p.spec_rows = spec_rows;
    MA_TRY(dispatch_cols(plan, p, false, plan->ctx->stream));
    return dispatch_rows_mul(plan, p, true, plan->ctx->stream);
}

// out[b][0..N) = inverse(forward(zero-padded in[b][0..valid)) * spectrum) for `batch` signals: three
// passes per chunk (columns forward, rows forward-multiply-inverse in place, columns inverse), the
// intermediate data staying in the L2-sized scratch.
ma_status launch_conv_large(ma_fft_plan* plan, const float* in, int64_t valid, int64_t in_stride,
                            const float2* spec_rows, float* out, int64_t batch) {
    const int64_t n = plan->n;
    return for_chunks(plan, batch, plan->d_scratch, plan->scratch_batch, plan->scratch_lanes,
                      [&](int64_t done, int64_t count, float2* lane_scratch, cudaStream_t st) {
        LargeParams p{};
        fill_tables(plan, p);
        p.scratch = lane_scratch;
        p.batch = count;
        p.in = in + done * in_stride;
        p.in_stride = in_stride;
        p.valid = valid;
        p.spec_rows = const_cast<float2*>(spec_rows);
        p.out_a = out + done * n;
        p.layout = LAYOUT_HALF_INTERLEAVED;
        MA_TRY(dispatch_cols(plan, p, false, st));
        MA_TRY(dispatch_rows_mul(plan, p, false, st));
        return dispatch_cols(plan, p, true, st);
    });
}

}  // namespace ma

// ---------------------------------------------------------------------------------------------
// Allocation-free forward transform (see ma_fft_forward_static_dev in the public header).
//
// The pass scratch lives in this file-scope device array.  In host code the name `g_static_scratch`
// is only a handle for the runtime, not a device address: handing it to a kernel would fault (or,
// where the GPU can reach host memory, silently use the wrong bytes).  The device address is
// looked up once per device with cudaGetSymbolAddress, with that device current, and that pointer
// is what the kernels receive.
static __device__ __align__(256) unsigned char g_static_scratch[MA_STATIC_SCRATCH_BYTES];

namespace {
std::atomic<float2*> g_static_scratch_addr[64];  // zero-initialised; one slot per device ordinal

// Device address of the static scratch on the current device (which must be `device`).  Threads
// that race on the first call all store the same address.
ma_status static_scratch_address(int device, float2** out) {
    if (device < 0 || device >= 64) return MA_ERR_INVALID_ARGUMENT;
    float2* addr = g_static_scratch_addr[device].load(std::memory_order_acquire);
    if (addr == nullptr) {
        void* ptr = nullptr;
        const cudaError_t e = cudaGetSymbolAddress(&ptr, g_static_scratch);
        if (e != cudaSuccess) return ma::cuda_fail(e);
        addr = static_cast<float2*>(ptr);
        g_static_scratch_addr[device].store(addr, std::memory_order_release);
    }
    *out = addr;
    return MA_OK;
}
}  // namespace

extern "C" ma_status ma_fft_forward_static_dev(ma_fft_plan* plan, const float* in, float* out_a, float* out_b,
                                               float* mag, int32_t mag_kind, float db_reference, int64_t batch,
                                               int32_t layout) {
    using namespace ma;
    if (plan == nullptr) return MA_ERR_INVALID_ARGUMENT;
    if (!plan->large)  // no scratch involved below 8192 points
        return ma_fft_forward_dev(plan, in, out_a, out_b, mag, mag_kind, db_reference, batch, layout);
    MA_TRY(enter(plan->ctx, MA_FAULT_LAUNCH));  // makes the context's device current
    if (batch == 0) return MA_OK;
    MA_TRY(check_forward_args(plan, in, out_a, out_b, mag, mag_kind, batch, layout));  // same checks as ma_fft_forward_dev
    const size_t per = (size_t)(plan->n2 / 2 + 1) * (size_t)plan->n1 * sizeof(float2);
    if (per > MA_STATIC_SCRATCH_BYTES) return MA_ERR_SCRATCH_LIMIT;
    float2* scratch = nullptr;
    MA_TRY(static_scratch_address(plan->ctx->device, &scratch));
    return launch_r2c_large(plan, in, out_a, out_b, mag, mag_kind, 1.0f / db_reference, batch, layout, scratch,
                            (int64_t)(MA_STATIC_SCRATCH_BYTES / per));
}
