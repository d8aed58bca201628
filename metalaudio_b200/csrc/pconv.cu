// Uniformly partitioned overlap-add convolution with a frequency-domain delay line (FDL).
//
// Data in HBM (all float2, "packed" half spectra: B complex bins per 2B-point block, bin 0
// holding (DC, Nyquist)):
//   H     [n_irs][P][B]      partition spectra of every impulse response
//   ring  [C][P][B]          delay line of the last P input-block spectra per channel
//   tl    [C][P-1+T][B]      whole-signal call: history followed by all T block spectra
//   Y     [C][T][B]          whole-signal call: accumulated output spectra
// Kernels:
//   r2c (fft_small.cu)       input blocks -> spectra (zero-padded to 2B in the loader)
//   pconv_mac_kernel         Y[c] = sum_p X[c][t-p] * H[ir(c)][p]; streams the delay line once,
//                            channels that share an IR are tiled so each H element is loaded
//                            once per tile and reused from registers
//   c2r / istft (fft_small)  inverse transform + block overlap-add
#include <cuda_pipeline.h>

#include <new>
#include <type_traits>
#include <vector>

#include "fft_plan.h"
#include "host_pipe.h"
#include "pconv_tiling.h"

struct ma_pconv {
    ma_context* ctx = nullptr;
    int block = 0;      // B
    int channels = 0;   // C
    ma_fft_plan* plan = nullptr;  // N = 2B
    int64_t taps = 0;
    int partitions = 0;  // P
    int n_irs = 0;
    int share = 1;       // channels per tile that share one IR (1, 2 or 4)
    float2* d_h = nullptr;
    int32_t* d_ch2ir = nullptr;
    float2* d_ring = nullptr;
    float* d_tail = nullptr;
    int write_index = 0;
    int splits = 1;              // partition splits of the streaming step
    float2* d_partial = nullptr; // [splits][C][B]
    int64_t reserved_len = 0;
    int64_t reserved_blocks = 0;
    float2* d_timeline = nullptr;
    float2* d_y = nullptr;
};

namespace ma {

struct MacParams {
    const float2* x;        // delay line or timeline
    int64_t x_chan_stride;  // float2 units
    const float2* h;
    const int32_t* ch2ir;
    float2* out;
    int64_t out_split_stride, out_chan_stride, out_t_stride;  // float2 units
    int block;       // B
    int partitions;  // P
    int w0;          // slot of partition 0 for t = 0
    int wrap;        // P for the ring, 0 for the timeline
    int splits;
    int p_per_split;
    int bin_tiles;
    int bpt;         // threads covering one spectrum tile (power of two <= 128)
    int dependent_launch;  // streaming step: launched with programmatic stream serialization
    int cluster;           // CTAs per thread-block cluster along the splits (1: none): their partial sums are
                           // added up through distributed shared memory and rank 0 alone writes
};

constexpr int kMacThreads = 128;

template <int VEC>
struct VecT;
template <>
struct VecT<1> { using type = float2; };
template <>
struct VecT<2> { using type = float4; };

// One CTA: CT channels sharing an IR, one tile of bins, one range of partitions, one block
// index t (blockIdx.y).  Threads along bins (VEC bins each); when a spectrum tile needs fewer
// than 128 threads the remaining thread rows take interleaved partitions and are reduced
// through shared memory.  STREAM selects evict-first loads for the delay line (read once).
template <int CT, int VEC, bool STREAM>
__global__ void __launch_bounds__(kMacThreads) pconv_mac_kernel(const MacParams q) {
    using V = typename VecT<VEC>::type;
    __shared__ float2 red[kMacThreads * CT * VEC];
    if (q.dependent_launch) {  // streaming step: the new delay-line slot comes from the kernel before this one
        asm volatile("griddepcontrol.wait;" ::: "memory");
        asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    }
    const int tid = threadIdx.x;
    const int bpt = q.bpt;
    const int kb = tid & (bpt - 1);
    const int pl = tid / bpt;
    const int PL = kMacThreads / bpt;
    int bx = blockIdx.x;
    const int split = bx % q.splits;
    bx /= q.splits;
    const int bt = bx % q.bin_tiles;
    const int ctile = bx / q.bin_tiles;
    const int t = blockIdx.y;
    const int c0 = ctile * CT;
    const int e = (bt * bpt + kb) * VEC;  // first bin of this thread
    const bool dc = (e == 0);
    const int B = q.block;
    const int p_beg = split * q.p_per_split;
    int p_end = p_beg + q.p_per_split;
    if (p_end > q.partitions) p_end = q.partitions;

    const float2* hb = q.h + (int64_t)__ldg(q.ch2ir + c0) * q.partitions * B + e;
    const float2* xb = q.x + (int64_t)c0 * q.x_chan_stride + e;
    const int w = q.w0 + t;

    float2 acc[CT][VEC];
#pragma unroll
    for (int c = 0; c < CT; ++c)
#pragma unroll
        for (int v = 0; v < VEC; ++v) acc[c][v] = make_float2(0.f, 0.f);

#pragma unroll 4
    for (int p = p_beg + pl; p < p_end; p += PL) {
        const V hv = __ldg(reinterpret_cast<const V*>(hb + (int64_t)p * B));
        float2 h[VEC];
        h[0] = make_float2(reinterpret_cast<const float*>(&hv)[0], reinterpret_cast<const float*>(&hv)[1]);
        if constexpr (VEC == 2)
            h[1] = make_float2(reinterpret_cast<const float*>(&hv)[2], reinterpret_cast<const float*>(&hv)[3]);
        // bin 0 carries (DC, Nyquist): component-wise product instead of a complex one
        const float ha = dc ? 0.f : h[0].y;
        const float hc = dc ? h[0].y : h[0].x;
        int slot = w - p;
        if (slot < 0) slot += q.wrap;
        const float2* xp = xb + (int64_t)slot * B;
#pragma unroll
        for (int c = 0; c < CT; ++c) {
            const V* src = reinterpret_cast<const V*>(xp + (int64_t)c * q.x_chan_stride);
            V xv;
            if (STREAM) xv = __ldcs(src);
            else xv = __ldg(src);
            const float* xf = reinterpret_cast<const float*>(&xv);
            acc[c][0].x = fmaf(xf[0], h[0].x, acc[c][0].x);
            acc[c][0].x = fmaf(-xf[1], ha, acc[c][0].x);
            acc[c][0].y = fmaf(xf[0], ha, acc[c][0].y);
            acc[c][0].y = fmaf(xf[1], hc, acc[c][0].y);
            if constexpr (VEC == 2) {
                acc[c][1].x = fmaf(xf[2], h[1].x, acc[c][1].x);
                acc[c][1].x = fmaf(-xf[3], h[1].y, acc[c][1].x);
                acc[c][1].y = fmaf(xf[2], h[1].y, acc[c][1].y);
                acc[c][1].y = fmaf(xf[3], h[1].x, acc[c][1].y);
            }
        }
    }

    if (PL > 1) {
#pragma unroll
        for (int c = 0; c < CT; ++c)
#pragma unroll
            for (int v = 0; v < VEC; ++v) red[(c * VEC + v) * kMacThreads + tid] = acc[c][v];
        __syncthreads();
        if (pl == 0) {
            for (int r = 1; r < PL; ++r) {
#pragma unroll
                for (int c = 0; c < CT; ++c)
#pragma unroll
                    for (int v = 0; v < VEC; ++v) {
                        const float2 o = red[(c * VEC + v) * kMacThreads + r * bpt + kb];
                        acc[c][v].x += o.x;
                        acc[c][v].y += o.y;
                    }
            }
        }
    }
    int out_split = split;
    bool writer = pl == 0;
    if (q.cluster > 1) {
        // The cluster's CTAs hold consecutive splits of one tile.  Each leaves its sums in its own shared
        // memory; after the cluster barrier rank 0 adds the others' in rank order (a fixed order: results
        // do not depend on timing) through distributed shared memory and writes one partial spectrum for
        // the whole cluster.  The second barrier keeps every CTA's shared memory alive until rank 0 has
        // read it.  Cluster barriers are hardware barriers among co-scheduled CTAs, not spin waits.
        uint32_t rank;
        asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(rank));
        if (PL > 1) __syncthreads();  // the intra-CTA reduction above is done with `red`
        if (pl == 0) {
#pragma unroll
            for (int c = 0; c < CT; ++c)
#pragma unroll
                for (int v = 0; v < VEC; ++v) red[(c * VEC + v) * kMacThreads + tid] = acc[c][v];
        }
        asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
        if (rank == 0 && pl == 0) {
            for (int r = 1; r < q.cluster; ++r) {
#pragma unroll
                for (int c = 0; c < CT; ++c)
#pragma unroll
                    for (int v = 0; v < VEC; ++v) {
                        const uint32_t local = static_cast<uint32_t>(__cvta_generic_to_shared(&red[(c * VEC + v) * kMacThreads + tid]));
                        uint32_t remote;
                        asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local), "r"(r));
                        float2 o;
                        asm volatile("ld.shared::cluster.v2.f32 {%0, %1}, [%2];" : "=f"(o.x), "=f"(o.y) : "r"(remote) : "memory");
                        acc[c][v].x += o.x;
                        acc[c][v].y += o.y;
                    }
            }
        }
        asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
        writer = pl == 0 && rank == 0;
        out_split = split / q.cluster;
    }
    if (writer) {
#pragma unroll
        for (int c = 0; c < CT; ++c) {
            float2* o = q.out + (int64_t)out_split * q.out_split_stride + (int64_t)(c0 + c) * q.out_chan_stride +
                        (int64_t)t * q.out_t_stride + e;
#pragma unroll
            for (int v = 0; v < VEC; ++v) o[v] = acc[c][v];
        }
    }
}

// Whole-signal form of the same multiply-accumulate, tiled over time.  With every block
// spectrum of the call already in the timeline, output blocks are independent, and TT consecutive
// outputs of one (channel, bin) reuse the same partition spectra: a thread keeps TT accumulators
// and a sliding window of TT timeline values in registers, and per partition takes ONE new
// timeline value and ONE partition value for TT complex multiply-accumulates (4*TT FMAs).
// A CTA is 4 warps = 4 consecutive time tiles of one channel and 32 bins (lanes along bins).
// Its warps need the same partition rows and overlapping timeline rows, so both are staged in
// shared memory by 16-byte asynchronous copies, a chunk of TT partitions ahead: the timeline
// rows in a ring of 128 rows (each row enters once per CTA), the partition rows double-buffered.
// That leaves about 0.25 byte of L2 traffic per complex multiply-accumulate and makes the FMA
// pipe the limiter.  One barrier per chunk (1024 FMAs per thread apart).
// TWO_LEVEL: every kFlushChunks chunks the running sums are added into a second set of
// accumulators and cleared, so no float32 sum runs over more than TT*kFlushChunks partitions
// (blocked summation: the rounding error of thousands of partitions grows with the block
// length, not with the partition count).
constexpr int kFlushChunks = 16;
template <int TT, bool TWO_LEVEL>
__global__ void __launch_bounds__(128) pconv_mac_tiled_kernel(const MacParams q, int t_total, int64_t tl_len) {
    using TL = MacTiling<TT>;
    constexpr int RING = TL::kRing;
    __shared__ __align__(16) float2 xs[RING][32];
    __shared__ __align__(16) float2 hs[2][TT][32];
    const int tid = threadIdx.x;
    const int lane = tid & 31;
    const int warp = tid >> 5;
    const int B = q.block, P = q.partitions;
    const int bin_tiles = B >> 5;
    const int bt = blockIdx.x % bin_tiles;
    const int c = blockIdx.x / bin_tiles;
    const bool dc = (bt == 0 && lane == 0);
    const int t0_cta = blockIdx.y * 4 * TT;
    if (t0_cta >= t_total) return;
    const float2* xc = q.x + (int64_t)c * q.x_chan_stride + bt * 32;
    const float2* hc = q.h + (int64_t)__ldg(q.ch2ir + c) * P * B + bt * 32;
    const int64_t base0 = TL::base0(P, t0_cta);          // timeline row of the CTA's first output at p = 0
    const int64_t base = base0 + warp * TT;              // ... of this warp's first output

    // 16-byte copies: a row of 32 bins is 16 segments
    auto load_x_rows = [&](int64_t first, int count) {
        for (int idx = tid; idx < count * 16; idx += 128) {
            const int64_t row = first + (idx >> 4);
            const int seg = idx & 15;
            const int64_t src = TL::fetch_row(row, tl_len);  // clamped into the channel's own timeline
            __pipeline_memcpy_async(&xs[row & (RING - 1)][seg * 2], xc + src * B + seg * 2, 16);
        }
    };
    auto load_h_rows = [&](int buf, int p0) {
        for (int idx = tid; idx < TT * 16; idx += 128) {
            const int pr = p0 + (idx >> 4);
            const int seg = idx & 15;
            if (pr < P) __pipeline_memcpy_async(&hs[buf][idx >> 4][seg * 2], hc + (int64_t)pr * B + seg * 2, 16);
        }
    };

    load_x_rows(TL::chunk0_first(P, t0_cta), TL::kChunk0Rows);  // rows of chunk 0: [base0-TT+1, base0+4TT-1]
    load_h_rows(0, 0);
    __pipeline_commit();
    __pipeline_wait_prior(0);
    __syncthreads();

    float2 acc[TT], xw[TT];
    float2 acc2[TWO_LEVEL ? TT : 1];
#pragma unroll
    for (int i = 0; i < TT; ++i) {
        acc[i] = make_float2(0.f, 0.f);
        if constexpr (TWO_LEVEL) acc2[i] = make_float2(0.f, 0.f);
        xw[i] = xs[(base + i) & (RING - 1)][lane];
    }
    int buf = 0;
    int since_flush = 0;
    for (int p0 = 0; p0 < P; p0 += TT) {
        if (p0 + TT < P) {  // stage the next chunk while this one is consumed
            load_x_rows(TL::lookahead_first(P, t0_cta, p0), TT);
            load_h_rows(buf ^ 1, p0 + TT);
        }
        __pipeline_commit();
        // one chunk of TT partitions; FULL: all of them exist, so no per-partition test
        auto chunk = [&](auto full) {
            constexpr bool FULL = decltype(full)::value;
            const float2* hrow = &hs[buf][0][lane];
#pragma unroll
            for (int j = 0; j < TT; ++j) {
                const int p = p0 + j;
                if (FULL || p < P) {
                    // slot (i - j) mod TT holds timeline row base + i - p; the row base - p enters at i = 0
                    if (j > 0 || p0 > 0) xw[(TT - j) % TT] = xs[(base - p) & (RING - 1)][lane];
                    const float2 h = hrow[j * 32];
                    const float ha = dc ? 0.f : h.y;   // bin 0 carries (DC, Nyquist): component-wise product
                    const float hb = dc ? h.y : h.x;
#pragma unroll
                    for (int i = 0; i < TT; ++i) {
                        const float2 xv = xw[(i - j + TT) % TT];
                        acc[i].x = fmaf(xv.x, h.x, acc[i].x);
                        acc[i].x = fmaf(-xv.y, ha, acc[i].x);
                        acc[i].y = fmaf(xv.x, ha, acc[i].y);
                        acc[i].y = fmaf(xv.y, hb, acc[i].y);
                    }
                }
            }
        };
        if (p0 + TT <= P) chunk(std::true_type{});
        else chunk(std::false_type{});
        if constexpr (TWO_LEVEL) {
            if (++since_flush == kFlushChunks) {
                since_flush = 0;
#pragma unroll
                for (int i = 0; i < TT; ++i) {
                    acc2[i].x += acc[i].x;
                    acc2[i].y += acc[i].y;
                    acc[i] = make_float2(0.f, 0.f);
                }
            }
        }
        __pipeline_wait_prior(0);
        __syncthreads();
        buf ^= 1;
    }
    if constexpr (TWO_LEVEL) {
#pragma unroll
        for (int i = 0; i < TT; ++i) {
            acc[i].x += acc2[i].x;
            acc[i].y += acc2[i].y;
        }
    }
    const int t0 = t0_cta + warp * TT;
    float2* o = q.out + (int64_t)c * q.out_chan_stride + (int64_t)t0 * q.out_t_stride + bt * 32 + lane;
#pragma unroll
    for (int i = 0; i < TT; ++i)
        if (t0 + i < t_total) o[(int64_t)i * q.out_t_stride] = acc[i];
}

constexpr int kTwoLevelFrom = 2048;

static ma_status launch_mac_tiled(ma_pconv* pc, const MacParams& q, int channels, int64_t t_count, int64_t tl_len) {
    constexpr int TT = 16;
    ma_context* ctx = pc->ctx;
    const int bin_tiles = pc->block >> 5;
    const int64_t t_ctas = (t_count + 4 * TT - 1) / (4 * TT);
    int64_t done = 0;
    while (done < t_ctas) {  // grid.y limit
        int64_t ny = t_ctas - done;
        if (ny > 32768) ny = 32768;
        MacParams qq = q;
        const int64_t t_first = done * 4 * TT;
        qq.out = q.out + t_first * q.out_t_stride;
        qq.x = q.x + t_first * pc->block;  // shifts the timeline origin by t_first rows
        dim3 grid((unsigned)(bin_tiles * channels), (unsigned)ny, 1);
        // Blocked summation once a running sum would cover more than kTwoLevelFrom partitions.
        if (pc->partitions >= kTwoLevelFrom)
            pconv_mac_tiled_kernel<TT, true><<<grid, 128, 0, ctx->stream>>>(qq, (int)(t_count - t_first), tl_len - t_first);
        else
            pconv_mac_tiled_kernel<TT, false><<<grid, 128, 0, ctx->stream>>>(qq, (int)(t_count - t_first), tl_len - t_first);
        MA_TRY(after_launch(ctx));
        done += ny;
    }
    return MA_OK;
}

template <int CT, int VEC, bool STREAM>
static ma_status launch_mac_t(ma_context* ctx, const MacParams& q, int chan_tiles, int64_t t_count) {
    int64_t done = 0;
    while (done < t_count) {
        int64_t ny = t_count - done;
        if (ny > 32768) ny = 32768;
        MacParams qq = q;
        qq.w0 = q.w0 + (int)done;
        qq.out = q.out + done * q.out_t_stride;
        dim3 grid((unsigned)(chan_tiles * q.bin_tiles * q.splits), (unsigned)ny, 1);
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = grid;
        cfg.blockDim = dim3(kMacThreads);
        cfg.stream = ctx->stream;
        cudaLaunchAttribute attr[2];
        int n_attr = 0;
        if (q.dependent_launch) {
            attr[n_attr].id = cudaLaunchAttributeProgrammaticStreamSerialization;
            attr[n_attr].val.programmaticStreamSerializationAllowed = 1;
            ++n_attr;
        }
        if (q.cluster > 1) {  // consecutive splits of a tile (consecutive blockIdx.x) form a cluster
            attr[n_attr].id = cudaLaunchAttributeClusterDimension;
            attr[n_attr].val.clusterDim.x = (unsigned)q.cluster;
            attr[n_attr].val.clusterDim.y = 1;
            attr[n_attr].val.clusterDim.z = 1;
            ++n_attr;
        }
        cfg.attrs = attr;
        cfg.numAttrs = n_attr;
        (void)cudaLaunchKernelEx(&cfg, pconv_mac_kernel<CT, VEC, STREAM>, qq);  // an error is picked up by after_launch
        MA_TRY(after_launch(ctx));
        done += ny;
    }
    return MA_OK;
}

static ma_status launch_mac(ma_pconv* pc, MacParams q, int channels, bool stream, int64_t t_count) {
    const int B = pc->block;
    const int vec = B >= 2 ? 2 : 1;
    const int bp = B / vec;  // threads per spectrum
    q.bpt = bp < kMacThreads ? bp : kMacThreads;
    q.bin_tiles = bp / q.bpt;
    const int ct = pc->share;
    const int chan_tiles = channels / ct;
    ma_context* ctx = pc->ctx;
#define MAC_CASE(CT_, VEC_)                                                                        \
    if (ct == CT_ && vec == VEC_)                                                                  \
        return stream ? launch_mac_t<CT_, VEC_, true>(ctx, q, chan_tiles, t_count)                 \
                      : launch_mac_t<CT_, VEC_, false>(ctx, q, chan_tiles, t_count);
    MAC_CASE(1, 1) MAC_CASE(2, 1) MAC_CASE(4, 1) MAC_CASE(1, 2) MAC_CASE(2, 2) MAC_CASE(4, 2)
#undef MAC_CASE
    return MA_ERR_UNSUPPORTED;
}

// Streaming step with many partition splits: adds the partial spectra up, split 0 first, and
// leaves the total in slot 0, one thread per 16 bytes with eight loads in flight.  The inverse
// transform behind it then reads one spectrum per channel; walking `splits` partials inside that
// kernel costs a memory round trip per partial on a handful of CTAs, which with few channels per
// GPU (many splits) was the longest part of a step.  Same summation order as that walk.
__global__ void __launch_bounds__(256) pconv_sum_partials_kernel(float4* __restrict__ partial, int64_t n4,
                                                                 int64_t split_stride4, int splits) {
    asm volatile("griddepcontrol.wait;" ::: "memory");  // the multiply-accumulate before this kernel has finished
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
    if (i >= n4) return;
    float4 acc = __ldcg(partial + i);
#pragma unroll 8
    for (int sp = 1; sp < splits; ++sp) {
        const float4 v = __ldcg(partial + sp * split_stride4 + i);
        acc.x += v.x;
        acc.y += v.y;
        acc.z += v.z;
        acc.w += v.w;
    }
    partial[i] = acc;
}

// Thread-block cluster size of the streaming step's multiply-accumulate: with many partition splits, groups
// of eight (four, two) consecutive splits reduce their sums on chip and write one partial spectrum.
static int step_cluster(int splits) {
    // Measured (block 256, 512 partitions): 16 / 64 / 128 channels 21.4 / 27.4 / 35.3 -> 14.8 / 24.1 / 33.4 us
    // per step; below 16 splits (256 channels and more) clusters cost 2-4 %, so those keep one CTA each.
    if (splits < 16) return 1;
    for (int s : {8, 4, 2})
        if (splits % s == 0) return s;
    return 1;
}

// Partial spectra are summed by their own kernel from this many splits up.
constexpr int kSumKernelFromSplits = 16;  // measured: 9 splits are faster summed inside the inverse kernel, 19 and 37 by this one

// Ordered copies between the ring and the timeline.
// to_timeline: tl[c][j] = ring[c][(w - (P-1-j)) mod P], j < P-1.
// to_ring:     ring[c][j] = tl[c][first + j], j < P.
__global__ void pconv_history_kernel(float2* __restrict__ ring, float2* __restrict__ tl, int64_t tl_chan_stride,
                                     int P, int B, int w, int64_t first, int to_timeline, int channels) {
    const int rows = to_timeline ? P - 1 : P;
    const int64_t total = (int64_t)channels * rows * B;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (int64_t)gridDim.x * blockDim.x) {
        const int k = (int)(i % B);
        const int64_t r = i / B;
        const int j = (int)(r % rows);
        const int64_t c = r / rows;
        if (to_timeline) {
            int slot = w - (P - 1 - j);
            slot %= P;
            if (slot < 0) slot += P;
            tl[c * tl_chan_stride + (int64_t)j * B + k] = ring[(c * P + slot) * B + k];
        } else {
            ring[(c * P + j) * B + k] = tl[c * tl_chan_stride + (first + j) * B + k];
        }
    }
}

static void free_signal_buffers(ma_pconv* pc) {
    if (pc->d_timeline) (void)cudaFree(pc->d_timeline);
    if (pc->d_y) (void)cudaFree(pc->d_y);
    pc->d_timeline = nullptr;
    pc->d_y = nullptr;
    pc->reserved_len = 0;
    pc->reserved_blocks = 0;
}

static void free_kernel_buffers(ma_pconv* pc) {
    if (pc->d_h) (void)cudaFree(pc->d_h);
    if (pc->d_ch2ir) (void)cudaFree(pc->d_ch2ir);
    if (pc->d_ring) (void)cudaFree(pc->d_ring);
    if (pc->d_tail) (void)cudaFree(pc->d_tail);
    if (pc->d_partial) (void)cudaFree(pc->d_partial);
    pc->d_h = nullptr;
    pc->d_ch2ir = nullptr;
    pc->d_ring = nullptr;
    pc->d_tail = nullptr;
    pc->d_partial = nullptr;
    free_signal_buffers(pc);
    (void)cudaGetLastError();
}

}  // namespace ma

using namespace ma;

extern "C" {

ma_status ma_pconv_create(ma_context* ctx, int32_t block_size, int32_t n_channels, ma_pconv** out) {
    if (out == nullptr) return MA_ERR_INVALID_ARGUMENT;
    *out = nullptr;
    MA_TRY(enter(ctx, MA_FAULT_ALLOC));
    if (block_size <= 0 || n_channels <= 0) return MA_ERR_INVALID_ARGUMENT;
    if ((block_size & (block_size - 1)) != 0) return MA_ERR_SIZE_NOT_POW2;
    if (2 * (int64_t)block_size > kMaxSmallN) return MA_ERR_UNSUPPORTED;
    ma_pconv* pc = new (std::nothrow) ma_pconv();
    if (pc == nullptr) return MA_ERR_ALLOC;
    pc->ctx = ctx;
    pc->block = block_size;
    pc->channels = n_channels;
    ma_status st = ma_fft_plan_create(ctx, 2 * block_size, nullptr, block_size, &pc->plan);
    if (st != MA_OK) {
        delete pc;
        return st;
    }
    *out = pc;
    return MA_OK;
}

ma_status ma_pconv_destroy(ma_pconv* pc) {
    if (pc == nullptr) return MA_OK;
    if (pc->ctx) {
        (void)cudaSetDevice(pc->ctx->device);
        (void)cudaStreamSynchronize(pc->ctx->stream);
    }
    free_kernel_buffers(pc);
    ma_fft_plan_destroy(pc->plan);
    delete pc;
    return MA_OK;
}

ma_status ma_pconv_set_kernels(ma_pconv* pc, const float* irs, int64_t taps, int32_t n_irs,
                               const int32_t* channel_to_ir) {
    if (pc == nullptr) return MA_ERR_INVALID_ARGUMENT;
    ma_context* ctx = pc->ctx;
    MA_TRY(enter(ctx, MA_FAULT_ALLOC));
    if (irs == nullptr || n_irs <= 0) return MA_ERR_INVALID_ARGUMENT;
    if (taps <= 0) return MA_ERR_EMPTY_KERNEL;
    const int B = pc->block, C = pc->channels;
    const int64_t P64 = (taps + B - 1) / B;
    if (P64 > (1 << 24)) return MA_ERR_OUTPUT_OVERFLOW;
    const int P = (int)P64;
    std::vector<int32_t> map((size_t)C, 0);
    if (channel_to_ir != nullptr) {
        for (int c = 0; c < C; ++c) {
            if (channel_to_ir[c] < 0 || channel_to_ir[c] >= n_irs) return MA_ERR_INVALID_ARGUMENT;
            map[(size_t)c] = channel_to_ir[c];
        }
    }
    // Largest aligned channel group (4, 2, 1) whose members all use one IR.
    int share = 1;
    for (int cand : {4, 2}) {
        if (C % cand != 0) continue;
        bool ok = true;
        for (int c = 0; c < C && ok; ++c) ok = map[(size_t)c] == map[(size_t)(c - c % cand)];
        if (ok) {
            share = cand;
            break;
        }
    }
    MA_CUDA(cudaStreamSynchronize(ctx->stream));
    free_kernel_buffers(pc);
    pc->taps = taps;
    pc->partitions = P;
    pc->n_irs = n_irs;
    pc->share = share;
    pc->write_index = 0;
    // Partition splits of the streaming step: about 5.25 CTAs per SM in all (the multiply-accumulate
    // kernel fits 7 of its 128-thread CTAs on an SM; measured for 512 / 256 / 128 channels of block 256
    // with 512 partitions: 768 CTAs 92 / 53 / 35 us per step, 640 CTAs 99 / 58 / 36 us, 1024 CTAs
    // 97 / 58 / 36 us - a wave that nearly fills the device, with room left for the step's other
    // kernels), each split still covering at least eight partitions per thread row.
    {
        const int vec = B >= 2 ? 2 : 1;
        const int bp = B / vec;
        const int bpt = bp < kMacThreads ? bp : kMacThreads;
        const int rows = kMacThreads / bpt;
        const int64_t tiles = (int64_t)(C / share) * (bp / bpt);
        int64_t want = ((int64_t)ctx->sm_count * 21 / 4 + tiles / 2) / tiles;
        int64_t max_splits = P / (8 * rows);
        if (max_splits < 1) max_splits = 1;
        if (want > max_splits) want = max_splits;
        if (want < 1) want = 1;
        if (want > 64) want = 64;
        if (want >= 16) want = (want + 4) / 8 * 8;  // whole clusters of eight splits (see step_cluster)
        if (want > max_splits) want = max_splits;
        pc->splits = (int)want;
    }
    const size_t spec_bytes = (size_t)P * B * sizeof(float2);
    ma_status st = MA_OK;
    cudaError_t e = cudaMalloc((void**)&pc->d_h, spec_bytes * (size_t)n_irs);
    if (e == cudaSuccess) e = cudaMalloc((void**)&pc->d_ch2ir, sizeof(int32_t) * (size_t)C);
    if (e == cudaSuccess) e = cudaMalloc((void**)&pc->d_ring, spec_bytes * (size_t)C);
    if (e == cudaSuccess) e = cudaMalloc((void**)&pc->d_tail, sizeof(float) * (size_t)C * B);
    if (e == cudaSuccess)
        e = cudaMalloc((void**)&pc->d_partial, sizeof(float2) * (size_t)pc->splits * (size_t)C * B);
    if (e != cudaSuccess) st = cuda_fail(e);
    if (st == MA_OK) st = copy_h2d(ctx, pc->d_ch2ir, map.data(), sizeof(int32_t) * (size_t)C);
    // Partition spectra: the taps are the "signals", partitions the "frames" at hop B, each
    // frame's samples beyond B (and beyond the end of the IR) read as zero.
    float* d_taps = nullptr;
    const int64_t tstride = taps + (taps & 1);
    if (st == MA_OK) st = temp_alloc(ctx, sizeof(float) * (size_t)(tstride * n_irs), (void**)&d_taps);
    for (int i = 0; i < n_irs && st == MA_OK; ++i)
        st = copy_h2d(ctx, d_taps + (int64_t)i * tstride, irs + (int64_t)i * taps, sizeof(float) * (size_t)taps);
    if (st == MA_OK) {
        R2CParams p{};
        p.in = d_taps;
        p.signal_stride = tstride;
        p.frames_per_signal = P;
        p.total_frames = (int64_t)P * n_irs;
        p.signal_len = taps;
        p.hop = B;
        p.frame_valid = B;
        p.out_a = reinterpret_cast<float*>(pc->d_h);
        p.out_signal_stride = (int64_t)P * B;
        p.out_frame_stride = B;
        p.layout = LAYOUT_HALF_PACKED;
        p.mag_kind = MAG_NONE;
        st = launch_r2c_small(pc->plan, p);
    }
    temp_free(ctx, d_taps);
    if (st == MA_OK) st = ma_pconv_reset(pc);
    if (st == MA_OK) {
        cudaError_t e2 = cudaStreamSynchronize(ctx->stream);
        if (e2 != cudaSuccess) st = cuda_fail(e2);
    }
    if (st != MA_OK) free_kernel_buffers(pc);
    return st;
}

ma_status ma_pconv_partition_count(ma_pconv* pc, int32_t* partitions) {
    if (pc == nullptr || partitions == nullptr) return MA_ERR_INVALID_ARGUMENT;
    *partitions = pc->partitions;
    return MA_OK;
}

ma_status ma_pconv_step_splits(ma_pconv* pc, int32_t set_to, int32_t* splits) {
    if (pc == nullptr) return MA_ERR_INVALID_ARGUMENT;
    if (pc->d_h == nullptr) return MA_ERR_KERNEL_NOT_CONFIGURED;
    if (set_to > 0) {
        ma_context* ctx = pc->ctx;
        MA_TRY(enter(ctx, MA_FAULT_ALLOC));
        if (set_to > pc->partitions || set_to > 64) return MA_ERR_INVALID_ARGUMENT;
        if (set_to != pc->splits) {
            // the partial spectra of earlier steps may still be in use: wait, then resize
            MA_CUDA(cudaStreamSynchronize(ctx->stream));
            float2* fresh = nullptr;
            MA_CUDA(cudaMalloc((void**)&fresh, sizeof(float2) * (size_t)set_to * (size_t)pc->channels * pc->block));
            if (pc->d_partial) (void)cudaFree(pc->d_partial);
            pc->d_partial = fresh;
            pc->splits = set_to;
        }
    }
    if (splits != nullptr) *splits = pc->splits;
    return MA_OK;
}

ma_status ma_pconv_reset(ma_pconv* pc) {
    if (pc == nullptr) return MA_ERR_INVALID_ARGUMENT;
    MA_TRY(enter(pc->ctx, MA_FAULT_LAUNCH));
    if (pc->d_ring == nullptr) return MA_OK;  // nothing configured yet
    const size_t ring_bytes = (size_t)pc->channels * pc->partitions * pc->block * sizeof(float2);
    MA_CUDA(cudaMemsetAsync(pc->d_ring, 0, ring_bytes, pc->ctx->stream));
    MA_CUDA(cudaMemsetAsync(pc->d_tail, 0, sizeof(float) * (size_t)pc->channels * pc->block, pc->ctx->stream));
    pc->write_index = 0;
    return MA_OK;
}

ma_status ma_pconv_reserve(ma_pconv* pc, int64_t max_len) {
    if (pc == nullptr) return MA_ERR_INVALID_ARGUMENT;
    ma_context* ctx = pc->ctx;
    MA_TRY(enter(ctx, MA_FAULT_ALLOC));
    if (pc->d_h == nullptr) return MA_ERR_KERNEL_NOT_CONFIGURED;
    if (max_len <= 0) return MA_ERR_INVALID_ARGUMENT;
    if (max_len <= pc->reserved_len) return MA_OK;
    int64_t full;
    if (__builtin_add_overflow(max_len, pc->taps - 1, &full)) return MA_ERR_OUTPUT_OVERFLOW;
    const int64_t blocks = (full + pc->block - 1) / pc->block;
    MA_CUDA(cudaStreamSynchronize(ctx->stream));
    free_signal_buffers(pc);
    const size_t row = (size_t)pc->block * sizeof(float2);
    const size_t tl_bytes = (size_t)pc->channels * (size_t)(pc->partitions - 1 + blocks) * row;
    const size_t y_bytes = (size_t)pc->channels * (size_t)blocks * row;
    cudaError_t e = cudaMalloc((void**)&pc->d_timeline, tl_bytes ? tl_bytes : 16);
    if (e == cudaSuccess) e = cudaMalloc((void**)&pc->d_y, y_bytes ? y_bytes : 16);
    if (e != cudaSuccess) {
        ma_status st = cuda_fail(e);
        free_signal_buffers(pc);
        return st;
    }
    pc->reserved_len = max_len;
    pc->reserved_blocks = blocks;
    return MA_OK;
}

}  // extern "C"

// Whole-signal convolution of channels [c0, c0 + nc) (nc a multiple of the IR-sharing group): `in`
// and `out` point at channel c0's rows.  Every buffer of the object is per channel, so a range runs
// on its own slices; the delay-line position is reset by the caller once all ranges are queued.
static ma_status process_range(ma_pconv* pc, int c0, int nc, const float* in, int64_t len, int64_t in_stride,
                               float* out, int64_t out_stride, int64_t full) {
    ma_context* ctx = pc->ctx;
    const int B = pc->block, P = pc->partitions;
    const int64_t T = (full + B - 1) / B;
    const int64_t tl_len = (int64_t)P - 1 + T;
    const int64_t tl_stride = tl_len * B;
    float2* ring = pc->d_ring + (int64_t)c0 * P * B;
    float2* timeline = pc->d_timeline + (int64_t)c0 * tl_stride;
    float2* y = pc->d_y + (int64_t)c0 * T * B;

    // 1. history -> timeline prefix
    if (P > 1) {
        const int64_t total = (int64_t)nc * (P - 1) * B;
        int grid = (int)((total + 255) / 256 < (int64_t)ctx->sm_count * 8 ? (total + 255) / 256 : (int64_t)ctx->sm_count * 8);
        pconv_history_kernel<<<grid, 256, 0, ctx->stream>>>(ring, timeline, tl_stride, P, B, pc->write_index, 0, 1, nc);
        MA_TRY(after_launch(ctx));
    }
    // 2. all input blocks -> spectra
    {
        R2CParams p{};
        p.in = in;
        p.signal_stride = in_stride;
        p.frames_per_signal = T;
        p.total_frames = T * nc;
        p.signal_len = len;
        p.hop = B;
        p.frame_valid = B;
        p.out_a = reinterpret_cast<float*>(timeline + (int64_t)(P - 1) * B);
        p.out_signal_stride = tl_stride;
        p.out_frame_stride = B;
        p.layout = LAYOUT_HALF_PACKED;
        p.mag_kind = MAG_NONE;
        MA_TRY(launch_r2c_small(pc->plan, p));
    }
    // 3. delay-line multiply-accumulate for every (channel, block)
    {
        MacParams q{};
        q.x = timeline;
        q.x_chan_stride = tl_stride;
        q.h = pc->d_h;
        q.ch2ir = pc->d_ch2ir + c0;
        q.out = y;
        q.out_split_stride = 0;
        q.out_chan_stride = T * B;
        q.out_t_stride = B;
        q.block = B;
        q.partitions = P;
        q.w0 = P - 1;
        q.wrap = 0;
        q.splits = 1;
        q.p_per_split = P;
        if (B >= 32 && T < (int64_t)1 << 30) MA_TRY(launch_mac_tiled(pc, q, nc, T, tl_len));
        else MA_TRY(launch_mac(pc, q, nc, false, T));
    }
    // 4. inverse transform + block overlap-add, truncated at len + taps - 1
    {
        C2RParams p{};
        p.in_a = reinterpret_cast<const float*>(y);
        p.in_signal_stride = T * B;
        p.in_frame_stride = B;
        p.frames_per_signal = T;
        p.n_signals = nc;
        p.layout = LAYOUT_HALF_PACKED;
        p.hop = B;
        p.window = nullptr;
        p.out = out;
        p.out_signal_stride = out_stride;
        p.out_len = full;
        p.floor = -1.0f;
        MA_TRY(launch_istft_small(pc->plan, p));
    }
    // 5. the last P block spectra become the delay line
    {
        const int64_t total = (int64_t)nc * P * B;
        int grid = (int)((total + 255) / 256 < (int64_t)ctx->sm_count * 8 ? (total + 255) / 256 : (int64_t)ctx->sm_count * 8);
        pconv_history_kernel<<<grid, 256, 0, ctx->stream>>>(ring, timeline, tl_stride, P, B, 0, T - 1, 0, nc);
        MA_TRY(after_launch(ctx));
        MA_CUDA(cudaMemsetAsync(pc->d_tail + (int64_t)c0 * B, 0, sizeof(float) * (size_t)nc * B, ctx->stream));
    }
    return MA_OK;
}

extern "C" {

ma_status ma_pconv_process_dev(ma_pconv* pc, const float* in, int64_t len, int64_t in_stride, float* out,
                               int64_t out_stride) {
    if (pc == nullptr) return MA_ERR_INVALID_ARGUMENT;
    ma_context* ctx = pc->ctx;
    MA_TRY(enter(ctx, MA_FAULT_LAUNCH));
    if (pc->d_h == nullptr) return MA_ERR_KERNEL_NOT_CONFIGURED;
    if (len == 0) return MA_OK;  // empty input -> empty output (Convolution.swift:339-342)
    if (len < 0 || in == nullptr || out == nullptr) return MA_ERR_INVALID_ARGUMENT;
    if (pc->write_index < 0 || pc->write_index >= pc->partitions) return MA_ERR_INVALID_PARTITION_STATE;
    int64_t full;
    if (__builtin_add_overflow(len, pc->taps - 1, &full)) return MA_ERR_OUTPUT_OVERFLOW;
    if (len > pc->reserved_len) return MA_ERR_INVALID_ARGUMENT;
    if (pc->channels > 1 && (in_stride < len || out_stride < full)) return MA_ERR_INVALID_ARGUMENT;
    MA_TRY(process_range(pc, 0, pc->channels, in, len, in_stride, out, out_stride, full));
    pc->write_index = 0;
    return MA_OK;
}

// Host form: groups of channels go through the context's three-stage pipeline (copy in, convolve,
// copy out on three streams, two workspace lanes deep) when both host arrays are pinned, so the
// transfers of neighbouring groups run under the convolution of the current one; pageable arrays
// take the same groups one after the other through the staging buffer.
ma_status ma_pconv_process_host(ma_pconv* pc, const float* in, int64_t len, int64_t in_stride, float* out,
                                int64_t out_stride) {
    if (pc == nullptr) return MA_ERR_INVALID_ARGUMENT;
    ma_context* ctx = pc->ctx;
    MA_TRY(enter(ctx, MA_FAULT_LAUNCH));
    if (pc->d_h == nullptr) return MA_ERR_KERNEL_NOT_CONFIGURED;
    if (len == 0) return MA_OK;
    if (len < 0 || in == nullptr || out == nullptr) return MA_ERR_INVALID_ARGUMENT;
    if (pc->write_index < 0 || pc->write_index >= pc->partitions) return MA_ERR_INVALID_PARTITION_STATE;
    int64_t full;
    if (__builtin_add_overflow(len, pc->taps - 1, &full)) return MA_ERR_OUTPUT_OVERFLOW;
    const int C = pc->channels;
    if (C > 1 && (in_stride < len || out_stride < full)) return MA_ERR_INVALID_ARGUMENT;
    MA_TRY(ma_pconv_reserve(pc, len));
    const int group = pc->share;  // channels that must stay together (they share one impulse response)
    const size_t in_row = round256(sizeof(float) * (size_t)len), out_row = round256(sizeof(float) * (size_t)full);
    const bool pinned = is_pinned(in) && is_pinned(out);
    Pipe pp;
    MA_TRY(pipe_open(pp, ctx, pinned, C / group, (in_row + out_row) * (size_t)group, 0));
    const int64_t step = pp.chunk * group;
    int64_t i = 0;
    for (int64_t c0 = 0; c0 < C && pp.st == MA_OK; c0 += step, ++i) {
        const int nc = (int)(C - c0 < step ? C - c0 : step);
        char* lane = pp.lane[i & 1];
        float* d_in = reinterpret_cast<float*>(lane);
        float* d_out = reinterpret_cast<float*>(lane + in_row * (size_t)nc);
        pp.before_copy_in(i);
        pp.in2d(d_in, in_row, in + c0 * in_stride, sizeof(float) * (size_t)in_stride, sizeof(float) * (size_t)len, (size_t)nc);
        pp.before_kernels(i);
        if (pp.st == MA_OK)
            pp.st = process_range(pc, (int)c0, nc, d_in, len, (int64_t)(in_row / sizeof(float)), d_out,
                                  (int64_t)(out_row / sizeof(float)), full);
        pp.before_copy_out(i);
        pp.out2d(out + c0 * out_stride, sizeof(float) * (size_t)out_stride, d_out, out_row, sizeof(float) * (size_t)full, (size_t)nc);
        pp.after_copy_out(i);
    }
    const ma_status st = pp.finish();
    if (st == MA_OK) pc->write_index = 0;
    return st;
}

ma_status ma_pconv_step_dev(ma_pconv* pc, const float* in_block, int64_t in_stride, float* out_block,
                            int64_t out_stride) {
    if (pc == nullptr) return MA_ERR_INVALID_ARGUMENT;
    ma_context* ctx = pc->ctx;
    MA_TRY(enter(ctx, MA_FAULT_LAUNCH));
    if (pc->d_h == nullptr) return MA_ERR_KERNEL_NOT_CONFIGURED;
    if (in_block == nullptr || out_block == nullptr) return MA_ERR_INVALID_ARGUMENT;
    const int B = pc->block, P = pc->partitions, C = pc->channels;
    if (C > 1 && (in_stride < B || out_stride < B)) return MA_ERR_INVALID_ARGUMENT;
    if (pc->write_index < 0 || pc->write_index >= P) return MA_ERR_INVALID_PARTITION_STATE;
    const int w = pc->write_index;
    // The three kernels are chained by programmatic dependent launch: this step's r2c may run
    // beside the previous step's c2r (see fft_small.cu).  That is only sound when the kernel right
    // before this r2c on the stream is that c2r and the two share no data: r2c reads its input
    // before it waits for the earlier kernel.  So r2c is launched plainly when the caller feeds the
    // previous step's output block straight back in, and whenever the library queued anything else
    // on this context since the last step (whose output might be this step's input).
    const float* in_end = in_block + (int64_t)(C - 1) * in_stride + B;
    const bool feeds_back = ctx->step_out != nullptr && in_block < ctx->step_out_end && ctx->step_out < in_end;
    const bool follows_step = ctx->launch_seq == ctx->step_end_seq;
    // 1. this block's spectrum into ring slot w
    {
        R2CParams p{};
        p.dependent_launch = (follows_step && !feeds_back) ? 1 : 0;
        p.in = in_block;
        p.signal_stride = in_stride;
        p.frames_per_signal = 1;
        p.total_frames = C;
        p.signal_len = B;
        p.hop = B;
        p.frame_valid = B;
        p.out_a = reinterpret_cast<float*>(pc->d_ring + (int64_t)w * B);
        p.out_signal_stride = (int64_t)P * B;
        p.out_frame_stride = 0;
        p.layout = LAYOUT_HALF_PACKED;
        p.mag_kind = MAG_NONE;
        MA_TRY(launch_r2c_small(pc->plan, p));
    }
    // 2. stream the whole delay line once: partial sums per partition split
    {
        MacParams q{};
        q.x = pc->d_ring;
        q.x_chan_stride = (int64_t)P * B;
        q.h = pc->d_h;
        q.ch2ir = pc->d_ch2ir;
        q.out = pc->d_partial;
        q.out_split_stride = (int64_t)C * B;
        q.out_chan_stride = B;
        q.out_t_stride = 0;
        q.block = B;
        q.partitions = P;
        q.w0 = w;
        q.wrap = P;
        q.splits = pc->splits;
        q.p_per_split = (P + pc->splits - 1) / pc->splits;
        q.dependent_launch = 1;
        q.cluster = step_cluster(pc->splits);
        MA_TRY(launch_mac(pc, q, pc->channels, true, 1));
    }
    // 3. sum the partials, inverse transform, add the kept tail, keep the new one
    const int partials = pc->splits / step_cluster(pc->splits);  // partial spectra the multiply-accumulate left
    const bool own_sum = partials >= kSumKernelFromSplits && ((int64_t)C * B) % 2 == 0;
    if (own_sum) {
        const int64_t n4 = (int64_t)C * B / 2;
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3((unsigned)((n4 + 255) / 256));
        cfg.blockDim = dim3(256);
        cfg.stream = ctx->stream;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        (void)cudaLaunchKernelEx(&cfg, pconv_sum_partials_kernel, reinterpret_cast<float4*>(pc->d_partial), n4, n4,
                                 partials);  // an error is picked up by after_launch
        MA_TRY(after_launch(ctx));
    }
    {
        C2RParams p{};
        p.in_a = reinterpret_cast<const float*>(pc->d_partial);
        p.in_signal_stride = B;
        p.in_frame_stride = 0;
        p.frames_per_signal = 1;
        p.n_signals = C;
        p.layout = LAYOUT_HALF_PACKED;
        p.n_partials = own_sum ? 1 : partials;
        p.partial_stride = (int64_t)C * B;
        p.out = out_block;
        p.out_signal_stride = out_stride;
        p.tail = pc->d_tail;
        p.dependent_launch = 1;
        MA_TRY(launch_c2r_small(pc->plan, p));
    }
    ctx->step_end_seq = ctx->launch_seq;
    ctx->step_out = out_block;
    ctx->step_out_end = out_block + (int64_t)(C - 1) * out_stride + B;
    pc->write_index = (w + 1) % P;
    return MA_OK;
}

}  // extern "C"
