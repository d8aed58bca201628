// __global__ wrappers and launchers for the in-shared-memory transforms (N <= 8192).
#include "bulk_copy.cuh"
#include "fft_plan.h"
#include "host_tables.h"

namespace ma {

struct DevCta {
    __device__ __forceinline__ int tid() const { return threadIdx.x; }
    __device__ __forceinline__ int bid() const { return blockIdx.x; }
    __device__ __forceinline__ int nblocks() const { return gridDim.x; }
    __device__ __forceinline__ void sync() { __syncthreads(); }
    __device__ __forceinline__ void bulk_init(uint64_t* bar) { bulk_barrier_init(bar); }
    __device__ __forceinline__ void bulk_copy(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
        bulk_copy_g2s(dst, src, bytes, bar);
    }
    __device__ __forceinline__ void bulk_expect(uint64_t* bar, uint32_t total_bytes) { bulk_barrier_expect(bar, total_bytes); }
    __device__ __forceinline__ void bulk_part(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
        bulk_copy_part(dst, src, bytes, bar);
    }
    __device__ __forceinline__ bool bulk_wait(uint64_t* bar, uint32_t parity) { return bulk_barrier_wait(bar, parity); }
};

extern __shared__ float4 ma_dyn_smem[];

// Programmatic dependent launch, used by the convolution's streaming step (r2c -> multiply-
// accumulate -> c2r, every block).  A kernel launched with the programmatic-stream-serialization
// attribute may become resident once every CTA of the kernel before it has executed
// launch_dependents; it must execute wait before it touches (or, for r2c, before it completes
// ahead of) anything the earlier kernel produces.  Without the attribute both are no-ops.
//   c2r: wait, then launch_dependents - the next step's r2c starts while this c2r still runs
//        (they share no data), but never before the multiply-accumulate that reads the delay line
//        slot r2c is about to overwrite has completed;
//   r2c: launch_dependents at once, wait only at the very end - so it completes after the c2r
//        before it, and everything later in the stream stays ordered after that c2r as well.
__device__ __forceinline__ void dependents_launch() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// cudaLaunchKernelEx with the attribute (dependent != 0) or a plain launch.
template <typename K, typename P>
static void launch_maybe_dependent(K kernel, int grid, int threads, size_t smem, cudaStream_t stream, const P& p,
                                   int dependent) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3((unsigned)threads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = dependent ? 1 : 0;
    (void)cudaLaunchKernelEx(&cfg, kernel, p);  // an error is picked up by after_launch
}

template <int M, bool ALIGNED, int LAYOUT, int MAGK>
__global__ void __launch_bounds__(CtaShape<M>::THREADS, 512 / CtaShape<M>::THREADS) r2c_kernel(const R2CParams p) {
    DevCta cta;
    if (p.dependent_launch) dependents_launch();
    r2c_body<M, ALIGNED, LAYOUT, MAGK, DevCta>(p, cta, reinterpret_cast<float2*>(ma_dyn_smem));
    if (p.dependent_launch) dependency_wait();
}

template <int M, int LAYOUT>
__global__ void __launch_bounds__(CtaShape<M>::THREADS, 512 / CtaShape<M>::THREADS) c2r_kernel(const C2RParams p) {
    DevCta cta;
    if (p.dependent_launch) {
        dependency_wait();
        dependents_launch();
    }
    c2r_body<M, LAYOUT, DevCta>(p, cta, reinterpret_cast<float2*>(ma_dyn_smem));
}

template <int M>
__global__ void __launch_bounds__(FftPlan<M>::T, (512 / FftPlan<M>::T) > 16 ? 16 : (512 / FftPlan<M>::T)) istft_kernel(const C2RParams p) {
    DevCta cta;
    istft_body<M, DevCta>(p, cta, reinterpret_cast<float2*>(ma_dyn_smem));
}

template <int M, int LAYOUT, int OVT>
__global__ void __launch_bounds__(FftPlan<M>::T, (512 / FftPlan<M>::T) > 16 ? 16 : (512 / FftPlan<M>::T))
istft_fast_kernel(const C2RParams p) {
    DevCta cta;
    if constexpr (plan_pairable<M>())
        istft_fast_body<M, LAYOUT, OVT, DevCta>(p, cta, reinterpret_cast<float2*>(ma_dyn_smem));
}

// Resident CTAs per SM for a kernel (cached per instantiation and device), after raising
// its dynamic shared-memory limit.
template <class K>
static ma_status occupancy(K kernel, int threads, size_t smem, int* per_sm) {
    MA_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    int n = 0;
    MA_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, kernel, threads, smem));
    *per_sm = n > 0 ? n : 1;
    return MA_OK;
}

template <int M, bool ALIGNED, int LAYOUT, int MAGK>
static ma_status launch_r2c_t(ma_fft_plan* plan, const R2CParams& p) {
    using S = CtaShape<M>;
    static int per_sm[64] = {0};
    ma_context* ctx = plan->ctx;
    int& occ = per_sm[ctx->device & 63];
    constexpr size_t smem = (ALIGNED && LAYOUT >= 0 && plan_pairable<M>()) ? S::SMEM_BYTES_PREFETCH : S::SMEM_BYTES;
    if (occ == 0) MA_TRY(occupancy(r2c_kernel<M, ALIGNED, LAYOUT, MAGK>, S::THREADS, smem, &occ));
    int64_t want = (p.total_frames + S::FPC - 1) / S::FPC;
    int64_t cap = (int64_t)ctx->sm_count * occ;
    int grid = (int)(want < cap ? want : cap);
    if (grid < 1) return MA_OK;
    launch_maybe_dependent(r2c_kernel<M, ALIGNED, LAYOUT, MAGK>, grid, S::THREADS, smem, ctx->stream, p, p.dependent_launch);
    return after_launch(ctx);
}

template <int M>
static ma_status launch_r2c_variant(ma_fft_plan* plan, const R2CParams& p, bool aligned, int magk) {
    if constexpr (plan_pairable<M>()) {
        if (aligned && magk != -2) {
#define MA_R2C_CASE(L_, K_) \
    if (p.layout == L_ && magk == K_) return launch_r2c_t<M, true, L_, K_>(plan, p);
            MA_R2C_CASE(LAYOUT_HALF_INTERLEAVED, 0)
            MA_R2C_CASE(LAYOUT_HALF_INTERLEAVED, -1)
            MA_R2C_CASE(LAYOUT_HALF_PACKED, 0)
            MA_R2C_CASE(LAYOUT_HALF_PACKED, -1)
            MA_R2C_CASE(LAYOUT_FULL_SPLIT, 0)
            MA_R2C_CASE(LAYOUT_FULL_SPLIT, -1)
            MA_R2C_CASE(LAYOUT_HALF_POLAR, -1)
#undef MA_R2C_CASE
        }
    }
    return aligned ? launch_r2c_t<M, true, -1, -2>(plan, p) : launch_r2c_t<M, false, -1, -2>(plan, p);
}

ma_status launch_r2c_small(ma_fft_plan* plan, R2CParams p) {
    p.twM = plan->d_twM;
    p.twN = plan->d_twN;
    if (p.total_frames <= 0) return MA_OK;
    const int n = plan->n;
    const int64_t last_end = (p.frames_per_signal - 1) * (int64_t)p.hop + n;
    const bool aligned = ((uintptr_t)p.in % 8 == 0) && (p.signal_stride % 2 == 0) && (p.hop % 2 == 0) &&
                         p.frame_valid >= n && last_end <= p.signal_len;
    p.bulk_ok = (aligned && (uintptr_t)p.in % 16 == 0 && p.signal_stride % 4 == 0 && p.hop % 4 == 0 && n % 4 == 0) ? 1 : 0;
    p.error_flag = plan->ctx->d_error_flag;
    ma_status st = MA_ERR_UNSUPPORTED;
    // Aligned launches of the paired plans get kernels with the layout and the magnitude kind
    // fixed at compile time (no per-store branches); everything else decides at run time.
    const int magk = p.mag == nullptr ? -1 : (p.mag_kind == MAG_MAGNITUDE ? 0 : -2);
#define RUN(MM) st = launch_r2c_variant<MM>(plan, p, aligned, magk);
    MA_DISPATCH_M(plan->m, RUN)
#undef RUN
    return st;
}

template <int M, int LAYOUT>
static ma_status launch_c2r_t(ma_fft_plan* plan, const C2RParams& p) {
    using S = CtaShape<M>;
    static int per_sm[64] = {0};
    ma_context* ctx = plan->ctx;
    int& occ = per_sm[ctx->device & 63];
    constexpr size_t smem = (plan_pairable<M>() && (LAYOUT == LAYOUT_HALF_INTERLEAVED || LAYOUT == LAYOUT_HALF_PACKED))
                                ? S::SMEM_BYTES_STAGED
                                : S::SMEM_BYTES;
    if (occ == 0) MA_TRY(occupancy(c2r_kernel<M, LAYOUT>, S::THREADS, smem, &occ));
    const int64_t total = p.n_signals * p.frames_per_signal;
    int64_t want = (total + S::FPC - 1) / S::FPC;
    int64_t cap = (int64_t)ctx->sm_count * occ;
    int grid = (int)(want < cap ? want : cap);
    if (grid < 1) return MA_OK;
    launch_maybe_dependent(c2r_kernel<M, LAYOUT>, grid, S::THREADS, smem, ctx->stream, p, p.dependent_launch);
    return after_launch(ctx);
}

template <int M>
static ma_status launch_c2r_variant(ma_fft_plan* plan, const C2RParams& p) {
    if constexpr (plan_pairable<M>()) {
        // plain batched inverse of a paired plan: layout fixed at compile time
        if (p.tail == nullptr && p.n_partials <= 1 && p.mul == nullptr) {
            if (p.layout == LAYOUT_HALF_INTERLEAVED) return launch_c2r_t<M, LAYOUT_HALF_INTERLEAVED>(plan, p);
            if (p.layout == LAYOUT_HALF_PACKED) return launch_c2r_t<M, LAYOUT_HALF_PACKED>(plan, p);
            if (p.layout == LAYOUT_FULL_SPLIT) return launch_c2r_t<M, LAYOUT_FULL_SPLIT>(plan, p);
        }
    }
    return launch_c2r_t<M, -1>(plan, p);
}

ma_status launch_c2r_small(ma_fft_plan* plan, C2RParams p) {
    p.twM = plan->d_twInv;
    p.twN = plan->d_twN;
    p.error_flag = plan->ctx->d_error_flag;
    if (p.n_signals * p.frames_per_signal <= 0) return MA_OK;
    ma_status st = MA_ERR_UNSUPPORTED;
#define RUN(MM) st = launch_c2r_variant<MM>(plan, p);
    MA_DISPATCH_M(plan->m, RUN)
#undef RUN
    return st;
}

template <int M>
static ma_status launch_istft_t(ma_fft_plan* plan, C2RParams& p) {
    constexpr int T = FftPlan<M>::T;
    const bool fast = istft_fast_ok<M>(p);
    const int ov = fast ? (2 * M) / p.hop : 0;
    // 0: general kernel; 1: fast, overlap count read at run time; 2: fast with the overlap count 4
    // fixed at compile time (register ring)
    const int kind = !fast ? 0 : (ov == 4 ? 2 : 1);
    const size_t smem = kind == 2 ? (size_t)IstftFastShape<M, 4>::SMEM_BYTES
                      : kind == 1 ? (size_t)IstftFastShape<M, 0>::SMEM_BYTES
                                  : 2 * smem_elems_per_fft<M, 1>() * sizeof(float2) + 2 * M * sizeof(float);
    static int per_sm[3][64] = {{0}, {0}, {0}};
    ma_context* ctx = plan->ctx;
    int& occ = per_sm[kind][ctx->device & 63];
    const int variant = !fast ? 0
                              : (p.layout == LAYOUT_HALF_INTERLEAVED ? 1 : (p.layout == LAYOUT_HALF_PACKED ? 3 : 5)) +
                                    (ov == 4 ? 1 : 0);
    if (occ == 0) {  // the layout variants of a kind share its footprint; raise every one's shared-memory limit
        int dummy;
        if (kind == 2) {
            MA_TRY(occupancy(istft_fast_kernel<M, LAYOUT_HALF_INTERLEAVED, 4>, T, smem, &occ));
            MA_TRY(occupancy(istft_fast_kernel<M, LAYOUT_HALF_PACKED, 4>, T, smem, &dummy));
            MA_TRY(occupancy(istft_fast_kernel<M, LAYOUT_HALF_POLAR, 4>, T, smem, &dummy));
        } else if (kind == 1) {
            MA_TRY(occupancy(istft_fast_kernel<M, LAYOUT_HALF_INTERLEAVED, 0>, T, smem, &occ));
            MA_TRY(occupancy(istft_fast_kernel<M, LAYOUT_HALF_PACKED, 0>, T, smem, &dummy));
            MA_TRY(occupancy(istft_fast_kernel<M, LAYOUT_HALF_POLAR, 0>, T, smem, &dummy));
        } else {
            MA_TRY(occupancy(istft_kernel<M>, T, smem, &occ));
        }
    }
    // Chunks per signal: enough CTAs to fill the device a few times over, but chunks long
    // enough that the recomputed lead-in frames stay a small fraction.
    const int64_t F = p.frames_per_signal;
    const int reach = (2 * M + p.hop - 1) / p.hop - 1;
    const int64_t cap = (int64_t)ctx->sm_count * occ;
    int64_t chunks = (2 * cap + p.n_signals - 1) / p.n_signals;
    const int64_t min_len = reach > 0 ? 16 * (int64_t)reach : 1;
    if (chunks > F / min_len) chunks = F / min_len;
    if (chunks < 1) chunks = 1;
    p.chunks_per_signal = (int32_t)chunks;
    int64_t total = chunks * p.n_signals;
    if (fast) {  // contiguous ranges of the global frame list, at least min_len frames each
        total = (F * p.n_signals) / min_len;
        if (total < 1) total = 1;
    }
    int grid = (int)(total < cap ? total : cap);
    if (grid < 1) return MA_OK;
    switch (variant) {
        case 1: istft_fast_kernel<M, LAYOUT_HALF_INTERLEAVED, 0><<<grid, T, smem, ctx->stream>>>(p); break;
        case 2: istft_fast_kernel<M, LAYOUT_HALF_INTERLEAVED, 4><<<grid, T, smem, ctx->stream>>>(p); break;
        case 3: istft_fast_kernel<M, LAYOUT_HALF_PACKED, 0><<<grid, T, smem, ctx->stream>>>(p); break;
        case 4: istft_fast_kernel<M, LAYOUT_HALF_PACKED, 4><<<grid, T, smem, ctx->stream>>>(p); break;
        case 5: istft_fast_kernel<M, LAYOUT_HALF_POLAR, 0><<<grid, T, smem, ctx->stream>>>(p); break;
        case 6: istft_fast_kernel<M, LAYOUT_HALF_POLAR, 4><<<grid, T, smem, ctx->stream>>>(p); break;
        default: istft_kernel<M><<<grid, T, smem, ctx->stream>>>(p); break;
    }
    return after_launch(ctx);
}

// Rebuilds the interior normaliser table (host_tables.h) when the floor changes.
static ma_status update_norm_table(ma_fft_plan* plan, int hop, float floor) {
    if (plan->norm_floor == floor) return MA_OK;
    std::vector<float> tab =
        make_norm_table(plan->h_window.empty() ? nullptr : plan->h_window.data(), plan->n, hop, floor);
    tab.resize(2 * (size_t)hop);
    for (int r = 0; r < hop; ++r) tab[(size_t)(hop + r)] = 1.0f / tab[(size_t)r];
    MA_CUDA(cudaMemcpyAsync(plan->d_norm, tab.data(), 2 * sizeof(float) * (size_t)hop, cudaMemcpyHostToDevice,
                            plan->ctx->stream));
    MA_CUDA(cudaStreamSynchronize(plan->ctx->stream));
    plan->norm_floor = floor;
    return MA_OK;
}

ma_status launch_istft_small(ma_fft_plan* plan, C2RParams p) {
    p.twM = plan->d_twInv;
    p.twN = plan->d_twN;
    if (p.n_signals <= 0 || p.frames_per_signal <= 0) return MA_OK;
    if (!(p.window == nullptr && p.floor < 0.f)) {
        if (p.hop != plan->hop) return MA_ERR_INVALID_ARGUMENT;
        MA_TRY(update_norm_table(plan, p.hop, p.floor));
    }
    p.norm_mid = plan->d_norm;
    p.norm_mid_inv = plan->d_norm + plan->hop;
    p.window_syn = p.window != nullptr ? reinterpret_cast<const float4*>(plan->d_window_syn) : nullptr;
    p.error_flag = plan->ctx->d_error_flag;
    ma_status st = MA_ERR_UNSUPPORTED;
#define RUN(MM) st = launch_istft_t<MM>(plan, p);
    MA_DISPATCH_M(plan->m, RUN)
#undef RUN
    return st;
}

// Magnitude family over bins 0..N/2 of full-N split spectra.
__global__ void magnitude_kernel(const float* __restrict__ re, const float* __restrict__ im,
                                 float* __restrict__ out, int64_t batch, int n, int kind, float db_scale) {
    const int kh = n / 2 + 1;
    const int64_t total = batch * kh;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t g = i / kh;
        const int k = (int)(i - g * kh);
        const float2 x = make_float2(__ldg(re + g * n + k), __ldg(im + g * n + k));
        out[i] = mag_value(x, kind, db_scale);
    }
}

ma_status launch_magnitude(ma_fft_plan* plan, const float* re, const float* im, float* out, int64_t batch,
                           int kind, float db_scale) {
    ma_context* ctx = plan->ctx;
    const int64_t total = batch * (plan->n / 2 + 1);
    if (total <= 0) return MA_OK;
    int64_t want = (total + 255) / 256;
    int64_t cap = (int64_t)ctx->sm_count * 8;
    int grid = (int)(want < cap ? want : cap);
    magnitude_kernel<<<grid, 256, 0, ctx->stream>>>(re, im, out, batch, plan->n, kind, db_scale);
    return after_launch(ctx);
}

}  // namespace ma
