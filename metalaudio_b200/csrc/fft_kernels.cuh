// Kernel bodies for real-input transforms that fit in shared memory (N <= 8192):
//   r2c_body   - forward: frame gather (STFT) + analysis window + packed-real complex FFT
//                + Hermitian post-process + optional magnitude, one HBM read and one HBM
//                write per frame.
//   c2r_body   - inverse: Hermitian pre-process + complex FFT + 1/N scale, optional
//                synthesis window, overlap-add and window-sum normalisation (iSTFT).
// The bodies are templated on a Cta type (barrier + ids) so the CPU emulator in the
// test-suite can execute exactly this index arithmetic.
#pragma once
#include "fft_core.cuh"

namespace ma {

enum : int { LAYOUT_HALF_INTERLEAVED = 0, LAYOUT_FULL_SPLIT = 1, LAYOUT_HALF_PACKED = 2, LAYOUT_HALF_POLAR = 3 };
enum : int { MAG_NONE = -1, MAG_MAGNITUDE = 0, MAG_POWER = 1, MAG_DB = 2 };

struct R2CParams {
    const float* in;            // signals
    int64_t signal_stride;      // floats between signals
    int64_t frames_per_signal;  // F
    int64_t total_frames;       // n_signals * F
    int64_t signal_len;         // samples at/after this index of a signal read as zero
    int32_t hop;                // frame f starts at f*hop
    int32_t frame_valid;        // samples at/after this index of a frame read as zero
    const float* window;        // N coefficients or nullptr
    float* out_a;               // half layouts: interleaved bins; FULL_SPLIT: real
    float* out_b;               // FULL_SPLIT: imag
    float* mag;                 // optional (N/2+1 per frame)
    int64_t out_signal_stride;  // float2 units, half layouts
    int64_t out_frame_stride;   // float2 units, half layouts
    int32_t layout;
    int32_t mag_kind;
    float db_scale;             // 1/reference for MAG_DB
    const float2* twM;          // stage twiddle tables of FftPlan<M> (fft_core.cuh layout)
    int32_t bulk_ok;            // frame starts and length are 16-byte multiples: bulk async staging allowed
    int32_t* error_flag;        // set to 1 when a bounded wait ran out
    int32_t dependent_launch;   // launched with programmatic stream serialization (see fft_small.cu)
    const float2* twN;          // Hermitian-step twiddles exp(-2 pi i k / N): [k], k <= M/2, or for
                                // plan_pairable<M>() the table [k][j] = W_N^(j + k*NL), j <= NL/2
};

MA_HD float mag_value(float2 x, int kind, float db_scale) {
    float p = x.x * x.x + x.y * x.y;
    if (kind == MAG_POWER) return p;
    float m = sqrtf(p);
    if (kind == MAG_MAGNITUDE) return m;
    return 20.0f * log10f(m * db_scale);
}

// Threads per CTA and frames per CTA for the contiguous-frame kernels.
template <int M>
struct CtaShape {
    static constexpr int T = FftPlan<M>::T;
    static constexpr int THREADS = T >= 128 ? T : 128;
    static constexpr int FPC = THREADS / T;
    static constexpr int ELEMS = smem_elems_per_fft<M, 1>();      // one buffer, one frame
    static constexpr int BUF_STRIDE = ELEMS * FPC;                // float2 between buffers
    static constexpr int SMEM_BYTES = 2 * BUF_STRIDE * (int)sizeof(float2);
    // Prefetching forward kernels add a staging frame per slot plus one mbarrier per slot.
    static constexpr int STAGE = FftPlan<M>::R * THREADS;
    static constexpr int SMEM_BYTES_PREFETCH = SMEM_BYTES + STAGE * (int)sizeof(float2) + 16 * FPC;
    // Staged inverse kernels: one spectrum row (M+2 bins with the alignment slack) per slot.
    static constexpr int ROW = M + 2;
    static constexpr int TW1_INV = stage1_table_elems<FftPlanRev<M>>();
    static constexpr int SMEM_BYTES_STAGED = SMEM_BYTES + FPC * ROW * (int)sizeof(float2) + 16 * FPC + TW1_INV * (int)sizeof(float2);
    static_assert(SMEM_BYTES % 16 == 0 && (ROW * sizeof(float2)) % 16 == 0 && (M * sizeof(float2)) % 16 == 0 || M < 2,
                  "bulk copy destinations must be 16-byte aligned");
};

// Hermitian post-process of one pair: a = Z[k], b = Z[(M-k) mod M], w = exp(-2 pi i k/N).
// xk = X[k], xm = X[M-k].
MA_HD void herm_post(float2 a, float2 b, float2 w, float2& xk, float2& xm) {
    float2 xe = make_float2(0.5f * (a.x + b.x), 0.5f * (a.y - b.y));
    float2 xo = make_float2(0.5f * (a.y + b.y), -0.5f * (a.x - b.x));
    float2 t = cmul(w, xo);
    xk = make_float2(xe.x + t.x, xe.y + t.y);
    xm = make_float2(xe.x - t.x, -(xe.y - t.y));
}

// Inverse of herm_post without the 1/2 (folded into the final 1/N):
// a = X[k], b = X[M-k]  ->  zk = 2 Z[k], zm = 2 Z[M-k].
MA_HD void herm_pre(float2 a, float2 b, float2 w, float2& zk, float2& zm) {
    float2 xe = make_float2(a.x + b.x, a.y - b.y);   // A + conj(B)
    float2 d = make_float2(a.x - b.x, a.y + b.y);    // A - conj(B) = W * Xo
    float2 xo = cmul(cconj(w), d);
    // Z[k] = Xe + i Xo ; Z[M-k] = conj(Xe - i Xo)
    zk = make_float2(xe.x - xo.y, xe.y + xo.x);
    zm = make_float2(xe.x + xo.y, -(xe.y - xo.x));
}

// exp(-2 pi i k / R2) for R2 in {4, 8, 16} and 0 <= k < R2/2; folds to immediates once the
// caller's loop over k is unrolled.
template <int R2>
MA_HD float2 root_const(int k) {
    constexpr float kS = 0.70710678118654752440f, kC1 = 0.92387953251128675613f, kS1 = 0.38268343236508977173f;
    switch (k * (16 / R2)) {
        case 0: return make_float2(1.f, 0.f);
        case 1: return make_float2(kC1, -kS1);
        case 2: return make_float2(kS, -kS);
        case 3: return make_float2(kS1, -kC1);
        case 4: return make_float2(0.f, -1.f);
        case 5: return make_float2(-kS1, -kC1);
        case 6: return make_float2(-kS, -kS);
        default: return make_float2(-kC1, -kS1);
    }
}

// Stores X[k] = xk and X[M-k] = xm of frame g in the requested layout (plus magnitudes).
// LAYOUT >= 0 fixes the layout at compile time (-1: read p.layout); MAGK >= 0 fixes the
// magnitude kind, -1 means no magnitude output, -2 reads p.mag / p.mag_kind.
template <int M, int LAYOUT, int MAGK>
MA_HD void r2c_store_pair(const R2CParams& p, int64_t g, int64_t half_off, int k, float2 xk, float2 xm) {
    constexpr int N = 2 * M;
    (void)N;
    const int layout = LAYOUT >= 0 ? LAYOUT : p.layout;
    const int km = M - k;
    if (layout == LAYOUT_HALF_INTERLEAVED) {
        float2* o = reinterpret_cast<float2*>(p.out_a) + half_off;
        o[k] = xk;
        o[km] = xm;
    } else if (layout == LAYOUT_HALF_PACKED) {
        float2* o = reinterpret_cast<float2*>(p.out_a) + half_off;
        if (k == 0) {
            o[0] = make_float2(xk.x, xm.x);
        } else {
            o[k] = xk;
            o[km] = xm;
        }
    } else if (layout == LAYOUT_HALF_POLAR) {
        float* mg = p.out_a + g * (int64_t)(M + 1);
        float* ph = p.out_b + g * (int64_t)(M + 1);
        mg[k] = sqrtf(xk.x * xk.x + xk.y * xk.y);
        ph[k] = fast_atan2(xk.y, xk.x);
        mg[km] = sqrtf(xm.x * xm.x + xm.y * xm.y);
        ph[km] = fast_atan2(xm.y, xm.x);
    } else {
        float* re = p.out_a + g * (int64_t)N;
        float* im = p.out_b + g * (int64_t)N;
        re[k] = xk.x;
        im[k] = xk.y;
        re[km] = xm.x;
        im[km] = xm.y;
        if (k > 0) {  // conjugate mirror, bins M+1 .. N-1
            re[N - k] = xk.x;
            im[N - k] = -xk.y;
            if (km < M) {
                re[N - km] = xm.x;
                im[N - km] = -xm.y;
            }
        }
    }
    if (MAGK == -1) return;
    if (MAGK >= 0 || p.mag != nullptr) {
        const int kind = MAGK >= 0 ? MAGK : p.mag_kind;
        float* mg = p.mag + g * (int64_t)(M + 1);
        mg[k] = mag_value(xk, kind, p.db_scale);
        mg[km] = mag_value(xm, kind, p.db_scale);
    }
}

// ALIGNED: every frame start is 8-byte aligned and no zero padding is requested, so
// sample pairs are fetched with one float2 load.  Otherwise scalar guarded loads.
template <int M, bool ALIGNED, int LAYOUT, int MAGK, class Cta>
MA_HD void r2c_body(const R2CParams& p, Cta& cta, float2* smem) {
    using P = FftPlan<M>;
    using S = CtaShape<M>;
    constexpr int R = P::R, T = P::T, N = 2 * M;
    const int tid = cta.tid();
    const int slot = tid / T;
    const int t = tid % T;
    float2* sbuf0 = smem + slot * S::ELEMS;
    int parity = 0;

    float2 wreg[R];
    if (p.window != nullptr) {
#pragma unroll
        for (int q = 0; q < R; ++q) {
            const int n = t + q * T;
            wreg[q] = make_float2(MA_LDG(p.window + 2 * n), MA_LDG(p.window + 2 * n + 1));
        }
    } else {
#pragma unroll
        for (int q = 0; q < R; ++q) wreg[q] = make_float2(1.0f, 1.0f);
    }

    // Kernels with the layout fixed at compile time keep their twiddles in registers and have the
    // whole next frame staged by one bulk asynchronous copy (TMA unit).  (Per-thread 8-byte
    // asynchronous copies were tried instead: they cost more load/store-pipe wavefronts than they hide.)
    constexpr bool TWALU = ALIGNED && LAYOUT >= 0 && plan_pairable<M>();
    constexpr bool BULK = TWALU;
    float2 twb[tw_base_count<P>()];
    float2 wherm[R / 2 + 1];
    (void)wherm;
    if constexpr (TWALU) {
        load_tw_bases<P, true>(twb, t, p.twM);
        constexpr int rl_ = P::radix(P::NS - 1), NL_ = M / rl_;
#pragma unroll
        for (int c = 0; c < R / rl_ / 2; ++c) wherm[c] = MA_LDG(p.twN + (c * T + t));
        (void)NL_;
    }
    float2* stage = smem + 2 * S::BUF_STRIDE;
    (void)stage;
    // (signal, frame) of this thread's first frame by one division; later frames advance by the
    // grid stride without dividing.
    const int64_t stride_frames = (int64_t)cta.nblocks() * S::FPC;
    int64_t g = (int64_t)cta.bid() * S::FPC + slot;
    int64_t s = g / p.frames_per_signal;
    int64_t f = g - s * p.frames_per_signal;
    const int64_t ds = stride_frames / p.frames_per_signal;
    const int64_t df = stride_frames - ds * p.frames_per_signal;
    // Bulk staging: slot-private frame buffer and mbarrier; thread 0 of the slot issues copies.
    float2* stage_slot = stage + slot * M;
    uint64_t* bar = reinterpret_cast<uint64_t*>(stage + S::STAGE) + 2 * slot;
    const bool bulk = BULK && p.bulk_ok != 0;
    uint32_t phase = 0;
    if (bulk) {
        if (t == 0) cta.bulk_init(bar);
        cta.sync();
        if (t == 0 && g < p.total_frames)
            cta.bulk_copy(stage_slot, p.in + s * p.signal_stride + f * (int64_t)p.hop, N * (uint32_t)sizeof(float), bar);
    }
    for (int64_t base = (int64_t)cta.bid() * S::FPC; base < p.total_frames;
         base += stride_frames, g += stride_frames, s += ds, f += df) {
        if (f >= p.frames_per_signal) {
            f -= p.frames_per_signal;
            ++s;
        }
        const bool active = S::FPC == 1 ? true : g < p.total_frames;
        const int64_t start = f * (int64_t)p.hop;
        const float* src = p.in + (active ? s * p.signal_stride + start : 0);

        float2 v[R];
        if (bulk) {
            if (active) {
                if (!cta.bulk_wait(bar, phase) && p.error_flag != nullptr) *p.error_flag = 1;
                phase ^= 1;
            }
#pragma unroll
            for (int q = 0; q < R; ++q) {
                const float2 x = active ? stage_slot[t + q * T] : make_float2(0.f, 0.f);
                v[q] = make_float2(x.x * wreg[q].x, x.y * wreg[q].y);
            }
        } else if (ALIGNED) {
#pragma unroll
            for (int q = 0; q < R; ++q) {
                const int n = t + q * T;
                float2 x = make_float2(0.f, 0.f);
                if (active) x = MA_LDG(reinterpret_cast<const float2*>(src) + n);
                v[q] = make_float2(x.x * wreg[q].x, x.y * wreg[q].y);
            }
        } else {
#pragma unroll
            for (int q = 0; q < R; ++q) {
                const int i0 = 2 * (t + q * T);
                float x0 = 0.f, x1 = 0.f;
                if (active && i0 < p.frame_valid && start + i0 < p.signal_len) x0 = MA_LDG(src + i0);
                if (active && i0 + 1 < p.frame_valid && start + i0 + 1 < p.signal_len)
                    x1 = MA_LDG(src + i0 + 1);
                v[q] = make_float2(x0 * wreg[q].x, x1 * wreg[q].y);
            }
        }

        const int64_t half_off = s * p.out_signal_stride + f * p.out_frame_stride;
        if constexpr (plan_pairable<M>()) {
            // Last stage with paired butterflies: bins k and M-k end up in the same thread,
            // so the Hermitian post-process needs no exchange.
            auto issue_next = [&]() {
                if (bulk && t == 0 && g + stride_frames < p.total_frames) {
                    int64_t fn = f + df, sn = s + ds;
                    if (fn >= p.frames_per_signal) {
                        fn -= p.frames_per_signal;
                        ++sn;
                    }
                    cta.bulk_copy(stage_slot, p.in + sn * p.signal_stride + fn * (int64_t)p.hop,
                                  N * (uint32_t)sizeof(float), bar);
                }
            };
            fft_run<P, 1, false, true, Cta, TWALU>(v, t, sbuf0, S::BUF_STRIDE, parity, p.twM, cta, twb, issue_next);
            constexpr int rl = P::radix(P::NS - 1), NBL = R / rl, NL = M / rl;
#pragma unroll
            for (int c = 0; c < NBL / 2; ++c) {
                const float2* A = v + (2 * c) * rl;
                const float2* Bf = v + (2 * c + 1) * rl;
                const int j = c * T + t;
                if (j != 0) {
#pragma unroll
                    for (int k = 0; k < rl; ++k) {
                        float2 xk, xm;
                        const float2 wk = TWALU ? cmul(wherm[c], root_const<2 * rl>(k))
                                                : MA_LDG(p.twN + k * (NL / 2 + 1) + j);
                        herm_post(A[k], Bf[rl - 1 - k], wk, xk, xm);
                        if (active) r2c_store_pair<M, LAYOUT, MAGK>(p, g, half_off, j + k * NL, xk, xm);
                    }
                } else {
                    // butterfly 0 pairs with itself (bins k*NL and M - k*NL) ...
#pragma unroll
                    for (int k = 0; k <= rl / 2; ++k) {
                        float2 xk, xm;
                        herm_post(A[k], A[(rl - k) % rl], root_const<2 * rl>(k), xk, xm);
                        if (active) r2c_store_pair<M, LAYOUT, MAGK>(p, g, half_off, k * NL, xk, xm);
                    }
                    // ... and so does butterfly NL/2 (bins NL/2 + k*NL).
#pragma unroll
                    for (int k = 0; k < rl / 2; ++k) {
                        float2 xk, xm;
                        herm_post(Bf[k], Bf[rl - 1 - k], MA_LDG(p.twN + k * (NL / 2 + 1) + NL / 2), xk, xm);
                        if (active) r2c_store_pair<M, LAYOUT, MAGK>(p, g, half_off, NL / 2 + k * NL, xk, xm);
                    }
                }
            }
        } else {
            fft_forward_regs<M, 1, Cta>(v, t, sbuf0, S::BUF_STRIDE, parity, p.twM, cta);
            // exchange for the Hermitian post-process
            float2* sb = sbuf0 + parity * S::BUF_STRIDE;
            parity ^= 1;
#pragma unroll
            for (int q = 0; q < R; ++q) sb[saddr<1>(t + q * T)] = v[q];
            cta.sync();
#pragma unroll
            for (int q = 0; q <= R / 2; ++q) {
                const int k = t + q * T;
                if (k > M / 2 || !active) continue;
                const float2 a = sb[saddr<1>(k)];
                const float2 b = sb[saddr<1>((M - k) & (M - 1))];
                float2 xk, xm;
                herm_post(a, b, MA_LDG(p.twN + k), xk, xm);
                r2c_store_pair<M, LAYOUT, MAGK>(p, g, half_off, k, xk, xm);
            }
        }
    }
}

struct C2RParams {
    const float* in_a;          // half layouts: interleaved bins; FULL_SPLIT: real
    const float* in_b;          // FULL_SPLIT: imag
    int64_t in_signal_stride;   // float2 units, half layouts
    int64_t in_frame_stride;    // float2 units, half layouts
    int64_t frames_per_signal;  // F
    int64_t n_signals;
    int32_t layout;
    int32_t hop;
    const float* window;        // synthesis window (iSTFT) or nullptr
    float* out;
    int64_t out_signal_stride;  // floats
    int64_t out_len;            // iSTFT: (F-1)*hop + N ; plain inverse: unused
    float floor;                // iSTFT window-sum floor
    int32_t chunks_per_signal;  // iSTFT: CTAs per signal
    int32_t n_partials;         // HALF_PACKED input: number of partial spectra to sum (>= 1)
    int64_t partial_stride;     // float2 units between partial spectra
    float* tail;                // streaming convolution step: per-signal overlap tail (N/2 floats)
    const float* norm_mid;      // iSTFT: clamped window sums of the interior, indexed by position mod hop
    const float* norm_mid_inv;  // iSTFT: their reciprocals
    int32_t* error_flag;        // set to 1 when a bounded wait ran out
    int32_t dependent_launch;   // launched with programmatic stream serialization (see fft_small.cu)
    const float4* window_syn;   // register-ring iSTFT: synthesis window in thread order with 1/N folded in
                                // (host_tables.h make_synthesis_table), or nullptr for no window
    const float2* mul;          // HALF_INTERLEAVED input only: every bin is multiplied by mul[k] on load (N/2+1 values), or nullptr
    const float2* twM;          // stage tables: FftPlanRev<M> when plan_pairable<M>(), else FftPlan<M>
    const float2* twN;
};

// Loads the pair (X[k], X[M-k]) of frame g for the inverse pre-process.  LAYOUT >= 0 fixes the
// layout at compile time (-1: read p.layout).  x is the frame's first bin for the half layouts.
template <int LAYOUT, bool STAGED = false>
MA_HD void c2r_load_pair(const C2RParams& p, const float2* x, int64_t g, int k, int M,
                         float2& a, float2& b, const float2* xg = nullptr) {
    const int layout = LAYOUT >= 0 ? LAYOUT : p.layout;
    const int km = M - k;
    if (layout == LAYOUT_FULL_SPLIT) {
        const int N = 2 * M;
        const float* re = p.in_a + g * (int64_t)N;
        const float* im = p.in_b + g * (int64_t)N;
        // Real part of the inverse of an arbitrary spectrum equals the inverse of its
        // Hermitian part: symmetrise with the mirror bins.
        if (k == 0) {
            a = make_float2(MA_LDG(re), 0.f);
            b = make_float2(MA_LDG(re + M), 0.f);
        } else {
            float2 xa = make_float2(MA_LDG(re + k), MA_LDG(im + k));
            float2 xan = make_float2(MA_LDG(re + N - k), MA_LDG(im + N - k));
            float2 xb = make_float2(MA_LDG(re + km), MA_LDG(im + km));
            float2 xbn = make_float2(MA_LDG(re + N - km), MA_LDG(im + N - km));
            a = make_float2(0.5f * (xa.x + xan.x), 0.5f * (xa.y - xan.y));
            b = make_float2(0.5f * (xb.x + xbn.x), 0.5f * (xb.y - xbn.y));
        }
    } else if (layout == LAYOUT_HALF_PACKED) {
        // Optionally the spectrum is the sum of n_partials partial spectra (the
        // partition-split accumulators of the convolution step).
        float2 xa = STAGED ? x[k] : MA_LDG(x + k);
        float2 xb = STAGED ? x[k == 0 ? 0 : km] : MA_LDG(x + (k == 0 ? 0 : km));
        if (LAYOUT < 0) {
            for (int i = 1; i < p.n_partials; ++i) {
                const float2* xi = x + (int64_t)i * p.partial_stride;
                const float2 ya = MA_LDG(xi + k);
                const float2 yb = MA_LDG(xi + (k == 0 ? 0 : km));
                xa.x += ya.x; xa.y += ya.y;
                xb.x += yb.x; xb.y += yb.y;
            }
        }
        if (k == 0) {
            a = make_float2(xa.x, 0.f);
            b = make_float2(xa.y, 0.f);
        } else {
            a = xa;
            b = xb;
        }
    } else if (layout == LAYOUT_HALF_POLAR) {
        const float* mg = p.in_a + g * (int64_t)(M + 1);
        const float* ph = p.in_b + g * (int64_t)(M + 1);
        float ma, pa, mb, pb;
        if (STAGED) {
            // x: M staged magnitudes followed by M staged phases, each copied from the 16-byte
            // boundary at or below its row (rows of M+1 floats start 4*(g mod 4) bytes past one),
            // so bin i sits at [i + shift] and the last shift bins plus bin M come from HBM.
            const float* sm = reinterpret_cast<const float*>(x);
            const int shift = (int)(g & 3), lim = M - shift;
            ma = k < lim ? sm[k + shift] : MA_LDG(mg + k);
            pa = k < lim ? sm[M + k + shift] : MA_LDG(ph + k);
            mb = km < lim ? sm[km + shift] : MA_LDG(mg + km);
            pb = km < lim ? sm[M + km + shift] : MA_LDG(ph + km);
        } else {
            ma = MA_LDG(mg + k);
            pa = MA_LDG(ph + k);
            mb = MA_LDG(mg + km);
            pb = MA_LDG(ph + km);
        }
        float sa, ca, sb, cb;
        fast_sincos(pa, &sa, &ca);
        fast_sincos(pb, &sb, &cb);
        a = make_float2(ma * ca, k == 0 ? 0.f : ma * sa);
        b = make_float2(mb * cb, k == 0 ? 0.f : mb * sb);
    } else {
        a = STAGED ? x[k] : MA_LDG(x + k);
        if (STAGED && k == 0) b = MA_LDG(xg + M);  // bin M is not staged
        else b = STAGED ? x[km] : MA_LDG(x + km);
        if (LAYOUT < 0 && p.mul != nullptr) {  // frequency-domain product fused into the inverse (FFT convolution)
            a = cmul(a, MA_LDG(p.mul + k));
            b = cmul(b, MA_LDG(p.mul + km));
        }
        if (k == 0) {
            a.y = 0.f;
            b.y = 0.f;
        }
    }
}

// A spectrum row (half layouts) prepared for a bulk copy of 16-byte granularity.  Only bins
// 0..M-1 are staged (the thread that needs bin M reads it from HBM itself), so the copy is
// M bins when the row starts on a 16-byte boundary and M+2 bins, beginning one bin early
// (shift = 1), when it starts on an odd 8-byte boundary; either way it stays inside the row's
// own neighbourhood and never runs past the end of the array.
struct StagedRow {
    const float2* row;   // first bin of the row (global)
    const float2* src;   // 16-byte aligned start of the copy
    uint32_t bytes;      // multiple of 16
    int shift;           // bins between src and row (0 or 1)
};

template <int M>
MA_HD StagedRow staged_row(const C2RParams& p, int64_t s, int64_t f) {
    StagedRow r;
    r.row = reinterpret_cast<const float2*>(p.in_a) + s * p.in_signal_stride + f * p.in_frame_stride;
    r.shift = (int)((reinterpret_cast<uintptr_t>(r.row) >> 3) & 1);
    r.src = r.row - r.shift;
    r.bytes = (uint32_t)(M + 2 * r.shift) * (uint32_t)sizeof(float2);
    return r;
}

// Pre-process + FFT of one frame: leaves v[q] = (x[2n+1], x[2n]) * N for n = t + q*T
// (real and imaginary parts swapped: the inverse transform is run as a forward transform
// of the swapped spectrum).
template <int M, int LAYOUT, bool TWALU, class Cta, bool STAGED = false, class Hook = NoHook, bool SINGLE = false,
          bool TWS1 = false>
MA_HD void c2r_frame(const C2RParams& p, bool active, int64_t s, int64_t f, int64_t g, int t,
                     float2* sbuf0, int buf_stride, int& parity, float2* v, Cta& cta,
                     const float2* twb = nullptr, const float2* wherm = nullptr,
                     const float2* staged = nullptr, const Hook& hook = Hook(), const float2* xg = nullptr,
                     const float2* tw_s1 = nullptr) {
    using P = FftPlan<M>;
    constexpr int R = P::R, T = P::T;
    const float2* x = STAGED ? staged
                             : reinterpret_cast<const float2*>(p.in_a) +
                                   (active ? s * p.in_signal_stride + f * p.in_frame_stride : 0);
    if constexpr (plan_pairable<M>()) {
        // First stage with paired butterflies (reversed radix order): the thread that loads
        // X[i] and X[M-i] also consumes both Z[i] and Z[M-i]; no exchange for the pre-process.
        using PR = FftPlanRev<M>;
        constexpr int r0 = PR::radix(0), NB0 = R / r0, N0 = M / r0;
        const float2 zero = make_float2(0.f, 0.f);
#pragma unroll
        for (int c = 0; c < NB0 / 2; ++c) {
            float2* A = v + (2 * c) * r0;
            float2* Bf = v + (2 * c + 1) * r0;
            const int j = c * T + t;
            if (j != 0) {
                // all loads first, then the arithmetic: one memory round trip per frame
                float2 a[r0], b[r0];
#pragma unroll
                for (int k = 0; k < r0; ++k) {
                    a[k] = zero;
                    b[k] = zero;
                    if (active) c2r_load_pair<LAYOUT, STAGED>(p, x, g, j + k * N0, M, a[k], b[k], xg);
                }
#pragma unroll
                for (int k = 0; k < r0; ++k) {
                    float2 zk, zm;
                    const float2 wk = TWALU ? cmul(wherm[c], root_const<2 * r0>(k))
                                            : MA_LDG(p.twN + k * (N0 / 2 + 1) + j);
                    herm_pre(a[k], b[k], wk, zk, zm);
                    A[k] = make_float2(zk.y, zk.x);
                    Bf[r0 - 1 - k] = make_float2(zm.y, zm.x);
                }
            } else {
#pragma unroll
                for (int k = 0; k <= r0 / 2; ++k) {
                    float2 a = zero, b = zero, zk, zm;
                    if (active) c2r_load_pair<LAYOUT, STAGED>(p, x, g, k * N0, M, a, b, xg);
                    herm_pre(a, b, root_const<2 * r0>(k), zk, zm);
                    A[k] = make_float2(zk.y, zk.x);
                    if (k > 0) A[r0 - k] = make_float2(zm.y, zm.x);
                }
#pragma unroll
                for (int k = 0; k < r0 / 2; ++k) {
                    float2 a = zero, b = zero, zk, zm;
                    if (active) c2r_load_pair<LAYOUT, STAGED>(p, x, g, N0 / 2 + k * N0, M, a, b, xg);
                    herm_pre(a, b, MA_LDG(p.twN + k * (N0 / 2 + 1) + N0 / 2), zk, zm);
                    Bf[k] = make_float2(zk.y, zk.x);
                    Bf[r0 - 1 - k] = make_float2(zm.y, zm.x);
                }
            }
        }
        fft_run<PR, 1, true, false, Cta, TWALU, Hook, SINGLE, TWS1>(v, t, sbuf0, buf_stride, parity, p.twM, cta, twb, hook, tw_s1);
    } else {
        float2* sb = sbuf0 + parity * buf_stride;
        parity ^= 1;
        // All loads first (one memory round trip per partial spectrum, not one per bin), then the
        // arithmetic.
        float2 pa[R / 2 + 1], pb[R / 2 + 1];
        const bool split_sum = LAYOUT < 0 && p.layout == LAYOUT_HALF_PACKED && p.n_partials > 1;
#pragma unroll
        for (int q = 0; q <= R / 2; ++q) {
            const int k = t + q * T;
            pa[q] = make_float2(0.f, 0.f);
            pb[q] = pa[q];
            if (k > M / 2 || !active) continue;
            if (split_sum) {  // raw bins of partial spectrum 0; bin 0 is unpacked after the sum
                pa[q] = MA_LDG(x + k);
                pb[q] = MA_LDG(x + (k == 0 ? 0 : M - k));
            } else {
                c2r_load_pair<LAYOUT>(p, x, g, k, M, pa[q], pb[q]);
            }
        }
        if (split_sum) {
            for (int i = 1; i < p.n_partials; ++i) {
                const float2* xi = x + (int64_t)i * p.partial_stride;
#pragma unroll
                for (int q = 0; q <= R / 2; ++q) {
                    const int k = t + q * T;
                    if (k > M / 2 || !active) continue;
                    const float2 ya = MA_LDG(xi + k);
                    const float2 yb = MA_LDG(xi + (k == 0 ? 0 : M - k));
                    pa[q].x += ya.x;
                    pa[q].y += ya.y;
                    pb[q].x += yb.x;
                    pb[q].y += yb.y;
                }
            }
            if (t == 0) {  // k == 0 (q == 0): bin 0 holds (DC, Nyquist)
                pb[0] = make_float2(pa[0].y, 0.f);
                pa[0] = make_float2(pa[0].x, 0.f);
            }
        }
#pragma unroll
        for (int q = 0; q <= R / 2; ++q) {
            const int k = t + q * T;
            if (k > M / 2) continue;
            const float2 w = MA_LDG(p.twN + k);
            float2 zk, zm;
            herm_pre(pa[q], pb[q], w, zk, zm);
            sb[saddr<1>(k)] = make_float2(zk.y, zk.x);
            if (k > 0) sb[saddr<1>(M - k)] = make_float2(zm.y, zm.x);
        }
        cta.sync();
#pragma unroll
        for (int q = 0; q < R; ++q) v[q] = sb[saddr<1>(t + q * T)];
        fft_forward_regs<M, 1, Cta>(v, t, sbuf0, buf_stride, parity, p.twM, cta);
    }
}

// Loads the frame-invariant twiddles of the register-resident mode for the inverse kernels.
template <int M>
MA_HD void c2r_load_tw_regs(const C2RParams& p, int t, float2* twb, float2* wherm) {
    if constexpr (plan_pairable<M>()) {
        using PR = FftPlanRev<M>;
        constexpr int NB0 = PR::R / PR::radix(0);
        load_tw_bases<PR, false>(twb, t, p.twM);
#pragma unroll
        for (int c = 0; c < NB0 / 2; ++c) wherm[c] = MA_LDG(p.twN + (c * PR::T + t));
    }
}

// Plain batched inverse: out[g][2n], out[g][2n+1].  LAYOUT >= 0: layout fixed at compile time
// and (for paired plans) twiddles kept in registers.
template <int M, int LAYOUT, class Cta>
MA_HD void c2r_body(const C2RParams& p, Cta& cta, float2* smem) {
    using P = FftPlan<M>;
    using S = CtaShape<M>;
    constexpr int R = P::R, T = P::T, N = 2 * M;
    constexpr bool TWALU = LAYOUT >= 0 && plan_pairable<M>();
    const int tid = cta.tid();
    const int slot = tid / T;
    const int t = tid % T;
    float2* sbuf0 = smem + slot * S::ELEMS;
    int parity = 0;
    const float scale = 1.0f / (float)N;
    const int64_t total = p.n_signals * p.frames_per_signal;
    float2 twb[tw_base_count<FftPlanRev<M>>()];
    float2 wherm[R / 2 + 1];
    if constexpr (TWALU) c2r_load_tw_regs<M>(p, t, twb, wherm);
    const int64_t stride_frames = (int64_t)cta.nblocks() * S::FPC;
    int64_t g = (int64_t)cta.bid() * S::FPC + slot;
    int64_t s = g / p.frames_per_signal;
    int64_t f = g - s * p.frames_per_signal;
    const int64_t ds = stride_frames / p.frames_per_signal;
    const int64_t df = stride_frames - ds * p.frames_per_signal;
    // Staged variant (half layouts of paired plans): the next frame's row is brought into shared
    // memory by one bulk asynchronous copy while this frame is transformed.
    constexpr bool STAGED = TWALU && (LAYOUT == LAYOUT_HALF_INTERLEAVED || LAYOUT == LAYOUT_HALF_PACKED);
    float2* stage_slot = smem + 2 * S::BUF_STRIDE + slot * S::ROW;
    uint64_t* bar = reinterpret_cast<uint64_t*>(smem + 2 * S::BUF_STRIDE + S::FPC * S::ROW) + 2 * slot;
    uint32_t phase = 0;
    (void)stage_slot;
    (void)bar;
    float2* tw1 = smem + 2 * S::BUF_STRIDE + S::FPC * S::ROW + 2 * S::FPC;  // stage-1 twiddle table (staged variant)
    (void)tw1;
    if constexpr (STAGED) {
        stage1_table_fill<FftPlanRev<M>>(tw1, p.twM, tid, S::THREADS);
        if (t == 0) cta.bulk_init(bar);
        cta.sync();
        if (t == 0 && g < total) {
            const StagedRow r0 = staged_row<M>(p, s, f);
            cta.bulk_copy(stage_slot, r0.src, r0.bytes, bar);
        }
    }
    for (int64_t base = (int64_t)cta.bid() * S::FPC; base < total;
         base += stride_frames, g += stride_frames, s += ds, f += df) {
        if (f >= p.frames_per_signal) {
            f -= p.frames_per_signal;
            ++s;
        }
        const bool active = S::FPC == 1 ? true : g < total;
        float2 v[R];
        if constexpr (STAGED) {
            StagedRow r;
            r.shift = 0;
            r.row = nullptr;
            if (active) {
                r = staged_row<M>(p, s, f);
                if (!cta.bulk_wait(bar, phase) && p.error_flag != nullptr) *p.error_flag = 1;
                phase ^= 1;
            }
            auto issue_next = [&]() {
                if (t == 0 && g + stride_frames < total) {
                    int64_t fn = f + df, sn = s + ds;
                    if (fn >= p.frames_per_signal) {
                        fn -= p.frames_per_signal;
                        ++sn;
                    }
                    const StagedRow rn = staged_row<M>(p, sn, fn);
                    cta.bulk_copy(stage_slot, rn.src, rn.bytes, bar);
                }
            };
            c2r_frame<M, LAYOUT, TWALU, Cta, true, decltype(issue_next), false, true>(
                p, active, s, f, g, t, sbuf0, S::BUF_STRIDE, parity, v, cta, twb, wherm, stage_slot + r.shift, issue_next, r.row, tw1);
        } else {
            c2r_frame<M, LAYOUT, TWALU, Cta>(p, active, s, f, g, t, sbuf0, S::BUF_STRIDE, parity, v, cta, twb, wherm);
        }
        if (active && p.tail == nullptr) {
            float2* o = reinterpret_cast<float2*>(p.out + g * (int64_t)N);
#pragma unroll
            for (int q = 0; q < R; ++q) o[t + q * T] = make_float2(v[q].y * scale, v[q].x * scale);
        } else if (active) {
            // Streaming convolution step: emit the first half plus the kept tail of the
            // previous block, keep the second half as the new tail.
            float* o = p.out + g * p.out_signal_stride;
            float* tl = p.tail + g * (int64_t)M;
            if constexpr (R == 1) {
                o[0] = v[0].y * scale + tl[0];
                tl[0] = v[0].x * scale;
            } else {
#pragma unroll
                for (int q = 0; q < R / 2; ++q) {
                    const int i0 = 2 * (t + q * T);
                    o[i0] = v[q].y * scale + tl[i0];
                    o[i0 + 1] = v[q].x * scale + tl[i0 + 1];
                    tl[i0] = v[q + R / 2].y * scale;
                    tl[i0 + 1] = v[q + R / 2].x * scale;
                }
            }
        }
    }
}

// Sum of squared window over the frames covering output position o, accumulated in
// increasing frame order in float32 (the order of the reference's sequential loop),
// denormal results zeroed, clamped to the floor.
MA_HD float window_sum_at(const float* __restrict__ window, int64_t o, int N, int hop,
                          int64_t frames, float floor) {
    int64_t f_lo = (o >= N) ? (o - N) / hop + 1 : 0;
    int64_t f_hi = o / hop;
    if (f_hi > frames - 1) f_hi = frames - 1;
    float acc = 0.f;
    for (int64_t f = f_lo; f <= f_hi; ++f) {
        float w = window ? MA_LDG(window + (o - f * hop)) : 1.0f;
        acc += w * w;
    }
    if (acc < 1.17549435e-38f) acc = 0.f;
    return acc > floor ? acc : floor;
}

// iSTFT: one CTA (T threads, one frame at a time) owns the frames [f0, f1) of one signal
// and the output samples [f0*hop, f1*hop) (through the end of the signal for the last
// chunk).  Overlap-add runs in a shared-memory ring of N floats; the frames before f0 that
// reach into the chunk are recomputed instead of exchanged, so no atomics and a fixed
// summation order.  smem: 2 exchange buffers (float2) followed by the ring (N floats).
//
// With window == nullptr and floor < 0 the normaliser is skipped (plain overlap-add of
// scaled inverse frames): that is the block overlap-add of partitioned convolution.
template <int M, class Cta>
MA_HD void istft_body(const C2RParams& p, Cta& cta, float2* smem) {
    using P = FftPlan<M>;
    constexpr int R = P::R, T = P::T, N = 2 * M;
    constexpr int ELEMS = smem_elems_per_fft<M, 1>();
    const int t = cta.tid();
    float* ring = reinterpret_cast<float*>(smem + 2 * ELEMS);
    int parity = 0;
    const float scale = 1.0f / (float)N;
    const int hop = p.hop;
    const int64_t F = p.frames_per_signal;
    const bool normalise = !(p.window == nullptr && p.floor < 0.f);

    float2 wreg[R];
#pragma unroll
    for (int q = 0; q < R; ++q) {
        const int n = t + q * T;
        if (p.window != nullptr)
            wreg[q] = make_float2(MA_LDG(p.window + 2 * n) * scale, MA_LDG(p.window + 2 * n + 1) * scale);
        else
            wreg[q] = make_float2(scale, scale);
    }

    const int64_t n_chunks = (int64_t)p.chunks_per_signal;
    const int64_t total_chunks = p.n_signals * n_chunks;
    const int64_t per = (F + n_chunks - 1) / n_chunks;
    const int reach = (N + hop - 1) / hop - 1;  // earlier frames overlapping a frame start

    for (int64_t c = cta.bid(); c < total_chunks; c += cta.nblocks()) {
        const int64_t s = c / n_chunks;
        const int64_t ci = c - s * n_chunks;
        const int64_t f0 = ci * per;
        int64_t f1 = f0 + per;
        if (f1 > F) f1 = F;
        if (f0 >= f1) continue;  // uniform across the CTA
        int64_t fh = f0 - reach;
        if (fh < 0) fh = 0;
        for (int i = t; i < N; i += T) ring[i] = 0.f;
        cta.sync();
        for (int64_t f = fh; f < f1; ++f) {
            float2 v[R];
            c2r_frame<M, -1, false, Cta>(p, true, s, f, s * F + f, t, smem, ELEMS, parity, v, cta);
            const int64_t start = f * (int64_t)hop;
            if ((hop & 1) == 0) {
                float2* ring2 = reinterpret_cast<float2*>(ring);
                const int h0 = (int)((start & (N - 1)) >> 1);
#pragma unroll
                for (int q = 0; q < R; ++q) {
                    const int pp = (h0 + t + q * T) & (M - 1);
                    float2 r = ring2[pp];
                    r.x += v[q].y * wreg[q].x;
                    r.y += v[q].x * wreg[q].y;
                    ring2[pp] = r;
                }
            } else {
#pragma unroll
                for (int q = 0; q < R; ++q) {
                    const int n2 = 2 * (t + q * T);
                    const int p0 = (int)((start + n2) & (N - 1));
                    const int p1 = (int)((start + n2 + 1) & (N - 1));
                    ring[p0] += v[q].y * wreg[q].x;
                    ring[p1] += v[q].x * wreg[q].y;
                }
            }
            cta.sync();
            // Samples [start, start+span) are complete: emit and clear them.
            const int span = (f == F - 1) ? N : hop;
            const bool emit = f >= f0;
            for (int i = t; i < span; i += T) {
                const int64_t o = start + i;
                const int rp = (int)(o & (N - 1));
                const float acc = ring[rp];
                ring[rp] = 0.f;
                if (emit && o < p.out_len) {
                    float r = acc;
                    if (normalise) {
                        // interior positions (all overlapping frames exist) share hop distinct sums
                        const bool mid = o >= (int64_t)(N - hop) && o < F * (int64_t)hop;
                        const float ws = mid ? MA_LDG(p.norm_mid + i) : window_sum_at(p.window, o, N, hop, F, p.floor);
                        r = acc / ws;
                    }
                    p.out[s * p.out_signal_stride + o] = r;
                }
            }
            cta.sync();
        }
    }
}

// Fast iSTFT for paired plans when hop/2 is a multiple of T (e.g. N = 4096, hop = 1024) and the
// spectra are in a half layout.  Differences from istft_body:
//  * thread t only ever touches overlap-add positions congruent to t modulo T, so the overlap-add
//    ring is thread-private: no barrier for accumulate or emit, only the two FFT exchanges remain;
//  * completed samples go straight from registers to HBM, multiplied by the precomputed
//    reciprocal of the interior window sum (frames near the ends of the signal take the exact
//    per-sample path);
//  * twiddles live in registers (power chains) and the layout is fixed at compile time.
// OVT is the overlap count N/hop when fixed at compile time (0: read it from p.hop).
//  * OVT > 0: the ring lives in REGISTERS.  Slots are numbered from the current frame's start, a
//    frame completes the first H = R/OVT of them, and the sum for slot q >= H is written to
//    register q - H, which is where the next frame expects it: the rotation costs nothing.  Window
//    multiply and accumulate are one packed multiply-add per sample pair.  The registers the ring
//    takes are the ones the window used to hold: the window (in thread order, 1/N folded in) sits
//    in the shared memory the ring used to take and is read with 16-byte loads.  (Reading it from
//    global memory through L1 instead, to afford a second exchange buffer, measured 27 % slower:
//    the loads' latency is exposed at four warps per scheduler.)
//  * OVT == 0: ring [R][T] float2 in shared memory, window in registers.
// smem: exchange buffer | ring or window table [R*T] float2 | staged row [M+2] float2 | mbarrier.
template <int M, int OVT = 0>
struct IstftFastShape {
    using P = FftPlan<M>;
    static constexpr bool REGRING = OVT > 0;
    static constexpr int ELEMS = smem_elems_per_fft<M, 1>();
    static constexpr int RING = P::R * P::T;  // the ring, or (REGRING) the window table
    static constexpr int ROW = M + 2;  // staged spectrum row with the alignment slack
    static constexpr int EXCH = 1;  // exchange buffers (1: a barrier before each write instead of a second buffer)
    static constexpr int EXCH_ELEMS = (EXCH * ELEMS + 1) & ~1;  // keeps the staged row 16-byte aligned
    static constexpr int TW1 = stage1_table_elems<FftPlanRev<M>>();  // stage-1 twiddle table behind the mbarrier
    static constexpr int SMEM_BYTES = (EXCH_ELEMS + RING + ROW + TW1) * (int)sizeof(float2) + 16;
    static_assert(!plan_pairable<M>() || ((EXCH_ELEMS + RING) * sizeof(float2)) % 16 == 0,
                  "bulk copy destination must be 16-byte aligned");
};

// Whether istft_fast_body serves these parameters.
template <int M>
inline bool istft_fast_ok(const C2RParams& p) {
    if constexpr (!plan_pairable<M>()) {
        (void)p;
        return false;
    } else {
        constexpr int R = FftPlan<M>::R, T = FftPlan<M>::T;
        if (p.layout != LAYOUT_HALF_INTERLEAVED && p.layout != LAYOUT_HALF_PACKED && p.layout != LAYOUT_HALF_POLAR) return false;
        // staged magnitude / phase rows are copied from 16-byte boundaries: the arrays must start on one
        if (p.layout == LAYOUT_HALF_POLAR && (M % 4 != 0 || ((reinterpret_cast<uintptr_t>(p.in_a) | reinterpret_cast<uintptr_t>(p.in_b)) & 15) != 0))
            return false;
        if (p.n_partials > 1 || p.hop <= 0 || p.hop % (2 * T) != 0) return false;
        const int h = p.hop / (2 * T);
        if (h > R || R % h != 0) return false;
        if ((reinterpret_cast<uintptr_t>(p.out) & 7) != 0 || (p.out_signal_stride & 1) != 0) return false;
        return true;
    }
}

template <int M, int LAYOUT, int OVT, class Cta>
MA_HD void istft_fast_body(const C2RParams& p, Cta& cta, float2* smem) {
    using P = FftPlan<M>;
    using SH = IstftFastShape<M, OVT>;
    constexpr int R = P::R, T = P::T, N = 2 * M;
    constexpr bool REGRING = SH::REGRING;
    // Every layout stages the next frame's spectrum row(s) with bulk copies: one copy of the complex
    // row, or one each of the magnitude and the phase row.
    constexpr bool POLAR = LAYOUT == LAYOUT_HALF_POLAR;
    float2* ring = smem + SH::EXCH_ELEMS;
    float2* stage = ring + SH::RING;
    uint64_t* bar = reinterpret_cast<uint64_t*>(stage + SH::ROW);
    float2* tw1 = stage + SH::ROW + 2;  // 16 bytes of barrier, then the stage-1 twiddle table
    auto start_copy = [&](int64_t s_, int64_t f_) {  // called by thread 0
        if constexpr (POLAR) {
            const int64_t g_ = s_ * p.frames_per_signal + f_;
            const int shift = (int)(g_ & 3);
            float* dst = reinterpret_cast<float*>(stage);
            cta.bulk_expect(bar, 2u * M * (uint32_t)sizeof(float));
            cta.bulk_part(dst, p.in_a + g_ * (int64_t)(M + 1) - shift, M * (uint32_t)sizeof(float), bar);
            cta.bulk_part(dst + M, p.in_b + g_ * (int64_t)(M + 1) - shift, M * (uint32_t)sizeof(float), bar);
        } else {
            const StagedRow r_ = staged_row<M>(p, s_, f_);
            cta.bulk_copy(stage, r_.src, r_.bytes, bar);
        }
    };
    const int t = cta.tid();
    int parity = 0;
    uint32_t phase = 0;
    const float scale = 1.0f / (float)N;
    const int hop = p.hop;
    const int h = OVT > 0 ? R / OVT : hop / (2 * T);  // ring slots completed per frame
    const int64_t F = p.frames_per_signal;
    const bool normalise = !(p.window == nullptr && p.floor < 0.f);

    float2 wreg[REGRING ? 1 : R];
    if constexpr (REGRING) {
        // window table into shared memory, once: entry [q2*T + t] is read by thread t alone
        float4* wtab = reinterpret_cast<float4*>(ring);
#pragma unroll
        for (int q2 = 0; q2 < R / 2; ++q2)
            wtab[q2 * T + t] = p.window_syn != nullptr ? MA_LDG(p.window_syn + q2 * T + t) : make_float4(scale, scale, scale, scale);
    } else {
#pragma unroll
        for (int q = 0; q < R; ++q) {
            const int n = t + q * T;
            if (p.window != nullptr)
                wreg[q] = make_float2(MA_LDG(p.window + 2 * n) * scale, MA_LDG(p.window + 2 * n + 1) * scale);
            else
                wreg[q] = make_float2(scale, scale);
        }
    }
    float2 twb[tw_base_count<FftPlanRev<M>>()];
    float2 wherm[R / 2 + 1];
    c2r_load_tw_regs<M>(p, t, twb, wherm);
    // reciprocal window sums of the samples an interior frame completes (positions modulo hop)
    constexpr int HN = OVT > 0 ? R / OVT : 1;
    float2 ninv[HN];
#pragma unroll
    for (int q = 0; q < HN; ++q)
        ninv[q] = (OVT > 0 && normalise) ? MA_LDG(reinterpret_cast<const float2*>(p.norm_mid_inv + 2 * (t + q * T)))
                                         : make_float2(1.f, 1.f);

    // This CTA owns the global frames [G0, G1) (frame G = signal*F + f) and the output samples
    // they complete.  It starts up to `reach` frames early inside the same signal to rebuild the
    // overlap (no emission for those), so no CTA depends on another and the summation order is
    // fixed.
    const int64_t total = p.n_signals * F;
    const int64_t per = (total + cta.nblocks() - 1) / cta.nblocks();
    const int64_t G0 = (int64_t)cta.bid() * per;
    int64_t G1 = G0 + per;
    if (G1 > total) G1 = total;
    if (G0 >= G1) return;  // uniform across the CTA
    const int reach = R / h - 1;
    int64_t s = G0 / F;
    int64_t f = G0 - s * F;
    int64_t lead = f < reach ? f : reach;
    f -= lead;
    int64_t G = G0 - lead;

    if (t == 0) cta.bulk_init(bar);
    stage1_table_fill<FftPlanRev<M>>(tw1, p.twM, t, T);
    // register ring (REGRING): racc[i] = (odd sample, even sample) partial sums of slot i of the next
    // frame, in the pair order the inverse transform produces
    constexpr int HR = REGRING ? R / OVT : R;
    float2 racc[REGRING ? R - HR : 1];
    if constexpr (REGRING) {
#pragma unroll
        for (int i = 0; i < R - HR; ++i) racc[i] = make_float2(0.f, 0.f);
    } else {
#pragma unroll
        for (int q = 0; q < R; ++q) ring[q * T + t] = make_float2(0.f, 0.f);
    }
    cta.sync();
    if (t == 0) start_copy(s, f);

    for (; G < G1; ++G, ++f) {
        if (f == F) {  // next signal: nothing overlaps across signals
            f = 0;
            ++s;
            if constexpr (REGRING) {
#pragma unroll
                for (int i = 0; i < R - HR; ++i) racc[i] = make_float2(0.f, 0.f);
            } else {
#pragma unroll
                for (int q = 0; q < R; ++q) ring[q * T + t] = make_float2(0.f, 0.f);
            }
        }
        float2 v[R];
        if (!cta.bulk_wait(bar, phase) && p.error_flag != nullptr) *p.error_flag = 1;
        phase ^= 1;
        auto issue_next = [&]() {
            if (t == 0 && G + 1 < G1) {
                const bool wrap = f + 1 == F;
                start_copy(wrap ? s + 1 : s, wrap ? 0 : f + 1);
            }
        };
        if constexpr (POLAR) {
            c2r_frame<M, LAYOUT, true, Cta, true, decltype(issue_next), SH::EXCH == 1, true>(
                p, true, s, f, G, t, smem, SH::ELEMS, parity, v, cta, twb, wherm, stage, issue_next, nullptr, tw1);
        } else {
            const StagedRow r = staged_row<M>(p, s, f);
            c2r_frame<M, LAYOUT, true, Cta, true, decltype(issue_next), SH::EXCH == 1, true>(
                p, true, s, f, G, t, smem, SH::ELEMS, parity, v, cta, twb, wherm, stage + r.shift, issue_next, r.row, tw1);
        }

        // v[q] = (x[2n+1], x[2n]) * N for n = t + q*T.  Overlap-add in this thread's ring column.
        const int64_t start = f * (int64_t)hop;
        const int rot = (int)((f * (int64_t)h) & (R - 1));
        const bool last = f == F - 1;
        const bool emit = G >= G0;
        // every sample this frame completes has all its overlapping frames present
        const bool interior = !last && start >= (int64_t)(N - hop);
        float* out = p.out + s * p.out_signal_stride + start;
        if constexpr (REGRING) {
            const float4* wtab = reinterpret_cast<const float4*>(ring) + t;
            if (emit && interior && normalise) {
                // The common frame (every overlapping frame present, inside this CTA's range): no
                // per-slot decisions, reciprocals of the window sum already in registers.
#pragma unroll
                for (int q2 = 0; q2 < R / 2; ++q2) {
                    const float4 w4 = wtab[q2 * T];
#pragma unroll
                    for (int e = 0; e < 2; ++e) {
                        const int q = 2 * q2 + e;
                        const float2 wsw = e == 0 ? make_float2(w4.x, w4.y) : make_float2(w4.z, w4.w);
                        // (odd, even) sample pair of slot q with every frame up to this one
                        const float2 acc = q < R - HR ? pfma(v[q], wsw, racc[q]) : pmul(v[q], wsw);
                        if (q < HR)
                            *reinterpret_cast<float2*>(out + 2 * (t + q * T)) =
                                make_float2(acc.y * ninv[q < HN ? q : 0].x, acc.x * ninv[q < HN ? q : 0].y);
                        else
                            racc[q - HR] = acc;  // slot q is slot q - H of the next frame
                    }
                }
                continue;
            }
#pragma unroll
            for (int q2 = 0; q2 < R / 2; ++q2) {
                const float4 w4 = wtab[q2 * T];
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const int q = 2 * q2 + e;
                    const float2 wsw = e == 0 ? make_float2(w4.x, w4.y) : make_float2(w4.z, w4.w);
                    const float2 acc = q < R - HR ? pfma(v[q], wsw, racc[q]) : pmul(v[q], wsw);
                    const int i0 = 2 * (t + q * T);
                    if ((q < HR || last) && emit) {
                        float2 r2 = make_float2(acc.y, acc.x);
                        if (normalise) {
                            if (interior) {
                                const float2 inv = MA_LDG(reinterpret_cast<const float2*>(p.norm_mid_inv + i0));
                                r2.x *= inv.x;
                                r2.y *= inv.y;
                            } else {
                                const int64_t o = start + i0;
                                r2.x = r2.x / window_sum_at(p.window, o, N, hop, F, p.floor);
                                r2.y = r2.y / window_sum_at(p.window, o + 1, N, hop, F, p.floor);
                            }
                        }
                        *reinterpret_cast<float2*>(out + i0) = r2;
                    }
                    if (q >= HR) racc[q - HR] = acc;
                }
            }
            continue;
        }
        // shared-memory ring (overlap count known only at run time)
#pragma unroll
        for (int q = 0; q < (REGRING ? 0 : R); ++q) {
            float2* slot = ring + ((q + rot) & (R - 1)) * T + t;
            float2 acc = make_float2(v[q].y * wreg[REGRING ? 0 : q].x, v[q].x * wreg[REGRING ? 0 : q].y);
            if (q < R - h) {  // slot already holds earlier frames
                const float2 old = *slot;
                acc.x += old.x;
                acc.y += old.y;
            }
            if (q < h || last) {  // complete after this frame: emit
                if (emit) {
                    const int i0 = 2 * (t + q * T);
                    float2 r2 = acc;
                    if (normalise) {
                        if (interior) {
                            const float2 inv = MA_LDG(reinterpret_cast<const float2*>(p.norm_mid_inv + i0));
                            r2.x = acc.x * inv.x;
                            r2.y = acc.y * inv.y;
                        } else {
                            const int64_t o = start + i0;
                            r2.x = acc.x / window_sum_at(p.window, o, N, hop, F, p.floor);
                            r2.y = acc.y / window_sum_at(p.window, o + 1, N, hop, F, p.floor);
                        }
                    }
                    *reinterpret_cast<float2*>(out + i0) = r2;
                }
            } else {
                *slot = acc;
            }
        }
    }
}

}  // namespace ma
