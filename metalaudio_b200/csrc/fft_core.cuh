// Register/shared-memory Stockham FFT building blocks (FP32 SIMT, sm_100a).
//
// A complex transform of length M is run by T = M/R threads that each hold R points in
// registers.  Stage 0 is an R-point butterfly on points loaded with stride T; every
// later stage exchanges through shared memory in the Stockham autosort pattern
// (read element jv + k*M/r, twiddle, r-point butterfly, write element
// (jv/Ns)*Ns*r + jv%Ns + k*Ns), so no bit-reversal pass exists.  The exchange buffer is
// double-buffered: one barrier per exchange.
//
// Everything here is __host__ __device__ and templated on a "Cta" type that supplies the
// barrier, so that the index arithmetic can be executed on the CPU by a thread-per-lane
// emulator in the test-suite as well as by the kernels.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#define MA_HD __host__ __device__ __forceinline__

#ifdef __CUDA_ARCH__
#include <cuda_pipeline.h>
#define MA_LDG(p) __ldg(p)
// Asynchronous 8-byte global -> shared copy (LDGSTS): no registers, no stall until the wait.
#define MA_ASYNC_COPY8(dst, src) __pipeline_memcpy_async((dst), (src), 8)
#define MA_ASYNC_COMMIT() __pipeline_commit()
#define MA_ASYNC_WAIT_ALL() __pipeline_wait_prior(0)
#else
#define MA_LDG(p) (*(p))
#define MA_ASYNC_COPY8(dst, src) (*(dst) = *(src))
#define MA_ASYNC_COMMIT() ((void)0)
#define MA_ASYNC_WAIT_ALL() ((void)0)
#endif

namespace ma {

// ---------------------------------------------------------------- complex helpers
// On the device a complex add / subtract is ONE packed two-wide FP32 instruction (add.f32x2 /
// fma.rn.f32x2 of sm_100): these kernels are bound by instruction issue, and half of a
// transform's arithmetic is complex additions.  a - b is fma(b, -1, a): exact negation, one
// rounding, the same result as the subtraction.
#if defined(__CUDA_ARCH__) && __CUDA_ARCH__ >= 1000 && !defined(MA_SCALAR_MATH)
#define MA_PACKED 1
MA_HD float2 cadd(float2 a, float2 b) { return __fadd2_rn(a, b); }
MA_HD float2 csub(float2 a, float2 b) { return __ffma2_rn(b, make_float2(-1.f, -1.f), a); }
// a + s*t and a - s*t for a real scale s, one instruction each
MA_HD float2 cfma_scaled(float2 t, float s, float2 a) { return __ffma2_rn(t, make_float2(s, s), a); }
// element-wise product and multiply-add of pairs
MA_HD float2 pmul(float2 a, float2 b) { return __fmul2_rn(a, b); }
MA_HD float2 pfma(float2 a, float2 b, float2 c) { return __ffma2_rn(a, b, c); }
#else
#define MA_PACKED 0
MA_HD float2 cadd(float2 a, float2 b) { return make_float2(a.x + b.x, a.y + b.y); }
MA_HD float2 csub(float2 a, float2 b) { return make_float2(a.x - b.x, a.y - b.y); }
MA_HD float2 cfma_scaled(float2 t, float s, float2 a) { return make_float2(fmaf(t.x, s, a.x), fmaf(t.y, s, a.y)); }
MA_HD float2 pmul(float2 a, float2 b) { return make_float2(a.x * b.x, a.y * b.y); }
MA_HD float2 pfma(float2 a, float2 b, float2 c) { return make_float2(fmaf(a.x, b.x, c.x), fmaf(a.y, b.y, c.y)); }
#endif
MA_HD float2 cmul(float2 a, float2 b) {
    return make_float2(a.x * b.x - a.y * b.y, a.x * b.y + a.y * b.x);
}
MA_HD float2 cconj(float2 a) { return make_float2(a.x, -a.y); }
// a * (-i)
MA_HD float2 cmul_mi(float2 a) { return make_float2(a.y, -a.x); }

// atan2 for finite arguments, about 4e-7 rad maximum error: odd polynomial in min/max (degree 15,
// near-minimax on [0, 1]) with the octant folded back afterwards.  Signed zeros of x count as +0.
MA_HD float fast_atan2(float y, float x) {
#ifdef __CUDA_ARCH__
    const float ax = fabsf(x), ay = fabsf(y);
    const float mx = fmaxf(ax, ay), mn = fminf(ax, ay);
    const float a = mx > 0.f ? __fdividef(mn, mx) : 0.f;
    const float s = a * a;
    float r = -0.004668773151934147f;
    r = fmaf(r, s, 0.02416618913412094f);
    r = fmaf(r, s, -0.0593671016395092f);
    r = fmaf(r, s, 0.09906096756458282f);
    r = fmaf(r, s, -0.14016585052013397f);
    r = fmaf(r, s, 0.19969235360622406f);
    r = fmaf(r, s, -0.33331960439682007f);
    r = fmaf(r, s, 0.9999998807907104f);
    r *= a;
    if (ay > ax) r = 1.5707963705062866f - r;
    if (x < 0.f) r = 3.1415927410125732f - r;
    return copysignf(r, y);
#else
    return atan2f(y, x);
#endif
}

// sin and cos with an explicit two-constant reduction by 2*pi followed by the hardware
// approximations: absolute error below 5e-7 for |x| up to about 1e4 rad.
MA_HD void fast_sincos(float x, float* sn, float* cs) {
#ifdef __CUDA_ARCH__
    const float k = rintf(x * 0.15915494309189535f);
    float r = fmaf(-k, 6.2831854820251465f, x);
    r = fmaf(k, 1.7484555e-7f, r);  // 2*pi = 6.2831854820251465 - 1.7484555e-7
    *sn = __sinf(r);
    *cs = __cosf(r);
#else
    sincosf(x, sn, cs);
#endif
}

// Multiply by W_R^K = exp(-2*pi*i*K/R) with the trivial cases resolved at compile time.
template <int R, int K>
MA_HD float2 mul_wconst(float2 v) {
    constexpr float kS = 0.70710678118654752440f;  // sqrt(1/2)
    constexpr float kC1 = 0.92387953251128675613f; // cos(pi/8)
    constexpr float kS1 = 0.38268343236508977173f; // sin(pi/8)
    if constexpr (K == 0) {
        return v;
    } else if constexpr (4 * K == R) {  // -i
        return make_float2(v.y, -v.x);
    } else if constexpr (8 * K == R) {  // (1 - i)/sqrt2
        return make_float2((v.x + v.y) * kS, (v.y - v.x) * kS);
    } else if constexpr (8 * K == 3 * R) {  // (-1 - i)/sqrt2
        return make_float2((v.y - v.x) * kS, -(v.x + v.y) * kS);
    } else if constexpr (16 * K == R) {  // W16^1 = (c1, -s1)
        return make_float2(v.x * kC1 + v.y * kS1, v.y * kC1 - v.x * kS1);
    } else if constexpr (16 * K == 3 * R) {  // W16^3 = (s1, -c1)
        return make_float2(v.x * kS1 + v.y * kC1, v.y * kS1 - v.x * kC1);
    } else if constexpr (16 * K == 5 * R) {  // W16^5 = (-s1, -c1)
        return make_float2(v.y * kC1 - v.x * kS1, -v.x * kC1 - v.y * kS1);
    } else {  // 16*K == 7*R : W16^7 = (-c1, -s1)
        static_assert(16 * K == 7 * R, "unsupported constant twiddle");
        return make_float2(v.y * kS1 - v.x * kC1, -v.x * kS1 - v.y * kC1);
    }
}

// ---------------------------------------------------------------- register butterflies
// In-place forward DFT (sign -) of R points held in registers, natural order in and out.
template <int R>
struct Bfly;

template <>
struct Bfly<1> {
    static MA_HD void run(float2* a) { (void)a; }
};
template <>
struct Bfly<2> {
    static MA_HD void run(float2* a) {
        float2 t = a[0];
        a[0] = cadd(t, a[1]);
        a[1] = csub(t, a[1]);
    }
};
// e + (-i)*d and e - (-i)*d.  (-i)*d = (d.y, -d.x) crosses the components, which a packed add cannot
// do without first moving registers, so these four sums stay scalar.
MA_HD void add_sub_mi(float2 e, float2 d, float2& plus, float2& minus) {
    plus = make_float2(e.x + d.y, e.y - d.x);
    minus = make_float2(e.x - d.y, e.y + d.x);
}

template <>
struct Bfly<4> {
    static MA_HD void run(float2* a) {
        float2 t0 = cadd(a[0], a[2]);
        float2 t1 = csub(a[0], a[2]);
        float2 t2 = cadd(a[1], a[3]);
        float2 d = csub(a[1], a[3]);
        a[0] = cadd(t0, t2);
        a[2] = csub(t0, t2);
        add_sub_mi(t1, d, a[1], a[3]);
    }
};

// a[K] = e[K] + W_R^K o[K], a[K + R/2] = e[K] - W_R^K o[K], with the constant twiddle folded into
// the sums where that saves instructions.
template <int R, int K>
struct BflyCombine {
    static MA_HD void run(float2* a, const float2* e, const float2* o) {
        constexpr float kS = 0.70710678118654752440f;  // sqrt(1/2)
        if constexpr (4 * K == R) {  // -i
            add_sub_mi(e[K], o[K], a[K], a[K + R / 2]);
        } else if constexpr (8 * K == R) {  // (1 - i)/sqrt2: t = (x + y, y - x) * kS
            const float2 t = make_float2(o[K].x + o[K].y, o[K].y - o[K].x);
            a[K] = cfma_scaled(t, kS, e[K]);
            a[K + R / 2] = cfma_scaled(t, -kS, e[K]);
        } else if constexpr (8 * K == 3 * R) {  // (-1 - i)/sqrt2: t = (y - x, -(x + y)) * kS
            const float2 t = make_float2(o[K].y - o[K].x, -(o[K].x + o[K].y));
            a[K] = cfma_scaled(t, kS, e[K]);
            a[K + R / 2] = cfma_scaled(t, -kS, e[K]);
        } else {
            float2 t = mul_wconst<R, K>(o[K]);
            a[K] = cadd(e[K], t);
            a[K + R / 2] = csub(e[K], t);
        }
        if constexpr (K + 1 < R / 2) BflyCombine<R, K + 1>::run(a, e, o);
    }
};

template <int R>
struct Bfly {
    static_assert(R == 8 || R == 16, "radix");
    static MA_HD void run(float2* a) {
        float2 e[R / 2], o[R / 2];
#pragma unroll
        for (int k = 0; k < R / 2; ++k) {
            e[k] = a[2 * k];
            o[k] = a[2 * k + 1];
        }
        Bfly<R / 2>::run(e);
        Bfly<R / 2>::run(o);
        BflyCombine<R, 0>::run(a, e, o);
    }
};

// ---------------------------------------------------------------- plans
// Radix chain per complex length M.  The first radix is always R (points per thread);
// later radices divide R.  Chains are chosen so that every shared-memory exchange is
// bank-conflict free with the 1-in-16 padding below.
template <int M>
struct FftPlan;

#define MA_DEFINE_PLAN(M_, R_, NS_, R0, R1, R2)                                     \
    template <>                                                                     \
    struct FftPlan<M_> {                                                            \
        static constexpr int M = M_;                                                \
        static constexpr int R = R_;                                                \
        static constexpr int T = M_ / R_;                                           \
        static constexpr int NS = NS_;                                              \
        static constexpr __host__ __device__ int radix(int s) { return s == 0 ? R0 : (s == 1 ? R1 : R2); } \
        static constexpr __host__ __device__ int ns_before(int s) {                                     \
            return s == 0 ? 1 : (s == 1 ? R0 : R0 * R1);                            \
        }                                                                           \
    };

MA_DEFINE_PLAN(1, 1, 1, 1, 1, 1)
MA_DEFINE_PLAN(2, 2, 1, 2, 1, 1)
MA_DEFINE_PLAN(4, 4, 1, 4, 1, 1)
MA_DEFINE_PLAN(8, 8, 1, 8, 1, 1)
MA_DEFINE_PLAN(16, 16, 1, 16, 1, 1)
MA_DEFINE_PLAN(32, 8, 2, 8, 4, 1)
MA_DEFINE_PLAN(64, 8, 2, 8, 8, 1)
MA_DEFINE_PLAN(128, 16, 2, 16, 8, 1)
MA_DEFINE_PLAN(256, 16, 2, 16, 16, 1)
MA_DEFINE_PLAN(512, 16, 3, 16, 8, 4)
MA_DEFINE_PLAN(1024, 16, 3, 16, 8, 8)
MA_DEFINE_PLAN(2048, 16, 3, 16, 16, 8)
MA_DEFINE_PLAN(4096, 16, 3, 16, 16, 16)
#undef MA_DEFINE_PLAN

// Threads per transform of the plan for length m (0 for a length without a plan).
inline int fft_plan_threads(int m) {
    switch (m) {
        case 32: return FftPlan<32>::T;
        case 64: return FftPlan<64>::T;
        case 128: return FftPlan<128>::T;
        case 256: return FftPlan<256>::T;
        case 512: return FftPlan<512>::T;
        case 1024: return FftPlan<1024>::T;
        case 2048: return FftPlan<2048>::T;
        case 4096: return FftPlan<4096>::T;
        default: return 0;
    }
}

// The same radices in reverse order (first stage the smallest radix, possibly several
// butterflies per thread).  Used by the inverse transforms, whose Hermitian pre-process
// feeds a paired first stage.
template <int M_>
struct FftPlanRev {
    using F = FftPlan<M_>;
    static constexpr int M = M_;
    static constexpr int R = F::R;
    static constexpr int T = F::T;
    static constexpr int NS = F::NS;
    static constexpr __host__ __device__ int radix(int s) { return F::radix(NS - 1 - s); }
    static constexpr __host__ __device__ int ns_before(int s) {
        int n = 1;
        for (int i = 0; i < s; ++i) n *= radix(i);
        return n;
    }
};

// True when the last forward stage (first reverse stage) runs at least two butterflies per
// thread, which is what the paired mapping needs.
template <int M_>
constexpr __host__ __device__ bool plan_pairable() {
    return FftPlan<M_>::NS >= 2 && (FftPlan<M_>::R / FftPlan<M_>::radix(FftPlan<M_>::NS - 1)) >= 2;
}

// Shared-memory addressing.  W == 1: one transform owns a contiguous region, element idx
// lives at idx + idx/16 (float2 units).  W > 1: W transforms are interleaved, element idx
// of transform slot i lives at idx*W + i (the caller passes the base already offset by i),
// which is conflict-free for any idx pattern when a half-warp spans 16 slots.
template <int W>
MA_HD int saddr(int idx) {
    if constexpr (W == 1) return idx + (idx >> 4);
    else return idx * W;
}

// float2 elements one transform needs in ONE exchange buffer.
template <int M, int W>
constexpr __host__ __device__ int smem_elems_per_fft() {
    if constexpr (W == 1) {
        constexpr int T = FftPlan<M>::T;
        int padded = M + (M >> 4) + 1;
        // Several small transforms share a half-warp: stagger their regions.
        if (T < 16) {
            while ((padded & 15) != (T & 15)) ++padded;
        }
        return padded;
    } else {
        return M;  // per slot; total M*W
    }
}

// ---------------------------------------------------------------- twiddled stages
// Stage twiddles live in one table per plan, stage after stage (stage 0 has none); inside a
// stage the layout is [k-1][j], j = jv % Ns, value exp(-2*pi*i*j*k/(Ns*r)).  Lanes run along
// j, so every load is contiguous across a warp (a gather from a single M-point table costs an
// L1 wavefront per distinct line), and all r-1 twiddles are exact table values.
template <class P>
constexpr __host__ __device__ int stage_tw_offset(int s) {
    int off = 0;
    for (int i = 1; i < s; ++i) off += P::ns_before(i) * (P::radix(i) - 1);
    return off;
}
template <class P>
constexpr __host__ __device__ int stage_tw_total() {
    return stage_tw_offset<P>(P::NS);
}

template <class P, int S>
MA_HD void load_stage_twiddles(float2* w, const float2* __restrict__ tws, int j) {
    constexpr int r = P::radix(S), Ns = P::ns_before(S), off = stage_tw_offset<P>(S);
#pragma unroll
    for (int k = 1; k < r; ++k) w[k] = MA_LDG(tws + off + (k - 1) * Ns + j);
}

// Register-resident alternative: the twiddles of a thread's butterflies do not change from
// frame to frame, and w^k follows from w^1 by a multiplication chain of depth <= 4, so a kernel
// that loops over many frames keeps one base twiddle per (stage, sub-butterfly) in registers
// and spends FMA-pipe work instead of load/store-pipe bandwidth (the scarcer resource here).
template <class P>
constexpr __host__ __device__ int tw_base_index(int s, int b) {
    int idx = 0;
    for (int i = 1; i < s; ++i) idx += P::R / P::radix(i);
    return idx + b;
}
template <class P>
constexpr __host__ __device__ int tw_base_count() {
    return tw_base_index<P>(P::NS, 0) > 0 ? tw_base_index<P>(P::NS, 0) : 1;
}

template <int r>
MA_HD void twiddle_powers(float2* w, float2 w1) {
    if constexpr (r >= 2) w[1] = w1;
    if constexpr (r >= 4) {
        w[2] = cmul(w1, w1);
        w[3] = cmul(w[2], w1);
    }
    if constexpr (r >= 8) {
        w[4] = cmul(w[2], w[2]);
        w[5] = cmul(w[4], w[1]);
        w[6] = cmul(w[4], w[2]);
        w[7] = cmul(w[4], w[3]);
    }
    if constexpr (r >= 16) {
        w[8] = cmul(w[4], w[4]);
#pragma unroll
        for (int k = 1; k < 8; ++k) w[8 + k] = cmul(w[8], w[k]);
    }
}

// Which butterfly of a stage a thread's b-th sub-butterfly is.  Natural: jv = t + b*T.
// Paired: the thread owns butterflies in pairs (j, nbfly - j), so that element i and element
// M - i of a stage input/output that is indexed jv + k*nbfly sit in the same thread; the two
// self-paired butterflies 0 and nbfly/2 go to thread 0.
template <class P, bool PAIRED>
MA_HD int stage_jv(int t, int b, int nbfly) {
    if constexpr (!PAIRED) {
        (void)nbfly;
        return t + b * P::T;
    } else {
        const int j = (b >> 1) * P::T + t;
        if ((b & 1) == 0) return j;
        return j == 0 ? (nbfly >> 1) : nbfly - j;
    }
}

// Padded address of element o0 + k*Ns as base(o0) + offset(k) with a compile-time offset, so
// that the r accesses of a butterfly need one address computation.  Valid because
// (o0 + k*Ns) >> 4 splits exactly in the three cases below (o0's low bits never carry).
template <int W, int Ns, int r>
struct ExchangeAddr {
    static constexpr bool kSplit = (W != 1) || (Ns % 16 == 0) || (Ns == 1 && (r == 16 || r == 8)) ||
                                   (Ns == 8 && r >= 2);
    static MA_HD int base(int o0) {
        if constexpr (W != 1) return o0 * W;
        else return o0 + (o0 >> 4);
    }
    static constexpr __host__ __device__ int offset(int k) {
        if (W != 1) return k * Ns * W;
        if (Ns % 16 == 0) return k * Ns + k * (Ns / 16);
        if (Ns == 1) return k;           // o0 = jv*r, r in {8, 16}: k < r never reaches bit 4 ... of o0's group
        return k * 8 + (k >> 1);         // Ns == 8: o0 % 16 < 8, so (o0%16 + 8k) >> 4 == k >> 1
    }
};

template <class P, int W, int S, bool PAIRED>
MA_HD void stage_write(const float2* v, int t, float2* sbuf) {
    constexpr int M = P::M, r = P::radix(S), Ns = P::ns_before(S), NB = P::R / r;
    using A = ExchangeAddr<W, Ns, r>;
#pragma unroll
    for (int b = 0; b < NB; ++b) {
        const int jv = stage_jv<P, PAIRED>(t, b, M / r);
        const int o0 = (jv / Ns) * (Ns * r) + (jv % Ns);
        if constexpr (A::kSplit) {
            float2* dst = sbuf + A::base(o0);
#pragma unroll
            for (int k = 0; k < r; ++k) dst[A::offset(k)] = v[b * r + k];
        } else {
#pragma unroll
            for (int k = 0; k < r; ++k) sbuf[saddr<W>(o0 + k * Ns)] = v[b * r + k];
        }
    }
}

// Stage-1 twiddles from shared memory.  The first twiddled stage has only Ns = radix(0) distinct
// twiddle sets (j = jv % Ns), so a table of Ns * r entries (1-2 KB) serves every thread of the CTA:
// r/2 16-byte loads per butterfly, all lanes of a warp inside one or two wavefronts, instead of the
// r-2 complex multiplications of a power chain.  Used by the inverse kernels (measured 1 % faster
// there and exact table values instead of chained products; in the forward kernel, whose
// load/store pipe is busier, the extra shared-memory reads cost 2 %).  Layout: entry [kp*Ns + j] (float4) =
// (w^(2kp+1), w^(2kp+2)) for butterfly-local twiddle base j; powers >= r are filled with 1.
template <class P>
constexpr __host__ __device__ bool stage1_table_ok() {
    return P::NS >= 2 && P::ns_before(1) <= 16 && P::radix(1) >= 4;
}
template <class P>
constexpr __host__ __device__ int stage1_table_elems() {  // float2 units, a multiple of 2
    return stage1_table_ok<P>() ? P::radix(1) * P::ns_before(1) : 0;
}
// Cooperative fill from the plan's global stage table (layout [k-1][j]); the caller synchronises.
template <class P>
MA_HD void stage1_table_fill(float2* tab, const float2* __restrict__ tws, int tid, int nthreads) {
    if constexpr (stage1_table_ok<P>()) {
        constexpr int r = P::radix(1), Ns = P::ns_before(1), off = stage_tw_offset<P>(1);
        for (int i = tid; i < r * Ns; i += nthreads) {
            const int e = i & 1, j = (i >> 1) % Ns, kp = (i >> 1) / Ns;
            const int k = 2 * kp + 1 + e;
            tab[i] = k < r ? MA_LDG(tws + off + (k - 1) * Ns + j) : make_float2(1.f, 0.f);
        }
    }
}

template <class P, int W, int S, bool PAIRED, bool TWALU, bool TWS1 = false>
MA_HD void stage_read_compute(float2* v, int t, const float2* sbuf,
                              const float2* __restrict__ twM, const float2* twb, const float2* tw_s1 = nullptr) {
    constexpr int M = P::M, r = P::radix(S), Ns = P::ns_before(S), NB = P::R / r;
    constexpr int stride = M / r;
    using A = ExchangeAddr<W, stride, r>;
#pragma unroll
    for (int b = 0; b < NB; ++b) {
        const int jv = stage_jv<P, PAIRED>(t, b, M / r);
        if constexpr (W != 1 || stride % 16 == 0) {
            const float2* src = sbuf + A::base(jv);
#pragma unroll
            for (int k = 0; k < r; ++k) v[b * r + k] = src[A::offset(k)];
        } else {
#pragma unroll
            for (int k = 0; k < r; ++k) v[b * r + k] = sbuf[saddr<W>(jv + k * stride)];
        }
        float2 w[r];
        if constexpr (TWS1 && S == 1 && stage1_table_ok<P>()) {
            const float4* tab = reinterpret_cast<const float4*>(tw_s1) + (jv % Ns);
#pragma unroll
            for (int kp = 0; kp < r / 2; ++kp) {
                const float4 w4 = tab[kp * Ns];
                w[2 * kp + 1] = make_float2(w4.x, w4.y);
                if (2 * kp + 2 < r) w[2 * kp + 2] = make_float2(w4.z, w4.w);
            }
        } else if constexpr (TWALU) twiddle_powers<r>(w, twb[tw_base_index<P>(S, b)]);
        else load_stage_twiddles<P, S>(w, twM, jv % Ns);
#pragma unroll
        for (int k = 1; k < r; ++k) v[b * r + k] = cmul(v[b * r + k], w[k]);
        Bfly<r>::run(v + b * r);
    }
}

template <class P, bool PAIRL, int S>
MA_HD void tw_bases_stage(float2* twb, int t, const float2* __restrict__ tws) {
    if constexpr (S < P::NS) {
        constexpr int r = P::radix(S), Ns = P::ns_before(S), NB = P::R / r;
#pragma unroll
        for (int b = 0; b < NB; ++b) {
            const int jv = stage_jv<P, (S == P::NS - 1) && PAIRL>(t, b, P::M / r);
            twb[tw_base_index<P>(S, b)] = MA_LDG(tws + stage_tw_offset<P>(S) + (jv % Ns));
        }
        tw_bases_stage<P, PAIRL, S + 1>(twb, t, tws);
    }
}

struct NoHook {
    MA_HD void operator()() const {}
};

template <class P, int W, int S, bool PAIR0, bool PAIRL, bool TWALU, class Cta, class Hook = NoHook,
          bool SINGLE = false, bool TWS1 = false>
struct StageChain {
    static MA_HD void run(float2* v, int t, float2* sbuf0, int buf_stride, int& parity,
                          const float2* __restrict__ twM, const float2* twb, Cta& cta, const Hook& hook = Hook(),
                          const float2* tw_s1 = nullptr) {
        if constexpr (S < P::NS) {
            // SINGLE: one exchange buffer only; a barrier before each write keeps it from
            // overtaking the previous exchange's reads (costs a barrier, saves a buffer).
            if constexpr (SINGLE) cta.sync();
            float2* sbuf = SINGLE ? sbuf0 : sbuf0 + parity * buf_stride;
            stage_write<P, W, S - 1, (S == 1) && PAIR0>(v, t, sbuf);
            cta.sync();
            if constexpr (S == 1) hook();  // every thread is past its reads of the frame's input
            stage_read_compute<P, W, S, (S == P::NS - 1) && PAIRL, TWALU, TWS1>(v, t, sbuf, twM, twb, tw_s1);
            parity ^= 1;
            StageChain<P, W, S + 1, PAIR0, PAIRL, TWALU, Cta, Hook, SINGLE, TWS1>::run(v, t, sbuf0, buf_stride, parity, twM, twb, cta, hook, tw_s1);
        }
    }
};

// Base twiddles (k = 1 entries of the stage tables) of this thread's butterflies, for the
// register-resident mode.
template <class P, bool PAIRL>
MA_HD void load_tw_bases(float2* twb, int t, const float2* __restrict__ tws) {
    twb[0] = make_float2(1.f, 0.f);
    tw_bases_stage<P, PAIRL, 1>(twb, t, tws);
}

// All stages of plan P on registers.
// In:  v[b*r0 + k] = z[jv0(b) + k*M/r0], r0 the first radix, jv0 natural or paired (PAIR0).
// Out: v[b*rl + k] = Z[jvl(b) + k*M/rl], rl the last radix, jvl natural or paired (PAIRL).
// sbuf0 is the transform's exchange region (already offset by the slot when W > 1);
// buf_stride is the distance in float2 between the two exchange buffers; parity selects the
// buffer of the next exchange and is updated.
// tw_s1 (with TWS1): the stage-1 twiddle table in shared memory (stage1_table_fill).
template <class P, int W, bool PAIR0, bool PAIRL, class Cta, bool TWALU = false, class Hook = NoHook,
          bool SINGLE = false, bool TWS1 = false>
MA_HD void fft_run(float2* v, int t, float2* sbuf0, int buf_stride, int& parity,
                   const float2* __restrict__ twM, Cta& cta, const float2* twb = nullptr,
                   const Hook& hook = Hook(), const float2* tw_s1 = nullptr) {
    constexpr int r0 = P::radix(0), NB0 = P::R / r0;
    static_assert(!(PAIRL && P::NS < 2), "a paired last stage needs at least two stages");
#pragma unroll
    for (int b = 0; b < NB0; ++b) Bfly<r0>::run(v + b * r0);  // stage 0: no twiddles
    StageChain<P, W, 1, PAIR0, PAIRL, TWALU, Cta, Hook, SINGLE, TWS1>::run(v, t, sbuf0, buf_stride, parity, twM, twb, cta, hook, tw_s1);
}

// Complex forward FFT of length M in natural order.  In: v[q] = z[t + q*T].
// Out: v[q] = Z[t + q*T].
// SINGLE: one exchange buffer (buf_stride is ignored), a barrier in front of every exchange write.
template <int M, int W, class Cta, bool SINGLE = false>
MA_HD void fft_forward_regs(float2* v, int t, float2* sbuf0, int buf_stride, int& parity,
                            const float2* __restrict__ twM, Cta& cta) {
    using P = FftPlan<M>;
    constexpr int R = P::R;
    fft_run<P, W, false, false, Cta, false, NoHook, SINGLE>(v, t, sbuf0, buf_stride, parity, twM, cta);
    // After the last stage, element (b, k) of the flat array is Z[t + (b + k*NB)*T].
    constexpr int rl = P::radix(P::NS - 1), NB = R / rl;
    if constexpr (NB > 1) {
        float2 tmp[R];
#pragma unroll
        for (int i = 0; i < R; ++i) tmp[i] = v[i];
#pragma unroll
        for (int b = 0; b < NB; ++b)
#pragma unroll
            for (int k = 0; k < rl; ++k) v[b + k * NB] = tmp[b * rl + k];
    }
}

}  // namespace ma
