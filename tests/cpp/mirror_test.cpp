// Exercises the C++ host mirror (include/MetalDSP.hpp) the way the reference's XCTest suites
// exercise the Swift API.  `--host-only` checks the host logic and the no-device behaviour
// (no GPU compute); without the flag it runs the known-answer tests on the GPU.
#include <cmath>
#include <cstdio>
#include <cstring>
#include <random>

#include "MetalDSP.hpp"

using namespace metalaudio;

static int failures = 0;
#define CHECK(cond)                                                      \
    do {                                                                 \
        if (!(cond)) {                                                   \
            std::printf("FAILED %s:%d: %s\n", __FILE__, __LINE__, #cond); \
            ++failures;                                                  \
        }                                                                \
    } while (0)

static void host_logic() {
    FFT::Config c(2048);
    CHECK(c.hopSize == 512 && c.windowType == WindowType::hann && !c.inverse);
    CHECK(FFT::Config(2).hopSize == 1);
    CHECK(FFT::Config(1024, false, WindowType::hann, 256).overlapPercent() == 75);
    CHECK(colaHopDivisors(WindowType::none) == std::vector<int>({1}));
    CHECK(colaHopDivisors(WindowType::hann) == std::vector<int>({2, 4}));
    CHECK(colaHopDivisors(WindowType::hamming).empty());
    CHECK(colaHopDivisors(WindowType::blackman) == std::vector<int>({3, 4}));
    CHECK(FFT::Config(2048, false, WindowType::hann, 512).colaCompliance() == COLACompliance::perfect);
    CHECK(FFT::Config(2048, false, WindowType::hann, 300).colaCompliance() == COLACompliance::nonCompliant);
    CHECK(FFT::Config(2048, false, WindowType::hamming, 512).colaCompliance() == COLACompliance::nearPerfect);
    auto v = FFT::Config(2048, false, WindowType::hann, 300).validateCOLA();
    CHECK(!v.first && v.second.find("1024 (50% overlap)") != std::string::npos);
    // symmetric window: w[i] == w[N-1-i] at N = 256, endpoints 0, centre ~1
    for (int i = 0; i < 256; ++i)
        CHECK(std::fabs(windowCoefficient(WindowType::hann, i, 256) - windowCoefficient(WindowType::hann, 255 - i, 256)) < 1e-5f);
    CHECK(windowCoefficient(WindowType::hann, 0, 256) == 0.f && windowCoefficient(WindowType::hann, 5, 1) == 1.f);
    CHECK(std::string(FFTError::inputTooShort(100, 256).what()).find("100") != std::string::npos);
    CHECK(std::string(FFTError::sizeNotPowerOf2(300).what()).find("300") != std::string::npos);
    CHECK(FFTError::invalidHopSize(0, 256).errorCase == "invalidHopSize");
    CHECK(ConvolutionError::emptyKernel().errorCase == "emptyKernel");
    // biquad coefficient design needs no device: DC gain 1 for a low-pass, zero at DC for a high-pass,
    // 0 dB peaking is an identity; validation errors name the parameter
    const auto lp = BiquadFilter::design(BiquadFilter::FilterType::lowpass(), 1000.f, 44100.f);
    CHECK(std::fabs((lp.b0 + lp.b1 + lp.b2) / (1.0 + lp.a1 + lp.a2) - 1.0) < 1e-4);
    const auto hp = BiquadFilter::design(BiquadFilter::FilterType::highpass(), 1000.f, 44100.f);
    CHECK(std::fabs(hp.b0 + hp.b1 + hp.b2) < 1e-6);
    const auto pk = BiquadFilter::design(BiquadFilter::FilterType::peaking(0.f), 1000.f, 44100.f);
    CHECK(std::fabs(pk.b0 - 1.f) < 1e-6f && std::fabs(pk.b1 - pk.a1) < 1e-6f && std::fabs(pk.b2 - pk.a2) < 1e-6f);
    bool caught = false;
    try {
        BiquadFilter::design(BiquadFilter::FilterType::lowpass(), 1000.f, 44100.f, 0.f);
    } catch (const FilterError& e) {
        caught = e.errorCase == "invalidParameter" && e.name == "q";
    }
    CHECK(caught);
    CHECK(std::string(FilterError::unstable("x").what()) == "Filter is unstable: x");
    // sampled output validation: off by default; a NaN on a sampled index and an Inf at the end are found
    std::vector<float> buf(1000, 0.f);
    buf[20] = std::nanf("");
    CHECK(!validateFFTOutput(buf.data(), 1000, "outputReal"));
    fftValidationEnabled() = true;
    CHECK(validateFFTOutput(buf.data(), 1000, "outputReal"));
    CHECK(fftValidationLog().back() == "[FFT] Warning: NaN detected in outputReal near index 20");
    std::vector<float> buf2(1000, 0.f);
    buf2[21] = INFINITY;
    CHECK(!validateFFTOutput(buf2.data(), 1000, "outputImag"));   // between two samples
    buf2[999] = INFINITY;
    CHECK(validateFFTOutput(buf2.data(), 1000, "outputImag"));
    fftValidationEnabled() = false;
}

static void no_device() {
    if (ma_device_count() > 0) return;
    bool threw = false;
    try {
        AudioDevice dev;
    } catch (const MetalAudioError& e) {
        threw = e.errorCase == "deviceNotFound";
    }
    CHECK(threw);
}

static double rel_rms(const std::vector<double>& a, const std::vector<double>& b) {
    double num = 0, den = 0;
    for (size_t i = 0; i < a.size(); ++i) {
        num += (a[i] - b[i]) * (a[i] - b[i]);
        den += b[i] * b[i];
    }
    return den > 0 ? std::sqrt(num / den) : std::sqrt(num);
}

static void gpu_tests() {
    {   // explicit-backend complex transform: a real impulse train as interleaved complex data
        AudioDevice dev;
        FFT fft(dev, FFT::Config(256, false, WindowType::none));
        std::vector<float> in(2 * 256 + 4, 0.f), out, back;
        in[2 * 3] = 1.f;                                   // delta at n = 3 -> X[k] = exp(-2 pi i 3k/256)
        CHECK(fft.forwardGPU(in, out) == Backend::cuda && out.size() == 512);
        for (int k = 0; k < 256; k += 17) {
            const double a = -2.0 * M_PI * 3.0 * k / 256.0;
            CHECK(std::fabs(out[2 * k] - std::cos(a)) < 1e-5 && std::fabs(out[2 * k + 1] - std::sin(a)) < 1e-5);
        }
        fft.inverseGPU(out, back);
        CHECK(std::fabs(back[6] - 1.f) < 1e-5f && std::fabs(back[8]) < 1e-5f && std::fabs(back[7]) < 1e-5f);
        bool threw = false;
        try { fft.forwardGPU(std::vector<float>(10), out); } catch (const MetalAudioError& e) { threw = e.errorCase == "bufferSizeMismatch"; }
        CHECK(threw);
        CHECK(!fft.shouldUseMetal() && !fft.shouldUseMPSGraph());
    }
    AudioDevice dev;
    std::printf("device: %s\n", dev.name().c_str());
    const int n = 1024;
    FFT fwd(dev, FFT::Config(n, false, WindowType::none));
    FFT inv(dev, FFT::Config(n, true, WindowType::none));
    std::vector<float> x(n, 0.f), re(n), im(n), y(n), mag(n / 2 + 1);
    x[0] = 1.f;  // impulse -> flat spectrum
    fwd.forward(x.data(), re.data(), im.data());
    for (int k = 0; k < n; ++k) CHECK(std::fabs(re[k] - 1.f) < 1e-6f && std::fabs(im[k]) < 1e-6f);
    std::fill(x.begin(), x.end(), 1.f);  // DC -> N at bin 0
    fwd.forward(x.data(), re.data(), im.data());
    CHECK(std::fabs(re[0] - n) < 1e-3f && std::fabs(re[5]) < 1e-3f);
    const int kbin = 37;  // sine at bin k peaks there with N/2
    for (int i = 0; i < n; ++i) x[i] = (float)std::sin(2.0 * M_PI * kbin * i / n);
    fwd.forward(x.data(), re.data(), im.data());
    fwd.magnitude(re.data(), im.data(), mag.data());
    int arg = 0;
    for (int k = 1; k <= n / 2; ++k)
        if (mag[k] > mag[arg]) arg = k;
    CHECK(arg == kbin && std::fabs(mag[kbin] - n / 2) < 1e-2f);
    std::mt19937 rng(7);
    std::normal_distribution<float> nd;
    for (auto& v : x) v = nd(rng);
    fwd.forward(x.data(), re.data(), im.data());
    inv.inverse(re.data(), im.data(), y.data());  // two-object round trip
    double err = 0;
    for (int i = 0; i < n; ++i) err = std::max(err, (double)std::fabs(y[i] - x[i]));
    CHECK(err < 1e-5);

    // STFT shape + reconstruction on the interior
    FFT st(dev, FFT::Config(512, false, WindowType::hann, 128));
    std::vector<float> sig(9000);
    for (auto& v : sig) v = nd(rng) * 0.3f;
    STFTResult r = st.stft(sig);
    CHECK(r.frameCount() == (9000 - 512) / 128 + 1 && r.binCount() == 512);
    std::vector<float> rec = st.istft(r);
    CHECK((int)rec.size() == (r.frameCount() - 1) * 128 + 512);
    std::vector<double> a, b;
    for (size_t i = 512; i + 512 < rec.size(); ++i) {
        a.push_back(rec[i]);
        b.push_back(sig[i]);
    }
    CHECK(rel_rms(a, b) < 1e-5);
    bool threw = false;
    try {
        st.stft(std::vector<float>(100));
    } catch (const FFTError& e) {
        threw = e.errorCase == "inputTooShort";
    }
    CHECK(threw);

    // partitioned convolution: delta kernel reproduces the input (ConvolutionTests identity row)
    Convolution conv(dev, Convolution::Mode::partitioned(64));
    conv.setKernel({1.0f});
    std::vector<float> ramp(256), out;
    for (int i = 0; i < 256; ++i) ramp[i] = i / 256.f;
    conv.process(ramp, out);
    CHECK(out.size() == 256);
    for (int i = 0; i < 256; ++i) CHECK(std::fabs(out[i] - ramp[i]) < 1e-4f);
    // short kernel against direct convolution
    std::vector<float> h = {0.5f, -0.25f, 0.125f, 0.0625f, 1.0f};
    Convolution c2(dev, Convolution::Mode::partitioned(16));
    c2.setKernel(h);
    std::vector<float> in(100), o2;
    for (auto& v : in) v = nd(rng);
    c2.process(in, o2);
    CHECK(o2.size() == 104 && c2.partitionCount() == 1);
    for (int i = 0; i < 104; ++i) {
        double acc = 0;
        for (int j = 0; j < 5; ++j)
            if (i - j >= 0 && i - j < 100) acc += (double)h[j] * in[i - j];
        CHECK(std::fabs(o2[i] - acc) < 1e-5);
    }
    threw = false;
    try {
        Convolution c3(dev, Convolution::Mode::partitioned(64));
        c3.setKernel({});
    } catch (const ConvolutionError& e) {
        threw = e.errorCase == "emptyKernel";
    }
    CHECK(threw);
    // .fft mode (the default): an impulse returns the kernel; oversize input is refused
    // (ConvolutionTests testFFTConvolutionImpulseResponse / InputSizeMismatchThrows)
    Convolution fc(dev);
    const std::vector<float> k4 = {1.0f, 0.5f, 0.25f, 0.125f};
    fc.setKernel(k4);
    std::vector<float> o4;
    fc.process({1.0f, 0.0f, 0.0f, 0.0f}, o4);
    CHECK(o4.size() == 8 && fc.fftSize() == 8 && fc.maxInputSize() == 4);
    for (int i = 0; i < 4; ++i) CHECK(std::fabs(o4[i] - k4[i]) < 1e-5f);
    fc.setKernel(k4, 64);
    threw = false;
    try {
        fc.process(std::vector<float>(128, 1.0f), o4);
    } catch (const ConvolutionError& e) {
        threw = e.errorCase == "inputSizeMismatch" && std::string(e.what()).find("circular convolution") != std::string::npos;
    }
    CHECK(threw);
    // magnitude / phase STFT and its inverse reproduce the signal away from the ends
    {
        FFT pf(dev, FFT::Config(1024, false, WindowType::hann, 256));
        std::vector<float> sig(16384), mg, ph;
        for (auto& v : sig) v = nd(rng);
        pf.stftPolar(sig, mg, ph);
        CHECK(mg.size() == (size_t)((16384 - 1024) / 256 + 1) * 513 && ph.size() == mg.size());
        const std::vector<float> back = pf.istftPolar(mg, ph);
        double err = 0, ref = 0;
        for (size_t i = 1024; i + 1024 < back.size(); ++i) {
            err += (back[i] - sig[i]) * (double)(back[i] - sig[i]);
            ref += sig[i] * (double)sig[i];
        }
        CHECK(std::sqrt(err / ref) < 1e-5);
    }
    // biquad: unity DC gain of a low-pass, streaming equals one call, filter bank of 0 dB bands is an identity
    {
        BiquadFilter lp(dev);
        lp.configure(BiquadFilter::FilterType::lowpass(), 1000.0f, 44100.0f, 0.707f);
        const std::vector<float> ones(20000, 1.0f);
        const std::vector<float> y = lp.process(ones);
        CHECK(std::fabs(y.back() - 1.0f) < 1e-4f && lp.isStable());
        lp.reset();
        std::vector<float> parts = lp.process(std::vector<float>(ones.begin(), ones.begin() + 9000));
        const std::vector<float> rest = lp.process(std::vector<float>(ones.begin() + 9000, ones.end()));
        parts.insert(parts.end(), rest.begin(), rest.end());
        for (size_t i = 0; i < y.size(); i += 97) CHECK(std::fabs(parts[i] - y[i]) < 1e-5f);
        threw = false;
        try {
            lp.configure(BiquadFilter::FilterType::lowpass(), 30000.0f, 44100.0f);
        } catch (const FilterError& e) {
            threw = e.errorCase == "invalidParameter" && e.name == "frequency";
        }
        CHECK(threw);
        FilterBank bank(dev, 5);
        bank.configureAsEQ(100.0f, 10000.0f, 44100.0f);
        std::vector<float> noise(5000);
        for (auto& v : noise) v = nd(rng);
        const std::vector<float> flat = bank.processSeries(noise), par = bank.processParallel(noise);
        for (size_t i = 0; i < noise.size(); i += 13) {
            CHECK(std::fabs(flat[i] - noise[i]) < 1e-4f);
            CHECK(std::fabs(par[i] - noise[i]) < 1e-4f);
        }
    }
    dev.markDeviceLost();
    threw = false;
    try {
        dev.ensureAvailable();
    } catch (const MetalAudioError& e) {
        threw = e.errorCase == "deviceLost";
    }
    CHECK(threw);
}

int main(int argc, char** argv) {
    const bool host_only = argc > 1 && std::strcmp(argv[1], "--host-only") == 0;
    host_logic();
    if (host_only) no_device();
    else gpu_tests();
    std::printf(failures ? "%d FAILURES\n" : "OK\n", failures);
    return failures ? 1 : 0;
}
