// MetalDSP.hpp - C++ host-side mirror of the reference's public Swift API for the DSP hot path,
// over the C ABI of metalaudio_cuda.h.  Header-only; link with -lmetalaudio_cuda.
//
// The reference is a Swift package; where a Swift toolchain exists the same calls are made from
// Swift through a system-library module.  This header gives compiled-language callers the same
// surface: names, argument meaning and error behaviour follow
//   AudioDevice                         Sources/MetalAudioKit/Core/AudioDevice.swift:222, :323, :434, :733
//   Tensor                              Sources/MetalAudioKit/Buffers/Tensor.swift:59, :272, :325
//   FFT, FFT::Config, WindowType, COLA  Sources/MetalDSP/FFT.swift:12-55, :155-348, :441-495, :818-919, :1780-1847
//   FFT::stft / istft / batches         Sources/MetalDSP/STFT.swift:10-22, :40-128, :327-527
//   Convolution (.fft, .partitioned)    Sources/MetalDSP/Convolution.swift:8-47, :112-125, :176-383, :437-493, :529-775
//   BiquadFilter, FilterBank            Sources/MetalDSP/Filters.swift:14-26, :65-96, :226-490, :515-716, :736-873
//   stftPolar / istftPolar              the magnitude / phase split and rebuild of Sources/MetalNN/HTDemucs.swift:726-741, :795-812
// Swift `throws` becomes C++ exceptions carrying the Swift case name and the same description.
// There is one backend (CUDA) and no CPU fallback.
#pragma once

#include <cmath>
#include <cstdint>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

#include "metalaudio_cuda.h"

namespace metalaudio {

// ------------------------------------------------------------------------------ errors
struct MetalAudioError : std::runtime_error {
    std::string errorCase;
    MetalAudioError(std::string c, const std::string& msg) : std::runtime_error(msg), errorCase(std::move(c)) {}
};

struct FFTError : std::runtime_error {
    std::string errorCase;
    FFTError(std::string c, const std::string& msg) : std::runtime_error(msg), errorCase(std::move(c)) {}
    static FFTError inputTooShort(int64_t inputSize, int64_t requiredSize) {
        return FFTError("inputTooShort", "Input size " + std::to_string(inputSize) +
                                             " is shorter than the required FFT size " + std::to_string(requiredSize) +
                                             ". Provide at least " + std::to_string(requiredSize) +
                                             " samples, or use a smaller FFT size.");
    }
    static FFTError sizeTooLarge(int64_t requested, int64_t maxSize) {
        return FFTError("sizeTooLarge", "FFT size " + std::to_string(requested) + " exceeds maximum supported size " +
                                            std::to_string(maxSize) + ".");
    }
    static FFTError sizeNotPowerOf2(int64_t size) {
        return FFTError("sizeNotPowerOf2", "FFT size " + std::to_string(size) +
                                               " is not a power of 2. Use sizes like 256, 512, 1024, 2048, etc.");
    }
    static FFTError invalidHopSize(int64_t hop, int64_t fftSize) {
        return FFTError("invalidHopSize", "Hop size " + std::to_string(hop) + " is invalid. Must be > 0 and <= FFT size (" +
                                              std::to_string(fftSize) + ").");
    }
    static FFTError istftOutputOverflow(int64_t frames, int64_t hop, int64_t fftSize) {
        return FFTError("istftOutputOverflow", "ISTFT output length calculation overflowed: frameCount=" +
                                                   std::to_string(frames) + ", hopSize=" + std::to_string(hop) +
                                                   ", fftSize=" + std::to_string(fftSize) +
                                                   ". Use smaller STFT result or process in chunks.");
    }
};

struct ConvolutionError : std::runtime_error {
    std::string errorCase;
    ConvolutionError(std::string c, const std::string& msg) : std::runtime_error(msg), errorCase(std::move(c)) {}
    static ConvolutionError emptyKernel() {
        return ConvolutionError("emptyKernel", "Convolution kernel cannot be empty. Provide at least one sample.");
    }
    static ConvolutionError fftNotInitialized() {
        return ConvolutionError("fftNotInitialized",
                                "FFT resources failed to initialize. This may indicate a Metal device error.");
    }
    static ConvolutionError inputSizeMismatch(int64_t inputSize, int64_t expectedMaxSize, int64_t fftSize) {
        return ConvolutionError("inputSizeMismatch",
                                "Convolution input size " + std::to_string(inputSize) + " exceeds expected maximum " +
                                    std::to_string(expectedMaxSize) + " (FFT size: " + std::to_string(fftSize) +
                                    "). This would cause circular convolution artifacts. Call setKernel() with a larger "
                                    "expectedInputSize parameter.");
    }
    static ConvolutionError outputSizeOverflow(int64_t inputSize, int64_t kernelSize) {
        return ConvolutionError("outputSizeOverflow", "Output size would overflow: input (" + std::to_string(inputSize) +
                                                          ") + kernel (" + std::to_string(kernelSize) +
                                                          ") - 1 exceeds Int.max. Use smaller buffers or process in chunks.");
    }
};

inline void throwStatus(ma_status st, const char* where) {
    if (st == MA_OK) return;
    const std::string text = std::string(where) + ": " + ma_status_string(st);
    switch (st) {
        case MA_ERR_DEVICE_LOST: throw MetalAudioError("deviceLost", text);
        case MA_ERR_TIMEOUT: throw MetalAudioError("gpuTimeout", text);
        case MA_ERR_ALLOC: throw MetalAudioError("bufferAllocationFailed", text);
        case MA_ERR_CUDA: throw MetalAudioError("gpuExecutionError", text + " (cudaError " + std::to_string(ma_last_cuda_error()) + ")");
        case MA_ERR_KERNEL_NOT_CONFIGURED: throw ConvolutionError::fftNotInitialized();
        default: throw MetalAudioError("invalidConfiguration", text);
    }
}

// ------------------------------------------------------------------------------ device / tensor
class AudioDevice {
public:
    explicit AudioDevice(int deviceIndex = 0, size_t pinnedBytes = 0) {
        const ma_status st = ma_context_create(deviceIndex, pinnedBytes, &ctx_);
        if (st == MA_ERR_DEVICE_LOST)
            throw MetalAudioError("deviceNotFound", "No CUDA device found; this library has no CPU fallback");
        throwStatus(st, "AudioDevice()");
    }
    ~AudioDevice() { ma_context_destroy(ctx_); }
    AudioDevice(const AudioDevice&) = delete;
    AudioDevice& operator=(const AudioDevice&) = delete;

    ma_context* handle() const { return ctx_; }
    std::string name() const {
        char buf[256];
        ma_context_device_name(ctx_, buf, sizeof buf);
        return buf;
    }
    bool isDeviceAvailable() const {
        int32_t v = 0;
        ma_context_is_available(ctx_, &v);
        return v != 0;
    }
    void markDeviceLost() { ma_context_mark_lost(ctx_); }
    void ensureAvailable() const {
        if (!isDeviceAvailable()) throw MetalAudioError("deviceLost", "GPU device was lost");
    }
    // ComputeContext.executeSync's wait; default timeout 2 s (ComputeContext.swift:137)
    void synchronize(double timeout = 2.0) { throwStatus(ma_context_sync(ctx_, timeout), "synchronize"); }
    void timingBegin() { throwStatus(ma_timing_begin(ctx_), "timingBegin"); }
    float timingEnd() {
        float ms = 0;
        throwStatus(ma_timing_end(ctx_, &ms), "timingEnd");
        return ms;
    }

private:
    ma_context* ctx_ = nullptr;
};

class Tensor {
public:
    Tensor(AudioDevice& device, std::vector<int64_t> shape) : device_(device), shape_(std::move(shape)) {
        count_ = 1;
        for (int64_t d : shape_) count_ *= d;
        throwStatus(ma_buffer_alloc(device_.handle(), (size_t)count_ * sizeof(float), &ptr_), "Tensor()");
    }
    ~Tensor() { ma_buffer_free(device_.handle(), ptr_); }
    Tensor(const Tensor&) = delete;
    Tensor& operator=(const Tensor&) = delete;

    int64_t count() const { return count_; }
    const std::vector<int64_t>& shape() const { return shape_; }
    float* devicePointer() const { return static_cast<float*>(ptr_); }
    void copy(const std::vector<float>& from) {
        if ((int64_t)from.size() != count_) throw MetalAudioError("bufferSizeMismatch", "Tensor.copy(from:) size mismatch");
        throwStatus(ma_memcpy_h2d(device_.handle(), ptr_, from.data(), from.size() * sizeof(float)), "Tensor.copy");
    }
    std::vector<float> toArray() const {
        std::vector<float> out((size_t)count_);
        throwStatus(ma_memcpy_d2h(device_.handle(), out.data(), ptr_, out.size() * sizeof(float)), "Tensor.toArray");
        return out;
    }
    void zero() { throwStatus(ma_buffer_zero(device_.handle(), ptr_, (size_t)count_ * sizeof(float)), "Tensor.zero"); }

private:
    AudioDevice& device_;
    std::vector<int64_t> shape_;
    int64_t count_ = 0;
    void* ptr_ = nullptr;
};

// ------------------------------------------------------------------------------ FFT
enum class WindowType { none, hann, hamming, blackman };
enum class COLACompliance { perfect, nearPerfect, nonCompliant };
enum class Backend { vdsp, gpu, mpsGraph, cuda };

// Symmetric window coefficient (denominator N-1) evaluated in double (FFT.swift:268-294).
inline float windowCoefficient(WindowType w, int index, int length) {
    if (length <= 1) return 1.0f;
    const double n = index, denom = (double)length - 1.0;
    switch (w) {
        case WindowType::none: return 1.0f;
        case WindowType::hann: return (float)(0.5 * (1.0 - std::cos(2.0 * M_PI * n / denom)));
        case WindowType::hamming: return (float)(0.54 - 0.46 * std::cos(2.0 * M_PI * n / denom));
        default:
            return (float)(0.42 - 0.5 * std::cos(2.0 * M_PI * n / denom) + 0.08 * std::cos(4.0 * M_PI * n / denom));
    }
}
inline std::vector<int> colaHopDivisors(WindowType w) {
    switch (w) {
        case WindowType::none: return {1};
        case WindowType::hann: return {2, 4};
        case WindowType::hamming: return {};
        default: return {3, 4};
    }
}
inline const char* windowName(WindowType w) {
    switch (w) {
        case WindowType::none: return "rectangular";
        case WindowType::hann: return "Hann";
        case WindowType::hamming: return "Hamming";
        default: return "Blackman";
    }
}

struct STFTResult {  // STFT.swift:10-22: full-N split rows
    std::vector<std::vector<float>> real, imag;
    int frameCount() const { return (int)real.size(); }
    int binCount() const { return real.empty() ? 0 : (int)real[0].size(); }
};

// FFT.swift:63-134: sampled NaN / Inf check on transform outputs, off unless the flag is set.  Looks
// at about 50 evenly spaced values plus the last one, reports the first of each kind, never throws.
inline bool& fftValidationEnabled() {
    static bool enabled = false;
    return enabled;
}
inline std::vector<std::string>& fftValidationLog() {
    static std::vector<std::string> log;
    return log;
}
inline bool validateFFTOutput(const float* buffer, int64_t count, const std::string& context) {
    if (!fftValidationEnabled() || count <= 0) return false;
    const int64_t sampleCount = count < 50 ? count : 50;
    const int64_t stride = std::max<int64_t>(1, count / sampleCount);
    int64_t nanAt = -1, infAt = -1;
    for (int64_t i = 0; i < count && (nanAt < 0 || infAt < 0); i += stride) {
        if (nanAt < 0 && std::isnan(buffer[i])) nanAt = i;
        if (infAt < 0 && std::isinf(buffer[i])) infAt = i;
    }
    if (count > 1) {
        if (nanAt < 0 && std::isnan(buffer[count - 1])) nanAt = count - 1;
        if (infAt < 0 && std::isinf(buffer[count - 1])) infAt = count - 1;
    }
    if (nanAt >= 0) fftValidationLog().push_back("[FFT] Warning: NaN detected in " + context + " near index " + std::to_string(nanAt));
    if (infAt >= 0) fftValidationLog().push_back("[FFT] Warning: Inf detected in " + context + " near index " + std::to_string(infAt));
    return nanAt >= 0 || infAt >= 0;
}

class FFT {
public:
    static constexpr int maxFFTSize = 1 << 24;  // FFT.swift:422

    struct Config {  // FFT.swift:158-258
        int size;
        bool inverse = false;
        WindowType windowType = WindowType::hann;
        int hopSize;
        Config(int size_, bool inverse_ = false, WindowType w = WindowType::hann, int hop = -1)
            : size(size_), inverse(inverse_), windowType(w), hopSize(hop > 0 ? hop : std::max(1, size_ / 4)) {}

        COLACompliance colaCompliance() const {
            const auto divs = colaHopDivisors(windowType);
            if (divs.empty()) {
                if (windowType == WindowType::hamming && (hopSize == size / 2 || hopSize == size / 4))
                    return COLACompliance::nearPerfect;
                return COLACompliance::nonCompliant;
            }
            for (int d : divs)
                if (size % d == 0 && hopSize == size / d) return COLACompliance::perfect;
            return COLACompliance::nonCompliant;
        }
        int overlapPercent() const { return 100 - (hopSize * 100 / size); }
        std::pair<bool, std::string> validateCOLA() const {
            const std::string w = windowName(windowType);
            switch (colaCompliance()) {
                case COLACompliance::perfect:
                    return {true, w + " window with hop size " + std::to_string(hopSize) + " (overlap " +
                                      std::to_string(overlapPercent()) + "%) satisfies COLA"};
                case COLACompliance::nearPerfect:
                    return {true, w + " window with hop size " + std::to_string(hopSize) + " is near-COLA (error < 0.1%)"};
                default: {
                    std::string hops;
                    for (int d : colaHopDivisors(windowType))
                        if (size % d == 0) {
                            const int hop = size / d;
                            if (!hops.empty()) hops += ", ";
                            hops += std::to_string(hop) + " (" + std::to_string(100 - (hop * 100 / size)) + "% overlap)";
                        }
                    const std::string sug = hops.empty() ? "Consider using Hann window for COLA-compliant STFT"
                                                         : "Suggested hop sizes: " + hops;
                    return {false, w + " window with hop size " + std::to_string(hopSize) + " does not satisfy COLA. " + sug};
                }
            }
        }
    };

    FFT(AudioDevice& device, const Config& config) : device_(device), config_(config) {
        const int n = config.size;
        if (n <= 0 || (n & (n - 1)) != 0) throw FFTError::sizeNotPowerOf2(n);  // order of FFT.swift:443-455
        if (n > maxFFTSize) throw FFTError::sizeTooLarge(n, maxFFTSize);
        if (config.hopSize <= 0 || config.hopSize > n) throw FFTError::invalidHopSize(config.hopSize, n);
        window_.resize((size_t)n);
        for (int i = 0; i < n; ++i) window_[(size_t)i] = windowCoefficient(config.windowType, i, n);
        throwStatus(ma_fft_plan_create(device.handle(), n, config.windowType == WindowType::none ? nullptr : window_.data(),
                                       config.hopSize, &plan_),
                    "FFT.init");
    }
    ~FFT() { ma_fft_plan_destroy(plan_); }
    FFT(const FFT&) = delete;
    FFT& operator=(const FFT&) = delete;

    int size() const { return config_.size; }
    const std::vector<float>& window() const { return window_; }

private:
    Backend complexTransform(const std::vector<float>& input, std::vector<float>& output, int inverse) {
        const size_t n2 = 2 * (size_t)config_.size;
        if (input.size() < n2)
            throw MetalAudioError("bufferSizeMismatch", "Buffer size mismatch: expected " + std::to_string(n2) +
                                                            " bytes, got " + std::to_string(input.size()));
        output.assign(n2, 0.f);
        throwStatus(ma_fft_complex_host(plan_, input.data(), output.data(), 1, inverse), inverse ? "inverseGPU" : "forwardGPU");
        return Backend::cuda;
    }

public:
    Backend optimalBackend() const { return Backend::cuda; }
    bool shouldUseGPU() const { return true; }
    // FFT.swift:1522-1539: the reference's size classes, kept as queries (one backend serves all).
    bool shouldUseMetal() const { return config_.size > 2048 && config_.size <= 8192; }
    bool shouldUseMPSGraph() const { return config_.size > 8192; }

    // FFT.swift:945-1107, :1176-1315: complex transform of N interleaved (re, im) pairs, forward
    // unscaled / inverse with 1/N.  Short inputs throw bufferSizeMismatch, longer ones are
    // truncated, the output is resized to 2N.
    Backend forwardGPU(const std::vector<float>& input, std::vector<float>& output) { return complexTransform(input, output, 0); }
    Backend inverseGPU(const std::vector<float>& input, std::vector<float>& output) { return complexTransform(input, output, 1); }

    // FFT.swift:818-855.  Non-throwing pointer API: outputs are zeroed on failure.  Direction
    // follows Config::inverse (one setup serves both methods in the reference).
    void forward(const float* input, float* outputReal, float* outputImag) {
        const int n = config_.size;
        const ma_status st = ma_fft_forward_host(plan_, input, outputReal, outputImag, nullptr, 0, 1.0f, 1, MA_LAYOUT_FULL_SPLIT);
        if (st != MA_OK) {
            for (int i = 0; i < n; ++i) outputReal[i] = outputImag[i] = 0.f;
            return;
        }
        if (config_.inverse)
            for (int i = 0; i < n; ++i) outputImag[i] = -outputImag[i];
        validateFFTOutput(outputReal, n, "outputReal");  // FFT.swift:853-854
        validateFFTOutput(outputImag, n, "outputImag");
    }
    // FFT.swift:889-919: real part of the transform in the object's direction, times 1/N.
    void inverse(const float* inputReal, const float* inputImag, float* output) {
        const int n = config_.size;
        const ma_status st = ma_fft_inverse_host(plan_, inputReal, inputImag, output, 1, MA_LAYOUT_FULL_SPLIT);
        if (st != MA_OK) {
            for (int i = 0; i < n; ++i) output[i] = 0.f;
            return;
        }
        if (!config_.inverse)  // a forward-configured object returns the time-reversed sequence
            for (int i = 1, j = n - 1; i < j; ++i, --j) std::swap(output[i], output[j]);
    }
    void magnitude(const float* real, const float* imag, float* out) { mag(real, imag, out, MA_MAG_MAGNITUDE, 1.0f); }
    void power(const float* real, const float* imag, float* out) { mag(real, imag, out, MA_MAG_POWER, 1.0f); }
    void magnitudeDB(const float* real, const float* imag, float* out, float reference = 1.0f) {
        mag(real, imag, out, MA_MAG_DB, reference);
    }

    int64_t frameCount(int64_t inputLength) const {
        if (inputLength < config_.size) throw FFTError::inputTooShort(inputLength, config_.size);
        return (inputLength - config_.size) / config_.hopSize + 1;
    }

    // STFT.swift:40-81
    STFTResult stft(const std::vector<float>& input) {
        const int n = config_.size;
        const int64_t f = frameCount((int64_t)input.size());
        std::vector<float> re((size_t)f * n), im((size_t)f * n);
        throwStatus(ma_stft_host(plan_, input.data(), (int64_t)input.size(), (int64_t)input.size(), 1, re.data(), im.data(),
                                 nullptr, 0, 1.0f, MA_LAYOUT_FULL_SPLIT),
                    "stft");
        STFTResult r;
        r.real.resize((size_t)f);
        r.imag.resize((size_t)f);
        for (int64_t i = 0; i < f; ++i) {
            r.real[(size_t)i].assign(re.begin() + i * n, re.begin() + (i + 1) * n);
            r.imag[(size_t)i].assign(im.begin() + i * n, im.begin() + (i + 1) * n);
        }
        return r;
    }

    // STFT.swift:384-527, with the true inverse transform per frame.
    std::vector<float> istft(const STFTResult& s, float windowFloorEpsilon = 1e-8f) {
        const int64_t f = s.frameCount();
        if (f == 0) return {};
        const int n = config_.size;
        int64_t outLen = 0;
        if (ma_istft_output_length(plan_, f, &outLen) != MA_OK) throw FFTError::istftOutputOverflow(f, config_.hopSize, n);
        std::vector<float> re((size_t)f * n), im((size_t)f * n), out((size_t)outLen);
        for (int64_t i = 0; i < f; ++i) {
            std::copy(s.real[(size_t)i].begin(), s.real[(size_t)i].begin() + n, re.begin() + i * n);
            std::copy(s.imag[(size_t)i].begin(), s.imag[(size_t)i].begin() + n, im.begin() + i * n);
        }
        float floor = windowFloorEpsilon;  // validated as STFT.swift:491-501
        if (floor < 1e-10f) floor = 1e-6f;
        else if (floor > 0.1f) floor = 0.1f;
        throwStatus(ma_istft_host(plan_, re.data(), im.data(), f, 1, out.data(), outLen, floor, MA_LAYOUT_FULL_SPLIT), "istft");
        return out;
    }

    // STFT straight to magnitude and phase, frames x (N/2+1) each, row-major: the split the
    // reference's STFT consumer does on the host (HTDemucs.swift:726-741), fused into the transform.
    void stftPolar(const std::vector<float>& input, std::vector<float>& magnitude, std::vector<float>& phase) {
        const int64_t f = frameCount((int64_t)input.size());
        const size_t count = (size_t)f * (size_t)(config_.size / 2 + 1);
        magnitude.resize(count);
        phase.resize(count);
        throwStatus(ma_stft_host(plan_, input.data(), (int64_t)input.size(), (int64_t)input.size(), 1, magnitude.data(),
                                 phase.data(), nullptr, 0, 1.0f, MA_LAYOUT_HALF_POLAR),
                    "stftPolar");
    }

    // iSTFT from magnitude and phase (polar rebuild + conjugate mirror of HTDemucs.swift:795-812, fused).
    std::vector<float> istftPolar(const std::vector<float>& magnitude, const std::vector<float>& phase,
                                  float windowFloorEpsilon = 1e-8f) {
        const int64_t kh = config_.size / 2 + 1;
        const int64_t f = (int64_t)magnitude.size() / kh;
        if (f == 0) return {};
        if (phase.size() != magnitude.size()) throw MetalAudioError("invalidConfiguration", "magnitude and phase sizes differ");
        int64_t outLen = 0;
        if (ma_istft_output_length(plan_, f, &outLen) != MA_OK) throw FFTError::istftOutputOverflow(f, config_.hopSize, config_.size);
        std::vector<float> out((size_t)outLen);
        float floor = windowFloorEpsilon;
        if (floor < 1e-10f) floor = 1e-6f;
        else if (floor > 0.1f) floor = 0.1f;
        throwStatus(ma_istft_host(plan_, magnitude.data(), phase.data(), f, 1, out.data(), outLen, floor, MA_LAYOUT_HALF_POLAR),
                    "istftPolar");
        return out;
    }

    // STFT.swift:94-128 / :327-373 on flat row-major batches.
    void forwardBatch(const std::vector<float>& inputs, int batch, std::vector<float>& outReal, std::vector<float>& outImag) {
        const int n = config_.size;
        if (batch == 0) return;
        if ((int64_t)inputs.size() < (int64_t)batch * n) throw FFTError::inputTooShort((int64_t)inputs.size() / std::max(1, batch), n);
        outReal.resize((size_t)batch * n);
        outImag.resize((size_t)batch * n);
        throwStatus(ma_fft_forward_host(plan_, inputs.data(), outReal.data(), outImag.data(), nullptr, 0, 1.0f, batch,
                                        MA_LAYOUT_FULL_SPLIT),
                    "forwardBatch");
    }
    void inverseBatch(const std::vector<float>& inReal, const std::vector<float>& inImag, int batch, std::vector<float>& out) {
        if (batch == 0) return;
        out.resize((size_t)batch * config_.size);
        throwStatus(ma_fft_inverse_host(plan_, inReal.data(), inImag.data(), out.data(), batch, MA_LAYOUT_FULL_SPLIT),
                    "inverseBatch");
    }

    ma_fft_plan* handle() const { return plan_; }

private:
    void mag(const float* real, const float* imag, float* out, int kind, float reference) {
        throwStatus(ma_fft_magnitude_host(plan_, real, imag, out, 1, kind, reference), "magnitude");
    }
    AudioDevice& device_;
    Config config_;
    std::vector<float> window_;
    ma_fft_plan* plan_ = nullptr;
};

// ------------------------------------------------------------------------------ convolution
class Convolution {
public:
    struct Mode {  // Convolution.swift:112-125; .fft and .partitioned are served, .direct is not
        enum Kind { kFFT, kPartitioned } kind;
        int blockSize;
        bool useMPSGraphFFT;
        static Mode fft() { return Mode{kFFT, 0, false}; }
        static Mode partitioned(int blockSize, bool useMPSGraphFFT = false) { return Mode{kPartitioned, blockSize, useMPSGraphFFT}; }
    };

    explicit Convolution(AudioDevice& device, Mode mode = Mode::fft(), int channels = 1)
        : device_(device), mode_(mode), channels_(channels) {}
    ~Convolution() {
        ma_pconv_destroy(pc_);
        ma_fftconv_destroy(fc_);
    }
    Convolution(const Convolution&) = delete;
    Convolution& operator=(const Convolution&) = delete;

    // Convolution.swift:188-208 -> :210-248 (.fft) or :250-322 (.partitioned).  expectedInputSize
    // (.fft only) defaults to the kernel length, as in the reference.
    void setKernel(const std::vector<float>& kernel, int64_t expectedInputSize = -1) {
        if (kernel.empty()) throw ConvolutionError::emptyKernel();
        if (mode_.kind == Mode::kFFT) {
            const int64_t expected = expectedInputSize < 0 ? (int64_t)kernel.size() : expectedInputSize;
            ma_fftconv_destroy(fc_);
            fc_ = nullptr;
            const ma_status st = ma_fftconv_create(device_.handle(), kernel.data(), (int64_t)kernel.size(), expected, channels_, &fc_);
            if (st == MA_ERR_SIZE_TOO_LARGE) throw FFTError::sizeTooLarge(expected + (int64_t)kernel.size() - 1, 1 << 24);
            throwStatus(st, "setKernel");
            ma_fftconv_fft_size(fc_, &fftSize_);
            expected_ = expected;
            taps_ = (int64_t)kernel.size();
            return;
        }
        if (mode_.blockSize <= 0)
            throw MetalAudioError("invalidConfiguration", "Block size must be positive, got " + std::to_string(mode_.blockSize));
        if ((mode_.blockSize & (mode_.blockSize - 1)) != 0) throw FFTError::sizeNotPowerOf2(2 * mode_.blockSize);
        if (pc_ == nullptr) throwStatus(ma_pconv_create(device_.handle(), mode_.blockSize, channels_, &pc_), "setKernel");
        throwStatus(ma_pconv_set_kernels(pc_, kernel.data(), (int64_t)kernel.size(), 1, nullptr), "setKernel");
        taps_ = (int64_t)kernel.size();
    }
    int64_t kernelTailLength() const { return taps_ > 0 ? taps_ - 1 : 0; }
    int64_t expectedOutputSize(int64_t inputSize) const { return taps_ > 0 ? inputSize + taps_ - 1 : inputSize; }
    int64_t maxInputSize() const { return mode_.kind == Mode::kFFT ? expected_ : 0; }  // Convolution.swift:377-383
    int64_t fftSize() const { return fftSize_; }
    int partitionCount() const {
        int32_t p = 0;
        if (pc_) ma_pconv_partition_count(pc_, &p);
        return p;
    }

    // Convolution.swift:336-352.  .partitioned (-> :529-758): channels x L in, channels x (L+K-1)
    // out (row-major).  .fft (-> :437-493): fftSize samples per signal, a smaller output is
    // replaced, a larger one keeps its tail.
    void process(const std::vector<float>& input, std::vector<float>& output) {
        if (input.empty()) {
            output.clear();
            return;
        }
        if (mode_.kind == Mode::kFFT) {
            if (fc_ == nullptr) throw ConvolutionError::fftNotInitialized();
            const int64_t len = (int64_t)input.size() / channels_;
            if (len > expected_) throw ConvolutionError::inputSizeMismatch(len, expected_, fftSize_);
            if ((int64_t)output.size() < fftSize_ * channels_) output.assign((size_t)(fftSize_ * channels_), 0.f);
            throwStatus(ma_fftconv_process_host(fc_, input.data(), len, len, channels_, output.data()), "process");
            return;
        }
        if (pc_ == nullptr) throw ConvolutionError::fftNotInitialized();
        const int64_t len = (int64_t)input.size() / channels_;
        const int64_t full = len + taps_ - 1;
        if ((int64_t)output.size() < full * channels_) output.assign((size_t)(full * channels_), 0.f);
        else std::fill(output.begin(), output.end(), 0.f);
        throwStatus(ma_pconv_process_host(pc_, input.data(), len, len, output.data(), full), "process");
    }
    void reset() {
        if (pc_) throwStatus(ma_pconv_reset(pc_), "reset");
    }

private:
    AudioDevice& device_;
    Mode mode_;
    int channels_;
    int64_t taps_ = 0, expected_ = 0, fftSize_ = 0;
    ma_pconv* pc_ = nullptr;
    ma_fftconv* fc_ = nullptr;
};

// ------------------------------------------------------------------------------ filters

struct FilterError : std::runtime_error {  // Filters.swift:14-26
    std::string errorCase, name;
    float value = 0.f;
    FilterError(std::string c, const std::string& msg, std::string n = "", float v = 0.f)
        : std::runtime_error(msg), errorCase(std::move(c)), name(std::move(n)), value(v) {}
    static FilterError unstable(const std::string& reason) { return FilterError("unstable", "Filter is unstable: " + reason); }
    static FilterError invalidParameter(const std::string& name, float value, const std::string& requirement) {
        return FilterError("invalidParameter",
                           "Invalid parameter '" + name + "' with value " + std::to_string(value) + ": " + requirement, name, value);
    }
};

class BiquadFilter {
public:
    enum class Kind { lowpass, highpass, bandpass, notch, allpass, peaking, lowshelf, highshelf };
    struct FilterType {  // Filters.swift:68-77
        Kind kind;
        float gainDB;
        static FilterType lowpass() { return {Kind::lowpass, 0.f}; }
        static FilterType highpass() { return {Kind::highpass, 0.f}; }
        static FilterType bandpass() { return {Kind::bandpass, 0.f}; }
        static FilterType notch() { return {Kind::notch, 0.f}; }
        static FilterType allpass() { return {Kind::allpass, 0.f}; }
        static FilterType peaking(float gainDB) { return {Kind::peaking, gainDB}; }
        static FilterType lowshelf(float gainDB) { return {Kind::lowshelf, gainDB}; }
        static FilterType highshelf(float gainDB) { return {Kind::highshelf, gainDB}; }
    };
    struct Coefficients {  // Filters.swift:80-96: a0 divided out, identity by default
        float b0 = 1.f, b1 = 0.f, b2 = 0.f, a1 = 0.f, a2 = 0.f;
    };

    explicit BiquadFilter(AudioDevice& device, int channels = 1) : device_(device), channels_(channels) {
        throwStatus(ma_biquad_create(device.handle(), channels, 1, &bq_), "BiquadFilter");
        upload();
    }
    ~BiquadFilter() { ma_biquad_destroy(bq_); }
    BiquadFilter(const BiquadFilter&) = delete;
    BiquadFilter& operator=(const BiquadFilter&) = delete;

    // Coefficient design and validation in the order of Filters.swift:346-482 (double precision
    // cookbook forms, rounded to float after the division by a0).
    static Coefficients design(FilterType type, float frequency, float sampleRate, float q = 0.7071067811865476f) {
        if (!(sampleRate > 0)) throw FilterError::invalidParameter("sampleRate", sampleRate, "must be > 0");
        const float nyquist = sampleRate / 2.0f;
        if (!(frequency > 0 && frequency < nyquist))
            throw FilterError::invalidParameter("frequency", frequency, "must be > 0 and < " + std::to_string(nyquist) + " Hz (Nyquist)");
        if (!(q > 0)) throw FilterError::invalidParameter("q", q, "must be > 0");
        if (!std::isfinite(frequency) || !std::isfinite(sampleRate) || !std::isfinite(q))
            throw FilterError::invalidParameter("input", 0.f, "parameters must not be NaN or Infinite");
        const double pi = 3.14159265358979323846;
        const double w = 2.0 * pi * (double)frequency / (double)sampleRate, sn = std::sin(w), cs = std::cos(w);
        const double al = sn / (2.0 * (double)q);
        const double A = std::pow(10.0, (double)type.gainDB / 40.0), rt = 2.0 * std::sqrt(A) * al;
        double b[3], a[3];
        auto set = [](double* d, double x, double y, double z) { d[0] = x; d[1] = y; d[2] = z; };
        switch (type.kind) {
            case Kind::lowpass: set(b, (1 - cs) / 2, 1 - cs, (1 - cs) / 2); set(a, 1 + al, -2 * cs, 1 - al); break;
            case Kind::highpass: set(b, (1 + cs) / 2, -(1 + cs), (1 + cs) / 2); set(a, 1 + al, -2 * cs, 1 - al); break;
            case Kind::bandpass: set(b, al, 0, -al); set(a, 1 + al, -2 * cs, 1 - al); break;
            case Kind::notch: set(b, 1, -2 * cs, 1); set(a, 1 + al, -2 * cs, 1 - al); break;
            case Kind::allpass: set(b, 1 - al, -2 * cs, 1 + al); set(a, 1 + al, -2 * cs, 1 - al); break;
            case Kind::peaking: set(b, 1 + al * A, -2 * cs, 1 - al * A); set(a, 1 + al / A, -2 * cs, 1 - al / A); break;
            case Kind::lowshelf:
                set(b, A * ((A + 1) - (A - 1) * cs + rt), 2 * A * ((A - 1) - (A + 1) * cs), A * ((A + 1) - (A - 1) * cs - rt));
                set(a, (A + 1) + (A - 1) * cs + rt, -2 * ((A - 1) + (A + 1) * cs), (A + 1) + (A - 1) * cs - rt);
                break;
            case Kind::highshelf:
                set(b, A * ((A + 1) + (A - 1) * cs + rt), -2 * A * ((A - 1) + (A + 1) * cs), A * ((A + 1) + (A - 1) * cs - rt));
                set(a, (A + 1) - (A - 1) * cs + rt, 2 * ((A - 1) - (A + 1) * cs), (A + 1) - (A - 1) * cs - rt);
                break;
        }
        const float a0f = (float)a[0];
        if (!(std::fabs(a0f) > 1e-6f))
            throw FilterError::invalidParameter("a0 (computed)", a0f, "denominator coefficient a0 must not be near zero (|a0| > 1e-6)");
        Coefficients c;
        c.b0 = (float)(b[0] / a[0]); c.b1 = (float)(b[1] / a[0]); c.b2 = (float)(b[2] / a[0]);
        c.a1 = (float)(a[1] / a[0]); c.a2 = (float)(a[2] / a[0]);
        if (!std::isfinite(c.b0) || !std::isfinite(c.b1) || !std::isfinite(c.b2) || !std::isfinite(c.a1) || !std::isfinite(c.a2))
            throw FilterError::invalidParameter("coefficients", 0.f, "normalized coefficients must not be NaN or Infinite");
        if (!(std::fabs(c.a2) < 1.0f)) throw FilterError::invalidParameter("a2 (stability)", c.a2, "|a2| must be < 1 for filter stability");
        if (!(std::fabs(c.a1) < 1.0f + c.a2))
            throw FilterError::invalidParameter("a1 (stability)", c.a1, "|a1| must be < 1 + a2 for filter stability");
        return c;
    }

    // Filters.swift:346-490: a failed validation leaves the previous coefficients in place.
    void configure(FilterType type, float frequency, float sampleRate, float q = 0.7071067811865476f) {
        coefficients_ = design(type, frequency, sampleRate, q);
        upload();
    }
    const Coefficients& currentCoefficients() const { return coefficients_; }
    bool isStable() const {
        return std::isfinite(coefficients_.a1) && std::isfinite(coefficients_.a2) && std::fabs(coefficients_.a2) < 1.0f &&
               std::fabs(coefficients_.a1) < 1.0f + coefficients_.a2;
    }
    void validateStability() const {  // Filters.swift:688-716
        if (!std::isfinite(coefficients_.a1) || !std::isfinite(coefficients_.a2))
            throw FilterError::unstable("coefficients contain NaN or Infinite values, filter is in invalid state");
        if (!(std::fabs(coefficients_.a2) < 1.0f)) throw FilterError::unstable("a2 coefficient magnitude >= 1, poles outside unit circle");
        if (!(std::fabs(coefficients_.a1) < 1.0f + coefficients_.a2)) throw FilterError::unstable("a1 coefficient violates stability condition |a1| < 1 + a2");
    }

    // process(input:) (Filters.swift:555-593): channels x L row-major in, same shape out; state carries over.
    std::vector<float> process(const std::vector<float>& input) {
        std::vector<float> out(input.size());
        if (input.empty()) return out;
        const int64_t len = (int64_t)input.size() / channels_;
        throwStatus(ma_biquad_process_host(bq_, input.data(), len, out.data(), len, len), "process");
        return out;
    }
    float process(float sample) {  // Filters.swift:515-537
        float y = 0.f;
        throwStatus(ma_biquad_process_host(bq_, &sample, 1, &y, 1, 1), "process");
        return y;
    }
    void reset() { throwStatus(ma_biquad_reset(bq_), "reset"); }

private:
    void upload() {
        const float c[5] = {coefficients_.b0, coefficients_.b1, coefficients_.b2, coefficients_.a1, coefficients_.a2};
        throwStatus(ma_biquad_set_coefficients(bq_, c, 1, nullptr), "configure");
    }
    AudioDevice& device_;
    int channels_;
    Coefficients coefficients_;
    ma_biquad* bq_ = nullptr;
};

class FilterBank {  // Filters.swift:736-873
public:
    FilterBank(AudioDevice& device, int bandCount) : device_(device), bands_(bandCount), coeffs_((size_t)(bandCount > 0 ? bandCount : 0)) {}
    ~FilterBank() {
        ma_biquad_destroy(series_);
        ma_biquad_destroy(parallel_);
    }
    FilterBank(const FilterBank&) = delete;
    FilterBank& operator=(const FilterBank&) = delete;

    void configureAsEQ(float lowFreq, float highFreq, float sampleRate, float q = 1.414f) {
        if (bands_ < 2) throw FilterError::invalidParameter("bandCount", (float)bands_, "must be >= 2 for logarithmic band spacing");
        if (!(lowFreq > 0)) throw FilterError::invalidParameter("lowFreq", lowFreq, "must be > 0");
        if (!(highFreq > 0 && highFreq > lowFreq)) throw FilterError::invalidParameter("highFreq", highFreq, "must be > 0 and > lowFreq");
        const float logLow = std::log10(lowFreq), logHigh = std::log10(highFreq), step = (logHigh - logLow) / (float)(bands_ - 1);
        for (int i = 0; i < bands_; ++i) {
            coeffs_[(size_t)i] = BiquadFilter::design(BiquadFilter::FilterType::peaking(0.f), std::pow(10.0f, logLow + (float)i * step), sampleRate, q);
            dirty_ = true;
        }
    }
    void setBandGain(int band, float gainDB, float frequency, float sampleRate, float q = 1.414f) {
        if (band < 0 || band >= bands_) throw FilterError::invalidParameter("band", (float)band, "must be in range 0..<" + std::to_string(bands_));
        coeffs_[(size_t)band] = BiquadFilter::design(BiquadFilter::FilterType::peaking(gainDB), frequency, sampleRate, q);
        dirty_ = true;
    }
    std::vector<float> processSeries(const std::vector<float>& input) {  // one cascade of bandCount sections
        if (input.empty() || bands_ <= 0) return input;
        prepare();
        std::vector<float> out(input.size());
        throwStatus(ma_biquad_process_host(series_, input.data(), (int64_t)input.size(), out.data(), (int64_t)input.size(), (int64_t)input.size()), "processSeries");
        return out;
    }
    std::vector<float> processParallel(const std::vector<float>& input) {  // every band on the same input, mixed with 1/bandCount
        std::vector<float> out(input.size(), 0.f);
        if (input.empty() || bands_ <= 0) return out;
        prepare();
        const int64_t n = (int64_t)input.size();
        Tensor in(device_, {n}), bands(device_, {(int64_t)bands_, n}), mix(device_, {n});
        in.copy(input);
        throwStatus(ma_biquad_process_dev(parallel_, in.devicePointer(), 0, bands.devicePointer(), n, n), "processParallel");
        throwStatus(ma_channel_mix_dev(device_.handle(), bands.devicePointer(), bands_, n, n, 1.0f / (float)bands_, mix.devicePointer()), "processParallel");
        return mix.toArray();
    }
    void reset() {
        if (series_) throwStatus(ma_biquad_reset(series_), "reset");
        if (parallel_) throwStatus(ma_biquad_reset(parallel_), "reset");
    }

private:
    void prepare() {
        if (series_ == nullptr) {
            throwStatus(ma_biquad_create(device_.handle(), 1, bands_, &series_), "FilterBank");
            throwStatus(ma_biquad_create(device_.handle(), bands_, 1, &parallel_), "FilterBank");
        }
        if (!dirty_) return;
        std::vector<float> c((size_t)bands_ * 5);
        std::vector<int32_t> map((size_t)bands_);
        for (int i = 0; i < bands_; ++i) {
            const auto& k = coeffs_[(size_t)i];
            const float v[5] = {k.b0, k.b1, k.b2, k.a1, k.a2};
            std::copy(v, v + 5, c.begin() + 5 * i);
            map[(size_t)i] = i;
        }
        throwStatus(ma_biquad_set_coefficients(series_, c.data(), 1, nullptr), "FilterBank");
        throwStatus(ma_biquad_set_coefficients(parallel_, c.data(), bands_, map.data()), "FilterBank");
        dirty_ = false;
    }
    AudioDevice& device_;
    int bands_;
    std::vector<BiquadFilter::Coefficients> coeffs_;
    ma_biquad* series_ = nullptr;
    ma_biquad* parallel_ = nullptr;
    bool dirty_ = true;
};

}  // namespace metalaudio
