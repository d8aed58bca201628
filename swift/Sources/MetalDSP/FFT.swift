// NOT COMPILED in the build image (no Swift toolchain); written against include/metalaudio_cuda.h.
// Public surface of FFT (Sources/MetalDSP/FFT.swift:12-55, :155-348, :441-495, :818-919, :945-1747,
// :1780-1847) with every transform routed to the CUDA library.  One backend, no size routing, no CPU
// fallback: a missing device is an error.
import CMetalAudioCUDA
import Foundation
import MetalAudioKit

public enum FFTError: Error, LocalizedError {
    case inputTooShort(inputSize: Int, requiredSize: Int)
    case sizeTooLarge(requestedSize: Int, maxSize: Int)
    case sizeNotPowerOf2(size: Int)
    case invalidHopSize(hopSize: Int, fftSize: Int)
    case batchSizeOverflow(batchSize: Int, fftSize: Int)
    case istftOutputOverflow(frameCount: Int, hopSize: Int, fftSize: Int)
    case istftFrameOverflow(frameIndex: Int, hopSize: Int, fftSize: Int, outputLength: Int)

    public var errorDescription: String? {
        switch self {
        case .inputTooShort(let i, let r):
            return "Input size \(i) is shorter than the required FFT size \(r). Provide at least \(r) samples, or use a smaller FFT size."
        case .sizeTooLarge(let s, let m): return "FFT size \(s) exceeds maximum supported size \(m)."
        case .sizeNotPowerOf2(let s): return "FFT size \(s) is not a power of 2. Use sizes like 256, 512, 1024, 2048, etc."
        case .invalidHopSize(let h, let n): return "Hop size \(h) is invalid. Must be > 0 and <= FFT size (\(n))."
        case .batchSizeOverflow(let b, let n): return "Batch size \(b) with FFT size \(n) would overflow buffer limits."
        case .istftOutputOverflow(let f, let h, let n):
            return "ISTFT output length calculation overflowed: frameCount=\(f), hopSize=\(h), fftSize=\(n). Use smaller STFT result or process in chunks."
        case .istftFrameOverflow(let i, let h, let n, let o):
            return "ISTFT frame \(i) position overflow: frameIndex*hopSize=\(i)*\(h) + fftSize=\(n) exceeds outputLength=\(o). STFT result may be corrupted or parameters are inconsistent."
        }
    }
}

/// Sampled NaN / Inf check on transform outputs, off unless this is set (FFT.swift:63).
nonisolated(unsafe) public var fftValidationEnabled = false

/// About 50 evenly spaced values plus the last one; logs, never throws (FFT.swift:80-134).
@discardableResult
func validateFFTOutput(_ p: UnsafePointer<Float>, count: Int, context: String) -> Bool {
    guard fftValidationEnabled, count > 0 else { return false }
    let step = max(1, count / min(50, count))
    var nanAt = -1, infAt = -1
    for i in stride(from: 0, to: count, by: step) + [count - 1] {
        if nanAt < 0 && p[i].isNaN { nanAt = i }
        if infAt < 0 && p[i].isInfinite { infAt = i }
    }
    if nanAt >= 0 { NSLog("[FFT] Warning: NaN detected in \(context) near index \(nanAt)") }
    if infAt >= 0 { NSLog("[FFT] Warning: Inf detected in \(context) near index \(infAt)") }
    return nanAt >= 0 || infAt >= 0
}

public final class FFT {
    public static let maxFFTSize = 1 << 24

    public enum COLACompliance { case perfect, nearPerfect, nonCompliant }

    public enum WindowType {
        case none, hann, hamming, blackman

        /// Symmetric window (denominator length - 1), evaluated in Double and rounded once.
        public func coefficient(at i: Int, length n: Int) -> Float {
            guard n > 1 else { return 1 }
            let x = 2.0 * Double.pi * Double(i) / Double(n - 1)
            switch self {
            case .none: return 1
            case .hann: return Float(0.5 - 0.5 * cos(x))
            case .hamming: return Float(0.54 - 0.46 * cos(x))
            case .blackman: return Float(0.42 - 0.5 * cos(x) + 0.08 * cos(2 * x))
            }
        }

        /// Hop = size / divisor gives constant overlap-add for these divisors.
        public var colaHopDivisors: [Int] {
            switch self {
            case .none: return [1]
            case .hann: return [2, 4]
            case .hamming: return []
            case .blackman: return [3, 4]
            }
        }
    }

    public struct Config {
        public let size: Int
        public let inverse: Bool
        public let windowType: WindowType
        public var hopSize: Int

        public init(size: Int, inverse: Bool = false, windowType: WindowType = .hann, hopSize: Int? = nil) {
            self.size = size
            self.inverse = inverse
            self.windowType = windowType
            self.hopSize = hopSize ?? max(1, size / 4)
        }

        public var colaCompliance: COLACompliance {
            for d in windowType.colaHopDivisors where size % d == 0 && hopSize == size / d { return .perfect }
            if case .hamming = windowType, hopSize == size / 2 || hopSize == size / 4 { return .nearPerfect }
            return .nonCompliant
        }

        public var overlapPercent: Int { 100 - hopSize * 100 / size }

        public func validateCOLA() -> (isValid: Bool, compliance: COLACompliance, message: String) {
            let w = "\(windowType)"
            switch colaCompliance {
            case .perfect:
                return (true, .perfect, "\(w) window with hop size \(hopSize) (overlap \(overlapPercent)%) satisfies COLA")
            case .nearPerfect:
                return (true, .nearPerfect, "\(w) window with hop size \(hopSize) is near-COLA (error < 0.1%)")
            case .nonCompliant:
                let hops = windowType.colaHopDivisors.filter { size % $0 == 0 }
                    .map { "\(size / $0) (\(100 - (size / $0) * 100 / size)% overlap)" }
                let hint = hops.isEmpty ? "Consider using Hann window for COLA-compliant STFT"
                                        : "Suggested hop sizes: " + hops.joined(separator: ", ")
                return (false, .nonCompliant, "\(w) window with hop size \(hopSize) does not satisfy COLA. \(hint)")
            }
        }
    }

    public enum Backend {
        case vdsp, gpu, mpsGraph, cuda
        public var description: String { self == .cuda ? "CUDA (sm_100a)" : "unavailable in this build" }
    }

    public let config: Config
    public var size: Int { config.size }
    let device: AudioDevice
    var plan: OpaquePointer?
    let window: [Float]

    public init(device: AudioDevice, config: Config) throws {
        let n = config.size
        guard n > 0 && n & (n - 1) == 0 else { throw FFTError.sizeNotPowerOf2(size: n) }
        guard n <= FFT.maxFFTSize else { throw FFTError.sizeTooLarge(requestedSize: n, maxSize: FFT.maxFFTSize) }
        guard config.hopSize > 0 && config.hopSize <= n else { throw FFTError.invalidHopSize(hopSize: config.hopSize, fftSize: n) }
        self.device = device
        self.config = config
        window = (0..<n).map { config.windowType.coefficient(at: $0, length: n) }
        let st = window.withUnsafeBufferPointer { w -> ma_status in
            var useWindow = true
            if case .none = config.windowType { useWindow = false }
            return ma_fft_plan_create(device.handle, Int32(n), useWindow ? w.baseAddress : nil, Int32(config.hopSize), &plan)
        }
        try maCheck(st)
    }

    deinit { ma_fft_plan_destroy(plan) }

    // MARK: single transforms (pointer API, non-throwing: outputs are zeroed on failure)

    public func forward(input: UnsafePointer<Float>, outputReal: UnsafeMutablePointer<Float>, outputImag: UnsafeMutablePointer<Float>) {
        let st = ma_fft_forward_host(plan, input, outputReal, outputImag, nil, 0, 1, 1, Int32(MA_LAYOUT_FULL_SPLIT))
        guard st == ma_status(MA_OK) else {
            outputReal.update(repeating: 0, count: size)
            outputImag.update(repeating: 0, count: size)
            return
        }
        // the reference's single vDSP setup runs in the direction Config.inverse names
        if config.inverse { for i in 0..<size { outputImag[i] = -outputImag[i] } }
        validateFFTOutput(outputReal, count: size, context: "outputReal")
        validateFFTOutput(outputImag, count: size, context: "outputImag")
    }

    public func inverse(inputReal: UnsafePointer<Float>, inputImag: UnsafePointer<Float>, output: UnsafeMutablePointer<Float>) {
        let st = ma_fft_inverse_host(plan, inputReal, inputImag, output, 1, Int32(MA_LAYOUT_FULL_SPLIT))
        guard st == ma_status(MA_OK) else { output.update(repeating: 0, count: size); return }
        if !config.inverse && size > 2 {   // forward-direction object: the sequence comes back time-reversed
            var i = 1, j = size - 1
            while i < j { swap(&output[i], &output[j]); i += 1; j -= 1 }
        }
        validateFFTOutput(output, count: size, context: "inverse.output")
    }

    private func magnitudeKind(_ kind: Int32, _ re: UnsafePointer<Float>, _ im: UnsafePointer<Float>,
                               _ out: UnsafeMutablePointer<Float>, _ reference: Float) {
        _ = ma_fft_magnitude_host(plan, re, im, out, 1, kind, reference)
    }
    public func magnitude(real: UnsafePointer<Float>, imag: UnsafePointer<Float>, magnitude: UnsafeMutablePointer<Float>) {
        magnitudeKind(Int32(MA_MAG_MAGNITUDE), real, imag, magnitude, 1)
    }
    public func power(real: UnsafePointer<Float>, imag: UnsafePointer<Float>, power: UnsafeMutablePointer<Float>) {
        magnitudeKind(Int32(MA_MAG_POWER), real, imag, power, 1)
    }
    public func magnitudeDB(real: UnsafePointer<Float>, imag: UnsafePointer<Float>, magnitudeDB: UnsafeMutablePointer<Float>, reference: Float = 1.0) {
        magnitudeKind(Int32(MA_MAG_DB), real, imag, magnitudeDB, reference)
    }

    // MARK: explicit-backend and auto API: one backend serves them all

    public var optimalBackend: Backend { .cuda }
    public var shouldUseGPU: Bool { true }
    public var shouldUseMetal: Bool { size > 2048 && size <= 8192 }
    public var shouldUseMPSGraph: Bool { size > 8192 }

    private func complexTransform(_ input: [Float], _ output: inout [Float], inverse: Bool) throws -> Backend {
        guard input.count >= 2 * size else { throw MetalAudioError.bufferSizeMismatch(expected: 2 * size, actual: input.count) }
        if output.count != 2 * size { output = [Float](repeating: 0, count: 2 * size) }
        let st = input.withUnsafeBufferPointer { i in
            output.withUnsafeMutableBufferPointer { o in ma_fft_complex_host(plan, i.baseAddress, o.baseAddress, 1, inverse ? 1 : 0) }
        }
        try maCheck(st)
        return .cuda
    }
    /// Complex transform of `size` interleaved (re, im) pairs, unscaled.
    @discardableResult
    public func forwardGPU(input: [Float], output: inout [Float]) throws -> Backend { try complexTransform(input, &output, inverse: false) }
    /// Its inverse with the 1/N scale.
    @discardableResult
    public func inverseGPU(input: [Float], output: inout [Float]) throws -> Backend { try complexTransform(input, &output, inverse: true) }

    public func forwardMPSGraph(input: [Float], outputReal: inout [Float], outputImag: inout [Float]) throws {
        _ = try forwardAuto(input: input, outputReal: &outputReal, outputImag: &outputImag)
    }
    public func inverseMPSGraph(inputReal: [Float], inputImag: [Float], output: inout [Float]) throws {
        var out = [[Float]]()
        try inverseBatch(inputsReal: [inputReal], inputsImag: [inputImag], outputs: &out)
        output = out[0]
    }

    @discardableResult
    public func forwardAuto(input: [Float], outputReal: inout [Float], outputImag: inout [Float]) throws -> Backend {
        guard input.count >= size else { throw FFTError.inputTooShort(inputSize: input.count, requiredSize: size) }
        if outputReal.count < size { outputReal = [Float](repeating: 0, count: size) }
        if outputImag.count < size { outputImag = [Float](repeating: 0, count: size) }
        input.withUnsafeBufferPointer { i in
            outputReal.withUnsafeMutableBufferPointer { r in
                outputImag.withUnsafeMutableBufferPointer { m in forward(input: i.baseAddress!, outputReal: r.baseAddress!, outputImag: m.baseAddress!) }
            }
        }
        return .cuda
    }

    @discardableResult
    public func inverseAuto(inputReal: [Float], inputImag: [Float], output: inout [Float]) throws -> Backend {
        guard inputReal.count >= size, inputImag.count >= size else {
            throw FFTError.inputTooShort(inputSize: min(inputReal.count, inputImag.count), requiredSize: size)
        }
        if output.count < size { output = [Float](repeating: 0, count: size) }
        inputReal.withUnsafeBufferPointer { r in
            inputImag.withUnsafeBufferPointer { m in
                output.withUnsafeMutableBufferPointer { o in inverse(inputReal: r.baseAddress!, inputImag: m.baseAddress!, output: o.baseAddress!) }
            }
        }
        return .cuda
    }

    /// Creates the CUDA context's lazily built state (first launch of the plan's kernels).
    public func warmup() {
        var x = [Float](repeating: 0, count: size), r = x, m = x
        _ = try? forwardAuto(input: x, outputReal: &r, outputImag: &m)
        x = r
    }

    /// Device tables are a few kilobytes; they are kept so the object stays usable.
    public func releaseGPUResources() {}
}

extension FFT: MemoryPressureResponder {
    public func didReceiveMemoryPressure(level: MemoryPressureLevel) {
        if level == .critical { releaseGPUResources() }
    }
}
