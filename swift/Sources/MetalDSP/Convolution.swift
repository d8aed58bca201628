// NOT COMPILED in the build image (no Swift toolchain); written against include/metalaudio_cuda.h.
// Convolution (Sources/MetalDSP/Convolution.swift:8-47, :112-125, :176-383, :437-493, :529-775) in
// its `.partitioned` and `.fft` modes on the CUDA library.  `.direct` (cross-correlation through
// vDSP_conv in the reference) is not served by this backend.
import CMetalAudioCUDA
import Foundation
import MetalAudioKit

public enum ConvolutionError: Error, LocalizedError {
    case inputSizeMismatch(inputSize: Int, expectedMaxSize: Int, fftSize: Int)
    case kernelNotConfigured
    case emptyKernel
    case fftNotInitialized
    case invalidPartitionState(reason: String)
    case outputSizeOverflow(inputSize: Int, kernelSize: Int)

    public var errorDescription: String? {
        switch self {
        case .inputSizeMismatch(let i, let e, let n):
            return "Convolution input size \(i) exceeds expected maximum \(e) (FFT size: \(n)). This would cause circular convolution artifacts. Call setKernel() with a larger expectedInputSize parameter."
        case .kernelNotConfigured: return "Convolution kernel has not been set. Call setKernel() before processing."
        case .emptyKernel: return "Convolution kernel cannot be empty. Provide at least one sample."
        case .fftNotInitialized: return "FFT resources failed to initialize. This may indicate a Metal device error."
        case .invalidPartitionState(let r): return "Partitioned convolution is in an invalid state: \(r)"
        case .outputSizeOverflow(let i, let k):
            return "Output size would overflow: input (\(i)) + kernel (\(k)) - 1 exceeds Int.max. Use smaller buffers or process in chunks."
        }
    }
}

public final class Convolution {
    public enum Mode {
        case direct
        case fft
        case partitioned(blockSize: Int, useMPSGraphFFT: Bool = false)
    }

    let device: AudioDevice
    let mode: Mode
    private var pconv: OpaquePointer?
    private var fftconv: OpaquePointer?
    private var kernelCount = 0
    private var expectedInput = 0
    private var fftSize = 0

    public init(device: AudioDevice, mode: Mode = .fft) {
        self.device = device
        self.mode = mode
    }

    deinit {
        ma_pconv_destroy(pconv)
        ma_fftconv_destroy(fftconv)
    }

    public func setKernel(_ kernel: [Float], expectedInputSize: Int? = nil) throws {
        switch mode {
        case .direct:
            throw MetalAudioError.invalidConfiguration("direct mode is not served by the CUDA backend")
        case .partitioned(let block, _):
            guard !kernel.isEmpty else { throw MetalAudioError.invalidConfiguration("Kernel must not be empty for partitioned convolution") }
            if pconv == nil { try maCheck(ma_pconv_create(device.handle, Int32(block), 1, &pconv)) }
            try maCheck(kernel.withUnsafeBufferPointer { ma_pconv_set_kernels(pconv, $0.baseAddress, Int64(kernel.count), 1, nil) })
        case .fft:
            guard !kernel.isEmpty else { throw ConvolutionError.emptyKernel }
            ma_fftconv_destroy(fftconv)
            fftconv = nil
            expectedInput = expectedInputSize ?? kernel.count
            try maCheck(kernel.withUnsafeBufferPointer {
                ma_fftconv_create(device.handle, $0.baseAddress, Int64(kernel.count), Int64(expectedInput), 1, &fftconv) })
            var n: Int64 = 0
            ma_fftconv_fft_size(fftconv, &n)
            fftSize = Int(n)
        }
        kernelCount = kernel.count
    }

    public var kernelTailLength: Int { max(0, kernelCount - 1) }
    public func expectedOutputSize(forInputSize inputSize: Int) -> Int { inputSize + kernelTailLength }
    public var maxInputSize: Int { if case .fft = mode { return expectedInput }; return 0 }

    /// Whole-signal call: `output` grows to input.count + kernel.count - 1 (or fftSize in `.fft`
    /// mode); an empty input gives an empty output.
    public func process(input: [Float], output: inout [Float]) throws {
        guard !input.isEmpty else { output = []; return }
        switch mode {
        case .direct:
            throw MetalAudioError.invalidConfiguration("direct mode is not served by the CUDA backend")
        case .partitioned:
            guard pconv != nil else { throw ConvolutionError.fftNotInitialized }
            let (full, over) = input.count.addingReportingOverflow(kernelCount - 1)
            guard !over else { throw ConvolutionError.outputSizeOverflow(inputSize: input.count, kernelSize: kernelCount) }
            if output.count < full { output = [Float](repeating: 0, count: full) } else { for i in full..<output.count { output[i] = 0 } }
            let st = input.withUnsafeBufferPointer { x in
                output.withUnsafeMutableBufferPointer { y in
                    ma_pconv_process_host(pconv, x.baseAddress, Int64(input.count), Int64(input.count), y.baseAddress, Int64(full))
                }
            }
            if st == ma_status(MA_ERR_INVALID_PARTITION_STATE) { throw ConvolutionError.invalidPartitionState(reason: "write index out of range") }
            try maCheck(st)
        case .fft:
            guard fftconv != nil else { throw ConvolutionError.kernelNotConfigured }
            guard input.count <= expectedInput else {
                throw ConvolutionError.inputSizeMismatch(inputSize: input.count, expectedMaxSize: expectedInput, fftSize: fftSize)
            }
            if output.count != fftSize { output = [Float](repeating: 0, count: fftSize) }
            try maCheck(input.withUnsafeBufferPointer { x in
                output.withUnsafeMutableBufferPointer { y in
                    ma_fftconv_process_host(fftconv, x.baseAddress, Int64(input.count), Int64(input.count), 1, y.baseAddress)
                }
            })
        }
    }

    /// Clears the delay line, its write index and the overlap tail.
    public func reset() { if pconv != nil { ma_pconv_reset(pconv) } }

    public func releaseFFTResources() {}
}

extension Convolution: MemoryPressureResponder {
    public func didReceiveMemoryPressure(level: MemoryPressureLevel) {
        if level == .critical { releaseFFTResources() }
    }
}
