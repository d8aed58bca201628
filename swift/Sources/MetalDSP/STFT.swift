// NOT COMPILED in the build image (no Swift toolchain); written against include/metalaudio_cuda.h.
// STFT extension of FFT (Sources/MetalDSP/STFT.swift:10-22, :40-128, :327-527): frames at i*hop,
// analysis window, forward DFT, full-N split result; the inverse overlap-adds and divides by
// max(sum of squared window, floor).  `istft` uses the true inverse transform (the reference pushes
// frames through the object's forward-direction setup, which returns them time-reversed).
import CMetalAudioCUDA
import MetalAudioKit

extension FFT {
    public struct STFTResult {
        public let real: [[Float]]
        public let imag: [[Float]]
        public var frameCount: Int { real.count }
        public var binCount: Int { real.first?.count ?? 0 }
        public init(real: [[Float]], imag: [[Float]]) { self.real = real; self.imag = imag }
    }

    private func rows(_ flat: [Float], _ width: Int) -> [[Float]] {
        stride(from: 0, to: flat.count, by: width).map { Array(flat[$0..<$0 + width]) }
    }

    public func stft(input: [Float]) throws -> STFTResult {
        var frames: Int64 = 0
        guard ma_stft_frame_count(plan, Int64(input.count), &frames) == ma_status(MA_OK) else {
            throw FFTError.inputTooShort(inputSize: input.count, requiredSize: size)
        }
        var re = [Float](repeating: 0, count: Int(frames) * size), im = re
        let st = input.withUnsafeBufferPointer { x in
            re.withUnsafeMutableBufferPointer { r in
                im.withUnsafeMutableBufferPointer { m in
                    ma_stft_host(plan, x.baseAddress, Int64(input.count), Int64(input.count), 1, r.baseAddress, m.baseAddress,
                                 nil, 0, 1, Int32(MA_LAYOUT_FULL_SPLIT))
                }
            }
        }
        try maCheck(st)
        return STFTResult(real: rows(re, size), imag: rows(im, size))
    }

    /// Window floor rule of the reference: tiny configured values become 1e-6, large ones 0.1.
    static func validatedWindowFloor() -> Float {
        let c = ToleranceProvider.shared.tolerances.windowFloorEpsilon
        return c < 1e-10 ? 1e-6 : (c > 0.1 ? 0.1 : c)
    }

    public func istft(stft: STFTResult) throws -> [Float] {
        let f = stft.frameCount
        guard f > 0 else { return [] }
        var outLen: Int64 = 0
        guard ma_istft_output_length(plan, Int64(f), &outLen) == ma_status(MA_OK) else {
            throw FFTError.istftOutputOverflow(frameCount: f, hopSize: config.hopSize, fftSize: size)
        }
        guard stft.imag.count >= f else { throw FFTError.inputTooShort(inputSize: stft.imag.count, requiredSize: f) }
        let re = stft.real.flatMap { $0 }, im = stft.imag.flatMap { $0 }
        var out = [Float](repeating: 0, count: Int(outLen))
        let st = re.withUnsafeBufferPointer { r in
            im.withUnsafeBufferPointer { m in
                out.withUnsafeMutableBufferPointer { o in
                    ma_istft_host(plan, r.baseAddress, m.baseAddress, Int64(f), 1, o.baseAddress, outLen,
                                  FFT.validatedWindowFloor(), Int32(MA_LAYOUT_FULL_SPLIT))
                }
            }
        }
        try maCheck(st)
        return out
    }

    public func forwardBatch(inputs: [[Float]], outputsReal: inout [[Float]], outputsImag: inout [[Float]]) throws {
        guard !inputs.isEmpty else { return }
        for x in inputs where x.count < size { throw FFTError.inputTooShort(inputSize: x.count, requiredSize: size) }
        let (total, overflow) = inputs.count.multipliedReportingOverflow(by: size)
        guard !overflow else { throw FFTError.batchSizeOverflow(batchSize: inputs.count, fftSize: size) }
        let flat = inputs.flatMap { $0[0..<size] }
        var re = [Float](repeating: 0, count: total), im = re
        let st = flat.withUnsafeBufferPointer { x in
            re.withUnsafeMutableBufferPointer { r in
                im.withUnsafeMutableBufferPointer { m in
                    ma_fft_forward_host(plan, x.baseAddress, r.baseAddress, m.baseAddress, nil, 0, 1, Int64(inputs.count), Int32(MA_LAYOUT_FULL_SPLIT))
                }
            }
        }
        try maCheck(st)
        outputsReal = rows(re, size)
        outputsImag = rows(im, size)
    }

    public func inverseBatch(inputsReal: [[Float]], inputsImag: [[Float]], outputs: inout [[Float]]) throws {
        guard !inputsReal.isEmpty else { return }
        let re = inputsReal.flatMap { $0[0..<size] }, im = inputsImag.flatMap { $0[0..<size] }
        var out = [Float](repeating: 0, count: re.count)
        let st = re.withUnsafeBufferPointer { r in
            im.withUnsafeBufferPointer { m in
                out.withUnsafeMutableBufferPointer { o in
                    ma_fft_inverse_host(plan, r.baseAddress, m.baseAddress, o.baseAddress, Int64(inputsReal.count), Int32(MA_LAYOUT_FULL_SPLIT))
                }
            }
        }
        try maCheck(st)
        outputs = rows(out, size)
    }

    // MARK: device-resident forms (flat Tensor results: no per-frame Swift arrays)

    /// STFT of an (S, L) signal tensor into an (S, F, N/2+1, 2) spectrum tensor and, optionally, an
    /// (S, F, N/2+1) magnitude tensor; queued on the device stream.
    public func stftTensor(signals: Tensor, spectrum: Tensor, magnitude: Tensor? = nil) throws {
        let s = signals.shape[0], l = signals.shape[1]
        try maCheck(ma_stft_dev(plan, signals.pointer.assumingMemoryBound(to: Float.self), Int64(l), Int64(l), Int64(s),
                                spectrum.pointer.assumingMemoryBound(to: Float.self), nil,
                                magnitude?.pointer.assumingMemoryBound(to: Float.self), Int32(MA_MAG_MAGNITUDE), 1,
                                Int32(MA_LAYOUT_HALF_INTERLEAVED)))
    }

    public func istftTensor(spectrum: Tensor, output: Tensor) throws {
        try maCheck(ma_istft_dev(plan, spectrum.pointer.assumingMemoryBound(to: Float.self), nil, Int64(spectrum.shape[1]),
                                 Int64(spectrum.shape[0]), output.pointer.assumingMemoryBound(to: Float.self),
                                 Int64(output.shape[1]), FFT.validatedWindowFloor(), Int32(MA_LAYOUT_HALF_INTERLEAVED)))
    }
}
