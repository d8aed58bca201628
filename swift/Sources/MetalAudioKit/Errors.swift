// NOT COMPILED in the build image (no Swift toolchain); written against include/metalaudio_cuda.h.
// Error vocabulary of the reference (Sources/MetalAudioKit/Core/AudioDevice.swift:11-77), the
// cases the hot path can raise, and the mapping from the library's status codes.
import CMetalAudioCUDA
import Foundation

public enum MetalAudioError: Error, LocalizedError {
    case deviceNotFound
    case bufferAllocationFailed(Int)
    case bufferSizeMismatch(expected: Int, actual: Int)
    case invalidConfiguration(String)
    case gpuTimeout(TimeInterval)
    case gpuExecutionError(String)
    case deviceLost
    case invalidPointer

    public var errorDescription: String? {
        switch self {
        case .deviceNotFound: return "No CUDA device found"
        case .bufferAllocationFailed(let n): return "Failed to allocate buffer of size \(n) bytes"
        case .bufferSizeMismatch(let e, let a): return "Buffer size mismatch: expected \(e) bytes, got \(a)"
        case .invalidConfiguration(let why): return "Invalid configuration: \(why)"
        case .gpuTimeout(let t): return "GPU operation timed out after \(t) seconds"
        case .gpuExecutionError(let why): return "GPU execution error: \(why)"
        case .deviceLost: return "GPU device was disconnected or lost"
        case .invalidPointer: return "Invalid or null pointer provided"
        }
    }
}

/// Throws the Swift error a non-zero library status stands for.
@inline(__always)
public func maCheck(_ status: ma_status, bytes: Int = 0, timeout: TimeInterval = 2.0) throws {
    switch status {
    case ma_status(MA_OK): return
    case ma_status(MA_ERR_ALLOC): throw MetalAudioError.bufferAllocationFailed(bytes)
    case ma_status(MA_ERR_TIMEOUT): throw MetalAudioError.gpuTimeout(timeout)
    case ma_status(MA_ERR_DEVICE_LOST): throw MetalAudioError.deviceLost
    case ma_status(MA_ERR_CUDA):
        throw MetalAudioError.gpuExecutionError("\(String(cString: ma_status_string(status))) (cudaError \(ma_last_cuda_error()))")
    default: throw MetalAudioError.invalidConfiguration(String(cString: ma_status_string(status)))
    }
}
