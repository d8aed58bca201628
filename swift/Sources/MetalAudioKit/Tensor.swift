// NOT COMPILED in the build image (no Swift toolchain); written against include/metalaudio_cuda.h.
// float32 slice of Tensor (Sources/MetalAudioKit/Buffers/Tensor.swift:12-438) with its storage in
// device memory.  The reference's `floatPointer` / `withUnsafe*BufferPointer` assumed CPU-addressable
// storage; here host access is an explicit copy (copy(from:), toArray(), copy(to:)).
import CMetalAudioCUDA

public final class Tensor {
    public let device: AudioDevice
    public let shape: [Int]
    /// Device address of the first element (pass to the `_dev` entry points).
    public let pointer: UnsafeMutableRawPointer

    public var count: Int { shape.reduce(1, *) }
    public var isEmpty: Bool { count == 0 }
    public var rank: Int { shape.count }
    public var byteSize: Int { count * MemoryLayout<Float>.stride }

    public init(device: AudioDevice, shape: [Int]) throws {
        guard shape.allSatisfy({ $0 >= 0 }) else { throw MetalAudioError.invalidConfiguration("negative dimension") }
        self.device = device
        self.shape = shape
        var p: UnsafeMutableRawPointer?
        let bytes = shape.reduce(1, *) * MemoryLayout<Float>.stride
        try maCheck(ma_buffer_alloc(device.handle, bytes, &p), bytes: bytes)
        guard let q = p else { throw MetalAudioError.bufferAllocationFailed(bytes) }
        pointer = q
    }

    deinit { ma_buffer_free(device.handle, pointer) }

    public func copy(from array: [Float]) throws {
        guard array.count == count else {
            throw MetalAudioError.bufferSizeMismatch(expected: byteSize, actual: array.count * MemoryLayout<Float>.stride)
        }
        try array.withUnsafeBufferPointer { try maCheck(ma_memcpy_h2d(device.handle, pointer, $0.baseAddress, byteSize)) }
    }

    public func toArray() -> [Float] {
        var out = [Float](repeating: 0, count: count)
        out.withUnsafeMutableBufferPointer { _ = ma_memcpy_d2h(device.handle, $0.baseAddress, pointer, byteSize) }
        return out
    }

    public func copy(to array: inout [Float]) throws {
        if array.count != count { array = [Float](repeating: 0, count: count) }
        try array.withUnsafeMutableBufferPointer { try maCheck(ma_memcpy_d2h(device.handle, $0.baseAddress, pointer, byteSize)) }
    }

    public func zero() { ma_buffer_zero(device.handle, pointer, byteSize) }
}
