// NOT COMPILED in the build image (no Swift toolchain); written against include/metalaudio_cuda.h.
// executeSync / executeSyncWithTiming of ComputeContext (Sources/MetalAudioKit/Core/
// ComputeContext.swift:137, :154-211, :232-297).  The closure no longer receives a Metal encoder: it
// queues library calls on the device's stream, and the context waits for them with a deadline.
import CMetalAudioCUDA
import Foundation

public final class ComputeContext {
    public static let defaultGPUTimeout: TimeInterval = 2.0
    public let device: AudioDevice

    public init(device: AudioDevice, maxInFlightBuffers: Int = 3) throws {
        try device.ensureAvailable()
        self.device = device
    }

    /// Runs `work`, then waits for everything it queued; `.gpuTimeout` when the deadline passes
    /// (the stream keeps draining), `.gpuExecutionError` for a CUDA error.
    public func executeSync(timeout: TimeInterval = ComputeContext.defaultGPUTimeout, _ work: () throws -> Void) throws {
        try work()
        try maCheck(ma_context_sync(device.handle, timeout), timeout: timeout)
    }

    /// Same, returning the device time of the queued work in seconds (CUDA events around it).
    public func executeSyncWithTiming(timeout: TimeInterval = ComputeContext.defaultGPUTimeout,
                                      _ work: () throws -> Void) throws -> TimeInterval {
        try maCheck(ma_timing_begin(device.handle))
        try work()
        var ms: Float = 0
        try maCheck(ma_timing_end(device.handle, &ms), timeout: timeout)
        return TimeInterval(ms) * 1e-3
    }
}
