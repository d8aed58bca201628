// NOT COMPILED in the build image (no Swift toolchain); written against include/metalaudio_cuda.h.
// The slice of AudioDevice (Sources/MetalAudioKit/Core/AudioDevice.swift:222, :323-332, :434-472,
// :733-741) the DSP path uses: one CUDA device + stream + pinned staging, a name, the loss flag.
import CMetalAudioCUDA

public protocol DeviceLossDelegate: AnyObject {
    func audioDeviceWasLost(_ device: AudioDevice)
}

public final class AudioDevice {
    /// Opaque ma_context*; every plan, convolution and tensor is created on it.
    public let handle: OpaquePointer
    public let deviceIndex: Int
    public weak var lossDelegate: DeviceLossDelegate?
    private var notified = false

    /// `deviceIndex` is new (the reference owns the single system Metal device); `pinnedBytes` sizes
    /// the staging buffer host copies of pageable memory go through (0: 64 MiB).
    public init(deviceIndex: Int = 0, pinnedBytes: Int = 0) throws {
        var h: OpaquePointer?
        let st = ma_context_create(Int32(deviceIndex), pinnedBytes, &h)
        guard st == ma_status(MA_OK), let ctx = h else {
            throw st == ma_status(MA_ERR_DEVICE_LOST) ? MetalAudioError.deviceNotFound
                                                       : MetalAudioError.gpuExecutionError(String(cString: ma_status_string(st)))
        }
        handle = ctx
        self.deviceIndex = deviceIndex
    }

    deinit { ma_context_destroy(handle) }

    public var name: String {
        var buf = [CChar](repeating: 0, count: 256)
        ma_context_device_name(handle, &buf, buf.count)
        return String(cString: buf)
    }

    public var isDeviceAvailable: Bool {
        var ok: Int32 = 0
        ma_context_is_available(handle, &ok)
        return ok != 0
    }

    /// After this every call on the device throws `.deviceLost`; there is no CPU path to fall back to.
    public func markDeviceLost() {
        ma_context_mark_lost(handle)
        if !notified {
            notified = true
            lossDelegate?.audioDeviceWasLost(self)
        }
    }

    public func ensureAvailable() throws {
        if !isDeviceAvailable { throw MetalAudioError.deviceLost }
    }

    /// Device memory for the host-array calls (stft / istft), allocated once instead of per call.
    public func reserveWorkspace(bytes: Int) throws { try maCheck(ma_context_reserve_workspace(handle, bytes), bytes: bytes) }
}
