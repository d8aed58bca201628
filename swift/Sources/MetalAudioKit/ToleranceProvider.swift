// NOT COMPILED in the build image (no Swift toolchain).
// The fields of ToleranceConfiguration the DSP path reads.  A B200 is no Apple GPU family, which the
// reference maps to its conservative set (Sources/MetalAudioKit/Config/ToleranceConfiguration.swift:158-181).
public struct ToleranceConfiguration {
    public var windowFloorEpsilon: Float = 1e-8
    public var fftAccuracy: Float = 1e-6
    public var convolutionAccuracy: Float = 1e-6
    public static func conservative() -> ToleranceConfiguration { ToleranceConfiguration() }
}

public final class ToleranceProvider {
    public static let shared = ToleranceProvider()
    public var tolerances = ToleranceConfiguration.conservative()
}

public enum MemoryPressureLevel { case normal, warning, critical }

public protocol MemoryPressureResponder: AnyObject {
    func didReceiveMemoryPressure(level: MemoryPressureLevel)
}
