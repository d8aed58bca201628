// swift-tools-version:5.9
// Swift surface of the reference's DSP hot path over the CUDA backend.  NOT COMPILED in the build
// image (no Swift toolchain there); see README.md in this directory.
import PackageDescription

let package = Package(
    name: "MetalAudioCUDA",
    products: [
        .library(name: "MetalAudioKit", targets: ["MetalAudioKit"]),
        .library(name: "MetalDSP", targets: ["MetalDSP"]),
    ],
    targets: [
        // C ABI of libmetalaudio_cuda.so (include/metalaudio_cuda.h at the repository root)
        .systemLibrary(name: "CMetalAudioCUDA", path: "Sources/CMetalAudioCUDA"),
        .target(name: "MetalAudioKit", dependencies: ["CMetalAudioCUDA"], path: "Sources/MetalAudioKit"),
        .target(name: "MetalDSP", dependencies: ["MetalAudioKit", "CMetalAudioCUDA"], path: "Sources/MetalDSP",
                linkerSettings: [.linkedLibrary("metalaudio_cuda")]),
    ]
)
