// swift-tools-version: 5.9
//
// SwiftPM manifest of the CUDA build of the PagedAttentionMetal API.  It takes the place of
// the reference's "PagedAttentionMetal" target (Package.swift:46-53 of the reference, a Swift
// target with kernels.metal as a processed resource): the Swift classes keep their names and
// signatures and call libpam_cuda.so through the C module CPamCuda (include/pam_cuda.h).
//
// Build the library first (python -m pagedattentionmetal_b200.build), then
//   swift build -Xlinker -L<repo>/pagedattentionmetal_b200 -Xlinker -rpath -Xlinker <repo>/pagedattentionmetal_b200
// The MLX, NIO and Hugging Face dependencies of the reference's manifest belong to targets
// outside this library (demo server, MLX adapters) and are not needed.
import PackageDescription

let package = Package(
    name: "PagedAttentionMetal",
    products: [
        .library(name: "PagedAttentionMetal", targets: ["PagedAttentionMetal"]),
    ],
    targets: [
        .systemLibrary(name: "CPamCuda", path: "Sources/CPamCuda"),
        .target(name: "PagedAttentionMetal", dependencies: ["CPamCuda"], path: "Sources/PagedAttentionMetal"),
    ]
)
