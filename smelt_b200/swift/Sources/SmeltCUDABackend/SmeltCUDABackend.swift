// SmeltCUDABackend — the Swift side of the drop-in: what SmeltRuntime's Metal-specific
// members become when the decode table is executed by libsmelt_cuda.
//
// Source only: no Swift toolchain exists on the build or GPU machines, so this file is not
// compiled or tested here; the C ABI it calls is exercised from C++ and Python instead.
// Each method names the SmeltRuntime member it replaces
// (Sources/SmeltRuntime/SmeltRuntime.swift in the reference).

import CSmeltCUDA
import Foundation

public struct SmeltCUDAError: Error, CustomStringConvertible {
    public let status: Int32
    public let message: String
    public var description: String { "libsmelt_cuda status \(status): \(message)" }
}

public final class SmeltCUDABackend {
    private var ctx: OpaquePointer?

    /// Replaces MTLCreateSystemDefaultDevice + makeCommandQueue (SmeltRuntime.swift:695-712).
    public init(deviceOrdinal: Int32 = 0) throws {
        var handle: OpaquePointer?
        let status = smelt_cuda_create(deviceOrdinal, &handle)
        guard status == SMELT_OK, let handle else {
            throw SmeltCUDAError(status: status, message: "no usable sm_100 CUDA device")
        }
        ctx = handle
    }

    deinit { smelt_cuda_destroy(ctx) }

    private func check(_ status: Int32) throws {
        guard status == SMELT_OK else {
            throw SmeltCUDAError(status: status, message: String(cString: smelt_cuda_last_error(ctx)))
        }
    }

    /// Replaces the weights mmap -> MTLBuffer segments (SmeltRuntime.swift:799-826): the whole
    /// weights.bin image goes into the weights slot; record offsets index it unchanged.
    public func uploadWeights(slot: Int32, image: UnsafeRawBufferPointer) throws {
        try check(smelt_cuda_upload_weights(ctx, slot, image.baseAddress, image.count))
    }

    /// Replaces buffer-slot allocation and zero fill (SmeltRuntime.swift:922-979).
    public func allocateSlot(_ slot: Int32, bytes: Int) throws {
        try check(smelt_cuda_alloc_slot(ctx, slot, bytes))
    }

    /// Replaces KV growth in resizeRequestScopedBuffers (SmeltRuntime.swift:6803-6913, :6957-6959).
    public func growKVSlot(_ slot: Int32, heads: Int32, headDim: Int32, from old: UInt32, to new: UInt32, live: UInt32) throws {
        try check(smelt_cuda_resize_kv_slot(ctx, slot, heads, headDim, old, new, live))
    }

    /// Replaces makeLibrary + lazy pipeline materialisation (SmeltRuntime.swift:881-915, :6229-6263):
    /// manifest.pipelines entries are registered by name; an unknown kernel is an error.
    public func registerPipelines(_ names: [String]) throws {
        for (index, name) in names.enumerated() {
            try check(name.withCString { smelt_cuda_register_pipeline(ctx, Int32(index), $0) })
        }
    }

    public func configure(_ config: smelt_cuda_runtime_config) throws {
        var c = config
        try check(smelt_cuda_configure(ctx, &c))
    }

    /// Replaces decodeStep's encode / commit / waitUntilCompleted / argmax read
    /// (SmeltRuntime.swift:1573-1641).  `table` is the mmap'd dispatches.bin.
    public func decodeStep(table: UnsafeBufferPointer<smelt_dispatch_record>, tokenId: Int32, position: Int32) throws -> Int32 {
        var token = tokenId
        var out: Int32 = -1
        try check(smelt_cuda_decode_step(ctx, table.baseAddress, table.count, &token, position, &out))
        return out
    }

    /// Replaces encodeTrunkDecode (SmeltRuntime.swift:5029-5091): enqueue only.
    public func enqueueDecode(table: UnsafeBufferPointer<smelt_dispatch_record>, tokenId: Int32, position: Int32) throws {
        var token = tokenId
        try check(smelt_cuda_enqueue_decode(ctx, table.baseAddress, table.count, &token, position))
    }

    /// One CUDA graph per table; replay decodes tokens without a host round trip.
    public func buildGraph(table: UnsafeBufferPointer<smelt_dispatch_record>) throws {
        try check(smelt_cuda_graph_build(ctx, table.baseAddress, table.count))
    }

    public func graphStep(tokenId: Int32, position: Int32) throws -> Int32 {
        var token = tokenId
        var out: Int32 = -1
        try check(smelt_cuda_graph_step(ctx, &token, position, &out))
        return out
    }
}
