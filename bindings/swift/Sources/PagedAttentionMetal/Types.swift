// Value types of the PagedAttentionMetal API (reference: PagedAttentionTypes.swift,
// KVCacheManager.swift:6-44, Scheduler.swift:5-40) for the CUDA build.  Names, cases, fields
// and raw values are the reference's; an MTLBuffer becomes a PagedBuffer (device or host
// pointer plus its length) and an MTLDevice a CUDA device ordinal.
import CPamCuda
import Foundation

/// PagedAttentionError (PagedAttentionTypes.swift:5-64).  `description` is what the library
/// stored for the failing call (the reference's texts).
public enum PagedAttentionError: Error, CustomStringConvertible {
    case deviceInitializationFailed
    case invalidConfiguration(String)
    case bufferTooSmall(String)
    case commandEncodingFailed(String)
    case commandExecutionFailed(String)
    case unsupportedPath(String)
    case resourceExhausted(String)
    case invalidState(String)
    case recurringFailure(String)

    public var description: String {
        switch self {
        case .deviceInitializationFailed: return "Metal device or command queue could not be initialized."
        case .invalidConfiguration(let m), .bufferTooSmall(let m), .commandEncodingFailed(let m),
             .commandExecutionFailed(let m), .unsupportedPath(let m), .resourceExhausted(let m),
             .invalidState(let m), .recurringFailure(let m):
            return m
        }
    }
}

/// KVCacheError (KVCacheManager.swift:6-11).
public enum KVCacheError: Error {
    case outOfMemory
    case sequenceNotFound
    case sequenceAlreadyExists
    case invalidRequest(String)
}

/// The error of the last failed call on a context, as the matching Swift error.
func lastError(of ctx: UnsafeMutableRawPointer?) -> Error {
    let code = pamc_last_error_code(ctx)
    let text = pam_last_error(ctx).map { String(cString: $0) } ?? "unknown error"
    switch code {
    case Int32(PAM_ERR_DEVICE_INIT): return PagedAttentionError.deviceInitializationFailed
    case Int32(PAM_ERR_INVALID_CONFIGURATION): return PagedAttentionError.invalidConfiguration(text)
    case Int32(PAM_ERR_BUFFER_TOO_SMALL): return PagedAttentionError.bufferTooSmall(text)
    case Int32(PAM_ERR_COMMAND_ENCODING): return PagedAttentionError.commandEncodingFailed(text)
    case Int32(PAM_ERR_UNSUPPORTED): return PagedAttentionError.unsupportedPath(text)
    case Int32(PAM_ERR_RESOURCE_EXHAUSTED): return PagedAttentionError.resourceExhausted(text)
    case Int32(PAM_ERR_INVALID_STATE): return PagedAttentionError.invalidState(text)
    case Int32(PAM_ERR_RECURRING): return PagedAttentionError.recurringFailure(text)
    case Int32(PAM_ERR_KV_OUT_OF_MEMORY): return KVCacheError.outOfMemory
    case Int32(PAM_ERR_KV_SEQUENCE_NOT_FOUND): return KVCacheError.sequenceNotFound
    case Int32(PAM_ERR_KV_SEQUENCE_EXISTS): return KVCacheError.sequenceAlreadyExists
    case Int32(PAM_ERR_KV_INVALID_REQUEST): return KVCacheError.invalidRequest(text)
    default: return PagedAttentionError.commandExecutionFailed(text)
    }
}

@inline(__always) func check(_ ctx: UnsafeMutableRawPointer?, _ rc: Int32) throws {
    if rc != 0 { throw lastError(of: ctx) }
}

/// PagedAttentionDataType (PagedAttentionTypes.swift:67-91); bfloat16 is an addition.
public enum PagedAttentionDataType: Int32, Sendable {
    case float32 = 0
    case float16 = 1
    case float8 = 2
    case bfloat16 = 3

    /// Bytes of one stored element.
    public var byteWidth: Int { self == .float32 ? 4 : self == .float8 ? 1 : 2 }
    /// Bytes of one query / output / new K-V element (float16 for an FP8 cache).
    public var ioByteWidth: Int { self == .float32 ? 4 : 2 }
}

/// What stands in for an MTLBuffer: bytes in CUDA device memory, or in host memory that the
/// library stages for the duration of a call.
public struct PagedBuffer: @unchecked Sendable {
    public var pointer: UnsafeMutableRawPointer?
    public var length: Int
    public init(pointer: UnsafeMutableRawPointer?, length: Int) {
        self.pointer = pointer
        self.length = length
    }
    var c: PamBuffer { PamBuffer(ptr: pointer, bytes: length) }
    static let none = PagedBuffer(pointer: nil, length: 0)
}

/// PagedLayerSpec (PagedAttentionTypes.swift:94-152).
public struct PagedLayerSpec: Sendable {
    public var headDim: Int
    public var numHeads: Int
    public var numKVHeads: Int
    public var blockSize: Int
    public var dataType: PagedAttentionDataType
    public var windowSize: Int

    public init(headDim: Int, numHeads: Int, numKVHeads: Int, blockSize: Int,
                dataType: PagedAttentionDataType = .float16, windowSize: Int = 0) {
        self.headDim = headDim
        self.numHeads = numHeads
        self.numKVHeads = numKVHeads
        self.blockSize = blockSize
        self.dataType = dataType
        self.windowSize = windowSize
    }

    /// PagedAttentionTypes.swift:126-142
    public func validate() throws {
        if headDim <= 0 { throw PagedAttentionError.invalidConfiguration("headDim must be positive.") }
        if numHeads <= 0 { throw PagedAttentionError.invalidConfiguration("numHeads must be positive.") }
        if numKVHeads <= 0 { throw PagedAttentionError.invalidConfiguration("numKVHeads must be positive.") }
        if numHeads % numKVHeads != 0 {
            throw PagedAttentionError.invalidConfiguration("numHeads must be divisible by numKVHeads for GQA/MQA mapping.")
        }
        if blockSize <= 0 { throw PagedAttentionError.invalidConfiguration("blockSize must be positive.") }
    }

    public var groupSize: Int { numHeads / numKVHeads }
    public var qBytesPerToken: Int { numHeads * headDim * dataType.byteWidth }
    public var kvBytesPerToken: Int { numKVHeads * headDim * dataType.byteWidth }

    var c: PamLayerSpec {
        PamLayerSpec(head_dim: Int32(headDim), num_heads: Int32(numHeads), num_kv_heads: Int32(numKVHeads),
                     block_size: Int32(blockSize), data_type: dataType.rawValue, window_size: Int32(windowSize))
    }
}

/// PagedAttentionStats (PagedAttentionTypes.swift:169-207).
public struct PagedAttentionStats: Sendable {
    public enum Operation: Int32, Sendable {
        case none = 0, prefillSinglePass, prefillMMA, prefillFlash, prefillTiledPass, decode, append, backward
    }
    public var operation: Operation = .none
    public var batchSize = 0
    public var sequenceLength = 0
    public var numBlocks = 0
    public var temporaryBytes = 0
    public var usedSplitPass = false
    public var elapsedMilliseconds = 0.0
}

/// PagedAttentionPrefillRequest (PagedAttentionTypes.swift:210-256).
public struct PagedAttentionPrefillRequest {
    public var q, kPool, vPool, blockTable, output: PagedBuffer
    public var seqLen: Int
    public var layer: PagedLayerSpec
    public var causal: Bool
    public var kScaleBuffer, vScaleBuffer: PagedBuffer
    public init(q: PagedBuffer, kPool: PagedBuffer, vPool: PagedBuffer, blockTable: PagedBuffer, output: PagedBuffer,
                seqLen: Int, layer: PagedLayerSpec, causal: Bool = true,
                kScaleBuffer: PagedBuffer? = nil, vScaleBuffer: PagedBuffer? = nil) {
        self.q = q; self.kPool = kPool; self.vPool = vPool; self.blockTable = blockTable; self.output = output
        self.seqLen = seqLen; self.layer = layer; self.causal = causal
        self.kScaleBuffer = kScaleBuffer ?? .none; self.vScaleBuffer = vScaleBuffer ?? .none
    }
}

/// PagedAttentionDecodeRequest (PagedAttentionTypes.swift:259-315).
public struct PagedAttentionDecodeRequest {
    public var q, kPool, vPool, blockTables, seqLengths, output: PagedBuffer
    public var batchSize, maxNumBlocks: Int
    public var layer: PagedLayerSpec
    public var kScaleBuffer, vScaleBuffer: PagedBuffer
    public init(q: PagedBuffer, kPool: PagedBuffer, vPool: PagedBuffer, blockTables: PagedBuffer, seqLengths: PagedBuffer,
                output: PagedBuffer, batchSize: Int, maxNumBlocks: Int, layer: PagedLayerSpec,
                kScaleBuffer: PagedBuffer? = nil, vScaleBuffer: PagedBuffer? = nil) {
        self.q = q; self.kPool = kPool; self.vPool = vPool; self.blockTables = blockTables; self.seqLengths = seqLengths
        self.output = output; self.batchSize = batchSize; self.maxNumBlocks = maxNumBlocks; self.layer = layer
        self.kScaleBuffer = kScaleBuffer ?? .none; self.vScaleBuffer = vScaleBuffer ?? .none
    }
}

/// PagedKVAppendRequest (PagedAttentionTypes.swift:318-364).
public struct PagedKVAppendRequest {
    public var keys, values, kPool, vPool, blockTable: PagedBuffer
    public var tokenOffset, numNewTokens: Int
    public var layer: PagedLayerSpec
    public var kScaleBuffer, vScaleBuffer: PagedBuffer
    public init(keys: PagedBuffer, values: PagedBuffer, kPool: PagedBuffer, vPool: PagedBuffer, blockTable: PagedBuffer,
                tokenOffset: Int, numNewTokens: Int, layer: PagedLayerSpec,
                kScaleBuffer: PagedBuffer? = nil, vScaleBuffer: PagedBuffer? = nil) {
        self.keys = keys; self.values = values; self.kPool = kPool; self.vPool = vPool; self.blockTable = blockTable
        self.tokenOffset = tokenOffset; self.numNewTokens = numNewTokens; self.layer = layer
        self.kScaleBuffer = kScaleBuffer ?? .none; self.vScaleBuffer = vScaleBuffer ?? .none
    }
}

/// PagedAttentionFusedPrefillRequest (PagedAttentionTypes.swift:367-421).
public struct PagedAttentionFusedPrefillRequest {
    public var q, rawK, rawV, blockTable, kPool, vPool, output: PagedBuffer
    public var seqLen: Int
    public var layer: PagedLayerSpec
    public var causal: Bool
    public var kScaleBuffer, vScaleBuffer: PagedBuffer
    public init(q: PagedBuffer, rawK: PagedBuffer, rawV: PagedBuffer, blockTable: PagedBuffer, kPool: PagedBuffer,
                vPool: PagedBuffer, output: PagedBuffer, seqLen: Int, layer: PagedLayerSpec, causal: Bool = true,
                kScaleBuffer: PagedBuffer? = nil, vScaleBuffer: PagedBuffer? = nil) {
        self.q = q; self.rawK = rawK; self.rawV = rawV; self.blockTable = blockTable; self.kPool = kPool; self.vPool = vPool
        self.output = output; self.seqLen = seqLen; self.layer = layer; self.causal = causal
        self.kScaleBuffer = kScaleBuffer ?? .none; self.vScaleBuffer = vScaleBuffer ?? .none
    }
}

/// BlockEvictionPolicy (KVCacheManager.swift:13-17).
public enum BlockEvictionPolicy: Int32, Sendable { case fifo = 0, lifo = 1, bestFit = 2 }

/// KVCacheMemoryStats (KVCacheManager.swift:19-32).
public struct KVCacheMemoryStats: Sendable {
    public var totalBlocks, usedBlocks, freeBlocks, activeSequences: Int
    public var totalMemoryBytes, usedMemoryBytes: Int
    public var partiallyFilledBlocks: Int
    public var fragmentationRatio: Float
    public var prefixCacheHits, prefixCacheEntries, sharedBlocks: Int
    public var evictionPolicy: BlockEvictionPolicy
}

/// LogicalSequence (KVCacheManager.swift:34-44).
public struct LogicalSequence: Sendable {
    public var blockTable: [Int32]
    public var sequenceLength: Int
}

/// SequenceStatus (Scheduler.swift:5-10) and SchedulerSequence (Scheduler.swift:24-40).
public enum SequenceStatus: Int32, Sendable { case waiting = 0, running, paused, completed }

public struct SchedulerSequence: Sendable {
    public var id: Int
    public var status: SequenceStatus
    public var numGeneratedTokens, maxNewTokens, promptLength, arrivalOrder: Int
    public var isDone: Bool { numGeneratedTokens >= maxNewTokens }
}
