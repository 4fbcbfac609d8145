// KVCacheManager and BatchKVCacheManager (reference: KVCacheManager.swift:47-703) over
// libpam_cuda.so.  Block tables, the free list with its policies, reference counts, the
// prefix cache and copy-on-write decisions are taken by the library's block manager and are
// bit-exact with the reference; the pools live in HBM, laid out
// [block][kv_head][block_size][head_dim].
import CPamCuda
import Foundation

public class KVCacheManager: @unchecked Sendable {
    let engine: PagedAttentionEngine
    let handle: UnsafeMutableRawPointer
    public let blockSize, headDim, numKVHeads, maxBlocks: Int
    public let dataType: PagedAttentionDataType
    public let kPoolBuffer, vPoolBuffer: PagedBuffer
    /// FP8 caches: float16 scales [block][kv_head]; nil otherwise.
    public let kScaleBuffer, vScaleBuffer: PagedBuffer?

    /// KVCacheManager.swift:76-104
    public init(engine: PagedAttentionEngine, maxBlocks: Int, blockSize: Int, headDim: Int, numKVHeads: Int,
                dataType: PagedAttentionDataType = .float16) throws {
        guard let h = pam_create_cache(engine.ctx, Int32(maxBlocks), Int32(blockSize), Int32(headDim), Int32(numKVHeads),
                                       dataType.rawValue) else { throw lastError(of: engine.ctx) }
        self.engine = engine
        handle = h
        self.maxBlocks = maxBlocks; self.blockSize = blockSize; self.headDim = headDim; self.numKVHeads = numKVHeads
        self.dataType = dataType
        var k: UnsafeMutableRawPointer?, v: UnsafeMutableRawPointer?, ks: UnsafeMutableRawPointer?, vs: UnsafeMutableRawPointer?
        var poolBytes = 0, scaleBytes = 0
        pamc_cache_pools(h, &k, &v, &ks, &vs, &poolBytes, &scaleBytes)
        kPoolBuffer = PagedBuffer(pointer: k, length: poolBytes)
        vPoolBuffer = PagedBuffer(pointer: v, length: poolBytes)
        kScaleBuffer = ks.map { PagedBuffer(pointer: $0, length: scaleBytes) }
        vScaleBuffer = vs.map { PagedBuffer(pointer: $0, length: scaleBytes) }
    }

    deinit { pam_destroy_cache(handle) }

    /// KVCacheManager.swift:65-67
    public var evictionPolicy: BlockEvictionPolicy = .fifo {
        didSet { pamc_cache_set_eviction_policy(handle, evictionPolicy.rawValue) }
    }

    public func allocateSequence(id: Int) throws {                       // :106-113
        try check(engine.ctx, pam_reserve_sequence(engine.ctx, handle, Int64(id)))
    }

    public func appendTokens(toSequence id: Int, count: Int, blockHashes: [UInt64]? = nil) throws {   // :115-174
        if let hashes = blockHashes {
            try check(engine.ctx, pamc_cache_append_tokens(engine.ctx, handle, Int64(id), Int32(count), hashes, Int32(hashes.count)))
        } else {
            try check(engine.ctx, pam_append_tokens(engine.ctx, handle, Int64(id), Int32(count)))
        }
    }

    public func registerBlockHash(_ hash: UInt64, physicalBlock: Int32) {   // :196-198
        pamc_cache_register_block_hash(handle, hash, physicalBlock)
    }

    public func ensureExclusiveAccess(sequenceId: Int, logicalBlockIndex: Int) throws {   // :200-214
        try check(engine.ctx, pamc_cache_ensure_exclusive(engine.ctx, handle, Int64(sequenceId), Int32(logicalBlockIndex)))
    }

    public func freeSequence(id: Int) { pam_free_sequence(handle, Int64(id)) }   // :216-239

    public func getBlockTable(forSequence id: Int) throws -> [Int32] {           // :299-303
        let n = pamc_cache_block_table(engine.ctx, handle, Int64(id), nil, 0)
        if n < 0 { throw lastError(of: engine.ctx) }
        var table = [Int32](repeating: 0, count: Int(n))
        if n > 0 { _ = pamc_cache_block_table(engine.ctx, handle, Int64(id), &table, n) }
        return table
    }

    public func getSequence(id: Int) throws -> LogicalSequence {                  // :323-327
        LogicalSequence(blockTable: try getBlockTable(forSequence: id), sequenceLength: try getSequenceLength(id))
    }

    public func getSequenceLength(_ id: Int) throws -> Int {                      // :329-333
        let n = pam_sequence_length(engine.ctx, handle, Int64(id))
        if n < 0 { throw lastError(of: engine.ctx) }
        return Int(n)
    }

    public func getNumBlocks(forSequence id: Int) throws -> Int {                 // :335-339
        let n = pamc_cache_num_blocks(engine.ctx, handle, Int64(id))
        if n < 0 { throw lastError(of: engine.ctx) }
        return Int(n)
    }

    public var availableBlocks: Int { Int(pam_available_blocks(handle)) }         // :341-345
    public var activeSequenceCount: Int { Int(pamc_cache_active_sequences(handle)) }   // :347-351

    public func memoryStats() -> KVCacheMemoryStats {                             // :353-378
        var s = PamMemoryStats()
        pamc_cache_memory_stats(handle, &s)
        return KVCacheMemoryStats(totalBlocks: Int(s.total_blocks), usedBlocks: Int(s.used_blocks),
                                  freeBlocks: Int(s.free_blocks), activeSequences: Int(s.active_sequences),
                                  totalMemoryBytes: Int(s.total_memory_bytes), usedMemoryBytes: Int(s.used_memory_bytes),
                                  partiallyFilledBlocks: Int(s.partially_filled_blocks),
                                  fragmentationRatio: s.fragmentation_ratio, prefixCacheHits: Int(s.prefix_cache_hits),
                                  prefixCacheEntries: Int(s.prefix_cache_entries), sharedBlocks: Int(s.shared_blocks),
                                  evictionPolicy: BlockEvictionPolicy(rawValue: s.eviction_policy) ?? .fifo)
    }

    // MARK: the attention calls of the reference's C ABI on this cache (PagedAttentionCABI.swift:203-337)

    public func appendKV(sequenceId: Int, keys: PagedBuffer, values: PagedBuffer, tokenOffset: Int, numNewTokens: Int,
                         numHeads: Int) throws {
        try check(engine.ctx, pam_append_kv(engine.ctx, handle, Int64(sequenceId), keys.pointer, values.pointer,
                                            Int32(tokenOffset), Int32(numNewTokens), Int32(numHeads)))
    }

    public func prefill(sequenceId: Int, q: PagedBuffer, output: PagedBuffer, seqLen: Int, numHeads: Int,
                        causal: Bool = true) throws {
        try check(engine.ctx, pam_prefill(engine.ctx, handle, Int64(sequenceId), q.pointer, output.pointer, Int32(seqLen),
                                          Int32(numHeads), causal))
    }

    public func decode(batch ids: [Int], q: PagedBuffer, output: PagedBuffer, numHeads: Int) throws {
        let ids64 = ids.map { Int64($0) }
        try check(engine.ctx, pam_decode(engine.ctx, handle, ids64, Int32(ids64.count), q.pointer, output.pointer, Int32(numHeads)))
    }
}

/// BatchKVCacheManager (KVCacheManager.swift:382-703): the same manager plus zero-padded
/// [maxBatchSize][maxSequenceBlocks] block tables and [maxBatchSize] lengths in device slabs
/// that every call overwrites.
public final class BatchKVCacheManager: KVCacheManager, @unchecked Sendable {
    public let maxBatchSize, maxSequenceBlocks: Int
    public let blockTablesSlab, seqLengthsSlab: PagedBuffer

    public init(engine: PagedAttentionEngine, maxBatchSize: Int, maxSequenceBlocks: Int, maxBlocks: Int, blockSize: Int,
                headDim: Int, numKVHeads: Int, dataType: PagedAttentionDataType = .float16) throws {   // :413-453
        self.maxBatchSize = maxBatchSize
        self.maxSequenceBlocks = maxSequenceBlocks
        blockTablesSlab = try engine.makeBuffer(length: maxBatchSize * maxSequenceBlocks * MemoryLayout<Int32>.size)
        seqLengthsSlab = try engine.makeBuffer(length: maxBatchSize * MemoryLayout<UInt32>.size)
        try super.init(engine: engine, maxBlocks: maxBlocks, blockSize: blockSize, headDim: headDim, numKVHeads: numKVHeads,
                       dataType: dataType)
    }

    deinit {
        engine.free(blockTablesSlab)
        engine.free(seqLengthsSlab)
    }

    private func fill(_ batch: [Int]) throws {
        if batch.count > maxBatchSize { throw KVCacheError.outOfMemory }            // :664-666
        let ids = batch.map { Int64($0) }
        try check(engine.ctx, pamc_cache_batch_tables(engine.ctx, handle, ids, Int32(ids.count), Int32(maxSequenceBlocks),
                                                      blockTablesSlab.pointer?.assumingMemoryBound(to: Int32.self),
                                                      seqLengthsSlab.pointer?.assumingMemoryBound(to: UInt32.self)))
    }

    public func getBatchBlockTableBuffer(forBatch batch: [Int]) throws -> PagedBuffer {   // :661-688
        try fill(batch)
        return blockTablesSlab
    }

    public func getSeqLengthsBuffer(forBatch batch: [Int]) throws -> PagedBuffer {        // :690-703
        try fill(batch)
        return seqLengthsSlab
    }
}
