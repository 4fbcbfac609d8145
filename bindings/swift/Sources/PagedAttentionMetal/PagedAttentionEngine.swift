// PagedAttentionEngine (reference: PagedAttentionEngine.swift:82) over libpam_cuda.so.
// Every operation is one pamc_* call; validation, the retry loop, the circuit breaker,
// graceful degradation and the statistics live in the library and behave like the
// reference's (PagedAttentionEngine.swift:375-414, 1897-1950).
import CPamCuda
import Foundation

public final class PagedAttentionEngine: @unchecked Sendable {
    let ctx: UnsafeMutableRawPointer
    /// CUDA device ordinal the engine runs on (the reference's private MTLDevice).
    public let deviceIndex: Int

    /// PagedAttentionEngine.swift:248 -- the current CUDA device.
    public convenience init() throws {
        try self.init(deviceIndex: nil)
    }

    public init(deviceIndex: Int?) throws {
        let handle = deviceIndex.map { pamc_create_context_on(Int32($0)) } ?? pam_create_context()
        guard let handle else { throw PagedAttentionError.deviceInitializationFailed }
        ctx = handle
        self.deviceIndex = deviceIndex ?? 0
    }

    deinit { pam_destroy_context(ctx) }

    // MARK: properties (PagedAttentionEngine.swift:116-129)

    public var splitThreshold: Int = 1024 { didSet { pamc_set_split_threshold(ctx, Int32(splitThreshold)) } }
    public var defaultWindowSize: Int = 0 { didSet { pamc_set_default_window(ctx, Int32(defaultWindowSize)) } }
    public var defaultChunkSize: Int = 0 { didSet { pamc_set_default_chunk(ctx, Int32(defaultChunkSize)) } }
    public var maxRetries: Int = 3 { didSet { pamc_set_max_retries(ctx, Int32(maxRetries)) } }
    public var enableGracefulDegradation: Bool = true {
        didSet { pamc_set_graceful_degradation(ctx, enableGracefulDegradation ? 1 : 0) }
    }

    /// PagedAttentionEngine.swift:137-141
    public var lastStats: PagedAttentionStats {
        var s = PamStats()
        pamc_last_stats(ctx, &s)
        return PagedAttentionStats(operation: PagedAttentionStats.Operation(rawValue: s.operation) ?? .none,
                                   batchSize: Int(s.batch_size), sequenceLength: Int(s.sequence_length),
                                   numBlocks: Int(s.num_blocks), temporaryBytes: Int(s.temporary_bytes),
                                   usedSplitPass: s.used_split_pass != 0, elapsedMilliseconds: s.elapsed_ms)
    }

    /// PagedAttentionEngine.swift:144-148
    public var lastError: String? { pam_last_error(ctx).map { String(cString: $0) } }

    /// recommendedMaxBlocks (PagedAttentionEngine.swift:201-217) with free device memory in
    /// place of recommendedMaxWorkingSetSize.
    public func recommendedMaxBlocks(blockSize: Int, numKVHeads: Int, headDim: Int, dataType: PagedAttentionDataType,
                                     memoryFraction: Float = 0.75, layerCount: Int = 1) -> Int {
        Int(pamc_recommended_max_blocks(ctx, Int32(blockSize), Int32(numKVHeads), Int32(headDim), dataType.rawValue,
                                        memoryFraction, Int32(layerCount)))
    }

    // MARK: device memory for callers without a CUDA runtime of their own

    public func makeBuffer(length: Int) throws -> PagedBuffer {
        guard let p = pamc_buffer_alloc(ctx, length) else {
            throw PagedAttentionError.resourceExhausted("GPU resource exhausted: cannot allocate \(length) bytes")
        }
        return PagedBuffer(pointer: p, length: length)
    }

    public func free(_ buffer: PagedBuffer) { pamc_buffer_free(ctx, buffer.pointer) }

    public func upload(_ bytes: UnsafeRawBufferPointer, to buffer: PagedBuffer) throws {
        try check(ctx, pamc_memcpy(ctx, buffer.pointer, bytes.baseAddress, min(bytes.count, buffer.length), 0))
    }

    public func download(_ buffer: PagedBuffer, into bytes: UnsafeMutableRawBufferPointer) throws {
        try check(ctx, pamc_memcpy(ctx, bytes.baseAddress, buffer.pointer, min(bytes.count, buffer.length), 1))
    }

    // MARK: operations, request form (PagedAttentionEngine.swift:405, 533, 585, 633)

    public func prefill(_ r: PagedAttentionPrefillRequest, chunkSize: Int = 0) throws {
        var c = PamPrefillRequest(q: r.q.c, k_pool: r.kPool.c, v_pool: r.vPool.c, block_table: r.blockTable.c,
                                  output: r.output.c, seq_len: Int32(r.seqLen), layer: r.layer.c,
                                  causal: r.causal ? 1 : 0, k_scale: r.kScaleBuffer.c, v_scale: r.vScaleBuffer.c,
                                  q_start: 0, q_len: 0)
        try check(ctx, pamc_prefill(ctx, &c, Int32(chunkSize)))
    }

    public func decode(_ r: PagedAttentionDecodeRequest) throws {
        var c = PamDecodeRequest(q: r.q.c, k_pool: r.kPool.c, v_pool: r.vPool.c, block_tables: r.blockTables.c,
                                 seq_lengths: r.seqLengths.c, output: r.output.c, batch_size: Int32(r.batchSize),
                                 max_num_blocks: Int32(r.maxNumBlocks), layer: r.layer.c,
                                 k_scale: r.kScaleBuffer.c, v_scale: r.vScaleBuffer.c)
        try check(ctx, pamc_decode(ctx, &c))
    }

    public func appendToCache(_ r: PagedKVAppendRequest) throws {
        var c = PamAppendRequest(keys: r.keys.c, values: r.values.c, k_pool: r.kPool.c, v_pool: r.vPool.c,
                                 block_table: r.blockTable.c, token_offset: Int32(r.tokenOffset),
                                 num_new_tokens: Int32(r.numNewTokens), layer: r.layer.c,
                                 k_scale: r.kScaleBuffer.c, v_scale: r.vScaleBuffer.c)
        try check(ctx, pamc_append_to_cache(ctx, &c))
    }

    /// cache: the manager that owns the pools (required for FP8, which needs its scale rows).
    public func fusedPrefill(_ r: PagedAttentionFusedPrefillRequest, cache: KVCacheManager? = nil) throws {
        var c = PamFusedPrefillRequest(q: r.q.c, raw_k: r.rawK.c, raw_v: r.rawV.c, block_table: r.blockTable.c,
                                       k_pool: r.kPool.c, v_pool: r.vPool.c, output: r.output.c, seq_len: Int32(r.seqLen),
                                       layer: r.layer.c, causal: r.causal ? 1 : 0, k_scale: r.kScaleBuffer.c,
                                       v_scale: r.vScaleBuffer.c)
        try check(ctx, pamc_fused_prefill(ctx, &c, cache?.handle))
    }

    /// PagedAttentionEngine.swift:1341-1395: dQ is written, dKPool and dVPool are added to; m and l are
    /// the float32 row maximum and row sum of the caller's forward pass, [seqLen][numHeads].
    public func backward(q: PagedBuffer, kPool: PagedBuffer, vPool: PagedBuffer, blockTable: PagedBuffer, dO: PagedBuffer,
                         m: PagedBuffer, l: PagedBuffer, dQ: PagedBuffer, dKPool: PagedBuffer, dVPool: PagedBuffer,
                         seqLen: Int, headDim: Int, numHeads: Int, numKVHeads: Int, blockSize: Int,
                         dataType: PagedAttentionDataType = .float32, windowSize: Int = 0) throws {
        let layer = PagedLayerSpec(headDim: headDim, numHeads: numHeads, numKVHeads: numKVHeads, blockSize: blockSize,
                                   dataType: dataType, windowSize: windowSize)
        var c = PamBackwardRequest(q: q.c, k_pool: kPool.c, v_pool: vPool.c, block_table: blockTable.c, d_out: dO.c,
                                   m: m.c, l: l.c, d_q: dQ.c, d_k_pool: dKPool.c, d_v_pool: dVPool.c,
                                   seq_len: Int32(seqLen), layer: layer.c)
        try check(ctx, pamc_backward(ctx, &c))
    }

    // MARK: operations, flat form (PagedAttentionEngine.swift:713, 1012, 1167)

    public func prefill(q: PagedBuffer, kPool: PagedBuffer, vPool: PagedBuffer, blockTable: PagedBuffer, seqLen: Int,
                        headDim: Int, numHeads: Int, numKVHeads: Int, blockSize: Int, causal: Bool = true,
                        output: PagedBuffer, dataType: PagedAttentionDataType = .float16, windowSize: Int = 0,
                        chunkSize: Int = 0) throws {
        let layer = PagedLayerSpec(headDim: headDim, numHeads: numHeads, numKVHeads: numKVHeads, blockSize: blockSize,
                                   dataType: dataType, windowSize: windowSize)
        try prefill(PagedAttentionPrefillRequest(q: q, kPool: kPool, vPool: vPool, blockTable: blockTable, output: output,
                                                 seqLen: seqLen, layer: layer, causal: causal), chunkSize: chunkSize)
    }

    public func decode(q: PagedBuffer, kPool: PagedBuffer, vPool: PagedBuffer, blockTables: PagedBuffer,
                       seqLengths: PagedBuffer, batchSize: Int, maxNumBlocks: Int, headDim: Int, numHeads: Int,
                       numKVHeads: Int, blockSize: Int, output: PagedBuffer, dataType: PagedAttentionDataType = .float16,
                       windowSize: Int = 0) throws {
        let layer = PagedLayerSpec(headDim: headDim, numHeads: numHeads, numKVHeads: numKVHeads, blockSize: blockSize,
                                   dataType: dataType, windowSize: windowSize)
        try decode(PagedAttentionDecodeRequest(q: q, kPool: kPool, vPool: vPool, blockTables: blockTables,
                                               seqLengths: seqLengths, output: output, batchSize: batchSize,
                                               maxNumBlocks: maxNumBlocks, layer: layer))
    }

    public func appendToCache(keys: PagedBuffer, values: PagedBuffer, kPool: PagedBuffer, vPool: PagedBuffer,
                              blockTable: PagedBuffer, tokenOffset: Int, numNewTokens: Int, numHeads: Int,
                              numKVHeads: Int, headDim: Int, blockSize: Int,
                              dataType: PagedAttentionDataType = .float16, windowSize: Int = 0) throws {
        let layer = PagedLayerSpec(headDim: headDim, numHeads: numHeads, numKVHeads: numKVHeads, blockSize: blockSize,
                                   dataType: dataType, windowSize: windowSize)
        try appendToCache(PagedKVAppendRequest(keys: keys, values: values, kPool: kPool, vPool: vPool,
                                               blockTable: blockTable, tokenOffset: tokenOffset,
                                               numNewTokens: numNewTokens, layer: layer))
    }

    // MARK: batched-layer calls (PagedAttentionEngine.swift:1433, 1641, 1744)

    public func decodeLayers(_ requests: [PagedAttentionDecodeRequest]) throws {
        var c = requests.map {
            PamDecodeRequest(q: $0.q.c, k_pool: $0.kPool.c, v_pool: $0.vPool.c, block_tables: $0.blockTables.c,
                             seq_lengths: $0.seqLengths.c, output: $0.output.c, batch_size: Int32($0.batchSize),
                             max_num_blocks: Int32($0.maxNumBlocks), layer: $0.layer.c, k_scale: $0.kScaleBuffer.c,
                             v_scale: $0.vScaleBuffer.c)
        }
        try check(ctx, pamc_decode_layers(ctx, &c, Int32(c.count)))
    }

    public func prefillLayers(_ requests: [PagedAttentionPrefillRequest]) throws {
        var c = requests.map {
            PamPrefillRequest(q: $0.q.c, k_pool: $0.kPool.c, v_pool: $0.vPool.c, block_table: $0.blockTable.c,
                              output: $0.output.c, seq_len: Int32($0.seqLen), layer: $0.layer.c,
                              causal: $0.causal ? 1 : 0, k_scale: $0.kScaleBuffer.c, v_scale: $0.vScaleBuffer.c,
                              q_start: 0, q_len: 0)
        }
        try check(ctx, pamc_prefill_layers(ctx, &c, Int32(c.count)))
    }

    public func appendLayers(_ requests: [PagedKVAppendRequest], caches: [KVCacheManager?] = []) throws {
        var c = requests.map {
            PamAppendRequest(keys: $0.keys.c, values: $0.values.c, k_pool: $0.kPool.c, v_pool: $0.vPool.c,
                             block_table: $0.blockTable.c, token_offset: Int32($0.tokenOffset),
                             num_new_tokens: Int32($0.numNewTokens), layer: $0.layer.c, k_scale: $0.kScaleBuffer.c,
                             v_scale: $0.vScaleBuffer.c)
        }
        var handles: [UnsafeMutableRawPointer?] = caches.map { $0?.handle }
        if handles.isEmpty {
            try check(ctx, pamc_append_layers(ctx, &c, Int32(c.count), nil))
        } else {
            try check(ctx, pamc_append_layers(ctx, &c, Int32(c.count), &handles))
        }
    }
}
