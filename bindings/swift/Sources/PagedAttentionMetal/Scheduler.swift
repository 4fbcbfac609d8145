// ContinuousBatchingScheduler (reference: Scheduler.swift:42-177) and PagedAttentionInference
// (reference: PagedAttentionInference.swift:7-299) over libpam_cuda.so; batch order, status
// changes and victim order are those of the reference.
import CPamCuda
import Foundation

public final class ContinuousBatchingScheduler: @unchecked Sendable {
    let handle: UnsafeMutableRawPointer
    private let owned: Bool
    public let maxBatchSize: Int

    public init(maxBatchSize: Int, maxSequences: Int = 128) {                     // :53-56
        handle = pamc_sched_create(Int32(maxBatchSize), Int32(maxSequences))
        owned = true
        self.maxBatchSize = maxBatchSize
    }

    init(borrowing handle: UnsafeMutableRawPointer, maxBatchSize: Int) {
        self.handle = handle
        owned = false
        self.maxBatchSize = maxBatchSize
    }

    deinit { if owned { pamc_sched_destroy(handle) } }

    public func sequence(id: Int) -> SchedulerSequence? {
        var s = PamSchedSequence()
        guard pamc_sched_get(handle, Int64(id), &s) == 0 else { return nil }
        return SchedulerSequence(id: Int(s.id), status: SequenceStatus(rawValue: s.status) ?? .waiting,
                                 numGeneratedTokens: Int(s.num_generated_tokens), maxNewTokens: Int(s.max_new_tokens),
                                 promptLength: Int(s.prompt_length), arrivalOrder: Int(s.arrival_order))
    }

    public func addRequest(promptTokenCount: Int, maxNewTokens: Int) -> Int {     // :58-70
        Int(pamc_sched_add_request(handle, Int32(promptTokenCount), Int32(maxNewTokens)))
    }

    public func completeSequence(id: Int) { pamc_sched_complete(handle, Int64(id)) }   // :72-76

    public func step() -> [SchedulerSequence] {                                   // :78-114
        var ids = [Int64](repeating: 0, count: max(maxBatchSize, 1))
        let n = Int(pamc_sched_step(handle, &ids, Int32(ids.count)))
        return ids.prefix(max(min(n, ids.count), 0)).compactMap { sequence(id: Int($0)) }
    }

    public func markPrefilled(id: Int) { pamc_sched_mark_prefilled(handle, Int64(id)) }     // :116-120
    public func markDecoded(id: Int) { pamc_sched_mark_decoded(handle, Int64(id)) }         // :122-126
    public func preemptSequence(id: Int) { pamc_sched_preempt(handle, Int64(id)) }          // :128-132

    /// :134-152 -- `availableBlocks` is evaluated before every preemption, like the reference's autoclosure.
    public func handleMemoryPressure(requiredBlocks: Int, availableBlocks: @escaping () -> Int) -> [Int] {
        final class Box { let f: () -> Int; init(_ f: @escaping () -> Int) { self.f = f } }
        let box = Box(availableBlocks)
        var ids = [Int64](repeating: 0, count: 1024)
        let n = withExtendedLifetime(box) {
            pamc_sched_handle_memory_pressure(handle, Int32(requiredBlocks), { user in
                Int32(Unmanaged<Box>.fromOpaque(user!).takeUnretainedValue().f())
            }, Unmanaged.passUnretained(box).toOpaque(), &ids, Int32(ids.count))
        }
        return ids.prefix(max(Int(n), 0)).map { Int($0) }
    }

    public var waitingCount: Int { Int(pamc_sched_count(handle, SequenceStatus.waiting.rawValue)) }       // :154-158
    public var runningCount: Int { Int(pamc_sched_count(handle, SequenceStatus.running.rawValue)) }       // :160-164
    public var completedCount: Int { Int(pamc_sched_count(handle, SequenceStatus.completed.rawValue)) }   // :166-170
    public var totalSequencesProcessed: Int { Int(pamc_sched_total(handle)) }                              // :172-176
}

public final class PagedAttentionInference: @unchecked Sendable {
    public let engine: PagedAttentionEngine
    public let scheduler: ContinuousBatchingScheduler
    let handle: UnsafeMutableRawPointer

    /// PagedAttentionInference.swift:47-90
    public init(engine: PagedAttentionEngine, maxBlocks: Int, blockSize: Int, layerSpecs: [PagedLayerSpec],
                maxBatchSize: Int = 16, maxSequences: Int = 128) throws {
        let specs = layerSpecs.map { $0.c }
        guard let h = pamc_infer_create(engine.ctx, Int32(maxBlocks), Int32(blockSize), specs, Int32(specs.count),
                                        Int32(maxBatchSize), Int32(maxSequences)) else { throw lastError(of: engine.ctx) }
        self.engine = engine
        handle = h
        scheduler = ContinuousBatchingScheduler(borrowing: pamc_infer_scheduler(h), maxBatchSize: maxBatchSize)
    }

    deinit { pamc_infer_destroy(handle) }

    public func addRequest(promptTokenCount: Int, maxNewTokens: Int) -> Int {     // :103-105
        Int(pamc_infer_add_request(handle, Int32(promptTokenCount), Int32(maxNewTokens)))
    }

    public func completeSequence(id: Int) { pamc_infer_complete_sequence(handle, Int64(id)) }   // :108-114

    @discardableResult
    public func step() throws -> [Int] {                                          // :119-148
        var ids = [Int64](repeating: 0, count: max(scheduler.maxBatchSize, 1))
        let n = pamc_infer_step(handle, &ids, Int32(ids.count))
        if n < 0 { throw lastError(of: engine.ctx) }
        return ids.prefix(min(Int(n), ids.count)).map { Int($0) }
    }

    public func runAll() throws { try check(engine.ctx, pamc_infer_run_all(handle)) }   // :151-156

    public var totalTokensGenerated: Int { Int(pamc_infer_total_tokens(handle)) }       // :166-170
    public var stepCount: Int { Int(pamc_infer_step_count(handle)) }                    // :34

    /// One prefill launch per layer and step for all prompts of the step, optionally bounded
    /// to `tokenBudget` prompt rows per step (not in the reference; off by default).
    public func setBatchedPrefill(_ on: Bool, tokenBudget: Int = 0) {
        pamc_infer_set_batched_prefill(handle, on ? 1 : 0, Int32(tokenBudget))
    }
}
