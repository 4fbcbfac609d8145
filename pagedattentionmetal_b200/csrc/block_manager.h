// Host-side bookkeeping of the paged KV cache and the continuous-batching
// scheduler.  Pure C++ (no CUDA): block tables, the free list with its three
// policies, reference counts, the caller-hashed prefix cache and copy-on-write
// decisions of KVCacheManager (KVCacheManager.swift:47-379), and
// ContinuousBatchingScheduler (Scheduler.swift:42-177).  Block tables, free
// counts and batch order are bit-exact with the reference.
#pragma once

#include <cstdint>
#include <deque>
#include <map>
#include <mutex>
#include <string>
#include <unordered_map>
#include <utility>
#include <vector>

namespace pam {

enum class KVStatus { ok, outOfMemory, sequenceNotFound, sequenceAlreadyExists, invalidRequest };

struct KVResult {
    KVStatus status = KVStatus::ok;
    std::string message;
    bool ok() const { return status == KVStatus::ok; }
};

struct LogicalSequence {            // KVCacheManager.swift:34-44
    std::vector<int32_t> blockTable;
    int64_t sequenceLength = 0;
    // Not in the reference: changes whenever an entry that already exists is replaced
    // (copy-on-write) and when the id is allocated again after a free; growing the table
    // leaves it alone.  A holder of a copy of the first n entries needs no more than the
    // entries from n on while this number stays the same.
    uint64_t rewriteVersion = 0;
};

// One sequence as seen under the manager's lock (BlockManager::visit).
struct SequenceView {
    const int32_t* table;
    int32_t numBlocks;
    int64_t length;
    uint64_t rewriteVersion;
};

struct MemoryStats {                // KVCacheManager.swift:19-32 (byte fields filled by the owner)
    int64_t totalBlocks = 0, usedBlocks = 0, freeBlocks = 0, activeSequences = 0;
    int64_t partiallyFilledBlocks = 0;
    float fragmentationRatio = 0.f;
    int64_t prefixCacheHits = 0, prefixCacheEntries = 0, sharedBlocks = 0;
    int policy = 0;
};

class BlockManager {
public:
    enum Policy { fifo = 0, lifo = 1, bestFit = 2 };   // KVCacheManager.swift:13-17

    BlockManager(int maxBlocks, int blockSize);

    // Each copy-on-write (source block, fresh block) is appended to `cow` in the
    // order the reference would have copied the bytes (KVCacheManager.swift:176-194).
    KVResult allocateSequence(int64_t id);
    KVResult appendTokens(int64_t id, int64_t count, const uint64_t* hashes, int numHashes,
                          std::vector<std::pair<int32_t, int32_t>>* cow);
    KVResult ensureExclusiveAccess(int64_t id, int64_t logicalBlock,
                                   std::vector<std::pair<int32_t, int32_t>>* cow);
    void registerBlockHash(uint64_t hash, int32_t block);
    void freeSequence(int64_t id);
    void setPolicy(int policy);
    // Two fixes of reference behaviour, both off by default so that block tables, free
    // counts and hit counts stay bit-exact with the reference:
    //  * a prefix-cache entry is dropped when its block's reference count reaches zero
    //    (the reference keeps the hash and later hands the recycled block to whoever
    //    presents it, KVCacheManager.swift:150-158, 216-239);
    //  * an append that runs out of blocks changes nothing (the reference has already
    //    done the copy-on-write of a shared last block by then, KVCacheManager.swift:134-146,
    //    which leaks the fresh block and drops a reference the sequence still uses).
    void setHygiene(bool on);
    bool hygiene() const;
    // fn(i, view) for ids[0 .. n) in order under one lock; stops at the first unknown id
    // and reports it.
    template <class F> KVResult visit(const int64_t* ids, int n, F fn) const;

    KVResult blockTable(int64_t id, std::vector<int32_t>* out) const;
    KVResult sequenceLength(int64_t id, int64_t* out) const;
    int availableBlocks() const;
    int activeSequences() const;
    MemoryStats stats() const;
    int maxBlocks() const { return maxBlocks_; }
    int blockSize() const { return blockSize_; }

private:
    int32_t allocateBlockLocked();
    KVResult copyOnWriteLocked(int32_t block, size_t index, LogicalSequence& seq,
                               std::vector<std::pair<int32_t, int32_t>>* cow);

    const int maxBlocks_, blockSize_;
    mutable std::mutex mu_;
    std::deque<int32_t> free_;
    std::unordered_map<int32_t, int> freeSizes_;
    int policy_ = fifo;
    std::unordered_map<int64_t, LogicalSequence> sequences_;
    std::unordered_map<uint64_t, int32_t> prefix_;
    std::vector<int32_t> refcounts_;
    int64_t prefixHits_ = 0;
    uint64_t versionCounter_ = 0;
    bool hygiene_ = false;
    std::unordered_map<int32_t, std::vector<uint64_t>> hashesOfBlock_;   // hygiene only
};

template <class F>
KVResult BlockManager::visit(const int64_t* ids, int n, F fn) const {
    std::lock_guard<std::mutex> g(mu_);
    for (int i = 0; i < n; ++i) {
        auto it = sequences_.find(ids[i]);
        if (it == sequences_.end()) return {KVStatus::sequenceNotFound, "sequenceNotFound"};
        const LogicalSequence& q = it->second;
        fn(i, SequenceView{q.blockTable.data(), static_cast<int32_t>(q.blockTable.size()), q.sequenceLength, q.rewriteVersion});
    }
    return {};
}

enum SeqStatus { waiting = 0, running = 1, paused = 2, completed = 3 };   // Scheduler.swift:5-10

struct SchedulerSequence {          // Scheduler.swift:24-40
    int64_t id = 0;
    int status = waiting;
    int numGeneratedTokens = 0, maxNewTokens = 0, promptLength = 0, arrivalOrder = 0;
    bool isDone() const { return numGeneratedTokens >= maxNewTokens; }
};

class Scheduler {
public:
    Scheduler(int maxBatchSize, int maxSequences) : maxBatch_(maxBatchSize), maxSeqs_(maxSequences) {}
    int64_t addRequest(int promptTokens, int maxNewTokens);
    void complete(int64_t id);
    std::vector<int64_t> step();
    void markPrefilled(int64_t id);
    void markDecoded(int64_t id);
    void preempt(int64_t id);
    template <class F> std::vector<int64_t> handleMemoryPressure(int required, F available);
    int count(int status) const;
    int total() const;
    bool get(int64_t id, SchedulerSequence* out) const;

private:
    const int maxBatch_, maxSeqs_;
    mutable std::mutex mu_;
    std::map<int64_t, SchedulerSequence> seqs_;
    int64_t nextId_ = 0;
    int arrival_ = 0;
};

// Scheduler.swift:134-152: newest running sequence is paused, one at a time,
// re-reading the available count before each.
template <class F>
std::vector<int64_t> Scheduler::handleMemoryPressure(int required, F available) {
    std::lock_guard<std::mutex> g(mu_);
    std::vector<int64_t> out;
    while (available() < required) {
        SchedulerSequence* victim = nullptr;
        for (auto& kv : seqs_)
            if (kv.second.status == running && (!victim || kv.second.arrivalOrder > victim->arrivalOrder))
                victim = &kv.second;
        if (!victim) break;
        victim->status = paused;
        out.push_back(victim->id);
    }
    return out;
}

}  // namespace pam
