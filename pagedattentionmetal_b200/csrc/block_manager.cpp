// See block_manager.h.  Every method names the reference lines it follows.
#include "block_manager.h"

#include <algorithm>
#include <climits>
#include <cstdlib>

namespace pam {

BlockManager::BlockManager(int maxBlocks, int blockSize)
    : maxBlocks_(maxBlocks), blockSize_(blockSize), refcounts_(static_cast<size_t>(maxBlocks), 0) {
    // KVCacheManager.swift:101 -- the deque holds max-1 ... 0 and blocks are
    // taken from its back, so a fresh manager hands out 0, 1, 2, ...
    for (int b = maxBlocks - 1; b >= 0; --b) free_.push_back(b);
}

KVResult BlockManager::allocateSequence(int64_t id) {          // KVCacheManager.swift:106-113
    std::lock_guard<std::mutex> g(mu_);
    if (sequences_.count(id)) return {KVStatus::sequenceAlreadyExists, "sequenceAlreadyExists"};
    LogicalSequence fresh;
    fresh.rewriteVersion = ++versionCounter_;
    sequences_[id] = std::move(fresh);
    return {};
}

int32_t BlockManager::allocateBlockLocked() {                  // KVCacheManager.swift:241-265
    if (policy_ != bestFit) {
        int32_t b = free_.back();
        free_.pop_back();
        return b;
    }
    size_t bestIdx = 0;
    long bestDelta = LONG_MAX;
    for (size_t i = 0; i < free_.size(); ++i) {
        auto it = freeSizes_.find(free_[i]);
        int held = it == freeSizes_.end() ? blockSize_ : it->second;
        long delta = std::labs(static_cast<long>(held) - blockSize_);
        if (delta < bestDelta) { bestDelta = delta; bestIdx = i; }
    }
    int32_t b = free_[bestIdx];
    free_.erase(free_.begin() + static_cast<std::ptrdiff_t>(bestIdx));
    freeSizes_.erase(b);
    return b;
}

KVResult BlockManager::copyOnWriteLocked(int32_t block, size_t index, LogicalSequence& seq,
                                         std::vector<std::pair<int32_t, int32_t>>* cow) {
    // KVCacheManager.swift:176-194; the byte copy itself is done by the owner
    // of the pools from the (block, fresh) pair recorded here.
    if (free_.empty()) return {KVStatus::outOfMemory, "outOfMemory"};
    int32_t fresh = allocateBlockLocked();
    if (cow) cow->emplace_back(block, fresh);
    refcounts_[static_cast<size_t>(block)] -= 1;
    refcounts_[static_cast<size_t>(fresh)] = 1;
    seq.blockTable[index] = fresh;
    seq.rewriteVersion = ++versionCounter_;
    return {};
}

KVResult BlockManager::appendTokens(int64_t id, int64_t count, const uint64_t* hashes, int numHashes,
                                    std::vector<std::pair<int32_t, int32_t>>* cow) {
    // KVCacheManager.swift:115-174
    std::lock_guard<std::mutex> g(mu_);
    if (count < 0) return {KVStatus::invalidRequest, "count must be non-negative"};
    if (count == 0) return {};
    auto it = sequences_.find(id);
    if (it == sequences_.end()) return {KVStatus::sequenceNotFound, "sequenceNotFound"};
    // The reference edits a copy and stores it back on success only (:122, :173).
    LogicalSequence seq = it->second;
    const int64_t bs = blockSize_;
    const int64_t cur = seq.sequenceLength, newLen = cur + count;
    const int64_t now = (cur + bs - 1) / bs, after = (newLen + bs - 1) / bs;
    const int64_t additional = after - now;

    if (hygiene_) {
        // nothing is changed by an append that cannot be completed
        const bool needsCopy = now > 0 && cur % bs != 0 &&
                               refcounts_[static_cast<size_t>(seq.blockTable[static_cast<size_t>(now - 1)])] > 1;
        if (static_cast<int64_t>(free_.size()) < additional + (needsCopy ? 1 : 0))
            return {KVStatus::outOfMemory, "outOfMemory"};
    }
    if (now > 0 && cur % bs != 0) {                            // :134-140
        int32_t last = seq.blockTable[static_cast<size_t>(now - 1)];
        if (refcounts_[static_cast<size_t>(last)] > 1) {
            KVResult r = copyOnWriteLocked(last, static_cast<size_t>(now - 1), seq, cow);
            if (!r.ok()) return r;
        }
    }
    if (additional > 0) {
        if (static_cast<int64_t>(free_.size()) < additional)   // :142-146, before any prefix hit
            return {KVStatus::outOfMemory, "outOfMemory"};
        for (int64_t i = 0; i < additional; ++i) {
            const bool hashed = hashes && i < numHashes;
            if (hashed) {                                      // :150-158
                auto hit = prefix_.find(hashes[i]);
                if (hit != prefix_.end()) {
                    seq.blockTable.push_back(hit->second);
                    refcounts_[static_cast<size_t>(hit->second)] += 1;
                    prefixHits_ += 1;
                    continue;
                }
            }
            int32_t b = allocateBlockLocked();                 // :161-168
            seq.blockTable.push_back(b);
            refcounts_[static_cast<size_t>(b)] = 1;
            if (hashed) {
                prefix_[hashes[i]] = b;
                if (hygiene_) hashesOfBlock_[b].push_back(hashes[i]);
            }
        }
    }
    seq.sequenceLength = newLen;
    it->second = std::move(seq);
    return {};
}

KVResult BlockManager::ensureExclusiveAccess(int64_t id, int64_t logicalBlock,
                                             std::vector<std::pair<int32_t, int32_t>>* cow) {
    // KVCacheManager.swift:200-214
    std::lock_guard<std::mutex> g(mu_);
    auto it = sequences_.find(id);
    if (it == sequences_.end()) return {KVStatus::sequenceNotFound, "sequenceNotFound"};
    LogicalSequence seq = it->second;
    if (logicalBlock < 0 || logicalBlock >= static_cast<int64_t>(seq.blockTable.size()))
        return {KVStatus::invalidRequest, "block index out of range"};
    int32_t b = seq.blockTable[static_cast<size_t>(logicalBlock)];
    if (refcounts_[static_cast<size_t>(b)] > 1) {
        KVResult r = copyOnWriteLocked(b, static_cast<size_t>(logicalBlock), seq, cow);
        if (!r.ok()) return r;
    }
    it->second = std::move(seq);
    return {};
}

void BlockManager::registerBlockHash(uint64_t hash, int32_t block) {   // KVCacheManager.swift:196-198
    std::lock_guard<std::mutex> g(mu_);   // the reference takes no lock here; taking one changes no result
    prefix_[hash] = block;
    if (hygiene_) hashesOfBlock_[block].push_back(hash);
}

void BlockManager::setHygiene(bool on) {
    std::lock_guard<std::mutex> g(mu_);
    hygiene_ = on;
    hashesOfBlock_.clear();
    // entries registered before the switch are tracked from now on
    if (on) for (auto& kv : prefix_) hashesOfBlock_[kv.second].push_back(kv.first);
}

bool BlockManager::hygiene() const {
    std::lock_guard<std::mutex> g(mu_);
    return hygiene_;
}

void BlockManager::freeSequence(int64_t id) {                  // KVCacheManager.swift:216-239
    std::lock_guard<std::mutex> g(mu_);
    auto it = sequences_.find(id);
    if (it == sequences_.end()) return;
    LogicalSequence seq = std::move(it->second);
    sequences_.erase(it);
    const size_t total = seq.blockTable.size();
    const int rem = static_cast<int>(seq.sequenceLength % blockSize_);
    const int lastTokens = rem == 0 ? blockSize_ : rem;
    for (size_t i = 0; i < total; ++i) {
        int32_t b = seq.blockTable[i];
        int32_t& rc = refcounts_[static_cast<size_t>(b)];
        rc -= 1;
        if (rc <= 0) {
            if (hygiene_) {
                // the block goes back to the free list: nobody may reach it through a hash any more
                auto h = hashesOfBlock_.find(b);
                if (h != hashesOfBlock_.end()) {
                    for (uint64_t hash : h->second) {
                        auto e = prefix_.find(hash);
                        if (e != prefix_.end() && e->second == b) prefix_.erase(e);
                    }
                    hashesOfBlock_.erase(h);
                }
            }
            switch (policy_) {
                case fifo: free_.push_front(b); break;
                case lifo: free_.push_back(b); break;
                default:
                    freeSizes_[b] = i + 1 < total ? blockSize_ : lastTokens;
                    free_.push_back(b);
            }
        }
    }
}

void BlockManager::setPolicy(int policy) {                     // KVCacheManager.swift:65-67, 267-283
    std::lock_guard<std::mutex> g(mu_);
    policy_ = policy;
    if (policy == fifo || policy == lifo) {
        std::reverse(free_.begin(), free_.end());
        freeSizes_.clear();
    } else {
        for (int32_t b : free_) freeSizes_.emplace(b, blockSize_);
        std::stable_sort(free_.begin(), free_.end(), [&](int32_t a, int32_t b) {
            return freeSizes_[a] > freeSizes_[b];
        });
    }
}

KVResult BlockManager::blockTable(int64_t id, std::vector<int32_t>* out) const {
    std::lock_guard<std::mutex> g(mu_);
    auto it = sequences_.find(id);
    if (it == sequences_.end()) return {KVStatus::sequenceNotFound, "sequenceNotFound"};
    *out = it->second.blockTable;
    return {};
}

KVResult BlockManager::sequenceLength(int64_t id, int64_t* out) const {
    std::lock_guard<std::mutex> g(mu_);
    auto it = sequences_.find(id);
    if (it == sequences_.end()) return {KVStatus::sequenceNotFound, "sequenceNotFound"};
    *out = it->second.sequenceLength;
    return {};
}

int BlockManager::availableBlocks() const {                    // KVCacheManager.swift:341-345
    std::lock_guard<std::mutex> g(mu_);
    return static_cast<int>(free_.size());
}

int BlockManager::activeSequences() const {                    // KVCacheManager.swift:347-351
    std::lock_guard<std::mutex> g(mu_);
    return static_cast<int>(sequences_.size());
}

MemoryStats BlockManager::stats() const {                      // KVCacheManager.swift:353-378
    std::lock_guard<std::mutex> g(mu_);
    MemoryStats s;
    s.totalBlocks = maxBlocks_;
    s.freeBlocks = static_cast<int64_t>(free_.size());
    s.usedBlocks = maxBlocks_ - s.freeBlocks;
    s.activeSequences = static_cast<int64_t>(sequences_.size());
    for (auto& kv : sequences_)
        if (kv.second.sequenceLength % blockSize_ > 0) s.partiallyFilledBlocks += 1;
    s.fragmentationRatio = static_cast<float>(s.partiallyFilledBlocks) /
                           static_cast<float>(std::max<int64_t>(s.activeSequences, 1));
    s.prefixCacheHits = prefixHits_;
    s.prefixCacheEntries = static_cast<int64_t>(prefix_.size());
    for (int32_t r : refcounts_) if (r > 1) s.sharedBlocks += 1;
    s.policy = policy_;
    return s;
}

// ---------------------------------------------------------------- scheduler

int64_t Scheduler::addRequest(int promptTokens, int maxNewTokens) {   // Scheduler.swift:58-70
    std::lock_guard<std::mutex> g(mu_);
    if (static_cast<int>(seqs_.size()) >= maxSeqs_) return -1;
    SchedulerSequence s;
    s.id = nextId_++;
    s.promptLength = promptTokens;
    s.maxNewTokens = maxNewTokens;
    s.arrivalOrder = arrival_++;
    seqs_[s.id] = s;
    return s.id;
}

void Scheduler::complete(int64_t id) {                         // Scheduler.swift:72-76
    std::lock_guard<std::mutex> g(mu_);
    auto it = seqs_.find(id);
    if (it != seqs_.end()) it->second.status = completed;
}

std::vector<int64_t> Scheduler::step() {                       // Scheduler.swift:78-114
    std::lock_guard<std::mutex> g(mu_);
    std::vector<SchedulerSequence*> byArrival;
    for (auto& kv : seqs_) byArrival.push_back(&kv.second);
    std::sort(byArrival.begin(), byArrival.end(),
              [](auto* a, auto* b) { return a->arrivalOrder < b->arrivalOrder; });
    std::vector<SchedulerSequence*> w, r, p;
    for (auto* s : byArrival) {
        if (s->status == waiting) w.push_back(s);
        else if (s->status == running && !s->isDone()) r.push_back(s);
        else if (s->status == paused) p.push_back(s);
    }
    std::vector<int64_t> batch;
    const size_t cap = static_cast<size_t>(std::max(maxBatch_, 0));
    for (size_t i = 0; i < w.size() && i < cap; ++i) { w[i]->status = running; batch.push_back(w[i]->id); }
    for (size_t i = 0; i < r.size() && batch.size() < cap; ++i) batch.push_back(r[i]->id);
    for (size_t i = 0; i < p.size() && batch.size() < cap; ++i) { p[i]->status = running; batch.push_back(p[i]->id); }
    return batch;
}

void Scheduler::markPrefilled(int64_t id) {                    // Scheduler.swift:116-120
    std::lock_guard<std::mutex> g(mu_);
    auto it = seqs_.find(id);
    if (it != seqs_.end()) it->second.status = running;
}

void Scheduler::markDecoded(int64_t id) {                      // Scheduler.swift:122-126
    std::lock_guard<std::mutex> g(mu_);
    auto it = seqs_.find(id);
    if (it != seqs_.end()) it->second.numGeneratedTokens += 1;
}

void Scheduler::preempt(int64_t id) {                          // Scheduler.swift:128-132
    std::lock_guard<std::mutex> g(mu_);
    auto it = seqs_.find(id);
    if (it != seqs_.end()) it->second.status = paused;
}

int Scheduler::count(int status) const {                       // Scheduler.swift:154-170
    std::lock_guard<std::mutex> g(mu_);
    int n = 0;
    for (auto& kv : seqs_) if (kv.second.status == status) ++n;
    return n;
}

int Scheduler::total() const {                                 // Scheduler.swift:172-176
    std::lock_guard<std::mutex> g(mu_);
    return static_cast<int>(seqs_.size());
}

bool Scheduler::get(int64_t id, SchedulerSequence* out) const {
    std::lock_guard<std::mutex> g(mu_);
    auto it = seqs_.find(id);
    if (it == seqs_.end()) return false;
    *out = it->second;
    return true;
}

}  // namespace pam
