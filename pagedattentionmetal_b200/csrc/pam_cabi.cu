// Host side of the library: context (engine), KV cache handles and the C ABI
// declared in include/pam_cuda.h.  Mirrors PagedAttentionEngine
// (PagedAttentionEngine.swift), KVCacheManager (KVCacheManager.swift),
// ContinuousBatchingScheduler (Scheduler.swift) and the reference's own C ABI
// (PagedAttentionCABI.swift); each function cites what it follows.
#include <cuda_runtime.h>
#include <unistd.h>

#include <algorithm>
#include <chrono>
#include <climits>
#include <map>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <set>
#include <string>
#include <unordered_set>
#include <vector>

#include "../../include/pam_cuda.h"
#include "block_manager.h"
#include "kernels.h"

namespace {

using pam::BlockManager;
using pam::KVResult;
using pam::KVStatus;

constexpr size_t kUnknownBytes = static_cast<size_t>(-1);

size_t alignUp(size_t v, size_t a) { return (v + a - 1) / a * a; }

// Device memory handed out in bump fashion for the duration of one call:
// staging copies of host arguments, block tables, the decode kernel's records.
class Arena {
public:
    ~Arena() { release(); }
    void release() {
        for (auto& c : chunks_) cudaFree(c.base);
        chunks_.clear();
    }
    // Start of a call: fold several chunks into one of their total size.
    void reset(cudaStream_t stream) {
        if (chunks_.size() > 1) {
            size_t total = 0;
            for (auto& c : chunks_) total += c.cap;
            cudaStreamSynchronize(stream);
            release();
            void* p = nullptr;
            if (cudaMalloc(&p, total) == cudaSuccess) chunks_.push_back({p, total, 0});
        }
        for (auto& c : chunks_) c.used = 0;
    }
    void* take(size_t bytes) {
        bytes = alignUp(std::max<size_t>(bytes, 1), 256);
        for (auto& c : chunks_)
            if (c.cap - c.used >= bytes) {
                void* p = static_cast<char*>(c.base) + c.used;
                c.used += bytes;
                return p;
            }
        size_t cap = std::max(bytes, chunks_.empty() ? size_t(1) << 20 : chunks_.back().cap * 2);
        void* p = nullptr;
        if (cudaMalloc(&p, cap) != cudaSuccess) { cudaGetLastError(); return nullptr; }
        chunks_.push_back({p, cap, bytes});
        return p;
    }

private:
    struct Chunk { void* base; size_t cap, used; };
    std::vector<Chunk> chunks_;
};

struct Context {
    int device = 0, smCount = 148;
    cudaStream_t ownStream = nullptr, stream = nullptr;
    bool async = false;
    std::mutex mu;            // serialises operations and guards the fields below
    std::string lastError;
    bool hasError = false;
    int lastCode = PAM_OK;
    // PagedAttentionEngine.swift:116-129
    int maxRetries = 3, splitThreshold = 1024, defaultWindow = 0, defaultChunk = 0;
    bool graceful = true;
    int consecutiveFailures = 0, injectFailures = 0;
    int64_t launches = 0;
    PamStats stats{};
    Arena arena;
    int* devErr = nullptr;    // set by a kernel whose bounded wait ran out
    int* hostErr = nullptr;   // pinned copy, read after the stream has been synchronised
    bool errPending = false;
    bool forceGeneralPrefill = false;
    int exactWeights = 1;
    void* pinned = nullptr;   // page-locked scratch for host arrays the library builds itself (batch tables)
    size_t pinnedCap = 0;
    void* qStage = nullptr;   // device copy of a host query of pam_decode, sent before the tables are built
    size_t qStageCap = 0;
    void* outStage = nullptr; // device side of a pageable host output of pam_decode
    size_t outStageCap = 0;
    int* mergeCounters = nullptr;                // zero between launches: three counting words per (sequence, kv head)
    int64_t mergeCountersCap = 0;
    long long waitLimitCycles = 0;               // 0: the prefill kernel's default bound on its waits
    int dropFirstVTile = 0;                      // test switch, see pamc_test_starve_prefill

    int32_t fail(int code, const std::string& msg) {            // CABI.swift:18-30
        lastError = msg;
        hasError = true;
        lastCode = code;
        return -1;
    }
    void clearError() { hasError = false; lastCode = PAM_OK; lastError.clear(); }   // CABI.swift:32-37
};

struct Cache {
    BlockManager mgr;
    bool bookkeeping = false;
    int device = 0, dtype = 0, headDim = 0, kvHeads = 0, blockSize = 0, maxBlocks = 0;
    void *kPool = nullptr, *vPool = nullptr, *kScale = nullptr, *vScale = nullptr;
    unsigned long long* amax = nullptr;    // FP8 append scratch, [block][kv_head][2]
    uint32_t epoch = 0;
    size_t poolBytes = 0, scaleBytes = 0;
    std::mutex mu;
    std::vector<std::pair<int32_t, int32_t>> cowLog;
    // The block tables of the batch pam_decode last ran, kept on the device: a decode step
    // changes at most one entry per sequence, so only what changed is sent again.
    struct Resident {
        int32_t* tables = nullptr;         // [rows][stride]
        uint32_t* upload = nullptr;        // lengths, then (row, column, block) patches
        int rows = 0, stride = 0;
        size_t uploadCap = 0;              // bytes
        std::vector<int64_t> ids;          // per row: what the device copy holds
        std::vector<uint64_t> versions;
        std::vector<int32_t> counts;
        unsigned char* pinned = nullptr;   // staging of `upload`
        size_t pinnedCap = 0;
        cudaEvent_t consumed = nullptr;    // the last upload has left `pinned`
    } res;
    Cache(int maxBlocks_, int blockSize_) : mgr(maxBlocks_, blockSize_), blockSize(blockSize_), maxBlocks(maxBlocks_) {}
    ~Cache() {
        if (bookkeeping) return;
        cudaSetDevice(device);
        cudaDeviceSynchronize();
        cudaFree(kPool); cudaFree(vPool); cudaFree(kScale); cudaFree(vScale); cudaFree(amax);
        cudaFree(res.tables); cudaFree(res.upload);
        if (res.pinned) cudaFreeHost(res.pinned);
        if (res.consumed) cudaEventDestroy(res.consumed);
    }
    size_t blockBytes() const { return static_cast<size_t>(blockSize) * kvHeads * headDim * pam::elemBytes(dtype); }
};

struct Sched {
    pam::Scheduler s;
    Sched(int b, int m) : s(b, m) {}
};

Context* asCtx(void* p) { return static_cast<Context*>(p); }
Cache* asCache(void* p) { return static_cast<Cache*>(p); }

bool isDevicePointer(const void* p) {
    cudaPointerAttributes a{};
    if (cudaPointerGetAttributes(&a, p) != cudaSuccess) { cudaGetLastError(); return false; }
    return a.type == cudaMemoryTypeDevice || a.type == cudaMemoryTypeManaged;
}

// Where a buffer argument lives, asked once per call.  `device` is the address a kernel
// may use: the pointer itself for device memory, the device-side alias for page-locked
// host memory, null for pageable host memory (which has to be staged).
struct Placement {
    bool onDevice = false;
    void* device = nullptr;
};
Placement placementOf(const void* p) {
    Placement r;
    cudaPointerAttributes a{};
    if (!p || cudaPointerGetAttributes(&a, p) != cudaSuccess) { cudaGetLastError(); return r; }
    r.onDevice = a.type == cudaMemoryTypeDevice || a.type == cudaMemoryTypeManaged;
    if (r.onDevice) r.device = const_cast<void*>(p);
    else if (a.type == cudaMemoryTypeHost) r.device = a.devicePointer;
    return r;
}

// One zeroed arrival word per (sequence, kv head) pair of the largest decode so far.
struct Context;
bool ensureMergeCounters(Context* c, int64_t pairs);

// Operations that need the GPU fail like a missing device (PagedAttentionTypes.swift:36-37).
int32_t noGpu(Context* c) {
    return c->fail(PAM_ERR_DEVICE_INIT, "Metal device or command queue could not be initialized.");
}

bool ensureMergeCounters(Context* c, int64_t pairs) {
    if (pairs <= c->mergeCountersCap) return true;
    cudaStreamSynchronize(c->stream);
    if (c->mergeCounters) cudaFree(c->mergeCounters);
    c->mergeCounters = nullptr;
    c->mergeCountersCap = 0;
    const int64_t cap = pairs + pairs / 2;
    if (cudaMalloc(reinterpret_cast<void**>(&c->mergeCounters), static_cast<size_t>(cap) * sizeof(int)) != cudaSuccess ||
        cudaMemsetAsync(c->mergeCounters, 0, static_cast<size_t>(cap) * sizeof(int), c->stream) != cudaSuccess) {
        cudaGetLastError();
        if (c->mergeCounters) cudaFree(c->mergeCounters);
        c->mergeCounters = nullptr;
        return false;
    }
    c->mergeCountersCap = cap;
    return true;
}

// Page-locked scratch of at least `bytes` (nullptr when it cannot be had: the caller then
// copies from its pageable array).  A copy from page-locked memory runs at the link's speed
// and does not hold the host; one block is reused by every call, so the caller must have
// the stream drained before the next call writes it (the synchronous mode does, and the
// cache-handle calls drain it themselves in async mode).
void* pinnedScratch(Context* c, size_t bytes) {
    if (bytes <= c->pinnedCap) return c->pinned;
    cudaStreamSynchronize(c->stream);
    if (c->pinned) cudaFreeHost(c->pinned);
    c->pinned = nullptr;
    c->pinnedCap = 0;
    const size_t cap = std::max<size_t>(bytes + bytes / 2, size_t(1) << 20);
    if (cudaHostAlloc(&c->pinned, cap, cudaHostAllocDefault) != cudaSuccess) {
        cudaGetLastError();
        c->pinned = nullptr;
        return nullptr;
    }
    c->pinnedCap = cap;
    return c->pinned;
}

int32_t kvFail(Context* c, const KVResult& r) {
    switch (r.status) {
        case KVStatus::outOfMemory: return c->fail(PAM_ERR_KV_OUT_OF_MEMORY, "KVCacheError.outOfMemory");
        case KVStatus::sequenceNotFound: return c->fail(PAM_ERR_KV_SEQUENCE_NOT_FOUND, "KVCacheError.sequenceNotFound");
        case KVStatus::sequenceAlreadyExists: return c->fail(PAM_ERR_KV_SEQUENCE_EXISTS, "KVCacheError.sequenceAlreadyExists");
        case KVStatus::invalidRequest: return c->fail(PAM_ERR_KV_INVALID_REQUEST, "KVCacheError.invalidRequest(\"" + r.message + "\")");
        default: return 0;
    }
}

// PagedAttentionError.description (PagedAttentionTypes.swift:34-63)
std::string invalidConfiguration(const std::string& m) { return "Invalid paged attention configuration: " + m; }
std::string bufferTooSmall(const char* name, size_t expected, size_t actual) {
    return std::string(name) + " buffer is too small: expected at least " + std::to_string(expected) +
           " bytes, got " + std::to_string(actual) + ".";
}
std::string commandExecutionFailed(const std::string& m) { return "Metal command execution failed: " + m; }

bool validDtype(int d) { return d >= 0 && d <= 3; }

// PagedLayerSpec.validate (PagedAttentionTypes.swift:126-142)
bool validateLayer(Context* c, const PamLayerSpec& l) {
    const char* m = nullptr;
    if (l.head_dim <= 0) m = "headDim must be positive.";
    else if (l.num_heads <= 0) m = "numHeads must be positive.";
    else if (l.num_kv_heads <= 0) m = "numKVHeads must be positive.";
    else if (l.num_heads % l.num_kv_heads != 0) m = "numHeads must be divisible by numKVHeads for GQA/MQA mapping.";
    else if (l.block_size <= 0) m = "blockSize must be positive.";
    if (m) { c->fail(PAM_ERR_INVALID_CONFIGURATION, invalidConfiguration(m)); return false; }
    if (!validDtype(l.data_type)) {                              // CABI.swift:64-69
        c->fail(PAM_ERR_INVALID_CONFIGURATION,
                invalidConfiguration("unknown dtype " + std::to_string(l.data_type) +
                                     "; use 0 for float32 or 1 for float16"));
        return false;
    }
    return true;
}

// requireBuffer (PagedAttentionEngine.swift:1994-1998)
bool requireBuffer(Context* c, const PamBuffer& b, const char* name, size_t expected) {
    if (b.bytes != kUnknownBytes && b.bytes < expected) {
        c->fail(PAM_ERR_BUFFER_TOO_SMALL, bufferTooSmall(name, expected, b.bytes));
        return false;
    }
    if (!b.ptr) {
        c->fail(PAM_ERR_BUFFER_TOO_SMALL, bufferTooSmall(name, expected, 0));
        return false;
    }
    return true;
}

// Query, output and new K/V rows of an FP8 layer are float16: the reference's
// qBytesPerToken / kvBytesPerToken count the cache's one byte per element there
// (PagedAttentionTypes.swift:149-151), half of what the kernels read and write.  A buffer
// of known length must hold what is really accessed.
bool requireIoBuffer(Context* c, const PamBuffer& b, const char* name, size_t referenceBytes, size_t accessedBytes) {
    return requireBuffer(c, b, name, std::max(referenceBytes, accessedBytes));
}

size_t qBytesPerToken(const PamLayerSpec& l) {                  // PagedAttentionTypes.swift:149
    return static_cast<size_t>(l.num_heads) * l.head_dim * pam::elemBytes(l.data_type);
}
size_t kvBytesPerToken(const PamLayerSpec& l) {                 // PagedAttentionTypes.swift:151
    return static_cast<size_t>(l.num_kv_heads) * l.head_dim * pam::elemBytes(l.data_type);
}
// Actual size of query/output rows: FP8 caches take float16 queries.
size_t ioBytesPerToken(const PamLayerSpec& l) {
    return static_cast<size_t>(l.num_heads) * l.head_dim * pam::ioBytes(l.data_type);
}

// Blocks a pool buffer of known length holds (table entries are clamped to it).
int poolBlocksOf(const PamBuffer& k, const PamBuffer& v, const PamLayerSpec& l) {
    if (k.bytes == kUnknownBytes || v.bytes == kUnknownBytes) return INT32_MAX;
    const size_t perBlock = std::max<size_t>(static_cast<size_t>(l.block_size) * kvBytesPerToken(l), 1);
    return static_cast<int>(std::min<size_t>(std::min(k.bytes, v.bytes) / perBlock, INT32_MAX));
}

// Host arguments are copied into the arena; outputs are copied back by finish().
class Stager {
public:
    explicit Stager(Context* c) : c_(c) {}
    const void* in(const void* p, size_t bytes) {
        if (!p || isDevicePointer(p)) return p;
        void* d = c_->arena.take(bytes);
        if (!d || cudaMemcpyAsync(d, p, bytes, cudaMemcpyHostToDevice, c_->stream) != cudaSuccess) { ok_ = false; return nullptr; }
        return d;
    }
    void* out(void* p, size_t bytes) {
        if (!p || isDevicePointer(p)) return p;
        void* d = c_->arena.take(bytes);
        if (!d) { ok_ = false; return nullptr; }
        outs_.push_back({p, d, bytes});
        return d;
    }
    // Upload a host array the library built itself (tables, lengths, ...).
    void* upload(const void* host, size_t bytes) {
        void* d = c_->arena.take(bytes);
        if (!d || cudaMemcpyAsync(d, host, bytes, cudaMemcpyHostToDevice, c_->stream) != cudaSuccess) { ok_ = false; return nullptr; }
        return d;
    }
    bool ok() const { return ok_; }
    bool hasOutputs() const { return !outs_.empty(); }
    cudaError_t copyBack() {
        for (auto& o : outs_) {
            cudaError_t e = cudaMemcpyAsync(o.host, o.dev, o.bytes, cudaMemcpyDeviceToHost, c_->stream);
            if (e != cudaSuccess) return e;
        }
        return cudaSuccess;
    }
    void zeroOutputs(void* devOrHostOut, size_t bytes) {
        if (!devOrHostOut) return;
        if (isDevicePointer(devOrHostOut)) cudaMemsetAsync(devOrHostOut, 0, bytes, c_->stream);
        else std::memset(devOrHostOut, 0, bytes);
    }

private:
    struct Out { void* host; void* dev; size_t bytes; };
    Context* c_;
    std::vector<Out> outs_;
    bool ok_ = true;
};

// withRetry (PagedAttentionEngine.swift:375-400): up to maxRetries attempts,
// a back-off of 10 ms * 2^attempt from the second failure on, and a circuit
// breaker after 2 * maxRetries consecutive failures.  `attempt` enqueues the
// work and returns a CUDA status; host-injected failures stand in for it.
template <class F>
int32_t withRetry(Context* c, const char* operation, F attempt) {
    std::string last = "no attempt made (maxRetries is 0)";
    for (int i = 0; i < c->maxRetries; ++i) {
        cudaError_t e;
        if (c->injectFailures > 0) {
            c->injectFailures -= 1;
            e = cudaErrorLaunchFailure;
            last = "injected launch failure";
        } else {
            e = attempt();
            if (e == cudaSuccess && !c->async) e = cudaStreamSynchronize(c->stream);
            if (e != cudaSuccess) { last = cudaGetErrorString(e); cudaGetLastError(); }
            else if (!c->async && c->errPending) {
                // a kernel gave up on a bounded wait and returned without finishing its work
                c->errPending = false;
                if (*c->hostErr != 0) {
                    last = "a kernel's bounded wait ran out (site " + std::to_string(*c->hostErr) + ")";
                    *c->hostErr = 0;
                    cudaMemsetAsync(c->devErr, 0, sizeof(int), c->stream);
                    e = cudaErrorLaunchTimeout;
                }
            }
        }
        if (e == cudaSuccess) { c->consecutiveFailures = 0; return 0; }
        c->consecutiveFailures += 1;
        if (c->consecutiveFailures >= c->maxRetries * 2) {
            return c->fail(PAM_ERR_RECURRING, "Recurring failure in '" + std::string(operation) + "' after " +
                                                  std::to_string(c->consecutiveFailures) +
                                                  " attempts \xE2\x80\x94 circuit breaker engaged.");
        }
        if (i > 0) usleep(static_cast<useconds_t>(0.01 * static_cast<double>(1 << i) * 1e6));
    }
    return c->fail(PAM_ERR_COMMAND_EXECUTION, commandExecutionFailed(last));
}

double nowMs() {
    return std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now().time_since_epoch()).count();
}

struct DeviceGuard {
    int prev = -1;
    explicit DeviceGuard(int dev) {
        if (dev < 0) return;
        cudaGetDevice(&prev);
        if (prev != dev) cudaSetDevice(dev);
        else prev = -1;
    }
    ~DeviceGuard() { if (prev >= 0) cudaSetDevice(prev); }
};

// ------------------------------------------------------------------ operations

// Copy-on-write pairs recorded by the block manager: copy K, V and scales on
// the GPU, one launch per run of pairs that do not feed one another.
int32_t runCopies(Context* c, Cache* k, const std::vector<std::pair<int32_t, int32_t>>& pairs) {
    if (pairs.empty() || k->bookkeeping) return 0;
    size_t begin = 0;
    while (begin < pairs.size()) {
        std::unordered_set<int32_t> written;
        size_t end = begin;
        while (end < pairs.size() && !written.count(pairs[end].first) && !written.count(pairs[end].second)) {
            written.insert(pairs[end].second);
            ++end;
        }
        if (end == begin) end = begin + 1;
        std::vector<int32_t> flat;
        for (size_t i = begin; i < end; ++i) { flat.push_back(pairs[i].first); flat.push_back(pairs[i].second); }
        const int n = static_cast<int>(end - begin);
        int32_t rc = withRetry(c, "copyBlocks", [&]() -> cudaError_t {
            Stager st(c);
            const int32_t* dev = static_cast<const int32_t*>(st.upload(flat.data(), flat.size() * sizeof(int32_t)));
            if (!st.ok()) return cudaErrorMemoryAllocation;
            int launches = 0;
            cudaError_t e = pam::launchCopyBlocks(k->kPool, k->vPool, k->kScale, k->vScale, dev, n, k->blockBytes(),
                                                  k->kvHeads, c->stream, &launches);
            c->launches += launches;
            // the upload buffer is read by the kernel: the caller keeps `flat` alive until the sync below
            if (e == cudaSuccess) e = cudaStreamSynchronize(c->stream);
            return e;
        });
        if (rc != 0) return rc;
        begin = end;
    }
    return 0;
}

int32_t appendImpl(Context* c, const PamAppendRequest& rq, Cache* cacheForScratch, const int64_t* hostSlots,
                   const int64_t* deviceSlots = nullptr) {
    // PagedAttentionEngine.swift:585-628; validateAppend :1935-1950
    if (!validateLayer(c, rq.layer)) return -1;
    if (rq.token_offset < 0) return c->fail(PAM_ERR_INVALID_CONFIGURATION, invalidConfiguration("tokenOffset must be non-negative."));
    if (rq.num_new_tokens <= 0) return c->fail(PAM_ERR_INVALID_CONFIGURATION, invalidConfiguration("numNewTokens must be positive."));
    const PamLayerSpec& l = rq.layer;
    const int T = rq.num_new_tokens;
    const size_t finalLen = static_cast<size_t>(rq.token_offset) + T;
    const size_t numBlocks = (finalLen + l.block_size - 1) / l.block_size;
    const size_t newBytes = static_cast<size_t>(T) * l.num_kv_heads * l.head_dim * pam::ioBytes(l.data_type);
    if (!requireIoBuffer(c, rq.keys, "new keys", static_cast<size_t>(T) * kvBytesPerToken(l), newBytes)) return -1;
    if (!requireIoBuffer(c, rq.values, "new values", static_cast<size_t>(T) * kvBytesPerToken(l), newBytes)) return -1;
    if (!hostSlots && !deviceSlots && !requireBuffer(c, rq.block_table, "blockTable", numBlocks * sizeof(int32_t))) return -1;
    if (!requireBuffer(c, rq.k_pool, "K pool", numBlocks * l.block_size * kvBytesPerToken(l))) return -1;
    if (!requireBuffer(c, rq.v_pool, "V pool", numBlocks * l.block_size * kvBytesPerToken(l))) return -1;
    const bool fp8 = l.data_type == PAM_DTYPE_FP8;
    if (fp8 && (!rq.k_scale.ptr || !rq.v_scale.ptr || !cacheForScratch))
        return c->fail(PAM_ERR_INVALID_CONFIGURATION, invalidConfiguration("FP8 append needs the cache's scale buffers."));
    if (!isDevicePointer(rq.k_pool.ptr) || !isDevicePointer(rq.v_pool.ptr))
        return c->fail(PAM_ERR_INVALID_CONFIGURATION, invalidConfiguration("KV pools must be device memory."));

    // Slots outside the pool are skipped by the kernels; the pool size comes
    // from the cache handle, else from the length given with the pool buffer.
    int64_t poolSlots = INT64_MAX;
    if (cacheForScratch) poolSlots = static_cast<int64_t>(cacheForScratch->maxBlocks) * cacheForScratch->blockSize;
    else if (rq.k_pool.bytes != kUnknownBytes) poolSlots = static_cast<int64_t>(std::min(rq.k_pool.bytes, rq.v_pool.bytes) / std::max<size_t>(kvBytesPerToken(l), 1));
    const double t0 = nowMs();
    c->arena.reset(c->stream);
    int32_t rc = withRetry(c, "appendToCacheFlat", [&]() -> cudaError_t {
        Stager st(c);
        const void* keys = st.in(rq.keys.ptr, newBytes);
        const void* values = st.in(rq.values.ptr, newBytes);
        pam::SlotSource src;
        src.numSlots = poolSlots;
        if (deviceSlots) src.slots = deviceSlots;
        else if (hostSlots) src.slots = static_cast<const int64_t*>(st.upload(hostSlots, sizeof(int64_t) * T));
        else {
            src.table = static_cast<const int32_t*>(st.in(rq.block_table.ptr, numBlocks * sizeof(int32_t)));
            src.tokenOffset = rq.token_offset;
        }
        if (!st.ok()) return cudaErrorMemoryAllocation;
        int launches = 0;
        cudaError_t e;
        if (fp8) {
            Cache* k = cacheForScratch;
            if (!k->amax) {
                const size_t bytes = static_cast<size_t>(k->maxBlocks) * k->kvHeads * 2 * sizeof(unsigned long long);
                e = cudaMalloc(reinterpret_cast<void**>(&k->amax), bytes);
                if (e != cudaSuccess) return e;
                e = cudaMemsetAsync(k->amax, 0, bytes, c->stream);
                if (e != cudaSuccess) return e;
                k->epoch = 0;
            }
            k->epoch += 1;
            e = pam::launchReshapeAndCacheFp8(keys, values, rq.k_pool.ptr, rq.v_pool.ptr, rq.k_scale.ptr, rq.v_scale.ptr,
                                              src, T, l.num_kv_heads, l.block_size, l.head_dim, k->amax, k->epoch,
                                              c->stream, &launches);
        } else {
            e = pam::launchReshapeAndCache(keys, values, rq.k_pool.ptr, rq.v_pool.ptr, src, T, l.num_kv_heads,
                                           l.block_size, l.head_dim, pam::elemBytes(l.data_type), c->stream, &launches);
        }
        c->launches += launches;
        return e;
    });
    if (rc != 0) {
        if (!c->graceful) return rc;                             // :588-596 swallows the error
        c->clearError();
    }
    c->stats = PamStats{PAM_OP_APPEND, 1, T, static_cast<int32_t>(numBlocks), 0, 0, nowMs() - t0};   // :616-626
    return 0;
}

// validateDecode (PagedAttentionEngine.swift:1916-1933) and the checks of decodeFlat's
// arguments; host work only, done before anything that needs the GPU.
int32_t validateDecode(Context* c, const PamDecodeRequest& rq) {
    if (!validateLayer(c, rq.layer)) return -1;
    if (rq.batch_size <= 0) return c->fail(PAM_ERR_INVALID_CONFIGURATION, invalidConfiguration("batchSize must be positive."));
    if (rq.max_num_blocks <= 0) return c->fail(PAM_ERR_INVALID_CONFIGURATION, invalidConfiguration("maxNumBlocks must be positive."));
    const PamLayerSpec& l = rq.layer;
    const size_t B = static_cast<size_t>(rq.batch_size), NB = static_cast<size_t>(rq.max_num_blocks);
    if (rq.block_tables.bytes != kUnknownBytes && NB > rq.block_tables.bytes / (B * sizeof(int32_t)))
        return c->fail(PAM_ERR_INVALID_CONFIGURATION, invalidConfiguration("maxNumBlocks exceeds blockTables buffer capacity"));
    if (!requireIoBuffer(c, rq.q, "Q", B * qBytesPerToken(l), B * ioBytesPerToken(l))) return -1;
    if (!requireBuffer(c, rq.block_tables, "blockTables", B * NB * sizeof(int32_t))) return -1;
    if (!requireBuffer(c, rq.seq_lengths, "seqLengths", B * sizeof(uint32_t))) return -1;
    if (!requireIoBuffer(c, rq.output, "output", B * qBytesPerToken(l), B * ioBytesPerToken(l))) return -1;
    if (!requireBuffer(c, rq.k_pool, "K pool", NB * l.block_size * kvBytesPerToken(l))) return -1;
    if (!requireBuffer(c, rq.v_pool, "V pool", NB * l.block_size * kvBytesPerToken(l))) return -1;
    if (l.data_type == PAM_DTYPE_FP8 && (!rq.k_scale.ptr || !rq.v_scale.ptr))
        return c->fail(PAM_ERR_INVALID_CONFIGURATION, invalidConfiguration("FP8 decode needs kScaleBuffer and vScaleBuffer."));
    if (l.head_dim > 256)
        return c->fail(PAM_ERR_UNSUPPORTED, "Unsupported paged attention path: headDim above 256.");
    return 0;
}

int32_t decodeImpl(Context* c, const PamDecodeRequest& rq) {
    // PagedAttentionEngine.swift:533-580
    if (validateDecode(c, rq) != 0) return -1;
    if (c->device < 0) return noGpu(c);
    const PamLayerSpec& l = rq.layer;
    const size_t B = static_cast<size_t>(rq.batch_size), NB = static_cast<size_t>(rq.max_num_blocks);
    if (!isDevicePointer(rq.k_pool.ptr) || !isDevicePointer(rq.v_pool.ptr))
        return c->fail(PAM_ERR_INVALID_CONFIGURATION, invalidConfiguration("KV pools must be device memory."));

    const int window = l.window_size > 0 ? l.window_size : c->defaultWindow;     // :1028
    const size_t ioBytes = B * ioBytesPerToken(l);
    const double t0 = nowMs();
    c->arena.reset(c->stream);
    size_t tempBytes = 0;
    Stager st(c);
    int32_t rc = withRetry(c, "decodeFlat", [&]() -> cudaError_t {
        pam::DecodeParams p{};
        p.q = st.in(rq.q.ptr, ioBytes);
        p.kPool = rq.k_pool.ptr;
        p.vPool = rq.v_pool.ptr;
        p.tables = static_cast<const int32_t*>(st.in(rq.block_tables.ptr, B * NB * sizeof(int32_t)));
        p.lens = static_cast<const uint32_t*>(st.in(rq.seq_lengths.ptr, B * sizeof(uint32_t)));
        p.out = st.out(rq.output.ptr, ioBytes);
        p.kScale = rq.k_scale.ptr;
        p.vScale = rq.v_scale.ptr;
        p.batch = rq.batch_size; p.heads = l.num_heads; p.kvHeads = l.num_kv_heads; p.headDim = l.head_dim;
        p.blockSize = l.block_size; p.maxNumBlocks = rq.max_num_blocks; p.window = window; p.dtype = l.data_type;
        p.poolBlocks = poolBlocksOf(rq.k_pool, rq.v_pool, l);
        if (!ensureMergeCounters(c, static_cast<int64_t>(rq.batch_size) * l.num_kv_heads)) return cudaErrorMemoryAllocation;
        p.counters = c->mergeCounters;
        p.countersCap = c->mergeCountersCap;
        if (!st.ok()) return cudaErrorMemoryAllocation;
        tempBytes = pam::decodeWorkspaceBytes(p, c->smCount);
        if (tempBytes) {
            p.workspace = static_cast<float*>(c->arena.take(tempBytes));
            p.workspaceBytes = tempBytes;
            if (!p.workspace) return cudaErrorMemoryAllocation;
        }
        if (!st.ok()) return cudaErrorMemoryAllocation;
        int launches = 0;
        cudaError_t e = pam::launchDecode(p, c->smCount, c->stream, &launches);
        c->launches += launches;
        if (e == cudaSuccess) e = st.copyBack();
        return e;
    });
    if (rc != 0) {
        // a launch that did not finish may have left arrivals counted
        if (c->mergeCounters) cudaMemsetAsync(c->mergeCounters, 0, static_cast<size_t>(c->mergeCountersCap) * sizeof(int), c->stream);
        if (!c->graceful) return rc;
        st.zeroOutputs(rq.output.ptr, rq.output.bytes != kUnknownBytes ? rq.output.bytes : ioBytes);   // :536-542
        c->clearError();
    }
    if (c->async && st.hasOutputs()) cudaStreamSynchronize(c->stream);   // host results must be there on return
    c->stats = PamStats{PAM_OP_DECODE, rq.batch_size, 0, rq.max_num_blocks, static_cast<int64_t>(tempBytes), 0, nowMs() - t0};   // :568-577
    return 0;
}

// Decode for callers that may not allocate: same checks and kernels as
// decodeImpl, but nothing is staged (every buffer must already be device
// memory), the context's arena is left alone, and the records of shared pairs go to the
// library's fixed scratch array.
int32_t decodeNoAllocImpl(Context* c, const PamDecodeRequest& rq) {
    if (validateDecode(c, rq) != 0) return -1;
    if (c->device < 0) return noGpu(c);
    const PamLayerSpec& l = rq.layer;
    const size_t B = static_cast<size_t>(rq.batch_size);
    const void* mustBeDevice[] = {rq.q.ptr, rq.k_pool.ptr, rq.v_pool.ptr, rq.block_tables.ptr, rq.seq_lengths.ptr, rq.output.ptr};
    for (const void* p : mustBeDevice)
        if (!isDevicePointer(p))
            return c->fail(PAM_ERR_INVALID_CONFIGURATION,
                           invalidConfiguration("the no-allocation decode takes device memory only: a host buffer would need a staging allocation."));
    pam::DecodeParams p{};
    p.q = rq.q.ptr; p.kPool = rq.k_pool.ptr; p.vPool = rq.v_pool.ptr;
    p.tables = static_cast<const int32_t*>(rq.block_tables.ptr);
    p.lens = static_cast<const uint32_t*>(rq.seq_lengths.ptr);
    p.out = rq.output.ptr; p.kScale = rq.k_scale.ptr; p.vScale = rq.v_scale.ptr;
    p.batch = rq.batch_size; p.heads = l.num_heads; p.kvHeads = l.num_kv_heads; p.headDim = l.head_dim;
    p.blockSize = l.block_size; p.maxNumBlocks = rq.max_num_blocks;
    p.window = l.window_size > 0 ? l.window_size : c->defaultWindow;
    p.dtype = l.data_type;
    p.poolBlocks = poolBlocksOf(rq.k_pool, rq.v_pool, l);
    p.counters = nullptr; p.countersCap = 0;
    // What the call needs of the built-in arrays: one counting word per (sequence, kv head)
    // pair (65 536 words) and records for the partial results: one per warp of the launch and
    // one per pair (8 MiB; the launch takes fewer warps when that is all the array holds, but
    // at least one CTA's worth).  The general kernel needs neither.
    const size_t pairs = std::min<size_t>(B, pam::kDecodeStreamMaxBatch) * static_cast<size_t>(l.num_kv_heads);
    const size_t words = pam::decodeStreamApplies(p) ? B * static_cast<size_t>(l.num_kv_heads) : 0;
    const size_t recordBytes = static_cast<size_t>(l.num_heads / l.num_kv_heads) * (static_cast<size_t>(l.head_dim) + 4) * sizeof(float);
    const size_t need = pam::decodeStreamApplies(p) ? std::min(pam::decodeWorkspaceBytes(p, c->smCount), (4 + pairs) * recordBytes) : 0;
    if (need > pam::decodeStaticScratchBytes() || words > (size_t(1) << 16))
        return c->fail(PAM_ERR_RESOURCE_EXHAUSTED,
                       "GPU resource exhausted: this decode needs " + std::to_string(need) +
                           " bytes of scratch for partial results and " + std::to_string(words) +
                           " counting words, the built-in arrays hold " +
                           std::to_string(pam::decodeStaticScratchBytes()) +
                           " bytes and 65536 words; use pamc_decode, or a smaller batch or fewer heads.");
    const double t0 = nowMs();
    // While the stream is being captured nothing may wait on it and nothing runs yet: the
    // launch is recorded once, without the wait and the retry loop of the eager call.
    cudaStreamCaptureStatus capture = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(c->stream, &capture) != cudaSuccess) { cudaGetLastError(); capture = cudaStreamCaptureStatusNone; }
    int32_t rc = 0;
    if (capture != cudaStreamCaptureStatusNone) {
        int launches = 0;
        cudaError_t e = pam::launchDecodeStatic(p, c->smCount, c->stream, &launches);
        c->launches += launches;
        if (e != cudaSuccess) {
            cudaGetLastError();
            return c->fail(PAM_ERR_COMMAND_EXECUTION, commandExecutionFailed(cudaGetErrorString(e)));
        }
    } else {
        rc = withRetry(c, "decodeFlat", [&]() -> cudaError_t {
            int launches = 0;
            cudaError_t e = pam::launchDecodeStatic(p, c->smCount, c->stream, &launches);
            c->launches += launches;
            return e;
        });
    }
    if (rc != 0) {
        if (!c->graceful) return rc;
        cudaMemsetAsync(rq.output.ptr, 0, rq.output.bytes != kUnknownBytes ? rq.output.bytes : B * ioBytesPerToken(l), c->stream);
        c->clearError();
    }
    c->stats = PamStats{PAM_OP_DECODE, rq.batch_size, 0, rq.max_num_blocks, static_cast<int64_t>(need), 0, nowMs() - t0};
    return 0;
}

struct PrefillSeq { int seqLen, qStart, qLen; };

int32_t prefillImpl(Context* c, const PamLayerSpec& l, const PamBuffer& q, const PamBuffer& kPool, const PamBuffer& vPool,
                    const PamBuffer& tables, const PamBuffer& output, const PamBuffer& kScale, const PamBuffer& vScale,
                    const std::vector<PrefillSeq>& seqs, int maxNumBlocks, bool causal, const char* tableName) {
    // PagedAttentionEngine.swift:405-528; validatePrefill :1897-1914
    if (!validateLayer(c, l)) return -1;
    int64_t totalRows = 0;
    int maxQLen = 0, maxSeqLen = 0;
    for (auto& s : seqs) {
        if (s.seqLen <= 0) return c->fail(PAM_ERR_INVALID_CONFIGURATION, invalidConfiguration("seqLen must be positive."));
        if (s.qStart < 0 || s.qLen <= 0 || s.qStart + s.qLen > s.seqLen)
            return c->fail(PAM_ERR_INVALID_CONFIGURATION, invalidConfiguration("chunk rows must lie inside the sequence."));
        totalRows += s.qLen;
        maxQLen = std::max(maxQLen, s.qLen);
        maxSeqLen = std::max(maxSeqLen, s.seqLen);
    }
    const size_t numBlocks = (static_cast<size_t>(maxSeqLen) + l.block_size - 1) / l.block_size;
    if (static_cast<size_t>(maxNumBlocks) < numBlocks)
        return c->fail(PAM_ERR_BUFFER_TOO_SMALL, bufferTooSmall(tableName, numBlocks * sizeof(int32_t), static_cast<size_t>(maxNumBlocks) * sizeof(int32_t)));
    if (!requireIoBuffer(c, q, "Q", static_cast<size_t>(totalRows) * qBytesPerToken(l), static_cast<size_t>(totalRows) * ioBytesPerToken(l))) return -1;
    if (!requireBuffer(c, tables, tableName, seqs.size() * static_cast<size_t>(maxNumBlocks) * sizeof(int32_t))) return -1;
    if (!requireIoBuffer(c, output, "output", static_cast<size_t>(totalRows) * qBytesPerToken(l), static_cast<size_t>(totalRows) * ioBytesPerToken(l))) return -1;
    if (!requireBuffer(c, kPool, "K pool", numBlocks * l.block_size * kvBytesPerToken(l))) return -1;
    if (!requireBuffer(c, vPool, "V pool", numBlocks * l.block_size * kvBytesPerToken(l))) return -1;
    if (l.data_type == PAM_DTYPE_FP8 && (!kScale.ptr || !vScale.ptr))
        return c->fail(PAM_ERR_INVALID_CONFIGURATION, invalidConfiguration("FP8 prefill needs kScaleBuffer and vScaleBuffer."));
    if (l.head_dim > 256)
        return c->fail(PAM_ERR_UNSUPPORTED, "Unsupported paged attention path: headDim above 256.");
    if (!isDevicePointer(kPool.ptr) || !isDevicePointer(vPool.ptr))
        return c->fail(PAM_ERR_INVALID_CONFIGURATION, invalidConfiguration("KV pools must be device memory."));

    const int window = l.window_size > 0 ? l.window_size : c->defaultWindow;     // :729
    const int n = static_cast<int>(seqs.size());
    std::vector<int32_t> meta(static_cast<size_t>(5) * n);
    int32_t rowOff = 0;
    for (int i = 0; i < n; ++i) {
        meta[i] = seqs[i].seqLen;
        meta[n + i] = seqs[i].qStart;
        meta[2 * n + i] = seqs[i].qLen;
        meta[3 * n + i] = rowOff;
        meta[4 * n + i] = window > 0 ? std::max(0, seqs[i].seqLen - window) : 0;   // :802, one start for all rows
        rowOff += seqs[i].qLen;
    }
    const size_t ioBytes = static_cast<size_t>(totalRows) * ioBytesPerToken(l);
    const double t0 = nowMs();
    c->arena.reset(c->stream);
    bool tensorPath = false;
    Stager st(c);
    int32_t rc = withRetry(c, "prefill", [&]() -> cudaError_t {
        pam::PrefillParams p{};
        // (Host queries and outputs go through copies in the arena, page-locked ones too.  Letting
        // the tensor-core kernel read and write page-locked host buffers in place through their
        // device-side addresses worked on single calls and then stalled a call for minutes after
        // some hundred calls in a row; it is not used.)
        p.q = st.in(q.ptr, ioBytes);
        p.kPool = kPool.ptr; p.vPool = vPool.ptr;
        p.tables = static_cast<const int32_t*>(st.in(tables.ptr, static_cast<size_t>(n) * maxNumBlocks * sizeof(int32_t)));
        p.out = st.out(output.ptr, ioBytes);
        p.kScale = kScale.ptr; p.vScale = vScale.ptr;
        if (n <= pam::kPrefillInlineSeqs) {
            p.inlineMeta = 1;
            for (int w = 0; w < 5; ++w)
                for (int i = 0; i < n; ++i) p.meta[w][i] = meta[static_cast<size_t>(w) * n + i];
        } else {
            const int32_t* dm = static_cast<const int32_t*>(st.upload(meta.data(), meta.size() * sizeof(int32_t)));
            if (!st.ok()) return cudaErrorMemoryAllocation;
            p.seqLens = dm; p.qStarts = dm + n; p.qLens = dm + 2 * n; p.qRowOffsets = dm + 3 * n; p.windowStarts = dm + 4 * n;
        }
        if (!st.ok()) return cudaErrorMemoryAllocation;
        p.numSeqs = n; p.maxQLen = maxQLen; p.heads = l.num_heads; p.kvHeads = l.num_kv_heads; p.headDim = l.head_dim;
        p.blockSize = l.block_size; p.maxNumBlocks = maxNumBlocks; p.causal = causal ? 1 : 0; p.dtype = l.data_type;
        p.poolBlocks = poolBlocksOf(kPool, vPool, l);
        p.totalRows = static_cast<int>(totalRows);
        p.errFlag = c->devErr;
        p.forceGeneral = c->forceGeneralPrefill ? 1 : 0;
        p.exactWeights = c->exactWeights;
        p.waitCycles = c->waitLimitCycles;
        p.starveV = 0;
        if (c->dropFirstVTile > 0) { c->dropFirstVTile -= 1; p.starveV = 1; }
        int launches = 0;
        if (pam::prefillFp8StagingApplies(p)) {
            // FP8 KV: the pages this launch can see are dequantised to float16 scratch pools
            // (the reference's all-half chain), which the tensor-core kernel then reads
            // through a table of scratch block numbers.
            int maxCount = 0;
            for (int i = 0; i < n; ++i) {
                const int lo = meta[static_cast<size_t>(4) * n + i] / l.block_size;
                const int hi = (meta[i] + l.block_size - 1) / l.block_size;
                maxCount = std::max(maxCount, hi - lo);
            }
            const size_t poolBytes = static_cast<size_t>(n) * maxCount * l.num_kv_heads * l.block_size * l.head_dim * 2;
            if (maxCount > 0 && poolBytes <= (size_t(1) << 30)) {
                const size_t tableBytes = static_cast<size_t>(n) * maxNumBlocks * sizeof(int32_t);
                void* kOut = c->arena.take(poolBytes);
                void* vOut = c->arena.take(poolBytes);
                int32_t* staged = static_cast<int32_t*>(c->arena.take(tableBytes));
                const int32_t* dm = static_cast<const int32_t*>(st.upload(meta.data(), meta.size() * sizeof(int32_t)));
                if (!kOut || !vOut || !staged || !st.ok()) return cudaErrorMemoryAllocation;
                cudaError_t se = cudaMemsetAsync(staged, 0, tableBytes, c->stream);
                if (se == cudaSuccess)
                    se = pam::launchFp8StagePages(p, dm, dm + static_cast<size_t>(4) * n, maxCount, kOut, vOut, staged, c->stream, &launches);
                if (se != cudaSuccess) return se;
                p.dtype = PAM_DTYPE_F16;
                p.kPool = kOut; p.vPool = vOut; p.tables = staged;
                p.kScale = nullptr; p.vScale = nullptr;
                p.poolBlocks = n * maxCount;
            }
        }
        cudaError_t e = pam::launchPrefill(p, c->smCount, c->stream, &launches, &tensorPath);
        c->launches += launches;
        if (e == cudaSuccess && tensorPath) {
            // the flag is fetched now when the call waits for the GPU anyway, else by pamc_synchronize
            if (!c->async) e = cudaMemcpyAsync(c->hostErr, c->devErr, sizeof(int), cudaMemcpyDeviceToHost, c->stream);
            c->errPending = true;
        }
        if (e == cudaSuccess) e = st.copyBack();
        // `meta` is read by an async copy from pageable memory, which the
        // runtime stages before returning; nothing else outlives this scope.
        return e;
    });
    if (rc != 0) {
        if (!c->graceful) return rc;
        st.zeroOutputs(output.ptr, output.bytes != kUnknownBytes ? output.bytes : ioBytes);       // :408-414
        c->clearError();
    }
    if (c->async && st.hasOutputs()) cudaStreamSynchronize(c->stream);
    c->stats = PamStats{tensorPath ? PAM_OP_PREFILL_MMA : PAM_OP_PREFILL_TILED, 1, maxSeqLen,
                        static_cast<int32_t>(numBlocks), 0, tensorPath ? 0 : 1, nowMs() - t0};      // :511-527
    return 0;
}

PamBuffer buf(const void* p, size_t bytes = kUnknownBytes) { return PamBuffer{const_cast<void*>(p), bytes}; }

PamLayerSpec layerOf(const Cache* k, int numHeads) {
    return PamLayerSpec{k->headDim, numHeads, k->kvHeads, k->blockSize, k->dtype, 0};
}

Cache* createCache(Context* c, int32_t maxBlocks, int32_t blockSize, int32_t headDim, int32_t kvHeads, int32_t dtype) {
    Cache* k = new Cache(maxBlocks, blockSize);
    k->device = c->device; k->dtype = dtype; k->headDim = headDim; k->kvHeads = kvHeads;
    k->poolBytes = static_cast<size_t>(maxBlocks) * k->blockBytes();            // KVCacheManager.swift:91-92
    cudaError_t e = cudaMalloc(&k->kPool, k->poolBytes);
    if (e == cudaSuccess) e = cudaMalloc(&k->vPool, k->poolBytes);
    if (e == cudaSuccess) e = cudaMemsetAsync(k->kPool, 0, k->poolBytes, c->stream);
    if (e == cudaSuccess) e = cudaMemsetAsync(k->vPool, 0, k->poolBytes, c->stream);
    if (e == cudaSuccess && dtype == PAM_DTYPE_FP8) {
        k->scaleBytes = static_cast<size_t>(maxBlocks) * kvHeads * 2;
        e = cudaMalloc(&k->kScale, k->scaleBytes);
        if (e == cudaSuccess) e = cudaMalloc(&k->vScale, k->scaleBytes);
        if (e == cudaSuccess) e = cudaMemsetAsync(k->kScale, 0, k->scaleBytes, c->stream);   // scales start at zero
        if (e == cudaSuccess) e = cudaMemsetAsync(k->vScale, 0, k->scaleBytes, c->stream);
    }
    if (e == cudaSuccess) e = cudaStreamSynchronize(c->stream);
    if (e != cudaSuccess) {
        cudaGetLastError();
        c->fail(PAM_ERR_COMMAND_ENCODING, "Metal command encoding failed: Failed to allocate KV pool buffers");   // KVCacheManager.swift:96
        delete k;
        return nullptr;
    }
    return k;
}

int32_t syncContext(Context* c) {
    cudaError_t e = cudaSuccess;
    if (c->errPending) e = cudaMemcpyAsync(c->hostErr, c->devErr, sizeof(int), cudaMemcpyDeviceToHost, c->stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(c->stream);
    if (e != cudaSuccess) { cudaGetLastError(); return c->fail(PAM_ERR_COMMAND_EXECUTION, commandExecutionFailed(cudaGetErrorString(e))); }
    if (c->errPending) {
        c->errPending = false;
        if (*c->hostErr != 0) {
            const int site = *c->hostErr;
            *c->hostErr = 0;
            cudaMemsetAsync(c->devErr, 0, sizeof(int), c->stream);
            return c->fail(PAM_ERR_COMMAND_EXECUTION, commandExecutionFailed("a kernel's bounded wait ran out (site " + std::to_string(site) + ")"));
        }
    }
    return 0;
}

// The *Layers calls (PagedAttentionEngine.swift:1433-1895) run the same operation once per
// layer and wait once at the end.  Here each layer's request is enqueued on the context's
// stream without a wait in between, and the stream is waited for once (unless the context
// is in async mode, where the caller waits).
template <class Rq, class F>
int32_t runLayers(void* ctx, const Rq* requests, int32_t numLayers, F one) {
    if (!ctx) return -1;
    Context* c = asCtx(ctx);
    std::lock_guard<std::mutex> g(c->mu);
    DeviceGuard dg(c->device);
    if (c->device < 0) return noGpu(c);
    if (!requests || numLayers <= 0) return c->fail(PAM_ERR_INVALID_CONFIGURATION, invalidConfiguration("buffer/layer count mismatch"));
    const bool wasAsync = c->async;
    c->async = true;
    int32_t rc = 0;
    const double t0 = nowMs();
    for (int i = 0; i < numLayers && rc == 0; ++i) rc = one(c, requests[i], i);
    c->async = wasAsync;
    if (!wasAsync) {
        const int32_t src = syncContext(c);
        if (rc == 0) rc = src;
    }
    if (rc == 0) {
        c->stats.elapsed_ms = nowMs() - t0;
        c->clearError();
    }
    return rc;
}

}  // namespace

// ======================================================================= C ABI

extern "C" {

int32_t pamc_device_count(void) {
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess) { cudaGetLastError(); return 0; }
    return n;
}

void* pamc_create_context_on(int32_t device) {
    int n = pamc_device_count();
    if (device < 0 || device >= n) return nullptr;                // deviceInitializationFailed
    if (cudaSetDevice(device) != cudaSuccess) { cudaGetLastError(); return nullptr; }
    Context* c = new Context();
    c->device = device;
    cudaDeviceProp prop{};
    if (cudaGetDeviceProperties(&prop, device) == cudaSuccess) c->smCount = prop.multiProcessorCount;
    if (cudaStreamCreateWithFlags(&c->ownStream, cudaStreamNonBlocking) != cudaSuccess) {
        cudaGetLastError();
        delete c;
        return nullptr;
    }
    c->stream = c->ownStream;
    if (cudaMalloc(reinterpret_cast<void**>(&c->devErr), sizeof(int)) != cudaSuccess ||
        cudaMemset(c->devErr, 0, sizeof(int)) != cudaSuccess ||
        cudaMallocHost(reinterpret_cast<void**>(&c->hostErr), sizeof(int)) != cudaSuccess) {
        cudaGetLastError();
        if (c->devErr) cudaFree(c->devErr);
        cudaStreamDestroy(c->ownStream);
        delete c;
        return nullptr;
    }
    *c->hostErr = 0;
    constexpr int64_t kCounters = 1 << 16;
    if (cudaMalloc(reinterpret_cast<void**>(&c->mergeCounters), kCounters * sizeof(int)) == cudaSuccess &&
        cudaMemset(c->mergeCounters, 0, kCounters * sizeof(int)) == cudaSuccess) {
        c->mergeCountersCap = kCounters;
    } else {
        // (asked for again by the first decode)
        cudaGetLastError();
        if (c->mergeCounters) cudaFree(c->mergeCounters);
        c->mergeCounters = nullptr;
    }
    return c;
}

void* pamc_create_host_context(void) {
    Context* c = new Context();
    c->device = -1;
    return c;
}

void* pam_create_context(void) {
    int dev = 0;
    if (pamc_device_count() <= 0) return nullptr;
    if (cudaGetDevice(&dev) != cudaSuccess) { cudaGetLastError(); return nullptr; }
    return pamc_create_context_on(dev);
}

void pam_destroy_context(void* ctx) {
    if (!ctx) return;
    Context* c = asCtx(ctx);
    if (c->device < 0) { delete c; return; }
    cudaSetDevice(c->device);
    cudaStreamSynchronize(c->stream);
    c->arena.release();
    if (c->devErr) cudaFree(c->devErr);
    if (c->hostErr) cudaFreeHost(c->hostErr);
    if (c->pinned) cudaFreeHost(c->pinned);
    if (c->qStage) cudaFree(c->qStage);
    if (c->outStage) cudaFree(c->outStage);
    if (c->mergeCounters) cudaFree(c->mergeCounters);
    if (c->ownStream) cudaStreamDestroy(c->ownStream);
    delete c;
}

const char* pam_last_error(void* ctx) {
    if (!ctx) return nullptr;
    Context* c = asCtx(ctx);
    return c->hasError ? c->lastError.c_str() : nullptr;
}

int32_t pamc_last_error_code(void* ctx) { return ctx ? asCtx(ctx)->lastCode : PAM_ERR_NULL_HANDLE; }

void* pam_create_cache(void* ctx, int32_t max_blocks, int32_t block_size, int32_t head_dim, int32_t num_kv_heads,
                       int32_t data_type) {
    if (!ctx) return nullptr;
    Context* c = asCtx(ctx);
    std::lock_guard<std::mutex> g(c->mu);
    DeviceGuard dg(c->device);
    if (c->device < 0) { noGpu(c); return nullptr; }
    PamLayerSpec l{head_dim, num_kv_heads, num_kv_heads, block_size, data_type, 0};   // CABI.swift:107-114
    if (!validateLayer(c, l)) return nullptr;
    if (max_blocks <= 0) { c->fail(PAM_ERR_INVALID_CONFIGURATION, invalidConfiguration("maxBlocks must be positive")); return nullptr; }
    Cache* k = createCache(c, max_blocks, block_size, head_dim, num_kv_heads, data_type);
    if (k) c->clearError();
    return k;
}

void* pamc_cache_create_bookkeeping(int32_t max_blocks, int32_t block_size) {
    if (max_blocks <= 0 || block_size <= 0) return nullptr;
    Cache* k = new Cache(max_blocks, block_size);
    k->bookkeeping = true;
    return k;
}

void pam_destroy_cache(void* cache) { delete asCache(cache); }

int32_t pam_reserve_sequence(void* ctx, void* cache, int64_t id) {
    if (!ctx || !cache) return -1;
    Context* c = asCtx(ctx);
    std::lock_guard<std::mutex> g(c->mu);
    KVResult r = asCache(cache)->mgr.allocateSequence(id);
    if (!r.ok()) return kvFail(c, r);
    c->clearError();
    return 0;
}

// The log of copy-on-write pairs is for callers that mirror the copies elsewhere (another
// GPU's pools, a test); one that never drains it must not grow without bound: beyond this
// many pairs the oldest are dropped.
constexpr size_t kCowLogLimit = size_t(1) << 16;
static void logCopies(Cache* k, const std::vector<std::pair<int32_t, int32_t>>& cow) {
    if (cow.empty()) return;
    std::lock_guard<std::mutex> gk(k->mu);
    k->cowLog.insert(k->cowLog.end(), cow.begin(), cow.end());
    if (k->cowLog.size() > kCowLogLimit) k->cowLog.erase(k->cowLog.begin(), k->cowLog.end() - static_cast<std::ptrdiff_t>(kCowLogLimit));
}

int32_t pamc_cache_append_tokens(void* ctx, void* cache, int64_t id, int32_t count, const uint64_t* hashes,
                                 int32_t num_hashes) {
    if (!ctx || !cache) return -1;
    Context* c = asCtx(ctx);
    Cache* k = asCache(cache);
    std::lock_guard<std::mutex> g(c->mu);
    std::vector<std::pair<int32_t, int32_t>> cow;
    KVResult r = k->mgr.appendTokens(id, count, hashes, hashes ? num_hashes : 0, &cow);
    logCopies(k, cow);
    // An append that failed after its copy-on-write (the reference's order,
    // KVCacheManager.swift:134-146) has left the sequence's table as it was: the fresh
    // block is in no table, so there is nothing to copy into it.
    if (r.ok() && !cow.empty() && !k->bookkeeping) {
        DeviceGuard dg(c->device);
        if (c->device < 0) return noGpu(c);
        c->arena.reset(c->stream);
        if (runCopies(c, k, cow) != 0) return -1;
    }
    if (!r.ok()) return kvFail(c, r);
    c->clearError();
    return 0;
}

int32_t pam_append_tokens(void* ctx, void* cache, int64_t id, int32_t count) {
    return pamc_cache_append_tokens(ctx, cache, id, count, nullptr, 0);
}

int32_t pamc_cache_ensure_exclusive(void* ctx, void* cache, int64_t id, int32_t logical_block) {
    if (!ctx || !cache) return -1;
    Context* c = asCtx(ctx);
    Cache* k = asCache(cache);
    std::lock_guard<std::mutex> g(c->mu);
    std::vector<std::pair<int32_t, int32_t>> cow;
    KVResult r = k->mgr.ensureExclusiveAccess(id, logical_block, &cow);
    logCopies(k, cow);
    if (r.ok() && !cow.empty() && !k->bookkeeping) {
        DeviceGuard dg(c->device);
        if (c->device < 0) return noGpu(c);
        c->arena.reset(c->stream);
        if (runCopies(c, k, cow) != 0) return -1;
    }
    if (!r.ok()) return kvFail(c, r);
    c->clearError();
    return 0;
}

void pamc_cache_register_block_hash(void* cache, uint64_t hash, int32_t physical_block) {
    if (cache) asCache(cache)->mgr.registerBlockHash(hash, physical_block);
}

void pam_free_sequence(void* cache, int64_t id) {
    if (cache) asCache(cache)->mgr.freeSequence(id);
}

int32_t pam_available_blocks(void* cache) { return cache ? asCache(cache)->mgr.availableBlocks() : -1; }

int32_t pam_sequence_length(void* ctx, void* cache, int64_t id) {
    if (!ctx || !cache) return -1;
    Context* c = asCtx(ctx);
    std::lock_guard<std::mutex> g(c->mu);
    int64_t len = 0;
    KVResult r = asCache(cache)->mgr.sequenceLength(id, &len);
    if (!r.ok()) return kvFail(c, r);
    c->clearError();
    return static_cast<int32_t>(len);
}

int32_t pamc_cache_block_table(void* ctx, void* cache, int64_t id, int32_t* out, int32_t capacity) {
    if (!ctx || !cache) return -1;
    Context* c = asCtx(ctx);
    std::lock_guard<std::mutex> g(c->mu);
    std::vector<int32_t> t;
    KVResult r = asCache(cache)->mgr.blockTable(id, &t);
    if (!r.ok()) return kvFail(c, r);
    if (out) for (int i = 0; i < capacity && i < static_cast<int>(t.size()); ++i) out[i] = t[static_cast<size_t>(i)];
    c->clearError();
    return static_cast<int32_t>(t.size());
}

int32_t pamc_cache_num_blocks(void* ctx, void* cache, int64_t id) {
    return pamc_cache_block_table(ctx, cache, id, nullptr, 0);
}

int32_t pamc_cache_active_sequences(void* cache) { return cache ? asCache(cache)->mgr.activeSequences() : -1; }

int32_t pamc_cache_set_eviction_policy(void* cache, int32_t policy) {
    if (!cache || policy < 0 || policy > 2) return -1;
    asCache(cache)->mgr.setPolicy(policy);
    return 0;
}

int32_t pamc_cache_set_hygiene(void* cache, int32_t on) {
    if (!cache) return -1;
    asCache(cache)->mgr.setHygiene(on != 0);
    return 0;
}

// Chained content hash of the full blocks of a token sequence: hash j covers the ids of
// blocks 0 .. j (64-bit FNV-1a over the ids, continued from the hash of the block before),
// so equal hashes mean equal prefixes up to a 64-bit collision.
int32_t pamc_block_hashes(const int32_t* token_ids, int32_t num_tokens, int32_t block_size, uint64_t seed, uint64_t* out,
                          int32_t capacity) {
    if (!token_ids || num_tokens < 0 || block_size <= 0) return -1;
    const int full = num_tokens / block_size;
    uint64_t h = 0xcbf29ce484222325ull ^ seed;
    for (int j = 0; j < full; ++j) {
        for (int t = 0; t < block_size; ++t) {
            uint32_t v = static_cast<uint32_t>(token_ids[static_cast<size_t>(j) * block_size + t]);
            for (int byte = 0; byte < 4; ++byte) {
                h ^= v & 0xFFu;
                h *= 0x100000001b3ull;
                v >>= 8;
            }
        }
        if (out && j < capacity) out[j] = h;
    }
    return full;
}

int32_t pamc_cache_memory_stats(void* cache, PamMemoryStats* out) {
    if (!cache || !out) return -1;
    Cache* k = asCache(cache);
    pam::MemoryStats s = k->mgr.stats();
    const int64_t bytesPerBlock = k->bookkeeping ? 0 : static_cast<int64_t>(k->blockBytes()) * 2;   // KVCacheManager.swift:357
    out->total_blocks = s.totalBlocks; out->used_blocks = s.usedBlocks; out->free_blocks = s.freeBlocks;
    out->active_sequences = s.activeSequences;
    out->total_memory_bytes = s.totalBlocks * bytesPerBlock; out->used_memory_bytes = s.usedBlocks * bytesPerBlock;
    out->partially_filled_blocks = s.partiallyFilledBlocks; out->fragmentation_ratio = s.fragmentationRatio;
    out->prefix_cache_hits = s.prefixCacheHits; out->prefix_cache_entries = s.prefixCacheEntries;
    out->shared_blocks = s.sharedBlocks; out->eviction_policy = s.policy;
    return 0;
}

int32_t pamc_cache_pools(void* cache, void** k_pool, void** v_pool, void** k_scale, void** v_scale,
                         size_t* pool_bytes, size_t* scale_bytes) {
    if (!cache) return -1;
    Cache* k = asCache(cache);
    if (k_pool) *k_pool = k->kPool;
    if (v_pool) *v_pool = k->vPool;
    if (k_scale) *k_scale = k->kScale;
    if (v_scale) *v_scale = k->vScale;
    if (pool_bytes) *pool_bytes = k->poolBytes;
    if (scale_bytes) *scale_bytes = k->scaleBytes;
    return 0;
}

int32_t pamc_cache_drain_cow_log(void* cache, int32_t* out_pairs, int32_t capacity) {
    if (!cache) return -1;
    Cache* k = asCache(cache);
    std::lock_guard<std::mutex> g(k->mu);
    int n = static_cast<int>(std::min<size_t>(k->cowLog.size(), static_cast<size_t>(std::max(capacity, 0))));
    for (int i = 0; i < n; ++i) {
        out_pairs[2 * i] = k->cowLog[static_cast<size_t>(i)].first;
        out_pairs[2 * i + 1] = k->cowLog[static_cast<size_t>(i)].second;
    }
    k->cowLog.erase(k->cowLog.begin(), k->cowLog.begin() + n);
    return n;
}

static int32_t buildBatchTables(Context* c, Cache* k, const int64_t* ids, int32_t n, int32_t maxNumBlocks,
                                std::vector<int32_t>* tables, std::vector<uint32_t>* lens, int* maxLen) {
    tables->assign(static_cast<size_t>(n) * maxNumBlocks, 0);   // zero padding, CABI.swift:360-363
    lens->assign(static_cast<size_t>(n), 0);
    if (maxLen) *maxLen = 0;
    std::vector<int32_t> t;
    for (int i = 0; i < n; ++i) {
        KVResult r = k->mgr.blockTable(ids[i], &t);
        if (!r.ok()) return kvFail(c, r);
        if (static_cast<int>(t.size()) > maxNumBlocks)           // KVCacheManager.swift:675-677
            return c->fail(PAM_ERR_KV_INVALID_REQUEST,
                           "KVCacheError.invalidRequest(\"sequence " + std::to_string(ids[i]) + " requires " +
                               std::to_string(t.size()) + " blocks, maxSequenceBlocks is " + std::to_string(maxNumBlocks) + "\")");
        std::copy(t.begin(), t.end(), tables->begin() + static_cast<std::ptrdiff_t>(i) * maxNumBlocks);
        int64_t len = 0;
        k->mgr.sequenceLength(ids[i], &len);
        (*lens)[static_cast<size_t>(i)] = static_cast<uint32_t>(len);
        if (maxLen) *maxLen = std::max(*maxLen, static_cast<int>(len));
    }
    return 0;
}

int32_t pamc_cache_batch_tables(void* ctx, void* cache, const int64_t* ids, int32_t n, int32_t max_num_blocks,
                                int32_t* tables, uint32_t* lens) {
    if (!ctx || !cache || !ids || n < 0 || max_num_blocks <= 0) return -1;
    Context* c = asCtx(ctx);
    std::lock_guard<std::mutex> g(c->mu);
    std::vector<int32_t> t;
    std::vector<uint32_t> l;
    if (buildBatchTables(c, asCache(cache), ids, n, max_num_blocks, &t, &l, nullptr) != 0) return -1;
    DeviceGuard dg(c->device);
    auto put = [&](void* dst, const void* src, size_t bytes) -> bool {
        if (!dst || bytes == 0) return true;
        if (c->device < 0 || !isDevicePointer(dst)) { std::memcpy(dst, src, bytes); return true; }
        return cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, c->stream) == cudaSuccess &&
               cudaStreamSynchronize(c->stream) == cudaSuccess;
    };
    if (!put(tables, t.data(), t.size() * sizeof(int32_t)) || !put(lens, l.data(), l.size() * sizeof(uint32_t)))
        return c->fail(PAM_ERR_COMMAND_EXECUTION, commandExecutionFailed("copy of batch tables failed"));
    c->clearError();
    return 0;
}

int32_t pamc_cache_slot_mapping(void* ctx, void* cache, int64_t id, int32_t token_offset, int32_t num_tokens,
                                int64_t* out) {
    if (!ctx || !cache || !out) return -1;
    Context* c = asCtx(ctx);
    Cache* k = asCache(cache);
    std::lock_guard<std::mutex> g(c->mu);
    std::vector<int32_t> t;
    KVResult r = k->mgr.blockTable(id, &t);
    if (!r.ok()) return kvFail(c, r);
    const int bs = k->blockSize;
    if (token_offset < 0 || num_tokens < 0 ||
        (static_cast<int64_t>(token_offset) + num_tokens + bs - 1) / bs > static_cast<int64_t>(t.size()))
        return c->fail(PAM_ERR_KV_INVALID_REQUEST, "KVCacheError.invalidRequest(\"tokens lie outside the block table\")");
    for (int i = 0; i < num_tokens; ++i) {
        const int pos = token_offset + i;                         // kernels.metal:1823-1827
        out[i] = static_cast<int64_t>(t[static_cast<size_t>(pos / bs)]) * bs + pos % bs;
    }
    c->clearError();
    return 0;
}

// ------------------------------------------------------------------ engine knobs

int32_t pamc_set_stream(void* ctx, void* cuda_stream) {
    if (!ctx) return -1;
    Context* c = asCtx(ctx);
    std::lock_guard<std::mutex> g(c->mu);
    if (c->device < 0) return noGpu(c);
    cudaStreamSynchronize(c->stream);
    c->stream = cuda_stream ? static_cast<cudaStream_t>(cuda_stream) : c->ownStream;
    return 0;
}
int32_t pamc_set_async(void* ctx, int32_t enabled) { if (!ctx) return -1; asCtx(ctx)->async = enabled != 0; return 0; }
int32_t pamc_synchronize(void* ctx) {
    if (!ctx) return -1;
    Context* c = asCtx(ctx);
    DeviceGuard dg(c->device);
    if (c->device < 0) return noGpu(c);
    return syncContext(c);
}
int32_t pamc_set_max_retries(void* ctx, int32_t n) { if (!ctx || n < 0) return -1; asCtx(ctx)->maxRetries = n; return 0; }
int32_t pamc_set_graceful_degradation(void* ctx, int32_t on) { if (!ctx) return -1; asCtx(ctx)->graceful = on != 0; return 0; }
int32_t pamc_set_split_threshold(void* ctx, int32_t t) { if (!ctx) return -1; asCtx(ctx)->splitThreshold = t; return 0; }
int32_t pamc_set_prefill_tensor_path(void* ctx, int32_t on) { if (!ctx) return -1; asCtx(ctx)->forceGeneralPrefill = on == 0; return 0; }
int32_t pamc_set_prefill_exact_weights(void* ctx, int32_t mode) { if (!ctx || mode < 0 || mode > 2) return -1; asCtx(ctx)->exactWeights = mode; return 0; }
int32_t pamc_set_default_window(void* ctx, int32_t t) { if (!ctx || t < 0) return -1; asCtx(ctx)->defaultWindow = t; return 0; }
int32_t pamc_set_default_chunk(void* ctx, int32_t t) { if (!ctx || t < 0) return -1; asCtx(ctx)->defaultChunk = t; return 0; }
int32_t pamc_inject_launch_failures(void* ctx, int32_t n) { if (!ctx || n < 0) return -1; asCtx(ctx)->injectFailures = n; return 0; }
int64_t pamc_kernel_launches(void* ctx) { return ctx ? asCtx(ctx)->launches : -1; }
int32_t pamc_set_wait_limit(void* ctx, int64_t sm_cycles) { if (!ctx || sm_cycles < 0) return -1; asCtx(ctx)->waitLimitCycles = sm_cycles; return 0; }
int32_t pamc_test_starve_prefill(void* ctx, int32_t launches) { if (!ctx || launches < 0) return -1; asCtx(ctx)->dropFirstVTile = launches; return 0; }

int32_t pamc_last_stats(void* ctx, PamStats* out) {
    if (!ctx || !out) return -1;
    Context* c = asCtx(ctx);
    std::lock_guard<std::mutex> g(c->mu);
    *out = c->stats;
    return 0;
}

int64_t pamc_recommended_max_blocks(void* ctx, int32_t block_size, int32_t num_kv_heads, int32_t head_dim,
                                    int32_t data_type, float memory_fraction, int32_t layer_count) {
    if (!ctx || !validDtype(data_type)) return -1;
    Context* c = asCtx(ctx);
    DeviceGuard dg(c->device);
    if (c->device < 0) return noGpu(c);
    size_t freeB = 0, totalB = 0;
    if (cudaMemGetInfo(&freeB, &totalB) != cudaSuccess) { cudaGetLastError(); return -1; }
    // PagedAttentionEngine.swift:201-217: fraction * budget / (bytes per block, K and V, all layers), at least 1
    const double perBlock = static_cast<double>(block_size) * num_kv_heads * head_dim * pam::elemBytes(data_type) * 2.0 *
                            std::max(layer_count, 1);
    if (perBlock <= 0) return 1;
    const int64_t n = static_cast<int64_t>(static_cast<double>(memory_fraction) * static_cast<double>(freeB) / perBlock);
    return std::max<int64_t>(n, 1);
}

void* pamc_buffer_alloc(void* ctx, size_t bytes) {
    if (!ctx) return nullptr;
    Context* c = asCtx(ctx);
    DeviceGuard dg(c->device);
    if (c->device < 0) { noGpu(c); return nullptr; }
    void* p = nullptr;
    if (cudaMalloc(&p, std::max<size_t>(bytes, 1)) != cudaSuccess) { cudaGetLastError(); return nullptr; }
    return p;
}
void pamc_buffer_free(void* ctx, void* ptr) {
    if (!ctx || !ptr) return;
    DeviceGuard dg(asCtx(ctx)->device);
    cudaFree(ptr);
}
int32_t pamc_memcpy(void* ctx, void* dst, const void* src, size_t bytes, int32_t kind) {
    if (!ctx) return -1;
    Context* c = asCtx(ctx);
    DeviceGuard dg(c->device);
    if (c->device < 0) return noGpu(c);
    cudaMemcpyKind k = kind == 0 ? cudaMemcpyHostToDevice : kind == 1 ? cudaMemcpyDeviceToHost : cudaMemcpyDeviceToDevice;
    cudaError_t e = cudaMemcpyAsync(dst, src, bytes, k, c->stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(c->stream);
    if (e != cudaSuccess) { cudaGetLastError(); return c->fail(PAM_ERR_COMMAND_EXECUTION, commandExecutionFailed(cudaGetErrorString(e))); }
    return 0;
}

// ------------------------------------------------------------------ operations

int32_t pamc_append_to_cache(void* ctx, const PamAppendRequest* request) {
    if (!ctx || !request) return -1;
    Context* c = asCtx(ctx);
    std::lock_guard<std::mutex> g(c->mu);
    DeviceGuard dg(c->device);
    if (c->device < 0) return noGpu(c);
    if (request->layer.data_type == PAM_DTYPE_FP8)
        return c->fail(PAM_ERR_UNSUPPORTED, "Unsupported paged attention path: FP8 append goes through a cache handle (pam_append_kv or pamc_reshape_and_cache), which owns the absmax scratch.");
    int32_t rc = appendImpl(c, *request, nullptr, nullptr);
    if (rc == 0) c->clearError();
    return rc;
}

int32_t pam_append_kv(void* ctx, void* cache, int64_t id, void* keys, void* values, int32_t token_offset,
                      int32_t num_new_tokens, int32_t num_heads) {
    if (!ctx || !cache || !keys || !values) return -1;           // CABI.swift:214-219
    Context* c = asCtx(ctx);
    Cache* k = asCache(cache);
    std::lock_guard<std::mutex> g(c->mu);
    DeviceGuard dg(c->device);
    if (c->device < 0) return noGpu(c);
    if (k->bookkeeping) return c->fail(PAM_ERR_INVALID_STATE, "Invalid engine state: cache has no pools");
    std::vector<int32_t> table;
    KVResult r = k->mgr.blockTable(id, &table);
    if (!r.ok()) return kvFail(c, r);
    PamAppendRequest rq{};
    rq.keys = buf(keys); rq.values = buf(values);
    rq.k_pool = buf(k->kPool, k->poolBytes); rq.v_pool = buf(k->vPool, k->poolBytes);
    // getBlockTableBuffer pads an empty table to one entry (KVCacheManager.swift:310)
    rq.block_table = buf(table.data(), std::max<size_t>(table.size(), 1) * sizeof(int32_t));
    rq.token_offset = token_offset; rq.num_new_tokens = num_new_tokens;
    rq.layer = layerOf(k, num_heads);
    rq.k_scale = buf(k->kScale, k->scaleBytes); rq.v_scale = buf(k->vScale, k->scaleBytes);
    // The table is known on the host: derive the slots here after the same checks.
    std::vector<int64_t> slots;
    if (token_offset >= 0 && num_new_tokens > 0) {
        const size_t need = (static_cast<size_t>(token_offset) + num_new_tokens + k->blockSize - 1) / k->blockSize;
        if (need * sizeof(int32_t) > rq.block_table.bytes)
            return c->fail(PAM_ERR_BUFFER_TOO_SMALL, bufferTooSmall("blockTable", need * sizeof(int32_t), rq.block_table.bytes));
        slots.resize(static_cast<size_t>(num_new_tokens));
        for (int i = 0; i < num_new_tokens; ++i) {
            const int pos = token_offset + i;
            slots[static_cast<size_t>(i)] = static_cast<int64_t>(table[static_cast<size_t>(pos / k->blockSize)]) * k->blockSize + pos % k->blockSize;
        }
    }
    int32_t rc = appendImpl(c, rq, k, slots.empty() ? nullptr : slots.data());
    if (rc == 0) c->clearError();
    return rc;
}

int32_t pamc_reshape_and_cache(void* ctx, void* cache, const void* keys, const void* values,
                               const int64_t* slot_mapping, int32_t num_tokens) {
    if (!ctx || !cache || !keys || !values || !slot_mapping) return -1;
    Context* c = asCtx(ctx);
    Cache* k = asCache(cache);
    std::lock_guard<std::mutex> g(c->mu);
    DeviceGuard dg(c->device);
    if (c->device < 0) return noGpu(c);
    if (k->bookkeeping) return c->fail(PAM_ERR_INVALID_STATE, "Invalid engine state: cache has no pools");
    if (num_tokens <= 0) return c->fail(PAM_ERR_INVALID_CONFIGURATION, invalidConfiguration("numNewTokens must be positive."));
    PamAppendRequest rq{};
    rq.keys = buf(keys); rq.values = buf(values);
    rq.k_pool = buf(k->kPool, k->poolBytes); rq.v_pool = buf(k->vPool, k->poolBytes);
    rq.block_table = buf(nullptr, 0);
    rq.token_offset = 0; rq.num_new_tokens = num_tokens;
    rq.layer = layerOf(k, k->kvHeads);
    rq.k_scale = buf(k->kScale, k->scaleBytes); rq.v_scale = buf(k->vScale, k->scaleBytes);
    // Host slot lists are checked here; device lists are checked by the kernel,
    // which skips tokens whose slot lies outside the pool.
    const bool onDevice = isDevicePointer(slot_mapping);
    if (!onDevice) {
        const int64_t poolSlots = static_cast<int64_t>(k->maxBlocks) * k->blockSize;
        for (int i = 0; i < num_tokens; ++i)
            if (slot_mapping[i] < 0 || slot_mapping[i] >= poolSlots)
                return c->fail(PAM_ERR_INVALID_CONFIGURATION, invalidConfiguration("slot " + std::to_string(slot_mapping[i]) + " lies outside the pool"));
    }
    // appendImpl's pool lower bound is counted from token_offset + tokens; the
    // slots were checked against the pool above, so keep that bound trivial.
    rq.num_new_tokens = num_tokens;
    PamAppendRequest small = rq;
    small.k_pool.bytes = kUnknownBytes; small.v_pool.bytes = kUnknownBytes;
    int32_t rc = appendImpl(c, small, k, onDevice ? nullptr : slot_mapping, onDevice ? slot_mapping : nullptr);
    if (rc == 0) c->clearError();
    return rc;
}

int32_t pamc_copy_blocks(void* ctx, void* cache, const int32_t* src, const int32_t* dst, int32_t n) {
    if (!ctx || !cache || (n > 0 && (!src || !dst))) return -1;
    Context* c = asCtx(ctx);
    Cache* k = asCache(cache);
    std::lock_guard<std::mutex> g(c->mu);
    DeviceGuard dg(c->device);
    if (c->device < 0) return noGpu(c);
    if (k->bookkeeping) return c->fail(PAM_ERR_INVALID_STATE, "Invalid engine state: cache has no pools");
    std::vector<std::pair<int32_t, int32_t>> pairs;
    for (int i = 0; i < n; ++i) {
        if (src[i] < 0 || src[i] >= k->maxBlocks || dst[i] < 0 || dst[i] >= k->maxBlocks)
            return c->fail(PAM_ERR_INVALID_CONFIGURATION, invalidConfiguration("block index outside the pool"));
        pairs.emplace_back(src[i], dst[i]);
    }
    c->arena.reset(c->stream);
    int32_t rc = runCopies(c, k, pairs);
    if (rc == 0) c->clearError();
    return rc;
}

int32_t pamc_decode(void* ctx, const PamDecodeRequest* request) {
    if (!ctx || !request) return -1;
    Context* c = asCtx(ctx);
    std::lock_guard<std::mutex> g(c->mu);
    DeviceGuard dg(c->device);
    int32_t rc = decodeImpl(c, *request);
    if (rc == 0) c->clearError();
    return rc;
}

int32_t pamc_decode_path(const PamDecodeRequest* request) {
    if (!request) return -1;
    const PamDecodeRequest& rq = *request;
    pam::DecodeParams p{};
    p.q = rq.q.ptr; p.kPool = rq.k_pool.ptr; p.vPool = rq.v_pool.ptr; p.out = rq.output.ptr;
    p.kScale = rq.k_scale.ptr; p.vScale = rq.v_scale.ptr;
    p.heads = rq.layer.num_heads; p.kvHeads = rq.layer.num_kv_heads; p.headDim = rq.layer.head_dim;
    p.blockSize = rq.layer.block_size; p.dtype = rq.layer.data_type;
    p.batch = rq.batch_size > 0 ? rq.batch_size : 1;
    p.maxNumBlocks = rq.max_num_blocks > 0 ? rq.max_num_blocks : 1;
    if (p.kvHeads <= 0 || p.heads <= 0 || p.blockSize <= 0) return -1;
    return pam::decodeTakesStreamPath(p) ? 1 : 0;
}

int32_t pamc_decode_noalloc(void* ctx, const PamDecodeRequest* request) {
    if (!ctx || !request) return -1;
    Context* c = asCtx(ctx);
    std::lock_guard<std::mutex> g(c->mu);
    DeviceGuard dg(c->device);
    int32_t rc = decodeNoAllocImpl(c, *request);
    if (rc == 0) c->clearError();
    return rc;
}

// Brings the device copy of the batch's block tables and lengths up to date
// (CABI.swift:306-330, 339-372 build and upload all of it on every call).  Row i of the copy
// belongs to batch_ids[i]; a row is sent again in full when it holds another sequence, or
// one whose existing entries were replaced (copy-on-write, free and re-allocation), and only
// from its old end on when the table merely grew.  The lengths go up every time.
static int32_t refreshResidentTables(Context* c, Cache* k, const int64_t* ids, int B, int* maxNumBlocks, int* maxLen,
                                     size_t* uploadedBytes) {
    Cache::Resident& r = k->res;
    std::lock_guard<std::mutex> gk(k->mu);
    auto fail = [&](cudaError_t e) {
        cudaGetLastError();
        r.ids.clear(); r.versions.clear(); r.counts.clear();
        return c->fail(PAM_ERR_COMMAND_EXECUTION, commandExecutionFailed(cudaGetErrorString(e)));
    };
    cudaError_t e = cudaSuccess;
    if (!r.consumed) {
        e = cudaEventCreateWithFlags(&r.consumed, cudaEventDisableTiming);
        if (e != cudaSuccess) return fail(e);
    } else {
        e = cudaEventSynchronize(r.consumed);        // the staging block is about to be rewritten
        if (e != cudaSuccess) return fail(e);
    }
    std::vector<int32_t> patches;
    std::vector<uint32_t> lens(static_cast<size_t>(B));
    for (int attempt = 0; attempt < 2; ++attempt) {
        patches.clear();
        if (static_cast<int>(r.ids.size()) < B) {
            r.ids.resize(static_cast<size_t>(B), INT64_MIN);
            r.versions.resize(static_cast<size_t>(B), 0);
            r.counts.resize(static_cast<size_t>(B), 0);
        }
        int widest = 1, longest = 0;                  // CABI.swift:308
        KVResult kr = k->mgr.visit(ids, B, [&](int i, const pam::SequenceView& v) {
            const size_t si = static_cast<size_t>(i);
            const bool keep = r.ids[si] == ids[i] && r.versions[si] == v.rewriteVersion && r.counts[si] <= v.numBlocks;
            for (int col = keep ? r.counts[si] : 0; col < v.numBlocks; ++col) {
                patches.push_back(i); patches.push_back(col); patches.push_back(v.table[col]);
            }
            r.ids[si] = ids[i]; r.versions[si] = v.rewriteVersion; r.counts[si] = v.numBlocks;
            lens[si] = static_cast<uint32_t>(v.length);
            widest = std::max(widest, static_cast<int>(v.numBlocks));
            longest = std::max(longest, static_cast<int>(v.length));
        });
        if (!kr.ok()) {
            r.ids.clear(); r.versions.clear(); r.counts.clear();   // rows up to the unknown id were marked as sent
            return kvFail(c, kr);
        }
        *maxNumBlocks = widest;
        *maxLen = longest;
        if (widest <= r.stride && B <= r.rows) break;
        // a wider or taller table: new device block, every row goes up again
        cudaStreamSynchronize(c->stream);
        cudaFree(r.tables);
        r.tables = nullptr;
        r.rows = std::max(B, r.rows);
        r.stride = std::max((widest + widest / 4 + 63) / 64 * 64, r.stride);
        e = cudaMalloc(reinterpret_cast<void**>(&r.tables), static_cast<size_t>(r.rows) * r.stride * sizeof(int32_t));
        if (e != cudaSuccess) { r.rows = r.stride = 0; return fail(e); }
        r.ids.assign(static_cast<size_t>(r.rows), INT64_MIN);
    }
    const size_t lenBytes = (static_cast<size_t>(B) * sizeof(uint32_t) + 15) & ~static_cast<size_t>(15);
    const size_t numPatches = patches.size() / 3;
    const size_t tableBytes = static_cast<size_t>(B) * r.stride * sizeof(int32_t);
    // many changes (a new batch): the rows go up whole, zero padded, which is fewer bytes
    const bool whole = patches.size() * sizeof(int32_t) > tableBytes;
    const size_t need = lenBytes + (whole ? tableBytes : patches.size() * sizeof(int32_t));
    if (need > r.pinnedCap) {
        if (r.pinned) cudaFreeHost(r.pinned);
        r.pinned = nullptr; r.pinnedCap = 0;
        const size_t cap = need + need / 2 + 4096;
        e = cudaHostAlloc(reinterpret_cast<void**>(&r.pinned), cap, cudaHostAllocDefault);
        if (e != cudaSuccess) return fail(e);
        r.pinnedCap = cap;
    }
    const size_t devNeed = lenBytes + (whole ? 0 : patches.size() * sizeof(int32_t));
    if (devNeed > r.uploadCap) {
        cudaStreamSynchronize(c->stream);
        cudaFree(r.upload);
        r.upload = nullptr; r.uploadCap = 0;
        const size_t cap = devNeed + devNeed / 2 + 4096;
        e = cudaMalloc(reinterpret_cast<void**>(&r.upload), cap);
        if (e != cudaSuccess) return fail(e);
        r.uploadCap = cap;
    }
    std::memcpy(r.pinned, lens.data(), static_cast<size_t>(B) * sizeof(uint32_t));
    int32_t* staged = reinterpret_cast<int32_t*>(r.pinned + lenBytes);
    if (whole) {
        std::memset(staged, 0, tableBytes);                       // zero padding, CABI.swift:360-363
        for (size_t t = 0; t < numPatches; ++t)
            staged[static_cast<size_t>(patches[3 * t]) * r.stride + patches[3 * t + 1]] = patches[3 * t + 2];
        e = cudaMemcpyAsync(r.upload, r.pinned, lenBytes, cudaMemcpyHostToDevice, c->stream);
        if (e == cudaSuccess) e = cudaMemcpyAsync(r.tables, staged, tableBytes, cudaMemcpyHostToDevice, c->stream);
    } else {
        if (numPatches) std::memcpy(staged, patches.data(), patches.size() * sizeof(int32_t));
        e = cudaMemcpyAsync(r.upload, r.pinned, need, cudaMemcpyHostToDevice, c->stream);
        int launches = 0;
        if (e == cudaSuccess)
            e = pam::launchPatchTables(r.tables, r.stride, reinterpret_cast<const int32_t*>(reinterpret_cast<unsigned char*>(r.upload) + lenBytes),
                                       static_cast<int>(numPatches), c->stream, &launches);
        c->launches += launches;
    }
    if (e == cudaSuccess) e = cudaEventRecord(r.consumed, c->stream);
    if (e != cudaSuccess) return fail(e);
    *uploadedBytes = need;
    return 0;
}

int32_t pam_decode(void* ctx, void* cache, const int64_t* batch_ids, int32_t batch_size, void* q, void* out,
                   int32_t num_heads) {
    if (!ctx || !cache || !batch_ids || !q || !out) return -1;   // CABI.swift:299-305
    Context* c = asCtx(ctx);
    Cache* k = asCache(cache);
    std::lock_guard<std::mutex> g(c->mu);
    DeviceGuard dg(c->device);
    if (c->device < 0) return noGpu(c);
    if (k->bookkeeping) return c->fail(PAM_ERR_INVALID_STATE, "Invalid engine state: cache has no pools");
    const PamLayerSpec layer = layerOf(k, num_heads);
    // PagedAttentionEngine.swift:533-580; validateDecode :1916-1933
    if (!validateLayer(c, layer)) return -1;
    if (batch_size <= 0) return c->fail(PAM_ERR_INVALID_CONFIGURATION, invalidConfiguration("batchSize must be positive."));
    if (layer.head_dim > 256) return c->fail(PAM_ERR_UNSUPPORTED, "Unsupported paged attention path: headDim above 256.");
    const double t0 = nowMs();
    const size_t ioBytes = static_cast<size_t>(batch_size) * ioBytesPerToken(layer);
    // each argument is looked at once: device memory is used in place; a page-locked host
    // output is written by the kernels themselves through its device-side address; a host
    // query, and a pageable host output, go through a device block the context keeps
    const Placement qAt = placementOf(q), outAt = placementOf(out);
    auto deviceBlock = [&](void*& block, size_t& cap) -> bool {
        if (ioBytes <= cap) return true;
        cudaStreamSynchronize(c->stream);
        if (block) cudaFree(block);
        block = nullptr; cap = 0;
        if (cudaMalloc(&block, ioBytes) != cudaSuccess) { cudaGetLastError(); block = nullptr; return false; }
        cap = ioBytes;
        return true;
    };
    bool callerMemoryInFlight = false;
    // every return below leaves no copy from or to the caller's memory behind
    auto failed = [&](int32_t rc) {
        if (callerMemoryInFlight) cudaStreamSynchronize(c->stream);
        return rc;
    };
    const void* qDev = q;
    if (!qAt.onDevice) {
        // the query goes up first, so that its copy runs while the tables are put together
        if (!deviceBlock(c->qStage, c->qStageCap)) return c->fail(PAM_ERR_RESOURCE_EXHAUSTED, "GPU resource exhausted: query staging block");
        cudaError_t e = cudaMemcpyAsync(c->qStage, q, ioBytes, cudaMemcpyHostToDevice, c->stream);
        if (e != cudaSuccess) { cudaGetLastError(); return c->fail(PAM_ERR_COMMAND_EXECUTION, commandExecutionFailed(cudaGetErrorString(e))); }
        qDev = c->qStage;
        callerMemoryInFlight = true;
    }
    void* outDev = outAt.device;
    if (!outDev) {
        if (!deviceBlock(c->outStage, c->outStageCap)) return failed(c->fail(PAM_ERR_RESOURCE_EXHAUSTED, "GPU resource exhausted: output staging block"));
        outDev = c->outStage;
    }
    int maxNumBlocks = 1, maxLen = 0;
    size_t uploaded = 0;
    if (int32_t rc = refreshResidentTables(c, k, batch_ids, batch_size, &maxNumBlocks, &maxLen, &uploaded)) return failed(rc);
    // validateDecode's pool bound uses maxNumBlocks (a lower bound, PagedAttentionEngine.swift:1931)
    const size_t poolNeed = static_cast<size_t>(maxNumBlocks) * layer.block_size * kvBytesPerToken(layer);
    if (k->poolBytes < poolNeed) return failed(c->fail(PAM_ERR_BUFFER_TOO_SMALL, bufferTooSmall("K pool", poolNeed, k->poolBytes)));

    pam::DecodeParams p{};
    p.q = qDev; p.kPool = k->kPool; p.vPool = k->vPool;
    p.tables = k->res.tables;
    p.lens = k->res.upload;
    p.out = outDev;
    p.kScale = k->kScale; p.vScale = k->vScale;
    p.batch = batch_size; p.heads = num_heads; p.kvHeads = k->kvHeads; p.headDim = k->headDim;
    p.blockSize = k->blockSize; p.maxNumBlocks = k->res.stride; p.window = c->defaultWindow; p.dtype = k->dtype;   // :1028
    p.poolBlocks = k->maxBlocks;
    if (!ensureMergeCounters(c, static_cast<int64_t>(batch_size) * k->kvHeads))
        return failed(c->fail(PAM_ERR_RESOURCE_EXHAUSTED, "GPU resource exhausted: counting words of the decode kernel"));
    p.counters = c->mergeCounters;
    p.countersCap = c->mergeCountersCap;
    c->arena.reset(c->stream);
    size_t tempBytes = 0;
    int32_t rc = withRetry(c, "decodeFlat", [&]() -> cudaError_t {
        tempBytes = pam::decodeWorkspaceBytes(p, c->smCount);
        if (tempBytes) {
            p.workspace = static_cast<float*>(c->arena.take(tempBytes));
            p.workspaceBytes = tempBytes;
            if (!p.workspace) return cudaErrorMemoryAllocation;
        }
        int launches = 0;
        cudaError_t e = pam::launchDecode(p, c->smCount, c->stream, &launches);
        c->launches += launches;
        if (e == cudaSuccess && outDev == c->outStage) {
            e = cudaMemcpyAsync(out, outDev, ioBytes, cudaMemcpyDeviceToHost, c->stream);
            callerMemoryInFlight = true;
        }
        return e;
    });
    if (rc != 0) {
        if (c->mergeCounters) cudaMemsetAsync(c->mergeCounters, 0, static_cast<size_t>(c->mergeCountersCap) * sizeof(int), c->stream);
        cudaStreamSynchronize(c->stream);
        callerMemoryInFlight = false;
        if (!c->graceful) return rc;
        if (outAt.onDevice) cudaMemsetAsync(out, 0, ioBytes, c->stream);       // :536-542
        else std::memset(out, 0, ioBytes);
        c->clearError();
    }
    // host memory of the caller's (the query on its way up, the output on its way down or
    // being written by the kernels) must be settled before this call returns; the
    // synchronous mode has waited already
    if (c->async && (!qAt.onDevice || !outAt.onDevice)) cudaStreamSynchronize(c->stream);
    c->stats = PamStats{PAM_OP_DECODE, batch_size, 0, maxNumBlocks, static_cast<int64_t>(tempBytes), 0, nowMs() - t0};   // :568-577
    c->clearError();
    return 0;
}

int32_t pamc_prefill(void* ctx, const PamPrefillRequest* request, int32_t chunk_size) {
    if (!ctx || !request) return -1;
    Context* c = asCtx(ctx);
    std::lock_guard<std::mutex> g(c->mu);
    DeviceGuard dg(c->device);
    if (c->device < 0) return noGpu(c);
    const PamPrefillRequest& rq = *request;
    if (rq.seq_len <= 0) return c->fail(PAM_ERR_INVALID_CONFIGURATION, invalidConfiguration("seqLen must be positive."));
    const int qLen = rq.q_len > 0 ? rq.q_len : rq.seq_len;
    const int qStart = rq.q_len > 0 ? rq.q_start : 0;
    const int chunk = chunk_size > 0 ? chunk_size : c->defaultChunk;            // PagedAttentionEngine.swift:730
    const int maxNumBlocks = rq.block_table.bytes != kUnknownBytes
                                 ? static_cast<int>(std::min<size_t>(rq.block_table.bytes / sizeof(int32_t), 1u << 30))
                                 : (rq.seq_len + std::max(rq.layer.block_size, 1) - 1) / std::max(rq.layer.block_size, 1);
    int32_t rc = 0;
    if (chunk > 0 && qLen > chunk && validDtype(rq.layer.data_type) && rq.layer.num_heads > 0 && rq.layer.head_dim > 0) {
        // PagedAttentionEngine.swift:740-756, each row computed once.
        const size_t rowBytes = ioBytesPerToken(rq.layer);
        for (int cs = 0; cs < qLen && rc == 0; cs += chunk) {
            const int n = std::min(chunk, qLen - cs);
            PamBuffer q = rq.q, o = rq.output;
            q.ptr = static_cast<char*>(q.ptr) + static_cast<size_t>(cs) * rowBytes;
            o.ptr = static_cast<char*>(o.ptr) + static_cast<size_t>(cs) * rowBytes;
            if (q.bytes != kUnknownBytes) q.bytes = q.bytes > static_cast<size_t>(cs) * rowBytes ? q.bytes - static_cast<size_t>(cs) * rowBytes : 0;
            if (o.bytes != kUnknownBytes) o.bytes = o.bytes > static_cast<size_t>(cs) * rowBytes ? o.bytes - static_cast<size_t>(cs) * rowBytes : 0;
            rc = prefillImpl(c, rq.layer, q, rq.k_pool, rq.v_pool, rq.block_table, o, rq.k_scale, rq.v_scale,
                             {PrefillSeq{rq.seq_len, qStart + cs, n}}, maxNumBlocks, rq.causal != 0, "blockTable");
        }
    } else {
        rc = prefillImpl(c, rq.layer, rq.q, rq.k_pool, rq.v_pool, rq.block_table, rq.output, rq.k_scale, rq.v_scale,
                         {PrefillSeq{rq.seq_len, qStart, qLen}}, maxNumBlocks, rq.causal != 0, "blockTable");
    }
    if (rc == 0) c->clearError();
    return rc;
}

int32_t pamc_prefill_batch(void* ctx, const PamBatchPrefillRequest* request) {
    if (!ctx || !request) return -1;
    Context* c = asCtx(ctx);
    std::lock_guard<std::mutex> g(c->mu);
    DeviceGuard dg(c->device);
    if (c->device < 0) return noGpu(c);
    const PamBatchPrefillRequest& rq = *request;
    if (rq.num_sequences <= 0 || !rq.seq_lens || !rq.q_starts || !rq.q_lens)
        return c->fail(PAM_ERR_INVALID_CONFIGURATION, invalidConfiguration("batchSize must be positive."));
    std::vector<PrefillSeq> seqs;
    for (int i = 0; i < rq.num_sequences; ++i) seqs.push_back({rq.seq_lens[i], rq.q_starts[i], rq.q_lens[i]});
    int32_t rc = prefillImpl(c, rq.layer, rq.q, rq.k_pool, rq.v_pool, rq.block_tables, rq.output, rq.k_scale, rq.v_scale,
                             seqs, rq.max_num_blocks, rq.causal != 0, "blockTables");
    if (rc == 0) c->clearError();
    return rc;
}

int32_t pamc_fused_prefill(void* ctx, const PamFusedPrefillRequest* request, void* cache) {
    // PagedAttentionEngine.swift:633-710.  The reference's kernels (kernels.metal:1963-2340)
    // have every threadgroup rewrite the whole sequence into the pools before its own
    // attention rows; here the rows are written once by the append kernels and the
    // prefill kernel follows on the same stream.
    if (!ctx || !request) return -1;
    Context* c = asCtx(ctx);
    std::lock_guard<std::mutex> g(c->mu);
    DeviceGuard dg(c->device);
    if (c->device < 0) return noGpu(c);
    const PamFusedPrefillRequest& rq = *request;
    if (!validateLayer(c, rq.layer)) return -1;
    if (rq.seq_len <= 0) return c->fail(PAM_ERR_INVALID_CONFIGURATION, invalidConfiguration("seqLen must be positive."));
    const PamLayerSpec& l = rq.layer;
    const size_t numBlocks = (static_cast<size_t>(rq.seq_len) + l.block_size - 1) / l.block_size;
    if (!requireBuffer(c, rq.block_table, "blockTable", numBlocks * sizeof(int32_t))) return -1;
    if (!requireIoBuffer(c, rq.output, "output", static_cast<size_t>(rq.seq_len) * qBytesPerToken(l), static_cast<size_t>(rq.seq_len) * ioBytesPerToken(l))) return -1;
    Cache* k = cache ? asCache(cache) : nullptr;
    if (l.data_type == PAM_DTYPE_FP8 && !k)
        return c->fail(PAM_ERR_INVALID_CONFIGURATION, invalidConfiguration("FP8 fused prefill needs the cache handle that owns the scale buffers."));
    const double t0 = nowMs();
    PamAppendRequest ap{};
    ap.keys = rq.raw_k; ap.values = rq.raw_v;
    ap.k_pool = rq.k_pool; ap.v_pool = rq.v_pool;
    ap.block_table = rq.block_table;
    ap.token_offset = 0; ap.num_new_tokens = rq.seq_len;
    ap.layer = l;
    ap.k_scale = rq.k_scale; ap.v_scale = rq.v_scale;
    int32_t rc = appendImpl(c, ap, k, nullptr);
    if (rc != 0) return rc;
    const int maxNumBlocks = rq.block_table.bytes != kUnknownBytes
                                 ? static_cast<int>(std::min<size_t>(rq.block_table.bytes / sizeof(int32_t), 1u << 30))
                                 : static_cast<int>(numBlocks);
    rc = prefillImpl(c, l, rq.q, rq.k_pool, rq.v_pool, rq.block_table, rq.output, rq.k_scale, rq.v_scale,
                     {PrefillSeq{rq.seq_len, 0, rq.seq_len}}, maxNumBlocks, rq.causal != 0, "blockTable");
    if (rc != 0) return rc;
    // the reference reports the fused call as a single pass over the sequence (:697-706)
    c->stats = PamStats{PAM_OP_PREFILL_SINGLE_PASS, 1, rq.seq_len, static_cast<int32_t>(numBlocks), 0, 0, nowMs() - t0};
    c->clearError();
    return 0;
}

int32_t pamc_backward(void* ctx, const PamBackwardRequest* request) {
    // PagedAttentionEngine.backward (PagedAttentionEngine.swift:1341-1395); kernels.metal:1217-1415
    if (!ctx || !request) return -1;
    Context* c = asCtx(ctx);
    std::lock_guard<std::mutex> g(c->mu);
    DeviceGuard dg(c->device);
    const PamBackwardRequest& rq = *request;
    const PamLayerSpec& l = rq.layer;
    if (!validateLayer(c, l)) return -1;
    if (rq.seq_len <= 0) return c->fail(PAM_ERR_INVALID_CONFIGURATION, invalidConfiguration("seqLen must be positive."));
    // the reference has a float32 and a float16 pipeline (:1366); bfloat16 is this library's addition
    if (l.data_type == PAM_DTYPE_FP8)
        return c->fail(PAM_ERR_UNSUPPORTED, "Unsupported paged attention path: backward over an FP8 cache.");
    if (l.head_dim > 256) return c->fail(PAM_ERR_UNSUPPORTED, "Unsupported paged attention path: headDim above 256.");
    const size_t rows = static_cast<size_t>(rq.seq_len);
    const size_t numBlocks = (rows + l.block_size - 1) / l.block_size;
    const size_t ioBytes = rows * ioBytesPerToken(l), statBytes = rows * l.num_heads * sizeof(float);
    const size_t poolNeed = numBlocks * l.block_size * kvBytesPerToken(l);
    if (!requireBuffer(c, rq.q, "Q", ioBytes)) return -1;
    if (!requireBuffer(c, rq.d_out, "dO", ioBytes)) return -1;
    if (!requireBuffer(c, rq.m, "m", statBytes)) return -1;
    if (!requireBuffer(c, rq.l, "l", statBytes)) return -1;
    if (!requireBuffer(c, rq.d_q, "dQ", ioBytes)) return -1;
    if (!requireBuffer(c, rq.block_table, "blockTable", numBlocks * sizeof(int32_t))) return -1;
    if (!requireBuffer(c, rq.k_pool, "K pool", poolNeed)) return -1;
    if (!requireBuffer(c, rq.v_pool, "V pool", poolNeed)) return -1;
    if (!requireBuffer(c, rq.d_k_pool, "dK pool", poolNeed)) return -1;
    if (!requireBuffer(c, rq.d_v_pool, "dV pool", poolNeed)) return -1;
    if (c->device < 0) return noGpu(c);
    const void* pools[] = {rq.k_pool.ptr, rq.v_pool.ptr, rq.d_k_pool.ptr, rq.d_v_pool.ptr};
    for (const void* ptr : pools)
        if (!isDevicePointer(ptr))
            return c->fail(PAM_ERR_INVALID_CONFIGURATION, invalidConfiguration("KV pools and their gradient pools must be device memory."));
    const int window = l.window_size > 0 ? l.window_size : 0;                 // (the call's own windowSize, :1358; no engine default)
    const int maxNumBlocks = rq.block_table.bytes != kUnknownBytes
                                 ? static_cast<int>(std::min<size_t>(rq.block_table.bytes / sizeof(int32_t), 1u << 30))
                                 : static_cast<int>(numBlocks);
    const double t0 = nowMs();
    c->arena.reset(c->stream);
    Stager st(c);
    size_t tempBytes = 0;
    int32_t rc = withRetry(c, "backward", [&]() -> cudaError_t {
        pam::BackwardParams p{};
        p.q = st.in(rq.q.ptr, ioBytes);
        p.dO = st.in(rq.d_out.ptr, ioBytes);
        p.m = static_cast<const float*>(st.in(rq.m.ptr, statBytes));
        p.l = static_cast<const float*>(st.in(rq.l.ptr, statBytes));
        p.table = static_cast<const int32_t*>(st.in(rq.block_table.ptr, static_cast<size_t>(maxNumBlocks) * sizeof(int32_t)));
        p.dQ = st.out(rq.d_q.ptr, ioBytes);
        p.kPool = rq.k_pool.ptr; p.vPool = rq.v_pool.ptr; p.dKPool = rq.d_k_pool.ptr; p.dVPool = rq.d_v_pool.ptr;
        p.seqLen = rq.seq_len; p.heads = l.num_heads; p.kvHeads = l.num_kv_heads; p.headDim = l.head_dim;
        p.blockSize = l.block_size; p.dtype = l.data_type;
        p.windowStart = window > 0 ? std::max(0, rq.seq_len - window) : 0;    // :1380
        p.maxNumBlocks = maxNumBlocks;
        const int kPoolBlocks = poolBlocksOf(rq.k_pool, rq.v_pool, l), dPoolBlocks = poolBlocksOf(rq.d_k_pool, rq.d_v_pool, l);
        p.poolBlocks = std::min(kPoolBlocks, dPoolBlocks);
        if (!st.ok()) return cudaErrorMemoryAllocation;
        tempBytes = pam::backwardWorkspaceBytes(p);
        unsigned char* ws = static_cast<unsigned char*>(c->arena.take(tempBytes));
        if (!ws) return cudaErrorMemoryAllocation;
        p.rowSum = reinterpret_cast<float*>(ws);
        const size_t rowSumBytes = (statBytes + 255) / 256 * 256;
        p.dQAcc = l.data_type == PAM_DTYPE_F32 ? static_cast<float*>(p.dQ) : reinterpret_cast<float*>(ws + rowSumBytes);
        int launches = 0;
        cudaError_t e = pam::launchBackward(p, c->stream, &launches);
        c->launches += launches;
        if (e == cudaSuccess) e = st.copyBack();
        return e;
    });
    if (rc != 0) {
        if (!c->graceful) return rc;
        st.zeroOutputs(rq.d_q.ptr, rq.d_q.bytes != kUnknownBytes ? rq.d_q.bytes : ioBytes);
        c->clearError();
    }
    if (c->async && st.hasOutputs()) cudaStreamSynchronize(c->stream);
    c->stats = PamStats{PAM_OP_BACKWARD, 1, rq.seq_len, static_cast<int32_t>(numBlocks), static_cast<int64_t>(tempBytes), 0, nowMs() - t0};
    return 0;
}

int32_t pamc_decode_layers(void* ctx, const PamDecodeRequest* requests, int32_t num_layers) {
    return runLayers(ctx, requests, num_layers, [](Context* c, const PamDecodeRequest& rq, int) { return decodeImpl(c, rq); });
}

int32_t pamc_prefill_layers(void* ctx, const PamPrefillRequest* requests, int32_t num_layers) {
    return runLayers(ctx, requests, num_layers, [](Context* c, const PamPrefillRequest& rq, int) -> int32_t {
        if (rq.seq_len <= 0) return c->fail(PAM_ERR_INVALID_CONFIGURATION, invalidConfiguration("seqLen must be positive."));
        const int qLen = rq.q_len > 0 ? rq.q_len : rq.seq_len;
        const int qStart = rq.q_len > 0 ? rq.q_start : 0;
        const int bs = std::max(rq.layer.block_size, 1);
        const int maxNumBlocks = rq.block_table.bytes != kUnknownBytes
                                     ? static_cast<int>(std::min<size_t>(rq.block_table.bytes / sizeof(int32_t), 1u << 30))
                                     : (rq.seq_len + bs - 1) / bs;
        return prefillImpl(c, rq.layer, rq.q, rq.k_pool, rq.v_pool, rq.block_table, rq.output, rq.k_scale, rq.v_scale,
                           {PrefillSeq{rq.seq_len, qStart, qLen}}, maxNumBlocks, rq.causal != 0, "blockTable");
    });
}

int32_t pamc_append_layers(void* ctx, const PamAppendRequest* requests, int32_t num_layers, void* const* caches) {
    return runLayers(ctx, requests, num_layers, [caches](Context* c, const PamAppendRequest& rq, int i) -> int32_t {
        Cache* k = caches && caches[i] ? asCache(caches[i]) : nullptr;
        if (rq.layer.data_type == PAM_DTYPE_FP8 && !k)
            return c->fail(PAM_ERR_INVALID_CONFIGURATION, invalidConfiguration("FP8 append needs the cache handle that owns the scale buffers."));
        return appendImpl(c, rq, k, nullptr);
    });
}

int32_t pam_prefill(void* ctx, void* cache, int64_t id, void* q, void* out, int32_t seq_len, int32_t num_heads,
                    bool causal) {
    if (!ctx || !cache || !q || !out) return -1;                 // CABI.swift:257-262
    Context* c = asCtx(ctx);
    Cache* k = asCache(cache);
    std::vector<int32_t> table;
    {
        std::lock_guard<std::mutex> g(c->mu);
        if (k->bookkeeping) return c->fail(PAM_ERR_INVALID_STATE, "Invalid engine state: cache has no pools");
        KVResult r = k->mgr.blockTable(id, &table);
        if (!r.ok()) return kvFail(c, r);
    }
    if (table.empty()) table.push_back(0);                        // KVCacheManager.swift:310
    PamPrefillRequest rq{};
    rq.q = buf(q); rq.output = buf(out);
    rq.k_pool = buf(k->kPool, k->poolBytes); rq.v_pool = buf(k->vPool, k->poolBytes);
    rq.block_table = buf(table.data(), table.size() * sizeof(int32_t));
    rq.seq_len = seq_len; rq.layer = layerOf(k, num_heads); rq.causal = causal ? 1 : 0;
    rq.k_scale = buf(k->kScale, k->scaleBytes); rq.v_scale = buf(k->vScale, k->scaleBytes);
    int32_t rc = pamc_prefill(ctx, &rq, 0);
    if (rc == 0 && c->async) cudaStreamSynchronize(c->stream);    // `table` is read by an async copy
    return rc;
}

// ------------------------------------------------------------------ head-sharded outputs

int32_t pamc_comm_unique_id(void* out_128_bytes) { return pam::commUniqueId(out_128_bytes) == 0 ? 0 : -1; }

void* pamc_comm_create(void* ctx, const void* unique_id_128_bytes, int32_t rank, int32_t num_ranks) {
    if (!ctx) return nullptr;
    Context* c = asCtx(ctx);
    std::lock_guard<std::mutex> g(c->mu);
    DeviceGuard dg(c->device);
    if (c->device < 0) { noGpu(c); return nullptr; }
    std::string why;
    pam::HeadComm* comm = pam::commCreate(unique_id_128_bytes, rank, num_ranks, c->device, &why);
    if (!comm) { c->fail(PAM_ERR_DEVICE_INIT, "Metal device or command queue could not be initialized: " + why); return nullptr; }
    c->clearError();
    return comm;
}

void pamc_comm_destroy(void* comm) { pam::commDestroy(static_cast<pam::HeadComm*>(comm)); }

int32_t pamc_allgather_heads(void* ctx, void* comm, const void* local, void* full, int32_t rows, int32_t heads_local,
                             int32_t head_dim, int32_t data_type) {
    if (!ctx || !comm || !local || !full) return -1;
    Context* c = asCtx(ctx);
    std::lock_guard<std::mutex> g(c->mu);
    DeviceGuard dg(c->device);
    if (c->device < 0) return noGpu(c);
    if (rows <= 0 || heads_local <= 0 || head_dim <= 0 || !validDtype(data_type))
        return c->fail(PAM_ERR_INVALID_CONFIGURATION, invalidConfiguration("rows, heads and headDim must be positive."));
    pam::HeadComm* hc = static_cast<pam::HeadComm*>(comm);
    const size_t slice = static_cast<size_t>(heads_local) * head_dim * pam::ioBytes(data_type);
    if (slice % 16 != 0)
        return c->fail(PAM_ERR_UNSUPPORTED, "Unsupported paged attention path: a GPU's head slice must be a multiple of 16 bytes.");
    if (!isDevicePointer(local) || !isDevicePointer(full))
        return c->fail(PAM_ERR_INVALID_CONFIGURATION, invalidConfiguration("the gathered tensors must be device memory."));
    c->arena.reset(c->stream);
    // A collective is not retried: the other ranks would not take part in the second attempt.
    std::string why;
    void* staging = pam::commSize(hc) > 1 ? c->arena.take(static_cast<size_t>(pam::commSize(hc)) * rows * slice) : const_cast<void*>(local);
    if (!staging) return c->fail(PAM_ERR_RESOURCE_EXHAUSTED, "GPU resource exhausted: staging block of the all-gather");
    int launches = 0;
    cudaError_t e = pam::launchAllGatherHeads(hc, local, staging, full, rows, slice, c->stream, &launches, &why);
    c->launches += launches;
    if (e == cudaSuccess && !c->async) e = cudaStreamSynchronize(c->stream);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return c->fail(PAM_ERR_COMMAND_EXECUTION, commandExecutionFailed(why.empty() ? cudaGetErrorString(e) : why));
    }
    c->clearError();
    return 0;
}

// ------------------------------------------------------------------ scheduler

void* pamc_sched_create(int32_t max_batch_size, int32_t max_sequences) { return new Sched(max_batch_size, max_sequences); }
void pamc_sched_destroy(void* s) { delete static_cast<Sched*>(s); }
int64_t pamc_sched_add_request(void* s, int32_t prompt, int32_t max_new) { return s ? static_cast<Sched*>(s)->s.addRequest(prompt, max_new) : -1; }
void pamc_sched_complete(void* s, int64_t id) { if (s) static_cast<Sched*>(s)->s.complete(id); }
int32_t pamc_sched_step(void* s, int64_t* out_ids, int32_t capacity) {
    if (!s) return -1;
    std::vector<int64_t> b = static_cast<Sched*>(s)->s.step();
    for (int i = 0; i < capacity && i < static_cast<int>(b.size()); ++i) out_ids[i] = b[static_cast<size_t>(i)];
    return static_cast<int32_t>(b.size());
}
void pamc_sched_mark_prefilled(void* s, int64_t id) { if (s) static_cast<Sched*>(s)->s.markPrefilled(id); }
void pamc_sched_mark_decoded(void* s, int64_t id) { if (s) static_cast<Sched*>(s)->s.markDecoded(id); }
void pamc_sched_preempt(void* s, int64_t id) { if (s) static_cast<Sched*>(s)->s.preempt(id); }
int32_t pamc_sched_handle_memory_pressure(void* s, int32_t required_blocks, pamc_available_fn available, void* user,
                                          int64_t* out_ids, int32_t capacity) {
    if (!s || !available) return -1;
    std::vector<int64_t> v = static_cast<Sched*>(s)->s.handleMemoryPressure(required_blocks, [&]() { return available(user); });
    for (int i = 0; i < capacity && i < static_cast<int>(v.size()); ++i) out_ids[i] = v[static_cast<size_t>(i)];
    return static_cast<int32_t>(v.size());
}
int32_t pamc_sched_count(void* s, int32_t status) { return s ? static_cast<Sched*>(s)->s.count(status) : -1; }
int32_t pamc_sched_total(void* s) { return s ? static_cast<Sched*>(s)->s.total() : -1; }
int32_t pamc_sched_get(void* s, int64_t id, PamSchedSequence* out) {
    if (!s || !out) return -1;
    pam::SchedulerSequence q;
    if (!static_cast<Sched*>(s)->s.get(id, &q)) return -1;
    out->id = q.id; out->status = q.status; out->num_generated_tokens = q.numGeneratedTokens;
    out->max_new_tokens = q.maxNewTokens; out->prompt_length = q.promptLength; out->arrival_order = q.arrivalOrder;
    return 0;
}

// ------------------------------------------------------------------ inference orchestration
// PagedAttentionInference (PagedAttentionInference.swift:7-299): scheduler + cache + engine
// driven step by step.  Like the reference it has no model: the queries are zeroed buffers
// and nothing is appended to the pools; what it exercises is the scheduling, the block
// bookkeeping and the batched-layer attention launches.

struct Inference {
    Context* c = nullptr;
    Cache* cache = nullptr;
    Sched* sched = nullptr;
    std::vector<PamLayerSpec> layers;
    int maxBatch = 0;
    bool incrementalPreemption = false;
    bool batchedPrefill = false;                      // one prefill launch per layer and step (not in the reference)
    int prefillTokenBudget = 0;                       // prompt rows per step with batchedPrefill; 0: no limit
    std::map<int64_t, int> prefillProgress;           // rows done of a prompt that spans steps
    long long prefillLaunchSets = 0;                  // prefill launch sets (one per layer set) issued so far
    std::set<int64_t> prefilled;                      // :29
    long long totalTokens = 0;                        // :31
    int stepCount = 0;                                // :34
    pamc_token_fn onToken = nullptr;                  // :27
    void* onTokenUser = nullptr;
    std::mutex mu;
    std::vector<void*> q, out;                        // per layer, grown on demand
    std::vector<size_t> cap;
    ~Inference() {
        if (c && c->device >= 0) {
            cudaSetDevice(c->device);
            cudaStreamSynchronize(c->stream);
            for (void* p : q) cudaFree(p);
            for (void* p : out) cudaFree(p);
        }
        delete sched;
        delete cache;
    }
};

static int32_t inferFail(Inference* inf, int code, const std::string& m) {
    std::lock_guard<std::mutex> g(inf->c->mu);
    return inf->c->fail(code, m);
}
static int32_t inferKvFail(Inference* inf, const KVResult& r) {
    std::lock_guard<std::mutex> g(inf->c->mu);
    return kvFail(inf->c, r);
}

// zeroed query rows and an output buffer per layer (the reference makes fresh shared
// buffers every step, PagedAttentionInference.swift:190-202, 241-253).  Sized by the type
// the queries really have: float16 for an FP8 layer, where the reference's
// qBytesPerToken counts one byte per element.
static int32_t inferBuffers(Inference* inf, size_t rows) {
    Context* c = inf->c;
    DeviceGuard dg(c->device);
    for (size_t l = 0; l < inf->layers.size(); ++l) {
        const size_t need = std::max<size_t>(rows * ioBytesPerToken(inf->layers[l]), 16);
        if (inf->cap[l] < need) {
            cudaStreamSynchronize(c->stream);
            cudaFree(inf->q[l]); cudaFree(inf->out[l]);
            inf->q[l] = inf->out[l] = nullptr; inf->cap[l] = 0;
            cudaError_t e = cudaMalloc(&inf->q[l], need);
            if (e == cudaSuccess) e = cudaMalloc(&inf->out[l], need);
            if (e != cudaSuccess) {
                cudaGetLastError();
                return inferFail(inf, PAM_ERR_COMMAND_ENCODING, "Failed to encode Metal command: unable to allocate attention buffers");
            }
            inf->cap[l] = need;
        }
        if (cudaMemsetAsync(inf->q[l], 0, need, c->stream) != cudaSuccess) {
            cudaGetLastError();
            return inferFail(inf, PAM_ERR_COMMAND_EXECUTION, commandExecutionFailed("memset of the query buffer failed"));
        }
    }
    return 0;
}

static void inferForget(Inference* inf, int64_t id) {
    inf->cache->mgr.freeSequence(id);
    inf->prefilled.erase(id);
    inf->prefillProgress.erase(id);
}

// ensureBlocksAvailable (PagedAttentionInference.swift:280-299).  The reference reads the
// free count once per call of handleMemoryPressure while the victims' blocks are only
// freed afterwards, so under pressure every running sequence is paused; with
// incrementalPreemption one victim is paused and freed at a time.
static int32_t inferEnsureBlocks(Inference* inf, int needed) {
    BlockManager& mgr = inf->cache->mgr;
    if (mgr.availableBlocks() >= needed) return 0;
    if (!inf->incrementalPreemption) {
        const int avail = mgr.availableBlocks();
        for (int64_t id : inf->sched->s.handleMemoryPressure(needed, [&]() { return avail; })) inferForget(inf, id);
    } else {
        while (mgr.availableBlocks() < needed) {
            bool first = true;
            std::vector<int64_t> v = inf->sched->s.handleMemoryPressure(needed, [&]() {
                const int a = first ? mgr.availableBlocks() : needed;
                first = false;
                return a;
            });
            if (v.empty()) break;
            for (int64_t id : v) inferForget(inf, id);
        }
    }
    if (mgr.availableBlocks() < needed) return inferKvFail(inf, KVResult{KVStatus::outOfMemory, ""});
    return 0;
}

static void inferComplete(Inference* inf, int64_t id) {     // :108-114
    inf->sched->s.complete(id);
    inferForget(inf, id);
}

// The block bookkeeping of a prompt (:172-186): room for its blocks, a fresh table, the
// prompt's tokens appended.
static int32_t inferReservePrompt(Inference* inf, const pam::SchedulerSequence& seq) {
    Cache* k = inf->cache;
    const int needed = (seq.promptLength + k->blockSize - 1) / k->blockSize;
    if (int32_t rc = inferEnsureBlocks(inf, needed)) return rc;
    KVResult r = k->mgr.allocateSequence(seq.id);
    if (r.status == KVStatus::sequenceAlreadyExists) {
        k->mgr.freeSequence(seq.id);
        r = k->mgr.allocateSequence(seq.id);
    }
    if (!r.ok()) return inferKvFail(inf, r);
    r = k->mgr.appendTokens(seq.id, seq.promptLength, nullptr, 0, nullptr);
    if (!r.ok()) return inferKvFail(inf, r);
    return 0;
}

// With batchedPrefill: the prompts of a step that are not prefilled yet go through the same
// bookkeeping as in the reference, one after the other in batch order (so block tables,
// preemptions and errors are those of the reference), but their attention rows are issued
// together, one launch per layer, instead of one launch set per sequence
// (PagedAttentionInference.swift:172-219).  With a token budget a step takes at most that
// many prompt rows: a long prompt is prefilled in chunks over several steps (rows
// [done, done + n) against keys [0, done + n)), and prompts that do not fit wait.
struct PendingPrefill { pam::SchedulerSequence seq; int start, rows; };

static int32_t inferFlushPrefill(Inference* inf, std::vector<PendingPrefill>& pend) {
    if (pend.empty()) return 0;
    Cache* k = inf->cache;
    const int n = static_cast<int>(pend.size());
    size_t totalRows = 0;
    int maxNumBlocks = 1;
    std::vector<std::vector<int32_t>> rowsOf(static_cast<size_t>(n));
    for (int i = 0; i < n; ++i) {
        KVResult r = k->mgr.blockTable(pend[static_cast<size_t>(i)].seq.id, &rowsOf[static_cast<size_t>(i)]);
        if (!r.ok()) return inferKvFail(inf, r);
        maxNumBlocks = std::max(maxNumBlocks, static_cast<int>(rowsOf[static_cast<size_t>(i)].size()));
        totalRows += static_cast<size_t>(pend[static_cast<size_t>(i)].rows);
    }
    std::vector<int32_t> tables(static_cast<size_t>(n) * maxNumBlocks, 0);
    std::vector<PrefillSeq> seqs;
    for (int i = 0; i < n; ++i) {
        std::copy(rowsOf[static_cast<size_t>(i)].begin(), rowsOf[static_cast<size_t>(i)].end(), tables.begin() + static_cast<std::ptrdiff_t>(i) * maxNumBlocks);
        const PendingPrefill& pp = pend[static_cast<size_t>(i)];
        seqs.push_back(PrefillSeq{pp.start + pp.rows, pp.start, pp.rows});
    }
    if (int32_t rc = inferBuffers(inf, totalRows)) return rc;
    Context* c = inf->c;
    int32_t rc = 0;
    {
        std::lock_guard<std::mutex> g(c->mu);
        DeviceGuard dg(c->device);
        const bool wasAsync = c->async;
        c->async = true;                                   // the layers are enqueued back to back, one wait at the end
        for (size_t l = 0; l < inf->layers.size() && rc == 0; ++l) {
            const size_t bytes = totalRows * ioBytesPerToken(inf->layers[l]);
            rc = prefillImpl(c, inf->layers[l], buf(inf->q[l], bytes), buf(k->kPool, k->poolBytes), buf(k->vPool, k->poolBytes),
                             buf(tables.data(), tables.size() * sizeof(int32_t)), buf(inf->out[l], bytes),
                             buf(k->kScale, k->scaleBytes), buf(k->vScale, k->scaleBytes), seqs, maxNumBlocks, true, "blockTables");
        }
        c->async = wasAsync;
        const int32_t src = syncContext(c);                // `tables` is read by async copies: wait in either mode
        if (rc == 0) rc = src;
        if (rc == 0) c->clearError();
    }
    if (rc != 0) return rc;
    inf->prefillLaunchSets += 1;
    for (const PendingPrefill& pp : pend) {
        const int done = pp.start + pp.rows;
        if (done >= pp.seq.promptLength) {
            inf->prefillProgress.erase(pp.seq.id);
            inf->sched->s.markPrefilled(pp.seq.id);
            inf->prefilled.insert(pp.seq.id);
            inf->totalTokens += pp.seq.promptLength;
        } else {
            inf->prefillProgress[pp.seq.id] = done;
        }
    }
    pend.clear();
    return 0;
}

static int32_t inferPrefillBatched(Inference* inf, const std::vector<pam::SchedulerSequence>& prefill) {
    std::vector<PendingPrefill> pend;
    int budget = inf->prefillTokenBudget > 0 ? inf->prefillTokenBudget : INT_MAX;
    for (const auto& sq : prefill) {
        if (budget <= 0) break;                            // the others wait for the next step
        auto at = inf->prefillProgress.find(sq.id);
        int done = at == inf->prefillProgress.end() ? -1 : at->second;
        if (done < 0) {
            // A reservation that has to pause sequences may take one that this step has already
            // prepared; the reference has by then issued and counted that sequence's prefill
            // (one dispatch per sequence), so what is prepared goes out first.
            const int needed = (sq.promptLength + inf->cache->blockSize - 1) / inf->cache->blockSize;
            if (!pend.empty() && inf->cache->mgr.availableBlocks() < needed)
                if (int32_t rc = inferFlushPrefill(inf, pend)) return rc;
            if (int32_t rc = inferReservePrompt(inf, sq)) {
                // what was prepared before the failing prompt is issued, as the reference
                // would have done by then; the step still fails
                inferFlushPrefill(inf, pend);
                return rc;
            }
            // a preemption inside the reservation may have taken sequences of this step
            pend.erase(std::remove_if(pend.begin(), pend.end(), [&](const PendingPrefill& pp) {
                           int64_t len = 0;
                           return !inf->cache->mgr.sequenceLength(pp.seq.id, &len).ok();
                       }), pend.end());
            done = 0;
        }
        const int rows = std::min(sq.promptLength - done, budget);
        if (sq.promptLength <= 0) {
            // the reference's prefill of an empty prompt fails its validation (seqLen must be positive)
            inferFlushPrefill(inf, pend);
            std::lock_guard<std::mutex> g(inf->c->mu);
            return inf->c->fail(PAM_ERR_INVALID_CONFIGURATION, invalidConfiguration("seqLen must be positive."));
        }
        pend.push_back(PendingPrefill{sq, done, rows});
        inf->prefillProgress[sq.id] = done;
        budget -= rows;
    }
    return inferFlushPrefill(inf, pend);
}

static int32_t inferPrefill(Inference* inf, const pam::SchedulerSequence& seq) {     // :169-220
    Cache* k = inf->cache;
    if (int32_t rc = inferReservePrompt(inf, seq)) return rc;
    KVResult r;
    std::vector<int32_t> table;
    r = k->mgr.blockTable(seq.id, &table);
    if (!r.ok()) return inferKvFail(inf, r);
    if (table.empty()) table.push_back(0);
    if (int32_t rc = inferBuffers(inf, static_cast<size_t>(std::max(seq.promptLength, 0)))) return rc;
    std::vector<PamPrefillRequest> rq(inf->layers.size());
    for (size_t l = 0; l < rq.size(); ++l) {
        const size_t bytes = static_cast<size_t>(std::max(seq.promptLength, 0)) * ioBytesPerToken(inf->layers[l]);
        rq[l] = PamPrefillRequest{};
        rq[l].q = buf(inf->q[l], bytes); rq[l].output = buf(inf->out[l], bytes);
        rq[l].k_pool = buf(k->kPool, k->poolBytes); rq[l].v_pool = buf(k->vPool, k->poolBytes);
        rq[l].block_table = buf(table.data(), table.size() * sizeof(int32_t));
        rq[l].seq_len = seq.promptLength; rq[l].layer = inf->layers[l]; rq[l].causal = 1;
        rq[l].k_scale = buf(k->kScale, k->scaleBytes); rq[l].v_scale = buf(k->vScale, k->scaleBytes);
    }
    if (int32_t rc = pamc_prefill_layers(inf->c, rq.data(), static_cast<int32_t>(rq.size()))) return rc;
    inf->prefillLaunchSets += 1;
    inf->sched->s.markPrefilled(seq.id);
    inf->prefilled.insert(seq.id);
    inf->totalTokens += seq.promptLength;
    return 0;
}

static int32_t inferDecode(Inference* inf, const std::vector<pam::SchedulerSequence>& seqs) {   // :222-278
    Cache* k = inf->cache;
    const int n = static_cast<int>(seqs.size());
    std::vector<int64_t> ids;
    int totalExtras = 0;
    for (auto& sq : seqs) {
        ids.push_back(sq.id);
        int64_t len = 0;
        if (!k->mgr.sequenceLength(sq.id, &len).ok()) len = sq.promptLength;
        const int64_t now = (len + k->blockSize - 1) / k->blockSize, after = (len + 1 + k->blockSize - 1) / k->blockSize;
        totalExtras += static_cast<int>(std::max<int64_t>(0, after - now));
    }
    if (totalExtras > 0)
        if (int32_t rc = inferEnsureBlocks(inf, totalExtras)) return rc;
    // The reference's table rows are maxSequenceBlocks (= maxBlocks) wide (:75, 238); the
    // widest table of the batch gives the same result with a smaller upload.
    int maxNumBlocks = 1;
    std::vector<int32_t> t;
    for (int64_t id : ids) {
        KVResult r = k->mgr.blockTable(id, &t);
        if (!r.ok()) return inferKvFail(inf, r);
        maxNumBlocks = std::max(maxNumBlocks, static_cast<int>(t.size()));
    }
    std::vector<int32_t> tables;
    std::vector<uint32_t> lens;
    {
        std::lock_guard<std::mutex> g(inf->c->mu);
        if (buildBatchTables(inf->c, k, ids.data(), n, maxNumBlocks, &tables, &lens, nullptr) != 0) return -1;
    }
    if (int32_t rc = inferBuffers(inf, static_cast<size_t>(n))) return rc;
    std::vector<PamDecodeRequest> rq(inf->layers.size());
    for (size_t l = 0; l < rq.size(); ++l) {
        const size_t bytes = static_cast<size_t>(n) * ioBytesPerToken(inf->layers[l]);
        rq[l] = PamDecodeRequest{};
        rq[l].q = buf(inf->q[l], bytes); rq[l].output = buf(inf->out[l], bytes);
        rq[l].k_pool = buf(k->kPool, k->poolBytes); rq[l].v_pool = buf(k->vPool, k->poolBytes);
        rq[l].block_tables = buf(tables.data(), tables.size() * sizeof(int32_t));
        rq[l].seq_lengths = buf(lens.data(), lens.size() * sizeof(uint32_t));
        rq[l].batch_size = n; rq[l].max_num_blocks = maxNumBlocks; rq[l].layer = inf->layers[l];
        rq[l].k_scale = buf(k->kScale, k->scaleBytes); rq[l].v_scale = buf(k->vScale, k->scaleBytes);
    }
    if (int32_t rc = pamc_decode_layers(inf->c, rq.data(), static_cast<int32_t>(rq.size()))) return rc;
    for (auto& sq : seqs) {
        KVResult r = k->mgr.appendTokens(sq.id, 1, nullptr, 0, nullptr);
        if (!r.ok()) return inferKvFail(inf, r);
        inf->sched->s.markDecoded(sq.id);
        inf->totalTokens += 1;
        if (inf->onToken) inf->onToken(inf->onTokenUser, sq.id, 0);
        pam::SchedulerSequence now;
        if (inf->sched->s.get(sq.id, &now) && now.isDone()) inferComplete(inf, sq.id);
    }
    return 0;
}

static int32_t inferStep(Inference* inf, std::vector<int64_t>* batch) {      // :119-148
    *batch = inf->sched->s.step();
    if (batch->empty()) return 0;
    std::vector<pam::SchedulerSequence> prefill, decode;
    for (int64_t id : *batch) {
        pam::SchedulerSequence sq;
        if (!inf->sched->s.get(id, &sq)) continue;
        (inf->prefilled.count(id) ? decode : prefill).push_back(sq);
    }
    if (inf->batchedPrefill) {
        if (!prefill.empty())
            if (int32_t rc = inferPrefillBatched(inf, prefill)) return rc;
    } else {
        for (auto& sq : prefill)
            if (int32_t rc = inferPrefill(inf, sq)) return rc;
    }
    if (!decode.empty())
        if (int32_t rc = inferDecode(inf, decode)) return rc;
    inf->stepCount += 1;
    return 0;
}

void* pamc_infer_create(void* ctx, int32_t max_blocks, int32_t block_size, const PamLayerSpec* layers, int32_t num_layers,
                        int32_t max_batch_size, int32_t max_sequences) {
    if (!ctx) return nullptr;
    Context* c = asCtx(ctx);
    if (!layers || num_layers <= 0) {                              // :55-57
        std::lock_guard<std::mutex> g(c->mu);
        c->fail(PAM_ERR_INVALID_CONFIGURATION, invalidConfiguration("at least one layer spec required"));
        return nullptr;
    }
    // pools are shaped by the first layer (:59-62, 76-85)
    void* cache = pam_create_cache(ctx, max_blocks, block_size, layers[0].head_dim, layers[0].num_kv_heads, layers[0].data_type);
    if (!cache) return nullptr;
    Inference* inf = new Inference();
    inf->c = c;
    inf->cache = asCache(cache);
    inf->sched = new Sched(max_batch_size, max_sequences);
    inf->layers.assign(layers, layers + num_layers);
    inf->maxBatch = max_batch_size;
    inf->q.assign(static_cast<size_t>(num_layers), nullptr);
    inf->out.assign(static_cast<size_t>(num_layers), nullptr);
    inf->cap.assign(static_cast<size_t>(num_layers), 0);
    return inf;
}
void pamc_infer_destroy(void* infer) { delete static_cast<Inference*>(infer); }
void* pamc_infer_cache(void* infer) { return infer ? static_cast<Inference*>(infer)->cache : nullptr; }
void* pamc_infer_scheduler(void* infer) { return infer ? static_cast<Inference*>(infer)->sched : nullptr; }
int64_t pamc_infer_add_request(void* infer, int32_t prompt_token_count, int32_t max_new_tokens) {     // :103-105
    return infer ? static_cast<Inference*>(infer)->sched->s.addRequest(prompt_token_count, max_new_tokens) : -1;
}
void pamc_infer_complete_sequence(void* infer, int64_t id) {
    if (!infer) return;
    Inference* inf = static_cast<Inference*>(infer);
    std::lock_guard<std::mutex> g(inf->mu);
    inferComplete(inf, id);
}
int32_t pamc_infer_step(void* infer, int64_t* out_ids, int32_t capacity) {
    if (!infer) return -1;
    Inference* inf = static_cast<Inference*>(infer);
    std::lock_guard<std::mutex> g(inf->mu);
    std::vector<int64_t> batch;
    if (inferStep(inf, &batch) != 0) return -1;
    for (int i = 0; out_ids && i < capacity && i < static_cast<int>(batch.size()); ++i) out_ids[i] = batch[static_cast<size_t>(i)];
    return static_cast<int32_t>(batch.size());
}
int32_t pamc_infer_run_all(void* infer) {                          // :151-156
    if (!infer) return -1;
    Inference* inf = static_cast<Inference*>(infer);
    std::lock_guard<std::mutex> g(inf->mu);
    while (inf->sched->s.count(pam::waiting) > 0 || inf->sched->s.count(pam::running) > 0) {
        std::vector<int64_t> batch;
        if (inferStep(inf, &batch) != 0) return -1;
        if (batch.empty()) break;
    }
    return 0;
}
int64_t pamc_infer_total_tokens(void* infer) {
    if (!infer) return -1;
    Inference* inf = static_cast<Inference*>(infer);
    std::lock_guard<std::mutex> g(inf->mu);
    return inf->totalTokens;
}
int32_t pamc_infer_step_count(void* infer) {
    if (!infer) return -1;
    Inference* inf = static_cast<Inference*>(infer);
    std::lock_guard<std::mutex> g(inf->mu);
    return inf->stepCount;
}
void pamc_infer_set_token_callback(void* infer, pamc_token_fn fn, void* user) {
    if (!infer) return;
    Inference* inf = static_cast<Inference*>(infer);
    std::lock_guard<std::mutex> g(inf->mu);
    inf->onToken = fn; inf->onTokenUser = user;
}
void pamc_infer_set_batched_prefill(void* infer, int32_t on, int32_t token_budget) {
    if (!infer) return;
    Inference* inf = static_cast<Inference*>(infer);
    std::lock_guard<std::mutex> g(inf->mu);
    inf->batchedPrefill = on != 0;
    inf->prefillTokenBudget = std::max(token_budget, 0);
}
int64_t pamc_infer_prefill_launch_sets(void* infer) {
    if (!infer) return -1;
    Inference* inf = static_cast<Inference*>(infer);
    std::lock_guard<std::mutex> g(inf->mu);
    return inf->prefillLaunchSets;
}
void pamc_infer_set_incremental_preemption(void* infer, int32_t on) {
    if (!infer) return;
    Inference* inf = static_cast<Inference*>(infer);
    std::lock_guard<std::mutex> g(inf->mu);
    inf->incrementalPreemption = on != 0;
}

}  // extern "C"
