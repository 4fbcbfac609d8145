// Launchers of the CUDA kernels (sm_100a).  All pointers are device pointers;
// every launcher enqueues on `stream` and returns the launch status without
// synchronising.
#pragma once

#include <cuda_runtime.h>

#include <cstddef>
#include <cstdint>
#include <string>

namespace pam {

enum DType { kF32 = 0, kF16 = 1, kFP8 = 2, kBF16 = 3 };

inline int elemBytes(int dtype) { return dtype == kF32 ? 4 : dtype == kFP8 ? 1 : 2; }
// Type of queries, new K/V rows and outputs for a cache of type `dtype`.
inline int ioBytes(int dtype) { return dtype == kF32 ? 4 : 2; }

// Where the slot of token t comes from: an explicit list, or one block table
// with a token offset (slot = table[(off+t)/bs]*bs + (off+t)%bs).
struct SlotSource {
    const int64_t* slots = nullptr;
    const int32_t* table = nullptr;
    int tokenOffset = 0;
    int64_t numSlots = 0;   // slots of the pool; tokens whose slot lies outside are skipped
};

// ---- KV append and block copies (cache_kernels.cu) ----
cudaError_t launchReshapeAndCache(const void* keys, const void* values, void* kPool, void* vPool,
                                  SlotSource src, int numTokens, int kvHeads, int blockSize,
                                  int headDim, int elemBytes, cudaStream_t stream, int* launches);
// amaxScratch: [blocks][kvHeads][2] 64-bit words, zero when first used; epoch
// must grow by one per call on the same scratch.
cudaError_t launchReshapeAndCacheFp8(const void* keysF16, const void* valuesF16, void* kCodes,
                                     void* vCodes, void* kScale, void* vScale, SlotSource src,
                                     int numTokens, int kvHeads, int blockSize, int headDim,
                                     unsigned long long* amaxScratch, uint32_t epoch,
                                     cudaStream_t stream, int* launches);
// pairs: [n][2] (src block, dst block).  scale pointers may be null.
cudaError_t launchCopyBlocks(void* kPool, void* vPool, void* kScale, void* vScale,
                             const int32_t* pairs, int n, size_t blockBytes, int kvHeads,
                             cudaStream_t stream, int* launches);

// patches: [n][3] (row, column, block) written into tables[row * stride + column]: the
// entries of a resident batch of block tables that changed since it was uploaded.
cudaError_t launchPatchTables(int32_t* tables, int stride, const int32_t* patches, int n, cudaStream_t stream,
                              int* launches);

// ---- decode (decode_kernels.cu) ----
struct DecodeParams {
    const void* q;            // [batch][heads][dim], io type
    const void* kPool;        // [block][kvHeads][blockSize][dim], storage type
    const void* vPool;
    const int32_t* tables;    // [batch][maxNumBlocks]
    const uint32_t* lens;     // [batch]
    void* out;                // [batch][heads][dim], io type
    const void* kScale;       // FP8: [block][kvHeads] float16
    const void* vScale;
    int batch, heads, kvHeads, headDim, blockSize, maxNumBlocks, window, dtype;
    int poolBlocks;           // blocks in the pools; table entries are clamped into [0, poolBlocks)
    float* workspace;         // partial results of the stream kernel, decodeWorkspaceBytes() bytes
    size_t workspaceBytes;
    // Counting words of the stream kernel: device ints, all zero between launches, one per
    // (sequence, kv head) pair, kept by the caller and written by nothing else.
    int* counters;
    int64_t countersCap;
};
// True when `p` runs on the stream kernel (type, shape and pointer alignment allow it).
bool decodeTakesStreamPath(const DecodeParams& p);
// Bytes of workspace the launch of `p` needs (0 for the general kernel).
size_t decodeWorkspaceBytes(const DecodeParams& p, int smCount);
cudaError_t launchDecode(const DecodeParams& p, int smCount, cudaStream_t stream, int* launches);
// The persistent stream kernel (decode_stream_kernel.cu): float16 / bfloat16 / FP8 pools,
// head_dim 128 (64 for 16-bit pools), block size a multiple of 16, at most 16 query heads
// per KV head, aligned pointers.  It needs `workspace` (decodeStreamWorkspaceBytes; with less
// it launches fewer warps) and `counters` (batch * kvHeads words).  Batches beyond
// kDecodeStreamMaxBatch run as several launches.
constexpr int kDecodeStreamMaxBatch = 2048;
bool decodeStreamApplies(const DecodeParams& p);
int decodeStreamWarps(const DecodeParams& p, int smCount);
size_t decodeStreamWorkspaceBytes(const DecodeParams& p, int smCount);
cudaError_t launchDecodeStream(const DecodeParams& p, int smCount, cudaStream_t stream, int* launches);
// Device addresses of the fixed arrays inside the library image (workspace, counting words).
cudaError_t decodeStaticScratch(float** scratch, int** counters, int64_t* countersCap);

// Same decode with the workspace and the counting words taken from fixed arrays inside the
// library (decodeStaticScratchBytes() bytes and 65 536 words per GPU) instead of
// p.workspace and p.counters.  Allocates nothing; fails with cudaErrorInvalidValue when the
// batch has more pairs than words or the array cannot hold one record per pair and a CTA's
// worth of warps.  The current device must be the one the pointers in `p` live on.
size_t decodeStaticScratchBytes();
cudaError_t launchDecodeStatic(const DecodeParams& p, int smCount, cudaStream_t stream, int* launches);

// ---- backward (backward_kernels.cu) ----
struct BackwardParams {
    const void* q;            // [seqLen][heads][dim], io type
    const void* kPool;        // [block][kvHeads][blockSize][dim], io type (float32 / float16 / bfloat16)
    const void* vPool;
    const int32_t* table;     // [maxNumBlocks]
    const void* dO;           // [seqLen][heads][dim]
    const float* m;           // [seqLen][heads]: row maximum of the forward pass
    const float* l;           // [seqLen][heads]: row sum of exp(s - m)
    void* dQ;                 // [seqLen][heads][dim], io type (written)
    void* dKPool;             // like kPool (added to)
    void* dVPool;
    float* dQAcc;             // float32 [seqLen][heads][dim]: dQ itself for float32, else workspace
    float* rowSum;            // float32 [seqLen][heads] workspace
    int seqLen, heads, kvHeads, headDim, blockSize, windowStart, dtype;
    int poolBlocks;           // blocks in the pools; table entries are clamped into [0, poolBlocks)
    int maxNumBlocks;         // entries of the table
};
// Bytes of workspace (rowSum first, 256-byte aligned, then dQAcc for the 16-bit types).
size_t backwardWorkspaceBytes(const BackwardParams& p);
cudaError_t launchBackward(const BackwardParams& p, cudaStream_t stream, int* launches);
// The tensor-core form (backward_mma_kernels.cu): float16 / bfloat16, head_dim 64 or 128,
// 16-byte aligned buffers; launchBackward takes it when it applies.
bool backwardTensorPathApplies(const BackwardParams& p);
cudaError_t launchBackwardTensor(const BackwardParams& p, cudaStream_t stream, int* launches);

// ---- prefill (prefill_kernels.cu) ----
constexpr int kPrefillInlineSeqs = 32;
struct PrefillParams {
    const void* q;            // rows of all sequences back to back, [rows][heads][dim]
    const void* kPool;
    const void* vPool;
    const int32_t* tables;    // [numSeqs][maxNumBlocks]
    void* out;
    const void* kScale;
    const void* vScale;
    // per sequence (device arrays, numSeqs entries)
    const int32_t* seqLens;       // tokens in the cache
    const int32_t* qStarts;       // first row of this launch within the sequence
    const int32_t* qLens;         // rows of this launch
    const int32_t* qRowOffsets;   // first row of the sequence within q/out
    const int32_t* windowStarts;  // first visible key
    int numSeqs, maxQLen, heads, kvHeads, headDim, blockSize, maxNumBlocks, causal, dtype;
    int poolBlocks;               // table entries are clamped into [0, poolBlocks)
    int totalRows;                // rows in q/out (all sequences of the launch)
    int* errFlag;                 // device word the tensor-core kernel sets when a bounded wait runs out
    int forceGeneral;             // 1: never take the tensor-core path
    // Up to kPrefillInlineSeqs sequences travel inside the kernel parameters
    // (no upload before the launch): rows seqLens, qStarts, qLens, qRowOffsets,
    // windowStarts; the pointers above are then unused.
    int inlineMeta;
    int32_t meta[5][kPrefillInlineSeqs];
    int exactWeights;             // bfloat16 tensor path: 0 = 8-bit weights, 1 = 16-bit on short rows, 2 = 16-bit always
    long long waitCycles;         // tensor path: bound of every wait on a barrier in SM cycles; 0 = the default (about 0.2 s)
    int starveV;                  // tensor path, test launches: the CTA's first value tile is not fetched (its wait runs out)
    // Filled by the tensor-core launcher: reciprocals for the work-item arithmetic (an item
    // index is split by numSeqs * heads, heads and heads / kvHeads; valid while the item
    // count stays below 2^22, else fastItems is 0 and the kernel divides).
    int fastItems;
    int pairHeads;   // set by launchPrefillTensor: the two row groups of a CTA take two heads of one KV head
    float invPer, invHeads, invGroup;
};
// Tensor-core path (prefill_tc_kernel.cu): bf16/f16, head_dim 128, block size multiple of 16.
bool prefillTensorPathApplies(const PrefillParams& p);
cudaError_t launchPrefillTensor(const PrefillParams& p, int totalRows, int* errFlag, cudaStream_t stream, int* launches);
#ifdef __CUDACC__
// Per-sequence fields, from the inline table or from the device arrays.
__device__ __forceinline__ int prefillMeta(const PrefillParams& p, int which, int seq) {
    if (p.inlineMeta) return p.meta[which][seq];
    const int32_t* const ptr = which == 0 ? p.seqLens : which == 1 ? p.qStarts : which == 2 ? p.qLens
                               : which == 3 ? p.qRowOffsets : p.windowStarts;
    return ptr[seq];
}
#endif
cudaError_t launchPrefill(const PrefillParams& p, int smCount, cudaStream_t stream, int* launches,
                          bool* usedTensorPath);
// FP8 KV on the tensor-core prefill path: the pages the launch can see (blocks
// windowStart / blockSize .. ceil(seqLen / blockSize) of every sequence, at most
// `maxCount` each) are dequantised to float16 with the reference's all-half chain
// (kernels.metal:553-562) into scratch pools of numSeqs * maxCount blocks, and
// `stagedTables` ([numSeqs][maxNumBlocks], zeroed by the caller) gets the scratch block
// of every such table entry.  `meta` holds seqLens and windowStarts (numSeqs each).
bool prefillFp8StagingApplies(const PrefillParams& p);
cudaError_t launchFp8StagePages(const PrefillParams& p, const int32_t* seqLens, const int32_t* windowStarts, int maxCount,
                                void* kOut, void* vOut, int32_t* stagedTables, cudaStream_t stream, int* launches);

// ---- all-gather of head-sharded outputs (comm.cu) ----
// local: [rows][slice] on this GPU (slice = heads/N * dim * element bytes, a multiple of 16);
// staging: N * rows * slice bytes of scratch; full: [rows][N][slice] on every GPU.
struct HeadComm;
bool commAvailable();
int commUniqueId(void* out128);
HeadComm* commCreate(const void* id128, int rank, int size, int device, std::string* error);
void commDestroy(HeadComm* comm);
int commRank(const HeadComm* comm);
int commSize(const HeadComm* comm);
cudaError_t launchAllGatherHeads(HeadComm* comm, const void* local, void* staging, void* full, int rows, size_t sliceBytes,
                                 cudaStream_t stream, int* launches, std::string* error);

}  // namespace pam
