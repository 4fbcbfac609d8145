/*
 * pam_cuda.h -- C ABI of the B200 (sm_100a) paged-KV attention library.
 *
 * Two groups of entry points:
 *
 *  pam_*   The C ABI the reference project exports from Swift
 *          (Sources/PagedAttentionMetal/PagedAttentionCABI.swift:71-337), with
 *          identical names, argument order, argument types and return
 *          conventions.  Where the reference takes an MTLBuffer object pointer,
 *          this library takes a raw pointer to the same bytes: either CUDA
 *          device memory, or host memory (the reference's buffers are host
 *          visible, CABI.swift:58-62); host pointers are staged through the
 *          context's device arena inside the call.
 *
 *  pamc_*  What the Swift classes PagedAttentionEngine, KVCacheManager,
 *          BatchKVCacheManager and ContinuousBatchingScheduler need beyond
 *          that, one function per public method; each cites the method it
 *          backs.
 *
 * Conventions (CABI.swift:18-37): int32 results are 0 on success and -1 on
 * failure, with a message kept in the context and returned by
 * pam_last_error() until the next call on that context; creators return NULL
 * on failure.  Handles are opaque; every handle is safe to use from several
 * threads (calls on one handle serialise).  Unless pamc_set_async() is on,
 * every operation has completed on the GPU when its call returns
 * (PagedAttentionEngine.swift:2008-2015).
 *
 * KV pools are [block][kv_head][block_size][head_dim] in HBM; FP8 pools carry
 * float16 scales [block][kv_head].  Element types: see PAM_DTYPE_*.
 */
#ifndef PAM_CUDA_H
#define PAM_CUDA_H

#include <stdbool.h>
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* PagedAttentionDataType (PagedAttentionTypes.swift:67-74); 3 is an addition. */
enum {
    PAM_DTYPE_F32 = 0,
    PAM_DTYPE_F16 = 1,
    PAM_DTYPE_FP8 = 2, /* e4m3 codes; queries, new K/V and outputs are float16 */
    PAM_DTYPE_BF16 = 3
};

/* Error classes: PagedAttentionError (PagedAttentionTypes.swift:5-31) and
 * KVCacheError (KVCacheManager.swift:6-11). */
enum {
    PAM_OK = 0,
    PAM_ERR_DEVICE_INIT = 1,
    PAM_ERR_INVALID_CONFIGURATION = 4,
    PAM_ERR_BUFFER_TOO_SMALL = 5,
    PAM_ERR_COMMAND_ENCODING = 6,
    PAM_ERR_COMMAND_EXECUTION = 7,
    PAM_ERR_UNSUPPORTED = 8,
    PAM_ERR_RESOURCE_EXHAUSTED = 10,
    PAM_ERR_INVALID_STATE = 12,
    PAM_ERR_RECURRING = 13,
    PAM_ERR_KV_OUT_OF_MEMORY = 20,
    PAM_ERR_KV_SEQUENCE_NOT_FOUND = 21,
    PAM_ERR_KV_SEQUENCE_EXISTS = 22,
    PAM_ERR_KV_INVALID_REQUEST = 23,
    PAM_ERR_NULL_HANDLE = 30
};

/* BlockEvictionPolicy (KVCacheManager.swift:13-17). */
enum { PAM_POLICY_FIFO = 0, PAM_POLICY_LIFO = 1, PAM_POLICY_BEST_FIT = 2 };

/* SequenceStatus (Scheduler.swift:5-10). */
enum { PAM_SEQ_WAITING = 0, PAM_SEQ_RUNNING = 1, PAM_SEQ_PAUSED = 2, PAM_SEQ_COMPLETED = 3 };

/* PagedAttentionStats.Operation (PagedAttentionTypes.swift:171-180).  The four
 * prefill values name reference kernel variants; this library reports
 * PAM_OP_PREFILL_MMA for its tensor-core prefill kernel and
 * PAM_OP_PREFILL_TILED for the general one. */
enum {
    PAM_OP_NONE = 0,
    PAM_OP_PREFILL_SINGLE_PASS = 1,
    PAM_OP_PREFILL_MMA = 2,
    PAM_OP_PREFILL_FLASH = 3,
    PAM_OP_PREFILL_TILED = 4,
    PAM_OP_DECODE = 5,
    PAM_OP_APPEND = 6,
    PAM_OP_BACKWARD = 7
};

/* ------------------------------------------------------------------------
 * Reference C ABI (PagedAttentionCABI.swift)
 * ---------------------------------------------------------------------- */

/* CABI.swift:71-79.  Uses the current CUDA device. */
void *pam_create_context(void);
/* CABI.swift:81-85 */
void pam_destroy_context(void *ctx);
/* CABI.swift:87-90 */
const char *pam_last_error(void *ctx);
/* CABI.swift:92-132.  data_type: PAM_DTYPE_*; unknown values fail. */
void *pam_create_cache(void *ctx, int32_t max_blocks, int32_t block_size, int32_t head_dim,
                       int32_t num_kv_heads, int32_t data_type);
/* CABI.swift:134-138 */
void pam_destroy_cache(void *cache);
/* CABI.swift:140-154 -> KVCacheManager.allocateSequence (KVCacheManager.swift:106-113) */
int32_t pam_reserve_sequence(void *ctx, void *cache, int64_t sequence_id);
/* CABI.swift:156-171 -> KVCacheManager.appendTokens without hashes (KVCacheManager.swift:115-174) */
int32_t pam_append_tokens(void *ctx, void *cache, int64_t sequence_id, int32_t count);
/* CABI.swift:173-179 -> KVCacheManager.freeSequence (KVCacheManager.swift:216-239) */
void pam_free_sequence(void *cache, int64_t sequence_id);
/* CABI.swift:181-185; -1 for a NULL cache */
int32_t pam_available_blocks(void *cache);
/* CABI.swift:187-201 */
int32_t pam_sequence_length(void *ctx, void *cache, int64_t sequence_id);
/* CABI.swift:203-244 -> PagedAttentionEngine.appendToCache (PagedAttentionEngine.swift:585-628).
 * keys/values: [num_new_tokens][num_kv_heads][head_dim] in the cache's type
 * (float16 for an FP8 cache). */
int32_t pam_append_kv(void *ctx, void *cache, int64_t sequence_id, void *keys, void *values,
                      int32_t token_offset, int32_t num_new_tokens, int32_t num_heads);
/* CABI.swift:246-287 -> PagedAttentionEngine.prefill (PagedAttentionEngine.swift:405-418).
 * q/out: [seq_len][num_heads][head_dim]. */
int32_t pam_prefill(void *ctx, void *cache, int64_t sequence_id, void *q, void *out,
                    int32_t seq_len, int32_t num_heads, bool causal);
/* CABI.swift:289-337 -> PagedAttentionEngine.decode (PagedAttentionEngine.swift:533-546).
 * q/out: [batch][num_heads][head_dim]. */
int32_t pam_decode(void *ctx, void *cache, const int64_t *batch_ids, int32_t batch_size, void *q,
                   void *out, int32_t num_heads);

/* ------------------------------------------------------------------------
 * Context / engine (PagedAttentionEngine.swift)
 * ---------------------------------------------------------------------- */

/* Number of CUDA devices; 0 when there is none (never fails). */
int32_t pamc_device_count(void);
/* PagedAttentionEngine.init (PagedAttentionEngine.swift:248-333) on a chosen device. */
void *pamc_create_context_on(int32_t device);
/* A context without a device: it carries the last error for calls on
 * bookkeeping-only managers (pamc_cache_create_bookkeeping) and needs no GPU.
 * Every operation that would launch a kernel fails on it. */
void *pamc_create_host_context(void);
/* Class of the last error on this context (PAM_ERR_*), PAM_OK if none. */
int32_t pamc_last_error_code(void *ctx);
/* Run on a caller-owned CUDA stream (a cudaStream_t); NULL restores the
 * context's own stream. */
int32_t pamc_set_stream(void *ctx, void *cuda_stream);
/* 1: operations return after enqueueing; 0 (default): they wait for the GPU
 * like the reference's commitAndWait (PagedAttentionEngine.swift:2008-2015). */
int32_t pamc_set_async(void *ctx, int32_t enabled);
/* Wait for everything enqueued on the context's stream. */
int32_t pamc_synchronize(void *ctx);
/* Engine properties (PagedAttentionEngine.swift:116-129). */
int32_t pamc_set_max_retries(void *ctx, int32_t n);            /* maxRetries, default 3 */
int32_t pamc_set_graceful_degradation(void *ctx, int32_t on);  /* enableGracefulDegradation, default 1 */
int32_t pamc_set_split_threshold(void *ctx, int32_t tokens);   /* splitThreshold, default 1024 */
int32_t pamc_set_default_window(void *ctx, int32_t tokens);    /* defaultWindowSize, default 0 */
int32_t pamc_set_default_chunk(void *ctx, int32_t tokens);     /* defaultChunkSize, default 0 */
/* 1 (default): prefill takes the tensor-core kernel where it applies (bf16/f16,
 * head_dim 128, block size a multiple of 16); 0: always the general kernel.
 * The reference picks its prefill variant the same way, by type and head_dim
 * (PagedAttentionEngine.swift:420-434). */
int32_t pamc_set_prefill_tensor_path(void *ctx, int32_t on);
/* bfloat16 tensor-core prefill: how the softmax weights are carried into the
 * second product.  0: one bfloat16 operand (8 significant bits, what bfloat16
 * attention kernels usually do); 1 (default): two operands, 16 bits, on query
 * tiles whose rows see fewer than 256 keys, where 8 bits can miss the 2e-3
 * bound; 2: two operands everywhere (about 1.5x the tensor work).  No
 * counterpart in the reference, which has no bfloat16. */
int32_t pamc_set_prefill_exact_weights(void *ctx, int32_t mode);
/* Host-side fault injection for tests of the retry loop, circuit breaker and
 * zero-fill path (PagedAttentionEngine.swift:375-414): the next n kernel
 * launches of this context report failure without touching the GPU. */
int32_t pamc_inject_launch_failures(void *ctx, int32_t n);
/* Number of this library's kernels launched on the context since creation. */
int64_t pamc_kernel_launches(void *ctx);
/* Every wait inside the tensor-core prefill kernel is bounded; a wait that runs out makes
 * the kernel return early and the call fail with "a kernel's bounded wait ran out (site n)"
 * (retried and degraded like any failed launch, PagedAttentionEngine.swift:375-414).
 * sm_cycles is that bound in SM clock cycles; 0 restores the default (about 0.2 s). */
int32_t pamc_set_wait_limit(void *ctx, int64_t sm_cycles);
/* Test switch for that path: in each of the next `launches` tensor-core prefill launches
 * no CTA fetches its first value tile, so the wait for it runs out after the wait limit and
 * the kernel returns through its error exit.  Nothing spins or faults; set a short limit
 * first.  The host-side counterpart of pamc_inject_launch_failures. */
int32_t pamc_test_starve_prefill(void *ctx, int32_t launches);

/* PagedAttentionStats (PagedAttentionTypes.swift:169-207). */
typedef struct PamStats {
    int32_t operation; /* PAM_OP_* */
    int32_t batch_size;
    int32_t sequence_length;
    int32_t num_blocks;
    int64_t temporary_bytes;
    int32_t used_split_pass;
    double elapsed_ms;
} PamStats;
/* PagedAttentionEngine.lastStats (PagedAttentionEngine.swift:137-141). */
int32_t pamc_last_stats(void *ctx, PamStats *out);

/* recommendedMaxBlocks (PagedAttentionEngine.swift:201-217) with free device
 * memory in place of recommendedMaxWorkingSetSize. */
int64_t pamc_recommended_max_blocks(void *ctx, int32_t block_size, int32_t num_kv_heads,
                                    int32_t head_dim, int32_t data_type, float memory_fraction,
                                    int32_t layer_count);

/* Plain device memory for callers without a CUDA runtime of their own (the
 * Swift veneer's PagedBuffer).  kind: 0 host->device, 1 device->host,
 * 2 device->device; copies are ordered on the context's stream and complete
 * on return. */
void *pamc_buffer_alloc(void *ctx, size_t bytes);
void pamc_buffer_free(void *ctx, void *ptr);
int32_t pamc_memcpy(void *ctx, void *dst, const void *src, size_t bytes, int32_t kind);

/* ------------------------------------------------------------------------
 * KV cache manager (KVCacheManager.swift)
 * ---------------------------------------------------------------------- */

/* A manager that keeps block tables, reference counts and the prefix cache
 * but owns no pools (max_blocks, block_size only).  Multi-GPU callers take
 * allocation decisions once on such a handle and replay them on each GPU;
 * it needs no CUDA device. */
void *pamc_cache_create_bookkeeping(int32_t max_blocks, int32_t block_size);

/* KVCacheManager.appendTokens(toSequence:count:blockHashes:) (KVCacheManager.swift:115-174).
 * hashes[i] belongs to the i-th block newly added by this call; a shared
 * partial last block is copied on the GPU (K, V and FP8 scales) before the
 * call returns (KVCacheManager.swift:134-140, 176-194). */
int32_t pamc_cache_append_tokens(void *ctx, void *cache, int64_t sequence_id, int32_t count,
                                 const uint64_t *hashes, int32_t num_hashes);
/* KVCacheManager.ensureExclusiveAccess (KVCacheManager.swift:200-214) */
int32_t pamc_cache_ensure_exclusive(void *ctx, void *cache, int64_t sequence_id,
                                    int32_t logical_block);
/* KVCacheManager.registerBlockHash (KVCacheManager.swift:196-198) */
void pamc_cache_register_block_hash(void *cache, uint64_t hash, int32_t physical_block);
/* KVCacheManager.getBlockTable (KVCacheManager.swift:299-303): copies up to
 * capacity entries to out (host memory), returns the table length or -1. */
int32_t pamc_cache_block_table(void *ctx, void *cache, int64_t sequence_id, int32_t *out,
                               int32_t capacity);
/* KVCacheManager.getNumBlocks (KVCacheManager.swift:335-339) */
int32_t pamc_cache_num_blocks(void *ctx, void *cache, int64_t sequence_id);
/* KVCacheManager.activeSequenceCount (KVCacheManager.swift:347-351) */
int32_t pamc_cache_active_sequences(void *cache);
/* KVCacheManager.evictionPolicy didSet (KVCacheManager.swift:65-67, 267-283) */
int32_t pamc_cache_set_eviction_policy(void *cache, int32_t policy);

/* Two fixes of reference behaviour for servers, off by default so that block tables, free
 * counts and hit counts stay bit-exact with the reference.  on != 0:
 *  - a prefix-cache hash is forgotten when its block's reference count reaches zero (the
 *    reference keeps it, KVCacheManager.swift:216-239, and a later appendTokens with that
 *    hash is handed a block that meanwhile holds other tokens, :150-158);
 *  - an appendTokens that runs out of blocks changes nothing (the reference has by then
 *    copied a shared last block, :134-146, leaking the fresh block and dropping a
 *    reference the sequence still uses). */
int32_t pamc_cache_set_hygiene(void *cache, int32_t on);
/* Content hashes for appendTokens' blockHashes (the reference takes caller-supplied
 * UInt64s, KVCacheManager.swift:115): hash j covers the token ids of blocks 0..j (64-bit
 * FNV-1a, chained), so equal hashes mean equal prefixes.  Writes up to capacity hashes of
 * the num_tokens / block_size full blocks to out (may be NULL) and returns their number. */
int32_t pamc_block_hashes(const int32_t *token_ids, int32_t num_tokens, int32_t block_size, uint64_t seed,
                          uint64_t *out, int32_t capacity);

/* KVCacheMemoryStats (KVCacheManager.swift:19-32). */
typedef struct PamMemoryStats {
    int64_t total_blocks, used_blocks, free_blocks, active_sequences;
    int64_t total_memory_bytes, used_memory_bytes;
    int64_t partially_filled_blocks;
    float fragmentation_ratio;
    int64_t prefix_cache_hits, prefix_cache_entries, shared_blocks;
    int32_t eviction_policy;
} PamMemoryStats;
/* KVCacheManager.memoryStats (KVCacheManager.swift:353-378) */
int32_t pamc_cache_memory_stats(void *cache, PamMemoryStats *out);

/* kPoolBuffer / vPoolBuffer (KVCacheManager.swift:59-60) plus the FP8 scale
 * arrays; device pointers, any out argument may be NULL. */
int32_t pamc_cache_pools(void *cache, void **k_pool, void **v_pool, void **k_scale, void **v_scale,
                         size_t *pool_bytes, size_t *scale_bytes);
/* Copy-on-write pairs (src block, dst block) recorded since the last call, in
 * order; returns how many were written to out (host, capacity pairs). */
int32_t pamc_cache_drain_cow_log(void *cache, int32_t *out_pairs, int32_t capacity);

/* BatchKVCacheManager.getBatchBlockTableBuffer / getSeqLengthsBuffer
 * (KVCacheManager.swift:661-703) and the C ABI's BatchKVCacheView
 * (CABI.swift:339-372): rows zero-padded to max_num_blocks.  tables
 * [n][max_num_blocks] int32 and lens [n] uint32 may be device or host memory. */
int32_t pamc_cache_batch_tables(void *ctx, void *cache, const int64_t *ids, int32_t n,
                                int32_t max_num_blocks, int32_t *tables, uint32_t *lens);
/* Slot of each token of a sequence (kernels.metal:1823-1827):
 * table[(off+t)/bs]*bs + (off+t)%bs, written to out (host). */
int32_t pamc_cache_slot_mapping(void *ctx, void *cache, int64_t sequence_id, int32_t token_offset,
                                int32_t num_tokens, int64_t *out);

/* ------------------------------------------------------------------------
 * Operations (PagedAttentionEngine.swift), flat form
 * ---------------------------------------------------------------------- */

/* A buffer argument with its length, for the reference's bufferTooSmall checks
 * (PagedAttentionEngine.swift:1994-1998).  ptr may be device or host memory. */
typedef struct PamBuffer {
    void *ptr;
    size_t bytes;
} PamBuffer;

/* PagedLayerSpec (PagedAttentionTypes.swift:94-152). */
typedef struct PamLayerSpec {
    int32_t head_dim, num_heads, num_kv_heads, block_size, data_type, window_size;
} PamLayerSpec;

/* PagedKVAppendRequest (PagedAttentionTypes.swift:318-364). */
typedef struct PamAppendRequest {
    PamBuffer keys, values, k_pool, v_pool, block_table;
    int32_t token_offset, num_new_tokens;
    PamLayerSpec layer;
    PamBuffer k_scale, v_scale; /* FP8 only: [block][kv_head] float16 */
} PamAppendRequest;
/* PagedAttentionEngine.appendToCache (PagedAttentionEngine.swift:585-628) */
int32_t pamc_append_to_cache(void *ctx, const PamAppendRequest *request);

/* Append by explicit slot mapping (one int64 slot per token, device or host):
 * the scatter of kernels.metal:1804-1961 with the slot supplied by the caller
 * instead of derived from one block table. */
int32_t pamc_reshape_and_cache(void *ctx, void *cache, const void *keys, const void *values,
                               const int64_t *slot_mapping, int32_t num_tokens);
/* Block copies of copy-on-write (KVCacheManager.swift:176-194): K, V and FP8
 * scale rows of src[i] to dst[i]; src/dst are host arrays. */
int32_t pamc_copy_blocks(void *ctx, void *cache, const int32_t *src, const int32_t *dst, int32_t n);

/* PagedAttentionDecodeRequest (PagedAttentionTypes.swift:259-315). */
typedef struct PamDecodeRequest {
    PamBuffer q, k_pool, v_pool, block_tables, seq_lengths, output;
    int32_t batch_size, max_num_blocks;
    PamLayerSpec layer;
    PamBuffer k_scale, v_scale;
} PamDecodeRequest;
/* PagedAttentionEngine.decode (PagedAttentionEngine.swift:533-580). */
int32_t pamc_decode(void *ctx, const PamDecodeRequest *request);
/* Which kernel a decode request would run on, without launching anything: 1 = the stream
 * kernel (float16 / bfloat16 / FP8 KV, head_dim 128 or 64 (FP8: 128), block size a multiple
 * of 16, at most 16 query heads per KV head, pools 16-byte aligned, queries and outputs 4-byte
 * aligned, queries 8-byte for FP8), 0 = the general kernel, -1 = bad request.  Only pointers,
 * types and shapes are read. */
int32_t pamc_decode_path(const PamDecodeRequest *request);

/* Decode without any allocation.  No counterpart in the reference.
 *
 * For callers that must not allocate device memory while they run: code that
 * is recording work to replay later, a serving loop that has handed all free
 * memory to the KV pools, or a host that only ever gets pointers from another
 * runtime's allocator and cannot reach cudaMalloc itself.  pamc_decode may grow
 * the context's arena (for staged host buffers and for the partial results of
 * shared sequences); this entry point never does.  It calls no cudaMalloc, cudaFree or
 * other allocating routine.
 *
 * Same request, checks, kernels and results as pamc_decode, with these limits:
 *  - q, output, pools, block tables and lengths must all be device memory
 *    (nothing is staged);
 *  - the partial results of sequences that several warps share live in an 8 MiB
 *    array, and the kernel counts on 65 536 words; both are part of the library
 *    image on every GPU that loads it (held until the process exits).  A request
 *    needs one word per (sequence, kv head) pair and, of the array, one record of
 *    (heads / kv_heads) * (head_dim + 4) * 4 bytes per pair of a launch (a launch
 *    takes at most 2048 sequences) and one per warp; the launch takes fewer warps
 *    when the array holds no more, but at least four.  A request that needs more
 *    fails with PAM_ERR_RESOURCE_EXHAUSTED and a message that states the numbers.
 *    Requests that run on the general kernel (pamc_decode_path() == 0) need neither.
 *  - The first call on each GPU looks up the array's device address (once per
 *    device, with that device current).  Make that first call before starting
 *    any stream capture.
 *  - While the context's stream is being captured the call only records its
 *    launches: it does not wait for the stream and does not run the retry loop
 *    (an eager call does both unless pamc_set_async is on).
 *  - All calls on one GPU share the arrays.  The counting words are zero when
 *    the library is loaded and every call leaves them zero (the warp that
 *    completes a pair's count puts its word back); of the records a call reads
 *    only what it has written itself.  Two such decodes that overlap on one GPU
 *    (different streams or contexts) race on both and give wrong results; keep
 *    them ordered. */
int32_t pamc_decode_noalloc(void *ctx, const PamDecodeRequest *request);

/* PagedAttentionPrefillRequest (PagedAttentionTypes.swift:210-256) plus the row
 * range of one chunk: rows [q_start, q_start+q_len) of a sequence whose cache
 * holds seq_len tokens.  q/output hold q_len rows.  q_len = 0 means the whole
 * sequence (q_start = 0, q_len = seq_len), the reference's call. */
typedef struct PamPrefillRequest {
    PamBuffer q, k_pool, v_pool, block_table, output;
    int32_t seq_len;
    PamLayerSpec layer;
    int32_t causal;
    PamBuffer k_scale, v_scale;
    int32_t q_start, q_len;
} PamPrefillRequest;
/* PagedAttentionEngine.prefill (PagedAttentionEngine.swift:405-528); with
 * chunk_size > 0 the rows are processed chunk by chunk like the reference's
 * loop (PagedAttentionEngine.swift:740-756) but each row only once. */
int32_t pamc_prefill(void *ctx, const PamPrefillRequest *request, int32_t chunk_size);

/* One launch for the same chunk of several sequences that share one cache:
 * sequence i contributes rows [q_start[i], q_start[i]+q_len[i]); q/output are
 * the rows of all sequences back to back.  tables [n][max_num_blocks]. */
typedef struct PamBatchPrefillRequest {
    PamBuffer q, k_pool, v_pool, block_tables, output;
    const int32_t *seq_lens, *q_starts, *q_lens; /* host arrays, n entries */
    int32_t num_sequences, max_num_blocks;
    PamLayerSpec layer;
    int32_t causal;
    PamBuffer k_scale, v_scale;
} PamBatchPrefillRequest;
int32_t pamc_prefill_batch(void *ctx, const PamBatchPrefillRequest *request);

/* PagedAttentionFusedPrefillRequest (PagedAttentionTypes.swift:367-421): the raw
 * keys and values of tokens [0, seq_len) are written to the pages of block_table
 * and the prefill of the same seq_len rows runs over them. */
typedef struct PamFusedPrefillRequest {
    PamBuffer q, raw_k, raw_v, block_table, k_pool, v_pool, output;
    int32_t seq_len;
    PamLayerSpec layer;
    int32_t causal;
    PamBuffer k_scale, v_scale;
} PamFusedPrefillRequest;
/* PagedAttentionEngine.fusedPrefill (PagedAttentionEngine.swift:633-710).  Pools
 * and output equal those of pamc_append_to_cache (token_offset 0) followed by
 * pamc_prefill, which is what the reference's own test of this call checks.
 * cache: the handle that owns the pools; required for FP8 (absmax scratch and
 * scale rows), may be NULL otherwise. */
int32_t pamc_fused_prefill(void *ctx, const PamFusedPrefillRequest *request, void *cache);

/* The arguments of PagedAttentionEngine.backward (PagedAttentionEngine.swift:1341-1359) as one
 * struct: gradients of the attention of rows [0, seq_len) over the keys [window_start,
 * seq_len) of one sequence (the kernels have no causal mask, kernels.metal:1217-1415) with
 * respect to the queries and to the paged keys and values.  m and l are the float32 row
 * maximum and row sum of exp(s - m) of the caller's forward pass, [seq_len][heads].  d_q is
 * written; d_k_pool and d_v_pool (shaped and typed like the pools, device memory) are added
 * to, as the reference's atomic adds do.  layer.window_size is the call's windowSize
 * (window_start = max(0, seq_len - window_size) when it is positive); layer.data_type is
 * float32 or float16 as in the reference, or bfloat16. */
typedef struct PamBackwardRequest {
    PamBuffer q, k_pool, v_pool, block_table, d_out, m, l, d_q, d_k_pool, d_v_pool;
    int32_t seq_len;
    PamLayerSpec layer;
} PamBackwardRequest;
int32_t pamc_backward(void *ctx, const PamBackwardRequest *request);

/* The batched-layer calls (PagedAttentionEngine.swift:1433-1895: prefillLayers,
 * decodeLayers, appendLayers): one request per layer, enqueued back to back on
 * the context's stream and waited for once.  The reference hands every layer
 * the same pools; here each request names its own, so one pool per layer works
 * too.  caches[i] (append only) is the handle that owns layer i's pools; it is
 * required for FP8 layers, caches may be NULL otherwise.  num_layers <= 0 is
 * the reference's "buffer/layer count mismatch". */
int32_t pamc_decode_layers(void *ctx, const PamDecodeRequest *requests, int32_t num_layers);
int32_t pamc_prefill_layers(void *ctx, const PamPrefillRequest *requests, int32_t num_layers);
int32_t pamc_append_layers(void *ctx, const PamAppendRequest *requests, int32_t num_layers,
                           void *const *caches);

/* ------------------------------------------------------------------------
 * Outputs of a cache sharded by KV head over several GPUs
 * ---------------------------------------------------------------------- */

/* No counterpart in the reference (one device: PagedAttentionEngine.swift:249,
 * PagedAttentionCABI.swift:104).  With N GPUs, GPU r owns KV heads [r*KVH/N, (r+1)*KVH/N)
 * and the query heads that map to them; attention needs no exchange.  A caller that wants
 * the whole [rows][heads][head_dim] output on every GPU gathers it with these calls
 * (ncclAllGather over NVLink, then one kernel that interleaves the head slices).  NCCL is
 * loaded at run time; without it pamc_comm_unique_id and pamc_comm_create fail.
 *
 * One process per GPU: rank 0 makes the id, the caller carries its 128 bytes to the other
 * ranks by any means, every rank creates its communicator (a collective call). */
int32_t pamc_comm_unique_id(void *out_128_bytes);
void *pamc_comm_create(void *ctx, const void *unique_id_128_bytes, int32_t rank, int32_t num_ranks);
void pamc_comm_destroy(void *comm);
/* local: this GPU's [rows][heads_local][head_dim]; full: [rows][heads_local * num_ranks][head_dim],
 * both device memory of the context's GPU, elements of the query type of data_type
 * (PAM_DTYPE_*).  heads_local * head_dim * element size must be a multiple of 16 bytes.
 * Collective: every rank calls it with the same shape, on its context's stream. */
int32_t pamc_allgather_heads(void *ctx, void *comm, const void *local, void *full, int32_t rows,
                             int32_t heads_local, int32_t head_dim, int32_t data_type);

/* ------------------------------------------------------------------------
 * Scheduler (Scheduler.swift)
 * ---------------------------------------------------------------------- */

/* ContinuousBatchingScheduler.init (Scheduler.swift:53-56) */
void *pamc_sched_create(int32_t max_batch_size, int32_t max_sequences);
void pamc_sched_destroy(void *sched);
/* addRequest (Scheduler.swift:58-70): new id, or -1 when the table is full */
int64_t pamc_sched_add_request(void *sched, int32_t prompt_token_count, int32_t max_new_tokens);
/* completeSequence (Scheduler.swift:72-76) */
void pamc_sched_complete(void *sched, int64_t id);
/* step (Scheduler.swift:78-114): ids of the batch in order; returns the batch
 * size (which may exceed capacity; only capacity ids are written). */
int32_t pamc_sched_step(void *sched, int64_t *out_ids, int32_t capacity);
/* markPrefilled / markDecoded / preemptSequence (Scheduler.swift:116-132) */
void pamc_sched_mark_prefilled(void *sched, int64_t id);
void pamc_sched_mark_decoded(void *sched, int64_t id);
void pamc_sched_preempt(void *sched, int64_t id);
/* handleMemoryPressure (Scheduler.swift:134-152).  available is evaluated
 * before every preemption like the reference's autoclosure. */
typedef int32_t (*pamc_available_fn)(void *user);
int32_t pamc_sched_handle_memory_pressure(void *sched, int32_t required_blocks,
                                          pamc_available_fn available, void *user,
                                          int64_t *out_ids, int32_t capacity);
/* waitingCount / runningCount / completedCount (Scheduler.swift:154-170), by status */
int32_t pamc_sched_count(void *sched, int32_t status);
/* totalSequencesProcessed (Scheduler.swift:172-176) */
int32_t pamc_sched_total(void *sched);
/* SchedulerSequence (Scheduler.swift:24-40) */
typedef struct PamSchedSequence {
    int64_t id;
    int32_t status, num_generated_tokens, max_new_tokens, prompt_length, arrival_order;
} PamSchedSequence;
int32_t pamc_sched_get(void *sched, int64_t id, PamSchedSequence *out);

/* ------------------------------------------------------------------------
 * Inference orchestration (PagedAttentionInference.swift:7-299)
 * ---------------------------------------------------------------------- */

/* PagedAttentionInference.init (:47-90): a cache shaped by the first layer spec
 * and a scheduler, owned by the handle; the engine is the given context.  NULL
 * on error (message in the context). */
void *pamc_infer_create(void *ctx, int32_t max_blocks, int32_t block_size, const PamLayerSpec *layers,
                        int32_t num_layers, int32_t max_batch_size, int32_t max_sequences);
void pamc_infer_destroy(void *infer);
/* the handle's cache and scheduler (borrowed; valid for pam_* / pamc_cache_* and pamc_sched_*) */
void *pamc_infer_cache(void *infer);
void *pamc_infer_scheduler(void *infer);
/* addRequest (:103-105), completeSequence (:108-114) */
int64_t pamc_infer_add_request(void *infer, int32_t prompt_token_count, int32_t max_new_tokens);
void pamc_infer_complete_sequence(void *infer, int64_t id);
/* step (:119-148): prefill of the batch's sequences that are not prefilled yet
 * (one prefillLayers each), one decodeLayers for the others, one token appended
 * to each decoded sequence, finished sequences completed.  Returns the batch
 * size (ids of the batch in out_ids, up to capacity), or -1 on error. */
int32_t pamc_infer_step(void *infer, int64_t *out_ids, int32_t capacity);
/* runAll (:151-156) */
int32_t pamc_infer_run_all(void *infer);
/* totalTokensGenerated (:166-170; prompt tokens count at prefill, :216), stepCount (:34) */
int64_t pamc_infer_total_tokens(void *infer);
int32_t pamc_infer_step_count(void *infer);
/* onTokenGenerated (:27): called with (sequence id, token id = 0) per decoded token */
typedef void (*pamc_token_fn)(void *user, int64_t sequence_id, int32_t token_id);
void pamc_infer_set_token_callback(void *infer, pamc_token_fn fn, void *user);
/* Under memory pressure the reference pauses every running sequence, because
 * the free count it hands to handleMemoryPressure does not change while the
 * victims are chosen (:280-299, Scheduler.swift:134-152).  on != 0: pause and
 * free one victim at a time until enough blocks are free.  Default off. */
void pamc_infer_set_incremental_preemption(void *infer, int32_t on);
/* The reference prefills one sequence per dispatch (:172-219).  on != 0: the prompts of a
 * step go through the same block bookkeeping in the same order, but their attention rows
 * are issued together, one launch per layer.  token_budget > 0 also bounds the prompt rows
 * of a step: a longer prompt is prefilled in chunks over several steps and prompts that do
 * not fit wait for the next step (they decode only once their whole prompt is done).
 * Default off; with on != 0 and token_budget 0 every step leaves the same state as the
 * reference's. */
void pamc_infer_set_batched_prefill(void *infer, int32_t on, int32_t token_budget);
/* Prefill launch sets issued so far (one per sequence in the reference's mode, one per
 * step with batched prefill). */
int64_t pamc_infer_prefill_launch_sets(void *infer);

#ifdef __cplusplus
}
#endif
#endif /* PAM_CUDA_H */
