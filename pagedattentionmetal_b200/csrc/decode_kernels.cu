// Batched paged decode for pools laid out [block][kv_head][block_size][head_dim].
//
// Semantics: paged_decode_single / _f16 / _fp8 (kernels.metal:1417-1620): per
// (sequence, query head) softmax(q.K^T / sqrt(dim)) V over tokens
// [window_start, L) reached through the block table, window_start = L - W when
// W > 0 and L > W (kernels.metal:1442), float32 accumulation.
//
// Two kernels:
//
//  * decodeSplitKernel -- the fast path (float16 / bfloat16 KV, head_dim 64 or
//    128, block_size a multiple of 16, at most 16 query heads per KV head).
//    Split-K flash decoding.  A CTA owns (sequence, kv_head, split); each of
//    its warps runs its own cp.async ring over 16-token tiles (a 16-token run
//    of one kv head is contiguous in the pool: 4 KB of K and 4 KB of V for
//    dim 128) into XOR-swizzled shared memory, multiplies with mma.sync
//    m16n8k16 (rows = the query heads of the GQA group, so every K/V byte is
//    read from HBM once for the whole group), keeps an online softmax in
//    registers, and the warps' partial (m, l, O) are merged through shared
//    memory.  With more than one split per sequence the CTA writes its partial
//    to a workspace and decodeMergeKernel combines the splits with a
//    log-sum-exp reduction.  The kernel is bound by HBM bandwidth; the tensor
//    cores only keep the arithmetic out of the way.
//
//  * decodeGeneralKernel -- any type (float32, FP8 with the reference's
//    half-precision dequantisation chain, kernels.metal:553-562), any block
//    size, head_dim up to 256.  One CTA per (sequence, kv_head), 16 tokens at a
//    time.  Used where the fast path does not apply; not tuned.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <atomic>
#include <cmath>
#include <cstdlib>
#include <cstring>
#include <vector>

#include "kernels.h"

namespace pam {
namespace {

constexpr int kTileTokens = 16;
constexpr float kLog2e = 1.4426950408889634f;


// ---------------------------------------------------------------- PTX helpers

__device__ __forceinline__ uint32_t smemAddr(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void cpAsync16(uint32_t dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(dst), "l"(src));
}
__device__ __forceinline__ void cpAsyncCommit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cpAsyncWait() {
    asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}

__device__ __forceinline__ void ldmatrixX4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr));
}
__device__ __forceinline__ void ldmatrixX4Trans(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr));
}

template <typename T>
__device__ __forceinline__ void mma16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1);
template <>
__device__ __forceinline__ void mma16816<__half>(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
template <>
__device__ __forceinline__ void mma16816<__nv_bfloat16>(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

template <typename T>
__device__ __forceinline__ uint32_t pack2(float lo, float hi);
template <>
__device__ __forceinline__ uint32_t pack2<__half>(float lo, float hi) {
    __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&h);
}
template <>
__device__ __forceinline__ uint32_t pack2<__nv_bfloat16>(float lo, float hi) {
    __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&h);
}

// The two 16-bit halves of a packed pair, widened.
template <typename T> __device__ __forceinline__ float lowHalf(uint32_t v);
template <typename T> __device__ __forceinline__ float highHalf(uint32_t v);
template <> __device__ __forceinline__ float lowHalf<__nv_bfloat16>(uint32_t v) { return __uint_as_float(v << 16); }
template <> __device__ __forceinline__ float highHalf<__nv_bfloat16>(uint32_t v) { return __uint_as_float(v & 0xFFFF0000u); }
template <> __device__ __forceinline__ float lowHalf<__half>(uint32_t v) { return __half2float(__ushort_as_half(static_cast<unsigned short>(v & 0xFFFFu))); }
template <> __device__ __forceinline__ float highHalf<__half>(uint32_t v) { return __half2float(__ushort_as_half(static_cast<unsigned short>(v >> 16))); }
template <typename T> __device__ __forceinline__ constexpr bool isHalf() { return false; }
template <> __device__ __forceinline__ constexpr bool isHalf<__half>() { return true; }
constexpr int kShortContextKeys = 256;

template <typename T>
__device__ __forceinline__ T fromFloat(float v);
template <>
__device__ __forceinline__ __half fromFloat<__half>(float v) { return __float2half_rn(v); }
template <>
__device__ __forceinline__ __nv_bfloat16 fromFloat<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
template <>
__device__ __forceinline__ float fromFloat<float>(float v) { return v; }

__device__ __forceinline__ float toFloat(float v) { return v; }
__device__ __forceinline__ float toFloat(__half v) { return __half2float(v); }
__device__ __forceinline__ float toFloat(__nv_bfloat16 v) { return __bfloat162float(v); }

// Split geometry shared by the decode and the merge kernel.
struct SplitInfo {
    int firstTile;   // first 16-token tile that holds a visible token
    int numTiles;    // tiles from there to the end of the sequence
    int windowStart; // first visible token
};
__device__ __forceinline__ SplitInfo splitInfo(uint32_t len, int window, int maxTokens) {
    SplitInfo s;
    uint32_t L = len < static_cast<uint32_t>(maxTokens) ? len : static_cast<uint32_t>(maxTokens);
    s.windowStart = (window > 0 && len > static_cast<uint32_t>(window)) ? static_cast<int>(len) - window : 0;
    if (s.windowStart > static_cast<int>(L)) s.windowStart = static_cast<int>(L);
    s.firstTile = s.windowStart / kTileTokens;
    s.numTiles = (static_cast<int>(L) + kTileTokens - 1) / kTileTokens - s.firstTile;
    return s;
}

// The tiles of a sequence are divided evenly over its splits (sizes differ by at most one
// tile, none is empty): split k of n covers tiles [begin, end) counted from the first
// visible tile.
__host__ __device__ __forceinline__ int splitCount(int numTiles, int chunkTiles) {
    const int n = (numTiles + chunkTiles - 1) / chunkTiles;
    return n < 1 ? 1 : n;
}
__host__ __device__ __forceinline__ void splitRange(int numTiles, int numSplits, int split, int& begin, int& end) {
    const int base = numTiles / numSplits, rem = numTiles - base * numSplits;
    begin = split * base + (split < rem ? split : rem);
    end = begin + base + (split < rem ? 1 : 0);
}

// The running maximum of a row is only raised when a tile exceeds it by more than this
// (log2 domain): the result is the same either way because the final division uses the
// same reference, and the accumulator is then rescaled a few times per split instead of
// once per tile.  Weights reach at most 2^kLazyMax, well inside float16 and bfloat16.
constexpr float kLazyMax = 6.0f;
// bfloat16 weights keep 8 significant bits: only with the exact maximum as the reference is
// the largest weight of a row exactly 1, and a row that one key dominates stays within the
// 2e-3 bound.  There the maximum is followed exactly (the accumulator is still only
// rescaled on the tiles that raise it); float16 weights (11 bits) take the lazy form.
template <typename T> __device__ __forceinline__ constexpr float lazyMaxOf() { return kLazyMax; }
template <> __device__ __forceinline__ constexpr float lazyMaxOf<__nv_bfloat16>() { return 0.f; }

// What a CTA of the split kernels works on.  Two launch shapes:
//  * grid (maxSplits, kv_heads, batch): the range follows from the sequence's length;
//  * grid (items, kv_heads) with a work list built on the host from the lengths (longest
//    ranges first, so that the short ones fill the end of the launch): item = (sequence,
//    first tile, end tile, split | splits << 16).
struct SplitWork {
    int b, kvh, split, numSplits, tileBegin, tileEnd;
    SplitInfo si;
    uint32_t len;
};
__device__ __forceinline__ SplitWork splitWork(const int4* __restrict__ items, const uint32_t* __restrict__ lens,
                                               int window, int maxTokens, int chunkTiles) {
    SplitWork w;
    if (items) {
        const int4 it = items[blockIdx.x];
        w.b = it.x; w.kvh = blockIdx.y;
        w.len = lens[w.b];
        w.si = splitInfo(w.len, window, maxTokens);
        w.split = it.w & 0xFFFF; w.numSplits = it.w >> 16;
        w.tileBegin = it.y; w.tileEnd = it.z;
    } else {
        w.b = blockIdx.z; w.kvh = blockIdx.y; w.split = blockIdx.x;
        w.len = lens[w.b];
        w.si = splitInfo(w.len, window, maxTokens);
        w.numSplits = splitCount(w.si.numTiles, chunkTiles);
        int begin = 0, end = 0;
        if (w.si.numTiles > 0 && w.split < w.numSplits) splitRange(w.si.numTiles, w.numSplits, w.split, begin, end);
        w.tileBegin = w.si.firstTile + begin;
        w.tileEnd = w.si.firstTile + end;
    }
    return w;
}

// End of a split: the warps' partial results (m, l, O per query head, in `red`,
// [NW][G][HD + 2]) are combined; a sequence with one split gets its output, else the
// partial goes to the workspace.  With `counters` (one zeroed word per (sequence, kv head))
// the CTA that finishes a (sequence, kv head) last combines its splits right away and puts
// the word back to zero; without, decodeMergeKernel does that in a launch of its own.
template <typename T, int HD, int NW>
__device__ __forceinline__ void finishSplit(const float* red, int G, const SplitWork& w, int heads, int kvHeads,
                                            int maxSplits, T* __restrict__ out, float* __restrict__ workspace,
                                            int* __restrict__ counters) {
    constexpr int RS = HD + 2;
    __shared__ int sIsLast;
    for (int idx = threadIdx.x; idx < G * HD; idx += NW * 32) {
        const int g = idx / HD, d = idx - g * HD;
        float M = -INFINITY;
#pragma unroll
        for (int x = 0; x < NW; ++x) M = fmaxf(M, red[(x * G + g) * RS + HD]);
        float acc = 0.f, lsum = 0.f;
#pragma unroll
        for (int x = 0; x < NW; ++x) {
            const float wgt = exp2f(red[(x * G + g) * RS + HD] - M);   // idle warps: exp2(-inf) = 0
            acc += wgt * red[(x * G + g) * RS + d];
            lsum += wgt * red[(x * G + g) * RS + HD + 1];
        }
        const int head = w.kvh * G + g;
        if (w.numSplits == 1) {
            out[(static_cast<int64_t>(w.b) * heads + head) * HD + d] = fromFloat<T>(acc / lsum);
        } else {
            float* part = workspace + ((static_cast<int64_t>(w.b) * heads + head) * maxSplits + w.split) * RS;
            part[d] = acc;
            if (d == 0) { part[HD] = M; part[HD + 1] = lsum; }
        }
    }
    if (w.numSplits == 1 || !counters) return;
    // The partial is published before the arrival is counted; the last arrival reads the
    // others' partials from L2.
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        int* cnt = counters + static_cast<int64_t>(w.b) * kvHeads + w.kvh;
        const int before = atomicAdd(cnt, 1);
        sIsLast = before == w.numSplits - 1 ? 1 : 0;
        if (sIsLast) *cnt = 0;                      // ready for the next launch
    }
    __syncthreads();
    if (!sIsLast) return;
    __threadfence();
    // The weights of the splits first (one thread per (head, split), all loads in flight
    // together), into the shared memory the warps' partials no longer need; then one thread
    // per output element sums over the splits with eight loads in flight.
    float* wgtOf = const_cast<float*>(red);                 // [G][maxSplits] weights, then [G] 1 / sum
    __syncthreads();
    for (int g = 0; g < G; ++g) {
        const float* part = workspace + (static_cast<int64_t>(w.b) * heads + w.kvh * G + g) * maxSplits * RS;
        float M = -INFINITY;
        for (int sp = threadIdx.x; sp < w.numSplits; sp += NW * 32) M = fmaxf(M, __ldcg(part + sp * RS + HD));
        // block maximum through the warps
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) M = fmaxf(M, __shfl_xor_sync(0xFFFFFFFFu, M, o));
        __shared__ float sM[NW], sL[NW];
        if ((threadIdx.x & 31) == 0) sM[threadIdx.x >> 5] = M;
        __syncthreads();
        M = sM[0];
#pragma unroll
        for (int x = 1; x < NW; ++x) M = fmaxf(M, sM[x]);
        float lsum = 0.f;
        for (int sp = threadIdx.x; sp < w.numSplits; sp += NW * 32) {
            const float wgt = exp2f(__ldcg(part + sp * RS + HD) - M);
            wgtOf[g * maxSplits + sp] = wgt;
            lsum += wgt * __ldcg(part + sp * RS + HD + 1);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) lsum += __shfl_xor_sync(0xFFFFFFFFu, lsum, o);
        if ((threadIdx.x & 31) == 0) sL[threadIdx.x >> 5] = lsum;
        __syncthreads();
        if (threadIdx.x == 0) {
            float total = 0.f;
#pragma unroll
            for (int x = 0; x < NW; ++x) total += sL[x];
            wgtOf[G * maxSplits + g] = 1.f / total;
        }
        __syncthreads();
    }
    for (int idx = threadIdx.x; idx < G * HD; idx += NW * 32) {
        const int g = idx / HD, d = idx - g * HD;
        const int head = w.kvh * G + g;
        const float* part = workspace + (static_cast<int64_t>(w.b) * heads + head) * maxSplits * RS + d;
        const float* wg = wgtOf + g * maxSplits;
        float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        int sp = 0;
        for (; sp + 8 <= w.numSplits; sp += 8) {
#pragma unroll
            for (int u = 0; u < 8; ++u) acc[u] += wg[sp + u] * __ldcg(part + (sp + u) * RS);
        }
        for (; sp < w.numSplits; ++sp) acc[0] += wg[sp] * __ldcg(part + sp * RS);
        const float total = ((acc[0] + acc[1]) + (acc[2] + acc[3])) + ((acc[4] + acc[5]) + (acc[6] + acc[7]));
        out[(static_cast<int64_t>(w.b) * heads + head) * HD + d] = fromFloat<T>(total * wgtOf[G * maxSplits + g]);
    }
}

// ------------------------------------------------------------ fast split kernel

template <typename T, int HD, int NW, int NS, bool UPPER>
__global__ void __launch_bounds__(NW * 32)
decodeSplitKernel(const T* __restrict__ q, const T* __restrict__ kPool, const T* __restrict__ vPool,
                  const int32_t* __restrict__ tables, const uint32_t* __restrict__ lens,
                  T* __restrict__ out, float* __restrict__ workspace, int heads, int kvHeads,
                  int blockSize, int maxNumBlocks, int window, int chunkTiles, int maxSplits,
                  float scaleLog2, int poolBlocks, const int4* __restrict__ items, int* __restrict__ counters) {
    constexpr int ROWB = HD * 2;                 // bytes per token row
    constexpr int CPR = ROWB / 16;               // 16-byte chunks per row
    constexpr int TILEB = kTileTokens * ROWB;    // bytes per K (or V) tile
    constexpr int CHUNKS = TILEB / 16;
    constexpr int KSTEPS = HD / 16;
    constexpr int NT = HD / 8;                   // output n-tiles

    extern __shared__ __align__(128) unsigned char smem[];

    const SplitWork work = splitWork(items, lens, window, maxNumBlocks * blockSize, chunkTiles);
    const int kvh = work.kvh, b = work.b;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int G = heads / kvHeads;
    const int r = lane >> 2, j = lane & 3;

    const uint32_t len = work.len;
    const SplitInfo si = work.si;
    if (si.numTiles <= 0) {
        // Empty context (the reference divides 0 by 0 here): write zeros.
        if (work.split == 0)
            for (int i = threadIdx.x; i < G * HD; i += NW * 32)
                out[(static_cast<int64_t>(b) * heads + kvh * G) * HD + i] = fromFloat<T>(0.f);
        return;
    }
    if (work.split >= work.numSplits) return;

    const int tileBegin = work.tileBegin, tileEnd = work.tileEnd;
    // A bfloat16 weight keeps 8 significant bits.  A sequence with few visible keys has large
    // weights, and 8 bits alone can then miss the 2e-3 bound on unit-variance values: such
    // sequences carry every weight as two bfloat16 operands (16 bits) into a second product.
    // With hundreds of keys the weights are small enough for 8 bits.
    const bool twoPartWeights = sizeof(T) == 2 && !isHalf<T>() && static_cast<int>(len) - si.windowStart < kShortContextKeys;
    // warp w takes tiles tileBegin + w, + NW, ...
    const int myTiles = (tileEnd - tileBegin - warp + NW - 1) / NW;
    const int tilesPerPage = blockSize / kTileTokens;
    const int32_t* table = tables + static_cast<int64_t>(b) * maxNumBlocks;

    unsigned char* ring = smem + static_cast<size_t>(warp) * NS * 2 * TILEB;
    const uint32_t ringAddr = smemAddr(ring);

    auto issue = [&](int it) {
        const int tile = tileBegin + warp + it * NW;
        const int page = tile / tilesPerPage, within = tile - page * tilesPerPage;
        const int64_t blk = min(max(table[page], 0), poolBlocks - 1);   // never read outside the pool
        const int64_t elemOff = ((blk * kvHeads + kvh) * blockSize + within * kTileTokens) * static_cast<int64_t>(HD);
        const unsigned char* gk = reinterpret_cast<const unsigned char*>(kPool + elemOff);
        const unsigned char* gv = reinterpret_cast<const unsigned char*>(vPool + elemOff);
        const uint32_t sk = ringAddr + (it % NS) * 2 * TILEB, sv = sk + TILEB;
#pragma unroll
        for (int i = 0; i < CHUNKS / 32; ++i) {
            const int idx = lane + 32 * i;
            const int row = idx / CPR, c = idx % CPR;
            const uint32_t dst = row * ROWB + ((c ^ (row & 7)) << 4);
            cpAsync16(sk + dst, gk + idx * 16);
            cpAsync16(sv + dst, gv + idx * 16);
        }
    };

    // Query rows of this GQA group as A fragments (rows >= G are zero).
    uint32_t qa[KSTEPS][4];
    {
        const T* qb = q + (static_cast<int64_t>(b) * heads + kvh * G) * HD;
#pragma unroll
        for (int ks = 0; ks < KSTEPS; ++ks) {
            const int d0 = ks * 16 + 2 * j;
            qa[ks][0] = r < G ? *reinterpret_cast<const uint32_t*>(qb + r * HD + d0) : 0u;
            qa[ks][2] = r < G ? *reinterpret_cast<const uint32_t*>(qb + r * HD + d0 + 8) : 0u;
            if (UPPER) {
                qa[ks][1] = r + 8 < G ? *reinterpret_cast<const uint32_t*>(qb + (r + 8) * HD + d0) : 0u;
                qa[ks][3] = r + 8 < G ? *reinterpret_cast<const uint32_t*>(qb + (r + 8) * HD + d0 + 8) : 0u;
            } else {
                qa[ks][1] = 0u;
                qa[ks][3] = 0u;
            }
        }
    }

    float o[NT][4];
#pragma unroll
    for (int n = 0; n < NT; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;

#pragma unroll
    for (int s = 0; s < NS; ++s) {
        if (s < myTiles) issue(s);
        cpAsyncCommit();
    }

    for (int it = 0; it < myTiles; ++it) {
        cpAsyncWait<NS - 1>();
        __syncwarp();
        const int tile = tileBegin + warp + it * NW;
        const int tokBase = tile * kTileTokens;
        const uint32_t sk = ringAddr + (it % NS) * 2 * TILEB, sv = sk + TILEB;
        const bool partial = tokBase < si.windowStart || tokBase + kTileTokens > static_cast<int>(len);
        if (partial) {
            // Rows outside [window_start, L) may hold anything; zero their V so
            // that a zero probability times that row stays zero.
            unsigned char* vt = ring + (it % NS) * 2 * TILEB + TILEB;
            for (int idx = lane; idx < CHUNKS; idx += 32) {
                const int row = idx / CPR;
                const int tok = tokBase + row;
                if (tok < si.windowStart || tok >= static_cast<int>(len))
                    *reinterpret_cast<uint4*>(vt + idx * 16) = make_uint4(0u, 0u, 0u, 0u);
            }
            __syncwarp();
        }

        // S = Q K^T for the 16 tokens of the tile (two n-tiles of 8 tokens).
        float s[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
        for (int ks = 0; ks < KSTEPS; ++ks) {
            const int mi = lane >> 3, rowIn = lane & 7;
            const int row = 8 * (mi >> 1) + rowIn, chunk = 2 * ks + (mi & 1);
            uint32_t kb[4];
            ldmatrixX4(kb, sk + row * ROWB + ((chunk ^ (row & 7)) << 4));
            mma16816<T>(s[0], qa[ks], kb[0], kb[1]);
            mma16816<T>(s[1], qa[ks], kb[2], kb[3]);
        }

        // Online softmax in the log2 domain.
        float tmax0 = -INFINITY, tmax1 = -INFINITY;
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int tok = tokBase + 8 * nt + 2 * j + e;
                const bool ok = !partial || (tok >= si.windowStart && tok < static_cast<int>(len));
                s[nt][e] = ok ? s[nt][e] * scaleLog2 : -INFINITY;
                tmax0 = fmaxf(tmax0, s[nt][e]);
                if (UPPER) {
                    s[nt][e + 2] = ok ? s[nt][e + 2] * scaleLog2 : -INFINITY;
                    tmax1 = fmaxf(tmax1, s[nt][e + 2]);
                }
            }
        }
        tmax0 = fmaxf(tmax0, __shfl_xor_sync(0xFFFFFFFFu, tmax0, 1));
        tmax0 = fmaxf(tmax0, __shfl_xor_sync(0xFFFFFFFFu, tmax0, 2));
        bool raise = tmax0 > m0 + lazyMaxOf<T>();  // m0 = -inf: the first tile always raises
        float c0 = 1.f, c1 = 1.f;
        if (raise) { c0 = exp2f(m0 - tmax0); m0 = tmax0; }   // m0 = -inf gives 0
        if (UPPER) {
            tmax1 = fmaxf(tmax1, __shfl_xor_sync(0xFFFFFFFFu, tmax1, 1));
            tmax1 = fmaxf(tmax1, __shfl_xor_sync(0xFFFFFFFFu, tmax1, 2));
            if (tmax1 > m1 + lazyMaxOf<T>()) { c1 = exp2f(m1 - tmax1); m1 = tmax1; raise = true; }
        }
        if (__any_sync(0xFFFFFFFFu, raise)) {
            l0 *= c0;
            if (UPPER) l1 *= c1;
#pragma unroll
            for (int n = 0; n < NT; ++n) {
                o[n][0] *= c0;
                o[n][1] *= c0;
                if (UPPER) {
                    o[n][2] *= c1;
                    o[n][3] *= c1;
                }
            }
        }
        uint32_t pa[4], pl[4] = {0u, 0u, 0u, 0u};
        {
            const float p00 = exp2f(s[0][0] - m0), p01 = exp2f(s[0][1] - m0);
            const float p10 = exp2f(s[1][0] - m0), p11 = exp2f(s[1][1] - m0);
            l0 += (p00 + p01) + (p10 + p11);
            pa[0] = pack2<T>(p00, p01);
            pa[2] = pack2<T>(p10, p11);
            if (twoPartWeights) {
                pl[0] = pack2<T>(p00 - lowHalf<T>(pa[0]), p01 - highHalf<T>(pa[0]));
                pl[2] = pack2<T>(p10 - lowHalf<T>(pa[2]), p11 - highHalf<T>(pa[2]));
            }
            if (UPPER) {
                const float q00 = exp2f(s[0][2] - m1), q01 = exp2f(s[0][3] - m1);
                const float q10 = exp2f(s[1][2] - m1), q11 = exp2f(s[1][3] - m1);
                l1 += (q00 + q01) + (q10 + q11);
                pa[1] = pack2<T>(q00, q01);
                pa[3] = pack2<T>(q10, q11);
                if (twoPartWeights) {
                    pl[1] = pack2<T>(q00 - lowHalf<T>(pa[1]), q01 - highHalf<T>(pa[1]));
                    pl[3] = pack2<T>(q10 - lowHalf<T>(pa[3]), q11 - highHalf<T>(pa[3]));
                }
            } else {
                pa[1] = 0u;
                pa[3] = 0u;
            }
        }

        // O += P V
#pragma unroll
        for (int cp = 0; cp < NT / 2; ++cp) {
            const int mi = lane >> 3, rowIn = lane & 7;
            const int row = (mi & 1) * 8 + rowIn, chunk = 2 * cp + (mi >> 1);
            uint32_t vb[4];
            ldmatrixX4Trans(vb, sv + row * ROWB + ((chunk ^ (row & 7)) << 4));
            mma16816<T>(o[2 * cp], pa, vb[0], vb[1]);
            mma16816<T>(o[2 * cp + 1], pa, vb[2], vb[3]);
            if (twoPartWeights) {
                mma16816<T>(o[2 * cp], pl, vb[0], vb[1]);
                mma16816<T>(o[2 * cp + 1], pl, vb[2], vb[3]);
            }
        }

        __syncwarp();
        if (it + NS < myTiles) issue(it + NS);
        cpAsyncCommit();
    }
    cpAsyncWait<0>();

    // Row sums live spread over the four lanes of a quad.
    l0 += __shfl_xor_sync(0xFFFFFFFFu, l0, 1);
    l0 += __shfl_xor_sync(0xFFFFFFFFu, l0, 2);
    if (UPPER) {
        l1 += __shfl_xor_sync(0xFFFFFFFFu, l1, 1);
        l1 += __shfl_xor_sync(0xFFFFFFFFu, l1, 2);
    }

    // Merge the warps of the CTA through shared memory (the rings are idle now).
    __syncthreads();
    float* red = reinterpret_cast<float*>(smem);            // [NW][G][HD + 2]
    constexpr int RS = HD + 2;
    {
        float* mine = red + static_cast<size_t>(warp) * G * RS;
        if (r < G) {
#pragma unroll
            for (int n = 0; n < NT; ++n) {
                mine[r * RS + 8 * n + 2 * j] = o[n][0];
                mine[r * RS + 8 * n + 2 * j + 1] = o[n][1];
            }
            if (j == 0) { mine[r * RS + HD] = m0; mine[r * RS + HD + 1] = l0; }
        }
        if (UPPER && r + 8 < G) {
#pragma unroll
            for (int n = 0; n < NT; ++n) {
                mine[(r + 8) * RS + 8 * n + 2 * j] = o[n][2];
                mine[(r + 8) * RS + 8 * n + 2 * j + 1] = o[n][3];
            }
            if (j == 0) { mine[(r + 8) * RS + HD] = m1; mine[(r + 8) * RS + HD + 1] = l1; }
        }
    }
    __syncthreads();
    finishSplit<T, HD, NW>(red, G, work, heads, kvHeads, maxSplits, out, workspace, counters);
}

// ------------------------------------------------------------ FP8 split kernel

// 2^x by the special-function unit alone (exp2f adds a range fix-up for results below the
// normal range, which a softmax weight does not need); 2^-inf = 0.
__device__ __forceinline__ float ex2Fast(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// Two e4m3 codes (low 16 bits of `v`) to two float16 values; exact, every e4m3
// value is a float16 value.
__device__ __forceinline__ uint32_t e4m3x2ToHalf2(uint32_t v) {
    uint32_t r;
    asm("{\n\t.reg .b16 lo, hi;\n\tmov.b32 {lo, hi}, %1;\n\tcvt.rn.f16x2.e4m3x2 %0, lo;\n\t}" : "=r"(r) : "r"(v));
    return r;
}
__device__ __forceinline__ uint32_t e4m3x2HiToHalf2(uint32_t v) {
    uint32_t r;
    asm("{\n\t.reg .b16 lo, hi;\n\tmov.b32 {lo, hi}, %1;\n\tcvt.rn.f16x2.e4m3x2 %0, hi;\n\t}" : "=r"(r) : "r"(v));
    return r;
}

// The fast path for FP8 e4m3 KV (head_dim 128, block size a multiple of 16,
// float16 queries and outputs).  Same structure as decodeSplitKernel; a
// 16-token tile is 2 KB of K codes and 2 KB of V codes.  Codes become float16
// in registers (exactly) and feed mma.sync.m16n8k16.f16; the group scales
// [block][kv_head] are applied outside the products: K's on the scores, V's on
// the weights (relative to the scale of the warp's first tile, so that the
// weights stay in float16's normal range).  The fragments are loaded with
// 16-byte shared-memory reads: the K-dimension of QK^T and the N-dimension of
// PV are permuted so that every thread reads contiguous codes, which no result
// depends on.
template <int NW, int NS, bool UPPER>
__global__ void __launch_bounds__(NW * 32)
decodeSplitFp8Kernel(const __half* __restrict__ q, const uint8_t* __restrict__ kPool, const uint8_t* __restrict__ vPool,
                     const __half* __restrict__ kScale, const __half* __restrict__ vScale,
                     const int32_t* __restrict__ tables, const uint32_t* __restrict__ lens,
                     __half* __restrict__ out, float* __restrict__ workspace, int heads, int kvHeads,
                     int blockSize, int maxNumBlocks, int window, int chunkTiles, int maxSplits,
                     float scaleLog2, int poolBlocks, const int4* __restrict__ items, int* __restrict__ counters) {
    constexpr int HD = 128;
    constexpr int ROWB = HD;                     // bytes per token row
    constexpr int TILEB = kTileTokens * ROWB;    // 2 KB per K (or V) tile
    constexpr int CHUNKS = TILEB / 16;           // 128 16-byte chunks
    constexpr int STAGEB = 2 * TILEB + 16;       // + the two group scales of the tile
    constexpr int KSTEPS = HD / 16;
    constexpr int NT = HD / 8;

    extern __shared__ __align__(128) unsigned char smem[];

    const SplitWork work = splitWork(items, lens, window, maxNumBlocks * blockSize, chunkTiles);
    const int kvh = work.kvh, b = work.b;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int G = heads / kvHeads;
    const int r = lane >> 2, j = lane & 3;

    const uint32_t len = work.len;
    const SplitInfo si = work.si;
    if (si.numTiles <= 0) {
        if (work.split == 0)
            for (int i = threadIdx.x; i < G * HD; i += NW * 32)
                out[(static_cast<int64_t>(b) * heads + kvh * G) * HD + i] = __float2half_rn(0.f);
        return;
    }
    if (work.split >= work.numSplits) return;

    const int tileBegin = work.tileBegin, tileEnd = work.tileEnd;
    const int myTiles = (tileEnd - tileBegin - warp + NW - 1) / NW;
    const int tilesPerPage = blockSize / kTileTokens;
    const int32_t* table = tables + static_cast<int64_t>(b) * maxNumBlocks;

    unsigned char* ring = smem + static_cast<size_t>(warp) * NS * STAGEB;
    const uint32_t ringAddr = smemAddr(ring);

    auto issue = [&](int it) {
        const int tile = tileBegin + warp + it * NW;
        const int page = tile / tilesPerPage, within = tile - page * tilesPerPage;
        const int64_t blk = min(max(table[page], 0), poolBlocks - 1);
        const int64_t off = ((blk * kvHeads + kvh) * blockSize + within * kTileTokens) * static_cast<int64_t>(HD);
        const unsigned char* gk = kPool + off;
        const unsigned char* gv = vPool + off;
        const uint32_t sk = ringAddr + (it % NS) * STAGEB, sv = sk + TILEB;
#pragma unroll
        for (int i = 0; i < CHUNKS / 32; ++i) {
            const int idx = lane + 32 * i;
            const int row = idx >> 3, c = idx & 7;
            const uint32_t dst = row * ROWB + ((c ^ (row & 7)) << 4);
            cpAsync16(sk + dst, gk + idx * 16);
            cpAsync16(sv + dst, gv + idx * 16);
        }
        if (lane == 0) {
            __half* sc = reinterpret_cast<__half*>(ring + (it % NS) * STAGEB + 2 * TILEB);
            sc[0] = kScale[blk * kvHeads + kvh];
            sc[1] = vScale[blk * kvHeads + kvh];
        }
    };

    // Query rows as A fragments with the permuted K order: step ks of thread
    // (r, j) covers dims 32j + 4ks + {0,1} (first half) and + {2,3} (second half).
    uint32_t qa[KSTEPS][4];
    {
        const __half* qb = q + (static_cast<int64_t>(b) * heads + kvh * G) * HD;
#pragma unroll
        for (int ks = 0; ks < KSTEPS; ++ks) {
            const int d0 = 32 * j + 4 * ks;
            uint2 lo = make_uint2(0u, 0u), hi = make_uint2(0u, 0u);
            if (r < G) lo = *reinterpret_cast<const uint2*>(qb + r * HD + d0);
            if (UPPER && r + 8 < G) hi = *reinterpret_cast<const uint2*>(qb + (r + 8) * HD + d0);
            qa[ks][0] = lo.x; qa[ks][2] = lo.y;
            qa[ks][1] = hi.x; qa[ks][3] = hi.y;
        }
    }

    float o[NT][4];
#pragma unroll
    for (int n = 0; n < NT; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
    float vRef = 0.f, invVRef = 0.f;             // V scale of the warp's first tile

#pragma unroll
    for (int s = 0; s < NS; ++s) {
        if (s < myTiles) issue(s);
        cpAsyncCommit();
    }

    for (int it = 0; it < myTiles; ++it) {
        cpAsyncWait<NS - 1>();
        __syncwarp();
        const int tile = tileBegin + warp + it * NW;
        const int tokBase = tile * kTileTokens;
        unsigned char* stage = ring + (it % NS) * STAGEB;
        const uint32_t sk = ringAddr + (it % NS) * STAGEB, sv = sk + TILEB;
        const __half* sc = reinterpret_cast<const __half*>(stage + 2 * TILEB);
        const float ks_ = __half2float(sc[0]), vs_ = __half2float(sc[1]);
        if (it == 0) { vRef = vs_ > 0.f ? vs_ : 1.f; invVRef = 1.f / vRef; }
        const bool partial = tokBase < si.windowStart || tokBase + kTileTokens > static_cast<int>(len);
        if (partial) {
            // rows outside [window_start, L): zero codes, so that a zero weight times that row is zero
            unsigned char* vt = stage + TILEB;
            for (int idx = lane; idx < CHUNKS; idx += 32) {
                const int tok = tokBase + (idx >> 3);
                if (tok < si.windowStart || tok >= static_cast<int>(len))
                    *reinterpret_cast<uint4*>(vt + idx * 16) = make_uint4(0u, 0u, 0u, 0u);
            }
            __syncwarp();
        }

        // S = Q K^T on the codes; the group scale and 1/sqrt(d) follow.
        float s[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
            const int row = 8 * nt + r;
            const uint4 w0 = *reinterpret_cast<const uint4*>(stage + row * ROWB + (((2 * j) ^ (row & 7)) << 4));
            const uint4 w1 = *reinterpret_cast<const uint4*>(stage + row * ROWB + (((2 * j + 1) ^ (row & 7)) << 4));
            const uint32_t w[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
            for (int ks = 0; ks < KSTEPS; ++ks)
                mma16816<__half>(s[nt], qa[ks], e4m3x2ToHalf2(w[ks]), e4m3x2HiToHalf2(w[ks]));
        }
        (void)sk;

        const float sScale = ks_ * scaleLog2;
        float tmax0 = -INFINITY, tmax1 = -INFINITY;
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int tok = tokBase + 8 * nt + 2 * j + e;
                const bool ok = !partial || (tok >= si.windowStart && tok < static_cast<int>(len));
                s[nt][e] = ok ? s[nt][e] * sScale : -INFINITY;
                tmax0 = fmaxf(tmax0, s[nt][e]);
                if (UPPER) {
                    s[nt][e + 2] = ok ? s[nt][e + 2] * sScale : -INFINITY;
                    tmax1 = fmaxf(tmax1, s[nt][e + 2]);
                }
            }
        }
        tmax0 = fmaxf(tmax0, __shfl_xor_sync(0xFFFFFFFFu, tmax0, 1));
        tmax0 = fmaxf(tmax0, __shfl_xor_sync(0xFFFFFFFFu, tmax0, 2));
        bool raise = tmax0 > m0 + kLazyMax;        // m0 = -inf: the first tile always raises
        float c0 = 1.f, c1 = 1.f;
        if (raise) { c0 = ex2Fast(m0 - tmax0); m0 = tmax0; }
        if (UPPER) {
            tmax1 = fmaxf(tmax1, __shfl_xor_sync(0xFFFFFFFFu, tmax1, 1));
            tmax1 = fmaxf(tmax1, __shfl_xor_sync(0xFFFFFFFFu, tmax1, 2));
            if (tmax1 > m1 + kLazyMax) { c1 = ex2Fast(m1 - tmax1); m1 = tmax1; raise = true; }
        }
        if (__any_sync(0xFFFFFFFFu, raise)) {
            l0 *= c0;
            if (UPPER) l1 *= c1;
#pragma unroll
            for (int n = 0; n < NT; ++n) {
                o[n][0] *= c0;
                o[n][1] *= c0;
                if (UPPER) {
                    o[n][2] *= c1;
                    o[n][3] *= c1;
                }
            }
        }
        // weights; those that enter the product carry V's group scale relative to vRef
        const float vw = vs_ * invVRef;
        uint32_t pa[4];
        {
            const float p00 = ex2Fast(s[0][0] - m0), p01 = ex2Fast(s[0][1] - m0);
            const float p10 = ex2Fast(s[1][0] - m0), p11 = ex2Fast(s[1][1] - m0);
            l0 += (p00 + p01) + (p10 + p11);
            pa[0] = pack2<__half>(p00 * vw, p01 * vw);
            pa[2] = pack2<__half>(p10 * vw, p11 * vw);
            if (UPPER) {
                const float q00 = ex2Fast(s[0][2] - m1), q01 = ex2Fast(s[0][3] - m1);
                const float q10 = ex2Fast(s[1][2] - m1), q11 = ex2Fast(s[1][3] - m1);
                l1 += (q00 + q01) + (q10 + q11);
                pa[1] = pack2<__half>(q00 * vw, q01 * vw);
                pa[3] = pack2<__half>(q10 * vw, q11 * vw);
            } else {
                pa[1] = 0u;
                pa[3] = 0u;
            }
        }

        // O += P V.  Thread (r, j) reads chunk r (dims 16r .. 16r+15) of the token rows
        // 2j, 2j+1, 2j+8, 2j+9; n-tile c takes byte c of each: output column n of
        // n-tile c is dim 16n + c.
        {
            const unsigned char* vt = stage + TILEB;
            uint4 x[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int row = 2 * j + (i & 1) + 8 * (i >> 1);
                x[i] = *reinterpret_cast<const uint4*>(vt + row * ROWB + ((r ^ (row & 7)) << 4));
            }
            const uint32_t* x0 = reinterpret_cast<const uint32_t*>(&x[0]);
            const uint32_t* x1 = reinterpret_cast<const uint32_t*>(&x[1]);
            const uint32_t* x2 = reinterpret_cast<const uint32_t*>(&x[2]);
            const uint32_t* x3 = reinterpret_cast<const uint32_t*>(&x[3]);
#pragma unroll
            for (int wi = 0; wi < 4; ++wi) {
                const uint32_t a01 = __byte_perm(x0[wi], x1[wi], 0x5140);   // bytes 0,1 of both tokens, interleaved
                const uint32_t a23 = __byte_perm(x0[wi], x1[wi], 0x7362);
                const uint32_t b01 = __byte_perm(x2[wi], x3[wi], 0x5140);
                const uint32_t b23 = __byte_perm(x2[wi], x3[wi], 0x7362);
                mma16816<__half>(o[4 * wi + 0], pa, e4m3x2ToHalf2(a01), e4m3x2ToHalf2(b01));
                mma16816<__half>(o[4 * wi + 1], pa, e4m3x2HiToHalf2(a01), e4m3x2HiToHalf2(b01));
                mma16816<__half>(o[4 * wi + 2], pa, e4m3x2ToHalf2(a23), e4m3x2ToHalf2(b23));
                mma16816<__half>(o[4 * wi + 3], pa, e4m3x2HiToHalf2(a23), e4m3x2HiToHalf2(b23));
            }
        }
        (void)sv;

        __syncwarp();
        if (it + NS < myTiles) issue(it + NS);
        cpAsyncCommit();
    }
    cpAsyncWait<0>();

    l0 += __shfl_xor_sync(0xFFFFFFFFu, l0, 1);
    l0 += __shfl_xor_sync(0xFFFFFFFFu, l0, 2);
    if (UPPER) {
        l1 += __shfl_xor_sync(0xFFFFFFFFu, l1, 1);
        l1 += __shfl_xor_sync(0xFFFFFFFFu, l1, 2);
    }

    __syncthreads();
    float* red = reinterpret_cast<float*>(smem);            // [NW][G][HD + 2]
    constexpr int RS = HD + 2;
    {
        float* mine = red + static_cast<size_t>(warp) * G * RS;
        if (r < G) {
#pragma unroll
            for (int n = 0; n < NT; ++n) {
                mine[r * RS + 16 * (2 * j) + n] = o[n][0] * vRef;
                mine[r * RS + 16 * (2 * j + 1) + n] = o[n][1] * vRef;
            }
            if (j == 0) { mine[r * RS + HD] = m0; mine[r * RS + HD + 1] = l0; }
        }
        if (UPPER && r + 8 < G) {
#pragma unroll
            for (int n = 0; n < NT; ++n) {
                mine[(r + 8) * RS + 16 * (2 * j) + n] = o[n][2] * vRef;
                mine[(r + 8) * RS + 16 * (2 * j + 1) + n] = o[n][3] * vRef;
            }
            if (j == 0) { mine[(r + 8) * RS + HD] = m1; mine[(r + 8) * RS + HD + 1] = l1; }
        }
    }
    __syncthreads();
    finishSplit<__half, HD, NW>(red, G, work, heads, kvHeads, maxSplits, out, workspace, counters);
}

// Combine the splits of one (sequence, head): out = sum_s 2^(m_s - M) O_s / sum_s 2^(m_s - M) l_s.
template <typename T, int HD>
__global__ void decodeMergeKernel(const float* __restrict__ workspace, const uint32_t* __restrict__ lens,
                                  T* __restrict__ out, int heads, int blockSize, int maxNumBlocks,
                                  int window, int chunkTiles, int maxSplits) {
    constexpr int RS = HD + 2;
    const int head = blockIdx.x, b = blockIdx.y;
    const SplitInfo si = splitInfo(lens[b], window, maxNumBlocks * blockSize);
    const int numSplits = si.numTiles > 0 ? splitCount(si.numTiles, chunkTiles) : 0;
    if (numSplits <= 1) return;                       // written by the decode kernel itself
    const float* part = workspace + (static_cast<int64_t>(b) * heads + head) * maxSplits * RS;
    float M = -INFINITY;
    for (int s = 0; s < numSplits; ++s) M = fmaxf(M, part[s * RS + HD]);
    for (int d = threadIdx.x; d < HD; d += blockDim.x) {
        float acc = 0.f, lsum = 0.f;
        for (int s = 0; s < numSplits; ++s) {
            const float wgt = exp2f(part[s * RS + HD] - M);
            acc += wgt * part[s * RS + d];
            lsum += wgt * part[s * RS + HD + 1];
        }
        out[(static_cast<int64_t>(b) * heads + head) * HD + d] = fromFloat<T>(acc / lsum);
    }
}

// ------------------------------------------------------------ general kernel

// dequant_fp8 (kernels.metal:553-562): every product rounded to half.
__device__ __forceinline__ float dequantE4m3(uint8_t v, __half scale) {
    const int e = (v >> 3) & 0xF, m = v & 7;
    if (e == 0 && m == 0) return 0.f;
    const __half ss = (v & 0x80) ? __hneg(scale) : scale;
    const __half frac = __float2half_rn(static_cast<float>(m) * 0.125f);
    if (e == 0) return __half2float(__hmul(__hmul(ss, frac), __float2half_rn(0.015625f)));
    const __half t = __hmul(ss, __hadd(__float2half_rn(1.0f), frac));
    return __half2float(__hmul(t, __float2half_rn(exp2f(static_cast<float>(e - 7)))));
}

template <typename QT, typename KT>
__global__ void __launch_bounds__(128)
decodeGeneralKernel(const QT* __restrict__ q, const KT* __restrict__ kPool, const KT* __restrict__ vPool,
                    const int32_t* __restrict__ tables, const uint32_t* __restrict__ lens,
                    QT* __restrict__ out, const __half* __restrict__ kScale,
                    const __half* __restrict__ vScale, int heads, int kvHeads, int headDim,
                    int blockSize, int maxNumBlocks, int window, int poolBlocks) {
    constexpr int TB = 16, GMAX = 8, DPT = 2;
    extern __shared__ __align__(128) unsigned char smem[];
    const int kvh = blockIdx.x, b = blockIdx.y, tid = threadIdx.x;
    const int G = heads / kvHeads, D = headDim;
    float* sq = reinterpret_cast<float*>(smem);       // [GMAX][D]
    float* sk = sq + GMAX * D;                        // [TB][D]
    float* sv = sk + TB * D;                          // [TB][D]
    float* ss = sv + TB * D;                          // [GMAX][TB]
    float* sm = ss + GMAX * TB;                       // m, l, corr: [3][GMAX]
    const uint32_t len = lens[b];
    uint32_t L = len;
    if (L > static_cast<uint32_t>(maxNumBlocks) * blockSize) L = static_cast<uint32_t>(maxNumBlocks) * blockSize;
    const uint32_t ws = (window > 0 && len > static_cast<uint32_t>(window)) ? len - window : 0;
    const float scale = 1.0f / sqrtf(static_cast<float>(D));          // kernels.metal:1441
    const int32_t* table = tables + static_cast<int64_t>(b) * maxNumBlocks;

    for (int g0 = 0; g0 < G; g0 += GMAX) {
        const int gn = min(GMAX, G - g0);
        __syncthreads();
        for (int i = tid; i < gn * D; i += 128)
            sq[i] = toFloat(q[(static_cast<int64_t>(b) * heads + kvh * G + g0) * D + i]);
        if (tid < GMAX) { sm[tid] = -INFINITY; sm[GMAX + tid] = 0.f; sm[2 * GMAX + tid] = 0.f; }
        float acc[GMAX][DPT];
#pragma unroll
        for (int g = 0; g < GMAX; ++g)
#pragma unroll
            for (int i = 0; i < DPT; ++i) acc[g][i] = 0.f;

        for (uint32_t j0 = ws; j0 < L; j0 += TB) {
            const int nt = static_cast<int>(min(static_cast<uint32_t>(TB), L - j0));
            __syncthreads();
            for (int i = tid; i < nt * D; i += 128) {
                const int t = i / D, d = i - t * D;
                const uint32_t tok = j0 + t;
                const int64_t blk = min(max(table[tok / blockSize], 0), poolBlocks - 1);
                const int64_t off = ((blk * kvHeads + kvh) * blockSize + tok % blockSize) * static_cast<int64_t>(D) + d;
                if constexpr (sizeof(KT) == 1) {
                    sk[i] = dequantE4m3(kPool[off], kScale[blk * kvHeads + kvh]);
                    sv[i] = dequantE4m3(vPool[off], vScale[blk * kvHeads + kvh]);
                } else {
                    sk[i] = toFloat(kPool[off]);
                    sv[i] = toFloat(vPool[off]);
                }
            }
            __syncthreads();
            for (int i = tid; i < gn * nt; i += 128) {
                const int g = i / nt, t = i - g * nt;
                float dot = 0.f;
                for (int d = 0; d < D; ++d) dot += sq[g * D + d] * sk[t * D + d];
                ss[g * TB + t] = dot * scale;
            }
            __syncthreads();
            if (tid < gn) {
                const int g = tid;
                float m = sm[g], mx = m;
                for (int t = 0; t < nt; ++t) mx = fmaxf(mx, ss[g * TB + t]);
                const float corr = expf(m - mx);
                float sum = 0.f;
                for (int t = 0; t < nt; ++t) {
                    const float p = expf(ss[g * TB + t] - mx);
                    ss[g * TB + t] = p;
                    sum += p;
                }
                sm[g] = mx;
                sm[GMAX + g] = sm[GMAX + g] * corr + sum;
                sm[2 * GMAX + g] = corr;
            }
            __syncthreads();
#pragma unroll
            for (int i = 0; i < DPT; ++i) {
                const int d = tid + 128 * i;
                if (d < D) {
#pragma unroll
                    for (int g = 0; g < GMAX; ++g) {
                        if (g < gn) {
                            float a = acc[g][i] * sm[2 * GMAX + g];
                            for (int t = 0; t < nt; ++t) a += ss[g * TB + t] * sv[t * D + d];
                            acc[g][i] = a;
                        }
                    }
                }
            }
        }
        __syncthreads();
#pragma unroll
        for (int i = 0; i < DPT; ++i) {
            const int d = tid + 128 * i;
            if (d < D) {
#pragma unroll
                for (int g = 0; g < GMAX; ++g) {
                    if (g < gn) {
                        const float l = sm[GMAX + g];
                        // An empty context is 0/0 in the reference; zeros here.
                        const float v = l > 0.f ? acc[g][i] / l : 0.f;
                        out[(static_cast<int64_t>(b) * heads + kvh * G + g0 + g) * D + d] = fromFloat<QT>(v);
                    }
                }
            }
        }
    }
}

// ---------------------------------------------------------------- launch plan

struct SplitPlan {
    bool fast;
    int chunkTiles, maxSplits;
    const int4* items;      // work list on the device (host-planned launches), else null
    int numItems;
};

constexpr int kWarps = 4, kStages = 3, kStagesFp8 = 4;

bool fastPathApplies(const DecodeParams& p) {
    const int G = p.kvHeads > 0 ? p.heads / p.kvHeads : 0;
    const bool shape = p.headDim > 0 && p.blockSize % kTileTokens == 0 && G >= 1 && G <= 16;
    // the split kernels copy pages with 16-byte cp.async and read the query rows as 4-byte
    // (FP8: 8-byte) words; anything less aligned goes to the general kernel
    const auto aligned = [](const void* ptr, uintptr_t a) { return (reinterpret_cast<uintptr_t>(ptr) & (a - 1)) == 0; };
    if (!shape || !aligned(p.kPool, 16) || !aligned(p.vPool, 16) || !aligned(p.out, 2)) return false;
    if (p.dtype == kF16 || p.dtype == kBF16) return (p.headDim == 128 || p.headDim == 64) && aligned(p.q, 4);
    if (p.dtype == kFP8) return p.headDim == 128 && p.kScale && p.vScale && aligned(p.q, 8) && aligned(p.kScale, 2) && aligned(p.vScale, 2);
    return false;
}

// CTAs of the split kernel an SM holds at once (bounded by shared memory).
int residentCtas(const DecodeParams& p) {
    if (p.dtype == kFP8) return 3;
    return p.headDim == 64 ? 4 : 2;
}

int maxTilesOf(const DecodeParams& p) {
    int maxTokens = p.maxNumBlocks * p.blockSize;
    if (p.maxContext > 0 && p.maxContext < maxTokens) maxTokens = p.maxContext;
    if (p.window > 0 && p.window + kTileTokens < maxTokens) maxTokens = p.window + kTileTokens;
    return (maxTokens + kTileTokens - 1) / kTileTokens;
}

// Lengths unknown on the host: one chunk size for the whole batch from the longest
// context the tables can hold.
SplitPlan planSplits(const DecodeParams& p, int smCount) {
    SplitPlan plan{false, 0, 1, nullptr, 0};
    plan.fast = fastPathApplies(p);
    if (!plan.fast) return plan;
    const int maxTiles = maxTilesOf(p);
    // Enough CTAs to fill the machine several times over, but no chunk shorter
    // than two tiles per warp.
    const int64_t pairs = static_cast<int64_t>(p.batch) * p.kvHeads;
    const int64_t wantCtas = static_cast<int64_t>(smCount) * 8;
    int chunk = 64 * kWarps / 4;                                 // 64 tiles = 1024 tokens
    while (chunk > 2 * kWarps && pairs * ((maxTiles + chunk - 1) / chunk) < wantCtas) chunk /= 2;
    plan.chunkTiles = chunk;
    plan.maxSplits = (maxTiles + chunk - 1) / chunk;
    if (plan.maxSplits < 1) plan.maxSplits = 1;
    return plan;
}

}  // namespace

// Work list of a decode whose lengths the host knows, kept between calls: most decode
// steps leave every sequence's tile count as it was, and the list on the device is then
// used again without any upload.
struct DecodePlanCache {
    static constexpr int kRing = 4;
    int device = -1;
    // what the list was built from
    std::vector<int> geometry;            // (first tile, tiles) per sequence
    int kvHeads = 0, slots = 0, waves = 0;
    // the list
    int chunkTiles = 0, maxSplits = 1, numItems = 0;
    std::vector<int4> host;
    int4* dev = nullptr;
    size_t devCap = 0;
    // page-locked staging, one slot per upload in flight
    int4* pinned[kRing] = {};
    size_t pinnedCap[kRing] = {};
    cudaEvent_t ev[kRing] = {};
    int next = 0;
    ~DecodePlanCache() {
        if (device < 0) return;
        int prev = -1;
        cudaGetDevice(&prev);
        cudaSetDevice(device);
        if (dev) cudaFree(dev);
        for (int i = 0; i < kRing; ++i) {
            if (pinned[i]) cudaFreeHost(pinned[i]);
            if (ev[i]) cudaEventDestroy(ev[i]);
        }
        if (prev >= 0) cudaSetDevice(prev);
    }
};

DecodePlanCache* createDecodePlanCache() { return new DecodePlanCache(); }
void destroyDecodePlanCache(DecodePlanCache* c) { delete c; }

namespace {

int planWaves() {
    // CTAs per resident slot the work list aims at (PAM_DECODE_WAVES overrides, for tuning runs)
    static const int waves = [] {
        const char* e = std::getenv("PAM_DECODE_WAVES");
        const int v = e ? std::atoi(e) : 0;
        return v > 0 ? v : 2;
    }();
    return waves;
}

// Builds (or finds unchanged) the work list for `p` from the host copy of the lengths and
// makes sure it is on the device.  The upload is ordered on `stream` before the launch.
cudaError_t planFromLengths(const DecodeParams& p, int smCount, cudaStream_t stream, SplitPlan& plan) {
    DecodePlanCache& c = *p.planCache;
    plan = SplitPlan{true, 0, 1, nullptr, 0};
    const int maxTokens = p.maxNumBlocks * p.blockSize;
    const int slots = smCount * residentCtas(p), waves = planWaves();
    std::vector<int> geometry(static_cast<size_t>(p.batch) * 2);
    int64_t totalTiles = 0;
    for (int b = 0; b < p.batch; ++b) {
        const uint32_t len = p.hostLens[b];
        uint32_t L = len < static_cast<uint32_t>(maxTokens) ? len : static_cast<uint32_t>(maxTokens);
        int ws = (p.window > 0 && len > static_cast<uint32_t>(p.window)) ? static_cast<int>(len) - p.window : 0;
        if (ws > static_cast<int>(L)) ws = static_cast<int>(L);
        const int first = ws / kTileTokens;
        const int tiles = (static_cast<int>(L) + kTileTokens - 1) / kTileTokens - first;
        geometry[2 * b] = first;
        geometry[2 * b + 1] = tiles;
        totalTiles += tiles > 0 ? tiles : 0;
    }
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    const bool same = c.device == dev && c.kvHeads == p.kvHeads && c.slots == slots && c.waves == waves &&
                      c.geometry == geometry && c.dev != nullptr;
    if (!same) {
        if (c.device >= 0 && c.device != dev) return cudaErrorInvalidDevice;   // one cache belongs to one GPU
        c.device = dev;
        // chunk: about `waves` CTAs per resident slot, between two tiles per warp and 1024 tokens
        int64_t chunk = totalTiles * p.kvHeads / (static_cast<int64_t>(slots) * waves);
        if (chunk < 2 * kWarps) chunk = 2 * kWarps;
        if (chunk > 64) chunk = 64;
        c.chunkTiles = static_cast<int>(chunk);
        c.maxSplits = 1;
        // ranges by decreasing size (counting sort; a range has at most `chunk` tiles)
        std::vector<int> count(static_cast<size_t>(chunk) + 2, 0);
        int items = 0;
        for (int b = 0; b < p.batch; ++b) {
            const int tiles = geometry[2 * b + 1];
            const int n = tiles > 0 ? splitCount(tiles, c.chunkTiles) : 1;
            if (n > c.maxSplits) c.maxSplits = n;
            if (n > 0x7FFF) return cudaErrorInvalidValue;
            for (int k = 0; k < n; ++k) {
                int begin = 0, end = 0;
                if (tiles > 0) splitRange(tiles, n, k, begin, end);
                count[static_cast<size_t>(end - begin)] += 1;
                ++items;
            }
        }
        std::vector<int> start(count.size(), 0);
        for (int sz = static_cast<int>(chunk); sz >= 0; --sz) start[static_cast<size_t>(sz)] = start[static_cast<size_t>(sz) + 1] + count[static_cast<size_t>(sz) + 1];
        c.host.assign(static_cast<size_t>(items), int4{0, 0, 0, 0});
        for (int b = 0; b < p.batch; ++b) {
            const int first = geometry[2 * b], tiles = geometry[2 * b + 1];
            const int n = tiles > 0 ? splitCount(tiles, c.chunkTiles) : 1;
            for (int k = 0; k < n; ++k) {
                int begin = 0, end = 0;
                if (tiles > 0) splitRange(tiles, n, k, begin, end);
                c.host[static_cast<size_t>(start[static_cast<size_t>(end - begin)]++)] = int4{b, first + begin, first + end, k | (n << 16)};
            }
        }
        c.numItems = items;
        if (static_cast<size_t>(items) > c.devCap) {
            if (c.dev) { cudaStreamSynchronize(stream); cudaFree(c.dev); c.dev = nullptr; c.devCap = 0; }
            const size_t cap = static_cast<size_t>(items) + static_cast<size_t>(items) / 2 + 64;
            e = cudaMalloc(reinterpret_cast<void**>(&c.dev), cap * sizeof(int4));
            if (e != cudaSuccess) { c.dev = nullptr; return e; }
            c.devCap = cap;
        }
        const int slot = c.next;
        c.next = (c.next + 1) % DecodePlanCache::kRing;
        if (!c.ev[slot]) {
            e = cudaEventCreateWithFlags(&c.ev[slot], cudaEventDisableTiming);
            if (e != cudaSuccess) return e;
        } else {
            e = cudaEventSynchronize(c.ev[slot]);           // the upload that last used this slot has been read
            if (e != cudaSuccess) return e;
        }
        if (static_cast<size_t>(items) > c.pinnedCap[slot]) {
            if (c.pinned[slot]) cudaFreeHost(c.pinned[slot]);
            c.pinned[slot] = nullptr;
            c.pinnedCap[slot] = 0;
            e = cudaHostAlloc(reinterpret_cast<void**>(&c.pinned[slot]), c.devCap * sizeof(int4), cudaHostAllocDefault);
            if (e != cudaSuccess) { c.pinned[slot] = nullptr; return e; }
            c.pinnedCap[slot] = c.devCap;
        }
        std::memcpy(c.pinned[slot], c.host.data(), static_cast<size_t>(items) * sizeof(int4));
        e = cudaMemcpyAsync(c.dev, c.pinned[slot], static_cast<size_t>(items) * sizeof(int4), cudaMemcpyHostToDevice, stream);
        if (e == cudaSuccess) e = cudaEventRecord(c.ev[slot], stream);
        if (e != cudaSuccess) { c.geometry.clear(); return e; }
        c.geometry.swap(geometry);
        c.kvHeads = p.kvHeads; c.slots = slots; c.waves = waves;
    }
    plan.chunkTiles = c.chunkTiles;
    plan.maxSplits = c.maxSplits;
    plan.items = c.dev;
    plan.numItems = c.numItems;
    return cudaSuccess;
}

// Bytes of split-K partials of a plan.
size_t partialBytes(const DecodeParams& p, const SplitPlan& plan) {
    if (!plan.fast || plan.maxSplits <= 1) return 0;
    return static_cast<size_t>(p.batch) * p.heads * plan.maxSplits * (p.headDim + 2) * sizeof(float);
}

// The dynamic shared memory limit of a kernel is raised once per device, not per launch.
template <class K>
cudaError_t allowSharedMemory(K kernel, size_t bytes, std::atomic<size_t>* granted) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
    if (granted[dev].load(std::memory_order_acquire) >= bytes) return cudaSuccess;
    e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(bytes));
    if (e == cudaSuccess) granted[dev].store(bytes, std::memory_order_release);
    return e;
}

dim3 splitGrid(const DecodeParams& p, const SplitPlan& plan) {
    if (plan.items) return dim3(static_cast<unsigned>(plan.numItems), static_cast<unsigned>(p.kvHeads));
    return dim3(static_cast<unsigned>(plan.maxSplits), static_cast<unsigned>(p.kvHeads), static_cast<unsigned>(p.batch));
}

// The last CTA of a (sequence, kv head) merges its splits when the caller gave counters
// for every such pair; else the merge kernel follows.
bool mergeInKernel(const DecodeParams& p, const SplitPlan& plan) {
    // (the merging CTA keeps one weight per (head, split) in its shared memory: 48 KB of the ring's space)
    const int64_t G = p.heads / p.kvHeads;
    return plan.maxSplits > 1 && p.counters && static_cast<int64_t>(p.batch) * p.kvHeads <= p.countersCap &&
           (G * plan.maxSplits + G) * static_cast<int64_t>(sizeof(float)) <= 48 * 1024;
}

template <typename T, int HD>
cudaError_t launchMerge(const DecodeParams& p, const SplitPlan& plan, cudaStream_t stream, int* launches) {
    dim3 mgrid(static_cast<unsigned>(p.heads), static_cast<unsigned>(p.batch));
    decodeMergeKernel<T, HD><<<mgrid, HD, 0, stream>>>(p.workspace, p.lens, static_cast<T*>(p.out), p.heads,
                                                      p.blockSize, p.maxNumBlocks, p.window, plan.chunkTiles,
                                                      plan.maxSplits);
    cudaError_t e = cudaGetLastError();
    if (e == cudaSuccess && launches) *launches += 1;
    return e;
}

template <typename T, int HD, bool UPPER>
cudaError_t launchFast(const DecodeParams& p, const SplitPlan& plan, cudaStream_t stream, int* launches) {
    constexpr int NW = kWarps, NS = kStages;
    static std::atomic<size_t> granted[64];
    const int G = p.heads / p.kvHeads;
    size_t ring = static_cast<size_t>(NW) * NS * 2 * kTileTokens * HD * 2;
    size_t red = static_cast<size_t>(NW) * G * (HD + 2) * sizeof(float);
    size_t smem = ring > red ? ring : red;
    auto kernel = decodeSplitKernel<T, HD, NW, NS, UPPER>;
    cudaError_t e = allowSharedMemory(kernel, smem, granted);
    if (e != cudaSuccess) return e;
    const bool fused = mergeInKernel(p, plan);
    const float scaleLog2 = (1.0f / sqrtf(static_cast<float>(p.headDim))) * kLog2e;
    kernel<<<splitGrid(p, plan), NW * 32, smem, stream>>>(static_cast<const T*>(p.q), static_cast<const T*>(p.kPool),
                                                          static_cast<const T*>(p.vPool), p.tables, p.lens,
                                                          static_cast<T*>(p.out), p.workspace, p.heads, p.kvHeads,
                                                          p.blockSize, p.maxNumBlocks, p.window, plan.chunkTiles,
                                                          plan.maxSplits, scaleLog2, p.poolBlocks, plan.items,
                                                          fused ? p.counters : nullptr);
    e = cudaGetLastError();
    if (e != cudaSuccess) return e;
    if (launches) *launches += 1;
    if (plan.maxSplits > 1 && !fused) e = launchMerge<T, HD>(p, plan, stream, launches);
    return e;
}

template <bool UPPER>
cudaError_t launchFastFp8(const DecodeParams& p, const SplitPlan& plan, cudaStream_t stream, int* launches) {
    constexpr int NW = kWarps, NS = kStagesFp8, HD = 128;
    static std::atomic<size_t> granted[64];
    const int G = p.heads / p.kvHeads;
    size_t ring = static_cast<size_t>(NW) * NS * (2 * kTileTokens * HD + 16);
    size_t red = static_cast<size_t>(NW) * G * (HD + 2) * sizeof(float);
    size_t smem = ring > red ? ring : red;
    auto kernel = decodeSplitFp8Kernel<NW, NS, UPPER>;
    cudaError_t e = allowSharedMemory(kernel, smem, granted);
    if (e != cudaSuccess) return e;
    const bool fused = mergeInKernel(p, plan);
    const float scaleLog2 = (1.0f / sqrtf(static_cast<float>(p.headDim))) * kLog2e;
    kernel<<<splitGrid(p, plan), NW * 32, smem, stream>>>(static_cast<const __half*>(p.q), static_cast<const uint8_t*>(p.kPool),
                                                          static_cast<const uint8_t*>(p.vPool), static_cast<const __half*>(p.kScale),
                                                          static_cast<const __half*>(p.vScale), p.tables, p.lens,
                                                          static_cast<__half*>(p.out), p.workspace, p.heads, p.kvHeads, p.blockSize,
                                                          p.maxNumBlocks, p.window, plan.chunkTiles, plan.maxSplits, scaleLog2,
                                                          p.poolBlocks, plan.items, fused ? p.counters : nullptr);
    e = cudaGetLastError();
    if (e != cudaSuccess) return e;
    if (launches) *launches += 1;
    if (plan.maxSplits > 1 && !fused) e = launchMerge<__half, HD>(p, plan, stream, launches);
    return e;
}

template <typename T>
cudaError_t launchFastT(const DecodeParams& p, const SplitPlan& plan, cudaStream_t stream, int* launches) {
    const bool upper = p.heads / p.kvHeads > 8;
    if (p.headDim == 128)
        return upper ? launchFast<T, 128, true>(p, plan, stream, launches)
                     : launchFast<T, 128, false>(p, plan, stream, launches);
    return upper ? launchFast<T, 64, true>(p, plan, stream, launches)
                 : launchFast<T, 64, false>(p, plan, stream, launches);
}

template <typename QT, typename KT>
cudaError_t launchGeneral(const DecodeParams& p, cudaStream_t stream, int* launches) {
    static std::atomic<size_t> granted[64];
    const size_t smem = (static_cast<size_t>(8 + 2 * 16) * p.headDim + 8 * 16 + 3 * 8) * sizeof(float);
    auto kernel = decodeGeneralKernel<QT, KT>;
    cudaError_t e = allowSharedMemory(kernel, smem, granted);
    if (e != cudaSuccess) return e;
    dim3 grid(static_cast<unsigned>(p.kvHeads), static_cast<unsigned>(p.batch));
    kernel<<<grid, 128, smem, stream>>>(static_cast<const QT*>(p.q), static_cast<const KT*>(p.kPool),
                                        static_cast<const KT*>(p.vPool), p.tables, p.lens,
                                        static_cast<QT*>(p.out), static_cast<const __half*>(p.kScale),
                                        static_cast<const __half*>(p.vScale), p.heads, p.kvHeads,
                                        p.headDim, p.blockSize, p.maxNumBlocks, p.window, p.poolBlocks);
    if (launches) *launches += 1;
    return cudaGetLastError();
}

cudaError_t makePlan(const DecodeParams& p, int smCount, cudaStream_t stream, SplitPlan& plan) {
    if (p.hostLens && p.planCache && fastPathApplies(p)) return planFromLengths(p, smCount, stream, plan);
    plan = planSplits(p, smCount);
    return cudaSuccess;
}

}  // namespace

namespace {
// (tuning runs only: PAM_DECODE_STREAM=0 takes the grid-per-split kernels instead of the stream kernel)
bool streamEnabled() {
    static const bool on = [] {
        const char* e = std::getenv("PAM_DECODE_STREAM");
        return !(e && e[0] == '0');
    }();
    return on;
}
bool takesStream(const DecodeParams& p) { return streamEnabled() && decodeStreamApplies(p); }
}  // namespace

bool decodeTakesSplitPath(const DecodeParams& p) { return decodeStreamApplies(p) || fastPathApplies(p); }

size_t decodeWorkspaceBytes(const DecodeParams& p, int smCount, cudaStream_t stream) {
    if (takesStream(p)) return decodeStreamWorkspaceBytes(p, smCount);
    SplitPlan plan{};
    if (makePlan(p, smCount, stream, plan) != cudaSuccess) { cudaGetLastError(); return 0; }
    return partialBytes(p, plan);
}

cudaError_t launchDecode(const DecodeParams& p, int smCount, cudaStream_t stream, int* launches) {
    if (p.batch <= 0) return cudaSuccess;
    if (p.headDim > 256 || p.poolBlocks <= 0) return cudaErrorInvalidValue;
    if (takesStream(p) && p.workspace && p.counters && static_cast<int64_t>(p.batch) * p.kvHeads <= p.countersCap)
        return launchDecodeStream(p, smCount, stream, launches);
    SplitPlan plan{};
    cudaError_t pe = makePlan(p, smCount, stream, plan);
    if (pe != cudaSuccess) return pe;
    if (plan.fast) {
        if (plan.maxSplits > 1 && (!p.workspace || p.workspaceBytes < partialBytes(p, plan)))
            return cudaErrorInvalidValue;
        if (p.dtype == kFP8)
            return p.heads / p.kvHeads > 8 ? launchFastFp8<true>(p, plan, stream, launches)
                                           : launchFastFp8<false>(p, plan, stream, launches);
        return p.dtype == kF16 ? launchFastT<__half>(p, plan, stream, launches)
                               : launchFastT<__nv_bfloat16>(p, plan, stream, launches);
    }
    switch (p.dtype) {
        case kF32: return launchGeneral<float, float>(p, stream, launches);
        case kF16: return launchGeneral<__half, __half>(p, stream, launches);
        case kBF16: return launchGeneral<__nv_bfloat16, __nv_bfloat16>(p, stream, launches);
        case kFP8: return launchGeneral<__half, uint8_t>(p, stream, launches);
    }
    return cudaErrorInvalidValue;
}

cudaError_t launchDecodeStatic(const DecodeParams& p, int smCount, cudaStream_t stream, int* launches) {
    // The scratch array and the arrival words are part of the library image on every GPU;
    // their device addresses are looked up once per device (decodeStaticScratch).
    float* scratch = nullptr;
    int* counters = nullptr;
    int64_t countersCap = 0;
    cudaError_t e = decodeStaticScratch(&scratch, &counters, &countersCap);
    if (e != cudaSuccess) return e;
    DecodeParams q = p;
    q.hostLens = nullptr;      // nothing here may depend on a cache that allocates
    q.planCache = nullptr;
    q.workspace = scratch;
    q.workspaceBytes = decodeStaticScratchBytes();
    q.counters = counters;
    q.countersCap = countersCap;
    if (takesStream(q)) {
        // the stream kernel sizes its grid to the scratch it is given; the arrival words bound the batch
        if (static_cast<int64_t>(q.batch) * q.kvHeads > countersCap) return cudaErrorInvalidValue;
        return launchDecodeStream(q, smCount, stream, launches);
    }
    q.counters = nullptr;
    q.countersCap = 0;
    if (decodeWorkspaceBytes(q, smCount, stream) > decodeStaticScratchBytes()) return cudaErrorInvalidValue;
    return launchDecode(q, smCount, stream, launches);
}

}  // namespace pam
