// Batched paged decode as one persistent stream of key/value tiles.
//
// Semantics: paged_decode_single / _f16 / _fp8 (kernels.metal:1417-1620): per (sequence,
// query head) softmax(q.K^T / sqrt(dim)) V over tokens [window_start, L) reached through the
// block table, float32 accumulation.  Pools are [block][kv_head][block_size][head_dim].
//
// The work of a launch is the list of 16-token tiles of all (sequence, kv head) pairs, laid
// end to end: sequence after sequence, kv head after kv head, tile after tile.  Every warp of
// the grid (one CTA per resident slot, four warps each) takes one contiguous piece of that
// list, all pieces the same length, found from a prefix sum of the sequences' tile counts
// that each CTA builds in shared memory from the lengths.  A warp streams its piece through
// its own cp.async ring (K tile + V tile per stage, XOR-swizzled 16-byte chunks) without a
// pause at the borders between sequences: the loads run ahead of the arithmetic across
// them.  Nothing in the kernel waits for another warp.
//
// A (sequence, kv head) pair that lies inside one warp's piece gets its output from that
// warp.  A pair that several warps share gets one partial result (m, l, O per query head)
// from each of them in a workspace, at a place fixed by the piece's number; every warp adds
// its tiles of the pair to the pair's counting word, and the warp that completes the count
// combines the partials, in the order of the pieces, with a log-sum-exp reduction and puts
// the word back to zero.  Equal inputs therefore give equal bits, whatever the timing.
// (A variant in which a warp that is through takes the rest of another warp's piece was
// measured and dropped: the warps finish apart because they share the memory system
// unevenly, not because their pieces differ, and taking work did not shorten a launch.)
//
// Arithmetic per tile: mma.sync m16n8k16 with the query heads of the GQA group as rows (every
// K/V byte is read once for the whole group), online softmax in registers in the log2
// domain; FP8 e4m3 codes become float16 in registers and the (block, kv_head) scales are
// applied outside the products.  FP8 pools with at most 8 query heads per KV head take the
// products transposed (tokens and dims as rows, heads as the 8 columns), which wastes no row
// of a product on padding.  The kernel is bound by HBM bandwidth.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <algorithm>
#include <atomic>
#include <cmath>
#include <type_traits>

#include "kernels.h"

namespace pam {
namespace {

constexpr int kTileTokens = 16;
constexpr int kWarps = 4;
constexpr float kLog2e = 1.4426950408889634f;
constexpr int kShortContextKeys = 256;
// The running maximum of a row is only raised when a tile exceeds it by more than this
// (log2 domain): the result is the same either way because the final division uses the
// same reference, and the accumulator is then rescaled a few times per sequence instead of
// once per tile.  Weights reach at most 2^kLazyMax, well inside float16.
constexpr float kLazyMax = 6.0f;

// Records of shared pairs and counting words for launchDecodeStatic(): device memory that belongs
// to the library image itself, so that a decode can run without any allocation call.  Every
// GPU that loads the library holds them until the process exits.
constexpr size_t kStaticScratchBytes = size_t(8) << 20;
constexpr int kStaticCounters = 1 << 16;
static __device__ __align__(256) float gStaticDecodeScratch[kStaticScratchBytes / sizeof(float)];
static __device__ __align__(256) int gStaticDecodeCounters[kStaticCounters];

// ---------------------------------------------------------------- PTX helpers

__device__ __forceinline__ uint32_t smemAddr(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }
__device__ __forceinline__ void cpAsync16(uint32_t dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(dst), "l"(src));
}
__device__ __forceinline__ void cpAsync4(uint32_t dst, const void* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" ::"r"(dst), "l"(src));
}
__device__ __forceinline__ void cpAsyncCommit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cpAsyncWait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

__device__ __forceinline__ void ldmatrixX4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrixX4Trans(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}

template <typename T>
__device__ __forceinline__ void mma16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1);
template <>
__device__ __forceinline__ void mma16816<__half>(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
template <>
__device__ __forceinline__ void mma16816<__nv_bfloat16>(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

template <typename T> __device__ __forceinline__ uint32_t pack2(float lo, float hi);
template <> __device__ __forceinline__ uint32_t pack2<__half>(float lo, float hi) {
    __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&h);
}
template <> __device__ __forceinline__ uint32_t pack2<__nv_bfloat16>(float lo, float hi) {
    __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&h);
}
// The two 16-bit halves of a packed bfloat16 pair, widened.
__device__ __forceinline__ float bf16Low(uint32_t v) { return __uint_as_float(v << 16); }
__device__ __forceinline__ float bf16High(uint32_t v) { return __uint_as_float(v & 0xFFFF0000u); }

template <typename T> __device__ __forceinline__ T fromFloat(float v);
template <> __device__ __forceinline__ __half fromFloat<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 fromFloat<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// 2^x by the special-function unit alone (exp2f adds a range fix-up for results below the
// normal range, which a softmax weight does not need); 2^-inf = 0.
__device__ __forceinline__ float ex2Fast(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
// Two e4m3 codes (low or high 16 bits of `v`) to two float16 values; exact, every e4m3 value
// is a float16 value.
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

// Visible tiles of a sequence.
struct Visible {
    int firstTile;   // first 16-token tile that holds a visible token
    int numTiles;    // tiles from there to the end of the sequence
    int windowStart; // first visible token
};
__device__ __forceinline__ Visible visibleOf(uint32_t len, int window, int maxTokens) {
    Visible s;
    uint32_t L = len < static_cast<uint32_t>(maxTokens) ? len : static_cast<uint32_t>(maxTokens);
    s.windowStart = (window > 0 && len > static_cast<uint32_t>(window)) ? static_cast<int>(len) - window : 0;   // kernels.metal:1442
    if (s.windowStart > static_cast<int>(L)) s.windowStart = static_cast<int>(L);
    s.firstTile = s.windowStart / kTileTokens;
    s.numTiles = (static_cast<int>(L) + kTileTokens - 1) / kTileTokens - s.firstTile;
    if (s.numTiles < 0) s.numTiles = 0;
    return s;
}

struct StreamArgs {
    const void* q;
    const void* kPool;
    const void* vPool;
    const void* kScale;
    const void* vScale;
    const int32_t* tables;
    const uint32_t* lens;
    void* out;
    float* records;       // partial results, G x (HD + 4) floats each
    int* counters;        // [batch][kvHeads]: tiles of the pair whose partial result is in; zero between launches
    int batch, heads, kvHeads, blockSize, maxNumBlocks, window, poolBlocks;
    float scaleLog2;
};

// ------------------------------------------------------------ tile arithmetic
//
// A policy says how one kind of pool is streamed and multiplied: the bytes of a ring stage,
// how a tile is fetched, how the query rows sit in registers, what one tile does to the
// running (m, l, O), and how the result leaves the registers.

// float16 / bfloat16 pools, head_dim 64 or 128.
template <typename T, int HD_, bool UPPER>
struct HalfTiles {
    using Out = T;
    static constexpr int HD = HD_, NS = 3;
    static constexpr int ROWB = HD * 2, CPR = ROWB / 16, TILEB = kTileTokens * ROWB, CHUNKS = TILEB / 16;
    static constexpr int STAGEB = 2 * TILEB, KSTEPS = HD / 16, NT = HD / 8;
    static constexpr bool kBf16 = sizeof(T) == 2 && !std::is_same<T, __half>::value;
    struct Query { uint32_t a[KSTEPS][4]; };
    struct Acc {
        float o[NT][4];
        float m0, m1, l0, l1;
        bool twoPart;        // bfloat16, few visible keys: weights as two operands (16 bits)
    };

    static __device__ __forceinline__ void issue(uint32_t stage, unsigned char*, const StreamArgs& a, int64_t blk, int kvh,
                                                 int within, int lane) {
        const int64_t off = ((blk * a.kvHeads + kvh) * a.blockSize + within * kTileTokens) * static_cast<int64_t>(ROWB);
        const unsigned char* gk = static_cast<const unsigned char*>(a.kPool) + off;
        const unsigned char* gv = static_cast<const unsigned char*>(a.vPool) + off;
#pragma unroll
        for (int i = 0; i < CHUNKS / 32; ++i) {
            const int idx = lane + 32 * i;
            const int row = idx / CPR, c = idx % CPR;
            const uint32_t dst = row * ROWB + ((c ^ (row & 7)) << 4);
            cpAsync16(stage + dst, gk + idx * 16);
            cpAsync16(stage + TILEB + dst, gv + idx * 16);
        }
    }

    // Query rows of a GQA group as A fragments (rows >= G are zero).
    static __device__ __forceinline__ void loadQuery(Query& q, const StreamArgs& a, int64_t row0, int G, int lane) {
        const int r = lane >> 2, j = lane & 3;
        const T* qb = static_cast<const T*>(a.q) + row0 * HD;
#pragma unroll
        for (int ks = 0; ks < KSTEPS; ++ks) {
            const int d0 = ks * 16 + 2 * j;
            q.a[ks][0] = r < G ? *reinterpret_cast<const uint32_t*>(qb + r * HD + d0) : 0u;
            q.a[ks][2] = r < G ? *reinterpret_cast<const uint32_t*>(qb + r * HD + d0 + 8) : 0u;
            q.a[ks][1] = (UPPER && r + 8 < G) ? *reinterpret_cast<const uint32_t*>(qb + (r + 8) * HD + d0) : 0u;
            q.a[ks][3] = (UPPER && r + 8 < G) ? *reinterpret_cast<const uint32_t*>(qb + (r + 8) * HD + d0 + 8) : 0u;
        }
    }

    static __device__ __forceinline__ void reset(Acc& c, int visibleTokens) {
#pragma unroll
        for (int n = 0; n < NT; ++n) c.o[n][0] = c.o[n][1] = c.o[n][2] = c.o[n][3] = 0.f;
        c.m0 = c.m1 = -INFINITY;
        c.l0 = c.l1 = 0.f;
        // A bfloat16 weight keeps 8 significant bits.  A sequence with few visible keys has
        // large weights, and 8 bits alone can then miss the 2e-3 bound on unit-variance
        // values: such sequences carry every weight as two bfloat16 operands into a second
        // product.  With hundreds of keys the weights are small enough for 8 bits.
        c.twoPart = kBf16 && visibleTokens < kShortContextKeys;
    }

    static __device__ __forceinline__ void tile(Acc& c, const Query& q, unsigned char* stagePtr, uint32_t stage, int tokBase,
                                                int windowStart, int len, float scaleLog2, int lane) {
        const int j = lane & 3;
        const uint32_t sk = stage, sv = stage + TILEB;
        const bool partial = tokBase < windowStart || tokBase + kTileTokens > len;
        if (partial) {
            // Rows outside [window_start, L) may hold anything; zero their V so that a zero
            // probability times that row stays zero.
            unsigned char* vt = stagePtr + TILEB;
            for (int idx = lane; idx < CHUNKS; idx += 32) {
                const int tok = tokBase + idx / CPR;
                if (tok < windowStart || tok >= len) *reinterpret_cast<uint4*>(vt + idx * 16) = make_uint4(0u, 0u, 0u, 0u);
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
            mma16816<T>(s[0], q.a[ks], kb[0], kb[1]);
            mma16816<T>(s[1], q.a[ks], kb[2], kb[3]);
        }
        // Online softmax in the log2 domain.
        float tmax0 = -INFINITY, tmax1 = -INFINITY;
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int tok = tokBase + 8 * nt + 2 * j + e;
                const bool ok = !partial || (tok >= windowStart && tok < len);
                s[nt][e] = ok ? s[nt][e] * scaleLog2 : -INFINITY;
                tmax0 = fmaxf(tmax0, s[nt][e]);
                if (UPPER) {
                    s[nt][e + 2] = ok ? s[nt][e + 2] * scaleLog2 : -INFINITY;
                    tmax1 = fmaxf(tmax1, s[nt][e + 2]);
                }
            }
        }
        // With bfloat16 weights the maximum is followed exactly: only then is the largest
        // weight of a row exactly 1, which a row that one key dominates needs for the bound.
        constexpr float lazy = kBf16 ? 0.f : kLazyMax;
        tmax0 = fmaxf(tmax0, __shfl_xor_sync(0xFFFFFFFFu, tmax0, 1));
        tmax0 = fmaxf(tmax0, __shfl_xor_sync(0xFFFFFFFFu, tmax0, 2));
        bool raise = tmax0 > c.m0 + lazy;              // m0 = -inf: the first tile always raises
        float c0 = 1.f, c1 = 1.f;
        if (raise) { c0 = exp2f(c.m0 - tmax0); c.m0 = tmax0; }   // m0 = -inf gives 0
        if (UPPER) {
            tmax1 = fmaxf(tmax1, __shfl_xor_sync(0xFFFFFFFFu, tmax1, 1));
            tmax1 = fmaxf(tmax1, __shfl_xor_sync(0xFFFFFFFFu, tmax1, 2));
            if (tmax1 > c.m1 + lazy) { c1 = exp2f(c.m1 - tmax1); c.m1 = tmax1; raise = true; }
        }
        if (__any_sync(0xFFFFFFFFu, raise)) {
            c.l0 *= c0;
            if (UPPER) c.l1 *= c1;
#pragma unroll
            for (int n = 0; n < NT; ++n) {
                c.o[n][0] *= c0;
                c.o[n][1] *= c0;
                if (UPPER) {
                    c.o[n][2] *= c1;
                    c.o[n][3] *= c1;
                }
            }
        }
        uint32_t pa[4], pl[4] = {0u, 0u, 0u, 0u};
        {
            const float p00 = exp2f(s[0][0] - c.m0), p01 = exp2f(s[0][1] - c.m0);
            const float p10 = exp2f(s[1][0] - c.m0), p11 = exp2f(s[1][1] - c.m0);
            c.l0 += (p00 + p01) + (p10 + p11);
            pa[0] = pack2<T>(p00, p01);
            pa[2] = pack2<T>(p10, p11);
            if (kBf16 && c.twoPart) {
                pl[0] = pack2<T>(p00 - bf16Low(pa[0]), p01 - bf16High(pa[0]));
                pl[2] = pack2<T>(p10 - bf16Low(pa[2]), p11 - bf16High(pa[2]));
            }
            if (UPPER) {
                const float q00 = exp2f(s[0][2] - c.m1), q01 = exp2f(s[0][3] - c.m1);
                const float q10 = exp2f(s[1][2] - c.m1), q11 = exp2f(s[1][3] - c.m1);
                c.l1 += (q00 + q01) + (q10 + q11);
                pa[1] = pack2<T>(q00, q01);
                pa[3] = pack2<T>(q10, q11);
                if (kBf16 && c.twoPart) {
                    pl[1] = pack2<T>(q00 - bf16Low(pa[1]), q01 - bf16High(pa[1]));
                    pl[3] = pack2<T>(q10 - bf16Low(pa[3]), q11 - bf16High(pa[3]));
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
            mma16816<T>(c.o[2 * cp], pa, vb[0], vb[1]);
            mma16816<T>(c.o[2 * cp + 1], pa, vb[2], vb[3]);
            if (kBf16 && c.twoPart) {
                mma16816<T>(c.o[2 * cp], pl, vb[0], vb[1]);
                mma16816<T>(c.o[2 * cp + 1], pl, vb[2], vb[3]);
            }
        }
    }

    // Row sums live spread over the four lanes of a quad.
    static __device__ __forceinline__ void finish(Acc& c) {
        c.l0 += __shfl_xor_sync(0xFFFFFFFFu, c.l0, 1);
        c.l0 += __shfl_xor_sync(0xFFFFFFFFu, c.l0, 2);
        if (UPPER) {
            c.l1 += __shfl_xor_sync(0xFFFFFFFFu, c.l1, 1);
            c.l1 += __shfl_xor_sync(0xFFFFFFFFu, c.l1, 2);
        }
    }

    // f(row g, column d, value) for every accumulator element this lane holds, and
    // g(row, m, l) once per row.
    template <class F, class Gf>
    static __device__ __forceinline__ void each(const Acc& c, int G, int lane, F f, Gf g) {
        const int r = lane >> 2, j = lane & 3;
        if (r < G) {
#pragma unroll
            for (int n = 0; n < NT; ++n) f(r, 8 * n + 2 * j, c.o[n][0], c.o[n][1]);
            if (j == 0) g(r, c.m0, c.l0);
        }
        if (UPPER && r + 8 < G) {
#pragma unroll
            for (int n = 0; n < NT; ++n) f(r + 8, 8 * n + 2 * j, c.o[n][2], c.o[n][3]);
            if (j == 0) g(r + 8, c.m1, c.l1);
        }
    }
    static constexpr int kPairStride = 1;     // the two values handed to f are columns d and d + 1
    static __device__ __forceinline__ float rowSum(const Acc& c, int g) { return g >= 8 ? c.l1 : c.l0; }
};

// FP8 e4m3 pools with float16 (block, kv_head) scales, head_dim 128, float16 queries and
// outputs.  A 16-token tile is 2 KB of K codes and 2 KB of V codes.  Codes become float16 in
// registers (exactly) and feed mma.sync.m16n8k16.f16; the group scales are applied outside
// the products: K's on the scores, V's on the weights (relative to the scale of the first
// tile of the sequence this warp sees, so that the weights stay in float16's normal range).
// The fragments are loaded with 16-byte shared-memory reads: the K-dimension of QK^T and
// the N-dimension of PV are permuted so that every thread reads contiguous codes, which no
// result depends on.
template <bool UPPER>
struct Fp8Tiles {
    using Out = __half;
    static constexpr int HD = 128, NS = 4;
    static constexpr int ROWB = HD, TILEB = kTileTokens * ROWB, CHUNKS = TILEB / 16;
    static constexpr int STAGEB = 2 * TILEB + 16;   // + the words that hold the tile's two group scales
    static constexpr int KSTEPS = HD / 16, NT = HD / 8;
    struct Query { uint32_t a[KSTEPS][4]; };
    struct Acc {
        float o[NT][4];
        float m0, m1, l0, l1;
        float vRef, invVRef;     // V scale of the first tile
        bool first;
    };

    static __device__ __forceinline__ void issue(uint32_t stage, unsigned char* stagePtr, const StreamArgs& a, int64_t blk,
                                                 int kvh, int within, int lane) {
        const int64_t off = ((blk * a.kvHeads + kvh) * a.blockSize + within * kTileTokens) * static_cast<int64_t>(ROWB);
        const unsigned char* gk = static_cast<const unsigned char*>(a.kPool) + off;
        const unsigned char* gv = static_cast<const unsigned char*>(a.vPool) + off;
#pragma unroll
        for (int i = 0; i < CHUNKS / 32; ++i) {
            const int idx = lane + 32 * i;
            const int row = idx >> 3, c = idx & 7;
            const uint32_t dst = row * ROWB + ((c ^ (row & 7)) << 4);
            cpAsync16(stage + dst, gk + idx * 16);
            cpAsync16(stage + TILEB + dst, gv + idx * 16);
        }
        // the aligned words that hold the two float16 scales travel with the tile; which half
        // of a word is the scale follows from the parity of its index
        if (lane < 2) {
            const int64_t si = blk * a.kvHeads + kvh;
            const unsigned char* base = static_cast<const unsigned char*>(lane == 0 ? a.kScale : a.vScale);
            cpAsync4(stage + 2 * TILEB + 4 * lane, base + ((si * 2) & ~static_cast<int64_t>(3)));
            if (lane == 0) stagePtr[2 * TILEB + 8] = static_cast<unsigned char>(si & 1);
        }
    }

    // Query rows as A fragments with the permuted K order: step ks of thread (r, j) covers
    // dims 32j + 4ks + {0,1} (first half) and + {2,3} (second half).
    static __device__ __forceinline__ void loadQuery(Query& q, const StreamArgs& a, int64_t row0, int G, int lane) {
        const int r = lane >> 2, j = lane & 3;
        const __half* qb = static_cast<const __half*>(a.q) + row0 * HD;
#pragma unroll
        for (int ks = 0; ks < KSTEPS; ++ks) {
            const int d0 = 32 * j + 4 * ks;
            uint2 lo = make_uint2(0u, 0u), hi = make_uint2(0u, 0u);
            if (r < G) lo = *reinterpret_cast<const uint2*>(qb + r * HD + d0);
            if (UPPER && r + 8 < G) hi = *reinterpret_cast<const uint2*>(qb + (r + 8) * HD + d0);
            q.a[ks][0] = lo.x; q.a[ks][2] = lo.y;
            q.a[ks][1] = hi.x; q.a[ks][3] = hi.y;
        }
    }

    static __device__ __forceinline__ void reset(Acc& c, int) {
#pragma unroll
        for (int n = 0; n < NT; ++n) c.o[n][0] = c.o[n][1] = c.o[n][2] = c.o[n][3] = 0.f;
        c.m0 = c.m1 = -INFINITY;
        c.l0 = c.l1 = 0.f;
        c.vRef = 1.f; c.invVRef = 1.f;
        c.first = true;
    }

    static __device__ __forceinline__ void tile(Acc& c, const Query& q, unsigned char* stagePtr, uint32_t, int tokBase,
                                                int windowStart, int len, float scaleLog2, int lane) {
        const int r = lane >> 2, j = lane & 3;
        const __half* sc = reinterpret_cast<const __half*>(stagePtr + 2 * TILEB);
        const int odd = stagePtr[2 * TILEB + 8];
        const float ks_ = __half2float(sc[odd]), vs_ = __half2float(sc[2 + odd]);
        if (c.first) { c.vRef = vs_ > 0.f ? vs_ : 1.f; c.invVRef = 1.f / c.vRef; c.first = false; }
        const bool partial = tokBase < windowStart || tokBase + kTileTokens > len;
        if (partial) {
            // rows outside [window_start, L): zero codes, so that a zero weight times that row is zero
            unsigned char* vt = stagePtr + TILEB;
            for (int idx = lane; idx < CHUNKS; idx += 32) {
                const int tok = tokBase + (idx >> 3);
                if (tok < windowStart || tok >= len) *reinterpret_cast<uint4*>(vt + idx * 16) = make_uint4(0u, 0u, 0u, 0u);
            }
            __syncwarp();
        }
        // S = Q K^T on the codes; the group scale and 1/sqrt(d) follow.
        float s[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
            const int row = 8 * nt + r;
            const uint4 w0 = *reinterpret_cast<const uint4*>(stagePtr + row * ROWB + (((2 * j) ^ (row & 7)) << 4));
            const uint4 w1 = *reinterpret_cast<const uint4*>(stagePtr + row * ROWB + (((2 * j + 1) ^ (row & 7)) << 4));
            const uint32_t w[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
            for (int ks = 0; ks < KSTEPS; ++ks) mma16816<__half>(s[nt], q.a[ks], e4m3x2ToHalf2(w[ks]), e4m3x2HiToHalf2(w[ks]));
        }
        const float sScale = ks_ * scaleLog2;
        float tmax0 = -INFINITY, tmax1 = -INFINITY;
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int tok = tokBase + 8 * nt + 2 * j + e;
                const bool ok = !partial || (tok >= windowStart && tok < len);
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
        bool raise = tmax0 > c.m0 + kLazyMax;          // m0 = -inf: the first tile always raises
        float c0 = 1.f, c1 = 1.f;
        if (raise) { c0 = ex2Fast(c.m0 - tmax0); c.m0 = tmax0; }
        if (UPPER) {
            tmax1 = fmaxf(tmax1, __shfl_xor_sync(0xFFFFFFFFu, tmax1, 1));
            tmax1 = fmaxf(tmax1, __shfl_xor_sync(0xFFFFFFFFu, tmax1, 2));
            if (tmax1 > c.m1 + kLazyMax) { c1 = ex2Fast(c.m1 - tmax1); c.m1 = tmax1; raise = true; }
        }
        if (__any_sync(0xFFFFFFFFu, raise)) {
            c.l0 *= c0;
            if (UPPER) c.l1 *= c1;
#pragma unroll
            for (int n = 0; n < NT; ++n) {
                c.o[n][0] *= c0;
                c.o[n][1] *= c0;
                if (UPPER) {
                    c.o[n][2] *= c1;
                    c.o[n][3] *= c1;
                }
            }
        }
        // weights; those that enter the product carry V's group scale relative to vRef
        const float vw = vs_ * c.invVRef;
        uint32_t pa[4];
        {
            const float p00 = ex2Fast(s[0][0] - c.m0), p01 = ex2Fast(s[0][1] - c.m0);
            const float p10 = ex2Fast(s[1][0] - c.m0), p11 = ex2Fast(s[1][1] - c.m0);
            c.l0 += (p00 + p01) + (p10 + p11);
            pa[0] = pack2<__half>(p00 * vw, p01 * vw);
            pa[2] = pack2<__half>(p10 * vw, p11 * vw);
            if (UPPER) {
                const float q00 = ex2Fast(s[0][2] - c.m1), q01 = ex2Fast(s[0][3] - c.m1);
                const float q10 = ex2Fast(s[1][2] - c.m1), q11 = ex2Fast(s[1][3] - c.m1);
                c.l1 += (q00 + q01) + (q10 + q11);
                pa[1] = pack2<__half>(q00 * vw, q01 * vw);
                pa[3] = pack2<__half>(q10 * vw, q11 * vw);
            } else {
                pa[1] = 0u;
                pa[3] = 0u;
            }
        }
        // O += P V.  Thread (r, j) reads chunk r (dims 16r .. 16r+15) of the token rows
        // 2j, 2j+1, 2j+8, 2j+9; n-tile c takes byte c of each: output column n of n-tile c
        // is dim 16n + c.
        {
            const unsigned char* vt = stagePtr + TILEB;
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
                mma16816<__half>(c.o[4 * wi + 0], pa, e4m3x2ToHalf2(a01), e4m3x2ToHalf2(b01));
                mma16816<__half>(c.o[4 * wi + 1], pa, e4m3x2HiToHalf2(a01), e4m3x2HiToHalf2(b01));
                mma16816<__half>(c.o[4 * wi + 2], pa, e4m3x2ToHalf2(a23), e4m3x2ToHalf2(b23));
                mma16816<__half>(c.o[4 * wi + 3], pa, e4m3x2HiToHalf2(a23), e4m3x2HiToHalf2(b23));
            }
        }
    }

    static __device__ __forceinline__ void finish(Acc& c) {
        c.l0 += __shfl_xor_sync(0xFFFFFFFFu, c.l0, 1);
        c.l0 += __shfl_xor_sync(0xFFFFFFFFu, c.l0, 2);
        if (UPPER) {
            c.l1 += __shfl_xor_sync(0xFFFFFFFFu, c.l1, 1);
            c.l1 += __shfl_xor_sync(0xFFFFFFFFu, c.l1, 2);
        }
    }

    // accumulator element n of a thread is dim 16 * (2j) + n (first value) and 16 * (2j + 1) + n
    template <class F, class Gf>
    static __device__ __forceinline__ void each(const Acc& c, int G, int lane, F f, Gf g) {
        const int r = lane >> 2, j = lane & 3;
        if (r < G) {
#pragma unroll
            for (int n = 0; n < NT; ++n) f(r, 16 * (2 * j) + n, c.o[n][0] * c.vRef, c.o[n][1] * c.vRef);
            if (j == 0) g(r, c.m0, c.l0);
        }
        if (UPPER && r + 8 < G) {
#pragma unroll
            for (int n = 0; n < NT; ++n) f(r + 8, 16 * (2 * j) + n, c.o[n][2] * c.vRef, c.o[n][3] * c.vRef);
            if (j == 0) g(r + 8, c.m1, c.l1);
        }
    }
    static constexpr int kPairStride = 16;    // the two values handed to f are columns d and d + 16
    static __device__ __forceinline__ float rowSum(const Acc& c, int g) { return g >= 8 ? c.l1 : c.l0; }
};

// The same pools with at most 8 query heads per KV head: the products are taken transposed,
// S^T = K Q^T (16 tokens x 8 heads) and O^T = V^T P^T (dims x 8 heads), so that the 8-wide side
// of mma.sync.m16n8k16 carries the heads and no row of a product is padding: half the
// products, half the accumulator registers.  Thread (r, j) of a warp (r = lane / 4,
// j = lane % 4) then holds the scores of tokens r and r + 8 for heads 2j and 2j + 1; the
// weights go back to the token-major operand layout with two movmatrix transposes.
__device__ __forceinline__ uint32_t movmatrixTrans(uint32_t v) {
    uint32_t r;
    asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(r) : "r"(v));
    return r;
}

struct Fp8TilesT {
    using Base = Fp8Tiles<false>;
    using Out = __half;
    static constexpr int HD = 128, NS = Base::NS;
    static constexpr int ROWB = Base::ROWB, TILEB = Base::TILEB, CHUNKS = Base::CHUNKS, STAGEB = Base::STAGEB;
    static constexpr int KSTEPS = HD / 16, MT = HD / 16;
    struct Query { uint32_t b[KSTEPS][2]; };
    struct Acc {
        float o[MT][4];          // m-tile t: (dim 16r + t, heads 2j, 2j+1), (dim 16r + 8 + t, heads 2j, 2j+1)
        float m0, m1, l0, l1;    // running maximum and sum of heads 2j and 2j + 1 (the sums over this thread's tokens)
        float vRef, invVRef;     // V scale of the first tile
        bool first;
    };

    static __device__ __forceinline__ void issue(uint32_t stage, unsigned char* stagePtr, const StreamArgs& a, int64_t blk,
                                                 int kvh, int within, int lane) {
        Base::issue(stage, stagePtr, a, blk, kvh, within, lane);
    }

    // Query rows as B fragments with the permuted K order: step ks of thread (r, j) covers
    // dims 32j + 4ks + {0,1} (first half) and + {2,3} (second half) of head r.
    static __device__ __forceinline__ void loadQuery(Query& q, const StreamArgs& a, int64_t row0, int G, int lane) {
        const int r = lane >> 2, j = lane & 3;
        const __half* qb = static_cast<const __half*>(a.q) + row0 * HD;
#pragma unroll
        for (int ks = 0; ks < KSTEPS; ++ks) {
            uint2 w = make_uint2(0u, 0u);
            if (r < G) w = *reinterpret_cast<const uint2*>(qb + r * HD + 32 * j + 4 * ks);
            q.b[ks][0] = w.x;
            q.b[ks][1] = w.y;
        }
    }

    static __device__ __forceinline__ void reset(Acc& c, int) {
#pragma unroll
        for (int t = 0; t < MT; ++t) c.o[t][0] = c.o[t][1] = c.o[t][2] = c.o[t][3] = 0.f;
        c.m0 = c.m1 = -INFINITY;
        c.l0 = c.l1 = 0.f;
        c.vRef = 1.f; c.invVRef = 1.f;
        c.first = true;
    }

    static __device__ __forceinline__ void tile(Acc& c, const Query& q, unsigned char* stagePtr, uint32_t, int tokBase,
                                                int windowStart, int len, float scaleLog2, int lane) {
        const int r = lane >> 2, j = lane & 3;
        const __half* sc = reinterpret_cast<const __half*>(stagePtr + 2 * TILEB);
        const int odd = stagePtr[2 * TILEB + 8];
        const float ks_ = __half2float(sc[odd]), vs_ = __half2float(sc[2 + odd]);
        if (c.first) { c.vRef = vs_ > 0.f ? vs_ : 1.f; c.invVRef = 1.f / c.vRef; c.first = false; }
        const bool partial = tokBase < windowStart || tokBase + kTileTokens > len;
        if (partial) {
            // rows outside [window_start, L): zero codes, so that a zero weight times that row is zero
            unsigned char* vt = stagePtr + TILEB;
            for (int idx = lane; idx < CHUNKS; idx += 32) {
                const int tok = tokBase + (idx >> 3);
                if (tok < windowStart || tok >= len) *reinterpret_cast<uint4*>(vt + idx * 16) = make_uint4(0u, 0u, 0u, 0u);
            }
            __syncwarp();
        }
        // S^T = K Q^T on the codes (two accumulators, so that the products do not form one
        // chain); the group scale and 1/sqrt(d) follow.
        float s[4] = {0.f, 0.f, 0.f, 0.f}, s2[4] = {0.f, 0.f, 0.f, 0.f};
        {
            const int rowA = r, rowB = r + 8;
            const uint4 a0 = *reinterpret_cast<const uint4*>(stagePtr + rowA * ROWB + (((2 * j) ^ (rowA & 7)) << 4));
            const uint4 a1 = *reinterpret_cast<const uint4*>(stagePtr + rowA * ROWB + (((2 * j + 1) ^ (rowA & 7)) << 4));
            const uint4 b0 = *reinterpret_cast<const uint4*>(stagePtr + rowB * ROWB + (((2 * j) ^ (rowB & 7)) << 4));
            const uint4 b1 = *reinterpret_cast<const uint4*>(stagePtr + rowB * ROWB + (((2 * j + 1) ^ (rowB & 7)) << 4));
            const uint32_t wa[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
            const uint32_t wb[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
#pragma unroll
            for (int ks = 0; ks < KSTEPS; ++ks) {
                const uint32_t frag[4] = {e4m3x2ToHalf2(wa[ks]), e4m3x2ToHalf2(wb[ks]), e4m3x2HiToHalf2(wa[ks]), e4m3x2HiToHalf2(wb[ks])};
                if (ks & 1) mma16816<__half>(s2, frag, q.b[ks][0], q.b[ks][1]);
                else mma16816<__half>(s, frag, q.b[ks][0], q.b[ks][1]);
            }
        }
        const float sScale = ks_ * scaleLog2;
        const bool okA = !partial || (tokBase + r >= windowStart && tokBase + r < len);
        const bool okB = !partial || (tokBase + r + 8 >= windowStart && tokBase + r + 8 < len);
        s[0] = okA ? (s[0] + s2[0]) * sScale : -INFINITY;      // token r, head 2j
        s[1] = okA ? (s[1] + s2[1]) * sScale : -INFINITY;      // token r, head 2j + 1
        s[2] = okB ? (s[2] + s2[2]) * sScale : -INFINITY;      // token r + 8, head 2j
        s[3] = okB ? (s[3] + s2[3]) * sScale : -INFINITY;      // token r + 8, head 2j + 1
        float tmax0 = fmaxf(s[0], s[2]), tmax1 = fmaxf(s[1], s[3]);
#pragma unroll
        for (int o = 4; o <= 16; o <<= 1) {
            tmax0 = fmaxf(tmax0, __shfl_xor_sync(0xFFFFFFFFu, tmax0, o));
            tmax1 = fmaxf(tmax1, __shfl_xor_sync(0xFFFFFFFFu, tmax1, o));
        }
        bool raise = false;                              // m = -inf: the first tile always raises
        float c0 = 1.f, c1 = 1.f;
        if (tmax0 > c.m0 + kLazyMax) { c0 = ex2Fast(c.m0 - tmax0); c.m0 = tmax0; raise = true; }
        if (tmax1 > c.m1 + kLazyMax) { c1 = ex2Fast(c.m1 - tmax1); c.m1 = tmax1; raise = true; }
        if (__any_sync(0xFFFFFFFFu, raise)) {
            c.l0 *= c0;
            c.l1 *= c1;
#pragma unroll
            for (int t = 0; t < MT; ++t) {
                c.o[t][0] *= c0;
                c.o[t][1] *= c1;
                c.o[t][2] *= c0;
                c.o[t][3] *= c1;
            }
        }
        // weights; those that enter the product carry V's group scale relative to vRef.  As the
        // B operand they must be token-major per head: two 8 x 8 transposes.
        const float vw = vs_ * c.invVRef;
        uint32_t pb[2];
        {
            const float p0 = ex2Fast(s[0] - c.m0), p1 = ex2Fast(s[1] - c.m1);
            const float p2 = ex2Fast(s[2] - c.m0), p3 = ex2Fast(s[3] - c.m1);
            c.l0 += p0 + p2;
            c.l1 += p1 + p3;
            pb[0] = movmatrixTrans(pack2<__half>(p0 * vw, p1 * vw));      // (head r; tokens 2j, 2j + 1)
            pb[1] = movmatrixTrans(pack2<__half>(p2 * vw, p3 * vw));      // (head r; tokens 2j + 8, 2j + 9)
        }
        // O^T += V^T P^T.  Thread (r, j) reads chunk r (dims 16r .. 16r+15) of the token rows
        // 2j, 2j+1, 2j+8, 2j+9; m-tile t takes bytes t and 8 + t of each: its rows r and r + 8
        // are dims 16r + t and 16r + 8 + t.
        {
            const unsigned char* vt = stagePtr + TILEB;
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
            for (int wi = 0; wi < 2; ++wi) {
                // words wi (dims 16r + 4wi ..) and wi + 2 (dims 16r + 8 + 4wi ..) of the four token rows
                const uint32_t lo01 = __byte_perm(x0[wi], x1[wi], 0x5140), lo23 = __byte_perm(x0[wi], x1[wi], 0x7362);
                const uint32_t hi01 = __byte_perm(x0[wi + 2], x1[wi + 2], 0x5140), hi23 = __byte_perm(x0[wi + 2], x1[wi + 2], 0x7362);
                const uint32_t lp01 = __byte_perm(x2[wi], x3[wi], 0x5140), lp23 = __byte_perm(x2[wi], x3[wi], 0x7362);
                const uint32_t hp01 = __byte_perm(x2[wi + 2], x3[wi + 2], 0x5140), hp23 = __byte_perm(x2[wi + 2], x3[wi + 2], 0x7362);
                {
                    const uint32_t f0[4] = {e4m3x2ToHalf2(lo01), e4m3x2ToHalf2(hi01), e4m3x2ToHalf2(lp01), e4m3x2ToHalf2(hp01)};
                    mma16816<__half>(c.o[4 * wi + 0], f0, pb[0], pb[1]);
                    const uint32_t f1[4] = {e4m3x2HiToHalf2(lo01), e4m3x2HiToHalf2(hi01), e4m3x2HiToHalf2(lp01), e4m3x2HiToHalf2(hp01)};
                    mma16816<__half>(c.o[4 * wi + 1], f1, pb[0], pb[1]);
                    const uint32_t f2[4] = {e4m3x2ToHalf2(lo23), e4m3x2ToHalf2(hi23), e4m3x2ToHalf2(lp23), e4m3x2ToHalf2(hp23)};
                    mma16816<__half>(c.o[4 * wi + 2], f2, pb[0], pb[1]);
                    const uint32_t f3[4] = {e4m3x2HiToHalf2(lo23), e4m3x2HiToHalf2(hi23), e4m3x2HiToHalf2(lp23), e4m3x2HiToHalf2(hp23)};
                    mma16816<__half>(c.o[4 * wi + 3], f3, pb[0], pb[1]);
                }
            }
        }
    }

    static __device__ __forceinline__ void finish(Acc& c) {
#pragma unroll
        for (int o = 4; o <= 16; o <<= 1) {
            c.l0 += __shfl_xor_sync(0xFFFFFFFFu, c.l0, o);
            c.l1 += __shfl_xor_sync(0xFFFFFFFFu, c.l1, o);
        }
    }

    template <class F, class Gf>
    static __device__ __forceinline__ void each(const Acc& c, int G, int lane, F f, Gf g) {
        const int r = lane >> 2, j = lane & 3;
        if (2 * j < G) {
#pragma unroll
            for (int t = 0; t < MT; ++t) f(2 * j, 16 * r + t, c.o[t][0] * c.vRef, c.o[t][2] * c.vRef);
            if (r == 0) g(2 * j, c.m0, c.l0);
        }
        if (2 * j + 1 < G) {
#pragma unroll
            for (int t = 0; t < MT; ++t) f(2 * j + 1, 16 * r + t, c.o[t][1] * c.vRef, c.o[t][3] * c.vRef);
            if (r == 0) g(2 * j + 1, c.m1, c.l1);
        }
    }
    static constexpr int kPairStride = 8;     // the two values handed to f are columns d and d + 8
    static __device__ __forceinline__ float rowSum(const Acc& c, int g) { return (g & 1) ? c.l1 : c.l0; }
};

// ------------------------------------------------------------ the stream

// Tile counts of the sequences as a prefix sum in shared memory: prefix[b] = tiles of all
// (sequence, kv head) pairs before sequence b, first[b] = the sequence's first visible tile.
__device__ __forceinline__ void buildPrefix(int* prefix, int* first, const StreamArgs& a) {
    const int tid = threadIdx.x, nt = blockDim.x, lane = tid & 31, warp = tid >> 5;
    const int per = (a.batch + nt - 1) / nt;
    const int b0 = min(tid * per, a.batch), b1 = min(b0 + per, a.batch);
    const int maxTokens = a.maxNumBlocks * a.blockSize;
    int sum = 0;
    for (int b = b0; b < b1; ++b) {
        const Visible v = visibleOf(a.lens[b], a.window, maxTokens);
        first[b] = v.firstTile;
        prefix[b + 1] = v.numTiles * a.kvHeads;
        sum += v.numTiles * a.kvHeads;
    }
    __shared__ int warpSums[kWarps];
    int incl = sum;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const int n = __shfl_up_sync(0xFFFFFFFFu, incl, o);
        if (lane >= o) incl += n;
    }
    if (lane == 31) warpSums[warp] = incl;
    __syncthreads();
    int run = incl - sum;
    for (int w = 0; w < warp; ++w) run += warpSums[w];
    for (int b = b0; b < b1; ++b) {
        run += prefix[b + 1];
        prefix[b + 1] = run;
    }
    if (tid == 0) prefix[0] = 0;
    __syncthreads();
}

// Position in the list of tiles.
struct Cursor {
    int b, kvh, tile;        // sequence, kv head, tile counted from the sequence's first visible tile
    int tilesB, firstTile;   // tiles of a (sequence, kv head) pair of this sequence, its first visible tile
};
__device__ __forceinline__ void locate(Cursor& c, int unit, const int* prefix, const int* first, int batch, int kvHeads) {
    int lo = 0, hi = batch - 1;
    while (lo < hi) {                       // the sequence with prefix[b] <= unit < prefix[b + 1]
        const int mid = (lo + hi) >> 1;
        if (prefix[mid + 1] <= unit) lo = mid + 1; else hi = mid;
    }
    c.b = lo;
    c.tilesB = (prefix[lo + 1] - prefix[lo]) / kvHeads;
    const int local = unit - prefix[lo];
    c.kvh = local / c.tilesB;
    c.tile = local - c.kvh * c.tilesB;
    c.firstTile = first[lo];
}
__device__ __forceinline__ void advance(Cursor& c, const int* prefix, const int* first, int batch, int kvHeads) {
    if (++c.tile < c.tilesB) return;
    c.tile = 0;
    if (++c.kvh < kvHeads) return;
    c.kvh = 0;
    do { ++c.b; } while (c.b < batch && prefix[c.b + 1] == prefix[c.b]);    // sequences without visible tiles
    if (c.b < batch) {
        c.tilesB = (prefix[c.b + 1] - prefix[c.b]) / kvHeads;
        c.firstTile = first[c.b];
    }
}

constexpr int kPartialPad = 4;      // a partial row is head_dim + 4 floats: O, then m and l (16-byte rows)

// Where the partial results of a pair go.  Piece w of the list (warp w's) covers tiles
// [w * quota, (w + 1) * quota).  A pair that begins in piece wf and is the i-th pair of the
// launch owns the records from wf + i on, one per piece it overlaps, in the order of the
// pieces: the pair before it ends in piece wf or earlier and owns records up to wf + i - 1.
__device__ __forceinline__ int64_t recordBase(int pairBegin, int pairIndex, int quota) {
    return static_cast<int64_t>(pairBegin / quota) + pairIndex;
}

// Combination of the partials of one (sequence, kv head) pair by the warp whose tiles
// completed it: records first .. first + n - 1, always in that order, so that equal inputs
// give equal bits.  Two heads at a time; the (m, l) of all contributions are read by the
// lanes in parallel, the columns with sixteen loads in flight per lane (each lane four
// columns of eight records of both heads): the pairs of a launch tend to complete together
// at its end, where nothing else hides the latency of these reads.
template <class P>
__device__ __forceinline__ void combine(const float* __restrict__ records, typename P::Out* __restrict__ out, int heads, int b,
                                        int kvh, int G, int64_t first, int n, int lane) {
    constexpr int HD = P::HD, RS = HD + kPartialPad, U = 8;
    using Out = typename P::Out;
    const bool holds = lane * 4 < HD;                    // head_dim 64: half the lanes hold columns
    const int64_t step = static_cast<int64_t>(G) * RS;   // from one contribution to the next
    for (int g = 0; g < G; g += 2) {
        const bool two = g + 1 < G;
        const float* base0 = records + (first * G + g) * RS;
        const float* base1 = base0 + (two ? RS : 0);
        float M0 = -INFINITY, M1 = -INFINITY;
        for (int i = lane; i < n; i += 32) {
            M0 = fmaxf(M0, __ldcg(base0 + i * step + HD));
            M1 = fmaxf(M1, __ldcg(base1 + i * step + HD));
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            M0 = fmaxf(M0, __shfl_xor_sync(0xFFFFFFFFu, M0, o));
            M1 = fmaxf(M1, __shfl_xor_sync(0xFFFFFFFFu, M1, o));
        }
        float l0 = 0.f, l1 = 0.f;
        float4 acc0 = make_float4(0.f, 0.f, 0.f, 0.f), acc1 = acc0;
        for (int c0 = 0; c0 < n; c0 += 32) {
            const int mine = c0 + lane;
            float w0 = 0.f, w1 = 0.f;
            if (mine < n) {
                const float2 ml0 = __ldcg(reinterpret_cast<const float2*>(base0 + mine * step + HD));
                const float2 ml1 = __ldcg(reinterpret_cast<const float2*>(base1 + mine * step + HD));
                w0 = exp2f(ml0.x - M0);
                w1 = exp2f(ml1.x - M1);
                l0 += w0 * ml0.y;
                l1 += w1 * ml1.y;
            }
            const int cnt = min(32, n - c0);
            for (int i0 = 0; i0 < cnt; i0 += U) {
                float4 v0[U], v1[U];
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    v0[u] = make_float4(0.f, 0.f, 0.f, 0.f);
                    v1[u] = v0[u];
                    if (holds && i0 + u < cnt) {
                        v0[u] = __ldcg(reinterpret_cast<const float4*>(base0 + (c0 + i0 + u) * step) + lane);
                        if (two) v1[u] = __ldcg(reinterpret_cast<const float4*>(base1 + (c0 + i0 + u) * step) + lane);
                    }
                }
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    const float a0 = __shfl_sync(0xFFFFFFFFu, w0, (i0 + u) & 31);     // (zero beyond cnt)
                    const float a1 = __shfl_sync(0xFFFFFFFFu, w1, (i0 + u) & 31);
                    acc0.x += a0 * v0[u].x; acc0.y += a0 * v0[u].y; acc0.z += a0 * v0[u].z; acc0.w += a0 * v0[u].w;
                    acc1.x += a1 * v1[u].x; acc1.y += a1 * v1[u].y; acc1.z += a1 * v1[u].z; acc1.w += a1 * v1[u].w;
                }
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            l0 += __shfl_xor_sync(0xFFFFFFFFu, l0, o);
            l1 += __shfl_xor_sync(0xFFFFFFFFu, l1, o);
        }
        if (holds) {
            Out* dst = out + (static_cast<int64_t>(b) * heads + kvh * G + g) * HD + lane * 4;
            const float inv0 = 1.f / l0;
            dst[0] = fromFloat<Out>(acc0.x * inv0);
            dst[1] = fromFloat<Out>(acc0.y * inv0);
            dst[2] = fromFloat<Out>(acc0.z * inv0);
            dst[3] = fromFloat<Out>(acc0.w * inv0);
            if (two) {
                const float inv1 = 1.f / l1;
                dst[HD + 0] = fromFloat<Out>(acc1.x * inv1);
                dst[HD + 1] = fromFloat<Out>(acc1.y * inv1);
                dst[HD + 2] = fromFloat<Out>(acc1.z * inv1);
                dst[HD + 3] = fromFloat<Out>(acc1.w * inv1);
            }
        }
    }
}

template <class P>
__global__ void __launch_bounds__(kWarps * 32)
decodeStreamKernel(const StreamArgs a) {
    constexpr int NS = P::NS, STAGEB = P::STAGEB, HD = P::HD, RS = HD + kPartialPad;
    using Out = typename P::Out;
    extern __shared__ __align__(128) unsigned char smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int G = a.heads / a.kvHeads;
    const int maxTokens = a.maxNumBlocks * a.blockSize;
    constexpr int kRingBytes = (kWarps * NS * STAGEB + 15) / 16 * 16;
    int* prefix = reinterpret_cast<int*>(smem + kRingBytes);     // [batch + 1]
    int* first = prefix + a.batch + 1;                           // [batch]
    const int warpsInGrid = gridDim.x * kWarps, wid = blockIdx.x * kWarps + warp;
    buildPrefix(prefix, first, a);

    // An empty context (the reference divides 0 by 0 there) gets zeros.
    for (int b = blockIdx.x; b < a.batch; b += gridDim.x) {
        if (prefix[b + 1] != prefix[b]) continue;
        Out* dst = static_cast<Out*>(a.out) + static_cast<int64_t>(b) * a.heads * HD;
        for (int i = threadIdx.x; i < a.heads * HD; i += kWarps * 32) dst[i] = fromFloat<Out>(0.f);
    }

    // This warp's piece of the list.
    const int total = prefix[a.batch];
    const int quota = max((total + warpsInGrid - 1) / warpsInGrid, 1);
    const int begin = min(wid * quota, total), end = min(begin + quota, total);
    if (begin >= end) return;                        // (no barrier below this line)
    const int tilesPerPage = a.blockSize / kTileTokens;
    // (a division by a run-time value is some twenty instructions per tile; block sizes are
    // powers of two in practice)
    const int pageShift = (tilesPerPage & (tilesPerPage - 1)) == 0 ? __ffs(tilesPerPage) - 1 : -1;
    unsigned char* ring = smem + static_cast<size_t>(warp) * NS * STAGEB;
    const uint32_t ringAddr = smemAddr(ring);

    Cursor ahead, cur;                       // where the loads are, where the arithmetic is
    locate(ahead, begin, prefix, first, a.batch, a.kvHeads);
    cur = ahead;
    int issued = begin;
    auto issueNext = [&](int slot) {
        if (issued >= end) return;
        const int tile = ahead.firstTile + ahead.tile;
        const int page = pageShift >= 0 ? tile >> pageShift : tile / tilesPerPage, within = tile - page * tilesPerPage;
        const int32_t* table = a.tables + static_cast<int64_t>(ahead.b) * a.maxNumBlocks;
        const int64_t blk = min(max(table[page], 0), a.poolBlocks - 1);     // never read outside the pool
        P::issue(ringAddr + slot * STAGEB, ring + slot * STAGEB, a, blk, ahead.kvh, within, lane);
        advance(ahead, prefix, first, a.batch, a.kvHeads);
        ++issued;
    };
#pragma unroll
    for (int s = 0; s < NS; ++s) {
        issueNext(s);
        cpAsyncCommit();
    }

    typename P::Query q;
    typename P::Acc acc;
    int len = 0, windowStart = 0, pairBegin = 0, pairTiles = 0;
    // The length and the query rows of the (sequence, kv head) pair at `c`.  At a border they are
    // asked for before the finished pair's result leaves, so that they arrive meanwhile.
    auto openPair = [&](const Cursor& c, int& newLen, int& newWindowStart, int& newPairBegin) {
        const uint32_t L = a.lens[c.b];
        const Visible v = visibleOf(L, a.window, maxTokens);
        newLen = static_cast<int>(L < static_cast<uint32_t>(maxTokens) ? L : static_cast<uint32_t>(maxTokens));
        newWindowStart = v.windowStart;
        newPairBegin = prefix[c.b] + c.kvh * c.tilesB;
        P::loadQuery(q, a, static_cast<int64_t>(c.b) * a.heads + c.kvh * G, G, lane);
    };
    openPair(cur, len, windowStart, pairBegin);
    P::reset(acc, len - windowStart);
    for (int done = begin; done < end;) {
        cpAsyncWait<NS - 1>();
        __syncwarp();
        const int slot = (done - begin) % NS;
        P::tile(acc, q, ring + slot * STAGEB, ringAddr + slot * STAGEB, (cur.firstTile + cur.tile) * kTileTokens, windowStart,
                len, a.scaleLog2, lane);
        __syncwarp();
        ++done;
        ++pairTiles;
        issueNext(slot);
        cpAsyncCommit();

        Cursor next = cur;
        advance(next, prefix, first, a.batch, a.kvHeads);
        if (cur.tile + 1 == cur.tilesB || done == end) {
            // the pair ends here, or the piece does
            P::finish(acc);
            int nextLen = 0, nextWindowStart = 0, nextPairBegin = 0;
            if (done < end) openPair(next, nextLen, nextWindowStart, nextPairBegin);       // (the query registers are free: the last tile is done)
            const int64_t outRow = static_cast<int64_t>(cur.b) * a.heads + cur.kvh * G;
            if (pairTiles == cur.tilesB) {
                // every tile of the pair was this warp's: its output
                Out* dst = static_cast<Out*>(a.out) + outRow * HD;
                P::each(acc, G, lane,
                        [&](int g, int d, float v0, float v1) {
                            const float inv = 1.f / P::rowSum(acc, g);
                            if (P::kPairStride == 1) {
                                *reinterpret_cast<uint32_t*>(dst + g * HD + d) = pack2<Out>(v0 * inv, v1 * inv);
                            } else {
                                dst[g * HD + d] = fromFloat<Out>(v0 * inv);
                                dst[g * HD + d + P::kPairStride] = fromFloat<Out>(v1 * inv);
                            }
                        },
                        [](int, float, float) {});
            } else {
                // one record per piece the pair overlaps, in the order of the pieces; the tiles
                // counted so far decide who combines
                const int pairIndex = cur.b * a.kvHeads + cur.kvh;
                const int firstPiece = pairBegin / quota;
                const int64_t base = recordBase(pairBegin, pairIndex, quota);
                float* part = a.records + ((base + (wid - firstPiece)) * G) * RS;
                P::each(acc, G, lane,
                        [&](int g, int d, float v0, float v1) {
                            part[g * RS + d] = v0;
                            part[g * RS + d + P::kPairStride] = v1;
                        },
                        [&](int g, float m, float l) {
                            part[g * RS + HD] = m;
                            part[g * RS + HD + 1] = l;
                        });
                // the record is published before its tiles are counted; whoever completes the
                // count reads the others' records from L2
                __threadfence();
                __syncwarp();
                int* tilesDone = a.counters + pairIndex;
                bool last = false;
                if (lane == 0) {
                    last = atomicAdd(tilesDone, pairTiles) + pairTiles == cur.tilesB;
                    if (last) *tilesDone = 0;                   // ready for the next launch
                }
                if (__shfl_sync(0xFFFFFFFFu, last ? 1 : 0, 0)) {
                    __threadfence();
                    const int n = (pairBegin + cur.tilesB - 1) / quota - firstPiece + 1;
                    combine<P>(a.records, static_cast<Out*>(a.out), a.heads, cur.b, cur.kvh, G, base, n, lane);
                }
            }
            len = nextLen;
            windowStart = nextWindowStart;
            pairBegin = nextPairBegin;
            pairTiles = 0;
            P::reset(acc, len - windowStart);
        }
        cur = next;
    }
    cpAsyncWait<0>();
}

// ---------------------------------------------------------------- launch

// The dynamic shared memory limit of a kernel is raised once per device, not per launch.
template <class K>
cudaError_t allowSharedMemory(K kernel, size_t bytes, std::atomic<size_t>* granted, int dev) {
    if (granted[dev].load(std::memory_order_acquire) >= bytes) return cudaSuccess;
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(bytes));
    if (e == cudaSuccess) granted[dev].store(bytes, std::memory_order_release);
    return e;
}

template <class P>
size_t streamSharedBytes(int batch) {
    const size_t ring = (static_cast<size_t>(kWarps) * P::NS * P::STAGEB + 15) / 16 * 16;
    return ring + (static_cast<size_t>(2) * batch + 1) * sizeof(int);
}

// CTAs of the launch: every resident slot of the GPU.
template <class P>
cudaError_t streamGrid(int batch, int smCount, int* grid) {
    static std::atomic<int> perSm[64][4];      // by device and by shared-memory class of the batch
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
    const int cls = batch <= 256 ? 0 : batch <= 512 ? 1 : batch <= 1024 ? 2 : 3;
    const int classBatch = cls == 0 ? 256 : cls == 1 ? 512 : cls == 2 ? 1024 : kDecodeStreamMaxBatch;
    int n = perSm[dev][cls].load(std::memory_order_acquire);
    if (n == 0) {
        static std::atomic<size_t> granted[64];
        const size_t smem = streamSharedBytes<P>(kDecodeStreamMaxBatch);
        e = allowSharedMemory(decodeStreamKernel<P>, smem, granted, dev);
        if (e != cudaSuccess) return e;
        e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, decodeStreamKernel<P>, kWarps * 32, streamSharedBytes<P>(classBatch));
        if (e != cudaSuccess) return e;
        if (n < 1) n = 1;
        perSm[dev][cls].store(n, std::memory_order_release);
    }
    *grid = smCount * n;
    return cudaSuccess;
}

// One record per piece and per pair bounds what recordBase() hands out.
size_t recordBytes(int grid, int pairs, int G, int headDim) {
    return (static_cast<size_t>(grid) * kWarps + static_cast<size_t>(pairs)) * G * (headDim + kPartialPad) * sizeof(float);
}

template <class P>
cudaError_t launchStreamT(const DecodeParams& p, int smCount, cudaStream_t stream, int* launches) {
    int grid = 0;
    cudaError_t e = streamGrid<P>(p.batch, smCount, &grid);
    if (e != cudaSuccess) return e;
    const int G = p.heads / p.kvHeads, pairs = p.batch * p.kvHeads;
    // Short lists get fewer warps.  With less than kMinTilesPerWarp tiles per warp (by the bound
    // the table width and the window give; the lengths are on the device) a third CTA per SM
    // costs more in records, combinations and starts than it hides latency: measured on one KV
    // head of the long-context FP8 workload, 9 tiles per warp at three CTAs per SM took 0.063 ms
    // against 0.048 ms at two (14 per warp), while 18 per warp at three beat 28 at two.
    {
        constexpr int64_t kMinTilesPerWarp = 14;
        int64_t tokens = static_cast<int64_t>(p.maxNumBlocks) * p.blockSize;
        if (p.window > 0) tokens = std::min<int64_t>(tokens, static_cast<int64_t>(p.window) + p.blockSize);
        const int64_t tiles = (tokens + kTileTokens - 1) / kTileTokens * pairs;
        int perSm = std::max(grid / std::max(smCount, 1), 1);
        while (perSm > 2 && tiles < kMinTilesPerWarp * smCount * perSm * kWarps) --perSm;
        grid = smCount * perSm;
    }
    // a smaller workspace (the fixed array of the no-allocation call) holds fewer warps' records
    while (grid > 1 && recordBytes(grid, pairs, G, P::HD) > p.workspaceBytes) grid = grid * 3 / 4;
    if (recordBytes(grid, pairs, G, P::HD) > p.workspaceBytes) return cudaErrorInvalidValue;
    StreamArgs a{};
    a.q = p.q; a.kPool = p.kPool; a.vPool = p.vPool; a.kScale = p.kScale; a.vScale = p.vScale;
    a.tables = p.tables; a.lens = p.lens; a.out = p.out; a.records = p.workspace; a.counters = p.counters;
    a.batch = p.batch; a.heads = p.heads; a.kvHeads = p.kvHeads; a.blockSize = p.blockSize; a.maxNumBlocks = p.maxNumBlocks;
    a.window = p.window; a.poolBlocks = p.poolBlocks;
    a.scaleLog2 = (1.0f / sqrtf(static_cast<float>(p.headDim))) * kLog2e;
    decodeStreamKernel<P><<<grid, kWarps * 32, streamSharedBytes<P>(p.batch), stream>>>(a);
    e = cudaGetLastError();
    if (e == cudaSuccess && launches) *launches += 1;
    return e;
}

template <class F>
auto dispatch(const DecodeParams& p, F f) {
    const bool upper = p.heads / p.kvHeads > 8;
    if (p.dtype == kFP8) return upper ? f(Fp8Tiles<true>{}) : f(Fp8TilesT{});
    if (p.dtype == kF16) {
        if (p.headDim == 128) return upper ? f(HalfTiles<__half, 128, true>{}) : f(HalfTiles<__half, 128, false>{});
        return upper ? f(HalfTiles<__half, 64, true>{}) : f(HalfTiles<__half, 64, false>{});
    }
    if (p.headDim == 128) return upper ? f(HalfTiles<__nv_bfloat16, 128, true>{}) : f(HalfTiles<__nv_bfloat16, 128, false>{});
    return upper ? f(HalfTiles<__nv_bfloat16, 64, true>{}) : f(HalfTiles<__nv_bfloat16, 64, false>{});
}

}  // namespace

bool decodeStreamApplies(const DecodeParams& p) {
    const int G = p.kvHeads > 0 ? p.heads / p.kvHeads : 0;
    const bool shape = p.headDim > 0 && p.blockSize > 0 && p.blockSize % kTileTokens == 0 && G >= 1 && G <= 16 && p.batch >= 1;
    // the kernel copies pages with 16-byte cp.async and reads the query rows as 4-byte (FP8:
    // 8-byte) words; anything less aligned goes to the general kernel
    const auto aligned = [](const void* ptr, uintptr_t a) { return (reinterpret_cast<uintptr_t>(ptr) & (a - 1)) == 0; };
    if (!shape || !aligned(p.kPool, 16) || !aligned(p.vPool, 16)) return false;
    // positions in the list of tiles are ints
    const int slice = p.batch < kDecodeStreamMaxBatch ? p.batch : kDecodeStreamMaxBatch;
    if (static_cast<int64_t>(p.maxNumBlocks) * p.blockSize / kTileTokens * p.kvHeads * slice >= (int64_t(1) << 30)) return false;
    if (p.dtype == kF16 || p.dtype == kBF16) return (p.headDim == 128 || p.headDim == 64) && aligned(p.q, 4) && aligned(p.out, 4);
    if (p.dtype == kFP8)
        return p.headDim == 128 && p.kScale && p.vScale && aligned(p.q, 8) && aligned(p.out, 2) && aligned(p.kScale, 4) &&
               aligned(p.vScale, 4);
    return false;
}

int decodeStreamWarps(const DecodeParams& p, int smCount) {
    int grid = 0;
    const int slice = p.batch < kDecodeStreamMaxBatch ? p.batch : kDecodeStreamMaxBatch;
    const cudaError_t e = dispatch(p, [&](auto tiles) { return streamGrid<decltype(tiles)>(slice, smCount, &grid); });
    if (e != cudaSuccess) { cudaGetLastError(); return 0; }
    return grid * kWarps;
}

size_t decodeStreamWorkspaceBytes(const DecodeParams& p, int smCount) {
    const int warps = decodeStreamWarps(p, smCount);
    if (warps == 0) return 0;
    const int slice = p.batch < kDecodeStreamMaxBatch ? p.batch : kDecodeStreamMaxBatch;
    const int pairs = slice * p.kvHeads;
    return recordBytes(warps / kWarps, pairs, p.heads / p.kvHeads, p.headDim);
}

cudaError_t launchDecodeStream(const DecodeParams& p, int smCount, cudaStream_t stream, int* launches) {
    if (!p.workspace || !p.counters || static_cast<int64_t>(p.batch) * p.kvHeads > p.countersCap) return cudaErrorInvalidValue;
    // batches beyond what the prefix sum in shared memory holds go in slices
    for (int b0 = 0; b0 < p.batch; b0 += kDecodeStreamMaxBatch) {
        DecodeParams s = p;
        s.batch = p.batch - b0 < kDecodeStreamMaxBatch ? p.batch - b0 : kDecodeStreamMaxBatch;
        const size_t io = static_cast<size_t>(p.heads) * p.headDim * ioBytes(p.dtype);
        s.q = static_cast<const char*>(p.q) + b0 * io;
        s.out = static_cast<char*>(p.out) + b0 * io;
        s.tables = p.tables + static_cast<int64_t>(b0) * p.maxNumBlocks;
        s.lens = p.lens + b0;
        s.counters = p.counters + static_cast<int64_t>(b0) * p.kvHeads;
        const cudaError_t e = dispatch(s, [&](auto tiles) { return launchStreamT<decltype(tiles)>(s, smCount, stream, launches); });
        if (e != cudaSuccess) return e;
    }
    return cudaSuccess;
}

size_t decodeStaticScratchBytes() { return kStaticScratchBytes; }

cudaError_t decodeStaticScratch(float** scratch, int** counters, int64_t* countersCap) {
    // In host code the arrays' names are only handles; the kernels need their device
    // addresses, which differ per GPU.  They are looked up once per device, with that device
    // current (the caller has made it so).  Two host threads may get here together for the
    // same GPU: both then store the same addresses.
    static std::atomic<float*> scratchOn[64];
    static std::atomic<int*> countersOn[64];
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
    float* s = scratchOn[dev].load(std::memory_order_acquire);
    int* c = countersOn[dev].load(std::memory_order_acquire);
    if (!s || !c) {
        void* ps = nullptr;
        void* pc = nullptr;
        e = cudaGetSymbolAddress(&ps, gStaticDecodeScratch);
        if (e == cudaSuccess) e = cudaGetSymbolAddress(&pc, gStaticDecodeCounters);
        if (e != cudaSuccess) return e;
        s = static_cast<float*>(ps);
        c = static_cast<int*>(pc);
        scratchOn[dev].store(s, std::memory_order_release);
        countersOn[dev].store(c, std::memory_order_release);
    }
    *scratch = s;
    *counters = c;
    *countersCap = kStaticCounters;
    return cudaSuccess;
}

}  // namespace pam
