// Chunked causal prefill on the 5th-generation tensor cores (sm_100a):
// tcgen05.mma with accumulators in tensor memory, operands staged in shared
// memory by TMA, for bfloat16 / float16 KV with head_dim 128 and a block size
// that is a multiple of 16.
//
// Semantics are those of prefillGeneralKernel (paged_attention_tiled,
// kernels.metal:693-765, plus the chunk rows of
// PagedAttentionEngine.swift:740-756).
//
// One CTA owns 128 query rows of one head of one sequence and walks the key
// tiles (128 keys each) those rows can see.  Tensor memory holds two S buffers
// (128 columns each, overwritten in place by the weights P) and the
// accumulator O (128 columns): while the softmax warps turn S of tile j into P,
// the tensor pipe finishes P V of tile j-1 and Q K^T of tile j+1.
//
//   warp 16              TMA producer of Q (once) and of K: per key tile 8
//                        pages (each 16 rows x 256 B, fetched as two
//                        128-byte-swizzled boxes, one page per lane) into a
//                        3-stage ring; completion on mbarriers.
//   warp 17              TMA producer of V, 2-stage ring.
//   warp 18 (one thread) MMA issuer: S = Q K^T (8 x tcgen05.mma 128x128x16,
//                        both operands from shared memory) two tiles ahead,
//                        and O += P V (P read from tensor memory, V as an
//                        MN-major operand straight from its row-major pages);
//                        tcgen05.commit signals the mbarriers.
//   warps 0-15           softmax: four threads per row, thread (t, c) owns row t
//                        and key columns [32c, 32c+32).  S is read from tensor
//                        memory (tcgen05.ld), scaled, masked (causal, window
//                        start, sequence end) only on edge tiles; the four
//                        parts of a row exchange their maxima through shared
//                        memory.  The running maximum is only raised when it
//                        grows by more than 2^8 (the result is exact either
//                        way, the final division uses the same reference), in
//                        which case O is rescaled in tensor memory.  The
//                        weights go back to tensor memory in the cache type
//                        (tcgen05.st); for bfloat16, on rows that see few keys,
//                        as two operands P_hi + P_lo (16 significant bits
//                        together) and twice the PV instructions, because 8-bit
//                        weights alone miss the 2e-3 bound there.
//
// Every wait on an mbarrier is bounded; a wait that runs out raises a flag the
// host reads and the CTA falls through to the common exit, where the tensor
// memory is released.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <cmath>

#include "kernels.h"

namespace pam {
namespace {

constexpr int kRows = 128;        // query rows per CTA
constexpr int kKeys = 128;        // keys per tile
constexpr int kHd = 128;
constexpr int kKStages = 3, kVStages = 2;
constexpr int kTileBytes = kRows * kHd * 2;            // 32 KB: one [128][128] 16-bit tile
constexpr int kHalfBytes = kTileBytes / 2;             // one 64-column block
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kRescaleThreshold = 8.0f;
constexpr int kShortRowKeys = 256;
constexpr long long kWaitCycles = 400000000LL;         // ~0.2 s

#ifdef PAM_PREFILL_TRACE
// Instrumented build only: CTA (0,0,0) keeps clock stamps [role][tile][event] in
// shared memory (no global traffic while it runs) and dumps them at the end.
constexpr int kTraceRoles = 4, kTraceTiles = 32, kTraceEvents = 12;
__device__ long long gTrace[kTraceRoles * kTraceTiles * kTraceEvents];
#define TRACE(role, tile, event)                                                                        \
    do {                                                                                                \
        if (blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && (threadIdx.x & 31) == 0 &&         \
            (role) < kTraceRoles && (tile) < kTraceTiles)                                               \
            s->trace[((role) * kTraceTiles + (tile)) * kTraceEvents + (event)] = clock64();             \
    } while (0)
#else
#define TRACE(role, tile, event)
#endif

struct Smem {
    // tiles first: each 1024-byte aligned (swizzle atoms)
    unsigned char q[kTileBytes];               // the query tile; reused to stage the output
    unsigned char k[kKStages][kTileBytes];
    unsigned char v[kVStages][kTileBytes];
    unsigned long long qFull, kFull[kKStages], kEmpty[kKStages], vFull[kVStages], vEmpty[kVStages];
    unsigned long long sFull[2], pFull, pvDone;
    unsigned long long maxReady[2], sumReady;  // exchange between the four parts of a row
    float rowMax[2][4][kRows];                 // [parity][column quarter][row]
    uint32_t tmemBase;
    int dead;
#ifdef PAM_PREFILL_TRACE
    long long trace[kTraceRoles * kTraceTiles * kTraceEvents];
#endif
};

__device__ __forceinline__ uint32_t smemAddr(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbarInit(unsigned long long* bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smemAddr(bar)), "r"(count));
}
__device__ __forceinline__ void mbarExpectTx(unsigned long long* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smemAddr(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbarArrive(unsigned long long* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smemAddr(bar)) : "memory");
}
__device__ __forceinline__ bool mbarTry(unsigned long long* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smemAddr(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// The same with a suspend-time hint: the warp sleeps in hardware until the
// phase completes or about that many nanoseconds have passed, instead of
// spinning through issue slots that the working warps need.
__device__ __forceinline__ bool mbarTrySleep(unsigned long long* bar, uint32_t parity, uint32_t ns) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smemAddr(bar)), "r"(parity), "r"(ns)
        : "memory");
    return ok != 0;
}
// Bounded wait.  Returns false (and marks the CTA dead) when the barrier did
// not complete in time or another thread of the CTA already gave up.
__device__ __forceinline__ bool mbarWait(unsigned long long* bar, uint32_t parity, int* dead, int* errFlag, int where) {
    if (mbarTry(bar, parity)) return true;
    const long long t0 = clock64();
    while (true) {
        if (mbarTrySleep(bar, parity, 20000u)) return true;
        if (*reinterpret_cast<volatile int*>(dead)) return false;
        if (clock64() - t0 > kWaitCycles) {
            *reinterpret_cast<volatile int*>(dead) = 1;
            atomicCAS(errFlag, 0, where);
            return false;
        }
    }
}

__device__ __forceinline__ void tmaLoad2d(void* dst, const CUtensorMap* map, unsigned long long* bar, int x, int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smemAddr(dst)), "l"(map), "r"(smemAddr(bar)), "r"(x), "r"(y)
        : "memory");
}
__device__ __forceinline__ void tmaLoad3d(void* dst, const CUtensorMap* map, unsigned long long* bar, int x, int y, int z) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(smemAddr(dst)), "l"(map), "r"(smemAddr(bar)), "r"(x), "r"(y), "r"(z)
        : "memory");
}

// Shared-memory matrix descriptor (128-byte swizzle, descriptor version 1).
// lbo/sbo in bytes.  K-major operands: sbo = 1024 (eight 128-byte rows),
// lbo unused (1).  MN-major operand (V): lbo = distance between 64-element
// column blocks, sbo = 1024 (eight keys).
__device__ __forceinline__ uint64_t makeDesc(uint32_t addr, uint32_t lboBytes, uint32_t sboBytes) {
    uint64_t d = (addr & 0x3FFFFu) >> 4;
    d |= static_cast<uint64_t>((lboBytes >> 4) & 0x3FFFu) << 16;
    d |= static_cast<uint64_t>((sboBytes >> 4) & 0x3FFFu) << 32;
    d |= 1ull << 46;       // version
    d |= 2ull << 61;       // SWIZZLE_128B
    return d;
}

// The two halves of a descriptor: the high word is the same for every tile of a
// layout, the low word is the start address (in 16-byte units) plus the LBO
// field, so that stepping through a tile is one integer add on the low word.
__device__ __forceinline__ uint32_t descHi(uint32_t sboBytes) { return ((sboBytes >> 4) & 0x3FFFu) | (1u << 14) | (2u << 29); }
__device__ __forceinline__ uint32_t descLo(uint32_t addr, uint32_t lboBytes) {
    return ((addr & 0x3FFFFu) >> 4) | (((lboBytes >> 4) & 0x3FFFu) << 16);
}
__device__ __forceinline__ uint64_t desc64(uint32_t lo, uint32_t hi) {
    uint64_t d;
    asm("mov.b64 %0, {%1, %2};" : "=l"(d) : "r"(lo), "r"(hi));
    return d;
}

__device__ __forceinline__ void umma(uint32_t tmemD, uint64_t descA, uint64_t descB, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}"
        ::"r"(tmemD), "l"(descA), "l"(descB), "r"(idesc), "r"(accumulate), "r"(0u)
        : "memory");
}
// Same with the A operand read from tensor memory (row = lane, two 16-bit
// elements of K per 32-bit column).
__device__ __forceinline__ void ummaTs(uint32_t tmemD, uint32_t tmemA, uint64_t descB, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, {%5, %5, %5, %5}, p;\n\t}"
        ::"r"(tmemD), "r"(tmemA), "l"(descB), "r"(idesc), "r"(accumulate), "r"(0u)
        : "memory");
}
__device__ __forceinline__ void ummaCommit(unsigned long long* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smemAddr(bar)) : "memory");
}
__device__ __forceinline__ void tcFenceBefore() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tcFenceAfter() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void tmemLd32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
        "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
// The same load without the wait, to keep several loads in flight.
__device__ __forceinline__ void tmemLd32NoWait(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
        "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr));
}
__device__ __forceinline__ void tmemLdWait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmemSt32(uint32_t taddr, const uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
        "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
          "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
          "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
}
__device__ __forceinline__ void tmemSt16(uint32_t taddr, const uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
        "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
        : "memory");
}
__device__ __forceinline__ void tmemStWait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

template <bool BF16>
__device__ __forceinline__ uint32_t pack16(float lo, float hi) {
    if (BF16) {
        __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
        return *reinterpret_cast<uint32_t*>(&h);
    }
    __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&h);
}

__device__ __forceinline__ float ex2Approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// Visibility of key `key` for the row at sequence position `rowPos`.
struct MaskInfo {
    int lo, hi;      // keys [lo, hi) are visible to the row
    __device__ __forceinline__ MaskInfo(int ws, int seqLen, int rowPos, int causal)
        : lo(ws), hi(causal ? min(seqLen, rowPos + 1) : seqLen) {}
    // key = firstKey + i with i a compile-time constant in the callers' unrolled loops
    __device__ __forceinline__ bool visible(int key) const {
        return static_cast<unsigned>(key - lo) < static_cast<unsigned>(max(hi - lo, 0));
    }
};

// Maximum of 32 raw scores; EDGE tiles mask invisible keys.
template <bool EDGE>
__device__ __forceinline__ float quarterRowMax(const uint32_t (&r)[32], const MaskInfo& mk, int firstKey) {
    float m4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
    for (int i = 0; i < 32; ++i) {
        float a = __uint_as_float(r[i]);
        if (EDGE && !mk.visible(firstKey + i)) a = -INFINITY;
        m4[i & 3] = fmaxf(m4[i & 3], a);
    }
    return fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3]));
}

// Maximum of 64 raw scores (two loaded chunks); EDGE tiles mask invisible keys.
template <bool EDGE>
__device__ __forceinline__ float halfRowMax(const uint32_t (&r0)[32], const uint32_t (&r1)[32], const MaskInfo& mk, int firstKey) {
    float m4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
    for (int i = 0; i < 32; ++i) {
        float a = __uint_as_float(r0[i]), b = __uint_as_float(r1[i]);
        if (EDGE) {
            if (!mk.visible(firstKey + i)) a = -INFINITY;
            if (!mk.visible(firstKey + 32 + i)) b = -INFINITY;
        }
        m4[i & 3] = fmaxf(m4[i & 3], fmaxf(a, b));
    }
    return fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3]));
}

// 32 scores -> 16 packed weight pairs (w[0..15]) and, with LO (bfloat16 only),
// the 16 pairs of their low-order parts (w[16..31]); returns the sum of the weights.
template <bool BF16, bool LO, bool EDGE>
__device__ __forceinline__ float weights32(const uint32_t (&r)[32], uint32_t (&w)[32], float scaleLog2, float negM,
                                           const MaskInfo& mk, int firstKey) {
    float s4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int i = 0; i < 32; i += 2) {
        float x0 = fmaf(__uint_as_float(r[i]), scaleLog2, negM);
        float x1 = fmaf(__uint_as_float(r[i + 1]), scaleLog2, negM);
        if (EDGE) {
            if (!mk.visible(firstKey + i)) x0 = -INFINITY;
            if (!mk.visible(firstKey + i + 1)) x1 = -INFINITY;
        }
        const float p0 = ex2Approx(x0), p1 = ex2Approx(x1);
        s4[(i >> 1) & 3] += p0 + p1;
        w[i / 2] = pack16<BF16>(p0, p1);
        if (LO) {
            // bfloat16 keeps 8 significant bits of a weight; the remainder goes into a
            // second operand so that P_hi + P_lo carries 16 bits
            const float h0 = __uint_as_float(w[i / 2] << 16);
            const float h1 = __uint_as_float(w[i / 2] & 0xFFFF0000u);
            w[16 + i / 2] = pack16<true>(p0 - h0, p1 - h1);
        }
    }
    return (s4[0] + s4[1]) + (s4[2] + s4[3]);
}

constexpr int kSoftmaxThreads = 512;                   // four threads per row
constexpr int kKProducerWarp = 16, kVProducerWarp = 17, kMmaWarp = 18;
constexpr int kThreads = kSoftmaxThreads + 96;

template <bool BF16>
__global__ void __launch_bounds__(kThreads, 1)
prefillTcKernel(const __grid_constant__ CUtensorMap mapQ, const __grid_constant__ CUtensorMap mapK,
                const __grid_constant__ CUtensorMap mapV, const __grid_constant__ PrefillParams p, float scaleLog2,
                int* errFlag) {
    // Dynamic shared memory starts on a 1024-byte boundary (the swizzle atoms
    // need that); if it ever does not, give up cleanly instead of computing garbage.
    extern __shared__ __align__(1024) unsigned char rawSmem[];
    Smem* s = reinterpret_cast<Smem*>(rawSmem);
    if ((smemAddr(rawSmem) & 1023u) != 0) {
        if (threadIdx.x == 0) atomicCAS(errFlag, 0, 20);
        return;
    }

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tile = static_cast<int>(gridDim.x) - 1 - static_cast<int>(blockIdx.x);   // long tiles first
    const int head = blockIdx.y, seq = blockIdx.z;
    const int qLen = prefillMeta(p, 2, seq);
    if (tile * kRows >= qLen) return;
    if (*reinterpret_cast<volatile int*>(errFlag) != 0) return;       // an earlier CTA gave up: do not pile up waits
    const int G = p.heads / p.kvHeads, kvh = head / G;
    const int qStart = prefillMeta(p, 1, seq), seqLen = prefillMeta(p, 0, seq), ws = prefillMeta(p, 4, seq);
    const int rowBase = prefillMeta(p, 3, seq) + tile * kRows;        // first row of the tile in q/out
    const int rowsValid = min(kRows, qLen - tile * kRows);
    const int firstPos = qStart + tile * kRows;                       // sequence position of row 0
    const int lastPos = firstPos + rowsValid - 1;
    // Key tiles tileLo .. tileLo + nT - 1 hold every key a row of this tile may see.
    const int keyEnd = p.causal ? min(seqLen, lastPos + 1) : seqLen;  // exclusive
    const int tileLo = ws / kKeys;
    const int nT = keyEnd > ws ? (keyEnd - 1) / kKeys - tileLo + 1 : 0;
    // Fewest keys any row of the tile sees.  A bfloat16 weight keeps 8 significant bits; on a
    // row with few keys (large weights) that alone can cost more than 2e-3 on unit-variance
    // values, so such tiles carry the weights as two bfloat16 operands (16 bits).  Rows with
    // hundreds of keys have weights small enough for 8 bits, as in every bfloat16 attention
    // kernel.  exactWeights: 0 never, 1 short rows, 2 always.
    const int fewest = p.causal ? firstPos + 1 - ws : seqLen - ws;
    const bool useLo = BF16 && (p.exactWeights == 2 || (p.exactWeights == 1 && fewest < kShortRowKeys));

    if (threadIdx.x == kKProducerWarp * 32) {
        asm volatile("prefetch.tensormap [%0];" ::"l"(&mapQ) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&mapK) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&mapV) : "memory");
    }
    TRACE(0, 31, 0);                                   // CTA start (instrumented build)
    if (threadIdx.x == 0) {
        mbarInit(&s->qFull, 1);
        for (int i = 0; i < kKStages; ++i) { mbarInit(&s->kFull[i], 1); mbarInit(&s->kEmpty[i], 1); }
        for (int i = 0; i < kVStages; ++i) { mbarInit(&s->vFull[i], 1); mbarInit(&s->vEmpty[i], 1); }
        for (int i = 0; i < 2; ++i) { mbarInit(&s->sFull[i], 1); mbarInit(&s->maxReady[i], kSoftmaxThreads); }
        mbarInit(&s->pFull, kSoftmaxThreads);
        mbarInit(&s->pvDone, 1);
        mbarInit(&s->sumReady, kSoftmaxThreads);
        s->dead = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == kMmaWarp) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smemAddr(&s->tmemBase)), "r"(512u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tcFenceBefore();
    __syncthreads();
    tcFenceAfter();
    const uint32_t tmem = s->tmemBase;
    TRACE(0, 31, 1);                                   // barriers and tensor memory ready
    const uint32_t tmemS[2] = {tmem, tmem + 128u};
    const uint32_t tmemO = tmem + 256u;

    // Row of the pool (block * kv_heads * block_size space) of the 16-token piece `lane`
    // of key tile j; lanes 0-7 of a producer warp fetch one piece each.
    const int32_t* table = p.tables + static_cast<int64_t>(seq) * p.maxNumBlocks;
    const int tilesPerPage = p.blockSize / 16;
    auto pieceRow = [&](int j) {
        const int t16 = (tileLo + j) * (kKeys / 16) + lane;
        const int page = min(t16 / tilesPerPage, p.maxNumBlocks - 1);
        const int blk = min(max(table[page], 0), p.poolBlocks - 1);
        return (blk * p.kvHeads + kvh) * p.blockSize + (t16 % tilesPerPage) * 16;
    };

    if (warp == kKProducerWarp) {
        // ------------------------------------------------------------ Q and K producer
        if (nT > 0) {
            if (lane == 0) {
                mbarExpectTx(&s->qFull, kTileBytes);
                tmaLoad3d(s->q, &mapQ, &s->qFull, 0, head, rowBase);
                tmaLoad3d(s->q + kHalfBytes, &mapQ, &s->qFull, 64, head, rowBase);
            }
            bool ok = true;
            for (int j = 0; j < nT && ok; ++j) {
                const int st = j % kKStages;
                const int row = lane < kKeys / 16 ? pieceRow(j) : 0;
                if (j >= kKStages) ok = mbarWait(&s->kEmpty[st], ((j / kKStages) - 1) & 1, &s->dead, errFlag, 1);
                ok = __all_sync(0xFFFFFFFFu, ok);
                if (!ok) break;
                if (lane == 0) mbarExpectTx(&s->kFull[st], kTileBytes);
                __syncwarp();
                if (lane < kKeys / 16) {
                    tmaLoad2d(s->k[st] + lane * 2048, &mapK, &s->kFull[st], 0, row);
                    tmaLoad2d(s->k[st] + kHalfBytes + lane * 2048, &mapK, &s->kFull[st], 64, row);
                }
            }
        }
    } else if (warp == kVProducerWarp) {
        // ------------------------------------------------------------ V producer
        bool ok = true;
        for (int j = 0; j < nT && ok; ++j) {
            const int st = j % kVStages;
            const int row = lane < kKeys / 16 ? pieceRow(j) : 0;
            if (j >= kVStages) ok = mbarWait(&s->vEmpty[st], ((j / kVStages) - 1) & 1, &s->dead, errFlag, 13);
            ok = __all_sync(0xFFFFFFFFu, ok);
            if (!ok) break;
            if (lane == 0) mbarExpectTx(&s->vFull[st], kTileBytes);
            __syncwarp();
            if (lane < kKeys / 16) {
                tmaLoad2d(s->v[st] + lane * 2048, &mapV, &s->vFull[st], 0, row);
                tmaLoad2d(s->v[st] + kHalfBytes + lane * 2048, &mapV, &s->vFull[st], 64, row);
            }
        }
    } else if (warp == kMmaWarp) {
        // ------------------------------------------------------------ MMA issuer
        // Tensor-core instructions of one thread execute in issue order: S of tile j+2 is
        // written over P of tile j right behind P V of tile j without a wait in between.
        if (lane == 0 && nT > 0) {
            const uint32_t fmt = BF16 ? 1u : 0u;
            // D = f32, A/B = bf16|f16, M = 128, N = 128; B of the second product is MN-major.
            const uint32_t idescS = (1u << 4) | (fmt << 7) | (fmt << 10) | ((128u >> 3) << 17) | ((128u >> 4) << 24);
            // P has the type of the cache: a float16 P against bfloat16 V is rejected by
            // the hardware (illegal instruction), the two operands must agree.
            const uint32_t idescO = idescS | (1u << 16);
            const uint32_t hiK = descHi(1024);                      // K-major tiles and the MN-major V tile share it
            const uint32_t qLo = descLo(smemAddr(s->q), 16);
            bool ok = mbarWait(&s->qFull, 0, &s->dead, errFlag, 2);
            auto issueQK = [&](int j) {
                const int st = j % kKStages;
                ok = mbarWait(&s->kFull[st], (j / kKStages) & 1, &s->dead, errFlag, 3);
                if (!ok) return;
                tcFenceAfter();
                const uint32_t kLo = descLo(smemAddr(s->k[st]), 16);
#pragma unroll
                for (int ks = 0; ks < kHd / 16; ++ks) {
                    const uint32_t off = ((ks >> 2) * kHalfBytes + (ks & 3) * 32) >> 4;
                    umma(tmemS[j & 1], desc64(qLo + off, hiK), desc64(kLo + off, hiK), idescS, ks > 0);
                }
                ummaCommit(&s->sFull[j & 1]);
                ummaCommit(&s->kEmpty[st]);
                TRACE(2, j, 3);
            };
            if (ok) issueQK(0);
            if (ok && nT > 1) issueQK(1);
            for (int j = 0; j < nT && ok; ++j) {
                const int st = j % kVStages;
                TRACE(2, j, 0);
                ok = mbarWait(&s->pFull, j & 1, &s->dead, errFlag, 5);
                if (ok) ok = mbarWait(&s->vFull[st], (j / kVStages) & 1, &s->dead, errFlag, 6);
                if (!ok) break;
                tcFenceAfter();
                TRACE(2, j, 1);
                const uint32_t vLo = descLo(smemAddr(s->v[st]), kHalfBytes);
                // P of keys 32c .. 32c+31 sits in columns 32c .. 32c+15 (and, with the low-order
                // pass, its remainder in columns 32c+16 .. 32c+31) of the S buffer
#pragma unroll
                for (int ks = 0; ks < kKeys / 16; ++ks) {
                    const uint32_t pCol = tmemS[j & 1] + 32u * (ks >> 1) + 8u * (ks & 1);
                    ummaTs(tmemO, pCol, desc64(vLo + ks * 128, hiK), idescO, (j > 0 || ks > 0) ? 1u : 0u);
                }
                if (useLo) {
#pragma unroll
                    for (int ks = 0; ks < kKeys / 16; ++ks) {
                        const uint32_t pCol = tmemS[j & 1] + 32u * (ks >> 1) + 8u * (ks & 1) + 16u;
                        ummaTs(tmemO, pCol, desc64(vLo + ks * 128, hiK), idescO, 1u);
                    }
                }
                ummaCommit(&s->pvDone);
                ummaCommit(&s->vEmpty[st]);
                TRACE(2, j, 2);
                if (j + 2 < nT) issueQK(j + 2);
            }
        }
    } else {
        // ------------------------------------------------------------ softmax warps
        // Thread (t, cq): row t, key columns [32cq, 32cq + 32) of every key tile and output
        // columns [32cq, 32cq + 32).  Warps w, w+4, w+8, w+12 share the tensor-memory lanes
        // 32(w&3) .. +31 (a warp may only touch the lane quarter of its index modulo 4).
        const int cq = warp >> 2, t = (warp & 3) * 32 + lane;
        const int rowPos = firstPos + t;
        const uint32_t laneBase = static_cast<uint32_t>((warp & 3) * 32) << 16;
        const uint32_t oBase = tmemO + laneBase + 32u * cq;
        const MaskInfo mk(ws, seqLen, rowPos, p.causal);
        float mUsed = -INFINITY, l = 0.f;
        bool ok = true;
        for (int j = 0; j < nT && ok; ++j) {
            const int b = j & 1;
            const int k0 = (tileLo + j) * kKeys;
            const int kq = k0 + 32 * cq;                                    // first key of this thread's columns
            const uint32_t sBase = tmemS[b] + laneBase + 32u * cq;
            const bool edge = k0 < ws || k0 + kKeys > seqLen || (p.causal && k0 + kKeys - 1 > firstPos);
            TRACE((warp == 0 ? 0 : warp == 8 ? 1 : 99), j, 0);
            ok = mbarWait(&s->sFull[b], (j >> 1) & 1, &s->dead, errFlag, 7);
            if (!ok) break;
            tcFenceAfter();
            TRACE((warp == 0 ? 0 : warp == 8 ? 1 : 99), j, 1);
            uint32_t r[32];
            tmemLd32(sBase, r);
            TRACE((warp == 0 ? 0 : warp == 8 ? 1 : 99), j, 4);
            // maximum of the raw scores of this quarter row (the scale is positive)
            float tmax = (edge ? quarterRowMax<true>(r, mk, kq) : quarterRowMax<false>(r, mk, kq)) * scaleLog2;
            s->rowMax[b][cq][t] = tmax;
            mbarArrive(&s->maxReady[b]);
            TRACE((warp == 0 ? 0 : warp == 8 ? 1 : 99), j, 5);
            ok = mbarWait(&s->maxReady[b], (j >> 1) & 1, &s->dead, errFlag, 11);
            if (!ok) break;
            tmax = fmaxf(fmaxf(s->rowMax[b][0][t], s->rowMax[b][1][t]), fmaxf(s->rowMax[b][2][t], s->rowMax[b][3][t]));
            TRACE((warp == 0 ? 0 : warp == 8 ? 1 : 99), j, 2);
            bool raise = false;
            float corr = 1.f;
            if (j == 0) mUsed = tmax;
            else if (tmax > mUsed + kRescaleThreshold) {
                raise = true;
                corr = ex2Approx(mUsed - tmax);
                mUsed = tmax;
            }
            if (j >= 1 && __any_sync(0xFFFFFFFFu, raise)) {
                // O is still being added to by P V of tile j-1: wait for it, then rescale
                ok = mbarWait(&s->pvDone, (j - 1) & 1, &s->dead, errFlag, 8);
                if (!ok) break;
                tcFenceAfter();
                uint32_t o[32];
                tmemLd32(oBase, o);
#pragma unroll
                for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * corr);
                tmemSt32(oBase, o);
                l *= corr;
            }
            // the weights replace the scores in tensor memory: 16 columns of packed pairs
            // (plus 16 columns of their low-order parts where the tile needs 16-bit weights)
            const float negM = mUsed == -INFINITY ? 0.f : -mUsed;
            uint32_t w[32];
            if (useLo) {
                l += edge ? weights32<BF16, true, true>(r, w, scaleLog2, negM, mk, kq)
                          : weights32<BF16, true, false>(r, w, scaleLog2, negM, mk, kq);
                tmemSt32(sBase, w);
            } else {
                l += edge ? weights32<BF16, false, true>(r, w, scaleLog2, negM, mk, kq)
                          : weights32<BF16, false, false>(r, w, scaleLog2, negM, mk, kq);
                tmemSt16(sBase, w);
            }
            tmemStWait();
            TRACE((warp == 0 ? 0 : warp == 8 ? 1 : 99), j, 10);
            if (k0 + kKeys > seqLen) {
                // rows of V past the end of the sequence may hold anything: zero them
                const int st = j % kVStages;
                ok = mbarWait(&s->vFull[st], (j / kVStages) & 1, &s->dead, errFlag, 9);
                if (!ok) break;
                if (k0 + t >= seqLen) {
#pragma unroll
                    for (int c16 = 0; c16 < 4; ++c16)
                        *reinterpret_cast<uint4*>(s->v[st] + (cq >> 1) * kHalfBytes + t * 128 + ((cq & 1) * 4 + c16) * 16) =
                            make_uint4(0u, 0u, 0u, 0u);
                }
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            }
            tcFenceBefore();
            mbarArrive(&s->pFull);
            TRACE((warp == 0 ? 0 : warp == 8 ? 1 : 99), j, 3);
        }
        // epilogue: O / l to global memory
        if (ok) {
            s->rowMax[nT & 1][cq][t] = l;            // the buffer the last tile did not use
            mbarArrive(&s->sumReady);
            ok = mbarWait(&s->sumReady, 0, &s->dead, errFlag, 12);
        }
        if (ok && nT > 0) ok = mbarWait(&s->pvDone, (nT - 1) & 1, &s->dead, errFlag, 10);
        TRACE((warp == 0 ? 0 : warp == 8 ? 1 : 99), 31, 2);   // last PV done
        if (ok) {
            tcFenceAfter();
            const float lt = (s->rowMax[nT & 1][0][t] + s->rowMax[nT & 1][1][t]) + (s->rowMax[nT & 1][2][t] + s->rowMax[nT & 1][3][t]);
            const float inv = (nT > 0 && lt > 0.f) ? 1.f / lt : 0.f;
            // The Q tile is no longer read: stage this warp's 32 rows x 64 bytes there (16-byte
            // chunks XOR-swizzled by row), then write them out eight rows per instruction,
            // 64 contiguous bytes per row.
            unsigned char* stage = s->q;
            uint32_t o[32];
            if (nT > 0) tmemLd32(oBase, o);
#pragma unroll
            for (int q4 = 0; q4 < 4; ++q4) {
                uint32_t wv[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float a = nT > 0 ? __uint_as_float(o[8 * q4 + 2 * e]) * inv : 0.f;
                    const float bb = nT > 0 ? __uint_as_float(o[8 * q4 + 2 * e + 1]) * inv : 0.f;
                    wv[e] = pack16<BF16>(a, bb);
                }
                *reinterpret_cast<uint4*>(stage + t * 256 + (((cq * 4 + q4) ^ (t & 7)) << 4)) =
                    make_uint4(wv[0], wv[1], wv[2], wv[3]);
            }
            __syncwarp();
            const int rowLo = (warp & 3) * 32;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int row = rowLo + 8 * i + (lane >> 2), chunk = cq * 4 + (lane & 3);
                if (row < rowsValid) {
                    const uint4 v = *reinterpret_cast<const uint4*>(stage + row * 256 + ((chunk ^ (row & 7)) << 4));
                    unsigned char* out = static_cast<unsigned char*>(p.out) +
                                         ((static_cast<int64_t>(rowBase) + row) * p.heads + head) * kHd * 2;
                    *reinterpret_cast<uint4*>(out + chunk * 16) = v;
                }
            }
        }
    }

    TRACE((warp == 0 ? 0 : warp == 8 ? 1 : 99), 31, 3);       // output stored
    tcFenceBefore();
    __syncthreads();
#ifdef PAM_PREFILL_TRACE
    if (blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0)
        for (int i = threadIdx.x; i < kTraceRoles * kTraceTiles * kTraceEvents; i += kThreads) gTrace[i] = s->trace[i];
#endif
    if (warp == kMmaWarp) {
        tcFenceAfter();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512u) : "memory");
    }
}

// cuTensorMapEncodeTiled through the runtime's driver entry point (no link
// against libcuda).
using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                              const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                              CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeFn encodeFn() {
    static EncodeFn fn = nullptr;
    if (!fn) {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeFn>(ptr);
    }
    return fn;
}

}  // namespace

bool prefillTensorPathApplies(const PrefillParams& p) {
    return (p.dtype == kF16 || p.dtype == kBF16) && p.headDim == kHd && p.blockSize % 16 == 0 && p.heads % p.kvHeads == 0 &&
           (reinterpret_cast<uintptr_t>(p.q) & 15) == 0 && (reinterpret_cast<uintptr_t>(p.out) & 15) == 0 &&
           (reinterpret_cast<uintptr_t>(p.kPool) & 15) == 0 && (reinterpret_cast<uintptr_t>(p.vPool) & 15) == 0 &&
           p.poolBlocks > 0 && p.poolBlocks < (1 << 30) / (p.kvHeads * p.blockSize);
}

cudaError_t launchPrefillTensor(const PrefillParams& p, int totalRows, int* errFlag, cudaStream_t stream, int* launches) {
    EncodeFn encode = encodeFn();
    if (!encode) return cudaErrorNotSupported;
    const CUtensorMapDataType dt = p.dtype == kBF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    CUtensorMap mapQ, mapK, mapV;
    {
        // Q: [rows][heads][128]; a box is 64 dims x 1 head x 128 rows
        cuuint64_t dims[3] = {static_cast<cuuint64_t>(kHd), static_cast<cuuint64_t>(p.heads), static_cast<cuuint64_t>(totalRows)};
        cuuint64_t strides[2] = {static_cast<cuuint64_t>(kHd) * 2, static_cast<cuuint64_t>(p.heads) * kHd * 2};
        cuuint32_t box[3] = {64, 1, static_cast<cuuint32_t>(kRows)};
        cuuint32_t es[3] = {1, 1, 1};
        if (encode(&mapQ, dt, 3, const_cast<void*>(p.q), dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return cudaErrorInvalidValue;
    }
    const cuuint64_t poolRows = static_cast<cuuint64_t>(p.poolBlocks) * p.kvHeads * p.blockSize;
    for (int which = 0; which < 2; ++which) {
        // pools: [block * kv_head * slot][128]; a box is 64 dims x 16 rows (one half of a 16-token page piece)
        cuuint64_t dims[2] = {static_cast<cuuint64_t>(kHd), poolRows};
        cuuint64_t strides[1] = {static_cast<cuuint64_t>(kHd) * 2};
        cuuint32_t box[2] = {64, 16};
        cuuint32_t es[2] = {1, 1};
        if (encode(which ? &mapV : &mapK, dt, 2, const_cast<void*>(which ? p.vPool : p.kPool), dims, strides, box, es,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return cudaErrorInvalidValue;
    }
    const size_t smem = sizeof(Smem);
    const float scaleLog2 = (1.0f / sqrtf(static_cast<float>(p.headDim))) * kLog2e;
    dim3 grid(static_cast<unsigned>((p.maxQLen + kRows - 1) / kRows), static_cast<unsigned>(p.heads), static_cast<unsigned>(p.numSeqs));
    cudaError_t e;
    if (p.dtype == kBF16) {
        e = cudaFuncSetAttribute(prefillTcKernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
        if (e != cudaSuccess) return e;
        prefillTcKernel<true><<<grid, kThreads, smem, stream>>>(mapQ, mapK, mapV, p, scaleLog2, errFlag);
    } else {
        e = cudaFuncSetAttribute(prefillTcKernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
        if (e != cudaSuccess) return e;
        prefillTcKernel<false><<<grid, kThreads, smem, stream>>>(mapQ, mapK, mapV, p, scaleLog2, errFlag);
    }
    if (launches) *launches += 1;
    return cudaGetLastError();
}

}  // namespace pam

#ifdef PAM_PREFILL_TRACE
extern "C" int pamc_debug_trace_read(long long* out) {
    cudaDeviceSynchronize();
    cudaMemcpyFromSymbol(out, pam::gTrace, sizeof(long long) * pam::kTraceRoles * pam::kTraceTiles * pam::kTraceEvents);
    return pam::kTraceRoles * pam::kTraceTiles * pam::kTraceEvents;
}
#endif
