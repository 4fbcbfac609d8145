// Chunked causal prefill on the 5th-generation tensor cores (sm_100a):
// tcgen05.mma with accumulators in tensor memory, operands staged in shared
// memory by TMA, for bfloat16 / float16 KV with head_dim 128 and a block size
// that is a multiple of 16.
//
// Semantics are those of prefillGeneralKernel (paged_attention_tiled,
// kernels.metal:693-765, plus the chunk rows of
// PagedAttentionEngine.swift:740-756).
//
// The kernel is persistent: one CTA per multiprocessor walks the work items
// round robin, longest items first.  An item is a pair of tiles of 128 query
// rows of one sequence that share a KV head: the same rows of two neighbouring
// query heads when the number of query heads per KV head is even (both tiles
// then see the same keys), else two consecutive tiles of one head.  It walks the
// key tiles (128 keys each) its rows can see, and every key and value tile is
// fetched once for both query tiles.  Each query tile belongs to one of two softmax groups, with
// its own S buffer and accumulator O in tensor memory (4 x 128 columns): while
// one group turns its S into the weights P, the tensor pipe works for the
// other.
//
//   warps 0-3, 4-7       softmax groups 0 and 1: thread t of a group owns query
//                        row t of the group's tile, all 128 key columns of a key
//                        tile, in registers (no exchange between threads).
//                        Scores are scaled, masked (causal, window start,
//                        sequence end) only on edge tiles.  The running maximum
//                        is only raised when it grows by more than 2^8 (the
//                        result is exact either way, the final division uses
//                        the same reference), in which case O is rescaled in
//                        tensor memory.  The weights go back to tensor memory
//                        over the scores, in the cache type (tcgen05.st); for
//                        bfloat16, on rows that see few keys, as two operands
//                        P_hi + P_lo (16 significant bits together) and twice
//                        the PV instructions, because 8-bit weights alone miss
//                        the 2e-3 bound there.  Thread 0 of a group fetches the
//                        group's next query tile by TMA during the last key
//                        tile of the current one.  At the end of an item the
//                        thread leaves its row's sum in shared memory and goes
//                        on with the next item.
//   warp 8               TMA producer of K: per key tile 8 pages (each 16 rows x
//                        256 B, fetched as two 128-byte-swizzled boxes, one page
//                        per lane) into a ring; completion on mbarriers.
//   warp 9               TMA producer of V, its own ring.
//   warp 10              MMA issuer (one elected lane): for every key tile and
//                        group, O += P V (P read from tensor memory, V as an
//                        MN-major operand straight from its row-major pages)
//                        and right behind it S = Q K^T of the group's next key
//                        tile (8 x tcgen05.mma 128x128x16, both operands from
//                        shared memory); tcgen05.commit signals the mbarriers.
//   warps 12-15          output: once the last P V product of a group's tile is
//                        complete, O / l goes from tensor memory to a staging
//                        buffer in the layout of a TMA box and out with a TMA
//                        store, then the accumulator goes back to the MMA
//                        issuer.  This keeps the output off the softmax warps,
//                        which are the busiest.
//
// The service and output warps hand registers to the softmax warps (setmaxnreg).
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
constexpr int kKStages = 2, kVStages = 2;
constexpr int kTileBytes = kRows * kHd * 2;            // 32 KB: one [128][128] 16-bit tile
constexpr int kHalfBytes = kTileBytes / 2;             // one 64-column block
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kRescaleThreshold = 8.0f;
constexpr int kShortRowKeys = 256;
constexpr long long kWaitCycles = 400000000LL;         // ~0.2 s: the bound of a wait unless the launch gives its own

struct Smem {
    // tiles first: each 1024-byte aligned (swizzle atoms)
    unsigned char q[2][kTileBytes];            // the query tile of each softmax group
    unsigned char k[kKStages][kTileBytes];
    unsigned char v[kVStages][kTileBytes];
    unsigned char stage[kTileBytes];           // finished rows of one group on their way out (TMA box layout)
    unsigned long long qFull[2], kFull[kKStages], kEmpty[kKStages], vFull[kVStages], vEmpty[kVStages];
    unsigned long long sFull[2], pFull[2], oFull[2], oEmpty[2], lReady[2];   // one of each per softmax group
    float rowL[2][kRows];                      // [group][row]: sum of the weights of the item just finished
    uint32_t tmemBase;
    int dead;
};

static_assert(sizeof(Smem) <= 227 * 1024, "the CTA's shared memory must fit the 227 KB a block may opt into");

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
__device__ __forceinline__ bool mbarWait(unsigned long long* bar, uint32_t parity, int* dead, int* errFlag, long long limit, int where) {
    if (mbarTry(bar, parity)) return true;
    const long long t0 = clock64();
    while (true) {
        if (mbarTrySleep(bar, parity, 20000u)) return true;
        if (*reinterpret_cast<volatile int*>(dead)) return false;
        if (clock64() - t0 > limit) {
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

__device__ __forceinline__ void tmaStore3d(const CUtensorMap* map, const void* src, int x, int y, int z) {
    asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];"
                 ::"l"(map), "r"(smemAddr(src)), "r"(x), "r"(y), "r"(z)
                 : "memory");
}

// Shared-memory matrix descriptors (128-byte swizzle, descriptor version 1): start address,
// leading and stride byte offsets in 16-byte units.  K-major operands: stride offset 1024
// (eight 128-byte rows), leading offset unused.  MN-major operand (V): leading offset =
// distance between 64-element column blocks, stride offset 1024 (eight keys).
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
// True in exactly one lane of a converged warp.
__device__ __forceinline__ bool electOne() {
    uint32_t pred;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "elect.sync _|p, 0xFFFFFFFF;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(pred));
    return pred != 0;
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

// Keys [lo, hi) are visible to the row at sequence position `rowPos`.
struct MaskInfo {
    int lo, hi;
    __device__ __forceinline__ MaskInfo(int ws, int seqLen, int rowPos, int causal)
        : lo(ws), hi(causal ? min(seqLen, rowPos + 1) : seqLen) {}
};

// Edge tiles only: the scores of invisible keys (key firstKey + i for score i) become -inf,
// after which the tile goes through the same code as an inner tile.
__device__ __forceinline__ void maskScores(uint32_t (&r)[32], const MaskInfo& mk, int firstKey) {
    const int a = mk.lo - firstKey, b = mk.hi - firstKey;      // visible: a <= i < b
    if (a <= 0) {
        // the usual case (the causal diagonal, the end of the sequence): an upper bound only
#pragma unroll
        for (int i = 0; i < 32; ++i)
            if (i >= b) r[i] = 0xFF800000u;
    } else {
#pragma unroll
        for (int i = 0; i < 32; ++i)
            if (i < a || i >= b) r[i] = 0xFF800000u;
    }
}

__device__ __forceinline__ float max3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}
// Two float lanes in one 64-bit register pair (packed single-precision instructions).
__device__ __forceinline__ unsigned long long pack2(float lo, float hi) {
    unsigned long long v;
    asm("mov.b64 %0, {%1, %2};" : "=l"(v) : "f"(lo), "f"(hi));
    return v;
}
__device__ __forceinline__ void unpack2(unsigned long long v, float& lo, float& hi) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ unsigned long long fma2(unsigned long long a, unsigned long long b, unsigned long long c) {
    unsigned long long d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}
__device__ __forceinline__ unsigned long long add2(unsigned long long a, unsigned long long b) {
    unsigned long long d;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}

// Maximum of 32 raw scores (masked ones are -inf already).
__device__ __forceinline__ float quarterRowMax(const uint32_t (&r)[32]) {
    float m4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
    for (int i = 0; i < 32; i += 2) m4[(i >> 1) & 3] = max3(m4[(i >> 1) & 3], __uint_as_float(r[i]), __uint_as_float(r[i + 1]));
    return fmaxf(max3(m4[0], m4[1], m4[2]), m4[3]);
}

// Scores r[BEGIN .. END) of a thread's 32 -> packed weight pairs w[BEGIN/2 .. END/2) and,
// with LO (bfloat16 only), the pairs of their low-order parts in w[16 + BEGIN/2 ..);
// returns the sum of the weights.  Masked scores are -inf and give weight 0.  (The loop is
// kept to five instructions per pair: with one warp per group on each scheduler the
// instruction count is what limits it; an integer-only pack and polynomial exponentials
// for part of the pairs, which relieve the special-function pipe, both made it slower.)
template <bool BF16, bool LO, int BEGIN, int END>
__device__ __forceinline__ float weightsRange(const uint32_t (&r)[32], uint32_t (&w)[32], float scaleLog2, float negM) {
    const unsigned long long scale2 = pack2(scaleLog2, scaleLog2), negM2 = pack2(negM, negM);
    unsigned long long acc[2] = {0ull, 0ull};
#pragma unroll
    for (int i = BEGIN; i < END; i += 2) {
        float x0, x1;
        unpack2(fma2(pack2(__uint_as_float(r[i]), __uint_as_float(r[i + 1])), scale2, negM2), x0, x1);
        const float p0 = ex2Approx(x0), p1 = ex2Approx(x1);
        acc[(i >> 1) & 1] = add2(acc[(i >> 1) & 1], pack2(p0, p1));
        w[i / 2] = pack16<BF16>(p0, p1);
        if (LO) {
            // bfloat16 keeps 8 significant bits of a weight; the remainder goes into a
            // second operand so that P_hi + P_lo carries 16 bits
            const float h0 = __uint_as_float(w[i / 2] << 16);
            const float h1 = __uint_as_float(w[i / 2] & 0xFFFF0000u);
            w[16 + i / 2] = pack16<true>(p0 - h0, p1 - h1);
        }
    }
    float s0, s1, s2, s3;
    unpack2(acc[0], s0, s1);
    unpack2(acc[1], s2, s3);
    return (s0 + s1) + (s2 + s3);
}

constexpr int kGroupThreads = 128;                     // one thread per query row
constexpr int kSoftmaxWarps = 8;                       // two groups of four warps
constexpr int kKProducerWarp = 8, kVProducerWarp = 9, kMmaWarp = 10, kIdleWarp = 11, kOutputWarp0 = 12;
constexpr int kThreads = (kSoftmaxWarps + 8) * 32;     // softmax, service and output warpgroups

// One unit of work: two tiles of 128 query rows of one sequence under one KV head (the same
// rows of two heads, or two consecutive tiles of one head: see loadItem).
// Softmax group x owns tile x of the pair: its own query tile, S buffer and accumulator;
// the key and value tiles are fetched once for both.
struct Item {
    int head, headStep, seq, kvh; // group x works on head + x * headStep
    __device__ __forceinline__ int headOf(int x) const { return head + x * headStep; }
    int tileLo, nT;              // key tiles tileLo .. tileLo + nT - 1 hold every key a row of the pair may see
    int nTg[2];                  // ... a row of group x may see (0: the group has no rows, or they see nothing)
    int rowBase[2], rowsValid[2];// first row in q/out, rows that exist
    int firstPos[2];             // sequence position of a group's row 0
    int seqLen, ws;
    bool useLo[2];
    const int32_t* table;
};

// Work item `w` of the launch.  Items are numbered pair-major with the last (longest) pairs
// first and the head running fastest, so that the CTAs working side by side share the keys
// of one KV head through L2 and the short items fill the end of the launch.  Returns false
// when the sequence has no rows in that pair.
// n / d and n % d for 0 <= n < 2^22, 0 < d, through the float reciprocal of d (a division
// by a run-time value is some twenty instructions, and the roles of the kernel split item
// indices at every item boundary on their critical paths).
__device__ __forceinline__ int fastDivMod(int n, int d, float inv, int& rem) {
    int q = __float2int_rz(__int2float_rn(n) * inv);
    int r = n - q * d;
    if (r < 0) {
        --q;
        r += d;
    } else if (r >= d) {
        ++q;
        r -= d;
    }
    rem = r;
    return q;
}

__device__ __forceinline__ bool loadItem(const PrefillParams& p, int w, int numPairs, Item& it) {
    // pairHeads: the two groups take the same query tile of two neighbouring heads of one KV
    // head (equal work for both); else two consecutive query tiles of one head
    const int heads = p.pairHeads ? p.heads / 2 : p.heads;
    const int per = p.numSeqs * heads, group = heads / p.kvHeads;
    int pairFromEnd, rem, unused, h;
    if (p.fastItems) {
        pairFromEnd = fastDivMod(w, per, p.invPer, rem);
        it.seq = fastDivMod(rem, heads, p.invHeads, h);
        it.kvh = fastDivMod(h, group, p.invGroup, unused);
    } else {
        pairFromEnd = w / per;
        rem = w % per;
        it.seq = rem / heads;
        h = rem % heads;
        it.kvh = h / group;
    }
    it.head = p.pairHeads ? 2 * h : h;
    it.headStep = p.pairHeads ? 1 : 0;
    const int tilesPer = p.pairHeads ? 1 : 2, tileStep = p.pairHeads ? 0 : 1;
    const int pair = numPairs - 1 - pairFromEnd;
    const int qLen = prefillMeta(p, 2, it.seq);
    if (pair * tilesPer * kRows >= qLen) return false;
    const int qStart = prefillMeta(p, 1, it.seq), rowOff = prefillMeta(p, 3, it.seq);
    it.seqLen = prefillMeta(p, 0, it.seq);
    it.ws = prefillMeta(p, 4, it.seq);
    it.tileLo = it.ws / kKeys;
    it.nT = 0;
#pragma unroll
    for (int x = 0; x < 2; ++x) {
        const int first = (pair * tilesPer + x * tileStep) * kRows;  // first row of the tile within the launch's rows
        const int rows = min(kRows, qLen - first);
        it.rowsValid[x] = max(rows, 0);
        it.rowBase[x] = rowOff + first;
        it.firstPos[x] = qStart + first;
        it.nTg[x] = 0;
        it.useLo[x] = false;
        if (rows > 0) {
            const int lastPos = it.firstPos[x] + rows - 1;
            const int keyEnd = p.causal ? min(it.seqLen, lastPos + 1) : it.seqLen;  // exclusive
            it.nTg[x] = keyEnd > it.ws ? (keyEnd - 1) / kKeys - it.tileLo + 1 : 0;
            // Fewest keys any row of the tile sees.  A bfloat16 weight keeps 8 significant bits;
            // on a row with few keys (large weights) that alone can cost more than 2e-3 on
            // unit-variance values, so such tiles carry the weights as two bfloat16 operands
            // (16 bits).  Rows with hundreds of keys have weights small enough for 8 bits, as in
            // every bfloat16 attention kernel.  exactWeights: 0 never, 1 short rows, 2 always.
            const int fewest = p.causal ? it.firstPos[x] + 1 - it.ws : it.seqLen - it.ws;
            it.useLo[x] = p.exactWeights == 2 || (p.exactWeights == 1 && fewest < kShortRowKeys);
        }
        it.nT = max(it.nT, it.nTg[x]);
    }
    it.table = p.tables + static_cast<int64_t>(it.seq) * p.maxNumBlocks;
    return true;
}

// Position of a role in the CTA's stream of key tiles: item w, tile j of it, g tiles done
// before.  Every role walks the same stream, so g gives the stage and the phase parity of the
// K and V rings without any communication.
struct Cursor {
    int w, j, g;
    bool valid;
    Item it;
    __device__ __forceinline__ void seek(const PrefillParams& p, int total, int numPairs) {
        valid = false;
        while (w < total) {
            if (loadItem(p, w, numPairs, it) && it.nT > 0) {
                valid = true;
                return;
            }
            w += gridDim.x;
        }
    }
    __device__ __forceinline__ void init(const PrefillParams& p, int total, int numPairs) {
        w = blockIdx.x;
        j = g = 0;
        seek(p, total, numPairs);
    }
    __device__ __forceinline__ void nextTile(const PrefillParams& p, int total, int numPairs) {
        ++j;
        ++g;
        if (j == it.nT) {
            j = 0;
            w += gridDim.x;
            seek(p, total, numPairs);
        }
    }
};

template <bool BF16>
__global__ void __launch_bounds__(kThreads, 1)
prefillTcKernel(const __grid_constant__ CUtensorMap mapQ, const __grid_constant__ CUtensorMap mapK,
                const __grid_constant__ CUtensorMap mapV, const __grid_constant__ CUtensorMap mapO,
                const __grid_constant__ PrefillParams p, float scaleLog2, int* errFlag) {
    // Dynamic shared memory starts on a 1024-byte boundary (the swizzle atoms
    // need that); if it ever does not, give up cleanly instead of computing garbage.
    extern __shared__ __align__(1024) unsigned char rawSmem[];
    Smem* s = reinterpret_cast<Smem*>(rawSmem);
    if ((smemAddr(rawSmem) & 1023u) != 0) {
        if (threadIdx.x == 0) atomicCAS(errFlag, 0, 20);
        return;
    }

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int numTiles = (p.maxQLen + kRows - 1) / kRows;
    const int numPairs = p.pairHeads ? numTiles : (numTiles + 1) / 2;      // item rows of the launch
    const int total = numPairs * p.numSeqs * (p.pairHeads ? p.heads / 2 : p.heads);

    if (threadIdx.x == kKProducerWarp * 32) asm volatile("prefetch.tensormap [%0];" ::"l"(&mapK) : "memory");
    if (threadIdx.x == kVProducerWarp * 32) asm volatile("prefetch.tensormap [%0];" ::"l"(&mapV) : "memory");
    if (threadIdx.x == kOutputWarp0 * 32) asm volatile("prefetch.tensormap [%0];" ::"l"(&mapO) : "memory");
    if (threadIdx.x == 0 || threadIdx.x == kGroupThreads) asm volatile("prefetch.tensormap [%0];" ::"l"(&mapQ) : "memory");
    if (threadIdx.x == 0) {
        for (int i = 0; i < 2; ++i) {
            mbarInit(&s->qFull[i], 1);
            mbarInit(&s->sFull[i], 1);
            mbarInit(&s->pFull[i], kGroupThreads);
            mbarInit(&s->oFull[i], 1);
            mbarInit(&s->oEmpty[i], 1);
            mbarInit(&s->lReady[i], kGroupThreads);
        }
        for (int i = 0; i < kKStages; ++i) { mbarInit(&s->kFull[i], 1); mbarInit(&s->kEmpty[i], 1); }
        for (int i = 0; i < kVStages; ++i) { mbarInit(&s->vFull[i], 1); mbarInit(&s->vEmpty[i], 1); }
        // an earlier CTA gave up: do not pile up waits
        s->dead = *reinterpret_cast<volatile int*>(errFlag) != 0 ? 1 : 0;
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
    // tensor memory columns: S of group 0 and 1 at 0 and 128, their accumulators at 256 and 384
    auto tmemS = [&](int grp) { return tmem + 128u * static_cast<uint32_t>(grp); };
    auto tmemO = [&](int grp) { return tmem + 256u + 128u * static_cast<uint32_t>(grp); };
    const bool live = *reinterpret_cast<volatile int*>(&s->dead) == 0;
    const long long waitLimit = p.waitCycles > 0 ? p.waitCycles : kWaitCycles;

    // Row of the pool (block * kv_heads * block_size space) of the 16-token piece `lane`
    // of key tile j of an item; lanes 0-7 of a producer warp fetch one piece each.
    const int tilesPerPage = p.blockSize / 16;
    auto pieceRow = [&](const Item& it, int j) {
        const int t16 = (it.tileLo + j) * (kKeys / 16) + lane;
        const int page = min(t16 / tilesPerPage, p.maxNumBlocks - 1);
        const int blk = min(max(it.table[page], 0), p.poolBlocks - 1);
        return (blk * p.kvHeads + it.kvh) * p.blockSize + (t16 % tilesPerPage) * 16;
    };

    // Registers move from the service and output warps to the softmax warps, which hold a whole
    // row of scores: first statement of every role's branch, the same value in all four warps
    // of a warpgroup (the instruction is defined per warpgroup).  512 x 128 registers at
    // launch; the service warps give up 48 each, the output warps 64, the softmax warps take 56.
    if (warp == kKProducerWarp) {
        // ------------------------------------------------------------ K producer
        asm volatile("setmaxnreg.dec.sync.aligned.u32 80;");
        if (!live) goto done;
        Cursor c;
        c.init(p, total, numPairs);
        bool ok = true;
        while (c.valid && ok) {
            const int st = c.g % kKStages;
            const int row = lane < kKeys / 16 ? pieceRow(c.it, c.j) : 0;
            if (c.g >= kKStages) ok = mbarWait(&s->kEmpty[st], ((c.g / kKStages) - 1) & 1, &s->dead, errFlag, waitLimit, 1);
            ok = __all_sync(0xFFFFFFFFu, ok);
            if (!ok) break;
            if (lane == 0) mbarExpectTx(&s->kFull[st], kTileBytes);
            __syncwarp();
            if (lane < kKeys / 16) {
                tmaLoad2d(s->k[st] + lane * 2048, &mapK, &s->kFull[st], 0, row);
                tmaLoad2d(s->k[st] + kHalfBytes + lane * 2048, &mapK, &s->kFull[st], 64, row);
            }
            c.nextTile(p, total, numPairs);
        }
    } else if (warp == kVProducerWarp) {
        // ------------------------------------------------------------ V producer
        asm volatile("setmaxnreg.dec.sync.aligned.u32 80;");
        if (!live) goto done;
        Cursor c;
        c.init(p, total, numPairs);
        bool ok = true;
        while (c.valid && ok) {
            const int st = c.g % kVStages;
            const int row = lane < kKeys / 16 ? pieceRow(c.it, c.j) : 0;
            if (c.g >= kVStages) ok = mbarWait(&s->vEmpty[st], ((c.g / kVStages) - 1) & 1, &s->dead, errFlag, waitLimit, 13);
            ok = __all_sync(0xFFFFFFFFu, ok);
            if (!ok) break;
            // (test launches only: the CTA's first value tile is never fetched, so that the wait
            // for it runs out; see pamc_test_starve_prefill)
            const bool starved = p.starveV != 0 && c.g == 0;
            if (lane == 0 && !starved) mbarExpectTx(&s->vFull[st], kTileBytes);
            __syncwarp();
            if (lane < kKeys / 16 && !starved) {
                tmaLoad2d(s->v[st] + lane * 2048, &mapV, &s->vFull[st], 0, row);
                tmaLoad2d(s->v[st] + kHalfBytes + lane * 2048, &mapV, &s->vFull[st], 64, row);
            }
            c.nextTile(p, total, numPairs);
        }
    } else if (warp == kMmaWarp) {
        // ------------------------------------------------------------ MMA issuer
        // For every key tile of the stream, for each group that takes part in it: O += P V
        // once the group has released P, then right behind it S = Q K^T of the group's next
        // tile (tensor-core instructions execute in issue order: S is written over P after
        // the product that read it).  When the group's next tile is the first of the next
        // item and at most two tiles ahead in the stream (so that the key ring can hold it),
        // that S product is issued here as well; otherwise when the stream gets there.
        // All 32 lanes walk the loop, so that the descriptor arithmetic is uniform across the
        // warp (it then runs on the uniform datapath, where the tensor-core instructions take
        // their operands from); one elected lane issues the tensor-core instructions.
        asm volatile("setmaxnreg.dec.sync.aligned.u32 80;");
        if (!live) goto done;
        const bool leader = electOne();
        const uint32_t fmt = BF16 ? 1u : 0u;
        // D = f32, A/B = bf16|f16, M = 128, N = 128; B of the second product is MN-major.
        const uint32_t idescS = (1u << 4) | (fmt << 7) | (fmt << 10) | ((128u >> 3) << 17) | ((128u >> 4) << 24);
        // P has the type of the cache: a float16 P against bfloat16 V is rejected by
        // the hardware (illegal instruction), the two operands must agree.
        const uint32_t idescO = idescS | (1u << 16);
        const uint32_t hiK = descHi(1024);                      // K-major tiles and the MN-major V tile share it
        bool ok = true;
        Cursor c;
        c.init(p, total, numPairs);
        int steps0 = 0, steps1 = 0;          // group tiles done: phase of sFull, pFull, pvDone
        int items0 = 0, items1 = 0;          // items a group took part in: phase of qFull, oEmpty
        int qkOpen0 = 0, qkOpen1 = 0;        // per key stage: S products still to issue on the tile it holds
        bool ahead0 = false, ahead1 = false; // the S product of the group's next tile is already issued
        // S = Q_x K^T for tile j (global tile gTile) of item `it`
        auto issueQK = [&](int x, const Item& it, int j, int gTile) {
            const int st = gTile % kKStages;
            if (j == 0) ok = mbarWait(&s->qFull[x], (x ? items1 : items0) & 1, &s->dead, errFlag, waitLimit, 2);
            if (ok) ok = mbarWait(&s->kFull[st], (gTile / kKStages) & 1, &s->dead, errFlag, waitLimit, 3);
            ok = __all_sync(0xFFFFFFFFu, ok);
            if (!ok) return;
            tcFenceAfter();
            const uint32_t qLo = descLo(smemAddr(s->q[x]), 16);
            const uint32_t kLo = descLo(smemAddr(s->k[st]), 16);
            const uint32_t dS = tmemS(x);
            uint64_t dq[kHd / 16], dk[kHd / 16];
#pragma unroll
            for (int ks = 0; ks < kHd / 16; ++ks) {
                const uint32_t off = ((ks >> 2) * kHalfBytes + (ks & 3) * 32) >> 4;
                dq[ks] = desc64(qLo + off, hiK);
                dk[ks] = desc64(kLo + off, hiK);
            }
            // the key stage goes back to its producer behind the last S product on it
            int& open = st ? qkOpen1 : qkOpen0;
            if (open == 0) open = (j < it.nTg[0] ? 1 : 0) + (j < it.nTg[1] ? 1 : 0);
            --open;
            if (leader) {
#pragma unroll
                for (int ks = 0; ks < kHd / 16; ++ks) umma(dS, dq[ks], dk[ks], idescS, ks > 0);
                ummaCommit(&s->sFull[x]);
                if (open == 0) ummaCommit(&s->kEmpty[st]);
            }
            __syncwarp();
            if (j == 0) { if (x) ++items1; else ++items0; }
        };
        while (c.valid && ok) {
            // S products not issued ahead (start of the stream, or a group whose next item was
            // too far away when it finished the one before)
#pragma unroll
            for (int x = 0; x < 2; ++x) {
                bool& ahead = x ? ahead1 : ahead0;
                if (c.j < c.it.nTg[x] && ok) {
                    if (!ahead) issueQK(x, c.it, c.j, c.g);
                    ahead = false;
                }
            }
            if (!ok) break;
            const int st = c.g % kVStages;
            // the next item of the stream, for the groups that finish this one here
            Cursor nx = c;
            const bool lastOfItem = c.j == c.it.nT - 1;
            const bool endsHere0 = c.j == c.it.nTg[0] - 1, endsHere1 = c.j == c.it.nTg[1] - 1;
            if (endsHere0 || endsHere1) {
                nx.g = c.g + (c.it.nT - 1 - c.j);      // last tile of this item
                nx.j = c.it.nT - 1;
                nx.nextTile(p, total, numPairs);       // first tile of the next item (or the end)
            }
#pragma unroll
            for (int x = 0; x < 2; ++x) {
                if (!(c.j < c.it.nTg[x]) || !ok) continue;
                int& steps = x ? steps1 : steps0;
                ok = mbarWait(&s->pFull[x], steps & 1, &s->dead, errFlag, waitLimit, 5);
                if (ok) ok = mbarWait(&s->vFull[st], (c.g / kVStages) & 1, &s->dead, errFlag, waitLimit, 6);
                // the accumulator is free once the output of the group's item before was read from it
                const int itemsX = x ? items1 : items0;
                if (ok && c.j == 0 && itemsX >= 2) ok = mbarWait(&s->oEmpty[x], (itemsX - 2) & 1, &s->dead, errFlag, waitLimit, 15);
                ok = __all_sync(0xFFFFFFFFu, ok);
                if (!ok) break;
                tcFenceAfter();
                const uint32_t vLo = descLo(smemAddr(s->v[st]), kHalfBytes);
                const uint32_t sCol = tmemS(x), dO = tmemO(x);
                const uint32_t first = c.j > 0 ? 1u : 0u;
                const bool lo = BF16 && c.it.useLo[x];
                const bool lastUser = x == 1 || !(c.j < c.it.nTg[1]);
                uint64_t dv[kKeys / 16];
#pragma unroll
                for (int ks = 0; ks < kKeys / 16; ++ks) dv[ks] = desc64(vLo + ks * 128, hiK);
                if (leader) {
                    // P of keys 32c .. 32c+31 sits in columns 32c .. 32c+15 (and, with the
                    // low-order pass, its remainder in columns 32c+16 .. 32c+31) of the S buffer
#pragma unroll
                    for (int ks = 0; ks < kKeys / 16; ++ks)
                        ummaTs(dO, sCol + 32u * (ks >> 1) + 8u * (ks & 1), dv[ks], idescO, ks > 0 ? 1u : first);
                    if (lo) {
#pragma unroll
                        for (int ks = 0; ks < kKeys / 16; ++ks)
                            ummaTs(dO, sCol + 32u * (ks >> 1) + 8u * (ks & 1) + 16u, dv[ks], idescO, 1u);
                    }
                    if (c.j == c.it.nTg[x] - 1) ummaCommit(&s->oFull[x]);     // the tile's accumulator is final
                    if (lastUser) ummaCommit(&s->vEmpty[st]);
                }
                __syncwarp();
                ++steps;
                // the group's next S product
                bool& ahead = x ? ahead1 : ahead0;
                if (c.j + 1 < c.it.nTg[x]) {
                    issueQK(x, c.it, c.j + 1, c.g + 1);
                    ahead = true;
                } else if (nx.valid && nx.it.nTg[x] > 0 && nx.g <= c.g + 2 &&
                           __all_sync(0xFFFFFFFFu, mbarTry(&s->qFull[x], (x ? items1 : items0) & 1))) {
                    // (only if the query tile is already there: the other group must not wait for it)
                    issueQK(x, nx.it, 0, nx.g);
                    ahead = true;
                }
            }
            (void)lastOfItem;
            c.nextTile(p, total, numPairs);
        }
    } else if (warp == kIdleWarp) {
        asm volatile("setmaxnreg.dec.sync.aligned.u32 80;");          // (the fourth warp of the service warpgroup)
    } else if (warp >= kOutputWarp0) {
        // ------------------------------------------------------------ output warps
        // Thread t of the warpgroup owns row t of the tile being written.  Per item and group,
        // in stream order: the row's sum from the softmax thread, the final accumulator from
        // tensor memory (its barrier gets one commit per tile, so its phases are taken in
        // order), O / l into the staging buffer in the layout of the two TMA boxes ([half]
        // [row][8 chunks of 16 bytes, chunk index XOR row % 8]), one TMA store.  Tiles with
        // fewer than 128 rows of the sequence go out with plain stores (a box would run into
        // the next sequence's rows).
        asm volatile("setmaxnreg.dec.sync.aligned.u32 64;");
        if (!live) goto done;
        const int t = (warp & 3) * 32 + lane;
        const uint32_t laneBase = static_cast<uint32_t>((warp & 3) * 32) << 16;
        const bool issuer = threadIdx.x == kOutputWarp0 * 32;
        int cnt0 = 0, cnt1 = 0;           // tiles written per group (phase of lReady, oFull)
        bool ok = true, storePending = false;
        for (int w = blockIdx.x; w < total && ok; w += gridDim.x) {
            Item it;
            if (!loadItem(p, w, numPairs, it)) continue;
#pragma unroll
            for (int x = 0; x < 2; ++x) {
                if (it.nTg[x] == 0 || it.rowsValid[x] == 0 || !ok) continue;
                int& cnt = x ? cnt1 : cnt0;
                ok = mbarWait(&s->lReady[x], cnt & 1, &s->dead, errFlag, waitLimit, 17);
                if (ok) ok = mbarWait(&s->oFull[x], cnt & 1, &s->dead, errFlag, waitLimit, 10);
                ok = __all_sync(0xFFFFFFFFu, ok);
                if (!ok) break;
                tcFenceAfter();
                const float l = s->rowL[x][t];
                const float inv = l > 0.f ? 1.f / l : 0.f;
                const bool full = it.rowsValid[x] == kRows;
                if (full && storePending) {
                    // the staging buffer is free once the store before has read it
                    if (issuer) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
                    asm volatile("bar.sync 1, 128;" ::: "memory");
                    storePending = false;
                }
                unsigned char* out = static_cast<unsigned char*>(p.out) + ((static_cast<int64_t>(it.rowBase[x]) + t) * p.heads + it.headOf(x)) * kHd * 2;
                const uint32_t oAddr = tmemO(x) + laneBase;
#pragma unroll 1
                for (int c = 0; c < 4; ++c) {
                    uint32_t o[32];
                    tmemLd32(oAddr + 32u * c, o);
#pragma unroll
                    for (int q4 = 0; q4 < 4; ++q4) {
                        uint32_t wv[4];
#pragma unroll
                        for (int e = 0; e < 4; ++e)
                            wv[e] = pack16<BF16>(__uint_as_float(o[8 * q4 + 2 * e]) * inv, __uint_as_float(o[8 * q4 + 2 * e + 1]) * inv);
                        const int chunk = c * 4 + q4;          // 16-byte chunk of the 256-byte row
                        if (full)
                            *reinterpret_cast<uint4*>(s->stage + (chunk >> 3) * kHalfBytes + t * 128 + (((chunk & 7) ^ (t & 7)) << 4)) =
                                make_uint4(wv[0], wv[1], wv[2], wv[3]);
                        else if (t < it.rowsValid[x])
                            *reinterpret_cast<uint4*>(out + chunk * 16) = make_uint4(wv[0], wv[1], wv[2], wv[3]);
                    }
                }
                tcFenceBefore();
                // the buffer is next read (TMA store) by the asynchronous proxy
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                asm volatile("bar.sync 1, 128;" ::: "memory");
                if (issuer) {
                    mbarArrive(&s->oEmpty[x]);                  // the accumulator may be overwritten
                    if (full) {
                        tmaStore3d(&mapO, s->stage, 0, it.headOf(x), it.rowBase[x]);
                        tmaStore3d(&mapO, s->stage + kHalfBytes, 64, it.headOf(x), it.rowBase[x]);
                        asm volatile("cp.async.bulk.commit_group;" ::: "memory");
                    }
                }
                if (full) storePending = true;
                ++cnt;
            }
        }
        if (issuer) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
    } else {
        // ------------------------------------------------------------ softmax warps
        // Two groups of 128 threads; group x owns query tile x of every item, thread t of a
        // group owns row t of it: all 128 key columns of a tile in registers, no exchange
        // between threads.  While one group turns its S into P, the tensor pipe works for the
        // other.
        asm volatile("setmaxnreg.inc.sync.aligned.u32 184;");
        if (!live) goto done;
        const int x = warp >> 2, t = (warp & 3) * 32 + lane;
        const bool loader = t == 0;                     // fetches the group's query tiles
        const uint32_t laneBase = static_cast<uint32_t>((warp & 3) * 32) << 16;
        const uint32_t sAddr = tmemS(x) + laneBase, oAddr = tmemO(x) + laneBase;
        bool ok = true;
        int steps = 0;      // key tiles this group has done (phase of its barriers)
        int items = 0;      // items this group has taken part in
        int g0 = 0;         // key tiles of the stream before the current item
        // the next query tile is brought into L2 an item early, so that its fetch during the
        // last key tile of the item before it is short
        auto prefetchQ = [&](const Item& it) {
            const int rowBase = x ? it.rowBase[1] : it.rowBase[0];
            asm volatile("cp.async.bulk.prefetch.tensor.3d.L2.global.tile [%0, {%1, %2, %3}];" ::"l"(&mapQ), "r"(0), "r"(it.headOf(x)), "r"(rowBase) : "memory");
            asm volatile("cp.async.bulk.prefetch.tensor.3d.L2.global.tile [%0, {%1, %2, %3}];" ::"l"(&mapQ), "r"(64), "r"(it.headOf(x)), "r"(rowBase) : "memory");
        };
        auto loadQ = [&](const Item& it) {
            const int rowBase = x ? it.rowBase[1] : it.rowBase[0];
            mbarExpectTx(&s->qFull[x], kTileBytes);
            tmaLoad3d(s->q[x], &mapQ, &s->qFull[x], 0, it.headOf(x), rowBase);
            tmaLoad3d(s->q[x] + kHalfBytes, &mapQ, &s->qFull[x], 64, it.headOf(x), rowBase);
        };
        // the first item the group takes part in: its query tile is fetched right away
        int wNext = blockIdx.x;
        Item nextIt;
        auto seekNext = [&]() {                          // first item at or after wNext in which the group has key tiles
            while (wNext < total) {
                if (loadItem(p, wNext, numPairs, nextIt) && (x ? nextIt.nTg[1] : nextIt.nTg[0]) > 0) return true;
                wNext += gridDim.x;
            }
            return false;
        };
        bool haveNext = seekNext();
        if (haveNext && loader) loadQ(nextIt);
        for (int w = blockIdx.x; w < total && ok; w += gridDim.x) {
            Item it;
            if (!loadItem(p, w, numPairs, it)) continue;
            const int gBase = g0;
            g0 += it.nT;
            // this group's half of the item
            const int rowsValid = x ? it.rowsValid[1] : it.rowsValid[0], nT = x ? it.nTg[1] : it.nTg[0];
            const int rowBase = x ? it.rowBase[1] : it.rowBase[0], firstPos = x ? it.firstPos[1] : it.firstPos[0];
            if (rowsValid == 0) continue;
            if (nT == 0) {
                // rows that see no key at all: zeros (no other role takes part)
                if (t < rowsValid) {
                    uint4* out = reinterpret_cast<uint4*>(static_cast<unsigned char*>(p.out) +
                                                          ((static_cast<int64_t>(rowBase) + t) * p.heads + it.headOf(x)) * kHd * 2);
#pragma unroll
                    for (int i = 0; i < 16; ++i) out[i] = make_uint4(0u, 0u, 0u, 0u);
                }
                continue;
            }
            // the item after this one in which the group has key tiles (its query tile is
            // fetched during this item's last key tile)
            wNext = w + gridDim.x;
            haveNext = seekNext();
            if (haveNext && loader) prefetchQ(nextIt);
            const MaskInfo mk(it.ws, it.seqLen, firstPos + t, p.causal);
            const bool useLo = BF16 && (x ? it.useLo[1] : it.useLo[0]);
            float mUsed = -INFINITY, l = 0.f;
            for (int j = 0; j < nT && ok; ++j, ++steps) {
                const int k0 = (it.tileLo + j) * kKeys;
                const bool edge = k0 < it.ws || k0 + kKeys > it.seqLen || (p.causal && k0 + kKeys - 1 > firstPos);
                ok = mbarWait(&s->sFull[x], steps & 1, &s->dead, errFlag, waitLimit, 7);
                if (!ok) break;
                tcFenceAfter();
                // S of the item's last tile is there, so its query tile is no longer read
                if (j == nT - 1 && haveNext && loader) loadQ(nextIt);
                // ---- the whole row of scores into registers, then its maximum (the scale is positive)
                uint32_t r0[32], r1[32], r2[32], r3[32];
                tmemLd32NoWait(sAddr, r0);
                tmemLd32NoWait(sAddr + 32u, r1);
                tmemLd32NoWait(sAddr + 64u, r2);
                tmemLd32NoWait(sAddr + 96u, r3);
                tmemLdWait();
                if (edge) {
                    maskScores(r0, mk, k0);
                    maskScores(r1, mk, k0 + 32);
                    maskScores(r2, mk, k0 + 64);
                    maskScores(r3, mk, k0 + 96);
                }
                const float tmax = fmaxf(fmaxf(quarterRowMax(r0), quarterRowMax(r1)), fmaxf(quarterRowMax(r2), quarterRowMax(r3))) * scaleLog2;
                // The running maximum is only raised when it grows by more than 2^8: the result is
                // exact either way, the final division uses the same reference.
                bool raise = false;
                float corr = 1.f;
                if (j == 0) mUsed = tmax;
                else if (tmax > mUsed + kRescaleThreshold) {
                    raise = true;
                    corr = ex2Approx(mUsed - tmax);
                    mUsed = tmax;
                }
                if (j >= 1 && __any_sync(0xFFFFFFFFu, raise)) {
                    // The accumulator is complete up to the tile before: this tile's S product was
                    // issued behind that P V product and has been seen complete.
#pragma unroll 1
                    for (int c = 0; c < 4; ++c) {
                        uint32_t o[32];
                        tmemLd32(oAddr + 32u * c, o);
#pragma unroll
                        for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * corr);
                        tmemSt32(oAddr + 32u * c, o);
                    }
                    tmemStWait();
                    l *= corr;
                }
                // ---- the weights replace the scores in tensor memory: per 32 keys 16 columns of
                // packed pairs (plus 16 columns of their low-order parts where the tile needs
                // 16-bit weights)
                const float negM = mUsed == -INFINITY ? 0.f : -mUsed;
                {
                    uint32_t wgt[32];
                    if (useLo) {
                        l += weightsRange<BF16, true, 0, 32>(r0, wgt, scaleLog2, negM);
                        tmemSt32(sAddr, wgt);
                        l += weightsRange<BF16, true, 0, 32>(r1, wgt, scaleLog2, negM);
                        tmemSt32(sAddr + 32u, wgt);
                        l += weightsRange<BF16, true, 0, 32>(r2, wgt, scaleLog2, negM);
                        tmemSt32(sAddr + 64u, wgt);
                        l += weightsRange<BF16, true, 0, 32>(r3, wgt, scaleLog2, negM);
                        tmemSt32(sAddr + 96u, wgt);
                    } else {
                        l += weightsRange<BF16, false, 0, 32>(r0, wgt, scaleLog2, negM);
                        tmemSt16(sAddr, wgt);
                        l += weightsRange<BF16, false, 0, 32>(r1, wgt, scaleLog2, negM);
                        tmemSt16(sAddr + 32u, wgt);
                        l += weightsRange<BF16, false, 0, 32>(r2, wgt, scaleLog2, negM);
                        tmemSt16(sAddr + 64u, wgt);
                        l += weightsRange<BF16, false, 0, 32>(r3, wgt, scaleLog2, negM);
                        tmemSt16(sAddr + 96u, wgt);
                    }
                }
                tmemStWait();
                if (k0 + kKeys > it.seqLen) {
                    // rows of V past the end of the sequence may hold anything: zero them (both
                    // groups may, with the same zeros)
                    const int gt = gBase + j, st = gt % kVStages;
                    ok = mbarWait(&s->vFull[st], (gt / kVStages) & 1, &s->dead, errFlag, waitLimit, 9);
                    if (!ok) break;
                    if (k0 + t >= it.seqLen) {
#pragma unroll
                        for (int c16 = 0; c16 < 16; ++c16)
                            *reinterpret_cast<uint4*>(s->v[st] + (c16 >> 3) * kHalfBytes + t * 128 + (c16 & 7) * 16) =
                                make_uint4(0u, 0u, 0u, 0u);
                    }
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                }
                tcFenceBefore();
                mbarArrive(&s->pFull[x]);
            }
            if (!ok) break;
            // The output warps write the tile once its last P V product is complete; this thread
            // leaves them the sum of its row's weights and goes on.  (The next write to this
            // slot comes at the end of the group's next item, whose first P V product waits for
            // the accumulator to be handed back, which happens after the sum was read.)
            s->rowL[x][t] = l;
            mbarArrive(&s->lReady[x]);
            ++items;
        }
    }

done:
    tcFenceBefore();
    __syncthreads();
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
    CUtensorMap mapQ, mapK, mapV, mapO;
    for (int which = 0; which < 2; ++which) {
        // Q and the output: [rows][heads][128]; a box is 64 dims x 1 head x 128 rows
        cuuint64_t dims[3] = {static_cast<cuuint64_t>(kHd), static_cast<cuuint64_t>(p.heads), static_cast<cuuint64_t>(totalRows)};
        cuuint64_t strides[2] = {static_cast<cuuint64_t>(kHd) * 2, static_cast<cuuint64_t>(p.heads) * kHd * 2};
        cuuint32_t box[3] = {64, 1, static_cast<cuuint32_t>(kRows)};
        cuuint32_t es[3] = {1, 1, 1};
        if (encode(which ? &mapO : &mapQ, dt, 3, which ? p.out : const_cast<void*>(p.q), dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
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
    // One resident CTA per multiprocessor walks the work items round robin.
    int dev = 0, sms = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e == cudaSuccess) e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (e != cudaSuccess) return e;
    // An even number of query heads per KV head: an item is one query tile of two heads,
    // so both softmax groups have the same key tiles; else two query tiles of one head.
    const int numTiles = (p.maxQLen + kRows - 1) / kRows;
    const bool pairHeads = (p.heads / p.kvHeads) % 2 == 0;
    const int itemHeads = pairHeads ? p.heads / 2 : p.heads;
    const long long items = static_cast<long long>(pairHeads ? numTiles : (numTiles + 1) / 2) * itemHeads * p.numSeqs;
    if (items <= 0 || items > 0x7FFFFFFF) return cudaErrorInvalidValue;
    PrefillParams pk = p;
    pk.pairHeads = pairHeads ? 1 : 0;
    pk.fastItems = items < (1 << 22) ? 1 : 0;
    pk.invPer = 1.0f / static_cast<float>(p.numSeqs * itemHeads);
    pk.invHeads = 1.0f / static_cast<float>(itemHeads);
    pk.invGroup = 1.0f / static_cast<float>(itemHeads / p.kvHeads);
    dim3 grid(static_cast<unsigned>(items < sms ? items : sms));
    if (p.dtype == kBF16) {
        e = cudaFuncSetAttribute(prefillTcKernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
        if (e != cudaSuccess) return e;
        prefillTcKernel<true><<<grid, kThreads, smem, stream>>>(mapQ, mapK, mapV, mapO, pk, scaleLog2, errFlag);
    } else {
        e = cudaFuncSetAttribute(prefillTcKernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
        if (e != cudaSuccess) return e;
        prefillTcKernel<false><<<grid, kThreads, smem, stream>>>(mapQ, mapK, mapV, mapO, pk, scaleLog2, errFlag);
    }
    if (launches) *launches += 1;
    return cudaGetLastError();
}

}  // namespace pam
