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
// (128 query rows of one head of one sequence) round robin, longest items
// first.  An item walks the key tiles (128 keys each) its rows can see; the
// tiles go alternately to two softmax groups, each with its own S buffer and
// accumulator O in tensor memory (4 x 128 columns), so that one group turns S
// into the weights P while the tensor pipe works for the other.  The two
// accumulators are merged (log-sum-exp) when the item is written out.
//
//   warps 0-3, 4-7       softmax groups 0 and 1: thread t of a group owns query
//                        row t, all 128 key columns of a tile, in registers (no
//                        exchange between threads).  Scores are scaled, masked
//                        (causal, window start, sequence end) only on edge
//                        tiles.  The running maximum is only raised when it
//                        grows by more than 2^8 (the result is exact either
//                        way, the final division uses the same reference), in
//                        which case O is rescaled in tensor memory.  The
//                        weights go back to tensor memory over the scores, in
//                        the cache type (tcgen05.st); for bfloat16, on rows that
//                        see few keys, as two operands P_hi + P_lo (16
//                        significant bits together) and twice the PV
//                        instructions, because 8-bit weights alone miss the
//                        2e-3 bound there.  The merged O / l of an item is
//                        staged in its (by then idle) query buffer in the
//                        layout of a TMA box.
//   warp 8               TMA producer of Q (two buffers, one per item in flight)
//                        and of K: per key tile 8 pages (each 16 rows x 256 B,
//                        fetched as two 128-byte-swizzled boxes, one page per
//                        lane) into a ring; completion on mbarriers.
//   warp 9               TMA producer of V, its own ring.
//   warp 10              MMA issuer (one elected lane): S = Q K^T (8 x
//                        tcgen05.mma 128x128x16, both operands from shared
//                        memory) and O += P V (P read from tensor memory, V as
//                        an MN-major operand straight from its row-major
//                        pages); tcgen05.commit signals the mbarriers.
//   warp 11              TMA store of the finished rows of an item.
//
// The service warps hand registers to the softmax warps (setmaxnreg).
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
// Instrumented build only: CTA 0 leaves clock stamps [role][tile][event] in global memory.
constexpr int kTraceRoles = 4, kTraceTiles = 32, kTraceEvents = 12;
__device__ long long gTrace[kTraceRoles * kTraceTiles * kTraceEvents];
__device__ unsigned long long gCtaTimes[4 * 256];      // start and end of every CTA: nanoseconds, then SM cycles
__device__ __forceinline__ unsigned long long globalTimerNs() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
#define TRACE(role, tile, event)                                                                        \
    do {                                                                                                \
        if (blockIdx.x == 0 && (threadIdx.x & 31) == 0 && (role) < kTraceRoles && (tile) < kTraceTiles) \
            gTrace[((role) * kTraceTiles + (tile)) * kTraceEvents + (event)] = clock64();               \
    } while (0)
#else
#define TRACE(role, tile, event)
#endif

struct Smem {
    // tiles first: each 1024-byte aligned (swizzle atoms)
    unsigned char q[2][kTileBytes];            // query tiles of two items in flight; each doubles as output staging
    unsigned char k[kKStages][kTileBytes];
    unsigned char v[kVStages][kTileBytes];
    unsigned long long qFull[2], qEmpty[2], kFull[kKStages], kEmpty[kKStages], vFull[kVStages], vEmpty[kVStages];
    unsigned long long sFull[2], pFull[2], pvDone[2];   // one of each per softmax group
    unsigned long long oEmpty, oStaged[2];
    unsigned long long stateReady, stateRead;  // the two softmax groups meet twice per item
    float2 rowState[2][kRows];                 // [group][row]: reference maximum and sum of weights of an item
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

__device__ __forceinline__ void tmaStore3d(const CUtensorMap* map, const void* src, int x, int y, int z) {
    asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];"
                 ::"l"(map), "r"(smemAddr(src)), "r"(x), "r"(y), "r"(z)
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
__device__ __forceinline__ uint32_t tmemLd1(uint32_t taddr) {
    uint32_t v;
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x1.b32 {%0}, [%1];" : "=r"(v) : "r"(taddr));
    return v;
}
__device__ __forceinline__ void tmemSt1(uint32_t taddr, uint32_t v) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x1.b32 [%0], {%1};" ::"r"(taddr), "r"(v) : "memory");
}
// A float as bfloat16 bits, rounded towards +infinity, and back.  Used for the reference
// maximum of a row: any value at or a little above the true maximum serves, as long as the
// four threads of the row use the same one.
__device__ __forceinline__ unsigned short bf16Up(float x) {
    const uint32_t b = __float_as_uint(x);
    return static_cast<unsigned short>(((b >> 31) ? b : b + 0xFFFFu) >> 16);
}
__device__ __forceinline__ float bf16ToFloat(unsigned short h) { return __uint_as_float(static_cast<uint32_t>(h) << 16); }
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
#pragma unroll
    for (int i = 0; i < 32; ++i)
        if (i < a || i >= b) r[i] = 0xFF800000u;
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
// returns the sum of the weights.  Masked scores are -inf and give weight 0.
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
constexpr int kKProducerWarp = 8, kVProducerWarp = 9, kMmaWarp = 10, kStoreWarp = 11;
constexpr int kThreads = (kSoftmaxWarps + 4) * 32;

// One unit of work: 128 query rows of one head of one sequence.
struct Item {
    int head, seq, kvh;
    int nT, tileLo;          // key tiles tileLo .. tileLo + nT - 1 hold every key a row may see
    int rowBase, rowsValid;  // first row in q/out, rows that exist
    int firstPos;            // sequence position of row 0
    int seqLen, ws;
    bool useLo;
    const int32_t* table;
};

// Work item `w` of the launch.  Items are numbered tile-major with the last (longest)
// query tiles first and the head running fastest, so that the CTAs working side by side
// share the keys of one KV head through L2 and the short items fill the end of the launch.
// Returns false when the sequence has no rows in that tile.
__device__ __forceinline__ bool loadItem(const PrefillParams& p, int w, int numTiles, Item& it) {
    const int per = p.numSeqs * p.heads;
    const int tile = numTiles - 1 - w / per;
    const int rem = w % per;
    it.seq = rem / p.heads;
    it.head = rem % p.heads;
    const int qLen = prefillMeta(p, 2, it.seq);
    if (tile * kRows >= qLen) return false;
    it.kvh = it.head / (p.heads / p.kvHeads);
    const int qStart = prefillMeta(p, 1, it.seq);
    it.seqLen = prefillMeta(p, 0, it.seq);
    it.ws = prefillMeta(p, 4, it.seq);
    it.rowBase = prefillMeta(p, 3, it.seq) + tile * kRows;
    it.rowsValid = min(kRows, qLen - tile * kRows);
    it.firstPos = qStart + tile * kRows;
    const int lastPos = it.firstPos + it.rowsValid - 1;
    const int keyEnd = p.causal ? min(it.seqLen, lastPos + 1) : it.seqLen;  // exclusive
    it.tileLo = it.ws / kKeys;
    it.nT = keyEnd > it.ws ? (keyEnd - 1) / kKeys - it.tileLo + 1 : 0;
    // Fewest keys any row of the tile sees.  A bfloat16 weight keeps 8 significant bits; on a
    // row with few keys (large weights) that alone can cost more than 2e-3 on unit-variance
    // values, so such tiles carry the weights as two bfloat16 operands (16 bits).  Rows with
    // hundreds of keys have weights small enough for 8 bits, as in every bfloat16 attention
    // kernel.  exactWeights: 0 never, 1 short rows, 2 always.
    const int fewest = p.causal ? it.firstPos + 1 - it.ws : it.seqLen - it.ws;
    it.useLo = p.exactWeights == 2 || (p.exactWeights == 1 && fewest < kShortRowKeys);
    it.table = p.tables + static_cast<int64_t>(it.seq) * p.maxNumBlocks;
    return true;
}

// Position of a role in the CTA's stream of key tiles: item w, tile j of it, g tiles and
// n items (with keys) done before.  Every role walks the same stream, so g and n give the
// stage and the phase parity of every barrier without any communication.
struct Cursor {
    int w, j, g, n;
    bool valid;
    Item it;
    __device__ __forceinline__ void seek(const PrefillParams& p, int total, int numTiles) {
        valid = false;
        while (w < total) {
            if (loadItem(p, w, numTiles, it) && it.nT > 0) {
                valid = true;
                return;
            }
            w += gridDim.x;
        }
    }
    __device__ __forceinline__ void init(const PrefillParams& p, int total, int numTiles) {
        w = blockIdx.x;
        j = g = n = 0;
        seek(p, total, numTiles);
    }
    __device__ __forceinline__ void nextTile(const PrefillParams& p, int total, int numTiles) {
        ++j;
        ++g;
        if (j == it.nT) nextItem(p, total, numTiles);
    }
    // to the first tile of the next item with keys (g must already count the tiles left behind)
    __device__ __forceinline__ void nextItem(const PrefillParams& p, int total, int numTiles) {
        j = 0;
        ++n;
        w += gridDim.x;
        seek(p, total, numTiles);
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

#ifdef PAM_PREFILL_TRACE
    if (threadIdx.x == 0 && blockIdx.x < 256) {
        gCtaTimes[4 * blockIdx.x] = globalTimerNs();
        gCtaTimes[4 * blockIdx.x + 2] = clock64();
    }
#endif
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int numTiles = (p.maxQLen + kRows - 1) / kRows;
    const int total = numTiles * p.numSeqs * p.heads;

    if (threadIdx.x == kKProducerWarp * 32) {
        asm volatile("prefetch.tensormap [%0];" ::"l"(&mapQ) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&mapK) : "memory");
    }
    if (threadIdx.x == kVProducerWarp * 32) asm volatile("prefetch.tensormap [%0];" ::"l"(&mapV) : "memory");
    if (threadIdx.x == kStoreWarp * 32) asm volatile("prefetch.tensormap [%0];" ::"l"(&mapO) : "memory");
    if (threadIdx.x == 0) {
        for (int i = 0; i < 2; ++i) {
            mbarInit(&s->qFull[i], 1);
            mbarInit(&s->qEmpty[i], 1);
            mbarInit(&s->oStaged[i], kSoftmaxWarps);
            mbarInit(&s->sFull[i], 1);
            mbarInit(&s->pFull[i], kGroupThreads);
            mbarInit(&s->pvDone[i], 1);
        }
        for (int i = 0; i < kKStages; ++i) { mbarInit(&s->kFull[i], 1); mbarInit(&s->kEmpty[i], 1); }
        for (int i = 0; i < kVStages; ++i) { mbarInit(&s->vFull[i], 1); mbarInit(&s->vEmpty[i], 1); }
        mbarInit(&s->oEmpty, kSoftmaxWarps);
        mbarInit(&s->stateReady, 2 * kGroupThreads);
        mbarInit(&s->stateRead, 2 * kGroupThreads);
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

    // Row of the pool (block * kv_heads * block_size space) of the 16-token piece `lane`
    // of key tile j of an item; lanes 0-7 of a producer warp fetch one piece each.
    const int tilesPerPage = p.blockSize / 16;
    auto pieceRow = [&](const Item& it, int j) {
        const int t16 = (it.tileLo + j) * (kKeys / 16) + lane;
        const int page = min(t16 / tilesPerPage, p.maxNumBlocks - 1);
        const int blk = min(max(it.table[page], 0), p.poolBlocks - 1);
        return (blk * p.kvHeads + it.kvh) * p.blockSize + (t16 % tilesPerPage) * 16;
    };

    // Registers move from the four service warps to the softmax warps, which hold a whole row
    // of scores: first statement of every role's branch, the same value in all four warps of
    // a warpgroup (the instruction is defined per warpgroup).  384 x 168 registers at launch;
    // 128 threads give up 72 each, 256 threads take 32 each.
    if (warp == kKProducerWarp) {
        // ------------------------------------------------------------ Q and K producer
        asm volatile("setmaxnreg.dec.sync.aligned.u32 96;");
        if (!live) goto done;
        Cursor c;
        c.init(p, total, numTiles);
        bool ok = true;
        while (c.valid && ok) {
            if (c.j == 0) {
                // the query tile of item n goes into buffer n & 1 once the output of item n - 2 left it
                const int qb = c.n & 1;
                if (c.n >= 2) ok = mbarWait(&s->qEmpty[qb], ((c.n >> 1) - 1) & 1, &s->dead, errFlag, 14);
                ok = __all_sync(0xFFFFFFFFu, ok);
                if (!ok) break;
                if (lane == 0) {
                    mbarExpectTx(&s->qFull[qb], kTileBytes);
                    tmaLoad3d(s->q[qb], &mapQ, &s->qFull[qb], 0, c.it.head, c.it.rowBase);
                    tmaLoad3d(s->q[qb] + kHalfBytes, &mapQ, &s->qFull[qb], 64, c.it.head, c.it.rowBase);
                }
            }
            const int st = c.g % kKStages;
            const int row = lane < kKeys / 16 ? pieceRow(c.it, c.j) : 0;
            if (c.g >= kKStages) ok = mbarWait(&s->kEmpty[st], ((c.g / kKStages) - 1) & 1, &s->dead, errFlag, 1);
            ok = __all_sync(0xFFFFFFFFu, ok);
            if (!ok) break;
            if (lane == 0) mbarExpectTx(&s->kFull[st], kTileBytes);
            __syncwarp();
            if (lane < kKeys / 16) {
                tmaLoad2d(s->k[st] + lane * 2048, &mapK, &s->kFull[st], 0, row);
                tmaLoad2d(s->k[st] + kHalfBytes + lane * 2048, &mapK, &s->kFull[st], 64, row);
            }
            c.nextTile(p, total, numTiles);
        }
    } else if (warp == kVProducerWarp) {
        // ------------------------------------------------------------ V producer
        asm volatile("setmaxnreg.dec.sync.aligned.u32 96;");
        if (!live) goto done;
        Cursor c;
        c.init(p, total, numTiles);
        bool ok = true;
        while (c.valid && ok) {
            const int st = c.g % kVStages;
            const int row = lane < kKeys / 16 ? pieceRow(c.it, c.j) : 0;
            if (c.g >= kVStages) ok = mbarWait(&s->vEmpty[st], ((c.g / kVStages) - 1) & 1, &s->dead, errFlag, 13);
            ok = __all_sync(0xFFFFFFFFu, ok);
            if (!ok) break;
            if (lane == 0) mbarExpectTx(&s->vFull[st], kTileBytes);
            __syncwarp();
            if (lane < kKeys / 16) {
                tmaLoad2d(s->v[st] + lane * 2048, &mapV, &s->vFull[st], 0, row);
                tmaLoad2d(s->v[st] + kHalfBytes + lane * 2048, &mapV, &s->vFull[st], 64, row);
            }
            c.nextTile(p, total, numTiles);
        }
    } else if (warp == kMmaWarp) {
        // ------------------------------------------------------------ MMA issuer
        // Key tile j of an item belongs to softmax group j & 1, with its own S buffer and
        // accumulator.  Tensor-core instructions execute in issue order: S of a group's next
        // tile is written over its P right behind the P V product that read it.
        // All 32 lanes walk the loop, so that the descriptor arithmetic is uniform across the
        // warp (it then runs on the uniform datapath, where the tensor-core instructions take
        // their operands from); one elected lane issues the tensor-core instructions.
        asm volatile("setmaxnreg.dec.sync.aligned.u32 96;");
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
        Cursor qk, pv;
        qk.init(p, total, numTiles);
        pv = qk;
        int qkCnt0 = 0, qkCnt1 = 0, pvCnt0 = 0, pvCnt1 = 0;     // S products and P V products issued, per group
        while (pv.valid && ok) {
            // An S product needs its group's buffer back (the P V product of the group's tile
            // before issued).  The query tile of a new item arrives only after the output of
            // the item two before left its buffer, which takes P V products still to come: so
            // the warp waits for it only when there is nothing else to issue.
            const int gq = qk.j & 1;
            const bool canQK = qk.valid && (gq ? qkCnt1 == pvCnt1 : qkCnt0 == pvCnt0);
            bool takeQK = canQK && (qk.j != 0 || qk.g == pv.g);
            if (canQK && !takeQK) takeQK = __all_sync(0xFFFFFFFFu, mbarTry(&s->qFull[qk.n & 1], (qk.n >> 1) & 1));
            if (takeQK) {
                const int st = qk.g % kKStages, qb = qk.n & 1;
                if (qk.j == 0) ok = mbarWait(&s->qFull[qb], (qk.n >> 1) & 1, &s->dead, errFlag, 2);
                if (ok) ok = mbarWait(&s->kFull[st], (qk.g / kKStages) & 1, &s->dead, errFlag, 3);
                ok = __all_sync(0xFFFFFFFFu, ok);
                if (!ok) break;
                tcFenceAfter();
                const uint32_t qLo = descLo(smemAddr(s->q[qb]), 16);
                const uint32_t kLo = descLo(smemAddr(s->k[st]), 16);
                const uint32_t dS = tmemS(gq);
                uint64_t dq[kHd / 16], dk[kHd / 16];
#pragma unroll
                for (int ks = 0; ks < kHd / 16; ++ks) {
                    const uint32_t off = ((ks >> 2) * kHalfBytes + (ks & 3) * 32) >> 4;
                    dq[ks] = desc64(qLo + off, hiK);
                    dk[ks] = desc64(kLo + off, hiK);
                }
                if (leader) {
#pragma unroll
                    for (int ks = 0; ks < kHd / 16; ++ks) umma(dS, dq[ks], dk[ks], idescS, ks > 0);
                    ummaCommit(&s->sFull[gq]);
                    ummaCommit(&s->kEmpty[st]);
                }
                __syncwarp();
                if (gq) ++qkCnt1; else ++qkCnt0;
                qk.nextTile(p, total, numTiles);
            } else {
                const int st = pv.g % kVStages, gp = pv.j & 1;
                ok = mbarWait(&s->pFull[gp], (gp ? pvCnt1 : pvCnt0) & 1, &s->dead, errFlag, 5);
                if (ok) ok = mbarWait(&s->vFull[st], (pv.g / kVStages) & 1, &s->dead, errFlag, 6);
                // the accumulators are free once the output of the item before was read from them
                if (ok && pv.j < 2 && pv.n >= 1) ok = mbarWait(&s->oEmpty, (pv.n - 1) & 1, &s->dead, errFlag, 15);
                ok = __all_sync(0xFFFFFFFFu, ok);
                if (!ok) break;
                tcFenceAfter();
                const uint32_t vLo = descLo(smemAddr(s->v[st]), kHalfBytes);
                const uint32_t sCol = tmemS(gp), dO = tmemO(gp);
                const uint32_t first = pv.j >= 2 ? 1u : 0u;
                const bool lo = BF16 && pv.it.useLo;
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
                    ummaCommit(&s->pvDone[gp]);
                    ummaCommit(&s->vEmpty[st]);
                }
                __syncwarp();
                if (gp) ++pvCnt1; else ++pvCnt0;
                pv.nextTile(p, total, numTiles);
            }
        }
    } else if (warp == kStoreWarp) {
        // ------------------------------------------------------------ output store
        // The softmax warps leave the finished rows of item n in its query buffer, in the
        // swizzled layout of a TMA box; one thread sends them to global memory and hands
        // the buffer back to the producer once the copy has read it.  Tiles with fewer
        // than 128 rows of this sequence were written by the softmax warps themselves (a
        // box would run into the next sequence's rows).
        asm volatile("setmaxnreg.dec.sync.aligned.u32 96;");
        if (!live) goto done;
        int n = 0;
        bool ok = true;
        for (int w = blockIdx.x; w < total && ok; w += gridDim.x) {
            Item it;
            if (!loadItem(p, w, numTiles, it) || it.nT == 0) continue;
            const int qb = n & 1;
            ok = mbarWait(&s->oStaged[qb], (n >> 1) & 1, &s->dead, errFlag, 16);
            ok = __all_sync(0xFFFFFFFFu, ok);
            if (!ok) break;
            if (lane == 0) {
                if (it.rowsValid == kRows) {
                    tmaStore3d(&mapO, s->q[qb], 0, it.head, it.rowBase);
                    tmaStore3d(&mapO, s->q[qb] + kHalfBytes, 64, it.head, it.rowBase);
                    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
                    asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
                }
                mbarArrive(&s->qEmpty[qb]);
            }
            ++n;
        }
        if (lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
    } else {
        // ------------------------------------------------------------ softmax warps
        // Two groups of 128 threads; group grp takes the key tiles j with j & 1 == grp of
        // every item, thread t of a group owns query row t (all 128 key columns of a tile):
        // no exchange between threads.  Each group keeps its own running maximum, sum and
        // accumulator; the two are merged when the item is written out.  A tile is read
        // from tensor memory twice, 32 columns at a time: once for the maximum, once for
        // the weights.
        asm volatile("setmaxnreg.inc.sync.aligned.u32 200;");
        if (!live) goto done;
        const int grp = warp >> 2, t = (warp & 3) * 32 + lane;
        const uint32_t laneBase = static_cast<uint32_t>((warp & 3) * 32) << 16;
        const uint32_t sAddr = tmemS(grp) + laneBase, oAddr = tmemO(grp) + laneBase;
        bool ok = true;
        int k = 0;          // key tiles this group has done (phase of its barriers)
        int g0 = 0;         // key tiles of the stream before the current item
        int n = 0;          // items with keys before the current one
        for (int w = blockIdx.x; w < total && ok; w += gridDim.x) {
            Item it;
            if (!loadItem(p, w, numTiles, it)) continue;
            if (it.nT == 0) {
                // rows that see no key at all: zeros (no other role takes part); each thread
                // writes half of its row
                if (t < it.rowsValid) {
                    uint4* out = reinterpret_cast<uint4*>(static_cast<unsigned char*>(p.out) +
                                                          ((static_cast<int64_t>(it.rowBase) + t) * p.heads + it.head) * kHd * 2 + grp * 128);
#pragma unroll
                    for (int i = 0; i < 8; ++i) out[i] = make_uint4(0u, 0u, 0u, 0u);
                }
                continue;
            }
            const MaskInfo mk(it.ws, it.seqLen, it.firstPos + t, p.causal);
            const bool useLo = BF16 && it.useLo;
            float mUsed = -INFINITY, l = 0.f;
            for (int j = grp; j < it.nT && ok; j += 2, ++k) {
                const int k0 = (it.tileLo + j) * kKeys;
                const bool edge = k0 < it.ws || k0 + kKeys > it.seqLen || (p.causal && k0 + kKeys - 1 > it.firstPos);
                ok = mbarWait(&s->sFull[grp], k & 1, &s->dead, errFlag, 7);
                if (!ok) break;
                tcFenceAfter();
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
                if (j < 2) mUsed = tmax;
                else if (tmax > mUsed + kRescaleThreshold) {
                    raise = true;
                    corr = ex2Approx(mUsed - tmax);
                    mUsed = tmax;
                }
                if (j >= 2 && __any_sync(0xFFFFFFFFu, raise)) {
                    // the group's accumulator is complete up to its tile before (seen at the end of
                    // that tile, before this tile's S could be made)
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
                // packed pairs (plus 16 columns of their low-order parts where the item needs
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
                    // rows of V past the end of the sequence may hold anything: zero them
                    const int gt = g0 + j, st = gt % kVStages;
                    ok = mbarWait(&s->vFull[st], (gt / kVStages) & 1, &s->dead, errFlag, 9);
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
                mbarArrive(&s->pFull[grp]);
                // Every thread sees every P V product of its group complete, in order: a wait on
                // a phase parity is only good for one step back, and the next product cannot
                // complete before this thread's next arrival.
                ok = mbarWait(&s->pvDone[grp], k & 1, &s->dead, errFlag, 10);
            }
            if (!ok) break;
            // ---- output of the item: (O_0 2^(m_0 - m) + O_1 2^(m_1 - m)) / (l_0 2^(m_0 - m) + l_1 2^(m_1 - m)).
            // Thread t of group grp writes columns [64 grp, 64 grp + 64) of row t.
            tcFenceAfter();
            s->rowState[grp][t] = make_float2(mUsed, l);
            mbarArrive(&s->stateReady);
            ok = mbarWait(&s->stateReady, n & 1, &s->dead, errFlag, 17);
            if (!ok) break;
            const float2 other = s->rowState[grp ^ 1][t];
            const float m = fmaxf(mUsed, other.x);
            const float wMine = m == -INFINITY ? 0.f : ex2Approx(mUsed - m), wOther = m == -INFINITY ? 0.f : ex2Approx(other.x - m);
            const float lt = l * wMine + other.y * wOther;
            const float inv = lt > 0.f ? 1.f / lt : 0.f;
            const float f0 = (grp == 0 ? wMine : wOther) * inv, f1 = (grp == 0 ? wOther : wMine) * inv;
            const bool has1 = it.nT >= 2;                     // group 1 had a tile: its accumulator holds numbers
            unsigned char* stage = s->q[n & 1] + grp * kHalfBytes + t * 128;
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                uint32_t o0[32], o1[32];
                tmemLd32(tmemO(0) + laneBase + 64u * grp + 32u * c, o0);
                if (has1) tmemLd32(tmemO(1) + laneBase + 64u * grp + 32u * c, o1);
#pragma unroll
                for (int q4 = 0; q4 < 4; ++q4) {
                    uint32_t wv[4];
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int i = 8 * q4 + 2 * e;
                        float a = __uint_as_float(o0[i]) * f0, b = __uint_as_float(o0[i + 1]) * f0;
                        if (has1) {
                            a = fmaf(__uint_as_float(o1[i]), f1, a);
                            b = fmaf(__uint_as_float(o1[i + 1]), f1, b);
                        }
                        wv[e] = pack16<BF16>(a, b);
                    }
                    *reinterpret_cast<uint4*>(stage + (((c * 4 + q4) ^ (t & 7)) << 4)) = make_uint4(wv[0], wv[1], wv[2], wv[3]);
                }
            }
            tcFenceBefore();
            __syncwarp();
            if (lane == 0) mbarArrive(&s->oEmpty);                 // the accumulators may be overwritten
            if (it.rowsValid < kRows) {
                // ragged tile: this thread writes its own 128 bytes
                if (t < it.rowsValid) {
                    uint4* out = reinterpret_cast<uint4*>(static_cast<unsigned char*>(p.out) +
                                                          ((static_cast<int64_t>(it.rowBase) + t) * p.heads + it.head) * kHd * 2 + grp * 128);
#pragma unroll
                    for (int i = 0; i < 8; ++i) out[i] = *reinterpret_cast<const uint4*>(stage + ((i ^ (t & 7)) << 4));
                }
            }
            // the buffer is next read (TMA store) and written (TMA load) by the asynchronous proxy
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbarArrive(&s->oStaged[n & 1]);
            // the other group must have read this group's row state before the next item overwrites it
            mbarArrive(&s->stateRead);
            ok = mbarWait(&s->stateRead, n & 1, &s->dead, errFlag, 18);
            g0 += it.nT;
            ++n;
        }
    }

done:
    tcFenceBefore();
    __syncthreads();
#ifdef PAM_PREFILL_TRACE
    if (threadIdx.x == 0 && blockIdx.x < 256) {
        gCtaTimes[4 * blockIdx.x + 1] = globalTimerNs();
        gCtaTimes[4 * blockIdx.x + 3] = clock64();
    }
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
    const long long items = static_cast<long long>((p.maxQLen + kRows - 1) / kRows) * p.heads * p.numSeqs;
    if (items <= 0 || items > 0x7FFFFFFF) return cudaErrorInvalidValue;
    dim3 grid(static_cast<unsigned>(items < sms ? items : sms));
    if (p.dtype == kBF16) {
        e = cudaFuncSetAttribute(prefillTcKernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
        if (e != cudaSuccess) return e;
        prefillTcKernel<true><<<grid, kThreads, smem, stream>>>(mapQ, mapK, mapV, mapO, p, scaleLog2, errFlag);
    } else {
        e = cudaFuncSetAttribute(prefillTcKernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
        if (e != cudaSuccess) return e;
        prefillTcKernel<false><<<grid, kThreads, smem, stream>>>(mapQ, mapK, mapV, mapO, p, scaleLog2, errFlag);
    }
    if (launches) *launches += 1;
    return cudaGetLastError();
}

}  // namespace pam

#ifdef PAM_PREFILL_TRACE
extern "C" int pamc_debug_cta_times(unsigned long long* out) {
    cudaDeviceSynchronize();
    cudaMemcpyFromSymbol(out, pam::gCtaTimes, sizeof(unsigned long long) * 1024);
    return 1024;
}
extern "C" int pamc_debug_trace_read(long long* out) {
    cudaDeviceSynchronize();
    cudaMemcpyFromSymbol(out, pam::gTrace, sizeof(long long) * pam::kTraceRoles * pam::kTraceTiles * pam::kTraceEvents);
    return pam::kTraceRoles * pam::kTraceTiles * pam::kTraceEvents;
}
#endif
