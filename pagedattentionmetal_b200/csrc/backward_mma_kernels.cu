// Gradients of paged attention for float16 / bfloat16 pools with head_dim 64 or 128 on the
// tensor cores (mma.sync.m16n8k16, float32 accumulation).  Same semantics and the same three
// steps as backward_kernels.cu (row sums; one CTA per tile of 64 keys and KV head that owns the
// tile's rows of dK and dV; dQ through float32 adds), with the five products
//
//     S = Q K^T,  dP = dO V^T,  dV += P^T dO,  dK += dS^T Q,  dQ += dS K
//
// taken from 16-bit tiles in shared memory through ldmatrix.  P and dS are rounded to the
// storage type between the first two products and the last three, like the operands of any
// 16-bit attention kernel; everything is accumulated in float32 and the gradient pools get one
// rounding, where the reference's half atomics round every term.
//
// A CTA has 8 warps.  For the 64 x 64 tile pair (rows, keys) of one head: warp (wr, wc) =
// (warp / 2, warp % 2) takes rows 16 wr .. + 15 and keys 32 wc .. + 31 of S and dP, writes its
// part of P and dS to shared memory, then keys 16 wr .. + 15 and dims wc * hd / 2 .. of dV and dK
// (kept in registers over all rows and all query heads of the KV head) and rows 16 wr .. + 15
// and the same dims of dQ.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <algorithm>
#include <atomic>
#include <cmath>

#include "kernels.h"

namespace pam {
namespace {

constexpr int kThreads = 256, kTile = 64;

__device__ __forceinline__ uint32_t smemAddr(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }
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
template <typename T> __device__ __forceinline__ float2 unpack2(uint32_t v);
template <> __device__ __forceinline__ float2 unpack2<__half>(uint32_t v) { return __half22float2(*reinterpret_cast<__half2*>(&v)); }
template <> __device__ __forceinline__ float2 unpack2<__nv_bfloat16>(uint32_t v) {
    return make_float2(__uint_as_float(v << 16), __uint_as_float(v & 0xFFFF0000u));
}

__device__ __forceinline__ int64_t tokenOffset(const BackwardParams& p, int j, int kvh) {
    const int page = min(j / p.blockSize, p.maxNumBlocks - 1);
    const int64_t blk = min(max(p.table[page], 0), p.poolBlocks - 1);
    return ((blk * p.kvHeads + kvh) * p.blockSize + j % p.blockSize) * static_cast<int64_t>(p.headDim);
}

// Shared memory: four 64 x (HD + 8) tiles and two 64 x 72 tiles of the storage type (the
// 16 bytes of padding per row keep the eight row addresses of an ldmatrix in distinct banks),
// then three 64-long float vectors.
template <typename T, int HD>
struct Tiles {
    static constexpr int RS = HD + 8, PS = kTile + 8;
    T *q, *dO, *k, *v, *p, *dS;
    float *m, *l, *rowSum;
    __device__ explicit Tiles(unsigned char* base) {
        q = reinterpret_cast<T*>(base);
        dO = q + kTile * RS;
        k = dO + kTile * RS;
        v = k + kTile * RS;
        p = v + kTile * RS;
        dS = p + kTile * PS;
        m = reinterpret_cast<float*>(dS + kTile * PS);
        l = m + kTile;
        rowSum = l + kTile;
    }
    static constexpr size_t bytes() { return (static_cast<size_t>(4) * kTile * RS + 2 * kTile * PS) * sizeof(T) + 3 * kTile * sizeof(float); }
};

// 64 rows of HD elements into a tile, 16 bytes per thread and step; `rowPtr(r)` gives the
// global address of row r or null (zeros).  The addresses (a block-table look-up each for
// pool rows) are all taken first and the loads all issued before the first store, so that a
// tile costs two memory round trips, not two per step.
template <typename T, int HD, class F>
__device__ __forceinline__ void loadTile(T* tile, F rowPtr) {
    constexpr int CPR = HD * 2 / 16, RS = HD + 8, N = kTile * CPR / kThreads;
    static_assert(kTile * CPR % kThreads == 0, "a tile is a whole number of steps");
    const T* src[N];
    uint4 val[N];
#pragma unroll
    for (int i = 0; i < N; ++i) src[i] = rowPtr((threadIdx.x + kThreads * i) / CPR);
#pragma unroll
    for (int i = 0; i < N; ++i) {
        val[i] = make_uint4(0u, 0u, 0u, 0u);
        if (src[i]) val[i] = *reinterpret_cast<const uint4*>(src[i] + ((threadIdx.x + kThreads * i) % CPR) * 8);
    }
#pragma unroll
    for (int i = 0; i < N; ++i) {
        const int idx = threadIdx.x + kThreads * i;
        *reinterpret_cast<uint4*>(tile + (idx / CPR) * RS + (idx % CPR) * 8) = val[i];
    }
}

// S and dP of rows 16 wr .. and keys 32 wc .. : s[nt], dp[nt] are the accumulators of the key
// columns 32 wc + 8 nt .. + 7.
template <typename T, int HD>
__device__ __forceinline__ void scoreTiles(const Tiles<T, HD>& t, int wr, int wc, int lane, float (&s)[4][4], float (&dp)[4][4]) {
    constexpr int RS = Tiles<T, HD>::RS;
#pragma unroll
    for (int nt = 0; nt < 4; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) s[nt][e] = dp[nt][e] = 0.f;
    const int aRow = 16 * wr + (lane & 15), aCol = (lane >> 4) * 8;
    const int bRow = 32 * wc + (lane & 7) + 8 * (lane >> 4), bCol = 8 * ((lane >> 3) & 1);
#pragma unroll
    for (int ks = 0; ks < HD / 16; ++ks) {
        uint32_t aq[4], ag[4];
        ldmatrixX4(aq, smemAddr(t.q + aRow * RS + 16 * ks + aCol));
        ldmatrixX4(ag, smemAddr(t.dO + aRow * RS + 16 * ks + aCol));
#pragma unroll
        for (int half = 0; half < 2; ++half) {           // two key tiles of 8 per ldmatrix
            uint32_t bk[4], bv[4];
            ldmatrixX4(bk, smemAddr(t.k + (bRow + 16 * half) * RS + 16 * ks + bCol));
            ldmatrixX4(bv, smemAddr(t.v + (bRow + 16 * half) * RS + 16 * ks + bCol));
            mma16816<T>(s[2 * half], aq, bk[0], bk[1]);
            mma16816<T>(s[2 * half + 1], aq, bk[2], bk[3]);
            mma16816<T>(dp[2 * half], ag, bv[0], bv[1]);
            mma16816<T>(dp[2 * half + 1], ag, bv[2], bv[3]);
        }
    }
}

template <typename T, int HD>
__global__ void __launch_bounds__(kThreads, 2)
backwardMmaRowSumKernel(const BackwardParams p) {
    extern __shared__ __align__(16) unsigned char smemB[];
    Tiles<T, HD> t(smemB);
    const int row0 = blockIdx.x * kTile, head = blockIdx.y;
    const int kvh = head / (p.heads / p.kvHeads);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, wr = warp >> 1, wc = warp & 1;
    const float scale = 1.0f / sqrtf(static_cast<float>(HD));
    const T* q = static_cast<const T*>(p.q);
    const T* dO = static_cast<const T*>(p.dO);
    auto rowOf = [&](const T* base) {
        return [=](int r) -> const T* { return row0 + r < p.seqLen ? base + (static_cast<int64_t>(row0 + r) * p.heads + head) * HD : nullptr; };
    };
    loadTile<T, HD>(t.q, rowOf(q));
    loadTile<T, HD>(t.dO, rowOf(dO));
    for (int r = threadIdx.x; r < kTile; r += kThreads) {
        const bool in = row0 + r < p.seqLen;
        t.m[r] = in ? p.m[static_cast<int64_t>(row0 + r) * p.heads + head] : 0.f;
        t.l[r] = in ? p.l[static_cast<int64_t>(row0 + r) * p.heads + head] : 1.f;
        t.rowSum[r] = 0.f;
    }
    const int rA = 16 * wr + (lane >> 2), rB = rA + 8;
    float sumA = 0.f, sumB = 0.f;
    for (int key0 = p.windowStart; key0 < p.seqLen; key0 += kTile) {
        __syncthreads();
        auto keyOf = [&](const void* pool) {
            const T* base = static_cast<const T*>(pool);
            return [=](int r) -> const T* { return key0 + r < p.seqLen ? base + tokenOffset(p, key0 + r, kvh) : nullptr; };
        };
        loadTile<T, HD>(t.k, keyOf(p.kPool));
        loadTile<T, HD>(t.v, keyOf(p.vPool));
        __syncthreads();
        float s[4][4], dp[4][4];
        scoreTiles<T, HD>(t, wr, wc, lane, s, dp);
        const float mA = t.m[rA], mB = t.m[rB], ilA = 1.f / t.l[rA], ilB = 1.f / t.l[rB];
#pragma unroll
        for (int nt = 0; nt < 4; ++nt)
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int j = key0 + 32 * wc + 8 * nt + 2 * (lane & 3) + e;
                if (j < p.seqLen) {
                    sumA += expf(s[nt][e] * scale - mA) * ilA * dp[nt][e];
                    sumB += expf(s[nt][e + 2] * scale - mB) * ilB * dp[nt][e + 2];
                }
            }
    }
    sumA += __shfl_xor_sync(0xFFFFFFFFu, sumA, 1);
    sumA += __shfl_xor_sync(0xFFFFFFFFu, sumA, 2);
    sumB += __shfl_xor_sync(0xFFFFFFFFu, sumB, 1);
    sumB += __shfl_xor_sync(0xFFFFFFFFu, sumB, 2);
    __syncthreads();
    if ((lane & 3) == 0) {                // the two warps of a row block hold the two halves of the keys
        atomicAdd(&t.rowSum[rA], sumA);
        atomicAdd(&t.rowSum[rB], sumB);
    }
    __syncthreads();
    for (int r = threadIdx.x; r < kTile; r += kThreads)
        if (row0 + r < p.seqLen) p.rowSum[static_cast<int64_t>(row0 + r) * p.heads + head] = t.rowSum[r];
}

template <typename T, int HD>
__global__ void __launch_bounds__(kThreads, 2)
backwardMmaKeyTileKernel(const BackwardParams p) {
    constexpr int RS = Tiles<T, HD>::RS, PS = Tiles<T, HD>::PS;
    constexpr int NT = HD / 16;                       // 8-wide dim tiles of a warp's half of the head
    extern __shared__ __align__(16) unsigned char smemB[];
    Tiles<T, HD> t(smemB);
    const int key0 = p.windowStart + blockIdx.x * kTile, kvh = blockIdx.y;
    const int G = p.heads / p.kvHeads;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, wr = warp >> 1, wc = warp & 1;
    const float scale = 1.0f / sqrtf(static_cast<float>(HD));
    const int dim0 = wc * (HD / 2);
    {
        auto keyOf = [&](const void* pool) {
            const T* base = static_cast<const T*>(pool);
            return [=](int r) -> const T* { return key0 + r < p.seqLen ? base + tokenOffset(p, key0 + r, kvh) : nullptr; };
        };
        loadTile<T, HD>(t.k, keyOf(p.kPool));
        loadTile<T, HD>(t.v, keyOf(p.vPool));
    }
    float dK[NT][4], dV[NT][4];           // keys 16 wr + lane / 4 (+ 8), dims dim0 + 8 nt + 2 (lane % 4) (+ 1)
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) dK[nt][e] = dV[nt][e] = 0.f;
    const int rA = 16 * wr + (lane >> 2), rB = rA + 8;

    for (int g = 0; g < G; ++g) {
        const int head = kvh * G + g;
        const T* q = static_cast<const T*>(p.q);
        const T* dO = static_cast<const T*>(p.dO);
        for (int row0 = 0; row0 < p.seqLen; row0 += kTile) {
            __syncthreads();
            auto rowOf = [&](const T* base) {
                return [=](int r) -> const T* { return row0 + r < p.seqLen ? base + (static_cast<int64_t>(row0 + r) * p.heads + head) * HD : nullptr; };
            };
            loadTile<T, HD>(t.q, rowOf(q));
            loadTile<T, HD>(t.dO, rowOf(dO));
            for (int r = threadIdx.x; r < kTile; r += kThreads) {
                const bool in = row0 + r < p.seqLen;
                const int64_t at = static_cast<int64_t>(row0 + r) * p.heads + head;
                t.m[r] = in ? p.m[at] : 0.f;
                t.l[r] = in ? p.l[at] : 1.f;
                t.rowSum[r] = in ? p.rowSum[at] : 0.f;
            }
            __syncthreads();
            {
                float s[4][4], dp[4][4];
                scoreTiles<T, HD>(t, wr, wc, lane, s, dp);
                const bool inA = row0 + rA < p.seqLen, inB = row0 + rB < p.seqLen;
                const float mA = t.m[rA], mB = t.m[rB], ilA = 1.f / t.l[rA], ilB = 1.f / t.l[rB];
                const float dA = t.rowSum[rA], dB = t.rowSum[rB];
#pragma unroll
                for (int nt = 0; nt < 4; ++nt) {
                    const int col = 32 * wc + 8 * nt + 2 * (lane & 3);
                    float pa[2], pb[2], sa[2], sb[2];
#pragma unroll
                    for (int e = 0; e < 2; ++e) {
                        const bool keyIn = key0 + col + e < p.seqLen;
                        pa[e] = inA && keyIn ? expf(s[nt][e] * scale - mA) * ilA : 0.f;
                        pb[e] = inB && keyIn ? expf(s[nt][e + 2] * scale - mB) * ilB : 0.f;
                        sa[e] = pa[e] * (dp[nt][e] - dA);
                        sb[e] = pb[e] * (dp[nt][e + 2] - dB);
                    }
                    *reinterpret_cast<uint32_t*>(t.p + rA * PS + col) = pack2<T>(pa[0], pa[1]);
                    *reinterpret_cast<uint32_t*>(t.p + rB * PS + col) = pack2<T>(pb[0], pb[1]);
                    *reinterpret_cast<uint32_t*>(t.dS + rA * PS + col) = pack2<T>(sa[0], sa[1]);
                    *reinterpret_cast<uint32_t*>(t.dS + rB * PS + col) = pack2<T>(sb[0], sb[1]);
                }
            }
            __syncthreads();
            // dV += P^T dO and dK += dS^T Q: A = the transposed 16 x 16 blocks of P / dS (keys 16 wr ..,
            // rows 16 ks ..), B = dO / Q rows 16 ks .. at this warp's dims
#pragma unroll
            for (int ks = 0; ks < kTile / 16; ++ks) {
                uint32_t ap[4], as[4];
                const int tRow = 16 * ks + (lane & 7) + 8 * (lane >> 4), tCol = 16 * wr + 8 * ((lane >> 3) & 1);
                ldmatrixX4Trans(ap, smemAddr(t.p + tRow * PS + tCol));
                ldmatrixX4Trans(as, smemAddr(t.dS + tRow * PS + tCol));
                const int bRow = 16 * ks + (lane & 7) + 8 * ((lane >> 3) & 1), bColBase = dim0 + 8 * (lane >> 4);
#pragma unroll
                for (int n2 = 0; n2 < NT / 2; ++n2) {
                    uint32_t bg[4], bq[4];
                    ldmatrixX4Trans(bg, smemAddr(t.dO + bRow * RS + bColBase + 16 * n2));
                    ldmatrixX4Trans(bq, smemAddr(t.q + bRow * RS + bColBase + 16 * n2));
                    mma16816<T>(dV[2 * n2], ap, bg[0], bg[1]);
                    mma16816<T>(dV[2 * n2 + 1], ap, bg[2], bg[3]);
                    mma16816<T>(dK[2 * n2], as, bq[0], bq[1]);
                    mma16816<T>(dK[2 * n2 + 1], as, bq[2], bq[3]);
                }
            }
            // dQ of rows 16 wr .. at this warp's dims: A = dS (rows, keys 16 ks ..), B = K rows 16 ks ..
            float dq[NT][4];
#pragma unroll
            for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                for (int e = 0; e < 4; ++e) dq[nt][e] = 0.f;
#pragma unroll
            for (int ks = 0; ks < kTile / 16; ++ks) {
                uint32_t as[4];
                ldmatrixX4(as, smemAddr(t.dS + (16 * wr + (lane & 15)) * PS + 16 * ks + (lane >> 4) * 8));
                const int bRow = 16 * ks + (lane & 7) + 8 * ((lane >> 3) & 1), bColBase = dim0 + 8 * (lane >> 4);
#pragma unroll
                for (int n2 = 0; n2 < NT / 2; ++n2) {
                    uint32_t bk[4];
                    ldmatrixX4Trans(bk, smemAddr(t.k + bRow * RS + bColBase + 16 * n2));
                    mma16816<T>(dq[2 * n2], as, bk[0], bk[1]);
                    mma16816<T>(dq[2 * n2 + 1], as, bk[2], bk[3]);
                }
            }
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                const int d = dim0 + 8 * nt + 2 * (lane & 3);
                if (row0 + rA < p.seqLen) {
                    float* dst = p.dQAcc + (static_cast<int64_t>(row0 + rA) * p.heads + head) * HD + d;
                    atomicAdd(dst, dq[nt][0] * scale);
                    atomicAdd(dst + 1, dq[nt][1] * scale);
                }
                if (row0 + rB < p.seqLen) {
                    float* dst = p.dQAcc + (static_cast<int64_t>(row0 + rB) * p.heads + head) * HD + d;
                    atomicAdd(dst, dq[nt][2] * scale);
                    atomicAdd(dst + 1, dq[nt][3] * scale);
                }
            }
        }
    }
    // the tile's rows of the gradient pools belong to this CTA alone
    T* dKPool = static_cast<T*>(p.dKPool);
    T* dVPool = static_cast<T*>(p.dVPool);
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        const int j = key0 + (half ? rB : rA);
        if (j >= p.seqLen) continue;
        const int64_t off = tokenOffset(p, j, kvh);
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            const int d = dim0 + 8 * nt + 2 * (lane & 3);
            uint32_t* kw = reinterpret_cast<uint32_t*>(dKPool + off + d);
            uint32_t* vw = reinterpret_cast<uint32_t*>(dVPool + off + d);
            const float2 k0 = unpack2<T>(*kw), v0 = unpack2<T>(*vw);
            *kw = pack2<T>(k0.x + dK[nt][2 * half] * scale, k0.y + dK[nt][2 * half + 1] * scale);
            *vw = pack2<T>(v0.x + dV[nt][2 * half], v0.y + dV[nt][2 * half + 1]);
        }
    }
}

template <typename T>
__global__ void backwardMmaStoreKernel(const float* __restrict__ acc, T* __restrict__ out, int64_t n) {
    for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < n; i += static_cast<int64_t>(gridDim.x) * blockDim.x)
        out[i] = static_cast<T>(acc[i]);
}

template <class K>
cudaError_t allowShared(K kernel, size_t bytes, std::atomic<size_t>* granted) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
    if (granted[dev].load(std::memory_order_acquire) >= bytes) return cudaSuccess;
    e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(bytes));
    if (e == cudaSuccess) granted[dev].store(bytes, std::memory_order_release);
    return e;
}

template <typename T, int HD>
cudaError_t launchT(const BackwardParams& p, cudaStream_t stream, int* launches) {
    static std::atomic<size_t> grantedRowSum[64], grantedKeyTile[64];
    constexpr size_t smem = Tiles<T, HD>::bytes();
    cudaError_t e = allowShared(backwardMmaRowSumKernel<T, HD>, smem, grantedRowSum);
    if (e == cudaSuccess) e = allowShared(backwardMmaKeyTileKernel<T, HD>, smem, grantedKeyTile);
    if (e != cudaSuccess) return e;
    const int64_t n = static_cast<int64_t>(p.seqLen) * p.heads * HD;
    e = cudaMemsetAsync(p.dQAcc, 0, static_cast<size_t>(n) * sizeof(float), stream);
    if (e != cudaSuccess) return e;
    const int rowTiles = (p.seqLen + kTile - 1) / kTile;
    const int keyTiles = (p.seqLen - p.windowStart + kTile - 1) / kTile;
    backwardMmaRowSumKernel<T, HD><<<dim3(rowTiles, p.heads), kThreads, smem, stream>>>(p);
    e = cudaGetLastError();
    if (e != cudaSuccess) return e;
    if (launches) *launches += 1;
    if (keyTiles > 0) {
        backwardMmaKeyTileKernel<T, HD><<<dim3(keyTiles, p.kvHeads), kThreads, smem, stream>>>(p);
        e = cudaGetLastError();
        if (e != cudaSuccess) return e;
        if (launches) *launches += 1;
    }
    backwardMmaStoreKernel<T><<<static_cast<unsigned>(std::min<int64_t>((n + 255) / 256, 148 * 8)), 256, 0, stream>>>(
        p.dQAcc, static_cast<T*>(p.dQ), n);
    e = cudaGetLastError();
    if (e == cudaSuccess && launches) *launches += 1;
    return e;
}

}  // namespace

bool backwardTensorPathApplies(const BackwardParams& p) {
    const auto aligned16 = [](const void* ptr) { return (reinterpret_cast<uintptr_t>(ptr) & 15) == 0; };
    return (p.dtype == kF16 || p.dtype == kBF16) && (p.headDim == 64 || p.headDim == 128) && aligned16(p.q) && aligned16(p.dO) &&
           aligned16(p.kPool) && aligned16(p.vPool) && aligned16(p.dKPool) && aligned16(p.dVPool);
}

cudaError_t launchBackwardTensor(const BackwardParams& p, cudaStream_t stream, int* launches) {
    if (p.dtype == kF16)
        return p.headDim == 128 ? launchT<__half, 128>(p, stream, launches) : launchT<__half, 64>(p, stream, launches);
    return p.headDim == 128 ? launchT<__nv_bfloat16, 128>(p, stream, launches) : launchT<__nv_bfloat16, 64>(p, stream, launches);
}

}  // namespace pam
