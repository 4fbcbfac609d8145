// Gradients of paged attention with respect to the queries and the paged keys and values.
//
// Semantics: paged_attention_backward / _f16 (kernels.metal:1217-1415), dispatched by
// PagedAttentionEngine.backward (PagedAttentionEngine.swift:1341-1395).  Every row i of every
// head sees the keys [window_start, L) reached through the block table (the kernel has no
// causal mask); the caller hands over the row maximum m and the row sum l of its forward
// pass.  With P_ij = exp(q_i.k_j / sqrt(d) - m_i) / l_i, dP_ij = dO_i.v_j,
// rowsum_i = sum_j P_ij dP_ij and dS_ij = P_ij (dP_ij - rowsum_i):
//
//     dQ_i  = sum_j dS_ij k_j / sqrt(d)
//     dK_j += sum over rows and the query heads of the KV head of dS_ij q_i / sqrt(d)
//     dV_j += sum over rows and heads of P_ij dO_i
//
// (the pool gradients are added to what the gradient pools hold, as the reference's atomic
// adds do).  The reference runs one thread per (dim, row, head), each of which walks all
// keys twice and adds its dK / dV terms with float (half) compare-and-swap atomics.  Here:
//
//  * backwardRowSumKernel -- one CTA per (tile of query rows, head): S = Q K^T and
//    dP = dO V^T tile by tile over the keys, rowsum_i reduced in registers.
//  * backwardKeyTileKernel -- one CTA per (tile of keys, KV head).  It owns the tile's rows
//    of dK and dV (no atomics on them: they are accumulated in registers over all rows and
//    all query heads of the KV head and added to the pool once, in float32 whatever the pool
//    type), recomputes S and dP against every tile of query rows, and adds its share of dQ
//    into a float32 buffer with red.global.add.f32.
//  * backwardStoreKernel -- float32 dQ to the output type (16-bit types only).
//
// The products of this file run on the CUDA cores in float32 (4 x 4 register blocks out of
// shared memory): the float32 path of the reference is float32 arithmetic, which tensor cores
// would only reach through split operands.  float16 / bfloat16 with head_dim 64 or 128 take the
// tensor-core form of backward_mma_kernels.cu instead.  Pools are
// [block][kv_head][block_size][head_dim] like everywhere here.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <algorithm>
#include <atomic>
#include <cmath>

#include "kernels.h"

namespace pam {
namespace {

constexpr int kThreads = 256;

__device__ __forceinline__ float asFloat(float v) { return v; }
__device__ __forceinline__ float asFloat(__half v) { return __half2float(v); }
__device__ __forceinline__ float asFloat(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T fromFloatB(float v);
template <> __device__ __forceinline__ float fromFloatB<float>(float v) { return v; }
template <> __device__ __forceinline__ __half fromFloatB<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 fromFloatB<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// Element offset of (token j, kv head, dim 0) in a pool; table entries are clamped into it.
__device__ __forceinline__ int64_t tokenOffset(const BackwardParams& p, int j, int kvh) {
    const int page = min(j / p.blockSize, p.maxNumBlocks - 1);
    const int64_t blk = min(max(p.table[page], 0), p.poolBlocks - 1);
    return ((blk * p.kvHeads + kvh) * p.blockSize + j % p.blockSize) * static_cast<int64_t>(p.headDim);
}

// Shared memory of both kernels, in floats: four TILE x HS tiles (HS = head_dim | 1, so that
// rows a multiple of 32 words apart do not meet in one bank), two TILE x (TILE + 1) tiles,
// three TILE-long row vectors.
template <int TILE>
struct Tiles {
    float *q, *dO, *k, *v, *p, *dS, *m, *l, *rowSum;
    int HS;
    __device__ Tiles(float* base, int headDim) {
        HS = headDim | 1;
        q = base;
        dO = q + TILE * HS;
        k = dO + TILE * HS;
        v = k + TILE * HS;
        p = v + TILE * HS;
        dS = p + TILE * (TILE + 1);
        m = dS + TILE * (TILE + 1);
        l = m + TILE;
        rowSum = l + TILE;
    }
};
template <int TILE>
size_t tilesBytes(int headDim) {
    return (static_cast<size_t>(4) * TILE * (headDim | 1) + 2 * TILE * (TILE + 1) + 3 * TILE) * sizeof(float);
}

// Rows [row0, row0 + TILE) of one head of a [rows][heads][dim] array into a tile (rows past the end: zeros).
template <typename T, int TILE>
__device__ __forceinline__ void loadRows(float* tile, int HS, const T* src, int row0, int head, const BackwardParams& p) {
    const int hd = p.headDim;
    for (int idx = threadIdx.x; idx < TILE * hd; idx += kThreads) {
        const int r = idx / hd, d = idx - r * hd;
        const int i = row0 + r;
        tile[r * HS + d] = i < p.seqLen ? asFloat(src[(static_cast<int64_t>(i) * p.heads + head) * hd + d]) : 0.f;
    }
}
// Keys [key0, key0 + TILE) of one KV head of a pool into a tile (keys past the end: zeros).
template <typename T, int TILE>
__device__ __forceinline__ void loadKeys(float* tile, int HS, const T* pool, int key0, int kvh, const BackwardParams& p) {
    const int hd = p.headDim;
    for (int idx = threadIdx.x; idx < TILE * hd; idx += kThreads) {
        const int r = idx / hd, d = idx - r * hd;
        const int j = key0 + r;
        tile[r * HS + d] = j < p.seqLen ? asFloat(pool[tokenOffset(p, j, kvh) + d]) : 0.f;
    }
}

// The R x R block (rows R ty .., keys R tx ..) of S = Q K^T and of dP = dO V^T.
template <int TILE, int R>
__device__ __forceinline__ void scoreBlocks(const Tiles<TILE>& t, int headDim, int ty, int tx, float (&s)[R][R], float (&dp)[R][R]) {
#pragma unroll
    for (int a = 0; a < R; ++a)
#pragma unroll
        for (int b = 0; b < R; ++b) s[a][b] = dp[a][b] = 0.f;
    const int HS = t.HS;
    for (int k = 0; k < headDim; ++k) {
        float qv[R], gv[R], kv[R], vv[R];
#pragma unroll
        for (int a = 0; a < R; ++a) {
            qv[a] = t.q[(R * ty + a) * HS + k];
            gv[a] = t.dO[(R * ty + a) * HS + k];
            kv[a] = t.k[(R * tx + a) * HS + k];
            vv[a] = t.v[(R * tx + a) * HS + k];
        }
#pragma unroll
        for (int a = 0; a < R; ++a)
#pragma unroll
            for (int b = 0; b < R; ++b) {
                s[a][b] += qv[a] * kv[b];
                dp[a][b] += gv[a] * vv[b];
            }
    }
}

template <typename T, int TILE>
__global__ void __launch_bounds__(kThreads)
backwardRowSumKernel(const BackwardParams p) {
    constexpr int R = TILE / 16;
    extern __shared__ __align__(16) float smemF[];
    Tiles<TILE> t(smemF, p.headDim);
    const int row0 = blockIdx.x * TILE, head = blockIdx.y;
    const int kvh = head / (p.heads / p.kvHeads);
    const int ty = threadIdx.x / 16, tx = threadIdx.x % 16;
    const float scale = 1.0f / sqrtf(static_cast<float>(p.headDim));          // kernels.metal:1243
    loadRows<T, TILE>(t.q, t.HS, static_cast<const T*>(p.q), row0, head, p);
    loadRows<T, TILE>(t.dO, t.HS, static_cast<const T*>(p.dO), row0, head, p);
    for (int r = threadIdx.x; r < TILE; r += kThreads) {
        const int i = row0 + r;
        t.m[r] = i < p.seqLen ? p.m[static_cast<int64_t>(i) * p.heads + head] : 0.f;
        t.l[r] = i < p.seqLen ? p.l[static_cast<int64_t>(i) * p.heads + head] : 1.f;
    }
    float sum[R];
#pragma unroll
    for (int a = 0; a < R; ++a) sum[a] = 0.f;
    for (int key0 = p.windowStart; key0 < p.seqLen; key0 += TILE) {
        __syncthreads();
        loadKeys<T, TILE>(t.k, t.HS, static_cast<const T*>(p.kPool), key0, kvh, p);
        loadKeys<T, TILE>(t.v, t.HS, static_cast<const T*>(p.vPool), key0, kvh, p);
        __syncthreads();
        float s[R][R], dp[R][R];
        scoreBlocks<TILE, R>(t, p.headDim, ty, tx, s, dp);
#pragma unroll
        for (int a = 0; a < R; ++a)
#pragma unroll
            for (int b = 0; b < R; ++b) {
                const int j = key0 + R * tx + b;
                if (j < p.seqLen) sum[a] += expf(s[a][b] * scale - t.m[R * ty + a]) / t.l[R * ty + a] * dp[a][b];     // :1283-1286
            }
    }
    // the 16 threads that share a block of rows sit in one half of a warp
#pragma unroll
    for (int a = 0; a < R; ++a) {
#pragma unroll
        for (int o = 1; o < 16; o <<= 1) sum[a] += __shfl_xor_sync(0xFFFFFFFFu, sum[a], o);
        const int i = row0 + R * ty + a;
        if (tx == 0 && i < p.seqLen) p.rowSum[static_cast<int64_t>(i) * p.heads + head] = sum[a];
    }
}

template <typename T, int TILE, int MAXHD>
__global__ void __launch_bounds__(kThreads)
backwardKeyTileKernel(const BackwardParams p) {
    constexpr int R = TILE / 16, C = MAXHD / 16;
    extern __shared__ __align__(16) float smemF[];
    Tiles<TILE> t(smemF, p.headDim);
    const int key0 = p.windowStart + blockIdx.x * TILE, kvh = blockIdx.y;
    const int G = p.heads / p.kvHeads, hd = p.headDim, HS = t.HS;
    const int ty = threadIdx.x / 16, tx = threadIdx.x % 16;
    const float scale = 1.0f / sqrtf(static_cast<float>(hd));
    loadKeys<T, TILE>(t.k, HS, static_cast<const T*>(p.kPool), key0, kvh, p);
    loadKeys<T, TILE>(t.v, HS, static_cast<const T*>(p.vPool), key0, kvh, p);
    // this thread's part of the tile's gradients: keys R ty + a, dims tx + 16 c
    float dK[R][C], dV[R][C];
#pragma unroll
    for (int a = 0; a < R; ++a)
#pragma unroll
        for (int c = 0; c < C; ++c) dK[a][c] = dV[a][c] = 0.f;

    for (int g = 0; g < G; ++g) {
        const int head = kvh * G + g;
        for (int row0 = 0; row0 < p.seqLen; row0 += TILE) {
            __syncthreads();
            loadRows<T, TILE>(t.q, HS, static_cast<const T*>(p.q), row0, head, p);
            loadRows<T, TILE>(t.dO, HS, static_cast<const T*>(p.dO), row0, head, p);
            for (int r = threadIdx.x; r < TILE; r += kThreads) {
                const int i = row0 + r;
                const bool in = i < p.seqLen;
                t.m[r] = in ? p.m[static_cast<int64_t>(i) * p.heads + head] : 0.f;
                t.l[r] = in ? p.l[static_cast<int64_t>(i) * p.heads + head] : 1.f;
                t.rowSum[r] = in ? p.rowSum[static_cast<int64_t>(i) * p.heads + head] : 0.f;
            }
            __syncthreads();
            {
                float s[R][R], dp[R][R];
                scoreBlocks<TILE, R>(t, hd, ty, tx, s, dp);
#pragma unroll
                for (int a = 0; a < R; ++a)
#pragma unroll
                    for (int b = 0; b < R; ++b) {
                        const int row = R * ty + a, col = R * tx + b;
                        const bool in = row0 + row < p.seqLen && key0 + col < p.seqLen;
                        const float pij = in ? expf(s[a][b] * scale - t.m[row]) / t.l[row] : 0.f;       // :1283
                        t.p[row * (TILE + 1) + col] = pij;
                        t.dS[row * (TILE + 1) + col] = pij * (dp[a][b] - t.rowSum[row]);               // :1285
                    }
            }
            __syncthreads();
            // dV += P^T dO, dK += dS^T Q (the factor 1/sqrt(d) at the end)
            for (int row = 0; row < TILE; ++row) {
                float pv[R], dv[R];
#pragma unroll
                for (int a = 0; a < R; ++a) {
                    pv[a] = t.p[row * (TILE + 1) + R * ty + a];
                    dv[a] = t.dS[row * (TILE + 1) + R * ty + a];
                }
#pragma unroll
                for (int c = 0; c < C; ++c) {
                    const int d = tx + 16 * c;
                    if (d < hd) {
                        const float x = t.dO[row * HS + d], y = t.q[row * HS + d];
#pragma unroll
                        for (int a = 0; a < R; ++a) {
                            dV[a][c] += pv[a] * x;
                            dK[a][c] += dv[a] * y;
                        }
                    }
                }
            }
            // this key tile's share of dQ: rows R ty + a, dims tx + 16 c
            float dq[R][C];
#pragma unroll
            for (int a = 0; a < R; ++a)
#pragma unroll
                for (int c = 0; c < C; ++c) dq[a][c] = 0.f;
            for (int key = 0; key < TILE; ++key) {
                float dv[R];
#pragma unroll
                for (int a = 0; a < R; ++a) dv[a] = t.dS[(R * ty + a) * (TILE + 1) + key];
#pragma unroll
                for (int c = 0; c < C; ++c) {
                    const int d = tx + 16 * c;
                    if (d < hd) {
                        const float kd = t.k[key * HS + d];
#pragma unroll
                        for (int a = 0; a < R; ++a) dq[a][c] += dv[a] * kd;
                    }
                }
            }
#pragma unroll
            for (int a = 0; a < R; ++a) {
                const int i = row0 + R * ty + a;
                if (i >= p.seqLen) continue;
                float* dst = p.dQAcc + (static_cast<int64_t>(i) * p.heads + head) * hd;
#pragma unroll
                for (int c = 0; c < C; ++c) {
                    const int d = tx + 16 * c;
                    if (d < hd) atomicAdd(dst + d, dq[a][c] * scale);                                   // :1287, 1300
                }
            }
        }
    }
    // the tile's rows of the gradient pools belong to this CTA alone
    T* dKPool = static_cast<T*>(p.dKPool);
    T* dVPool = static_cast<T*>(p.dVPool);
#pragma unroll
    for (int a = 0; a < R; ++a) {
        const int j = key0 + R * ty + a;
        if (j >= p.seqLen) continue;
        const int64_t off = tokenOffset(p, j, kvh);
#pragma unroll
        for (int c = 0; c < C; ++c) {
            const int d = tx + 16 * c;
            if (d < hd) {
                dKPool[off + d] = fromFloatB<T>(asFloat(dKPool[off + d]) + dK[a][c] * scale);           // :1289-1291
                dVPool[off + d] = fromFloatB<T>(asFloat(dVPool[off + d]) + dV[a][c]);                   // :1293-1295
            }
        }
    }
}

template <typename T>
__global__ void backwardStoreKernel(const float* __restrict__ acc, T* __restrict__ out, int64_t n) {
    for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < n; i += static_cast<int64_t>(gridDim.x) * blockDim.x)
        out[i] = fromFloatB<T>(acc[i]);
}

// The dynamic shared memory limit of a kernel is raised once per device, not per launch.
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

template <typename T, int TILE, int MAXHD>
cudaError_t launchT(const BackwardParams& p, cudaStream_t stream, int* launches) {
    static std::atomic<size_t> grantedRowSum[64], grantedKeyTile[64];
    const size_t smem = tilesBytes<TILE>(p.headDim);
    cudaError_t e = allowShared(backwardRowSumKernel<T, TILE>, smem, grantedRowSum);
    if (e == cudaSuccess) e = allowShared(backwardKeyTileKernel<T, TILE, MAXHD>, smem, grantedKeyTile);
    if (e != cudaSuccess) return e;
    const size_t dqBytes = static_cast<size_t>(p.seqLen) * p.heads * p.headDim * sizeof(float);
    e = cudaMemsetAsync(p.dQAcc, 0, dqBytes, stream);
    if (e != cudaSuccess) return e;
    const int rowTiles = (p.seqLen + TILE - 1) / TILE;
    const int keyTiles = (p.seqLen - p.windowStart + TILE - 1) / TILE;
    backwardRowSumKernel<T, TILE><<<dim3(rowTiles, p.heads), kThreads, smem, stream>>>(p);
    e = cudaGetLastError();
    if (e != cudaSuccess) return e;
    if (launches) *launches += 1;
    if (keyTiles > 0) {
        backwardKeyTileKernel<T, TILE, MAXHD><<<dim3(keyTiles, p.kvHeads), kThreads, smem, stream>>>(p);
        e = cudaGetLastError();
        if (e != cudaSuccess) return e;
        if (launches) *launches += 1;
    }
    if (static_cast<void*>(p.dQAcc) != p.dQ) {
        const int64_t n = static_cast<int64_t>(p.seqLen) * p.heads * p.headDim;
        backwardStoreKernel<T><<<static_cast<unsigned>(std::min<int64_t>((n + 255) / 256, 148 * 8)), 256, 0, stream>>>(
            p.dQAcc, static_cast<T*>(p.dQ), n);
        e = cudaGetLastError();
        if (e == cudaSuccess && launches) *launches += 1;
    }
    return e;
}

template <typename T>
cudaError_t launchByDim(const BackwardParams& p, cudaStream_t stream, int* launches) {
    if (p.headDim <= 128) return launchT<T, 64, 128>(p, stream, launches);
    return launchT<T, 32, 256>(p, stream, launches);
}

}  // namespace

size_t backwardWorkspaceBytes(const BackwardParams& p) {
    const size_t rows = static_cast<size_t>(p.seqLen) * p.heads;
    size_t bytes = (rows * sizeof(float) + 255) / 256 * 256;                                   // rowsum_i
    if (p.dtype != kF32) bytes += rows * p.headDim * sizeof(float);                            // float32 dQ
    return bytes;
}

cudaError_t launchBackward(const BackwardParams& p, cudaStream_t stream, int* launches) {
    if (p.seqLen <= 0) return cudaSuccess;
    if (p.headDim <= 0 || p.headDim > 256 || p.kvHeads <= 0 || p.heads % p.kvHeads != 0 || p.poolBlocks <= 0 || p.maxNumBlocks <= 0 ||
        p.windowStart < 0 || p.windowStart > p.seqLen)
        return cudaErrorInvalidValue;
    if (backwardTensorPathApplies(p)) return launchBackwardTensor(p, stream, launches);
    switch (p.dtype) {
        case kF32: return launchByDim<float>(p, stream, launches);
        case kF16: return launchByDim<__half>(p, stream, launches);
        case kBF16: return launchByDim<__nv_bfloat16>(p, stream, launches);
    }
    return cudaErrorInvalidValue;
}

}  // namespace pam
