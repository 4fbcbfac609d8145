// KV append ("reshape_and_cache"), FP8 e4m3 quantising append and copy-on-write
// block copies for pools laid out [block][kv_head][block_size][head_dim].
//
// Semantics follow kv_cache_append[_f16] (kernels.metal:1804-1874),
// kv_cache_scale_fp8 + kv_cache_append_fp8 (kernels.metal:1876-1961), the
// software codec quantize_fp8 (kernels.metal:564-601) and the host memcpy of
// KVCacheManager.copyOnWrite (KVCacheManager.swift:176-194).  The FP8 scale
// group is (block, kv_head) instead of the reference's whole block.
//
// These are byte-moving kernels bound by HBM bandwidth: every thread moves
// 16-byte vectors, rows of one (token, kv_head) are contiguous on both sides.
#include <cuda_fp16.h>

#include "kernels.h"

namespace pam {
namespace {

// Slot of token t, or -1 when it lies outside the pool (such a token is skipped
// instead of written out of bounds).
__device__ __forceinline__ int64_t slotOf(const SlotSource& s, int t, int blockSize) {
    int64_t slot;
    if (s.slots) slot = s.slots[t];
    else {
        int pos = s.tokenOffset + t;                               // kernels.metal:1823-1827
        slot = static_cast<int64_t>(s.table[pos / blockSize]) * blockSize + pos % blockSize;
    }
    return (slot >= 0 && slot < s.numSlots) ? slot : -1;
}

// One thread per VEC-byte piece of a (token, kv_head) row, K and V together.
template <typename Vec>
__global__ void reshapeAndCacheKernel(const Vec* __restrict__ keys, const Vec* __restrict__ values,
                                      Vec* __restrict__ kPool, Vec* __restrict__ vPool,
                                      SlotSource src, int numTokens, int kvHeads, int blockSize,
                                      int rowVecs) {
    const int64_t total = static_cast<int64_t>(numTokens) * kvHeads * rowVecs;
    for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total;
         i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        const int c = static_cast<int>(i % rowVecs);
        const int64_t row = i / rowVecs;
        const int kvh = static_cast<int>(row % kvHeads);
        const int t = static_cast<int>(row / kvHeads);
        const int64_t slot = slotOf(src, t, blockSize);
        if (slot < 0) continue;
        const int64_t blk = slot / blockSize, off = slot % blockSize;
        const int64_t dst = ((blk * kvHeads + kvh) * blockSize + off) * rowVecs + c;
        kPool[dst] = keys[i];
        vPool[dst] = values[i];
    }
}

// ---- FP8 ----------------------------------------------------------------

// quantize_fp8 (kernels.metal:564-601) on the float32 quotient, with Metal's
// round() (half away from zero) done in integer arithmetic.
__device__ __forceinline__ uint32_t quantizeE4m3(float value, float scale) {
    float v = __fdiv_rn(value, scale);                             // :565, IEEE divide
    v = fminf(fmaxf(v, -448.0f), 448.0f);                          // :566
    const uint32_t sign = v < 0.0f ? 0x80u : 0u;                   // :568 (-0.0 is not < 0)
    const float a = fabsf(v);
    if (a == 0.0f) return 0u;                                      // :571
    if (a < 0x1p-6f) {                                             // :573-578
        // round(a*512) = floor(a*512 + 1/2) = (floor(a*1024) + 1) >> 1
        uint32_t m = (static_cast<uint32_t>(a * 1024.0f) + 1u) >> 1;
        return sign | (m > 7u ? 7u : m);
    }
    const uint32_t bits = __float_as_uint(a);
    int eb = static_cast<int>(bits >> 23) - 127 + 7;               // :580-589, a = 1.f * 2^(eb-7)
    uint32_t m = ((bits & 0x7FFFFFu) + (1u << 19)) >> 20;          // :590-591, round((1.f-1)*8)
    if (m > 7u) { m = 0u; ++eb; }                                  // :592
    if (eb > 15) return sign | 0x7Eu;                              // :585-586, :593-595
    if (eb == 15 && m > 6u) m = 6u;                                // :596-598
    return sign | (static_cast<uint32_t>(eb) << 3) | m;
}

__device__ __forceinline__ float warpMax(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xFFFFFFFFu, v, o));
    return v;
}

// Pass 1 (kernels.metal:1876-1905): absmax of every new (token, kv_head) row
// folded into its group's word.  A word is (epoch << 32) | float bits, so one
// 64-bit atomicMax both resets stale values of earlier calls and takes the
// maximum within this call; nothing has to be cleared between calls.
__global__ void fp8AbsmaxKernel(const __half* __restrict__ keys, const __half* __restrict__ values,
                                SlotSource src, int numTokens, int kvHeads, int blockSize,
                                int headDim, unsigned long long* __restrict__ amax, uint32_t epoch) {
    const int lane = threadIdx.x & 31;
    const int64_t rows = static_cast<int64_t>(numTokens) * kvHeads;
    const int64_t warpsTotal = (static_cast<int64_t>(gridDim.x) * blockDim.x) >> 5;
    for (int64_t row = (blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x) >> 5;
         row < rows; row += warpsTotal) {
        const __half* k = keys + row * headDim;
        const __half* v = values + row * headDim;
        float ka = 0.f, va = 0.f;
        if ((headDim & 7) == 0) {
            for (int d = lane * 8; d < headDim; d += 256) {
                uint4 kk = *reinterpret_cast<const uint4*>(k + d);
                uint4 vv = *reinterpret_cast<const uint4*>(v + d);
                const __half2* kh = reinterpret_cast<const __half2*>(&kk);
                const __half2* vh = reinterpret_cast<const __half2*>(&vv);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    float2 a = __half22float2(kh[j]), b = __half22float2(vh[j]);
                    ka = fmaxf(ka, fmaxf(fabsf(a.x), fabsf(a.y)));
                    va = fmaxf(va, fmaxf(fabsf(b.x), fabsf(b.y)));
                }
            }
        } else {
            for (int d = lane; d < headDim; d += 32) {
                ka = fmaxf(ka, fabsf(__half2float(k[d])));
                va = fmaxf(va, fabsf(__half2float(v[d])));
            }
        }
        ka = warpMax(ka);
        va = warpMax(va);
        if (lane == 0) {
            const int t = static_cast<int>(row / kvHeads), kvh = static_cast<int>(row % kvHeads);
            const int64_t slot = slotOf(src, t, blockSize);
            if (slot < 0) continue;
            const int64_t blk = slot / blockSize;
            unsigned long long* w = amax + (blk * kvHeads + kvh) * 2;
            const unsigned long long tag = static_cast<unsigned long long>(epoch) << 32;
            atomicMax(w + 0, tag | __float_as_uint(ka));
            atomicMax(w + 1, tag | __float_as_uint(va));
        }
    }
}

// Pass 2 (kernels.metal:1907-1961): group scale from this call's absmax and the
// stored scale, quantise the row with it, store codes and scale.  Warps of one
// group may read the stored scale before or after another warp has replaced
// it; the rule max(absmax, s*448)/448 returns the same half either way, so
// every warp derives the same scale.
__global__ void fp8QuantizeKernel(const __half* __restrict__ keys, const __half* __restrict__ values,
                                  uint8_t* __restrict__ kCodes, uint8_t* __restrict__ vCodes,
                                  __half* kScale, __half* vScale, SlotSource src, int numTokens,
                                  int kvHeads, int blockSize, int headDim,
                                  const unsigned long long* __restrict__ amax) {
    const int lane = threadIdx.x & 31;
    const int64_t rows = static_cast<int64_t>(numTokens) * kvHeads;
    const int64_t warpsTotal = (static_cast<int64_t>(gridDim.x) * blockDim.x) >> 5;
    for (int64_t row = (blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x) >> 5;
         row < rows; row += warpsTotal) {
        const int t = static_cast<int>(row / kvHeads), kvh = static_cast<int>(row % kvHeads);
        const int64_t slot = slotOf(src, t, blockSize);
        if (slot < 0) continue;
        const int64_t blk = slot / blockSize, off = slot % blockSize;
        const int64_t group = blk * kvHeads + kvh;
        float ks, vs;
        {
            const float ka = __uint_as_float(static_cast<uint32_t>(amax[group * 2 + 0]));
            const float va = __uint_as_float(static_cast<uint32_t>(amax[group * 2 + 1]));
            const float km = fmaxf(ka, __half2float(*(volatile __half*)(kScale + group)) * 448.0f);   // :1945-1947
            const float vm = fmaxf(va, __half2float(*(volatile __half*)(vScale + group)) * 448.0f);   // :1949-1951
            const __half kh = km > 0.f ? __float2half_rn(__fdiv_rn(km, 448.0f)) : __float2half_rn(1.0f);  // :1953
            const __half vh = vm > 0.f ? __float2half_rn(__fdiv_rn(vm, 448.0f)) : __float2half_rn(1.0f);  // :1954
            if (lane == 0) { kScale[group] = kh; vScale[group] = vh; }                                  // :1959-1960
            ks = __half2float(kh);
            vs = __half2float(vh);
        }
        const __half* k = keys + row * headDim;
        const __half* v = values + row * headDim;
        uint8_t* kd = kCodes + ((blk * kvHeads + kvh) * blockSize + off) * headDim;
        uint8_t* vd = vCodes + ((blk * kvHeads + kvh) * blockSize + off) * headDim;
        if ((headDim & 7) == 0) {
            for (int d = lane * 8; d < headDim; d += 256) {
                uint4 kk = *reinterpret_cast<const uint4*>(k + d);
                uint4 vv = *reinterpret_cast<const uint4*>(v + d);
                const __half* kh = reinterpret_cast<const __half*>(&kk);
                const __half* vh = reinterpret_cast<const __half*>(&vv);
                uint2 ko = make_uint2(0u, 0u), vo = make_uint2(0u, 0u);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    ko.x |= quantizeE4m3(__half2float(kh[j]), ks) << (8 * j);
                    ko.y |= quantizeE4m3(__half2float(kh[j + 4]), ks) << (8 * j);
                    vo.x |= quantizeE4m3(__half2float(vh[j]), vs) << (8 * j);
                    vo.y |= quantizeE4m3(__half2float(vh[j + 4]), vs) << (8 * j);
                }
                *reinterpret_cast<uint2*>(kd + d) = ko;
                *reinterpret_cast<uint2*>(vd + d) = vo;
            }
        } else {
            for (int d = lane; d < headDim; d += 32) {
                kd[d] = static_cast<uint8_t>(quantizeE4m3(__half2float(k[d]), ks));
                vd[d] = static_cast<uint8_t>(quantizeE4m3(__half2float(v[d]), vs));
            }
        }
    }
}

// ---- FP8, 16-byte pieces ----------------------------------------------------
// The same two passes with one thread per 16-byte piece (8 values) of a (token, kv_head)
// row and 32-bit index arithmetic: every lane of a warp works, consecutive lanes read
// consecutive pieces, and a row of head_dim / 8 = 2^k <= 32 pieces is reduced inside its
// group of lanes.  Used when the row splits that way and the launch has fewer than 2^31
// pieces; results are those of the row-per-warp kernels above, bit for bit.

// quantize_fp8 (kernels.metal:564-601) without the division.  `inv` is the reciprocal of
// the scale, rounded to nearest, times (1 + 2^-20).  The code of a quotient only depends
// on comparisons with thresholds of at most five significant bits (the rounding points of
// the 3-bit mantissa, the sub-normal steps k/512 + 1/1024, 2^-6 and 448).  Value and scale
// are float16 numbers (11 significant bits), so value / scale either equals such a
// threshold or is at least 2^-17 away from it in relative terms: a product that lies
// between value / scale and value / scale * (1 + 2^-19) falls on the same side of every
// threshold as the correctly rounded quotient, and on the threshold's upper side when
// they are equal, which is where round-half-away puts it.
__device__ __forceinline__ uint32_t quantizeE4m3Scaled(float value, float inv) {
    const float q = value * inv;
    const float a = fminf(fabsf(q), 448.0f);                                  // :566
    // exponent and mantissa rounded to 3 bits, half up; a carry moves into the exponent (:580-592)
    const uint32_t normal = min(((__float_as_uint(a) + 0x80000u) >> 20) - 960u, 0x7Eu);   // :585-586, :593-598
    // round(a * 512), at most 7 (:573-578); also yields 0 for a == 0 (:571)
    const uint32_t sub = min(static_cast<uint32_t>(__float2int_rz(fmaf(a, 512.0f, 0.5f))), 7u);
    return (a < 0x1p-6f ? sub : normal) | (q < 0.0f ? 0x80u : 0u);            // :568 (-0.0 is not < 0)
}

__device__ __forceinline__ float absmax8(const uint4& x) {
    // |x| of eight float16 values: clear the sign bits, then compare as float16 pairs
    const uint32_t w[4] = {x.x & 0x7FFF7FFFu, x.y & 0x7FFF7FFFu, x.z & 0x7FFF7FFFu, x.w & 0x7FFF7FFFu};
    __half2 m = __hmax2(__hmax2(*reinterpret_cast<const __half2*>(&w[0]), *reinterpret_cast<const __half2*>(&w[1])),
                        __hmax2(*reinterpret_cast<const __half2*>(&w[2]), *reinterpret_cast<const __half2*>(&w[3])));
    return fmaxf(__low2float(m), __high2float(m));
}

struct PieceIndex {
    uint32_t t, kvh, c;
};
__device__ __forceinline__ PieceIndex pieceIndex(uint32_t i, int pieceShift, uint32_t kvHeads) {
    PieceIndex p;
    const uint32_t row = i >> pieceShift;
    p.c = i & ((1u << pieceShift) - 1u);
    p.t = row / kvHeads;
    p.kvh = row - p.t * kvHeads;
    return p;
}
// block and offset of a slot; block sizes are powers of two in practice
__device__ __forceinline__ void splitSlot(int64_t slot, int blockSize, int64_t& blk, int& off) {
    if ((blockSize & (blockSize - 1)) == 0) {
        blk = slot >> (__ffs(blockSize) - 1);
        off = static_cast<int>(slot & (blockSize - 1));
    } else {
        blk = slot / blockSize;
        off = static_cast<int>(slot - blk * blockSize);
    }
}

__global__ void __launch_bounds__(256)
fp8AbsmaxPiecesKernel(const uint4* __restrict__ keys, const uint4* __restrict__ values, SlotSource src,
                      uint32_t pieces, int pieceShift, int kvHeads, int blockSize,
                      unsigned long long* __restrict__ amax, uint32_t epoch) {
    const uint32_t rowLanes = 1u << pieceShift;
    const uint32_t rounded = (pieces + 31u) & ~31u;               // whole warps stay in the loop for the shuffles
    const uint32_t stride = gridDim.x * blockDim.x;
    const unsigned long long tag = static_cast<unsigned long long>(epoch) << 32;
    // two pieces per thread and trip, a grid apart: four 16-byte loads in flight per thread
    for (uint32_t i0 = blockIdx.x * blockDim.x + threadIdx.x; i0 < rounded; i0 += 2u * stride) {
        const uint32_t idx[2] = {i0, i0 + stride};
        uint4 kk[2], vv[2];
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            kk[u] = vv[u] = make_uint4(0u, 0u, 0u, 0u);
            if (idx[u] < pieces) { kk[u] = keys[idx[u]]; vv[u] = values[idx[u]]; }
        }
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            if (idx[u] >= rounded) continue;                       // the same for the whole warp
            float ka = absmax8(kk[u]), va = absmax8(vv[u]);
            for (uint32_t o = rowLanes >> 1; o > 0; o >>= 1) {
                ka = fmaxf(ka, __shfl_xor_sync(0xFFFFFFFFu, ka, o));
                va = fmaxf(va, __shfl_xor_sync(0xFFFFFFFFu, va, o));
            }
            if (idx[u] < pieces && (idx[u] & (rowLanes - 1u)) == 0u) {
                const PieceIndex p = pieceIndex(idx[u], pieceShift, static_cast<uint32_t>(kvHeads));
                const int64_t slot = slotOf(src, static_cast<int>(p.t), blockSize);
                if (slot >= 0) {
                    int64_t blk;
                    int off;
                    splitSlot(slot, blockSize, blk, off);
                    unsigned long long* w = amax + (blk * kvHeads + p.kvh) * 2;
                    atomicMax(w + 0, tag | __float_as_uint(ka));
                    atomicMax(w + 1, tag | __float_as_uint(va));
                }
            }
        }
    }
}

__global__ void __launch_bounds__(256)
fp8QuantizePiecesKernel(const uint4* __restrict__ keys, const uint4* __restrict__ values,
                        uint8_t* __restrict__ kCodes, uint8_t* __restrict__ vCodes, __half* kScale, __half* vScale,
                        SlotSource src, uint32_t pieces, int pieceShift, int kvHeads, int blockSize,
                        const unsigned long long* __restrict__ amax) {
    const uint32_t stride = gridDim.x * blockDim.x;
    const int headDim = 8 << pieceShift;
    for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < pieces; i += stride) {
        const uint4 kk = keys[i], vv = values[i];
        const PieceIndex p = pieceIndex(i, pieceShift, static_cast<uint32_t>(kvHeads));
        const int64_t slot = slotOf(src, static_cast<int>(p.t), blockSize);
        if (slot < 0) continue;
        int64_t blk;
        int off;
        splitSlot(slot, blockSize, blk, off);
        const int64_t group = blk * kvHeads + p.kvh;
        // the group's scale, derived by every thread of the row (kernels.metal:1942-1960)
        const float ka = __uint_as_float(static_cast<uint32_t>(amax[group * 2 + 0]));
        const float va = __uint_as_float(static_cast<uint32_t>(amax[group * 2 + 1]));
        const float km = fmaxf(ka, __half2float(*(volatile __half*)(kScale + group)) * 448.0f);
        const float vm = fmaxf(va, __half2float(*(volatile __half*)(vScale + group)) * 448.0f);
        const __half kh = km > 0.f ? __float2half_rn(__fdiv_rn(km, 448.0f)) : __float2half_rn(1.0f);
        const __half vh = vm > 0.f ? __float2half_rn(__fdiv_rn(vm, 448.0f)) : __float2half_rn(1.0f);
        if (p.c == 0) { kScale[group] = kh; vScale[group] = vh; }
        const float kInv = __frcp_rn(__half2float(kh)) * 1.00000095367431640625f;
        const float vInv = __frcp_rn(__half2float(vh)) * 1.00000095367431640625f;
        const __half2* k2 = reinterpret_cast<const __half2*>(&kk);
        const __half2* v2 = reinterpret_cast<const __half2*>(&vv);
        uint2 ko = make_uint2(0u, 0u), vo = make_uint2(0u, 0u);
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            const float2 a = __half22float2(k2[j]), b = __half22float2(k2[j + 2]);
            const float2 c = __half22float2(v2[j]), d = __half22float2(v2[j + 2]);
            ko.x |= (quantizeE4m3Scaled(a.x, kInv) | (quantizeE4m3Scaled(a.y, kInv) << 8)) << (16 * j);
            ko.y |= (quantizeE4m3Scaled(b.x, kInv) | (quantizeE4m3Scaled(b.y, kInv) << 8)) << (16 * j);
            vo.x |= (quantizeE4m3Scaled(c.x, vInv) | (quantizeE4m3Scaled(c.y, vInv) << 8)) << (16 * j);
            vo.y |= (quantizeE4m3Scaled(d.x, vInv) | (quantizeE4m3Scaled(d.y, vInv) << 8)) << (16 * j);
        }
        const int64_t dst = ((blk * kvHeads + p.kvh) * blockSize + off) * headDim + static_cast<int64_t>(p.c) * 8;
        *reinterpret_cast<uint2*>(kCodes + dst) = ko;
        *reinterpret_cast<uint2*>(vCodes + dst) = vo;
    }
}

// ---- copy-on-write block copies -------------------------------------------

// grid.x = pair, grid.y = slice of the block; 16-byte vectors, K and V.
__global__ void copyBlocksKernel(uint4* __restrict__ kPool, uint4* __restrict__ vPool,
                                 __half* kScale, __half* vScale, const int32_t* __restrict__ pairs,
                                 int64_t blockVecs, int kvHeads) {
    const int64_t srcBlk = pairs[2 * blockIdx.x], dstBlk = pairs[2 * blockIdx.x + 1];
    const uint4* ks = kPool + srcBlk * blockVecs;
    const uint4* vs = vPool + srcBlk * blockVecs;
    uint4* kd = kPool + dstBlk * blockVecs;
    uint4* vd = vPool + dstBlk * blockVecs;
    for (int64_t i = blockIdx.y * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < blockVecs;
         i += static_cast<int64_t>(gridDim.y) * blockDim.x) {
        kd[i] = ks[i];
        vd[i] = vs[i];
    }
    if (kScale && blockIdx.y == 0 && threadIdx.x < kvHeads) {
        kScale[dstBlk * kvHeads + threadIdx.x] = kScale[srcBlk * kvHeads + threadIdx.x];
        vScale[dstBlk * kvHeads + threadIdx.x] = vScale[srcBlk * kvHeads + threadIdx.x];
    }
}

template <typename Vec>
cudaError_t launchScatter(const void* keys, const void* values, void* kPool, void* vPool,
                          SlotSource src, int T, int kvHeads, int blockSize, int rowBytes,
                          cudaStream_t stream) {
    const int rowVecs = rowBytes / static_cast<int>(sizeof(Vec));
    const int64_t total = static_cast<int64_t>(T) * kvHeads * rowVecs;
    const int threads = 256;
    int64_t blocks = (total + threads - 1) / threads;
    if (blocks > 148 * 32) blocks = 148 * 32;                      // grid-stride beyond 32 CTAs per SM
    reshapeAndCacheKernel<Vec><<<static_cast<unsigned>(blocks), threads, 0, stream>>>(
        static_cast<const Vec*>(keys), static_cast<const Vec*>(values), static_cast<Vec*>(kPool),
        static_cast<Vec*>(vPool), src, T, kvHeads, blockSize, rowVecs);
    return cudaGetLastError();
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

}  // namespace

cudaError_t launchReshapeAndCache(const void* keys, const void* values, void* kPool, void* vPool,
                                  SlotSource src, int numTokens, int kvHeads, int blockSize,
                                  int headDim, int elemBytes, cudaStream_t stream, int* launches) {
    if (numTokens <= 0) return cudaSuccess;
    const int rowBytes = headDim * elemBytes;
    if (launches) *launches += 1;
    if (rowBytes % 16 == 0 && aligned16(keys) && aligned16(values) && aligned16(kPool) && aligned16(vPool))
        return launchScatter<uint4>(keys, values, kPool, vPool, src, numTokens, kvHeads, blockSize, rowBytes, stream);
    if (elemBytes == 4)
        return launchScatter<uint32_t>(keys, values, kPool, vPool, src, numTokens, kvHeads, blockSize, rowBytes, stream);
    if (elemBytes == 2)
        return launchScatter<uint16_t>(keys, values, kPool, vPool, src, numTokens, kvHeads, blockSize, rowBytes, stream);
    return launchScatter<uint8_t>(keys, values, kPool, vPool, src, numTokens, kvHeads, blockSize, rowBytes, stream);
}

cudaError_t launchReshapeAndCacheFp8(const void* keysF16, const void* valuesF16, void* kCodes,
                                     void* vCodes, void* kScale, void* vScale, SlotSource src,
                                     int numTokens, int kvHeads, int blockSize, int headDim,
                                     unsigned long long* amaxScratch, uint32_t epoch,
                                     cudaStream_t stream, int* launches) {
    if (numTokens <= 0) return cudaSuccess;
    const int64_t rows = static_cast<int64_t>(numTokens) * kvHeads;
    const int threads = 256;                                       // 8 rows per CTA
    int64_t blocks = (rows + 7) / 8;
    if (blocks > 148 * 16) blocks = 148 * 16;
    // The kernels take the 16-byte path whenever headDim % 8 == 0; it needs
    // 16-byte aligned inputs and 8-byte aligned code pools.
    if (headDim % 8 == 0 &&
        (!aligned16(keysF16) || !aligned16(valuesF16) ||
         ((reinterpret_cast<uintptr_t>(kCodes) | reinterpret_cast<uintptr_t>(vCodes)) & 7u) != 0))
        return cudaErrorMisalignedAddress;
    const int rowPieces = headDim / 8;
    const int64_t pieces = rows * rowPieces;
    if (headDim % 8 == 0 && rowPieces <= 32 && (rowPieces & (rowPieces - 1)) == 0 && pieces < (int64_t(1) << 31)) {
        int pieceShift = 0;
        while ((1 << pieceShift) < rowPieces) ++pieceShift;
        int64_t grid = (pieces + threads - 1) / threads;
        if (grid > 148 * 32) grid = 148 * 32;                      // grid-stride beyond four waves of eight CTAs per SM
        fp8AbsmaxPiecesKernel<<<static_cast<unsigned>(grid), threads, 0, stream>>>(
            static_cast<const uint4*>(keysF16), static_cast<const uint4*>(valuesF16), src, static_cast<uint32_t>(pieces),
            pieceShift, kvHeads, blockSize, amaxScratch, epoch);
        cudaError_t pe = cudaGetLastError();
        if (pe != cudaSuccess) return pe;
        if (launches) *launches += 1;
        fp8QuantizePiecesKernel<<<static_cast<unsigned>(grid), threads, 0, stream>>>(
            static_cast<const uint4*>(keysF16), static_cast<const uint4*>(valuesF16), static_cast<uint8_t*>(kCodes),
            static_cast<uint8_t*>(vCodes), static_cast<__half*>(kScale), static_cast<__half*>(vScale), src,
            static_cast<uint32_t>(pieces), pieceShift, kvHeads, blockSize, amaxScratch);
        if (launches) *launches += 1;
        return cudaGetLastError();
    }
    fp8AbsmaxKernel<<<static_cast<unsigned>(blocks), threads, 0, stream>>>(
        static_cast<const __half*>(keysF16), static_cast<const __half*>(valuesF16), src, numTokens,
        kvHeads, blockSize, headDim, amaxScratch, epoch);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return e;
    if (launches) *launches += 1;
    fp8QuantizeKernel<<<static_cast<unsigned>(blocks), threads, 0, stream>>>(
        static_cast<const __half*>(keysF16), static_cast<const __half*>(valuesF16),
        static_cast<uint8_t*>(kCodes), static_cast<uint8_t*>(vCodes), static_cast<__half*>(kScale),
        static_cast<__half*>(vScale), src, numTokens, kvHeads, blockSize, headDim, amaxScratch);
    if (launches) *launches += 1;
    return cudaGetLastError();
}

cudaError_t launchCopyBlocks(void* kPool, void* vPool, void* kScale, void* vScale,
                             const int32_t* pairs, int n, size_t blockBytes, int kvHeads,
                             cudaStream_t stream, int* launches) {
    if (n <= 0) return cudaSuccess;
    if (blockBytes % 16 != 0 || !aligned16(kPool) || !aligned16(vPool)) return cudaErrorMisalignedAddress;
    const int64_t vecs = static_cast<int64_t>(blockBytes / 16);
    const int threads = 256;
    int slices = static_cast<int>((vecs + threads * 4 - 1) / (threads * 4));   // 4 vectors per thread
    if (slices < 1) slices = 1;
    if (slices > 64) slices = 64;
    dim3 grid(static_cast<unsigned>(n), static_cast<unsigned>(slices));
    copyBlocksKernel<<<grid, threads, 0, stream>>>(static_cast<uint4*>(kPool), static_cast<uint4*>(vPool),
                                                   static_cast<__half*>(kScale), static_cast<__half*>(vScale),
                                                   pairs, vecs, kvHeads);
    if (launches) *launches += 1;
    return cudaGetLastError();
}

// Block-table entries that changed since the device copy was made.
__global__ void patchTablesKernel(int32_t* __restrict__ tables, int stride, const int32_t* __restrict__ patches, int n) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const int row = patches[3 * i], col = patches[3 * i + 1];
    tables[static_cast<int64_t>(row) * stride + col] = patches[3 * i + 2];
}

cudaError_t launchPatchTables(int32_t* tables, int stride, const int32_t* patches, int n, cudaStream_t stream, int* launches) {
    if (n <= 0) return cudaSuccess;
    patchTablesKernel<<<(n + 255) / 256, 256, 0, stream>>>(tables, stride, patches, n);
    if (launches) *launches += 1;
    return cudaGetLastError();
}

}  // namespace pam
