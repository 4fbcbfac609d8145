// Batched paged decode for pools laid out [block][kv_head][block_size][head_dim]: the
// dispatch between the two decode kernels, and the general one.
//
// Semantics: paged_decode_single / _f16 / _fp8 (kernels.metal:1417-1620): per
// (sequence, query head) softmax(q.K^T / sqrt(dim)) V over tokens
// [window_start, L) reached through the block table, window_start = L - W when
// W > 0 and L > W (kernels.metal:1442), float32 accumulation.
//
//  * decodeStreamKernel (decode_stream_kernel.cu) -- float16 / bfloat16 / FP8 KV, head_dim
//    64 or 128 (FP8: 128), block_size a multiple of 16, at most 16 query heads per KV head,
//    16-byte aligned pools: one launch for the whole batch, bound by HBM bandwidth.
//
//  * decodeGeneralKernel -- any type (float32, FP8 with the reference's
//    half-precision dequantisation chain, kernels.metal:553-562), any block
//    size, head_dim up to 256.  One CTA per (sequence, kv_head), 16 tokens at a
//    time.  Used where the stream kernel does not apply; not tuned.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <atomic>
#include <cmath>

#include "kernels.h"

namespace pam {
namespace {

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

}  // namespace

bool decodeTakesStreamPath(const DecodeParams& p) { return decodeStreamApplies(p); }

size_t decodeWorkspaceBytes(const DecodeParams& p, int smCount) {
    return decodeStreamApplies(p) ? decodeStreamWorkspaceBytes(p, smCount) : 0;
}

cudaError_t launchDecode(const DecodeParams& p, int smCount, cudaStream_t stream, int* launches) {
    if (p.batch <= 0) return cudaSuccess;
    if (p.headDim > 256 || p.poolBlocks <= 0) return cudaErrorInvalidValue;
    if (decodeStreamApplies(p)) return launchDecodeStream(p, smCount, stream, launches);
    switch (p.dtype) {
        case kF32: return launchGeneral<float, float>(p, stream, launches);
        case kF16: return launchGeneral<__half, __half>(p, stream, launches);
        case kBF16: return launchGeneral<__nv_bfloat16, __nv_bfloat16>(p, stream, launches);
        case kFP8: return launchGeneral<__half, uint8_t>(p, stream, launches);
    }
    return cudaErrorInvalidValue;
}

cudaError_t launchDecodeStatic(const DecodeParams& p, int smCount, cudaStream_t stream, int* launches) {
    // The scratch array and the counting words are part of the library image on every GPU;
    // their device addresses are looked up once per device (decodeStaticScratch).
    DecodeParams q = p;
    float* scratch = nullptr;
    const cudaError_t e = decodeStaticScratch(&scratch, &q.counters, &q.countersCap);
    if (e != cudaSuccess) return e;
    q.workspace = scratch;
    q.workspaceBytes = decodeStaticScratchBytes();
    // (the stream kernel sizes its grid to the scratch it is given; the general kernel needs none)
    return launchDecode(q, smCount, stream, launches);
}

}  // namespace pam
