// Chunked causal / sliding-window prefill over paged KV laid out
// [block][kv_head][block_size][head_dim].
//
// Semantics: paged_attention_tiled (kernels.metal:693-765) and the reference's
// chunk loop (PagedAttentionEngine.swift:740-756): row i of a sequence attends
// keys [window_start, S) of its paged cache, key j visible iff j <= i when
// causal; scores are scaled by 1/sqrt(dim), accumulation is float32.  A launch
// covers one chunk of rows [q_start, q_start + q_len) of each of several
// sequences.  Rows that see no key (0/0 in the reference) are written as zeros.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <cmath>

#include "kernels.h"

namespace pam {
namespace {

__device__ __forceinline__ float toFloat(float v) { return v; }
__device__ __forceinline__ float toFloat(__half v) { return __half2float(v); }
__device__ __forceinline__ float toFloat(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T>
__device__ __forceinline__ T fromFloat(float v);
template <>
__device__ __forceinline__ __half fromFloat<__half>(float v) { return __float2half_rn(v); }
template <>
__device__ __forceinline__ __nv_bfloat16 fromFloat<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
template <>
__device__ __forceinline__ float fromFloat<float>(float v) { return v; }

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

// General kernel: one CTA per (16-row tile, head, sequence), 16 keys at a time.
// Works for every storage type, block size and head_dim up to 256; not tuned.
template <typename QT, typename KT>
__global__ void __launch_bounds__(128)
prefillGeneralKernel(const __grid_constant__ PrefillParams p) {
    constexpr int QR = 16, TB = 16, DPT = 2;
    extern __shared__ __align__(16) unsigned char smem[];
    const int tile = blockIdx.x, head = blockIdx.y, seq = blockIdx.z, tid = threadIdx.x;
    const int D = p.headDim, G = p.heads / p.kvHeads, kvh = head / G;
    const int qLen = prefillMeta(p, 2, seq);
    if (tile * QR >= qLen) return;
    const int qStart = prefillMeta(p, 1, seq), seqLen = prefillMeta(p, 0, seq), ws = prefillMeta(p, 4, seq);
    const int64_t rowBase = prefillMeta(p, 3, seq) + tile * QR;
    const int rows = min(QR, qLen - tile * QR);
    const int firstRow = qStart + tile * QR;             // sequence position of local row 0

    float* sq = reinterpret_cast<float*>(smem);          // [QR][D]
    float* sk = sq + QR * D;                             // [TB][D]
    float* sv = sk + TB * D;                             // [TB][D]
    float* ss = sv + TB * D;                             // [QR][TB]
    float* sm = ss + QR * TB;                            // m, l, corr: [3][QR]
    const QT* q = static_cast<const QT*>(p.q);
    const KT* kPool = static_cast<const KT*>(p.kPool);
    const KT* vPool = static_cast<const KT*>(p.vPool);
    const __half* kScale = static_cast<const __half*>(p.kScale);
    const __half* vScale = static_cast<const __half*>(p.vScale);
    QT* out = static_cast<QT*>(p.out);
    const int32_t* table = p.tables + static_cast<int64_t>(seq) * p.maxNumBlocks;
    const float scale = 1.0f / sqrtf(static_cast<float>(D));      // kernels.metal:719

    for (int i = tid; i < rows * D; i += 128) {
        const int r = i / D, d = i - r * D;
        sq[i] = toFloat(q[((rowBase + r) * p.heads + head) * D + d]);
    }
    if (tid < QR) { sm[tid] = -INFINITY; sm[QR + tid] = 0.f; sm[2 * QR + tid] = 0.f; }
    float acc[QR][DPT];
#pragma unroll
    for (int r = 0; r < QR; ++r)
#pragma unroll
        for (int i = 0; i < DPT; ++i) acc[r][i] = 0.f;

    int keyEnd = seqLen;
    if (p.causal) keyEnd = min(keyEnd, firstRow + rows);        // kernels.metal:745
    for (int j0 = ws; j0 < keyEnd; j0 += TB) {
        const int nt = min(TB, keyEnd - j0);
        __syncthreads();
        for (int i = tid; i < nt * D; i += 128) {
            const int t = i / D, d = i - t * D;
            const int tok = j0 + t;
            const int64_t blk = min(max(table[tok / p.blockSize], 0), p.poolBlocks - 1);
            const int64_t off = ((blk * p.kvHeads + kvh) * p.blockSize + tok % p.blockSize) * static_cast<int64_t>(D) + d;
            if constexpr (sizeof(KT) == 1) {
                sk[i] = dequantE4m3(kPool[off], kScale[blk * p.kvHeads + kvh]);
                sv[i] = dequantE4m3(vPool[off], vScale[blk * p.kvHeads + kvh]);
            } else {
                sk[i] = toFloat(kPool[off]);
                sv[i] = toFloat(vPool[off]);
            }
        }
        __syncthreads();
        for (int i = tid; i < rows * nt; i += 128) {
            const int r = i / nt, t = i - r * nt;
            float dot = 0.f;
            for (int d = 0; d < D; ++d) dot += sq[r * D + d] * sk[t * D + d];
            const bool visible = !p.causal || (j0 + t <= firstRow + r);
            ss[r * TB + t] = visible ? dot * scale : -INFINITY;
        }
        __syncthreads();
        if (tid < rows) {
            const int r = tid;
            float m = sm[r], mx = m;
            for (int t = 0; t < nt; ++t) mx = fmaxf(mx, ss[r * TB + t]);
            if (mx == -INFINITY) {
                for (int t = 0; t < nt; ++t) ss[r * TB + t] = 0.f;
                sm[2 * QR + r] = 1.f;
            } else {
                const float corr = expf(m - mx);
                float sum = 0.f;
                for (int t = 0; t < nt; ++t) {
                    const float pr = expf(ss[r * TB + t] - mx);
                    ss[r * TB + t] = pr;
                    sum += pr;
                }
                sm[r] = mx;
                sm[QR + r] = sm[QR + r] * corr + sum;
                sm[2 * QR + r] = corr;
            }
        }
        __syncthreads();
#pragma unroll
        for (int i = 0; i < DPT; ++i) {
            const int d = tid + 128 * i;
            if (d < D) {
#pragma unroll
                for (int r = 0; r < QR; ++r) {
                    if (r < rows) {
                        float a = acc[r][i] * sm[2 * QR + r];
                        for (int t = 0; t < nt; ++t) a += ss[r * TB + t] * sv[t * D + d];
                        acc[r][i] = a;
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
            for (int r = 0; r < QR; ++r) {
                if (r < rows) {
                    const float l = sm[QR + r];
                    out[((rowBase + r) * p.heads + head) * D + d] = fromFloat<QT>(l > 0.f ? acc[r][i] / l : 0.f);
                }
            }
        }
    }
}

template <typename QT, typename KT>
cudaError_t launchGeneral(const PrefillParams& p, cudaStream_t stream, int* launches) {
    const size_t smem = (static_cast<size_t>(16 + 2 * 16) * p.headDim + 16 * 16 + 3 * 16) * sizeof(float);
    auto kernel = prefillGeneralKernel<QT, KT>;
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (e != cudaSuccess) return e;
    dim3 grid(static_cast<unsigned>((p.maxQLen + 15) / 16), static_cast<unsigned>(p.heads),
              static_cast<unsigned>(p.numSeqs));
    kernel<<<grid, 128, smem, stream>>>(p);
    if (launches) *launches += 1;
    return cudaGetLastError();
}

// Two codes (the low two bytes of `c2`) to two float16 values by the reference's chain
// (dequant_fp8, kernels.metal:553-562: every product rounded to half) for normal codes:
// (+-scale) * (1 + m/8), then * 2^(e-7), as two half2 products.  1 + m/8 and 2^(e-7) are
// built from their float16 bit patterns.  `anySpecial` is set when one of the two codes
// has a zero exponent field (zero or sub-normal), for which the caller takes the scalar
// function.
__device__ __forceinline__ uint32_t dequantPairNormal(uint32_t c2, uint32_t scale2, bool& anySpecial) {
    const uint32_t lanes = __byte_perm(c2, 0u, 0x4140);                      // code 0 and code 1, one per 16-bit lane
    const uint32_t e = (lanes >> 3) & 0x000F000Fu;
    anySpecial = (e & 0x0000FFFFu) == 0u || (e >> 16) == 0u;
    const uint32_t onePlus = 0x3C003C00u | ((lanes & 0x00070007u) << 7);     // 1 + m/8
    const uint32_t pow2 = (e + 0x00080008u) << 10;                           // 2^(e-7): exponent field e - 7 + 15
    const uint32_t signedScale = scale2 ^ ((lanes & 0x00800080u) << 8);
    const __half2 t = __hmul2(*reinterpret_cast<const __half2*>(&signedScale), *reinterpret_cast<const __half2*>(&onePlus));
    const __half2 r = __hmul2(t, *reinterpret_cast<const __half2*>(&pow2));
    return *reinterpret_cast<const uint32_t*>(&r);
}

// One CTA per (visible block of a sequence, KV head): codes -> float16, K and V, 16 codes
// per thread and step.
__global__ void __launch_bounds__(256)
fp8StagePagesKernel(const uint8_t* __restrict__ kCodes, const uint8_t* __restrict__ vCodes, const __half* __restrict__ kScale,
                    const __half* __restrict__ vScale, const int32_t* __restrict__ tables, const int32_t* __restrict__ seqLens,
                    const int32_t* __restrict__ windowStarts, __half* __restrict__ kOut, __half* __restrict__ vOut,
                    int32_t* __restrict__ stagedTables, int maxNumBlocks, int maxCount, int kvHeads, int blockSize, int headDim,
                    int poolBlocks) {
    const int seq = blockIdx.y, c = blockIdx.x, kvh = blockIdx.z;
    const int lo = windowStarts[seq] / blockSize, hi = (seqLens[seq] + blockSize - 1) / blockSize;
    const int b = lo + c;
    if (b >= hi || b >= maxNumBlocks) return;
    const int src = min(max(tables[static_cast<int64_t>(seq) * maxNumBlocks + b], 0), poolBlocks - 1);
    const int dst = seq * maxCount + c;
    if (threadIdx.x == 0 && kvh == 0) stagedTables[static_cast<int64_t>(seq) * maxNumBlocks + b] = dst;
    const int perHead = blockSize * headDim;                 // elements of one (block, kv head)
    const int chunks = perHead / 16;
    const __half ksc = kScale[src * kvHeads + kvh], vsc = vScale[src * kvHeads + kvh];
    for (int i = threadIdx.x; i < 2 * chunks; i += blockDim.x) {
        const bool isV = i >= chunks;
        const int ch = isV ? i - chunks : i;
        const int64_t inHead = static_cast<int64_t>(kvh) * perHead + static_cast<int64_t>(ch) * 16;
        const uint4 codes = *reinterpret_cast<const uint4*>((isV ? vCodes : kCodes) + static_cast<int64_t>(src) * kvHeads * perHead + inHead);
        const __half scale = isV ? vsc : ksc;
        const uint32_t scale2 = static_cast<uint32_t>(__half_as_ushort(scale)) * 0x00010001u;
        const uint32_t w[4] = {codes.x, codes.y, codes.z, codes.w};
        uint32_t h[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            const uint32_t c2 = (w[e >> 1] >> (16 * (e & 1))) & 0xFFFFu;
            bool special;
            h[e] = dequantPairNormal(c2, scale2, special);
            if (special) {
                const __half a = __float2half_rn(dequantE4m3(static_cast<uint8_t>(c2 & 0xFFu), scale));   // exact: the value is a half
                const __half bb = __float2half_rn(dequantE4m3(static_cast<uint8_t>(c2 >> 8), scale));
                h[e] = static_cast<uint32_t>(__half_as_ushort(a)) | (static_cast<uint32_t>(__half_as_ushort(bb)) << 16);
            }
        }
        uint4* out = reinterpret_cast<uint4*>((isV ? vOut : kOut) + static_cast<int64_t>(dst) * kvHeads * perHead + inHead);
        out[0] = make_uint4(h[0], h[1], h[2], h[3]);
        out[1] = make_uint4(h[4], h[5], h[6], h[7]);
    }
}

}  // namespace

bool prefillFp8StagingApplies(const PrefillParams& p) {
    if (p.dtype != kFP8 || p.forceGeneral || !p.errFlag || !p.kScale || !p.vScale) return false;
    PrefillParams f = p;
    f.dtype = kF16;
    return prefillTensorPathApplies(f) && (p.blockSize * p.headDim) % 16 == 0;
}

cudaError_t launchFp8StagePages(const PrefillParams& p, const int32_t* seqLens, const int32_t* windowStarts, int maxCount,
                                void* kOut, void* vOut, int32_t* stagedTables, cudaStream_t stream, int* launches) {
    if (maxCount <= 0 || p.numSeqs <= 0) return cudaSuccess;
    dim3 grid(static_cast<unsigned>(maxCount), static_cast<unsigned>(p.numSeqs), static_cast<unsigned>(p.kvHeads));
    fp8StagePagesKernel<<<grid, 256, 0, stream>>>(static_cast<const uint8_t*>(p.kPool), static_cast<const uint8_t*>(p.vPool),
                                                  static_cast<const __half*>(p.kScale), static_cast<const __half*>(p.vScale),
                                                  p.tables, seqLens, windowStarts, static_cast<__half*>(kOut),
                                                  static_cast<__half*>(vOut), stagedTables, p.maxNumBlocks, maxCount, p.kvHeads,
                                                  p.blockSize, p.headDim, p.poolBlocks);
    if (launches) *launches += 1;
    return cudaGetLastError();
}

namespace {
}  // namespace

cudaError_t launchPrefill(const PrefillParams& p, int smCount, cudaStream_t stream, int* launches,
                          bool* usedTensorPath) {
    (void)smCount;
    if (usedTensorPath) *usedTensorPath = false;
    if (p.numSeqs <= 0 || p.maxQLen <= 0) return cudaSuccess;
    if (p.headDim > 256 || p.poolBlocks <= 0) return cudaErrorInvalidValue;
    if (!p.forceGeneral && p.errFlag && prefillTensorPathApplies(p)) {
        if (usedTensorPath) *usedTensorPath = true;
        return launchPrefillTensor(p, p.totalRows, p.errFlag, stream, launches);
    }
    switch (p.dtype) {
        case kF32: return launchGeneral<float, float>(p, stream, launches);
        case kF16: return launchGeneral<__half, __half>(p, stream, launches);
        case kBF16: return launchGeneral<__nv_bfloat16, __nv_bfloat16>(p, stream, launches);
        case kFP8: return launchGeneral<__half, uint8_t>(p, stream, launches);
    }
    return cudaErrorInvalidValue;
}

}  // namespace pam
