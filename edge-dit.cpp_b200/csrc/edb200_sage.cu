// SageAttention-style INT8 quantisation of Q and K and the driver that runs
// quantisation + the INT8-QK attention kernel out of one caller-provided
// scratch buffer.
//
// Quantiser semantics follow the reference's CUDA kernels bit for bit
// (src/core/backend/ggml/cuda/ed_cuda_sage_attn.cu):
//   channel means   sequential f32 sum in token order, one division   (:209-244)
//   Q               per 32-token tile of (q - qm): amax = max(1e-7, |.|),
//                   scale = amax/127, q8 = rn_even(clamp(v * (1/scale), +-127)) (:61-138)
//   K               the same per 64-token block of (k - km)            (:144-204)
//   smooth-Q bias   bias[j] = sum_d qm[d] * K_orig[j][d], 32-lane xor butterfly
//                   per 32 channels, then sequential over the groups  (:253-281)
#include "edb200_internal.h"

#include <cuda_fp16.h>

#include <cstdint>

namespace edb {
namespace sage {

constexpr int kQTile = 32;
constexpr int kKBlock = 64;

// x [HN, L, D] f16 -> mean [HN, D]; thread per (hn, d), sequential over tokens.
template <int D>
__global__ void __launch_bounds__(D)
channel_mean_kernel(const __half* __restrict__ x, float* __restrict__ mean, int L, int64_t head_rows) {
    const int hn = blockIdx.x;
    const int d = threadIdx.x;
    const __half* p = x + (int64_t)hn * head_rows * D + d;
    float sum = 0.0f;
    int t = 0;
    for (; t + 8 <= L; t += 8) {
        float v[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = __half2float(p[(int64_t)(t + i) * D]);
#pragma unroll
        for (int i = 0; i < 8; ++i) sum = __fadd_rn(sum, v[i]);
    }
    for (; t < L; ++t) sum = __fadd_rn(sum, __half2float(p[(int64_t)t * D]));
    mean[hn * D + d] = __fdiv_rn(sum, static_cast<float>(L));
}

// Fast (not bit-compatible) channel means: the token axis is cut into chunks of
// kMeanChunk rows that are summed in parallel (channel_partial_kernel), then the chunk
// sums are added in chunk order.  Deterministic, but the f32 rounding differs from the
// sequential sum above, so the means can differ in the last bits.  Any vector subtracted
// from K cancels in the softmax, and the smooth-Q bias compensates the Q mean
// exactly, so attention results are unaffected beyond rounding.
constexpr int kMeanChunk = 128;

// One CTA of 128 threads per (head, chunk, q|k).  Thread = (row group g, run of 8 channels): it adds rows
// g, g + G, g + 2G, ... of the chunk (G = 128 / (D / 8) row groups) in that order into one f32 sum per
// channel, with all of its 16-byte loads issued before the first add; the G sums of a channel are then
// added as a pairwise tree ((s0 + s1) + (s2 + s3)) + ... in shared memory.
template <int D>
__global__ void __launch_bounds__(128)
channel_partial_kernel(const __half* __restrict__ q, const __half* __restrict__ k, float* __restrict__ part_q,
                       float* __restrict__ part_k, int L, int n_chunks, int64_t head_rows) {
    constexpr int CG = D / 8;            // channel runs per row
    constexpr int G = 128 / CG;          // row groups
    constexpr int RPT = kMeanChunk / G;  // rows per thread
    __shared__ float sh[G][D];
    const int hn = blockIdx.x, chunk = blockIdx.y;
    const __half* x = blockIdx.z == 0 ? k : q;
    float* part = blockIdx.z == 0 ? part_k : part_q;
    const int g = threadIdx.x / CG, d0 = (threadIdx.x % CG) * 8;
    const int t0 = chunk * kMeanChunk;
    const __half* p = x + ((int64_t)hn * head_rows + t0) * D + d0;
    uint4 raw[RPT];
#pragma unroll
    for (int i = 0; i < RPT; ++i) {
        const int t = g + i * G;
        raw[i] = make_uint4(0u, 0u, 0u, 0u);
        if (t0 + t < L) {
            // volatile: the compiler must not sink the loads to their uses, all of them are to be in flight at once
            asm volatile("ld.global.nc.v4.u32 {%0, %1, %2, %3}, [%4];"
                         : "=r"(raw[i].x), "=r"(raw[i].y), "=r"(raw[i].z), "=r"(raw[i].w)
                         : "l"(p + (int64_t)t * D));
        }
    }
    // every value passes an empty volatile statement placed after the last load: no add can be
    // scheduled between the loads
#pragma unroll
    for (int i = 0; i < RPT; ++i) {
        asm volatile("" : "+r"(raw[i].x), "+r"(raw[i].y), "+r"(raw[i].z), "+r"(raw[i].w));
    }
    float s[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int i = 0; i < RPT; ++i) {
        const uint32_t w[4] = {raw[i].x, raw[i].y, raw[i].z, raw[i].w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[e]));
            s[2 * e] = __fadd_rn(s[2 * e], f.x);
            s[2 * e + 1] = __fadd_rn(s[2 * e + 1], f.y);
        }
    }
#pragma unroll
    for (int e = 0; e < 8; ++e) sh[g][d0 + e] = s[e];
    __syncthreads();
    for (int d = threadIdx.x; d < D; d += 128) {
        float v[G];
#pragma unroll
        for (int i = 0; i < G; ++i) v[i] = sh[i][d];
#pragma unroll
        for (int m = 1; m < G; m <<= 1) {
#pragma unroll
            for (int i = 0; i < G; i += 2 * m) v[i] = __fadd_rn(v[i], v[i + m]);
        }
        part[((int64_t)hn * n_chunks + chunk) * D + d] = v[0];
    }
}

template <int D>
__global__ void __launch_bounds__(D)
channel_finalize_kernel(const float* __restrict__ part_q, const float* __restrict__ part_k, float* __restrict__ qm,
                        float* __restrict__ km, int L, int n_chunks) {
    const int hn = blockIdx.x, d = threadIdx.x;
    const float* part = blockIdx.y == 0 ? part_k : part_q;
    float* mean = blockIdx.y == 0 ? km : qm;
    float s = 0.0f;
    for (int c = 0; c < n_chunks; ++c) s += part[((int64_t)hn * n_chunks + c) * D + d];
    mean[hn * D + d] = s / static_cast<float>(L);
}

// One CTA (128 threads) per (token block, head).  BLK tokens share one scale.  Every thread
// owns runs of 8 consecutive channels (16-byte loads, 8-byte stores); the arithmetic per
// element and the (exact) maximum are those of the reference kernels.
template <int D, int BLK>
__global__ void __launch_bounds__(128)
quant_block_kernel(const __half* __restrict__ x, const float* __restrict__ mean, int8_t* __restrict__ x8,
                   float* __restrict__ scale, int L, int scale_stride, int64_t head_rows) {
    __shared__ float sh[4];
    __shared__ float s_inv;
    const int blk = blockIdx.x, hn = blockIdx.y, tid = threadIdx.x;
    const int tok0 = blk * BLK;
    const __half* xp = x + (int64_t)hn * head_rows * D;
    const float* mrow = mean ? mean + hn * D : nullptr;
    constexpr int VPT = BLK * D / 8 / 128;   // 8-channel vectors per thread
    float vals[VPT][8];
    float amax = 1e-7f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
        const int idx = tid + i * 128;
        const int t = idx / (D / 8), d0 = (idx % (D / 8)) * 8;
        uint4 raw = make_uint4(0u, 0u, 0u, 0u);
        const bool live = tok0 + t < L;
        if (live) raw = *reinterpret_cast<const uint4*>(xp + (int64_t)(tok0 + t) * D + d0);
        const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
        float m8[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        if (mrow != nullptr) {
            const float4 m0 = __ldg(reinterpret_cast<const float4*>(mrow + d0));
            const float4 m1 = __ldg(reinterpret_cast<const float4*>(mrow + d0 + 4));
            m8[0] = m0.x, m8[1] = m0.y, m8[2] = m0.z, m8[3] = m0.w;
            m8[4] = m1.x, m8[5] = m1.y, m8[6] = m1.z, m8[7] = m1.w;
        }
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[e]));
            float v0 = f.x, v1 = f.y;
            if (mrow != nullptr) {
                v0 = __fsub_rn(v0, m8[2 * e]);
                v1 = __fsub_rn(v1, m8[2 * e + 1]);
            }
            if (!live) v0 = v1 = 0.0f;
            vals[i][2 * e] = v0;
            vals[i][2 * e + 1] = v1;
            amax = fmaxf(amax, fmaxf(fabsf(v0), fabsf(v1)));
        }
    }
#pragma unroll
    for (int m = 16; m > 0; m >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, m));
    if ((tid & 31) == 0) sh[tid >> 5] = amax;
    __syncthreads();
    if (tid == 0) {
        const float a = fmaxf(fmaxf(sh[0], sh[1]), fmaxf(sh[2], sh[3]));
        const float sc = __fdiv_rn(a, 127.0f);
        scale[(int64_t)hn * scale_stride + blk] = sc;
        s_inv = __fdiv_rn(1.0f, sc);
    }
    __syncthreads();
    const float inv = s_inv;
    int8_t* op = x8 + (int64_t)hn * L * D;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
        const int idx = tid + i * 128;
        const int t = idx / (D / 8), d0 = (idx % (D / 8)) * 8;
        if (tok0 + t < L) {
            uint32_t packed[2] = {0u, 0u};
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                float v = __fmul_rn(vals[i][e], inv);
                v = fmaxf(fminf(v, 127.0f), -127.0f);
                packed[e >> 2] |= (static_cast<uint32_t>(__float2int_rn(v)) & 0xffu) << (8 * (e & 3));
            }
            *reinterpret_cast<uint2*>(op + (int64_t)(tok0 + t) * D + d0) = make_uint2(packed[0], packed[1]);
        }
    }
}

// One thread per (key, head): bias = sum_d qm[d] * k[d], added in the order of the
// reference's warp kernel (per 32 channels the xor-butterfly tree 16, 8, 4, 2, 1 over
// the lanes, then the four group sums one after the other), so the result is bit-identical
// without any shuffle.
template <int D>
__global__ void __launch_bounds__(256)
smooth_q_bias_kernel(const __half* __restrict__ k, const float* __restrict__ qm, float* __restrict__ bias, int L,
                     int HN, int bias_stride, int64_t head_rows) {
    __shared__ float q_sh[D];
    const int hn = blockIdx.y;
    for (int i = threadIdx.x; i < D; i += blockDim.x) q_sh[i] = qm[hn * D + i];
    __syncthreads();
    const int tok = blockIdx.x * blockDim.x + threadIdx.x;
    if (tok >= L) return;
    const uint4* kp = reinterpret_cast<const uint4*>(k + ((int64_t)hn * head_rows + tok) * D);
    float total = 0.0f;
#pragma unroll
    for (int w = 0; w < D / 32; ++w) {
        float p[32];
#pragma unroll
        for (int v = 0; v < 4; ++v) {
            const uint4 raw = kp[w * 4 + v];
            const uint32_t u[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&u[e]));
                p[v * 8 + 2 * e] = __fmul_rn(f.x, q_sh[w * 32 + v * 8 + 2 * e]);
                p[v * 8 + 2 * e + 1] = __fmul_rn(f.y, q_sh[w * 32 + v * 8 + 2 * e + 1]);
            }
        }
#pragma unroll
        for (int m = 16; m > 0; m >>= 1) {
#pragma unroll
            for (int i = 0; i < m; ++i) p[i] = __fadd_rn(p[i], p[i + m]);
        }
        total = __fadd_rn(total, p[0]);
    }
    bias[(int64_t)hn * bias_stride + tok] = total;
}

constexpr int kFusedQuantThreads = 256;
#ifndef FQ_MIN_BLOCKS
#define FQ_MIN_BLOCKS 4
#endif

// Fast pre-pass, one launch for everything after the channel means: CTA (256 threads) per
// (64-token block, head) quantises the K block (one scale) and the two 32-token Q tiles of the same
// rows (one scale each) with the arithmetic of quant_block_kernel, and, with smooth-Q, produces the
// bias of its 64 keys from the K values it already holds.  The bias sum runs in a fixed order of its
// own (not the reference kernel's): per thread the 8 products of its channels as
// ((p0+p1)+(p2+p3))+((p4+p5)+(p6+p7)), then a pairwise tree over the D/8 threads of the token
// (xor-shuffles 1, 2, 4[, 8]).  Rows between l and the padded end of a bias row are set to zero.
template <int D>
__global__ void __launch_bounds__(kFusedQuantThreads, FQ_MIN_BLOCKS)
fused_quant_kernel(const __half* __restrict__ q, const __half* __restrict__ k, const float* __restrict__ qm,
                   const float* __restrict__ km, int8_t* __restrict__ q8, int8_t* __restrict__ k8,
                   float* __restrict__ q_scale, float* __restrict__ k_scale, float* __restrict__ bias, int L,
                   int q_scale_stride, int k_scale_stride, int bias_stride, int64_t head_rows) {
    constexpr int NT = kFusedQuantThreads, NW = NT / 32;
    __shared__ float sh[2 * NW];
    __shared__ float s_inv[2];
    constexpr int TPT = D / 8;                 // threads per token
    constexpr int VK = 64 * D / 8 / NT;        // 8-channel vectors per thread for 64 tokens
    const int blk = blockIdx.x, hn = blockIdx.y, tid = threadIdx.x;
    const int tok0 = blk * 64;
    const int d0 = (tid % TPT) * 8;
    const __half* kp = k + (int64_t)hn * head_rows * D;
    const __half* qp = q + (int64_t)hn * head_rows * D;
    float km8[8], qm8[8];
    {
        const float4 a = __ldg(reinterpret_cast<const float4*>(km + hn * D + d0));
        const float4 b = __ldg(reinterpret_cast<const float4*>(km + hn * D + d0 + 4));
        km8[0] = a.x, km8[1] = a.y, km8[2] = a.z, km8[3] = a.w, km8[4] = b.x, km8[5] = b.y, km8[6] = b.z, km8[7] = b.w;
    }
    const bool smooth = qm != nullptr;
    if (smooth) {
        const float4 a = __ldg(reinterpret_cast<const float4*>(qm + hn * D + d0));
        const float4 b = __ldg(reinterpret_cast<const float4*>(qm + hn * D + d0 + 4));
        qm8[0] = a.x, qm8[1] = a.y, qm8[2] = a.z, qm8[3] = a.w, qm8[4] = b.x, qm8[5] = b.y, qm8[6] = b.z, qm8[7] = b.w;
    } else {
#pragma unroll
        for (int e = 0; e < 8; ++e) qm8[e] = 0.0f;
    }
    float vals[VK][8];
    // ---- K block: subtract the mean, exact maximum, bias from the unsmoothed values
    float amax = 1e-7f;
#pragma unroll
    for (int i = 0; i < VK; ++i) {
        const int t = (tid + i * NT) / TPT;
        const bool live = tok0 + t < L;
        uint4 raw = make_uint4(0u, 0u, 0u, 0u);
        if (live) raw = *reinterpret_cast<const uint4*>(kp + (int64_t)(tok0 + t) * D + d0);
        const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
        float p[8];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[e]));
            p[2 * e] = __fmul_rn(f.x, qm8[2 * e]);
            p[2 * e + 1] = __fmul_rn(f.y, qm8[2 * e + 1]);
            float v0 = __fsub_rn(f.x, km8[2 * e]), v1 = __fsub_rn(f.y, km8[2 * e + 1]);
            if (!live) v0 = v1 = 0.0f;
            vals[i][2 * e] = v0;
            vals[i][2 * e + 1] = v1;
            amax = fmaxf(amax, fmaxf(fabsf(v0), fabsf(v1)));
        }
        if (smooth) {
            float b = __fadd_rn(__fadd_rn(__fadd_rn(p[0], p[1]), __fadd_rn(p[2], p[3])),
                                __fadd_rn(__fadd_rn(p[4], p[5]), __fadd_rn(p[6], p[7])));
#pragma unroll
            for (int m = 1; m < TPT; m <<= 1) b = __fadd_rn(b, __shfl_xor_sync(0xffffffffu, b, m));
            if (tid % TPT == 0) bias[(int64_t)hn * bias_stride + tok0 + t] = live ? b : 0.0f;
        }
    }
#pragma unroll
    for (int m = 16; m > 0; m >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, m));
    if ((tid & 31) == 0) sh[tid >> 5] = amax;
    __syncthreads();
    if (tid == 0) {
        float a = sh[0];
#pragma unroll
        for (int w = 1; w < NW; ++w) a = fmaxf(a, sh[w]);
        const float sc = __fdiv_rn(a, 127.0f);
        k_scale[(int64_t)hn * k_scale_stride + blk] = sc;
        s_inv[0] = __fdiv_rn(1.0f, sc);
    }
    __syncthreads();
    {
        const float inv = s_inv[0];
        int8_t* op = k8 + (int64_t)hn * L * D;
#pragma unroll
        for (int i = 0; i < VK; ++i) {
            const int t = (tid + i * NT) / TPT;
            if (tok0 + t < L) {
                uint32_t packed[2] = {0u, 0u};
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    float v = __fmul_rn(vals[i][e], inv);
                    v = fmaxf(fminf(v, 127.0f), -127.0f);
                    packed[e >> 2] |= (static_cast<uint32_t>(__float2int_rn(v)) & 0xffu) << (8 * (e & 3));
                }
                *reinterpret_cast<uint2*>(op + (int64_t)(tok0 + t) * D + d0) = make_uint2(packed[0], packed[1]);
            }
        }
    }
    // ---- Q: the same 64 rows as two 32-token tiles; vectors i < VK/2 belong to tile 0, the rest to tile 1
    float am[2] = {1e-7f, 1e-7f};
#pragma unroll
    for (int i = 0; i < VK; ++i) {
        const int t = (tid + i * NT) / TPT;
        const bool live = tok0 + t < L;
        uint4 raw = make_uint4(0u, 0u, 0u, 0u);
        if (live) raw = *reinterpret_cast<const uint4*>(qp + (int64_t)(tok0 + t) * D + d0);
        const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[e]));
            float v0 = f.x, v1 = f.y;
            if (smooth) {
                v0 = __fsub_rn(v0, qm8[2 * e]);
                v1 = __fsub_rn(v1, qm8[2 * e + 1]);
            }
            if (!live) v0 = v1 = 0.0f;
            vals[i][2 * e] = v0;
            vals[i][2 * e + 1] = v1;
            am[i / (VK / 2)] = fmaxf(am[i / (VK / 2)], fmaxf(fabsf(v0), fabsf(v1)));
        }
    }
#pragma unroll
    for (int m = 16; m > 0; m >>= 1) {
        am[0] = fmaxf(am[0], __shfl_xor_sync(0xffffffffu, am[0], m));
        am[1] = fmaxf(am[1], __shfl_xor_sync(0xffffffffu, am[1], m));
    }
    __syncthreads();   // sh and s_inv of the K part are no longer read
    if ((tid & 31) == 0) {
        sh[tid >> 5] = am[0];
        sh[NW + (tid >> 5)] = am[1];
    }
    __syncthreads();
    if (tid < 2) {
        float a = sh[NW * tid];
#pragma unroll
        for (int w = 1; w < NW; ++w) a = fmaxf(a, sh[NW * tid + w]);
        const float sc = __fdiv_rn(a, 127.0f);
        q_scale[(int64_t)hn * q_scale_stride + 2 * blk + tid] = sc;
        s_inv[tid] = __fdiv_rn(1.0f, sc);
    }
    __syncthreads();
    {
        int8_t* op = q8 + (int64_t)hn * L * D;
#pragma unroll
        for (int i = 0; i < VK; ++i) {
            const int t = (tid + i * NT) / TPT;
            const float inv = s_inv[i / (VK / 2)];
            if (tok0 + t < L) {
                uint32_t packed[2] = {0u, 0u};
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    float v = __fmul_rn(vals[i][e], inv);
                    v = fmaxf(fminf(v, 127.0f), -127.0f);
                    packed[e >> 2] |= (static_cast<uint32_t>(__float2int_rn(v)) & 0xffu) << (8 * (e & 3));
                }
                *reinterpret_cast<uint2*>(op + (int64_t)(tok0 + t) * D + d0) = make_uint2(packed[0], packed[1]);
            }
        }
    }
}

struct Layout {
    int64_t q8, k8, q_scale, k_scale, qm, km, bias, part_q, part_k, total;
    int q_scale_stride, k_scale_stride, bias_stride, n_chunks;
};

static Layout make_layout(int hn, int64_t l, int d) {
    Layout lo;
    const int64_t lpad = (l + 127) / 128 * 128;
    auto align = [](int64_t x) { return (x + 255) & ~int64_t(255); };
    int64_t off = 0;
    lo.q8 = off;
    off = align(off + (int64_t)hn * l * d);
    lo.k8 = off;
    off = align(off + (int64_t)hn * l * d);
    lo.q_scale_stride = static_cast<int>(lpad / kQTile);
    lo.k_scale_stride = static_cast<int>(lpad / kKBlock);
    lo.bias_stride = static_cast<int>(lpad);
    lo.q_scale = off;
    off = align(off + (int64_t)hn * lo.q_scale_stride * 4);
    lo.k_scale = off;
    off = align(off + (int64_t)hn * lo.k_scale_stride * 4);
    lo.qm = off;
    off = align(off + (int64_t)hn * d * 4);
    lo.km = off;
    off = align(off + (int64_t)hn * d * 4);
    lo.bias = off;
    off = align(off + (int64_t)hn * lo.bias_stride * 4);
    lo.n_chunks = static_cast<int>(lpad / kMeanChunk);
    lo.part_q = off;
    off = align(off + (int64_t)hn * lo.n_chunks * d * 4);
    lo.part_k = off;
    off = align(off + (int64_t)hn * lo.n_chunks * d * 4);
    lo.total = off;
    return lo;
}

}  // namespace sage

// Where the pieces of the quantised operands live: one caller buffer cut up by make_layout, or the
// separate buffers of the reference's plugin interface (ed_cuda_sage_attn_scratch).
SagePtrs sage_ptrs_from_scratch(void* scratch, int hn, int64_t l, int d) {
    const sage::Layout lo = sage::make_layout(hn, l, d);
    char* sc = static_cast<char*>(scratch);
    SagePtrs p;
    p.q8 = reinterpret_cast<int8_t*>(sc + lo.q8);
    p.k8 = reinterpret_cast<int8_t*>(sc + lo.k8);
    p.q_scale = reinterpret_cast<float*>(sc + lo.q_scale);
    p.k_scale = reinterpret_cast<float*>(sc + lo.k_scale);
    p.qm = reinterpret_cast<float*>(sc + lo.qm);
    p.km = reinterpret_cast<float*>(sc + lo.km);
    p.bias = reinterpret_cast<float*>(sc + lo.bias);
    p.part_q = reinterpret_cast<float*>(sc + lo.part_q);
    p.part_k = reinterpret_cast<float*>(sc + lo.part_k);
    p.q_scale_stride = lo.q_scale_stride;
    p.k_scale_stride = lo.k_scale_stride;
    p.bias_stride = lo.bias_stride;
    return p;
}

namespace sage {

template <int D>
static edb200_status_t quantize(const __half* q, const __half* k, int hn, int l, int64_t head_rows, bool smooth_q,
                                bool fast_means, const SagePtrs& sp, cudaStream_t s) {
    float* qm = sp.qm;
    float* km = sp.km;
    // algorithmic traffic: read q,k (f16) for the means, again for the quantisers (the bit-compatible path reads k
    // once more for the bias); write int8
    ProfScope prof(s, PROF_ELEMENTWISE, 0.0, (double)hn * l * D * (fast_means ? 10.0 : (smooth_q ? 13.0 : 8.0)));
    int launches = 0;
    if (fast_means) {
        const int nc = (l + kMeanChunk - 1) / kMeanChunk;
        channel_partial_kernel<D><<<dim3(hn, nc, smooth_q ? 2 : 1), 128, 0, s>>>(q, k, sp.part_q, sp.part_k, l, nc, head_rows);
        channel_finalize_kernel<D><<<dim3(hn, smooth_q ? 2 : 1), D, 0, s>>>(sp.part_q, sp.part_k, qm, km, l, nc);
        launches += 2;
    } else {
        channel_mean_kernel<D><<<hn, D, 0, s>>>(k, km, l, head_rows);
        if (smooth_q) channel_mean_kernel<D><<<hn, D, 0, s>>>(q, qm, l, head_rows);
        launches += 1 + (smooth_q ? 1 : 0);
    }
    const int lpad = (l + 127) / 128 * 128;
    if (fast_means) {
        // the fast pre-pass: everything after the means in one launch (K and Q read once more, no memset)
        fused_quant_kernel<D><<<dim3(lpad / kKBlock, hn), kFusedQuantThreads, 0, s>>>(q, k, smooth_q ? qm : nullptr, km, sp.q8, sp.k8,
                                                                       sp.q_scale, sp.k_scale, sp.bias, l,
                                                                       sp.q_scale_stride, sp.k_scale_stride,
                                                                       sp.bias_stride, head_rows);
        ++launches;
    } else {
        quant_block_kernel<D, kQTile><<<dim3(lpad / kQTile, hn), 128, 0, s>>>(q, smooth_q ? qm : nullptr, sp.q8, sp.q_scale,
                                                                              l, sp.q_scale_stride, head_rows);
        quant_block_kernel<D, kKBlock><<<dim3(lpad / kKBlock, hn), 128, 0, s>>>(k, km, sp.k8, sp.k_scale, l,
                                                                                sp.k_scale_stride, head_rows);
        launches += 2;
        if (smooth_q) {
            // the padded tail of each bias row is read by the attention kernel: keep it finite
            cudaMemsetAsync(sp.bias, 0, (size_t)hn * sp.bias_stride * 4, s);
            smooth_q_bias_kernel<D><<<dim3((l + 255) / 256, hn), 256, 0, s>>>(k, qm, sp.bias, l, hn, sp.bias_stride,
                                                                               head_rows);
            ++launches;
        }
    }
    count_launch(launches);
    return check_cuda(cudaGetLastError(), "sage quantize launch");
}

}  // namespace sage

// Quantise + attend on separately placed buffers (shared by the scratch-buffer entry points and the
// plugin entry point).
edb200_status_t sage_run(const void* q_f16, const void* k_f16, const void* v_f16, int hn, int64_t l, int64_t head_rows,
                         int64_t v_head_rows, int d_head, float scale, int smooth_q, const SagePtrs& sp, void* out,
                         int out_dtype, int64_t ld_out, const edb200_sp_peers_t* dst, void* stream, bool attend) {
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    edb200_status_t st;
    if (d_head == 128) {
        st = sage::quantize<128>(static_cast<const __half*>(q_f16), static_cast<const __half*>(k_f16), hn,
                                 static_cast<int>(l), head_rows, (smooth_q & 1) != 0, (smooth_q & 2) != 0, sp, s);
    } else {
        st = sage::quantize<64>(static_cast<const __half*>(q_f16), static_cast<const __half*>(k_f16), hn,
                                static_cast<int>(l), head_rows, (smooth_q & 1) != 0, (smooth_q & 2) != 0, sp, s);
    }
    if (st != EDB200_OK || !attend) return st;
    return edb200_attention_sage_int8_strided(sp.q8, sp.k8, v_f16, v_head_rows, sp.q_scale, sp.q_scale_stride, sp.k_scale,
                                              sp.k_scale_stride, (smooth_q & 1) ? sp.bias : nullptr, sp.bias_stride, hn, l,
                                              d_head, scale, out, out_dtype, ld_out, dst, stream);
}

namespace sage {

// ---------------------------------------------------------------------------
// Key-mean entry point without any caller- or library-side allocation: the chunk
// sums of the fast channel mean live in this fixed device array.  Every partial
// sum that the finalize pass reads is written by the partial pass of the same
// call, so nothing in the array has to start at zero.
constexpr int64_t kStaticScratchBytes = 1 << 20;   // 1 MiB = 2048 chunk rows of 128 floats
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

constexpr int kMaxDevices = 64;
static float* g_static_scratch_ptr[kMaxDevices];   // resolved once per device

static edb200_status_t static_scratch(float** out) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return check_cuda(e, "cudaGetDevice");
    if (dev < 0 || dev >= kMaxDevices) return fail(EDB200_ERR_UNSUPPORTED, "static scratch: device ordinal %d", dev);
    if (g_static_scratch_ptr[dev] == nullptr) {
        void* ptr = nullptr;
        e = cudaGetSymbolAddress(&ptr, g_static_scratch);
        if (e != cudaSuccess) return check_cuda(e, "cudaGetSymbolAddress(static scratch)");
        if (ptr == nullptr) return fail(EDB200_ERR_CUDA, "static scratch: null device address");
        g_static_scratch_ptr[dev] = static_cast<float*>(ptr);
    }
    *out = g_static_scratch_ptr[dev];
    return EDB200_OK;
}

template <int D>
static edb200_status_t key_means_static(const __half* k, int hn, int l, float* part, float* mean_out, cudaStream_t s) {
    const int nc = (l + kMeanChunk - 1) / kMeanChunk;
    ProfScope prof(s, PROF_ELEMENTWISE, 0.0, (double)hn * l * D * 2.0);
    channel_partial_kernel<D><<<dim3(hn, nc, 1), 128, 0, s>>>(nullptr, k, nullptr, part, l, nc, l);
    channel_finalize_kernel<D><<<dim3(hn, 1), D, 0, s>>>(nullptr, part, nullptr, mean_out, l, nc);
    count_launch(2);
    return check_cuda(cudaGetLastError(), "sage key means launch");
}

}  // namespace sage
}  // namespace edb

using namespace edb;

extern "C" {

int64_t edb200_sage_scratch_bytes(int hn, int64_t l, int d_head) {
    if (hn <= 0 || l <= 0 || d_head <= 0) return 0;
    return sage::make_layout(hn, l, d_head).total;
}

edb200_status_t edb200_sage_scratch_layout(int hn, int64_t l, int d_head, int64_t* offsets, int* strides) {
    if (offsets == nullptr || strides == nullptr || hn <= 0 || l <= 0 || d_head <= 0) {
        return fail(EDB200_ERR_INVALID, "sage_scratch_layout: bad argument");
    }
    const sage::Layout lo = sage::make_layout(hn, l, d_head);
    offsets[0] = lo.q8;
    offsets[1] = lo.k8;
    offsets[2] = lo.q_scale;
    offsets[3] = lo.k_scale;
    offsets[4] = lo.qm;
    offsets[5] = lo.km;
    offsets[6] = lo.bias;
    offsets[7] = lo.total;
    strides[0] = lo.q_scale_stride;
    strides[1] = lo.k_scale_stride;
    strides[2] = lo.bias_stride;
    return EDB200_OK;
}

edb200_status_t edb200_sage_quantize_qk(const void* q_f16, const void* k_f16, int hn, int64_t l, int d_head,
                                        int smooth_q, void* scratch, int64_t scratch_bytes, void* stream) {
    return edb200_sage_quantize_qk_strided(q_f16, k_f16, hn, l, l, d_head, smooth_q, scratch, scratch_bytes, stream);
}

edb200_status_t edb200_sage_quantize_qk_strided(const void* q_f16, const void* k_f16, int hn, int64_t l,
                                                int64_t head_rows, int d_head, int smooth_q, void* scratch,
                                                int64_t scratch_bytes, void* stream) {
    if (q_f16 == nullptr || k_f16 == nullptr || scratch == nullptr || hn <= 0 || l <= 0 || head_rows < l) {
        return fail(EDB200_ERR_INVALID, "sage_quantize_qk: null or empty argument");
    }
    if (d_head != 64 && d_head != 128) return fail(EDB200_ERR_UNSUPPORTED, "sage_quantize_qk: d_head must be 64 or 128");
    const sage::Layout lo = sage::make_layout(hn, l, d_head);
    if (scratch_bytes < lo.total || (reinterpret_cast<uintptr_t>(scratch) & 255u)) {
        return fail(EDB200_ERR_INVALID, "sage_quantize_qk: scratch must be 256-byte aligned and hold %lld bytes",
                    (long long)lo.total);
    }
    return sage_run(q_f16, k_f16, nullptr, hn, l, head_rows, head_rows, d_head, 0.0f, smooth_q,
                    sage_ptrs_from_scratch(scratch, hn, l, d_head), nullptr, 0, 0, nullptr, stream, false);
}

edb200_status_t edb200_sage_attention(const void* q_f16, const void* k_f16, const void* v_f16, int hn, int64_t l,
                                      int d_head, float scale, int smooth_q, void* scratch, int64_t scratch_bytes,
                                      void* out, int out_dtype, int64_t ld_out, void* stream) {
    return edb200_sage_attention_strided(q_f16, k_f16, v_f16, hn, l, l, d_head, scale, smooth_q, scratch, scratch_bytes,
                                         out, out_dtype, ld_out, nullptr, stream);
}

edb200_status_t edb200_sage_attention_sp(const void* q_f16, const void* k_f16, const void* v_f16, int hn, int64_t l,
                                         int d_head, float scale, int smooth_q, void* scratch, int64_t scratch_bytes,
                                         void* out, int out_dtype, int64_t ld_out, const edb200_sp_peers_t* dst,
                                         void* stream) {
    return edb200_sage_attention_strided(q_f16, k_f16, v_f16, hn, l, l, d_head, scale, smooth_q, scratch, scratch_bytes,
                                         out, out_dtype, ld_out, dst, stream);
}

edb200_status_t edb200_sage_attention_strided(const void* q_f16, const void* k_f16, const void* v_f16, int hn, int64_t l,
                                              int64_t head_rows, int d_head, float scale, int smooth_q, void* scratch,
                                              int64_t scratch_bytes, void* out, int out_dtype, int64_t ld_out,
                                              const edb200_sp_peers_t* dst, void* stream) {
    if (v_f16 == nullptr || (out == nullptr && dst == nullptr)) {
        return fail(EDB200_ERR_INVALID, "sage_attention: null argument");
    }
    if (d_head != 128 && d_head != 64) return fail(EDB200_ERR_UNSUPPORTED, "sage_attention: d_head must be 64 or 128");
    if (q_f16 == nullptr || k_f16 == nullptr || scratch == nullptr || hn <= 0 || l <= 0 || head_rows < l) {
        return fail(EDB200_ERR_INVALID, "sage_attention: null or empty argument");
    }
    const sage::Layout lo = sage::make_layout(hn, l, d_head);
    if (scratch_bytes < lo.total || (reinterpret_cast<uintptr_t>(scratch) & 255u)) {
        return fail(EDB200_ERR_INVALID, "sage_attention: scratch must be 256-byte aligned and hold %lld bytes",
                    (long long)lo.total);
    }
    return sage_run(q_f16, k_f16, v_f16, hn, l, head_rows, head_rows, d_head, scale, smooth_q,
                    sage_ptrs_from_scratch(scratch, hn, l, d_head), out, out_dtype, ld_out, dst, stream, true);
}

edb200_status_t edb200_sage_key_means_static(const void* k_f16, int hn, int64_t l, int d_head, float* mean_out,
                                             void* stream) {
    if (k_f16 == nullptr || mean_out == nullptr || hn <= 0 || l <= 0) {
        return fail(EDB200_ERR_INVALID, "sage_key_means_static: null or empty argument");
    }
    if (d_head != 64 && d_head != 128) {
        return fail(EDB200_ERR_UNSUPPORTED, "sage_key_means_static: d_head must be 64 or 128");
    }
    const int64_t nc = (l + sage::kMeanChunk - 1) / sage::kMeanChunk;
    const int64_t need = (int64_t)hn * nc * d_head * 4;
    if (l > INT32_MAX || need > sage::kStaticScratchBytes) {
        return fail(EDB200_ERR_UNSUPPORTED,
                    "sage_key_means_static: hn * ceil(l/128) * d_head * 4 = %lld bytes exceeds the fixed %lld-byte scratch",
                    (long long)need, (long long)sage::kStaticScratchBytes);
    }
    float* part = nullptr;
    edb200_status_t st = sage::static_scratch(&part);
    if (st != EDB200_OK) return st;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (d_head == 128) {
        return sage::key_means_static<128>(static_cast<const __half*>(k_f16), hn, static_cast<int>(l), part, mean_out, s);
    }
    return sage::key_means_static<64>(static_cast<const __half*>(k_f16), hn, static_cast<int>(l), part, mean_out, s);
}

}  // extern "C"
