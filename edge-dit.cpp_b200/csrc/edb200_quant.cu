// ggml block codecs on the device, the one-time weight repack, the small-m
// weight-streaming GEMV and the dense f32 linear used by prelude / final layers.
#include "edb200_internal.h"

#include <cuda_fp16.h>

namespace edb {

// ------------------------------------------------------------------ codecs --

// raw q8_0 block: f16 d, int8 q[32]  (34 bytes, 2-byte aligned)
__global__ void dequant_q8_0_kernel(const uint8_t* __restrict__ blocks, float* __restrict__ out, int64_t n_blocks) {
    const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;  // one thread per weight
    const int64_t b = idx >> 5;
    if (b >= n_blocks) return;
    const int i = idx & 31;
    const uint8_t* p = blocks + b * 34;
    const __half d = *reinterpret_cast<const __half*>(p);
    const int8_t q = static_cast<int8_t>(p[2 + i]);
    out[idx] = __fmul_rn(static_cast<float>(q), __half2float(d));
}

__device__ __forceinline__ void q4k_scale_min(int j, const uint8_t* s, uint32_t& sc, uint32_t& mn) {
    // 12 bytes -> eight 6-bit scales and mins (ggml get_scale_min_k4 packing).
    if (j < 4) {
        sc = s[j] & 63;
        mn = s[j + 4] & 63;
    } else {
        sc = (s[j + 4] & 0x0F) | ((s[j - 4] >> 6) << 4);
        mn = (s[j + 4] >> 4) | ((s[j] >> 6) << 4);
    }
}

// raw q4_K block: f16 d, f16 dmin, u8 scales[12], u8 qs[128]  (144 bytes)
__global__ void dequant_q4_k_kernel(const uint8_t* __restrict__ blocks, float* __restrict__ out, int64_t n_blocks) {
    const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;  // one thread per weight
    const int64_t b = idx >> 8;
    if (b >= n_blocks) return;
    const int i = idx & 255;
    const int sub = i >> 5;   // 0..7
    const int e = i & 31;
    const uint8_t* p = blocks + b * 144;
    const float d = __half2float(*reinterpret_cast<const __half*>(p));
    const float dmin = __half2float(*reinterpret_cast<const __half*>(p + 2));
    uint32_t sc, mn;
    q4k_scale_min(sub, p + 4, sc, mn);
    const uint8_t byte = p[16 + (sub >> 1) * 32 + e];
    const uint32_t q = (sub & 1) ? (byte >> 4) : (byte & 0x0F);
    const float dl = __fmul_rn(d, static_cast<float>(sc));
    const float ml = __fmul_rn(dmin, static_cast<float>(mn));
    out[idx] = __fsub_rn(__fmul_rn(dl, static_cast<float>(q)), ml);
}

// One warp per 32-weight block; follows quantize_row_q8_0_ref: d = amax/127,
// id = d ? 1/d : 0, q = roundf(x*id), d stored as f16.
__global__ void quant_q8_0_kernel(const float* __restrict__ x, uint8_t* __restrict__ blocks, int64_t n_blocks) {
    const int64_t b = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (b >= n_blocks) return;
    const float v = x[b * 32 + lane];
    float amax = fabsf(v);
#pragma unroll
    for (int m = 16; m > 0; m >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, m));
    const float d = __fdiv_rn(amax, 127.0f);
    const float id = d != 0.0f ? __fdiv_rn(1.0f, d) : 0.0f;
    const float q = roundf(__fmul_rn(v, id));
    uint8_t* p = blocks + b * 34;
    if (lane == 0) *reinterpret_cast<__half*>(p) = __float2half_rn(d);
    p[2 + lane] = static_cast<uint8_t>(static_cast<int8_t>(q));
}

__device__ __forceinline__ uint64_t splitmix64(uint64_t x) {
    x += 0x9E3779B97F4A7C15ull;
    x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
    x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
    return x ^ (x >> 31);
}

__global__ void fill_normal_kernel(float* __restrict__ out, int64_t n, uint64_t seed, float mean, float std) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;  // one pair per thread
    if (2 * i >= n) return;
    const uint64_t h = splitmix64(seed ^ splitmix64(static_cast<uint64_t>(i)));
    const float u1 = (static_cast<float>(h >> 40) + 1.0f) * (1.0f / 16777217.0f);  // (0,1)
    const float u2 = static_cast<float>((h >> 8) & 0xFFFFFFu) * (1.0f / 16777216.0f);
    const float r = sqrtf(-2.0f * logf(u1));
    float s, c;
    sincospif(2.0f * u2, &s, &c);
    out[2 * i] = mean + std * r * c;
    if (2 * i + 1 < n) out[2 * i + 1] = mean + std * r * s;
}

// ------------------------------------------------------------------ repack --

// q8_0: one thread per block -> int8 plane [n][k] and f16 scale plane [k/32][n_pad].
__global__ void repack_q8_0_kernel(const uint8_t* __restrict__ blocks, int8_t* __restrict__ qs,
                                   __half* __restrict__ sa, int64_t n_out, int64_t kb, int64_t n_pad) {
    const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= n_out * kb) return;
    const int64_t n = idx / kb;
    const int64_t b = idx % kb;
    const uint16_t* p = reinterpret_cast<const uint16_t*>(blocks + idx * 34);
    uint16_t w[17];
#pragma unroll
    for (int i = 0; i < 17; ++i) w[i] = p[i];
    sa[b * n_pad + n] = *reinterpret_cast<const __half*>(&w[0]);
    uint32_t o[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) o[i] = static_cast<uint32_t>(w[1 + 2 * i]) | (static_cast<uint32_t>(w[2 + 2 * i]) << 16);
    uint4* dst = reinterpret_cast<uint4*>(qs + (n * kb + b) * 32);
    dst[0] = make_uint4(o[0], o[1], o[2], o[3]);
    dst[1] = make_uint4(o[4], o[5], o[6], o[7]);
}

// q4_K: one thread per 256-block -> nibble plane [n][k/2] (ggml's own nibble
// arrangement: byte i of a 32-byte group = weight i | weight 32+i << 4) and the
// per-32 products a = d*sc, b = dmin*m as f16 (GEMM) and f32 (exact dequant).
__global__ void repack_q4_k_kernel(const uint8_t* __restrict__ blocks, uint8_t* __restrict__ qs,
                                   __half* __restrict__ sa, __half* __restrict__ sb, float* __restrict__ sa32,
                                   float* __restrict__ sb32, int64_t n_out, int64_t kb256, int64_t n_pad) {
    const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= n_out * kb256) return;
    const int64_t n = idx / kb256;
    const int64_t b = idx % kb256;
    const uint8_t* p = blocks + idx * 144;
    const float d = __half2float(*reinterpret_cast<const __half*>(p));
    const float dmin = __half2float(*reinterpret_cast<const __half*>(p + 2));
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        uint32_t sc, mn;
        q4k_scale_min(j, p + 4, sc, mn);
        const float a = __fmul_rn(d, static_cast<float>(sc));
        const float m = __fmul_rn(dmin, static_cast<float>(mn));
        const int64_t o = (b * 8 + j) * n_pad + n;
        sa[o] = __float2half_rn(a);
        sb[o] = __float2half_rn(m);
        sa32[o] = a;
        sb32[o] = m;
    }
    const uint4* src = reinterpret_cast<const uint4*>(p + 16);
    uint4* dst = reinterpret_cast<uint4*>(qs + (n * kb256 + b) * 128);
#pragma unroll
    for (int i = 0; i < 8; ++i) dst[i] = src[i];
}

__global__ void qweight_dequant_q8_0_kernel(const int8_t* __restrict__ qs, const __half* __restrict__ sa,
                                            float* __restrict__ out, int64_t n_out, int64_t k, int64_t n_pad) {
    const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= n_out * k) return;
    const int64_t n = idx / k;
    const int64_t kk = idx % k;
    out[idx] = __fmul_rn(static_cast<float>(qs[idx]), __half2float(sa[(kk >> 5) * n_pad + n]));
}

__global__ void qweight_dequant_q4_k_kernel(const uint8_t* __restrict__ qs, const float* __restrict__ sa32,
                                            const float* __restrict__ sb32, float* __restrict__ out, int64_t n_out,
                                            int64_t k, int64_t n_pad) {
    const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= n_out * k) return;
    const int64_t n = idx / k;
    const int64_t kk = idx % k;
    const int64_t g = kk >> 6;          // 64-weight group = 32 bytes
    const int e = kk & 63;
    const uint8_t byte = qs[n * (k >> 1) + g * 32 + (e & 31)];
    const uint32_t q = (e >= 32) ? (byte >> 4) : (byte & 0x0F);
    const int64_t o = (kk >> 5) * n_pad + n;
    out[idx] = __fsub_rn(__fmul_rn(sa32[o], static_cast<float>(q)), sb32[o]);
}

// -------------------------------------------------------------------- GEMV --
// y[mm][n] = sum_k act(x[mm][k]) * W[n][k] + bias[n],  mm < m <= 8.
// CTA = 8 warps, 4 consecutive weight rows per warp (32 rows per CTA share the
// scale-plane sectors).  x is staged once per CTA in shared memory as f32.
constexpr int GEMV_ROWS_PER_WARP = 4;
constexpr int GEMV_WARPS = 8;
constexpr int GEMV_MAX_M = 8;

template <int WT, int M>
__global__ void __launch_bounds__(GEMV_WARPS * 32)
gemv_q_kernel(const uint8_t* __restrict__ qs, const __half* __restrict__ sa, const __half* __restrict__ sb,
              const float* __restrict__ x, int64_t ldx, int pre_silu, const float* __restrict__ bias,
              float* __restrict__ y, int64_t ldy, int n_out, int k, int64_t n_pad) {
    extern __shared__ float xs[];  // [M][k]
    for (int i = threadIdx.x; i < M * k; i += blockDim.x) {
        const int mm = i / k, kk = i % k;
        float v = x[(int64_t)mm * ldx + kk];
        if (pre_silu) v = v / (1.0f + __expf(-v));
        xs[i] = v;
    }
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n0 = (blockIdx.x * GEMV_WARPS + warp) * GEMV_ROWS_PER_WARP;
    float acc[GEMV_ROWS_PER_WARP][M];
#pragma unroll
    for (int r = 0; r < GEMV_ROWS_PER_WARP; ++r)
#pragma unroll
        for (int mm = 0; mm < M; ++mm) acc[r][mm] = 0.0f;

    if (WT == EDB200_TYPE_Q8_0) {
        // lane handles 16 consecutive k per step: half a 32-block.
        for (int k0 = lane * 16; k0 < k; k0 += 32 * 16) {
            uint4 raw[GEMV_ROWS_PER_WARP];
            float d[GEMV_ROWS_PER_WARP];
#pragma unroll
            for (int r = 0; r < GEMV_ROWS_PER_WARP; ++r) {
                const int n = n0 + r;
                if (n < n_out) {
                    raw[r] = __ldg(reinterpret_cast<const uint4*>(qs + (int64_t)n * k + k0));
                    d[r] = __half2float(sa[(int64_t)(k0 >> 5) * n_pad + n]);
                } else {
                    raw[r] = make_uint4(0, 0, 0, 0);
                    d[r] = 0.0f;
                }
            }
#pragma unroll
            for (int r = 0; r < GEMV_ROWS_PER_WARP; ++r) {
                const uint32_t w[4] = {raw[r].x, raw[r].y, raw[r].z, raw[r].w};
#pragma unroll
                for (int mm = 0; mm < M; ++mm) {
                    const float* xp = xs + mm * k + k0;
                    float part = 0.0f;
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const float4 xv = *reinterpret_cast<const float4*>(xp + 4 * j);
                        // int8 -> f32 without conversion instructions: byte u = q + 128 placed in the
                        // mantissa of 2^23 gives 8388608 + u exactly; subtract 8388736 to get q.
                        const uint32_t u = w[j] ^ 0x80808080u;
                        const float q0 = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7650)) - 8388736.0f;
                        const float q1 = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7651)) - 8388736.0f;
                        const float q2 = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7652)) - 8388736.0f;
                        const float q3 = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7653)) - 8388736.0f;
                        part = fmaf(q0, xv.x, part);
                        part = fmaf(q1, xv.y, part);
                        part = fmaf(q2, xv.z, part);
                        part = fmaf(q3, xv.w, part);
                    }
                    acc[r][mm] += d[r] * part;
                }
            }
        }
    } else {
        // q4_K: lane handles 16 bytes = weights k0..k0+15 (low) and k0+32..k0+47 (high) of a 64-group.
        const int kbytes = k >> 1;
        for (int b0 = lane * 16; b0 < kbytes; b0 += 32 * 16) {
            const int g = b0 >> 5;             // 64-weight group
            const int off = b0 & 31;           // 0 or 16
#pragma unroll
            for (int r = 0; r < GEMV_ROWS_PER_WARP; ++r) {
                const int n = n0 + r;
                if (n >= n_out) continue;
                const uint4 raw = __ldg(reinterpret_cast<const uint4*>(qs + (int64_t)n * kbytes + b0));
                const float a_lo = __half2float(sa[(int64_t)(2 * g) * n_pad + n]);
                const float a_hi = __half2float(sa[(int64_t)(2 * g + 1) * n_pad + n]);
                const float b_lo = __half2float(sb[(int64_t)(2 * g) * n_pad + n]);
                const float b_hi = __half2float(sb[(int64_t)(2 * g + 1) * n_pad + n]);
                const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
                for (int mm = 0; mm < M; ++mm) {
                    const float* xl = xs + mm * k + g * 64 + off;
                    const float* xh = xl + 32;
                    float pl = 0.f, ph = 0.f, sl = 0.f, sh = 0.f;
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const uint32_t byte = (w[j] >> (8 * e)) & 0xFF;
                            const float xlo = xl[4 * j + e], xhi = xh[4 * j + e];
                            pl += static_cast<float>(byte & 0x0F) * xlo;
                            ph += static_cast<float>(byte >> 4) * xhi;
                            sl += xlo;
                            sh += xhi;
                        }
                    }
                    acc[r][mm] += a_lo * pl - b_lo * sl + a_hi * ph - b_hi * sh;
                }
            }
        }
    }
#pragma unroll
    for (int r = 0; r < GEMV_ROWS_PER_WARP; ++r) {
#pragma unroll
        for (int mm = 0; mm < M; ++mm) {
            float v = acc[r][mm];
#pragma unroll
            for (int s = 16; s > 0; s >>= 1) v += __shfl_xor_sync(0xffffffffu, v, s);
            const int n = n0 + r;
            if (lane == 0 && n < n_out) y[(int64_t)mm * ldy + n] = v + (bias ? bias[n] : 0.0f);
        }
    }
}

// ------------------------------------------------------------ dense f32 ----
// Small-m: one warp per output column, float4 streaming of the weight row.
template <int M>
__global__ void __launch_bounds__(256)
gemv_f32_kernel(const float* __restrict__ w, const float* __restrict__ bias, const float* __restrict__ x,
                int64_t ldx, int pre_silu, int act, float* __restrict__ y, int64_t ldy, int n_out, int k) {
    extern __shared__ float xs[];
    for (int i = threadIdx.x; i < M * k; i += blockDim.x) {
        float v = x[(int64_t)(i / k) * ldx + (i % k)];
        if (pre_silu) v = v / (1.0f + __expf(-v));
        xs[i] = v;
    }
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n = blockIdx.x * 8 + warp;
    if (n >= n_out) return;
    float acc[M];
#pragma unroll
    for (int mm = 0; mm < M; ++mm) acc[mm] = 0.0f;
    const float* wr = w + (int64_t)n * k;
    for (int k0 = lane * 4; k0 < k; k0 += 128) {
        const float4 wv = __ldg(reinterpret_cast<const float4*>(wr + k0));
#pragma unroll
        for (int mm = 0; mm < M; ++mm) {
            const float4 xv = *reinterpret_cast<const float4*>(xs + mm * k + k0);
            acc[mm] += wv.x * xv.x + wv.y * xv.y + wv.z * xv.z + wv.w * xv.w;
        }
    }
#pragma unroll
    for (int mm = 0; mm < M; ++mm) {
        float v = acc[mm];
#pragma unroll
        for (int s = 16; s > 0; s >>= 1) v += __shfl_xor_sync(0xffffffffu, v, s);
        if (lane == 0) {
            v += bias ? bias[n] : 0.0f;
            if (act == EDB200_ACT_SILU) v = v / (1.0f + __expf(-v));
            if (act == EDB200_ACT_GELU_TANH) {
                v = 0.5f * v * (1.0f + tanhf(0.7978845608028654f * v * (1.0f + 0.044715f * v * v)));
            }
            y[(int64_t)mm * ldy + n] = v;
        }
    }
}

// Larger m: 64x64 output tile per CTA, 16-wide k slices through shared memory.
__global__ void __launch_bounds__(256)
sgemm_nt_kernel(const float* __restrict__ w, const float* __restrict__ bias, const float* __restrict__ x,
                int64_t ldx, int act, float* __restrict__ y, int64_t ldy, int m, int n_out, int k) {
    __shared__ float xs[16][64 + 1];
    __shared__ float ws[16][64 + 1];
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;  // 16 x 16 threads, 4x4 outputs each
    const int m0 = blockIdx.y * 64, n0 = blockIdx.x * 64;
    float acc[4][4] = {};
    for (int k0 = 0; k0 < k; k0 += 16) {
        for (int i = threadIdx.x; i < 64 * 16; i += 256) {
            const int r = i >> 4, c = i & 15;
            const int mm = m0 + r, nn = n0 + r, kk = k0 + c;
            xs[c][r] = (mm < m && kk < k) ? x[(int64_t)mm * ldx + kk] : 0.0f;
            ws[c][r] = (nn < n_out && kk < k) ? w[(int64_t)nn * k + kk] : 0.0f;
        }
        __syncthreads();
#pragma unroll
        for (int c = 0; c < 16; ++c) {
            float a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                a[i] = xs[c][ty * 4 + i];
                b[i] = ws[c][tx * 4 + i];
            }
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] += a[i] * b[j];
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int mm = m0 + ty * 4 + i;
        if (mm >= m) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int nn = n0 + tx * 4 + j;
            if (nn >= n_out) continue;
            float v = acc[i][j] + (bias ? bias[nn] : 0.0f);
            if (act == EDB200_ACT_SILU) v = v / (1.0f + __expf(-v));
            if (act == EDB200_ACT_GELU_TANH) {
                v = 0.5f * v * (1.0f + tanhf(0.7978845608028654f * v * (1.0f + 0.044715f * v * v)));
            }
            y[(int64_t)mm * ldy + nn] = v;
        }
    }
}

template <int WT>
static edb200_status_t launch_gemv_q(const edb200_qweight_t* w, const float* x, int64_t m, int64_t ldx, int pre_silu,
                                     const float* bias, float* y, int64_t ldy, cudaStream_t stream) {
    const int rows_per_cta = GEMV_ROWS_PER_WARP * GEMV_WARPS;
    const int grid = static_cast<int>((w->n_out + rows_per_cta - 1) / rows_per_cta);
    const size_t smem = static_cast<size_t>(m) * w->k * sizeof(float);
    ProfScope prof(stream, PROF_GEMV, 2.0 * (double)m * (double)w->n_out * (double)w->k, (double)w->bytes);
#define EDB_GEMV_CASE(MM)                                                                                           \
    case MM: {                                                                                                      \
        auto kern = gemv_q_kernel<WT, MM>;                                                                          \
        if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);   \
        kern<<<grid, GEMV_WARPS * 32, smem, stream>>>(static_cast<const uint8_t*>(w->qs),                           \
                                                      static_cast<const __half*>(w->sa),                           \
                                                      static_cast<const __half*>(w->sb), x, ldx, pre_silu, bias, y, \
                                                      ldy, (int)w->n_out, (int)w->k, w->n_pad);                     \
        break;                                                                                                      \
    }
    switch (m) {
        EDB_GEMV_CASE(1)
        EDB_GEMV_CASE(2)
        EDB_GEMV_CASE(3)
        EDB_GEMV_CASE(4)
        EDB_GEMV_CASE(5)
        EDB_GEMV_CASE(6)
        EDB_GEMV_CASE(7)
        EDB_GEMV_CASE(8)
        default:
            return fail(EDB200_ERR_INVALID, "gemv_q: m must be in 1..8");
    }
#undef EDB_GEMV_CASE
    count_launch();
    return check_cuda(cudaGetLastError(), "gemv_q launch");
}

}  // namespace edb

using namespace edb;

extern "C" {

edb200_status_t edb200_dequantize_rows(int ggml_type, const void* blocks, float* out, int64_t rows, int64_t k,
                                       void* stream) {
    if (blocks == nullptr || out == nullptr || rows <= 0 || k <= 0) {
        return fail(EDB200_ERR_INVALID, "dequantize_rows: null or empty argument");
    }
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int64_t total = rows * k;
    const int grid = static_cast<int>((total + 255) / 256);
    if (ggml_type == EDB200_TYPE_Q8_0) {
        if (k % 32) return fail(EDB200_ERR_INVALID, "dequantize_rows: q8_0 needs k %% 32 == 0");
        dequant_q8_0_kernel<<<grid, 256, 0, s>>>(static_cast<const uint8_t*>(blocks), out, total / 32);
    } else if (ggml_type == EDB200_TYPE_Q4_K) {
        if (k % 256) return fail(EDB200_ERR_INVALID, "dequantize_rows: q4_K needs k %% 256 == 0");
        dequant_q4_k_kernel<<<grid, 256, 0, s>>>(static_cast<const uint8_t*>(blocks), out, total / 256);
    } else {
        return fail(EDB200_ERR_UNSUPPORTED, "dequantize_rows: type %d", ggml_type);
    }
    count_launch();
    return check_cuda(cudaGetLastError(), "dequantize_rows launch");
}

edb200_status_t edb200_quantize_rows_q8_0(const float* x, void* blocks, int64_t rows, int64_t k, void* stream) {
    if (x == nullptr || blocks == nullptr || rows <= 0 || k <= 0 || k % 32) {
        return fail(EDB200_ERR_INVALID, "quantize_rows_q8_0: bad argument (k %% 32 == 0 required)");
    }
    const int64_t n_blocks = rows * k / 32;
    const int grid = static_cast<int>((n_blocks * 32 + 255) / 256);
    quant_q8_0_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(x, static_cast<uint8_t*>(blocks), n_blocks);
    count_launch();
    return check_cuda(cudaGetLastError(), "quantize_rows_q8_0 launch");
}

edb200_status_t edb200_fill_normal(float* out, int64_t n, uint64_t seed, float mean, float std, void* stream) {
    if (out == nullptr || n <= 0) return fail(EDB200_ERR_INVALID, "fill_normal: bad argument");
    const int64_t pairs = (n + 1) / 2;
    fill_normal_kernel<<<static_cast<int>((pairs + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        out, n, seed, mean, std);
    count_launch();
    return check_cuda(cudaGetLastError(), "fill_normal launch");
}

edb200_status_t edb200_qweight_create(int ggml_type, const void* blocks, int64_t n_out, int64_t k, void* stream,
                                      edb200_qweight_t** out) {
    if (blocks == nullptr || out == nullptr || n_out <= 0 || k <= 0) {
        return fail(EDB200_ERR_INVALID, "qweight_create: null or empty argument");
    }
    if (ggml_type != EDB200_TYPE_Q8_0 && ggml_type != EDB200_TYPE_Q4_K) {
        return fail(EDB200_ERR_UNSUPPORTED, "qweight_create: type %d", ggml_type);
    }
    const int blk = ggml_type == EDB200_TYPE_Q8_0 ? 32 : 256;
    if (k % blk) return fail(EDB200_ERR_INVALID, "qweight_create: k must be a multiple of %d", blk);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    edb200_qweight_t* w = new (std::nothrow) edb200_qweight_t();
    if (w == nullptr) return fail(EDB200_ERR_NOMEM, "qweight_create: host allocation failed");
    w->ggml_type = ggml_type;
    w->n_out = n_out;
    w->k = k;
    w->n_pad = (n_out + 7) & ~int64_t(7);
    const int64_t kb32 = k / 32;
    const int64_t qs_bytes = ggml_type == EDB200_TYPE_Q8_0 ? n_out * k : n_out * k / 2;
    const int64_t plane = kb32 * w->n_pad;
    cudaError_t e = cudaMalloc(&w->qs, qs_bytes);
    if (e == cudaSuccess) e = cudaMalloc(&w->sa, plane * 2);
    if (e == cudaSuccess && ggml_type == EDB200_TYPE_Q4_K) {
        e = cudaMalloc(&w->sb, plane * 2);
        if (e == cudaSuccess) e = cudaMalloc(reinterpret_cast<void**>(&w->sa32), plane * 4);
        if (e == cudaSuccess) e = cudaMalloc(reinterpret_cast<void**>(&w->sb32), plane * 4);
    }
    if (e != cudaSuccess) {
        edb200_qweight_destroy(w);
        return fail(EDB200_ERR_NOMEM, "qweight_create: cudaMalloc: %s", cudaGetErrorString(e));
    }
    w->bytes = qs_bytes + plane * 2 * (ggml_type == EDB200_TYPE_Q4_K ? 6 : 1);
    cudaMemsetAsync(w->sa, 0, plane * 2, s);
    if (ggml_type == EDB200_TYPE_Q8_0) {
        const int64_t nb = n_out * kb32;
        repack_q8_0_kernel<<<static_cast<int>((nb + 255) / 256), 256, 0, s>>>(
            static_cast<const uint8_t*>(blocks), static_cast<int8_t*>(w->qs), static_cast<__half*>(w->sa), n_out,
            kb32, w->n_pad);
    } else {
        cudaMemsetAsync(w->sb, 0, plane * 2, s);
        const int64_t nb = n_out * (k / 256);
        repack_q4_k_kernel<<<static_cast<int>((nb + 127) / 128), 128, 0, s>>>(
            static_cast<const uint8_t*>(blocks), static_cast<uint8_t*>(w->qs), static_cast<__half*>(w->sa),
            static_cast<__half*>(w->sb), w->sa32, w->sb32, n_out, k / 256, w->n_pad);
    }
    count_launch();
    e = cudaGetLastError();
    if (e == cudaSuccess) e = cudaStreamSynchronize(s);
    if (e != cudaSuccess) {
        edb200_qweight_destroy(w);
        return check_cuda(e, "qweight_create repack");
    }
    edb200_status_t st;
    if (ggml_type == EDB200_TYPE_Q8_0) {
        st = make_tmap_2d(&w->map_qs, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, w->qs, (uint64_t)k, (uint64_t)n_out,
                          (uint64_t)k, 64, 128, CU_TENSOR_MAP_SWIZZLE_NONE);
    } else {
        st = make_tmap_2d(&w->map_qs, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, w->qs, (uint64_t)k / 2, (uint64_t)n_out,
                          (uint64_t)k / 2, 32, 128, CU_TENSOR_MAP_SWIZZLE_NONE);
    }
    if (st == EDB200_OK) {
        st = make_tmap_2d(&w->map_sa, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, w->sa, (uint64_t)w->n_pad, (uint64_t)kb32,
                          (uint64_t)w->n_pad * 2, 128, 2, CU_TENSOR_MAP_SWIZZLE_NONE);
    }
    if (st == EDB200_OK && ggml_type == EDB200_TYPE_Q4_K) {
        st = make_tmap_2d(&w->map_sb, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, w->sb, (uint64_t)w->n_pad, (uint64_t)kb32,
                          (uint64_t)w->n_pad * 2, 128, 2, CU_TENSOR_MAP_SWIZZLE_NONE);
    }
    if (st != EDB200_OK) {
        edb200_qweight_destroy(w);
        return st;
    }
    *out = w;
    return EDB200_OK;
}

void edb200_qweight_destroy(edb200_qweight_t* w) {
    if (w == nullptr) return;
    cudaFree(w->qs);
    cudaFree(w->sa);
    cudaFree(w->sb);
    cudaFree(w->sa32);
    cudaFree(w->sb32);
    delete w;
}

int64_t edb200_qweight_bytes(const edb200_qweight_t* w) { return w ? w->bytes : 0; }

edb200_status_t edb200_qweight_dequantize(const edb200_qweight_t* w, float* out, void* stream) {
    if (w == nullptr || out == nullptr) return fail(EDB200_ERR_INVALID, "qweight_dequantize: null argument");
    const int64_t total = w->n_out * w->k;
    const int grid = static_cast<int>((total + 255) / 256);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (w->ggml_type == EDB200_TYPE_Q8_0) {
        qweight_dequant_q8_0_kernel<<<grid, 256, 0, s>>>(static_cast<const int8_t*>(w->qs),
                                                         static_cast<const __half*>(w->sa), out, w->n_out, w->k,
                                                         w->n_pad);
    } else {
        qweight_dequant_q4_k_kernel<<<grid, 256, 0, s>>>(static_cast<const uint8_t*>(w->qs), w->sa32, w->sb32, out,
                                                         w->n_out, w->k, w->n_pad);
    }
    count_launch();
    return check_cuda(cudaGetLastError(), "qweight_dequantize launch");
}

edb200_status_t edb200_gemv_q(const edb200_qweight_t* w, const float* x, int64_t m, int64_t ldx, int pre_silu,
                              const float* bias, float* y, int64_t ldy, void* stream) {
    if (w == nullptr || x == nullptr || y == nullptr) return fail(EDB200_ERR_INVALID, "gemv_q: null argument");
    if (m < 1 || m > GEMV_MAX_M) return fail(EDB200_ERR_INVALID, "gemv_q: m must be in 1..8");
    if (w->k % 512 != 0 && w->ggml_type == EDB200_TYPE_Q8_0 && w->k % 16 != 0) {
        return fail(EDB200_ERR_UNSUPPORTED, "gemv_q: k must be a multiple of 16");
    }
    if (ldx < w->k || ldy < w->n_out) return fail(EDB200_ERR_INVALID, "gemv_q: leading dimension too small");
    if (static_cast<size_t>(m) * w->k * 4 > 200 * 1024) {
        return fail(EDB200_ERR_UNSUPPORTED, "gemv_q: m*k too large for the shared-memory stage");
    }
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (w->ggml_type == EDB200_TYPE_Q8_0) return launch_gemv_q<EDB200_TYPE_Q8_0>(w, x, m, ldx, pre_silu, bias, y, ldy, s);
    return launch_gemv_q<EDB200_TYPE_Q4_K>(w, x, m, ldx, pre_silu, bias, y, ldy, s);
}

edb200_status_t edb200_linear_f32(const float* w, const float* bias, const float* x, int64_t m, int64_t k, int64_t n,
                                  int64_t ldx, int pre_silu, int act, float* y, int64_t ldy, void* stream) {
    if (w == nullptr || x == nullptr || y == nullptr || m <= 0 || k <= 0 || n <= 0) {
        return fail(EDB200_ERR_INVALID, "linear_f32: null or empty argument");
    }
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    ProfScope prof(s, PROF_OTHER, 2.0 * (double)m * (double)n * (double)k, 4.0 * ((double)n * k + (double)m * (k + n)));
    if (m <= 8 && (k % 4) == 0 && (reinterpret_cast<uintptr_t>(w) & 15u) == 0 && m * k * 4 <= 160 * 1024) {
        const size_t smem = static_cast<size_t>(m) * k * 4;
        const int grid = static_cast<int>((n + 7) / 8);
#define EDB_GEMVF_CASE(MM)                                                                                         \
    case MM: {                                                                                                     \
        auto kern = gemv_f32_kernel<MM>;                                                                           \
        if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);  \
        kern<<<grid, 256, smem, s>>>(w, bias, x, ldx, pre_silu, act, y, ldy, (int)n, (int)k);                      \
        break;                                                                                                     \
    }
        switch (m) {
            EDB_GEMVF_CASE(1)
            EDB_GEMVF_CASE(2)
            EDB_GEMVF_CASE(3)
            EDB_GEMVF_CASE(4)
            EDB_GEMVF_CASE(5)
            EDB_GEMVF_CASE(6)
            EDB_GEMVF_CASE(7)
            EDB_GEMVF_CASE(8)
        }
#undef EDB_GEMVF_CASE
    } else {
        if (pre_silu) return fail(EDB200_ERR_UNSUPPORTED, "linear_f32: pre_silu only for m <= 8");
        dim3 grid(static_cast<unsigned>((n + 63) / 64), static_cast<unsigned>((m + 63) / 64));
        sgemm_nt_kernel<<<grid, 256, 0, s>>>(w, bias, x, ldx, act, y, ldy, (int)m, (int)n, (int)k);
    }
    count_launch();
    return check_cuda(cudaGetLastError(), "linear_f32 launch");
}

}  // extern "C"
