// ggml block codecs on the device (raw blocks <-> f32), the synthetic-weight
// generator and the dense f32 linear used by prelude / final layers.
#include "edb200_internal.h"
#include "edb200_codec.cuh"

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
            if (act == EDB200_ACT_GELU_ERF) v = 0.5f * v * (1.0f + erff(v * 0.70710678118654752f));
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
            if (act == EDB200_ACT_GELU_ERF) v = 0.5f * v * (1.0f + erff(v * 0.70710678118654752f));
            if (act == EDB200_ACT_GELU_TANH) {
                v = 0.5f * v * (1.0f + tanhf(0.7978845608028654f * v * (1.0f + 0.044715f * v * v)));
            }
            y[(int64_t)mm * ldy + nn] = v;
        }
    }
}


__device__ __forceinline__ float apply_act(float v, int act) {
    if (act == EDB200_ACT_SILU) v = v / (1.0f + __expf(-v));
    if (act == EDB200_ACT_GELU_ERF) v = 0.5f * v * (1.0f + erff(v * 0.70710678118654752f));
    if (act == EDB200_ACT_GELU_TANH) v = 0.5f * v * (1.0f + tanhf(0.7978845608028654f * v * (1.0f + 0.044715f * v * v)));
    return v;
}

// Register-tiled variant for aligned shapes (k % 16 == 0, 16-byte aligned rows): 64 tokens x
// 128 outputs per CTA, 4 x 8 outputs per thread, 16-k slabs double-buffered in shared memory
// with the next slab's global loads in flight during the multiply.  Every output is one
// accumulator summed over k in ascending order, like the simple kernel above.
constexpr int SG_BM = 64, SG_BN = 128, SG_BK = 16;

__global__ void __launch_bounds__(256)
sgemm_nt_tiled_kernel(const float* __restrict__ w, const float* __restrict__ bias, const float* __restrict__ x,
                      int64_t ldx, int act, float* __restrict__ y, int64_t ldy, int m, int n_out, int k) {
    __shared__ __align__(16) float xs[2][SG_BK][SG_BM + 4];
    __shared__ __align__(16) float ws[2][SG_BK][SG_BN + 4];
    const int tid = threadIdx.x;
    const int tx = tid & 15, ty = tid >> 4;
    const int m0 = blockIdx.y * SG_BM, n0 = blockIdx.x * SG_BN;
    const int lr = tid >> 2, lq = (tid & 3) * 4;   // loader: row of the tile, first of its 4 k
    const float4 zero = make_float4(0.f, 0.f, 0.f, 0.f);
    const float* xrow = (m0 + lr < m) ? x + (int64_t)(m0 + lr) * ldx + lq : nullptr;
    const float* wrow0 = (n0 + lr < n_out) ? w + (int64_t)(n0 + lr) * k + lq : nullptr;
    const float* wrow1 = (n0 + 64 + lr < n_out) ? w + (int64_t)(n0 + 64 + lr) * k + lq : nullptr;

    float acc[4][8];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[i][j] = 0.0f;

    float4 gx = xrow ? *reinterpret_cast<const float4*>(xrow) : zero;
    float4 gw0 = wrow0 ? __ldg(reinterpret_cast<const float4*>(wrow0)) : zero;
    float4 gw1 = wrow1 ? __ldg(reinterpret_cast<const float4*>(wrow1)) : zero;
    int buf = 0;
    for (int k0 = 0; k0 < k; k0 += SG_BK) {
        xs[buf][lq + 0][lr] = gx.x;
        xs[buf][lq + 1][lr] = gx.y;
        xs[buf][lq + 2][lr] = gx.z;
        xs[buf][lq + 3][lr] = gx.w;
        ws[buf][lq + 0][lr] = gw0.x;
        ws[buf][lq + 1][lr] = gw0.y;
        ws[buf][lq + 2][lr] = gw0.z;
        ws[buf][lq + 3][lr] = gw0.w;
        ws[buf][lq + 0][64 + lr] = gw1.x;
        ws[buf][lq + 1][64 + lr] = gw1.y;
        ws[buf][lq + 2][64 + lr] = gw1.z;
        ws[buf][lq + 3][64 + lr] = gw1.w;
        __syncthreads();
        if (k0 + SG_BK < k) {
            gx = xrow ? *reinterpret_cast<const float4*>(xrow + k0 + SG_BK) : zero;
            gw0 = wrow0 ? __ldg(reinterpret_cast<const float4*>(wrow0 + k0 + SG_BK)) : zero;
            gw1 = wrow1 ? __ldg(reinterpret_cast<const float4*>(wrow1 + k0 + SG_BK)) : zero;
        }
#pragma unroll
        for (int c = 0; c < SG_BK; ++c) {
            const float4 a4 = *reinterpret_cast<const float4*>(&xs[buf][c][ty * 4]);
            const float4 b0 = *reinterpret_cast<const float4*>(&ws[buf][c][tx * 4]);
            const float4 b1 = *reinterpret_cast<const float4*>(&ws[buf][c][64 + tx * 4]);
            const float a[4] = {a4.x, a4.y, a4.z, a4.w};
            const float b[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 8; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        buf ^= 1;   // the other buffer was last read before the barrier above
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int mm = m0 + ty * 4 + i;
        if (mm >= m) continue;
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int nn = n0 + hh * 64 + tx * 4 + j;
                if (nn < n_out) y[(int64_t)mm * ldy + nn] = apply_act(acc[i][hh * 4 + j] + (bias ? bias[nn] : 0.0f), act);
            }
        }
    }
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
    } else if (!pre_silu && linear_tf32_usable(w, x, m, k, n, ldx)) {
        // enough rows for the tensor cores: tf32 MMA straight on the f32 operands (edb200_linear_tf32.cu)
        EDB_TRY(launch_linear_tf32(w, bias, x, m, k, n, ldx, act, y, ldy, s));
    } else {
        if (pre_silu) return fail(EDB200_ERR_UNSUPPORTED, "linear_f32: pre_silu only for m <= 8");
        const bool aligned = (k % SG_BK) == 0 && (ldx % 4) == 0 && ((reinterpret_cast<uintptr_t>(w) |
                                                                       reinterpret_cast<uintptr_t>(x)) & 15u) == 0;
        if (aligned) {
            dim3 grid(static_cast<unsigned>((n + SG_BN - 1) / SG_BN), static_cast<unsigned>((m + SG_BM - 1) / SG_BM));
            sgemm_nt_tiled_kernel<<<grid, 256, 0, s>>>(w, bias, x, ldx, act, y, ldy, (int)m, (int)n, (int)k);
        } else {
            dim3 grid(static_cast<unsigned>((n + 63) / 64), static_cast<unsigned>((m + 63) / 64));
            sgemm_nt_kernel<<<grid, 256, 0, s>>>(w, bias, x, ldx, act, y, ldy, (int)m, (int)n, (int)k);
        }
    }
    count_launch();
    return check_cuda(cudaGetLastError(), "linear_f32 launch");
}

}  // extern "C"
