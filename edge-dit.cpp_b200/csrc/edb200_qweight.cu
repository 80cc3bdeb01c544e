// The repacked ("tiled") device form of a quantised weight: one-time repack from
// raw ggml blocks, the exact dequantiser that proves the repack changes no value,
// and the small-m weight-streaming GEMV that reads the tiles directly.
#include "edb200_internal.h"
#include "edb200_codec.cuh"

#include <cuda_fp16.h>

namespace edb {

// ------------------------------------------------------------------ repack --

// q8_0: one thread per 32-block of raw input (row n, block b).
__global__ void repack_q8_0_kernel(const uint8_t* __restrict__ blocks, uint8_t* __restrict__ tiles, int64_t n_out,
                                   int64_t kb, int64_t ksteps) {
    const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= n_out * kb) return;
    const int64_t n = idx / kb;
    const int64_t b = idx % kb;
    const uint16_t* p = reinterpret_cast<const uint16_t*>(blocks + idx * 34);
    uint16_t w[17];
#pragma unroll
    for (int i = 0; i < 17; ++i) w[i] = p[i];
    uint32_t o[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        // stored as u = q + 128 (sign bit flipped): the consumers build floats from the unsigned byte
        o[i] = (static_cast<uint32_t>(w[1 + 2 * i]) | (static_cast<uint32_t>(w[2 + 2 * i]) << 16)) ^ 0x80808080u;
    }
    const int64_t t = n / kQwTileRows;
    const int r = static_cast<int>(n % kQwTileRows);
    const int64_t s = b >> 1;
    const int h = static_cast<int>(b & 1);
    uint8_t* tile = tiles + (t * ksteps + s) * kQwTileBytesQ8;
    *reinterpret_cast<uint4*>(tile + ((2 * h + 0) * 128 + r) * 16) = make_uint4(o[0], o[1], o[2], o[3]);
    *reinterpret_cast<uint4*>(tile + ((2 * h + 1) * 128 + r) * 16) = make_uint4(o[4], o[5], o[6], o[7]);
    *reinterpret_cast<uint16_t*>(tile + 8192 + (h * 128 + r) * 2) = w[0];
}

// q4_K: one thread per 256-block of raw input (row n, super-block B).
__global__ void repack_q4_k_kernel(const uint8_t* __restrict__ blocks, uint8_t* __restrict__ tiles,
                                   uint8_t* __restrict__ hdr, int64_t n_out, int64_t kb256, int64_t ksteps) {
    const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= n_out * kb256) return;
    const int64_t n = idx / kb256;
    const int64_t B = idx % kb256;
    const uint8_t* p = blocks + idx * 144;
    const uint4 head = *reinterpret_cast<const uint4*>(p);
    *reinterpret_cast<uint4*>(hdr + idx * 16) = head;
    const float d = __half2float(*reinterpret_cast<const __half*>(p));
    const float dmin = __half2float(*reinterpret_cast<const __half*>(p + 2));
    const int64_t t = n / kQwTileRows;
    const int r = static_cast<int>(n % kQwTileRows);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        uint8_t* tile = tiles + (t * ksteps + B * 4 + j) * kQwTileBytesQ4;
        const uint4* src = reinterpret_cast<const uint4*>(p + 16 + j * 32);
        *reinterpret_cast<uint4*>(tile + (0 * 128 + r) * 16) = src[0];
        *reinterpret_cast<uint4*>(tile + (1 * 128 + r) * 16) = src[1];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            uint32_t sc, mn;
            q4k_scale_min(2 * j + h, p + 4, sc, mn);
            *reinterpret_cast<__half*>(tile + 4096 + (h * 128 + r) * 2) =
                __float2half_rn(__fmul_rn(d, static_cast<float>(sc)));
            *reinterpret_cast<__half*>(tile + 4608 + (h * 128 + r) * 2) =
                __float2half_rn(__fmul_rn(dmin, static_cast<float>(mn)));
        }
    }
}

// Exact f32 dequantisation from the tiled form (one thread per weight).
__global__ void qweight_dequant_q8_0_kernel(const uint8_t* __restrict__ tiles, float* __restrict__ out, int64_t n_out,
                                            int64_t k, int64_t ksteps) {
    const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= n_out * k) return;
    const int64_t n = idx / k, kk = idx % k;
    const uint8_t* tile = tiles + ((n / kQwTileRows) * ksteps + (kk >> 6)) * kQwTileBytesQ8;
    const int r = static_cast<int>(n % kQwTileRows), e = static_cast<int>(kk & 63);
    const int q = static_cast<int>(tile[((e >> 4) * 128 + r) * 16 + (e & 15)]) - 128;
    const __half d = *reinterpret_cast<const __half*>(tile + 8192 + ((e >> 5) * 128 + r) * 2);
    out[idx] = __fmul_rn(static_cast<float>(q), __half2float(d));
}

__global__ void qweight_dequant_q4_k_kernel(const uint8_t* __restrict__ tiles, const uint8_t* __restrict__ hdr,
                                            float* __restrict__ out, int64_t n_out, int64_t k, int64_t ksteps) {
    const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= n_out * k) return;
    const int64_t n = idx / k, kk = idx % k;
    const uint8_t* tile = tiles + ((n / kQwTileRows) * ksteps + (kk >> 6)) * kQwTileBytesQ4;
    const int r = static_cast<int>(n % kQwTileRows), e = static_cast<int>(kk & 63);
    const int i = e & 31;
    const uint8_t byte = tile[((i >> 4) * 128 + r) * 16 + (i & 15)];
    const uint32_t q = (e >= 32) ? (byte >> 4) : (byte & 0x0F);
    const uint8_t* h = hdr + (n * (k >> 8) + (kk >> 8)) * 16;
    const float d = __half2float(*reinterpret_cast<const __half*>(h));
    const float dmin = __half2float(*reinterpret_cast<const __half*>(h + 2));
    uint32_t sc, mn;
    q4k_scale_min(static_cast<int>((kk & 255) >> 5), h + 4, sc, mn);
    const float dl = __fmul_rn(d, static_cast<float>(sc));
    const float ml = __fmul_rn(dmin, static_cast<float>(mn));
    out[idx] = __fsub_rn(__fmul_rn(dl, static_cast<float>(q)), ml);
}

// -------------------------------------------------------------------- GEMV --
// y[mm][n] = sum_k act(x[mm][k]) * W[n][k] + bias[n],  mm < M <= 8.
// CTA = 8 warps on 32 consecutive weight rows (one lane per row); warp g takes
// k-steps g, g+8, ...: every load is 32 rows x 16 B = 512 contiguous bytes of a
// tile.  x is staged once per CTA in shared memory as f32 (read as a broadcast).
// The eight partial sums per row are added in warp order through shared memory.
constexpr int GEMV_WARPS = 8;
constexpr int GEMV_MAX_M = 8;

__device__ __forceinline__ float dot16_s8(const uint4& raw, const float* xp) {
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
    float part = 0.0f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const float4 xv = *reinterpret_cast<const float4*>(xp + 4 * j);
        // int8 -> f32 without conversion instructions: the stored byte u = q + 128 placed in
        // the mantissa of 2^23 gives 8388608 + u exactly; subtract 8388736 to get q.
        const uint32_t u = w[j];
        const float q0 = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7650)) - 8388736.0f;
        const float q1 = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7651)) - 8388736.0f;
        const float q2 = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7652)) - 8388736.0f;
        const float q3 = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7653)) - 8388736.0f;
        part = fmaf(q0, xv.x, part);
        part = fmaf(q1, xv.y, part);
        part = fmaf(q2, xv.z, part);
        part = fmaf(q3, xv.w, part);
    }
    return part;
}

template <int WT, int M>
__global__ void __launch_bounds__(GEMV_WARPS * 32)
gemv_q_kernel(const uint8_t* __restrict__ tiles, const float* __restrict__ x, int64_t ldx, int pre_silu,
              const float* __restrict__ bias, float* __restrict__ y, int64_t ldy, int n_out, int k, int ksteps) {
    extern __shared__ float xs[];  // [M][k], then [GEMV_WARPS][M][32] partial sums
    for (int i = threadIdx.x; i < M * k; i += blockDim.x) {
        const int mm = i / k, kk = i % k;
        float v = x[(int64_t)mm * ldx + kk];
        if (pre_silu) v = v / (1.0f + __expf(-v));
        xs[i] = v;
    }
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n = blockIdx.x * 32 + lane;
    const int64_t t = n / kQwTileRows;
    const int r = n % kQwTileRows;
    constexpr int TB = WT == EDB200_TYPE_Q8_0 ? kQwTileBytesQ8 : kQwTileBytesQ4;
    const uint8_t* base = tiles + t * ksteps * (int64_t)TB;
    float acc[M];
#pragma unroll
    for (int mm = 0; mm < M; ++mm) acc[mm] = 0.0f;

    for (int s = warp; s < ksteps; s += GEMV_WARPS) {
        const uint8_t* tile = base + (int64_t)s * TB;
        if (WT == EDB200_TYPE_Q8_0) {
            uint4 raw[4];
#pragma unroll
            for (int c = 0; c < 4; ++c) raw[c] = __ldg(reinterpret_cast<const uint4*>(tile + (c * 128 + r) * 16));
            const float d0 = __half2float(*reinterpret_cast<const __half*>(tile + 8192 + r * 2));
            const float d1 = __half2float(*reinterpret_cast<const __half*>(tile + 8192 + (128 + r) * 2));
#pragma unroll
            for (int mm = 0; mm < M; ++mm) {
                const float* xp = xs + mm * k + s * 64;
                const float p0 = dot16_s8(raw[0], xp) + dot16_s8(raw[1], xp + 16);
                const float p1 = dot16_s8(raw[2], xp + 32) + dot16_s8(raw[3], xp + 48);
                acc[mm] += d0 * p0 + d1 * p1;
            }
        } else {
            uint4 raw[2];
#pragma unroll
            for (int c = 0; c < 2; ++c) raw[c] = __ldg(reinterpret_cast<const uint4*>(tile + (c * 128 + r) * 16));
            const float a0 = __half2float(*reinterpret_cast<const __half*>(tile + 4096 + r * 2));
            const float a1 = __half2float(*reinterpret_cast<const __half*>(tile + 4096 + (128 + r) * 2));
            const float b0 = __half2float(*reinterpret_cast<const __half*>(tile + 4608 + r * 2));
            const float b1 = __half2float(*reinterpret_cast<const __half*>(tile + 4608 + (128 + r) * 2));
#pragma unroll
            for (int mm = 0; mm < M; ++mm) {
                const float* xl = xs + mm * k + s * 64;
                float pl = 0.f, ph = 0.f, sl = 0.f, sh = 0.f;
#pragma unroll
                for (int c = 0; c < 2; ++c) {
                    const uint32_t w[4] = {raw[c].x, raw[c].y, raw[c].z, raw[c].w};
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const uint32_t byte = (w[j] >> (8 * e)) & 0xFF;
                            const float xlo = xl[c * 16 + 4 * j + e], xhi = xl[32 + c * 16 + 4 * j + e];
                            pl = fmaf(static_cast<float>(byte & 0x0F), xlo, pl);
                            ph = fmaf(static_cast<float>(byte >> 4), xhi, ph);
                            sl += xlo;
                            sh += xhi;
                        }
                    }
                }
                acc[mm] += a0 * pl - b0 * sl + a1 * ph - b1 * sh;
            }
        }
    }
    float* part = xs + M * k;
#pragma unroll
    for (int mm = 0; mm < M; ++mm) part[(warp * M + mm) * 32 + lane] = acc[mm];
    __syncthreads();
    for (int i = threadIdx.x; i < M * 32; i += blockDim.x) {
        const int mm = i / 32, ln = i % 32;
        float v = 0.0f;
#pragma unroll
        for (int g = 0; g < GEMV_WARPS; ++g) v += part[(g * M + mm) * 32 + ln];
        const int nn = blockIdx.x * 32 + ln;
        if (nn < n_out) y[(int64_t)mm * ldy + nn] = v + (bias ? bias[nn] : 0.0f);
    }
}

template <int WT>
static edb200_status_t launch_gemv_q(const edb200_qweight_t* w, const float* x, int64_t m, int64_t ldx, int pre_silu,
                                     const float* bias, float* y, int64_t ldy, cudaStream_t stream) {
    const int grid = static_cast<int>(w->n_tiles * (kQwTileRows / 32));
    const size_t smem = (static_cast<size_t>(m) * w->k + GEMV_WARPS * m * 32) * sizeof(float);
    ProfScope prof(stream, PROF_GEMV, 2.0 * (double)m * (double)w->n_out * (double)w->k, (double)w->bytes);
#define EDB_GEMV_CASE(MM)                                                                                         \
    case MM: {                                                                                                    \
        auto kern = gemv_q_kernel<WT, MM>;                                                                        \
        if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        kern<<<grid, GEMV_WARPS * 32, smem, stream>>>(w->tiles, x, ldx, pre_silu, bias, y, ldy, (int)w->n_out,    \
                                                      (int)w->k, (int)w->ksteps);                                 \
        break;                                                                                                    \
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

edb200_status_t edb200_qweight_create(int ggml_type, const void* blocks, int64_t n_out, int64_t k, void* stream,
                                      edb200_qweight_t** out) {
    if (blocks == nullptr || out == nullptr || n_out <= 0 || k <= 0) {
        return fail(EDB200_ERR_INVALID, "qweight_create: null or empty argument");
    }
    if (ggml_type != EDB200_TYPE_Q8_0 && ggml_type != EDB200_TYPE_Q4_K) {
        return fail(EDB200_ERR_UNSUPPORTED, "qweight_create: type %d", ggml_type);
    }
    const int blk = ggml_type == EDB200_TYPE_Q8_0 ? 64 : 256;
    if (k % blk) return fail(EDB200_ERR_INVALID, "qweight_create: k must be a multiple of %d", blk);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    edb200_qweight_t* w = new (std::nothrow) edb200_qweight_t();
    if (w == nullptr) return fail(EDB200_ERR_NOMEM, "qweight_create: host allocation failed");
    w->ggml_type = ggml_type;
    w->n_out = n_out;
    w->k = k;
    w->n_tiles = (n_out + kQwTileRows - 1) / kQwTileRows;
    w->ksteps = k / kQwTileK;
    w->tile_bytes = ggml_type == EDB200_TYPE_Q8_0 ? kQwTileBytesQ8 : kQwTileBytesQ4;
    // one spare (zero) tile row so that the GEMM may always fetch weight tiles in pairs
    const int64_t tiles_bytes = (w->n_tiles + (w->n_tiles & 1)) * w->ksteps * w->tile_bytes;
    const int64_t hdr_bytes = ggml_type == EDB200_TYPE_Q4_K ? n_out * (k / 256) * 16 : 0;
    cudaError_t e = cudaMalloc(reinterpret_cast<void**>(&w->tiles), tiles_bytes);
    if (e == cudaSuccess && hdr_bytes > 0) e = cudaMalloc(reinterpret_cast<void**>(&w->hdr), hdr_bytes);
    if (e != cudaSuccess) {
        edb200_qweight_destroy(w);
        return fail(EDB200_ERR_NOMEM, "qweight_create: cudaMalloc: %s", cudaGetErrorString(e));
    }
    w->bytes = tiles_bytes + hdr_bytes;
    if ((n_out % kQwTileRows) || (w->n_tiles & 1)) cudaMemsetAsync(w->tiles, 0, tiles_bytes, s);   // zero the padding
    if (ggml_type == EDB200_TYPE_Q8_0) {
        const int64_t nb = n_out * (k / 32);
        repack_q8_0_kernel<<<static_cast<unsigned>((nb + 255) / 256), 256, 0, s>>>(
            static_cast<const uint8_t*>(blocks), w->tiles, n_out, k / 32, w->ksteps);
    } else {
        const int64_t nb = n_out * (k / 256);
        repack_q4_k_kernel<<<static_cast<unsigned>((nb + 127) / 128), 128, 0, s>>>(
            static_cast<const uint8_t*>(blocks), w->tiles, w->hdr, n_out, k / 256, w->ksteps);
    }
    count_launch();
    e = cudaGetLastError();
    if (e == cudaSuccess) e = cudaStreamSynchronize(s);
    if (e != cudaSuccess) {
        edb200_qweight_destroy(w);
        return check_cuda(e, "qweight_create repack");
    }
    *out = w;
    return EDB200_OK;
}

void edb200_qweight_destroy(edb200_qweight_t* w) {
    if (w == nullptr) return;
    cudaFree(w->tiles);
    cudaFree(w->hdr);
    delete w;
}

int64_t edb200_qweight_bytes(const edb200_qweight_t* w) { return w ? w->bytes : 0; }

edb200_status_t edb200_qweight_dequantize(const edb200_qweight_t* w, float* out, void* stream) {
    if (w == nullptr || out == nullptr) return fail(EDB200_ERR_INVALID, "qweight_dequantize: null argument");
    const int64_t total = w->n_out * w->k;
    const unsigned grid = static_cast<unsigned>((total + 255) / 256);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (w->ggml_type == EDB200_TYPE_Q8_0) {
        qweight_dequant_q8_0_kernel<<<grid, 256, 0, s>>>(w->tiles, out, w->n_out, w->k, w->ksteps);
    } else {
        qweight_dequant_q4_k_kernel<<<grid, 256, 0, s>>>(w->tiles, w->hdr, out, w->n_out, w->k, w->ksteps);
    }
    count_launch();
    return check_cuda(cudaGetLastError(), "qweight_dequantize launch");
}

edb200_status_t edb200_gemv_q(const edb200_qweight_t* w, const float* x, int64_t m, int64_t ldx, int pre_silu,
                              const float* bias, float* y, int64_t ldy, void* stream) {
    if (w == nullptr || x == nullptr || y == nullptr) return fail(EDB200_ERR_INVALID, "gemv_q: null argument");
    if (m < 1 || m > GEMV_MAX_M) return fail(EDB200_ERR_INVALID, "gemv_q: m must be in 1..8");
    if (ldx < w->k || ldy < w->n_out) return fail(EDB200_ERR_INVALID, "gemv_q: leading dimension too small");
    if ((static_cast<size_t>(m) * w->k + GEMV_WARPS * m * 32) * 4 > 200 * 1024) {
        return fail(EDB200_ERR_UNSUPPORTED, "gemv_q: m*k too large for the shared-memory stage");
    }
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (w->ggml_type == EDB200_TYPE_Q8_0) return launch_gemv_q<EDB200_TYPE_Q8_0>(w, x, m, ldx, pre_silu, bias, y, ldy, s);
    return launch_gemv_q<EDB200_TYPE_Q4_K>(w, x, m, ldx, pre_silu, bias, y, ldy, s);
}

}  // extern "C"
