// The repacked ("tiled") device form of a quantised weight: one-time repack from
// raw ggml blocks, the exact dequantiser that proves the repack changes no value,
// and the small-m weight-streaming GEMV that reads the tiles directly.
#include "edb200_internal.h"

#include <cstring>
#include <new>
#include <vector>
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


// ------------------------------------------------------------ batched GEMV --
// Every adaLN projection of a denoise step has the same input vector (silu of the conditioning
// vector) and the same row length, so all of them run as ONE launch that streams their weights
// back to back: CTA b works on 32 rows of the weight that owns row block b (table of first
// blocks, binary search), the input is activated once by a small kernel and staged per CTA with
// 16-byte loads, and every warp has the loads of two k-steps in flight before it waits for the
// staging barrier.  Sequence-parallel ranks split the row blocks between them and store their
// results into every rank's output (peer pointers), so the weight stream is not replicated.
struct GemvBatchItem {
    const uint8_t* tiles;
    const float* bias;
    float* y;
    int n_out;
    int block0;   // first row block (32 rows) of this weight in the launch
};

__global__ void gemv_activate_kernel(const float* __restrict__ x, float* __restrict__ xa, int k, int pre_silu) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= k) return;
    float v = x[i];
    if (pre_silu) v = v / (1.0f + __expf(-v));
    xa[i] = v;
}

struct GemvPeers {
    long long delta[8];   // byte offset from this rank's output address to the same place on rank p
    int world;
};

template <int WT>
__global__ void __launch_bounds__(GEMV_WARPS * 32)
gemv_q_batch_kernel(const GemvBatchItem* __restrict__ items, int n_items, const float* __restrict__ xa, int k, int ksteps,
                    int block_first, const GemvPeers peers) {
    extern __shared__ float xs[];  // [k], then [GEMV_WARPS][32] partial sums
    const int b = block_first + blockIdx.x;
    int lo = 0, hi = n_items - 1;
    while (lo < hi) {
        const int mid = (lo + hi + 1) >> 1;
        if (items[mid].block0 <= b) lo = mid; else hi = mid - 1;
    }
    const GemvBatchItem it = items[lo];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n = (b - it.block0) * 32 + lane;
    const int64_t t = n / kQwTileRows;
    const int r = n % kQwTileRows;
    constexpr int TB = WT == EDB200_TYPE_Q8_0 ? kQwTileBytesQ8 : kQwTileBytesQ4;
    constexpr int NV = WT == EDB200_TYPE_Q8_0 ? 4 : 2;
    const uint8_t* base = it.tiles + t * ksteps * (int64_t)TB;
    // weight loads of the first two k-steps go out before the input is staged
    uint4 raw[2][NV];
    uint32_t sc[2][2];
#pragma unroll
    for (int u = 0; u < 2; ++u) {
        const int s = warp + u * GEMV_WARPS;
        if (s < ksteps) {
            const uint8_t* tile = base + (int64_t)s * TB;
#pragma unroll
            for (int c = 0; c < NV; ++c) raw[u][c] = __ldg(reinterpret_cast<const uint4*>(tile + (c * 128 + r) * 16));
            if (WT == EDB200_TYPE_Q8_0) {
                sc[u][0] = *reinterpret_cast<const uint16_t*>(tile + 8192 + r * 2) |
                           (static_cast<uint32_t>(*reinterpret_cast<const uint16_t*>(tile + 8192 + (128 + r) * 2)) << 16);
            } else {
                sc[u][0] = *reinterpret_cast<const uint16_t*>(tile + 4096 + r * 2) |
                           (static_cast<uint32_t>(*reinterpret_cast<const uint16_t*>(tile + 4096 + (128 + r) * 2)) << 16);
                sc[u][1] = *reinterpret_cast<const uint16_t*>(tile + 4608 + r * 2) |
                           (static_cast<uint32_t>(*reinterpret_cast<const uint16_t*>(tile + 4608 + (128 + r) * 2)) << 16);
            }
        }
    }
    for (int i = threadIdx.x; i < k / 4; i += blockDim.x) {
        reinterpret_cast<float4*>(xs)[i] = __ldg(reinterpret_cast<const float4*>(xa) + i);
    }
    __syncthreads();
    float acc = 0.0f;
    for (int s0 = warp; s0 < ksteps; s0 += 2 * GEMV_WARPS) {
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            const int s = s0 + u * GEMV_WARPS;
            if (s >= ksteps) break;
            const float* xp = xs + s * 64;
            const __half2 h0 = *reinterpret_cast<const __half2*>(&sc[u][0]);
            if (WT == EDB200_TYPE_Q8_0) {
                const float p0 = dot16_s8(raw[u][0], xp) + dot16_s8(raw[u][1], xp + 16);
                const float p1 = dot16_s8(raw[u][2], xp + 32) + dot16_s8(raw[u][3], xp + 48);
                acc += __low2float(h0) * p0 + __high2float(h0) * p1;
            } else {
                const __half2 h1 = *reinterpret_cast<const __half2*>(&sc[u][1]);
                float pl = 0.f, ph = 0.f, sl = 0.f, sh = 0.f;
#pragma unroll
                for (int c = 0; c < 2; ++c) {
                    const uint32_t w[4] = {raw[u][c].x, raw[u][c].y, raw[u][c].z, raw[u][c].w};
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const uint32_t byte = (w[j] >> (8 * e)) & 0xFF;
                            const float xlo = xp[c * 16 + 4 * j + e], xhi = xp[32 + c * 16 + 4 * j + e];
                            pl = fmaf(static_cast<float>(byte & 0x0F), xlo, pl);
                            ph = fmaf(static_cast<float>(byte >> 4), xhi, ph);
                            sl += xlo;
                            sh += xhi;
                        }
                    }
                }
                acc += __low2float(h0) * pl - __low2float(h1) * sl + __high2float(h0) * ph - __high2float(h1) * sh;
            }
            // refill this slot with the k-step two rounds ahead
            const int sn = s + 2 * GEMV_WARPS;
            if (sn < ksteps) {
                const uint8_t* tile = base + (int64_t)sn * TB;
#pragma unroll
                for (int c = 0; c < NV; ++c) raw[u][c] = __ldg(reinterpret_cast<const uint4*>(tile + (c * 128 + r) * 16));
                if (WT == EDB200_TYPE_Q8_0) {
                    sc[u][0] = *reinterpret_cast<const uint16_t*>(tile + 8192 + r * 2) |
                               (static_cast<uint32_t>(*reinterpret_cast<const uint16_t*>(tile + 8192 + (128 + r) * 2)) << 16);
                } else {
                    sc[u][0] = *reinterpret_cast<const uint16_t*>(tile + 4096 + r * 2) |
                               (static_cast<uint32_t>(*reinterpret_cast<const uint16_t*>(tile + 4096 + (128 + r) * 2)) << 16);
                    sc[u][1] = *reinterpret_cast<const uint16_t*>(tile + 4608 + r * 2) |
                               (static_cast<uint32_t>(*reinterpret_cast<const uint16_t*>(tile + 4608 + (128 + r) * 2)) << 16);
                }
            }
        }
    }
    float* part = xs + k;
    part[warp * 32 + lane] = acc;
    __syncthreads();
    if (warp == 0) {
        float v = 0.0f;
#pragma unroll
        for (int g = 0; g < GEMV_WARPS; ++g) v += part[g * 32 + lane];
        if (n < it.n_out) {
            v += it.bias ? it.bias[n] : 0.0f;
            char* dst = reinterpret_cast<char*>(it.y + n);
            for (int p = 0; p < peers.world; ++p) *reinterpret_cast<float*>(dst + peers.delta[p]) = v;
        }
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

struct edb200_gemv_batch {
    int n = 0;
    int ggml_type = 0;
    int64_t k = 0, ksteps = 0;
    int total_blocks = 0;
    double weight_bytes = 0.0, flops = 0.0;
    edb::GemvBatchItem* items = nullptr;   // device
    float* xa = nullptr;                   // device, [k]
};

edb200_status_t edb200_gemv_batch_create(const edb200_qweight_t* const* w, const float* const* bias, float* const* y, int n,
                                         void* stream, edb200_gemv_batch_t** out) {
    if (w == nullptr || y == nullptr || out == nullptr || n <= 0) return fail(EDB200_ERR_INVALID, "gemv_batch_create: null or empty argument");
    std::vector<edb::GemvBatchItem> items(n);
    edb200_gemv_batch* b = new (std::nothrow) edb200_gemv_batch();
    if (b == nullptr) return fail(EDB200_ERR_NOMEM, "gemv_batch_create: host allocation failed");
    int blocks = 0;
    for (int i = 0; i < n; ++i) {
        if (w[i] == nullptr || y[i] == nullptr) {
            delete b;
            return fail(EDB200_ERR_INVALID, "gemv_batch_create: null weight or output %d", i);
        }
        if (i == 0) {
            b->ggml_type = w[i]->ggml_type;
            b->k = w[i]->k;
            b->ksteps = w[i]->ksteps;
        } else if (w[i]->ggml_type != b->ggml_type || w[i]->k != b->k) {
            delete b;
            return fail(EDB200_ERR_INVALID, "gemv_batch_create: all weights must share one block type and row length");
        }
        items[i].tiles = w[i]->tiles;
        items[i].bias = bias ? bias[i] : nullptr;
        items[i].y = y[i];
        items[i].n_out = static_cast<int>(w[i]->n_out);
        items[i].block0 = blocks;
        blocks += static_cast<int>(w[i]->n_tiles * (kQwTileRows / 32));
        b->weight_bytes += (double)w[i]->n_out * (double)w[i]->k * (w[i]->ggml_type == EDB200_TYPE_Q8_0 ? 34.0 / 32.0 : 144.0 / 256.0);
        b->flops += 2.0 * (double)w[i]->n_out * (double)w[i]->k;
    }
    if ((b->k * 4 + GEMV_WARPS * 32 * 4) > 200 * 1024 || b->k % 4) {
        delete b;
        return fail(EDB200_ERR_UNSUPPORTED, "gemv_batch_create: row length too large for the shared-memory stage");
    }
    b->n = n;
    b->total_blocks = blocks;
    cudaError_t e = cudaMalloc(reinterpret_cast<void**>(&b->items), sizeof(edb::GemvBatchItem) * n);
    if (e == cudaSuccess) e = cudaMalloc(reinterpret_cast<void**>(&b->xa), b->k * 4);
    if (e == cudaSuccess) {
        e = cudaMemcpyAsync(b->items, items.data(), sizeof(edb::GemvBatchItem) * n, cudaMemcpyHostToDevice,
                            static_cast<cudaStream_t>(stream));
    }
    if (e == cudaSuccess) e = cudaStreamSynchronize(static_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) {
        edb200_gemv_batch_destroy(b);
        return check_cuda(e, "gemv_batch_create");
    }
    *out = b;
    return EDB200_OK;
}

void edb200_gemv_batch_destroy(edb200_gemv_batch_t* b) {
    if (b == nullptr) return;
    cudaFree(b->items);
    cudaFree(b->xa);
    delete b;
}

edb200_status_t edb200_gemv_batch_run(const edb200_gemv_batch_t* b, const float* x, int pre_silu, const edb200_sp_peers_t* share,
                                      void* stream) {
    if (b == nullptr || x == nullptr) return fail(EDB200_ERR_INVALID, "gemv_batch_run: null argument");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    edb::GemvPeers peers;
    memset(&peers, 0, sizeof(peers));
    peers.world = 1;
    int first = 0, count = b->total_blocks;
    if (share != nullptr) {
        if (share->world <= 0 || share->world > 8 || share->rank < 0 || share->rank >= share->world) {
            return fail(EDB200_ERR_INVALID, "gemv_batch_run: bad peer description");
        }
        // rank r computes row blocks [r * per, (r + 1) * per) and stores them on every rank:
        // buf[0][p] is rank p's copy of one common reference address
        peers.world = share->world;
        for (int p = 0; p < share->world; ++p) {
            if (share->buf[0][p] == nullptr) return fail(EDB200_ERR_INVALID, "gemv_batch_run: null peer buffer");
            peers.delta[p] = static_cast<const char*>(share->buf[0][p]) - static_cast<const char*>(share->buf[0][share->rank]);
        }
        const int per = (b->total_blocks + share->world - 1) / share->world;
        first = share->rank * per;
        count = b->total_blocks - first;
        if (count > per) count = per;
        if (count < 0) count = 0;
    }
    const size_t smem = (static_cast<size_t>(b->k) + GEMV_WARPS * 32) * sizeof(float);
    const double frac = b->total_blocks > 0 ? (double)count / b->total_blocks : 0.0;
    ProfScope prof(s, PROF_GEMV, b->flops * frac, b->weight_bytes * frac);
    gemv_activate_kernel<<<static_cast<unsigned>((b->k + 255) / 256), 256, 0, s>>>(x, b->xa, static_cast<int>(b->k), pre_silu);
    count_launch();
    if (count > 0) {
        if (b->ggml_type == EDB200_TYPE_Q8_0) {
            auto kern = edb::gemv_q_batch_kernel<EDB200_TYPE_Q8_0>;
            if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            kern<<<count, GEMV_WARPS * 32, smem, s>>>(b->items, b->n, b->xa, (int)b->k, (int)b->ksteps, first, peers);
        } else {
            auto kern = edb::gemv_q_batch_kernel<EDB200_TYPE_Q4_K>;
            if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            kern<<<count, GEMV_WARPS * 32, smem, s>>>(b->items, b->n, b->xa, (int)b->k, (int)b->ksteps, first, peers);
        }
        count_launch();
    }
    return check_cuda(cudaGetLastError(), "gemv_batch launch");
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
