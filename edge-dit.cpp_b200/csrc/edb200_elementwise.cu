// Memory-bound kernels of the DiT block: LayerNorm + adaLN modulate, the
// bit-exact f32 modulate / residual-gate / RoPE ops of the reference's custom-op
// surface, and the fused QK-RMSNorm + RoPE + head-major pack that feeds attention.
// All global accesses are 128-bit where the layout allows; reductions use warp
// shuffles.
#include "edb200_internal.h"

#include <type_traits>

#include <cstring>

#include <cuda_bf16.h>
#include <cuda_fp16.h>

namespace edb {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int m = 16; m > 0; m >>= 1) v += __shfl_xor_sync(0xffffffffu, v, m);
    return v;
}

template <int THREADS>
__device__ __forceinline__ float block_sum(float v, float* sh) {
    v = warp_sum(v);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    __syncthreads();  // protect sh from the previous reduction
    if (lane == 0) sh[warp] = v;
    __syncthreads();
    float t = (lane < THREADS / 32) ? sh[lane] : 0.0f;
    return warp_sum(t);
}

__device__ __forceinline__ void store_vec4(void* base, int dtype, int64_t elem_off, float a, float b, float c,
                                           float d) {
    if (dtype == EDB200_TYPE_F32) {
        *reinterpret_cast<float4*>(static_cast<float*>(base) + elem_off) = make_float4(a, b, c, d);
    } else if (dtype == EDB200_TYPE_BF16) {
        __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
        uint2 u;
        u.x = *reinterpret_cast<uint32_t*>(&lo);
        u.y = *reinterpret_cast<uint32_t*>(&hi);
        *reinterpret_cast<uint2*>(static_cast<__nv_bfloat16*>(base) + elem_off) = u;
    } else {
        __half2 lo = __floats2half2_rn(a, b), hi = __floats2half2_rn(c, d);
        uint2 u;
        u.x = *reinterpret_cast<uint32_t*>(&lo);
        u.y = *reinterpret_cast<uint32_t*>(&hi);
        *reinterpret_cast<uint2*>(static_cast<__half*>(base) + elem_off) = u;
    }
}

__device__ __forceinline__ float4 load_vec4(const void* base, int dtype, int64_t elem_off) {
    if (dtype == EDB200_TYPE_F32) {
        return *reinterpret_cast<const float4*>(static_cast<const float*>(base) + elem_off);
    }
    const uint2 u = *reinterpret_cast<const uint2*>(static_cast<const uint16_t*>(base) + elem_off);
    if (dtype == EDB200_TYPE_BF16) {
        const float2 lo = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.x));
        const float2 hi = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.y));
        return make_float4(lo.x, lo.y, hi.x, hi.y);
    }
    const float2 lo = __half22float2(*reinterpret_cast<const __half2*>(&u.x));
    const float2 hi = __half22float2(*reinterpret_cast<const __half2*>(&u.y));
    return make_float4(lo.x, lo.y, hi.x, hi.y);
}

// ---------------------------------------------------- LayerNorm + modulate --
// One CTA per token row.  y = (xn + xn*scale) + shift with xn = (x-mean)*rstd,
// the association the reference's modulate uses
// (src/core/backend/ggml/ed_ggml_modulation_ext.hpp:168-199) applied to ggml_norm's output.
constexpr int LN_THREADS = 256;
#ifndef LN_MIN_BLOCKS
#define LN_MIN_BLOCKS 1
#endif
constexpr int LN_MAXV = 8;  // float4 per thread -> H <= 8192

// NV > 0: the row is exactly NV * LN_THREADS float4 wide and every bound check folds away (the common hidden
// sizes: 3072 -> 3, 5120 -> 5); NV == 0: any width up to LN_MAXV * LN_THREADS float4.  Same arithmetic, same
// order of additions in both.
template <int NV>
__global__ void __launch_bounds__(LN_THREADS, LN_MIN_BLOCKS)
layernorm_modulate_kernel(const float* __restrict__ x, int64_t ldx, const float* __restrict__ shift,
                          const float* __restrict__ scale, const float* __restrict__ ln_w,
                          const float* __restrict__ ln_b, int H, float eps, void* __restrict__ y, int y_dtype,
                          int64_t ldy) {
    __shared__ float sh[LN_THREADS / 32];
    const int64_t row = blockIdx.x;
    const float* xr = x + row * ldx;
    const int nvec = H >> 2;
    constexpr bool EXACT = NV > 0;
    constexpr int NI = EXACT ? NV : LN_MAXV;
    float4 v[NI];
    float s = 0.0f;
#pragma unroll
    for (int i = 0; i < NI; ++i) {
        const int c = threadIdx.x + i * LN_THREADS;
        if (EXACT || c < nvec) {
            v[i] = *reinterpret_cast<const float4*>(xr + 4 * c);
            s += (v[i].x + v[i].y) + (v[i].z + v[i].w);
        }
    }
    const float mean = block_sum<LN_THREADS>(s, sh) / static_cast<float>(H);
    float q = 0.0f;
#pragma unroll
    for (int i = 0; i < NI; ++i) {
        const int c = threadIdx.x + i * LN_THREADS;
        if (EXACT || c < nvec) {
            v[i].x -= mean;
            v[i].y -= mean;
            v[i].z -= mean;
            v[i].w -= mean;
            q += (v[i].x * v[i].x + v[i].y * v[i].y) + (v[i].z * v[i].z + v[i].w * v[i].w);
        }
    }
    const float var = block_sum<LN_THREADS>(q, sh) / static_cast<float>(H);
    const float rstd = 1.0f / sqrtf(var + eps);
#pragma unroll
    for (int i = 0; i < NI; ++i) {
        const int c = threadIdx.x + i * LN_THREADS;
        if (EXACT || c < nvec) {
            float o[4] = {v[i].x * rstd, v[i].y * rstd, v[i].z * rstd, v[i].w * rstd};
            if (ln_w != nullptr) {
                const float4 w4 = __ldg(reinterpret_cast<const float4*>(ln_w) + c);
                o[0] *= w4.x, o[1] *= w4.y, o[2] *= w4.z, o[3] *= w4.w;
            }
            if (ln_b != nullptr) {
                const float4 b4 = __ldg(reinterpret_cast<const float4*>(ln_b) + c);
                o[0] += b4.x, o[1] += b4.y, o[2] += b4.z, o[3] += b4.w;
            }
            if (scale != nullptr) {
                const float4 sc = __ldg(reinterpret_cast<const float4*>(scale) + c);
                o[0] = __fadd_rn(o[0], __fmul_rn(o[0], sc.x));
                o[1] = __fadd_rn(o[1], __fmul_rn(o[1], sc.y));
                o[2] = __fadd_rn(o[2], __fmul_rn(o[2], sc.z));
                o[3] = __fadd_rn(o[3], __fmul_rn(o[3], sc.w));
            }
            if (shift != nullptr) {
                const float4 sf = __ldg(reinterpret_cast<const float4*>(shift) + c);
                o[0] = __fadd_rn(o[0], sf.x);
                o[1] = __fadd_rn(o[1], sf.y);
                o[2] = __fadd_rn(o[2], sf.z);
                o[3] = __fadd_rn(o[3], sf.w);
            }
            store_vec4(y, y_dtype, row * ldy + 4 * c, o[0], o[1], o[2], o[3]);
        }
    }
}

// ------------------------------------------- bit-exact f32 modulate / gate --
// y = (x + x*scale) + shift ; y = residual + x*gate, every op rounded to f32
// separately (no FMA), broadcast of the [H] vectors over rows.
// (src/core/backend/ggml/ed_ggml_modulation_ext.hpp:168-226, cuda/ed_cuda_modulation.cu:77-301)
__global__ void fused_modulate_kernel(const float4* __restrict__ x, const float4* __restrict__ shift,
                                      const float4* __restrict__ scale, float4* __restrict__ y, int64_t total4,
                                      int h4) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total4) return;
    const int c = static_cast<int>(i % h4);
    const float4 xv = x[i], sc = __ldg(scale + c), sf = __ldg(shift + c);
    float4 o;
    o.x = __fadd_rn(__fadd_rn(xv.x, __fmul_rn(xv.x, sc.x)), sf.x);
    o.y = __fadd_rn(__fadd_rn(xv.y, __fmul_rn(xv.y, sc.y)), sf.y);
    o.z = __fadd_rn(__fadd_rn(xv.z, __fmul_rn(xv.z, sc.z)), sf.z);
    o.w = __fadd_rn(__fadd_rn(xv.w, __fmul_rn(xv.w, sc.w)), sf.w);
    y[i] = o;
}

__global__ void fused_residual_gate_kernel(const float4* __restrict__ res, const float4* __restrict__ x,
                                           const float4* __restrict__ gate, float4* __restrict__ y, int64_t total4,
                                           int h4) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total4) return;
    const int c = static_cast<int>(i % h4);
    const float4 rv = res[i], xv = x[i], g = __ldg(gate + c);
    float4 o;
    o.x = __fadd_rn(rv.x, __fmul_rn(xv.x, g.x));
    o.y = __fadd_rn(rv.y, __fmul_rn(xv.y, g.y));
    o.z = __fadd_rn(rv.z, __fmul_rn(xv.z, g.z));
    o.w = __fadd_rn(rv.w, __fmul_rn(xv.w, g.w));
    y[i] = o;
}

__global__ void advance_step_kernel(int* step) { *step += 1; }

// SD3's form of the sampler update (sd3_pipeline.cpp:697): x += model_out * (sigma_next - sigma).
// `sched` != NULL: dt = sched[*step + 1] - sched[*step], read on the device.
__global__ void flow_update_kernel(float* __restrict__ x, const float* __restrict__ v, float dt,
                                   const float* __restrict__ sched, const int* __restrict__ step, int64_t n) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    if (sched != nullptr) {
        const int k = *step;
        dt = __fsub_rn(sched[k + 1], sched[k]);
    }
    x[i] = __fadd_rn(x[i], __fmul_rn(v[i], dt));
}

__global__ void sub_kernel(const float4* __restrict__ a, const float4* __restrict__ b, float4* __restrict__ out, int64_t n4) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n4) return;
    const float4 x = a[i], y = b[i];
    out[i] = make_float4(__fsub_rn(x.x, y.x), __fsub_rn(x.y, y.y), __fsub_rn(x.z, y.z), __fsub_rn(x.w, y.w));
}

// Sampler update of one step (flux_pipeline.cpp:1290-1297): every operation rounded on its own.
// `sched` != NULL: sigma = sched[*step], sigma_next = sched[*step + 1], read on the device.
__global__ void euler_update_kernel(float* __restrict__ x, const float* __restrict__ v, float sigma, float sigma_next,
                                    const float* __restrict__ sched, const int* __restrict__ step, int64_t n) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    if (sched != nullptr) {
        const int k = *step;
        sigma = sched[k];
        sigma_next = sched[k + 1];
    }
    const float xi = x[i];
    const float denoised = __fadd_rn(__fmul_rn(v[i], -sigma), xi);   // model_out * c_out + x * c_skip, c_skip = 1
    if (sigma == 0.0f) {
        x[i] = denoised;
    } else {
        const float d = __fdiv_rn(__fsub_rn(xi, denoised), sigma);
        x[i] = __fadd_rn(xi, __fmul_rn(d, __fsub_rn(sigma_next, sigma)));
    }
}

// ---------------------------------------- QK-RMSNorm + RoPE + head-major pack --
// One warp per (token, head); lane owns 4 consecutive channels (two RoPE pairs)
// of a 128-wide head, or 2 channels (one pair) of a 64-wide head.
// q,k: x * rsqrt(mean(x^2)+eps) * w  (src/dit_models/components/common/normalization.cpp:42-61)
// then y0 = x0*pe00 + x1*pe10, y1 = x0*pe01 + x1*pe11 with the stored
// [[cos,-sin],[sin,cos]] table (src/core/backend/ggml/ed_ggml_rope_ext.hpp:105-184),
// written head-major [head][token][d] like the reference's fused RoPE op.
// Sequence-parallel destination: head h of the local tokens belongs to rank h / hp and is
// stored straight into that rank's [hp, L_total, D] buffers (peer-mapped pointers), at the
// global token position.  hp == 0: plain local output.
struct PackPeers {
    void* q[8];
    void* k[8];
    void* v[8];
    int hp;
    long long global_first;   // global position of this rank's token 0
    // Whole-row RMSNorm (Wan: over all heads before the head split, wan.hpp:3504-3532):
    // rstd per token computed beforehand, weights indexed by head * D + channel.
    const float* rstd_q;
    const float* rstd_k;
    int w_head_stride;        // 0: one [D] weight vector for every head, D: [heads * D]
    int skip_mask;            // bit i set: tensor i (0 q, 1 k, 2 v) is not produced
};

// A warp walks `heads_per_warp` consecutive heads of one token: the token's RoPE table and the norm weights
// are read once, the address arithmetic is incremental, and the rows of the next two heads are already on
// their way while one head is normalised and rotated (about 1.5 KB in flight per warp).
template <int D, bool IN16>
__global__ void __launch_bounds__(256, 3)
qk_norm_rope_pack_kernel(const void* __restrict__ qkv, int in_dtype, int64_t ld, int64_t q_off, int64_t k_off,
                         int64_t v_off, int64_t T, int n_heads, int heads_per_warp, const float* __restrict__ q_w,
                         const float* __restrict__ k_w, float eps, const float* __restrict__ pe, int64_t tok_off,
                         int64_t L_total, void* __restrict__ q_out, void* __restrict__ k_out,
                         void* __restrict__ v_out, int out_dtype, const PackPeers peers) {
    constexpr int E = D / 32;  // elements per lane: 4 or 2
    constexpr int AHEAD = 2;   // heads fetched ahead of the one being processed
    using Raw = typename std::conditional<IN16, uint2, float4>::type;   // E values as loaded
    const int lane = threadIdx.x & 31;
    const int groups = n_heads / heads_per_warp;
    const int64_t n_warps = ((int64_t)gridDim.x * blockDim.x) >> 5;
    // items (token, head group) are dealt round-robin to the warps of a grid that is resident all at once
#pragma unroll 1
    for (int64_t item = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5; item < T * groups; item += n_warps) {
    const int64_t t = item / groups;
    const int h_first = static_cast<int>(item % groups) * heads_per_warp;
    const int64_t row = t * ld + lane * E;

    float pe_v[E * 2];  // per pair: pe00, pe10, pe01, pe11  (ggml [row,col] = flat row + 2*col)
    if (pe != nullptr) {
        const float* pp = pe + ((tok_off + t) * (D / 2) + lane * (E / 2)) * 4;
#pragma unroll
        for (int p = 0; p < E / 2; ++p) {
            const float4 m = __ldg(reinterpret_cast<const float4*>(pp) + p);
            pe_v[4 * p + 0] = m.x;  // (row0,col0)
            pe_v[4 * p + 1] = m.y;  // (row1,col0)
            pe_v[4 * p + 2] = m.z;  // (row0,col1)
            pe_v[4 * p + 3] = m.w;  // (row1,col1)
        }
    }
    const bool need[3] = {!(peers.skip_mask & 1), !(peers.skip_mask & 2), !(peers.skip_mask & 4)};
    const int64_t offs[3] = {q_off, k_off, v_off};
    // per-token scale of a whole-row norm; per-head weights are fetched inside the loop, shared ones here
    float rs[2] = {1.0f, 1.0f};
    if (q_w != nullptr && peers.rstd_q != nullptr) rs[0] = __ldg(peers.rstd_q + t);
    if (k_w != nullptr && peers.rstd_k != nullptr) rs[1] = __ldg(peers.rstd_k + t);
    float wsh[2][E];
#pragma unroll
    for (int which = 0; which < 2; ++which) {
        const float* w = which == 0 ? q_w : k_w;
#pragma unroll
        for (int e = 0; e < E; ++e) wsh[which][e] = (w != nullptr && peers.w_head_stride == 0) ? __ldg(w + lane * E + e) : 1.0f;
    }

    auto fetch = [&](int h, Raw (&dst)[3]) {
#pragma unroll
        for (int which = 0; which < 3; ++which) {
            if (!need[which]) continue;   // uniform
            const int64_t off = row + offs[which] + (int64_t)h * D;
            if (IN16) {
                if (E == 4) {
                    *reinterpret_cast<uint2*>(&dst[which]) = *reinterpret_cast<const uint2*>(static_cast<const uint16_t*>(qkv) + off);
                } else {
                    reinterpret_cast<uint2*>(&dst[which])->x = *reinterpret_cast<const uint32_t*>(static_cast<const uint16_t*>(qkv) + off);
                }
            } else {
                if (E == 4) {
                    *reinterpret_cast<float4*>(&dst[which]) = *reinterpret_cast<const float4*>(static_cast<const float*>(qkv) + off);
                } else {
                    const float2 f = *reinterpret_cast<const float2*>(static_cast<const float*>(qkv) + off);
                    reinterpret_cast<float4*>(&dst[which])->x = f.x;
                    reinterpret_cast<float4*>(&dst[which])->y = f.y;
                }
            }
        }
    };
    auto widen = [&](const Raw& r, float (&v)[E]) {
        if (IN16) {
            const uint2& u = *reinterpret_cast<const uint2*>(&r);
            float2 lo, hi = make_float2(0.f, 0.f);
            if (in_dtype == EDB200_TYPE_BF16) {
                lo = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.x));
                if (E == 4) hi = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.y));
            } else {
                lo = __half22float2(*reinterpret_cast<const __half2*>(&u.x));
                if (E == 4) hi = __half22float2(*reinterpret_cast<const __half2*>(&u.y));
            }
            v[0] = lo.x, v[1] = lo.y;
            if (E == 4) v[E - 2] = hi.x, v[E - 1] = hi.y;
        } else {
            const float4& f = *reinterpret_cast<const float4*>(&r);
            v[0] = f.x, v[1] = f.y;
            if (E == 4) v[E - 2] = f.z, v[E - 1] = f.w;
        }
    };

    Raw ring[AHEAD + 1][3];
#pragma unroll
    for (int a = 0; a < AHEAD; ++a) {
        if (a < heads_per_warp) fetch(h_first + a, ring[a]);
    }
#pragma unroll 1
    for (int hh0 = 0; hh0 < heads_per_warp; hh0 += AHEAD + 1) {
#pragma unroll
        for (int slot = 0; slot < AHEAD + 1; ++slot) {   // ring slots are compile-time indices
            const int hh = hh0 + slot;
            if (hh >= heads_per_warp) break;   // uniform
            const int h = h_first + hh;
            if (hh + AHEAD < heads_per_warp) fetch(h + AHEAD, ring[(slot + AHEAD) % (AHEAD + 1)]);
            int64_t out_base = ((int64_t)h * L_total + tok_off + t) * D + lane * E;
            void* dsts[3] = {q_out, k_out, v_out};
            if (peers.hp > 0) {
                const int dst_rank = h / peers.hp;
                out_base = ((int64_t)(h % peers.hp) * L_total + peers.global_first + tok_off + t) * D + lane * E;
                dsts[0] = peers.q[dst_rank];
                dsts[1] = peers.k[dst_rank];
                dsts[2] = peers.v[dst_rank];
            }
#pragma unroll
            for (int which = 0; which < 3; ++which) {
                if (!need[which]) continue;   // uniform
                float v[E];
                widen(ring[slot][which], v);
                if (which < 2) {
                    const float* w = which == 0 ? q_w : k_w;
                    if (w != nullptr) {
                        float sc = rs[which];
                        if ((which == 0 ? peers.rstd_q : peers.rstd_k) == nullptr) {
                            float ss = 0.0f;
#pragma unroll
                            for (int e = 0; e < E; ++e) ss += v[e] * v[e];
                            ss = warp_sum(ss);
                            sc = 1.0f / sqrtf(ss / static_cast<float>(D) + eps);
                        }
                        if (peers.w_head_stride == 0) {
#pragma unroll
                            for (int e = 0; e < E; ++e) v[e] = (v[e] * sc) * wsh[which][e];
                        } else {
                            const float* wh = w + (int64_t)h * peers.w_head_stride + lane * E;
#pragma unroll
                            for (int e = 0; e < E; ++e) v[e] = (v[e] * sc) * __ldg(wh + e);
                        }
                    }
                    if (pe != nullptr) {
#pragma unroll
                        for (int p = 0; p < E / 2; ++p) {
                            const float x0 = v[2 * p], x1 = v[2 * p + 1];
                            v[2 * p] = __fadd_rn(__fmul_rn(x0, pe_v[4 * p + 0]), __fmul_rn(x1, pe_v[4 * p + 1]));
                            v[2 * p + 1] = __fadd_rn(__fmul_rn(x0, pe_v[4 * p + 2]), __fmul_rn(x1, pe_v[4 * p + 3]));
                        }
                    }
                }
                void* dst = dsts[which];
                if (E == 4) {
                    store_vec4(dst, out_dtype, out_base, v[0], v[1], v[E - 2], v[E - 1]);
                } else {
                    if (out_dtype == EDB200_TYPE_F32) {
                        *reinterpret_cast<float2*>(static_cast<float*>(dst) + out_base) = make_float2(v[0], v[1]);
                    } else if (out_dtype == EDB200_TYPE_BF16) {
                        *reinterpret_cast<__nv_bfloat162*>(static_cast<__nv_bfloat16*>(dst) + out_base) =
                            __floats2bfloat162_rn(v[0], v[1]);
                    } else {
                        *reinterpret_cast<__half2*>(static_cast<__half*>(dst) + out_base) = __floats2half2_rn(v[0], v[1]);
                    }
                }
            }
        }
    }
    }   // items
}

__global__ void cast_kernel(const void* __restrict__ x, int in_dtype, void* __restrict__ y, int out_dtype,
                            int64_t n4) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n4) return;
    const float4 v = load_vec4(x, in_dtype, 4 * i);
    store_vec4(y, out_dtype, 4 * i, v.x, v.y, v.z, v.w);
}

static bool dtype_ok(int dt) { return dt == EDB200_TYPE_F32 || dt == EDB200_TYPE_F16 || dt == EDB200_TYPE_BF16; }

}  // namespace edb

using namespace edb;

extern "C" {

edb200_status_t edb200_layernorm_modulate(const float* x, int64_t ldx, const float* shift, const float* scale,
                                          const float* ln_weight, const float* ln_bias, int64_t rows, int64_t h,
                                          float eps, void* y, int y_dtype, int64_t ldy, void* stream) {
    if (x == nullptr || y == nullptr || rows <= 0 || h <= 0) {
        return fail(EDB200_ERR_INVALID, "layernorm_modulate: null or empty argument");
    }
    if (h % 4 != 0 || h > 4 * LN_MAXV * LN_THREADS || ldx % 4 != 0 || ldy % 4 != 0 || !dtype_ok(y_dtype)) {
        return fail(EDB200_ERR_UNSUPPORTED, "layernorm_modulate: h must be a multiple of 4 and <= 8192");
    }
    ProfScope prof(static_cast<cudaStream_t>(stream), PROF_ELEMENTWISE, 0.0,
                   (double)rows * (double)h * (4.0 + (y_dtype == EDB200_TYPE_F32 ? 4.0 : 2.0)));
    const unsigned grid = static_cast<unsigned>(rows);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int hi = static_cast<int>(h);
    const int nv = (h % (4 * LN_THREADS) == 0) ? static_cast<int>(h / (4 * LN_THREADS)) : 0;
#define EDB_LN_LAUNCH(NVAL) \
    layernorm_modulate_kernel<NVAL><<<grid, LN_THREADS, 0, s>>>(x, ldx, shift, scale, ln_weight, ln_bias, hi, eps, y, y_dtype, ldy)
    switch (nv) {
        case 1: EDB_LN_LAUNCH(1); break;
        case 2: EDB_LN_LAUNCH(2); break;
        case 3: EDB_LN_LAUNCH(3); break;
        case 4: EDB_LN_LAUNCH(4); break;
        case 5: EDB_LN_LAUNCH(5); break;
        case 6: EDB_LN_LAUNCH(6); break;
        default: EDB_LN_LAUNCH(0); break;
    }
#undef EDB_LN_LAUNCH
    count_launch();
    return check_cuda(cudaGetLastError(), "layernorm_modulate launch");
}

edb200_status_t edb200_fused_modulate(const float* x, const float* shift, const float* scale, float* y, int64_t rows,
                                      int64_t h, void* stream) {
    if (x == nullptr || shift == nullptr || scale == nullptr || y == nullptr || rows <= 0 || h <= 0 || h % 4) {
        return fail(EDB200_ERR_INVALID, "fused_modulate: bad argument (h %% 4 == 0 required)");
    }
    const int64_t total4 = rows * h / 4;
    fused_modulate_kernel<<<static_cast<unsigned>((total4 + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        reinterpret_cast<const float4*>(x), reinterpret_cast<const float4*>(shift),
        reinterpret_cast<const float4*>(scale), reinterpret_cast<float4*>(y), total4, static_cast<int>(h / 4));
    count_launch();
    return check_cuda(cudaGetLastError(), "fused_modulate launch");
}

edb200_status_t edb200_fused_residual_gate(const float* residual, const float* x, const float* gate, float* y,
                                           int64_t rows, int64_t h, void* stream) {
    if (residual == nullptr || x == nullptr || gate == nullptr || y == nullptr || rows <= 0 || h <= 0 || h % 4) {
        return fail(EDB200_ERR_INVALID, "fused_residual_gate: bad argument (h %% 4 == 0 required)");
    }
    const int64_t total4 = rows * h / 4;
    fused_residual_gate_kernel<<<static_cast<unsigned>((total4 + 255) / 256), 256, 0,
                                 static_cast<cudaStream_t>(stream)>>>(
        reinterpret_cast<const float4*>(residual), reinterpret_cast<const float4*>(x),
        reinterpret_cast<const float4*>(gate), reinterpret_cast<float4*>(y), total4, static_cast<int>(h / 4));
    count_launch();
    return check_cuda(cudaGetLastError(), "fused_residual_gate launch");
}

edb200_status_t edb200_euler_update(float* x, const float* model_out, float sigma, float sigma_next, int64_t n,
                                    void* stream) {
    if (x == nullptr || model_out == nullptr || n <= 0) return fail(EDB200_ERR_INVALID, "euler_update: null or empty argument");
    euler_update_kernel<<<static_cast<unsigned>((n + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        x, model_out, sigma, sigma_next, nullptr, nullptr, n);
    count_launch();
    return check_cuda(cudaGetLastError(), "euler_update launch");
}

edb200_status_t edb200_flow_update(float* x, const float* model_out, float sigma, float sigma_next, int64_t n,
                                   void* stream) {
    if (x == nullptr || model_out == nullptr || n <= 0) return fail(EDB200_ERR_INVALID, "flow_update: null or empty argument");
    flow_update_kernel<<<static_cast<unsigned>((n + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        x, model_out, sigma_next - sigma, nullptr, nullptr, n);
    count_launch();
    return check_cuda(cudaGetLastError(), "flow_update launch");
}

edb200_status_t edb200_flow_update_sched(float* x, const float* model_out, const float* sigmas, int* step, int64_t n,
                                         void* stream) {
    if (x == nullptr || model_out == nullptr || sigmas == nullptr || step == nullptr || n <= 0) {
        return fail(EDB200_ERR_INVALID, "flow_update_sched: null or empty argument");
    }
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    flow_update_kernel<<<static_cast<unsigned>((n + 255) / 256), 256, 0, s>>>(x, model_out, 0.0f, sigmas, step, n);
    count_launch();
    advance_step_kernel<<<1, 1, 0, s>>>(step);   // after every thread above has read the old value (stream order)
    count_launch();
    return check_cuda(cudaGetLastError(), "flow_update_sched launch");
}

edb200_status_t edb200_sub_f32(const float* a, const float* b, float* out, int64_t n, void* stream) {
    if (a == nullptr || b == nullptr || out == nullptr || n <= 0 || n % 4) {
        return fail(EDB200_ERR_INVALID, "sub_f32: bad argument (n %% 4 == 0 required)");
    }
    sub_kernel<<<static_cast<unsigned>((n / 4 + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        reinterpret_cast<const float4*>(a), reinterpret_cast<const float4*>(b), reinterpret_cast<float4*>(out), n / 4);
    count_launch();
    return check_cuda(cudaGetLastError(), "sub_f32 launch");
}

edb200_status_t edb200_euler_update_sched(float* x, const float* model_out, const float* sigmas, int* step, int64_t n,
                                          void* stream) {
    if (x == nullptr || model_out == nullptr || sigmas == nullptr || step == nullptr || n <= 0) {
        return fail(EDB200_ERR_INVALID, "euler_update_sched: null or empty argument");
    }
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    euler_update_kernel<<<static_cast<unsigned>((n + 255) / 256), 256, 0, s>>>(x, model_out, 0.0f, 0.0f, sigmas, step, n);
    count_launch();
    advance_step_kernel<<<1, 1, 0, s>>>(step);   // after every thread above has read the old value (stream order)
    count_launch();
    return check_cuda(cudaGetLastError(), "euler_update_sched launch");
}

static edb200_status_t qk_pack_launch(const void* qkv, int in_dtype, int64_t ld, int64_t q_off, int64_t k_off,
                                      int64_t v_off, int64_t tokens, int n_heads, int d_head, const float* q_weight,
                                      const float* k_weight, float eps, const float* pe, int64_t tok_off,
                                      int64_t l_total, void* q_out, void* k_out, void* v_out, int out_dtype,
                                      const PackPeers& peers, void* stream) {
    const bool need[3] = {!(peers.skip_mask & 1), !(peers.skip_mask & 2), !(peers.skip_mask & 4)};
    if (qkv == nullptr || (need[0] && q_out == nullptr) || (need[1] && k_out == nullptr) ||
        (need[2] && v_out == nullptr) || tokens <= 0 || n_heads <= 0) {
        return fail(EDB200_ERR_INVALID, "qk_norm_rope_pack: null or empty argument");
    }
    if ((d_head != 64 && d_head != 128) || !dtype_ok(in_dtype) || !dtype_ok(out_dtype)) {
        return fail(EDB200_ERR_UNSUPPORTED, "qk_norm_rope_pack: d_head must be 64 or 128");
    }
    if (ld % 4 || q_off % 4 || k_off % 4 || v_off % 4 || tok_off < 0 ||
        peers.global_first + tok_off + tokens > l_total) {
        return fail(EDB200_ERR_INVALID, "qk_norm_rope_pack: offsets must be multiples of 4 and fit l_total");
    }
    // An item is one token x a group of at most 8 consecutive heads (more groups when tokens are few, so that
    // there are about 16 warps of work per SM); the grid is no larger than what is resident at once.
    int groups = 1;
    while (groups < n_heads &&
           (n_heads % groups != 0 || n_heads / groups > 8 || tokens * groups < (int64_t)sm_count() * 16)) {
        ++groups;
    }
    const int heads_per_warp = n_heads / groups;
    const int64_t items = tokens * groups;
    int64_t blocks = (items + 7) / 8;
    if (blocks > (int64_t)sm_count() * 3) blocks = (int64_t)sm_count() * 3;
    const unsigned grid = static_cast<unsigned>(blocks);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    ProfScope prof(s, PROF_ELEMENTWISE, 0.0,
                   (double)tokens * 3.0 * n_heads * d_head *
                       ((in_dtype == EDB200_TYPE_F32 ? 4.0 : 2.0) + (out_dtype == EDB200_TYPE_F32 ? 4.0 : 2.0)));
    const bool in16 = in_dtype != EDB200_TYPE_F32;
#define EDB_PACK_LAUNCH(DH, I16)                                                                                      \
    qk_norm_rope_pack_kernel<DH, I16><<<grid, 256, 0, s>>>(qkv, in_dtype, ld, q_off, k_off, v_off, tokens, n_heads,   \
                                                           heads_per_warp, q_weight, k_weight, eps, pe, tok_off,      \
                                                           l_total, q_out, k_out, v_out, out_dtype, peers)
    if (d_head == 128) {
        if (in16) EDB_PACK_LAUNCH(128, true); else EDB_PACK_LAUNCH(128, false);
    } else {
        if (in16) EDB_PACK_LAUNCH(64, true); else EDB_PACK_LAUNCH(64, false);
    }
#undef EDB_PACK_LAUNCH
    count_launch();
    return check_cuda(cudaGetLastError(), "qk_norm_rope_pack launch");
}

edb200_status_t edb200_qk_norm_rope_pack(const void* qkv, int in_dtype, int64_t ld, int64_t q_off, int64_t k_off,
                                         int64_t v_off, int64_t tokens, int n_heads, int d_head, const float* q_weight,
                                         const float* k_weight, float eps, const float* pe, int64_t tok_off,
                                         int64_t l_total, void* q_out, void* k_out, void* v_out, int out_dtype,
                                         void* stream) {
    PackPeers none;
    memset(&none, 0, sizeof(none));
    return qk_pack_launch(qkv, in_dtype, ld, q_off, k_off, v_off, tokens, n_heads, d_head, q_weight, k_weight, eps, pe,
                          tok_off, l_total, q_out, k_out, v_out, out_dtype, none, stream);
}

edb200_status_t edb200_qk_norm_rope_pack_sp(const void* qkv, int in_dtype, int64_t ld, int64_t q_off, int64_t k_off,
                                            int64_t v_off, int64_t tokens, int n_heads, int d_head,
                                            const float* q_weight, const float* k_weight, float eps, const float* pe,
                                            int64_t tok_off, int64_t l_total, const edb200_sp_peers_t* dst,
                                            int out_dtype, void* stream) {
    if (dst == nullptr || dst->world <= 0 || dst->world > 8 || dst->rank < 0 || dst->rank >= dst->world ||
        n_heads % dst->world || dst->t_loc <= 0) {
        return fail(EDB200_ERR_INVALID, "qk_norm_rope_pack_sp: bad peer description");
    }
    PackPeers pp;
    memset(&pp, 0, sizeof(pp));
    for (int r = 0; r < dst->world; ++r) {
        pp.q[r] = dst->buf[0][r];
        pp.k[r] = dst->buf[1][r];
        pp.v[r] = dst->buf[2][r];
        if (pp.q[r] == nullptr || pp.k[r] == nullptr || pp.v[r] == nullptr) {
            return fail(EDB200_ERR_INVALID, "qk_norm_rope_pack_sp: null peer buffer");
        }
    }
    pp.hp = n_heads / dst->world;
    pp.global_first = (long long)dst->rank * dst->t_loc;
    // the position table is addressed by tok_off + t of the local slice: shift it to the global rows
    const float* pe_g = pe ? pe + pp.global_first * (d_head / 2) * 4 : nullptr;
    return qk_pack_launch(qkv, in_dtype, ld, q_off, k_off, v_off, tokens, n_heads, d_head, q_weight, k_weight, eps,
                          pe_g, tok_off, l_total, pp.q[dst->rank], pp.k[dst->rank], pp.v[dst->rank], out_dtype, pp,
                          stream);
}

// rstd[row] = 1/sqrt(mean(x[row, :]^2) + eps); one warp per row, 16-byte loads.
__global__ void __launch_bounds__(256)
row_rstd_kernel(const void* __restrict__ x, int dtype, int64_t ld, int64_t rows, int cols, float eps,
                float* __restrict__ out) {
    const int64_t row = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (row >= rows) return;
    float ss = 0.0f;
    for (int c = lane * 4; c < cols; c += 128) {
        const float4 f = load_vec4(x, dtype, row * ld + c);
        ss += (f.x * f.x + f.y * f.y) + (f.z * f.z + f.w * f.w);
    }
    ss = warp_sum(ss);
    if (lane == 0) out[row] = 1.0f / sqrtf(ss / static_cast<float>(cols) + eps);
}

edb200_status_t edb200_row_rstd(const void* x, int dtype, int64_t ld, int64_t rows, int64_t cols, float eps, float* out,
                                void* stream) {
    if (x == nullptr || out == nullptr || rows <= 0 || cols <= 0 || cols % 4 || ld % 4 || !dtype_ok(dtype)) {
        return fail(EDB200_ERR_INVALID, "row_rstd: bad argument (cols and ld multiples of 4)");
    }
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    ProfScope prof(s, PROF_ELEMENTWISE, 0.0, (double)rows * cols * (dtype == EDB200_TYPE_F32 ? 4.0 : 2.0));
    row_rstd_kernel<<<static_cast<unsigned>((rows * 32 + 255) / 256), 256, 0, s>>>(x, dtype, ld, rows,
                                                                                   static_cast<int>(cols), eps, out);
    count_launch();
    return check_cuda(cudaGetLastError(), "row_rstd launch");
}

edb200_status_t edb200_qk_rownorm_rope_pack(const void* qkv, int in_dtype, int64_t ld, int64_t q_off, int64_t k_off,
                                            int64_t v_off, int64_t tokens, int n_heads, int d_head,
                                            const float* q_weight, const float* k_weight, const float* rstd_q,
                                            const float* rstd_k, const float* pe, int64_t tok_off, int64_t l_total,
                                            void* q_out, void* k_out, void* v_out, int out_dtype,
                                            const edb200_sp_peers_t* dst, void* stream) {
    PackPeers pp;
    memset(&pp, 0, sizeof(pp));
    pp.rstd_q = rstd_q;
    pp.rstd_k = rstd_k;
    pp.w_head_stride = d_head;
    if ((q_weight != nullptr && rstd_q == nullptr) || (k_weight != nullptr && rstd_k == nullptr)) {
        return fail(EDB200_ERR_INVALID, "qk_rownorm_rope_pack: a weight needs its row rstd");
    }
    const float* pe_g = pe;
    if (dst != nullptr) {
        if (dst->world <= 0 || dst->world > 8 || dst->rank < 0 || dst->rank >= dst->world || n_heads % dst->world ||
            dst->t_loc <= 0) {
            return fail(EDB200_ERR_INVALID, "qk_rownorm_rope_pack: bad peer description");
        }
        for (int r = 0; r < dst->world; ++r) {
            pp.q[r] = dst->buf[0][r];
            pp.k[r] = dst->buf[1][r];
            pp.v[r] = dst->buf[2][r];
        }
        pp.hp = n_heads / dst->world;
        pp.global_first = (long long)dst->rank * dst->t_loc;
        pe_g = pe ? pe + pp.global_first * (d_head / 2) * 4 : nullptr;
        q_out = pp.q[dst->rank], k_out = pp.k[dst->rank], v_out = pp.v[dst->rank];
    } else {
        pp.skip_mask = (q_out == nullptr ? 1 : 0) | (k_out == nullptr ? 2 : 0) | (v_out == nullptr ? 4 : 0);
    }
    return qk_pack_launch(qkv, in_dtype, ld, q_off, k_off, v_off, tokens, n_heads, d_head, q_weight, k_weight, 0.0f,
                          pe_g, tok_off, l_total, q_out, k_out, v_out, out_dtype, pp, stream);
}

edb200_status_t edb200_cast(const void* x, int in_dtype, void* y, int out_dtype, int64_t n, void* stream) {
    if (x == nullptr || y == nullptr || n <= 0 || n % 4 || !dtype_ok(in_dtype) || !dtype_ok(out_dtype)) {
        return fail(EDB200_ERR_INVALID, "cast: bad argument (n %% 4 == 0 required)");
    }
    cast_kernel<<<static_cast<unsigned>((n / 4 + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        x, in_dtype, y, out_dtype, n / 4);
    count_launch();
    return check_cuda(cudaGetLastError(), "cast launch");
}

}  // extern "C"
