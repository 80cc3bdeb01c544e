// Non-causal multi-head attention for sm_100a on tcgen05 / tensor memory.
//
//   O = softmax(Q K^T * scale) V      Q [HN, Lq, D], K/V [HN, Lk, D], D in {64, 128}
//
// Two variants of one kernel:
//   plain : f16 Q/K, kind::f16 QK^T  (stands in for ggml_flash_attn_ext / cuDNN SDPA,
//           reference src/core/backend/ggml/ggml_extend.hpp:1749-1984)
//   Sage  : INT8 Q/K (per-32-row / per-64-key scales, optional smooth-Q bias),
//           kind::i8 QK^T into s32 accumulators (reference
//           src/core/backend/ggml/cuda/sage/sage_qk_int_sv_f16_kernel.cuh:25-683)
// Both keep the softmax in f32 base 2, P in f16 and the PV product in kind::f16
// with f32 accumulation, V in f16 (as the reference feeds it).
//
// One CTA per (128-query tile, head); 640 threads, warp-specialised:
//   warp 0     TMA producer (Q once; K and V tiles of 128 keys, 2-stage rings)
//   warp 1     tcgen05.mma issuer: S_j = Q K_j^T into one of two S buffers in
//              tensor memory, O += P_j V_j
//   warp 2     tensor-memory allocator
//   warps 4-19 softmax: four threads per query row, each owning 32 score columns
//              (four warps per scheduler hide the dependent-issue latency a
//              single warp cannot); tcgen05.ld S, exp2, P -> shared memory
//              (128B-swizzled K-major operand), lazy rescale of O in tensor
//              memory (only when a row maximum grows by more than 2^8)
#include "edb200_internal.h"
#include "edb200_ptx.cuh"

namespace edb {
namespace attn {

constexpr int BQ = 128;   // query rows per CTA
constexpr int BKV = 128;  // keys per block
constexpr int KV_STAGES = 2;
constexpr int NSPLIT = 4;          // softmax threads per query row
constexpr int NUM_THREADS = 128 + NSPLIT * 128;
constexpr uint32_t TMEM_COLS = 512;
constexpr uint32_t TMEM_S0 = 0, TMEM_S1 = 128, TMEM_O = 256, TMEM_P = 384;
constexpr float kRescaleThreshold = 8.0f;  // log2(256)

struct Params {
    void* out;           // [Lq, ld_out] token-major, head hn at column hn*D
    long long ld_out;
    int out_dtype;
    int Lq, Lk, HN;
    float scale_log2;    // softmax scale * log2(e)
    // Sage only
    const float* q_scale;  // [HN, q_scale_stride]  one per 32 query rows
    const float* k_scale;  // [HN, k_scale_stride]  one per 64 keys
    const float* bias;     // [HN, bias_stride] f32 per key (smooth-Q) or NULL
    int q_scale_stride, k_scale_stride, bias_stride;
    int* err;
};

template <int D, bool SAGE>
struct Cfg {
    static constexpr int QK_ELEM = SAGE ? 1 : 2;
    static constexpr int Q_BYTES = BQ * D * QK_ELEM;
    static constexpr int K_BYTES = BKV * D * QK_ELEM;
    static constexpr int V_BYTES = BKV * D * 2;
    static constexpr int OFF_Q = 0;
    static constexpr int OFF_K = OFF_Q + Q_BYTES;
    static constexpr int OFF_V = OFF_K + KV_STAGES * K_BYTES;
    static constexpr int OFF_BAR = OFF_V + KV_STAGES * V_BYTES;
    static constexpr int OFF_XCH = OFF_BAR + 256;                  // row-maximum exchange [2][NSPLIT][BQ] f32
    static constexpr int SMEM_BYTES = OFF_XCH + 2 * NSPLIT * BQ * 4 + 1024;
    // Q/K panels: rows of 128 bytes (64 f16 or 128 int8); a tile is D*QK_ELEM/128 panels.
    static constexpr int QK_PANELS = D * QK_ELEM / 128;
    static constexpr int QK_PANEL_BYTES = 128 * 128;
    static constexpr int QK_KSTEPS = SAGE ? D / 32 : D / 16;   // 32 bytes of K per MMA either way
    static constexpr int V_PANELS = D / 64;
};

__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

__device__ __forceinline__ uint32_t pack_h2(float a, float b) {
    __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
}

template <int D, bool SAGE>
__global__ void __launch_bounds__(NUM_THREADS, 1)
attention_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                 const __grid_constant__ CUtensorMap map_v, const __grid_constant__ Params P) {
    using C = Cfg<D, SAGE>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::OFF_BAR);
    uint64_t* q_full = bars;                 // [1]
    uint64_t* k_full = q_full + 1;           // [2]
    uint64_t* k_empty = k_full + KV_STAGES;  // [2]
    uint64_t* v_full = k_empty + KV_STAGES;  // [2]
    uint64_t* v_empty = v_full + KV_STAGES;  // [2]
    uint64_t* s_full = v_empty + KV_STAGES;  // [2]
    uint64_t* s_empty = s_full + 2;          // [2]
    uint64_t* p_full = s_empty + 2;          // [1]
    uint64_t* pv_done = p_full + 1;          // [1]
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(pv_done + 1);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int q0 = blockIdx.x * BQ;
    const int hn = blockIdx.y;
    const int n_kv = (P.Lk + BKV - 1) / BKV;

    if (threadIdx.x == 0) {
        mbar_init(q_full, 1);
        for (int i = 0; i < KV_STAGES; ++i) {
            mbar_init(&k_full[i], 1);
            mbar_init(&k_empty[i], 1);
            mbar_init(&v_full[i], 1);
            mbar_init(&v_empty[i], 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(&s_full[i], 1);
            mbar_init(&s_empty[i], 4 * NSPLIT);
        }
        mbar_init(p_full, 4 * NSPLIT);
        mbar_init(pv_done, 1);
        *abort_flag = 0;
        fence_mbar_init();
    }
    if (warp == 2) {
        tmem_alloc(tmem_slot, TMEM_COLS);
        tmem_relinquish();
    }
    if (warp == 0 && lane == 0) {
        tma_prefetch_desc(&map_q);
        tma_prefetch_desc(&map_k);
        tma_prefetch_desc(&map_v);
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ------------------------------------------------------ TMA producer
        if (lane == 0) {
            mbar_arrive_expect_tx(q_full, C::Q_BYTES);
#pragma unroll
            for (int p = 0; p < C::QK_PANELS; ++p) {
                tma_load_3d(smem + C::OFF_Q + p * C::QK_PANEL_BYTES, &map_q, q_full, p * (128 / C::QK_ELEM), q0, hn);
            }
            for (int j = 0; j < n_kv; ++j) {
                const int st = j % KV_STAGES;
                const uint32_t ph = (j / KV_STAGES) & 1;
                if (!mbar_wait(&k_empty[st], ph ^ 1u, abort_flag, P.err)) break;
                mbar_arrive_expect_tx(&k_full[st], C::K_BYTES);
#pragma unroll
                for (int p = 0; p < C::QK_PANELS; ++p) {
                    tma_load_3d(smem + C::OFF_K + st * C::K_BYTES + p * C::QK_PANEL_BYTES, &map_k, &k_full[st],
                                p * (128 / C::QK_ELEM), j * BKV, hn);
                }
                if (!mbar_wait(&v_empty[st], ph ^ 1u, abort_flag, P.err)) break;
                mbar_arrive_expect_tx(&v_full[st], C::V_BYTES);
#pragma unroll
                for (int p = 0; p < C::V_PANELS; ++p) {
                    tma_load_3d(smem + C::OFF_V + st * C::V_BYTES + p * (BKV * 128), &map_v, &v_full[st], p * 64,
                                j * BKV, hn);
                }
            }
        }
    } else if (warp == 1) {
        // -------------------------------------------------------- MMA issuer
        const uint32_t idesc_qk = SAGE ? make_idesc(kDFmtS32, kFmtS8, kFmtS8, 0, 0, BQ, BKV)
                                       : make_idesc(kDFmtF32, kFmtF16, kFmtF16, 0, 0, BQ, BKV);
        const uint32_t idesc_pv = make_idesc(kDFmtF32, kFmtF16, kFmtF16, 0, 1, BQ, D);
        const uint32_t q_addr = smem_u32(smem + C::OFF_Q);
        bool ok = mbar_wait(q_full, 0, abort_flag, P.err);

        auto issue_qk = [&](int j) -> bool {
            const int st = j % KV_STAGES;
            const uint32_t kph = (j / KV_STAGES) & 1;
            const int sb = j & 1;
            const uint32_t sph = (j >> 1) & 1;
            if (!mbar_wait(&k_full[st], kph, abort_flag, P.err)) return false;
            if (!mbar_wait(&s_empty[sb], sph ^ 1u, abort_flag, P.err)) return false;
            tc_fence_after_sync();
            if (elect_one()) {
                const uint32_t k_addr = smem_u32(smem + C::OFF_K + st * C::K_BYTES);
                const uint32_t tmem_s = tmem_base + (sb ? TMEM_S1 : TMEM_S0);
#pragma unroll
                for (int ks = 0; ks < C::QK_KSTEPS; ++ks) {
                    const uint32_t off = (ks / 4) * C::QK_PANEL_BYTES + (ks % 4) * 32;
                    const uint64_t ad = make_smem_desc_sw128(q_addr + off, 16, 1024);
                    const uint64_t bd = make_smem_desc_sw128(k_addr + off, 16, 1024);
                    if (SAGE) {
                        mma_i8_ss(tmem_s, ad, bd, idesc_qk, ks > 0 ? 1u : 0u);
                    } else {
                        mma_f16_ss(tmem_s, ad, bd, idesc_qk, ks > 0 ? 1u : 0u);
                    }
                }
                mma_commit(&s_full[sb]);
                mma_commit(&k_empty[st]);
            }
            __syncwarp();
            return true;
        };

        if (ok) ok = issue_qk(0);
        for (int j = 0; ok && j < n_kv; ++j) {
            if (j + 1 < n_kv) {
                if (!issue_qk(j + 1)) break;
            }
            const int st = j % KV_STAGES;
            const uint32_t vph = (j / KV_STAGES) & 1;
            if (!mbar_wait(&v_full[st], vph, abort_flag, P.err) ||
                !mbar_wait(p_full, static_cast<uint32_t>(j & 1), abort_flag, P.err)) {
                break;
            }
            tc_fence_after_sync();
            if (elect_one()) {
                const uint32_t v_addr = smem_u32(smem + C::OFF_V + st * C::V_BYTES);
#pragma unroll
                for (int ks = 0; ks < BKV / 16; ++ks) {
                    // P: tensor memory, 8 columns (16 keys) per step; V: MN-major, 16 keys = 2 KB per step
                    const uint64_t bd = make_smem_desc_sw128(v_addr + ks * 2048, BKV * 128, 1024);
                    mma_f16_ts(tmem_base + TMEM_O, tmem_base + TMEM_P + ks * 8, bd, idesc_pv, (j > 0 || ks > 0) ? 1u : 0u);
                }
                mma_commit(pv_done);
                mma_commit(&v_empty[st]);
            }
            __syncwarp();
        }
    } else if (warp >= 4) {
        // ------------------------------------------------------------ softmax
        // NSPLIT threads share one query row: thread `split` owns score columns
        // [split*CW, split*CW+CW) and output columns [split*OW, split*OW+OW).  The
        // row maximum is exchanged through shared memory behind a named barrier
        // per lane quarter, so every thread of a row takes the same rescale decision.
        constexpr int CW = BKV / NSPLIT;
        constexpr int OW = D / NSPLIT;
        const int quarter = warp & 3;
        const int split = (warp - 4) >> 2;
        const int r = quarter * 32 + lane;          // row inside the tile
        const int q_row = q0 + r;
        const uint32_t lane_base = static_cast<uint32_t>(quarter * 32) << 16;
        float* xch = reinterpret_cast<float*>(smem + C::OFF_XCH);   // [2][NSPLIT][BQ]
        float m_used = -INFINITY;
        float l_sum = 0.0f;
        float row_scale = P.scale_log2;
        const float* bias_row = nullptr;
        if (SAGE) {
            row_scale *= P.q_scale[(long long)hn * P.q_scale_stride + (q0 >> 5) + quarter];
            if (P.bias != nullptr) bias_row = P.bias + (long long)hn * P.bias_stride + split * CW;
        }
        bool ok = true;

        for (int j = 0; j < n_kv; ++j) {
            // After an abort every wait returns false at once; the loop still runs to
            // the end so that all threads of a row group meet at the named barrier.
            const int sb = j & 1;
            ok = mbar_wait(&s_full[sb], static_cast<uint32_t>((j >> 1) & 1), abort_flag, P.err) && ok;
            tc_fence_after_sync();
            float s[CW];
            {
                const uint32_t taddr = tmem_base + lane_base + (sb ? TMEM_S1 : TMEM_S0) + split * CW;
                uint32_t rr[CW];
                tmem_ld_cols<CW>(taddr, rr);
                tmem_wait_ld();
#pragma unroll
                for (int i = 0; i < CW; ++i) s[i] = __uint_as_float(rr[i]);
            }
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(&s_empty[sb]);

            // scores in the log2 domain
            const int valid = P.Lk - j * BKV - split * CW;  // own columns >= valid are padding
            if (SAGE) {
                const float ks = P.k_scale[(long long)hn * P.k_scale_stride + 2 * j + (split * CW >= 64 ? 1 : 0)];
                const float c0 = row_scale * ks;
                // s32 -> f32 without a conversion instruction (valid for |s| < 2^22):
                // as_float(s + 0x4B400000) = 12582912 + s exactly.
                if (bias_row != nullptr) {
                    const float4* b4 = reinterpret_cast<const float4*>(bias_row + j * BKV);
#pragma unroll
                    for (int i = 0; i < CW / 4; ++i) {
                        const float4 b = __ldg(b4 + i);
                        const float bb[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const float f = __int_as_float(__float_as_int(s[4 * i + e]) + 0x4B400000) - 12582912.0f;
                            s[4 * i + e] = fmaf(f, c0, bb[e] * P.scale_log2);
                        }
                    }
                } else {
#pragma unroll
                    for (int i = 0; i < CW; ++i) {
                        const float f = __int_as_float(__float_as_int(s[i]) + 0x4B400000) - 12582912.0f;
                        s[i] = f * c0;
                    }
                }
            } else {
#pragma unroll
                for (int i = 0; i < CW; ++i) s[i] *= row_scale;
            }
            if (valid < CW) {
#pragma unroll
                for (int i = 0; i < CW; ++i) {
                    if (i >= valid) s[i] = -INFINITY;
                }
            }
            float mx4[4] = {s[0], s[1], s[2], s[3]};
#pragma unroll
            for (int i = 4; i < CW; ++i) mx4[i & 3] = fmaxf(mx4[i & 3], s[i]);
            float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
            if (NSPLIT > 1) {
                float* xb = xch + (j & 1) * (NSPLIT * BQ);
                xb[split * BQ + r] = mx;
                named_bar_sync(1 + quarter, NSPLIT * 32);
#pragma unroll
                for (int sp = 0; sp < NSPLIT; ++sp) mx = fmaxf(mx, xb[sp * BQ + r]);
            }

            // lazy rescale: keep exponentiating against the old maximum until it is stale by > 2^8
            float alpha = 1.0f;
            const bool grow = mx > m_used + kRescaleThreshold;
            if (grow) {
                alpha = ex2(m_used - mx);   // 0 on the first block (m_used = -inf)
                m_used = mx;
                l_sum *= alpha;
            }
            uint32_t p2[CW / 2];
            float part[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int i = 0; i < CW / 2; ++i) {
                const float a = ex2(s[2 * i] - m_used);
                const float b = ex2(s[2 * i + 1] - m_used);
                part[i & 3] += a + b;
                p2[i] = pack_h2(a, b);
            }
            l_sum += (part[0] + part[1]) + (part[2] + part[3]);

            // P buffer and O are free once the previous PV product has completed
            if (j > 0) {
                ok = mbar_wait(pv_done, static_cast<uint32_t>((j - 1) & 1), abort_flag, P.err) && ok;
                tc_fence_after_sync();
                if (__any_sync(0xffffffffu, grow)) {
                    const uint32_t oaddr = tmem_base + lane_base + TMEM_O + split * OW;
                    uint32_t rr[OW];
                    tmem_ld_cols<OW>(oaddr, rr);
                    tmem_wait_ld();
#pragma unroll
                    for (int i = 0; i < OW; ++i) rr[i] = __float_as_uint(__uint_as_float(rr[i]) * alpha);
                    tmem_st_cols<OW>(oaddr, rr);
                    tmem_wait_st();
                }
            }
            // P (f16 pairs, two keys per 32-bit column) goes to tensor memory as the A operand of PV
            tmem_st_cols<CW / 2>(tmem_base + lane_base + TMEM_P + split * (CW / 2), p2);
            tmem_wait_st();
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(p_full);
        }

        // ----------------------------------------------------------- epilogue
        if (NSPLIT > 1) {
            // row sum = fixed-order sum of the NSPLIT partial sums (all scaled by the same alphas)
            float* xb = xch + (n_kv & 1) * (NSPLIT * BQ);
            xb[split * BQ + r] = l_sum;
            named_bar_sync(1 + quarter, NSPLIT * 32);
            l_sum = 0.0f;
#pragma unroll
            for (int sp = 0; sp < NSPLIT; ++sp) l_sum += xb[sp * BQ + r];
        }
        ok = mbar_wait(pv_done, static_cast<uint32_t>((n_kv - 1) & 1), abort_flag, P.err) && ok;
        if (ok) {
            tc_fence_after_sync();
            const float inv_l = 1.0f / l_sum;
            const uint32_t oaddr = tmem_base + lane_base + TMEM_O + split * OW;
            const bool row_ok = q_row < P.Lq;
            char* obase = static_cast<char*>(P.out);
            const long long ocol = (long long)q_row * P.ld_out + (long long)hn * D + split * OW;
            uint32_t rr[OW];
            tmem_ld_cols<OW>(oaddr, rr);
            tmem_wait_ld();
            if (row_ok) {
                float v[OW];
#pragma unroll
                for (int i = 0; i < OW; ++i) v[i] = __uint_as_float(rr[i]) * inv_l;
                if (P.out_dtype == EDB200_TYPE_F32) {
                    float4* o = reinterpret_cast<float4*>(obase + ocol * 4);
#pragma unroll
                    for (int i = 0; i < OW / 4; ++i) o[i] = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
                } else {
                    uint4* o = reinterpret_cast<uint4*>(obase + ocol * 2);
                    const bool bf = P.out_dtype == EDB200_TYPE_BF16;
#pragma unroll
                    for (int i = 0; i < OW / 8; ++i) {
                        uint32_t u[4];
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            if (bf) {
                                __nv_bfloat162 h = __floats2bfloat162_rn(v[8 * i + 2 * e], v[8 * i + 2 * e + 1]);
                                u[e] = *reinterpret_cast<uint32_t*>(&h);
                            } else {
                                u[e] = pack_h2(v[8 * i + 2 * e], v[8 * i + 2 * e + 1]);
                            }
                        }
                        o[i] = make_uint4(u[0], u[1], u[2], u[3]);
                    }
                }
            }
        }
    }

    tc_fence_before_sync();
    __syncthreads();
    if (*abort_flag) {
        for (int i = 0; i < 200; ++i) __nanosleep(1000);
        __syncthreads();
    }
    if (warp == 2) {
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, TMEM_COLS);
    }
}

template <int D, bool SAGE>
static edb200_status_t launch(const void* q, const void* k, const void* v, const Params& P, cudaStream_t stream) {
    using C = Cfg<D, SAGE>;
    CUtensorMap mq, mk, mv;
    const CUtensorMapDataType qk_dt = SAGE ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    const int es = C::QK_ELEM;
    const uint32_t box_inner = 128 / es;
    edb200_status_t st = make_tmap_3d(&mq, qk_dt, es, q, D, P.Lq, P.HN, (uint64_t)D * es, (uint64_t)P.Lq * D * es,
                                      box_inner, BQ, 1, CU_TENSOR_MAP_SWIZZLE_128B);
    if (st != EDB200_OK) return st;
    st = make_tmap_3d(&mk, qk_dt, es, k, D, P.Lk, P.HN, (uint64_t)D * es, (uint64_t)P.Lk * D * es, box_inner, BKV, 1,
                      CU_TENSOR_MAP_SWIZZLE_128B);
    if (st != EDB200_OK) return st;
    st = make_tmap_3d(&mv, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, v, D, P.Lk, P.HN, (uint64_t)D * 2,
                      (uint64_t)P.Lk * D * 2, 64, BKV, 1, CU_TENSOR_MAP_SWIZZLE_128B);
    if (st != EDB200_OK) return st;
    auto kern = attention_kernel<D, SAGE>;
    static bool attr_set = false;
    if (!attr_set) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES);
        if (e != cudaSuccess) return check_cuda(e, "cudaFuncSetAttribute(attention)");
        attr_set = true;
    }
    dim3 grid((P.Lq + BQ - 1) / BQ, P.HN);
    ProfScope prof(stream, PROF_ATTENTION, 4.0 * (double)P.Lq * (double)P.Lk * D * P.HN,
                   (double)P.HN * D * ((double)P.Lq * (C::QK_ELEM + 2) + (double)P.Lk * (C::QK_ELEM + 2)));
    kern<<<grid, NUM_THREADS, C::SMEM_BYTES, stream>>>(mq, mk, mv, P);
    count_launch();
    return check_cuda(cudaGetLastError(), "attention launch");
}

}  // namespace attn
}  // namespace edb

using namespace edb;

extern "C" {

edb200_status_t edb200_attention_f16(const void* q, const void* k, const void* v, int hn, int64_t lq, int64_t lk,
                                     int d_head, float scale, void* out, int out_dtype, int64_t ld_out,
                                     void* stream) {
    if (q == nullptr || k == nullptr || v == nullptr || out == nullptr || hn <= 0 || lq <= 0 || lk <= 0) {
        return fail(EDB200_ERR_INVALID, "attention_f16: null or empty argument");
    }
    if (d_head != 64 && d_head != 128) return fail(EDB200_ERR_UNSUPPORTED, "attention_f16: d_head must be 64 or 128");
    if (out_dtype != EDB200_TYPE_F32 && out_dtype != EDB200_TYPE_F16 && out_dtype != EDB200_TYPE_BF16) {
        return fail(EDB200_ERR_INVALID, "attention_f16: bad out_dtype");
    }
    const int esz = out_dtype == EDB200_TYPE_F32 ? 4 : 2;
    if (ld_out < (int64_t)hn * d_head || (ld_out * esz) % 16 != 0 || (reinterpret_cast<uintptr_t>(out) & 15u)) {
        return fail(EDB200_ERR_INVALID, "attention_f16: out rows must be 16-byte aligned and ld_out >= hn*d_head");
    }
    int* err = device_error_word();
    if (err == nullptr) return fail(EDB200_ERR_CUDA, "attention_f16: no CUDA device");
    attn::Params P;
    memset(&P, 0, sizeof(P));
    P.out = out;
    P.ld_out = ld_out;
    P.out_dtype = out_dtype;
    P.Lq = static_cast<int>(lq);
    P.Lk = static_cast<int>(lk);
    P.HN = hn;
    P.scale_log2 = scale * 1.4426950408889634f;
    P.err = err;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (d_head == 128) return attn::launch<128, false>(q, k, v, P, s);
    return attn::launch<64, false>(q, k, v, P, s);
}

edb200_status_t edb200_attention_sage_int8(const void* q_i8, const void* k_i8, const void* v_f16,
                                           const float* q_scale, int q_scale_stride, const float* k_scale,
                                           int k_scale_stride, const float* bias, int bias_stride, int hn, int64_t l,
                                           int d_head, float scale, void* out, int out_dtype, int64_t ld_out,
                                           void* stream) {
    if (q_i8 == nullptr || k_i8 == nullptr || v_f16 == nullptr || q_scale == nullptr || k_scale == nullptr ||
        out == nullptr || hn <= 0 || l <= 0) {
        return fail(EDB200_ERR_INVALID, "attention_sage_int8: null or empty argument");
    }
    if (d_head != 128) return fail(EDB200_ERR_UNSUPPORTED, "attention_sage_int8: d_head must be 128");
    const int esz = out_dtype == EDB200_TYPE_F32 ? 4 : 2;
    if (ld_out < (int64_t)hn * d_head || (ld_out * esz) % 16 != 0 || (reinterpret_cast<uintptr_t>(out) & 15u)) {
        return fail(EDB200_ERR_INVALID, "attention_sage_int8: out rows must be 16-byte aligned");
    }
    const int64_t lpad = (l + 127) / 128 * 128;
    if (q_scale_stride < lpad / 32 || k_scale_stride < lpad / 64 || (bias != nullptr && bias_stride < lpad) ||
        (bias != nullptr && ((bias_stride % 4) || (reinterpret_cast<uintptr_t>(bias) & 15u)))) {
        return fail(EDB200_ERR_INVALID, "attention_sage_int8: scale / bias rows must cover l rounded up to 128");
    }
    int* err = device_error_word();
    if (err == nullptr) return fail(EDB200_ERR_CUDA, "attention_sage_int8: no CUDA device");
    attn::Params P;
    memset(&P, 0, sizeof(P));
    P.out = out;
    P.ld_out = ld_out;
    P.out_dtype = out_dtype;
    P.Lq = P.Lk = static_cast<int>(l);
    P.HN = hn;
    P.scale_log2 = scale * 1.4426950408889634f;
    P.q_scale = q_scale;
    P.k_scale = k_scale;
    P.bias = bias;
    P.q_scale_stride = q_scale_stride;
    P.k_scale_stride = k_scale_stride;
    P.bias_stride = bias_stride;
    P.err = err;
    return attn::launch<128, true>(q_i8, k_i8, v_f16, P, static_cast<cudaStream_t>(stream));
}

}  // extern "C"
