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
// One CTA per (256-query slab, head): two 128-row query tiles share every K/V tile
// that is fetched.  The exponentials bound this kernel (16 ex2 per clock per SM:
// 1024 clocks for a 128 x 128 score tile, as long as its two f16 products), so
// the design keeps the softmax threads busy all the time.  384 threads,
// warp-specialised:
//   warp 0      TMA producer (both Q tiles once; K and V tiles of 128 keys, 2-stage
//               rings; with a smooth-Q bias its 512-byte row piece per key tile)
//   warp 1      tcgen05.mma issuer (elect.sync).  Scores are produced per 64-key
//               half g into buffer g % 2 of the tile's 128 S columns; per half and
//               query tile t:  O_t += P_t[g] V_g,  then  S_t[g + 2] = Q_t K_{g+2}^T
//   warp 2      tensor-memory allocator
//   warps 4-7   softmax of query tile 0: one thread per query row owns all 64 scores
//               of the half (no cross-thread exchange), tcgen05.ld, packed f32x2
//               arithmetic, exp2, P as f16 pairs back over the first 32 columns of
//               the buffer just read (tcgen05.st), where the PV product reads it as
//               its A operand
//   warps 8-11  the same for query tile 1
// Tensor memory: S0 | S1 | O0 | O1, 128 columns each.  The tensor pipe executes in
// issue order, so S_t[g + 2] may overwrite the buffer once O_t += P_t[g] V_g has been
// issued.  O_t is rescaled in place, after the tile's last PV product has completed,
// only when a row maximum grows by more than 2^8.
#include "edb200_internal.h"
#include "edb200_ptx.cuh"

#include <cstdlib>

namespace edb {
namespace attn {

constexpr int BQ = 128;   // query rows per tile (two tiles per CTA)
constexpr int QT = 2;     // query tiles per CTA
constexpr int BKV = 128;  // keys per K/V tile in shared memory
constexpr int HK = 64;    // keys per softmax step (half a tile): S is double-buffered per query tile
constexpr int KV_STAGES = 2;
constexpr int BIAS_STAGES = 4;      // smooth-Q bias ring (one 512-byte row piece per key block)
constexpr int NUM_THREADS = 128 + QT * 128;
constexpr uint32_t TMEM_COLS = 512;
constexpr uint32_t TMEM_S = 0, TMEM_O = 256;       // + tile * 128
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
    // Sequence-parallel output (t_loc > 0): query row r belongs to rank r / t_loc and is
    // stored into that rank's buffer (peer-mapped) at row r % t_loc; `out` is unused.
    void* out_peer[8];
    int t_loc;
    int one;   // always 1: an operand the compiler cannot fold (see magic_i2f_biased)
    int qt;    // query tiles per CTA: 2, or 1 when two would leave SMs without a CTA
    // Mixed schedule (n_mixed_two >= 0; the grid is then 1-D): the first n_mixed_two CTAs take two-tile slabs in
    // (head, slab) order, the CTAs after them the remaining slabs one tile each - the last, partial wave of
    // two-tile CTAs becomes a wave of one-tile CTAs, which finish in about two thirds of the time.
    int n_mixed_two;
    int slabs2;   // two-tile slabs per head
};

template <int D, bool SAGE>
struct Cfg {
    static constexpr int QK_ELEM = SAGE ? 1 : 2;
    static constexpr int Q_BYTES = BQ * D * QK_ELEM;      // one query tile
    static constexpr int K_BYTES = BKV * D * QK_ELEM;
    static constexpr int V_BYTES = BKV * D * 2;
    static constexpr int OFF_Q = 0;
    static constexpr int OFF_K = OFF_Q + QT * Q_BYTES;
    static constexpr int OFF_V = OFF_K + KV_STAGES * K_BYTES;
    static constexpr int OFF_BAR = OFF_V + KV_STAGES * V_BYTES;
    static constexpr int OFF_BIAS = OFF_BAR + 256;
    static constexpr int SMEM_BYTES = OFF_BIAS + BIAS_STAGES * BKV * 4 + 1024;
    // Q/K panels: rows of QK_ROW_BYTES (128: 64 f16 or 128 int8; 64: the 64 int8 of a 64-wide head, which
    // takes the 64-byte swizzle); a tile is D*QK_ELEM/QK_ROW_BYTES panels.
    static constexpr int QK_ROW_BYTES = D * QK_ELEM < 128 ? D * QK_ELEM : 128;
    static constexpr int QK_PANELS = D * QK_ELEM / QK_ROW_BYTES;
    static constexpr int QK_PANEL_BYTES = 128 * QK_ROW_BYTES;
    static constexpr int QK_KSTEPS = SAGE ? D / 32 : D / 16;   // 32 bytes of K per MMA either way
    static constexpr int QK_KSTEPS_PER_PANEL = QK_ROW_BYTES / 32;
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

// Two f32 operations per instruction (sm_100 packed f32x2 pipe).
__device__ __forceinline__ void fma2(float& d0, float& d1, float a0, float a1, float b0, float b1, float c0, float c1) {
    asm("{\n .reg .b64 a, b, c, d;\n mov.b64 a, {%2, %3};\n mov.b64 b, {%4, %5};\n mov.b64 c, {%6, %7};\n"
        " fma.rn.f32x2 d, a, b, c;\n mov.b64 {%0, %1}, d;\n}"
        : "=f"(d0), "=f"(d1)
        : "f"(a0), "f"(a1), "f"(b0), "f"(b1), "f"(c0), "f"(c1));
}
__device__ __forceinline__ void add2(float& d0, float& d1, float a0, float a1, float b0, float b1) {
    asm("{\n .reg .b64 a, b, d;\n mov.b64 a, {%2, %3};\n mov.b64 b, {%4, %5};\n"
        " add.rn.f32x2 d, a, b;\n mov.b64 {%0, %1}, d;\n}"
        : "=f"(d0), "=f"(d1)
        : "f"(a0), "f"(a1), "f"(b0), "f"(b1));
}
__device__ __forceinline__ void mul2(float& d0, float& d1, float a0, float a1, float b0, float b1) {
    asm("{\n .reg .b64 a, b, d;\n mov.b64 a, {%2, %3};\n mov.b64 b, {%4, %5};\n"
        " mul.rn.f32x2 d, a, b;\n mov.b64 {%0, %1}, d;\n}"
        : "=f"(d0), "=f"(d1)
        : "f"(a0), "f"(a1), "f"(b0), "f"(b1));
}

// s32 -> f32 without a conversion instruction (valid for |s| < 2^22):
// as_float(s + 0x4B400000) = 12582912 + s exactly.
constexpr int kMagicInt = 0x4B400000;
constexpr float kMagicFloat = 12582912.0f;

__device__ __forceinline__ float max3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}

// s32 dot product -> f32 (valid for |s| < 2^22): as_float(s + 0x4B400000) = 12582912 + s
// exactly.  The add is written as a multiply-add by a run-time 1 so that it issues on the
// FMA pipe, which has twice the integer-add pipe's rate and is the less loaded one here.
__device__ __forceinline__ float magic_i2f_biased(uint32_t s, int one) {
    int r;
    asm("mad.lo.s32 %0, %1, %2, %3;" : "=r"(r) : "r"(static_cast<int>(s)), "r"(one), "r"(kMagicInt));
    return __int_as_float(r);
}

// Half a score row (64 columns, raw tensor-memory words) -> maximum of the scaled scores (log2
// domain).  MASKED: only the first `valid` columns are real keys.  The words are not changed.
// Only the first half of a row, a ragged last half and halves whose scores outgrow the running
// maximum take this sweep (see the softmax loop).
template <bool SAGE, bool MASKED>
__device__ __forceinline__ float half_row_max(const uint32_t (&rr)[64], float c0, float cq, const float4* bias, float sl2,
                                              int valid, int one) {
    if (SAGE && bias == nullptr) {
        int mi[4] = {INT_MIN, INT_MIN, INT_MIN, INT_MIN};
#pragma unroll
        for (int i = 0; i < 64; ++i) {
            if (!MASKED || i < valid) mi[i & 3] = max(mi[i & 3], static_cast<int>(rr[i]));
        }
        const int m = max(max(mi[0], mi[1]), max(mi[2], mi[3]));
        return m == INT_MIN ? -INFINITY : static_cast<float>(m) * c0;   // c0 > 0
    }
    float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
    if (SAGE) {
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            const float4 b = bias[i];   // shared memory, same address in every lane
            float f0 = magic_i2f_biased(rr[4 * i + 0], one);
            float f1 = magic_i2f_biased(rr[4 * i + 1], one);
            float f2 = magic_i2f_biased(rr[4 * i + 2], one);
            float f3 = magic_i2f_biased(rr[4 * i + 3], one);
            add2(f0, f1, f0, f1, -kMagicFloat, -kMagicFloat);
            add2(f2, f3, f2, f3, -kMagicFloat, -kMagicFloat);
            fma2(f0, f1, f0, f1, cq, cq, b.x, b.y);
            fma2(f2, f3, f2, f3, cq, cq, b.z, b.w);
            if (MASKED) {
                if (4 * i + 0 >= valid) f0 = -INFINITY;
                if (4 * i + 1 >= valid) f1 = -INFINITY;
                if (4 * i + 2 >= valid) f2 = -INFINITY;
                if (4 * i + 3 >= valid) f3 = -INFINITY;
            }
            mx[i & 1] = max3(mx[i & 1], f0, f1);
            mx[2 + (i & 1)] = max3(mx[2 + (i & 1)], f2, f3);
        }
        return fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3])) * sl2;   // sl2 > 0
    } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) {
            float f0 = __uint_as_float(rr[2 * i]), f1 = __uint_as_float(rr[2 * i + 1]);
            if (MASKED) {
                if (2 * i + 0 >= valid) f0 = -INFINITY;
                if (2 * i + 1 >= valid) f1 = -INFINITY;
            }
            mx[i & 3] = max3(mx[i & 3], f0, f1);
        }
        return fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3])) * c0;   // c0 > 0
    }
}

// exp2 of two non-positive-ish arguments (<= 8 by the lazy-rescale rule) on the FMA
// pipe: round to nearest integer with the 1.5 * 2^23 trick, degree-3 polynomial of
// 2^f on [-0.5, 0.5] (relative error 7.5e-5, below the f16 rounding of P), integer
// part added into the exponent field.  Relieves the 16-per-clock-per-SM ex2 unit.
__device__ __forceinline__ void ex2_poly2(float e0, float e1, float& a, float& b) {
    e0 = fmaxf(e0, -126.0f);
    e1 = fmaxf(e1, -126.0f);
    float r0, r1, x0, x1, f0, f1, p0, p1;
    add2(r0, r1, e0, e1, kMagicFloat, kMagicFloat);
    add2(x0, x1, r0, r1, -kMagicFloat, -kMagicFloat);
    fma2(f0, f1, x0, x1, -1.0f, -1.0f, e0, e1);
    fma2(p0, p1, f0, f1, 0.05517162f, 0.05517162f, 0.24261113f, 0.24261113f);
    fma2(p0, p1, p0, p1, f0, f1, 0.69326097f, 0.69326097f);
    fma2(p0, p1, p0, p1, f0, f1, 0.99992806f, 0.99992806f);
    a = __int_as_float(__float_as_int(p0) + (__float_as_int(r0) << 23));
    b = __int_as_float(__float_as_int(p1) + (__float_as_int(r1) << 23));
}

// POLY: one score pair in POLY takes the polynomial path (0: none)

// Half a score row -> P = exp2(score - m) as 32 packed f16 pairs in ONE sweep over the raw words; the
// pair (sum0, sum1) accumulates the row sum of this half.  MASKED: columns >= valid are padding and get
// P = 0.  MODE 0: the words are f32 scores, exponent = s * c0 - m.  MODE 1: s32 dot products; with
// f = 12582912 + s (the magic-number reinterpretation) the exponent is f * c0 + kr, kr = -(m + 12582912 * c0),
// one multiply-add and no separate subtraction.  MODE 2: s32 dot products plus a per-key smooth-Q bias b
// (shared memory, not yet scaled): exponent = f * c0 + (b * sl2 + kr).  Rounding kr (magnitude about
// 12582912 * c0, a few thousand at most) costs below 1e-4 of absolute exponent error, under the f16
// rounding of P.
template <int MODE, bool MASKED, int POLY>
__device__ __forceinline__ void half_row_exp(const uint32_t (&rr)[64], uint32_t (&p2)[32], float c0, float m,
                                             const float4* bias, float sl2, int valid, float& sum0, float& sum1,
                                             int one) {
    const float kr = MODE == 0 ? -m : -fmaf(kMagicFloat, c0, m);
#pragma unroll
    for (int i = 0; i < 32; ++i) {
        float e0, e1;
        if (MODE == 0) {
            fma2(e0, e1, __uint_as_float(rr[2 * i]), __uint_as_float(rr[2 * i + 1]), c0, c0, kr, kr);
        } else {
            const float f0 = magic_i2f_biased(rr[2 * i + 0], one);
            const float f1 = magic_i2f_biased(rr[2 * i + 1], one);
            if (MODE == 2) {
                const float2 b = reinterpret_cast<const float2*>(bias)[i];   // same address in every lane
                float t0, t1;
                fma2(t0, t1, b.x, b.y, sl2, sl2, kr, kr);
                fma2(e0, e1, f0, f1, c0, c0, t0, t1);
            } else {
                fma2(e0, e1, f0, f1, c0, c0, kr, kr);
            }
        }
        float a, b;
        if (POLY > 0 && i % (POLY > 0 ? POLY : 1) == (POLY > 0 ? POLY : 1) - 1) {
            ex2_poly2(e0, e1, a, b);
        } else {
            a = ex2(e0);
            b = ex2(e1);
        }
        if (MASKED) {
            if (2 * i + 0 >= valid) a = 0.0f;
            if (2 * i + 1 >= valid) b = 0.0f;
        }
        add2(sum0, sum1, sum0, sum1, a, b);
        p2[i] = pack_h2(a, b);
    }
}

// A half whose row sum (against the running maximum the row already uses) stays below this needs no new
// maximum: every P of it is below the limit too, far inside the f16 range.
constexpr float kHalfSumLimit = 4096.0f;

template <int D, bool SAGE, int POLY>
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
    uint64_t* s_full = v_empty + KV_STAGES;  // [QT][2]  S of (tile, half) complete
    uint64_t* p_full = s_full + QT * 2;      // [QT][2]  P of (tile, half) written
    uint64_t* pv_done = p_full + QT * 2;     // [QT]     one phase per PV product of the tile
    uint64_t* o_done = pv_done + QT;         // [QT]     the tile's last PV product
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(o_done + QT);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    // which query rows and head this CTA owns, and how many 128-row tiles (qt)
    int qt = P.qt, q0 = blockIdx.x * (P.qt * BQ), hn = blockIdx.y;
    if (P.n_mixed_two >= 0) {
        const int b = blockIdx.x;
        if (b < P.n_mixed_two) {
            qt = 2;
            hn = b / P.slabs2;
            q0 = (b % P.slabs2) * (2 * BQ);
        } else {
            const int j = b - P.n_mixed_two;
            const int item = P.n_mixed_two + (j >> 1);
            qt = 1;
            hn = item / P.slabs2;
            q0 = (item % P.slabs2) * (2 * BQ) + (j & 1) * BQ;
            if (q0 >= P.Lq) return;   // the second half of a slab that holds one tile only (whole CTA leaves)
        }
    }
    const int n_kv = (P.Lk + BKV - 1) / BKV;

    if (threadIdx.x == 0) {
        mbar_init(q_full, 1);
        for (int i = 0; i < KV_STAGES; ++i) {
            mbar_init(&k_full[i], 1);
            mbar_init(&k_empty[i], qt);
            mbar_init(&v_full[i], 1);
            mbar_init(&v_empty[i], qt);
        }
        for (int i = 0; i < QT; ++i) {
            for (int b = 0; b < 2; ++b) {
                mbar_init(&s_full[i * 2 + b], 1);
                mbar_init(&p_full[i * 2 + b], 4);
            }
            mbar_init(&pv_done[i], 1);
            mbar_init(&o_done[i], 1);
        }
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
        if (elect_one()) {
            mbar_arrive_expect_tx(q_full, qt * C::Q_BYTES);
            for (int t = 0; t < qt; ++t) {
#pragma unroll
                for (int p = 0; p < C::QK_PANELS; ++p) {
                    tma_load_3d(smem + C::OFF_Q + t * C::Q_BYTES + p * C::QK_PANEL_BYTES, &map_q, q_full,
                                p * (C::QK_ROW_BYTES / C::QK_ELEM), q0 + t * BQ, hn);
                }
            }
            for (int j = 0; j < n_kv; ++j) {
                const int st = j % KV_STAGES;
                const uint32_t ph = (j / KV_STAGES) & 1;
                if (!mbar_wait(&k_empty[st], ph ^ 1u, abort_flag, P.err)) break;
                const bool with_bias = SAGE && P.bias != nullptr;
                mbar_arrive_expect_tx(&k_full[st], C::K_BYTES + (with_bias ? BKV * 4 : 0));
#pragma unroll
                for (int p = 0; p < C::QK_PANELS; ++p) {
                    tma_load_3d(smem + C::OFF_K + st * C::K_BYTES + p * C::QK_PANEL_BYTES, &map_k, &k_full[st],
                                p * (C::QK_ROW_BYTES / C::QK_ELEM), j * BKV, hn);
                }
                if (with_bias) {
                    // The bias piece of key block j is read by the softmax threads until their P of block j
                    // is complete.  Piece j + 4 is fetched after S(j + 2) of the second query tile finished,
                    // which the issue order puts after P(j + 1) of both tiles: four stages cannot collide.
                    bulk_load_1d(smem + C::OFF_BIAS + (j % BIAS_STAGES) * (BKV * 4),
                                 P.bias + (long long)hn * P.bias_stride + (long long)j * BKV, BKV * 4, &k_full[st]);
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
    } else if (warp == 1 || (warp == 3 && qt == 2)) {
        // ------------------------------------------- MMA issuers, one per query tile
        // (one thread cannot issue the small products of both tiles fast enough)
        const int t = warp >> 1;
        const uint32_t idesc_qk = SAGE ? make_idesc(kDFmtS32, kFmtS8, kFmtS8, 0, 0, BQ, HK)
                                       : make_idesc(kDFmtF32, kFmtF16, kFmtF16, 0, 0, BQ, HK);
        const uint32_t idesc_pv = make_idesc(kDFmtF32, kFmtF16, kFmtF16, 0, 1, BQ, D);
        bool ok = mbar_wait(q_full, 0, abort_flag, P.err);
        const int n_half = 2 * n_kv;     // 64-key halves; half g = keys [64 g, 64 g + 64) = block g/2, buffer g%2

        // S_t[g % 2] = Q_t K_g^T.  The buffer is free: the PV product that read P from it
        // (half g - 2) was issued before, and the tensor pipe runs in issue order.
        auto issue_qk = [&](int g) -> bool {
            const int j = g >> 1, hb = g & 1;
            const int st = j % KV_STAGES;
            if (!mbar_wait(&k_full[st], static_cast<uint32_t>((j / KV_STAGES) & 1), abort_flag, P.err)) return false;
            tc_fence_after_sync();
            if (elect_one()) {
                const uint32_t q_addr = smem_u32(smem + C::OFF_Q + t * C::Q_BYTES);
                // K-major rows of QK_ROW_BYTES: 64 keys further = 64 rows inside every panel
                const uint32_t k_addr = smem_u32(smem + C::OFF_K + st * C::K_BYTES) + hb * (HK * C::QK_ROW_BYTES);
                const uint32_t tmem_s = tmem_base + TMEM_S + t * 128 + hb * HK;
#pragma unroll
                for (int ks = 0; ks < C::QK_KSTEPS; ++ks) {
                    const uint32_t off = (ks / C::QK_KSTEPS_PER_PANEL) * C::QK_PANEL_BYTES + (ks % C::QK_KSTEPS_PER_PANEL) * 32;
                    const uint64_t ad = C::QK_ROW_BYTES == 128 ? make_smem_desc_sw128(q_addr + off, 16, 1024)
                                                               : make_smem_desc_sw64(q_addr + off, 16, 512);
                    const uint64_t bd = C::QK_ROW_BYTES == 128 ? make_smem_desc_sw128(k_addr + off, 16, 1024)
                                                               : make_smem_desc_sw64(k_addr + off, 16, 512);
                    if (SAGE) {
                        mma_i8_ss(tmem_s, ad, bd, idesc_qk, ks > 0 ? 1u : 0u);
                    } else {
                        mma_f16_ss(tmem_s, ad, bd, idesc_qk, ks > 0 ? 1u : 0u);
                    }
                }
                mma_commit(&s_full[t * 2 + hb]);
                if (hb == 1) mma_commit(&k_empty[st]);
            }
            __syncwarp();
            return true;
        };
        // O_t += P_t[g % 2] V_g
        auto issue_pv = [&](int g) -> bool {
            const int j = g >> 1, hb = g & 1;
            const int st = j % KV_STAGES;
            if (!mbar_wait(&v_full[st], static_cast<uint32_t>((j / KV_STAGES) & 1), abort_flag, P.err) ||
                !mbar_wait(&p_full[t * 2 + hb], static_cast<uint32_t>(j & 1), abort_flag, P.err)) {
                return false;
            }
            tc_fence_after_sync();
            if (elect_one()) {
                const uint32_t v_addr = smem_u32(smem + C::OFF_V + st * C::V_BYTES);
                const uint32_t tmem_p = tmem_base + TMEM_S + t * 128 + hb * HK;
#pragma unroll
                for (int ks = 0; ks < HK / 16; ++ks) {
                    // P: tensor memory, 8 columns (16 keys) per step; V: MN-major, 16 keys = 2 KB per step
                    const uint64_t bd = make_smem_desc_sw128(v_addr + (hb * (HK / 16) + ks) * 2048, BKV * 128, 1024);
                    mma_f16_ts(tmem_base + TMEM_O + t * 128, tmem_p + ks * 8, bd, idesc_pv, (g > 0 || ks > 0) ? 1u : 0u);
                }
                mma_commit(&pv_done[t]);
                if (g == n_half - 1) mma_commit(&o_done[t]);
                if (hb == 1) mma_commit(&v_empty[st]);
            }
            __syncwarp();
            return true;
        };

        for (int g = 0; ok && g < 2; ++g) ok = issue_qk(g);
        for (int g = 0; ok && g < n_half; ++g) {
            ok = issue_pv(g);
            if (ok && g + 2 < n_half) ok = issue_qk(g + 2);
        }
    } else if (warp >= 4 && warp < 4 + 4 * qt) {
        // ------------------------------------------------------------ softmax
        const int t = (warp - 4) >> 2;              // query tile
        const int quarter = warp & 3;
        const int r = quarter * 32 + lane;          // row inside the tile = tensor-memory lane
        const int q_row = q0 + t * BQ + r;
        const uint32_t lane_base = static_cast<uint32_t>(quarter * 32) << 16;
        const uint32_t s_addr = tmem_base + lane_base + TMEM_S + t * 128;
        const uint32_t o_addr = tmem_base + lane_base + TMEM_O + t * 128;
        float m_used = -INFINITY;
        float sum0 = 0.0f, sum1 = 0.0f;
        float row_scale = P.scale_log2;
        float q_scale = 1.0f;
        const float* bias_row = nullptr;
        const float* ks_row = nullptr;
        if (SAGE) {
            // a query tile that lies wholly beyond Lq (second tile of the last slab) has no scale row
            if (q0 + t * BQ < P.Lq) {
                q_scale = P.q_scale[(long long)hn * P.q_scale_stride + ((q0 + t * BQ) >> 5) + quarter];
            }
            row_scale *= q_scale;
            ks_row = P.k_scale + (long long)hn * P.k_scale_stride;
            if (P.bias != nullptr) bias_row = P.bias + (long long)hn * P.bias_stride;
        }
        bool ok = true;

        const bool biased = SAGE && bias_row != nullptr;   // uniform over the CTA
        const int n_half = 2 * n_kv;
        // One online-softmax step per 64-key half g: its scores sit in buffer g % 2 of the tile's S
        // columns, and the other buffer is filled by the tensor pipe meanwhile, so a softmax warp goes
        // from one half straight to the next.
        // The tensor-memory read of half g + 1 is issued before P of half g is stored, so its
        // latency and that of the store / barrier hand-over overlap.
        uint32_t rr[64];
        ok = mbar_wait(&s_full[t * 2], 0, abort_flag, P.err);
        tc_fence_after_sync();
        if (ok) tmem_ld_cols<64>(s_addr, rr);
        for (int g = 0; ok && g < n_half; ++g) {
            const int j = g >> 1, hb = g & 1;
            const int valid = P.Lk - g * HK;        // columns >= valid are padding (last block only)
            float c0 = row_scale;                   // score multiplier
            float cq = 1.0f;                        // the same without the softmax scale
            if (SAGE) {
                const float kscale = __ldg(ks_row + g);
                c0 *= kscale;
                cq = q_scale * kscale;
            }
            const uint32_t sb_addr = s_addr + hb * HK;
            tmem_wait_ld();
            const float4* bias_h =
                biased ? reinterpret_cast<const float4*>(smem + C::OFF_BIAS + (j % BIAS_STAGES) * (BKV * 4)) + 16 * hb
                       : nullptr;
            // P = exp2(score - m) as f16 pairs over the first 32 columns of the buffer just read.
            // Fast path: one sweep against the maximum the row already uses (it may be stale: any maximum
            // gives the same softmax as long as nothing overflows), accepted when the half's row sum shows
            // that no score has outgrown it.  Otherwise, and for the first and a ragged last half: the
            // maximum sweep, a rescale of what has been accumulated if the maximum moved by more than 2^8,
            // and the exponentials again.
            uint32_t p2[32];
            const bool ragged = valid < HK;          // uniform; only the last key block can be ragged
            bool slow = g == 0 || ragged;
            if (!slow) {
                float h0 = 0.0f, h1 = 0.0f;
                if (!SAGE) {
                    half_row_exp<0, false, POLY>(rr, p2, c0, m_used, nullptr, P.scale_log2, valid, h0, h1, P.one);
                } else if (biased) {
                    half_row_exp<2, false, POLY>(rr, p2, c0, m_used, bias_h, P.scale_log2, valid, h0, h1, P.one);
                } else {
                    half_row_exp<1, false, POLY>(rr, p2, c0, m_used, nullptr, P.scale_log2, valid, h0, h1, P.one);
                }
                const bool over = !(h0 + h1 <= kHalfSumLimit);   // also true for inf / NaN
                if (__any_sync(0xffffffffu, over)) {
                    slow = true;
                } else {
                    sum0 += h0;
                    sum1 += h1;
                }
            }
            if (slow) {
                const float mx = ragged ? half_row_max<SAGE, true>(rr, c0, cq, bias_h, P.scale_log2, valid, P.one)
                                        : half_row_max<SAGE, false>(rr, c0, cq, bias_h, P.scale_log2, valid, P.one);
                // lazy rescale: keep exponentiating against the old maximum until it is stale by > 2^8
                float alpha = 1.0f;
                const bool grow = mx > m_used + kRescaleThreshold;
                if (grow) {
                    alpha = ex2(m_used - mx);   // 0 on the very first half (m_used = -inf)
                    m_used = mx;
                    sum0 *= alpha;
                    sum1 *= alpha;
                }
                if (g > 0 && __any_sync(0xffffffffu, grow)) {
                    // O_t holds the PV products up to half g - 1; the next one waits for this thread's P.
                    // S(g) complete means the product of half g - 2 has completed, so pv_done is in
                    // phase g - 1 or g and the parity wait below cannot alias.
                    if (!mbar_wait(&pv_done[t], static_cast<uint32_t>((g - 1) & 1), abort_flag, P.err)) {
                        ok = false;
                        break;
                    }
                    tc_fence_after_sync();
#pragma unroll
                    for (int c = 0; c < D / 32; ++c) {
                        uint32_t oo[32];
                        tmem_ld_cols<32>(o_addr + c * 32, oo);
                        tmem_wait_ld();
#pragma unroll
                        for (int i = 0; i < 32; ++i) oo[i] = __float_as_uint(__uint_as_float(oo[i]) * alpha);
                        tmem_st_cols<32>(o_addr + c * 32, oo);
                    }
                }
                float h0 = 0.0f, h1 = 0.0f;
                if (!ragged) {
                    if (!SAGE) {
                        half_row_exp<0, false, POLY>(rr, p2, c0, m_used, nullptr, P.scale_log2, valid, h0, h1, P.one);
                    } else if (biased) {
                        half_row_exp<2, false, POLY>(rr, p2, c0, m_used, bias_h, P.scale_log2, valid, h0, h1, P.one);
                    } else {
                        half_row_exp<1, false, POLY>(rr, p2, c0, m_used, nullptr, P.scale_log2, valid, h0, h1, P.one);
                    }
                } else {
                    if (!SAGE) {
                        half_row_exp<0, true, POLY>(rr, p2, c0, m_used, nullptr, P.scale_log2, valid, h0, h1, P.one);
                    } else if (biased) {
                        half_row_exp<2, true, POLY>(rr, p2, c0, m_used, bias_h, P.scale_log2, valid, h0, h1, P.one);
                    } else {
                        half_row_exp<1, true, POLY>(rr, p2, c0, m_used, nullptr, P.scale_log2, valid, h0, h1, P.one);
                    }
                }
                sum0 += h0;
                sum1 += h1;
            }
            if (g + 1 < n_half) {
                // all of rr has been consumed; the other buffer holds the next half
                if (!mbar_wait(&s_full[t * 2 + (hb ^ 1)], static_cast<uint32_t>(((g + 1) >> 1) & 1), abort_flag, P.err)) {
                    ok = false;
                    break;
                }
                tc_fence_after_sync();
                tmem_ld_cols<64>(s_addr + (hb ^ 1) * HK, rr);
            }
            tmem_st_cols<32>(sb_addr, p2);
            tmem_wait_st();
            tc_fence_before_sync();
            __syncwarp();
            if (elect_one()) mbar_arrive(&p_full[t * 2 + hb]);
        }

        // ----------------------------------------------------------- epilogue
        if (ok) ok = mbar_wait(&o_done[t], 0, abort_flag, P.err);
        if (ok) {
            tc_fence_after_sync();
            const float inv_l = 1.0f / (sum0 + sum1);
            const bool row_ok = q_row < P.Lq;
            char* obase = static_cast<char*>(P.out);
            long long orow = q_row;
            if (P.t_loc > 0 && row_ok) {
                obase = static_cast<char*>(P.out_peer[q_row / P.t_loc]);
                orow = q_row % P.t_loc;
            }
            const long long ocol = orow * P.ld_out + (long long)hn * D;
#pragma unroll
            for (int c = 0; c < D / 32; ++c) {
                __syncwarp();
                uint32_t oo[32];
                tmem_ld_cols<32>(o_addr + c * 32, oo);
                tmem_wait_ld();
                if (!row_ok) continue;
                float v[32];
#pragma unroll
                for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(oo[i]) * inv_l;
                if (P.out_dtype == EDB200_TYPE_F32) {
                    float4* o = reinterpret_cast<float4*>(obase + (ocol + c * 32) * 4);
#pragma unroll
                    for (int i = 0; i < 8; ++i) o[i] = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
                } else {
                    uint4* o = reinterpret_cast<uint4*>(obase + (ocol + c * 32) * 2);
                    const bool bf = P.out_dtype == EDB200_TYPE_BF16;
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
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

template <int D, bool SAGE, int POLY>
static edb200_status_t launch_poly(const void* q, const void* k, const void* v, int64_t q_head_rows, int64_t k_head_rows,
                              int64_t v_head_rows, const Params& P_in, cudaStream_t stream) {
    using C = Cfg<D, SAGE>;
    Params P = P_in;
    // Two query tiles per CTA share K/V and overlap softmax with the tensor pipe; when that leaves SMs
    // without a CTA (few heads per rank under sequence parallelism) one tile per CTA fills the GPU better.
    // One CTA fits per SM (it holds all of tensor memory), so the kernel runs in waves; a two-tile CTA
    // takes about 1.5x as long as a one-tile CTA.
    {
        const int64_t sms = sm_count();
        const int64_t w2 = (((P.Lq + QT * BQ - 1) / (QT * BQ)) * P.HN + sms - 1) / sms;
        const int64_t w1 = (((P.Lq + BQ - 1) / BQ) * P.HN + sms - 1) / sms;
        P.qt = (P.Lq > BQ && 2 * w1 < 3 * w2) ? 1 : QT;
    }
    P.n_mixed_two = -1;
    P.slabs2 = static_cast<int>((P.Lq + QT * BQ - 1) / (QT * BQ));
    if (P.qt == QT) {
        // at least one full wave of two-tile CTAs and a partial last wave whose slabs, taken one tile per CTA,
        // still fit one wave: run that last wave as one-tile CTAs
        const int64_t sms = sm_count();
        const int64_t items = (int64_t)P.slabs2 * P.HN, tail = items % sms;
        static int mix = -1;   // EDB200_ATTN_MIX=0: every CTA takes two tiles (comparison runs)
        if (mix < 0) {
            const char* e = getenv("EDB200_ATTN_MIX");
            mix = (e != nullptr && atoi(e) == 0) ? 0 : 1;
        }
        if (mix == 1 && items / sms >= 1 && tail > 0 && 2 * tail <= sms) P.n_mixed_two = static_cast<int>(items - tail);
    }
    if (const char* e = getenv("EDB200_ATTN_QT")) {   // tuning and tests: force one of the schedules
        if (e[0] == '1') P.qt = 1, P.n_mixed_two = -1;
        if (e[0] == '2') P.qt = QT, P.n_mixed_two = -1;
    }

    CUtensorMap mq, mk, mv;
    const CUtensorMapDataType qk_dt = SAGE ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    const int es = C::QK_ELEM;
    const uint32_t box_inner = C::QK_ROW_BYTES / es;
    const CUtensorMapSwizzle qk_swz = C::QK_ROW_BYTES == 128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B;
    edb200_status_t st = make_tmap_3d(&mq, qk_dt, es, q, D, P.Lq, P.HN, (uint64_t)D * es, (uint64_t)q_head_rows * D * es,
                                      box_inner, BQ, 1, qk_swz);
    if (st != EDB200_OK) return st;
    st = make_tmap_3d(&mk, qk_dt, es, k, D, P.Lk, P.HN, (uint64_t)D * es, (uint64_t)k_head_rows * D * es, box_inner, BKV, 1,
                      qk_swz);
    if (st != EDB200_OK) return st;
    st = make_tmap_3d(&mv, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, v, D, P.Lk, P.HN, (uint64_t)D * 2,
                      (uint64_t)v_head_rows * D * 2, 64, BKV, 1, CU_TENSOR_MAP_SWIZZLE_128B);
    if (st != EDB200_OK) return st;
    auto kern = attention_kernel<D, SAGE, POLY>;
    static bool attr_set[64] = {false};   // the attribute is per device
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64 || !attr_set[dev]) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES);
        if (e != cudaSuccess) return check_cuda(e, "cudaFuncSetAttribute(attention)");
        if (dev >= 0 && dev < 64) attr_set[dev] = true;
    }
    dim3 grid((P.Lq + P.qt * BQ - 1) / (P.qt * BQ), P.HN);
    if (P.n_mixed_two >= 0) {
        const int64_t items = (int64_t)P.slabs2 * P.HN;
        grid = dim3(static_cast<unsigned>(P.n_mixed_two + 2 * (items - P.n_mixed_two)), 1);
    }
    ProfScope prof(stream, PROF_ATTENTION, 4.0 * (double)P.Lq * (double)P.Lk * D * P.HN,
                   (double)P.HN * D * ((double)P.Lq * (C::QK_ELEM + 2) + (double)P.Lk * (C::QK_ELEM + 2)));
    kern<<<grid, NUM_THREADS, C::SMEM_BYTES, stream>>>(mq, mk, mv, P);
    count_launch();
    return check_cuda(cudaGetLastError(), "attention launch");
}

// Share of the exponentials evaluated as a polynomial on the FMA pipe instead of the ex2 unit, per variant
// (measured at 24 heads x 4608 and 5 heads x 75600 tokens, d 128): the f16 kernel is fastest with one
// pair in eight (1148 / 1271 TFLOP/s against 1147 / 1199 with one in four and 1089 / 1196 with none), the
// INT8 kernel, which already spends more FMA-pipe instructions per score, with none (930 / 1087 against
// 917 / 1059 and 891 / 1025).
template <int D, bool SAGE>
static edb200_status_t launch(const void* q, const void* k, const void* v, int64_t q_head_rows, int64_t k_head_rows,
                              int64_t v_head_rows, const Params& P_in, cudaStream_t stream) {
    return launch_poly<D, SAGE, SAGE ? 0 : 8>(q, k, v, q_head_rows, k_head_rows, v_head_rows, P_in, stream);
}

}  // namespace attn
}  // namespace edb

using namespace edb;

extern "C" {

// Fills the peer-output part of the kernel parameters: the column block of this rank's heads
// inside every rank's [t_loc, ld_out] buffer.
static edb200_status_t set_peer_out(attn::Params& P, const edb200_sp_peers_t* dst, int hn, int d_head, int out_dtype) {
    if (dst == nullptr) return EDB200_OK;
    if (dst->world <= 0 || dst->world > 8 || dst->rank < 0 || dst->rank >= dst->world || dst->t_loc <= 0 ||
        dst->t_loc * dst->world < P.Lq) {
        return fail(EDB200_ERR_INVALID, "attention: bad peer description");
    }
    const int esz = out_dtype == EDB200_TYPE_F32 ? 4 : 2;
    for (int r = 0; r < dst->world; ++r) {
        if (dst->buf[0][r] == nullptr) return fail(EDB200_ERR_INVALID, "attention: null peer buffer");
        P.out_peer[r] = static_cast<char*>(dst->buf[0][r]) + (int64_t)dst->rank * hn * d_head * esz;
    }
    P.t_loc = static_cast<int>(dst->t_loc);
    P.out = P.out_peer[dst->rank];
    return EDB200_OK;
}

edb200_status_t edb200_attention_f16(const void* q, const void* k, const void* v, int hn, int64_t lq, int64_t lk,
                                     int d_head, float scale, void* out, int out_dtype, int64_t ld_out,
                                     void* stream) {
    return edb200_attention_f16_strided(q, k, v, hn, lq, lk, lq, lk, d_head, scale, out, out_dtype, ld_out, nullptr, stream);
}

edb200_status_t edb200_attention_f16_sp(const void* q, const void* k, const void* v, int hn, int64_t lq, int64_t lk,
                                        int d_head, float scale, void* out, int out_dtype, int64_t ld_out,
                                        const edb200_sp_peers_t* dst, void* stream) {
    return edb200_attention_f16_strided(q, k, v, hn, lq, lk, lq, lk, d_head, scale, out, out_dtype, ld_out, dst, stream);
}

edb200_status_t edb200_attention_f16_strided(const void* q, const void* k, const void* v, int hn, int64_t lq, int64_t lk,
                                             int64_t q_head_rows, int64_t kv_head_rows, int d_head, float scale,
                                             void* out, int out_dtype, int64_t ld_out, const edb200_sp_peers_t* dst,
                                             void* stream) {
    if (dst != nullptr && out == nullptr) out = dst->buf[0][dst->rank < 8 && dst->rank >= 0 ? dst->rank : 0];
    if (q == nullptr || k == nullptr || v == nullptr || out == nullptr || hn <= 0 || lq <= 0 || lk <= 0) {
        return fail(EDB200_ERR_INVALID, "attention_f16: null or empty argument");
    }
    if (q_head_rows < lq || kv_head_rows < lk) {
        return fail(EDB200_ERR_INVALID, "attention_f16: the rows between heads must cover the sequence");
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
    P.one = 1;
    P.out = out;
    P.ld_out = ld_out;
    P.out_dtype = out_dtype;
    P.Lq = static_cast<int>(lq);
    P.Lk = static_cast<int>(lk);
    P.HN = hn;
    P.scale_log2 = scale * 1.4426950408889634f;
    P.err = err;
    EDB_TRY(set_peer_out(P, dst, hn, d_head, out_dtype));
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (d_head == 128) return attn::launch<128, false>(q, k, v, q_head_rows, kv_head_rows, kv_head_rows, P, s);
    return attn::launch<64, false>(q, k, v, q_head_rows, kv_head_rows, kv_head_rows, P, s);
}

edb200_status_t edb200_attention_sage_int8(const void* q_i8, const void* k_i8, const void* v_f16,
                                           const float* q_scale, int q_scale_stride, const float* k_scale,
                                           int k_scale_stride, const float* bias, int bias_stride, int hn, int64_t l,
                                           int d_head, float scale, void* out, int out_dtype, int64_t ld_out,
                                           void* stream) {
    return edb200_attention_sage_int8_strided(q_i8, k_i8, v_f16, l, q_scale, q_scale_stride, k_scale, k_scale_stride, bias,
                                              bias_stride, hn, l, d_head, scale, out, out_dtype, ld_out, nullptr, stream);
}

edb200_status_t edb200_attention_sage_int8_sp(const void* q_i8, const void* k_i8, const void* v_f16,
                                              const float* q_scale, int q_scale_stride, const float* k_scale,
                                              int k_scale_stride, const float* bias, int bias_stride, int hn,
                                              int64_t l, int d_head, float scale, void* out, int out_dtype,
                                              int64_t ld_out, const edb200_sp_peers_t* dst, void* stream) {
    return edb200_attention_sage_int8_strided(q_i8, k_i8, v_f16, l, q_scale, q_scale_stride, k_scale, k_scale_stride, bias,
                                              bias_stride, hn, l, d_head, scale, out, out_dtype, ld_out, dst, stream);
}

edb200_status_t edb200_attention_sage_int8_strided(const void* q_i8, const void* k_i8, const void* v_f16,
                                                   int64_t v_head_rows, const float* q_scale, int q_scale_stride,
                                                   const float* k_scale, int k_scale_stride, const float* bias,
                                                   int bias_stride, int hn, int64_t l, int d_head, float scale,
                                                   void* out, int out_dtype, int64_t ld_out,
                                                   const edb200_sp_peers_t* dst, void* stream) {
    if (dst != nullptr && out == nullptr) out = dst->buf[0][dst->rank < 8 && dst->rank >= 0 ? dst->rank : 0];
    if (q_i8 == nullptr || k_i8 == nullptr || v_f16 == nullptr || q_scale == nullptr || k_scale == nullptr ||
        out == nullptr || hn <= 0 || l <= 0 || v_head_rows < l) {
        return fail(EDB200_ERR_INVALID, "attention_sage_int8: null or empty argument");
    }
    if (d_head != 128 && d_head != 64) return fail(EDB200_ERR_UNSUPPORTED, "attention_sage_int8: d_head must be 64 or 128");
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
    P.one = 1;
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
    EDB_TRY(set_peer_out(P, dst, hn, d_head, out_dtype));
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (d_head == 64) return attn::launch<64, true>(q_i8, k_i8, v_f16, l, l, v_head_rows, P, s);
    return attn::launch<128, true>(q_i8, k_i8, v_f16, l, l, v_head_rows, P, s);
}

}  // extern "C"
