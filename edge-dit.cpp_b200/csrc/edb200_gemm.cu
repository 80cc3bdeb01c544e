// Dequant-fused quantised GEMM for sm_100a.
//
//   y[m, n] = sum_k x[m, k] * dequant(W)[n, k]   (+ bias, activation, gated residual)
//
// Stands in for ggml_mul_mat on q8_0 / q4_K weights reached through
// ggml_ext_linear (reference src/core/backend/ggml/ggml_extend.hpp:1308-1347).
//
// The kernel computes the transposed tile  D[n, m] = W[n, :] . x[m, :]  so that
// the *weights* are the tcgen05 A operand.  A may live in tensor memory, which is
// what makes the fusion cheap: the dequantisers write f16 weights straight into
// tensor memory (tcgen05.st) and never touch shared memory with them.  Per 64-deep
// k-step a CTA moves 24 KB of activations in (TMA) and out (MMA B operand) plus
// 8.5 KB of raw weights per weight tile, instead of also writing and re-reading
// 16-32 KB of dequantised weights.
//
// Two kernels share this scheme.  qgemm_pair_kernel (further down; the default) runs it on pairs of CTAs
// with tcgen05 .cta_group::2, each CTA staging half of the token tile; qgemm_kernel, described here, is the
// single-CTA form kept for comparison (EDB200_GEMM_PAIR=0).
//
// One persistent CTA per SM, 896 threads, warp-specialised:
//   warp 0       producer (elect.sync): TMA tile of 192 tokens x 64 k (f16, 128B
//                swizzle) and one bulk copy per 128-row x 64-k weight tile record,
//                5-stage ring
//   warp 1       tcgen05.mma issuer (elect.sync): 128 x 192 x 16 kind::f16, A from
//                tensor memory, B from shared memory, four MMAs per A-stage
//                barrier; fp32 accumulators in tensor memory (384 columns)
//   warp 2       tensor-memory allocator
//   warps 4-11   epilogue: tcgen05.ld (lane = output feature, column = token),
//                bias / GELU / gate*y+residual, stores coalesced across lanes
//   warps 12-27  dequantisers: thread = one weight row x 32 k; int8 / 4-bit
//                payload -> f16 -> tcgen05.st into one of four 32-column A stages
// Issuing tcgen05.mma / tcgen05.commit from an `if (lane == 0)` branch costs about a
// hundred cycles per batch on B200; elect.sync issue runs at the tensor pipe's rate.
// The dequantised f16 weight equals rn_f16(d*q) for q8_0 (one rounding of the
// exact product) and rn_f16(a*q - b) for q4_K with a = rn_f16(d*sc), b = rn_f16(dmin*m).
#include "edb200_internal.h"
#include "edb200_ptx.cuh"

namespace edb {
namespace gemm {

constexpr int TW = 128;            // weight rows (output features) per tile = tensor-memory lanes
constexpr int TN = 192;            // tokens per tile = accumulator columns
constexpr int BK = 64;
constexpr int LD_STAGES = 5;
constexpr int X_BYTES = TN * BK * 2;          // 24 KB
constexpr int W_BYTES_MAX = 8704;             // one weight tile record (8704 / 5120 B)
constexpr int STAGE_BYTES = X_BYTES + 2 * W_BYTES_MAX;    // 41 KB (room for two weight tiles)
constexpr int OFF_BAR = LD_STAGES * STAGE_BYTES;
constexpr int SMEM_BYTES = OFF_BAR + 256 + 1024;  // + alignment slack

constexpr int NUM_THREADS = 896;
constexpr int EPI_WARPS = 8;       // warps 4-7 (weight half 0) and 8-11 (weight half 1)
constexpr int EC = 16;             // accumulator columns (tokens) per epilogue step
constexpr uint32_t TMEM_COLS = 512;
constexpr uint32_t TMEM_ACC = 0;                       // 384 accumulator columns, A stages above them

struct Problem {
    const float* bias;
    void* out;
    const float* residual;
    const float* gate;
    void* out2;
    const uint8_t* tiles;      // repacked weight
    long long ldo, ld_res, ldo2, split_n;
    int out_dtype, act, out2_dtype, act2;
    int M, N, K;
    int m_tiles, n_tiles;
    int chunk;   // token tiles per L2-resident activation chunk (tile order below)
    // Fused head-major pack of the leading q | k | v features (edb200_qk_pack_t); n_pack = 0: off.
    int n_pack;          // 3 * heads * 128, or heads * 128 when the output is q, k or v alone
    int pk_first;        // kind of the first packed head block: 0 q, 1 k, 2 v
    int pk_d;            // head width: 128 (one head per weight tile) or 64 (two)
    int pk_heads, pk_hp; // heads; heads per rank when the destination is sharded (0: local)
    float pk_eps;
    const float* pk_qw;
    const float* pk_kw;
    const float* pk_pe;      // row i of the problem reads table row pk_pe_row0 + i
    long long pk_pe_row0;
    long long pk_pos0;       // token position of row 0 in the destination
    long long pk_ltotal;
    void* pk_dst[3][8];      // q, k, v of every destination rank (index 0 when local)
    int ksplit;  // parts the reduction is cut into (1: whole k per tile); parts add into `out` atomically
};

struct Params {
    Problem p[2];
    int tiles0;       // tiles of problem 0
    int total_tiles;
    int* err;
};

struct TileCoord {
    int prob, m0, n_tile;   // n_tile = first of the WH consecutive weight tiles
    int kpart;              // which part of the reduction (0 .. ksplit-1)
};

__device__ __forceinline__ TileCoord tile_coord(const Params& P, int t, int wh) {
    TileCoord c;
    c.prob = (t >= P.tiles0) ? 1 : 0;
    int tt = c.prob ? t - P.tiles0 : t;
    const Problem& pr = c.prob ? P.p[1] : P.p[0];
    const int mn_tiles = pr.m_tiles * pr.n_tiles;
    c.kpart = tt / mn_tiles;   // reduction part outermost: 0 for unsplit problems
    tt -= c.kpart * mn_tiles;
    // Order: activation chunk (pr.chunk token tiles, sized to stay in L2) > weight tile row > token
    // tile.  CTAs running at the same time share one weight tile row through L2, and all weight
    // rows pass over a chunk before the next chunk is touched, so neither operand is re-read
    // from DRAM more than (number of chunks) times, however many tokens there are.
    const int per_chunk = pr.chunk * pr.n_tiles;
    const int full = pr.m_tiles / pr.chunk;
    int chunk_idx = tt / per_chunk, r = tt % per_chunk, width = pr.chunk;
    if (chunk_idx >= full) {   // the last, narrower chunk
        chunk_idx = full;
        r = tt - full * per_chunk;
        width = pr.m_tiles - full * pr.chunk;
    }
    c.n_tile = (r / width) * wh;
    c.m0 = (chunk_idx * pr.chunk + r % width) * TN;
    return c;
}

__device__ __forceinline__ float gelu_tanh_fast(float x) {
    const float u = 0.7978845608028654f * x * (1.0f + 0.044715f * x * x);
    float t;
    asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(u));
    return 0.5f * x * (1.0f + t);
}

__device__ __forceinline__ float apply_act(float v, int act) {
    if (act == EDB200_ACT_GELU_TANH) return gelu_tanh_fast(v);
    if (act == EDB200_ACT_SILU) return v / (1.0f + __expf(-v));
    return v;
}

// EC tokens (m_first..) of one output feature n; lanes of a warp hold
// consecutive n, so every global access below is contiguous across the warp.
__device__ __forceinline__ void epilogue_store(const Problem& P, float (&v)[EC], int n, int m_first, bool n_ok,
                                               int kpart) {
    if (P.ksplit > 1) {
        // Split reduction (host guarantees: gated residual in place, f32, no activation):
        // out += gate * (partial + bias once).  The parts of one output add in any order.
        if (!n_ok) return;
        const float b = (P.bias != nullptr && kpart == 0) ? __ldg(P.bias + n) : 0.0f;
        const float g = __ldg(P.gate + n);
        const int rows = min(EC, P.M - m_first);
        float* o = reinterpret_cast<float*>(P.out) + (long long)m_first * P.ldo + n;
#pragma unroll
        for (int i = 0; i < EC; ++i) {
            if (i < rows) atomicAdd(o + (long long)i * P.ldo, g * (v[i] + b));
        }
        return;
    }
    const bool second = (P.split_n > 0) && (n >= P.split_n);
    const int act = second ? P.act2 : P.act;
    const float b = (P.bias != nullptr && n_ok) ? __ldg(P.bias + n) : 0.0f;
#pragma unroll
    for (int i = 0; i < EC; ++i) v[i] = apply_act(v[i] + b, act);
    const int rows = min(EC, P.M - m_first);   // uniform across the warp
    if (!second && P.gate != nullptr) {
        const float g = n_ok ? __ldg(P.gate + n) : 0.0f;
        const float* rp = P.residual + (long long)m_first * P.ld_res + n;
#pragma unroll
        for (int i = 0; i < EC; ++i) {
            if (i < rows && n_ok) v[i] = rp[(long long)i * P.ld_res] + g * v[i];
        }
    }
    if (!n_ok) return;
    const int dt = second ? P.out2_dtype : P.out_dtype;
    const long long ld = second ? P.ldo2 : P.ldo;
    const long long col = second ? (n - P.split_n) : n;
    char* base = reinterpret_cast<char*>(second ? P.out2 : P.out);
    if (dt == EDB200_TYPE_F32) {
        float* o = reinterpret_cast<float*>(base) + (long long)m_first * ld + col;
#pragma unroll
        for (int i = 0; i < EC; ++i) {
            if (i < rows) o[(long long)i * ld] = v[i];
        }
    } else if (dt == EDB200_TYPE_BF16) {
        __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(base) + (long long)m_first * ld + col;
#pragma unroll
        for (int i = 0; i < EC; ++i) {
            if (i < rows) o[(long long)i * ld] = __float2bfloat16_rn(v[i]);
        }
    } else {
        __half* o = reinterpret_cast<__half*>(base) + (long long)m_first * ld + col;
#pragma unroll
        for (int i = 0; i < EC; ++i) {
            if (i < rows) o[(long long)i * ld] = __float2half_rn(v[i]);
        }
    }
}

__device__ __forceinline__ uint32_t h2_sub_mul(uint32_t packed, __half2 bias, __half2 scale) {
    __half2 h = *reinterpret_cast<__half2*>(&packed);
    h = __hmul2(__hsub2(h, bias), scale);
    return *reinterpret_cast<uint32_t*>(&h);
}

__device__ __forceinline__ uint32_t h2_sub_fma(uint32_t packed, __half2 bias, __half2 a, __half2 negb) {
    __half2 h = *reinterpret_cast<__half2*>(&packed);
    h = __hfma2(__hsub2(h, bias), a, negb);
    return *reinterpret_cast<uint32_t*>(&h);
}

// q8_0 tile record: payload [c][r][16 bytes u = q + 128], scales [h][r] f16.  Thread (row r,
// half h) converts weights h*32 .. h*32+31 of its row into 16 packed f16 pairs.
__device__ __forceinline__ void dequant_q8_0(const uint8_t* tile, int r, int h, uint32_t (&o)[16]) {
    const __half2 k1152 = __float2half2_rn(1152.0f);
    const __half2 d2 = __half2half2(*reinterpret_cast<const __half*>(tile + 8192 + (h * 128 + r) * 2));
#pragma unroll
    for (int cc = 0; cc < 2; ++cc) {
        const uint4 raw = *reinterpret_cast<const uint4*>(tile + ((2 * h + cc) * 128 + r) * 16);
        const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const uint32_t x = w[j];                                      // bytes hold u = q + 128
            const uint32_t lo = __byte_perm(x, 0x64646464u, 0x4140);      // f16 (1024 + u0, 1024 + u1)
            const uint32_t hi = __byte_perm(x, 0x64646464u, 0x4342);
            o[cc * 8 + 2 * j + 0] = h2_sub_mul(lo, k1152, d2);
            o[cc * 8 + 2 * j + 1] = h2_sub_mul(hi, k1152, d2);
        }
    }
}

// q4_K tile record: payload [c][r][16 B] (low nibble = weight c*16+i, high nibble
// = weight 32+c*16+i), a [h][r] f16 at +4096, b [h][r] f16 at +4608.
__device__ __forceinline__ void dequant_q4_k(const uint8_t* tile, int r, int h, uint32_t (&o)[16]) {
    const __half2 k1024 = __float2half2_rn(1024.0f);
    const __half2 a2 = __half2half2(*reinterpret_cast<const __half*>(tile + 4096 + (h * 128 + r) * 2));
    const __half2 nb2 = __hneg2(__half2half2(*reinterpret_cast<const __half*>(tile + 4608 + (h * 128 + r) * 2)));
#pragma unroll
    for (int cc = 0; cc < 2; ++cc) {
        const uint4 raw = *reinterpret_cast<const uint4*>(tile + (cc * 128 + r) * 16);
        const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const uint32_t x = (h ? (w[j] >> 4) : w[j]) & 0x0F0F0F0Fu;
            o[cc * 8 + 2 * j + 0] = h2_sub_fma(__byte_perm(x, 0x64646464u, 0x4140), k1024, a2, nb2);
            o[cc * 8 + 2 * j + 1] = h2_sub_fma(__byte_perm(x, 0x64646464u, 0x4342), k1024, a2, nb2);
        }
    }
}

// WH = weight tiles (128-row halves) per CTA tile.
//   WH = 2: 256 weight rows x 192 tokens, one accumulator set (epilogue not overlapped):
//           least operand traffic per MAC, best for long reductions
//   WH = 1: 128 weight rows x 192 tokens, accumulators double-buffered (epilogue
//           overlaps the next tile's main loop), twice as many tiles
template <int WT, int WH>  // WT: EDB200_TYPE_Q8_0 or EDB200_TYPE_Q4_K
__global__ void __launch_bounds__(NUM_THREADS, 1)
qgemm_kernel(const __grid_constant__ CUtensorMap map_x0, const __grid_constant__ CUtensorMap map_x1,
             const __grid_constant__ Params P) {
    constexpr bool kQ4 = (WT == EDB200_TYPE_Q4_K);
    constexpr uint32_t kWBytes = kQ4 ? kQwTileBytesQ4 : kQwTileBytesQ8;
    constexpr uint32_t kTxBytes = X_BYTES + WH * kWBytes;
    constexpr int ACC_STAGES = WH == 1 ? 2 : 1;
    constexpr int A_COLS = 32;                       // tensor-memory columns of one A stage
    constexpr int AKW = 64 / WH;                     // k per A stage: 32 k of both halves, or 64 k of the one half
    constexpr int A_STAGES = 128 / A_COLS;           // 4
    constexpr uint32_t TMEM_A = 384;                 // accumulators occupy WH * ACC_STAGES * TN = 384 columns
    constexpr int DQ_PER_LD = WH == 1 ? 8 : 16;      // dequantiser warps that read one shared-memory stage
    static_assert(WH * ACC_STAGES * TN == 384, "tensor-memory plan");

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + OFF_BAR);
    uint64_t* ld_full = bars;                       // [LD_STAGES]
    uint64_t* ld_empty = ld_full + LD_STAGES;       // [LD_STAGES]
    uint64_t* a_full = ld_empty + LD_STAGES;        // [8]
    uint64_t* a_empty = a_full + 8;                 // [8]
    uint64_t* acc_full = a_empty + 8;               // [2]
    uint64_t* acc_empty = acc_full + 2;             // [2]
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int i = 0; i < LD_STAGES; ++i) {
            mbar_init(&ld_full[i], 1);
            mbar_init(&ld_empty[i], 1 + DQ_PER_LD);
        }
        for (int i = 0; i < A_STAGES; ++i) {
            mbar_init(&a_full[i], 8);
            mbar_init(&a_empty[i], 1);
        }
        for (int i = 0; i < ACC_STAGES; ++i) {
            mbar_init(&acc_full[i], 1);
            mbar_init(&acc_empty[i], EPI_WARPS);
        }
        *abort_flag = 0;
        fence_mbar_init();
    }
    if (warp == 2) {
        tmem_alloc(tmem_slot, TMEM_COLS);
        tmem_relinquish();
    }
    if (warp == 0 && lane == 0) {
        tma_prefetch_desc(&map_x0);
        if (P.total_tiles > P.tiles0) tma_prefetch_desc(&map_x1);
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ---------------------------------------------------------- producer
        uint32_t s = 0, ph = 0;
        bool ok = true;
        for (int t = blockIdx.x; ok && t < P.total_tiles; t += gridDim.x) {
            const TileCoord tc = tile_coord(P, t, WH);
            const Problem& pr = tc.prob ? P.p[1] : P.p[0];
            const int ksteps_all = pr.K / BK;
            const int k_first = tc.kpart * (ksteps_all / pr.ksplit);
            const int k_last = k_first + ksteps_all / pr.ksplit;
            const CUtensorMap* mx = tc.prob ? &map_x1 : &map_x0;
            const uint8_t* wsrc = pr.tiles + (long long)tc.n_tile * ksteps_all * kWBytes;
            for (int ks = k_first; ks < k_last; ++ks) {
                if (!mbar_wait(&ld_empty[s], ph ^ 1u, abort_flag, P.err)) {
                    ok = false;
                    break;
                }
                if (elect_one()) {
                    uint8_t* stage = smem + s * STAGE_BYTES;
                    mbar_arrive_expect_tx(&ld_full[s], kTxBytes);
                    tma_load_2d(stage, mx, &ld_full[s], ks * BK, tc.m0);
#pragma unroll
                    for (int hw = 0; hw < WH; ++hw) {
                        bulk_load_1d(stage + X_BYTES + hw * W_BYTES_MAX,
                                  wsrc + ((long long)hw * ksteps_all + ks) * kWBytes, kWBytes, &ld_full[s]);
                    }
                }
                __syncwarp();
                if (++s == LD_STAGES) {
                    s = 0;
                    ph ^= 1u;
                }
            }
        }
    } else if (warp == 1) {
        // -------------------------------------------------------- MMA issuer
        // tcgen05 instructions are issued under elect.sync: issuing them from an
        // `if (lane == 0)` branch costs ~100 cycles per batch on B200.
        const uint32_t idesc = make_idesc(kDFmtF32, kFmtF16, kFmtF16, 0, 0, TW, TN);
        uint32_t s = 0, ph = 0, as = 0, aph = 0, cs = 0, cph = 0;
        bool ok = true;
        for (int t = blockIdx.x; ok && t < P.total_tiles; t += gridDim.x) {
            const TileCoord tc = tile_coord(P, t, WH);
            const int ksteps = (tc.prob ? P.p[1].K / P.p[1].ksplit : P.p[0].K / P.p[0].ksplit) / BK;
            if (!mbar_wait(&acc_empty[cs], cph ^ 1u, abort_flag, P.err)) {
                ok = false;
                break;
            }
            tc_fence_after_sync();
            const uint32_t tmem_d = tmem_base + TMEM_ACC + cs * (WH * TN);
            for (int ks = 0; ok && ks < ksteps; ++ks) {
                if (!mbar_wait(&ld_full[s], ph, abort_flag, P.err)) {
                    ok = false;
                    break;
                }
                const uint32_t x_addr = smem_u32(smem + s * STAGE_BYTES);
#pragma unroll
                for (int kh = 0; kh < BK / AKW; ++kh) {
                    if (!mbar_wait(&a_full[as], aph, abort_flag, P.err)) {
                        ok = false;
                        break;
                    }
                    tc_fence_after_sync();
                    if (elect_one()) {
#pragma unroll
                        for (int j = 0; j < AKW / 16; ++j) {
                            const uint64_t bd = make_smem_desc_sw128(x_addr + (kh * (AKW / 16) + j) * 32, 16, 1024);
#pragma unroll
                            for (int hw = 0; hw < WH; ++hw) {
                                // WH = 2: columns [hw*16 + j*8 ...) ; WH = 1: columns [j*8 ...) of the stage
                                const uint32_t a_tmem = tmem_base + TMEM_A + as * A_COLS + hw * 16 + j * 8;
                                mma_f16_ts(tmem_d + hw * TN, a_tmem, bd, idesc, (ks > 0 || kh > 0 || j > 0) ? 1u : 0u);
                            }
                        }
                        mma_commit(&a_empty[as]);
                        if (kh == BK / AKW - 1) mma_commit(&ld_empty[s]);
                    }
                    __syncwarp();
                    if (++as == A_STAGES) {
                        as = 0;
                        aph ^= 1u;
                    }
                }
                if (++s == LD_STAGES) {
                    s = 0;
                    ph ^= 1u;
                }
            }
            if (!ok) break;
            if (elect_one()) mma_commit(&acc_full[cs]);
            __syncwarp();
            if (++cs == ACC_STAGES) {
                cs = 0;
                cph ^= 1u;
            }
        }
    } else if (warp >= 4 && warp < 12) {
        // ----------------------------------------------------------- epilogue
        // WH = 2: warps 4-7 drain weight half 0, warps 8-11 half 1.
        // WH = 1: both warp sets drain the one half, alternating 16-token steps.
        const int quarter = warp & 3;
        const int set = warp >= 8 ? 1 : 0;
        const int hw = WH == 2 ? set : 0;
        uint32_t cs = 0, cph = 0;
        bool ok = true;
        for (int t = blockIdx.x; ok && t < P.total_tiles; t += gridDim.x) {
            const TileCoord tc = tile_coord(P, t, WH);
            const Problem& pr = tc.prob ? P.p[1] : P.p[0];
            if (!mbar_wait(&acc_full[cs], cph, abort_flag, P.err)) {
                ok = false;
                break;
            }
            tc_fence_after_sync();
            const int n = (tc.n_tile + hw) * TW + quarter * 32 + lane;
            const bool n_ok = n < pr.N;
            const uint32_t taddr =
                tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + TMEM_ACC + (cs * WH + hw) * TN;
            if ((tc.n_tile + hw) * TW < pr.N) {   // uniform: the whole half may lie beyond N
#pragma unroll 1
                for (int c = (WH == 1 ? set : 0); c < TN / EC; c += (WH == 1 ? 2 : 1)) {
                    const int m_first = tc.m0 + c * EC;
                    if (m_first >= pr.M) break;   // uniform
                    uint32_t r[EC];
                    tmem_ld_32x32b_x16(taddr + c * EC, r);
                    tmem_wait_ld();
                    float v[EC];
#pragma unroll
                    for (int j = 0; j < EC; ++j) v[j] = __uint_as_float(r[j]);
                    epilogue_store(pr, v, n, m_first, n_ok, tc.kpart);
                }
            }
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(&acc_empty[cs]);
            if (++cs == ACC_STAGES) {
                cs = 0;
                cph ^= 1u;
            }
        }
    } else if (warp >= 12) {
        // -------------------------------------------------------- dequantisers
        // Every warp converts 32 k of 32 weight rows per job and has a whole 64-k
        // stage's MMA time (or two, WH = 1) for its load -> convert -> tcgen05.st ->
        // arrive chain, so the chain's latency stays off the tensor pipe's critical path.
        //   WH = 2: warp = (lane quarter, weight half, k half), works on every stage
        //   WH = 1: warp = (lane quarter, k half, stage parity), works on every other stage
        const int quarter = warp & 3;
        const int b2 = ((warp - 12) >> 2) & 1;
        const int b3 = (warp - 12) >> 3;
        const int hw = WH == 2 ? b2 : 0;
        const int kh = WH == 2 ? b3 : b2;
        const uint32_t par = WH == 2 ? 0u : static_cast<uint32_t>(b3);
        const int r = quarter * 32 + lane;       // weight row of the tile = tensor-memory lane
        const uint32_t lane_base = static_cast<uint32_t>(quarter * 32) << 16;
        uint32_t g = 0;   // 64-k stages seen so far (all tiles)
        bool ok = true;
        for (int t = blockIdx.x; ok && t < P.total_tiles; t += gridDim.x) {
            const TileCoord tc = tile_coord(P, t, WH);
            const int ksteps = (tc.prob ? P.p[1].K / P.p[1].ksplit : P.p[0].K / P.p[0].ksplit) / BK;
            for (int ks = 0; ok && ks < ksteps; ++ks, ++g) {
                if (WH == 1 && (g & 1u) != par) continue;
                const uint32_t s = g % LD_STAGES;
                const uint32_t ph = (g / LD_STAGES) & 1u;
                if (!mbar_wait(&ld_full[s], ph, abort_flag, P.err)) {
                    ok = false;
                    break;
                }
                const uint8_t* tile = smem + s * STAGE_BYTES + X_BYTES + hw * W_BYTES_MAX;
                uint32_t o[16];
                if (kQ4) {
                    dequant_q4_k(tile, r, kh, o);
                } else {
                    dequant_q8_0(tile, r, kh, o);
                }
                const uint32_t ai = WH == 2 ? 2u * g + kh : g;   // running A stage number
                const uint32_t as = ai % A_STAGES;
                const uint32_t aph = (ai / A_STAGES) & 1u;
                if (!mbar_wait(&a_empty[as], aph ^ 1u, abort_flag, P.err)) {
                    ok = false;
                    break;
                }
                tc_fence_after_sync();
                tmem_st_32x32b_x16(tmem_base + lane_base + TMEM_A + as * A_COLS + (WH == 2 ? hw : kh) * 16, o);
                tmem_wait_st();
                tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) {
                    mbar_arrive(&a_full[as]);
                    mbar_arrive(&ld_empty[s]);
                }
            }
        }
    }

    // ---------------------------------------------------------------- teardown
    tc_fence_before_sync();
    __syncthreads();
    if (*abort_flag) {
        // Give copies and MMAs still in flight time to land before the CTA's
        // shared and tensor memory are released.
        for (int i = 0; i < 200; ++i) __nanosleep(1000);
        __syncthreads();
    }
    if (warp == 2) {
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, TMEM_COLS);
    }
}

// ------------------------------------------------------------------------------------------------
// The same GEMM on CTA pairs (a cluster of two CTAs on neighbouring SMs, tcgen05 .cta_group::2).
//
// A pair computes 256 weight rows x 192 tokens.  Each CTA owns one 128-row weight tile (raw record in its
// shared memory, dequantised into its tensor memory, accumulators in its tensor memory, its own epilogue)
// and stages only HALF of the token tile: 96 tokens x 64 k = 12 KB per k-step instead of 24 KB.  One
// 256 x 192 x 16 MMA issued by the leader CTA reads rows 0-95 of B from the leader's shared memory and rows
// 96-191 from the peer's.  Per SM and k-step the shared-memory traffic drops from about 65 KB (24 KB TMA
// write + 24 KB MMA read + 2 x 8.5 KB weights) to about 41 KB for the same 384 tensor clocks, which takes
// the single-CTA kernel's limit (the 128 B/clk shared-memory port) out of the way.
//
// Signals across the pair (all others stay inside a CTA):
//   a_full     16 arrivals on the LEADER's barrier: the 8 dequantiser warps of either CTA.  A dequantiser
//              arrives only after it has seen its own CTA's ld_full for that stage, so a_full also tells
//              the leader that both halves of the token tile have landed.
//   a_empty, ld_empty, acc_full   tcgen05.commit signalling the barrier of the same name in both CTAs
//   acc_empty  16 arrivals on the leader's barrier: the 8 epilogue warps of either CTA
// Loads are addressed to the issuing CTA only.
#ifdef EDB200_GEMM_STATS
// Tuning build only: cycles spent waiting, per role, of the first pair of a launch.
__device__ long long g_pair_stats[16];
#define PAIR_STAT_T0() const long long stat_t0 = clock64()
#define PAIR_STAT_ADD(acc) acc += clock64() - stat_t0
#define PAIR_STAT_FLUSH(slot, v) atomicAdd(reinterpret_cast<unsigned long long*>(&g_pair_stats[slot]), (unsigned long long)(v))
#else
#define PAIR_STAT_T0()
#define PAIR_STAT_ADD(acc)
#define PAIR_STAT_FLUSH(slot, v)
#endif

constexpr int PAIR_TOK = TN / 2;                                  // tokens staged per CTA
constexpr int PAIR_X_BYTES = PAIR_TOK * BK * 2;                   // 12 KB
constexpr int PAIR_STAGE_BYTES = PAIR_X_BYTES + 9 * 1024;         // + one weight tile record, 1 KB granular
constexpr int PAIR_LD_STAGES = 8;
constexpr int PAIR_OFF_STAGE = PAIR_LD_STAGES * PAIR_STAGE_BYTES;    // epilogue transposition: 2 sets x 2 buffers
constexpr int PAIR_STAGE_OUT_BYTES = 2 * 2 * EC * TW * 4;           //   of 16 tokens x 128 features f32 (32 KB)
constexpr int PAIR_OFF_BAR = PAIR_OFF_STAGE + PAIR_STAGE_OUT_BYTES;
constexpr int PAIR_SMEM_BYTES = PAIR_OFF_BAR + 512 + 1024;
static_assert(PAIR_SMEM_BYTES <= 227 * 1024, "shared memory plan");
static_assert(W_BYTES_MAX <= 9 * 1024, "weight tile record must fit its slot");

// Epilogue of a weight tile that holds one head (D 128) or two heads (D 64) of q, k or v: RMSNorm over the head's
// features and the rotary embedding on the f32 accumulators, then f16 rows of the head-major attention operand
// (edb200_qk_pack_t).  Run by the 128 threads of one epilogue warp set; after the transposition through `stage`
// a token's 128 features sit in 8 neighbouring lanes, 2 x 8 each (features cc*8.. and 64 + cc*8..: with D 64 one
// group per head).
template <int D>
__device__ __forceinline__ void pack_qkv_tile(const Problem& pr, float* stage, uint32_t& buf, uint32_t taddr, int set,
                                              int tid, int n0, int n, bool n_ok, int m0) {
    const int blk = n0 / (pr.pk_heads * D);
    const int which = pr.pk_first + blk;                   // 0 q, 1 k, 2 v
    const int head0 = (n0 - blk * pr.pk_heads * D) / D;    // first head of the tile
    const float* wn = which == 0 ? pr.pk_qw : which == 1 ? pr.pk_kw : nullptr;
    const bool rope = which < 2 && pr.pk_pe != nullptr;
    const float bias_v = (pr.bias != nullptr && n_ok) ? __ldg(pr.bias + n) : 0.0f;
    const int row = tid >> 3, cc = tid & 7;
#pragma unroll 1
    for (int c = set; c < TN / EC; c += 2) {
        const int m_first = m0 + c * EC;
        if (m_first >= pr.M) break;   // uniform over the set
        uint32_t r[EC];
        tmem_ld_32x32b_x16(taddr + c * EC, r);
        tmem_wait_ld();
        float* st = stage + buf * (EC * TW);
#pragma unroll
        for (int j = 0; j < EC; ++j) st[j * TW + tid] = __uint_as_float(r[j]) + bias_v;
        named_bar_sync(1u + static_cast<uint32_t>(set), 128u);
        const long long m = m_first + row;
        const long long mc = m < pr.M ? m : pr.M - 1;   // rows past the end compute on the last row, store nothing
        float v[16];
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            const float* sp = st + row * TW + j * 64 + cc * 8;
            const float4 a = *reinterpret_cast<const float4*>(sp);
            const float4 b = *reinterpret_cast<const float4*>(sp + 4);
            v[8 * j + 0] = a.x, v[8 * j + 1] = a.y, v[8 * j + 2] = a.z, v[8 * j + 3] = a.w;
            v[8 * j + 4] = b.x, v[8 * j + 5] = b.y, v[8 * j + 6] = b.z, v[8 * j + 7] = b.w;
        }
        if (wn != nullptr) {   // uniform
            float ss[2] = {0.0f, 0.0f};
#pragma unroll
            for (int j = 0; j < 2; ++j) {
#pragma unroll
                for (int e = 0; e < 8; ++e) ss[j] += v[8 * j + e] * v[8 * j + e];
            }
            if (D == TW) ss[0] = ss[1] = ss[0] + ss[1];
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                if (D == TW && j == 1) {
                    ss[1] = ss[0];
                } else {
                    ss[j] += __shfl_xor_sync(0xffffffffu, ss[j], 1);
                    ss[j] += __shfl_xor_sync(0xffffffffu, ss[j], 2);
                    ss[j] += __shfl_xor_sync(0xffffffffu, ss[j], 4);
                }
                const float sc = 1.0f / sqrtf(ss[j] / static_cast<float>(D) + pr.pk_eps);
                const int fh = (D == TW ? j * 64 : 0) + cc * 8;     // feature within the head
                const float4 wa = __ldg(reinterpret_cast<const float4*>(wn + fh));
                const float4 wb = __ldg(reinterpret_cast<const float4*>(wn + fh + 4));
                v[8 * j + 0] = (v[8 * j + 0] * sc) * wa.x, v[8 * j + 1] = (v[8 * j + 1] * sc) * wa.y;
                v[8 * j + 2] = (v[8 * j + 2] * sc) * wa.z, v[8 * j + 3] = (v[8 * j + 3] * sc) * wa.w;
                v[8 * j + 4] = (v[8 * j + 4] * sc) * wb.x, v[8 * j + 5] = (v[8 * j + 5] * sc) * wb.y;
                v[8 * j + 6] = (v[8 * j + 6] * sc) * wb.z, v[8 * j + 7] = (v[8 * j + 7] * sc) * wb.w;
            }
        }
        if (rope) {   // uniform
            const float4* pp = reinterpret_cast<const float4*>(pr.pk_pe) + (pr.pk_pe_row0 + mc) * (D / 2);
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                const int fh = (D == TW ? j * 64 : 0) + cc * 8;
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const float4 mt = __ldg(pp + fh / 2 + q);   // pe00, pe10, pe01, pe11
                    const float x0 = v[8 * j + 2 * q], x1 = v[8 * j + 2 * q + 1];
                    v[8 * j + 2 * q] = __fadd_rn(__fmul_rn(x0, mt.x), __fmul_rn(x1, mt.y));
                    v[8 * j + 2 * q + 1] = __fadd_rn(__fmul_rn(x0, mt.z), __fmul_rn(x1, mt.w));
                }
            }
        }
        if (m < pr.M) {
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                const int head = head0 + (D == TW ? 0 : j);
                const int fh = (D == TW ? j * 64 : 0) + cc * 8;
                const int dst_rank = pr.pk_hp > 0 ? head / pr.pk_hp : 0;
                const int head_l = pr.pk_hp > 0 ? head % pr.pk_hp : head;
                __half* dst = reinterpret_cast<__half*>(pr.pk_dst[which][dst_rank]) +
                              ((long long)head_l * pr.pk_ltotal + pr.pk_pos0 + m) * D + fh;
                uint4 o;
                __half2 h0 = __floats2half2_rn(v[8 * j + 0], v[8 * j + 1]);
                __half2 h1 = __floats2half2_rn(v[8 * j + 2], v[8 * j + 3]);
                __half2 h2 = __floats2half2_rn(v[8 * j + 4], v[8 * j + 5]);
                __half2 h3 = __floats2half2_rn(v[8 * j + 6], v[8 * j + 7]);
                o.x = *reinterpret_cast<uint32_t*>(&h0);
                o.y = *reinterpret_cast<uint32_t*>(&h1);
                o.z = *reinterpret_cast<uint32_t*>(&h2);
                o.w = *reinterpret_cast<uint32_t*>(&h3);
                *reinterpret_cast<uint4*>(dst) = o;
            }
        }
        buf ^= 1u;
    }
}

template <int WT, int DQ>   // DQ: 64-k stages whose conversion is in flight at once per CTA (2 or 4)
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(NUM_THREADS, 1)
qgemm_pair_kernel(const __grid_constant__ CUtensorMap map_x0, const __grid_constant__ CUtensorMap map_x1,
                  const __grid_constant__ Params P) {
    constexpr bool kQ4 = (WT == EDB200_TYPE_Q4_K);
    constexpr uint32_t kWBytes = kQ4 ? kQwTileBytesQ4 : kQwTileBytesQ8;
    constexpr uint32_t kTxBytes = PAIR_X_BYTES + kWBytes;
    constexpr int ACC_STAGES = 2;
    constexpr int A_COLS = 32;            // tensor-memory columns of one A stage: 64 k of the CTA's 128 rows
    constexpr int A_STAGES = 4;
    constexpr uint32_t TMEM_A = 384;      // accumulators: 2 stages x 192 columns
    constexpr int LDS = PAIR_LD_STAGES;

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + PAIR_OFF_BAR);
    uint64_t* ld_full = bars;                       // [LDS]
    uint64_t* ld_empty = ld_full + LDS;             // [LDS]
    uint64_t* a_full = ld_empty + LDS;              // [4]  (the leader's are used)
    uint64_t* a_empty = a_full + A_STAGES;          // [4]
    uint64_t* acc_full = a_empty + A_STAGES;        // [2]
    uint64_t* acc_empty = acc_full + ACC_STAGES;    // [2]  (the leader's are used)
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + ACC_STAGES);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();        // 0: leader (issues the MMAs), 1: peer
    const int pair = blockIdx.x >> 1;
    const int n_pairs = gridDim.x >> 1;

    if (threadIdx.x == 0) {
        for (int i = 0; i < LDS; ++i) {
            mbar_init(&ld_full[i], 1);
            mbar_init(&ld_empty[i], 1 + 16 / DQ);    // the commit + this CTA's dequantiser warps of the stage
        }
        for (int i = 0; i < A_STAGES; ++i) {
            mbar_init(&a_full[i], 2 * (16 / DQ));   // the stage's dequantiser warps of both CTAs
            mbar_init(&a_empty[i], 1);
        }
        for (int i = 0; i < ACC_STAGES; ++i) {
            mbar_init(&acc_full[i], 1);
            mbar_init(&acc_empty[i], 2 * EPI_WARPS);
        }
        *abort_flag = 0;
        fence_mbar_init();
    }
    if (warp == 2) {
        tmem_alloc_pair(tmem_slot, TMEM_COLS);
        tmem_relinquish_pair();
    }
    if (warp == 0 && lane == 0) {
        tma_prefetch_desc(&map_x0);
        if (P.total_tiles > P.tiles0) tma_prefetch_desc(&map_x1);
    }
    tc_fence_before_sync();
    __syncthreads();
    cluster_sync_all();     // the peer's barriers are initialised before anything arrives on them
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ---------------------------------------------------------- producer (both CTAs)
        uint32_t s = 0, ph = 0;
        bool ok = true;
        long long st_wait = 0;
        (void)st_wait;
        for (int t = pair; ok && t < P.total_tiles; t += n_pairs) {
            const TileCoord tc = tile_coord(P, t, 2);
            const Problem& pr = tc.prob ? P.p[1] : P.p[0];
            const int ksteps_all = pr.K / BK;
            const int k_first = tc.kpart * (ksteps_all / pr.ksplit);
            const int k_last = k_first + ksteps_all / pr.ksplit;
            const CUtensorMap* mx = tc.prob ? &map_x1 : &map_x0;
            const uint8_t* wsrc = pr.tiles + (long long)(tc.n_tile + (int)rank) * ksteps_all * kWBytes;
            const int m_half = tc.m0 + (int)rank * PAIR_TOK;
            for (int ks = k_first; ks < k_last; ++ks) {
                PAIR_STAT_T0();
                if (!mbar_wait(&ld_empty[s], ph ^ 1u, abort_flag, P.err)) {
                    ok = false;
                    break;
                }
                PAIR_STAT_ADD(st_wait);
                if (elect_one()) {
                    uint8_t* stage = smem + s * PAIR_STAGE_BYTES;
                    mbar_arrive_expect_tx(&ld_full[s], kTxBytes);
                    tma_load_2d(stage, mx, &ld_full[s], ks * BK, m_half);
                    bulk_load_1d(stage + PAIR_X_BYTES, wsrc + (long long)ks * kWBytes, kWBytes, &ld_full[s]);
                }
                __syncwarp();
                if (++s == LDS) {
                    s = 0;
                    ph ^= 1u;
                }
            }
        }
        if (blockIdx.x < 2 && lane == 0) PAIR_STAT_FLUSH(3 + 8 * rank, st_wait);
    } else if (warp == 1) {
        // -------------------------------------------------------- MMA issuer (leader CTA only)
        if (rank == 0) {
            const uint32_t idesc = make_idesc(kDFmtF32, kFmtF16, kFmtF16, 0, 0, 2 * TW, TN);
            uint32_t s = 0, as = 0, aph = 0, cs = 0, cph = 0;
            bool ok = true;
            long long st_acc = 0, st_a = 0;
            (void)st_acc;
            (void)st_a;
#ifdef EDB200_GEMM_STATS
            const long long st_begin = clock64();
#endif
            for (int t = pair; ok && t < P.total_tiles; t += n_pairs) {
                const TileCoord tc = tile_coord(P, t, 2);
                const int ksteps = (tc.prob ? P.p[1].K / P.p[1].ksplit : P.p[0].K / P.p[0].ksplit) / BK;
                {
                    PAIR_STAT_T0();
                    if (!mbar_wait(&acc_empty[cs], cph ^ 1u, abort_flag, P.err)) {
                        ok = false;
                        break;
                    }
                    PAIR_STAT_ADD(st_acc);
                }
                tc_fence_after_sync();
                const uint32_t tmem_d = tmem_base + TMEM_ACC + cs * TN;
                for (int ks = 0; ok && ks < ksteps; ++ks) {
                    {
                        PAIR_STAT_T0();
                        if (!mbar_wait(&a_full[as], aph, abort_flag, P.err)) {
                            ok = false;
                            break;
                        }
                        PAIR_STAT_ADD(st_a);
                    }
                    tc_fence_after_sync();
                    if (elect_one()) {
                        const uint32_t x_addr = smem_u32(smem + s * PAIR_STAGE_BYTES);
#pragma unroll
                        for (int j = 0; j < BK / 16; ++j) {
                            const uint64_t bd = make_smem_desc_sw128(x_addr + j * 32, 16, 1024);
                            mma_f16_ts_pair(tmem_d, tmem_base + TMEM_A + as * A_COLS + j * 8, bd, idesc,
                                            (ks > 0 || j > 0) ? 1u : 0u);
                        }
                        mma_commit_pair(&a_empty[as]);
                        mma_commit_pair(&ld_empty[s]);
                    }
                    __syncwarp();
                    if (++as == A_STAGES) {
                        as = 0;
                        aph ^= 1u;
                    }
                    if (++s == LDS) s = 0;
                }
                if (!ok) break;
                if (elect_one()) mma_commit_pair(&acc_full[cs]);
                __syncwarp();
                if (++cs == ACC_STAGES) {
                    cs = 0;
                    cph ^= 1u;
                }
            }
#ifdef EDB200_GEMM_STATS
            if (blockIdx.x == 0 && lane == 0) {
                PAIR_STAT_FLUSH(0, clock64() - st_begin);
                PAIR_STAT_FLUSH(1, st_acc);
                PAIR_STAT_FLUSH(2, st_a);
            }
#endif
        }
    } else if (warp >= 4 && warp < 12) {
        // ----------------------------------------------------------- epilogue (both CTAs, own weight rows)
        const int quarter = warp & 3;
        const int set = warp >= 8 ? 1 : 0;   // the two warp sets alternate 16-token steps
        const int tid = quarter * 32 + lane;  // thread of the set
        float* stage = reinterpret_cast<float*>(smem + PAIR_OFF_STAGE) + set * (2 * EC * TW);
        uint32_t buf = 0;
        uint32_t cs = 0, cph = 0;
        bool ok = true;
        long long st_wait = 0, st_busy = 0;
        (void)st_wait;
        (void)st_busy;
        for (int t = pair; ok && t < P.total_tiles; t += n_pairs) {
            const TileCoord tc = tile_coord(P, t, 2);
            const Problem& pr = tc.prob ? P.p[1] : P.p[0];
            {
                PAIR_STAT_T0();
                if (!mbar_wait(&acc_full[cs], cph, abort_flag, P.err)) {
                    ok = false;
                    break;
                }
                PAIR_STAT_ADD(st_wait);
            }
            PAIR_STAT_T0();
            tc_fence_after_sync();
            const int n_tile = tc.n_tile + (int)rank;
            const int n0 = n_tile * TW;
            const int n = n0 + tid;                  // this thread's weight row = its tensor-memory lane
            const bool n_ok = n < pr.N;
            const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + TMEM_ACC + cs * TN;
            if (n0 < pr.N && pr.ksplit > 1) {
                // split reduction: atomic adds, one output feature per lane
#pragma unroll 1
                for (int c = set; c < TN / EC; c += 2) {
                    const int m_first = tc.m0 + c * EC;
                    if (m_first >= pr.M) break;   // uniform
                    uint32_t r[EC];
                    tmem_ld_32x32b_x16(taddr + c * EC, r);
                    tmem_wait_ld();
                    float v[EC];
#pragma unroll
                    for (int j = 0; j < EC; ++j) v[j] = __uint_as_float(r[j]);
                    epilogue_store(pr, v, n, m_first, n_ok, tc.kpart);
                }
            } else if (n0 < pr.n_pack) {
                // one head (or two) of q, k or v: norm, rotary embedding and the head-major store happen here
                if (pr.pk_d == TW) {
                    pack_qkv_tile<TW>(pr, stage, buf, taddr, set, tid, n0, n, n_ok, tc.m0);
                } else {
                    pack_qkv_tile<64>(pr, stage, buf, taddr, set, tid, n0, n, n_ok, tc.m0);
                }
            } else if (n0 < pr.N) {   // uniform: the whole weight tile may lie beyond N
                // The accumulators arrive one output feature per lane, 16 tokens per step; memory wants whole
                // 128-byte lines of one token's consecutive features.  Each warp set transposes its 16 x 128
                // step through shared memory (two buffers, one named barrier per step) and stores 16 bytes
                // per thread: a lane-per-feature store of 64 B per token row ran at a seventh of this rate.
                const bool second = (pr.split_n > 0) && (n0 >= pr.split_n);   // tile-uniform: split_n % 128 == 0
                const int act = second ? pr.act2 : pr.act;
                const int dt = second ? pr.out2_dtype : pr.out_dtype;
                const long long ld = second ? pr.ldo2 : pr.ldo;
                const long long col0 = second ? (n0 - pr.split_n) : n0;
                char* obase = reinterpret_cast<char*>(second ? pr.out2 : pr.out);
                const bool gated = !second && pr.gate != nullptr;
                const float bias_v = (pr.bias != nullptr && n_ok) ? __ldg(pr.bias + n) : 0.0f;
                const int row = tid >> 3, cc = tid & 7;
#pragma unroll 1
                for (int c = set; c < TN / EC; c += 2) {
                    const int m_first = tc.m0 + c * EC;
                    if (m_first >= pr.M) break;   // uniform over the set
                    uint32_t r[EC];
                    tmem_ld_32x32b_x16(taddr + c * EC, r);
                    tmem_wait_ld();
                    float* st = stage + buf * (EC * TW);
                    if (dt == EDB200_TYPE_F32) {
#pragma unroll
                        for (int j = 0; j < EC; ++j) st[j * TW + tid] = apply_act(__uint_as_float(r[j]) + bias_v, act);
                    } else if (dt == EDB200_TYPE_BF16) {
                        __nv_bfloat16* sh = reinterpret_cast<__nv_bfloat16*>(st);
#pragma unroll
                        for (int j = 0; j < EC; ++j) {
                            sh[j * TW + tid] = __float2bfloat16_rn(apply_act(__uint_as_float(r[j]) + bias_v, act));
                        }
                    } else {
                        __half* sh = reinterpret_cast<__half*>(st);
#pragma unroll
                        for (int j = 0; j < EC; ++j) {
                            sh[j * TW + tid] = __float2half_rn(apply_act(__uint_as_float(r[j]) + bias_v, act));
                        }
                    }
                    named_bar_sync(1u + static_cast<uint32_t>(set), 128u);
                    const long long m = m_first + row;
                    if (m < pr.M) {
                        if (dt == EDB200_TYPE_F32) {
                            float* orow = reinterpret_cast<float*>(obase) + m * ld + col0;
#pragma unroll
                            for (int j = 0; j < 4; ++j) {
                                const int nl = j * 32 + cc * 4;
                                if (n0 + nl >= pr.N) continue;
                                float4 x = *reinterpret_cast<const float4*>(st + row * TW + nl);
                                if (gated) {
                                    const float4 g = __ldg(reinterpret_cast<const float4*>(pr.gate + n0 + nl));
                                    const float4 q = *reinterpret_cast<const float4*>(pr.residual + m * pr.ld_res + n0 + nl);
                                    x.x = q.x + g.x * x.x;
                                    x.y = q.y + g.y * x.y;
                                    x.z = q.z + g.z * x.z;
                                    x.w = q.w + g.w * x.w;
                                }
                                *reinterpret_cast<float4*>(orow + nl) = x;
                            }
                        } else {
                            const uint16_t* sh = reinterpret_cast<const uint16_t*>(st);
                            uint16_t* orow = reinterpret_cast<uint16_t*>(obase) + m * ld + col0;
#pragma unroll
                            for (int j = 0; j < 2; ++j) {
                                const int nl = j * 64 + cc * 8;
                                if (n0 + nl >= pr.N) continue;
                                *reinterpret_cast<uint4*>(orow + nl) = *reinterpret_cast<const uint4*>(sh + row * TW + nl);
                            }
                        }
                    }
                    buf ^= 1u;
                }
            }
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive_leader(&acc_empty[cs]);
            PAIR_STAT_ADD(st_busy);
            if (++cs == ACC_STAGES) {
                cs = 0;
                cph ^= 1u;
            }
        }
        if (blockIdx.x < 2 && warp == 4 && lane == 0) {
            PAIR_STAT_FLUSH(6 + 8 * rank, st_wait);
            PAIR_STAT_FLUSH(7 + 8 * rank, st_busy);
        }
    } else if (warp >= 12) {
        // -------------------------------------------------------- dequantisers (both CTAs, own weight tile)
        // DQ = 2: warp = (lane quarter, k half, stage parity): 32 rows x 32 k per job, every other 64-k stage.
        // DQ = 4: warp = (lane quarter, stage mod 4): 32 rows x 64 k per job (two stores, one wait), every fourth
        //         stage - as many conversions in flight as there are A stages, so the chain load -> convert ->
        //         tcgen05.st -> wait -> arrive of one stage has four stages' tensor time to complete.
        const int quarter = warp & 3;
        const int kh0 = DQ == 2 ? ((warp - 12) >> 2) & 1 : 0;
        const uint32_t slot = DQ == 2 ? static_cast<uint32_t>((warp - 12) >> 3) : static_cast<uint32_t>((warp - 12) >> 2);
        const int r = quarter * 32 + lane;       // weight row of the tile = tensor-memory lane
        const uint32_t lane_base = static_cast<uint32_t>(quarter * 32) << 16;
        uint32_t g = 0;   // 64-k stages seen so far (all tiles)
        bool ok = true;
        long long st_ld = 0, st_a = 0;
        (void)st_ld;
        (void)st_a;
        for (int t = pair; ok && t < P.total_tiles; t += n_pairs) {
            const TileCoord tc = tile_coord(P, t, 2);
            const int ksteps = (tc.prob ? P.p[1].K / P.p[1].ksplit : P.p[0].K / P.p[0].ksplit) / BK;
            for (int ks = 0; ok && ks < ksteps; ++ks, ++g) {
                if ((g % DQ) != slot) continue;
                const uint32_t s = g % LDS;
                const uint32_t ph = (g / LDS) & 1u;
                {
                    PAIR_STAT_T0();
                    if (!mbar_wait(&ld_full[s], ph, abort_flag, P.err)) {
                        ok = false;
                        break;
                    }
                    PAIR_STAT_ADD(st_ld);
                }
                const uint8_t* tile = smem + s * PAIR_STAGE_BYTES + PAIR_X_BYTES;
                const uint32_t as = g % A_STAGES;
                const uint32_t aph = (g / A_STAGES) & 1u;
                uint32_t o[16];
                if (kQ4) {
                    dequant_q4_k(tile, r, kh0, o);
                } else {
                    dequant_q8_0(tile, r, kh0, o);
                }
                {
                    PAIR_STAT_T0();
                    if (!mbar_wait(&a_empty[as], aph ^ 1u, abort_flag, P.err)) {
                        ok = false;
                        break;
                    }
                    PAIR_STAT_ADD(st_a);
                }
                tc_fence_after_sync();
                tmem_st_32x32b_x16(tmem_base + lane_base + TMEM_A + as * A_COLS + kh0 * 16, o);
                if (DQ == 4) {   // the other 32 k of the same rows
                    if (kQ4) {
                        dequant_q4_k(tile, r, 1, o);
                    } else {
                        dequant_q8_0(tile, r, 1, o);
                    }
                    tmem_st_32x32b_x16(tmem_base + lane_base + TMEM_A + as * A_COLS + 16, o);
                }
                tmem_wait_st();
                tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) {
                    mbar_arrive_leader(&a_full[as]);
                    mbar_arrive(&ld_empty[s]);
                }
            }
        }
        if (blockIdx.x < 2 && warp == 12 && lane == 0) {
            PAIR_STAT_FLUSH(4 + 8 * rank, st_ld);
            PAIR_STAT_FLUSH(5 + 8 * rank, st_a);
        }
    }

    // ---------------------------------------------------------------- teardown
    tc_fence_before_sync();
    __syncthreads();
    if (*abort_flag) {
        // Give copies and MMAs still in flight time to land before shared and tensor memory are released.
        for (int i = 0; i < 200; ++i) __nanosleep(1000);
        __syncthreads();
    }
    // Neither CTA leaves while the other may still signal its barriers or the pair's MMAs read its memory.
    cluster_sync_all();
    if (warp == 2) {
        tc_fence_after_sync();
        tmem_dealloc_pair(tmem_base, TMEM_COLS);
    }
}

}  // namespace gemm


static edb200_status_t validate_problem(const edb200_qweight_t* w, const void* x, int64_t m, int64_t ldx,
                                        const edb200_epilogue_t* ep) {
    if (w == nullptr || x == nullptr || ep == nullptr || ep->out == nullptr) {
        return fail(EDB200_ERR_INVALID, "mul_mat_q: null argument");
    }
    if (m <= 0) return fail(EDB200_ERR_INVALID, "mul_mat_q: m must be positive");
    if (w->k % gemm::BK != 0) return fail(EDB200_ERR_UNSUPPORTED, "mul_mat_q: k must be a multiple of 64");
    if (w->n_out % 32 != 0) return fail(EDB200_ERR_UNSUPPORTED, "mul_mat_q: n_out must be a multiple of 32");
    if (ldx < w->k || (ldx * 2) % 16 != 0 || (reinterpret_cast<uintptr_t>(x) & 15u)) {
        return fail(EDB200_ERR_INVALID, "mul_mat_q: x rows must be 16-byte aligned and ldx >= k");
    }
    auto dt_ok = [](int dt) { return dt == EDB200_TYPE_F32 || dt == EDB200_TYPE_F16 || dt == EDB200_TYPE_BF16; };
    if (!dt_ok(ep->out_dtype)) return fail(EDB200_ERR_INVALID, "mul_mat_q: bad out_dtype");
    const int64_t n_primary = ep->split_n > 0 ? ep->split_n : w->n_out;
    const int esz = ep->out_dtype == EDB200_TYPE_F32 ? 4 : 2;
    if (ep->ldo < n_primary || (ep->ldo * esz) % 16 != 0 || (reinterpret_cast<uintptr_t>(ep->out) & 15u)) {
        return fail(EDB200_ERR_INVALID, "mul_mat_q: out rows must be 16-byte aligned and ldo >= columns");
    }
    if (ep->gate != nullptr) {
        if (ep->out_dtype != EDB200_TYPE_F32 || ep->residual == nullptr || (ep->ld_res % 4) != 0 ||
            (reinterpret_cast<uintptr_t>(ep->residual) & 15u) || (reinterpret_cast<uintptr_t>(ep->gate) & 15u)) {
            return fail(EDB200_ERR_INVALID, "mul_mat_q: gated residual needs f32 out, residual and aligned pointers");
        }
    }
    if (ep->split_k != EDB200_SPLIT_K_NEVER && ep->split_k != EDB200_SPLIT_K_UNORDERED) {
        return fail(EDB200_ERR_INVALID, "mul_mat_q: split_k must be EDB200_SPLIT_K_NEVER or EDB200_SPLIT_K_UNORDERED");
    }
    if (ep->bias != nullptr && (reinterpret_cast<uintptr_t>(ep->bias) & 15u)) {
        return fail(EDB200_ERR_INVALID, "mul_mat_q: bias must be 16-byte aligned");
    }
    if (ep->pack != nullptr) {
        const edb200_qk_pack_t& k = *ep->pack;
        const int64_t n_pack = (k.only ? 1ll : 3ll) * k.n_heads * k.d_head;
        const int64_t n_primary_cols = ep->split_n > 0 ? ep->split_n : w->n_out;
        if ((k.d_head != 128 && k.d_head != 64) || k.n_heads <= 0 || (k.n_heads * k.d_head) % 128 != 0 || k.only < 0 ||
            k.only > 3 || n_pack != n_primary_cols || ep->gate != nullptr ||
            ep->act != EDB200_ACT_NONE || ep->split_k != EDB200_SPLIT_K_NEVER || k.l_total <= 0 || k.tok_off < 0) {
            return fail(EDB200_ERR_INVALID,
                        "mul_mat_q: a fused q/k/v pack needs d_head 64 or 128 and (3 or 1) * n_heads * d_head plain primary columns");
        }
        auto al16 = [](const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15u) == 0; };
        if (!al16(k.q_weight) || !al16(k.k_weight) || !al16(k.pe)) {
            return fail(EDB200_ERR_INVALID, "mul_mat_q: pack weights and position table must be 16-byte aligned");
        }
        if (k.peers != nullptr) {
            const edb200_sp_peers_t& pp = *k.peers;
            if (pp.world <= 0 || pp.world > 8 || pp.rank < 0 || pp.rank >= pp.world || k.n_heads % pp.world ||
                (long long)pp.rank * pp.t_loc + k.tok_off + m > k.l_total) {
                return fail(EDB200_ERR_INVALID, "mul_mat_q: bad peer description of the fused pack");
            }
            for (int t = 0; t < 3; ++t) {
                for (int r = 0; r < pp.world; ++r) {
                    if (pp.buf[t][r] == nullptr || !al16(pp.buf[t][r])) {
                        return fail(EDB200_ERR_INVALID, "mul_mat_q: null or unaligned peer buffer of the fused pack");
                    }
                }
            }
        } else if (k.q_out == nullptr || k.k_out == nullptr || k.v_out == nullptr || !al16(k.q_out) || !al16(k.k_out) ||
                   !al16(k.v_out) || k.tok_off + m > k.l_total) {
            return fail(EDB200_ERR_INVALID, "mul_mat_q: pack outputs must be set, 16-byte aligned and hold tok_off + m rows");
        }
    }
    if (ep->split_n > 0) {
        if (ep->split_n % gemm::TW != 0 || ep->split_n >= w->n_out || ep->out2 == nullptr || !dt_ok(ep->out2_dtype)) {
            return fail(EDB200_ERR_INVALID, "mul_mat_q: split_n must be a multiple of 128 below n_out with out2 set");
        }
        const int esz2 = ep->out2_dtype == EDB200_TYPE_F32 ? 4 : 2;
        if (ep->ldo2 < w->n_out - ep->split_n || (ep->ldo2 * esz2) % 16 != 0 ||
            (reinterpret_cast<uintptr_t>(ep->out2) & 15u)) {
            return fail(EDB200_ERR_INVALID, "mul_mat_q: out2 rows must be 16-byte aligned");
        }
    }
    return EDB200_OK;
}

static void fill_problem(gemm::Problem& p, const edb200_qweight_t* w, int64_t m, const edb200_epilogue_t* ep,
                         int wh) {
    p.bias = ep->bias;
    p.out = ep->out;
    p.residual = ep->residual;
    p.gate = ep->gate;
    p.out2 = ep->out2;
    p.ldo = ep->ldo;
    p.ld_res = ep->ld_res;
    p.ldo2 = ep->ldo2;
    p.split_n = ep->split_n;
    p.out_dtype = ep->out_dtype;
    p.act = ep->act;
    p.out2_dtype = ep->out2_dtype;
    p.act2 = ep->act2;
    p.M = static_cast<int>(m);
    p.N = static_cast<int>(w->n_out);
    p.K = static_cast<int>(w->k);
    p.tiles = w->tiles;
    p.ksplit = 1;
    p.m_tiles = static_cast<int>((m + gemm::TN - 1) / gemm::TN);
    p.n_tiles = static_cast<int>((w->n_tiles + wh - 1) / wh);   // CTA tiles of `wh` weight tiles
    {
        // about 32 MB of f16 activations per chunk: a quarter of the 126 MB L2
        const int64_t per_tile = (int64_t)gemm::TN * w->k * 2;
        int64_t ch = (32ll << 20) / per_tile;
        if (ch < 4) ch = 4;
        if (ch > p.m_tiles) ch = p.m_tiles;
        p.chunk = static_cast<int>(ch);
    }
    p.n_pack = 0;
    if (ep->pack != nullptr) {
        const edb200_qk_pack_t& k = *ep->pack;
        p.n_pack = (k.only ? 1 : 3) * k.n_heads * k.d_head;
        p.pk_first = k.only ? k.only - 1 : 0;
        p.pk_heads = k.n_heads;
        p.pk_d = k.d_head;
        p.pk_eps = k.eps;
        p.pk_qw = k.q_weight;
        p.pk_kw = k.k_weight;
        p.pk_pe = k.pe;
        p.pk_pe_row0 = k.tok_off;
        p.pk_ltotal = k.l_total;
        if (k.peers != nullptr) {
            p.pk_hp = k.n_heads / k.peers->world;
            p.pk_pos0 = (long long)k.peers->rank * k.peers->t_loc + k.tok_off;
            for (int t = 0; t < 3; ++t) {
                for (int r = 0; r < k.peers->world; ++r) p.pk_dst[t][r] = k.peers->buf[t][r];
            }
        } else {
            p.pk_hp = 0;
            p.pk_pos0 = k.tok_off;
            p.pk_dst[0][0] = k.q_out;
            p.pk_dst[1][0] = k.k_out;
            p.pk_dst[2][0] = k.v_out;
        }
    }
}

static edb200_status_t launch_qgemm(int nprob, const edb200_qweight_t* const* ws, const void* const* xs,
                                    const int64_t* ms, const int64_t* ldxs, const edb200_epilogue_t* const* eps,
                                    int x_dtype, cudaStream_t stream) {
    // tcgen05 kind::f16 raises an illegal-instruction fault when the A and B
    // formats differ (measured on B200), and the dequantised weights are f16
    // (rn(d*q) keeps 11 significant bits), so activations must be f16 too.
    if (x_dtype != EDB200_TYPE_F16) {
        return fail(x_dtype == EDB200_TYPE_BF16 ? EDB200_ERR_UNSUPPORTED : EDB200_ERR_INVALID,
                    "mul_mat_q: x_dtype must be f16 (operands of one tcgen05.mma share a 16-bit format)");
    }
    for (int i = 0; i < nprob; ++i) {
        edb200_status_t st = validate_problem(ws[i], xs[i], ms[i], ldxs[i], eps[i]);
        if (st != EDB200_OK) return st;
        if (ws[i]->ggml_type != ws[0]->ggml_type) {
            return fail(EDB200_ERR_UNSUPPORTED, "mul_mat_q_pair: both weights must share one block type");
        }
    }
    int* err = device_error_word();
    if (err == nullptr) return fail(EDB200_ERR_CUDA, "mul_mat_q: no CUDA device");

    // Two weight tiles per CTA (least operand traffic, epilogue not overlapped) pay off
    // when the reduction is long; short reductions take one tile with double-buffered
    // accumulators.  EDB200_GEMM_WH=1|2 overrides the choice (tuning only).
    int wh = ws[0]->k >= 8192 ? 2 : 1;
    {
        static int force = -1;
        if (force < 0) {
            const char* e = getenv("EDB200_GEMM_WH");
            force = e ? atoi(e) : 0;
        }
        if (force == 1 || force == 2) wh = force;
    }
    // CTA pairs (256 weight rows x 192 tokens per pair, half the token tile staged per CTA) are the
    // default; EDB200_GEMM_PAIR=0 selects the single-CTA kernels (tuning and comparison only).
    static int pair_mode = -1;
    if (pair_mode < 0) {
        const char* e = getenv("EDB200_GEMM_PAIR");
        pair_mode = (e != nullptr && atoi(e) == 0) ? 0 : 1;
    }
    const bool pair = pair_mode == 1;
    if (pair) wh = 2;   // tile bookkeeping: two weight tiles per (pair) tile
    for (int i = 0; i < nprob; ++i) {
        if (eps[i]->pack != nullptr && !pair) {
            return fail(EDB200_ERR_UNSUPPORTED, "mul_mat_q: the fused q/k/v pack exists in the CTA-pair kernel only");
        }
    }
    gemm::Params P;
    memset(&P, 0, sizeof(P));
    CUtensorMap map_a[2];
    const CUtensorMapDataType adt =
        x_dtype == EDB200_TYPE_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    for (int i = 0; i < nprob; ++i) {
        fill_problem(P.p[i], ws[i], ms[i], eps[i], wh);
        edb200_status_t st = make_tmap_2d(&map_a[i], adt, 2, xs[i], (uint64_t)ws[i]->k, (uint64_t)ms[i],
                                          (uint64_t)ldxs[i] * 2, gemm::BK, pair ? gemm::PAIR_TOK : gemm::TN,
                                          CU_TENSOR_MAP_SWIZZLE_128B);
        if (st != EDB200_OK) return st;
    }
    if (nprob == 1) {
        map_a[1] = map_a[0];
        P.p[1].ksplit = 1;
    }
    // Long reductions into few outputs (the out-projections of a sequence-parallel rank) leave most
    // SMs without a tile.  When every problem of the launch asks for it (split_k =
    // EDB200_SPLIT_K_UNORDERED) and is an in-place gated residual, the reduction is cut into up to 4
    // parts, each a tile of its own, while every tile still gets its own CTA; the parts add
    // `gate * partial` into the f32 residual stream with atomics, in whatever order they finish.
    {
        int base_tiles = 0;
        bool eligible = true;
        for (int i = 0; i < nprob; ++i) {
            const edb200_epilogue_t* ep = eps[i];
            base_tiles += P.p[i].m_tiles * P.p[i].n_tiles;
            eligible = eligible && ep->split_k == EDB200_SPLIT_K_UNORDERED && ws[i]->k >= 8192 &&
                       ep->gate != nullptr && ep->out == ep->residual && ep->ldo == ep->ld_res &&
                       ep->out_dtype == EDB200_TYPE_F32 && ep->act == EDB200_ACT_NONE && ep->split_n == 0;
        }
        if (eligible) {
            int parts = (pair ? sm_count() / 2 : sm_count()) / base_tiles;
            if (parts > 4) parts = 4;
            for (; parts > 1; --parts) {
                bool divides = true;
                for (int i = 0; i < nprob; ++i) {
                    const int64_t ksteps = ws[i]->k / gemm::BK;
                    divides = divides && ksteps % parts == 0 && ksteps / parts >= 16;
                }
                if (divides) break;
            }
            if (parts > 1) {
                for (int i = 0; i < nprob; ++i) P.p[i].ksplit = parts;
            }
        }
    }
    P.tiles0 = P.p[0].m_tiles * P.p[0].n_tiles * P.p[0].ksplit;
    P.total_tiles = P.tiles0 + (nprob == 2 ? P.p[1].m_tiles * P.p[1].n_tiles * P.p[1].ksplit : 0);
    P.err = err;

    const bool q4 = ws[0]->ggml_type == EDB200_TYPE_Q4_K;
    using KernT = void (*)(const CUtensorMap, const CUtensorMap, const gemm::Params);
    static const KernT kerns[8] = {gemm::qgemm_kernel<EDB200_TYPE_Q8_0, 1>,       gemm::qgemm_kernel<EDB200_TYPE_Q8_0, 2>,
                                   gemm::qgemm_kernel<EDB200_TYPE_Q4_K, 1>,       gemm::qgemm_kernel<EDB200_TYPE_Q4_K, 2>,
                                   gemm::qgemm_pair_kernel<EDB200_TYPE_Q8_0, 2>, gemm::qgemm_pair_kernel<EDB200_TYPE_Q4_K, 2>,
                                   gemm::qgemm_pair_kernel<EDB200_TYPE_Q8_0, 4>, gemm::qgemm_pair_kernel<EDB200_TYPE_Q4_K, 4>};
    static int dq_depth = 0;   // EDB200_GEMM_DQ=2|4: conversions in flight per CTA (tuning)
    if (dq_depth == 0) {
        const char* e = getenv("EDB200_GEMM_DQ");
        dq_depth = (e != nullptr && atoi(e) == 2) ? 2 : 4;
    }
    const int ki = pair ? 4 + (dq_depth == 4 ? 2 : 0) + (q4 ? 1 : 0) : (q4 ? 2 : 0) + (wh - 1);
    KernT kern = kerns[ki];
    const int smem_bytes = pair ? gemm::PAIR_SMEM_BYTES : gemm::SMEM_BYTES;
    static bool attr_set_dev[64][8] = {};   // the attribute is per device
    static int max_pairs = 0;   // CTA pairs that can be resident at once
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) dev = 0;
    bool* attr_set = attr_set_dev[dev];
    if (!attr_set[ki]) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes);
        if (e != cudaSuccess) return check_cuda(e, "cudaFuncSetAttribute(qgemm)");
        if (pair && max_pairs == 0) {
            cudaLaunchConfig_t cfg;
            memset(&cfg, 0, sizeof(cfg));
            cfg.gridDim = dim3(static_cast<unsigned>(sm_count() & ~1), 1, 1);
            cfg.blockDim = dim3(gemm::NUM_THREADS, 1, 1);
            cfg.dynamicSmemBytes = static_cast<size_t>(smem_bytes);
            int n = 0;
            e = cudaOccupancyMaxActiveClusters(&n, kern, &cfg);
            if (e != cudaSuccess || n <= 0) {
                (void)cudaGetLastError();
                n = sm_count() / 2;
            }
            max_pairs = n < sm_count() / 2 ? n : sm_count() / 2;
#ifdef EDB200_GEMM_STATS
            fprintf(stderr, "qgemm: %d CTA pairs resident (occupancy query %d)\n", max_pairs, n);
#endif
        }
        attr_set[ki] = true;
    }
    const int grid = pair ? 2 * (P.total_tiles < max_pairs ? P.total_tiles : max_pairs)
                          : (P.total_tiles < sm_count() ? P.total_tiles : sm_count());
    double flops = 0.0, bytes = 0.0;
    for (int i = 0; i < nprob; ++i) {
        flops += 2.0 * (double)ms[i] * (double)ws[i]->n_out * (double)ws[i]->k;
        bytes += (double)ws[i]->bytes + 2.0 * (double)ms[i] * (double)ws[i]->k +
                 (double)ms[i] * (double)ws[i]->n_out * (eps[i]->out_dtype == EDB200_TYPE_F32 ? 4.0 : 2.0);
    }
    ProfScope prof(stream, PROF_GEMM, flops, bytes);
    kern<<<grid, gemm::NUM_THREADS, smem_bytes, stream>>>(map_a[0], map_a[1], P);
    count_launch();
    return check_cuda(cudaGetLastError(), "qgemm launch");
}

}  // namespace edb

extern "C" {

#ifdef EDB200_GEMM_STATS
EDB200_API void edb200_debug_pair_stats(long long* out16, int reset) {
    cudaDeviceSynchronize();
    if (out16) cudaMemcpyFromSymbol(out16, edb::gemm::g_pair_stats, 16 * sizeof(long long));
    if (reset) {
        long long zero[16] = {0};
        cudaMemcpyToSymbol(edb::gemm::g_pair_stats, zero, sizeof(zero));
    }
}
#endif

int edb200_mul_mat_q_fuses_qk_pack(void) {
    const char* e = getenv("EDB200_GEMM_PAIR");
    return (e != nullptr && atoi(e) == 0) ? 0 : 1;
}

edb200_status_t edb200_mul_mat_q(const edb200_qweight_t* w, const void* x, int x_dtype, int64_t m, int64_t ldx,
                                 const edb200_epilogue_t* ep, void* stream) {
    const edb200_qweight_t* ws[1] = {w};
    const void* xs[1] = {x};
    const int64_t ms[1] = {m};
    const int64_t lds[1] = {ldx};
    const edb200_epilogue_t* eps[1] = {ep};
    return edb::launch_qgemm(1, ws, xs, ms, lds, eps, x_dtype, static_cast<cudaStream_t>(stream));
}

edb200_status_t edb200_mul_mat_q_pair(const edb200_qweight_t* w0, const void* x0, int64_t m0, int64_t ldx0,
                                      const edb200_epilogue_t* ep0, const edb200_qweight_t* w1, const void* x1,
                                      int64_t m1, int64_t ldx1, const edb200_epilogue_t* ep1, int x_dtype,
                                      void* stream) {
    const edb200_qweight_t* ws[2] = {w0, w1};
    const void* xs[2] = {x0, x1};
    const int64_t ms[2] = {m0, m1};
    const int64_t lds[2] = {ldx0, ldx1};
    const edb200_epilogue_t* eps[2] = {ep0, ep1};
    return edb::launch_qgemm(2, ws, xs, ms, lds, eps, x_dtype, static_cast<cudaStream_t>(stream));
}

}  // extern "C"
