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
    gemm::Params P;
    memset(&P, 0, sizeof(P));
    CUtensorMap map_a[2];
    const CUtensorMapDataType adt =
        x_dtype == EDB200_TYPE_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    for (int i = 0; i < nprob; ++i) {
        fill_problem(P.p[i], ws[i], ms[i], eps[i], wh);
        edb200_status_t st = make_tmap_2d(&map_a[i], adt, 2, xs[i], (uint64_t)ws[i]->k, (uint64_t)ms[i],
                                          (uint64_t)ldxs[i] * 2, gemm::BK, gemm::TN, CU_TENSOR_MAP_SWIZZLE_128B);
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
            int parts = sm_count() / base_tiles;
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

    const int grid = P.total_tiles < sm_count() ? P.total_tiles : sm_count();
    const bool q4 = ws[0]->ggml_type == EDB200_TYPE_Q4_K;
    using KernT = void (*)(const CUtensorMap, const CUtensorMap, const gemm::Params);
    static const KernT kerns[4] = {gemm::qgemm_kernel<EDB200_TYPE_Q8_0, 1>, gemm::qgemm_kernel<EDB200_TYPE_Q8_0, 2>,
                                   gemm::qgemm_kernel<EDB200_TYPE_Q4_K, 1>, gemm::qgemm_kernel<EDB200_TYPE_Q4_K, 2>};
    const int ki = (q4 ? 2 : 0) + (wh - 1);
    KernT kern = kerns[ki];
    static bool attr_set[4] = {false, false, false, false};
    if (!attr_set[ki]) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, gemm::SMEM_BYTES);
        if (e != cudaSuccess) return check_cuda(e, "cudaFuncSetAttribute(qgemm)");
        attr_set[ki] = true;
    }
    double flops = 0.0, bytes = 0.0;
    for (int i = 0; i < nprob; ++i) {
        flops += 2.0 * (double)ms[i] * (double)ws[i]->n_out * (double)ws[i]->k;
        bytes += (double)ws[i]->bytes + 2.0 * (double)ms[i] * (double)ws[i]->k +
                 (double)ms[i] * (double)ws[i]->n_out * (eps[i]->out_dtype == EDB200_TYPE_F32 ? 4.0 : 2.0);
    }
    ProfScope prof(stream, PROF_GEMM, flops, bytes);
    kern<<<grid, gemm::NUM_THREADS, gemm::SMEM_BYTES, stream>>>(
        map_a[0], map_a[1], P);
    count_launch();
    return check_cuda(cudaGetLastError(), "qgemm launch");
}

}  // namespace edb

extern "C" {

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
