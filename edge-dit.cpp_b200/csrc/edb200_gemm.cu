// Dequant-fused quantised GEMM for sm_100a.
//
//   y[m, n] = sum_k x[m, k] * dequant(W)[n, k]   (+ bias, activation, gated residual)
//
// Stands in for ggml_mul_mat on q8_0 / q4_K weights reached through
// ggml_ext_linear (reference src/core/backend/ggml/ggml_extend.hpp:1308-1347).
//
// One persistent CTA per SM, 512 threads, warp-specialised:
//   warp 0      TMA producer: activation tile (bf16/f16, 128B swizzle), raw
//               quantised weight tile and its per-32 scale rows, 4-stage ring
//   warp 1      tcgen05.mma issuer (one lane): CTA tile 256x128, two 128x128x16 kind::f16
//               MMAs per k16 share one dequantised weight tile; fp32 accumulators
//               double-buffered in tensor memory (2 stages x 2 halves x 128 columns)
//   warp 2      tensor-memory allocator
//   warps 4-7   epilogue: tcgen05.ld, bias / GELU / gate*y+residual, stores
//   warps 8-15  dequantisers: raw int8 / 4-bit payload -> f16 = rn(d*q) written
//               straight into the 128B-swizzled K-major operand layout
// The dequantised f16 weight equals rn_f16(d*q) for q8_0 (one rounding of the
// exact product) and rn_f16(a*q - b) for q4_K with a = rn_f16(d*sc), b = rn_f16(dmin*m).
#include "edb200_internal.h"
#include "edb200_ptx.cuh"

namespace edb {
namespace gemm {

constexpr int BM = 256;      // rows per CTA tile = two 128-row MMA halves sharing one weight tile
constexpr int MMA_M = 128;
constexpr int BN = 128;
constexpr int BK = 64;
constexpr int LD_STAGES = 4;
constexpr int B_STAGES = 3;
constexpr int ACC_STAGES = 2;
constexpr int A_BYTES = BM * BK * 2;      // 32 KB
constexpr int WQ_BYTES = BN * BK;         // 8 KB (q8_0); q4_K uses half of it
constexpr int SC_PLANE_BYTES = 2 * BN * 2;  // two 32-blocks x 128 rows x f16
constexpr int SC_BYTES = 2 * SC_PLANE_BYTES;
constexpr int B_BYTES = BN * BK * 2;      // 16 KB

constexpr int OFF_A = 0;
constexpr int OFF_W = OFF_A + LD_STAGES * A_BYTES;
constexpr int OFF_B = OFF_W + LD_STAGES * WQ_BYTES;
constexpr int OFF_S = OFF_B + B_STAGES * B_BYTES;
constexpr int OFF_BAR = OFF_S + LD_STAGES * SC_BYTES;
constexpr int SMEM_BYTES = OFF_BAR + 256 + 1024;  // + alignment slack

constexpr int NUM_THREADS = 512;
constexpr int DQ_WARPS = 8;
constexpr int EPI_WARPS = 4;
constexpr uint32_t TMEM_COLS = 512;

struct Problem {
    const float* bias;
    void* out;
    const float* residual;
    const float* gate;
    void* out2;
    long long ldo, ld_res, ldo2, split_n;
    int out_dtype, act, out2_dtype, act2;
    int M, N, K;
    int m_tiles, n_tiles;
};

struct Params {
    Problem p[2];
    int tiles0;       // tiles of problem 0
    int total_tiles;
    uint32_t a_fmt;   // kFmtF16 / kFmtBF16
    int* err;
};

struct TileCoord {
    int prob, m0, n0;
};

__device__ __forceinline__ TileCoord tile_coord(const Params& P, int t) {
    TileCoord c;
    c.prob = (t >= P.tiles0) ? 1 : 0;
    const int tt = c.prob ? t - P.tiles0 : t;
    const int m_tiles = c.prob ? P.p[1].m_tiles : P.p[0].m_tiles;
    // m fastest: CTAs running at the same time share one weight column block.
    c.n0 = (tt / m_tiles) * BN;
    c.m0 = (tt % m_tiles) * BM;
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

__device__ __forceinline__ uint32_t pack_bf16(float a, float b) {
    __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
}
__device__ __forceinline__ uint32_t pack_f16(float a, float b) {
    __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
}

// One 32-column slice of one accumulator row.
__device__ __forceinline__ void epilogue_store(const Problem& P, float (&v)[32], int m, int n, bool row_ok) {
    if (P.bias != nullptr) {
        const float4* b4 = reinterpret_cast<const float4*>(P.bias + n);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const float4 b = __ldg(b4 + j);
            v[4 * j + 0] += b.x;
            v[4 * j + 1] += b.y;
            v[4 * j + 2] += b.z;
            v[4 * j + 3] += b.w;
        }
    }
    const bool second = (P.split_n > 0) && (n >= P.split_n);
    const int act = second ? P.act2 : P.act;
    if (act != EDB200_ACT_NONE) {
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = apply_act(v[j], act);
    }
    if (!second && P.gate != nullptr) {
        const float4* g4 = reinterpret_cast<const float4*>(P.gate + n);
        const float4* r4 = reinterpret_cast<const float4*>(P.residual + (long long)m * P.ld_res + n);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const float4 g = __ldg(g4 + j);
            float4 r = make_float4(0.f, 0.f, 0.f, 0.f);
            if (row_ok) r = r4[j];
            v[4 * j + 0] = r.x + g.x * v[4 * j + 0];
            v[4 * j + 1] = r.y + g.y * v[4 * j + 1];
            v[4 * j + 2] = r.z + g.z * v[4 * j + 2];
            v[4 * j + 3] = r.w + g.w * v[4 * j + 3];
        }
    }
    if (!row_ok) return;
    const int dt = second ? P.out2_dtype : P.out_dtype;
    const long long ld = second ? P.ldo2 : P.ldo;
    const long long col = second ? (n - P.split_n) : n;
    char* base = reinterpret_cast<char*>(second ? P.out2 : P.out);
    if (dt == EDB200_TYPE_F32) {
        float4* o = reinterpret_cast<float4*>(base + ((long long)m * ld + col) * 4);
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
    } else {
        uint4* o = reinterpret_cast<uint4*>(base + ((long long)m * ld + col) * 2);
        const bool bf = (dt == EDB200_TYPE_BF16);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            uint4 u;
            if (bf) {
                u.x = pack_bf16(v[8 * j + 0], v[8 * j + 1]);
                u.y = pack_bf16(v[8 * j + 2], v[8 * j + 3]);
                u.z = pack_bf16(v[8 * j + 4], v[8 * j + 5]);
                u.w = pack_bf16(v[8 * j + 6], v[8 * j + 7]);
            } else {
                u.x = pack_f16(v[8 * j + 0], v[8 * j + 1]);
                u.y = pack_f16(v[8 * j + 2], v[8 * j + 3]);
                u.z = pack_f16(v[8 * j + 4], v[8 * j + 5]);
                u.w = pack_f16(v[8 * j + 6], v[8 * j + 7]);
            }
            o[j] = u;
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

// q8_0: 128 rows x 64 int8 -> 128 rows x 64 f16 in the swizzled operand layout.
__device__ __forceinline__ void dequant_q8_0(const uint8_t* wq, const __half* sc, uint8_t* bdst, int dq_tid) {
    const __half2 k1152 = __float2half2_rn(1152.0f);
#pragma unroll
    for (int it = 0; it < BN * 4 / 256; ++it) {
        const int id = it * 256 + dq_tid;
        const int row = id >> 2;
        const int c = id & 3;
        const uint4 raw = *reinterpret_cast<const uint4*>(wq + row * 64 + c * 16);
        const __half2 d2 = __half2half2(sc[(c >> 1) * BN + row]);
        const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
        uint32_t o[8];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const uint32_t x = w[j] ^ 0x80808080u;                       // q + 128 in each byte
            const uint32_t lo = __byte_perm(x, 0x64646464u, 0x4140);      // f16 (1024 + u0, 1024 + u1)
            const uint32_t hi = __byte_perm(x, 0x64646464u, 0x4342);
            o[2 * j + 0] = h2_sub_mul(lo, k1152, d2);
            o[2 * j + 1] = h2_sub_mul(hi, k1152, d2);
        }
        const uint32_t rbase = (row >> 3) * 1024 + (row & 7) * 128;
        const uint32_t sw = row & 7;
        *reinterpret_cast<uint4*>(bdst + rbase + (((2 * c + 0) ^ sw) << 4)) = make_uint4(o[0], o[1], o[2], o[3]);
        *reinterpret_cast<uint4*>(bdst + rbase + (((2 * c + 1) ^ sw) << 4)) = make_uint4(o[4], o[5], o[6], o[7]);
    }
}

// q4_K: 128 rows x 32 bytes; byte i of a row holds weight k=i (low nibble, first
// 32-block) and weight k=32+i (high nibble, second 32-block).
__device__ __forceinline__ void dequant_q4_k(const uint8_t* wq, const __half* sa, const __half* sb, uint8_t* bdst,
                                             int dq_tid) {
    const __half2 k1024 = __float2half2_rn(1024.0f);
#pragma unroll
    for (int it = 0; it < BN * 2 / 256; ++it) {
        const int id = it * 256 + dq_tid;
        const int row = id >> 1;
        const int c = id & 1;  // bytes c*16 .. c*16+15
        const uint4 raw = *reinterpret_cast<const uint4*>(wq + row * 32 + c * 16);
        const __half2 a_lo = __half2half2(sa[row]);
        const __half2 a_hi = __half2half2(sa[BN + row]);
        const __half2 nb_lo = __hneg2(__half2half2(sb[row]));
        const __half2 nb_hi = __hneg2(__half2half2(sb[BN + row]));
        const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
        uint32_t lo_o[8], hi_o[8];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const uint32_t xl = w[j] & 0x0F0F0F0Fu;
            const uint32_t xh = (w[j] >> 4) & 0x0F0F0F0Fu;
            lo_o[2 * j + 0] = h2_sub_fma(__byte_perm(xl, 0x64646464u, 0x4140), k1024, a_lo, nb_lo);
            lo_o[2 * j + 1] = h2_sub_fma(__byte_perm(xl, 0x64646464u, 0x4342), k1024, a_lo, nb_lo);
            hi_o[2 * j + 0] = h2_sub_fma(__byte_perm(xh, 0x64646464u, 0x4140), k1024, a_hi, nb_hi);
            hi_o[2 * j + 1] = h2_sub_fma(__byte_perm(xh, 0x64646464u, 0x4342), k1024, a_hi, nb_hi);
        }
        const uint32_t rbase = (row >> 3) * 1024 + (row & 7) * 128;
        const uint32_t sw = row & 7;
        // low nibbles: k = c*16 .. c*16+15 -> 16-byte chunks 2c, 2c+1; high: k+32 -> chunks 4+2c, 5+2c
        *reinterpret_cast<uint4*>(bdst + rbase + (((2 * c + 0) ^ sw) << 4)) =
            make_uint4(lo_o[0], lo_o[1], lo_o[2], lo_o[3]);
        *reinterpret_cast<uint4*>(bdst + rbase + (((2 * c + 1) ^ sw) << 4)) =
            make_uint4(lo_o[4], lo_o[5], lo_o[6], lo_o[7]);
        *reinterpret_cast<uint4*>(bdst + rbase + (((4 + 2 * c + 0) ^ sw) << 4)) =
            make_uint4(hi_o[0], hi_o[1], hi_o[2], hi_o[3]);
        *reinterpret_cast<uint4*>(bdst + rbase + (((4 + 2 * c + 1) ^ sw) << 4)) =
            make_uint4(hi_o[4], hi_o[5], hi_o[6], hi_o[7]);
    }
}

template <int WT>  // EDB200_TYPE_Q8_0 or EDB200_TYPE_Q4_K
__global__ void __launch_bounds__(NUM_THREADS, 1)
qgemm_kernel(const __grid_constant__ CUtensorMap map_a0, const __grid_constant__ CUtensorMap map_q0,
             const __grid_constant__ CUtensorMap map_sa0, const __grid_constant__ CUtensorMap map_sb0,
             const __grid_constant__ CUtensorMap map_a1, const __grid_constant__ CUtensorMap map_q1,
             const __grid_constant__ CUtensorMap map_sa1, const __grid_constant__ CUtensorMap map_sb1,
             const __grid_constant__ Params P) {
    constexpr bool kQ4 = (WT == EDB200_TYPE_Q4_K);
    constexpr uint32_t kWqStageBytes = kQ4 ? (BN * BK / 2) : (BN * BK);
    constexpr uint32_t kTxBytes = A_BYTES + kWqStageBytes + (kQ4 ? 2 : 1) * SC_PLANE_BYTES;

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + OFF_BAR);
    uint64_t* ld_full = bars;                       // [LD_STAGES]
    uint64_t* ld_empty = ld_full + LD_STAGES;       // [LD_STAGES]
    uint64_t* b_full = ld_empty + LD_STAGES;        // [B_STAGES]
    uint64_t* b_empty = b_full + B_STAGES;          // [B_STAGES]
    uint64_t* acc_full = b_empty + B_STAGES;        // [ACC_STAGES]
    uint64_t* acc_empty = acc_full + ACC_STAGES;    // [ACC_STAGES]
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + ACC_STAGES);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int i = 0; i < LD_STAGES; ++i) {
            mbar_init(&ld_full[i], 1);
            mbar_init(&ld_empty[i], 1 + DQ_WARPS);
        }
        for (int i = 0; i < B_STAGES; ++i) {
            mbar_init(&b_full[i], DQ_WARPS);
            mbar_init(&b_empty[i], 1);
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
        tma_prefetch_desc(&map_a0);
        tma_prefetch_desc(&map_q0);
        tma_prefetch_desc(&map_sa0);
        if (P.total_tiles > P.tiles0) {
            tma_prefetch_desc(&map_a1);
            tma_prefetch_desc(&map_q1);
            tma_prefetch_desc(&map_sa1);
        }
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ------------------------------------------------------ TMA producer
        if (lane == 0) {
            uint32_t s = 0, ph = 0;
            bool ok = true;
            for (int t = blockIdx.x; ok && t < P.total_tiles; t += gridDim.x) {
                const TileCoord tc = tile_coord(P, t);
                const int ksteps = (tc.prob ? P.p[1].K : P.p[0].K) / BK;
                const CUtensorMap* ma = tc.prob ? &map_a1 : &map_a0;
                const CUtensorMap* mq = tc.prob ? &map_q1 : &map_q0;
                const CUtensorMap* msa = tc.prob ? &map_sa1 : &map_sa0;
                const CUtensorMap* msb = tc.prob ? &map_sb1 : &map_sb0;
                for (int ks = 0; ks < ksteps; ++ks) {
                    if (!mbar_wait(&ld_empty[s], ph ^ 1u, abort_flag, P.err)) {
                        ok = false;
                        break;
                    }
                    mbar_arrive_expect_tx(&ld_full[s], kTxBytes);
                    tma_load_2d(smem + OFF_A + s * A_BYTES, ma, &ld_full[s], ks * BK, tc.m0);
                    tma_load_2d(smem + OFF_W + s * WQ_BYTES, mq, &ld_full[s], kQ4 ? ks * (BK / 2) : ks * BK, tc.n0);
                    tma_load_2d(smem + OFF_S + s * SC_BYTES, msa, &ld_full[s], tc.n0, ks * 2);
                    if (kQ4) {
                        tma_load_2d(smem + OFF_S + s * SC_BYTES + SC_PLANE_BYTES, msb, &ld_full[s], tc.n0, ks * 2);
                    }
                    if (++s == LD_STAGES) {
                        s = 0;
                        ph ^= 1u;
                    }
                }
            }
        }
    } else if (warp == 1) {
        // -------------------------------------------------------- MMA issuer
        const uint32_t idesc = make_idesc(kDFmtF32, P.a_fmt, kFmtF16, 0, 0, MMA_M, BN);
        uint32_t s = 0, ph = 0, bs = 0, bph = 0, as = 0, aph = 0;
        bool ok = true;
        for (int t = blockIdx.x; ok && t < P.total_tiles; t += gridDim.x) {
            const TileCoord tc = tile_coord(P, t);
            const int ksteps = (tc.prob ? P.p[1].K : P.p[0].K) / BK;
            if (!mbar_wait(&acc_empty[as], aph ^ 1u, abort_flag, P.err)) {
                ok = false;
                break;
            }
            tc_fence_after_sync();
            const uint32_t tmem_d = tmem_base + as * (2 * BN);
            for (int ks = 0; ks < ksteps; ++ks) {
                if (!mbar_wait(&ld_full[s], ph, abort_flag, P.err) ||
                    !mbar_wait(&b_full[bs], bph, abort_flag, P.err)) {
                    ok = false;
                    break;
                }
                tc_fence_after_sync();
                if (lane == 0) {
                    const uint32_t a_addr = smem_u32(smem + OFF_A + s * A_BYTES);
                    const uint32_t b_addr = smem_u32(smem + OFF_B + bs * B_BYTES);
#pragma unroll
                    for (int j = 0; j < BK / 16; ++j) {
                        const uint64_t bd = make_smem_desc_sw128(b_addr + j * 32, 16, 1024);
#pragma unroll
                        for (int h = 0; h < BM / MMA_M; ++h) {
                            // rows h*128.. of the activation tile: 128 rows x 128 B further on
                            const uint64_t ad = make_smem_desc_sw128(a_addr + h * (MMA_M * 128) + j * 32, 16, 1024);
                            mma_f16_ss(tmem_d + h * BN, ad, bd, idesc, (ks > 0 || j > 0) ? 1u : 0u);
                        }
                    }
                    mma_commit(&ld_empty[s]);
                    mma_commit(&b_empty[bs]);
                }
                __syncwarp();
                if (++s == LD_STAGES) {
                    s = 0;
                    ph ^= 1u;
                }
                if (++bs == B_STAGES) {
                    bs = 0;
                    bph ^= 1u;
                }
            }
            if (!ok) break;
            if (lane == 0) mma_commit(&acc_full[as]);
            __syncwarp();
            if (++as == ACC_STAGES) {
                as = 0;
                aph ^= 1u;
            }
        }
    } else if (warp >= 4 && warp < 8) {
        // ----------------------------------------------------------- epilogue
        const int quarter = warp & 3;
        uint32_t as = 0, aph = 0;
        bool ok = true;
        for (int t = blockIdx.x; ok && t < P.total_tiles; t += gridDim.x) {
            const TileCoord tc = tile_coord(P, t);
            const Problem& pr = tc.prob ? P.p[1] : P.p[0];
            if (!mbar_wait(&acc_full[as], aph, abort_flag, P.err)) {
                ok = false;
                break;
            }
            tc_fence_after_sync();
            const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + as * (2 * BN);
#pragma unroll 1
            for (int hc = 0; hc < (BM / MMA_M) * (BN / 32); ++hc) {
                const int h = hc / (BN / 32), c = hc % (BN / 32);
                const int m = tc.m0 + h * MMA_M + quarter * 32 + lane;
                const bool row_ok = m < pr.M;
                const int n = tc.n0 + c * 32;
                if (n >= pr.N) continue;   // uniform: N is a multiple of 32
                if (tc.m0 + h * MMA_M >= pr.M) continue;   // uniform: whole half beyond the last row
                uint32_t r[32];
                tmem_ld_32x32b_x32(taddr + h * BN + c * 32, r);
                tmem_wait_ld();
                float v[32];
#pragma unroll
                for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
                epilogue_store(pr, v, m, n, row_ok);
            }
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(&acc_empty[as]);
            if (++as == ACC_STAGES) {
                as = 0;
                aph ^= 1u;
            }
        }
    } else if (warp >= 8) {
        // -------------------------------------------------------- dequantisers
        const int dq_tid = threadIdx.x - 8 * 32;
        uint32_t s = 0, ph = 0, bs = 0, bph = 0;
        bool ok = true;
        for (int t = blockIdx.x; ok && t < P.total_tiles; t += gridDim.x) {
            const TileCoord tc = tile_coord(P, t);
            const int ksteps = (tc.prob ? P.p[1].K : P.p[0].K) / BK;
            for (int ks = 0; ks < ksteps; ++ks) {
                if (!mbar_wait(&ld_full[s], ph, abort_flag, P.err) ||
                    !mbar_wait(&b_empty[bs], bph ^ 1u, abort_flag, P.err)) {
                    ok = false;
                    break;
                }
                const uint8_t* wq = smem + OFF_W + s * WQ_BYTES;
                const __half* sc = reinterpret_cast<const __half*>(smem + OFF_S + s * SC_BYTES);
                uint8_t* bdst = smem + OFF_B + bs * B_BYTES;
                if (kQ4) {
                    dequant_q4_k(wq, sc, sc + 2 * BN, bdst, dq_tid);
                } else {
                    dequant_q8_0(wq, sc, bdst, dq_tid);
                }
                fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) {
                    mbar_arrive(&b_full[bs]);
                    mbar_arrive(&ld_empty[s]);
                }
                if (++s == LD_STAGES) {
                    s = 0;
                    ph ^= 1u;
                }
                if (++bs == B_STAGES) {
                    bs = 0;
                    bph ^= 1u;
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
    if (ep->bias != nullptr && (reinterpret_cast<uintptr_t>(ep->bias) & 15u)) {
        return fail(EDB200_ERR_INVALID, "mul_mat_q: bias must be 16-byte aligned");
    }
    if (ep->split_n > 0) {
        if (ep->split_n % gemm::BN != 0 || ep->split_n >= w->n_out || ep->out2 == nullptr || !dt_ok(ep->out2_dtype)) {
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

static void fill_problem(gemm::Problem& p, const edb200_qweight_t* w, int64_t m, const edb200_epilogue_t* ep) {
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
    p.m_tiles = static_cast<int>((m + gemm::BM - 1) / gemm::BM);
    p.n_tiles = static_cast<int>((w->n_out + gemm::BN - 1) / gemm::BN);
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

    gemm::Params P;
    memset(&P, 0, sizeof(P));
    CUtensorMap map_a[2];
    const CUtensorMapDataType adt =
        x_dtype == EDB200_TYPE_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    for (int i = 0; i < nprob; ++i) {
        fill_problem(P.p[i], ws[i], ms[i], eps[i]);
        edb200_status_t st = make_tmap_2d(&map_a[i], adt, 2, xs[i], (uint64_t)ws[i]->k, (uint64_t)ms[i],
                                          (uint64_t)ldxs[i] * 2, gemm::BK, gemm::BM, CU_TENSOR_MAP_SWIZZLE_128B);
        if (st != EDB200_OK) return st;
    }
    if (nprob == 1) map_a[1] = map_a[0];
    const edb200_qweight_t* w1 = nprob == 2 ? ws[1] : ws[0];
    P.tiles0 = P.p[0].m_tiles * P.p[0].n_tiles;
    P.total_tiles = P.tiles0 + (nprob == 2 ? P.p[1].m_tiles * P.p[1].n_tiles : 0);
    P.a_fmt = x_dtype == EDB200_TYPE_BF16 ? kFmtBF16 : kFmtF16;
    P.err = err;

    const int grid = P.total_tiles < sm_count() ? P.total_tiles : sm_count();
    const bool q4 = ws[0]->ggml_type == EDB200_TYPE_Q4_K;
    auto kern = q4 ? gemm::qgemm_kernel<EDB200_TYPE_Q4_K> : gemm::qgemm_kernel<EDB200_TYPE_Q8_0>;
    static bool attr_set[2] = {false, false};
    if (!attr_set[q4 ? 1 : 0]) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, gemm::SMEM_BYTES);
        if (e != cudaSuccess) return check_cuda(e, "cudaFuncSetAttribute(qgemm)");
        attr_set[q4 ? 1 : 0] = true;
    }
    double flops = 0.0, bytes = 0.0;
    for (int i = 0; i < nprob; ++i) {
        flops += 2.0 * (double)ms[i] * (double)ws[i]->n_out * (double)ws[i]->k;
        bytes += (double)ws[i]->bytes + 2.0 * (double)ms[i] * (double)ws[i]->k +
                 (double)ms[i] * (double)ws[i]->n_out * (eps[i]->out_dtype == EDB200_TYPE_F32 ? 4.0 : 2.0);
    }
    ProfScope prof(stream, PROF_GEMM, flops, bytes);
    kern<<<grid, gemm::NUM_THREADS, gemm::SMEM_BYTES, stream>>>(
        map_a[0], ws[0]->map_qs, ws[0]->map_sa, q4 ? ws[0]->map_sb : ws[0]->map_sa, map_a[1], w1->map_qs, w1->map_sa,
        q4 ? w1->map_sb : w1->map_sa, P);
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
