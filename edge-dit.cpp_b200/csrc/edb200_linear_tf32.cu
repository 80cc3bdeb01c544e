// Dense f32 linear on the tensor cores (tcgen05 kind::tf32) for the unquantised layers of a step's prelude
// and tail - txt_in / img_in / context embedders / patch embedders / final linears (the tensors
// tensor_should_be_converted leaves unquantised, reference src/core/runtime/model_loader.cpp:2141-2172), which
// ggml runs as plain mul_mat on f32 / f16 weights (src/core/backend/ggml/ggml_extend.hpp:1308-1347).
//
//   y[m, n] = act(x[m, :] . W[n, :] + bias[n])        x, W, y f32 in global memory, read as they are
//
// Both operands go from global to shared memory by TMA as f32 rows of 32 k (128 bytes, 128-byte swizzle) and
// into the MMA from there (SS form): no repacked or converted copy of the weights exists, so nothing has to be
// kept in step with the parameter table.  The tensor core reads the f32 words as tf32 (10 mantissa bits; the
// accumulation is f32).  Transposed tile D[n, m] = W . x^T like the quantised GEMM, so a lane of the epilogue
// is an output feature and a row store is 128 contiguous bytes.
//
// One CTA per 128 features x 128 rows, 192 threads: warp 0 TMA producer (4-stage ring), warp 1 tensor-memory
// allocator and MMA issuer (four 128 x 128 x 8 MMAs per 32-k stage), warps 2-5 epilogue.  k, m and n tails are
// zero-filled by TMA and masked in the epilogue.
#include "edb200_internal.h"
#include "edb200_ptx.cuh"

namespace edb {
namespace lin32 {

constexpr int TW = 128;          // output features per tile = tensor-memory lanes
constexpr int TM = 128;          // rows (tokens) per tile = accumulator columns
constexpr int BK = 32;           // f32 per stage row = 128 bytes
constexpr int STAGES = 4;
constexpr int A_BYTES = TW * BK * 4, B_BYTES = TM * BK * 4, STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int OFF_BAR = STAGES * STAGE_BYTES;
constexpr int SMEM_BYTES = OFF_BAR + 128 + 1024;
constexpr int NUM_THREADS = 192;
constexpr uint32_t kFmtTF32 = 2;

struct Params {
    const float* bias;
    float* y;
    long long ldy;
    int M, N, K, act;
    int* err;
};

__device__ __forceinline__ void mma_tf32_ss(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                            uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t"
        "}\n"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}

__device__ __forceinline__ float act_apply(float v, int act) {
    if (act == EDB200_ACT_GELU_TANH) {
        const float u = 0.7978845608028654f * v * (1.0f + 0.044715f * v * v);
        return 0.5f * v * (1.0f + tanhf(u));
    }
    if (act == EDB200_ACT_SILU) return v / (1.0f + expf(-v));
    if (act == EDB200_ACT_GELU_ERF) return 0.5f * v * (1.0f + erff(v * 0.70710678118654752f));
    return v;
}

__global__ void __launch_bounds__(NUM_THREADS, 1)
linear_tf32_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x, const Params P) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + OFF_BAR);   // [STAGES]
    uint64_t* empty = full + STAGES;                                // [STAGES]
    uint64_t* acc_full = empty + STAGES;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_full + 1);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n0 = blockIdx.x * TW, m0 = blockIdx.y * TM;
    const int ksteps = (P.K + BK - 1) / BK;

    if (threadIdx.x == 0) {
        for (int i = 0; i < STAGES; ++i) {
            mbar_init(&full[i], 1);
            mbar_init(&empty[i], 1);
        }
        mbar_init(acc_full, 1);
        *abort_flag = 0;
        fence_mbar_init();
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, 128);
        tmem_relinquish();
    }
    if (warp == 0 && lane == 0) {
        tma_prefetch_desc(&map_w);
        tma_prefetch_desc(&map_x);
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        uint32_t s = 0, ph = 0;
        for (int ks = 0; ks < ksteps; ++ks) {
            if (!mbar_wait(&empty[s], ph ^ 1u, abort_flag, P.err)) break;
            if (elect_one()) {
                uint8_t* stage = smem + s * STAGE_BYTES;
                mbar_arrive_expect_tx(&full[s], STAGE_BYTES);
                tma_load_2d(stage, &map_w, &full[s], ks * BK, n0);
                tma_load_2d(stage + A_BYTES, &map_x, &full[s], ks * BK, m0);
            }
            __syncwarp();
            if (++s == STAGES) {
                s = 0;
                ph ^= 1u;
            }
        }
    } else if (warp == 1) {
        const uint32_t idesc = make_idesc(kDFmtF32, kFmtTF32, kFmtTF32, 0, 0, TW, TM);
        uint32_t s = 0, ph = 0;
        bool ok = true;
        for (int ks = 0; ks < ksteps; ++ks) {
            if (!mbar_wait(&full[s], ph, abort_flag, P.err)) {
                ok = false;
                break;
            }
            tc_fence_after_sync();
            if (elect_one()) {
                const uint32_t a_addr = smem_u32(smem + s * STAGE_BYTES), b_addr = a_addr + A_BYTES;
#pragma unroll
                for (int j = 0; j < BK / 8; ++j) {   // 8 tf32 = 32 bytes of k per instruction
                    mma_tf32_ss(tmem_base, make_smem_desc_sw128(a_addr + j * 32, 16, 1024),
                                make_smem_desc_sw128(b_addr + j * 32, 16, 1024), idesc, (ks > 0 || j > 0) ? 1u : 0u);
                }
                mma_commit(&empty[s]);
            }
            __syncwarp();
            if (++s == STAGES) {
                s = 0;
                ph ^= 1u;
            }
        }
        if (ok && elect_one()) mma_commit(acc_full);
        __syncwarp();
    } else {
        // epilogue: warp w reads the lanes of its quarter (w % 4); lane = output feature, register = row
        const int quarter = warp & 3;
        if (mbar_wait(acc_full, 0, abort_flag, P.err)) {
            tc_fence_after_sync();
            const int n = n0 + quarter * 32 + lane;
            const bool n_ok = n < P.N;
            const float b = (P.bias != nullptr && n_ok) ? __ldg(P.bias + n) : 0.0f;
            const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
#pragma unroll 1
            for (int c = 0; c < TM / 16; ++c) {
                const int m_first = m0 + c * 16;
                if (m_first >= P.M) break;   // uniform
                uint32_t r[16];
                tmem_ld_32x32b_x16(taddr + c * 16, r);
                tmem_wait_ld();
                if (n_ok) {
                    float* o = P.y + (long long)m_first * P.ldy + n;
#pragma unroll
                    for (int i = 0; i < 16; ++i) {
                        if (m_first + i < P.M) o[(long long)i * P.ldy] = act_apply(__uint_as_float(r[i]) + b, P.act);
                    }
                }
            }
        }
    }
    tc_fence_before_sync();
    __syncthreads();
    if (*abort_flag) {
        for (int i = 0; i < 200; ++i) __nanosleep(1000);   // let copies and MMAs in flight land
        __syncthreads();
    }
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, 128);
    }
}

}  // namespace lin32

// True when the tensor-core kernel can take the problem (otherwise the caller uses its SIMT kernels).
bool linear_tf32_usable(const float* w, const float* x, int64_t m, int64_t k, int64_t n, int64_t ldx) {
    static int on = -1;
    if (on < 0) {
        const char* e = getenv("EDB200_LINEAR_TF32");
        on = (e != nullptr && atoi(e) == 0) ? 0 : 1;
    }
    // every row count the GEMV does not take, so that a sequence-parallel rank with few rows rounds like the rest
    return on == 1 && m > 8 && n >= 32 && k >= 32 && (k % 4) == 0 && (ldx % 4) == 0 &&
           ((reinterpret_cast<uintptr_t>(w) | reinterpret_cast<uintptr_t>(x)) & 15u) == 0;
}

edb200_status_t launch_linear_tf32(const float* w, const float* bias, const float* x, int64_t m, int64_t k, int64_t n,
                                   int64_t ldx, int act, float* y, int64_t ldy, cudaStream_t s) {
    int* err = device_error_word();
    if (err == nullptr) return fail(EDB200_ERR_CUDA, "linear_f32: no CUDA device");
    CUtensorMap map_w, map_x;
    EDB_TRY(make_tmap_2d(&map_w, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, w, (uint64_t)k, (uint64_t)n, (uint64_t)k * 4, lin32::BK,
                         lin32::TW, CU_TENSOR_MAP_SWIZZLE_128B));
    EDB_TRY(make_tmap_2d(&map_x, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, x, (uint64_t)k, (uint64_t)m, (uint64_t)ldx * 4, lin32::BK,
                         lin32::TM, CU_TENSOR_MAP_SWIZZLE_128B));
    static bool attr_set[64] = {false};   // the attribute is per device
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) dev = 0;
    if (!attr_set[dev]) {
        EDB_TRY(check_cuda(cudaFuncSetAttribute(lin32::linear_tf32_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                lin32::SMEM_BYTES),
                           "cudaFuncSetAttribute(linear_tf32)"));
        attr_set[dev] = true;
    }
    lin32::Params P;
    P.bias = bias;
    P.y = y;
    P.ldy = ldy;
    P.M = static_cast<int>(m);
    P.N = static_cast<int>(n);
    P.K = static_cast<int>(k);
    P.act = act;
    P.err = err;
    dim3 grid(static_cast<unsigned>((n + lin32::TW - 1) / lin32::TW), static_cast<unsigned>((m + lin32::TM - 1) / lin32::TM));
    lin32::linear_tf32_kernel<<<grid, lin32::NUM_THREADS, lin32::SMEM_BYTES, s>>>(map_w, map_x, P);
    return check_cuda(cudaGetLastError(), "linear_tf32 launch");
}

}  // namespace edb
