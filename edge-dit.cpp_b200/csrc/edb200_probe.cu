// Tensor-pipe rate probe: every SM issues tcgen05.mma 128 x 256 (SS form, operands resident in shared
// memory and never reloaded) back to back, so the time measures the tensor pipe alone.  kind::f16
// (K = 16 per instruction) and kind::i8 (K = 32) run the same loop; their ratio carries the measured
// dense bf16 GEMM peak of a machine over to an INT8 figure for rooflines of INT8 kernels.
#include "edb200_internal.h"
#include "edb200_ptx.cuh"

namespace edb {
namespace {

template <bool I8>
__global__ void __launch_bounds__(128, 1) mma_rate_kernel(int iters, int* err) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    __shared__ uint64_t bar;
    __shared__ uint32_t slot;
    __shared__ int abort_flag;
    const int warp = threadIdx.x >> 5;
    if (threadIdx.x == 0) {
        mbar_init(&bar, 1);
        abort_flag = 0;
        fence_mbar_init();
    }
    if (warp == 0) {
        tmem_alloc(&slot, 256);
        tmem_relinquish();
    }
    // A: 128 rows x 128 bytes, B: 256 rows x 128 bytes, all zero
    for (int i = threadIdx.x; i < 48 * 1024 / 4; i += blockDim.x) reinterpret_cast<uint32_t*>(smem)[i] = 0;
    fence_proxy_async_smem();
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tb = slot;
    if (warp == 1) {
        const uint32_t idesc = I8 ? make_idesc(kDFmtS32, kFmtS8, kFmtS8, 0, 0, 128, 256)
                                  : make_idesc(kDFmtF32, kFmtF16, kFmtF16, 0, 0, 128, 256);
        const uint32_t a_addr = smem_u32(smem), b_addr = smem_u32(smem + 16384);
        if (elect_one()) {
            for (int it = 0; it < iters; ++it) {
#pragma unroll
                for (int j = 0; j < 4; ++j) {   // 32 bytes of K per instruction in both kinds
                    const uint64_t ad = make_smem_desc_sw128(a_addr + j * 32, 16, 1024);
                    const uint64_t bd = make_smem_desc_sw128(b_addr + j * 32, 16, 1024);
                    if (I8) {
                        mma_i8_ss(tb, ad, bd, idesc, 1u);
                    } else {
                        mma_f16_ss(tb, ad, bd, idesc, 1u);
                    }
                }
            }
            mma_commit(&bar);
        }
        __syncwarp();
        mbar_wait(&bar, 0, &abort_flag, err);
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 0) {
        tc_fence_after_sync();
        tmem_dealloc(tb, 256);
    }
}

}  // namespace
}  // namespace edb

using namespace edb;

extern "C" edb200_status_t edb200_probe_mma_rate(int kind, int iters, double* tera_ops, void* stream) {
    if (tera_ops == nullptr || iters <= 0 || iters > 100000 || (kind != 0 && kind != 1)) {
        return fail(EDB200_ERR_INVALID, "probe_mma_rate: kind 0 (f16) or 1 (i8), 1..100000 iterations");
    }
    int* err = device_error_word();
    if (err == nullptr) return fail(EDB200_ERR_CUDA, "probe_mma_rate: no CUDA device");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int smem = 64 * 1024;
    cudaError_t e = kind == 1 ? cudaFuncSetAttribute(mma_rate_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem)
                              : cudaFuncSetAttribute(mma_rate_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return check_cuda(e, "probe_mma_rate attribute");
    const int sms = sm_count();
    cudaEvent_t e0, e1;
    cudaEventCreate(&e0);
    cudaEventCreate(&e1);
    auto launch = [&](int n) {
        if (kind == 1) {
            mma_rate_kernel<true><<<sms, 128, smem, s>>>(n, err);
        } else {
            mma_rate_kernel<false><<<sms, 128, smem, s>>>(n, err);
        }
        count_launch();
    };
    launch(100);
    cudaEventRecord(e0, s);
    launch(iters);
    cudaEventRecord(e1, s);
    e = cudaStreamSynchronize(s);
    float ms = 0.0f;
    if (e == cudaSuccess) cudaEventElapsedTime(&ms, e0, e1);
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    if (e != cudaSuccess) return check_cuda(e, "probe_mma_rate");
    EDB_TRY(poll_device_error(s));
    const double k_per_mma = kind == 1 ? 32.0 : 16.0;
    const double ops = (double)sms * iters * 4.0 * 2.0 * 128.0 * 256.0 * k_per_mma;
    *tera_ops = ops / (ms * 1e-3) / 1e12;
    return EDB200_OK;
}
