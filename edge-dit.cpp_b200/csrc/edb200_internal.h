// Internal host-side declarations shared by the .cu files of libedb200.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <atomic>
#include <string>

#include "edb200_ops.h"

namespace edb {

// Records the message returned by edb200_last_error() and passes `st` through.
edb200_status_t fail(edb200_status_t st, const char* fmt, ...);
edb200_status_t check_cuda(cudaError_t e, const char* what);
void count_launch(int n = 1);

// Device status word shared by all kernels with bounded waits (zero = healthy).
// Lazily allocated per device; never freed.
int* device_error_word();
// Reads and clears the status word (synchronises the stream).
edb200_status_t poll_device_error(cudaStream_t stream);

// cuTensorMapEncodeTiled through the runtime's driver entry point (libcuda is
// not linked directly).
typedef CUresult (*PFN_encodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                    const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                    CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
PFN_encodeTiled get_encode_tiled();

// Dense f32 linear on the tensor cores (edb200_linear_tf32.cu): whether the problem qualifies, and the launch.
bool linear_tf32_usable(const float* w, const float* x, int64_t m, int64_t k, int64_t n, int64_t ldx);
edb200_status_t launch_linear_tf32(const float* w, const float* bias, const float* x, int64_t m, int64_t k, int64_t n,
                                   int64_t ldx, int act, float* y, int64_t ldy, cudaStream_t s);

// 2-D row-major tensor map: dims {inner, outer}, row pitch in bytes, box {box_inner, box_outer}.
edb200_status_t make_tmap_2d(CUtensorMap* map, CUtensorMapDataType dt, int elem_bytes, const void* base,
                             uint64_t inner, uint64_t outer, uint64_t pitch_bytes, uint32_t box_inner,
                             uint32_t box_outer, CUtensorMapSwizzle swz);
edb200_status_t make_tmap_3d(CUtensorMap* map, CUtensorMapDataType dt, int elem_bytes, const void* base,
                             uint64_t d0, uint64_t d1, uint64_t d2, uint64_t pitch1_bytes, uint64_t pitch2_bytes,
                             uint32_t b0, uint32_t b1, uint32_t b2, CUtensorMapSwizzle swz);

int sm_count();

// Optional per-kernel-class timing (off by default).  While enabled every
// launch site brackets its kernel with two CUDA events on the launching stream
// and records the algorithmic work; edb200_profile_end sums them per class.
enum ProfClass { PROF_GEMM = 0, PROF_ATTENTION = 1, PROF_GEMV = 2, PROF_ELEMENTWISE = 3, PROF_OTHER = 4, PROF_NCLASS = 5 };
bool profiling_enabled();
void profile_begin_launch(cudaStream_t s);
void profile_end_launch(cudaStream_t s, ProfClass cls, double flops, double bytes);

struct ProfScope {
    cudaStream_t s;
    ProfClass cls;
    double flops, bytes;
    bool on;
    ProfScope(cudaStream_t stream, ProfClass c, double f, double b) : s(stream), cls(c), flops(f), bytes(b), on(profiling_enabled()) {
        if (on) profile_begin_launch(s);
    }
    ~ProfScope() {
        if (on) profile_end_launch(s, cls, flops, bytes);
    }
};


// Buffers of the Sage quantisation (int8 Q/K, their scales, channel means, smooth-Q bias, chunk sums of the
// fast channel mean) and the strides of the scale / bias rows.
struct SagePtrs {
    int8_t* q8 = nullptr;
    int8_t* k8 = nullptr;
    float* q_scale = nullptr;
    float* k_scale = nullptr;
    float* qm = nullptr;
    float* km = nullptr;
    float* bias = nullptr;
    float* part_q = nullptr;
    float* part_k = nullptr;
    int q_scale_stride = 0, k_scale_stride = 0, bias_stride = 0;
};
SagePtrs sage_ptrs_from_scratch(void* scratch, int hn, int64_t l, int d);
// Quantise q and k ([hn, l, d] f16, heads head_rows rows apart) and, if `attend`, run the INT8-QK attention
// with v ([hn, l, d] f16, heads v_head_rows rows apart).  smooth_q is the EDB200_SAGE_* bit set.
edb200_status_t sage_run(const void* q_f16, const void* k_f16, const void* v_f16, int hn, int64_t l, int64_t head_rows,
                         int64_t v_head_rows, int d_head, float scale, int smooth_q, const SagePtrs& sp, void* out,
                         int out_dtype, int64_t ld_out, const edb200_sp_peers_t* dst, void* stream, bool attend);

}  // namespace edb

#define EDB_TRY(expr)                          \
    do {                                       \
        edb200_status_t _st = (expr);          \
        if (_st != EDB200_OK) return _st;      \
    } while (0)

// Repacked quantised weight (device resident), tiled for the GEMM's
// "one thread per weight row" dequantisers.
//
// The weight [n_out][k] is cut into tiles of kQwTileRows rows x kQwTileK weights.
// Tile (t, s) = rows t*128.., weights s*64.. is one contiguous record of
// `tile_bytes` at tiles + (t * ksteps + s) * tile_bytes, fetched with one bulk copy:
//   q8_0 (8704 B): payload [c = 0..3][r = 0..127][16 bytes q + 128] = weights s*64 + c*16 + i of row r
//                  scales  [h = 0..1][r] f16                 = d of 32-block 2s + h
//   q4_K (5120 B): payload [c = 0..1][r][16 B], byte c*16+i = weight s*64+c*16+i (low nibble)
//                  | weight s*64+32+c*16+i (high nibble): ggml's own nibble order
//                  a [h][r] f16 = rn(d*sc), b [h][r] f16 = rn(dmin*m) of sub-block 2s + h
//                  hdr (separate array): the 16 header bytes (d, dmin, scales[12]) of every
//                  256-block, kept so the exact f32 dequantiser can be restated
// Rows beyond n_out in the last tile are zero.
constexpr int kQwTileRows = 128;
constexpr int kQwTileK = 64;
constexpr int kQwTileBytesQ8 = 4 * 128 * 16 + 2 * 128 * 2;          // 8704
constexpr int kQwTileBytesQ4 = 2 * 128 * 16 + 2 * 2 * 128 * 2;      // 5120

struct edb200_qweight {
    int ggml_type = 0;
    int64_t n_out = 0;
    int64_t k = 0;
    int64_t n_tiles = 0;      // ceil(n_out / 128)
    int64_t ksteps = 0;       // k / 64
    int tile_bytes = 0;
    uint8_t* tiles = nullptr;
    uint8_t* hdr = nullptr;   // q4_K only: [n_out][k/256][16]
    int64_t bytes = 0;
};
