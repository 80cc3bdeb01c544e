/*
 * edb200_ops.h -- C ABI of the B200 (sm_100a) DiT denoise-step library.
 *
 * Plain C: opaque handles, raw device pointers, sizes and a CUDA stream passed
 * as void*.  Every entry point returns edb200_status_t, never throws and never
 * aborts; edb200_last_error() returns the message of the calling thread's last
 * failure.  All launches are asynchronous on the given stream unless stated.
 * There is no CPU fallback: without a CUDA device every compute entry point
 * returns EDB200_ERR_CUDA.
 *
 * Each declaration names the interface of the reference (THU-MIG/edge-dit.cpp,
 * paths relative to its root) that it stands in for.
 */
#ifndef EDB200_OPS_H
#define EDB200_OPS_H

#include <stddef.h>
#include <stdint.h>

#if defined(__GNUC__)
#define EDB200_API __attribute__((visibility("default")))
#else
#define EDB200_API
#endif

#ifdef __cplusplus
extern "C" {
#endif

typedef enum {
    EDB200_OK = 0,
    EDB200_ERR_INVALID = 1,     /* bad argument (null pointer, shape, alignment) */
    EDB200_ERR_UNSUPPORTED = 2, /* valid request this build has no kernel for */
    EDB200_ERR_CUDA = 3,        /* CUDA runtime / driver error, or no device */
    EDB200_ERR_TIMEOUT = 4,     /* a bounded device-side wait gave up */
    EDB200_ERR_NOMEM = 5
} edb200_status_t;

/* Element / block types.  Values are the ggml type ids the reference uses in
 * ed_dtype_t (include/edge-dit.h:47-62). */
enum {
    EDB200_TYPE_F32 = 0,
    EDB200_TYPE_F16 = 1,
    EDB200_TYPE_Q8_0 = 8,
    EDB200_TYPE_Q4_K = 12,
    EDB200_TYPE_I8 = 24,
    EDB200_TYPE_BF16 = 30
};

enum { EDB200_SPLIT_K_NEVER = 0, EDB200_SPLIT_K_UNORDERED = 1 };
enum { EDB200_ACT_NONE = 0, EDB200_ACT_GELU_TANH = 1, EDB200_ACT_SILU = 2, EDB200_ACT_GELU_ERF = 3 /* dense f32 linear only */ };

/* Buffers of every rank of the group as this GPU addresses them (peer mappings over
 * NVLink, see edb200_comm_map_peers): buf[i][r] = buffer i of rank r.  Kernels that
 * take this description store their results straight into the owning rank's memory,
 * so the exchange costs no extra pass over the data. */
typedef struct {
    int world, rank;
    int64_t t_loc;        /* tokens per rank */
    void* buf[3][8];
} edb200_sp_peers_t;

/* Message of the calling thread's last failed call ("" if none).  Stands in for
 * ed_get_last_error (include/edge-dit.h:333, src/edge_dit.cpp:347-353). */
EDB200_API const char* edb200_last_error(void);
/* Library version string and the compute capability it was built for. */
EDB200_API const char* edb200_version(void);
/* Number of kernels this library has launched in the calling process. */
EDB200_API int64_t edb200_launch_count(void);

/* Status of the device-side bounded waits.  Kernels of this library never wait without a limit (TMA
 * and tensor-pipe barriers about two seconds, the cross-GPU barrier edb200_comm_set_timeout_ms); a wait
 * that gives up sets a status word on the device and the kernel returns.  This call synchronises
 * `stream`, reads and clears the word: EDB200_OK, or EDB200_ERR_TIMEOUT when a wait has given up since
 * the last poll (results produced after that point are not valid).  The *_compute_host entry points
 * poll by themselves; callers of the device-resident *_step entry points poll where they synchronise. */
EDB200_API edb200_status_t edb200_poll_status(void* stream);

/* Per-kernel-class timing for measurement runs.  Between begin and end every
 * kernel launch of this library is bracketed by CUDA events on its stream;
 * end synchronises the device and fills arrays of 5 entries indexed by class
 * {0 quantised GEMM, 1 attention, 2 GEMV, 3 memory-bound ops, 4 other} with the
 * summed device time (ms), algorithmic FLOPs, algorithmic bytes and launch
 * counts.  Counterpart of ED_PROFILE_RUNNER / ED_PROFILE_FLUX
 * (src/core/backend/ggml/ggml_extend.hpp:2842, src/dit_models/models/flux.hpp:82-95). */
EDB200_API edb200_status_t edb200_profile_begin(void);
EDB200_API edb200_status_t edb200_profile_end(double* ms, double* flops, double* bytes, int64_t* launches);

/* Tensor-pipe rate of this GPU: every SM issues tcgen05.mma 128 x 256 instructions back to back with
 * operands resident in shared memory (no loads), kind 0 = kind::f16 (f32 accumulate), 1 = kind::i8
 * (s32 accumulate); *tera_ops = 2 * MACs / time / 1e12.  Synchronises the stream.  A measurement aid
 * without a counterpart in the reference: the i8 / f16 ratio carries a measured dense bf16 GEMM peak
 * over to an INT8 peak for the roofline of the INT8-QK attention kernel. */
EDB200_API edb200_status_t edb200_probe_mma_rate(int kind, int iters, double* tera_ops, void* stream);

/* CUDA graphs.  Everything this library enqueues on `stream` between begin and end (for
 * example one whole edb200_*_step with fixed buffers) is recorded instead of executed and
 * can then be replayed with one launch: a step of several hundred small kernels stops being
 * bound by launch overhead.  Run the sequence once normally first (the first call of a kernel
 * sets attributes that cannot be captured), use a non-default stream, keep every buffer the
 * sequence touches alive and in place, and do not capture the NCCL exchange path.  Counterpart
 * of the reference's compiled-graph cache (ED_CACHE_COMPILED_GRAPHS,
 * src/dit_models/models/flux.hpp:5243-5270). */
typedef struct edb200_graph edb200_graph_t;
EDB200_API edb200_status_t edb200_graph_begin(void* stream);
EDB200_API edb200_status_t edb200_graph_end(void* stream, edb200_graph_t** out);
EDB200_API edb200_status_t edb200_graph_launch(edb200_graph_t* g, void* stream);
EDB200_API void edb200_graph_destroy(edb200_graph_t* g);

/* ------------------------------------------------------------------ codecs
 * ggml block codecs on the device.  Stand in for ggml_quantize_chunk /
 * type_traits->to_float as called from src/core/runtime/model_loader.cpp:663-704. */

/* Dequantise `rows` rows of `k` weights from raw ggml blocks (q8_0: 34 B per 32,
 * q4_K: 144 B per 256) to f32, bit-exact with ggml's dequantize_row_*. */
EDB200_API edb200_status_t edb200_dequantize_rows(int ggml_type, const void* blocks, float* out, int64_t rows, int64_t k,
                                       void* stream);
/* Quantise f32 rows to raw q8_0 blocks, bit-exact with quantize_row_q8_0_ref. */
EDB200_API edb200_status_t edb200_quantize_rows_q8_0(const float* x, void* blocks, int64_t rows, int64_t k, void* stream);
/* Fill `n` floats with N(mean, std) from a counter-based generator (synthetic weights). */
EDB200_API edb200_status_t edb200_fill_normal(float* out, int64_t n, uint64_t seed, float mean, float std, void* stream);

/* ----------------------------------------------------------------- weights
 * A quantised linear weight repacked once into the TMA-friendly device layout
 * (payload plane + per-32 scale planes).  Repacking changes no value: the
 * dequantised weight is identical to the ggml block's. */
typedef struct edb200_qweight edb200_qweight_t;

/* Build from raw ggml blocks resident on the device ([n_out rows] of k weights).
 * The raw buffer is not referenced after the call returns (the call
 * synchronises the stream).  Replaces the reference's bind_weights step
 * (src/core/runtime/model_loader.cpp:663-704) for the device copy. */
EDB200_API edb200_status_t edb200_qweight_create(int ggml_type, const void* blocks, int64_t n_out, int64_t k, void* stream,
                                      edb200_qweight_t** out);
EDB200_API void edb200_qweight_destroy(edb200_qweight_t* w);
/* Dequantise the repacked form back to f32 [n_out, k] (parity check of the repack). */
EDB200_API edb200_status_t edb200_qweight_dequantize(const edb200_qweight_t* w, float* out, void* stream);
/* Bytes of device memory held by the repacked weight. */
EDB200_API int64_t edb200_qweight_bytes(const edb200_qweight_t* w);

/* ----------------------------------------------------------------- mul_mat
 * y[m, n_out] = x[m, k] . W^T (+ bias) with a fused epilogue.  Stands in for
 * ggml_mul_mat on q8_0/q4_K weights as reached through ggml_ext_linear
 * (src/core/backend/ggml/ggml_extend.hpp:1308-1347) and Linear::forward
 * (:7675-7698), forward_output_slice (:7700-7731) and
 * forward_input_concat_residual_gate_fused (:7733-7831). */
/* Optional last stage of a QKV projection's epilogue: the first 3 * n_heads * d_head output features
 * (q heads | k heads | v heads; or one of the three, see `only`) do not go to `out` but straight to head-major attention operands, with the
 * per-head RMSNorm of q and k and the rotary embedding applied to the f32 accumulators on the way
 * (QKNorm, src/dit_models/components/common/normalization.cpp:71-99; apply_rope,
 * src/dit_models/components/common/rope.hpp:733-778) - the work of edb200_qk_norm_rope_pack without the
 * round trip of the projection's output through memory.  d_head is 128 (one 128-row weight tile = one head) or
 * 64 (two heads; n_heads must then be even); available when edb200_mul_mat_q_fuses_qk_pack() returns 1. */
typedef struct edb200_qk_pack {
    int n_heads, d_head;
    int only;                /* 0: the packed features are q | k | v (3 * n_heads * d_head of them);
                              * 1, 2, 3: they are the heads of q, k or v alone (n_heads * d_head), for models
                              * with separate to_q / to_k / to_v projections */
    const float* q_weight;   /* [d_head] RMSNorm weights, NULL = no norm */
    const float* k_weight;
    float eps;
    const float* pe;         /* [positions, d_head/2, 2, 2] f32 as edb200_qk_norm_rope_pack takes it, NULL = no RoPE;
                              * row `tok_off + i` belongs to output row i */
    int64_t tok_off;         /* position of output row 0 on the token axis of q_out / k_out / v_out */
    int64_t l_total;         /* tokens per head in the destination */
    void* q_out;             /* f16 [n_heads, l_total, d_head] (unused when `peers` is given) */
    void* k_out;
    void* v_out;
    /* sequence parallel: head h goes to rank h / (n_heads / world), at token position
     * rank * t_loc + tok_off + i of that rank's [n_heads / world, l_total, d_head] buffers */
    const edb200_sp_peers_t* peers;
} edb200_qk_pack_t;

typedef struct {
    const float* bias;     /* [n_out] or NULL */
    int act;               /* EDB200_ACT_* applied to columns < split_n */
    void* out;             /* primary output, row-major [m, ldo] */
    int out_dtype;         /* EDB200_TYPE_F32 / F16 / BF16 */
    int64_t ldo;           /* elements between output rows */
    /* Gated residual: out = residual + gate[n] * (acc + bias).  Requires
     * out_dtype F32; residual may alias out.  NULL gate = plain output. */
    const float* residual; /* [m, ld_res] f32 */
    int64_t ld_res;
    const float* gate;     /* [n_out] f32 */
    /* Column split: columns >= split_n are written to out2[:, col - split_n]
     * with act2 (0 = no split).  split_n must be a multiple of 128. */
    int64_t split_n;
    void* out2;
    int out2_dtype;
    int64_t ldo2;
    int act2;
    /* EDB200_SPLIT_K_NEVER (0): every output is one sum over k in a fixed order; the same bits
     * every run.  EDB200_SPLIT_K_UNORDERED: an in-place gated residual (out == residual, f32,
     * no activation, no column split, k >= 8192) whose output tiles are fewer than half the
     * SMs may cut the reduction into up to 4 parts that add into `out` with atomics; the order
     * of those adds, hence the last bit of the result, can differ between runs.  The
     * sequence-parallel executors ask for it: a rank's out-projections have few output tiles. */
    int split_k;
    /* NULL, or the head-major destination of the leading q | k | v features (see edb200_qk_pack_t).  The
     * packed features must end where the column split starts (split_n) or cover the whole output. */
    const edb200_qk_pack_t* pack;
} edb200_epilogue_t;

/* 1 when edb200_mul_mat_q honours edb200_epilogue_t.pack (the CTA-pair kernel is in use), else 0. */
EDB200_API int edb200_mul_mat_q_fuses_qk_pack(void);

/* x: [m, ldx] f16 (x_dtype = EDB200_TYPE_F16), 16-byte aligned rows.  Tensor-core
 * path (tcgen05 kind::f16: both operands share one 16-bit format and the weights
 * dequantise to f16 = rn(d*q), so bf16 activations return EDB200_ERR_UNSUPPORTED).
 * For m <= 8 use edb200_gemv_q. */
EDB200_API edb200_status_t edb200_mul_mat_q(const edb200_qweight_t* w, const void* x, int x_dtype, int64_t m, int64_t ldx,
                                 const edb200_epilogue_t* ep, void* stream);

/* Two independent problems in one launch (txt and img streams of a joint block). */
EDB200_API edb200_status_t edb200_mul_mat_q_pair(const edb200_qweight_t* w0, const void* x0, int64_t m0, int64_t ldx0,
                                      const edb200_epilogue_t* ep0, const edb200_qweight_t* w1, const void* x1,
                                      int64_t m1, int64_t ldx1, const edb200_epilogue_t* ep1, int x_dtype,
                                      void* stream);

/* y[n_out] = act_in(x[k]) . W^T + bias for `m` (<= 8) f32 input rows; weight
 * streaming, HBM bound.  pre_silu applies SiLU to x first (adaLN producers:
 * Modulation::forward, src/dit_models/models/flux.hpp:1617-1634). */
EDB200_API edb200_status_t edb200_gemv_q(const edb200_qweight_t* w, const float* x, int64_t m, int64_t ldx, int pre_silu,
                              const float* bias, float* y, int64_t ldy, void* stream);

/* Many weight-streaming products of ONE input vector in one launch: y_i[n_out_i] = act(x[k]) . W_i^T + bias_i
 * for i < n.  All weights share one block type and row length.  The adaLN projections of a whole
 * denoise step are such a batch (every Modulation::forward of the step reads silu(vec),
 * src/dit_models/models/flux.hpp:1617-1634, :3547-3555): one launch streams all their weights back to
 * back instead of one small launch per projection.  create stores the weight / bias / output
 * addresses on the device (they must stay valid; bias may be NULL, or hold NULL entries); run
 * may be recorded into a CUDA graph.  `share` != NULL (sequence parallel, peer memory mapped): the
 * ranks split the rows of the batch between them and store their part into every rank's outputs;
 * share->buf[0][p] is rank p's mapping of one common address (e.g. the start of the output
 * area), outputs must lie at the same offsets on every rank, and a barrier (edb200_sp_barrier)
 * must follow before the results are read. */
typedef struct edb200_gemv_batch edb200_gemv_batch_t;
EDB200_API edb200_status_t edb200_gemv_batch_create(const edb200_qweight_t* const* w, const float* const* bias,
                                                    float* const* y, int n, void* stream, edb200_gemv_batch_t** out);
EDB200_API void edb200_gemv_batch_destroy(edb200_gemv_batch_t* b);
EDB200_API edb200_status_t edb200_gemv_batch_run(const edb200_gemv_batch_t* b, const float* x, int pre_silu,
                                                 const edb200_sp_peers_t* share, void* stream);

/* Dense f32 weight, the unquantised linears of the prelude / final layer:
 * y[m, n] = act(x[m, k] . W[n, k]^T + bias).  x f32, y f32.  Up to 8 rows: weight-streaming GEMV (exact f32).
 * From 9 rows on (k >= 32 and a multiple of 4, n >= 32, 16-byte aligned operands): tensor cores, which read the f32 operands as
 * tf32 - 10 mantissa bits, f32 accumulation (EDB200_LINEAR_TF32=0 in the environment keeps it on SIMT f32). */
EDB200_API edb200_status_t edb200_linear_f32(const float* w, const float* bias, const float* x, int64_t m, int64_t k,
                                  int64_t n, int64_t ldx, int pre_silu, int act, float* y, int64_t ldy,
                                  void* stream);

/* ------------------------------------------------------ memory-bound ops */

/* y = modulate(LayerNorm(x)):  xn = (x - mean) * rsqrt(var + eps) [* ln_weight + ln_bias],
 * y = (xn + xn*scale) + shift.  x f32 [rows, ldx]; shift/scale/ln_* f32 [h] or
 * NULL; y f32/f16/bf16 [rows, ldy].  Fuses LayerNorm::forward
 * (src/core/backend/ggml/ggml_extend.hpp:8127-8155, ggml_norm eps 1e-6) with
 * dit::modulate (src/dit_models/components/common/modulation.cpp:9-47). */
EDB200_API edb200_status_t edb200_layernorm_modulate(const float* x, int64_t ldx, const float* shift, const float* scale,
                                          const float* ln_weight, const float* ln_bias, int64_t rows, int64_t h,
                                          float eps, void* y, int y_dtype, int64_t ldy, void* stream);

/* y = (x + x*scale) + shift, f32, no FMA contraction: bit-identical to
 * fused_modulate_cpu_custom_op (src/core/backend/ggml/ed_ggml_modulation_ext.hpp:168-199)
 * and ed_cuda_fused_modulate_custom_compute (cuda/ed_cuda_modulation.cu:528-532).
 * x,y [rows, h] contiguous; shift/scale [h] broadcast over rows. */
EDB200_API edb200_status_t edb200_fused_modulate(const float* x, const float* shift, const float* scale, float* y, int64_t rows,
                                      int64_t h, void* stream);

/* y = residual + x*gate, f32, bit-identical to fused_residual_gate_cpu_custom_op
 * (src/core/backend/ggml/ed_ggml_modulation_ext.hpp:201-226). */
EDB200_API edb200_status_t edb200_fused_residual_gate(const float* residual, const float* x, const float* gate, float* y,
                                           int64_t rows, int64_t h, void* stream);

/* The sampler's latent update of one denoise step, in place on the device, so that the latent
 * never returns to the host between steps (src/dit_models/pipelines/flux_pipeline.cpp:1111-1112,
 * :1290-1297; the same form in sd3_pipeline.cpp):
 *   denoised = model_out * (-sigma) + x;
 *   sigma == 0 ? x = denoised : x += ((x - denoised) / sigma) * (sigma_next - sigma)
 * f32, each operation rounded on its own in that order (no FMA contraction): the reference's bits. */
EDB200_API edb200_status_t edb200_euler_update(float* x, const float* model_out, float sigma, float sigma_next, int64_t n,
                                    void* stream);
/* SD3's form of the same update (src/dit_models/pipelines/sd3_pipeline.cpp:697):
 * x += model_out * (sigma_next - sigma), f32, the difference, the product and the sum each rounded. */
EDB200_API edb200_status_t edb200_flow_update(float* x, const float* model_out, float sigma, float sigma_next, int64_t n,
                                   void* stream);
/* SD3's update with the schedule on the device: dt = sigmas[*step + 1] - sigmas[*step], then *step is
 * incremented (see edb200_euler_update_sched). */
EDB200_API edb200_status_t edb200_flow_update_sched(float* x, const float* model_out, const float* sigmas, int* step,
                                                    int64_t n, void* stream);
/* out = a - b, f32, n a multiple of 4 (e.g. the block stack's residual ModelOut - ModelIn that a reuse policy
 * stores, src/core/optimization/cache/tensor_cache_utils.hpp). */
EDB200_API edb200_status_t edb200_sub_f32(const float* a, const float* b, float* out, int64_t n, void* stream);
/* The same update with the schedule on the device: sigma = sigmas[*step], sigma_next =
 * sigmas[*step + 1]; afterwards *step is incremented (a second, one-thread kernel).  Together with
 * edb200_flux_step_sched this makes one recorded step + update (edb200_graph_*) replayable for
 * every step of a schedule: nothing in it depends on a by-value sigma. */
EDB200_API edb200_status_t edb200_euler_update_sched(float* x, const float* model_out, const float* sigmas, int* step,
                                          int64_t n, void* stream);

/* Per-head RMSNorm of q and k (weights [d_head] or NULL), RoPE with the
 * reference's pe table [l_total, d_head/2, 2, 2] (NULL = none), and head-major
 * pack of q, k, v into [n_heads, l_total, d_head] at token offset tok_off.
 * qkv is [tokens, ld] with q/k/v starting at element offsets q_off/k_off/v_off
 * of each row, heads contiguous.  Stands in for QKNorm::query_norm/key_norm
 * (src/dit_models/components/common/normalization.cpp:71-99), rope_custom_3d
 * (src/core/backend/ggml/ed_ggml_rope_ext.hpp:226-262), the txt||img concat
 * (src/dit_models/models/flux.hpp:1842-1844) and attention_v_prep /
 * attention_qkv_pair_pack (src/core/backend/ggml/ed_ggml_attention_ext.hpp:269-369). */
EDB200_API edb200_status_t edb200_qk_norm_rope_pack(const void* qkv, int in_dtype, int64_t ld, int64_t q_off, int64_t k_off,
                                         int64_t v_off, int64_t tokens, int n_heads, int d_head, const float* q_weight,
                                         const float* k_weight, float eps, const float* pe, int64_t tok_off,
                                         int64_t l_total, void* q_out, void* k_out, void* v_out, int out_dtype,
                                         void* stream);
/* The same with the heads exchange of sequence parallelism fused in: head h of the
 * local tokens is written into rank h / (n_heads / world)'s
 * [n_heads / world, l_total, d_head] q, k, v buffers (dst->buf[0..2]) at global token
 * position rank * t_loc + tok_off + t; `pe` is the table of the whole sequence.
 * Replaces the SP pack callbacks plus the seq->head all-to-all
 * (src/core/parallel/sp_parallel.cpp:99-469, src/core/parallel/backends/nccl/nccl_process_group.cpp:394-459). */
EDB200_API edb200_status_t edb200_qk_norm_rope_pack_sp(const void* qkv, int in_dtype, int64_t ld, int64_t q_off,
                                                       int64_t k_off, int64_t v_off, int64_t tokens, int n_heads,
                                                       int d_head, const float* q_weight, const float* k_weight,
                                                       float eps, const float* pe, int64_t tok_off, int64_t l_total,
                                                       const edb200_sp_peers_t* dst, int out_dtype, void* stream);

/* Whole-row RMSNorm in two parts (Wan norms q and k over all heads before the head
 * split: WanSelfAttention::forward, src/dit_models/models/wan.hpp:3504-3532; ggml-side
 * RMSNorm, src/core/backend/ggml/ggml_extend.hpp:8248-8282):
 *   out[row] = 1 / sqrt(mean(x[row, 0..cols)^2) + eps)                       */
EDB200_API edb200_status_t edb200_row_rstd(const void* x, int dtype, int64_t ld, int64_t rows, int64_t cols, float eps,
                                           float* out, void* stream);
/* ... and the pack that applies it: like edb200_qk_norm_rope_pack, but q and k are
 * scaled by rstd_q / rstd_k [tokens] and by weights over the whole row
 * [n_heads * d_head]; weight NULL = no norm, pe NULL = no RoPE, an output pointer
 * NULL = that tensor is skipped (cross-attention packs q alone, or k and v alone).
 * dst != NULL stores into the owning ranks as edb200_qk_norm_rope_pack_sp does. */
EDB200_API edb200_status_t edb200_qk_rownorm_rope_pack(const void* qkv, int in_dtype, int64_t ld, int64_t q_off,
                                                       int64_t k_off, int64_t v_off, int64_t tokens, int n_heads,
                                                       int d_head, const float* q_weight, const float* k_weight,
                                                       const float* rstd_q, const float* rstd_k, const float* pe,
                                                       int64_t tok_off, int64_t l_total, void* q_out, void* k_out,
                                                       void* v_out, int out_dtype, const edb200_sp_peers_t* dst,
                                                       void* stream);

/* Elementwise dtype conversion (f32/f16/bf16), n a multiple of 4
 * (ggml_cast call sites, e.g. src/dit_models/models/flux.hpp:101-111). */
EDB200_API edb200_status_t edb200_cast(const void* x, int in_dtype, void* y, int out_dtype, int64_t n, void* stream);

/* -------------------------------------------------------------- attention
 * Non-causal softmax(Q K^T * scale) V.  q [hn, lq, d_head], k/v [hn, lk, d_head]
 * f16 head-major (d contiguous); out [lq, ld_out] token-major with head h at
 * columns h*d_head.., f32/f16/bf16.  d_head 64 or 128.  Stands in for
 * ggml_ext_attention_ext -> ggml_flash_attn_ext / cuDNN SDPA
 * (src/core/backend/ggml/ggml_extend.hpp:1749-1984, src/core/backend/cuDNN/ed_cudnn_sdpa.cu:1115)
 * including the head-major -> [d*H, L] re-layout that follows it. */
EDB200_API edb200_status_t edb200_attention_f16(const void* q, const void* k, const void* v, int hn, int64_t lq,
                                                int64_t lk, int d_head, float scale, void* out, int out_dtype,
                                                int64_t ld_out, void* stream);

/* The same on buffers laid out for a longer (padded) sequence: consecutive heads are q_head_rows
 * (>= lq) rows apart in q and kv_head_rows (>= lk) rows apart in k and v, and only the first lq / lk
 * rows of every head are read.  This is how a sequence-parallel rank attends over a sequence that was
 * padded to a multiple of the world size (src/core/parallel/sp_parallel.cpp:757-768) without computing
 * on the padding.  dst may be NULL (plain output) or the peer description of edb200_attention_f16_sp. */
EDB200_API edb200_status_t edb200_attention_f16_strided(const void* q, const void* k, const void* v, int hn, int64_t lq,
                                                        int64_t lk, int64_t q_head_rows, int64_t kv_head_rows,
                                                        int d_head, float scale, void* out, int out_dtype,
                                                        int64_t ld_out, const edb200_sp_peers_t* dst, void* stream);

/* Sage path.  Scratch is caller-allocated like the reference's
 * (src/core/backend/ggml/cuda/ed_cuda_sage_attn.h:19-71): query the size, pass a
 * 256-byte aligned device buffer. */
EDB200_API int64_t edb200_sage_scratch_bytes(int hn, int64_t l, int d_head);
/* Byte offsets of {q8, k8, q_scale, k_scale, q_mean, k_mean, bias, total} and the
 * row strides {q_scale, k_scale, bias} inside the scratch buffer. */
EDB200_API edb200_status_t edb200_sage_scratch_layout(int hn, int64_t l, int d_head, int64_t* offsets, int* strides);
/* `smooth_q` arguments below are a bit set: EDB200_SAGE_SMOOTH_Q subtracts the
 * per-channel Q mean and adds the rank-1 bias back (ED_SAGE_SMOOTH_Q);
 * EDB200_SAGE_FAST_MEANS computes the channel means with a chunked parallel sum
 * instead of the reference's sequential one (deterministic, last-bit different;
 * the means cancel in the softmax, so only rounding changes). */
enum { EDB200_SAGE_SMOOTH_Q = 1, EDB200_SAGE_FAST_MEANS = 2 };
/* INT8 quantisation of smoothed Q and K, bit-exact with the reference kernels
 * sage_k_mean / sage_q_mean / sage_quant_q_perwarp / sage_quant_k_perblock_smoothk /
 * sage_smooth_q_bias (src/core/backend/ggml/cuda/ed_cuda_sage_attn.cu:61-281). */
EDB200_API edb200_status_t edb200_sage_quantize_qk(const void* q_f16, const void* k_f16, int hn, int64_t l, int d_head,
                                                   int smooth_q, void* scratch, int64_t scratch_bytes, void* stream);
/* INT8 QK^T attention on already quantised operands (main kernel of run_sage,
 * src/core/backend/ggml/cuda/ed_cuda_sage_attn.cu:834-1122).  q_scale one per 32
 * query rows, k_scale one per 64 keys, bias one per key (NULL = no smooth-Q);
 * rows of all three must cover l rounded up to 128.  d_head 64 or 128 (the reference gates its
 * Sage path on exactly these, src/core/backend/ggml/ggml_extend.hpp:1916-1928). */
EDB200_API edb200_status_t edb200_attention_sage_int8(const void* q_i8, const void* k_i8, const void* v_f16,
                                                      const float* q_scale, int q_scale_stride,
                                                      const float* k_scale, int k_scale_stride, const float* bias,
                                                      int bias_stride, int hn, int64_t l, int d_head, float scale,
                                                      void* out, int out_dtype, int64_t ld_out, void* stream);
/* Quantise + attend (sage_attn_custom, src/core/backend/ggml/ed_ggml_sage_attn_ext.hpp:252-288). */
EDB200_API edb200_status_t edb200_sage_attention(const void* q_f16, const void* k_f16, const void* v_f16, int hn,
                                                 int64_t l, int d_head, float scale, int smooth_q, void* scratch,
                                                 int64_t scratch_bytes, void* out, int out_dtype, int64_t ld_out,
                                                 void* stream);
/* Variants for inputs whose heads are head_rows (>= l) rows apart (padded sequence, see
 * edb200_attention_f16_strided); the INT8 copies and their scales in the scratch buffer stay dense. */
EDB200_API edb200_status_t edb200_sage_quantize_qk_strided(const void* q_f16, const void* k_f16, int hn, int64_t l,
                                                           int64_t head_rows, int d_head, int smooth_q, void* scratch,
                                                           int64_t scratch_bytes, void* stream);
EDB200_API edb200_status_t edb200_attention_sage_int8_strided(const void* q_i8, const void* k_i8, const void* v_f16,
                                                              int64_t v_head_rows, const float* q_scale,
                                                              int q_scale_stride, const float* k_scale,
                                                              int k_scale_stride, const float* bias, int bias_stride,
                                                              int hn, int64_t l, int d_head, float scale, void* out,
                                                              int out_dtype, int64_t ld_out,
                                                              const edb200_sp_peers_t* dst, void* stream);
EDB200_API edb200_status_t edb200_sage_attention_strided(const void* q_f16, const void* k_f16, const void* v_f16, int hn,
                                                         int64_t l, int64_t head_rows, int d_head, float scale,
                                                         int smooth_q, void* scratch, int64_t scratch_bytes, void* out,
                                                         int out_dtype, int64_t ld_out, const edb200_sp_peers_t* dst,
                                                         void* stream);
/* Per-channel key means (the smooth-K vector, chunked sum as with
 * EDB200_SAGE_FAST_MEANS) for callers that cannot hand over or allocate device
 * scratch.  No counterpart in the reference, whose means always live in the
 * caller's scratch buffer.  The chunk sums go to a 1 MiB array that is part of the
 * library image, so the call performs no allocation of any kind; mean_out
 * [hn, d_head] f32 is the only buffer the caller provides.
 *  - Limit: hn * ceil(l / 128) * d_head * 4 bytes <= 1 MiB (24 heads x 128 reach
 *    10880 tokens); larger problems return EDB200_ERR_UNSUPPORTED.
 *  - The first call on each device looks up the array's device address; make that
 *    call before starting a stream capture.
 *  - All calls on one device share the array: two calls whose kernels may overlap
 *    (different streams, no ordering) race on it.  Nothing in it needs clearing. */
EDB200_API edb200_status_t edb200_sage_key_means_static(const void* k_f16, int hn, int64_t l, int d_head,
                                                        float* mean_out, void* stream);

/* --------------------------------------- sequence-parallel (Ulysses) exchange
 * One process per GPU.  Every rank owns n_tokens / world consecutive tokens of the
 * [text ; image] sequence for the per-token work and heads / world heads for
 * attention.  Replaces the reference's SP pack / split / gather callbacks
 * (src/core/parallel/sp_parallel.cpp:99-469,793-831) and NCCL all-to-all
 * (src/core/parallel/backends/nccl/nccl_process_group.cpp:394-459). */
typedef struct edb200_comm edb200_comm_t;
/* Token slice of `rank`.  The sequence is padded to a multiple of the world size like the reference's
 * sp_sequence_padding (src/core/parallel/sp_parallel.cpp:757-768): every rank has a slot of
 * t_loc = ceil(n_tokens / world) rows, of which it owns the first t_rows (less than t_loc, possibly 0,
 * on the last ranks when the sequence does not divide); the first n_txt_local of them are text rows;
 * img_first = index of its first image token among the image tokens.  Padding rows are never
 * computed: attention runs over the n_tokens real rows of buffers laid out for world * t_loc.
 * Pure host arithmetic (no device needed). */
EDB200_API edb200_status_t edb200_sp_shard(int64_t n_tokens, int64_t n_txt, int rank, int world, int64_t* t_loc,
                                           int64_t* n_txt_local, int64_t* img_first, int64_t* t_rows);
/* Message list of the heads exchange [heads, t_loc, row] -> [heads/world, T, row]:
 * message i goes to and comes from peer[i], `bytes[i]` bytes from send_off[i] of the
 * send buffer and to recv_off[i] of the receive buffer.  Returns the number of
 * messages (call with peer == NULL to size the arrays), -1 on a bad argument.
 * Pure host arithmetic; the NCCL path below executes exactly this list. */
EDB200_API int edb200_sp_heads_plan(int rank, int world, int heads, int64_t t_loc, int64_t row_bytes, int* peer,
                                    int64_t* send_off, int64_t* recv_off, int64_t* bytes, int cap);
/* NCCL communicator over the ranks of one node (libnccl.so.2 is resolved from the
 * running process at first use).  Rank 0 makes the 128-byte id, the host program
 * distributes it (e.g. torch.distributed broadcast), every rank calls create. */
EDB200_API edb200_status_t edb200_comm_unique_id(void* id128);
EDB200_API edb200_status_t edb200_comm_create(const void* id128, int rank, int world, edb200_comm_t** out);
EDB200_API void edb200_comm_destroy(edb200_comm_t* c);
/* A communicator of `world` ranks with no transport behind it: edb200_comm_map_peers maps every
 * "peer" onto the caller's own allocation, the NCCL exchanges return EDB200_ERR_UNSUPPORTED.  For
 * single-process tests of code that needs a mapped communicator, e.g. letting edb200_sp_barrier run
 * into its time limit because no other rank ever arrives (ProcessGroup stubs of the reference:
 * src/core/parallel/backends/cpu/cpu_process_group.cpp). */
EDB200_API edb200_status_t edb200_comm_create_loopback(int rank, int world, edb200_comm_t** out);
/* Limit of the device-side wait of edb200_sp_barrier in milliseconds (default 2000, 1..60000). */
EDB200_API edb200_status_t edb200_comm_set_timeout_ms(edb200_comm_t* c, int64_t ms);
/* The decision rule of edb200_comm_map_peers, exported for host tests: 1 when ok[p * stride] == 1
 * for every rank p, else 0.  Every rank evaluates it on the same gathered bytes. */
EDB200_API int edb200_comm_all_ok(const unsigned char* ok, int stride, int world);
EDB200_API int edb200_comm_rank(const edb200_comm_t* c);
EDB200_API int edb200_comm_world(const edb200_comm_t* c);
/* Peer memory.  Every rank passes ONE device allocation of the same size and layout
 * (`base`, from cudaMalloc); afterwards edb200_comm_peer_ptr translates an address
 * inside this rank's allocation into the same place of `peer`'s allocation as
 * addressed from this GPU (CUDA IPC mapping, plain loads and stores over NVLink).
 * flags_off names 1024 bytes inside the allocation that the barrier below owns (eight flag
 * words and the barrier's epoch counter).
 * Collective over the communicator: every rank runs both of its rendezvous even when its own
 * handle export or one of its handle imports fails, and carries that failure in the message, so
 * all ranks return the same status together: EDB200_OK, or EDB200_ERR_UNSUPPORTED (nothing stays
 * mapped on any rank) where IPC mappings are not available on some rank, and the NCCL
 * exchanges below remain usable.  unmap is collective too and must come before the
 * allocation is freed. */
EDB200_API edb200_status_t edb200_comm_map_peers(edb200_comm_t* c, void* base, int64_t bytes, int64_t flags_off,
                                                 void* stream);
EDB200_API edb200_status_t edb200_comm_unmap_peers(edb200_comm_t* c);
EDB200_API int edb200_comm_peers_mapped(const edb200_comm_t* c);
EDB200_API void* edb200_comm_peer_ptr(const edb200_comm_t* c, int peer, const void* local_ptr);
/* Barrier across the ranks' streams, one small kernel per rank: everything this rank
 * enqueued before it (including its stores into peer memory) is visible to every
 * rank's work enqueued after it.  The barrier's epoch counter lives in device memory and the
 * kernel advances it, so a recorded barrier (edb200_graph_*) works on every replay.  The
 * device-side wait gives up after the communicator's time limit (edb200_comm_set_timeout_ms,
 * default two seconds) and edb200_poll_status then reports EDB200_ERR_TIMEOUT. */
EDB200_API edb200_status_t edb200_sp_barrier(edb200_comm_t* c, void* stream);
/* Heads exchange of n_tensors buffers (Q, K, V) in one NCCL group; no pack or
 * unpack kernel: every message is contiguous on both sides. */
EDB200_API edb200_status_t edb200_sp_all_to_all_heads(edb200_comm_t* c, const void* const* send, void* const* recv,
                                                      int n_tensors, int heads, int64_t t_loc, int64_t row_bytes,
                                                      void* stream);
/* Tokens exchange of the attention output: send [T, chunk] (this rank's heads, all
 * tokens) -> out [t_loc, world * chunk] with row pitch ld_out_bytes (all heads,
 * this rank's tokens), through `staging` (world * t_loc * chunk bytes). */
EDB200_API edb200_status_t edb200_sp_all_to_all_tokens(edb200_comm_t* c, const void* send, void* staging, void* out,
                                                       int64_t t_loc, int64_t chunk_bytes, int64_t ld_out_bytes,
                                                       void* stream);
/* All-gather of row blocks of unequal length: rank p contributes row_count[p] rows
 * that land at row row_first[p] of every rank's `recv`. */
EDB200_API edb200_status_t edb200_sp_all_gather_rows(edb200_comm_t* c, const void* send, void* recv,
                                                     const int64_t* row_first, const int64_t* row_count,
                                                     int64_t row_bytes, void* stream);

/* The same over peer memory (needs edb200_comm_map_peers; `recv` must lie inside the mapped allocation at the
 * same offset on every rank): a kernel stores this rank's rows into every rank's `recv`, then
 * edb200_sp_barrier orders the stores before whatever reads `recv` next.  No library exchange is
 * involved, so the call can be recorded into a CUDA graph.  Rows must be multiples of 16 bytes. */
EDB200_API edb200_status_t edb200_sp_all_gather_rows_peer(edb200_comm_t* c, const void* send, void* recv,
                                                          const int64_t* row_first, const int64_t* row_count,
                                                          int64_t row_bytes, void* stream);

/* Attention with the tokens exchange of sequence parallelism fused in: this rank
 * computes `hn` heads for all l tokens and stores query row r into rank r / t_loc's
 * buffer dst->buf[0][..] (row r % t_loc, columns (rank * hn + head) * d_head .., row
 * pitch ld_out).  `out` may be NULL.  Replaces the head->seq all-to-all and its
 * pack / recv-prep kernels (src/core/backend/ggml/cuda/ed_cuda_sp_flux.cu:443-1628). */
EDB200_API edb200_status_t edb200_attention_f16_sp(const void* q, const void* k, const void* v, int hn, int64_t lq,
                                                   int64_t lk, int d_head, float scale, void* out, int out_dtype,
                                                   int64_t ld_out, const edb200_sp_peers_t* dst, void* stream);
EDB200_API edb200_status_t edb200_attention_sage_int8_sp(const void* q_i8, const void* k_i8, const void* v_f16,
                                                         const float* q_scale, int q_scale_stride,
                                                         const float* k_scale, int k_scale_stride, const float* bias,
                                                         int bias_stride, int hn, int64_t l, int d_head, float scale,
                                                         void* out, int out_dtype, int64_t ld_out,
                                                         const edb200_sp_peers_t* dst, void* stream);
EDB200_API edb200_status_t edb200_sage_attention_sp(const void* q_f16, const void* k_f16, const void* v_f16, int hn,
                                                    int64_t l, int d_head, float scale, int smooth_q, void* scratch,
                                                    int64_t scratch_bytes, void* out, int out_dtype, int64_t ld_out,
                                                    const edb200_sp_peers_t* dst, void* stream);

/* CFG-parallel step on a 2-rank communicator (cfg_all_gather, src/core/parallel/cfg_parallel.cpp:38-108):
 * rank 0 has run the conditional pass, rank 1 the unconditional one; both receive
 * out = uncond + scale * (cond - uncond).  `gathered` is scratch for 2 * n floats.  Combine it with
 * sequence parallelism by giving every branch its own edb200_comm_t for the model. */
EDB200_API edb200_status_t edb200_cfg_parallel_combine(edb200_comm_t* c, const float* mine, float scale,
                                                       float* gathered, float* out, int64_t n, void* stream);

/* The same with Qwen-Image's norm-preserving combine (edb200_cfg_combine_rescaled) after the gather;
 * tensors f32 [channels, height, width], `gathered` holds 2 * channels * height * width floats. */
EDB200_API edb200_status_t edb200_cfg_parallel_combine_rescaled(edb200_comm_t* c, const float* mine, float scale,
                                                                int patch_size, int channels, int height, int width,
                                                                float* gathered, float* out, void* stream);

/* ------------------------------------------------------------ weight ingest
 * Reader for GGUF files, the container the reference's converter writes and its loader reads
 * (src/utils/model_io/gguf_io.cpp, src/core/runtime/model_loader.cpp).  The file is mapped; tensor
 * data pointers stay valid until edb200_gguf_close.  ggml_type is the file's own type code
 * (0 f32, 1 f16, 8 q8_0, 12 q4_K, 30 bf16, ...); dims are in ggml order (dims[0] = row length);
 * nbytes is -1 for a type this library does not read.  Host code: no GPU is needed. */
typedef struct edb200_gguf edb200_gguf_t;
EDB200_API edb200_status_t edb200_gguf_open(const char* path, edb200_gguf_t** out);
EDB200_API void edb200_gguf_close(edb200_gguf_t* g);
EDB200_API int edb200_gguf_tensor_count(const edb200_gguf_t* g);
EDB200_API edb200_status_t edb200_gguf_tensor_info(const edb200_gguf_t* g, int index, char* name, int name_cap,
                                                   int* ggml_type, int* n_dims, int64_t* dims /* [4] */,
                                                   int64_t* nbytes);
EDB200_API const void* edb200_gguf_tensor_data(const edb200_gguf_t* g, int index);

/* Reader for safetensors files (src/utils/model_io/safetensors_io.h): name, dtype string ("F32", "F16",
 * "BF16", ...), row-major shape (up to 8 extents) and the mapped data of every tensor.  Host code. */
typedef struct edb200_safetensors edb200_safetensors_t;
EDB200_API edb200_status_t edb200_safetensors_open(const char* path, edb200_safetensors_t** out);
EDB200_API void edb200_safetensors_close(edb200_safetensors_t* f);
EDB200_API int edb200_safetensors_tensor_count(const edb200_safetensors_t* f);
EDB200_API edb200_status_t edb200_safetensors_tensor_info(const edb200_safetensors_t* f, int index, char* name,
                                                          int name_cap, char* dtype, int dtype_cap, int* n_dims,
                                                          int64_t* dims /* [8] */, int64_t* nbytes);
EDB200_API const void* edb200_safetensors_tensor_data(const edb200_safetensors_t* f, int index);
/* The shard files a `*.safetensors.index.json` names in its weight_map (src/core/runtime/model_loader.cpp:296-327),
 * each once, resolved against the index's directory, written to `out` one per line.  The
 * edb200_*_load_safetensors calls accept such an index in place of a single file. */
EDB200_API edb200_status_t edb200_safetensors_index_files(const char* index_path, char* out, int out_cap, int* n_files);

/* Tensor-name canonicalisation of the weight loaders.  A checkpoint in the diffusers layout names the DiT's
 * tensors differently from the layout the step executors register; convert_diffusion_model_name
 * (src/utils/name_conversion.cpp:802-822, per family :439-543 SD3, :545-657 FLUX, :773-800 Wan) maps one to
 * the other, marking the 2nd, 3rd, ... projection of a fused tensor (q,k,v -> qkv; q,k,v,mlp -> linear1) with a
 * numeric suffix.  `out` receives the base name, `*part` the part index (0 for whole tensors and first parts).
 * Names already in the executors' layout pass through.  Qwen-Image keeps the diffusers names natively.
 * Every edb200_*_load_gguf / _load_safetensors call applies this, assembles fused tensors from their parts in
 * part order (ModelLoader::load_tensors, src/core/runtime/model_loader.cpp:2019-2113) and converts a tensor
 * stored in another type than the model keeps (f32 / f16 / bf16 / q8_0 / q4_K in, convert_tensor_data,
 * src/core/runtime/model_loader.cpp:663-704).  Host code. */
enum { EDB200_FAMILY_FLUX = 0, EDB200_FAMILY_SD3 = 1, EDB200_FAMILY_QWEN = 2, EDB200_FAMILY_WAN = 3 };
EDB200_API edb200_status_t edb200_canonical_tensor_name(int family, const char* name, char* out, int64_t capacity,
                                                        int* part);

/* ------------------------------------------------- FLUX.1 denoise-step model
 * A whole-step replacement at the reference's model seam
 * DiffusionModel::compute(n_threads, DiffusionParams) -> sd::Tensor<float>
 * (src/dit_models/diffusion_model.hpp:67-70) for FluxModel / FluxRunner::compute
 * (src/dit_models/models/flux.hpp:5158-5296).  Field names follow FluxParams
 * (src/dit_models/models/flux.hpp:3717-3745). */
enum { EDB200_ATTN_F16 = 0, EDB200_ATTN_SAGE_INT8 = 1 };

typedef struct {
    int hidden_size;          /* 3072 */
    int num_heads;            /* 24 */
    int depth;                /* double-stream blocks, 19 */
    int depth_single_blocks;  /* 38 */
    int mlp_hidden;           /* hidden_size * mlp_ratio, 12288 */
    int in_channels;          /* latent channels * patch^2, 64 */
    int context_in_dim;       /* 4096 */
    int vec_in_dim;           /* 768 */
    int patch_size;           /* 2 */
    int axes_dim[3];          /* RoPE axes, (16, 56, 56) */
    int theta;                /* 10000 */
    int guidance_embed;       /* 1 for FLUX.1-dev */
    int wtype;                /* EDB200_TYPE_Q8_0 or EDB200_TYPE_Q4_K */
    int attention;            /* EDB200_ATTN_* (ED_SAGE_ATTN in the reference) */
    int sage_smooth_q;        /* ED_SAGE_SMOOTH_Q */
} edb200_flux_config_t;

typedef struct edb200_flux edb200_flux_t;

EDB200_API edb200_status_t edb200_flux_create(const edb200_flux_config_t* cfg, edb200_flux_t** out);
EDB200_API void edb200_flux_destroy(edb200_flux_t* m);
/* Parameter table: names are the reference's tensor names without the
 * "model.diffusion_model." prefix (e.g. "double_blocks.0.img_attn.qkv.weight").
 * Stands in for GGMLRunner::get_param_tensors (src/core/backend/ggml/ggml_extend.hpp). */
EDB200_API int edb200_flux_tensor_count(const edb200_flux_t* m);
EDB200_API edb200_status_t edb200_flux_tensor_info(const edb200_flux_t* m, int index, char* name, int name_cap,
                                                   int* ggml_type, int64_t* n_out, int64_t* k, int64_t* nbytes);
/* Upload one tensor from host (on_device = 0) or device memory: raw ggml blocks
 * for quantised weights, f32 for everything else. */
EDB200_API edb200_status_t edb200_flux_set_tensor(edb200_flux_t* m, const char* name, int ggml_type, const void* data,
                                                  int64_t nbytes, int on_device, void* stream);
/* Reads one tensor back as f32 [n_out, k] into host (on_device = 0) or device memory; a quantised weight
 * is dequantised from its repacked device form (the values ggml's dequantize_row gives for the blocks
 * that were loaded).  n_floats must equal n_out * k.  Synchronises the stream.  Lets a checker run on
 * exactly the weights the device holds, e.g. after edb200_flux_init_random. */
EDB200_API edb200_status_t edb200_flux_get_tensor_f32(const edb200_flux_t* m, const char* name, float* out,
                                                      int64_t n_floats, int on_device, void* stream);
/* Loads every tensor of a GGUF file this model has a parameter for (names compared after removing
 * `strip_prefix`, e.g. "model.diffusion_model."; NULL = none); other tensors are skipped.  Quantised
 * weights must be stored in the model's block type; f16 / bf16 vectors are widened to f32.
 * *n_loaded (may be NULL) = tensors taken. */
EDB200_API edb200_status_t edb200_flux_load_gguf(edb200_flux_t* m, const char* path, const char* strip_prefix,
                                               int* n_loaded, void* stream);
/* The same from a safetensors file (F32 / F16 / BF16 tensors).  Parameters the model keeps quantised are
 * encoded on the device in its block type while they load: q8_0 by ggml's rule (bit for bit), q4_K by this
 * library's min/max encoder. */
EDB200_API edb200_status_t edb200_flux_load_safetensors(edb200_flux_t* m, const char* path, const char* strip_prefix,
                                                      int* n_loaded, void* stream);
/* Synthetic weights N(0, std) generated and quantised on the device. */
EDB200_API edb200_status_t edb200_flux_init_random(edb200_flux_t* m, uint64_t seed, float std, void* stream);
EDB200_API int64_t edb200_flux_weight_bytes(const edb200_flux_t* m);
EDB200_API int64_t edb200_flux_workspace_bytes(const edb200_flux_t* m);
/* Allocate the activation workspace and build the RoPE table for one
 * (latent height, latent width, text tokens) shape; a no-op when unchanged. */
EDB200_API edb200_status_t edb200_flux_prepare(edb200_flux_t* m, int latent_h, int latent_w, int n_txt, void* stream);
/* Optional debug tap: after block b (double blocks first) the f32 residual
 * stream [n_txt + n_img, hidden] is copied to tap + b * T * hidden.  NULL disables. */
EDB200_API edb200_status_t edb200_flux_set_tap(edb200_flux_t* m, float* tap);
/* Computation-reuse seam: the three anchors the reference's cache engine taps in the FLUX graph
 * (src/dit_models/models/flux.hpp:3968-3978 ModelIn, :4260-4266 BlockOut[i] with the probe stop,
 * :4511-4520 whole-stack inject and ModelOut).  All of them are views of the IMAGE stream
 * [image tokens (of this rank), hidden] f32.
 *   set_anchor_capture  during the following steps the stream at `anchor` is copied to dst (device);
 *                       anchor = EDB200_ANCHOR_MODEL_IN / _MODEL_OUT or a double-block index; NULL stops it
 *   set_stop_after      the step returns right after double block `block` (its BlockOut capture made,
 *                       `out` untouched): the probe pass of a policy that decides from an early block; -1 = off
 *   set_stream_override the step runs no block at all: the stream after the stack is ModelIn + residual
 *                       (device, same shape), then the final layer as usual; NULL = off */
enum { EDB200_ANCHOR_MODEL_IN = -1, EDB200_ANCHOR_MODEL_OUT = -2 };
EDB200_API edb200_status_t edb200_flux_set_anchor_capture(edb200_flux_t* m, int anchor, float* dst);
EDB200_API edb200_status_t edb200_flux_set_stop_after(edb200_flux_t* m, int block);
EDB200_API edb200_status_t edb200_flux_set_stream_override(edb200_flux_t* m, const float* residual);
/* One denoise step on device-resident tensors, asynchronous on `stream`:
 * latent/out f32 [C, H, W]; context f32 [n_txt, context_in_dim]; y f32 [vec_in_dim];
 * timestep and guidance as the reference passes them (sigma in 0..1, guidance scale). */
EDB200_API edb200_status_t edb200_flux_step(edb200_flux_t* m, const float* latent, float timestep,
                                            const float* context, const float* y, float guidance, float* out,
                                            void* stream);
/* The same step with the timestep read on the device: timestep = sigmas[*step] (f32 device array,
 * int device word).  See edb200_euler_update_sched. */
EDB200_API edb200_status_t edb200_flux_step_sched(edb200_flux_t* m, const float* latent, const float* sigmas,
                                                  const int* step, const float* context, const float* y,
                                                  float guidance, float* out, void* stream);
/* The same step with host tensors in and out (the reference's compute seam):
 * prepares the shape if needed, copies through pinned staging, runs the step,
 * copies the result back and synchronises. */
EDB200_API edb200_status_t edb200_flux_compute_host(edb200_flux_t* m, const float* latent, int latent_h, int latent_w,
                                                    float timestep, const float* context, int n_txt, const float* y,
                                                    float guidance, float* out, void* stream);

/* Sequence-parallel execution of the step (FLUX forward_sp, src/dit_models/models/flux.hpp:4529-5156):
 * call before edb200_flux_prepare; NULL returns to single-GPU execution.  Every
 * rank passes the full inputs and receives the full output latent; num_heads must divide
 * by the communicator size, the token count need not (edb200_sp_shard pads it).  The
 * communicator is borrowed. */
EDB200_API edb200_status_t edb200_flux_set_comm(edb200_flux_t* m, edb200_comm_t* comm);

/* ------------------------------------------------ SD3-medium (MMDiT) denoise pass
 * The same seam for MMDiTModel / MMDiTRunner::compute (src/dit_models/models/mmdit.hpp:3403-3487;
 * members :3165-3182).  One call is one batch-1 pass; classifier-free guidance runs the
 * conditional and the unconditional pass and combines them with edb200_cfg_combine. */
typedef struct {
    int hidden_size;        /* 1536 = 64 * depth */
    int num_heads;          /* 24 (head dim 64) */
    int depth;              /* 24 joint blocks; the last one's context side is pre_only */
    int mlp_hidden;         /* 4 * hidden_size */
    int in_channels;        /* latent channels, 16 */
    int out_channels;       /* 16 */
    int patch_size;         /* 2 */
    int adm_in_channels;    /* pooled vector, 2048 */
    int context_size;       /* 4096 */
    int pos_embed_max_size; /* 192 */
    int wtype;              /* EDB200_TYPE_Q8_0 / EDB200_TYPE_Q4_K */
    int attention;          /* EDB200_ATTN_F16 / EDB200_ATTN_SAGE_INT8 (ED_SAGE_ATTN) */
    int sage_smooth_q;      /* ED_SAGE_SMOOTH_Q; the reference's default for head dim 64 is off
                               (src/core/backend/ggml/ed_ggml_sage_attn_ext.hpp:67-86) */
    int sage_skip_first;    /* ED_SAGE_SKIP_FIRST / ED_SAGE_SKIP_LAST: that many first / last joint blocks keep f16 */
    int sage_skip_last;     /* attention (reference default 2 and 2, ed_ggml_sage_attn_ext.hpp:146-159) */
} edb200_sd3_config_t;

typedef struct edb200_sd3 edb200_sd3_t;

EDB200_API edb200_status_t edb200_sd3_create(const edb200_sd3_config_t* cfg, edb200_sd3_t** out);
EDB200_API void edb200_sd3_destroy(edb200_sd3_t* m);
EDB200_API int edb200_sd3_tensor_count(const edb200_sd3_t* m);
EDB200_API edb200_status_t edb200_sd3_tensor_info(const edb200_sd3_t* m, int index, char* name, int name_cap,
                                                  int* ggml_type, int64_t* n_out, int64_t* k, int64_t* nbytes);
EDB200_API edb200_status_t edb200_sd3_set_tensor(edb200_sd3_t* m, const char* name, int ggml_type, const void* data,
                                                 int64_t nbytes, int on_device, void* stream);
/* Reads one tensor back as f32 [n_out, k] into host (on_device = 0) or device memory; a quantised weight
 * is dequantised from its repacked device form (the values ggml's dequantize_row gives for the blocks
 * that were loaded).  n_floats must equal n_out * k.  Synchronises the stream.  Lets a checker run on
 * exactly the weights the device holds, e.g. after edb200_sd3_init_random. */
EDB200_API edb200_status_t edb200_sd3_get_tensor_f32(const edb200_sd3_t* m, const char* name, float* out,
                                                      int64_t n_floats, int on_device, void* stream);
/* Loads every tensor of a GGUF file this model has a parameter for (names compared after removing
 * `strip_prefix`, e.g. "model.diffusion_model."; NULL = none); other tensors are skipped.  Quantised
 * weights must be stored in the model's block type; f16 / bf16 vectors are widened to f32.
 * *n_loaded (may be NULL) = tensors taken. */
EDB200_API edb200_status_t edb200_sd3_load_gguf(edb200_sd3_t* m, const char* path, const char* strip_prefix,
                                               int* n_loaded, void* stream);
/* The same from a safetensors file (F32 / F16 / BF16 tensors).  Parameters the model keeps quantised are
 * encoded on the device in its block type while they load: q8_0 by ggml's rule (bit for bit), q4_K by this
 * library's min/max encoder. */
EDB200_API edb200_status_t edb200_sd3_load_safetensors(edb200_sd3_t* m, const char* path, const char* strip_prefix,
                                                      int* n_loaded, void* stream);
EDB200_API edb200_status_t edb200_sd3_init_random(edb200_sd3_t* m, uint64_t seed, float std, void* stream);
EDB200_API int64_t edb200_sd3_weight_bytes(const edb200_sd3_t* m);
EDB200_API edb200_status_t edb200_sd3_prepare(edb200_sd3_t* m, int lat_h, int lat_w, int n_ctx, void* stream);
/* The computation-reuse seam of edb200_flux_set_anchor_capture / _set_stop_after / _set_stream_override for
 * this family (src/dit_models/models/mmdit.hpp:3318-3385): the anchors are views of the stream the blocks transform,
 * the image rows of this rank, [rows, hidden], f32 on the device. */
EDB200_API edb200_status_t edb200_sd3_set_anchor_capture(edb200_sd3_t* m, int anchor, float* dst);
EDB200_API edb200_status_t edb200_sd3_set_stop_after(edb200_sd3_t* m, int block);
EDB200_API edb200_status_t edb200_sd3_set_stream_override(edb200_sd3_t* m, const float* residual);
/* Region inject (src/dit_models/models/mmdit.hpp:3336-3343): at block `at` the stream becomes ModelIn + residual and the
 * blocks [at, resume) are skipped.  A region that starts after block 0 rebuilds the stream from the ModelIn
 * capture buffer, which must be set.  residual NULL or at < 0 switches it off. */
EDB200_API edb200_status_t edb200_sd3_set_region_inject(edb200_sd3_t* m, int at, int resume, const float* residual);
/* Optional f32 tap [depth, n_ctx + image tokens, hidden]: both streams after every block. */
EDB200_API edb200_status_t edb200_sd3_set_tap(edb200_sd3_t* m, float* tap);
/* Sequence parallel over `comm` (MMDiT forward_sp, src/dit_models/models/mmdit.hpp:3117-3128, 3439-3466):
 * before prepare; NULL returns to single-GPU execution. */
EDB200_API edb200_status_t edb200_sd3_set_comm(edb200_sd3_t* m, edb200_comm_t* comm);
/* latent f32 [in_channels, lat_h, lat_w], context f32 [n_ctx, context_size], y f32 [adm_in_channels]. */
EDB200_API edb200_status_t edb200_sd3_step(edb200_sd3_t* m, const float* latent, float timestep, const float* context,
                                           const float* y, float* out, void* stream);
/* The same pass with the timestep read on the device: timestep = sigmas[*step] * t_scale (the pipelines pass
 * sigma * 1000).  With edb200_flow_update_sched and edb200_cfg_combine, one recorded (conditional pass,
 * unconditional pass, combine, update) replays for every step of a schedule. */
EDB200_API edb200_status_t edb200_sd3_step_sched(edb200_sd3_t* m, const float* latent, const float* sigmas, const int* step,
                                                 float t_scale, const float* context, const float* y, float* out,
                                                 void* stream);
EDB200_API edb200_status_t edb200_sd3_compute_host(edb200_sd3_t* m, const float* latent, int lat_h, int lat_w,
                                                   float timestep, const float* context, int n_ctx, const float* y,
                                                   float* out, void* stream);
/* out = uncond + scale * (cond - uncond), f32, n a multiple of 4: the pipeline-side CFG combine
 * (src/dit_models/pipelines/sd3_pipeline.cpp:631-669, src/dit_models/pipelines/flux_pipeline.cpp:1218-1258). */
EDB200_API edb200_status_t edb200_cfg_combine(const float* uncond, const float* cond, float scale, float* out, int64_t n,
                                              void* stream);
/* Qwen-Image's guidance combine (ed_qwen_apply_true_cfg, src/dit_models/pipelines/qwen_image_pipeline.cpp:29-85):
 * out = guided * (||cond|| / ||guided||) with guided = uncond + scale * (cond - uncond) and the two norms taken
 * per patch_size x patch_size latent patch over all channels (sums of squares in double, order dy, dx, channel);
 * 0 where ||guided|| is 0.  Tensors f32 [channels, height, width].  Bit-identical to the reference. */
EDB200_API edb200_status_t edb200_cfg_combine_rescaled(const float* uncond, const float* cond, float scale, int patch_size,
                                            int channels, int height, int width, float* out, void* stream);

/* ---------------------------------------------------- Qwen-Image denoise pass
 * The same seam for QwenImageModel (src/dit_models/models/qwen_image.hpp:3116-3301; members
 * QwenImageParams :3074-3114).  One call is one batch-1 pass (CFG = two passes + combine). */
typedef struct {
    int num_layers;           /* 60 */
    int num_heads;            /* 24 */
    int head_dim;             /* 128 */
    int mlp_hidden;           /* 12288 */
    int in_channels;          /* 64 = 16 latent channels x 2 x 2 patch */
    int out_channels;         /* 16 */
    int joint_attention_dim;  /* 3584 */
    int patch_size;           /* 2 */
    int axes_dim[3];          /* (16, 56, 56) */
    int theta;
    int wtype;                /* EDB200_TYPE_Q8_0 / EDB200_TYPE_Q4_K for every 2-D weight with row length % 256 == 0
                                 except img_in / txt_in (kept f32, src/core/runtime/model_loader.cpp:2152-2155);
                                 img_mod.1 / txt_mod.1 are at least q8_0 (:1746-1761) */
    int attention;            /* EDB200_ATTN_F16 / EDB200_ATTN_SAGE_INT8 */
    int sage_smooth_q;
} edb200_qwen_config_t;

typedef struct edb200_qwen edb200_qwen_t;

EDB200_API edb200_status_t edb200_qwen_create(const edb200_qwen_config_t* cfg, edb200_qwen_t** out);
EDB200_API void edb200_qwen_destroy(edb200_qwen_t* m);
EDB200_API int edb200_qwen_tensor_count(const edb200_qwen_t* m);
EDB200_API edb200_status_t edb200_qwen_tensor_info(const edb200_qwen_t* m, int index, char* name, int name_cap,
                                                   int* ggml_type, int64_t* n_out, int64_t* k, int64_t* nbytes);
EDB200_API edb200_status_t edb200_qwen_set_tensor(edb200_qwen_t* m, const char* name, int ggml_type, const void* data,
                                                  int64_t nbytes, int on_device, void* stream);
/* Reads one tensor back as f32 [n_out, k] into host (on_device = 0) or device memory; a quantised weight
 * is dequantised from its repacked device form (the values ggml's dequantize_row gives for the blocks
 * that were loaded).  n_floats must equal n_out * k.  Synchronises the stream.  Lets a checker run on
 * exactly the weights the device holds, e.g. after edb200_qwen_init_random. */
EDB200_API edb200_status_t edb200_qwen_get_tensor_f32(const edb200_qwen_t* m, const char* name, float* out,
                                                      int64_t n_floats, int on_device, void* stream);
/* Loads every tensor of a GGUF file this model has a parameter for (names compared after removing
 * `strip_prefix`, e.g. "model.diffusion_model."; NULL = none); other tensors are skipped.  Quantised
 * weights must be stored in the model's block type; f16 / bf16 vectors are widened to f32.
 * *n_loaded (may be NULL) = tensors taken. */
EDB200_API edb200_status_t edb200_qwen_load_gguf(edb200_qwen_t* m, const char* path, const char* strip_prefix,
                                               int* n_loaded, void* stream);
/* The same from a safetensors file (F32 / F16 / BF16 tensors).  Parameters the model keeps quantised are
 * encoded on the device in its block type while they load: q8_0 by ggml's rule (bit for bit), q4_K by this
 * library's min/max encoder. */
EDB200_API edb200_status_t edb200_qwen_load_safetensors(edb200_qwen_t* m, const char* path, const char* strip_prefix,
                                                      int* n_loaded, void* stream);
EDB200_API edb200_status_t edb200_qwen_init_random(edb200_qwen_t* m, uint64_t seed, float std, void* stream);
EDB200_API int64_t edb200_qwen_weight_bytes(const edb200_qwen_t* m);
EDB200_API edb200_status_t edb200_qwen_prepare(edb200_qwen_t* m, int lat_h, int lat_w, int n_txt, void* stream);
/* The computation-reuse seam of edb200_flux_set_anchor_capture / _set_stop_after / _set_stream_override for
 * this family (src/dit_models/models/qwen_image.hpp:3209-3274): the anchors are views of the stream the blocks transform,
 * the image rows of this rank, [rows, hidden], f32 on the device. */
EDB200_API edb200_status_t edb200_qwen_set_anchor_capture(edb200_qwen_t* m, int anchor, float* dst);
EDB200_API edb200_status_t edb200_qwen_set_stop_after(edb200_qwen_t* m, int block);
EDB200_API edb200_status_t edb200_qwen_set_stream_override(edb200_qwen_t* m, const float* residual);
/* Optional f32 tap [num_layers, n_txt + image tokens, hidden]: both streams after every block. */
EDB200_API edb200_status_t edb200_qwen_set_tap(edb200_qwen_t* m, float* tap);
/* Sequence parallel over `comm` (QwenImageTransformerBlock::forward_sp, qwen_image.hpp:2969-3040): before prepare. */
EDB200_API edb200_status_t edb200_qwen_set_comm(edb200_qwen_t* m, edb200_comm_t* comm);
/* latent f32 [in_channels / patch^2, lat_h, lat_w], context f32 [n_txt, joint_attention_dim]. */
EDB200_API edb200_status_t edb200_qwen_step(edb200_qwen_t* m, const float* latent, float timestep, const float* context,
                                            float* out, void* stream);
/* The same pass with the timestep read on the device: timestep = sigmas[*step] * t_scale. */
EDB200_API edb200_status_t edb200_qwen_step_sched(edb200_qwen_t* m, const float* latent, const float* sigmas,
                                                  const int* step, float t_scale, const float* context, float* out,
                                                  void* stream);
EDB200_API edb200_status_t edb200_qwen_compute_host(edb200_qwen_t* m, const float* latent, int lat_h, int lat_w,
                                                    float timestep, const float* context, int n_txt, float* out,
                                                    void* stream);

/* -------------------------------------------------- Wan 2.1 (t2v) denoise step
 * The same seam for WanModel / WanRunner::compute (src/dit_models/models/wan.hpp:4811-5529,
 * graph Wan::forward :4759-4808).  Field names follow WanParams (:4382-4405). */
typedef struct {
    int dim;            /* 5120 */
    int num_heads;      /* 40 (head dim 128) */
    int ffn_dim;        /* 13824 */
    int num_layers;     /* 40 */
    int in_dim;         /* latent channels, 16 */
    int out_dim;        /* 16 */
    int text_dim;       /* 4096 */
    int freq_dim;       /* 256 */
    int patch_size[3];  /* (1, 2, 2) */
    int axes_dim[3];    /* (44, 42, 42) over (t, h, w) */
    int theta;
    int wtype;          /* EDB200_TYPE_Q8_0 / EDB200_TYPE_Q4_K for the block linears */
    int attention;      /* self-attention: EDB200_ATTN_F16 / EDB200_ATTN_SAGE_INT8; cross-attention is always f16 */
    int sage_smooth_q;
    int sage_skip_first;  /* ED_SAGE_SKIP_FIRST / ED_SAGE_SKIP_LAST: that many first / last layers keep f16 */
    int sage_skip_last;   /* self-attention (reference default 2 and 2, ed_ggml_sage_attn_ext.hpp:146-159) */
} edb200_wan_config_t;

typedef struct edb200_wan edb200_wan_t;

EDB200_API edb200_status_t edb200_wan_create(const edb200_wan_config_t* cfg, edb200_wan_t** out);
EDB200_API void edb200_wan_destroy(edb200_wan_t* m);
EDB200_API int edb200_wan_tensor_count(const edb200_wan_t* m);
EDB200_API edb200_status_t edb200_wan_tensor_info(const edb200_wan_t* m, int index, char* name, int name_cap,
                                                  int* ggml_type, int64_t* n_out, int64_t* k, int64_t* nbytes);
EDB200_API edb200_status_t edb200_wan_set_tensor(edb200_wan_t* m, const char* name, int ggml_type, const void* data,
                                                 int64_t nbytes, int on_device, void* stream);
/* Reads one tensor back as f32 [n_out, k] into host (on_device = 0) or device memory; a quantised weight
 * is dequantised from its repacked device form (the values ggml's dequantize_row gives for the blocks
 * that were loaded).  n_floats must equal n_out * k.  Synchronises the stream.  Lets a checker run on
 * exactly the weights the device holds, e.g. after edb200_wan_init_random. */
EDB200_API edb200_status_t edb200_wan_get_tensor_f32(const edb200_wan_t* m, const char* name, float* out,
                                                      int64_t n_floats, int on_device, void* stream);
/* Loads every tensor of a GGUF file this model has a parameter for (names compared after removing
 * `strip_prefix`, e.g. "model.diffusion_model."; NULL = none); other tensors are skipped.  Quantised
 * weights must be stored in the model's block type; f16 / bf16 vectors are widened to f32.
 * *n_loaded (may be NULL) = tensors taken. */
EDB200_API edb200_status_t edb200_wan_load_gguf(edb200_wan_t* m, const char* path, const char* strip_prefix,
                                               int* n_loaded, void* stream);
/* The same from a safetensors file (F32 / F16 / BF16 tensors).  Parameters the model keeps quantised are
 * encoded on the device in its block type while they load: q8_0 by ggml's rule (bit for bit), q4_K by this
 * library's min/max encoder. */
EDB200_API edb200_status_t edb200_wan_load_safetensors(edb200_wan_t* m, const char* path, const char* strip_prefix,
                                                      int* n_loaded, void* stream);
EDB200_API edb200_status_t edb200_wan_init_random(edb200_wan_t* m, uint64_t seed, float std, void* stream);
EDB200_API int64_t edb200_wan_weight_bytes(const edb200_wan_t* m);
EDB200_API int64_t edb200_wan_workspace_bytes(const edb200_wan_t* m);
/* Latent [in_dim, frames, lat_h, lat_w] (frames, lat_h, lat_w multiples of the patch), n_ctx text tokens. */
EDB200_API edb200_status_t edb200_wan_prepare(edb200_wan_t* m, int frames, int lat_h, int lat_w, int n_ctx,
                                              void* stream);
/* The computation-reuse seam of edb200_flux_set_anchor_capture / _set_stop_after / _set_stream_override for
 * this family (src/dit_models/models/wan.hpp:4640-4729): the anchors are views of the stream the blocks transform,
 * the video-token rows of this rank, [rows, dim], f32 on the device. */
EDB200_API edb200_status_t edb200_wan_set_anchor_capture(edb200_wan_t* m, int anchor, float* dst);
EDB200_API edb200_status_t edb200_wan_set_stop_after(edb200_wan_t* m, int block);
EDB200_API edb200_status_t edb200_wan_set_stream_override(edb200_wan_t* m, const float* residual);
/* Region inject (src/dit_models/models/wan.hpp:4658-4665): at block `at` the stream becomes ModelIn + residual and the
 * blocks [at, resume) are skipped.  A region that starts after block 0 rebuilds the stream from the ModelIn
 * capture buffer, which must be set.  residual NULL or at < 0 switches it off. */
EDB200_API edb200_status_t edb200_wan_set_region_inject(edb200_wan_t* m, int at, int resume, const float* residual);
/* Optional f32 tap [num_layers, tokens (this rank's), dim]: residual stream after every block. */
EDB200_API edb200_status_t edb200_wan_set_tap(edb200_wan_t* m, float* tap);
/* Sequence parallel over `comm` (WanAttentionBlock::forward_sp, wan.hpp:4189-4235): before prepare. */
EDB200_API edb200_status_t edb200_wan_set_comm(edb200_wan_t* m, edb200_comm_t* comm);
/* One denoise step on device tensors: latent f32 [in_dim, frames, lat_h, lat_w], context f32
 * [n_ctx, text_dim], out f32 like latent. */
EDB200_API edb200_status_t edb200_wan_step(edb200_wan_t* m, const float* latent, float timestep, const float* context,
                                           float* out, void* stream);
/* The same step with the timestep read on the device: timestep = sigmas[*step] * t_scale. */
EDB200_API edb200_status_t edb200_wan_step_sched(edb200_wan_t* m, const float* latent, const float* sigmas, const int* step,
                                                 float t_scale, const float* context, float* out, void* stream);
/* The same with host tensors (DiffusionModel::compute seam); synchronises. */
EDB200_API edb200_status_t edb200_wan_compute_host(edb200_wan_t* m, const float* latent, int frames, int lat_h,
                                                   int lat_w, float timestep, const float* context, int n_ctx,
                                                   float* out, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* EDB200_OPS_H */
