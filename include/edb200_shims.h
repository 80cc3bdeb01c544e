/*
 * edb200_shims.h -- the reference's operator plugin ABI, implemented on this library's kernels.
 *
 * The reference dispatches each of its custom graph operators to a pair of functions
 *   bool ed_cuda_<op>_custom_supported(const ggml_tensor* dst);
 *   bool ed_cuda_<op>_custom_compute(ggml_tensor* dst, void* stream);
 * (headers src/core/backend/ggml/cuda/ed_cuda_{modulation,norm,rope,attention_v_prep,sage_attn}.h):
 * inputs are dst->src[i], the operator's parameters travel in dst->op_params as
 * {function pointer, n_tasks, userdata} with a 32-bit magic and small integers packed into
 * `userdata` (src/core/backend/ggml/ed_ggml_*_ext.hpp), `false` means "not mine / unsupported"
 * and the caller falls back, work is enqueued on the given CUDA stream without a host sync.
 * The functions below keep those names, signatures and semantics, so a build of the reference can
 * link its dispatcher against libedb200.so in place of its own cuda/ed_cuda_*.cu objects.  Results
 * are the reference CPU callbacks' to the bit (every one of these operators is elementwise or a
 * copy / cast, evaluated with the same operations in the same order).
 *
 * The tensors are described by ggml's own structure: see edb200_ggml.h for how it is provided.
 */
#ifndef EDB200_SHIMS_H
#define EDB200_SHIMS_H

#include <stddef.h>

#include "edb200_ggml.h"
#include "edb200_ops.h"

#ifdef __cplusplus

/* y = (x + x*scale) + shift | y = residual + x*gate | y = mod_0 + index*(mod_1 - mod_0), f32, operands
 * broadcast per dimension; which of the three is told by the magic in the op parameters
 * (cuda/ed_cuda_modulation.h:7-9, ed_ggml_modulation_ext.hpp:168-253). */
EDB200_API bool ed_cuda_fused_modulate_custom_supported(const ggml_tensor* dst);
EDB200_API bool ed_cuda_fused_modulate_custom_compute(ggml_tensor* dst, void* stream);

/* y = f16(x * rsqrt(mean(x^2) + eps) * w) over rows of ne[0] (cuda/ed_cuda_norm.h:33-35,
 * ed_ggml_norm_ext.hpp:223-263); eps travels in the op parameters. */
EDB200_API bool ed_cuda_rms_norm_mul_f16_custom_supported(const ggml_tensor* dst);
EDB200_API bool ed_cuda_rms_norm_mul_f16_custom_compute(ggml_tensor* dst, void* stream);

/* Rotary embedding with the stored 2x2 table, three input layouts, interleaved or split pairs, f32 or
 * bf16 in, f32 / f16 / bf16 out [d_head, seq, heads] (cuda/ed_cuda_rope.h:7-9, ed_ggml_rope_ext.hpp:105-184). */
EDB200_API bool ed_cuda_rope_custom_supported(const ggml_tensor* dst);
EDB200_API bool ed_cuda_rope_custom_compute(ggml_tensor* dst, void* stream);

/* Layout glue in front of attention, f32 in, f16 out (cuda/ed_cuda_attention_v_prep.h:7-21,
 * ed_ggml_attention_ext.hpp:269-369): V to [d_head, seq, heads * batch]; two streams' rows
 * concatenated head-major; the same for q, k and v of two streams at once. */
EDB200_API bool ed_cuda_attention_v_prep_custom_supported(const ggml_tensor* dst);
EDB200_API bool ed_cuda_attention_v_prep_custom_compute(ggml_tensor* dst, void* stream);
EDB200_API bool ed_cuda_attention_pair_pack_custom_supported(const ggml_tensor* dst);
EDB200_API bool ed_cuda_attention_pair_pack_custom_compute(ggml_tensor* dst, void* stream);
EDB200_API bool ed_cuda_attention_qkv_pair_pack_custom_supported(const ggml_tensor* dst);
EDB200_API bool ed_cuda_attention_qkv_pair_pack_custom_compute(ggml_tensor* dst, void* stream);

/* INT8-QK attention with caller-provided scratch (cuda/ed_cuda_sage_attn.h:13-71): the caller asks for
 * the sizes, allocates the buffers from its pool and passes them back.  q, k [d_head, L, heads * N] f16,
 * v [d_head, heads, L, N] or [d_head, L, heads] f16 or f32, dst f32 [d_head, heads * N, L].  f32 q / k
 * are reported unsupported (the caller falls back): this library quantises from f16 operands.  Fields of
 * the scratch description this implementation does not need are given size 0; o_half holds the chunk
 * sums of the channel means. */
struct ed_cuda_sage_attn_scratch {
    void* q_int8 = nullptr;
    void* k_int8 = nullptr;
    void* q_scale = nullptr;
    void* k_scale = nullptr;
    void* km = nullptr;
    void* v_f16 = nullptr;
    void* o_half = nullptr;
    void* qm = nullptr;
    void* qk_bias = nullptr;
    void* v_fp8 = nullptr;
    void* v_scale = nullptr;
    void* uniform_flag = nullptr;
    void* head_entropy = nullptr;
    void* detect_acc = nullptr;
};
struct ed_cuda_sage_attn_scratch_sizes {
    size_t q_int8_bytes = 0;
    size_t k_int8_bytes = 0;
    size_t q_scale_bytes = 0;
    size_t k_scale_bytes = 0;
    size_t km_bytes = 0;
    size_t v_f16_bytes = 0;
    size_t o_half_bytes = 0;
    size_t qm_bytes = 0;
    size_t qk_bias_bytes = 0;
    size_t v_fp8_bytes = 0;
    size_t v_scale_bytes = 0;
    size_t uniform_flag_bytes = 0;
    size_t head_entropy_bytes = 0;
    size_t detect_acc_bytes = 0;
};
EDB200_API bool ed_cuda_sage_attn_custom_supported(const ggml_tensor* dst);
EDB200_API bool ed_cuda_sage_attn_scratch_sizes_for(const ggml_tensor* dst, ed_cuda_sage_attn_scratch_sizes* out);
EDB200_API bool ed_cuda_sage_attn_custom_compute(ggml_tensor* dst, const ed_cuda_sage_attn_scratch* scratch, void* stream);

#endif /* __cplusplus */

/* Plain-C doors to the same entry points for callers without a C++ toolchain (ctypes tests):
 * `which` selects the operator, the tensor is passed as a pointer. */
#ifdef __cplusplus
extern "C" {
#endif
enum {
    EDB200_PLUGIN_MODULATE = 0,       /* modulate / residual gate / where-select */
    EDB200_PLUGIN_RMS_NORM_MUL_F16 = 1,
    EDB200_PLUGIN_ROPE = 2,
    EDB200_PLUGIN_V_PREP = 3,
    EDB200_PLUGIN_PAIR_PACK = 4,
    EDB200_PLUGIN_QKV_PAIR_PACK = 5,
    EDB200_PLUGIN_SAGE_ATTN = 6
};
EDB200_API int edb200_plugin_supported(int which, const struct ggml_tensor* dst);
/* For EDB200_PLUGIN_SAGE_ATTN `scratch` is an ed_cuda_sage_attn_scratch*, otherwise NULL. */
EDB200_API int edb200_plugin_compute(int which, struct ggml_tensor* dst, const void* scratch, void* stream);
/* sizes[14] in the order of ed_cuda_sage_attn_scratch_sizes. */
EDB200_API int edb200_plugin_sage_scratch_sizes(const struct ggml_tensor* dst, size_t* sizes);
/* sizeof(struct ggml_tensor) and the offsets of type, ne, nb, op, op_params, src, data as this library was
 * built, so that a caller can check its own view of the structure. */
EDB200_API void edb200_plugin_tensor_layout(size_t* out8);
#ifdef __cplusplus
}
#endif

#endif /* EDB200_SHIMS_H */
