// Calls the reference's own CPU callbacks (compiled from the reference tree against
// ref_shim/ggml.h) on plain arrays.  Test infrastructure: used to pin the numpy oracle
// and to generate the golden vectors under tests/golden/; never part of the product path.
//   modulate / residual gate  src/core/backend/ggml/ed_ggml_modulation_ext.hpp:168-228
//   rms_norm_mul_f16          src/core/backend/ggml/ed_ggml_norm_ext.hpp:223-263
//   rope                      src/core/backend/ggml/ed_ggml_rope_ext.hpp:105-184
//   attention layout glue     src/core/backend/ggml/ed_ggml_attention_ext.hpp:269-369
//   GELU (bf16 out), concat-linear (+ gated residual)  src/core/backend/ggml/ed_ggml_sp_flux_ext.hpp:675-804
#include "ed_ggml_attention_ext.hpp"
#include "ed_ggml_modulation_ext.hpp"
#include "ed_ggml_norm_ext.hpp"
#include "ed_ggml_rope_ext.hpp"
#include "ed_ggml_sp_flux_ext.hpp"

namespace {

ggml_tensor make(ggml_type type, void* data, int64_t n0, int64_t n1 = 1, int64_t n2 = 1, int64_t n3 = 1) {
    ggml_tensor t;
    std::memset(&t, 0, sizeof(t));
    t.type = type;
    t.ne[0] = n0, t.ne[1] = n1, t.ne[2] = n2, t.ne[3] = n3;
    t.nb[0] = ggml_type_size(type);
    for (int i = 1; i < GGML_MAX_DIMS; ++i) t.nb[i] = t.nb[i - 1] * (size_t)t.ne[i - 1];
    t.data = data;
    return t;
}

}  // namespace

using namespace edgedit::ggml_ext;

extern "C" {

// x [rows, h] f32; shift, scale [h]; out = (x + x*scale) + shift
void ref_fused_modulate(const float* x, const float* shift, const float* scale, float* out, int64_t rows, int64_t h) {
    ggml_tensor tx = make(GGML_TYPE_F32, const_cast<float*>(x), h, rows);
    ggml_tensor ts = make(GGML_TYPE_F32, const_cast<float*>(shift), h);
    ggml_tensor tc = make(GGML_TYPE_F32, const_cast<float*>(scale), h);
    ggml_tensor dst = make(GGML_TYPE_F32, out, h, rows);
    dst.src[0] = &tx, dst.src[1] = &ts, dst.src[2] = &tc;
    fused_modulate_cpu_custom_op(&dst, 0, 1, fused_modulate_params_to_userdata());
}

// out = residual + x*gate
void ref_fused_residual_gate(const float* residual, const float* x, const float* gate, float* out, int64_t rows,
                             int64_t h) {
    ggml_tensor tr = make(GGML_TYPE_F32, const_cast<float*>(residual), h, rows);
    ggml_tensor tx = make(GGML_TYPE_F32, const_cast<float*>(x), h, rows);
    ggml_tensor tg = make(GGML_TYPE_F32, const_cast<float*>(gate), h);
    ggml_tensor dst = make(GGML_TYPE_F32, out, h, rows);
    dst.src[0] = &tr, dst.src[1] = &tx, dst.src[2] = &tg;
    fused_residual_gate_cpu_custom_op(&dst, 0, 1, fused_residual_gate_params_to_userdata());
}

// x [rows, d] f32, w [d] -> out [rows, d] f16 bits
void ref_rms_norm_mul_f16(const float* x, const float* w, uint16_t* out, int64_t rows, int64_t d, float eps) {
    ggml_tensor tx = make(GGML_TYPE_F32, const_cast<float*>(x), d, rows);
    ggml_tensor tw = make(GGML_TYPE_F32, const_cast<float*>(w), d);
    ggml_tensor dst = make(GGML_TYPE_F16, out, d, rows);
    dst.src[0] = &tx, dst.src[1] = &tw;
    rms_norm_mul_f16_cpu_custom_op(&dst, 0, 1, rms_norm_mul_f16_params_to_userdata(eps));
}

// x [seq, heads, d] f32 (ggml ne = [d, heads, seq, 1]), pe [seq, d/2, 2, 2] (ggml ne = [2, 2, d/2, seq]),
// interleaved pairs -> out [heads, seq, d] f32 (ggml ne = [d, seq, heads, 1])
void ref_rope_interleaved(const float* x, const float* pe, float* out, int64_t seq, int64_t heads, int64_t d) {
    ggml_tensor tx = make(GGML_TYPE_F32, const_cast<float*>(x), d, heads, seq, 1);
    ggml_tensor tp = make(GGML_TYPE_F32, const_cast<float*>(pe), 2, 2, d / 2, seq);
    ggml_tensor dst = make(GGML_TYPE_F32, out, d, seq, heads, 1);
    dst.src[0] = &tx, dst.src[1] = &tp;
    rope_cpu_custom_op(&dst, 0, 1, rope_params_to_userdata(RopeInputLayout::NSeqHeadDim, true, d));
}

// Runs the reference CPU callback that a custom-op node describes: `dst` is a ggml_tensor (the structure of
// include/edb200_ggml.h) in host memory whose op_params hold {callback, n_tasks, userdata} and whose src[]
// point at host tensors.  The callback is chosen by the magic in userdata, as the reference's dispatch does.
// Returns 0 when the magic is not one of the operators below.
int ref_custom_op(ggml_tensor* dst) {
    struct Params {
        ggml_custom_op_t fun;
        int n_tasks;
        void* userdata;
    } p;
    std::memcpy(&p, dst->op_params, sizeof(p));
    const uint32_t magic = static_cast<uint32_t>(reinterpret_cast<uintptr_t>(p.userdata) & 0xffffffffu);
    switch (magic) {
        case kFusedModulateCustomMagic: fused_modulate_cpu_custom_op(dst, 0, 1, p.userdata); return 1;
        case kFusedResidualGateCustomMagic: fused_residual_gate_cpu_custom_op(dst, 0, 1, p.userdata); return 1;
        case kFusedWhereSelectCustomMagic: fused_where_select_cpu_custom_op(dst, 0, 1, p.userdata); return 1;
        case kRmsNormMulF16CustomMagic: rms_norm_mul_f16_cpu_custom_op(dst, 0, 1, p.userdata); return 1;
        case kRopeCustomMagic: rope_cpu_custom_op(dst, 0, 1, p.userdata); return 1;
        case kAttentionVPrepCustomMagic: attention_v_prep_cpu_custom_op(dst, 0, 1, p.userdata); return 1;
        case kAttentionPairPackCustomMagic: attention_pair_pack_cpu_custom_op(dst, 0, 1, p.userdata); return 1;
        case kAttentionQKVPairPackCustomMagic: attention_qkv_pair_pack_cpu_custom_op(dst, 0, 1, p.userdata); return 1;
        case kFluxSPGeluBF16CustomMagic: flux_sp_gelu_bf16_cpu_custom_op(dst, 0, 1, p.userdata); return 1;
        case kFluxSPConcatLinearCustomMagic: flux_sp_concat_linear_cpu_custom_op(dst, 0, 1, p.userdata); return 1;
        case kFluxSPConcatLinearResidualGateCustomMagic:
            flux_sp_concat_linear_residual_gate_cpu_custom_op(dst, 0, 1, p.userdata);
            return 1;
        default: return 0;
    }
}

// The userdata words the reference's graph builders attach to these operators.
uint64_t ref_userdata(int which, int64_t a, int64_t b, int64_t c, float f) {
    void* u = nullptr;
    switch (which) {
        case 0: u = fused_modulate_params_to_userdata(); break;
        case 1: u = fused_residual_gate_params_to_userdata(); break;
        case 2: u = fused_where_select_params_to_userdata(); break;
        case 3: u = rms_norm_mul_f16_params_to_userdata(f); break;
        case 4: u = rope_params_to_userdata(static_cast<RopeInputLayout>(a), b != 0, c); break;
        case 5: u = attention_v_prep_params_to_userdata(a != 0); break;
        case 6: u = attention_pair_pack_params_to_userdata(a); break;
        case 7: u = attention_qkv_pair_pack_params_to_userdata(a); break;
        case 8: u = flux_sp_gelu_bf16_params_to_userdata(); break;
        case 9: u = flux_sp_concat_linear_params_to_userdata(); break;
        case 10: u = flux_sp_concat_linear_residual_gate_params_to_userdata(); break;
        default: break;
    }
    return static_cast<uint64_t>(reinterpret_cast<uintptr_t>(u));
}

}  // extern "C"
