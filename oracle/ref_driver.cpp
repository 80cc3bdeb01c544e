// Calls the reference's own CPU callbacks (compiled from the reference tree against
// ref_shim/ggml.h) on plain arrays.  Test infrastructure: used to pin the numpy oracle
// and to generate the golden vectors under tests/golden/; never part of the product path.
//   modulate / residual gate  src/core/backend/ggml/ed_ggml_modulation_ext.hpp:168-228
//   rms_norm_mul_f16          src/core/backend/ggml/ed_ggml_norm_ext.hpp:223-263
//   rope                      src/core/backend/ggml/ed_ggml_rope_ext.hpp:105-184
#include "ed_ggml_modulation_ext.hpp"
#include "ed_ggml_norm_ext.hpp"
#include "ed_ggml_rope_ext.hpp"

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

}  // extern "C"
