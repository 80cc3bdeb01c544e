// Evaluates the pipelines' per-step latent arithmetic with the reference's own tensor class
// (src/utils/tensor.hpp, compiled from the reference tree): the expressions below are written
// as they stand in the pipelines, so the element type, the scalar conversions and the order of
// the roundings are the reference's.  Test infrastructure: pins the numpy oracle
// (O.euler_update, O.flow_update, O.cfg_combine) and feeds tests/golden/; never part of the
// product path.
//   FLUX / Qwen-Image update  src/dit_models/pipelines/flux_pipeline.cpp:1111-1112, :1290-1297
//   SD3 update                src/dit_models/pipelines/sd3_pipeline.cpp:697
//   guidance combine          src/dit_models/pipelines/flux_pipeline.cpp:1258
#include "utils/tensor.hpp"

#include <cstdint>
#include <cstring>
#include <vector>

namespace {

sd::Tensor<float> wrap(const float* p, int64_t n) {
    return sd::Tensor<float>({n}, std::vector<float>(p, p + n));
}

void unwrap(const sd::Tensor<float>& t, float* p) {
    for (int64_t i = 0; i < t.numel(); ++i) p[i] = t[i];
}

}  // namespace

extern "C" {

void ref_tensor_euler_update(float* x_io, const float* model_out_p, int64_t n, float sigma, float sigma_next) {
    sd::Tensor<float> x = wrap(x_io, n);
    const sd::Tensor<float> model_out = wrap(model_out_p, n);
    const float c_skip = 1.0f;
    const float c_out = -sigma;
    sd::Tensor<float> denoised = model_out * c_out + x * c_skip;
    if (sigma == 0.0f) {
        x = denoised;
    } else {
        const sd::Tensor<float> d = (x - denoised) / sigma;
        x += d * (sigma_next - sigma);
    }
    unwrap(x, x_io);
}

void ref_tensor_flow_update(float* x_io, const float* model_out_p, int64_t n, float sigma, float sigma_next) {
    sd::Tensor<float> x = wrap(x_io, n);
    const sd::Tensor<float> model_out = wrap(model_out_p, n);
    x += model_out * (sigma_next - sigma);
    unwrap(x, x_io);
}

void ref_tensor_cfg_combine(const float* uncond_p, const float* cond_p, int64_t n, float cfg_scale, float* out) {
    const sd::Tensor<float> uncond_out = wrap(uncond_p, n);
    sd::Tensor<float> model_out = wrap(cond_p, n);
    model_out = uncond_out + cfg_scale * (model_out - uncond_out);
    unwrap(model_out, out);
}

}  // extern "C"
