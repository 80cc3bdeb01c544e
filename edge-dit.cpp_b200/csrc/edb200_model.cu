// Parameter table, activation workspace and the small layout kernels shared by
// the denoise-step executors.
#include "edb200_model.h"

#include <cuda_fp16.h>
#include <cstring>

namespace edb {

int64_t ggml_row_bytes(int ggml_type, int64_t k) {
    switch (ggml_type) {
        case EDB200_TYPE_F32: return k * 4;
        case EDB200_TYPE_F16:
        case EDB200_TYPE_BF16: return k * 2;
        case EDB200_TYPE_Q8_0: return k / 32 * 34;
        case EDB200_TYPE_Q4_K: return k / 256 * 144;
        default: return -1;
    }
}

// ------------------------------------------------------------------ kernels --

// latent [C, H, W] -> tokens [(H/p)*(W/p), C*p*p], feature = c*p*p + py*p + px
// (DiT::patchify with patch_last = true, reference
// src/dit_models/components/common/common_dit.hpp:7-36).
__global__ void patchify_kernel(const float* __restrict__ x, float* __restrict__ t, int C, int H, int W, int p) {
    const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int64_t total = (int64_t)C * H * W;
    if (idx >= total) return;
    const int F = C * p * p;
    const int f = static_cast<int>(idx % F);
    const int64_t tok = idx / F;
    const int w_tok = W / p;
    const int ty = static_cast<int>(tok / w_tok), tx = static_cast<int>(tok % w_tok);
    const int c = f / (p * p), py = (f / p) % p, px = f % p;
    t[idx] = x[((int64_t)c * H + ty * p + py) * W + tx * p + px];
}

// inverse (DiT::unpatchify, common_dit.hpp:38-64)
__global__ void unpatchify_kernel(const float* __restrict__ t, float* __restrict__ x, int C, int H, int W, int p) {
    const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int64_t total = (int64_t)C * H * W;
    if (idx >= total) return;
    const int px_full = static_cast<int>(idx % W);
    const int py_full = static_cast<int>((idx / W) % H);
    const int c = static_cast<int>(idx / ((int64_t)W * H));
    const int w_tok = W / p;
    const int64_t tok = (int64_t)(py_full / p) * w_tok + px_full / p;
    const int f = c * p * p + (py_full % p) * p + (px_full % p);
    x[idx] = t[tok * (C * p * p) + f];
}

// `sched` != NULL: the timestep is sched[*step], read on the device (a recorded step then follows a
// schedule without being re-recorded).
__global__ void timestep_embedding_kernel(const float* __restrict__ freq, float t, const float* __restrict__ sched,
                                          const int* __restrict__ step, float pre_scale, float scale, int half,
                                          float* __restrict__ out) {
    const int j = blockIdx.x * blockDim.x + threadIdx.x;
    if (j >= half) return;
    if (sched != nullptr) t = __fmul_rn(sched[*step], pre_scale);   // the f32 product a host caller would pass
    const float arg = __fmul_rn(__fmul_rn(t, freq[j]), scale);
    out[j] = cosf(arg);
    out[half + j] = sinf(arg);
}

__global__ void add_inplace_kernel(float* __restrict__ dst, const float* __restrict__ src, int64_t n) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) dst[i] += src[i];
}

__global__ void add_one_kernel(float* __restrict__ dst, int64_t n) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) dst[i] += 1.0f;
}

// One thread per 256-weight super-block; the same min/max encoder as the CPU
// oracle's q4_k_quantize, operation for operation in f32.
__global__ void quant_q4_k_kernel(const float* __restrict__ x, uint8_t* __restrict__ blocks, int64_t n_blocks) {
    const int64_t b = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= n_blocks) return;
    const float* xb = x + b * 256;
    float mins[8], scale[8];
    float smax = 0.0f, mmax = 0.0f;
    for (int j = 0; j < 8; ++j) {
        float mn = 0.0f, mx = -INFINITY;
        for (int i = 0; i < 32; ++i) {
            const float v = xb[j * 32 + i];
            mn = fminf(mn, v);
            mx = fmaxf(mx, v);
        }
        mins[j] = mn;
        scale[j] = __fdiv_rn(__fsub_rn(mx, mn), 15.0f);
        smax = fmaxf(smax, scale[j]);
        mmax = fmaxf(mmax, -mn);
    }
    const __half d16 = __float2half_rn(__fdiv_rn(smax, 63.0f));
    const __half dmin16 = __float2half_rn(__fdiv_rn(mmax, 63.0f));
    const float df = __half2float(d16), dmf = __half2float(dmin16);
    uint8_t sc[8], mn8[8];
    uint8_t* out = blocks + b * 144;
    *reinterpret_cast<__half*>(out) = d16;
    *reinterpret_cast<__half*>(out + 2) = dmin16;
    for (int j = 0; j < 8; ++j) {
        float s = df > 0.0f ? rintf(__fdiv_rn(scale[j], df)) : 0.0f;
        float m = dmf > 0.0f ? rintf(__fdiv_rn(-mins[j], dmf)) : 0.0f;
        sc[j] = static_cast<uint8_t>(fminf(fmaxf(s, 0.0f), 63.0f));
        mn8[j] = static_cast<uint8_t>(fminf(fmaxf(m, 0.0f), 63.0f));
    }
    for (int j = 0; j < 4; ++j) {
        out[4 + j] = (sc[j] & 0x3F) | ((sc[j + 4] & 0x30) << 2);
        out[8 + j] = (mn8[j] & 0x3F) | ((mn8[j + 4] & 0x30) << 2);
        out[12 + j] = (sc[j + 4] & 0x0F) | ((mn8[j + 4] & 0x0F) << 4);
    }
    for (int g = 0; g < 4; ++g) {
        const float es0 = __fmul_rn(df, static_cast<float>(sc[2 * g])), em0 = __fmul_rn(dmf, static_cast<float>(mn8[2 * g]));
        const float es1 = __fmul_rn(df, static_cast<float>(sc[2 * g + 1])),
                    em1 = __fmul_rn(dmf, static_cast<float>(mn8[2 * g + 1]));
        for (int i = 0; i < 32; ++i) {
            float q0 = es0 > 0.0f ? rintf(__fdiv_rn(__fadd_rn(xb[(2 * g) * 32 + i], em0), es0)) : 0.0f;
            float q1 = es1 > 0.0f ? rintf(__fdiv_rn(__fadd_rn(xb[(2 * g + 1) * 32 + i], em1), es1)) : 0.0f;
            q0 = fminf(fmaxf(q0, 0.0f), 15.0f);
            q1 = fminf(fmaxf(q1, 0.0f), 15.0f);
            out[16 + g * 32 + i] = static_cast<uint8_t>(q0) | (static_cast<uint8_t>(q1) << 4);
        }
    }
}

void launch_patchify(const float* latent, float* tokens, int C, int H, int W, int p, cudaStream_t s) {
    const int64_t total = (int64_t)C * H * W;
    patchify_kernel<<<static_cast<unsigned>((total + 255) / 256), 256, 0, s>>>(latent, tokens, C, H, W, p);
    count_launch();
}

void launch_unpatchify(const float* tokens, float* latent, int C, int H, int W, int p, cudaStream_t s) {
    const int64_t total = (int64_t)C * H * W;
    unpatchify_kernel<<<static_cast<unsigned>((total + 255) / 256), 256, 0, s>>>(tokens, latent, C, H, W, p);
    count_launch();
}

void launch_timestep_embedding(const float* freq, float t, float scale, int half, float* out, cudaStream_t s) {
    timestep_embedding_kernel<<<(half + 127) / 128, 128, 0, s>>>(freq, t, nullptr, nullptr, 1.0f, scale, half, out);
    count_launch();
}

void launch_timestep_embedding_sched(const float* freq, const float* sched, const int* step, float pre_scale, float scale,
                                     int half, float* out, cudaStream_t s) {
    timestep_embedding_kernel<<<(half + 127) / 128, 128, 0, s>>>(freq, 0.0f, sched, step, pre_scale, scale, half, out);
    count_launch();
}

void launch_add_inplace(float* dst, const float* src, int64_t n, cudaStream_t s) {
    add_inplace_kernel<<<static_cast<unsigned>((n + 255) / 256), 256, 0, s>>>(dst, src, n);
    count_launch();
}

edb200_status_t quantize_rows_q4_k_device(const float* x, void* blocks, int64_t rows, int64_t k, cudaStream_t s) {
    if (k % 256) return fail(EDB200_ERR_INVALID, "quantize_rows_q4_k: k must be a multiple of 256");
    const int64_t nb = rows * k / 256;
    quant_q4_k_kernel<<<static_cast<unsigned>((nb + 127) / 128), 128, 0, s>>>(x, static_cast<uint8_t*>(blocks), nb);
    count_launch();
    return check_cuda(cudaGetLastError(), "quantize_rows_q4_k launch");
}

// -------------------------------------------------------------- ParamTable --

ParamTable::~ParamTable() {
    for (Param& p : params_) {
        if (p.qw) edb200_qweight_destroy(p.qw);
        if (p.f32) cudaFree(p.f32);
    }
}

void ParamTable::add(const std::string& name, int64_t n_out, int64_t k, bool quantised, int wtype) {
    Param p;
    p.spec.name = name;
    p.spec.n_out = n_out;
    p.spec.k = k;
    p.spec.quantised = quantised;
    p.spec.ggml_type = quantised ? wtype : EDB200_TYPE_F32;
    index_[name] = params_.size();
    params_.push_back(p);
}

Param* ParamTable::find(const std::string& name) {
    auto it = index_.find(name);
    return it == index_.end() ? nullptr : &params_[it->second];
}

const Param* ParamTable::get(const std::string& name) const {
    auto it = index_.find(name);
    return it == index_.end() ? nullptr : &params_[it->second];
}

edb200_status_t ParamTable::set(const std::string& name, int ggml_type, const void* data, int64_t nbytes,
                                bool on_device, cudaStream_t stream) {
    Param* p = find(name);
    if (p == nullptr) return fail(EDB200_ERR_INVALID, "set_tensor: unknown tensor '%s'", name.c_str());
    if (data == nullptr) return fail(EDB200_ERR_INVALID, "set_tensor: null data for '%s'", name.c_str());
    if (ggml_type != p->spec.ggml_type) {
        return fail(EDB200_ERR_INVALID, "set_tensor: '%s' expects ggml type %d, got %d", name.c_str(),
                    p->spec.ggml_type, ggml_type);
    }
    const int64_t want = p->spec.n_out * ggml_row_bytes(ggml_type, p->spec.k);
    if (nbytes != want) {
        return fail(EDB200_ERR_INVALID, "set_tensor: '%s' expects %lld bytes, got %lld", name.c_str(),
                    (long long)want, (long long)nbytes);
    }
    if (p->spec.quantised) {
        const void* dev_src = data;
        void* tmp = nullptr;
        if (!on_device) {
            cudaError_t e = cudaMalloc(&tmp, nbytes);
            if (e != cudaSuccess) return fail(EDB200_ERR_NOMEM, "set_tensor: cudaMalloc: %s", cudaGetErrorString(e));
            e = cudaMemcpyAsync(tmp, data, nbytes, cudaMemcpyHostToDevice, stream);
            if (e != cudaSuccess) {
                cudaFree(tmp);
                return check_cuda(e, "set_tensor H2D");
            }
            dev_src = tmp;
        }
        if (p->qw) {
            bytes_ -= edb200_qweight_bytes(p->qw);
            edb200_qweight_destroy(p->qw);
            p->qw = nullptr;
        }
        edb200_status_t st = edb200_qweight_create(ggml_type, dev_src, p->spec.n_out, p->spec.k, stream, &p->qw);
        if (tmp) cudaFree(tmp);
        if (st != EDB200_OK) return st;
        bytes_ += edb200_qweight_bytes(p->qw);
    } else {
        if (p->f32 == nullptr) {
            // pad to a multiple of 16 bytes so float4 readers may run past a short vector's end
            cudaError_t e = cudaMalloc(reinterpret_cast<void**>(&p->f32), (nbytes + 15) & ~int64_t(15));
            if (e != cudaSuccess) return fail(EDB200_ERR_NOMEM, "set_tensor: cudaMalloc: %s", cudaGetErrorString(e));
            bytes_ += nbytes;
        }
        cudaError_t e = cudaMemcpyAsync(p->f32, data, nbytes, on_device ? cudaMemcpyDeviceToDevice : cudaMemcpyHostToDevice,
                                        stream);
        if (e == cudaSuccess) e = cudaStreamSynchronize(stream);
        if (e != cudaSuccess) return check_cuda(e, "set_tensor copy");
    }
    p->loaded = true;
    ++generation_;
    return EDB200_OK;
}

static uint64_t name_seed(uint64_t seed, const std::string& name) {
    uint64_t h = 1469598103934665603ull;
    for (unsigned char c : name) h = (h ^ c) * 1099511628211ull;
    return h ^ (seed * 0x9E3779B97F4A7C15ull);
}

edb200_status_t ParamTable::init_random(uint64_t seed, float std, cudaStream_t stream) {
    int64_t max_elems = 0, max_raw = 0;
    for (const Param& p : params_) {
        const int64_t n = p.spec.n_out * p.spec.k;
        max_elems = n > max_elems ? n : max_elems;
        if (p.spec.quantised) {
            const int64_t raw = p.spec.n_out * ggml_row_bytes(p.spec.ggml_type, p.spec.k);
            max_raw = raw > max_raw ? raw : max_raw;
        }
    }
    float* tmp = nullptr;
    void* raw = nullptr;
    cudaError_t e = cudaMalloc(reinterpret_cast<void**>(&tmp), max_elems * 4);
    if (e == cudaSuccess && max_raw > 0) e = cudaMalloc(&raw, max_raw);
    if (e != cudaSuccess) {
        cudaFree(tmp);
        return fail(EDB200_ERR_NOMEM, "init_random: cudaMalloc: %s", cudaGetErrorString(e));
    }
    edb200_status_t st = EDB200_OK;
    for (Param& p : params_) {
        const int64_t n = p.spec.n_out * p.spec.k;
        st = edb200_fill_normal(tmp, n, name_seed(seed, p.spec.name), 0.0f, std, stream);
        if (st != EDB200_OK) break;
        const std::string& nm = p.spec.name;
        auto ends_with = [&](const char* suf) {
            const size_t n = strlen(suf);
            return nm.size() >= n && nm.compare(nm.size() - n, n, suf) == 0;
        };
        // norm weights are centred on one
        if (ends_with(".scale") || ends_with(".norm_q.weight") || ends_with(".norm_k.weight") || ends_with("norm3.weight") ||
            ends_with(".norm_added_q.weight") || ends_with(".norm_added_k.weight") || ends_with("txt_norm.weight")) {
            add_one_kernel<<<static_cast<unsigned>((n + 255) / 256), 256, 0, stream>>>(tmp, n);
            count_launch();
        }
        if (p.spec.quantised) {
            if (p.spec.ggml_type == EDB200_TYPE_Q8_0) {
                st = edb200_quantize_rows_q8_0(tmp, raw, p.spec.n_out, p.spec.k, stream);
            } else {
                st = quantize_rows_q4_k_device(tmp, raw, p.spec.n_out, p.spec.k, stream);
            }
            if (st != EDB200_OK) break;
            st = set(nm, p.spec.ggml_type, raw, p.spec.n_out * ggml_row_bytes(p.spec.ggml_type, p.spec.k), true, stream);
        } else {
            st = set(nm, EDB200_TYPE_F32, tmp, n * 4, true, stream);
        }
        if (st != EDB200_OK) break;
    }
    cudaStreamSynchronize(stream);
    cudaFree(tmp);
    cudaFree(raw);
    return st;
}

edb200_status_t ParamTable::fetch_f32(const std::string& name, float* out, int64_t n_floats, bool on_device,
                                      cudaStream_t stream) const {
    const Param* p = get(name);
    if (p == nullptr) return fail(EDB200_ERR_INVALID, "get_tensor: unknown tensor '%s'", name.c_str());
    if (!p->loaded) return fail(EDB200_ERR_INVALID, "get_tensor: '%s' has not been set", name.c_str());
    const int64_t n = p->spec.n_out * p->spec.k;
    if (out == nullptr || n_floats != n) {
        return fail(EDB200_ERR_INVALID, "get_tensor: '%s' has %lld values, room for %lld given", name.c_str(),
                    (long long)n, (long long)n_floats);
    }
    float* dev = out;
    if (!on_device && p->spec.quantised) {
        cudaError_t e = cudaMalloc(reinterpret_cast<void**>(&dev), n * 4);
        if (e != cudaSuccess) return fail(EDB200_ERR_NOMEM, "get_tensor: cudaMalloc: %s", cudaGetErrorString(e));
    }
    edb200_status_t st = EDB200_OK;
    cudaError_t e = cudaSuccess;
    if (p->spec.quantised) {
        st = edb200_qweight_dequantize(p->qw, dev, stream);
        if (st == EDB200_OK && !on_device) e = cudaMemcpyAsync(out, dev, n * 4, cudaMemcpyDeviceToHost, stream);
    } else {
        e = cudaMemcpyAsync(out, p->f32, n * 4, on_device ? cudaMemcpyDeviceToDevice : cudaMemcpyDeviceToHost, stream);
    }
    if (e == cudaSuccess) e = cudaStreamSynchronize(stream);
    if (dev != out) cudaFree(dev);
    if (st != EDB200_OK) return st;
    return check_cuda(e, "get_tensor copy");
}

edb200_status_t ParamTable::all_loaded() const {
    for (const Param& p : params_) {
        if (!p.loaded) return fail(EDB200_ERR_INVALID, "tensor '%s' has not been set", p.spec.name.c_str());
    }
    return EDB200_OK;
}

// --------------------------------------------------------------- Workspace --

Workspace::~Workspace() { cudaFree(base_); }

edb200_status_t Workspace::reserve(int64_t bytes) {
    cudaFree(base_);
    base_ = nullptr;
    cap_ = used_ = 0;
    cudaError_t e = cudaMalloc(reinterpret_cast<void**>(&base_), bytes);
    if (e != cudaSuccess) return fail(EDB200_ERR_NOMEM, "workspace: cudaMalloc(%lld): %s", (long long)bytes, cudaGetErrorString(e));
    cap_ = bytes;
    return EDB200_OK;
}

void* Workspace::take(int64_t bytes) {
    const int64_t aligned = (bytes + 255) & ~int64_t(255);
    if (used_ + aligned > cap_) return nullptr;
    void* p = base_ + used_;
    used_ += aligned;
    return p;
}

edb200_status_t ReuseAnchors::set_capture(int anchor, float* dst, int depth, const char* who) {
    if (anchor == EDB200_ANCHOR_MODEL_IN) {
        in = dst;
    } else if (anchor == EDB200_ANCHOR_MODEL_OUT) {
        out = dst;
    } else if (anchor >= 0 && anchor < depth) {
        block.resize(static_cast<size_t>(depth), nullptr);
        block[static_cast<size_t>(anchor)] = dst;
    } else {
        return fail(EDB200_ERR_INVALID, "%s_set_anchor_capture: anchor %d (block outputs are 0..%d)", who, anchor, depth - 1);
    }
    return EDB200_OK;
}

edb200_status_t ReuseAnchors::set_stop(int blk, int depth, const char* who) {
    if (blk < -1 || blk >= depth) {
        return fail(EDB200_ERR_INVALID, "%s_set_stop_after: block must be -1 (off) or a block index below %d", who, depth);
    }
    stop_after = blk;
    return EDB200_OK;
}

edb200_status_t ReuseAnchors::set_region(int at, int resume, const float* residual, int depth, const char* who) {
    if (residual == nullptr || at < 0) {   // off
        inject_at = -1;
        inject_residual = nullptr;
        return EDB200_OK;
    }
    if (at >= depth || resume <= at || resume > depth) {
        return fail(EDB200_ERR_INVALID, "%s_set_region_inject: need 0 <= at < resume <= %d", who, depth);
    }
    if (at > 0 && in == nullptr) {
        return fail(EDB200_ERR_INVALID,
                    "%s_set_region_inject: a region that starts after block 0 needs the ModelIn capture buffer set "
                    "(the stream is rebuilt from it)", who);
    }
    inject_at = at;
    inject_resume = resume;
    inject_residual = residual;
    return EDB200_OK;
}

bool ReuseAnchors::region_inject(int& i, float* stream, int64_t n, cudaStream_t s) const {
    if (inject_residual == nullptr || i != inject_at) return false;
    if (n > 0) {
        // x = x_before + residual; at block 0 the stream still is x_before
        if (i > 0) cudaMemcpyAsync(stream, in, static_cast<size_t>(n) * 4, cudaMemcpyDeviceToDevice, s);
        launch_add_inplace(stream, inject_residual, n, s);
    }
    i = inject_resume - 1;
    return true;
}

void ReuseAnchors::capture_in(const float* stream, int64_t n, cudaStream_t s) const {
    if (in != nullptr && n > 0) cudaMemcpyAsync(in, stream, static_cast<size_t>(n) * 4, cudaMemcpyDeviceToDevice, s);
}

void ReuseAnchors::capture_block(int i, const float* stream, int64_t n, cudaStream_t s) const {
    if (i < static_cast<int>(block.size()) && block[static_cast<size_t>(i)] != nullptr && n > 0) {
        cudaMemcpyAsync(block[static_cast<size_t>(i)], stream, static_cast<size_t>(n) * 4, cudaMemcpyDeviceToDevice, s);
    }
}

void ReuseAnchors::finish(float* stream, int64_t n, cudaStream_t s) const {
    if (n <= 0) return;
    if (stream_override != nullptr) launch_add_inplace(stream, stream_override, n, s);
    if (out != nullptr) cudaMemcpyAsync(out, stream, static_cast<size_t>(n) * 4, cudaMemcpyDeviceToDevice, s);
}

}  // namespace edb
