// SD3-medium (MMDiT) denoise-pass executor: the op schedule of MMDiT::forward
// (reference src/dit_models/models/mmdit.hpp:3403-3487, block_mixing :2685-2775,
// DismantledBlock::pre_attention :2454-2491 / post_attention :2606-2626,
// FinalLayer::forward :3143-3160) on the kernels of this library, for the
// SD3-medium variant (no q/k norm, no second self-attention, no RoPE: a learned
// position table is added to the patch embedding instead).
//
// Context rows first, image rows after them, in every [T, ...] buffer, so the
// joint attention needs no concat.  Per joint block, with c = t_emb + y_emb:
//   m_ctx, m_x = adaLN(silu(c))                       weight-streaming GEMVs, all up front
//   XMOD = modulate(LN(stream), shift_msa, scale_msa) both streams
//   QKV  = XMOD Wqkv + b                              one two-problem GEMM launch
//   Q,K,V head-major (no norm, no RoPE)               pack kernel
//   ATT  = attention(Q, K, V) over context + image    f16 kernel (head dim 64)
//   stream += gate_msa * (ATT Wproj + b)              two-problem GEMM, fused epilogue
//   stream += gate_mlp * fc2(gelu(fc1(modulate(LN(stream), shift_mlp, scale_mlp))))
// The last block's context side is "pre_only": it only feeds the attention
// (2 modulation vectors in (scale, shift) order).
#include "edb200_model.h"

#include <cuda_fp16.h>

#include <cmath>
#include <cstdlib>
#include <cstring>
#include <vector>

using namespace edb;

struct edb200_sd3 {
    edb200_sd3_config_t cfg;
    ParamTable params;
    Workspace ws;
    int lat_h = 0, lat_w = 0, n_ctx = 0, n_img = 0;
    float* X = nullptr;   // [n_ctx + n_img, H]: context rows, then image rows
    void *XMOD = nullptr, *QKV = nullptr, *Q = nullptr, *K = nullptr, *V = nullptr, *ATT = nullptr, *HID = nullptr;
    float *MODS = nullptr, *CVEC = nullptr, *TMP = nullptr, *TEMB = nullptr, *FREQ = nullptr, *TOK_IN = nullptr,
          *TOK_OUT = nullptr, *LAT_IN = nullptr, *LAT_OUT = nullptr, *CTX_IN = nullptr, *Y_IN = nullptr;
    void* SAGE = nullptr;
    int64_t sage_bytes = 0;
    float* tap = nullptr;
    ReuseAnchors anchors;   // computation-reuse seam (capture / probe stop / whole-stack inject)
    float* pinned = nullptr;
    int64_t pinned_bytes = 0;
    // sequence-parallel execution (world > 1): this rank's slice [context rows ; image rows] of the
    // [context ; image] sequence and the exchange buffers (see edb200_flux.cu for the scheme)
    edb200_comm_t* comm = nullptr;
    int rank = 0, world = 1;
    int64_t t_loc = 0, t_rows = 0, ctx_l = 0, img_l = 0, img_first = 0;
    bool p2p = false;
    void *QL = nullptr, *KL = nullptr, *VL = nullptr, *AOUT = nullptr, *STG = nullptr;
    float* TOK_LOC = nullptr;
    edb200_sp_peers_t qkv_peers, att_peers;
    // all adaLN projections of a pass (and the final layer's) as one weight-streaming launch
    edb200_gemv_batch_t* mod_batch = nullptr;
    uint64_t mod_batch_gen = 0;
    edb200_sp_peers_t mods_peers;
};

namespace {

struct Lin {
    const edb200_qweight_t* w;
    const float* b;
};

Lin qlin(edb200_sd3* m, const std::string& name) {
    Lin l;
    l.w = m->params.get(name + ".weight")->qw;
    l.b = m->params.get(name + ".bias")->f32;
    return l;
}

const float* fparam(edb200_sd3* m, const std::string& name) { return m->params.get(name)->f32; }

edb200_status_t dense(edb200_sd3* m, const std::string& name, const float* x, int64_t rows, int64_t ldx, int act,
                      float* y, int64_t ldy, cudaStream_t s) {
    const Param* w = m->params.get(name + ".weight");
    return edb200_linear_f32(w->f32, fparam(m, name + ".bias"), x, rows, w->spec.k, w->spec.n_out, ldx, 0, act, y, ldy, s);
}

edb200_epilogue_t make_ep(void* out, int dt, int64_t ldo, const float* bias) {
    edb200_epilogue_t ep;
    memset(&ep, 0, sizeof(ep));
    ep.out = out;
    ep.out_dtype = dt;
    ep.ldo = ldo;
    ep.bias = bias;
    return ep;
}

int64_t mods_per_block(const edb200_sd3_config_t& c) { return 12 * (int64_t)c.hidden_size; }

void register_params(edb200_sd3* m) {
    const edb200_sd3_config_t& c = m->cfg;
    const int64_t H = c.hidden_size, M = c.mlp_hidden;
    ParamTable& t = m->params;
    auto lin = [&](const std::string& name, int64_t n_out, int64_t k, bool q) {
        t.add(name + ".weight", n_out, k, q, c.wtype);
        t.add(name + ".bias", 1, n_out, false, c.wtype);
    };
    // Not quantised: biases, pos_embed and the x_/t_/y_/context_ embedders
    // (tensor_should_be_converted, reference src/core/runtime/model_loader.cpp:2141-2172).
    lin("x_embedder.proj", H, (int64_t)c.in_channels * c.patch_size * c.patch_size, false);
    t.add("pos_embed", (int64_t)c.pos_embed_max_size * c.pos_embed_max_size, H, false, c.wtype);
    lin("t_embedder.mlp.0", H, 256, false);
    lin("t_embedder.mlp.2", H, H, false);
    lin("y_embedder.mlp.0", H, c.adm_in_channels, false);
    lin("y_embedder.mlp.2", H, H, false);
    lin("context_embedder", H, c.context_size, false);
    for (int i = 0; i < c.depth; ++i) {
        for (const char* side : {"context_block", "x_block"}) {
            const std::string p = "joint_blocks." + std::to_string(i) + "." + side + ".";
            const bool pre_only = strcmp(side, "context_block") == 0 && i == c.depth - 1;
            lin(p + "adaLN_modulation.1", (pre_only ? 2 : 6) * H, H, true);
            lin(p + "attn.qkv", 3 * H, H, true);
            if (!pre_only) {
                lin(p + "attn.proj", H, H, true);
                lin(p + "mlp.fc1", M, H, true);
                lin(p + "mlp.fc2", H, M, true);
            }
        }
    }
    lin("final_layer.adaLN_modulation.1", 2 * H, H, true);
    lin("final_layer.linear", (int64_t)c.patch_size * c.patch_size * c.out_channels, H, true);
}

// x[t, :] += pos_embed[(top + t / w_tok) * max + left + t % w_tok, :]  (cropped_pos_embed, mmdit.hpp:3263-3301);
// row 0 of x is image token t0.
__global__ void add_pos_embed_kernel(float* __restrict__ x, const float* __restrict__ pos, int H, int w_tok, int max_size,
                                     int top, int left, int64_t t0, int64_t total) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const int64_t t = t0 + i / H;
    const int c = static_cast<int>(i % H);
    const int64_t row = (int64_t)(top + t / w_tok) * max_size + left + t % w_tok;
    x[i] += pos[row * H + c];
}

// tokens [h*w, p*p*C] with feature = c + C*(px + p*py) -> [C, h*p, w*p]
// (DiT::unpatchify, patch_last = false, common_dit.hpp:38-64)
__global__ void unpatchify_cf_kernel(const float* __restrict__ tok, float* __restrict__ lat, int C, int H, int W, int p) {
    const int64_t total = (int64_t)C * H * W;
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const int x = static_cast<int>(i % W), y = static_cast<int>((i / W) % H), c = static_cast<int>(i / ((int64_t)W * H));
    const int64_t token = (int64_t)(y / p) * (W / p) + x / p;
    const int feat = c + C * ((x % p) + p * (y % p));
    lat[i] = tok[token * ((int64_t)C * p * p) + feat];
}

__global__ void cfg_combine_kernel(const float4* __restrict__ u, const float4* __restrict__ c, float s, float4* __restrict__ o,
                                   int64_t n4) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n4) return;
    const float4 a = u[i], b = c[i];
    // uncond + scale * (cond - uncond), each operation rounded on its own like the reference's tensor
    // arithmetic (flux_pipeline.cpp:1258): no FMA contraction
    o[i] = make_float4(__fadd_rn(a.x, __fmul_rn(s, __fsub_rn(b.x, a.x))), __fadd_rn(a.y, __fmul_rn(s, __fsub_rn(b.y, a.y))),
                       __fadd_rn(a.z, __fmul_rn(s, __fsub_rn(b.z, a.z))), __fadd_rn(a.w, __fmul_rn(s, __fsub_rn(b.w, a.w))));
}

// Qwen-Image's guidance combine (ed_qwen_apply_true_cfg, src/dit_models/pipelines/qwen_image_pipeline.cpp:29-85):
// per p x p latent patch (all channels), guided = u + s*(c - u) in f32, then scaled by
// ||c|| / ||guided|| with both sums of squares accumulated in double in the order (dy, dx, channel).
// One thread per patch walks its p*p*C values in that order, so the result has the reference's bits.
__global__ void cfg_combine_rescaled_kernel(const float* __restrict__ cond, const float* __restrict__ uncond, float s,
                                            int p, int C, int H, int W, float* __restrict__ out) {
    const int pw = W / p, ph = H / p;
    const int idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= pw * ph) return;
    const int px = (idx % pw) * p, py = (idx / pw) * p;
    double cond_sq = 0.0, guided_sq = 0.0;
    for (int dy = 0; dy < p; ++dy) {
        for (int dx = 0; dx < p; ++dx) {
            for (int c = 0; c < C; ++c) {
                const int64_t off = (px + dx) + (int64_t)W * ((py + dy) + (int64_t)H * c);
                const float cv = cond[off], uv = uncond[off];
                const float g = __fadd_rn(uv, __fmul_rn(s, __fsub_rn(cv, uv)));
                cond_sq = __dadd_rn(cond_sq, __dmul_rn((double)cv, (double)cv));
                guided_sq = __dadd_rn(guided_sq, __dmul_rn((double)g, (double)g));
            }
        }
    }
    const float rescale = guided_sq > 0.0 ? (float)__ddiv_rn(__dsqrt_rn(cond_sq), __dsqrt_rn(guided_sq)) : 0.0f;
    for (int dy = 0; dy < p; ++dy) {
        for (int dx = 0; dx < p; ++dx) {
            for (int c = 0; c < C; ++c) {
                const int64_t off = (px + dx) + (int64_t)W * ((py + dy) + (int64_t)H * c);
                const float cv = cond[off], uv = uncond[off];
                out[off] = __fmul_rn(__fadd_rn(uv, __fmul_rn(s, __fsub_rn(cv, uv))), rescale);
            }
        }
    }
}

edb200_status_t ln_mod(const float* x, int64_t H, const float* shift, const float* scale, int64_t rows, void* y,
                       int y_dtype, cudaStream_t s) {
    if (rows == 0) return EDB200_OK;
    return edb200_layernorm_modulate(x, H, shift, scale, nullptr, nullptr, rows, H, 1e-6f, y, y_dtype, H, s);
}

// Row-count-tolerant two-problem GEMM: under sequence parallelism a rank may own no context rows.
edb200_status_t mm_pair(const edb200_qweight_t* w0, const void* x0, int64_t m0, int64_t ldx0, const edb200_epilogue_t* e0,
                        const edb200_qweight_t* w1, const void* x1, int64_t m1, int64_t ldx1, const edb200_epilogue_t* e1,
                        cudaStream_t s) {
    if (m0 > 0 && m1 > 0) return edb200_mul_mat_q_pair(w0, x0, m0, ldx0, e0, w1, x1, m1, ldx1, e1, EDB200_TYPE_F16, s);
    if (m0 > 0) return edb200_mul_mat_q(w0, x0, EDB200_TYPE_F16, m0, ldx0, e0, s);
    if (m1 > 0) return edb200_mul_mat_q(w1, x1, EDB200_TYPE_F16, m1, ldx1, e1, s);
    return EDB200_OK;
}

// Joint attention over [context ; image] into the local rows of ATT: single GPU, NCCL exchange, or
// peer-memory exchange with flag barriers (MMDiT forward_sp, mmdit.hpp:3117-3128, 3439-3466).
// INT8 scores (when configured) run on the middle layers only: sage_attn_skip_layer,
// src/core/backend/ggml/ed_ggml_sage_attn_ext.hpp:146-159, layer index from mmdit.hpp:3349-3350.
edb200_status_t joint_attention(edb200_sd3* m, int layer, int64_t T, cudaStream_t s) {
    const edb200_sd3_config_t& c = m->cfg;
    const int64_t H = c.hidden_size;
    const int d = static_cast<int>(H / c.num_heads);
    const int heads = c.num_heads / m->world;
    const float scale = 1.0f / std::sqrt(static_cast<float>(d));
    const int flags = (c.sage_smooth_q ? EDB200_SAGE_SMOOTH_Q : 0) | EDB200_SAGE_FAST_MEANS;
    const bool sage = c.attention == EDB200_ATTN_SAGE_INT8 && layer >= c.sage_skip_first &&
                      layer < c.depth - c.sage_skip_last;
    const int64_t head_rows = m->world > 1 ? m->t_loc * m->world : T;
    __half* att = static_cast<__half*>(m->ATT);
    if (m->p2p) {
        EDB_TRY(edb200_sp_barrier(m->comm, s));
        if (sage) {
            EDB_TRY(edb200_sage_attention_strided(m->Q, m->K, m->V, heads, T, head_rows, d, scale, flags, m->SAGE,
                                                  m->sage_bytes, nullptr, EDB200_TYPE_F16, H, &m->att_peers, s));
        } else {
            EDB_TRY(edb200_attention_f16_strided(m->Q, m->K, m->V, heads, T, T, head_rows, head_rows, d, scale, nullptr,
                                                 EDB200_TYPE_F16, H, &m->att_peers, s));
        }
        return edb200_sp_barrier(m->comm, s);
    }
    void* att_out = att;
    int64_t att_ld = H;
    if (m->world > 1) {
        const void* send[3] = {m->QL, m->KL, m->VL};
        void* recv[3] = {m->Q, m->K, m->V};
        EDB_TRY(edb200_sp_all_to_all_heads(m->comm, send, recv, 3, c.num_heads, m->t_loc, (int64_t)d * 2, s));
        att_out = m->AOUT;
        att_ld = (int64_t)heads * d;
    }
    if (sage) {
        EDB_TRY(edb200_sage_attention_strided(m->Q, m->K, m->V, heads, T, head_rows, d, scale, flags, m->SAGE,
                                              m->sage_bytes, att_out, EDB200_TYPE_F16, att_ld, nullptr, s));
    } else {
        EDB_TRY(edb200_attention_f16_strided(m->Q, m->K, m->V, heads, T, T, head_rows, head_rows, d, scale, att_out,
                                             EDB200_TYPE_F16, att_ld, nullptr, s));
    }
    if (m->world > 1) {
        EDB_TRY(edb200_sp_all_to_all_tokens(m->comm, m->AOUT, m->STG, att, m->t_loc, (int64_t)heads * d * 2, H * 2, s));
    }
    return EDB200_OK;
}

// Every adaLN projection of the pass as one batch (block i: context 6H (2H on the pre_only side), x 6H; then
// the final layer's 2H); built at the first pass after prepare or after a tensor was reloaded.
edb200_status_t ensure_mod_batch(edb200_sd3* m, cudaStream_t s) {
    if (m->mod_batch != nullptr && m->mod_batch_gen == m->params.generation()) return EDB200_OK;
    const edb200_sd3_config_t& c = m->cfg;
    const int64_t H = c.hidden_size;
    edb200_gemv_batch_destroy(m->mod_batch);
    m->mod_batch = nullptr;
    std::vector<const edb200_qweight_t*> bw;
    std::vector<const float*> bb;
    std::vector<float*> by;
    for (int i = 0; i < c.depth; ++i) {
        const std::string pb = "joint_blocks." + std::to_string(i) + ".";
        const Lin lc = qlin(m, pb + "context_block.adaLN_modulation.1"), lx = qlin(m, pb + "x_block.adaLN_modulation.1");
        bw.push_back(lc.w), bb.push_back(lc.b), by.push_back(m->MODS + (int64_t)i * 12 * H);
        bw.push_back(lx.w), bb.push_back(lx.b), by.push_back(m->MODS + ((int64_t)i * 12 + 6) * H);
    }
    const Lin lf = qlin(m, "final_layer.adaLN_modulation.1");
    bw.push_back(lf.w), bb.push_back(lf.b), by.push_back(m->MODS + (int64_t)c.depth * 12 * H);
    EDB_TRY(edb200_gemv_batch_create(bw.data(), bb.data(), by.data(), (int)bw.size(), s, &m->mod_batch));
    m->mod_batch_gen = m->params.generation();
    memset(&m->mods_peers, 0, sizeof(m->mods_peers));
    if (m->p2p) {
        m->mods_peers.world = m->world;
        m->mods_peers.rank = m->rank;
        for (int r = 0; r < m->world; ++r) m->mods_peers.buf[0][r] = edb200_comm_peer_ptr(m->comm, r, m->MODS);
    }
    return EDB200_OK;
}

}  // namespace

extern "C" {

edb200_status_t edb200_cfg_combine(const float* uncond, const float* cond, float scale, float* out, int64_t n,
                                   void* stream) {
    if (uncond == nullptr || cond == nullptr || out == nullptr || n <= 0 || n % 4) {
        return fail(EDB200_ERR_INVALID, "cfg_combine: bad argument (n %% 4 == 0 required)");
    }
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    ProfScope prof(s, PROF_ELEMENTWISE, 0.0, 12.0 * (double)n);
    cfg_combine_kernel<<<static_cast<unsigned>((n / 4 + 255) / 256), 256, 0, s>>>(
        reinterpret_cast<const float4*>(uncond), reinterpret_cast<const float4*>(cond), scale,
        reinterpret_cast<float4*>(out), n / 4);
    count_launch();
    return check_cuda(cudaGetLastError(), "cfg_combine launch");
}

edb200_status_t edb200_cfg_combine_rescaled(const float* uncond, const float* cond, float scale, int patch_size,
                                            int channels, int height, int width, float* out, void* stream) {
    if (uncond == nullptr || cond == nullptr || out == nullptr || patch_size <= 0 || channels <= 0 || height <= 0 ||
        width <= 0 || height % patch_size || width % patch_size) {
        return fail(EDB200_ERR_INVALID, "cfg_combine_rescaled: bad argument (height, width multiples of the patch size)");
    }
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int patches = (height / patch_size) * (width / patch_size);
    ProfScope prof(s, PROF_ELEMENTWISE, 0.0, 20.0 * (double)channels * height * width);
    cfg_combine_rescaled_kernel<<<(patches + 127) / 128, 128, 0, s>>>(cond, uncond, scale, patch_size, channels, height,
                                                                      width, out);
    count_launch();
    return check_cuda(cudaGetLastError(), "cfg_combine_rescaled launch");
}

edb200_status_t edb200_sd3_create(const edb200_sd3_config_t* cfg, edb200_sd3_t** out) {
    if (cfg == nullptr || out == nullptr) return fail(EDB200_ERR_INVALID, "sd3_create: null argument");
    const edb200_sd3_config_t& c = *cfg;
    if (c.hidden_size <= 0 || c.num_heads <= 0 || c.hidden_size % c.num_heads || c.depth <= 0) {
        return fail(EDB200_ERR_INVALID, "sd3_create: hidden_size must be a positive multiple of num_heads");
    }
    const int d = c.hidden_size / c.num_heads;
    if (d != 64 && d != 128) return fail(EDB200_ERR_UNSUPPORTED, "sd3_create: head dim must be 64 or 128");
    if (c.wtype != EDB200_TYPE_Q8_0 && c.wtype != EDB200_TYPE_Q4_K) {
        return fail(EDB200_ERR_UNSUPPORTED, "sd3_create: wtype must be q8_0 or q4_K");
    }
    if (c.hidden_size % 256 || c.mlp_hidden % 256 || c.hidden_size > 8192) {
        return fail(EDB200_ERR_UNSUPPORTED, "sd3_create: hidden_size (<= 8192) and mlp_hidden must be multiples of 256");
    }
    if (c.attention != EDB200_ATTN_F16 && c.attention != EDB200_ATTN_SAGE_INT8) {
        return fail(EDB200_ERR_INVALID, "sd3_create: attention must be EDB200_ATTN_F16 or EDB200_ATTN_SAGE_INT8");
    }
    if (c.sage_skip_first < 0 || c.sage_skip_last < 0) return fail(EDB200_ERR_INVALID, "sd3_create: negative layer skip");
    const int pf = c.patch_size * c.patch_size * c.out_channels;
    if (c.patch_size <= 0 || pf % 32 || (c.patch_size * c.patch_size * c.in_channels) % 4 || c.adm_in_channels % 4 ||
        c.context_size % 4 || c.pos_embed_max_size <= 0) {
        return fail(EDB200_ERR_UNSUPPORTED, "sd3_create: patch_size^2 * out_channels must be a multiple of 32");
    }
    if (device_error_word() == nullptr) return fail(EDB200_ERR_CUDA, "sd3_create: no CUDA device");
    edb200_sd3* m = new (std::nothrow) edb200_sd3();
    if (m == nullptr) return fail(EDB200_ERR_NOMEM, "sd3_create: host allocation failed");
    m->cfg = c;
    register_params(m);
    *out = m;
    return EDB200_OK;
}

void edb200_sd3_destroy(edb200_sd3_t* m) {
    if (m == nullptr) return;
    if (m->pinned) cudaFreeHost(m->pinned);
    edb200_gemv_batch_destroy(m->mod_batch);
    delete m;
}

int edb200_sd3_tensor_count(const edb200_sd3_t* m) {
    return m ? static_cast<int>(const_cast<edb200_sd3_t*>(m)->params.params().size()) : 0;
}

edb200_status_t edb200_sd3_tensor_info(const edb200_sd3_t* m, int index, char* name, int name_cap, int* ggml_type,
                                       int64_t* n_out, int64_t* k, int64_t* nbytes) {
    if (m == nullptr || index < 0 || index >= edb200_sd3_tensor_count(m)) {
        return fail(EDB200_ERR_INVALID, "sd3_tensor_info: bad index");
    }
    const Param& p = const_cast<edb200_sd3_t*>(m)->params.params()[index];
    if (name != nullptr && name_cap > 0) {
        strncpy(name, p.spec.name.c_str(), name_cap - 1);
        name[name_cap - 1] = '\0';
    }
    if (ggml_type) *ggml_type = p.spec.ggml_type;
    if (n_out) *n_out = p.spec.n_out;
    if (k) *k = p.spec.k;
    if (nbytes) *nbytes = p.spec.n_out * ggml_row_bytes(p.spec.ggml_type, p.spec.k);
    return EDB200_OK;
}

edb200_status_t edb200_sd3_set_tensor(edb200_sd3_t* m, const char* name, int ggml_type, const void* data, int64_t nbytes,
                                      int on_device, void* stream) {
    if (m == nullptr || name == nullptr) return fail(EDB200_ERR_INVALID, "sd3_set_tensor: null argument");
    return m->params.set(name, ggml_type, data, nbytes, on_device != 0, static_cast<cudaStream_t>(stream));
}

edb200_status_t edb200_sd3_get_tensor_f32(const edb200_sd3_t* m, const char* name, float* out, int64_t n_floats,
                                          int on_device, void* stream) {
    if (m == nullptr || name == nullptr) return fail(EDB200_ERR_INVALID, "sd3_get_tensor_f32: null argument");
    return m->params.fetch_f32(name, out, n_floats, on_device != 0, static_cast<cudaStream_t>(stream));
}

edb200_status_t edb200_sd3_load_gguf(edb200_sd3_t* m, const char* path, const char* strip_prefix, int* n_loaded,
                                    void* stream) {
    if (m == nullptr || path == nullptr) return fail(EDB200_ERR_INVALID, "sd3_load_gguf: null argument");
    return load_gguf(m->params, EDB200_FAMILY_SD3, path, strip_prefix, static_cast<cudaStream_t>(stream), n_loaded);
}

edb200_status_t edb200_sd3_load_safetensors(edb200_sd3_t* m, const char* path, const char* strip_prefix, int* n_loaded,
                                           void* stream) {
    if (m == nullptr || path == nullptr) return fail(EDB200_ERR_INVALID, "sd3_load_safetensors: null argument");
    return load_safetensors(m->params, EDB200_FAMILY_SD3, path, strip_prefix, static_cast<cudaStream_t>(stream), n_loaded);
}

edb200_status_t edb200_sd3_init_random(edb200_sd3_t* m, uint64_t seed, float std, void* stream) {
    if (m == nullptr) return fail(EDB200_ERR_INVALID, "sd3_init_random: null model");
    return m->params.init_random(seed, std, static_cast<cudaStream_t>(stream));
}

int64_t edb200_sd3_weight_bytes(const edb200_sd3_t* m) { return m ? m->params.device_bytes() : 0; }

edb200_status_t edb200_sd3_set_comm(edb200_sd3_t* m, edb200_comm_t* comm) {
    if (m == nullptr) return fail(EDB200_ERR_INVALID, "sd3_set_comm: null model");
    if (m->comm != nullptr && m->comm != comm) edb200_comm_unmap_peers(m->comm);   // collective
    m->comm = comm;
    m->rank = comm ? edb200_comm_rank(comm) : 0;
    m->world = comm ? edb200_comm_world(comm) : 1;
    m->lat_h = m->lat_w = m->n_ctx = 0;   // the workspace must be prepared again
    m->p2p = false;
    return EDB200_OK;
}

edb200_status_t edb200_sd3_set_anchor_capture(edb200_sd3_t* m, int anchor, float* dst) {
    if (m == nullptr) return fail(EDB200_ERR_INVALID, "sd3_set_anchor_capture: null model");
    return m->anchors.set_capture(anchor, dst, m->cfg.depth, "sd3");
}

edb200_status_t edb200_sd3_set_stop_after(edb200_sd3_t* m, int block) {
    if (m == nullptr) return fail(EDB200_ERR_INVALID, "sd3_set_stop_after: null model");
    return m->anchors.set_stop(block, m->cfg.depth, "sd3");
}

edb200_status_t edb200_sd3_set_stream_override(edb200_sd3_t* m, const float* residual) {
    if (m == nullptr) return fail(EDB200_ERR_INVALID, "sd3_set_stream_override: null model");
    m->anchors.stream_override = residual;
    return EDB200_OK;
}

edb200_status_t edb200_sd3_set_region_inject(edb200_sd3_t* m, int at, int resume, const float* residual) {
    if (m == nullptr) return fail(EDB200_ERR_INVALID, "sd3_set_region_inject: null model");
    return m->anchors.set_region(at, resume, residual, m->cfg.depth, "sd3");
}

edb200_status_t edb200_sd3_set_tap(edb200_sd3_t* m, float* tap) {
    if (m == nullptr) return fail(EDB200_ERR_INVALID, "sd3_set_tap: null model");
    m->tap = tap;
    return EDB200_OK;
}

edb200_status_t edb200_sd3_prepare(edb200_sd3_t* m, int lat_h, int lat_w, int n_ctx, void* stream) {
    if (m == nullptr) return fail(EDB200_ERR_INVALID, "sd3_prepare: null model");
    const edb200_sd3_config_t& c = m->cfg;
    const int p = c.patch_size;
    if (lat_h <= 0 || lat_w <= 0 || n_ctx <= 0 || lat_h % p || lat_w % p || lat_h / p > c.pos_embed_max_size ||
        lat_w / p > c.pos_embed_max_size) {
        return fail(EDB200_ERR_INVALID, "sd3_prepare: latent must be a multiple of the patch size and fit the position table");
    }
    if (m->lat_h == lat_h && m->lat_w == lat_w && m->n_ctx == n_ctx) return EDB200_OK;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int64_t H = c.hidden_size, M = c.mlp_hidden;
    const int64_t n_img = (int64_t)(lat_h / p) * (lat_w / p), T = n_img + n_ctx;
    const int64_t pf_in = (int64_t)c.in_channels * p * p, pf_out = (int64_t)c.out_channels * p * p;
    const int64_t lat_in = (int64_t)c.in_channels * lat_h * lat_w, lat_out = (int64_t)c.out_channels * lat_h * lat_w;
    auto al = [](int64_t b) { return (b + 255) & ~int64_t(255); };
    int64_t t_loc = T, t_rows = T, ctx_l = n_ctx, img_first = 0;
    if (m->world > 1) {
        if (c.num_heads % m->world) {
            return fail(EDB200_ERR_UNSUPPORTED, "sd3_prepare: %d heads do not divide over %d ranks", c.num_heads, m->world);
        }
        EDB_TRY(edb200_sp_shard(T, n_ctx, m->rank, m->world, &t_loc, &ctx_l, &img_first, &t_rows));
        if (t_rows == 0) return fail(EDB200_ERR_UNSUPPORTED, "sd3_prepare: %lld tokens leave rank %d without rows", (long long)T, m->rank);
    }
    const int64_t sage = c.attention == EDB200_ATTN_SAGE_INT8
                             ? edb200_sage_scratch_bytes(c.num_heads / m->world, T, static_cast<int>(H / c.num_heads))
                             : 0;
    int64_t total = al(T * H * 4) + al(T * H * 2) + al(T * 3 * H * 2) + 4 * al(T * H * 2) + al(T * M * 2);
    total += al((mods_per_block(c) * c.depth + 2 * H) * 4) + al(H * 4) + al(2 * H * 4) + al(256 * 4) + al(128 * 4);
    total += al(n_img * pf_in * 4) + al(n_img * pf_out * 4) + al(lat_in * 4) + al(lat_out * 4) +
             al((int64_t)n_ctx * c.context_size * 4) + al(c.adm_in_channels * 4) + al(sage) + 8192;
    if (m->world > 1) total += 5 * al(t_loc * H * 2) + al(n_img * pf_out * 4) + 2048;
    cudaStreamSynchronize(s);
    if (m->comm != nullptr) EDB_TRY(edb200_comm_unmap_peers(m->comm));   // collective; the old workspace goes away
    m->p2p = false;
    EDB_TRY(m->ws.reserve(total));
    edb200_gemv_batch_destroy(m->mod_batch);   // it points into the old workspace: rebuilt at the next pass
    m->mod_batch = nullptr;
    Workspace& w = m->ws;
    m->X = w.take_n<float>(T * H);
    m->XMOD = w.take(T * H * 2);
    m->QKV = w.take(T * 3 * H * 2);
    m->Q = w.take(T * H * 2);
    m->K = w.take(T * H * 2);
    m->V = w.take(T * H * 2);
    m->ATT = w.take(T * H * 2);
    m->HID = w.take(T * M * 2);
    m->MODS = w.take_n<float>(mods_per_block(c) * c.depth + 2 * H);
    m->CVEC = w.take_n<float>(H);
    m->TMP = w.take_n<float>(2 * H);
    m->TEMB = w.take_n<float>(256);
    m->FREQ = w.take_n<float>(128);
    m->TOK_IN = w.take_n<float>(n_img * pf_in);
    m->TOK_OUT = w.take_n<float>(n_img * pf_out);
    m->LAT_IN = w.take_n<float>(lat_in);
    m->LAT_OUT = w.take_n<float>(lat_out);
    m->CTX_IN = w.take_n<float>((int64_t)n_ctx * c.context_size);
    m->Y_IN = w.take_n<float>(c.adm_in_channels);
    m->SAGE = sage > 0 ? w.take(sage) : nullptr;
    m->sage_bytes = sage;
    if (m->Y_IN == nullptr || (sage > 0 && m->SAGE == nullptr)) {
        return fail(EDB200_ERR_NOMEM, "sd3_prepare: workspace accounting error");
    }
    m->QL = m->KL = m->VL = m->AOUT = m->STG = nullptr;
    m->TOK_LOC = nullptr;
    if (m->world > 1) {
        void* flags = w.take(1024);   // barrier flags + epoch
        m->QL = w.take(t_loc * H * 2);
        m->KL = w.take(t_loc * H * 2);
        m->VL = w.take(t_loc * H * 2);
        m->AOUT = w.take(t_loc * H * 2);
        m->STG = w.take(t_loc * H * 2);
        m->TOK_LOC = w.take_n<float>(n_img * pf_out);
        if (flags == nullptr || m->TOK_LOC == nullptr) return fail(EDB200_ERR_NOMEM, "sd3_prepare: workspace accounting error");
        const char* how = getenv("EDB200_SP_EXCHANGE");
        const bool want_p2p = how == nullptr || strcmp(how, "nccl") != 0;
        edb200_status_t st = want_p2p ? edb200_comm_map_peers(m->comm, w.base(), w.capacity(),
                                                              static_cast<char*>(flags) - static_cast<char*>(w.base()), s)
                                      : EDB200_ERR_UNSUPPORTED;
        if (st == EDB200_OK) {
            m->p2p = true;
            memset(&m->qkv_peers, 0, sizeof(m->qkv_peers));
            memset(&m->att_peers, 0, sizeof(m->att_peers));
            m->qkv_peers.world = m->att_peers.world = m->world;
            m->qkv_peers.rank = m->att_peers.rank = m->rank;
            m->qkv_peers.t_loc = m->att_peers.t_loc = t_loc;
            for (int r = 0; r < m->world; ++r) {
                m->qkv_peers.buf[0][r] = edb200_comm_peer_ptr(m->comm, r, m->Q);
                m->qkv_peers.buf[1][r] = edb200_comm_peer_ptr(m->comm, r, m->K);
                m->qkv_peers.buf[2][r] = edb200_comm_peer_ptr(m->comm, r, m->V);
                m->att_peers.buf[0][r] = edb200_comm_peer_ptr(m->comm, r, m->ATT);
            }
        } else if (st != EDB200_ERR_UNSUPPORTED) {
            return st;
        }
    }
    m->t_loc = t_loc;
    m->t_rows = t_rows;
    m->ctx_l = ctx_l;
    m->img_l = t_rows - ctx_l;
    m->img_first = img_first;
    std::vector<float> freq(128);
    for (int i = 0; i < 128; ++i) freq[i] = (float)std::exp(-std::log(10000) * i / 128);
    cudaError_t e = cudaMemcpyAsync(m->FREQ, freq.data(), 128 * 4, cudaMemcpyHostToDevice, s);
    if (e == cudaSuccess) e = cudaStreamSynchronize(s);
    if (e != cudaSuccess) return check_cuda(e, "sd3_prepare upload");
    const int64_t need = (lat_in + lat_out + (int64_t)n_ctx * c.context_size + c.adm_in_channels) * 4;
    if (need > m->pinned_bytes) {
        if (m->pinned) cudaFreeHost(m->pinned);
        m->pinned = nullptr;
        e = cudaMallocHost(reinterpret_cast<void**>(&m->pinned), need);
        if (e != cudaSuccess) return fail(EDB200_ERR_NOMEM, "sd3_prepare: cudaMallocHost: %s", cudaGetErrorString(e));
        m->pinned_bytes = need;
    }
    m->lat_h = lat_h;
    m->lat_w = lat_w;
    m->n_ctx = n_ctx;
    m->n_img = static_cast<int>(n_img);
    return EDB200_OK;
}

static edb200_status_t sd3_step_body(edb200_sd3_t* m, const float* latent, float timestep, const float* sched,
                                     const int* sched_step, float t_scale, const float* context, const float* y, float* out,
                                     void* stream) {
    if (m == nullptr || latent == nullptr || context == nullptr || y == nullptr || out == nullptr) {
        return fail(EDB200_ERR_INVALID, "sd3_step: null argument");
    }
    if (m->lat_h == 0) return fail(EDB200_ERR_INVALID, "sd3_step: call edb200_sd3_prepare first");
    EDB_TRY(m->params.all_loaded());
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const edb200_sd3_config_t& c = m->cfg;
    const int64_t H = c.hidden_size, M = c.mlp_hidden;
    const int d = static_cast<int>(H / c.num_heads);
    const int p = c.patch_size;
    const int64_t T = (int64_t)m->n_ctx + m->n_img;            // whole sequence (attention length)
    const int64_t n_ctx = m->ctx_l, n_img = m->img_l;          // rows this rank owns
    const int64_t TL = m->t_rows;
    const bool sp = m->world > 1;
    const int64_t ctx_first = sp ? (int64_t)m->rank * m->t_loc : 0;
    // few output tiles per rank: let the long out-projection reductions be cut along k (unordered adds)
    const int split_k = sp ? EDB200_SPLIT_K_UNORDERED : EDB200_SPLIT_K_NEVER;
    // q / k / v packed head-major by the QKV projections' own epilogue (EDB200_FUSED_QK_PACK=0: separate pass)
    static int fused_env = -1;
    if (fused_env < 0) {
        const char* e = getenv("EDB200_FUSED_QK_PACK");
        fused_env = (e != nullptr && atoi(e) == 0) ? 0 : edb200_mul_mat_q_fuses_qk_pack();
    }
    const bool fused = fused_env == 1 && (d == 64 || d == 128) && (H % 128) == 0;
    const int64_t pf_in = (int64_t)c.in_channels * p * p, pf_out = (int64_t)c.out_channels * p * p;
    const int F16 = EDB200_TYPE_F16;
    float* X_ctx = m->X;
    float* X_img = m->X + n_ctx * H;
    __half* xmod = static_cast<__half*>(m->XMOD);
    __half* qkv = static_cast<__half*>(m->QKV);
    __half* att = static_cast<__half*>(m->ATT);
    __half* hid = static_cast<__half*>(m->HID);

    // ---- prelude (MMDiT::forward, mmdit.hpp:3409-3428)
    launch_patchify(latent, m->TOK_IN, c.in_channels, m->lat_h, m->lat_w, p, s);
    if (n_img > 0) {
        EDB_TRY(dense(m, "x_embedder.proj", m->TOK_IN + m->img_first * pf_in, n_img, pf_in, EDB200_ACT_NONE, X_img, H, s));
        const int h_tok = m->lat_h / p, w_tok = m->lat_w / p;
        const int top = (c.pos_embed_max_size - h_tok) / 2, left = (c.pos_embed_max_size - w_tok) / 2;
        const int64_t total = n_img * H;
        add_pos_embed_kernel<<<static_cast<unsigned>((total + 255) / 256), 256, 0, s>>>(
            X_img, fparam(m, "pos_embed"), static_cast<int>(H), w_tok, c.pos_embed_max_size, top, left, m->img_first, total);
        count_launch();
    }
    if (sched != nullptr) {
        launch_timestep_embedding_sched(m->FREQ, sched, sched_step, t_scale, 1.0f, 128, m->TEMB, s);
    } else {
        launch_timestep_embedding(m->FREQ, timestep, 1.0f, 128, m->TEMB, s);
    }
    EDB_TRY(dense(m, "t_embedder.mlp.0", m->TEMB, 1, 256, EDB200_ACT_SILU, m->TMP, H, s));
    EDB_TRY(dense(m, "t_embedder.mlp.2", m->TMP, 1, H, EDB200_ACT_NONE, m->CVEC, H, s));
    EDB_TRY(dense(m, "y_embedder.mlp.0", y, 1, c.adm_in_channels, EDB200_ACT_SILU, m->TMP, H, s));
    EDB_TRY(dense(m, "y_embedder.mlp.2", m->TMP, 1, H, EDB200_ACT_NONE, m->TMP + H, H, s));
    launch_add_inplace(m->CVEC, m->TMP + H, H, s);
    if (n_ctx > 0) {
        EDB_TRY(dense(m, "context_embedder", context + ctx_first * c.context_size, n_ctx, c.context_size, EDB200_ACT_NONE,
                      X_ctx, H, s));
    }

    // ---- every adaLN vector of the pass: lin(silu(c)), weight streaming, one launch for all of them
    // (sequence-parallel ranks with peer memory each stream 1/N of the weights and store to all)
    float* mods = m->MODS;
    float* fmods = mods + (int64_t)c.depth * 12 * H;
    EDB_TRY(ensure_mod_batch(m, s));
    EDB_TRY(edb200_gemv_batch_run(m->mod_batch, m->CVEC, 1, m->p2p ? &m->mods_peers : nullptr, s));
    if (m->p2p) EDB_TRY(edb200_sp_barrier(m->comm, s));

    m->anchors.capture_in(X_img, n_img * H, s);
    // ---- joint blocks (block_mixing, mmdit.hpp:2685-2775)
    for (int i = 0; i < (m->anchors.inject() ? 0 : c.depth); ++i) {
        if (m->anchors.region_inject(i, X_img, n_img * H, s)) continue;   // skip a cached span of blocks
        const std::string pc = "joint_blocks." + std::to_string(i) + ".context_block.";
        const std::string px = "joint_blocks." + std::to_string(i) + ".x_block.";
        const bool pre_only = i == c.depth - 1;
        const float* mc = mods + (int64_t)i * 12 * H;   // shift_msa scale_msa gate_msa shift_mlp scale_mlp gate_mlp
        const float* mx = mc + 6 * H;
        const float* c_shift = pre_only ? mc + H : mc;   // pre_only: (scale, shift)
        const float* c_scale = pre_only ? mc : mc + H;
        EDB_TRY(ln_mod(X_ctx, H, c_shift, c_scale, n_ctx, xmod, F16, s));
        EDB_TRY(ln_mod(X_img, H, mx, mx + H, n_img, xmod + n_ctx * H, F16, s));
        {
            const Lin lx = qlin(m, px + "attn.qkv"), lc = qlin(m, pc + "attn.qkv");
            edb200_epilogue_t ex = make_ep(qkv + n_ctx * 3 * H, F16, 3 * H, lx.b);
            edb200_epilogue_t ec = make_ep(qkv, F16, 3 * H, lc.b);
            // head-major pack of the local rows (no norm, no RoPE) by the projections' own epilogue
            edb200_qk_pack_t px_, pc_;
            memset(&px_, 0, sizeof(px_));
            px_.n_heads = c.num_heads;
            px_.d_head = d;
            px_.eps = 1e-6f;
            if (m->p2p) {
                px_.peers = &m->qkv_peers;
                px_.l_total = m->t_loc * m->world;
            } else {
                px_.l_total = sp ? m->t_loc : T;
                px_.q_out = sp ? m->QL : m->Q;
                px_.k_out = sp ? m->KL : m->K;
                px_.v_out = sp ? m->VL : m->V;
            }
            pc_ = px_;
            px_.tok_off = n_ctx;   // the context rows of this rank come first
            if (fused) ex.pack = &px_, ec.pack = &pc_;
            EDB_TRY(mm_pair(lx.w, xmod + n_ctx * H, n_img, H, &ex, lc.w, xmod, n_ctx, H, &ec, s));
        }
        // the same as a separate pass; under the peer-memory exchange straight into the owning ranks' Q/K/V
        if (fused) {
        } else if (m->p2p) {
            EDB_TRY(edb200_qk_norm_rope_pack_sp(qkv, F16, 3 * H, 0, H, 2 * H, TL, c.num_heads, d, nullptr, nullptr, 1e-6f,
                                                nullptr, 0, m->t_loc * m->world, &m->qkv_peers, F16, s));
        } else {
            EDB_TRY(edb200_qk_norm_rope_pack(qkv, F16, 3 * H, 0, H, 2 * H, TL, c.num_heads, d, nullptr, nullptr, 1e-6f,
                                             nullptr, 0, sp ? m->t_loc : T, sp ? m->QL : m->Q, sp ? m->KL : m->K,
                                             sp ? m->VL : m->V, F16, s));
        }
        EDB_TRY(joint_attention(m, i, T, s));
        {
            const Lin lx = qlin(m, px + "attn.proj");
            edb200_epilogue_t ex = make_ep(X_img, EDB200_TYPE_F32, H, lx.b);
            ex.residual = X_img, ex.ld_res = H, ex.gate = mx + 2 * H, ex.split_k = split_k;
            if (!pre_only) {
                const Lin lc = qlin(m, pc + "attn.proj");
                edb200_epilogue_t ec = make_ep(X_ctx, EDB200_TYPE_F32, H, lc.b);
                ec.residual = X_ctx, ec.ld_res = H, ec.gate = mc + 2 * H, ec.split_k = split_k;
                EDB_TRY(mm_pair(lx.w, att + n_ctx * H, n_img, H, &ex, lc.w, att, n_ctx, H, &ec, s));
            } else if (n_img > 0) {
                EDB_TRY(edb200_mul_mat_q(lx.w, att + n_ctx * H, F16, n_img, H, &ex, s));
            }
        }
        EDB_TRY(ln_mod(X_img, H, mx + 3 * H, mx + 4 * H, n_img, xmod + n_ctx * H, F16, s));
        if (!pre_only) EDB_TRY(ln_mod(X_ctx, H, mc + 3 * H, mc + 4 * H, n_ctx, xmod, F16, s));
        {
            const Lin l1 = qlin(m, px + "mlp.fc1"), l2 = qlin(m, px + "mlp.fc2");
            edb200_epilogue_t e1 = make_ep(hid + n_ctx * M, F16, M, l1.b);
            e1.act = EDB200_ACT_GELU_TANH;
            edb200_epilogue_t e2 = make_ep(X_img, EDB200_TYPE_F32, H, l2.b);
            e2.residual = X_img, e2.ld_res = H, e2.gate = mx + 5 * H, e2.split_k = split_k;
            if (!pre_only) {
                const Lin c1 = qlin(m, pc + "mlp.fc1"), c2 = qlin(m, pc + "mlp.fc2");
                edb200_epilogue_t f1 = make_ep(hid, F16, M, c1.b);
                f1.act = EDB200_ACT_GELU_TANH;
                edb200_epilogue_t f2 = make_ep(X_ctx, EDB200_TYPE_F32, H, c2.b);
                f2.residual = X_ctx, f2.ld_res = H, f2.gate = mc + 5 * H, f2.split_k = split_k;
                EDB_TRY(mm_pair(l1.w, xmod + n_ctx * H, n_img, H, &e1, c1.w, xmod, n_ctx, H, &f1, s));
                EDB_TRY(mm_pair(l2.w, hid + n_ctx * M, n_img, M, &e2, c2.w, hid, n_ctx, M, &f2, s));
            } else if (n_img > 0) {
                EDB_TRY(edb200_mul_mat_q(l1.w, xmod + n_ctx * H, F16, n_img, H, &e1, s));
                EDB_TRY(edb200_mul_mat_q(l2.w, hid + n_ctx * M, F16, n_img, M, &e2, s));
            }
        }
        if (m->tap) cudaMemcpyAsync(m->tap + (int64_t)i * TL * H, m->X, TL * H * 4, cudaMemcpyDeviceToDevice, s);
        m->anchors.capture_block(i, X_img, n_img * H, s);
        if (m->anchors.stop_after == i) return check_cuda(cudaGetLastError(), "sd3_step");
    }

    m->anchors.finish(X_img, n_img * H, s);   // whole-stack inject, ModelOut

    // ---- final layer: (scale, shift) order (FinalLayer::forward, mmdit.hpp:3143-3160) + unpatchify
    EDB_TRY(ln_mod(X_img, H, fmods + H, fmods, n_img, xmod, F16, s));
    if (n_img > 0) {
        const Lin lf = qlin(m, "final_layer.linear");
        edb200_epilogue_t ep = make_ep(sp ? m->TOK_LOC : m->TOK_OUT, EDB200_TYPE_F32, pf_out, lf.b);
        EDB_TRY(edb200_mul_mat_q(lf.w, xmod, F16, n_img, H, &ep, s));
    }
    if (sp) {
        std::vector<int64_t> first(m->world), count(m->world);
        for (int r = 0; r < m->world; ++r) {
            int64_t tx = 0, f = 0, rows = 0;
            EDB_TRY(edb200_sp_shard(T, m->n_ctx, r, m->world, nullptr, &tx, &f, &rows));
            first[r] = f;
            count[r] = rows - tx;
        }
        if (m->p2p) {
            // peer stores + barrier: nothing of the step goes through a library exchange
            EDB_TRY(edb200_sp_all_gather_rows_peer(m->comm, m->TOK_LOC, m->TOK_OUT, first.data(), count.data(), pf_out * 4, s));
        } else {
            EDB_TRY(edb200_sp_all_gather_rows(m->comm, m->TOK_LOC, m->TOK_OUT, first.data(), count.data(), pf_out * 4, s));
        }
    }
    {
        const int64_t total = (int64_t)c.out_channels * m->lat_h * m->lat_w;
        unpatchify_cf_kernel<<<static_cast<unsigned>((total + 255) / 256), 256, 0, s>>>(m->TOK_OUT, out, c.out_channels,
                                                                                        m->lat_h, m->lat_w, p);
        count_launch();
    }
    return check_cuda(cudaGetLastError(), "sd3_step");
}

edb200_status_t edb200_sd3_step(edb200_sd3_t* m, const float* latent, float timestep, const float* context,
                                const float* y, float* out, void* stream) {
    return sd3_step_body(m, latent, timestep, nullptr, nullptr, 1.0f, context, y, out, stream);
}

edb200_status_t edb200_sd3_step_sched(edb200_sd3_t* m, const float* latent, const float* sigmas, const int* step, float t_scale,
                                      const float* context, const float* y, float* out, void* stream) {
    if (sigmas == nullptr || step == nullptr) return fail(EDB200_ERR_INVALID, "sd3_step_sched: null schedule");
    return sd3_step_body(m, latent, 0.0f, sigmas, step, t_scale, context, y, out, stream);
}

edb200_status_t edb200_sd3_compute_host(edb200_sd3_t* m, const float* latent, int lat_h, int lat_w, float timestep,
                                        const float* context, int n_ctx, const float* y, float* out, void* stream) {
    if (m == nullptr || latent == nullptr || context == nullptr || y == nullptr || out == nullptr) {
        return fail(EDB200_ERR_INVALID, "sd3_compute_host: null argument");
    }
    EDB_TRY(edb200_sd3_prepare(m, lat_h, lat_w, n_ctx, stream));
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const edb200_sd3_config_t& c = m->cfg;
    const int64_t lat_in = (int64_t)c.in_channels * lat_h * lat_w, lat_out = (int64_t)c.out_channels * lat_h * lat_w;
    const int64_t ctx_elems = (int64_t)n_ctx * c.context_size;
    float* p_lat = m->pinned;
    float* p_ctx = p_lat + lat_in;
    float* p_y = p_ctx + ctx_elems;
    float* p_out = p_y + c.adm_in_channels;
    memcpy(p_lat, latent, lat_in * 4);
    memcpy(p_ctx, context, ctx_elems * 4);
    memcpy(p_y, y, (size_t)c.adm_in_channels * 4);
    cudaError_t e = cudaMemcpyAsync(m->LAT_IN, p_lat, lat_in * 4, cudaMemcpyHostToDevice, s);
    if (e == cudaSuccess) e = cudaMemcpyAsync(m->CTX_IN, p_ctx, ctx_elems * 4, cudaMemcpyHostToDevice, s);
    if (e == cudaSuccess) e = cudaMemcpyAsync(m->Y_IN, p_y, (size_t)c.adm_in_channels * 4, cudaMemcpyHostToDevice, s);
    if (e != cudaSuccess) return check_cuda(e, "sd3_compute_host H2D");
    EDB_TRY(edb200_sd3_step(m, m->LAT_IN, timestep, m->CTX_IN, m->Y_IN, m->LAT_OUT, stream));
    e = cudaMemcpyAsync(p_out, m->LAT_OUT, lat_out * 4, cudaMemcpyDeviceToHost, s);
    if (e != cudaSuccess) return check_cuda(e, "sd3_compute_host D2H");
    EDB_TRY(poll_device_error(s));   // synchronises the stream
    memcpy(out, p_out, lat_out * 4);
    return EDB200_OK;
}

}  // extern "C"
