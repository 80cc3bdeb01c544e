// Qwen-Image denoise-pass executor: the op schedule of QwenImageModel::forward_orig
// (reference src/dit_models/models/qwen_image.hpp:3116-3301, QwenImageTransformerBlock::forward
// :2825-2967, QwenImageAttention::forward :2276-2470, AdaLayerNormContinuous :3040-3070) on the
// kernels of this library.
//
// Text rows first, image rows after them, in every [T, ...] buffer.  With t = time embedding:
//   m_img, m_txt = mod.1(silu(t))                      weight-streaming GEMVs, all up front
//   XMOD = modulate(LN(stream), shift1, scale1)        both streams
//   Q|K|V = XMOD W{q,k,v} + b                          three two-problem GEMM launches into one [T, 3H] buffer
//   Q,K  = rope(RMSNorm_d(q) w), V -> head-major       pack kernel (per-head norm, text and image weights)
//   ATT  = attention over text + image                 INT8-QK or f16
//   stream += gate1 * (ATT Wout + b)                   two-problem GEMM, fused epilogue
//   stream += gate2 * net.2(gelu(net.0.proj(modulate(LN(stream), shift2, scale2))))
// The reference's 1/128 K/V pre-scale and 1/32, 1/128 linear pre-scales keep f16 accumulators in
// range and cancel exactly; accumulation here is f32, so they are not needed.
#include "edb200_model.h"

#include <cuda_fp16.h>

#include <cmath>
#include <cstdlib>
#include <cstring>
#include <vector>

using namespace edb;

struct edb200_qwen {
    edb200_qwen_config_t cfg;
    ParamTable params;
    Workspace ws;
    int lat_h = 0, lat_w = 0, n_txt = 0, n_img = 0;
    float* X = nullptr;   // [n_txt + n_img, H]
    void *XMOD = nullptr, *QKV = nullptr, *Q = nullptr, *K = nullptr, *V = nullptr, *ATT = nullptr, *HID = nullptr,
         *CTXN = nullptr;
    float *MODS = nullptr, *TVEC = nullptr, *TMP = nullptr, *TEMB = nullptr, *FREQ = nullptr, *PE = nullptr, *RSTD = nullptr,
          *TOK_IN = nullptr, *TOK_OUT = nullptr, *LAT_IN = nullptr, *LAT_OUT = nullptr, *CTX_IN = nullptr;
    void* SAGE = nullptr;
    int64_t sage_bytes = 0;
    float* tap = nullptr;
    ReuseAnchors anchors;   // computation-reuse seam (capture / probe stop / whole-stack inject)
    float* pinned = nullptr;
    int64_t pinned_bytes = 0;
    // sequence-parallel execution (world > 1): this rank's slice [text rows ; image rows] of the
    // [text ; image] sequence and the exchange buffers (see edb200_flux.cu for the scheme)
    edb200_comm_t* comm = nullptr;
    int rank = 0, world = 1;
    int64_t t_loc = 0, t_rows = 0, txt_l = 0, img_l = 0, img_first = 0;   // slot rows, owned rows, ...
    bool p2p = false;
    void *QL = nullptr, *KL = nullptr, *VL = nullptr, *AOUT = nullptr, *STG = nullptr;
    float* TOK_LOC = nullptr;
    edb200_sp_peers_t qkv_peers, att_peers;
    // all img_mod.1 / txt_mod.1 projections of a pass as one weight-streaming launch
    edb200_gemv_batch_t* mod_batch = nullptr;
    uint64_t mod_batch_gen = 0;
    edb200_sp_peers_t mods_peers;
};

namespace {

struct Lin {
    const edb200_qweight_t* w;
    const float* b;
};

int64_t hidden(const edb200_qwen_config_t& c) { return (int64_t)c.num_heads * c.head_dim; }

Lin qlin(edb200_qwen* m, const std::string& name) {
    Lin l;
    l.w = m->params.get(name + ".weight")->qw;
    l.b = m->params.get(name + ".bias")->f32;
    return l;
}

const float* fparam(edb200_qwen* m, const std::string& name) { return m->params.get(name)->f32; }

edb200_epilogue_t make_ep(void* out, int dt, int64_t ldo, const float* bias) {
    edb200_epilogue_t ep;
    memset(&ep, 0, sizeof(ep));
    ep.out = out;
    ep.out_dtype = dt;
    ep.ldo = ldo;
    ep.bias = bias;
    return ep;
}

void register_params(edb200_qwen* m) {
    const edb200_qwen_config_t& c = m->cfg;
    const int64_t H = hidden(c), M = c.mlp_hidden;
    ParamTable& t = m->params;
    // Quantised: 2-D weights whose row length is a multiple of 256, except the in-embedders `img_in.`
    // and `txt_in.` that tensor_should_be_converted excludes by name (reference
    // src/core/runtime/model_loader.cpp:2141-2172).  The modulation projections img_mod.1 / txt_mod.1
    // are floored at q8_0: a block type with fewer bits per weight is lifted (set_wtype_override, :1746-1761).
    auto lin = [&](const std::string& name, int64_t n_out, int64_t k) {
        const bool embedder = name.rfind("img_in", 0) == 0 || name.rfind("txt_in", 0) == 0;
        const bool mod = name.size() > 6 && name.compare(name.size() - 6, 6, "_mod.1") == 0;
        const int wt = (mod && c.wtype == EDB200_TYPE_Q4_K) ? EDB200_TYPE_Q8_0 : c.wtype;
        t.add(name + ".weight", n_out, k, k % 256 == 0 && !embedder, wt);
        t.add(name + ".bias", 1, n_out, false, c.wtype);
    };
    lin("time_text_embed.timestep_embedder.linear_1", H, 256);
    lin("time_text_embed.timestep_embedder.linear_2", H, H);
    t.add("txt_norm.weight", 1, c.joint_attention_dim, false, c.wtype);
    lin("img_in", H, c.in_channels);
    lin("txt_in", H, c.joint_attention_dim);
    for (int i = 0; i < c.num_layers; ++i) {
        const std::string p = "transformer_blocks." + std::to_string(i) + ".";
        lin(p + "img_mod.1", 6 * H, H);
        lin(p + "txt_mod.1", 6 * H, H);
        for (const char* l : {"to_q", "to_k", "to_v", "add_q_proj", "add_k_proj", "add_v_proj", "to_out.0", "to_add_out"}) {
            lin(p + "attn." + l, H, H);
        }
        for (const char* n : {"norm_q", "norm_k", "norm_added_q", "norm_added_k"}) {
            t.add(p + "attn." + n + ".weight", 1, c.head_dim, false, c.wtype);
        }
        for (const char* s : {"img_mlp", "txt_mlp"}) {
            lin(p + s + ".net.0.proj", M, H);
            lin(p + s + ".net.2", H, M);
        }
    }
    lin("norm_out.linear", 2 * H, H);
    lin("proj_out", (int64_t)c.patch_size * c.patch_size * c.out_channels, H);
}

// pe[L, d/2, 2, 2]: text ids (s, s, s) with s = max(h_tok/2, w_tok/2) + j first, then image ids
// (0, row - h_tok/2, col - w_tok/2) (gen_qwen_image_ids, reference
// src/dit_models/components/common/rope.hpp:405-438; gen_flux_img_ids with scale_rope :142-182).
std::vector<float> build_qwen_pe(const edb200_qwen_config_t& c, int h_tok, int w_tok, int n_txt) {
    const int L = n_txt + h_tok * w_tok;
    int half_total = 0;
    for (int a = 0; a < 3; ++a) half_total += c.axes_dim[a] / 2;
    std::vector<float> pe((size_t)L * half_total * 4, 0.0f);
    const int start = std::max(h_tok / 2, w_tok / 2);
    int off = 0;
    for (int a = 0; a < 3; ++a) {
        const int dim = c.axes_dim[a], half = dim / 2;
        std::vector<float> omega(half);
        const float end = (dim * 1.f - 2) / dim;
        const float step = half > 1 ? (end - 0.f) / (half - 1) : 0.f;
        for (int i = 0; i < half; ++i) omega[i] = 1.0f / ::powf(1.f * c.theta, 0.f + i * step);
        for (int t = 0; t < L; ++t) {
            float pos;
            if (t < n_txt) {
                pos = static_cast<float>(start + t);
            } else {
                const int it = t - n_txt;
                pos = a == 0 ? 0.0f : a == 1 ? static_cast<float>(it / w_tok - h_tok / 2) : static_cast<float>(it % w_tok - w_tok / 2);
            }
            for (int j = 0; j < half; ++j) {
                const float ang = pos * omega[j];
                float* o = &pe[((size_t)t * half_total + off + j) * 4];
                o[0] = std::cos(ang);
                o[1] = -std::sin(ang);
                o[2] = std::sin(ang);
                o[3] = std::cos(ang);
            }
        }
        off += half;
    }
    return pe;
}

// y[row, c] = (x[row, c] * rstd[row]) * w[c]   (txt_norm: RMSNorm over the whole context row, f32 like
// the f32 txt_in linear that reads it)
__global__ void rms_apply_kernel(const float* __restrict__ x, const float* __restrict__ rstd, const float* __restrict__ w,
                                 float* __restrict__ y, int cols, int64_t total) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    y[i] = (x[i] * rstd[i / cols]) * w[i % cols];
}

edb200_status_t ln_mod(const float* x, int64_t H, const float* shift, const float* scale, int64_t rows, void* y,
                       int y_dtype, cudaStream_t s) {
    if (rows == 0) return EDB200_OK;
    return edb200_layernorm_modulate(x, H, shift, scale, nullptr, nullptr, rows, H, 1e-6f, y, y_dtype, H, s);
}

// Row-count-tolerant two-problem GEMM: under sequence parallelism a rank may own no text rows.
edb200_status_t mm_pair(const edb200_qweight_t* w0, const void* x0, int64_t m0, int64_t ldx0, const edb200_epilogue_t* e0,
                        const edb200_qweight_t* w1, const void* x1, int64_t m1, int64_t ldx1, const edb200_epilogue_t* e1,
                        cudaStream_t s) {
    if (m0 > 0 && m1 > 0) return edb200_mul_mat_q_pair(w0, x0, m0, ldx0, e0, w1, x1, m1, ldx1, e1, EDB200_TYPE_F16, s);
    if (m0 > 0) return edb200_mul_mat_q(w0, x0, EDB200_TYPE_F16, m0, ldx0, e0, s);
    if (m1 > 0) return edb200_mul_mat_q(w1, x1, EDB200_TYPE_F16, m1, ldx1, e1, s);
    return EDB200_OK;
}

edb200_status_t qk_pack(edb200_qwen* m, const __half* qkv, int64_t rows, int64_t local_first, const float* qs,
                        const float* ks, cudaStream_t s) {
    if (rows == 0) return EDB200_OK;
    const edb200_qwen_config_t& c = m->cfg;
    const int64_t H = hidden(c);
    const int d = c.head_dim;
    const bool sp = m->world > 1;
    if (m->p2p) {
        return edb200_qk_norm_rope_pack_sp(qkv, EDB200_TYPE_F16, 3 * H, 0, H, 2 * H, rows, c.num_heads, d, qs, ks, 1e-6f,
                                           m->PE, local_first, m->t_loc * m->world, &m->qkv_peers, EDB200_TYPE_F16, s);
    }
    const float* pe = m->PE + (int64_t)m->rank * m->t_loc * (d / 2) * 4;   // position rows of this rank's tokens
    return edb200_qk_norm_rope_pack(qkv, EDB200_TYPE_F16, 3 * H, 0, H, 2 * H, rows, c.num_heads, d, qs, ks, 1e-6f, pe,
                                    local_first, m->t_loc, sp ? m->QL : m->Q, sp ? m->KL : m->K, sp ? m->VL : m->V,
                                    EDB200_TYPE_F16, s);
}

// Whether the q / k / v projections pack their output themselves (fused epilogue) instead of a separate pass.
bool fused_pack(const edb200_qwen* m) {
    static int on = -1;
    if (on < 0) {
        const char* e = getenv("EDB200_FUSED_QK_PACK");
        on = (e != nullptr && atoi(e) == 0) ? 0 : edb200_mul_mat_q_fuses_qk_pack();
    }
    return on == 1 && m->cfg.head_dim == 128;
}

// The destination of qk_pack() as a fused-epilogue description (same positions, same table rows).
edb200_qk_pack_t pack_desc(edb200_qwen* m, int64_t local_first, const float* qs, const float* ks) {
    const edb200_qwen_config_t& c = m->cfg;
    const int d = c.head_dim;
    const bool sp = m->world > 1;
    edb200_qk_pack_t k;
    memset(&k, 0, sizeof(k));
    k.n_heads = c.num_heads;
    k.d_head = d;
    k.q_weight = qs;
    k.k_weight = ks;
    k.eps = 1e-6f;
    k.pe = m->PE + (int64_t)m->rank * m->t_loc * (d / 2) * 4;
    k.tok_off = local_first;
    if (m->p2p) {
        k.peers = &m->qkv_peers;
        k.l_total = m->t_loc * m->world;
    } else {
        k.l_total = m->t_loc;
        k.q_out = sp ? m->QL : m->Q;
        k.k_out = sp ? m->KL : m->K;
        k.v_out = sp ? m->VL : m->V;
    }
    return k;
}

// Joint attention over the whole sequence into the local rows of ATT (single GPU, NCCL exchange,
// or peer-memory exchange with flag barriers; QwenImageTransformerBlock::forward_sp, qwen_image.hpp:2969-3040).
edb200_status_t joint_attention(edb200_qwen* m, int64_t T, cudaStream_t s) {
    const edb200_qwen_config_t& c = m->cfg;
    const int64_t H = hidden(c);
    const int d = c.head_dim;
    const int heads = c.num_heads / m->world;
    const float scale = 1.0f / std::sqrt(static_cast<float>(d));
    const int flags = (c.sage_smooth_q ? EDB200_SAGE_SMOOTH_Q : 0) | EDB200_SAGE_FAST_MEANS;
    const bool sage = c.attention == EDB200_ATTN_SAGE_INT8;
    // rows between heads in Q/K/V: the sequence padded to a multiple of the world size
    const int64_t head_rows = m->world > 1 ? m->t_loc * m->world : T;
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
    void* att_out = m->ATT;
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
        EDB_TRY(edb200_sp_all_to_all_tokens(m->comm, m->AOUT, m->STG, m->ATT, m->t_loc, (int64_t)heads * d * 2, H * 2, s));
    }
    return EDB200_OK;
}

// Every img_mod.1 / txt_mod.1 projection of the pass as one batch (block i: img 6H then txt 6H); built at the
// first pass after prepare or after a tensor was reloaded (it caches device addresses).
edb200_status_t ensure_mod_batch(edb200_qwen* m, cudaStream_t s) {
    if (m->mod_batch != nullptr && m->mod_batch_gen == m->params.generation()) return EDB200_OK;
    const edb200_qwen_config_t& c = m->cfg;
    const int64_t H = hidden(c);
    edb200_gemv_batch_destroy(m->mod_batch);
    m->mod_batch = nullptr;
    std::vector<const edb200_qweight_t*> bw;
    std::vector<const float*> bb;
    std::vector<float*> by;
    for (int i = 0; i < c.num_layers; ++i) {
        const std::string pb = "transformer_blocks." + std::to_string(i) + ".";
        const Lin li = qlin(m, pb + "img_mod.1"), lt = qlin(m, pb + "txt_mod.1");
        bw.push_back(li.w), bb.push_back(li.b), by.push_back(m->MODS + (int64_t)i * 12 * H);
        bw.push_back(lt.w), bb.push_back(lt.b), by.push_back(m->MODS + ((int64_t)i * 12 + 6) * H);
    }
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

edb200_status_t edb200_qwen_create(const edb200_qwen_config_t* cfg, edb200_qwen_t** out) {
    if (cfg == nullptr || out == nullptr) return fail(EDB200_ERR_INVALID, "qwen_create: null argument");
    const edb200_qwen_config_t& c = *cfg;
    if (c.num_heads <= 0 || c.num_layers <= 0 || (c.head_dim != 64 && c.head_dim != 128)) {
        return fail(EDB200_ERR_UNSUPPORTED, "qwen_create: head dim must be 64 or 128");
    }
    const int64_t H = hidden(c);
    if (c.axes_dim[0] + c.axes_dim[1] + c.axes_dim[2] != c.head_dim) {
        return fail(EDB200_ERR_INVALID, "qwen_create: axes_dim must sum to the head dim");
    }
    if (c.wtype != EDB200_TYPE_Q8_0 && c.wtype != EDB200_TYPE_Q4_K) {
        return fail(EDB200_ERR_UNSUPPORTED, "qwen_create: wtype must be q8_0 or q4_K");
    }
    if (H % 256 || c.mlp_hidden % 256 || H > 8192 || c.joint_attention_dim % 256) {
        return fail(EDB200_ERR_UNSUPPORTED, "qwen_create: hidden (<= 8192), mlp_hidden and joint_attention_dim must be multiples of 256");
    }
    if (c.attention == EDB200_ATTN_SAGE_INT8 && c.head_dim != 128) {
        return fail(EDB200_ERR_UNSUPPORTED, "qwen_create: INT8 attention needs head dim 128");
    }
    const int pf = c.patch_size * c.patch_size * c.out_channels;
    if (c.patch_size <= 0 || pf % 32 || c.in_channels % 4 || c.in_channels % (c.patch_size * c.patch_size)) {
        return fail(EDB200_ERR_UNSUPPORTED, "qwen_create: patch_size^2 * out_channels must be a multiple of 32");
    }
    if (device_error_word() == nullptr) return fail(EDB200_ERR_CUDA, "qwen_create: no CUDA device");
    edb200_qwen* m = new (std::nothrow) edb200_qwen();
    if (m == nullptr) return fail(EDB200_ERR_NOMEM, "qwen_create: host allocation failed");
    m->cfg = c;
    register_params(m);
    *out = m;
    return EDB200_OK;
}

void edb200_qwen_destroy(edb200_qwen_t* m) {
    if (m == nullptr) return;
    if (m->pinned) cudaFreeHost(m->pinned);
    edb200_gemv_batch_destroy(m->mod_batch);
    delete m;
}

int edb200_qwen_tensor_count(const edb200_qwen_t* m) {
    return m ? static_cast<int>(const_cast<edb200_qwen_t*>(m)->params.params().size()) : 0;
}

edb200_status_t edb200_qwen_tensor_info(const edb200_qwen_t* m, int index, char* name, int name_cap, int* ggml_type,
                                        int64_t* n_out, int64_t* k, int64_t* nbytes) {
    if (m == nullptr || index < 0 || index >= edb200_qwen_tensor_count(m)) {
        return fail(EDB200_ERR_INVALID, "qwen_tensor_info: bad index");
    }
    const Param& p = const_cast<edb200_qwen_t*>(m)->params.params()[index];
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

edb200_status_t edb200_qwen_set_tensor(edb200_qwen_t* m, const char* name, int ggml_type, const void* data,
                                       int64_t nbytes, int on_device, void* stream) {
    if (m == nullptr || name == nullptr) return fail(EDB200_ERR_INVALID, "qwen_set_tensor: null argument");
    return m->params.set(name, ggml_type, data, nbytes, on_device != 0, static_cast<cudaStream_t>(stream));
}

edb200_status_t edb200_qwen_get_tensor_f32(const edb200_qwen_t* m, const char* name, float* out, int64_t n_floats,
                                          int on_device, void* stream) {
    if (m == nullptr || name == nullptr) return fail(EDB200_ERR_INVALID, "qwen_get_tensor_f32: null argument");
    return m->params.fetch_f32(name, out, n_floats, on_device != 0, static_cast<cudaStream_t>(stream));
}

edb200_status_t edb200_qwen_load_gguf(edb200_qwen_t* m, const char* path, const char* strip_prefix, int* n_loaded,
                                    void* stream) {
    if (m == nullptr || path == nullptr) return fail(EDB200_ERR_INVALID, "qwen_load_gguf: null argument");
    return load_gguf(m->params, EDB200_FAMILY_QWEN, path, strip_prefix, static_cast<cudaStream_t>(stream), n_loaded);
}

edb200_status_t edb200_qwen_load_safetensors(edb200_qwen_t* m, const char* path, const char* strip_prefix, int* n_loaded,
                                           void* stream) {
    if (m == nullptr || path == nullptr) return fail(EDB200_ERR_INVALID, "qwen_load_safetensors: null argument");
    return load_safetensors(m->params, EDB200_FAMILY_QWEN, path, strip_prefix, static_cast<cudaStream_t>(stream), n_loaded);
}

edb200_status_t edb200_qwen_init_random(edb200_qwen_t* m, uint64_t seed, float std, void* stream) {
    if (m == nullptr) return fail(EDB200_ERR_INVALID, "qwen_init_random: null model");
    return m->params.init_random(seed, std, static_cast<cudaStream_t>(stream));
}

int64_t edb200_qwen_weight_bytes(const edb200_qwen_t* m) { return m ? m->params.device_bytes() : 0; }

edb200_status_t edb200_qwen_set_comm(edb200_qwen_t* m, edb200_comm_t* comm) {
    if (m == nullptr) return fail(EDB200_ERR_INVALID, "qwen_set_comm: null model");
    if (m->comm != nullptr && m->comm != comm) edb200_comm_unmap_peers(m->comm);   // collective
    m->comm = comm;
    m->rank = comm ? edb200_comm_rank(comm) : 0;
    m->world = comm ? edb200_comm_world(comm) : 1;
    m->lat_h = m->lat_w = m->n_txt = 0;   // the workspace must be prepared again
    m->p2p = false;
    return EDB200_OK;
}

edb200_status_t edb200_qwen_set_anchor_capture(edb200_qwen_t* m, int anchor, float* dst) {
    if (m == nullptr) return fail(EDB200_ERR_INVALID, "qwen_set_anchor_capture: null model");
    return m->anchors.set_capture(anchor, dst, m->cfg.num_layers, "qwen");
}

edb200_status_t edb200_qwen_set_stop_after(edb200_qwen_t* m, int block) {
    if (m == nullptr) return fail(EDB200_ERR_INVALID, "qwen_set_stop_after: null model");
    return m->anchors.set_stop(block, m->cfg.num_layers, "qwen");
}

edb200_status_t edb200_qwen_set_stream_override(edb200_qwen_t* m, const float* residual) {
    if (m == nullptr) return fail(EDB200_ERR_INVALID, "qwen_set_stream_override: null model");
    m->anchors.stream_override = residual;
    return EDB200_OK;
}

edb200_status_t edb200_qwen_set_tap(edb200_qwen_t* m, float* tap) {
    if (m == nullptr) return fail(EDB200_ERR_INVALID, "qwen_set_tap: null model");
    m->tap = tap;
    return EDB200_OK;
}

edb200_status_t edb200_qwen_prepare(edb200_qwen_t* m, int lat_h, int lat_w, int n_txt, void* stream) {
    if (m == nullptr) return fail(EDB200_ERR_INVALID, "qwen_prepare: null model");
    const edb200_qwen_config_t& c = m->cfg;
    const int p = c.patch_size;
    if (lat_h <= 0 || lat_w <= 0 || n_txt <= 0 || lat_h % p || lat_w % p) {
        return fail(EDB200_ERR_INVALID, "qwen_prepare: latent must be a positive multiple of the patch size");
    }
    if (m->lat_h == lat_h && m->lat_w == lat_w && m->n_txt == n_txt) return EDB200_OK;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int64_t H = hidden(c), M = c.mlp_hidden, d = c.head_dim;
    const int h_tok = lat_h / p, w_tok = lat_w / p;
    const int64_t n_img = (int64_t)h_tok * w_tok, T = n_img + n_txt;
    const int lat_c = c.in_channels / (p * p);
    const int64_t pf_out = (int64_t)c.out_channels * p * p;
    const int64_t lat_in = (int64_t)lat_c * lat_h * lat_w, lat_out = (int64_t)c.out_channels * lat_h * lat_w;
    int64_t t_loc = T, t_rows = T, txt_l = n_txt, img_first = 0;
    if (m->world > 1) {
        if (c.num_heads % m->world) {
            return fail(EDB200_ERR_UNSUPPORTED, "qwen_prepare: %d heads do not divide over %d ranks", c.num_heads, m->world);
        }
        EDB_TRY(edb200_sp_shard(T, n_txt, m->rank, m->world, &t_loc, &txt_l, &img_first, &t_rows));
        if (t_rows == 0) return fail(EDB200_ERR_UNSUPPORTED, "qwen_prepare: %lld tokens leave rank %d without rows", (long long)T, m->rank);
    }
    const int64_t sage =
        c.attention == EDB200_ATTN_SAGE_INT8 ? edb200_sage_scratch_bytes(c.num_heads / m->world, T, (int)d) : 0;
    const int64_t pe_elems = T * (d / 2) * 4;
    auto al = [](int64_t b) { return (b + 255) & ~int64_t(255); };
    int64_t total = al(T * H * 4) + al(T * H * 2) + al(T * 3 * H * 2) + 4 * al(T * H * 2) + al(T * M * 2);
    total += al(((int64_t)12 * c.num_layers + 2) * H * 4) + al(H * 4) + al(H * 4) + al(256 * 4) + al(128 * 4) + al(pe_elems * 4);
    total += al((int64_t)n_txt * c.joint_attention_dim * 4) + al(n_txt * 4) + al(n_img * c.in_channels * 4) +
             al(n_img * pf_out * 4) + al(lat_in * 4) + al(lat_out * 4) + al((int64_t)n_txt * c.joint_attention_dim * 4) +
             al(sage) + 8192;
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
    m->MODS = w.take_n<float>(((int64_t)12 * c.num_layers + 2) * H);
    m->TVEC = w.take_n<float>(H);
    m->TMP = w.take_n<float>(H);
    m->TEMB = w.take_n<float>(256);
    m->FREQ = w.take_n<float>(128);
    m->PE = w.take_n<float>(pe_elems);
    m->CTXN = w.take((int64_t)n_txt * c.joint_attention_dim * 4);
    m->RSTD = w.take_n<float>(n_txt);
    m->TOK_IN = w.take_n<float>(n_img * c.in_channels);
    m->TOK_OUT = w.take_n<float>(n_img * pf_out);
    m->LAT_IN = w.take_n<float>(lat_in);
    m->LAT_OUT = w.take_n<float>(lat_out);
    m->CTX_IN = w.take_n<float>((int64_t)n_txt * c.joint_attention_dim);
    m->SAGE = sage > 0 ? w.take(sage) : nullptr;
    m->sage_bytes = sage;
    if (m->CTX_IN == nullptr || (sage > 0 && m->SAGE == nullptr)) {
        return fail(EDB200_ERR_NOMEM, "qwen_prepare: workspace accounting error");
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
        if (flags == nullptr || m->TOK_LOC == nullptr) return fail(EDB200_ERR_NOMEM, "qwen_prepare: workspace accounting error");
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
    m->txt_l = txt_l;
    m->img_l = t_rows - txt_l;
    m->img_first = img_first;
    std::vector<float> pe = build_qwen_pe(c, h_tok, w_tok, n_txt);
    std::vector<float> freq(128);
    for (int i = 0; i < 128; ++i) freq[i] = (float)std::exp(-std::log(10000) * i / 128);
    cudaError_t e = cudaMemcpyAsync(m->PE, pe.data(), pe.size() * 4, cudaMemcpyHostToDevice, s);
    if (e == cudaSuccess) e = cudaMemcpyAsync(m->FREQ, freq.data(), 128 * 4, cudaMemcpyHostToDevice, s);
    if (e == cudaSuccess) e = cudaStreamSynchronize(s);
    if (e != cudaSuccess) return check_cuda(e, "qwen_prepare upload");
    const int64_t need = (lat_in + lat_out + (int64_t)n_txt * c.joint_attention_dim) * 4;
    if (need > m->pinned_bytes) {
        if (m->pinned) cudaFreeHost(m->pinned);
        m->pinned = nullptr;
        e = cudaMallocHost(reinterpret_cast<void**>(&m->pinned), need);
        if (e != cudaSuccess) return fail(EDB200_ERR_NOMEM, "qwen_prepare: cudaMallocHost: %s", cudaGetErrorString(e));
        m->pinned_bytes = need;
    }
    m->lat_h = lat_h;
    m->lat_w = lat_w;
    m->n_txt = n_txt;
    m->n_img = static_cast<int>(n_img);
    return EDB200_OK;
}

static edb200_status_t qwen_step_body(edb200_qwen_t* m, const float* latent, float timestep, const float* sched,
                                      const int* sched_step, float t_scale, const float* context, float* out, void* stream) {
    if (m == nullptr || latent == nullptr || context == nullptr || out == nullptr) {
        return fail(EDB200_ERR_INVALID, "qwen_step: null argument");
    }
    if (m->lat_h == 0) return fail(EDB200_ERR_INVALID, "qwen_step: call edb200_qwen_prepare first");
    EDB_TRY(m->params.all_loaded());
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const edb200_qwen_config_t& c = m->cfg;
    const int64_t H = hidden(c), M = c.mlp_hidden;
    const int p = c.patch_size;
    const int64_t T = (int64_t)m->n_txt + m->n_img;            // whole sequence (attention length)
    const int64_t n_txt = m->txt_l, n_img = m->img_l;          // rows this rank owns
    const int64_t txt_first = m->world > 1 ? (int64_t)m->rank * m->t_loc : 0;
    const bool sp = m->world > 1;
    // few output tiles per rank: let the long out-projection reductions be cut along k (unordered adds)
    const int split_k = sp ? EDB200_SPLIT_K_UNORDERED : EDB200_SPLIT_K_NEVER;
    const bool fused = fused_pack(m);   // q / k / v packed by their projections' own epilogue
    const int lat_c = c.in_channels / (p * p);
    const int64_t pf_out = (int64_t)c.out_channels * p * p;
    const int F16 = EDB200_TYPE_F16;
    float* X_txt = m->X;
    float* X_img = m->X + n_txt * H;
    __half* xmod = static_cast<__half*>(m->XMOD);
    __half* qkv = static_cast<__half*>(m->QKV);
    __half* att = static_cast<__half*>(m->ATT);
    __half* hid = static_cast<__half*>(m->HID);

    // ---- prelude (forward_orig, qwen_image.hpp:3131-3160)
    launch_patchify(latent, m->TOK_IN, lat_c, m->lat_h, m->lat_w, p, s);
    {
        const Param* w = m->params.get("img_in.weight");
        if (n_img > 0) {
            EDB_TRY(edb200_linear_f32(w->f32, fparam(m, "img_in.bias"), m->TOK_IN + m->img_first * c.in_channels, n_img,
                                      c.in_channels, H, c.in_channels, 0, EDB200_ACT_NONE, X_img, H, s));
        }
    }
    if (n_txt > 0) {
        const float* ctx_l = context + txt_first * c.joint_attention_dim;
        EDB_TRY(edb200_row_rstd(ctx_l, EDB200_TYPE_F32, c.joint_attention_dim, n_txt, c.joint_attention_dim, 1e-6f, m->RSTD, s));
        const int64_t total = n_txt * c.joint_attention_dim;
        rms_apply_kernel<<<static_cast<unsigned>((total + 255) / 256), 256, 0, s>>>(
            ctx_l, m->RSTD, fparam(m, "txt_norm.weight"), static_cast<float*>(m->CTXN), c.joint_attention_dim, total);
        count_launch();
        EDB_TRY(edb200_linear_f32(m->params.get("txt_in.weight")->f32, fparam(m, "txt_in.bias"),
                                  static_cast<const float*>(m->CTXN), n_txt, c.joint_attention_dim, H,
                                  c.joint_attention_dim, 0, EDB200_ACT_NONE, X_txt, H, s));
    }
    if (sched != nullptr) {
        launch_timestep_embedding_sched(m->FREQ, sched, sched_step, t_scale, 1.0f, 128, m->TEMB, s);
    } else {
        launch_timestep_embedding(m->FREQ, timestep, 1.0f, 128, m->TEMB, s);
    }
    {
        const Lin l1 = qlin(m, "time_text_embed.timestep_embedder.linear_1");
        const Lin l2 = qlin(m, "time_text_embed.timestep_embedder.linear_2");
        EDB_TRY(edb200_gemv_q(l1.w, m->TEMB, 1, 256, 0, l1.b, m->TMP, H, s));
        EDB_TRY(edb200_gemv_q(l2.w, m->TMP, 1, H, 1, l2.b, m->TVEC, H, s));   // SiLU between the two
    }

    // ---- every adaLN vector of the pass: mod.1(silu(t)), weight streaming, one launch for all of them
    // (sequence-parallel ranks with peer memory each stream 1/N of the weights and store to all)
    float* mods = m->MODS;
    EDB_TRY(ensure_mod_batch(m, s));
    EDB_TRY(edb200_gemv_batch_run(m->mod_batch, m->TVEC, 1, m->p2p ? &m->mods_peers : nullptr, s));
    if (m->p2p) EDB_TRY(edb200_sp_barrier(m->comm, s));
    float* fmods = mods + (int64_t)c.num_layers * 12 * H;
    {
        const Lin lf = qlin(m, "norm_out.linear");
        EDB_TRY(edb200_gemv_q(lf.w, m->TVEC, 1, H, 1, lf.b, fmods, 2 * H, s));
    }

    m->anchors.capture_in(X_img, n_img * H, s);
    // ---- blocks (QwenImageTransformerBlock::forward, qwen_image.hpp:2825-2967)
    for (int i = 0; i < (m->anchors.inject() ? 0 : c.num_layers); ++i) {
        const std::string pb = "transformer_blocks." + std::to_string(i) + ".";
        const std::string pa = pb + "attn.";
        const float* im = mods + (int64_t)i * 12 * H;   // shift1 scale1 gate1 shift2 scale2 gate2
        const float* tm = im + 6 * H;
        EDB_TRY(ln_mod(X_img, H, im, im + H, n_img, xmod + n_txt * H, F16, s));
        EDB_TRY(ln_mod(X_txt, H, tm, tm + H, n_txt, xmod, F16, s));
        {
            const char* img_names[3] = {"to_q", "to_k", "to_v"};
            const char* txt_names[3] = {"add_q_proj", "add_k_proj", "add_v_proj"};
            const float* iq = fparam(m, pa + "norm_q.weight");
            const float* ik = fparam(m, pa + "norm_k.weight");
            const float* tq = fparam(m, pa + "norm_added_q.weight");
            const float* tk = fparam(m, pa + "norm_added_k.weight");
            for (int j = 0; j < 3; ++j) {
                const Lin li = qlin(m, pa + img_names[j]), lt = qlin(m, pa + txt_names[j]);
                edb200_epilogue_t ei = make_ep(qkv + n_txt * 3 * H + j * H, F16, 3 * H, li.b);
                edb200_epilogue_t et = make_ep(qkv + j * H, F16, 3 * H, lt.b);
                // each projection's epilogue packs its own tensor head-major (norm and RoPE for q and k)
                edb200_qk_pack_t pi = pack_desc(m, n_txt, iq, ik), pt = pack_desc(m, 0, tq, tk);
                pi.only = pt.only = j + 1;
                if (fused) ei.pack = &pi, et.pack = &pt;
                EDB_TRY(mm_pair(li.w, xmod + n_txt * H, n_img, H, &ei, lt.w, xmod, n_txt, H, &et, s));
            }
            if (!fused) {
                EDB_TRY(qk_pack(m, qkv + n_txt * 3 * H, n_img, n_txt, iq, ik, s));
                EDB_TRY(qk_pack(m, qkv, n_txt, 0, tq, tk, s));
            }
        }
        EDB_TRY(joint_attention(m, T, s));
        {
            const Lin li = qlin(m, pa + "to_out.0"), lt = qlin(m, pa + "to_add_out");
            edb200_epilogue_t ei = make_ep(X_img, EDB200_TYPE_F32, H, li.b);
            ei.residual = X_img, ei.ld_res = H, ei.gate = im + 2 * H, ei.split_k = split_k;
            edb200_epilogue_t et = make_ep(X_txt, EDB200_TYPE_F32, H, lt.b);
            et.residual = X_txt, et.ld_res = H, et.gate = tm + 2 * H, et.split_k = split_k;
            EDB_TRY(mm_pair(li.w, att + n_txt * H, n_img, H, &ei, lt.w, att, n_txt, H, &et, s));
        }
        EDB_TRY(ln_mod(X_img, H, im + 3 * H, im + 4 * H, n_img, xmod + n_txt * H, F16, s));
        EDB_TRY(ln_mod(X_txt, H, tm + 3 * H, tm + 4 * H, n_txt, xmod, F16, s));
        {
            const Lin i0 = qlin(m, pb + "img_mlp.net.0.proj"), t0 = qlin(m, pb + "txt_mlp.net.0.proj");
            edb200_epilogue_t ei = make_ep(hid + n_txt * M, F16, M, i0.b);
            ei.act = EDB200_ACT_GELU_TANH;
            edb200_epilogue_t et = make_ep(hid, F16, M, t0.b);
            et.act = EDB200_ACT_GELU_TANH;
            EDB_TRY(mm_pair(i0.w, xmod + n_txt * H, n_img, H, &ei, t0.w, xmod, n_txt, H, &et, s));
            const Lin i2 = qlin(m, pb + "img_mlp.net.2"), t2 = qlin(m, pb + "txt_mlp.net.2");
            edb200_epilogue_t fi = make_ep(X_img, EDB200_TYPE_F32, H, i2.b);
            fi.residual = X_img, fi.ld_res = H, fi.gate = im + 5 * H, fi.split_k = split_k;
            edb200_epilogue_t ft = make_ep(X_txt, EDB200_TYPE_F32, H, t2.b);
            ft.residual = X_txt, ft.ld_res = H, ft.gate = tm + 5 * H, ft.split_k = split_k;
            EDB_TRY(mm_pair(i2.w, hid + n_txt * M, n_img, M, &fi, t2.w, hid, n_txt, M, &ft, s));
        }
        if (m->tap) {
            cudaMemcpyAsync(m->tap + (int64_t)i * m->t_rows * H, m->X, m->t_rows * H * 4, cudaMemcpyDeviceToDevice, s);
        }
        m->anchors.capture_block(i, X_img, n_img * H, s);
        if (m->anchors.stop_after == i) return check_cuda(cudaGetLastError(), "qwen_step");
    }

    m->anchors.finish(X_img, n_img * H, s);   // whole-stack inject, ModelOut

    // ---- norm_out: (scale, shift) order (AdaLayerNormContinuous, qwen_image.hpp:3062-3068), proj_out, unpatchify
    EDB_TRY(ln_mod(X_img, H, fmods + H, fmods, n_img, xmod, F16, s));
    if (n_img > 0) {
        const Lin lf = qlin(m, "proj_out");
        edb200_epilogue_t ep = make_ep(sp ? m->TOK_LOC : m->TOK_OUT, EDB200_TYPE_F32, pf_out, lf.b);
        EDB_TRY(edb200_mul_mat_q(lf.w, xmod, F16, n_img, H, &ep, s));
    }
    if (sp) {
        std::vector<int64_t> first(m->world), count(m->world);
        for (int r = 0; r < m->world; ++r) {
            int64_t tx = 0, f = 0, rows = 0;
            EDB_TRY(edb200_sp_shard(T, m->n_txt, r, m->world, nullptr, &tx, &f, &rows));
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
    launch_unpatchify(m->TOK_OUT, out, c.out_channels, m->lat_h, m->lat_w, p, s);
    return check_cuda(cudaGetLastError(), "qwen_step");
}

edb200_status_t edb200_qwen_step(edb200_qwen_t* m, const float* latent, float timestep, const float* context, float* out,
                                 void* stream) {
    return qwen_step_body(m, latent, timestep, nullptr, nullptr, 1.0f, context, out, stream);
}

edb200_status_t edb200_qwen_step_sched(edb200_qwen_t* m, const float* latent, const float* sigmas, const int* step, float t_scale,
                                       const float* context, float* out, void* stream) {
    if (sigmas == nullptr || step == nullptr) return fail(EDB200_ERR_INVALID, "qwen_step_sched: null schedule");
    return qwen_step_body(m, latent, 0.0f, sigmas, step, t_scale, context, out, stream);
}

edb200_status_t edb200_qwen_compute_host(edb200_qwen_t* m, const float* latent, int lat_h, int lat_w, float timestep,
                                         const float* context, int n_txt, float* out, void* stream) {
    if (m == nullptr || latent == nullptr || context == nullptr || out == nullptr) {
        return fail(EDB200_ERR_INVALID, "qwen_compute_host: null argument");
    }
    EDB_TRY(edb200_qwen_prepare(m, lat_h, lat_w, n_txt, stream));
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const edb200_qwen_config_t& c = m->cfg;
    const int lat_c = c.in_channels / (c.patch_size * c.patch_size);
    const int64_t lat_in = (int64_t)lat_c * lat_h * lat_w, lat_out = (int64_t)c.out_channels * lat_h * lat_w;
    const int64_t ctx_elems = (int64_t)n_txt * c.joint_attention_dim;
    float* p_lat = m->pinned;
    float* p_ctx = p_lat + lat_in;
    float* p_out = p_ctx + ctx_elems;
    memcpy(p_lat, latent, lat_in * 4);
    memcpy(p_ctx, context, ctx_elems * 4);
    cudaError_t e = cudaMemcpyAsync(m->LAT_IN, p_lat, lat_in * 4, cudaMemcpyHostToDevice, s);
    if (e == cudaSuccess) e = cudaMemcpyAsync(m->CTX_IN, p_ctx, ctx_elems * 4, cudaMemcpyHostToDevice, s);
    if (e != cudaSuccess) return check_cuda(e, "qwen_compute_host H2D");
    EDB_TRY(edb200_qwen_step(m, m->LAT_IN, timestep, m->CTX_IN, m->LAT_OUT, stream));
    e = cudaMemcpyAsync(p_out, m->LAT_OUT, lat_out * 4, cudaMemcpyDeviceToHost, s);
    if (e != cudaSuccess) return check_cuda(e, "qwen_compute_host D2H");
    EDB_TRY(poll_device_error(s));   // synchronises the stream
    memcpy(out, p_out, lat_out * 4);
    return EDB200_OK;
}

}  // extern "C"
