// FLUX.1 denoise-step executor: a fixed op schedule (no graph interpreter) over
// device-resident activations.  Mirrors the reference graph
// (src/dit_models/models/flux.hpp): Flux::forward_orig :3872-4527,
// DoubleStreamBlock::forward :1747-1925, SingleStreamBlock::forward :2974-3034,
// LastLayer::forward :3533-3559, Modulation::forward :1617-1634, and the runner
// seam FluxRunner::compute :5158-5296 (host tensors in, host tensor out).
//
// Data layout in HBM for one step (T = T_txt + T_img, text rows first):
//   X      f32 [T, H]        residual stream, both streams in one buffer so the
//                            single-stream stack needs no concat
//   XMOD   f16 [T, H]        LayerNorm+modulate output = GEMM operand
//   QKV    f16 [T, 3H]       QKV projection output
//   Q,K,V  f16 [heads, T, d] head-major attention operands (RoPE'd, RMS-normed)
//   CAT    f16 [T, H + M]    [attention | GELU(mlp)] = linear2 operand of single
//                            blocks; double blocks use its first H columns and HID
//   HID    f16 [T, M]        GELU(mlp.0) of double blocks
//   MODS   f32               every adaLN shift/scale/gate vector of the step
#include "edb200_model.h"

#include <cuda_fp16.h>
#include <cmath>
#include <cstdlib>
#include <cstring>
#include <vector>

using namespace edb;

struct edb200_flux {
    edb200_flux_config_t cfg;
    ParamTable params;
    Workspace ws;
    // shape the workspace was prepared for
    int lat_h = 0, lat_w = 0, n_txt = 0, n_img = 0;
    // activations
    float* X = nullptr;
    void *XMOD = nullptr, *QKV = nullptr, *Q = nullptr, *K = nullptr, *V = nullptr, *CAT = nullptr, *HID = nullptr;
    float *MODS = nullptr, *VEC = nullptr, *TMP_H = nullptr, *TEMB = nullptr, *TOK_IN = nullptr, *TOK_OUT = nullptr;
    float *FIN = nullptr, *PE = nullptr, *FREQ = nullptr, *LAT_IN = nullptr, *LAT_OUT = nullptr, *CTX = nullptr,
          *YVEC = nullptr;
    void* SAGE = nullptr;
    int64_t sage_bytes = 0;
    // sequence-parallel execution (world > 1): this rank's token slice and exchange buffers
    edb200_comm_t* comm = nullptr;
    int rank = 0, world = 1;
    int64_t t_loc = 0, t_rows = 0, txt_l = 0, img_l = 0, img_first = 0;   // slot rows, owned rows, ...
    void *QL = nullptr, *KL = nullptr, *VL = nullptr, *AOUT = nullptr, *STG = nullptr;
    float* TOK_LOC = nullptr;
    // peer-memory exchange: producers store into the owning rank's buffers, flag barriers order them
    bool p2p = false;
    edb200_sp_peers_t qkv_peers, cat_peers;
    // all adaLN projections of a step as one weight-streaming launch (built in prepare)
    edb200_gemv_batch_t* mod_batch = nullptr;
    uint64_t mod_batch_gen = 0;
    edb200_sp_peers_t mods_peers;
    float* tap = nullptr;
    // computation-reuse seam: captures of the image stream at the anchors, probe stop, whole-stack inject
    float* anchor_in = nullptr;
    float* anchor_out = nullptr;
    std::vector<float*> anchor_block;   // [depth], NULL = not captured
    int stop_after = -1;
    const float* stream_override = nullptr;
    // host staging for compute_host
    float* pinned = nullptr;
    int64_t pinned_bytes = 0;
};

namespace {

int64_t mods_per_step(const edb200_flux_config_t& c) {
    return (int64_t)c.hidden_size * (12 * c.depth + 3 * c.depth_single_blocks + 2);
}

void register_params(edb200_flux* m) {
    const edb200_flux_config_t& c = m->cfg;
    const int64_t H = c.hidden_size, M = c.mlp_hidden, d = H / c.num_heads;
    ParamTable& t = m->params;
    auto lin = [&](const std::string& name, int64_t n_out, int64_t k, bool q) {
        t.add(name + ".weight", n_out, k, q, c.wtype);
        t.add(name + ".bias", 1, n_out, false, c.wtype);
    };
    // Which tensors are quantised follows tensor_should_be_converted
    // (reference src/core/runtime/model_loader.cpp:2141-2172): the in/out
    // embedders and final_layer stay f32.
    lin("img_in", H, c.in_channels, false);
    lin("txt_in", H, c.context_in_dim, false);
    lin("time_in.in_layer", H, 256, false);
    lin("time_in.out_layer", H, H, false);
    if (c.guidance_embed) {
        lin("guidance_in.in_layer", H, 256, false);
        lin("guidance_in.out_layer", H, H, false);
    }
    lin("vector_in.in_layer", H, c.vec_in_dim, false);
    lin("vector_in.out_layer", H, H, false);
    for (int i = 0; i < c.depth; ++i) {
        const std::string p = "double_blocks." + std::to_string(i) + ".";
        for (const char* s : {"img", "txt"}) {
            const std::string sp = p + s;
            lin(sp + "_mod.lin", 6 * H, H, true);
            lin(sp + "_attn.qkv", 3 * H, H, true);
            t.add(sp + "_attn.norm.query_norm.scale", 1, d, false, c.wtype);
            t.add(sp + "_attn.norm.key_norm.scale", 1, d, false, c.wtype);
            lin(sp + "_attn.proj", H, H, true);
            lin(sp + "_mlp.0", M, H, true);
            lin(sp + "_mlp.2", H, M, true);
        }
    }
    for (int i = 0; i < c.depth_single_blocks; ++i) {
        const std::string p = "single_blocks." + std::to_string(i) + ".";
        lin(p + "modulation.lin", 3 * H, H, true);
        lin(p + "linear1", 3 * H + M, H, true);
        lin(p + "linear2", H, H + M, true);
        t.add(p + "norm.query_norm.scale", 1, d, false, c.wtype);
        t.add(p + "norm.key_norm.scale", 1, d, false, c.wtype);
    }
    lin("final_layer.adaLN_modulation.1", 2 * H, H, false);
    lin("final_layer.linear", c.in_channels, H, false);
}

// pe[L, d/2, 2, 2] = [[cos, -sin], [sin, cos]] per (token, pair); text tokens
// first with all-zero ids, image token ids (0, row, col).  Follows
// Rope::rope / embed_nd / gen_flux_ids (reference
// src/dit_models/components/common/rope.hpp:77-127,201-260,130-199).
std::vector<float> build_flux_pe(const edb200_flux_config_t& c, int h_tok, int w_tok, int n_txt) {
    const int L = n_txt + h_tok * w_tok;
    int half_total = 0;
    for (int a = 0; a < 3; ++a) half_total += c.axes_dim[a] / 2;
    std::vector<float> pe((size_t)L * half_total * 4, 0.0f);
    int off = 0;
    for (int a = 0; a < 3; ++a) {
        const int dim = c.axes_dim[a], half = dim / 2;
        std::vector<float> omega(half);
        const float end = (dim * 1.f - 2) / dim;
        const float step = half > 1 ? (end - 0.f) / (half - 1) : 0.f;
        for (int i = 0; i < half; ++i) omega[i] = 1.0f / ::powf(1.f * c.theta, 0.f + i * step);
        for (int t = 0; t < L; ++t) {
            float pos = 0.0f;
            if (t >= n_txt) {
                const int it = t - n_txt;
                pos = a == 0 ? 0.0f : a == 1 ? static_cast<float>(it / w_tok) : static_cast<float>(it % w_tok);
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

edb200_epilogue_t make_ep(void* out, int dt, int64_t ldo, const float* bias) {
    edb200_epilogue_t ep;
    memset(&ep, 0, sizeof(ep));
    ep.out = out;
    ep.out_dtype = dt;
    ep.ldo = ldo;
    ep.bias = bias;
    return ep;
}

struct Lin {
    const edb200_qweight_t* w;
    const float* b;
};

Lin qlin(edb200_flux* m, const std::string& name) {
    Lin l;
    l.w = m->params.get(name + ".weight")->qw;
    l.b = m->params.get(name + ".bias")->f32;
    return l;
}

const float* fparam(edb200_flux* m, const std::string& name) { return m->params.get(name)->f32; }

edb200_status_t dense(edb200_flux* m, const std::string& name, const float* x, int64_t rows, int64_t ldx, int pre_silu,
                      int act, float* y, int64_t ldy, cudaStream_t s) {
    const Param* w = m->params.get(name + ".weight");
    return edb200_linear_f32(w->f32, fparam(m, name + ".bias"), x, rows, w->spec.k, w->spec.n_out, ldx, pre_silu, act,
                             y, ldy, s);
}

// Attention over the whole sequence.  Single GPU: all heads, output straight into `out`.
// Sequence parallel: Q/K/V of the local tokens (QL/KL/VL, head-major) are exchanged for
// all tokens of this rank's heads, attention runs on those, and its output is exchanged
// back into the local token rows of `out` (FLUX forward_sp, flux.hpp:1928-2369).
edb200_status_t attention(edb200_flux* m, int64_t T, void* out, int64_t ld_out, cudaStream_t s) {
    const edb200_flux_config_t& c = m->cfg;
    const int d = c.hidden_size / c.num_heads;
    const int heads = c.num_heads / m->world;
    const float scale = 1.0f / std::sqrt(static_cast<float>(d));
    // rows between heads in Q/K/V: the sequence padded to a multiple of the world size under
    // sequence parallelism (only the T real rows are attended over)
    const int64_t head_rows = m->world > 1 ? m->t_loc * m->world : T;
    if (m->p2p) {
        // Q/K/V rows were stored into their owners by the pack kernels; wait until every rank's are in,
        // let the attention epilogue store each output row into its owner's `out` rows, and meet
        // again before those rows are read.  The second barrier also tells the peers that this
        // rank has finished reading its Q/K/V, so the next block's pack kernels may overwrite them.
        EDB_TRY(edb200_sp_barrier(m->comm, s));
        if (c.attention == EDB200_ATTN_SAGE_INT8) {
            EDB_TRY(edb200_sage_attention_strided(m->Q, m->K, m->V, heads, T, head_rows, d, scale,
                                                  (c.sage_smooth_q ? EDB200_SAGE_SMOOTH_Q : 0) | EDB200_SAGE_FAST_MEANS,
                                                  m->SAGE, m->sage_bytes, nullptr, EDB200_TYPE_F16, ld_out,
                                                  &m->cat_peers, s));
        } else {
            EDB_TRY(edb200_attention_f16_strided(m->Q, m->K, m->V, heads, T, T, head_rows, head_rows, d, scale, nullptr,
                                                 EDB200_TYPE_F16, ld_out, &m->cat_peers, s));
        }
        return edb200_sp_barrier(m->comm, s);
    }
    void* att_out = out;
    int64_t att_ld = ld_out;
    if (m->world > 1) {
        const void* send[3] = {m->QL, m->KL, m->VL};
        void* recv[3] = {m->Q, m->K, m->V};
        EDB_TRY(edb200_sp_all_to_all_heads(m->comm, send, recv, 3, c.num_heads, m->t_loc, (int64_t)d * 2, s));
        att_out = m->AOUT;
        att_ld = (int64_t)heads * d;
    }
    if (c.attention == EDB200_ATTN_SAGE_INT8) {
        EDB_TRY(edb200_sage_attention_strided(m->Q, m->K, m->V, heads, T, head_rows, d, scale,
                                              (c.sage_smooth_q ? EDB200_SAGE_SMOOTH_Q : 0) | EDB200_SAGE_FAST_MEANS,
                                              m->SAGE, m->sage_bytes, att_out, EDB200_TYPE_F16, att_ld, nullptr, s));
    } else {
        EDB_TRY(edb200_attention_f16_strided(m->Q, m->K, m->V, heads, T, T, head_rows, head_rows, d, scale, att_out,
                                             EDB200_TYPE_F16, att_ld, nullptr, s));
    }
    if (m->world > 1) {
        EDB_TRY(edb200_sp_all_to_all_tokens(m->comm, m->AOUT, m->STG, out, m->t_loc, (int64_t)heads * d * 2, ld_out * 2, s));
    }
    return EDB200_OK;
}

// Row-count-tolerant wrappers: under sequence parallelism a rank may own no text rows.
edb200_status_t ln_mod(const float* x, int64_t H, const float* shift, const float* scale, int64_t rows, void* y,
                       int y_dtype, cudaStream_t s) {
    if (rows == 0) return EDB200_OK;
    return edb200_layernorm_modulate(x, H, shift, scale, nullptr, nullptr, rows, H, 1e-6f, y, y_dtype, H, s);
}

edb200_status_t mm_pair(const edb200_qweight_t* w0, const void* x0, int64_t m0, int64_t ldx0, const edb200_epilogue_t* e0,
                        const edb200_qweight_t* w1, const void* x1, int64_t m1, int64_t ldx1, const edb200_epilogue_t* e1,
                        cudaStream_t s) {
    if (m0 > 0 && m1 > 0) return edb200_mul_mat_q_pair(w0, x0, m0, ldx0, e0, w1, x1, m1, ldx1, e1, EDB200_TYPE_F16, s);
    if (m0 > 0) return edb200_mul_mat_q(w0, x0, EDB200_TYPE_F16, m0, ldx0, e0, s);
    if (m1 > 0) return edb200_mul_mat_q(w1, x1, EDB200_TYPE_F16, m1, ldx1, e1, s);
    return EDB200_OK;
}

edb200_status_t qk_pack(edb200_flux* m, const __half* qkv, int64_t rows, int64_t local_first, const float* qs,
                        const float* ks, cudaStream_t s) {
    if (rows == 0) return EDB200_OK;
    const edb200_flux_config_t& c = m->cfg;
    const int64_t H = c.hidden_size;
    const int d = static_cast<int>(H / c.num_heads);
    const bool sp = m->world > 1;
    if (m->p2p) {
        return edb200_qk_norm_rope_pack_sp(qkv, EDB200_TYPE_F16, 3 * H, 0, H, 2 * H, rows, c.num_heads, d, qs, ks, 1e-6f,
                                           m->PE, local_first, m->t_loc * m->world, &m->qkv_peers, EDB200_TYPE_F16, s);
    }
    // the position table is indexed by the global row: shift it by this rank's first token
    const float* pe = m->PE + (int64_t)m->rank * m->t_loc * (d / 2) * 4;
    return edb200_qk_norm_rope_pack(qkv, EDB200_TYPE_F16, 3 * H, 0, H, 2 * H, rows, c.num_heads, d, qs, ks, 1e-6f, pe,
                                    local_first, m->t_loc, sp ? m->QL : m->Q, sp ? m->KL : m->K, sp ? m->VL : m->V,
                                    EDB200_TYPE_F16, s);
}

// Whether the QKV projections pack q / k / v themselves (fused epilogue) instead of a separate pass.
bool fused_pack(const edb200_flux* m) {
    static int on = -1;
    if (on < 0) {
        const char* e = getenv("EDB200_FUSED_QK_PACK");
        on = (e != nullptr && atoi(e) == 0) ? 0 : edb200_mul_mat_q_fuses_qk_pack();
    }
    return on == 1 && m->cfg.hidden_size / m->cfg.num_heads == 128;
}

// The destination of qk_pack() as a fused-epilogue description (same positions, same table rows).
edb200_qk_pack_t pack_desc(edb200_flux* m, int64_t local_first, const float* qs, const float* ks) {
    const edb200_flux_config_t& c = m->cfg;
    const int d = static_cast<int>(c.hidden_size / c.num_heads);
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

// The adaLN projections of the whole step as one batch: [double i: img 6H, txt 6H] ... [single i: 3H].
// Built at the first step after prepare or after a tensor was reloaded (it caches device addresses).
edb200_status_t ensure_mod_batch(edb200_flux* m, cudaStream_t s) {
    if (m->mod_batch != nullptr && m->mod_batch_gen == m->params.generation()) return EDB200_OK;
    const edb200_flux_config_t& c = m->cfg;
    const int64_t H = c.hidden_size;
    edb200_gemv_batch_destroy(m->mod_batch);
    m->mod_batch = nullptr;
    std::vector<const edb200_qweight_t*> bw;
    std::vector<const float*> bb;
    std::vector<float*> by;
    for (int i = 0; i < c.depth; ++i) {
        const std::string p = "double_blocks." + std::to_string(i) + ".";
        for (int st = 0; st < 2; ++st) {
            const Lin l = qlin(m, p + (st == 0 ? "img" : "txt") + "_mod.lin");
            bw.push_back(l.w), bb.push_back(l.b), by.push_back(m->MODS + ((int64_t)i * 12 + st * 6) * H);
        }
    }
    for (int i = 0; i < c.depth_single_blocks; ++i) {
        const Lin l = qlin(m, "single_blocks." + std::to_string(i) + ".modulation.lin");
        bw.push_back(l.w), bb.push_back(l.b), by.push_back(m->MODS + ((int64_t)c.depth * 12 + (int64_t)i * 3) * H);
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

edb200_status_t edb200_flux_create(const edb200_flux_config_t* cfg, edb200_flux_t** out) {
    if (cfg == nullptr || out == nullptr) return fail(EDB200_ERR_INVALID, "flux_create: null argument");
    const edb200_flux_config_t& c = *cfg;
    if (c.hidden_size <= 0 || c.num_heads <= 0 || c.hidden_size % c.num_heads) {
        return fail(EDB200_ERR_INVALID, "flux_create: hidden_size must be a positive multiple of num_heads");
    }
    const int d = c.hidden_size / c.num_heads;
    if (d != 64 && d != 128) return fail(EDB200_ERR_UNSUPPORTED, "flux_create: head dim must be 64 or 128");
    if (c.axes_dim[0] + c.axes_dim[1] + c.axes_dim[2] != d) {
        return fail(EDB200_ERR_INVALID, "flux_create: axes_dim must sum to the head dim");
    }
    if (c.wtype != EDB200_TYPE_Q8_0 && c.wtype != EDB200_TYPE_Q4_K) {
        return fail(EDB200_ERR_UNSUPPORTED, "flux_create: wtype must be q8_0 or q4_K");
    }
    const int blk = c.wtype == EDB200_TYPE_Q4_K ? 256 : 64;
    if (c.hidden_size % 256 || c.mlp_hidden % 256 || (c.hidden_size + c.mlp_hidden) % blk) {
        return fail(EDB200_ERR_UNSUPPORTED, "flux_create: hidden_size and mlp_hidden must be multiples of 256");
    }
    if (c.attention == EDB200_ATTN_SAGE_INT8 && d != 128) {
        return fail(EDB200_ERR_UNSUPPORTED, "flux_create: INT8 attention needs head dim 128");
    }
    if (c.in_channels % 4 || c.context_in_dim % 4 || c.vec_in_dim % 4 || c.patch_size <= 0) {
        return fail(EDB200_ERR_INVALID, "flux_create: input dims must be multiples of 4");
    }
    if (device_error_word() == nullptr) return fail(EDB200_ERR_CUDA, "flux_create: no CUDA device");
    edb200_flux* m = new (std::nothrow) edb200_flux();
    if (m == nullptr) return fail(EDB200_ERR_NOMEM, "flux_create: host allocation failed");
    m->cfg = c;
    register_params(m);
    *out = m;
    return EDB200_OK;
}

void edb200_flux_destroy(edb200_flux_t* m) {
    if (m == nullptr) return;
    if (m->pinned) cudaFreeHost(m->pinned);
    edb200_gemv_batch_destroy(m->mod_batch);
    delete m;
}

int edb200_flux_tensor_count(const edb200_flux_t* m) {
    return m ? static_cast<int>(const_cast<edb200_flux_t*>(m)->params.params().size()) : 0;
}

edb200_status_t edb200_flux_tensor_info(const edb200_flux_t* m, int index, char* name, int name_cap, int* ggml_type,
                                        int64_t* n_out, int64_t* k, int64_t* nbytes) {
    if (m == nullptr || index < 0 || index >= edb200_flux_tensor_count(m)) {
        return fail(EDB200_ERR_INVALID, "flux_tensor_info: bad index");
    }
    const Param& p = const_cast<edb200_flux_t*>(m)->params.params()[index];
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

edb200_status_t edb200_flux_set_tensor(edb200_flux_t* m, const char* name, int ggml_type, const void* data,
                                       int64_t nbytes, int on_device, void* stream) {
    if (m == nullptr || name == nullptr) return fail(EDB200_ERR_INVALID, "flux_set_tensor: null argument");
    return m->params.set(name, ggml_type, data, nbytes, on_device != 0, static_cast<cudaStream_t>(stream));
}

edb200_status_t edb200_flux_get_tensor_f32(const edb200_flux_t* m, const char* name, float* out, int64_t n_floats,
                                          int on_device, void* stream) {
    if (m == nullptr || name == nullptr) return fail(EDB200_ERR_INVALID, "flux_get_tensor_f32: null argument");
    return m->params.fetch_f32(name, out, n_floats, on_device != 0, static_cast<cudaStream_t>(stream));
}

edb200_status_t edb200_flux_load_gguf(edb200_flux_t* m, const char* path, const char* strip_prefix, int* n_loaded,
                                    void* stream) {
    if (m == nullptr || path == nullptr) return fail(EDB200_ERR_INVALID, "flux_load_gguf: null argument");
    return load_gguf(m->params, EDB200_FAMILY_FLUX, path, strip_prefix, static_cast<cudaStream_t>(stream), n_loaded);
}

edb200_status_t edb200_flux_load_safetensors(edb200_flux_t* m, const char* path, const char* strip_prefix, int* n_loaded,
                                           void* stream) {
    if (m == nullptr || path == nullptr) return fail(EDB200_ERR_INVALID, "flux_load_safetensors: null argument");
    return load_safetensors(m->params, EDB200_FAMILY_FLUX, path, strip_prefix, static_cast<cudaStream_t>(stream), n_loaded);
}

edb200_status_t edb200_flux_init_random(edb200_flux_t* m, uint64_t seed, float std, void* stream) {
    if (m == nullptr) return fail(EDB200_ERR_INVALID, "flux_init_random: null model");
    return m->params.init_random(seed, std, static_cast<cudaStream_t>(stream));
}

int64_t edb200_flux_weight_bytes(const edb200_flux_t* m) { return m ? m->params.device_bytes() : 0; }
int64_t edb200_flux_workspace_bytes(const edb200_flux_t* m) { return m ? m->ws.capacity() : 0; }

edb200_status_t edb200_flux_prepare(edb200_flux_t* m, int latent_h, int latent_w, int n_txt, void* stream) {
    if (m == nullptr) return fail(EDB200_ERR_INVALID, "flux_prepare: null model");
    const edb200_flux_config_t& c = m->cfg;
    const int p = c.patch_size;
    if (latent_h <= 0 || latent_w <= 0 || n_txt <= 0 || latent_h % p || latent_w % p) {
        return fail(EDB200_ERR_INVALID, "flux_prepare: latent must be a positive multiple of the patch size");
    }
    if (m->lat_h == latent_h && m->lat_w == latent_w && m->n_txt == n_txt) return EDB200_OK;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int64_t H = c.hidden_size, M = c.mlp_hidden, d = H / c.num_heads;
    const int h_tok = latent_h / p, w_tok = latent_w / p;
    const int64_t n_img = (int64_t)h_tok * w_tok, T = n_img + n_txt;
    const int lat_c = c.in_channels / (p * p);
    int64_t t_loc = T, t_rows = T, txt_l = n_txt, img_first = 0;
    if (m->world > 1) {
        if (c.num_heads % m->world) {
            return fail(EDB200_ERR_UNSUPPORTED, "flux_prepare: %d heads do not divide over %d ranks", c.num_heads, m->world);
        }
        EDB_TRY(edb200_sp_shard(T, n_txt, m->rank, m->world, &t_loc, &txt_l, &img_first, &t_rows));
        if (t_rows == 0) return fail(EDB200_ERR_UNSUPPORTED, "flux_prepare: %lld tokens leave rank %d without rows", (long long)T, m->rank);
    }
    const int64_t sage =
        c.attention == EDB200_ATTN_SAGE_INT8 ? edb200_sage_scratch_bytes(c.num_heads / m->world, T, (int)d) : 0;
    const int64_t lat_elems = (int64_t)lat_c * latent_h * latent_w;
    const int64_t pe_elems = T * (d / 2) * 4;
    auto al = [](int64_t b) { return (b + 255) & ~int64_t(255); };
    int64_t total = 0;
    total += al(T * H * 4) + al(T * H * 2) + al(T * 3 * H * 2) + 3 * al(T * H * 2) + al(T * (H + M) * 2) +
             al(T * M * 2);
    total += al(mods_per_step(c) * 4) + 3 * al(H * 4) + al(256 * 4) + 2 * al(n_img * c.in_channels * 4);
    total += al(n_img * H * 4) + al(pe_elems * 4) + al(128 * 4) + 2 * al(lat_elems * 4) +
             al((int64_t)n_txt * c.context_in_dim * 4) + al(c.vec_in_dim * 4) + al(sage) + 4096;
    if (m->world > 1) total += 5 * al(t_loc * H * 2) + al(n_img * c.in_channels * 4);
    cudaStreamSynchronize(s);
    if (m->comm != nullptr) EDB_TRY(edb200_comm_unmap_peers(m->comm));   // collective; the old workspace goes away
    m->p2p = false;
    if (m->world > 1) total += 2048;
    EDB_TRY(m->ws.reserve(total));
    Workspace& w = m->ws;
    m->X = w.take_n<float>(T * H);
    m->XMOD = w.take(T * H * 2);
    m->QKV = w.take(T * 3 * H * 2);
    m->Q = w.take(T * H * 2);
    m->K = w.take(T * H * 2);
    m->V = w.take(T * H * 2);
    m->CAT = w.take(T * (H + M) * 2);
    m->HID = w.take(T * M * 2);
    m->MODS = w.take_n<float>(mods_per_step(c));
    m->VEC = w.take_n<float>(H);
    m->TMP_H = w.take_n<float>(2 * H);
    m->TEMB = w.take_n<float>(256);
    m->TOK_IN = w.take_n<float>(n_img * c.in_channels);
    m->TOK_OUT = w.take_n<float>(n_img * c.in_channels);
    m->FIN = w.take_n<float>(n_img * H);
    m->PE = w.take_n<float>(pe_elems);
    m->FREQ = w.take_n<float>(128);
    m->LAT_IN = w.take_n<float>(lat_elems);
    m->LAT_OUT = w.take_n<float>(lat_elems);
    m->CTX = w.take_n<float>((int64_t)n_txt * c.context_in_dim);
    m->YVEC = w.take_n<float>(c.vec_in_dim);
    m->SAGE = sage > 0 ? w.take(sage) : nullptr;
    m->sage_bytes = sage;
    m->QL = m->KL = m->VL = m->AOUT = m->STG = nullptr;
    m->TOK_LOC = nullptr;
    if (m->world > 1) {
        m->QL = w.take(t_loc * H * 2);
        m->KL = w.take(t_loc * H * 2);
        m->VL = w.take(t_loc * H * 2);
        m->AOUT = w.take(t_loc * H * 2);   // [T, (heads / world) * d] = the same number of elements
        m->STG = w.take(t_loc * H * 2);
        m->TOK_LOC = w.take_n<float>(n_img * c.in_channels);
        if (m->TOK_LOC == nullptr) return fail(EDB200_ERR_NOMEM, "flux_prepare: workspace accounting error");
    }
    if (m->world > 1) {
        void* flags = w.take(1024);   // barrier flags + epoch
        if (flags == nullptr) return fail(EDB200_ERR_NOMEM, "flux_prepare: workspace accounting error");
        const char* how = getenv("EDB200_SP_EXCHANGE");   // "nccl" keeps the library exchanges (comparison runs)
        const bool want_p2p = how == nullptr || strcmp(how, "nccl") != 0;
        // every rank takes the same decision: the mapping call is collective
        edb200_status_t st = want_p2p ? edb200_comm_map_peers(m->comm, w.base(), w.capacity(),
                                                              static_cast<char*>(flags) - static_cast<char*>(w.base()), s)
                                      : EDB200_ERR_UNSUPPORTED;
        if (st == EDB200_OK) {
            m->p2p = true;
            memset(&m->qkv_peers, 0, sizeof(m->qkv_peers));
            memset(&m->cat_peers, 0, sizeof(m->cat_peers));
            m->qkv_peers.world = m->cat_peers.world = m->world;
            m->qkv_peers.rank = m->cat_peers.rank = m->rank;
            m->qkv_peers.t_loc = m->cat_peers.t_loc = t_loc;
            for (int r = 0; r < m->world; ++r) {
                m->qkv_peers.buf[0][r] = edb200_comm_peer_ptr(m->comm, r, m->Q);
                m->qkv_peers.buf[1][r] = edb200_comm_peer_ptr(m->comm, r, m->K);
                m->qkv_peers.buf[2][r] = edb200_comm_peer_ptr(m->comm, r, m->V);
                m->cat_peers.buf[0][r] = edb200_comm_peer_ptr(m->comm, r, m->CAT);
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
    if (m->YVEC == nullptr || (sage > 0 && m->SAGE == nullptr)) {
        return fail(EDB200_ERR_NOMEM, "flux_prepare: workspace accounting error");
    }
    // the batch of adaLN projections points into the workspace: rebuilt at the next step
    edb200_gemv_batch_destroy(m->mod_batch);
    m->mod_batch = nullptr;
    // position table and sinusoid frequencies are computed once per shape on the host
    std::vector<float> pe = build_flux_pe(c, h_tok, w_tok, n_txt);
    std::vector<float> freq(128);
    for (int i = 0; i < 128; ++i) freq[i] = (float)std::exp(-std::log(10000) * i / 128);
    cudaError_t e = cudaMemcpyAsync(m->PE, pe.data(), pe.size() * 4, cudaMemcpyHostToDevice, s);
    if (e == cudaSuccess) e = cudaMemcpyAsync(m->FREQ, freq.data(), 128 * 4, cudaMemcpyHostToDevice, s);
    if (e == cudaSuccess) e = cudaStreamSynchronize(s);
    if (e != cudaSuccess) return check_cuda(e, "flux_prepare upload");
    // pinned staging for the host-tensor entry point
    const int64_t need = (2 * lat_elems + (int64_t)n_txt * c.context_in_dim + c.vec_in_dim) * 4;
    if (need > m->pinned_bytes) {
        if (m->pinned) cudaFreeHost(m->pinned);
        m->pinned = nullptr;
        e = cudaMallocHost(reinterpret_cast<void**>(&m->pinned), need);
        if (e != cudaSuccess) return fail(EDB200_ERR_NOMEM, "flux_prepare: cudaMallocHost: %s", cudaGetErrorString(e));
        m->pinned_bytes = need;
    }
    m->lat_h = latent_h;
    m->lat_w = latent_w;
    m->n_txt = n_txt;
    m->n_img = static_cast<int>(n_img);
    return EDB200_OK;
}

edb200_status_t edb200_flux_set_comm(edb200_flux_t* m, edb200_comm_t* comm) {
    if (m == nullptr) return fail(EDB200_ERR_INVALID, "flux_set_comm: null model");
    if (m->comm != nullptr && m->comm != comm) edb200_comm_unmap_peers(m->comm);   // collective
    m->comm = comm;
    m->rank = comm ? edb200_comm_rank(comm) : 0;
    m->world = comm ? edb200_comm_world(comm) : 1;
    m->lat_h = m->lat_w = m->n_txt = 0;   // the workspace must be prepared again
    m->p2p = false;
    return EDB200_OK;
}

edb200_status_t edb200_flux_set_anchor_capture(edb200_flux_t* m, int anchor, float* dst) {
    if (m == nullptr) return fail(EDB200_ERR_INVALID, "flux_set_anchor_capture: null model");
    if (anchor == EDB200_ANCHOR_MODEL_IN) {
        m->anchor_in = dst;
    } else if (anchor == EDB200_ANCHOR_MODEL_OUT) {
        m->anchor_out = dst;
    } else if (anchor >= 0 && anchor < m->cfg.depth) {
        m->anchor_block.resize(m->cfg.depth, nullptr);
        m->anchor_block[anchor] = dst;
    } else {
        return fail(EDB200_ERR_INVALID, "flux_set_anchor_capture: anchor %d (block outputs are 0..%d)", anchor, m->cfg.depth - 1);
    }
    return EDB200_OK;
}

edb200_status_t edb200_flux_set_stop_after(edb200_flux_t* m, int block) {
    if (m == nullptr || block < -1 || block >= m->cfg.depth) {
        return fail(EDB200_ERR_INVALID, "flux_set_stop_after: block must be -1 (off) or a double block index");
    }
    m->stop_after = block;
    return EDB200_OK;
}

edb200_status_t edb200_flux_set_stream_override(edb200_flux_t* m, const float* residual) {
    if (m == nullptr) return fail(EDB200_ERR_INVALID, "flux_set_stream_override: null model");
    m->stream_override = residual;
    return EDB200_OK;
}

edb200_status_t edb200_flux_set_tap(edb200_flux_t* m, float* tap) {
    if (m == nullptr) return fail(EDB200_ERR_INVALID, "flux_set_tap: null model");
    m->tap = tap;
    return EDB200_OK;
}

static edb200_status_t flux_step_body(edb200_flux_t* m, const float* latent, float timestep, const float* sched,
                                      const int* sched_step, const float* context, const float* y, float guidance,
                                      float* out, void* stream) {
    if (m == nullptr || latent == nullptr || context == nullptr || y == nullptr || out == nullptr) {
        return fail(EDB200_ERR_INVALID, "flux_step: null argument");
    }
    if (m->lat_h == 0) return fail(EDB200_ERR_INVALID, "flux_step: call edb200_flux_prepare first");
    EDB_TRY(m->params.all_loaded());
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const edb200_flux_config_t& c = m->cfg;
    const int64_t H = c.hidden_size, M = c.mlp_hidden;
    const int64_t T = (int64_t)m->n_txt + m->n_img;   // whole sequence (attention length)
    // rows this rank owns: all of them on one GPU, a slice [text rows ; image rows] otherwise
    const int64_t n_txt = m->txt_l, n_img = m->img_l, TL = m->t_rows;
    const int64_t txt_first = m->world > 1 ? (int64_t)m->rank * m->t_loc : 0;   // first owned text row (if any)
    // A sequence-parallel rank's out-projections have few output tiles and long reductions: let
    // them be cut along k (their adds into the residual stream are then unordered).  A single
    // GPU keeps every sum in one fixed order.
    const int split_k = m->world > 1 ? EDB200_SPLIT_K_UNORDERED : EDB200_SPLIT_K_NEVER;
    const int lat_c = c.in_channels / (c.patch_size * c.patch_size);
    const int F16 = EDB200_TYPE_F16;
    float* X_txt = m->X;
    float* X_img = m->X + n_txt * H;
    __half* xmod = static_cast<__half*>(m->XMOD);
    __half* qkv = static_cast<__half*>(m->QKV);
    __half* cat = static_cast<__half*>(m->CAT);
    __half* hid = static_cast<__half*>(m->HID);

    // ---- prelude (Flux::forward_orig, flux.hpp:3886-3965)
    launch_patchify(latent, m->TOK_IN, lat_c, m->lat_h, m->lat_w, c.patch_size, s);
    if (n_img > 0) {
        EDB_TRY(dense(m, "img_in", m->TOK_IN + m->img_first * c.in_channels, n_img, c.in_channels, 0, EDB200_ACT_NONE,
                      X_img, H, s));
    }
    if (n_txt > 0) {
        EDB_TRY(dense(m, "txt_in", context + txt_first * c.context_in_dim, n_txt, c.context_in_dim, 0, EDB200_ACT_NONE,
                      X_txt, H, s));
    }
    if (sched != nullptr) {
        launch_timestep_embedding_sched(m->FREQ, sched, sched_step, 1.0f, 1000.0f, 128, m->TEMB, s);
    } else {
        launch_timestep_embedding(m->FREQ, timestep, 1000.0f, 128, m->TEMB, s);
    }
    EDB_TRY(dense(m, "time_in.in_layer", m->TEMB, 1, 256, 0, EDB200_ACT_SILU, m->TMP_H, H, s));
    EDB_TRY(dense(m, "time_in.out_layer", m->TMP_H, 1, H, 0, EDB200_ACT_NONE, m->VEC, H, s));
    if (c.guidance_embed) {
        launch_timestep_embedding(m->FREQ, guidance, 1000.0f, 128, m->TEMB, s);
        EDB_TRY(dense(m, "guidance_in.in_layer", m->TEMB, 1, 256, 0, EDB200_ACT_SILU, m->TMP_H, H, s));
        EDB_TRY(dense(m, "guidance_in.out_layer", m->TMP_H, 1, H, 0, EDB200_ACT_NONE, m->TMP_H + H, H, s));
        launch_add_inplace(m->VEC, m->TMP_H + H, H, s);
    }
    EDB_TRY(dense(m, "vector_in.in_layer", y, 1, c.vec_in_dim, 0, EDB200_ACT_SILU, m->TMP_H, H, s));
    EDB_TRY(dense(m, "vector_in.out_layer", m->TMP_H, 1, H, 0, EDB200_ACT_NONE, m->TMP_H + H, H, s));
    launch_add_inplace(m->VEC, m->TMP_H + H, H, s);

    // ---- reuse seam (Flux::forward_orig, flux.hpp:3968-3978): the block stack transforms the image stream;
    // ModelIn is that stream before the stack
    if (m->anchor_in != nullptr && n_img > 0) {
        cudaMemcpyAsync(m->anchor_in, X_img, n_img * H * 4, cudaMemcpyDeviceToDevice, s);
    }
    const bool whole_inject = m->stream_override != nullptr;
    const bool fused = fused_pack(m);   // q / k / v packed by the QKV projections' own epilogue

    // ---- every adaLN vector of the step: lin(silu(vec)), weight streaming, one launch for all of them
    // (sequence-parallel ranks with peer memory each stream 1/N of the weights and store to all)
    float* mods = m->MODS;
    float* smods = mods + (int64_t)c.depth * 12 * H;
    EDB_TRY(ensure_mod_batch(m, s));
    EDB_TRY(edb200_gemv_batch_run(m->mod_batch, m->VEC, 1, m->p2p ? &m->mods_peers : nullptr, s));
    if (m->p2p) EDB_TRY(edb200_sp_barrier(m->comm, s));
    float* fmods = smods + (int64_t)c.depth_single_blocks * 3 * H;
    EDB_TRY(dense(m, "final_layer.adaLN_modulation.1", m->VEC, 1, H, 1, EDB200_ACT_NONE, fmods, 2 * H, s));

    // ---- double-stream blocks (none of them under a whole-stack inject, flux.hpp:4511-4515)
    for (int i = 0; i < (whole_inject ? 0 : c.depth); ++i) {
        const std::string p = "double_blocks." + std::to_string(i) + ".";
        const float* im = mods + (int64_t)i * 12 * H;   // shift1 scale1 gate1 shift2 scale2 gate2
        const float* tm = im + 6 * H;
        EDB_TRY(ln_mod(X_img, H, im, im + H, n_img, xmod + n_txt * H, F16, s));
        EDB_TRY(ln_mod(X_txt, H, tm, tm + H, n_txt, xmod, F16, s));
        {
            const Lin li = qlin(m, p + "img_attn.qkv"), lt = qlin(m, p + "txt_attn.qkv");
            edb200_epilogue_t ei = make_ep(qkv + n_txt * 3 * H, F16, 3 * H, li.b);
            edb200_epilogue_t et = make_ep(qkv, F16, 3 * H, lt.b);
            const float* iq = fparam(m, p + "img_attn.norm.query_norm.scale");
            const float* ik = fparam(m, p + "img_attn.norm.key_norm.scale");
            const float* tq = fparam(m, p + "txt_attn.norm.query_norm.scale");
            const float* tk = fparam(m, p + "txt_attn.norm.key_norm.scale");
            const edb200_qk_pack_t pi = pack_desc(m, n_txt, iq, ik), pt = pack_desc(m, 0, tq, tk);
            if (fused) ei.pack = &pi, et.pack = &pt;
            EDB_TRY(mm_pair(li.w, xmod + n_txt * H, n_img, H, &ei, lt.w, xmod, n_txt, H, &et, s));
            if (!fused) {
                EDB_TRY(qk_pack(m, qkv + n_txt * 3 * H, n_img, n_txt, iq, ik, s));
                EDB_TRY(qk_pack(m, qkv, n_txt, 0, tq, tk, s));
            }
        }
        EDB_TRY(attention(m, T, cat, H + M, s));
        {
            const Lin li = qlin(m, p + "img_attn.proj"), lt = qlin(m, p + "txt_attn.proj");
            edb200_epilogue_t ei = make_ep(X_img, EDB200_TYPE_F32, H, li.b);
            ei.residual = X_img, ei.ld_res = H, ei.gate = im + 2 * H, ei.split_k = split_k;
            edb200_epilogue_t et = make_ep(X_txt, EDB200_TYPE_F32, H, lt.b);
            et.residual = X_txt, et.ld_res = H, et.gate = tm + 2 * H, et.split_k = split_k;
            EDB_TRY(mm_pair(li.w, cat + n_txt * (H + M), n_img, H + M, &ei, lt.w, cat, n_txt, H + M, &et, s));
        }
        EDB_TRY(ln_mod(X_img, H, im + 3 * H, im + 4 * H, n_img, xmod + n_txt * H, F16, s));
        EDB_TRY(ln_mod(X_txt, H, tm + 3 * H, tm + 4 * H, n_txt, xmod, F16, s));
        {
            const Lin li = qlin(m, p + "img_mlp.0"), lt = qlin(m, p + "txt_mlp.0");
            edb200_epilogue_t ei = make_ep(hid + n_txt * M, F16, M, li.b);
            ei.act = EDB200_ACT_GELU_TANH;
            edb200_epilogue_t et = make_ep(hid, F16, M, lt.b);
            et.act = EDB200_ACT_GELU_TANH;
            EDB_TRY(mm_pair(li.w, xmod + n_txt * H, n_img, H, &ei, lt.w, xmod, n_txt, H, &et, s));
        }
        {
            const Lin li = qlin(m, p + "img_mlp.2"), lt = qlin(m, p + "txt_mlp.2");
            edb200_epilogue_t ei = make_ep(X_img, EDB200_TYPE_F32, H, li.b);
            ei.residual = X_img, ei.ld_res = H, ei.gate = im + 5 * H, ei.split_k = split_k;
            edb200_epilogue_t et = make_ep(X_txt, EDB200_TYPE_F32, H, lt.b);
            et.residual = X_txt, et.ld_res = H, et.gate = tm + 5 * H, et.split_k = split_k;
            EDB_TRY(mm_pair(li.w, hid + n_txt * M, n_img, M, &ei, lt.w, hid, n_txt, M, &et, s));
        }
        if (m->tap) {
            cudaMemcpyAsync(m->tap + (int64_t)i * TL * H, m->X, TL * H * 4, cudaMemcpyDeviceToDevice, s);
        }
        // BlockOut[i]: the image stream after double block i, and the probe stop (flux.hpp:4260-4266)
        if (i < (int)m->anchor_block.size() && m->anchor_block[i] != nullptr && n_img > 0) {
            cudaMemcpyAsync(m->anchor_block[i], X_img, n_img * H * 4, cudaMemcpyDeviceToDevice, s);
        }
        if (m->stop_after == i) return check_cuda(cudaGetLastError(), "flux_step");
    }

    // ---- single-stream blocks over [txt ; img]
    for (int i = 0; i < (whole_inject ? 0 : c.depth_single_blocks); ++i) {
        const std::string p = "single_blocks." + std::to_string(i) + ".";
        const float* sm = smods + (int64_t)i * 3 * H;   // shift scale gate
        EDB_TRY(ln_mod(m->X, H, sm, sm + H, TL, xmod, F16, s));
        {
            const Lin l1 = qlin(m, p + "linear1");
            edb200_epilogue_t ep = make_ep(qkv, F16, 3 * H, l1.b);
            ep.split_n = 3 * H;
            ep.out2 = cat + H;
            ep.out2_dtype = F16;
            ep.ldo2 = H + M;
            ep.act2 = EDB200_ACT_GELU_TANH;
            const float* nq = fparam(m, p + "norm.query_norm.scale");
            const float* nk = fparam(m, p + "norm.key_norm.scale");
            const edb200_qk_pack_t pk = pack_desc(m, 0, nq, nk);
            if (fused) ep.pack = &pk;
            EDB_TRY(edb200_mul_mat_q(l1.w, xmod, F16, TL, H, &ep, s));
            if (!fused) EDB_TRY(qk_pack(m, qkv, TL, 0, nq, nk, s));
        }
        EDB_TRY(attention(m, T, cat, H + M, s));
        {
            const Lin l2 = qlin(m, p + "linear2");
            edb200_epilogue_t ep = make_ep(m->X, EDB200_TYPE_F32, H, l2.b);
            ep.residual = m->X, ep.ld_res = H, ep.gate = sm + 2 * H, ep.split_k = split_k;
            EDB_TRY(edb200_mul_mat_q(l2.w, cat, F16, TL, H + M, &ep, s));
        }
        if (m->tap) {
            cudaMemcpyAsync(m->tap + (int64_t)(c.depth + i) * TL * H, m->X, TL * H * 4, cudaMemcpyDeviceToDevice, s);
        }
    }

    // whole-stack inject: the loops ran zero blocks; the stream after the stack is rebuilt as
    // x_before + residual (build_stream_override, flux.hpp:4511-4515)
    if (whole_inject && n_img > 0) launch_add_inplace(X_img, m->stream_override, n_img * H, s);
    // ModelOut: the image stream after the stack, before the final layer (flux.hpp:4516-4520)
    if (m->anchor_out != nullptr && n_img > 0) {
        cudaMemcpyAsync(m->anchor_out, X_img, n_img * H * 4, cudaMemcpyDeviceToDevice, s);
    }

    // ---- final layer on the image rows + unpatchify (LastLayer::forward, flux.hpp:3533-3559)
    EDB_TRY(ln_mod(X_img, H, fmods, fmods + H, n_img, m->FIN, EDB200_TYPE_F32, s));
    if (m->world == 1) {
        EDB_TRY(dense(m, "final_layer.linear", m->FIN, n_img, H, 0, EDB200_ACT_NONE, m->TOK_OUT, c.in_channels, s));
    } else {
        // every rank projects its image rows, then all ranks gather the whole token grid
        if (n_img > 0) {
            EDB_TRY(dense(m, "final_layer.linear", m->FIN, n_img, H, 0, EDB200_ACT_NONE, m->TOK_LOC, c.in_channels, s));
        }
        std::vector<int64_t> first(m->world), count(m->world);
        for (int r = 0; r < m->world; ++r) {
            int64_t tx = 0, f = 0, rows = 0;
            EDB_TRY(edb200_sp_shard(T, m->n_txt, r, m->world, nullptr, &tx, &f, &rows));
            first[r] = f;
            count[r] = rows - tx;
        }
        if (m->p2p) {
            // peer stores + barrier: nothing of the step goes through a library exchange
            EDB_TRY(edb200_sp_all_gather_rows_peer(m->comm, m->TOK_LOC, m->TOK_OUT, first.data(), count.data(), (int64_t)c.in_channels * 4, s));
        } else {
            EDB_TRY(edb200_sp_all_gather_rows(m->comm, m->TOK_LOC, m->TOK_OUT, first.data(), count.data(), (int64_t)c.in_channels * 4, s));
        }
    }
    launch_unpatchify(m->TOK_OUT, out, lat_c, m->lat_h, m->lat_w, c.patch_size, s);
    return check_cuda(cudaGetLastError(), "flux_step");
}

edb200_status_t edb200_flux_step(edb200_flux_t* m, const float* latent, float timestep, const float* context,
                                 const float* y, float guidance, float* out, void* stream) {
    return flux_step_body(m, latent, timestep, nullptr, nullptr, context, y, guidance, out, stream);
}

edb200_status_t edb200_flux_step_sched(edb200_flux_t* m, const float* latent, const float* sigmas, const int* step,
                                       const float* context, const float* y, float guidance, float* out,
                                       void* stream) {
    if (sigmas == nullptr || step == nullptr) return fail(EDB200_ERR_INVALID, "flux_step_sched: null schedule");
    return flux_step_body(m, latent, 0.0f, sigmas, step, context, y, guidance, out, stream);
}

edb200_status_t edb200_flux_compute_host(edb200_flux_t* m, const float* latent, int latent_h, int latent_w,
                                         float timestep, const float* context, int n_txt, const float* y,
                                         float guidance, float* out, void* stream) {
    if (m == nullptr || latent == nullptr || context == nullptr || y == nullptr || out == nullptr) {
        return fail(EDB200_ERR_INVALID, "flux_compute_host: null argument");
    }
    EDB_TRY(edb200_flux_prepare(m, latent_h, latent_w, n_txt, stream));
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const edb200_flux_config_t& c = m->cfg;
    const int lat_c = c.in_channels / (c.patch_size * c.patch_size);
    const int64_t lat_elems = (int64_t)lat_c * latent_h * latent_w;
    const int64_t ctx_elems = (int64_t)n_txt * c.context_in_dim;
    // stage through pinned memory so the copies are truly asynchronous
    float* p_lat = m->pinned;
    float* p_ctx = p_lat + lat_elems;
    float* p_y = p_ctx + ctx_elems;
    float* p_out = p_y + c.vec_in_dim;
    memcpy(p_lat, latent, lat_elems * 4);
    memcpy(p_ctx, context, ctx_elems * 4);
    memcpy(p_y, y, (size_t)c.vec_in_dim * 4);
    cudaError_t e = cudaMemcpyAsync(m->LAT_IN, p_lat, lat_elems * 4, cudaMemcpyHostToDevice, s);
    if (e == cudaSuccess) e = cudaMemcpyAsync(m->CTX, p_ctx, ctx_elems * 4, cudaMemcpyHostToDevice, s);
    if (e == cudaSuccess) e = cudaMemcpyAsync(m->YVEC, p_y, (size_t)c.vec_in_dim * 4, cudaMemcpyHostToDevice, s);
    if (e != cudaSuccess) return check_cuda(e, "flux_compute_host H2D");
    EDB_TRY(edb200_flux_step(m, m->LAT_IN, timestep, m->CTX, m->YVEC, guidance, m->LAT_OUT, stream));
    e = cudaMemcpyAsync(p_out, m->LAT_OUT, lat_elems * 4, cudaMemcpyDeviceToHost, s);
    if (e != cudaSuccess) return check_cuda(e, "flux_compute_host D2H");
    EDB_TRY(poll_device_error(s));   // synchronises the stream
    memcpy(out, p_out, lat_elems * 4);
    return EDB200_OK;
}

}  // extern "C"
