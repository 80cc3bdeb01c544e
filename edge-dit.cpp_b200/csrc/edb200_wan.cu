// Wan 2.1 (t2v) denoise-step executor: the op schedule of Wan::forward
// (reference src/dit_models/models/wan.hpp:4759-4808, forward_orig :4516-4758,
// WanAttentionBlock::forward :4136-4187, WanSelfAttention::forward :3523-3543,
// WanT2VCrossAttention::forward_named :3830-3895, Head::forward :4309-4330) on the
// kernels of this library.
//
// Per block, T video tokens of width D:
//   es = e0 + modulation                                           one small kernel
//   XMOD = modulate(LN(X), es0, es1)                               layernorm_modulate
//   QKV  = XMOD Wq|Wk|Wv + b                                       3 quantised GEMMs into one [T, 3D] buffer
//   Q,K  = rope(RMSNorm_D(q) w), V -> head-major                   row_rstd x2 + pack (stores to peers under SP)
//   ATT  = attention(Q, K, V)                                      INT8-QK or f16
//   X   += es2 * (ATT Wo + b)                                      GEMM epilogue
//   QC   = LN3(X) Wcq + b; Q = RMSNorm_D(QC) w                     LN (affine), GEMM, row_rstd, pack (q only)
//   KC,VC from the embedded text (512 tokens), K = RMSNorm_D(KC) w GEMM pair, row_rstd, pack (k, v only)
//   X   += attention(Q, K, V; Lq = T, Lk = n_ctx) Wco + b          f16 attention, GEMM epilogue (gate of ones)
//   X   += es5 * (gelu(modulate(LN(X), es3, es4) W0 + b) W2 + b)   two GEMMs
// Cross-attention needs no exchange under sequence parallelism: every rank holds the
// whole text context and attends with its own query rows.
#include "edb200_model.h"

#include <cuda_fp16.h>

#include <algorithm>
#include <cmath>
#include <cstdlib>
#include <cstring>
#include <vector>

using namespace edb;

struct edb200_wan {
    edb200_wan_config_t cfg;
    ParamTable params;
    Workspace ws;
    int frames = 0, lat_h = 0, lat_w = 0, n_ctx = 0;
    int64_t T = 0;           // video tokens of the whole clip
    float* X = nullptr;
    void *XMOD = nullptr, *QKV = nullptr, *Q = nullptr, *K = nullptr, *V = nullptr, *ATT = nullptr, *HID = nullptr;
    void *CTXE = nullptr, *KVC = nullptr, *KC = nullptr, *VC = nullptr, *QX = nullptr;
    float *ES = nullptr, *E = nullptr, *E0 = nullptr, *TMP = nullptr, *TEMB = nullptr, *FREQ = nullptr, *PE = nullptr;
    float *RSTD = nullptr, *ONES = nullptr, *TOK_IN = nullptr, *TOK_OUT = nullptr, *TOK_LOC = nullptr, *CTX32 = nullptr;
    float *LAT_IN = nullptr, *LAT_OUT = nullptr, *CTX_IN = nullptr, *HMOD = nullptr;
    void* SAGE = nullptr;
    int64_t sage_bytes = 0;
    float* tap = nullptr;
    ReuseAnchors anchors;   // computation-reuse seam (capture / probe stop / whole-stack inject)
    float* pinned = nullptr;
    int64_t pinned_bytes = 0;
    // sequence parallel
    edb200_comm_t* comm = nullptr;
    int rank = 0, world = 1;
    int64_t t_loc = 0, t_rows = 0;   // this rank's slot of the padded sequence and the rows it owns
    bool p2p = false;
    void *QL = nullptr, *KL = nullptr, *VL = nullptr, *AOUT = nullptr, *STG = nullptr;
    edb200_sp_peers_t qkv_peers, att_peers;
};

namespace {

struct Lin {
    const edb200_qweight_t* w;
    const float* b;
};

Lin qlin(edb200_wan* m, const std::string& name) {
    Lin l;
    l.w = m->params.get(name + ".weight")->qw;
    l.b = m->params.get(name + ".bias")->f32;
    return l;
}

const float* fparam(edb200_wan* m, const std::string& name) { return m->params.get(name)->f32; }

edb200_status_t dense(edb200_wan* m, const std::string& name, const float* x, int64_t rows, int64_t ldx, int pre_silu,
                      int act, float* y, int64_t ldy, cudaStream_t s) {
    const Param* w = m->params.get(name + ".weight");
    return edb200_linear_f32(w->f32, fparam(m, name + ".bias"), x, rows, w->spec.k, w->spec.n_out, ldx, pre_silu, act,
                             y, ldy, s);
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

void register_params(edb200_wan* m) {
    const edb200_wan_config_t& c = m->cfg;
    const int64_t D = c.dim, F = c.ffn_dim;
    const int64_t pf = (int64_t)c.in_dim * c.patch_size[0] * c.patch_size[1] * c.patch_size[2];
    ParamTable& t = m->params;
    auto lin = [&](const std::string& name, int64_t n_out, int64_t k, bool q) {
        t.add(name + ".weight", n_out, k, q, c.wtype);
        t.add(name + ".bias", 1, n_out, false, c.wtype);
    };
    // Quantised: every 2-D weight except biases, norm weights and names containing "embedding"
    // (tensor_should_be_converted, reference src/core/runtime/model_loader.cpp:2141-2172).
    lin("patch_embedding", D, pf, false);   // Conv3d (1,2,2) as its [D, in_dim*pt*ph*pw] matrix
    lin("text_embedding.0", D, c.text_dim, false);
    lin("text_embedding.2", D, D, false);
    lin("time_embedding.0", D, c.freq_dim, false);
    lin("time_embedding.2", D, D, false);
    lin("time_projection.1", 6 * D, D, true);
    for (int i = 0; i < c.num_layers; ++i) {
        const std::string p = "blocks." + std::to_string(i) + ".";
        t.add(p + "modulation", 6, D, false, c.wtype);
        for (const char* a : {"self_attn", "cross_attn"}) {
            for (const char* l : {"q", "k", "v", "o"}) lin(p + a + "." + l, D, D, true);
            t.add(p + a + ".norm_q.weight", 1, D, false, c.wtype);
            t.add(p + a + ".norm_k.weight", 1, D, false, c.wtype);
        }
        t.add(p + "norm3.weight", 1, D, false, c.wtype);
        t.add(p + "norm3.bias", 1, D, false, c.wtype);
        lin(p + "ffn.0", F, D, true);
        lin(p + "ffn.2", D, F, true);
    }
    t.add("head.modulation", 2, D, false, c.wtype);
    lin("head.head", (int64_t)c.out_dim * c.patch_size[0] * c.patch_size[1] * c.patch_size[2], D, true);
}

// pe[L, d/2, 2, 2] for token ids (t, h, w), w fastest (gen_vid_ids / gen_wan_pe,
// reference src/dit_models/components/common/rope.hpp:570-622; Rope::rope :77-127).
std::vector<float> build_wan_pe(const edb200_wan_config_t& c, int t_len, int h_len, int w_len) {
    const int64_t L = (int64_t)t_len * h_len * w_len;
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
        for (int64_t t = 0; t < L; ++t) {
            const int64_t it = t / ((int64_t)h_len * w_len), ih = (t / w_len) % h_len, iw = t % w_len;
            const float pos = static_cast<float>(a == 0 ? it : a == 1 ? ih : iw);
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

// latent [C, T, H, W] -> tokens [(t, h, w)][c*ph*pw*pt...]: feature (c, kt, kh, kw), the Conv3d
// (kernel = stride = patch) seen as a linear layer.
__global__ void patchify3d_kernel(const float* __restrict__ lat, float* __restrict__ tok, int C, int T, int H, int W,
                                  int pt, int ph, int pw) {
    const int64_t total = (int64_t)C * T * H * W;
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const int w = static_cast<int>(i % W), h = static_cast<int>((i / W) % H);
    const int t = static_cast<int>((i / ((int64_t)W * H)) % T), c = static_cast<int>(i / ((int64_t)W * H * T));
    const int h_len = H / ph, w_len = W / pw;
    const int64_t token = ((int64_t)(t / pt) * h_len + h / ph) * w_len + w / pw;
    const int feat = ((c * pt + t % pt) * ph + h % ph) * pw + w % pw;
    tok[token * ((int64_t)C * pt * ph * pw) + feat] = lat[i];
}

// tokens [L, pt*ph*pw*C] with feature = c + C*(kw + pw*(kh + ph*kt)) -> [C, T, H, W]
// (Wan::unpatchify, wan.hpp:4489-4514).
__global__ void unpatchify3d_kernel(const float* __restrict__ tok, float* __restrict__ lat, int C, int T, int H, int W,
                                    int pt, int ph, int pw) {
    const int64_t total = (int64_t)C * T * H * W;
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const int w = static_cast<int>(i % W), h = static_cast<int>((i / W) % H);
    const int t = static_cast<int>((i / ((int64_t)W * H)) % T), c = static_cast<int>(i / ((int64_t)W * H * T));
    const int h_len = H / ph, w_len = W / pw;
    const int64_t token = ((int64_t)(t / pt) * h_len + h / ph) * w_len + w / pw;
    const int feat = c + C * ((w % pw) + pw * ((h % ph) + ph * (t % pt)));
    lat[i] = tok[token * ((int64_t)C * pt * ph * pw) + feat];
}

// es[layer][j][:] = e0[j][:] + modulation_layer[j][:] for all layers; hm[j][:] = e[:] + head.modulation[j][:]
__global__ void add_rows_kernel(const float* __restrict__ a, int a_rows, const float* __restrict__ b, float* __restrict__ out,
                                int64_t n, int D) {
    // out[i] = a[(i / D) % a_rows][i % D] + b[i]
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    out[i] = a[((i / D) % a_rows) * D + i % D] + b[i];
}

__global__ void fill_kernel(float* p, int64_t n, float v) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) p[i] = v;
}

edb200_status_t ln_mod(const float* x, int64_t D, const float* shift, const float* scale, const float* w, const float* b,
                       int64_t rows, void* y, int y_dtype, cudaStream_t s) {
    if (rows == 0) return EDB200_OK;
    return edb200_layernorm_modulate(x, D, shift, scale, w, b, rows, D, 1e-6f, y, y_dtype, D, s);
}

}  // namespace

namespace {

// Self-attention over the whole clip (see edb200_flux.cu for the single-GPU / NCCL / peer-memory cases).
edb200_status_t self_attention(edb200_wan* m, int layer, cudaStream_t s) {
    const edb200_wan_config_t& c = m->cfg;
    const int d = c.dim / c.num_heads;
    const int heads = c.num_heads / m->world;
    const float scale = 1.0f / std::sqrt(static_cast<float>(d));
    const int flags = (c.sage_smooth_q ? EDB200_SAGE_SMOOTH_Q : 0) | EDB200_SAGE_FAST_MEANS;
    // INT8 scores only on the middle layers: the first sage_skip_first and the last sage_skip_last stay f16
    // (sage_attn_skip_layer, reference src/core/backend/ggml/ed_ggml_sage_attn_ext.hpp:146-159; the layer
    // index reaches it from WanAttentionBlock, wan.hpp:4673-4674)
    const bool sage = c.attention == EDB200_ATTN_SAGE_INT8 && layer >= c.sage_skip_first &&
                      layer < c.num_layers - c.sage_skip_last;
    const int64_t head_rows = m->world > 1 ? m->t_loc * m->world : m->T;   // padded sequence under SP
    if (m->p2p) {
        EDB_TRY(edb200_sp_barrier(m->comm, s));
        if (sage) {
            EDB_TRY(edb200_sage_attention_strided(m->Q, m->K, m->V, heads, m->T, head_rows, d, scale, flags, m->SAGE,
                                                  m->sage_bytes, nullptr, EDB200_TYPE_F16, c.dim, &m->att_peers, s));
        } else {
            EDB_TRY(edb200_attention_f16_strided(m->Q, m->K, m->V, heads, m->T, m->T, head_rows, head_rows, d, scale,
                                                 nullptr, EDB200_TYPE_F16, c.dim, &m->att_peers, s));
        }
        return edb200_sp_barrier(m->comm, s);
    }
    void* att_out = m->ATT;
    int64_t att_ld = c.dim;
    if (m->world > 1) {
        const void* send[3] = {m->QL, m->KL, m->VL};
        void* recv[3] = {m->Q, m->K, m->V};
        EDB_TRY(edb200_sp_all_to_all_heads(m->comm, send, recv, 3, c.num_heads, m->t_loc, (int64_t)d * 2, s));
        att_out = m->AOUT;
        att_ld = (int64_t)heads * d;
    }
    if (sage) {
        EDB_TRY(edb200_sage_attention_strided(m->Q, m->K, m->V, heads, m->T, head_rows, d, scale, flags, m->SAGE,
                                              m->sage_bytes, att_out, EDB200_TYPE_F16, att_ld, nullptr, s));
    } else {
        EDB_TRY(edb200_attention_f16_strided(m->Q, m->K, m->V, heads, m->T, m->T, head_rows, head_rows, d, scale, att_out,
                                             EDB200_TYPE_F16, att_ld, nullptr, s));
    }
    if (m->world > 1) {
        EDB_TRY(edb200_sp_all_to_all_tokens(m->comm, m->AOUT, m->STG, m->ATT, m->t_loc, (int64_t)heads * d * 2,
                                            (int64_t)c.dim * 2, s));
    }
    return EDB200_OK;
}

}  // namespace

extern "C" {

edb200_status_t edb200_wan_create(const edb200_wan_config_t* cfg, edb200_wan_t** out) {
    if (cfg == nullptr || out == nullptr) return fail(EDB200_ERR_INVALID, "wan_create: null argument");
    const edb200_wan_config_t& c = *cfg;
    if (c.dim <= 0 || c.num_heads <= 0 || c.dim % c.num_heads || c.num_layers <= 0) {
        return fail(EDB200_ERR_INVALID, "wan_create: dim must be a positive multiple of num_heads");
    }
    const int d = c.dim / c.num_heads;
    if (d != 64 && d != 128) return fail(EDB200_ERR_UNSUPPORTED, "wan_create: head dim must be 64 or 128");
    if (c.axes_dim[0] + c.axes_dim[1] + c.axes_dim[2] != d) {
        return fail(EDB200_ERR_INVALID, "wan_create: axes_dim must sum to the head dim");
    }
    if (c.wtype != EDB200_TYPE_Q8_0 && c.wtype != EDB200_TYPE_Q4_K) {
        return fail(EDB200_ERR_UNSUPPORTED, "wan_create: wtype must be q8_0 or q4_K");
    }
    if (c.dim % 256 || c.ffn_dim % 256 || c.dim > 8192) {
        return fail(EDB200_ERR_UNSUPPORTED, "wan_create: dim (<= 8192) and ffn_dim must be multiples of 256");
    }
    if (c.attention == EDB200_ATTN_SAGE_INT8 && d != 128) {
        return fail(EDB200_ERR_UNSUPPORTED, "wan_create: INT8 attention needs head dim 128");
    }
    const int pf = c.out_dim * c.patch_size[0] * c.patch_size[1] * c.patch_size[2];
    if (c.patch_size[0] <= 0 || c.patch_size[1] <= 0 || c.patch_size[2] <= 0 || pf % 32 || c.text_dim % 4 ||
        c.freq_dim != 256 || (c.in_dim * c.patch_size[0] * c.patch_size[1] * c.patch_size[2]) % 4) {
        return fail(EDB200_ERR_UNSUPPORTED,
                    "wan_create: freq_dim must be 256, out_dim * patch volume a multiple of 32, text_dim of 4");
    }
    if (device_error_word() == nullptr) return fail(EDB200_ERR_CUDA, "wan_create: no CUDA device");
    edb200_wan* m = new (std::nothrow) edb200_wan();
    if (m == nullptr) return fail(EDB200_ERR_NOMEM, "wan_create: host allocation failed");
    m->cfg = c;
    register_params(m);
    *out = m;
    return EDB200_OK;
}

void edb200_wan_destroy(edb200_wan_t* m) {
    if (m == nullptr) return;
    if (m->pinned) cudaFreeHost(m->pinned);
    delete m;
}

int edb200_wan_tensor_count(const edb200_wan_t* m) {
    return m ? static_cast<int>(const_cast<edb200_wan_t*>(m)->params.params().size()) : 0;
}

edb200_status_t edb200_wan_tensor_info(const edb200_wan_t* m, int index, char* name, int name_cap, int* ggml_type,
                                       int64_t* n_out, int64_t* k, int64_t* nbytes) {
    if (m == nullptr || index < 0 || index >= edb200_wan_tensor_count(m)) {
        return fail(EDB200_ERR_INVALID, "wan_tensor_info: bad index");
    }
    const Param& p = const_cast<edb200_wan_t*>(m)->params.params()[index];
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

edb200_status_t edb200_wan_set_tensor(edb200_wan_t* m, const char* name, int ggml_type, const void* data, int64_t nbytes,
                                      int on_device, void* stream) {
    if (m == nullptr || name == nullptr) return fail(EDB200_ERR_INVALID, "wan_set_tensor: null argument");
    return m->params.set(name, ggml_type, data, nbytes, on_device != 0, static_cast<cudaStream_t>(stream));
}

edb200_status_t edb200_wan_get_tensor_f32(const edb200_wan_t* m, const char* name, float* out, int64_t n_floats,
                                          int on_device, void* stream) {
    if (m == nullptr || name == nullptr) return fail(EDB200_ERR_INVALID, "wan_get_tensor_f32: null argument");
    return m->params.fetch_f32(name, out, n_floats, on_device != 0, static_cast<cudaStream_t>(stream));
}

edb200_status_t edb200_wan_load_gguf(edb200_wan_t* m, const char* path, const char* strip_prefix, int* n_loaded,
                                    void* stream) {
    if (m == nullptr || path == nullptr) return fail(EDB200_ERR_INVALID, "wan_load_gguf: null argument");
    return load_gguf(m->params, EDB200_FAMILY_WAN, path, strip_prefix, static_cast<cudaStream_t>(stream), n_loaded);
}

edb200_status_t edb200_wan_load_safetensors(edb200_wan_t* m, const char* path, const char* strip_prefix, int* n_loaded,
                                           void* stream) {
    if (m == nullptr || path == nullptr) return fail(EDB200_ERR_INVALID, "wan_load_safetensors: null argument");
    return load_safetensors(m->params, EDB200_FAMILY_WAN, path, strip_prefix, static_cast<cudaStream_t>(stream), n_loaded);
}

edb200_status_t edb200_wan_init_random(edb200_wan_t* m, uint64_t seed, float std, void* stream) {
    if (m == nullptr) return fail(EDB200_ERR_INVALID, "wan_init_random: null model");
    return m->params.init_random(seed, std, static_cast<cudaStream_t>(stream));
}

int64_t edb200_wan_weight_bytes(const edb200_wan_t* m) { return m ? m->params.device_bytes() : 0; }
int64_t edb200_wan_workspace_bytes(const edb200_wan_t* m) { return m ? m->ws.capacity() : 0; }

edb200_status_t edb200_wan_set_anchor_capture(edb200_wan_t* m, int anchor, float* dst) {
    if (m == nullptr) return fail(EDB200_ERR_INVALID, "wan_set_anchor_capture: null model");
    return m->anchors.set_capture(anchor, dst, m->cfg.num_layers, "wan");
}

edb200_status_t edb200_wan_set_stop_after(edb200_wan_t* m, int block) {
    if (m == nullptr) return fail(EDB200_ERR_INVALID, "wan_set_stop_after: null model");
    return m->anchors.set_stop(block, m->cfg.num_layers, "wan");
}

edb200_status_t edb200_wan_set_stream_override(edb200_wan_t* m, const float* residual) {
    if (m == nullptr) return fail(EDB200_ERR_INVALID, "wan_set_stream_override: null model");
    m->anchors.stream_override = residual;
    return EDB200_OK;
}

edb200_status_t edb200_wan_set_region_inject(edb200_wan_t* m, int at, int resume, const float* residual) {
    if (m == nullptr) return fail(EDB200_ERR_INVALID, "wan_set_region_inject: null model");
    return m->anchors.set_region(at, resume, residual, m->cfg.num_layers, "wan");
}

edb200_status_t edb200_wan_set_tap(edb200_wan_t* m, float* tap) {
    if (m == nullptr) return fail(EDB200_ERR_INVALID, "wan_set_tap: null model");
    m->tap = tap;
    return EDB200_OK;
}

edb200_status_t edb200_wan_set_comm(edb200_wan_t* m, edb200_comm_t* comm) {
    if (m == nullptr) return fail(EDB200_ERR_INVALID, "wan_set_comm: null model");
    if (m->comm != nullptr && m->comm != comm) edb200_comm_unmap_peers(m->comm);   // collective
    m->comm = comm;
    m->rank = comm ? edb200_comm_rank(comm) : 0;
    m->world = comm ? edb200_comm_world(comm) : 1;
    m->frames = m->lat_h = m->lat_w = m->n_ctx = 0;   // the workspace must be prepared again
    m->p2p = false;
    return EDB200_OK;
}

edb200_status_t edb200_wan_prepare(edb200_wan_t* m, int frames, int lat_h, int lat_w, int n_ctx, void* stream) {
    if (m == nullptr) return fail(EDB200_ERR_INVALID, "wan_prepare: null model");
    const edb200_wan_config_t& c = m->cfg;
    const int pt = c.patch_size[0], ph = c.patch_size[1], pw = c.patch_size[2];
    if (frames <= 0 || lat_h <= 0 || lat_w <= 0 || n_ctx <= 0 || frames % pt || lat_h % ph || lat_w % pw) {
        return fail(EDB200_ERR_INVALID, "wan_prepare: latent must be a positive multiple of the patch size");
    }
    if (m->frames == frames && m->lat_h == lat_h && m->lat_w == lat_w && m->n_ctx == n_ctx) return EDB200_OK;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int64_t D = c.dim, F = c.ffn_dim, d = D / c.num_heads;
    const int t_len = frames / pt, h_len = lat_h / ph, w_len = lat_w / pw;
    const int64_t T = (int64_t)t_len * h_len * w_len;
    const int64_t pf_in = (int64_t)c.in_dim * pt * ph * pw, pf_out = (int64_t)c.out_dim * pt * ph * pw;
    int64_t TL = T, t_rows = T;   // TL: rows of a rank's slot (buffers are laid out for it), t_rows: rows owned
    if (m->world > 1) {
        if (c.num_heads % m->world) {
            return fail(EDB200_ERR_UNSUPPORTED, "wan_prepare: %d heads do not divide over %d ranks", c.num_heads, m->world);
        }
        EDB_TRY(edb200_sp_shard(T, 0, m->rank, m->world, &TL, nullptr, nullptr, &t_rows));
        if (t_rows == 0) return fail(EDB200_ERR_UNSUPPORTED, "wan_prepare: %lld tokens leave rank %d without rows", (long long)T, m->rank);
    }
    const int64_t sage =
        c.attention == EDB200_ATTN_SAGE_INT8 ? edb200_sage_scratch_bytes(c.num_heads / m->world, T, (int)d) : 0;
    const int64_t lat_in = (int64_t)c.in_dim * frames * lat_h * lat_w, lat_out = (int64_t)c.out_dim * frames * lat_h * lat_w;
    const int64_t pe_elems = T * (d / 2) * 4;
    auto al = [](int64_t b) { return (b + 255) & ~int64_t(255); };
    int64_t total = al(TL * D * 4) + al(TL * D * 2) + al(TL * 3 * D * 2) + 6 * al(TL * D * 2) + al(TL * F * 2);
    total += al(n_ctx * D * 4) * 2 + al(n_ctx * D * 2) * 3 + al(n_ctx * 2 * D * 2);
    total += al(6 * D * 4) * 2 + al(D * 4) * 2 + al(2 * D * 4) * 2 + al(256 * 4) + al(128 * 4) + al(pe_elems * 4);
    total += al((2 * TL + n_ctx) * 4) + al(T * pf_in * 4) + 2 * al(T * pf_out * 4) + al(lat_in * 4) + al(lat_out * 4);
    total += al((int64_t)n_ctx * c.text_dim * 4) + al(sage) + 8192;
    if (m->world > 1) total += 6 * al(TL * D * 2) + 2048;
    cudaStreamSynchronize(s);
    if (m->comm != nullptr) EDB_TRY(edb200_comm_unmap_peers(m->comm));   // collective; the old workspace goes away
    m->p2p = false;
    EDB_TRY(m->ws.reserve(total));
    Workspace& w = m->ws;
    m->X = w.take_n<float>(TL * D);
    m->XMOD = w.take(TL * D * 2);
    m->QKV = w.take(TL * 3 * D * 2);
    m->Q = w.take(TL * D * 2);
    m->K = w.take(TL * D * 2);
    m->V = w.take(TL * D * 2);
    m->ATT = w.take(TL * D * 2);
    m->KVC = w.take((int64_t)n_ctx * 2 * D * 2);
    m->HID = w.take(TL * F * 2);
    m->CTX32 = w.take_n<float>((int64_t)n_ctx * D);
    m->TMP = w.take_n<float>((int64_t)n_ctx * D > 2 * D ? (int64_t)n_ctx * D : 2 * D);
    m->CTXE = w.take((int64_t)n_ctx * D * 2);
    m->KC = w.take((int64_t)n_ctx * D * 2);
    m->VC = w.take((int64_t)n_ctx * D * 2);
    m->ES = w.take_n<float>(6 * D);
    m->E0 = w.take_n<float>(6 * D);
    m->E = w.take_n<float>(D);
    m->ONES = w.take_n<float>(D);
    m->HMOD = w.take_n<float>(2 * D);
    float* spare = w.take_n<float>(2 * D);
    (void)spare;
    m->TEMB = w.take_n<float>(256);
    m->FREQ = w.take_n<float>(128);
    m->PE = w.take_n<float>(pe_elems);
    m->RSTD = w.take_n<float>(2 * TL + n_ctx);
    m->TOK_IN = w.take_n<float>(T * pf_in);
    m->TOK_OUT = w.take_n<float>(T * pf_out);
    m->TOK_LOC = w.take_n<float>(T * pf_out);
    m->LAT_IN = w.take_n<float>(lat_in);
    m->LAT_OUT = w.take_n<float>(lat_out);
    m->CTX_IN = w.take_n<float>((int64_t)n_ctx * c.text_dim);
    m->SAGE = sage > 0 ? w.take(sage) : nullptr;
    m->sage_bytes = sage;
    if (m->CTX_IN == nullptr || (sage > 0 && m->SAGE == nullptr)) {
        return fail(EDB200_ERR_NOMEM, "wan_prepare: workspace accounting error");
    }
    m->QL = m->KL = m->VL = m->AOUT = m->STG = nullptr;
    // the cross-attention queries get a buffer of their own: under the peer-memory exchange the
    // peers may already be storing the next block's Q/K/V into m->Q/K/V
    m->QX = w.take(TL * D * 2);
    if (m->QX == nullptr) return fail(EDB200_ERR_NOMEM, "wan_prepare: workspace accounting error");
    if (m->world > 1) {
        void* flags = w.take(1024);   // barrier flags + epoch
        m->QL = w.take(TL * D * 2);
        m->KL = w.take(TL * D * 2);
        m->VL = w.take(TL * D * 2);
        m->AOUT = w.take(TL * D * 2);
        m->STG = w.take(TL * D * 2);
        if (flags == nullptr || m->STG == nullptr) return fail(EDB200_ERR_NOMEM, "wan_prepare: workspace accounting error");
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
            m->qkv_peers.t_loc = m->att_peers.t_loc = TL;
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
    std::vector<float> pe = build_wan_pe(c, t_len, h_len, w_len);
    std::vector<float> freq(128);
    for (int i = 0; i < 128; ++i) freq[i] = (float)std::exp(-std::log(10000) * i / 128);
    cudaError_t e = cudaMemcpyAsync(m->PE, pe.data(), pe.size() * 4, cudaMemcpyHostToDevice, s);
    if (e == cudaSuccess) e = cudaMemcpyAsync(m->FREQ, freq.data(), 128 * 4, cudaMemcpyHostToDevice, s);
    fill_kernel<<<static_cast<unsigned>((D + 255) / 256), 256, 0, s>>>(m->ONES, D, 1.0f);
    count_launch();
    if (e == cudaSuccess) e = cudaStreamSynchronize(s);
    if (e != cudaSuccess) return check_cuda(e, "wan_prepare upload");
    const int64_t need = (lat_in + lat_out + (int64_t)n_ctx * c.text_dim) * 4;
    if (need > m->pinned_bytes) {
        if (m->pinned) cudaFreeHost(m->pinned);
        m->pinned = nullptr;
        e = cudaMallocHost(reinterpret_cast<void**>(&m->pinned), need);
        if (e != cudaSuccess) return fail(EDB200_ERR_NOMEM, "wan_prepare: cudaMallocHost: %s", cudaGetErrorString(e));
        m->pinned_bytes = need;
    }
    m->frames = frames;
    m->lat_h = lat_h;
    m->lat_w = lat_w;
    m->n_ctx = n_ctx;
    m->T = T;
    m->t_loc = TL;
    m->t_rows = t_rows;
    return EDB200_OK;
}

static edb200_status_t wan_step_body(edb200_wan_t* m, const float* latent, float timestep, const float* sched,
                                     const int* sched_step, float t_scale, const float* context, float* out, void* stream) {
    if (m == nullptr || latent == nullptr || context == nullptr || out == nullptr) {
        return fail(EDB200_ERR_INVALID, "wan_step: null argument");
    }
    if (m->frames == 0) return fail(EDB200_ERR_INVALID, "wan_step: call edb200_wan_prepare first");
    EDB_TRY(m->params.all_loaded());
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const edb200_wan_config_t& c = m->cfg;
    // TL: rows this rank owns (computed on); SL: rows of a rank's slot of the padded sequence (layout)
    const int64_t D = c.dim, F = c.ffn_dim, T = m->T, TL = m->t_rows, SL = m->t_loc, n_ctx = m->n_ctx;
    const int d = static_cast<int>(D / c.num_heads);
    const int pt = c.patch_size[0], ph = c.patch_size[1], pw = c.patch_size[2];
    const int64_t pf_in = (int64_t)c.in_dim * pt * ph * pw, pf_out = (int64_t)c.out_dim * pt * ph * pw;
    const int64_t first = (int64_t)m->rank * SL;   // first token this rank owns
    const int F16 = EDB200_TYPE_F16;
    __half* xmod = static_cast<__half*>(m->XMOD);
    __half* qkv = static_cast<__half*>(m->QKV);
    __half* kvc = static_cast<__half*>(m->KVC);
    __half* att = static_cast<__half*>(m->ATT);
    __half* hid = static_cast<__half*>(m->HID);
    const bool sp = m->world > 1;

    // ---- prelude (Wan::forward_orig, wan.hpp:4545-4567)
    {
        const int64_t total = (int64_t)c.in_dim * m->frames * m->lat_h * m->lat_w;
        patchify3d_kernel<<<static_cast<unsigned>((total + 255) / 256), 256, 0, s>>>(latent, m->TOK_IN, c.in_dim, m->frames,
                                                                                     m->lat_h, m->lat_w, pt, ph, pw);
        count_launch();
    }
    EDB_TRY(dense(m, "patch_embedding", m->TOK_IN + first * pf_in, TL, pf_in, 0, EDB200_ACT_NONE, m->X, D, s));
    if (sched != nullptr) {
        launch_timestep_embedding_sched(m->FREQ, sched, sched_step, t_scale, 1.0f, 128, m->TEMB, s);
    } else {
        launch_timestep_embedding(m->FREQ, timestep, 1.0f, 128, m->TEMB, s);
    }
    EDB_TRY(dense(m, "time_embedding.0", m->TEMB, 1, 256, 0, EDB200_ACT_SILU, m->TMP, D, s));
    EDB_TRY(dense(m, "time_embedding.2", m->TMP, 1, D, 0, EDB200_ACT_NONE, m->E, D, s));
    {
        const Lin l = qlin(m, "time_projection.1");
        EDB_TRY(edb200_gemv_q(l.w, m->E, 1, D, 1, l.b, m->E0, 6 * D, s));
    }
    add_rows_kernel<<<static_cast<unsigned>((2 * D + 255) / 256), 256, 0, s>>>(m->E, 1, fparam(m, "head.modulation"),
                                                                               m->HMOD, 2 * D, static_cast<int>(D));
    count_launch();
    EDB_TRY(dense(m, "text_embedding.0", context, n_ctx, c.text_dim, 0, EDB200_ACT_GELU_ERF, m->TMP, D, s));
    EDB_TRY(dense(m, "text_embedding.2", m->TMP, n_ctx, D, 0, EDB200_ACT_NONE, m->CTX32, D, s));
    EDB_TRY(edb200_cast(m->CTX32, EDB200_TYPE_F32, m->CTXE, F16, n_ctx * D, s));

    m->anchors.capture_in(m->X, TL * D, s);
    // ---- blocks (WanAttentionBlock::forward, wan.hpp:4136-4187)
    for (int i = 0; i < (m->anchors.inject() ? 0 : c.num_layers); ++i) {
        if (m->anchors.region_inject(i, m->X, TL * D, s)) continue;   // skip a cached span of blocks
        const std::string p = "blocks." + std::to_string(i) + ".";
        add_rows_kernel<<<static_cast<unsigned>((6 * D + 255) / 256), 256, 0, s>>>(m->E0, 6, fparam(m, p + "modulation"),
                                                                                   m->ES, 6 * D, static_cast<int>(D));
        count_launch();
        const float* es = m->ES;   // shift1 scale1 gate1 shift2 scale2 gate2

        // self-attention
        EDB_TRY(ln_mod(m->X, D, es, es + D, nullptr, nullptr, TL, xmod, F16, s));
        {
            const Lin lq = qlin(m, p + "self_attn.q"), lk = qlin(m, p + "self_attn.k"), lv = qlin(m, p + "self_attn.v");
            edb200_epilogue_t eq = make_ep(qkv, F16, 3 * D, lq.b);
            edb200_epilogue_t ek = make_ep(qkv + D, F16, 3 * D, lk.b);
            edb200_epilogue_t ev = make_ep(qkv + 2 * D, F16, 3 * D, lv.b);
            EDB_TRY(edb200_mul_mat_q_pair(lq.w, xmod, TL, D, &eq, lk.w, xmod, TL, D, &ek, F16, s));
            EDB_TRY(edb200_mul_mat_q(lv.w, xmod, F16, TL, D, &ev, s));
        }
        EDB_TRY(edb200_row_rstd(qkv, F16, 3 * D, TL, D, 1e-6f, m->RSTD, s));
        EDB_TRY(edb200_row_rstd(qkv + D, F16, 3 * D, TL, D, 1e-6f, m->RSTD + TL, s));
        {
            const float* wq = fparam(m, p + "self_attn.norm_q.weight");
            const float* wk = fparam(m, p + "self_attn.norm_k.weight");
            if (m->p2p) {
                EDB_TRY(edb200_qk_rownorm_rope_pack(qkv, F16, 3 * D, 0, D, 2 * D, TL, c.num_heads, d, wq, wk, m->RSTD,
                                                    m->RSTD + TL, m->PE, 0, SL * m->world, nullptr, nullptr, nullptr, F16,
                                                    &m->qkv_peers, s));
            } else {
                // NCCL exchange: local head-major buffers, position rows of this rank's tokens
                const float* pe = m->PE + first * (d / 2) * 4;
                EDB_TRY(edb200_qk_rownorm_rope_pack(qkv, F16, 3 * D, 0, D, 2 * D, TL, c.num_heads, d, wq, wk, m->RSTD,
                                                    m->RSTD + TL, pe, 0, SL, sp ? m->QL : m->Q, sp ? m->KL : m->K,
                                                    sp ? m->VL : m->V, F16, nullptr, s));
            }
        }
        EDB_TRY(self_attention(m, i, s));
        {
            const Lin lo = qlin(m, p + "self_attn.o");
            edb200_epilogue_t ep = make_ep(m->X, EDB200_TYPE_F32, D, lo.b);
            ep.residual = m->X, ep.ld_res = D, ep.gate = es + 2 * D;
            EDB_TRY(edb200_mul_mat_q(lo.w, att, F16, TL, D, &ep, s));
        }

        // cross-attention with the embedded text: local query rows, every head, no exchange
        EDB_TRY(ln_mod(m->X, D, nullptr, nullptr, fparam(m, p + "norm3.weight"), fparam(m, p + "norm3.bias"), TL, xmod, F16, s));
        {
            const Lin lq = qlin(m, p + "cross_attn.q");
            edb200_epilogue_t eq = make_ep(qkv, F16, 3 * D, lq.b);
            EDB_TRY(edb200_mul_mat_q(lq.w, xmod, F16, TL, D, &eq, s));
            const Lin lk = qlin(m, p + "cross_attn.k"), lv = qlin(m, p + "cross_attn.v");
            edb200_epilogue_t ek = make_ep(kvc, F16, 2 * D, lk.b);
            edb200_epilogue_t ev = make_ep(kvc + D, F16, 2 * D, lv.b);
            EDB_TRY(edb200_mul_mat_q_pair(lk.w, m->CTXE, n_ctx, D, &ek, lv.w, m->CTXE, n_ctx, D, &ev, F16, s));
        }
        EDB_TRY(edb200_row_rstd(qkv, F16, 3 * D, TL, D, 1e-6f, m->RSTD, s));
        EDB_TRY(edb200_row_rstd(kvc, F16, 2 * D, n_ctx, D, 1e-6f, m->RSTD + 2 * TL, s));
        EDB_TRY(edb200_qk_rownorm_rope_pack(qkv, F16, 3 * D, 0, 0, 0, TL, c.num_heads, d,
                                            fparam(m, p + "cross_attn.norm_q.weight"), nullptr, m->RSTD, nullptr, nullptr,
                                            0, TL, m->QX, nullptr, nullptr, F16, nullptr, s));
        EDB_TRY(edb200_qk_rownorm_rope_pack(kvc, F16, 2 * D, 0, 0, D, n_ctx, c.num_heads, d, nullptr,
                                            fparam(m, p + "cross_attn.norm_k.weight"), nullptr, m->RSTD + 2 * TL, nullptr,
                                            0, n_ctx, nullptr, m->KC, m->VC, F16, nullptr, s));
        EDB_TRY(edb200_attention_f16(m->QX, m->KC, m->VC, c.num_heads, TL, n_ctx, d, 1.0f / std::sqrt((float)d), att, F16,
                                     D, s));
        {
            const Lin lo = qlin(m, p + "cross_attn.o");
            edb200_epilogue_t ep = make_ep(m->X, EDB200_TYPE_F32, D, lo.b);
            ep.residual = m->X, ep.ld_res = D, ep.gate = m->ONES;
            EDB_TRY(edb200_mul_mat_q(lo.w, att, F16, TL, D, &ep, s));
        }

        // feed-forward
        EDB_TRY(ln_mod(m->X, D, es + 3 * D, es + 4 * D, nullptr, nullptr, TL, xmod, F16, s));
        {
            const Lin l0 = qlin(m, p + "ffn.0"), l2 = qlin(m, p + "ffn.2");
            edb200_epilogue_t e0 = make_ep(hid, F16, F, l0.b);
            e0.act = EDB200_ACT_GELU_TANH;
            EDB_TRY(edb200_mul_mat_q(l0.w, xmod, F16, TL, D, &e0, s));
            edb200_epilogue_t e2 = make_ep(m->X, EDB200_TYPE_F32, D, l2.b);
            e2.residual = m->X, e2.ld_res = D, e2.gate = es + 5 * D;
            EDB_TRY(edb200_mul_mat_q(l2.w, hid, F16, TL, F, &e2, s));
        }
        if (m->tap) cudaMemcpyAsync(m->tap + (int64_t)i * TL * D, m->X, TL * D * 4, cudaMemcpyDeviceToDevice, s);
        m->anchors.capture_block(i, m->X, TL * D, s);
        if (m->anchors.stop_after == i) return check_cuda(cudaGetLastError(), "wan_step");
    }

    m->anchors.finish(m->X, TL * D, s);   // whole-stack inject, ModelOut

    // ---- head (Head::forward, wan.hpp:4309-4330) + unpatchify (:4489-4514)
    EDB_TRY(ln_mod(m->X, D, m->HMOD, m->HMOD + D, nullptr, nullptr, TL, xmod, F16, s));
    {
        const Lin lh = qlin(m, "head.head");
        edb200_epilogue_t ep = make_ep(sp ? m->TOK_LOC : m->TOK_OUT, EDB200_TYPE_F32, pf_out, lh.b);
        EDB_TRY(edb200_mul_mat_q(lh.w, xmod, F16, TL, D, &ep, s));
    }
    if (sp) {
        std::vector<int64_t> firsts(m->world), counts(m->world);
        for (int r = 0; r < m->world; ++r) {
            firsts[r] = std::min<int64_t>((int64_t)r * SL, T);
            counts[r] = std::min<int64_t>(SL, T - firsts[r]);
        }
        if (m->p2p) {
            // peer stores + barrier: nothing of the step goes through a library exchange
            EDB_TRY(edb200_sp_all_gather_rows_peer(m->comm, m->TOK_LOC, m->TOK_OUT, firsts.data(), counts.data(), pf_out * 4, s));
        } else {
            EDB_TRY(edb200_sp_all_gather_rows(m->comm, m->TOK_LOC, m->TOK_OUT, firsts.data(), counts.data(), pf_out * 4, s));
        }
    }
    {
        const int64_t total = (int64_t)c.out_dim * m->frames * m->lat_h * m->lat_w;
        unpatchify3d_kernel<<<static_cast<unsigned>((total + 255) / 256), 256, 0, s>>>(m->TOK_OUT, out, c.out_dim, m->frames,
                                                                                       m->lat_h, m->lat_w, pt, ph, pw);
        count_launch();
    }
    return check_cuda(cudaGetLastError(), "wan_step");
}

edb200_status_t edb200_wan_step(edb200_wan_t* m, const float* latent, float timestep, const float* context, float* out,
                                void* stream) {
    return wan_step_body(m, latent, timestep, nullptr, nullptr, 1.0f, context, out, stream);
}

edb200_status_t edb200_wan_step_sched(edb200_wan_t* m, const float* latent, const float* sigmas, const int* step, float t_scale,
                                      const float* context, float* out, void* stream) {
    if (sigmas == nullptr || step == nullptr) return fail(EDB200_ERR_INVALID, "wan_step_sched: null schedule");
    return wan_step_body(m, latent, 0.0f, sigmas, step, t_scale, context, out, stream);
}

edb200_status_t edb200_wan_compute_host(edb200_wan_t* m, const float* latent, int frames, int lat_h, int lat_w,
                                        float timestep, const float* context, int n_ctx, float* out, void* stream) {
    if (m == nullptr || latent == nullptr || context == nullptr || out == nullptr) {
        return fail(EDB200_ERR_INVALID, "wan_compute_host: null argument");
    }
    EDB_TRY(edb200_wan_prepare(m, frames, lat_h, lat_w, n_ctx, stream));
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const edb200_wan_config_t& c = m->cfg;
    const int64_t lat_in = (int64_t)c.in_dim * frames * lat_h * lat_w, lat_out = (int64_t)c.out_dim * frames * lat_h * lat_w;
    const int64_t ctx_elems = (int64_t)n_ctx * c.text_dim;
    float* p_lat = m->pinned;
    float* p_ctx = p_lat + lat_in;
    float* p_out = p_ctx + ctx_elems;
    memcpy(p_lat, latent, lat_in * 4);
    memcpy(p_ctx, context, ctx_elems * 4);
    cudaError_t e = cudaMemcpyAsync(m->LAT_IN, p_lat, lat_in * 4, cudaMemcpyHostToDevice, s);
    if (e == cudaSuccess) e = cudaMemcpyAsync(m->CTX_IN, p_ctx, ctx_elems * 4, cudaMemcpyHostToDevice, s);
    if (e != cudaSuccess) return check_cuda(e, "wan_compute_host H2D");
    EDB_TRY(edb200_wan_step(m, m->LAT_IN, timestep, m->CTX_IN, m->LAT_OUT, stream));
    e = cudaMemcpyAsync(p_out, m->LAT_OUT, lat_out * 4, cudaMemcpyDeviceToHost, s);
    if (e != cudaSuccess) return check_cuda(e, "wan_compute_host D2H");
    EDB_TRY(poll_device_error(s));   // synchronises the stream
    memcpy(out, p_out, lat_out * 4);
    return EDB200_OK;
}

}  // extern "C"
