// Weight ingest shared by the GGUF and safetensors readers: tensor-name canonicalisation, assembly of
// fused tensors from their parts, and conversion between storage types.
//
// Names.  A checkpoint in the diffusers layout names the DiT's tensors differently from the layout the
// executors register (the "original" one): convert_diffusion_model_name and the per-family converters of
// src/utils/name_conversion.cpp (SD3 :439-543, FLUX :545-657, Wan :773-800) map one to the other.  Where
// the original layout fuses projections (q, k, v -> qkv; q, k, v, mlp -> linear1) the converted name of
// the 2nd, 3rd, ... projection carries a numeric suffix (".weight.1", ".bias.2", ...).  canonical_name()
// returns the base name and that number as the part index.
//
// Parts.  ModelLoader::load_tensors (src/core/runtime/model_loader.cpp:2019-2113) places part i of a fused
// tensor after parts 0..i-1 along the dimension in which the part is shorter than the fused tensor (rows
// for a weight, elements for a bias).  Ingest stages the parts on the host and hands the tensor to the
// parameter table once parts 0..m cover it exactly.
//
// Types.  convert_tensor_data (src/core/runtime/model_loader.cpp:663-704): a tensor stored in another type
// than the model keeps is dequantised to f32 and encoded again.  Here the f32 rows are encoded on the device
// (q8_0: ggml's reference rule bit for bit; q4_K: this library's min/max encoder, not ggml's iterative
// search - the blocks differ from the ones `ed-convert` would write, the step's tolerance holds).
#include "edb200_internal.h"
#include "edb200_model.h"

#include <cuda_fp16.h>

#include <cstring>
#include <map>
#include <string>
#include <vector>

namespace edb {
namespace {

constexpr int kTypeF16 = 1;
constexpr int kTypeBF16 = 30;

struct Rule {
    const char* from;
    const char* to;
    int part;
};

bool starts_with(const std::string& s, const char* prefix) { return s.compare(0, strlen(prefix), prefix) == 0; }

// The first rule whose `from` is a prefix of `s` rewrites that prefix.
bool apply_prefix_rules(const Rule* rules, size_t n, std::string& s, int& part) {
    for (size_t i = 0; i < n; ++i) {
        if (starts_with(s, rules[i].from)) {
            s = std::string(rules[i].to) + s.substr(strlen(rules[i].from));
            part = rules[i].part;
            return true;
        }
    }
    return false;
}

// "<scope>.<index>.<rest>" -> index and rest; false when `s` is not of that form.
bool split_block(const std::string& s, const char* scope, std::string& index, std::string& rest) {
    const size_t n = strlen(scope);
    if (s.compare(0, n, scope) != 0 || s.size() <= n || s[n] != '.') return false;
    size_t i = n + 1;
    const size_t first = i;
    while (i < s.size() && s[i] >= '0' && s[i] <= '9') ++i;
    if (i == first || i >= s.size() || s[i] != '.') return false;
    index = s.substr(first, i - first);
    rest = s.substr(i + 1);
    return true;
}

// The two embedder MLPs and the final layer are named alike in the FLUX and SD3 diffusers layouts.
const Rule kFluxTop[] = {
    {"time_text_embed.timestep_embedder.linear_1.", "time_in.in_layer.", 0},
    {"time_text_embed.timestep_embedder.linear_2.", "time_in.out_layer.", 0},
    {"time_text_embed.text_embedder.linear_1.", "vector_in.in_layer.", 0},
    {"time_text_embed.text_embedder.linear_2.", "vector_in.out_layer.", 0},
    {"time_text_embed.guidance_embedder.linear_1.", "guidance_in.in_layer.", 0},
    {"time_text_embed.guidance_embedder.linear_2.", "guidance_in.out_layer.", 0},
    {"context_embedder.", "txt_in.", 0},
    {"x_embedder.", "img_in.", 0},
    {"proj_out.", "final_layer.linear.", 0},
    {"norm_out.linear.", "final_layer.adaLN_modulation.1.", 0},
};
// Inside transformer_blocks.<i>. (image stream first, then the "added"/context stream).
const Rule kFluxDouble[] = {
    {"norm1.linear.", "img_mod.lin.", 0},
    {"norm1_context.linear.", "txt_mod.lin.", 0},
    {"attn.to_q.", "img_attn.qkv.", 0},
    {"attn.to_k.", "img_attn.qkv.", 1},
    {"attn.to_v.", "img_attn.qkv.", 2},
    {"attn.add_q_proj.", "txt_attn.qkv.", 0},
    {"attn.add_k_proj.", "txt_attn.qkv.", 1},
    {"attn.add_v_proj.", "txt_attn.qkv.", 2},
    {"attn.norm_q.weight", "img_attn.norm.query_norm.scale", 0},
    {"attn.norm_k.weight", "img_attn.norm.key_norm.scale", 0},
    {"attn.norm_added_q.weight", "txt_attn.norm.query_norm.scale", 0},
    {"attn.norm_added_k.weight", "txt_attn.norm.key_norm.scale", 0},
    {"attn.to_out.0.", "img_attn.proj.", 0},
    {"attn.to_add_out.", "txt_attn.proj.", 0},
    {"ff.net.0.proj.", "img_mlp.0.", 0},
    {"ff.net.2.", "img_mlp.2.", 0},
    {"ff_context.net.0.proj.", "txt_mlp.0.", 0},
    {"ff_context.net.2.", "txt_mlp.2.", 0},
};
// Inside single_transformer_blocks.<i>.: q, k, v and the MLP's first projection share linear1.
const Rule kFluxSingle[] = {
    {"norm.linear.", "modulation.lin.", 0},
    {"attn.to_q.", "linear1.", 0},
    {"attn.to_k.", "linear1.", 1},
    {"attn.to_v.", "linear1.", 2},
    {"proj_mlp.", "linear1.", 3},
    {"attn.norm_q.weight", "norm.query_norm.scale", 0},
    {"attn.norm_k.weight", "norm.key_norm.scale", 0},
    {"proj_out.", "linear2.", 0},
};

const Rule kSd3Top[] = {
    {"time_text_embed.timestep_embedder.linear_1.", "t_embedder.mlp.0.", 0},
    {"time_text_embed.timestep_embedder.linear_2.", "t_embedder.mlp.2.", 0},
    {"time_text_embed.text_embedder.linear_1.", "y_embedder.mlp.0.", 0},
    {"time_text_embed.text_embedder.linear_2.", "y_embedder.mlp.2.", 0},
    {"pos_embed.pos_embed", "pos_embed", 0},
    {"pos_embed.proj.", "x_embedder.proj.", 0},
    {"proj_out.", "final_layer.linear.", 0},
    {"norm_out.linear.", "final_layer.adaLN_modulation.1.", 0},
};
// Inside transformer_blocks.<i>. ; "attn2" is the second self-attention of the SD3.5-medium x blocks.
const Rule kSd3Block[] = {
    {"norm1.linear.", "x_block.adaLN_modulation.1.", 0},
    {"norm1_context.linear.", "context_block.adaLN_modulation.1.", 0},
    {"attn.to_q.", "x_block.attn.qkv.", 0},
    {"attn.to_k.", "x_block.attn.qkv.", 1},
    {"attn.to_v.", "x_block.attn.qkv.", 2},
    {"attn.add_q_proj.", "context_block.attn.qkv.", 0},
    {"attn.add_k_proj.", "context_block.attn.qkv.", 1},
    {"attn.add_v_proj.", "context_block.attn.qkv.", 2},
    {"attn2.to_q.", "x_block.attn2.qkv.", 0},
    {"attn2.to_k.", "x_block.attn2.qkv.", 1},
    {"attn2.to_v.", "x_block.attn2.qkv.", 2},
    {"attn2.add_q_proj.", "context_block.attn2.qkv.", 0},
    {"attn2.add_k_proj.", "context_block.attn2.qkv.", 1},
    {"attn2.add_v_proj.", "context_block.attn2.qkv.", 2},
    {"attn.norm_q.", "x_block.attn.ln_q.", 0},
    {"attn.norm_k.", "x_block.attn.ln_k.", 0},
    {"attn.norm_added_q.", "context_block.attn.ln_q.", 0},
    {"attn.norm_added_k.", "context_block.attn.ln_k.", 0},
    {"attn2.norm_q.", "x_block.attn2.ln_q.", 0},
    {"attn2.norm_k.", "x_block.attn2.ln_k.", 0},
    {"attn.to_out.0.", "x_block.attn.proj.", 0},
    {"attn.to_add_out.", "context_block.attn.proj.", 0},
    {"attn2.to_out.0.", "x_block.attn2.proj.", 0},
    {"attn2.to_add_out.", "context_block.attn2.proj.", 0},
    {"ff.net.0.proj.", "x_block.mlp.fc1.", 0},
    {"ff.net.2.", "x_block.mlp.fc2.", 0},
    {"ff_context.net.0.proj.", "context_block.mlp.fc1.", 0},
    {"ff_context.net.2.", "context_block.mlp.fc2.", 0},
};

const Rule kWanTop[] = {
    {"condition_embedder.text_embedder.linear_1.", "text_embedding.0.", 0},
    {"condition_embedder.text_embedder.linear_2.", "text_embedding.2.", 0},
    {"condition_embedder.time_embedder.linear_1.", "time_embedding.0.", 0},
    {"condition_embedder.time_embedder.linear_2.", "time_embedding.2.", 0},
    {"condition_embedder.time_proj.", "time_projection.1.", 0},
    {"proj_out.", "head.head.", 0},
    {"scale_shift_table", "head.modulation", 0},
};
// Wan block names change piecewise: each listed fragment is replaced wherever it first occurs.
const Rule kWanFragments[] = {
    {".attn1.", ".self_attn.", 0},    {".attn2.", ".cross_attn.", 0},
    {".to_q.", ".q.", 0},             {".to_k.", ".k.", 0},
    {".to_v.", ".v.", 0},             {".to_out.0.", ".o.", 0},
    {".ffn.net.0.proj.", ".ffn.0.", 0}, {".ffn.net.2.", ".ffn.2.", 0},
    {".norm2.", ".norm3.", 0},        {".scale_shift_table", ".modulation", 0},
};

template <size_t N>
bool top(const Rule (&rules)[N], std::string& s, int& part) {
    return apply_prefix_rules(rules, N, s, part);
}

template <size_t N>
bool in_block(const Rule (&rules)[N], const std::string& s, const char* scope, const char* new_scope, std::string& out,
              int& part) {
    std::string index, rest;
    if (!split_block(s, scope, index, rest)) return false;
    if (!apply_prefix_rules(rules, N, rest, part)) return false;
    out = std::string(new_scope) + "." + index + "." + rest;
    return true;
}

float f16_bits_to_f32(uint16_t h) { return __half2float(__ushort_as_half(h)); }

// ggml q4_K: 6-bit scale / min pairs of the 8 sub-blocks packed in 12 bytes.
void q4k_scale_min(int j, const uint8_t* q, uint8_t& sc, uint8_t& m) {
    if (j < 4) {
        sc = q[j] & 63;
        m = q[j + 4] & 63;
    } else {
        sc = (q[j + 4] & 0xF) | ((q[j - 4] >> 6) << 4);
        m = (q[j + 4] >> 4) | ((q[j] >> 6) << 4);
    }
}

}  // namespace

// `name` (prefix already removed) in the layout the executors register, with the part index of a fused
// tensor (0 for whole tensors and first parts).  A name that already carries a numeric part suffix
// ("….weight.2") is split the same way, whatever the family.
void canonical_name(int family, const std::string& name, std::string& out, int& part) {
    out = name;
    part = 0;
    std::string s = name;
    int p = 0;
    bool hit = false;
    if (family == EDB200_FAMILY_FLUX) {
        hit = in_block(kFluxDouble, s, "transformer_blocks", "double_blocks", out, p) ||
              in_block(kFluxSingle, s, "single_transformer_blocks", "single_blocks", out, p);
        if (!hit && top(kFluxTop, s, p)) {
            out = s;
            hit = true;
        }
    } else if (family == EDB200_FAMILY_SD3) {
        hit = in_block(kSd3Block, s, "transformer_blocks", "joint_blocks", out, p);
        if (!hit && top(kSd3Top, s, p)) {
            out = s;
            hit = true;
        }
    } else if (family == EDB200_FAMILY_WAN) {
        top(kWanTop, s, p);
        for (const Rule& r : kWanFragments) {
            const size_t at = s.find(r.from);
            if (at != std::string::npos) s.replace(at, strlen(r.from), r.to);
        }
        out = s;
        hit = true;
    }
    if (hit) part = p;
    // "<base>.weight.<n>" / "<base>.bias.<n>": an explicit part suffix.
    const size_t dot = out.rfind('.');
    if (dot != std::string::npos && dot + 1 < out.size()) {
        int value = 0;
        bool digits = true;
        for (size_t i = dot + 1; i < out.size() && digits; ++i) {
            digits = out[i] >= '0' && out[i] <= '9' && value < 100000;
            if (digits) value = value * 10 + (out[i] - '0');
        }
        const std::string base = out.substr(0, dot);
        const auto ends = [&](const char* suffix) {
            const size_t n = strlen(suffix);
            return base.size() >= n && base.compare(base.size() - n, n, suffix) == 0;
        };
        if (digits && (ends(".weight") || ends(".bias"))) {
            out = base;
            part = value;
        }
    }
}

// Elements of `data` (stored as `type`) as f32.  False for a type that is not read.
bool to_f32(int type, const void* data, int64_t n, int64_t row_len, float* out) {
    switch (type) {
        case EDB200_TYPE_F32: memcpy(out, data, static_cast<size_t>(n) * 4); return true;
        case kTypeF16: {
            const uint16_t* h = static_cast<const uint16_t*>(data);
            for (int64_t i = 0; i < n; ++i) out[i] = f16_bits_to_f32(h[i]);
            return true;
        }
        case kTypeBF16: {
            const uint16_t* h = static_cast<const uint16_t*>(data);
            for (int64_t i = 0; i < n; ++i) {
                const uint32_t bits = static_cast<uint32_t>(h[i]) << 16;
                memcpy(out + i, &bits, 4);
            }
            return true;
        }
        case EDB200_TYPE_Q8_0: {   // 34-byte blocks: f16 d, 32 x int8; value = d * q
            if (row_len % 32) return false;
            const uint8_t* b = static_cast<const uint8_t*>(data);
            for (int64_t blk = 0; blk < n / 32; ++blk, b += 34) {
                uint16_t dh;
                memcpy(&dh, b, 2);
                const float d = f16_bits_to_f32(dh);
                const int8_t* q = reinterpret_cast<const int8_t*>(b + 2);
                for (int j = 0; j < 32; ++j) out[blk * 32 + j] = d * static_cast<float>(q[j]);
            }
            return true;
        }
        case EDB200_TYPE_Q4_K: {   // 144-byte super-blocks of 256: f16 d, f16 dmin, 12 scale bytes, 128 nibble bytes
            if (row_len % 256) return false;
            const uint8_t* b = static_cast<const uint8_t*>(data);
            for (int64_t blk = 0; blk < n / 256; ++blk, b += 144) {
                uint16_t dh, mh;
                memcpy(&dh, b, 2);
                memcpy(&mh, b + 2, 2);
                const float d = f16_bits_to_f32(dh), dmin = f16_bits_to_f32(mh);
                const uint8_t* scales = b + 4;
                const uint8_t* q = b + 16;
                float* y = out + blk * 256;
                for (int j = 0; j < 4; ++j, q += 32, y += 64) {   // 64 values: low nibbles, then high nibbles
                    uint8_t sc, m;
                    q4k_scale_min(2 * j, scales, sc, m);
                    const float d1 = d * sc, m1 = dmin * m;
                    q4k_scale_min(2 * j + 1, scales, sc, m);
                    const float d2 = d * sc, m2 = dmin * m;
                    for (int l = 0; l < 32; ++l) y[l] = d1 * (q[l] & 0xF) - m1;
                    for (int l = 0; l < 32; ++l) y[32 + l] = d2 * (q[l] >> 4) - m2;
                }
            }
            return true;
        }
        default: return false;
    }
}

Ingest::Ingest(ParamTable& table, int family, const char* strip_prefix, cudaStream_t stream)
    : table_(table), family_(family), prefix_(strip_prefix ? strip_prefix : ""), stream_(stream) {}

// f32 rows on the host -> the parameter's storage (device encode for quantised parameters).
edb200_status_t Ingest::set_from_f32(const std::string& name, Param* p, const float* src) {
    const int64_t rows = p->spec.n_out, k = p->spec.k, n = rows * k;
    if (!p->spec.quantised) return table_.set(name, EDB200_TYPE_F32, src, n * 4, false, stream_);
    const int wt = p->spec.ggml_type;
    const int64_t qbytes = rows * ggml_row_bytes(wt, k);
    float* x_dev = nullptr;
    void* q_dev = nullptr;
    cudaError_t e = cudaMalloc(reinterpret_cast<void**>(&x_dev), static_cast<size_t>(n) * 4);
    if (e == cudaSuccess) e = cudaMalloc(&q_dev, static_cast<size_t>(qbytes));
    if (e == cudaSuccess) e = cudaMemcpyAsync(x_dev, src, static_cast<size_t>(n) * 4, cudaMemcpyHostToDevice, stream_);
    if (e != cudaSuccess) {
        cudaFree(x_dev);
        cudaFree(q_dev);
        return fail(EDB200_ERR_NOMEM, "weight ingest: staging '%s': %s", name.c_str(), cudaGetErrorString(e));
    }
    edb200_status_t st = wt == EDB200_TYPE_Q8_0 ? edb200_quantize_rows_q8_0(x_dev, q_dev, rows, k, stream_)
                                                : quantize_rows_q4_k_device(x_dev, q_dev, rows, k, stream_);
    if (st == EDB200_OK) st = table_.set(name, wt, q_dev, qbytes, true, stream_);
    cudaStreamSynchronize(stream_);   // the caller's host buffer and the staging buffers are reused or freed next
    cudaFree(x_dev);
    cudaFree(q_dev);
    return st;
}

edb200_status_t Ingest::offer(const SourceTensor& t) {
    std::string name = t.name;
    if (!prefix_.empty() && name.compare(0, prefix_.size(), prefix_) == 0) name = name.substr(prefix_.size());
    Param* p = table_.find(name);
    int part = 0;
    if (p == nullptr) {
        std::string canon;
        canonical_name(family_, name, canon, part);
        p = table_.find(canon);
        if (p == nullptr) return EDB200_OK;   // another component's tensor (VAE, text encoder)
        name = canon;
    }
    const int64_t rows = p->spec.n_out, k = p->spec.k, full = rows * k;
    const bool matrix = rows > 1;
    if (t.nbytes < 0) {
        return fail(EDB200_ERR_UNSUPPORTED, "weight ingest: '%s' is stored as ggml type %d, which is not read here",
                    t.name.c_str(), t.type);
    }
    if (t.n_elements == full && part == 0) {   // a whole tensor
        if (t.row_len > 0 && matrix && t.row_len != k) {
            return fail(EDB200_ERR_INVALID, "weight ingest: '%s' has rows of %lld, the model expects %lld x %lld",
                        t.name.c_str(), (long long)t.row_len, (long long)rows, (long long)k);
        }
        edb200_status_t st;
        if (t.type == p->spec.ggml_type) {
            st = table_.set(name, t.type, t.data, t.nbytes, false, stream_);
        } else {
            scratch_.resize(static_cast<size_t>(full));
            if (!to_f32(t.type, t.data, full, k, scratch_.data())) {
                return fail(EDB200_ERR_UNSUPPORTED, "weight ingest: '%s' is stored as ggml type %d, the model keeps type %d",
                            t.name.c_str(), t.type, p->spec.ggml_type);
            }
            st = set_from_f32(name, p, scratch_.data());
        }
        if (st == EDB200_OK) ++count_;
        return st;
    }
    // A part of a fused tensor: weights are cut along rows, vectors along their length.
    if (t.n_elements >= full || (matrix && (t.row_len != k || t.n_elements % k != 0))) {
        return fail(EDB200_ERR_INVALID,
                    "weight ingest: '%s' (%lld elements, rows of %lld) is neither '%s' (%lld x %lld) nor a part of it",
                    t.name.c_str(), (long long)t.n_elements, (long long)t.row_len, name.c_str(), (long long)rows,
                    (long long)k);
    }
    Staged& s = staged_[name];
    if (s.parts.count(part)) {
        return fail(EDB200_ERR_INVALID, "weight ingest: part %d of '%s' appears twice ('%s')", part, name.c_str(),
                    t.name.c_str());
    }
    Part& part_rec = s.parts[part];
    part_rec.n = t.n_elements;
    part_rec.type = t.type;
    // Same storage type as the model's and whole blocks: keep the raw bytes (rows of a block type are independent).
    const bool raw = t.type == p->spec.ggml_type && (matrix || t.type == EDB200_TYPE_F32);
    if (raw) {
        part_rec.bytes.assign(static_cast<const uint8_t*>(t.data), static_cast<const uint8_t*>(t.data) + t.nbytes);
    } else {
        part_rec.type = EDB200_TYPE_F32;
        part_rec.bytes.resize(static_cast<size_t>(t.n_elements) * 4);
        if (!to_f32(t.type, t.data, t.n_elements, matrix ? k : t.n_elements,
                    reinterpret_cast<float*>(part_rec.bytes.data()))) {
            return fail(EDB200_ERR_UNSUPPORTED, "weight ingest: '%s' is stored as ggml type %d, which is not converted",
                        t.name.c_str(), t.type);
        }
    }
    s.elements += t.n_elements;
    if (s.elements < full) return EDB200_OK;
    if (s.elements > full) {
        return fail(EDB200_ERR_INVALID, "weight ingest: the parts of '%s' hold %lld elements, the model expects %lld",
                    name.c_str(), (long long)s.elements, (long long)full);
    }
    const edb200_status_t st = assemble(name, p, s);
    staged_.erase(name);
    if (st == EDB200_OK) ++count_;
    return st;
}

// Parts 0..m in order, back to back (part i starts where parts 0..i-1 end).
edb200_status_t Ingest::assemble(const std::string& name, Param* p, Staged& s) {
    const int64_t k = p->spec.k, full = p->spec.n_out * k;
    const bool matrix = p->spec.n_out > 1;
    int expect = 0;
    bool all_raw = true;
    for (const auto& kv : s.parts) {
        if (kv.first != expect++) {
            return fail(EDB200_ERR_INVALID, "weight ingest: '%s' is complete in size but part %d is missing", name.c_str(),
                        expect - 1);
        }
        all_raw = all_raw && kv.second.type == p->spec.ggml_type;
    }
    if (all_raw) {
        std::vector<uint8_t> fused;
        fused.reserve(static_cast<size_t>(p->spec.n_out * ggml_row_bytes(p->spec.ggml_type, k)));
        for (const auto& kv : s.parts) fused.insert(fused.end(), kv.second.bytes.begin(), kv.second.bytes.end());
        return table_.set(name, p->spec.ggml_type, fused.data(), static_cast<int64_t>(fused.size()), false, stream_);
    }
    scratch_.resize(static_cast<size_t>(full));
    int64_t at = 0;
    for (const auto& kv : s.parts) {
        const Part& part = kv.second;
        if (part.type == EDB200_TYPE_F32) {
            memcpy(scratch_.data() + at, part.bytes.data(), static_cast<size_t>(part.n) * 4);
        } else if (!to_f32(part.type, part.bytes.data(), part.n, matrix ? k : part.n, scratch_.data() + at)) {
            return fail(EDB200_ERR_UNSUPPORTED, "weight ingest: a part of '%s' has ggml type %d, which is not converted",
                        name.c_str(), part.type);
        }
        at += part.n;
    }
    return set_from_f32(name, p, scratch_.data());
}

edb200_status_t Ingest::finish(int* n_loaded) {
    if (n_loaded) *n_loaded = count_;
    if (!staged_.empty()) {
        const auto& first = *staged_.begin();
        return fail(EDB200_ERR_INVALID, "weight ingest: '%s' is incomplete: %d part(s) with %lld elements were found",
                    first.first.c_str(), (int)first.second.parts.size(), (long long)first.second.elements);
    }
    return EDB200_OK;
}

}  // namespace edb

using namespace edb;

extern "C" edb200_status_t edb200_canonical_tensor_name(int family, const char* name, char* out, int64_t capacity,
                                                         int* part) {
    if (name == nullptr || out == nullptr || capacity <= 0) {
        return fail(EDB200_ERR_INVALID, "canonical_tensor_name: null argument");
    }
    if (family < EDB200_FAMILY_FLUX || family > EDB200_FAMILY_WAN) {
        return fail(EDB200_ERR_INVALID, "canonical_tensor_name: unknown family %d", family);
    }
    std::string canon;
    int p = 0;
    canonical_name(family, name, canon, p);
    if (static_cast<int64_t>(canon.size()) + 1 > capacity) {
        return fail(EDB200_ERR_INVALID, "canonical_tensor_name: the name needs %lld bytes", (long long)canon.size() + 1);
    }
    memcpy(out, canon.c_str(), canon.size() + 1);
    if (part) *part = p;
    return EDB200_OK;
}
