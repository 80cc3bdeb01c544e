// The reference's operator plugin ABI (ed_cuda_<op>_custom_supported / _compute on ggml_tensor,
// reference src/core/backend/ggml/cuda/ed_cuda_{modulation,norm,rope,attention_v_prep,sage_attn}.h)
// on this library's kernels.  Every operator here is elementwise, a norm over one row, or a copy /
// cast with a re-layout; the kernels index through the tensors' byte strides exactly as the
// reference's CPU callbacks do (src/core/backend/ggml/ed_ggml_*_ext.hpp), with the same f32
// operations in the same order, so the results are those callbacks' bits.  The parameter packing
// (a 32-bit magic plus small integers in the `userdata` word of dst->op_params) is the interface
// and is decoded as the reference's *_params_from_userdata functions do.
#include "edb200_shims.h"

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <cstdlib>
#include <cstring>

#include "edb200_internal.h"

using namespace edb;

namespace {

// ---- op parameter words (magics: ed_ggml_modulation_ext.hpp:10-12, ed_ggml_norm_ext.hpp, ed_ggml_rope_ext.hpp:13,
// ed_ggml_attention_ext.hpp:10-12, ed_ggml_sage_attn_ext.hpp:19)
constexpr uint32_t kMagicModulate = 0x45464d4fu;      // "EFMO"
constexpr uint32_t kMagicResidualGate = 0x45465247u;  // "EFRG"
constexpr uint32_t kMagicWhereSelect = 0x45465753u;   // "EFWS"
constexpr uint32_t kMagicRmsNormMulF16 = 0x45524d48u; // "ERMH"
constexpr uint32_t kMagicRope = 0x45525250u;          // "ERRP"
constexpr uint32_t kMagicVPrep = 0x45565050u;         // "EVPP"
constexpr uint32_t kMagicPairPack = 0x45505150u;      // "EPQP"
constexpr uint32_t kMagicQkvPairPack = 0x45514b50u;   // "EQKP"
constexpr uint32_t kMagicSageAttn = 0x53414751u;      // "SAGQ"

// dst->op_params holds {callback, n_tasks, userdata}; the operator's parameters are packed into userdata.
bool userdata_of(const ggml_tensor* dst, uint64_t* out) {
    if (dst == nullptr || dst->op != GGML_OP_CUSTOM) return false;
    struct Params {
        ggml_custom_op_t fun;
        int n_tasks;
        void* userdata;
    } p;
    static_assert(sizeof(p) <= GGML_MAX_OP_PARAMS, "custom op params do not fit");
    memcpy(&p, dst->op_params, sizeof(p));
    *out = static_cast<uint64_t>(reinterpret_cast<uintptr_t>(p.userdata));
    return true;
}

struct View {   // a tensor as the kernels see it: extents, strides in ELEMENTS, data
    long long ne[4];
    long long s[4];
    const void* data;
};

size_t elem_size(int type) {
    switch (type) {
        case GGML_TYPE_F32: return 4;
        case GGML_TYPE_F16: return 2;
        case GGML_TYPE_BF16: return 2;
        case GGML_TYPE_I8: return 1;
        default: return 0;
    }
}

bool make_view(const ggml_tensor* t, View* v) {
    const size_t es = elem_size(t->type);
    if (es == 0) return false;
    for (int i = 0; i < 4; ++i) {
        if (t->nb[i] % es) return false;
        v->ne[i] = t->ne[i];
        v->s[i] = static_cast<long long>(t->nb[i] / es);
    }
    v->data = t->data;
    return true;
}

bool contiguous(const ggml_tensor* t) {
    size_t expect = elem_size(t->type);
    if (expect == 0) return false;
    for (int i = 0; i < 4; ++i) {
        if (t->nb[i] != expect) return false;
        expect *= static_cast<size_t>(t->ne[i]);
    }
    return true;
}

bool positive(const ggml_tensor* t) { return t->ne[0] > 0 && t->ne[1] > 0 && t->ne[2] > 0 && t->ne[3] > 0; }

long long nelements(const ggml_tensor* t) { return (long long)t->ne[0] * t->ne[1] * t->ne[2] * t->ne[3]; }

bool broadcasts_into(const ggml_tensor* src, const ggml_tensor* dst) {
    for (int i = 0; i < 4; ++i) {
        if (src->ne[i] <= 0 || dst->ne[i] <= 0 || dst->ne[i] % src->ne[i]) return false;
    }
    return true;
}

bool same_shape(const ggml_tensor* a, const ggml_tensor* b) {
    for (int i = 0; i < 4; ++i) {
        if (a->ne[i] != b->ne[i]) return false;
    }
    return true;
}

bool env_disabled(const char* name) {
    const char* e = getenv(name);
    return e != nullptr && atoi(e) != 0;
}

__device__ __forceinline__ float bcast_at(const View& v, long long i0, long long i1, long long i2, long long i3) {
    return static_cast<const float*>(v.data)[(i0 % v.ne[0]) * v.s[0] + (i1 % v.ne[1]) * v.s[1] + (i2 % v.ne[2]) * v.s[2] +
                                             (i3 % v.ne[3]) * v.s[3]];
}

// which: 0 modulate (a x, b shift, c scale), 1 residual gate (a residual, b x, c gate), 2 where-select
// (a index, b mod_0, c mod_1).  dst contiguous f32; operands broadcast per dimension by modulo.
__global__ void modulation_kernel(int which, const View a, const View b, const View c, float* __restrict__ dst, long long n0,
                                  long long n1, long long n2, long long total) {
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const long long i0 = idx % n0;
    long long rest = idx / n0;
    const long long i1 = rest % n1;
    rest /= n1;
    const long long i2 = rest % n2, i3 = rest / n2;
    const float av = bcast_at(a, i0, i1, i2, i3), bv = bcast_at(b, i0, i1, i2, i3), cv = bcast_at(c, i0, i1, i2, i3);
    float y;
    if (which == 0) {
        y = __fadd_rn(__fadd_rn(av, __fmul_rn(av, cv)), bv);      // (x + x*scale) + shift
    } else if (which == 1) {
        y = __fadd_rn(av, __fmul_rn(bv, cv));                      // residual + x*gate
    } else {
        y = __fadd_rn(bv, __fmul_rn(av, __fsub_rn(cv, bv)));       // mod_0 + index*(mod_1 - mod_0)
    }
    dst[idx] = y;
}

// One warp per row: sum of squares in channel order is the CPU callback's (a sequential f32 sum), so the
// row is walked by ONE lane for the sum and by all lanes for the scaled output.
__global__ void rms_norm_mul_f16_kernel(const View x, const float* __restrict__ w, __half* __restrict__ dst, long long d_s1,
                                        long long d_s2, long long d_s3, long long rows, float eps) {
    const long long row = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (row >= rows) return;
    long long rem = row;
    const long long i1 = rem % x.ne[1];
    rem /= x.ne[1];
    const long long i2 = rem % x.ne[2], i3 = rem / x.ne[2];
    const float* xr = static_cast<const float*>(x.data) + i1 * x.s[1] + i2 * x.s[2] + i3 * x.s[3];
    float sum = 0.0f;
    if (lane == 0) {
        for (long long i0 = 0; i0 < x.ne[0]; ++i0) {
            const float v = xr[i0];
            sum = __fadd_rn(sum, __fmul_rn(v, v));
        }
    }
    sum = __shfl_sync(0xffffffffu, sum, 0);
    const float scale = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(sum, static_cast<float>(x.ne[0])), eps)));
    __half* dr = dst + i1 * d_s1 + i2 * d_s2 + i3 * d_s3;
    for (long long i0 = lane; i0 < x.ne[0]; i0 += 32) {
        dr[i0] = __float2half_rn(__fmul_rn(__fmul_rn(xr[i0], scale), w[i0]));
    }
}

template <typename T>
__device__ __forceinline__ float load_as_f32(const void* p, long long off);
template <>
__device__ __forceinline__ float load_as_f32<float>(const void* p, long long off) {
    return static_cast<const float*>(p)[off];
}
template <>
__device__ __forceinline__ float load_as_f32<__nv_bfloat16>(const void* p, long long off) {
    return __bfloat162float(static_cast<const __nv_bfloat16*>(p)[off]);
}
template <typename T>
__device__ __forceinline__ void store_from_f32(void* p, long long off, float v);
template <>
__device__ __forceinline__ void store_from_f32<float>(void* p, long long off, float v) {
    static_cast<float*>(p)[off] = v;
}
template <>
__device__ __forceinline__ void store_from_f32<__half>(void* p, long long off, float v) {
    static_cast<__half*>(p)[off] = __float2half_rn(v);
}
template <>
__device__ __forceinline__ void store_from_f32<__nv_bfloat16>(void* p, long long off, float v) {
    static_cast<__nv_bfloat16*>(p)[off] = __float2bfloat16_rn(v);
}

// layout 0: x [d, heads, seq, batch]; 1: x [d, seq, heads, batch]; 2: x [d/2, seq, heads, 2] (pair halves in ne[3]).
// pe: "matrix" [2, 2, d/2, seq] or "prepared" [2, d/2, seq, 2].  dst [d, seq, heads * batch] contiguous.
template <typename TI, typename TO>
__global__ void rope_kernel(const View x, const View pe, bool pe_prepared, void* __restrict__ dst, int layout, int interleaved,
                            int d_head, long long seq, long long n_head, long long total) {
    const long long idx0 = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx0 >= total) return;
    const int half = d_head / 2;
    const long long p = idx0 % half;
    long long idx = idx0 / half;
    const long long s = idx % seq;
    const long long h_total = idx / seq;
    float x0, x1;
    if (layout == 0) {
        const long long h = h_total % n_head, b = h_total / n_head;
        const long long base = h * x.s[1] + s * x.s[2] + b * x.s[3];
        x0 = load_as_f32<TI>(x.data, (interleaved ? 2 * p : p) * x.s[0] + base);
        x1 = load_as_f32<TI>(x.data, (interleaved ? 2 * p + 1 : p + half) * x.s[0] + base);
    } else if (layout == 1) {
        const long long h = h_total % n_head, b = h_total / n_head;
        const long long base = s * x.s[1] + h * x.s[2] + b * x.s[3];
        x0 = load_as_f32<TI>(x.data, (interleaved ? 2 * p : p) * x.s[0] + base);
        x1 = load_as_f32<TI>(x.data, (interleaved ? 2 * p + 1 : p + half) * x.s[0] + base);
    } else {
        const long long base = p * x.s[0] + s * x.s[1] + h_total * x.s[2];
        x0 = load_as_f32<TI>(x.data, base);
        x1 = load_as_f32<TI>(x.data, base + x.s[3]);
    }
    const float* pt = static_cast<const float*>(pe.data);
    float m[2][2];   // m[row][col]
#pragma unroll
    for (int row = 0; row < 2; ++row) {
#pragma unroll
        for (int col = 0; col < 2; ++col) {
            m[row][col] = pe_prepared ? pt[row * pe.s[0] + p * pe.s[1] + s * pe.s[2] + col * pe.s[3]]
                                      : pt[row * pe.s[0] + col * pe.s[1] + p * pe.s[2] + s * pe.s[3]];
        }
    }
    const float y0 = __fadd_rn(__fmul_rn(x0, m[0][0]), __fmul_rn(x1, m[1][0]));
    const float y1 = __fadd_rn(__fmul_rn(x0, m[0][1]), __fmul_rn(x1, m[1][1]));
    const long long dbase = h_total * d_head * seq + s * d_head;
    if (interleaved || layout == 2) {
        store_from_f32<TO>(dst, dbase + 2 * p, y0);
        store_from_f32<TO>(dst, dbase + 2 * p + 1, y1);
    } else {
        store_from_f32<TO>(dst, dbase + p, y0);
        store_from_f32<TO>(dst, dbase + p + half, y1);
    }
}

// mode 0 v_prep: src0 [d, seq, heads, batch] (seq-major) or [d, heads, seq, batch] -> dst [d, seq, heads*batch]
// mode 1 pair pack: src0, src1 [d*heads, seq_i, batch] -> dst [d, seq0+seq1, heads, batch]
// mode 2 qkv pair pack: planes q, k, v of two streams -> dst [d, seq0+seq1, heads, 3]
struct PackArgs {
    View first[3];
    View second[3];
    long long d_head, first_seq, total_seq, n_head, outer;   // outer: batch (modes 0, 1) or 3 planes (mode 2)
    long long d_s[4];
    int mode, v_is_seq_major;
};

__global__ void attention_pack_kernel(const PackArgs a, __half* __restrict__ dst, long long total) {
    const long long idx0 = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx0 >= total) return;
    const long long d = idx0 % a.d_head;
    long long idx = idx0 / a.d_head;
    const long long s = idx % a.total_seq;
    idx /= a.total_seq;
    const long long h = idx % a.n_head, o = idx / a.n_head;
    float v;
    long long off;
    if (a.mode == 0) {
        const View& x = a.first[0];
        v = static_cast<const float*>(x.data)[a.v_is_seq_major ? d * x.s[0] + s * x.s[1] + h * x.s[2] + o * x.s[3]
                                                               : d * x.s[0] + h * x.s[1] + s * x.s[2] + o * x.s[3]];
        off = d * a.d_s[0] + s * a.d_s[1] + (h + o * a.n_head) * a.d_s[2];
    } else {
        const int plane = a.mode == 2 ? static_cast<int>(o) : 0;
        const bool in_first = s < a.first_seq;
        const View& x = in_first ? a.first[plane] : a.second[plane];
        const long long ss = in_first ? s : s - a.first_seq;
        const long long b = a.mode == 2 ? 0 : o;
        v = static_cast<const float*>(x.data)[(d + h * a.d_head) * x.s[0] + ss * x.s[1] + b * x.s[2]];
        off = d * a.d_s[0] + s * a.d_s[1] + h * a.d_s[2] + o * a.d_s[3];
    }
    dst[off] = __float2half_rn(v);
}

// v of the Sage operator -> f16 [heads*N, L, d]: from [d, heads, L, N] (token-major) or [d, L, heads] (packed)
template <typename T>
__global__ void sage_v_to_f16_kernel(const View v, int packed, long long d_head, long long L, long long n_head,
                                     __half* __restrict__ dst, long long total) {
    const long long idx0 = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx0 >= total) return;
    const long long d = idx0 % d_head;
    long long idx = idx0 / d_head;
    const long long l = idx % L, hn = idx / L;
    const long long h = hn % n_head, n = hn / n_head;
    const long long off = packed ? d * v.s[0] + l * v.s[1] + h * v.s[2] : d * v.s[0] + h * v.s[1] + l * v.s[2] + n * v.s[3];
    if constexpr (sizeof(T) == 2) {
        dst[idx0] = static_cast<const __half*>(v.data)[off];
    } else {
        dst[idx0] = __float2half_rn(static_cast<const float*>(v.data)[off]);
    }
}

unsigned blocks_for(long long total) { return static_cast<unsigned>((total + 255) / 256); }

// ------------------------------------------------------------------ modulation
int modulation_kind(const ggml_tensor* dst) {
    uint64_t ud = 0;
    if (!userdata_of(dst, &ud) || dst->src[0] == nullptr || dst->src[1] == nullptr || dst->src[2] == nullptr) return -1;
    const uint32_t magic = static_cast<uint32_t>(ud & 0xffffffffu);
    const ggml_tensor *a = dst->src[0], *b = dst->src[1], *c = dst->src[2];
    if (a->type != GGML_TYPE_F32 || b->type != GGML_TYPE_F32 || c->type != GGML_TYPE_F32 || dst->type != GGML_TYPE_F32) return -1;
    if (!contiguous(dst) || !positive(dst)) return -1;
    if (magic == kMagicModulate) {
        // x, shift, scale: shift and scale broadcast into x; dst has x's shape
        return positive(a) && broadcasts_into(b, a) && broadcasts_into(c, a) && same_shape(dst, a) ? 0 : -1;
    }
    if (magic == kMagicResidualGate) {
        // residual, x, gate: residual has x's shape, gate broadcasts into x
        return positive(b) && same_shape(a, b) && broadcasts_into(c, b) && same_shape(dst, b) ? 1 : -1;
    }
    if (magic == kMagicWhereSelect) {
        return broadcasts_into(a, dst) && broadcasts_into(b, dst) && broadcasts_into(c, dst) ? 2 : -1;
    }
    return -1;
}

// ------------------------------------------------------------------ rope
struct RopeParams {
    int layout, interleaved, d_head;
};

bool rope_params(const ggml_tensor* dst, RopeParams* rp) {
    uint64_t ud = 0;
    if (!userdata_of(dst, &ud) || static_cast<uint32_t>(ud & 0xffffffffu) != kMagicRope) return false;
    rp->layout = static_cast<int>((ud >> 32) & 0xffu);
    rp->interleaved = static_cast<int>((ud >> 40) & 0xffu);
    rp->d_head = static_cast<int>((ud >> 48) & 0xffffu);
    return rp->d_head > 0 && rp->d_head % 2 == 0 && rp->layout >= 0 && rp->layout <= 2;
}

bool rope_shapes(const ggml_tensor* dst, const RopeParams& rp, long long* seq, long long* n_head, long long* batch,
                 bool* prepared) {
    const ggml_tensor *x = dst->src[0], *pe = dst->src[1];
    if (x == nullptr || pe == nullptr || env_disabled("ED_DISABLE_CUDA_ROPE")) return false;
    if ((x->type != GGML_TYPE_F32 && x->type != GGML_TYPE_BF16) || pe->type != GGML_TYPE_F32) return false;
    if (dst->type != GGML_TYPE_F32 && dst->type != GGML_TYPE_F16 && dst->type != GGML_TYPE_BF16) return false;
    if (!rp.interleaved && rp.layout == 2) return false;
    const long long half = rp.d_head / 2;
    if (rp.layout == 0) {
        *seq = x->ne[2], *n_head = x->ne[1], *batch = x->ne[3];
        if (x->ne[0] != rp.d_head) return false;
    } else if (rp.layout == 1) {
        *seq = x->ne[1], *n_head = x->ne[2], *batch = x->ne[3];
        if (x->ne[0] != rp.d_head) return false;
    } else {
        *seq = x->ne[1], *n_head = x->ne[2], *batch = 1;
        if (x->ne[0] != half || x->ne[3] != 2) return false;
    }
    if (*seq <= 0 || *n_head <= 0 || *batch <= 0) return false;
    // the output is [d_head, seq, heads * batch], contiguous in its first three dimensions
    const size_t es = elem_size(dst->type);
    if (dst->ne[0] != rp.d_head || dst->ne[1] != *seq || dst->ne[2] != *n_head * *batch) return false;
    if (dst->nb[0] != es || dst->nb[1] != es * dst->ne[0] || dst->nb[2] != es * dst->ne[0] * dst->ne[1]) return false;
    const bool is_prepared = pe->ne[0] == 2 && pe->ne[1] >= half && pe->ne[2] >= *seq && pe->ne[3] == 2;
    const bool is_matrix = pe->ne[0] == 2 && pe->ne[1] == 2 && pe->ne[2] >= half && pe->ne[3] >= *seq;
    *prepared = is_prepared;
    return is_prepared || is_matrix;
}

// ------------------------------------------------------------------ attention layout glue
bool pair_ok(const ggml_tensor* first, const ggml_tensor* second, long long n_head) {
    if (first == nullptr || second == nullptr || first->type != GGML_TYPE_F32 || second->type != GGML_TYPE_F32 || n_head <= 0) {
        return false;
    }
    if (first->ne[0] <= 0 || first->ne[1] <= 0 || first->ne[2] <= 0 || second->ne[0] <= 0 || second->ne[1] <= 0 ||
        second->ne[2] <= 0) {
        return false;
    }
    return first->ne[0] == second->ne[0] && first->ne[2] == second->ne[2] && first->ne[3] == 1 && second->ne[3] == 1 &&
           first->ne[0] % n_head == 0;
}

bool pack_args(const ggml_tensor* dst, int mode, PackArgs* a) {
    uint64_t ud = 0;
    if (!userdata_of(dst, &ud) || dst->type != GGML_TYPE_F16) return false;
    const uint32_t magic = static_cast<uint32_t>(ud & 0xffffffffu);
    memset(a, 0, sizeof(*a));
    a->mode = mode;
    for (int i = 0; i < 4; ++i) a->d_s[i] = static_cast<long long>(dst->nb[i] / 2);
    if (mode == 0) {
        const ggml_tensor* v = dst->src[0];
        const int seq_major = static_cast<int>((ud >> 32) & 0xffu);
        if (magic != kMagicVPrep || (seq_major != 0 && seq_major != 1) || v == nullptr || v->type != GGML_TYPE_F32 ||
            !positive(v) || env_disabled("ED_DISABLE_CUDA_ATTENTION_V_PREP")) {
            return false;
        }
        a->v_is_seq_major = seq_major;
        a->d_head = v->ne[0];
        a->total_seq = seq_major ? v->ne[1] : v->ne[2];
        a->n_head = seq_major ? v->ne[2] : v->ne[1];
        a->outer = v->ne[3];
        a->first_seq = a->total_seq;
        if (dst->ne[0] != a->d_head || dst->ne[1] != a->total_seq || dst->ne[2] != a->n_head * a->outer) return false;
        return make_view(v, &a->first[0]);
    }
    const long long n_head = static_cast<long long>((ud >> 32) & 0x7fffffffu);
    if (mode == 1) {
        if (magic != kMagicPairPack || !pair_ok(dst->src[0], dst->src[1], n_head)) return false;
        a->d_head = dst->src[0]->ne[0] / n_head;
        a->first_seq = dst->src[0]->ne[1];
        a->total_seq = a->first_seq + dst->src[1]->ne[1];
        a->n_head = n_head;
        a->outer = dst->src[0]->ne[2];
        if (dst->ne[0] != a->d_head || dst->ne[1] != a->total_seq || dst->ne[2] != n_head || dst->ne[3] != a->outer) return false;
        return make_view(dst->src[0], &a->first[0]) && make_view(dst->src[1], &a->second[0]);
    }
    if (magic != kMagicQkvPairPack) return false;
    for (int p = 0; p < 3; ++p) {
        if (!pair_ok(dst->src[p], dst->src[3 + p], n_head)) return false;
        if (dst->src[p]->ne[0] != dst->src[0]->ne[0] || dst->src[p]->ne[1] != dst->src[0]->ne[1] ||
            dst->src[3 + p]->ne[0] != dst->src[3]->ne[0] || dst->src[3 + p]->ne[1] != dst->src[3]->ne[1]) {
            return false;
        }
    }
    if (dst->src[0]->ne[2] != 1 || dst->src[3]->ne[2] != 1) return false;
    a->d_head = dst->src[0]->ne[0] / n_head;
    a->first_seq = dst->src[0]->ne[1];
    a->total_seq = a->first_seq + dst->src[3]->ne[1];
    a->n_head = n_head;
    a->outer = 3;
    if (dst->ne[0] != a->d_head || dst->ne[1] != a->total_seq || dst->ne[2] != n_head || dst->ne[3] != 3) return false;
    for (int p = 0; p < 3; ++p) {
        if (!make_view(dst->src[p], &a->first[p]) || !make_view(dst->src[3 + p], &a->second[p])) return false;
    }
    return true;
}

bool pack_compute(ggml_tensor* dst, int mode, void* stream) {
    PackArgs a;
    if (!pack_args(dst, mode, &a)) return false;
    const long long total = a.d_head * a.total_seq * a.n_head * a.outer;
    attention_pack_kernel<<<blocks_for(total), 256, 0, static_cast<cudaStream_t>(stream)>>>(a, static_cast<__half*>(dst->data),
                                                                                           total);
    count_launch();
    return cudaGetLastError() == cudaSuccess;
}

// ------------------------------------------------------------------ sage
struct SageShape {
    long long d_head, L, HN, n_head, N;
    int v_packed;
    bool smooth_q;
};

bool sage_shape(const ggml_tensor* dst, SageShape* sh) {
    uint64_t ud = 0;
    if (!userdata_of(dst, &ud) || static_cast<uint32_t>(ud & 0xffffffffu) != kMagicSageAttn) return false;
    const long long n_head = static_cast<long long>((ud >> 32) & 0x7fffffffu);
    const ggml_tensor *q = dst->src[0], *k = dst->src[1], *v = dst->src[2];
    if (n_head <= 0 || q == nullptr || k == nullptr || v == nullptr) return false;
    // this library quantises from f16 operands: f32 q / k are left to the caller's fallback
    if (q->type != GGML_TYPE_F16 || k->type != GGML_TYPE_F16) return false;
    if (v->type != GGML_TYPE_F16 && v->type != GGML_TYPE_F32) return false;
    const long long d = q->ne[0], L = q->ne[1];
    if ((d != 64 && d != 128) || L <= 0 || k->ne[1] != L || k->ne[0] != d) return false;   // self-attention lengths only
    if (q->ne[2] % n_head || k->ne[2] != q->ne[2] || q->ne[3] != 1 || k->ne[3] != 1) return false;
    const long long N = q->ne[2] / n_head;
    if (N <= 0 || !contiguous(q) || !contiguous(k)) return false;
    const bool v4 = v->ne[0] == d && v->ne[1] == n_head && v->ne[2] == L && v->ne[3] == N;
    const bool v3 = N == 1 && v->ne[0] == d && v->ne[1] == L && v->ne[2] == n_head && v->ne[3] == 1;
    if (!v4 && !v3) return false;
    if (dst->type != GGML_TYPE_F32 || dst->ne[0] != d || dst->ne[1] != q->ne[2] || dst->ne[2] != L || dst->ne[3] != 1 ||
        !contiguous(dst)) {
        return false;
    }
    sh->d_head = d, sh->L = L, sh->HN = q->ne[2], sh->n_head = n_head, sh->N = N;
    sh->v_packed = v4 ? 0 : 1;
    // ED_SAGE_SMOOTH_Q unset: on for head dim 128, off for 64 (sage_smooth_q_enabled, ed_ggml_sage_attn_ext.hpp:76-86)
    const char* e = getenv("ED_SAGE_SMOOTH_Q");
    if (e == nullptr || e[0] == '\0') {
        sh->smooth_q = d == 128;
    } else {
        sh->smooth_q = strcmp(e, "0") != 0 && strcmp(e, "false") != 0 && strcmp(e, "FALSE") != 0 && strcmp(e, "off") != 0 &&
                       strcmp(e, "OFF") != 0;
    }
    return true;
}

}  // namespace

// ======================================================================= entry points

bool ed_cuda_fused_modulate_custom_supported(const ggml_tensor* dst) { return modulation_kind(dst) >= 0; }

bool ed_cuda_fused_modulate_custom_compute(ggml_tensor* dst, void* stream) {
    const int kind = modulation_kind(dst);
    if (kind < 0) return false;
    View a, b, c;
    if (!make_view(dst->src[0], &a) || !make_view(dst->src[1], &b) || !make_view(dst->src[2], &c)) return false;
    const long long total = nelements(dst);
    modulation_kernel<<<blocks_for(total), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        kind, a, b, c, static_cast<float*>(dst->data), dst->ne[0], dst->ne[1], dst->ne[2], total);
    count_launch();
    return cudaGetLastError() == cudaSuccess;
}

bool ed_cuda_rms_norm_mul_f16_custom_supported(const ggml_tensor* dst) {
    uint64_t ud = 0;
    if (!userdata_of(dst, &ud) || static_cast<uint32_t>(ud & 0xffffffffu) != kMagicRmsNormMulF16) return false;
    const ggml_tensor *x = dst->src[0], *w = dst->src[1];
    if (x == nullptr || w == nullptr || x->type != GGML_TYPE_F32 || w->type != GGML_TYPE_F32 || dst->type != GGML_TYPE_F16) {
        return false;
    }
    if (!positive(x) || w->ne[0] != x->ne[0] || w->ne[1] != 1 || w->ne[2] != 1 || w->ne[3] != 1) return false;
    if (x->nb[0] != 4 || !contiguous(w) || !same_shape(dst, x) || dst->nb[0] != 2) return false;
    for (int i = 1; i < 4; ++i) {
        if (x->nb[i] % 4 || dst->nb[i] % 2) return false;
    }
    return true;
}

bool ed_cuda_rms_norm_mul_f16_custom_compute(ggml_tensor* dst, void* stream) {
    if (!ed_cuda_rms_norm_mul_f16_custom_supported(dst)) return false;
    uint64_t ud = 0;
    userdata_of(dst, &ud);
    const uint32_t eps_bits = static_cast<uint32_t>((ud >> 32) & 0xffffffffu);
    float eps;
    memcpy(&eps, &eps_bits, 4);
    View x;
    make_view(dst->src[0], &x);
    const long long rows = (long long)x.ne[1] * x.ne[2] * x.ne[3];
    rms_norm_mul_f16_kernel<<<blocks_for(rows * 32), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        x, static_cast<const float*>(dst->src[1]->data), static_cast<__half*>(dst->data), (long long)(dst->nb[1] / 2),
        (long long)(dst->nb[2] / 2), (long long)(dst->nb[3] / 2), rows, eps);
    count_launch();
    return cudaGetLastError() == cudaSuccess;
}

bool ed_cuda_rope_custom_supported(const ggml_tensor* dst) {
    RopeParams rp;
    long long seq, n_head, batch;
    bool prepared;
    return rope_params(dst, &rp) && rope_shapes(dst, rp, &seq, &n_head, &batch, &prepared);
}

bool ed_cuda_rope_custom_compute(ggml_tensor* dst, void* stream) {
    RopeParams rp;
    long long seq = 0, n_head = 0, batch = 0;
    bool prepared = false;
    if (!rope_params(dst, &rp) || !rope_shapes(dst, rp, &seq, &n_head, &batch, &prepared)) return false;
    View x, pe;
    if (!make_view(dst->src[0], &x) || !make_view(dst->src[1], &pe)) return false;
    const long long total = (long long)(rp.d_head / 2) * seq * n_head * batch;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int ti = dst->src[0]->type, to = dst->type;
#define EDB_ROPE(TI, TO)                                                                                              \
    rope_kernel<TI, TO><<<blocks_for(total), 256, 0, s>>>(x, pe, prepared, dst->data, rp.layout, rp.interleaved, rp.d_head, \
                                                          seq, n_head, total)
    if (ti == GGML_TYPE_F32 && to == GGML_TYPE_F32) {
        EDB_ROPE(float, float);
    } else if (ti == GGML_TYPE_F32 && to == GGML_TYPE_F16) {
        EDB_ROPE(float, __half);
    } else if (ti == GGML_TYPE_F32 && to == GGML_TYPE_BF16) {
        EDB_ROPE(float, __nv_bfloat16);
    } else if (ti == GGML_TYPE_BF16 && to == GGML_TYPE_F32) {
        EDB_ROPE(__nv_bfloat16, float);
    } else if (ti == GGML_TYPE_BF16 && to == GGML_TYPE_F16) {
        EDB_ROPE(__nv_bfloat16, __half);
    } else {
        EDB_ROPE(__nv_bfloat16, __nv_bfloat16);
    }
#undef EDB_ROPE
    count_launch();
    return cudaGetLastError() == cudaSuccess;
}

bool ed_cuda_attention_v_prep_custom_supported(const ggml_tensor* dst) {
    PackArgs a;
    return pack_args(dst, 0, &a);
}
bool ed_cuda_attention_v_prep_custom_compute(ggml_tensor* dst, void* stream) { return pack_compute(dst, 0, stream); }
bool ed_cuda_attention_pair_pack_custom_supported(const ggml_tensor* dst) {
    PackArgs a;
    return pack_args(dst, 1, &a);
}
bool ed_cuda_attention_pair_pack_custom_compute(ggml_tensor* dst, void* stream) { return pack_compute(dst, 1, stream); }
bool ed_cuda_attention_qkv_pair_pack_custom_supported(const ggml_tensor* dst) {
    PackArgs a;
    return pack_args(dst, 2, &a);
}
bool ed_cuda_attention_qkv_pair_pack_custom_compute(ggml_tensor* dst, void* stream) { return pack_compute(dst, 2, stream); }

bool ed_cuda_sage_attn_custom_supported(const ggml_tensor* dst) {
    SageShape sh;
    return sage_shape(dst, &sh);
}

bool ed_cuda_sage_attn_scratch_sizes_for(const ggml_tensor* dst, ed_cuda_sage_attn_scratch_sizes* out) {
    SageShape sh;
    if (out == nullptr || !sage_shape(dst, &sh)) return false;
    *out = ed_cuda_sage_attn_scratch_sizes();
    const size_t lpad = static_cast<size_t>((sh.L + 127) / 128 * 128);
    const size_t elems = static_cast<size_t>(sh.HN * sh.L * sh.d_head);
    out->q_int8_bytes = elems;
    out->k_int8_bytes = elems;
    out->q_scale_bytes = static_cast<size_t>(sh.HN) * (lpad / 32) * 4;
    out->k_scale_bytes = static_cast<size_t>(sh.HN) * (lpad / 64) * 4;
    out->km_bytes = static_cast<size_t>(sh.HN * sh.d_head) * 4;
    out->v_f16_bytes = elems * 2;
    // chunk sums of the two channel means (q and k): [2][HN][lpad / 128][d] floats
    out->o_half_bytes = 2 * static_cast<size_t>(sh.HN) * (lpad / 128) * sh.d_head * 4;
    out->qm_bytes = sh.smooth_q ? static_cast<size_t>(sh.HN * sh.d_head) * 4 : 0;
    out->qk_bias_bytes = sh.smooth_q ? static_cast<size_t>(sh.HN) * lpad * 4 : 0;
    return true;
}

bool ed_cuda_sage_attn_custom_compute(ggml_tensor* dst, const ed_cuda_sage_attn_scratch* scratch, void* stream) {
    SageShape sh;
    if (scratch == nullptr || !sage_shape(dst, &sh)) return false;
    if (scratch->q_int8 == nullptr || scratch->k_int8 == nullptr || scratch->q_scale == nullptr || scratch->k_scale == nullptr ||
        scratch->km == nullptr || scratch->v_f16 == nullptr || scratch->o_half == nullptr ||
        (sh.smooth_q && (scratch->qm == nullptr || scratch->qk_bias == nullptr))) {
        return false;
    }
    const long long lpad = (sh.L + 127) / 128 * 128;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    View v;
    if (!make_view(dst->src[2], &v)) return false;
    const long long total = sh.HN * sh.L * sh.d_head;
    if (dst->src[2]->type == GGML_TYPE_F16) {
        sage_v_to_f16_kernel<uint16_t><<<blocks_for(total), 256, 0, s>>>(v, sh.v_packed, sh.d_head, sh.L, sh.n_head,
                                                                         static_cast<__half*>(scratch->v_f16), total);
    } else {
        sage_v_to_f16_kernel<uint32_t><<<blocks_for(total), 256, 0, s>>>(v, sh.v_packed, sh.d_head, sh.L, sh.n_head,
                                                                         static_cast<__half*>(scratch->v_f16), total);
    }
    count_launch();
    SagePtrs sp;
    sp.q8 = static_cast<int8_t*>(scratch->q_int8);
    sp.k8 = static_cast<int8_t*>(scratch->k_int8);
    sp.q_scale = static_cast<float*>(scratch->q_scale);
    sp.k_scale = static_cast<float*>(scratch->k_scale);
    sp.qm = static_cast<float*>(scratch->qm);
    sp.km = static_cast<float*>(scratch->km);
    sp.bias = static_cast<float*>(scratch->qk_bias);
    sp.part_q = static_cast<float*>(scratch->o_half);
    sp.part_k = sp.part_q + sh.HN * (lpad / 128) * sh.d_head;
    sp.q_scale_stride = static_cast<int>(lpad / 32);
    sp.k_scale_stride = static_cast<int>(lpad / 64);
    sp.bias_stride = static_cast<int>(lpad);
    // the reference's own quantisation arithmetic and summation orders (no EDB200_SAGE_FAST_MEANS): this
    // entry point stands in for its kernels one to one
    const int flags = sh.smooth_q ? EDB200_SAGE_SMOOTH_Q : 0;
    const float scale = 1.0f / sqrtf(static_cast<float>(sh.d_head));
    // dst f32 [d, HN, L]: row l holds all HN heads, head hn at column hn * d
    const edb200_status_t st =
        sage_run(dst->src[0]->data, dst->src[1]->data, scratch->v_f16, static_cast<int>(sh.HN), sh.L, sh.L, sh.L,
                 static_cast<int>(sh.d_head), scale, flags, sp, dst->data, EDB200_TYPE_F32, sh.HN * sh.d_head, nullptr, stream, true);
    return st == EDB200_OK;
}

extern "C" {

int edb200_plugin_supported(int which, const struct ggml_tensor* dst) {
    switch (which) {
        case EDB200_PLUGIN_MODULATE: return ed_cuda_fused_modulate_custom_supported(dst);
        case EDB200_PLUGIN_RMS_NORM_MUL_F16: return ed_cuda_rms_norm_mul_f16_custom_supported(dst);
        case EDB200_PLUGIN_ROPE: return ed_cuda_rope_custom_supported(dst);
        case EDB200_PLUGIN_V_PREP: return ed_cuda_attention_v_prep_custom_supported(dst);
        case EDB200_PLUGIN_PAIR_PACK: return ed_cuda_attention_pair_pack_custom_supported(dst);
        case EDB200_PLUGIN_QKV_PAIR_PACK: return ed_cuda_attention_qkv_pair_pack_custom_supported(dst);
        case EDB200_PLUGIN_SAGE_ATTN: return ed_cuda_sage_attn_custom_supported(dst);
        default: return 0;
    }
}

int edb200_plugin_compute(int which, struct ggml_tensor* dst, const void* scratch, void* stream) {
    switch (which) {
        case EDB200_PLUGIN_MODULATE: return ed_cuda_fused_modulate_custom_compute(dst, stream);
        case EDB200_PLUGIN_RMS_NORM_MUL_F16: return ed_cuda_rms_norm_mul_f16_custom_compute(dst, stream);
        case EDB200_PLUGIN_ROPE: return ed_cuda_rope_custom_compute(dst, stream);
        case EDB200_PLUGIN_V_PREP: return ed_cuda_attention_v_prep_custom_compute(dst, stream);
        case EDB200_PLUGIN_PAIR_PACK: return ed_cuda_attention_pair_pack_custom_compute(dst, stream);
        case EDB200_PLUGIN_QKV_PAIR_PACK: return ed_cuda_attention_qkv_pair_pack_custom_compute(dst, stream);
        case EDB200_PLUGIN_SAGE_ATTN:
            return ed_cuda_sage_attn_custom_compute(dst, static_cast<const ed_cuda_sage_attn_scratch*>(scratch), stream);
        default: return 0;
    }
}

int edb200_plugin_sage_scratch_sizes(const struct ggml_tensor* dst, size_t* sizes) {
    ed_cuda_sage_attn_scratch_sizes s;
    if (sizes == nullptr || !ed_cuda_sage_attn_scratch_sizes_for(dst, &s)) return 0;
    static_assert(sizeof(s) == 14 * sizeof(size_t), "fourteen size fields");
    memcpy(sizes, &s, sizeof(s));
    return 1;
}

void edb200_plugin_tensor_layout(size_t* out8) {
    if (out8 == nullptr) return;
    out8[0] = sizeof(ggml_tensor);
    out8[1] = offsetof(ggml_tensor, type);
    out8[2] = offsetof(ggml_tensor, ne);
    out8[3] = offsetof(ggml_tensor, nb);
    out8[4] = offsetof(ggml_tensor, op);
    out8[5] = offsetof(ggml_tensor, op_params);
    out8[6] = offsetof(ggml_tensor, src);
    out8[7] = offsetof(ggml_tensor, data);
}

}  // extern "C"
