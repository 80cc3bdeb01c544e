/* Minimal stand-in for the ggml declarations that the reference's header-only CPU
 * callbacks use (tensor fields, type ids, f16/bf16 conversions, GGML_ASSERT).  Written
 * for the parity oracle only: it lets those callbacks compile from where they lie in
 * the reference tree, unmodified, without the ggml library.  Test infrastructure; never
 * part of the product path. */
#ifndef EDB_REF_SHIM_GGML_H
#define EDB_REF_SHIM_GGML_H

#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>

/* the tensor structure, type ids and operation kinds are the ones the library's plugin entry points use */
#include "../../include/edb200_ggml.h"

#define GGML_ASSERT(x)                                                                  \
    do {                                                                                \
        if (!(x)) {                                                                     \
            std::fprintf(stderr, "ref shim: assertion failed: %s (%s:%d)\n", #x, __FILE__, __LINE__); \
            std::abort();                                                               \
        }                                                                               \
    } while (0)

typedef uint16_t ggml_fp16_t;
typedef struct {
    uint16_t bits;
} ggml_bf16_t;

struct ggml_context;

static inline size_t ggml_type_size(enum ggml_type t) {
    switch (t) {
        case GGML_TYPE_F32: return 4;
        case GGML_TYPE_F16: return 2;
        case GGML_TYPE_BF16: return 2;
        case GGML_TYPE_I8: return 1;
        case GGML_TYPE_Q8_0: return 34;  /* bytes per block */
        case GGML_TYPE_Q4_K: return 144;
        default: return 0;
    }
}

/* array extents in the reference's loader headers; no table here is indexed beyond the ids above */
#define GGML_TYPE_COUNT ((enum ggml_type)64)

static inline int64_t ggml_blck_size(enum ggml_type t) {
    switch (t) {
        case GGML_TYPE_Q8_0: return 32;
        case GGML_TYPE_Q4_K: return 256;
        default: return 1;
    }
}

static inline const char* ggml_type_name(enum ggml_type t) {
    switch (t) {
        case GGML_TYPE_F32: return "f32";
        case GGML_TYPE_F16: return "f16";
        case GGML_TYPE_BF16: return "bf16";
        case GGML_TYPE_Q8_0: return "q8_0";
        case GGML_TYPE_Q4_K: return "q4_K";
        case GGML_TYPE_I8: return "i8";
        default: return "?";
    }
}

static inline int64_t ggml_nelements(const struct ggml_tensor* t) { return t->ne[0] * t->ne[1] * t->ne[2] * t->ne[3]; }

static inline bool ggml_is_contiguous(const struct ggml_tensor* t) {
    size_t expect = ggml_type_size(t->type);
    for (int i = 0; i < GGML_MAX_DIMS; ++i) {
        if (t->ne[i] != 1 && t->nb[i] != expect) return false;
        expect *= (size_t)t->ne[i];
    }
    return true;
}

static inline bool ggml_are_same_shape(const struct ggml_tensor* a, const struct ggml_tensor* b) {
    return a->ne[0] == b->ne[0] && a->ne[1] == b->ne[1] && a->ne[2] == b->ne[2] && a->ne[3] == b->ne[3];
}

/* rows (dimension 0) are dense; the rows themselves may be strided */
static inline bool ggml_is_contiguous_rows(const struct ggml_tensor* t) {
    return t->ne[0] == 1 || t->nb[0] == ggml_type_size(t->type);
}

static inline float ggml_fp16_to_fp32(ggml_fp16_t h) {
    _Float16 v;
    std::memcpy(&v, &h, 2);
    return (float)v;
}
static inline ggml_fp16_t ggml_fp32_to_fp16(float f) {
    _Float16 v = (_Float16)f; /* IEEE round to nearest even */
    ggml_fp16_t h;
    std::memcpy(&h, &v, 2);
    return h;
}
static inline float ggml_bf16_to_fp32(ggml_bf16_t h) {
    uint32_t u = (uint32_t)h.bits << 16;
    float f;
    std::memcpy(&f, &u, 4);
    return f;
}
static inline ggml_bf16_t ggml_fp32_to_bf16(float f) {
    uint32_t u;
    std::memcpy(&u, &f, 4);
    ggml_bf16_t h;
    if ((u & 0x7fffffffu) > 0x7f800000u) { /* NaN: keep it quiet */
        h.bits = (uint16_t)((u >> 16) | 64);
        return h;
    }
    h.bits = (uint16_t)((u + (0x7fffu + ((u >> 16) & 1u))) >> 16); /* round to nearest even */
    return h;
}

/* Graph construction is not part of the oracle: the builders in the reference headers
 * only need these to exist. */
static inline struct ggml_tensor* ggml_custom_4d(struct ggml_context*, enum ggml_type, int64_t, int64_t, int64_t, int64_t,
                                                 struct ggml_tensor**, int, ggml_custom_op_t, int, void*) {
    return nullptr;
}
static inline struct ggml_tensor* ggml_set_name(struct ggml_tensor* t, const char*) { return t; }

#endif
