/*
 * edb200_ggml.h -- the ggml declarations that the operator plugin entry points of this library
 * (edb200_shims.h) are written against.
 *
 * The plugin ABI of the reference passes `ggml_tensor*` (src/core/backend/ggml/cuda/ed_cuda_*.h).
 * Where ggml's own header is available, build with -DEDB200_USE_GGML_HEADER and it is included
 * instead, so the entry points see the real structure.  Otherwise this file declares a stand-in with
 * the fields those entry points read (type, ne, nb, op, op_params, src, data) under ggml's names and
 * ggml's type ids; its memory layout is NOT ggml's, so a binary built this way is for callers that
 * build their tensors from this header too (the tests of this repository do).
 */
#ifndef EDB200_GGML_H
#define EDB200_GGML_H

#ifdef EDB200_USE_GGML_HEADER
#include "ggml.h"
#else

#include <stddef.h>
#include <stdint.h>

#define GGML_MAX_DIMS 4
#define GGML_MAX_SRC 10
#define GGML_MAX_OP_PARAMS 64
#define GGML_N_TASKS_MAX (-1)

enum ggml_type {
    GGML_TYPE_F32 = 0,
    GGML_TYPE_F16 = 1,
    GGML_TYPE_Q8_0 = 8,
    GGML_TYPE_Q4_K = 12,
    GGML_TYPE_I8 = 24,
    GGML_TYPE_BF16 = 30
};

/* only the operation kinds the plugin entry points test for */
enum ggml_op {
    GGML_OP_NONE = 0,
    GGML_OP_CUSTOM = 1
};

struct ggml_tensor {
    enum ggml_type type;
    int64_t ne[GGML_MAX_DIMS]; /* elements per dimension, fastest first */
    size_t nb[GGML_MAX_DIMS];  /* stride in bytes per dimension */
    enum ggml_op op;
    int32_t op_params[GGML_MAX_OP_PARAMS / sizeof(int32_t)];
    struct ggml_tensor* src[GGML_MAX_SRC];
    void* data;
    char name[64];
};

typedef void (*ggml_custom_op_t)(struct ggml_tensor* dst, int ith, int nth, void* userdata);

#endif /* EDB200_USE_GGML_HEADER */
#endif /* EDB200_GGML_H */
