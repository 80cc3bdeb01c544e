/* Stand-in for ggml-backend.h: the reference's loader headers only name these handle types.
 * Test infrastructure for the parity oracle; never part of the product path. */
#ifndef EDB_REF_SHIM_GGML_BACKEND_H
#define EDB_REF_SHIM_GGML_BACKEND_H
#include "ggml.h"
typedef struct ggml_backend* ggml_backend_t;
typedef struct ggml_backend_buffer* ggml_backend_buffer_t;
#endif
