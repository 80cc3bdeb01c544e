// Host-side building blocks shared by the per-family denoise-step executors:
// a named parameter table (quantised weights repacked for the GEMM, f32 vectors
// as plain device arrays) and a bump allocator for the step's activations.
#pragma once

#include <map>
#include <string>
#include <vector>

#include "edb200_internal.h"

namespace edb {

struct ParamSpec {
    std::string name;
    int64_t n_out = 0;   // rows (1 for vectors)
    int64_t k = 0;       // row length
    bool quantised = false;
    int ggml_type = EDB200_TYPE_F32;  // storage type expected by set_tensor
};

struct Param {
    ParamSpec spec;
    edb200_qweight_t* qw = nullptr;  // quantised linear weight
    float* f32 = nullptr;            // everything else
    bool loaded = false;
};

// Raw bytes of `rows` rows of `k` weights in a ggml type.
int64_t ggml_row_bytes(int ggml_type, int64_t k);

class ParamTable {
public:
    ~ParamTable();
    void add(const std::string& name, int64_t n_out, int64_t k, bool quantised, int wtype);
    Param* find(const std::string& name);
    const Param* get(const std::string& name) const;
    // Upload one tensor (host or device source) and, for quantised weights, repack it.
    edb200_status_t set(const std::string& name, int ggml_type, const void* data, int64_t nbytes, bool on_device,
                        cudaStream_t stream);
    // Synthetic weights generated on the device: N(0, std) (norm scales 1 + N(0, std)),
    // quantised with the device q8_0 / q4_K encoders.
    edb200_status_t init_random(uint64_t seed, float std, cudaStream_t stream);
    // The tensor's values as f32 [n_out, k] (quantised weights dequantised from the repacked device form,
    // bit-identical to ggml's dequantize_row of the blocks that were loaded) into host or device memory.
    edb200_status_t fetch_f32(const std::string& name, float* out, int64_t n_floats, bool on_device,
                              cudaStream_t stream) const;
    edb200_status_t all_loaded() const;
    int64_t device_bytes() const { return bytes_; }
    // Changes whenever a tensor is (re)loaded: cached views of the weights (e.g. a GEMV batch) are rebuilt.
    uint64_t generation() const { return generation_; }
    std::vector<Param>& params() { return params_; }

private:
    std::vector<Param> params_;
    std::map<std::string, size_t> index_;
    int64_t bytes_ = 0;
    uint64_t generation_ = 0;
};

// One tensor of a checkpoint file as the readers see it.
struct SourceTensor {
    std::string name;
    int type = 0;             // ggml type code (f32 0, f16 1, q8_0 8, q4_K 12, bf16 30)
    int64_t n_elements = 0;
    int64_t row_len = 0;      // innermost extent of a 2-D tensor, 0 otherwise
    const void* data = nullptr;
    int64_t nbytes = 0;       // < 0: a storage type this library does not read
};

// `name` in the layout the executors register, plus the part index of a fused tensor (edb200_ingest.cu).
void canonical_name(int family, const std::string& name, std::string& out, int& part);

// Takes the tensors of one or more files in any order and hands the ones `table` knows to it: names
// canonicalised for the model family, parts of fused tensors assembled, storage types converted.
class Ingest {
public:
    Ingest(ParamTable& table, int family, const char* strip_prefix, cudaStream_t stream);
    edb200_status_t offer(const SourceTensor& t);
    // Fails if a fused tensor was left incomplete; *n_loaded = parameters set.
    edb200_status_t finish(int* n_loaded);

private:
    struct Part {
        int type = 0;
        int64_t n = 0;
        std::vector<uint8_t> bytes;
    };
    struct Staged {
        std::map<int, Part> parts;
        int64_t elements = 0;
    };
    edb200_status_t set_from_f32(const std::string& name, Param* p, const float* src);
    edb200_status_t assemble(const std::string& name, Param* p, Staged& s);

    ParamTable& table_;
    int family_;
    std::string prefix_;
    cudaStream_t stream_;
    std::map<std::string, Staged> staged_;
    std::vector<float> scratch_;
    int count_ = 0;
};

// Loads every tensor of a GGUF file that `table` knows (edb200_gguf.cu); `family` is an EDB200_FAMILY_* code.
edb200_status_t load_gguf(ParamTable& table, int family, const char* path, const char* strip_prefix, cudaStream_t stream,
                          int* n_loaded);

// The same from a safetensors file or a sharded checkpoint's index (edb200_safetensors.cu).
edb200_status_t load_safetensors(ParamTable& table, int family, const char* path, const char* strip_prefix,
                                 cudaStream_t stream, int* n_loaded);

// The computation-reuse seam of a step executor: the three anchors the reference's cache engine taps in every
// model graph (ModelIn before the block stack, BlockOut[i] after block i with the probe stop, ModelOut after
// the stack with the whole-stack inject; src/dit_models/models/mmdit.hpp:3318-3385, wan.hpp:4640-4729,
// qwen_image.hpp:3209-3274).  All of them are views of the stream the blocks transform, f32 [rows of this
// rank, width].
struct ReuseAnchors {
    float* in = nullptr;
    float* out = nullptr;
    std::vector<float*> block;           // [depth], NULL = not captured
    int stop_after = -1;                 // probe pass: return right after this block
    const float* stream_override = nullptr;   // whole-stack inject: stream after the stack = ModelIn + this
    // region inject (substep reuse, mmdit.hpp:3336-3343, wan.hpp:4658-4665): at block `inject_at` the stream becomes
    // ModelIn + inject_residual and the loop resumes at block `inject_resume`
    int inject_at = -1, inject_resume = 0;
    const float* inject_residual = nullptr;

    edb200_status_t set_capture(int anchor, float* dst, int depth, const char* who);
    edb200_status_t set_stop(int blk, int depth, const char* who);
    bool inject() const { return stream_override != nullptr; }
    edb200_status_t set_region(int at, int resume, const float* residual, int depth, const char* who);
    // true when block i starts an injected region: the stream has been rebuilt and `i` moved to the block before
    // the one to resume at (the caller's loop increment does the rest)
    bool region_inject(int& i, float* stream, int64_t n, cudaStream_t s) const;
    // copies on `s`; no-ops where nothing was asked for
    void capture_in(const float* stream, int64_t n, cudaStream_t s) const;
    void capture_block(int i, const float* stream, int64_t n, cudaStream_t s) const;
    void finish(float* stream, int64_t n, cudaStream_t s) const;   // inject (stream += override), then ModelOut
};

// One cudaMalloc carved into 256-byte aligned pieces.
class Workspace {
public:
    ~Workspace();
    edb200_status_t reserve(int64_t bytes);
    void* take(int64_t bytes);   // nullptr when exhausted
    template <typename T>
    T* take_n(int64_t n) { return static_cast<T*>(take(n * (int64_t)sizeof(T))); }
    int64_t capacity() const { return cap_; }
    int64_t used() const { return used_; }
    void* base() const { return base_; }

private:
    char* base_ = nullptr;
    int64_t cap_ = 0, used_ = 0;
};

// Small kernels used by the executors (defined in edb200_model.cu).
void launch_patchify(const float* latent, float* tokens, int C, int H, int W, int p, cudaStream_t s);
void launch_unpatchify(const float* tokens, float* latent, int C, int H, int W, int p, cudaStream_t s);
// out[j] = cos((t*freq[j])*scale), out[half+j] = sin(...); freq is a device table of `half` floats.
void launch_timestep_embedding(const float* freq, float t, float scale, int half, float* out, cudaStream_t s);
// The same with the timestep read on the device: t = sched[*step] * pre_scale.
void launch_timestep_embedding_sched(const float* freq, const float* sched, const int* step, float pre_scale, float scale,
                                     int half, float* out, cudaStream_t s);
void launch_add_inplace(float* dst, const float* src, int64_t n, cudaStream_t s);
// Device q4_K encoder used for synthetic weights (min/max per 32 sub-block).
edb200_status_t quantize_rows_q4_k_device(const float* x, void* blocks, int64_t rows, int64_t k, cudaStream_t s);

}  // namespace edb
