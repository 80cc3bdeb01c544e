// Weight ingest: a reader for GGUF files (the container `ed-convert` writes,
// src/utils/model_io/gguf_io.cpp) and the loop that hands the tensors a model asks
// for to its parameter table.  Host code only; the file is mapped, never copied.
//
// GGUF v2/v3 layout (little endian):
//   u32 magic "GGUF" | u32 version | u64 n_tensors | u64 n_kv
//   n_kv  x { string key | u32 type | value }          string = u64 length + bytes
//   n_tensors x { string name | u32 n_dims | u64 dims[n_dims] | u32 ggml_type | u64 offset }
//   padding to `general.alignment` (default 32) | tensor data, each at data_start + offset
// dims are in ggml order: dims[0] is the row length (k), dims[1] the number of rows.
#include "edb200_internal.h"
#include "edb200_model.h"

#include <cuda_fp16.h>

#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cstring>
#include <string>
#include <vector>

struct edb200_gguf {
    int fd = -1;
    const uint8_t* base = nullptr;
    size_t size = 0;
    struct Tensor {
        std::string name;
        int ggml_type = 0;
        int n_dims = 0;
        int64_t dims[4] = {1, 1, 1, 1};
        int64_t nbytes = 0;
        uint64_t offset = 0;   // from the start of the file
    };
    std::vector<Tensor> tensors;
    uint32_t version = 0;
    uint64_t alignment = 32;
};

namespace edb {
namespace {

constexpr int kGgufTypeF16 = 1;
constexpr int kGgufTypeBF16 = 30;

// Bounds-checked cursor over the mapped file.
struct Cursor {
    const uint8_t* p;
    const uint8_t* end;
    bool ok = true;
    template <typename T>
    T get() {
        T v{};
        if (!ok || static_cast<size_t>(end - p) < sizeof(T)) {
            ok = false;
            return v;
        }
        memcpy(&v, p, sizeof(T));
        p += sizeof(T);
        return v;
    }
    bool skip(uint64_t n) {
        if (!ok || static_cast<uint64_t>(end - p) < n) {
            ok = false;
            return false;
        }
        p += n;
        return true;
    }
    std::string str() {
        const uint64_t n = get<uint64_t>();
        if (!ok || static_cast<uint64_t>(end - p) < n || n > (1u << 20)) {
            ok = false;
            return std::string();
        }
        std::string s(reinterpret_cast<const char*>(p), static_cast<size_t>(n));
        p += n;
        return s;
    }
};

// Size of one scalar of a key/value type; 0 for strings and arrays.
size_t kv_scalar_size(uint32_t t) {
    switch (t) {
        case 0: case 1: case 7: return 1;      // u8, i8, bool
        case 2: case 3: return 2;              // u16, i16
        case 4: case 5: case 6: return 4;      // u32, i32, f32
        case 10: case 11: case 12: return 8;   // u64, i64, f64
        default: return 0;
    }
}

// Skips one value; for `general.alignment` the caller reads it instead.
bool skip_value(Cursor& c, uint32_t type, int depth = 0) {
    if (type == 8) {   // string
        c.str();
        return c.ok;
    }
    if (type == 9) {   // array: element type, count, elements
        if (depth > 2) return false;
        const uint32_t et = c.get<uint32_t>();
        const uint64_t n = c.get<uint64_t>();
        if (!c.ok) return false;
        const size_t es = kv_scalar_size(et);
        if (es) return c.skip(n * es);
        for (uint64_t i = 0; i < n; ++i) {
            if (!skip_value(c, et, depth + 1)) return false;
        }
        return c.ok;
    }
    const size_t s = kv_scalar_size(type);
    return s ? c.skip(s) : false;
}

// Bytes of a tensor of `n` elements with rows of `k`, or -1 for a type this library does not read.
int64_t tensor_bytes(int ggml_type, int64_t n, int64_t k) {
    switch (ggml_type) {
        case EDB200_TYPE_F32: return n * 4;
        case kGgufTypeF16: case kGgufTypeBF16: return n * 2;
        case EDB200_TYPE_Q8_0: return (k % 32) ? -1 : n / 32 * 34;
        case EDB200_TYPE_Q4_K: return (k % 256) ? -1 : n / 256 * 144;
        default: return -1;
    }
}

}  // namespace

// Hands every tensor of the file to the ingest stage, which keeps the ones `table` knows (after removing
// `strip_prefix`, e.g. "model.diffusion_model.", and canonicalising the name for `family`).  Tensors of
// other components (VAE, text encoders) are skipped; tensors the model needs and the file lacks are
// reported by all_loaded() at the first step.
edb200_status_t load_gguf(ParamTable& table, int family, const char* path, const char* strip_prefix, cudaStream_t stream,
                          int* n_loaded) {
    if (n_loaded) *n_loaded = 0;
    edb200_gguf_t* g = nullptr;
    edb200_status_t st = edb200_gguf_open(path, &g);
    if (st != EDB200_OK) return st;
    struct Closer {
        edb200_gguf_t* g;
        ~Closer() { edb200_gguf_close(g); }
    } closer{g};
    Ingest ingest(table, family, strip_prefix, stream);
    for (const auto& t : g->tensors) {
        SourceTensor src;
        src.name = t.name;
        src.type = t.ggml_type;
        src.n_elements = 1;
        for (int d = 0; d < t.n_dims; ++d) src.n_elements *= t.dims[d];
        src.row_len = t.n_dims == 2 ? t.dims[0] : 0;
        src.data = g->base + t.offset;
        src.nbytes = t.nbytes;
        st = ingest.offer(src);
        if (st != EDB200_OK) return st;
    }
    return ingest.finish(n_loaded);
}

}  // namespace edb

using namespace edb;

extern "C" {

edb200_status_t edb200_gguf_open(const char* path, edb200_gguf_t** out) {
    if (path == nullptr || out == nullptr) return fail(EDB200_ERR_INVALID, "gguf_open: null argument");
    *out = nullptr;
    const int fd = open(path, O_RDONLY);
    if (fd < 0) return fail(EDB200_ERR_INVALID, "gguf_open: cannot open '%s'", path);
    struct stat st;
    if (fstat(fd, &st) != 0 || st.st_size < 24) {
        close(fd);
        return fail(EDB200_ERR_INVALID, "gguf_open: '%s' is too short to be a GGUF file", path);
    }
    void* map = mmap(nullptr, static_cast<size_t>(st.st_size), PROT_READ, MAP_PRIVATE, fd, 0);
    if (map == MAP_FAILED) {
        close(fd);
        return fail(EDB200_ERR_NOMEM, "gguf_open: mmap of '%s' failed", path);
    }
    edb200_gguf* g = new (std::nothrow) edb200_gguf();
    if (g == nullptr) {
        munmap(map, static_cast<size_t>(st.st_size));
        close(fd);
        return fail(EDB200_ERR_NOMEM, "gguf_open: host allocation failed");
    }
    g->fd = fd;
    g->base = static_cast<const uint8_t*>(map);
    g->size = static_cast<size_t>(st.st_size);
    auto bail = [&](const char* what) {
        edb200_gguf_close(g);
        return fail(EDB200_ERR_INVALID, "gguf_open: '%s': %s", path, what);
    };

    Cursor c{g->base, g->base + g->size};
    if (c.get<uint32_t>() != 0x46554747u) return bail("not a GGUF file (magic)");
    g->version = c.get<uint32_t>();
    if (g->version < 2 || g->version > 3) return bail("unsupported GGUF version (2 and 3 are read)");
    const uint64_t n_tensors = c.get<uint64_t>();
    const uint64_t n_kv = c.get<uint64_t>();
    if (!c.ok || n_tensors > (1u << 24) || n_kv > (1u << 24)) return bail("implausible header counts");
    for (uint64_t i = 0; i < n_kv; ++i) {
        const std::string key = c.str();
        const uint32_t type = c.get<uint32_t>();
        if (!c.ok) return bail("truncated key/value section");
        if (key == "general.alignment" && type == 4) {
            g->alignment = c.get<uint32_t>();
            if (g->alignment == 0 || (g->alignment & (g->alignment - 1))) return bail("alignment is not a power of two");
        } else if (!skip_value(c, type)) {
            return bail("malformed key/value section");
        }
    }
    g->tensors.reserve(static_cast<size_t>(n_tensors));
    for (uint64_t i = 0; i < n_tensors; ++i) {
        edb200_gguf::Tensor t;
        t.name = c.str();
        const uint32_t nd = c.get<uint32_t>();
        if (!c.ok || nd == 0 || nd > 4) return bail("tensor with 0 or more than 4 dimensions");
        t.n_dims = static_cast<int>(nd);
        int64_t n = 1;
        for (uint32_t d = 0; d < nd; ++d) {
            const uint64_t e = c.get<uint64_t>();
            if (!c.ok || e == 0 || e > (1ull << 40)) return bail("implausible tensor extent");
            t.dims[d] = static_cast<int64_t>(e);
            n *= t.dims[d];
        }
        t.ggml_type = static_cast<int>(c.get<uint32_t>());
        t.offset = c.get<uint64_t>();   // relative to the data section for now
        if (!c.ok) return bail("truncated tensor table");
        t.nbytes = tensor_bytes(t.ggml_type, n, t.dims[0]);   // -1: a type this library does not read
        g->tensors.push_back(t);
    }
    const uint64_t table_end = static_cast<uint64_t>(c.p - g->base);
    const uint64_t data_start = (table_end + g->alignment - 1) / g->alignment * g->alignment;
    for (auto& t : g->tensors) {
        t.offset += data_start;
        if (t.nbytes >= 0 && (t.offset > g->size || static_cast<uint64_t>(t.nbytes) > g->size - t.offset)) {
            return bail("tensor data runs past the end of the file");
        }
    }
    *out = g;
    return EDB200_OK;
}

void edb200_gguf_close(edb200_gguf_t* g) {
    if (g == nullptr) return;
    if (g->base != nullptr) munmap(const_cast<uint8_t*>(g->base), g->size);
    if (g->fd >= 0) close(g->fd);
    delete g;
}

int edb200_gguf_tensor_count(const edb200_gguf_t* g) { return g ? static_cast<int>(g->tensors.size()) : 0; }

edb200_status_t edb200_gguf_tensor_info(const edb200_gguf_t* g, int index, char* name, int name_cap, int* ggml_type,
                                        int* n_dims, int64_t* dims, int64_t* nbytes) {
    if (g == nullptr || index < 0 || index >= static_cast<int>(g->tensors.size())) {
        return fail(EDB200_ERR_INVALID, "gguf_tensor_info: bad handle or index");
    }
    const auto& t = g->tensors[static_cast<size_t>(index)];
    if (name != nullptr && name_cap > 0) {
        strncpy(name, t.name.c_str(), static_cast<size_t>(name_cap) - 1);
        name[name_cap - 1] = 0;
    }
    if (ggml_type) *ggml_type = t.ggml_type;
    if (n_dims) *n_dims = t.n_dims;
    if (dims) {
        for (int d = 0; d < 4; ++d) dims[d] = t.dims[d];
    }
    if (nbytes) *nbytes = t.nbytes;
    return EDB200_OK;
}

const void* edb200_gguf_tensor_data(const edb200_gguf_t* g, int index) {
    if (g == nullptr || index < 0 || index >= static_cast<int>(g->tensors.size())) return nullptr;
    const auto& t = g->tensors[static_cast<size_t>(index)];
    return t.nbytes < 0 ? nullptr : g->base + t.offset;
}

}  // extern "C"
