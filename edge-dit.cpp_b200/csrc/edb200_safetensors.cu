// Weight ingest from safetensors files (src/utils/model_io/safetensors_io.h in the reference):
//   u64 header length | JSON header | tensor data
// The header maps tensor names to {"dtype": "F32"|"F16"|"BF16"|..., "shape": [...],
// "data_offsets": [begin, end]} (offsets from the end of the header) plus an optional
// "__metadata__" object of strings.  Shapes are row-major: the last extent is the row length.
// Host code; the file is mapped.  Unquantised checkpoints are quantised on the device while
// they load (q8_0: the bit-exact ggml-rule encoder of edb200_quantize_rows_q8_0).
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

struct edb200_safetensors {
    int fd = -1;
    const uint8_t* base = nullptr;
    size_t size = 0;
    struct Tensor {
        std::string name, dtype;
        int n_dims = 0;
        int64_t dims[8] = {1, 1, 1, 1, 1, 1, 1, 1};
        uint64_t begin = 0, end = 0;   // from the start of the file
    };
    std::vector<Tensor> tensors;
};

namespace edb {
namespace {

// Just enough JSON for a safetensors header: objects, arrays, strings and non-negative integers.
struct Json {
    const char* p;
    const char* end;
    bool ok = true;
    void ws() {
        while (p < end && (*p == ' ' || *p == '\n' || *p == '\t' || *p == '\r')) ++p;
    }
    bool eat(char c) {
        ws();
        if (p < end && *p == c) {
            ++p;
            return true;
        }
        return false;
    }
    bool peek(char c) {
        ws();
        return p < end && *p == c;
    }
    std::string str() {
        std::string s;
        if (!eat('"')) {
            ok = false;
            return s;
        }
        while (p < end && *p != '"') {
            if (*p == '\\' && p + 1 < end) {
                ++p;
                switch (*p) {
                    case 'n': s.push_back('\n'); break;
                    case 't': s.push_back('\t'); break;
                    case 'u':   // keep the escape as written: names are compared byte for byte
                        s += "\\u";
                        break;
                    default: s.push_back(*p); break;
                }
                ++p;
            } else {
                s.push_back(*p++);
            }
        }
        if (p >= end) {
            ok = false;
            return s;
        }
        ++p;
        return s;
    }
    uint64_t num() {
        ws();
        if (p >= end || *p < '0' || *p > '9') {
            ok = false;
            return 0;
        }
        uint64_t v = 0;
        while (p < end && *p >= '0' && *p <= '9') {
            if (v > (~0ull - 9) / 10) {
                ok = false;
                return 0;
            }
            v = v * 10 + static_cast<uint64_t>(*p++ - '0');
        }
        return v;
    }
    // Skips any value (used for "__metadata__" and unknown fields).
    void skip(int depth = 0) {
        ws();
        if (!ok || p >= end || depth > 8) {
            ok = false;
            return;
        }
        if (*p == '"') {
            str();
        } else if (*p == '{' || *p == '[') {
            const char close = *p == '{' ? '}' : ']';
            const bool object = *p == '{';
            ++p;
            if (eat(close)) return;
            do {
                if (object) {
                    str();
                    if (!eat(':')) ok = false;
                }
                skip(depth + 1);
            } while (ok && eat(','));
            if (!eat(close)) ok = false;
        } else {
            while (p < end && *p != ',' && *p != '}' && *p != ']') ++p;   // number / true / false / null
        }
    }
};

// Shard files named by a `*.safetensors.index.json` ({"metadata": {...}, "weight_map": {tensor: file}}),
// each once, in order of first appearance, resolved against the index file's directory.
edb200_status_t index_shards(const char* path, std::vector<std::string>& files) {
    files.clear();
    const int fd = open(path, O_RDONLY);
    if (fd < 0) return fail(EDB200_ERR_INVALID, "safetensors index: cannot open '%s'", path);
    struct stat st;
    std::string text;
    if (fstat(fd, &st) == 0 && st.st_size > 0 && st.st_size < (1 << 28)) {
        text.resize(static_cast<size_t>(st.st_size));
        size_t got = 0;
        while (got < text.size()) {
            const ssize_t r = read(fd, &text[got], text.size() - got);
            if (r <= 0) break;
            got += static_cast<size_t>(r);
        }
        text.resize(got);
    }
    close(fd);
    std::string dir(path);
    const size_t slash = dir.find_last_of('/');
    dir = slash == std::string::npos ? std::string() : dir.substr(0, slash + 1);
    Json j{text.data(), text.data() + text.size()};
    bool found = false;
    if (!j.eat('{')) return fail(EDB200_ERR_INVALID, "safetensors index '%s': not a JSON object", path);
    if (!j.peek('}')) {
        do {
            const std::string key = j.str();
            if (!j.ok || !j.eat(':')) break;
            if (key != "weight_map") {
                j.skip();
                continue;
            }
            found = true;
            if (!j.eat('{')) {
                j.ok = false;
                break;
            }
            if (!j.peek('}')) {
                do {
                    j.str();   // tensor name
                    if (!j.ok || !j.eat(':')) {
                        j.ok = false;
                        break;
                    }
                    const std::string file = j.str();
                    if (!j.ok) break;
                    if (file.empty() || file.find('/') != std::string::npos || file.find("..") != std::string::npos) {
                        return fail(EDB200_ERR_INVALID, "safetensors index '%s': shard name '%s' is not a plain file name",
                                    path, file.c_str());
                    }
                    const std::string full = dir + file;
                    bool seen = false;
                    for (const auto& f : files) seen = seen || f == full;
                    if (!seen) files.push_back(full);
                } while (j.ok && j.eat(','));
            }
            if (!j.eat('}')) j.ok = false;
        } while (j.ok && j.eat(','));
    }
    if (!j.ok || !found || files.empty()) {
        return fail(EDB200_ERR_INVALID, "safetensors index '%s': no readable weight_map", path);
    }
    return EDB200_OK;
}

bool is_index(const char* path) {
    static const char kSuffix[] = ".index.json";
    const size_t n = strlen(path), m = sizeof(kSuffix) - 1;
    return n >= m && strcmp(path + n - m, kSuffix) == 0;
}

int dtype_bytes(const std::string& d) {
    if (d == "F32" || d == "I32" || d == "U32") return 4;
    if (d == "F16" || d == "BF16" || d == "I16" || d == "U16") return 2;
    if (d == "F64" || d == "I64" || d == "U64") return 8;
    if (d == "I8" || d == "U8" || d == "BOOL" || d == "F8_E4M3" || d == "F8_E5M2") return 1;
    return 0;
}

}  // namespace

// Hands every F32 / F16 / BF16 tensor of one file to the ingest stage.
static edb200_status_t offer_file(Ingest& ingest, const char* path) {
    edb200_safetensors_t* f = nullptr;
    edb200_status_t st = edb200_safetensors_open(path, &f);
    if (st != EDB200_OK) return st;
    struct Closer {
        edb200_safetensors_t* f;
        ~Closer() { edb200_safetensors_close(f); }
    } closer{f};
    for (const auto& t : f->tensors) {
        SourceTensor src;
        src.name = t.name;
        src.n_elements = 1;
        for (int d = 0; d < t.n_dims; ++d) src.n_elements *= t.dims[d];
        src.row_len = t.n_dims == 2 ? t.dims[1] : 0;
        src.data = f->base + t.begin;
        src.nbytes = static_cast<int64_t>(t.end - t.begin);
        if (t.dtype == "F32") {
            src.type = EDB200_TYPE_F32;
        } else if (t.dtype == "F16") {
            src.type = 1;
        } else if (t.dtype == "BF16") {
            src.type = 30;
        } else {
            src.type = -1;   // integer tables and the like: refused only if the model asks for the tensor
            src.nbytes = -1;
        }
        st = ingest.offer(src);
        if (st != EDB200_OK) return st;
    }
    return EDB200_OK;
}

// Parameters the model keeps as f32 are widened on the host; parameters it keeps quantised are uploaded as
// f32 rows and encoded on the device in the model's block type (q8_0: ggml's rule, bit for bit; q4_K: this
// library's min/max encoder, the one init_random uses), then repacked like any other tensor.  The parts of
// a fused tensor may sit in different shards of a sharded checkpoint.
edb200_status_t load_safetensors(ParamTable& table, int family, const char* path, const char* strip_prefix,
                                 cudaStream_t stream, int* n_loaded) {
    if (n_loaded) *n_loaded = 0;
    std::vector<std::string> files;
    if (is_index(path)) {   // a sharded checkpoint: every shard of the index in turn
        const edb200_status_t ist = index_shards(path, files);
        if (ist != EDB200_OK) return ist;
    } else {
        files.push_back(path);
    }
    Ingest ingest(table, family, strip_prefix, stream);
    for (const auto& file : files) {
        const edb200_status_t st = offer_file(ingest, file.c_str());
        if (st != EDB200_OK) return st;
    }
    return ingest.finish(n_loaded);
}

}  // namespace edb

using namespace edb;

extern "C" {

void edb200_safetensors_close(edb200_safetensors_t* f) {
    if (f == nullptr) return;
    if (f->base != nullptr) munmap(const_cast<uint8_t*>(f->base), f->size);
    if (f->fd >= 0) close(f->fd);
    delete f;
}

edb200_status_t edb200_safetensors_open(const char* path, edb200_safetensors_t** out) {
    if (path == nullptr || out == nullptr) return fail(EDB200_ERR_INVALID, "safetensors_open: null argument");
    *out = nullptr;
    const int fd = open(path, O_RDONLY);
    if (fd < 0) return fail(EDB200_ERR_INVALID, "safetensors_open: cannot open '%s'", path);
    struct stat st;
    if (fstat(fd, &st) != 0 || st.st_size < 10) {
        close(fd);
        return fail(EDB200_ERR_INVALID, "safetensors_open: '%s' is too short", path);
    }
    void* map = mmap(nullptr, static_cast<size_t>(st.st_size), PROT_READ, MAP_PRIVATE, fd, 0);
    if (map == MAP_FAILED) {
        close(fd);
        return fail(EDB200_ERR_NOMEM, "safetensors_open: mmap of '%s' failed", path);
    }
    edb200_safetensors* f = new (std::nothrow) edb200_safetensors();
    if (f == nullptr) {
        munmap(map, static_cast<size_t>(st.st_size));
        close(fd);
        return fail(EDB200_ERR_NOMEM, "safetensors_open: host allocation failed");
    }
    f->fd = fd;
    f->base = static_cast<const uint8_t*>(map);
    f->size = static_cast<size_t>(st.st_size);
    auto bail = [&](const char* what) {
        edb200_safetensors_close(f);
        return fail(EDB200_ERR_INVALID, "safetensors_open: '%s': %s", path, what);
    };
    uint64_t hlen = 0;
    memcpy(&hlen, f->base, 8);
    if (hlen < 2 || hlen > f->size - 8 || hlen > (1ull << 28)) return bail("implausible header length");
    const uint64_t data_start = 8 + hlen;
    Json j{reinterpret_cast<const char*>(f->base + 8), reinterpret_cast<const char*>(f->base + data_start)};
    if (!j.eat('{')) return bail("header is not a JSON object");
    if (!j.peek('}')) {
        do {
            edb200_safetensors::Tensor t;
            t.name = j.str();
            if (!j.ok || !j.eat(':')) return bail("malformed header");
            if (t.name == "__metadata__") {
                j.skip();
                if (!j.ok) return bail("malformed __metadata__");
                continue;
            }
            if (!j.eat('{')) return bail("tensor entry is not an object");
            bool have_off = false;
            if (!j.peek('}')) {
                do {
                    const std::string key = j.str();
                    if (!j.ok || !j.eat(':')) return bail("malformed tensor entry");
                    if (key == "dtype") {
                        t.dtype = j.str();
                    } else if (key == "shape") {
                        if (!j.eat('[')) return bail("shape is not an array");
                        if (!j.peek(']')) {
                            do {
                                if (t.n_dims >= 8) return bail("more than 8 dimensions");
                                t.dims[t.n_dims++] = static_cast<int64_t>(j.num());
                            } while (j.ok && j.eat(','));
                        }
                        if (!j.eat(']')) return bail("malformed shape");
                    } else if (key == "data_offsets") {
                        if (!j.eat('[')) return bail("data_offsets is not an array");
                        t.begin = j.num();
                        if (!j.eat(',')) return bail("malformed data_offsets");
                        t.end = j.num();
                        if (!j.eat(']')) return bail("malformed data_offsets");
                        have_off = true;
                    } else {
                        j.skip();
                    }
                    if (!j.ok) return bail("malformed tensor entry");
                } while (j.eat(','));
            }
            if (!j.eat('}')) return bail("malformed tensor entry");
            const int es = dtype_bytes(t.dtype);
            int64_t n = 1;
            for (int d = 0; d < t.n_dims; ++d) n *= t.dims[d];
            if (!have_off || es == 0) return bail("tensor entry without dtype or data_offsets");
            if (t.end < t.begin || t.end - t.begin != static_cast<uint64_t>(n) * es) {
                return bail("data_offsets do not match shape and dtype");
            }
            t.begin += data_start;
            t.end += data_start;
            if (t.end > f->size) return bail("tensor data runs past the end of the file");
            f->tensors.push_back(t);
        } while (j.ok && j.eat(','));
    }
    if (!j.ok || !j.eat('}')) return bail("malformed header");
    *out = f;
    return EDB200_OK;
}

edb200_status_t edb200_safetensors_index_files(const char* index_path, char* out, int out_cap, int* n_files) {
    if (index_path == nullptr || out == nullptr || out_cap <= 0) {
        return fail(EDB200_ERR_INVALID, "safetensors_index_files: null argument");
    }
    std::vector<std::string> files;
    edb200_status_t st = index_shards(index_path, files);
    if (st != EDB200_OK) return st;
    std::string joined;
    for (const auto& f : files) {
        joined += f;
        joined.push_back('\n');
    }
    if (static_cast<int>(joined.size()) >= out_cap) {
        return fail(EDB200_ERR_INVALID, "safetensors_index_files: %d bytes needed, %d given", (int)joined.size() + 1, out_cap);
    }
    memcpy(out, joined.c_str(), joined.size() + 1);
    if (n_files) *n_files = static_cast<int>(files.size());
    return EDB200_OK;
}

int edb200_safetensors_tensor_count(const edb200_safetensors_t* f) { return f ? static_cast<int>(f->tensors.size()) : 0; }

edb200_status_t edb200_safetensors_tensor_info(const edb200_safetensors_t* f, int index, char* name, int name_cap,
                                               char* dtype, int dtype_cap, int* n_dims, int64_t* dims,
                                               int64_t* nbytes) {
    if (f == nullptr || index < 0 || index >= static_cast<int>(f->tensors.size())) {
        return fail(EDB200_ERR_INVALID, "safetensors_tensor_info: bad handle or index");
    }
    const auto& t = f->tensors[static_cast<size_t>(index)];
    if (name != nullptr && name_cap > 0) {
        strncpy(name, t.name.c_str(), static_cast<size_t>(name_cap) - 1);
        name[name_cap - 1] = 0;
    }
    if (dtype != nullptr && dtype_cap > 0) {
        strncpy(dtype, t.dtype.c_str(), static_cast<size_t>(dtype_cap) - 1);
        dtype[dtype_cap - 1] = 0;
    }
    if (n_dims) *n_dims = t.n_dims;
    if (dims) {
        for (int d = 0; d < 8; ++d) dims[d] = t.dims[d];
    }
    if (nbytes) *nbytes = static_cast<int64_t>(t.end - t.begin);
    return EDB200_OK;
}

const void* edb200_safetensors_tensor_data(const edb200_safetensors_t* f, int index) {
    if (f == nullptr || index < 0 || index >= static_cast<int>(f->tensors.size())) return nullptr;
    return f->base + f->tensors[static_cast<size_t>(index)].begin;
}

}  // extern "C"
