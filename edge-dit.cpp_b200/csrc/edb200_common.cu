// Host-side plumbing shared by every entry point: error strings, launch
// counter, device status word, TMA descriptor encoding.
#include "edb200_internal.h"

#include <cstdarg>
#include <cstdio>
#include <mutex>
#include <vector>

namespace edb {

static thread_local char g_last_error[512] = "";
static std::atomic<int64_t> g_launches{0};

edb200_status_t fail(edb200_status_t st, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_last_error, sizeof(g_last_error), fmt, ap);
    va_end(ap);
    return st;
}

edb200_status_t check_cuda(cudaError_t e, const char* what) {
    if (e == cudaSuccess) return EDB200_OK;
    return fail(EDB200_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e));
}

void count_launch(int n) { g_launches.fetch_add(n, std::memory_order_relaxed); }

static int* g_err_word[64] = {nullptr};
static std::mutex g_err_mu;

int* device_error_word() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    std::lock_guard<std::mutex> lk(g_err_mu);
    if (g_err_word[dev] == nullptr) {
        int* p = nullptr;
        if (cudaMalloc(&p, sizeof(int)) != cudaSuccess) return nullptr;
        cudaMemset(p, 0, sizeof(int));
        g_err_word[dev] = p;
    }
    return g_err_word[dev];
}

edb200_status_t poll_device_error(cudaStream_t stream) {
    int* w = device_error_word();
    if (w == nullptr) return fail(EDB200_ERR_CUDA, "no CUDA device");
    int host = 0;
    cudaError_t e = cudaMemcpyAsync(&host, w, sizeof(int), cudaMemcpyDeviceToHost, stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(stream);
    if (e != cudaSuccess) return check_cuda(e, "poll_device_error");
    if (host != 0) {
        cudaMemsetAsync(w, 0, sizeof(int), stream);
        return fail(EDB200_ERR_TIMEOUT, "device-side wait timed out (code %d)", host);
    }
    return EDB200_OK;
}

PFN_encodeTiled get_encode_tiled() {
    static PFN_encodeTiled fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess) {
            fn = reinterpret_cast<PFN_encodeTiled>(p);
        }
    });
    return fn;
}

edb200_status_t make_tmap_2d(CUtensorMap* map, CUtensorMapDataType dt, int elem_bytes, const void* base,
                             uint64_t inner, uint64_t outer, uint64_t pitch_bytes, uint32_t box_inner,
                             uint32_t box_outer, CUtensorMapSwizzle swz) {
    PFN_encodeTiled enc = get_encode_tiled();
    if (enc == nullptr) return fail(EDB200_ERR_CUDA, "cuTensorMapEncodeTiled unavailable");
    if ((reinterpret_cast<uintptr_t>(base) & 15u) != 0 || (pitch_bytes & 15u) != 0 ||
        ((uint64_t)box_inner * elem_bytes) % 16 != 0) {
        return fail(EDB200_ERR_INVALID, "tensor map: base/pitch/box not 16-byte aligned");
    }
    cuuint64_t dims[2] = {inner, outer};
    cuuint64_t strides[1] = {pitch_bytes};
    cuuint32_t box[2] = {box_inner, box_outer};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = enc(map, dt, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swz,
                     CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(EDB200_ERR_CUDA, "cuTensorMapEncodeTiled(2d) failed: %d", (int)r);
    return EDB200_OK;
}

edb200_status_t make_tmap_3d(CUtensorMap* map, CUtensorMapDataType dt, int elem_bytes, const void* base,
                             uint64_t d0, uint64_t d1, uint64_t d2, uint64_t pitch1_bytes, uint64_t pitch2_bytes,
                             uint32_t b0, uint32_t b1, uint32_t b2, CUtensorMapSwizzle swz) {
    PFN_encodeTiled enc = get_encode_tiled();
    if (enc == nullptr) return fail(EDB200_ERR_CUDA, "cuTensorMapEncodeTiled unavailable");
    if ((reinterpret_cast<uintptr_t>(base) & 15u) != 0 || (pitch1_bytes & 15u) != 0 || (pitch2_bytes & 15u) != 0 ||
        ((uint64_t)b0 * elem_bytes) % 16 != 0) {
        return fail(EDB200_ERR_INVALID, "tensor map: base/pitch/box not 16-byte aligned");
    }
    cuuint64_t dims[3] = {d0, d1, d2};
    cuuint64_t strides[2] = {pitch1_bytes, pitch2_bytes};
    cuuint32_t box[3] = {b0, b1, b2};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = enc(map, dt, 3, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swz,
                     CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(EDB200_ERR_CUDA, "cuTensorMapEncodeTiled(3d) failed: %d", (int)r);
    return EDB200_OK;
}

int sm_count() {
    static int n = 0;
    if (n == 0) {
        int dev = 0;
        cudaDeviceProp p;
        if (cudaGetDevice(&dev) == cudaSuccess && cudaGetDeviceProperties(&p, dev) == cudaSuccess) {
            n = p.multiProcessorCount;
        } else {
            n = 148;
        }
    }
    return n;
}

struct ProfRecord {
    cudaEvent_t a, b;
    ProfClass cls;
    double flops, bytes;
};
static bool g_prof_on = false;
static std::vector<ProfRecord> g_prof;
static cudaEvent_t g_prof_pending = nullptr;

bool profiling_enabled() { return g_prof_on; }

void profile_begin_launch(cudaStream_t s) {
    cudaEvent_t e;
    cudaEventCreate(&e);
    cudaEventRecord(e, s);
    g_prof_pending = e;
}

void profile_end_launch(cudaStream_t s, ProfClass cls, double flops, double bytes) {
    ProfRecord r;
    r.a = g_prof_pending;
    cudaEventCreate(&r.b);
    cudaEventRecord(r.b, s);
    r.cls = cls;
    r.flops = flops;
    r.bytes = bytes;
    g_prof.push_back(r);
}

}  // namespace edb

extern "C" {

edb200_status_t edb200_profile_begin(void) {
    edb::g_prof.clear();
    edb::g_prof_on = true;
    return EDB200_OK;
}

edb200_status_t edb200_profile_end(double* ms, double* flops, double* bytes, int64_t* launches) {
    edb::g_prof_on = false;
    cudaError_t e = cudaDeviceSynchronize();
    if (e != cudaSuccess) return edb::check_cuda(e, "profile_end");
    for (int c = 0; c < edb::PROF_NCLASS; ++c) {
        if (ms) ms[c] = 0;
        if (flops) flops[c] = 0;
        if (bytes) bytes[c] = 0;
        if (launches) launches[c] = 0;
    }
    for (edb::ProfRecord& r : edb::g_prof) {
        float t = 0.0f;
        cudaEventElapsedTime(&t, r.a, r.b);
        if (ms) ms[r.cls] += t;
        if (flops) flops[r.cls] += r.flops;
        if (bytes) bytes[r.cls] += r.bytes;
        if (launches) launches[r.cls] += 1;
        cudaEventDestroy(r.a);
        cudaEventDestroy(r.b);
    }
    edb::g_prof.clear();
    return EDB200_OK;
}

const char* edb200_last_error(void) { return edb::g_last_error; }

const char* edb200_version(void) { return "edb200 0.1 (sm_100a)"; }

int64_t edb200_launch_count(void) { return edb::g_launches.load(std::memory_order_relaxed); }

// ---------------------------------------------------------------- CUDA graphs
struct edb200_graph {
    cudaGraphExec_t exec = nullptr;
    int64_t launches = 0;   // kernels of this library recorded in the graph
};

static thread_local int64_t g_capture_launches0 = 0;

edb200_status_t edb200_graph_begin(void* stream) {
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (s == nullptr) return edb::fail(EDB200_ERR_INVALID, "graph_begin: capture needs a non-default stream");
    if (edb::profiling_enabled()) return edb::fail(EDB200_ERR_INVALID, "graph_begin: end the profile first");
    g_capture_launches0 = edb::g_launches.load(std::memory_order_relaxed);
    return edb::check_cuda(cudaStreamBeginCapture(s, cudaStreamCaptureModeThreadLocal), "cudaStreamBeginCapture");
}

edb200_status_t edb200_graph_end(void* stream, edb200_graph_t** out) {
    if (out == nullptr) return edb::fail(EDB200_ERR_INVALID, "graph_end: null argument");
    cudaGraph_t graph = nullptr;
    cudaError_t e = cudaStreamEndCapture(static_cast<cudaStream_t>(stream), &graph);
    if (e != cudaSuccess || graph == nullptr) {
        cudaGetLastError();
        return edb::fail(EDB200_ERR_CUDA, "graph_end: cudaStreamEndCapture: %s", cudaGetErrorString(e));
    }
    edb200_graph* g = new (std::nothrow) edb200_graph();
    if (g == nullptr) {
        cudaGraphDestroy(graph);
        return edb::fail(EDB200_ERR_NOMEM, "graph_end: host allocation failed");
    }
    e = cudaGraphInstantiate(&g->exec, graph, 0);
    cudaGraphDestroy(graph);
    if (e != cudaSuccess) {
        delete g;
        return edb::check_cuda(e, "cudaGraphInstantiate");
    }
    g->launches = edb::g_launches.load(std::memory_order_relaxed) - g_capture_launches0;
    *out = g;
    return EDB200_OK;
}

edb200_status_t edb200_graph_launch(edb200_graph_t* g, void* stream) {
    if (g == nullptr || g->exec == nullptr) return edb::fail(EDB200_ERR_INVALID, "graph_launch: null graph");
    edb::count_launch(static_cast<int>(g->launches));
    return edb::check_cuda(cudaGraphLaunch(g->exec, static_cast<cudaStream_t>(stream)), "cudaGraphLaunch");
}

void edb200_graph_destroy(edb200_graph_t* g) {
    if (g == nullptr) return;
    if (g->exec != nullptr) cudaGraphExecDestroy(g->exec);
    delete g;
}

}  // extern "C"
