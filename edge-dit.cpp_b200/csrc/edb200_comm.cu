// Sequence-parallel (Ulysses) redistribution between the ranks of one node.
//
// Every rank owns T_loc = T / P consecutive tokens for the per-token work (norms,
// linears, residuals) and H / P heads for attention.  Around attention the layout
// changes twice:
//   heads a2a   [H, T_loc, d] on every rank  ->  [H/P, T, d]   (Q, K and V)
//   tokens a2a  [T, (H/P) d]  on every rank  ->  [T_loc, H d]  (attention output)
// This stands in for the reference's SP pack / split / gather callbacks and their
// NCCL all-to-all (src/core/parallel/sp_parallel.cpp:99-469,757-831,
// src/core/parallel/backends/nccl/nccl_process_group.cpp:394-459).
//
// The head-major layout makes every message of the first exchange one contiguous
// run on both sides, so it needs no pack or unpack kernel at all: one grouped
// ncclSend / ncclRecv per (peer, head, tensor).  The second exchange lands in a
// staging buffer ordered by source rank and one small copy kernel interleaves the
// head groups into the token-major rows that the next linear reads.
//
// NCCL is resolved at run time from the already loaded libnccl.so.2 (the process
// that owns the ranks brings it); the library itself links cudart only.
//
// The faster path needs no exchange kernels at all: once every rank's workspace is
// mapped into its peers (CUDA IPC over NVLink, edb200_comm_map_peers) the producing
// kernels store each result row straight into the owning rank's buffer (Q/K/V pack
// kernel, attention epilogue) and a one-kernel flag barrier (edb200_sp_barrier)
// orders producers and consumers across GPUs.
#include "edb200_internal.h"
#include "edb200_ptx.cuh"

#include <dlfcn.h>

#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <vector>

namespace edb {
namespace {

struct NcclId {
    char internal[128];
};
using nccl_comm_t = void*;
constexpr int kNcclUint8 = 1;

struct NcclApi {
    int (*GetUniqueId)(NcclId*) = nullptr;
    int (*CommInitRank)(nccl_comm_t*, int, NcclId, int) = nullptr;
    int (*CommDestroy)(nccl_comm_t) = nullptr;
    int (*GroupStart)() = nullptr;
    int (*GroupEnd)() = nullptr;
    int (*Send)(const void*, size_t, int, int, nccl_comm_t, cudaStream_t) = nullptr;
    int (*Recv)(void*, size_t, int, int, nccl_comm_t, cudaStream_t) = nullptr;
    const char* (*GetErrorString)(int) = nullptr;
    bool ok = false;
};

NcclApi* nccl_api() {
    static NcclApi api;
    static std::once_flag once;
    std::call_once(once, [] {
        void* h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
        if (h == nullptr) h = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
        if (h == nullptr) return;
        auto sym = [&](const char* n) { return dlsym(h, n); };
        api.GetUniqueId = reinterpret_cast<decltype(api.GetUniqueId)>(sym("ncclGetUniqueId"));
        api.CommInitRank = reinterpret_cast<decltype(api.CommInitRank)>(sym("ncclCommInitRank"));
        api.CommDestroy = reinterpret_cast<decltype(api.CommDestroy)>(sym("ncclCommDestroy"));
        api.GroupStart = reinterpret_cast<decltype(api.GroupStart)>(sym("ncclGroupStart"));
        api.GroupEnd = reinterpret_cast<decltype(api.GroupEnd)>(sym("ncclGroupEnd"));
        api.Send = reinterpret_cast<decltype(api.Send)>(sym("ncclSend"));
        api.Recv = reinterpret_cast<decltype(api.Recv)>(sym("ncclRecv"));
        api.GetErrorString = reinterpret_cast<decltype(api.GetErrorString)>(sym("ncclGetErrorString"));
        api.ok = api.GetUniqueId && api.CommInitRank && api.CommDestroy && api.GroupStart && api.GroupEnd && api.Send &&
                 api.Recv && api.GetErrorString;
    });
    return api.ok ? &api : nullptr;
}

edb200_status_t check_nccl(int r, const char* what) {
    if (r == 0) return EDB200_OK;
    NcclApi* a = nccl_api();
    return fail(EDB200_ERR_CUDA, "%s: NCCL error %d (%s)", what, r, a ? a->GetErrorString(r) : "?");
}

__global__ void interleave_heads_kernel(const uint4* __restrict__ staging, uint4* __restrict__ out, int world,
                                        long long t_loc, int chunk16, long long ld16) {
    // staging [world][t_loc][chunk16] -> out[t][p * chunk16 + c], 16-byte units
    const long long total = (long long)world * t_loc * chunk16;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        const int c = static_cast<int>(i % chunk16);
        const long long t = (i / chunk16) % t_loc;
        const int p = static_cast<int>(i / ((long long)chunk16 * t_loc));
        out[t * ld16 + (long long)p * chunk16 + c] = staging[i];
    }
}

// All-gather over peer memory: this rank's rows go straight into every rank's receive buffer.
struct GatherArgs {
    uint4* dst[8];
    int world;
};

__global__ void gather_rows_peer_kernel(const uint4* __restrict__ src, const GatherArgs a, long long n16) {
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n16; i += (long long)gridDim.x * blockDim.x) {
        const uint4 v = src[i];
        for (int p = 0; p < a.world; ++p) a.dst[p][i] = v;
    }
}

// Cross-GPU barrier of one kernel per rank.  The epoch lives in device memory (one word per
// communicator, next to the flags): lane 0 reads it, the kernel uses epoch + 1 and writes that
// back at the end, so a recorded launch (CUDA graph) advances it on every replay just like an
// eager one.  Thread p tells rank p "rank `rank` has reached epoch e" (a release store at
// system scope into p's flag word for this rank, after a system fence that orders the stream's
// earlier peer stores), then waits until rank p has told this rank the same.  The wait is
// bounded by wall clock (`limit_ns`); on expiry the error word is set and the kernel returns.
struct BarrierArgs {
    uint32_t* flags[8];   // flags[p] = rank p's flag array (8 words, 64 bytes apart)
    uint32_t* epoch;      // this rank's epoch word
    int rank, world;
    unsigned long long limit_ns;
    int* err;
};

__global__ void sp_barrier_kernel(const BarrierArgs a) {
    const int p = threadIdx.x;
    uint32_t e = 0;
    if (p == 0) e = *a.epoch + 1u;
    e = __shfl_sync(0xffffffffu, e, 0);
    if (p < a.world) {
        __threadfence_system();
        uint32_t* theirs = a.flags[p] + a.rank * 16;
        asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(theirs), "r"(e) : "memory");
        const uint32_t* mine = a.flags[a.rank] + p * 16;
        const unsigned long long t0 = globaltimer_ns();
        uint32_t v;
        for (;;) {
            asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(mine) : "memory");
            if (static_cast<int32_t>(v - e) >= 0) break;
            if (globaltimer_ns() - t0 > a.limit_ns) {
                atomicExch(a.err, 3);
                break;
            }
            __nanosleep(100);
        }
    }
    __syncwarp();
    if (p == 0) *a.epoch = e;
}

}  // namespace
}  // namespace edb

using namespace edb;

struct edb200_comm {
    nccl_comm_t comm = nullptr;
    int rank = 0, world = 1;
    // peer mappings of one device allocation per rank (same size and layout on every rank)
    char* base[8] = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr};
    bool mapped = false;
    int64_t flags_off = 0;   // 8 flag words of 64 bytes each, then the epoch word, inside the allocation
    int64_t timeout_ms = 2000;   // limit of the barrier's device-side wait
    bool loopback = false;       // no NCCL behind it: every "peer" is this rank's own allocation
};

// Bytes of the mapped allocation that the barrier owns (from flags_off).
static constexpr int64_t kBarrierBytes = 1024;
static constexpr int64_t kEpochOff = 8 * 64;

extern "C" {

edb200_status_t edb200_sp_shard(int64_t n_tokens, int64_t n_txt, int rank, int world, int64_t* t_loc,
                                int64_t* n_txt_local, int64_t* img_first, int64_t* t_rows) {
    if (world <= 0 || rank < 0 || rank >= world || n_tokens <= 0 || n_txt < 0 || n_txt > n_tokens) {
        return fail(EDB200_ERR_INVALID, "sp_shard: bad argument");
    }
    // The sequence is padded to a multiple of the world size (sp_sequence_padding, reference
    // src/core/parallel/sp_parallel.cpp:757-768): every rank's slot is t_loc = ceil(T / P) rows, and the
    // slots past the last real token stay empty (the last ranks own fewer rows, possibly none).
    const int64_t tl = (n_tokens + world - 1) / world;
    const int64_t first = (int64_t)rank * tl;
    int64_t rows = n_tokens - first;
    if (rows < 0) rows = 0;
    if (rows > tl) rows = tl;
    int64_t txt = n_txt - first;
    if (txt < 0) txt = 0;
    if (txt > rows) txt = rows;
    if (t_loc) *t_loc = tl;
    if (t_rows) *t_rows = rows;
    if (n_txt_local) *n_txt_local = txt;
    if (img_first) {
        int64_t f = (first > n_txt ? first : n_txt) - n_txt;
        if (f > n_tokens - n_txt) f = n_tokens - n_txt;
        *img_first = f;
    }
    return EDB200_OK;
}

int edb200_sp_heads_plan(int rank, int world, int heads, int64_t t_loc, int64_t row_bytes, int* peer,
                         int64_t* send_off, int64_t* recv_off, int64_t* bytes, int cap) {
    if (world <= 0 || rank < 0 || rank >= world || heads <= 0 || heads % world || t_loc <= 0 || row_bytes <= 0) return -1;
    const int hp = heads / world;
    const int n = world * hp;
    if (peer == nullptr) return n;
    if (cap < n) return -1;
    const int64_t T = t_loc * world;
    int i = 0;
    for (int p = 0; p < world; ++p) {
        for (int hl = 0; hl < hp; ++hl, ++i) {
            peer[i] = p;
            bytes[i] = t_loc * row_bytes;
            // to rank p: its head hl is this rank's head p*hp + hl, all local tokens
            send_off[i] = ((int64_t)(p * hp + hl) * t_loc) * row_bytes;
            // from rank p: tokens [p*t_loc, (p+1)*t_loc) of local head hl
            recv_off[i] = ((int64_t)hl * T + (int64_t)p * t_loc) * row_bytes;
        }
    }
    return n;
}

edb200_status_t edb200_comm_unique_id(void* id128) {
    if (id128 == nullptr) return fail(EDB200_ERR_INVALID, "comm_unique_id: null argument");
    NcclApi* a = nccl_api();
    if (a == nullptr) return fail(EDB200_ERR_UNSUPPORTED, "comm_unique_id: libnccl.so.2 not available");
    NcclId id;
    EDB_TRY(check_nccl(a->GetUniqueId(&id), "ncclGetUniqueId"));
    memcpy(id128, id.internal, 128);
    return EDB200_OK;
}

edb200_status_t edb200_comm_create(const void* id128, int rank, int world, edb200_comm_t** out) {
    if (id128 == nullptr || out == nullptr || world <= 0 || rank < 0 || rank >= world) {
        return fail(EDB200_ERR_INVALID, "comm_create: bad argument");
    }
    NcclApi* a = nccl_api();
    if (a == nullptr) return fail(EDB200_ERR_UNSUPPORTED, "comm_create: libnccl.so.2 not available");
    NcclId id;
    memcpy(id.internal, id128, 128);
    edb200_comm* c = new (std::nothrow) edb200_comm();
    if (c == nullptr) return fail(EDB200_ERR_NOMEM, "comm_create: host allocation failed");
    c->rank = rank;
    c->world = world;
    edb200_status_t st = check_nccl(a->CommInitRank(&c->comm, world, id, rank), "ncclCommInitRank");
    if (st != EDB200_OK) {
        delete c;
        return st;
    }
    *out = c;
    return EDB200_OK;
}

edb200_status_t edb200_comm_create_loopback(int rank, int world, edb200_comm_t** out) {
    if (out == nullptr || world <= 0 || world > 8 || rank < 0 || rank >= world) {
        return fail(EDB200_ERR_INVALID, "comm_create_loopback: bad argument");
    }
    edb200_comm* c = new (std::nothrow) edb200_comm();
    if (c == nullptr) return fail(EDB200_ERR_NOMEM, "comm_create_loopback: host allocation failed");
    c->rank = rank;
    c->world = world;
    c->loopback = true;
    *out = c;
    return EDB200_OK;
}

edb200_status_t edb200_comm_set_timeout_ms(edb200_comm_t* c, int64_t ms) {
    if (c == nullptr || ms <= 0 || ms > 60000) return fail(EDB200_ERR_INVALID, "comm_set_timeout_ms: 1..60000 ms");
    c->timeout_ms = ms;
    return EDB200_OK;
}

void edb200_comm_destroy(edb200_comm_t* c) {
    if (c == nullptr) return;
    edb200_comm_unmap_peers(c);
    NcclApi* a = nccl_api();
    if (a != nullptr && c->comm != nullptr) a->CommDestroy(c->comm);
    delete c;
}

// Host-side rendezvous over NCCL: every rank sends `bytes` to every rank.
static edb200_status_t nccl_all_gather_small(edb200_comm_t* c, const void* dev_send, void* dev_recv, size_t bytes,
                                             cudaStream_t s) {
    NcclApi* a = nccl_api();
    EDB_TRY(check_nccl(a->GroupStart(), "ncclGroupStart"));
    int rc = 0;
    for (int p = 0; p < c->world && rc == 0; ++p) {
        rc = a->Send(dev_send, bytes, kNcclUint8, p, c->comm, s);
        if (rc == 0) rc = a->Recv(static_cast<char*>(dev_recv) + (size_t)p * bytes, bytes, kNcclUint8, p, c->comm, s);
    }
    const int rc_end = a->GroupEnd();
    EDB_TRY(check_nccl(rc, "ncclSend/ncclRecv"));
    EDB_TRY(check_nccl(rc_end, "ncclGroupEnd"));
    return check_cuda(cudaStreamSynchronize(s), "comm rendezvous");
}

edb200_status_t edb200_comm_unmap_peers(edb200_comm_t* c) {
    if (c == nullptr) return fail(EDB200_ERR_INVALID, "comm_unmap_peers: null communicator");
    if (!c->mapped) return EDB200_OK;
    // nobody may still be writing into a mapping that is about to go away
    cudaDeviceSynchronize();
    if (!c->loopback) {
        char* dev = nullptr;
        if (cudaMalloc(reinterpret_cast<void**>(&dev), 16 * 9) == cudaSuccess) {
            nccl_all_gather_small(c, dev, dev + 16, 16, nullptr);
            cudaFree(dev);
        }
        for (int p = 0; p < c->world; ++p) {
            if (p != c->rank && c->base[p] != nullptr) cudaIpcCloseMemHandle(c->base[p]);
        }
    }
    for (int p = 0; p < c->world; ++p) c->base[p] = nullptr;
    c->mapped = false;
    return EDB200_OK;
}

// What every rank sends in the two rendezvous of the mapping: its handle with a flag that says
// whether it has one, then whether it could open everybody else's.
struct MapMsg {
    cudaIpcMemHandle_t handle;
    unsigned char ok;
    unsigned char pad[15];
};
static_assert(sizeof(cudaIpcMemHandle_t) == 64 && sizeof(MapMsg) == 80, "IPC handle size");

int edb200_comm_all_ok(const unsigned char* ok, int stride, int world) {
    if (ok == nullptr || world <= 0) return 0;
    for (int p = 0; p < world; ++p) {
        if (ok[(size_t)p * stride] != 1) return 0;
    }
    return 1;
}

edb200_status_t edb200_comm_map_peers(edb200_comm_t* c, void* base, int64_t bytes, int64_t flags_off, void* stream) {
    if (c == nullptr || base == nullptr || bytes <= 0 || flags_off < 0 || flags_off + kBarrierBytes > bytes ||
        flags_off % 64) {
        return fail(EDB200_ERR_INVALID, "comm_map_peers: bad argument");
    }
    if (c->world > 8) return fail(EDB200_ERR_UNSUPPORTED, "comm_map_peers: at most 8 ranks");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (c->loopback) {
        EDB_TRY(edb200_comm_unmap_peers(c));
        EDB_TRY(check_cuda(cudaMemsetAsync(static_cast<char*>(base) + flags_off, 0, kBarrierBytes, s), "flags memset"));
        EDB_TRY(check_cuda(cudaStreamSynchronize(s), "comm_map_peers"));
        for (int p = 0; p < c->world; ++p) c->base[p] = static_cast<char*>(base);
        c->mapped = true;
        c->flags_off = flags_off;
        return EDB200_OK;
    }
    if (nccl_api() == nullptr) return fail(EDB200_ERR_UNSUPPORTED, "comm_map_peers: libnccl.so.2 not available");
    EDB_TRY(edb200_comm_unmap_peers(c));
    // The call is collective: from here on every rank runs BOTH rendezvous whatever fails locally, and
    // carries its failure in the message, so that all ranks take the same decision together and
    // nobody is left waiting in a rendezvous that a peer has abandoned.
    MapMsg mine;
    memset(&mine, 0, sizeof(mine));
    char local_err[160] = "";
    cudaError_t e = cudaIpcGetMemHandle(&mine.handle, base);
    const char* inject = getenv("EDB200_TEST_FAIL_IPC_RANK");   // host-side fault injection for the tests
    if (e == cudaSuccess && inject != nullptr && atoi(inject) == c->rank) e = cudaErrorNotSupported;
    if (e != cudaSuccess) {
        cudaGetLastError();
        snprintf(local_err, sizeof(local_err), "cudaIpcGetMemHandle: %s", cudaGetErrorString(e));
        memset(&mine.handle, 0, sizeof(mine.handle));
    } else {
        mine.ok = 1;
    }
    char* dev = nullptr;
    e = cudaMalloc(reinterpret_cast<void**>(&dev), sizeof(MapMsg) * 9);
    if (e != cudaSuccess) {
        // without device scratch this rank cannot even say so: this is the one failure the peers only
        // see as a time-out of NCCL itself
        return check_cuda(e, "comm_map_peers scratch");
    }
    MapMsg all[8];
    memset(all, 0, sizeof(all));
    cudaMemcpyAsync(dev, &mine, sizeof(MapMsg), cudaMemcpyHostToDevice, s);
    cudaMemsetAsync(static_cast<char*>(base) + flags_off, 0, kBarrierBytes, s);
    edb200_status_t st = nccl_all_gather_small(c, dev, dev + sizeof(MapMsg), sizeof(MapMsg), s);
    if (st == EDB200_OK) {
        st = check_cuda(cudaMemcpy(all, dev + sizeof(MapMsg), (size_t)c->world * sizeof(MapMsg), cudaMemcpyDeviceToHost),
                        "handles");
    }
    if (st != EDB200_OK) {   // the transport itself failed: no second rendezvous is possible either
        cudaFree(dev);
        return st;
    }
    bool have_all = edb200_comm_all_ok(&all[0].ok, (int)sizeof(MapMsg), c->world) == 1;
    bool opened_all = have_all;
    if (have_all) {
        for (int p = 0; p < c->world; ++p) {
            if (p == c->rank) {
                c->base[p] = static_cast<char*>(base);
                continue;
            }
            void* ptr = nullptr;
            e = cudaIpcOpenMemHandle(&ptr, all[p].handle, cudaIpcMemLazyEnablePeerAccess);
            if (e != cudaSuccess) {
                cudaGetLastError();
                snprintf(local_err, sizeof(local_err), "cudaIpcOpenMemHandle(rank %d): %s", p, cudaGetErrorString(e));
                opened_all = false;
                break;
            }
            c->base[p] = static_cast<char*>(ptr);
        }
    }
    // second rendezvous: did everybody open everything?  It also orders every rank's flag memset
    // before anybody's first signal.
    MapMsg second;
    memset(&second, 0, sizeof(second));
    second.ok = opened_all ? 1 : 0;
    cudaMemcpyAsync(dev, &second, sizeof(MapMsg), cudaMemcpyHostToDevice, s);
    st = nccl_all_gather_small(c, dev, dev + sizeof(MapMsg), sizeof(MapMsg), s);
    if (st == EDB200_OK) {
        st = check_cuda(cudaMemcpy(all, dev + sizeof(MapMsg), (size_t)c->world * sizeof(MapMsg), cudaMemcpyDeviceToHost),
                        "map result");
    }
    cudaFree(dev);
    const bool everybody = st == EDB200_OK && edb200_comm_all_ok(&all[0].ok, (int)sizeof(MapMsg), c->world) == 1;
    if (!everybody) {
        for (int p = 0; p < c->world; ++p) {
            if (p != c->rank && c->base[p] != nullptr) cudaIpcCloseMemHandle(c->base[p]);
            c->base[p] = nullptr;
        }
        if (st != EDB200_OK) return st;
        return fail(EDB200_ERR_UNSUPPORTED, "comm_map_peers: peer mappings unavailable (%s)",
                    local_err[0] ? local_err : "another rank could not map");
    }
    c->mapped = true;
    c->flags_off = flags_off;
    return EDB200_OK;
}

int edb200_comm_peers_mapped(const edb200_comm_t* c) { return c != nullptr && c->mapped ? 1 : 0; }

void* edb200_comm_peer_ptr(const edb200_comm_t* c, int peer, const void* local_ptr) {
    if (c == nullptr || !c->mapped || peer < 0 || peer >= c->world || local_ptr == nullptr) return nullptr;
    return c->base[peer] + (static_cast<const char*>(local_ptr) - c->base[c->rank]);
}

edb200_status_t edb200_sp_barrier(edb200_comm_t* c, void* stream) {
    if (c == nullptr || !c->mapped) return fail(EDB200_ERR_INVALID, "sp_barrier: peers are not mapped");
    int* err = device_error_word();
    if (err == nullptr) return fail(EDB200_ERR_CUDA, "sp_barrier: no CUDA device");
    BarrierArgs a;
    memset(&a, 0, sizeof(a));
    for (int p = 0; p < c->world; ++p) a.flags[p] = reinterpret_cast<uint32_t*>(c->base[p] + c->flags_off);
    a.epoch = reinterpret_cast<uint32_t*>(c->base[c->rank] + c->flags_off + kEpochOff);
    a.rank = c->rank;
    a.world = c->world;
    a.limit_ns = static_cast<unsigned long long>(c->timeout_ms) * 1000000ull;
    a.err = err;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    ProfScope prof(s, PROF_OTHER, 0.0, 0.0);
    sp_barrier_kernel<<<1, 32, 0, s>>>(a);
    count_launch();
    return check_cuda(cudaGetLastError(), "sp_barrier launch");
}

edb200_status_t edb200_poll_status(void* stream) { return poll_device_error(static_cast<cudaStream_t>(stream)); }

int edb200_comm_rank(const edb200_comm_t* c) { return c ? c->rank : 0; }
int edb200_comm_world(const edb200_comm_t* c) { return c ? c->world : 1; }

edb200_status_t edb200_sp_all_to_all_heads(edb200_comm_t* c, const void* const* send, void* const* recv, int n_tensors,
                                           int heads, int64_t t_loc, int64_t row_bytes, void* stream) {
    if (c == nullptr || send == nullptr || recv == nullptr || n_tensors <= 0) {
        return fail(EDB200_ERR_INVALID, "sp_all_to_all_heads: null argument");
    }
    NcclApi* a = nccl_api();
    if (a == nullptr) return fail(EDB200_ERR_UNSUPPORTED, "sp_all_to_all_heads: libnccl.so.2 not available");
    if (c->comm == nullptr) return fail(EDB200_ERR_UNSUPPORTED, "sp_all_to_all_heads: a loopback communicator has no transport");
    const int n = edb200_sp_heads_plan(c->rank, c->world, heads, t_loc, row_bytes, nullptr, nullptr, nullptr, nullptr, 0);
    if (n < 0) return fail(EDB200_ERR_INVALID, "sp_all_to_all_heads: heads must divide over the ranks");
    std::vector<int> peer(n);
    std::vector<int64_t> so(n), ro(n), nb(n);
    edb200_sp_heads_plan(c->rank, c->world, heads, t_loc, row_bytes, peer.data(), so.data(), ro.data(), nb.data(), n);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    EDB_TRY(check_nccl(a->GroupStart(), "ncclGroupStart"));
    int rc = 0;
    for (int t = 0; t < n_tensors && rc == 0; ++t) {
        const char* sb = static_cast<const char*>(send[t]);
        char* rb = static_cast<char*>(recv[t]);
        for (int i = 0; i < n && rc == 0; ++i) {
            rc = a->Send(sb + so[i], (size_t)nb[i], kNcclUint8, peer[i], c->comm, s);
            if (rc == 0) rc = a->Recv(rb + ro[i], (size_t)nb[i], kNcclUint8, peer[i], c->comm, s);
        }
    }
    const int rc_end = a->GroupEnd();
    EDB_TRY(check_nccl(rc, "ncclSend/ncclRecv"));
    return check_nccl(rc_end, "ncclGroupEnd");
}

edb200_status_t edb200_sp_all_to_all_tokens(edb200_comm_t* c, const void* send, void* staging, void* out, int64_t t_loc,
                                            int64_t chunk_bytes, int64_t ld_out_bytes, void* stream) {
    if (c == nullptr || send == nullptr || staging == nullptr || out == nullptr || t_loc <= 0 || chunk_bytes <= 0) {
        return fail(EDB200_ERR_INVALID, "sp_all_to_all_tokens: bad argument");
    }
    if (chunk_bytes % 16 || ld_out_bytes % 16 || ld_out_bytes < chunk_bytes * c->world ||
        (reinterpret_cast<uintptr_t>(staging) & 15u) || (reinterpret_cast<uintptr_t>(out) & 15u)) {
        return fail(EDB200_ERR_INVALID, "sp_all_to_all_tokens: rows must be multiples of 16 bytes and 16-byte aligned");
    }
    NcclApi* a = nccl_api();
    if (a == nullptr) return fail(EDB200_ERR_UNSUPPORTED, "sp_all_to_all_tokens: libnccl.so.2 not available");
    if (c->comm == nullptr) return fail(EDB200_ERR_UNSUPPORTED, "sp_all_to_all_tokens: a loopback communicator has no transport");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const size_t piece = (size_t)(t_loc * chunk_bytes);
    EDB_TRY(check_nccl(a->GroupStart(), "ncclGroupStart"));
    int rc = 0;
    for (int p = 0; p < c->world && rc == 0; ++p) {
        rc = a->Send(static_cast<const char*>(send) + (size_t)p * piece, piece, kNcclUint8, p, c->comm, s);
        if (rc == 0) rc = a->Recv(static_cast<char*>(staging) + (size_t)p * piece, piece, kNcclUint8, p, c->comm, s);
    }
    const int rc_end = a->GroupEnd();
    EDB_TRY(check_nccl(rc, "ncclSend/ncclRecv"));
    EDB_TRY(check_nccl(rc_end, "ncclGroupEnd"));
    const long long total16 = (long long)c->world * t_loc * (chunk_bytes / 16);
    const int threads = 256;
    long long blocks = (total16 + threads - 1) / threads;
    if (blocks > 148 * 16) blocks = 148 * 16;
    ProfScope prof(s, PROF_ELEMENTWISE, 0.0, 2.0 * (double)total16 * 16.0);
    interleave_heads_kernel<<<static_cast<unsigned>(blocks), threads, 0, s>>>(
        static_cast<const uint4*>(staging), static_cast<uint4*>(out), c->world, t_loc, static_cast<int>(chunk_bytes / 16),
        ld_out_bytes / 16);
    count_launch();
    return check_cuda(cudaGetLastError(), "sp interleave launch");
}

edb200_status_t edb200_sp_all_gather_rows(edb200_comm_t* c, const void* send, void* recv, const int64_t* row_first,
                                          const int64_t* row_count, int64_t row_bytes, void* stream) {
    if (c == nullptr || recv == nullptr || row_first == nullptr || row_count == nullptr || row_bytes <= 0) {
        return fail(EDB200_ERR_INVALID, "sp_all_gather_rows: bad argument");
    }
    NcclApi* a = nccl_api();
    if (a == nullptr) return fail(EDB200_ERR_UNSUPPORTED, "sp_all_gather_rows: libnccl.so.2 not available");
    if (c->comm == nullptr) return fail(EDB200_ERR_UNSUPPORTED, "sp_all_gather_rows: a loopback communicator has no transport");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const size_t mine = (size_t)(row_count[c->rank] * row_bytes);
    EDB_TRY(check_nccl(a->GroupStart(), "ncclGroupStart"));
    int rc = 0;
    for (int p = 0; p < c->world && rc == 0; ++p) {
        if (mine > 0) rc = a->Send(send, mine, kNcclUint8, p, c->comm, s);
        const size_t theirs = (size_t)(row_count[p] * row_bytes);
        if (rc == 0 && theirs > 0) {
            rc = a->Recv(static_cast<char*>(recv) + (size_t)(row_first[p] * row_bytes), theirs, kNcclUint8, p, c->comm, s);
        }
    }
    const int rc_end = a->GroupEnd();
    EDB_TRY(check_nccl(rc, "ncclSend/ncclRecv"));
    return check_nccl(rc_end, "ncclGroupEnd");
}

edb200_status_t edb200_sp_all_gather_rows_peer(edb200_comm_t* c, const void* send, void* recv, const int64_t* row_first,
                                               const int64_t* row_count, int64_t row_bytes, void* stream) {
    if (c == nullptr || recv == nullptr || row_first == nullptr || row_count == nullptr || row_bytes <= 0) {
        return fail(EDB200_ERR_INVALID, "sp_all_gather_rows_peer: bad argument");
    }
    if (!c->mapped) return fail(EDB200_ERR_INVALID, "sp_all_gather_rows_peer: peers are not mapped");
    if (row_bytes % 16 || (reinterpret_cast<uintptr_t>(recv) & 15u) || (reinterpret_cast<uintptr_t>(send) & 15u)) {
        return fail(EDB200_ERR_INVALID, "sp_all_gather_rows_peer: rows must be multiples of 16 bytes and 16-byte aligned");
    }
    const char* lo = c->base[c->rank];
    if (static_cast<const char*>(recv) < lo) return fail(EDB200_ERR_INVALID, "sp_all_gather_rows_peer: recv is outside the mapped allocation");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const long long n16 = (long long)(row_count[c->rank] * row_bytes / 16);
    if (n16 > 0) {
        if (send == nullptr) return fail(EDB200_ERR_INVALID, "sp_all_gather_rows_peer: null send buffer");
        GatherArgs a;
        memset(&a, 0, sizeof(a));
        a.world = c->world;
        for (int p = 0; p < c->world; ++p) {
            char* base = static_cast<char*>(edb200_comm_peer_ptr(c, p, recv));
            a.dst[p] = reinterpret_cast<uint4*>(base + row_first[c->rank] * row_bytes);
        }
        long long blocks = (n16 + 255) / 256;
        if (blocks > 148 * 8) blocks = 148 * 8;
        ProfScope prof(s, PROF_ELEMENTWISE, 0.0, (double)n16 * 16.0 * (1 + c->world));
        gather_rows_peer_kernel<<<static_cast<unsigned>(blocks), 256, 0, s>>>(static_cast<const uint4*>(send), a, n16);
        count_launch();
        EDB_TRY(check_cuda(cudaGetLastError(), "sp gather launch"));
    }
    // every rank's rows have landed everywhere once all ranks have passed this point
    return edb200_sp_barrier(c, stream);
}

edb200_status_t edb200_cfg_parallel_combine(edb200_comm_t* c, const float* mine, float scale, float* gathered, float* out,
                                            int64_t n, void* stream) {
    if (c == nullptr || mine == nullptr || gathered == nullptr || out == nullptr || n <= 0 || n % 4) {
        return fail(EDB200_ERR_INVALID, "cfg_parallel_combine: bad argument (n %% 4 == 0 required)");
    }
    if (c->world != 2) return fail(EDB200_ERR_UNSUPPORTED, "cfg_parallel_combine: the communicator must have 2 ranks");
    const int64_t first[2] = {0, 1}, count[2] = {1, 1};
    EDB_TRY(edb200_sp_all_gather_rows(c, mine, gathered, first, count, n * 4, stream));
    // rank 0 ran the conditional branch, rank 1 the unconditional one
    return edb200_cfg_combine(gathered + n, gathered, scale, out, n, stream);
}

edb200_status_t edb200_cfg_parallel_combine_rescaled(edb200_comm_t* c, const float* mine, float scale, int patch_size,
                                                     int channels, int height, int width, float* gathered, float* out,
                                                     void* stream) {
    const int64_t n = (int64_t)channels * height * width;
    if (c == nullptr || mine == nullptr || gathered == nullptr || out == nullptr || n <= 0) {
        return fail(EDB200_ERR_INVALID, "cfg_parallel_combine_rescaled: bad argument");
    }
    if (c->world != 2) {
        return fail(EDB200_ERR_UNSUPPORTED, "cfg_parallel_combine_rescaled: the communicator must have 2 ranks");
    }
    const int64_t first[2] = {0, 1}, count[2] = {1, 1};
    EDB_TRY(edb200_sp_all_gather_rows(c, mine, gathered, first, count, n * 4, stream));
    return edb200_cfg_combine_rescaled(gathered + n, gathered, scale, patch_size, channels, height, width, out, stream);
}

}  // extern "C"
