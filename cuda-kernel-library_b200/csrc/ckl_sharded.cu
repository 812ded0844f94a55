// Multi-GPU layer of the C ABI (include/ckl_gemm.h, "one process or thread per GPU").
//
// The reference library is single-GPU: it never calls cudaSetDevice and its test driver
// uploads, launches and downloads on one device (tests/test_gemm_tensor.cpp:69-85).  This
// file is the N-sharded form of that sequence for the GPUs of one box.  Output columns are
// independent, so rank r owns a column block of B and C; the rows of A are dealt to the ranks
// for the trip over the host link and replicated over NVLink afterwards.
//
//   ckl_comm                 the ranks of one job: an NCCL communicator (loaded with dlopen,
//                            so the library still links only the CUDA runtime), the streams
//                            and events of the pipelines below, device staging, and the peer
//                            mappings of buffers made with ckl_comm_alloc_shared.
//   ckl_gemm_host_sharded    host buffers in, host buffers out.  Each rank uploads ITS rows of
//                            A and its column blocks of B and C over its own host link, the
//                            ranks all-gather the A row panels (NCCL, every buffer in the
//                            rank's own memory), and panel j is multiplied and sent back while
//                            panel j+1 is still arriving.
//   ckl_gemm_gathered        device buffers; every rank ends with the whole row-major C.  The
//                            local GEMM runs in row panels; behind each panel a copy kernel of
//                            this library writes the panel's column block straight into every
//                            rank's C with plain 16-byte stores to peer memory (no staging
//                            buffer, no interleave pass, no TMA and no multicast on any peer
//                            address), so the NVLink transfer of panel i overlaps the
//                            multiplication of panel i+1.
//
// Nothing here waits inside a kernel for another GPU: ranks meet only in NCCL calls, which
// are ordered on one stream per rank.

#include <dlfcn.h>
#include <unistd.h>

#include <algorithm>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <mutex>
#include <string>
#include <vector>

#include <cuda_runtime.h>

#include "ckl_gemm.h"
#include "ckl_internal.h"

namespace {

using ckl::set_error;

#define SH_TRY_CUDA(expr)                                                                        \
    do {                                                                                         \
        const cudaError_t err__ = (expr);                                                        \
        if (err__ != cudaSuccess) {                                                              \
            return set_error(CKL_ERR_CUDA, "%s failed: %s (%s)", #expr, cudaGetErrorName(err__), \
                             cudaGetErrorString(err__));                                         \
        }                                                                                        \
    } while (0)

// ---- NCCL, bound at run time -------------------------------------------------------------
// Only the handful of entry points used here, with the public signatures of nccl.h
// (result codes: 0 = success; data type 1 = uint8, 2 = int32; reduction 0 = sum).

struct NcclUniqueId {
    char internal[CKL_COMM_ID_BYTES];
};
using NcclComm = void*;
constexpr int kNcclUint8 = 1;
constexpr int kNcclInt32 = 2;
constexpr int kNcclSum = 0;

struct NcclApi {
    void* lib = nullptr;
    int (*GetUniqueId)(NcclUniqueId*) = nullptr;
    int (*CommInitRank)(NcclComm*, int, NcclUniqueId, int) = nullptr;
    int (*CommDestroy)(NcclComm) = nullptr;
    int (*CommAbort)(NcclComm) = nullptr;
    int (*AllGather)(const void*, void*, size_t, int, NcclComm, cudaStream_t) = nullptr;
    int (*AllReduce)(const void*, void*, size_t, int, int, NcclComm, cudaStream_t) = nullptr;
    const char* (*GetErrorString)(int) = nullptr;
    std::string error;
};

NcclApi* load_nccl() {
    static NcclApi api;
    static std::once_flag once;
    std::call_once(once, [] {
        // A process that already carries an NCCL (a framework's bundled copy) gets that one:
        // dlopen by soname returns the mapped library.
        const char* names[] = {std::getenv("CKL_NCCL_LIB"), "libnccl.so.2", "libnccl.so"};
        for (const char* name : names) {
            if (name != nullptr && name[0] != '\0') {
                api.lib = dlopen(name, RTLD_NOW | RTLD_GLOBAL);
                if (api.lib != nullptr) {
                    break;
                }
            }
        }
        if (api.lib == nullptr) {
            api.error = "libnccl.so.2 could not be loaded (set CKL_NCCL_LIB to its path)";
            return;
        }
        auto sym = [&](const char* name) {
            void* p = dlsym(api.lib, name);
            if (p == nullptr && api.error.empty()) {
                api.error = std::string("NCCL symbol missing: ") + name;
            }
            return p;
        };
        api.GetUniqueId = reinterpret_cast<decltype(api.GetUniqueId)>(sym("ncclGetUniqueId"));
        api.CommInitRank = reinterpret_cast<decltype(api.CommInitRank)>(sym("ncclCommInitRank"));
        api.CommDestroy = reinterpret_cast<decltype(api.CommDestroy)>(sym("ncclCommDestroy"));
        api.CommAbort = reinterpret_cast<decltype(api.CommAbort)>(sym("ncclCommAbort"));
        api.AllGather = reinterpret_cast<decltype(api.AllGather)>(sym("ncclAllGather"));
        api.AllReduce = reinterpret_cast<decltype(api.AllReduce)>(sym("ncclAllReduce"));
        api.GetErrorString = reinterpret_cast<decltype(api.GetErrorString)>(sym("ncclGetErrorString"));
    });
    return &api;
}

int nccl_fail(const NcclApi* api, int result, const char* what) {
    return set_error(CKL_ERR_CUDA, "%s failed: NCCL result %d (%s)", what, result,
                     api->GetErrorString != nullptr ? api->GetErrorString(result) : "?");
}

#define SH_TRY_NCCL(api, expr)                       \
    do {                                             \
        const int res__ = (expr);                    \
        if (res__ != 0) {                            \
            return nccl_fail((api), res__, #expr);   \
        }                                            \
    } while (0)

size_t dtype_bytes(int dtype) { return dtype == CKL_F32 ? 4 : 2; }

struct Buffer {
    void* ptr = nullptr;
    size_t bytes = 0;
};

int ensure(Buffer* b, size_t bytes) {
    if (b->bytes >= bytes) {
        return CKL_OK;
    }
    if (b->ptr != nullptr) {
        SH_TRY_CUDA(cudaFree(b->ptr));
        b->ptr = nullptr;
        b->bytes = 0;
    }
    SH_TRY_CUDA(cudaMalloc(&b->ptr, bytes));
    // padding rows of a ragged problem are multiplied like any other row: keep them finite
    SH_TRY_CUDA(cudaMemset(b->ptr, 0, bytes));
    b->bytes = bytes;
    return CKL_OK;
}

constexpr int kMaxPanels = 8;
constexpr int kMaxWorld = 64;

struct SharedAlloc {
    size_t bytes = 0;
    std::vector<void*> peers;     // address of every rank's copy in THIS process (own = local)
    std::vector<bool> opened;     // mapped with cudaIpcOpenMemHandle (to be closed)
};

// What one rank publishes about a shared buffer.
struct ShareRecord {
    cudaIpcMemHandle_t handle;
    unsigned long long address;   // usable directly by ranks of the same process
    long long pid;
    int device;
    int pad;
};

}  // namespace

struct ckl_comm {
    int world = 1;
    int rank = 0;
    int device = 0;
    NcclComm nccl = nullptr;
    cudaStream_t s_in = nullptr, s_run = nullptr, s_out = nullptr, s_coll = nullptr;
    cudaEvent_t ev_b = nullptr, ev_entry = nullptr, ev_exit = nullptr;
    cudaEvent_t ev_a[kMaxPanels] = {}, ev_g[kMaxPanels] = {}, ev_c[kMaxPanels] = {},
                ev_done[kMaxPanels] = {};
    Buffer dev_a, dev_b, dev_c, exchange;
    int* barrier_word = nullptr;
    std::map<void*, SharedAlloc> shared;
    std::mutex mu;
};

namespace {

// Stream-ordered meeting point of all ranks on s_coll: a one-word all-reduce.
int rank_barrier(ckl_comm* comm) {
    if (comm->world == 1) {
        return CKL_OK;
    }
    NcclApi* api = load_nccl();
    SH_TRY_NCCL(api, api->AllReduce(comm->barrier_word, comm->barrier_word, 1, kNcclInt32, kNcclSum,
                                    comm->nccl, comm->s_coll));
    return CKL_OK;
}

// Copies `rows` rows of `row_bytes` bytes from a packed block (pitch row_bytes) to column
// offset `col_bytes` of row-major matrices of pitch `dst_pitch`, one per destination.
struct ScatterDsts {
    void* ptr[kMaxWorld];
};

template <typename T>
__global__ void __launch_bounds__(256)
scatter_column_block_kernel(ScatterDsts dsts, int parts, const T* __restrict__ src, size_t per_row,
                            size_t dst_pitch_units, size_t col_units, int rows) {
    const size_t total = per_row * static_cast<size_t>(rows);
    const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
    for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
        const size_t r = i / per_row;
        const size_t c = i - r * per_row;
        const T v = src[i];
        const size_t off = r * dst_pitch_units + col_units + c;
        for (int d = 0; d < parts; ++d) {
            static_cast<T*>(dsts.ptr[d])[off] = v;
        }
    }
}

int launch_scatter(const ScatterDsts& dsts, int parts, const void* src, int elem_size, int rows,
                   int width, int n, int col0, size_t row0, cudaStream_t stream) {
    if (rows <= 0 || width <= 0) {
        return CKL_OK;
    }
    const size_t es = static_cast<size_t>(elem_size);
    const size_t row_bytes = static_cast<size_t>(width) * es;
    const size_t pitch = static_cast<size_t>(n) * es;
    const size_t col_bytes = static_cast<size_t>(col0) * es;
    ScatterDsts moved = dsts;
    bool vec = row_bytes % 16 == 0 && pitch % 16 == 0 && col_bytes % 16 == 0 &&
               reinterpret_cast<uintptr_t>(src) % 16 == 0;
    for (int d = 0; d < parts; ++d) {
        moved.ptr[d] = static_cast<unsigned char*>(dsts.ptr[d]) + row0 * pitch;
        vec = vec && reinterpret_cast<uintptr_t>(moved.ptr[d]) % 16 == 0;
    }
    const size_t unit = vec ? 16 : es;
    const size_t per_row = row_bytes / unit;
    const size_t total = per_row * static_cast<size_t>(rows);
    // two resident blocks per SM beside the GEMM's one: enough stores in flight for NVLink
    const int blocks = static_cast<int>(std::min<size_t>((total + 255) / 256, 148 * 2));
    if (vec) {
        scatter_column_block_kernel<uint4><<<blocks, 256, 0, stream>>>(
            moved, parts, static_cast<const uint4*>(src), per_row, pitch / 16, col_bytes / 16, rows);
    } else if (elem_size == 4) {
        scatter_column_block_kernel<uint32_t><<<blocks, 256, 0, stream>>>(
            moved, parts, static_cast<const uint32_t*>(src), per_row, pitch / 4, col_bytes / 4, rows);
    } else {
        scatter_column_block_kernel<uint16_t><<<blocks, 256, 0, stream>>>(
            moved, parts, static_cast<const uint16_t*>(src), per_row, pitch / 2, col_bytes / 2, rows);
    }
    SH_TRY_CUDA(cudaGetLastError());
    return CKL_OK;
}

int check_comm(const ckl_comm* comm, const char* who) {
    if (comm == nullptr) {
        return set_error(CKL_ERR_INVALID_ARG, "%s: comm is null", who);
    }
    int dev = -1;
    SH_TRY_CUDA(cudaGetDevice(&dev));
    if (dev != comm->device) {
        return set_error(CKL_ERR_INVALID_ARG,
                         "%s: the communicator belongs to device %d but device %d is current", who,
                         comm->device, dev);
    }
    return CKL_OK;
}

int sync_all(ckl_comm* comm, int rc) {
    // Nothing of a call may still be in flight when it returns, whatever happened before.
    const cudaError_t e0 = cudaStreamSynchronize(comm->s_in);
    const cudaError_t e1 = cudaStreamSynchronize(comm->s_coll);
    const cudaError_t e2 = cudaStreamSynchronize(comm->s_run);
    const cudaError_t e3 = cudaStreamSynchronize(comm->s_out);
    if (rc != CKL_OK) {
        return rc;
    }
    SH_TRY_CUDA(e0);
    SH_TRY_CUDA(e1);
    SH_TRY_CUDA(e2);
    SH_TRY_CUDA(e3);
    return CKL_OK;
}

}  // namespace

extern "C" {

int ckl_column_shard(int n, int world, int rank, int align, int* col0, int* width) {
    if (world <= 0 || rank < 0 || rank >= world || n < 0 || align <= 0 || col0 == nullptr ||
        width == nullptr) {
        return set_error(CKL_ERR_INVALID_ARG, "ckl_column_shard: bad request n=%d world=%d rank=%d align=%d",
                         n, world, rank, align);
    }
    const long long per = (static_cast<long long>(n) + world - 1) / world;
    const long long block = (per + align - 1) / align * align;
    const long long first = std::min<long long>(static_cast<long long>(rank) * block, n);
    *col0 = static_cast<int>(first);
    *width = static_cast<int>(std::min<long long>(block, n - first));
    return CKL_OK;
}

int ckl_plan_host_sharded(int m, int world, int rank, ckl_host_shard_plan* out) {
    if (out == nullptr || world <= 0 || world > kMaxWorld || rank < 0 || rank >= world || m < 0) {
        return set_error(CKL_ERR_INVALID_ARG, "ckl_plan_host_sharded: bad request m=%d world=%d rank=%d",
                         m, world, rank);
    }
    std::memset(out, 0, sizeof *out);
    const int rpr = (m + world - 1) / world;
    out->rows_per_rank = rpr;
    out->row0 = static_cast<int>(std::min<long long>(static_cast<long long>(rank) * rpr, m));
    out->rows = std::min(rpr, m - out->row0);
    // Panels of at least 128 rows per rank, at most eight: each panel is one all-gather and
    // one GEMM over world * panel_rows rows; finer panels let the downloads start earlier and
    // shorten the tail of the pipeline, at the price of launches and smaller GEMMs (8 GPUs,
    // 8192^3, ms per call with 1 / 2 / 4 / 8 panels: 3.93 / 3.58 / 3.49 / 3.29).
    int panels = std::max(1, std::min(kMaxPanels, rpr / 128));
    if (const char* forced = std::getenv("CKL_HOST_PANELS")) {  // tuning knob: 1..8, the same on every rank
        panels = std::max(1, std::min(kMaxPanels, std::atoi(forced)));
    }
    int panel_rows = (rpr + panels - 1) / panels;
    panel_rows = (panel_rows + 7) / 8 * 8;
    panels = rpr > 0 ? (rpr + panel_rows - 1) / panel_rows : 0;
    out->panels = panels;
    out->panel_rows = panel_rows;
    out->padded_rows = panels * world * panel_rows;
    return CKL_OK;
}

int ckl_comm_get_unique_id(void* id) {
    if (id == nullptr) {
        return set_error(CKL_ERR_INVALID_ARG, "ckl_comm_get_unique_id: id is null");
    }
    NcclApi* api = load_nccl();
    if (!api->error.empty()) {
        return set_error(CKL_ERR_UNSUPPORTED, "%s", api->error.c_str());
    }
    NcclUniqueId uid;
    SH_TRY_NCCL(api, api->GetUniqueId(&uid));
    std::memcpy(id, uid.internal, CKL_COMM_ID_BYTES);
    return CKL_OK;
}

int ckl_comm_init(ckl_comm** out, int world, int rank, const void* id) {
    if (out == nullptr || world <= 0 || world > kMaxWorld || rank < 0 || rank >= world ||
        (world > 1 && id == nullptr)) {
        return set_error(CKL_ERR_INVALID_ARG, "ckl_comm_init: bad arguments (world=%d rank=%d)", world, rank);
    }
    *out = nullptr;
    int dev = 0;
    SH_TRY_CUDA(cudaGetDevice(&dev));
    ckl_comm* comm = new ckl_comm;
    comm->world = world;
    comm->rank = rank;
    comm->device = dev;
    auto fail_with = [&](int rc) {
        ckl_comm_destroy(comm);
        return rc;
    };
    auto cuda = [&](cudaError_t e, const char* what) {
        return e == cudaSuccess ? CKL_OK
                                : set_error(CKL_ERR_CUDA, "ckl_comm_init: %s failed: %s", what,
                                            cudaGetErrorString(e));
    };
    int rc = CKL_OK;
    cudaStream_t* streams[] = {&comm->s_in, &comm->s_run, &comm->s_out, &comm->s_coll};
    for (cudaStream_t* s : streams) {
        if ((rc = cuda(cudaStreamCreateWithFlags(s, cudaStreamNonBlocking), "stream creation")) != CKL_OK) {
            return fail_with(rc);
        }
    }
    std::vector<cudaEvent_t*> events = {&comm->ev_b, &comm->ev_entry, &comm->ev_exit};
    for (int j = 0; j < kMaxPanels; ++j) {
        events.push_back(&comm->ev_a[j]);
        events.push_back(&comm->ev_g[j]);
        events.push_back(&comm->ev_c[j]);
        events.push_back(&comm->ev_done[j]);
    }
    for (cudaEvent_t* e : events) {
        if ((rc = cuda(cudaEventCreateWithFlags(e, cudaEventDisableTiming), "event creation")) != CKL_OK) {
            return fail_with(rc);
        }
    }
    if ((rc = cuda(cudaMalloc(&comm->barrier_word, sizeof(int)), "cudaMalloc")) != CKL_OK ||
        (rc = cuda(cudaMemset(comm->barrier_word, 0, sizeof(int)), "cudaMemset")) != CKL_OK) {
        return fail_with(rc);
    }
    if (world > 1) {
        NcclApi* api = load_nccl();
        if (!api->error.empty()) {
            return fail_with(set_error(CKL_ERR_UNSUPPORTED, "%s", api->error.c_str()));
        }
        NcclUniqueId uid;
        std::memcpy(uid.internal, id, CKL_COMM_ID_BYTES);
        const int res = api->CommInitRank(&comm->nccl, world, uid, rank);
        if (res != 0) {
            comm->nccl = nullptr;
            return fail_with(nccl_fail(api, res, "ncclCommInitRank"));
        }
    }
    *out = comm;
    return CKL_OK;
}

int ckl_comm_world(const ckl_comm* comm) { return comm != nullptr ? comm->world : 0; }
int ckl_comm_rank(const ckl_comm* comm) { return comm != nullptr ? comm->rank : -1; }

int ckl_comm_destroy(ckl_comm* comm) {
    if (comm == nullptr) {
        return CKL_OK;
    }
    int prev = 0;
    const bool have_prev = cudaGetDevice(&prev) == cudaSuccess;
    cudaSetDevice(comm->device);
    cudaDeviceSynchronize();
    for (auto& kv : comm->shared) {
        for (size_t r = 0; r < kv.second.peers.size(); ++r) {
            if (kv.second.opened[r]) {
                cudaIpcCloseMemHandle(kv.second.peers[r]);
            }
        }
        cudaFree(kv.first);
    }
    comm->shared.clear();
    if (comm->nccl != nullptr) {
        load_nccl()->CommDestroy(comm->nccl);
    }
    cudaFree(comm->dev_a.ptr);
    cudaFree(comm->dev_b.ptr);
    cudaFree(comm->dev_c.ptr);
    cudaFree(comm->exchange.ptr);
    cudaFree(comm->barrier_word);
    cudaStream_t streams[] = {comm->s_in, comm->s_run, comm->s_out, comm->s_coll};
    for (cudaStream_t s : streams) {
        if (s != nullptr) {
            cudaStreamDestroy(s);
        }
    }
    cudaEvent_t singles[] = {comm->ev_b, comm->ev_entry, comm->ev_exit};
    for (cudaEvent_t e : singles) {
        if (e != nullptr) {
            cudaEventDestroy(e);
        }
    }
    for (int j = 0; j < kMaxPanels; ++j) {
        cudaEvent_t per_panel[] = {comm->ev_a[j], comm->ev_g[j], comm->ev_c[j], comm->ev_done[j]};
        for (cudaEvent_t e : per_panel) {
            if (e != nullptr) {
                cudaEventDestroy(e);
            }
        }
    }
    (void)cudaGetLastError();
    delete comm;
    if (have_prev) {
        cudaSetDevice(prev);
    }
    return CKL_OK;
}

int ckl_comm_alloc_shared(ckl_comm* comm, size_t bytes, void** local) {
    if (const int rc = check_comm(comm, "ckl_comm_alloc_shared"); rc != CKL_OK) {
        return rc;
    }
    if (local == nullptr || bytes == 0) {
        return set_error(CKL_ERR_INVALID_ARG, "ckl_comm_alloc_shared: null result pointer or zero bytes");
    }
    std::lock_guard<std::mutex> lock(comm->mu);
    void* mine = nullptr;
    SH_TRY_CUDA(cudaMalloc(&mine, bytes));
    SharedAlloc entry;
    entry.bytes = bytes;
    entry.peers.assign(static_cast<size_t>(comm->world), nullptr);
    entry.opened.assign(static_cast<size_t>(comm->world), false);
    entry.peers[static_cast<size_t>(comm->rank)] = mine;
    if (comm->world > 1) {
        // Every rank publishes an IPC handle of its buffer; the records travel through a
        // small device buffer with one all-gather.
        NcclApi* api = load_nccl();
        const size_t rec = sizeof(ShareRecord);
        auto release = [&](int rc) {
            cudaFree(mine);
            return rc;
        };
        if (const int rc = ensure(&comm->exchange, rec * static_cast<size_t>(comm->world)); rc != CKL_OK) {
            return release(rc);
        }
        ShareRecord own;
        std::memset(&own, 0, sizeof own);
        cudaError_t e = cudaIpcGetMemHandle(&own.handle, mine);
        if (e != cudaSuccess) {
            return release(set_error(CKL_ERR_CUDA, "cudaIpcGetMemHandle failed: %s", cudaGetErrorString(e)));
        }
        own.address = reinterpret_cast<unsigned long long>(mine);
        own.pid = static_cast<long long>(getpid());
        own.device = comm->device;
        auto* slots = static_cast<unsigned char*>(comm->exchange.ptr);
        e = cudaMemcpyAsync(slots + rec * static_cast<size_t>(comm->rank), &own, rec, cudaMemcpyHostToDevice,
                            comm->s_coll);
        if (e != cudaSuccess) {
            return release(set_error(CKL_ERR_CUDA, "record upload failed: %s", cudaGetErrorString(e)));
        }
        const int res = api->AllGather(slots + rec * static_cast<size_t>(comm->rank), slots, rec, kNcclUint8,
                                       comm->nccl, comm->s_coll);
        if (res != 0) {
            return release(nccl_fail(api, res, "ncclAllGather of the buffer records"));
        }
        std::vector<ShareRecord> all(static_cast<size_t>(comm->world));
        e = cudaMemcpyAsync(all.data(), slots, rec * static_cast<size_t>(comm->world), cudaMemcpyDeviceToHost,
                            comm->s_coll);
        if (e == cudaSuccess) {
            e = cudaStreamSynchronize(comm->s_coll);
        }
        if (e != cudaSuccess) {
            return release(set_error(CKL_ERR_CUDA, "record download failed: %s", cudaGetErrorString(e)));
        }
        for (int r = 0; r < comm->world; ++r) {
            if (r == comm->rank) {
                continue;
            }
            const ShareRecord& other = all[static_cast<size_t>(r)];
            void* mapped = nullptr;
            if (other.pid == own.pid) {
                // same process (one thread per GPU): the address is valid here, the devices
                // only need peer access switched on
                mapped = reinterpret_cast<void*>(other.address);
                const cudaError_t pe = cudaDeviceEnablePeerAccess(other.device, 0);
                if (pe != cudaSuccess && pe != cudaErrorPeerAccessAlreadyEnabled) {
                    return release(set_error(CKL_ERR_CUDA, "peer access to device %d refused: %s",
                                             other.device, cudaGetErrorString(pe)));
                }
                (void)cudaGetLastError();
            } else {
                e = cudaIpcOpenMemHandle(&mapped, other.handle, cudaIpcMemLazyEnablePeerAccess);
                if (e != cudaSuccess) {
                    for (int q = 0; q < r; ++q) {
                        if (entry.opened[static_cast<size_t>(q)]) {
                            cudaIpcCloseMemHandle(entry.peers[static_cast<size_t>(q)]);
                        }
                    }
                    return release(set_error(CKL_ERR_CUDA, "cudaIpcOpenMemHandle for rank %d failed: %s", r,
                                             cudaGetErrorString(e)));
                }
                entry.opened[static_cast<size_t>(r)] = true;
            }
            entry.peers[static_cast<size_t>(r)] = mapped;
        }
    }
    comm->shared[mine] = std::move(entry);
    *local = mine;
    return CKL_OK;
}

int ckl_comm_free_shared(ckl_comm* comm, void* local) {
    if (const int rc = check_comm(comm, "ckl_comm_free_shared"); rc != CKL_OK) {
        return rc;
    }
    std::lock_guard<std::mutex> lock(comm->mu);
    auto it = comm->shared.find(local);
    if (it == comm->shared.end()) {
        return set_error(CKL_ERR_INVALID_ARG, "ckl_comm_free_shared: not a buffer of this communicator");
    }
    SH_TRY_CUDA(cudaDeviceSynchronize());
    // every rank must be past its last store into the others' copies before they go
    if (const int rc = rank_barrier(comm); rc != CKL_OK) {
        return rc;
    }
    SH_TRY_CUDA(cudaStreamSynchronize(comm->s_coll));
    for (size_t r = 0; r < it->second.peers.size(); ++r) {
        if (it->second.opened[r]) {
            cudaIpcCloseMemHandle(it->second.peers[r]);
        }
    }
    SH_TRY_CUDA(cudaFree(local));
    comm->shared.erase(it);
    return CKL_OK;
}

int ckl_scatter_column_block(void* const* dsts, int parts, const void* src, int elem_size, int rows,
                             int width, int n, int col0, ckl_stream_t stream) {
    if (rows <= 0 || width <= 0 || parts <= 0) {
        return CKL_OK;
    }
    if (dsts == nullptr || src == nullptr || parts > kMaxWorld || (elem_size != 2 && elem_size != 4) ||
        col0 < 0 || col0 + width > n) {
        return set_error(CKL_ERR_INVALID_ARG, "ckl_scatter_column_block: bad arguments");
    }
    ScatterDsts d = {};
    for (int i = 0; i < parts; ++i) {
        if (dsts[i] == nullptr) {
            return set_error(CKL_ERR_INVALID_ARG, "ckl_scatter_column_block: destination %d is null", i);
        }
        d.ptr[i] = dsts[i];
    }
    return launch_scatter(d, parts, src, elem_size, rows, width, n, col0, 0, static_cast<cudaStream_t>(stream));
}

int ckl_gemm_gathered(ckl_comm* comm, int ab_dtype, const void* a, const void* b_shard, void* c_shard,
                      void* c_full, int c_dtype, int m, int n, int k, int lda, int ldb, float alpha,
                      float beta, ckl_stream_t stream_) {
    if (const int rc = check_comm(comm, "ckl_gemm_gathered"); rc != CKL_OK) {
        return rc;
    }
    if (m <= 0 || n <= 0) {
        return CKL_OK;
    }
    if (c_dtype != CKL_F32 && c_dtype != CKL_F16 && c_dtype != CKL_BF16) {
        return set_error(CKL_ERR_INVALID_ARG, "C dtype must be CKL_F32, CKL_F16 or CKL_BF16");
    }
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    std::lock_guard<std::mutex> lock(comm->mu);
    auto it = comm->shared.find(c_full);
    const size_t csz = dtype_bytes(c_dtype);
    if (it == comm->shared.end() || it->second.bytes < static_cast<size_t>(m) * n * csz) {
        return set_error(CKL_ERR_INVALID_ARG,
                         "ckl_gemm_gathered: c_full must come from ckl_comm_alloc_shared of this "
                         "communicator and hold m*n elements");
    }
    int col0 = 0, width = 0;
    if (const int rc = ckl_column_shard(n, comm->world, comm->rank, 8, &col0, &width); rc != CKL_OK) {
        return rc;
    }
    if (width > 0 && c_shard == nullptr) {
        return set_error(CKL_ERR_INVALID_ARG, "ckl_gemm_gathered: c_shard is null");
    }
    ScatterDsts dsts = {};
    for (int r = 0; r < comm->world; ++r) {
        dsts.ptr[r] = it->second.peers[static_cast<size_t>(r)];
    }
    // Row panels: the copy of panel i to every rank runs on s_coll while `stream` multiplies
    // panel i+1.  CKL_GATHER_PANELS overrides the count (1..8).
    const char* forced = std::getenv("CKL_GATHER_PANELS");
    const int forced_panels = forced != nullptr ? std::max(1, std::min(kMaxPanels, std::atoi(forced))) : 0;
    // Each panel should still be a GEMM of about two waves of 256x256 tiles: finer panels
    // hide more of the transfer but run the multiplication less efficiently (8192^3, 0.425 ms
    // with 4 panels against 0.435 with 2 at 2 GPUs, 0.283 with 2 against 0.334 with 4 at 4).
    const long long rank_tiles = static_cast<long long>((m + 255) / 256) * ((width + 255) / 256);
    int panels = forced_panels > 0 ? forced_panels
                                   : static_cast<int>(std::max<long long>(2, std::min<long long>(4, rank_tiles / 128)));
    panels = std::max(1, std::min(panels, m / 256));
    if (comm->world == 1) {
        panels = 1;
    }
    const int panel_rows = ((m + panels - 1) / panels + 255) / 256 * 256;
    // Entry: no rank may overwrite a peer's C before that peer has reached this call in its
    // own stream order (it may still be reading the previous result).
    SH_TRY_CUDA(cudaEventRecord(comm->ev_entry, stream));
    SH_TRY_CUDA(cudaStreamWaitEvent(comm->s_coll, comm->ev_entry, 0));
    if (const int rc = rank_barrier(comm); rc != CKL_OK) {
        return rc;
    }
    int used = 0;
    for (int row0 = 0; row0 < m; row0 += panel_rows, ++used) {
        const int rows = std::min(panel_rows, m - row0);
        if (width > 0) {
            const auto* a_panel = static_cast<const unsigned char*>(a) + static_cast<size_t>(row0) * lda * 2;
            auto* c_panel = static_cast<unsigned char*>(c_shard) + static_cast<size_t>(row0) * width * csz;
            if (const int rc = ckl_gemm_ex(ab_dtype, a_panel, b_shard, c_panel, c_dtype, rows, width, k, lda,
                                           ldb, width, alpha, beta, CKL_ALGO_AUTO, stream);
                rc != CKL_OK) {
                return rc;
            }
            SH_TRY_CUDA(cudaEventRecord(comm->ev_done[used], stream));
            SH_TRY_CUDA(cudaStreamWaitEvent(comm->s_coll, comm->ev_done[used], 0));
            if (const int rc = launch_scatter(dsts, comm->world, c_panel, static_cast<int>(csz), rows, width, n,
                                              col0, static_cast<size_t>(row0), comm->s_coll);
                rc != CKL_OK) {
                return rc;
            }
        }
    }
    // Exit: every rank's stores have been issued and completed (kernel boundaries) before
    // anybody's `stream` goes on.
    if (const int rc = rank_barrier(comm); rc != CKL_OK) {
        return rc;
    }
    SH_TRY_CUDA(cudaEventRecord(comm->ev_exit, comm->s_coll));
    SH_TRY_CUDA(cudaStreamWaitEvent(stream, comm->ev_exit, 0));
    return CKL_OK;
}

int ckl_gemm_host_sharded(ckl_comm* comm, int ab_dtype, const void* a_rows_host, const void* b_shard_host,
                          void* c_shard_host, int c_dtype, int m, int n_shard, int k, float alpha,
                          float beta) {
    if (const int rc = check_comm(comm, "ckl_gemm_host_sharded"); rc != CKL_OK) {
        return rc;
    }
    if (ab_dtype != CKL_F16 && ab_dtype != CKL_BF16) {
        return set_error(CKL_ERR_INVALID_ARG, "A/B dtype must be CKL_F16 or CKL_BF16 (got %d)", ab_dtype);
    }
    if (c_dtype != CKL_F32 && c_dtype != CKL_F16 && c_dtype != CKL_BF16) {
        return set_error(CKL_ERR_INVALID_ARG, "C dtype must be CKL_F32, CKL_F16 or CKL_BF16");
    }
    if (m <= 0) {
        return CKL_OK;
    }
    ckl_host_shard_plan plan;
    if (const int rc = ckl_plan_host_sharded(m, comm->world, comm->rank, &plan); rc != CKL_OK) {
        return rc;
    }
    const size_t kk = static_cast<size_t>(std::max(k, 0));
    const size_t nn = static_cast<size_t>(std::max(n_shard, 0));
    if ((nn > 0 && c_shard_host == nullptr) || (kk > 0 && nn > 0 && b_shard_host == nullptr) ||
        (kk > 0 && plan.rows > 0 && a_rows_host == nullptr)) {
        return set_error(CKL_ERR_INVALID_ARG, "ckl_gemm_host_sharded: null host pointer");
    }
    std::lock_guard<std::mutex> lock(comm->mu);
    NcclApi* api = comm->world > 1 ? load_nccl() : nullptr;
    const size_t csz = dtype_bytes(c_dtype);
    const size_t a_row = kk * 2, c_row = nn * csz;
    const size_t pr = static_cast<size_t>(plan.panel_rows);
    const size_t world = static_cast<size_t>(comm->world);
    if (int rc = ensure(&comm->dev_a, std::max<size_t>(static_cast<size_t>(plan.padded_rows) * a_row, 16)); rc != CKL_OK) return rc;
    if (int rc = ensure(&comm->dev_b, std::max<size_t>(kk * nn * 2, 16)); rc != CKL_OK) return rc;
    if (int rc = ensure(&comm->dev_c, std::max<size_t>(static_cast<size_t>(plan.padded_rows) * c_row, 16)); rc != CKL_OK) return rc;
    auto* dev_a = static_cast<unsigned char*>(comm->dev_a.ptr);
    auto* dev_c = static_cast<unsigned char*>(comm->dev_c.ptr);
    const auto* host_a = static_cast<const unsigned char*>(a_rows_host);
    auto* host_c = static_cast<unsigned char*>(c_shard_host);

    int rc = CKL_OK;
    auto cuda_ok = [&rc](cudaError_t e, const char* what) {
        if (e != cudaSuccess && rc == CKL_OK) {
            rc = set_error(CKL_ERR_CUDA, "ckl_gemm_host_sharded: %s failed: %s", what, cudaGetErrorString(e));
        }
        return rc == CKL_OK;
    };
    // Device layout of A and C: [panel j][rank r][panel_rows] rows, so that the all-gather of
    // panel j fills one contiguous block and GEMM j runs over world * panel_rows whole rows.
    // Row i of rank r's panel j is global row r * rows_per_rank + j * panel_rows + i.
    auto rows_of = [&](int r, int j) {  // rows rank r really owns in panel j
        const long long first = static_cast<long long>(r) * plan.rows_per_rank;
        const long long own = std::max<long long>(0, std::min<long long>(plan.rows_per_rank, m - first));
        return static_cast<int>(std::max<long long>(0, std::min<long long>(plan.panel_rows, own - static_cast<long long>(j) * plan.panel_rows)));
    };
    // One panel of the column block of C between host (row-major, packed) and device layout.
    auto move_c_panel = [&](int j, bool to_device, cudaStream_t s) {
        if (c_row == 0) {
            return true;
        }
        const size_t chunk = pr * c_row;
        const size_t host_pitch = static_cast<size_t>(plan.rows_per_rank) * c_row;
        unsigned char* dev = dev_c + static_cast<size_t>(j) * world * chunk;
        unsigned char* host = host_c + static_cast<size_t>(j) * chunk;
        const bool whole = rows_of(comm->world - 1, j) == plan.panel_rows && host_pitch <= 0x7fffffffull;
        if (whole) {
            // every rank's chunk is complete: one strided copy of `world` chunks
            return to_device ? cuda_ok(cudaMemcpy2DAsync(dev, chunk, host, host_pitch, chunk, world,
                                                         cudaMemcpyHostToDevice, s), "copy of C")
                             : cuda_ok(cudaMemcpy2DAsync(host, host_pitch, dev, chunk, chunk, world,
                                                         cudaMemcpyDeviceToHost, s), "copy of the result");
        }
        for (int r = 0; r < comm->world; ++r) {
            const size_t bytes = static_cast<size_t>(rows_of(r, j)) * c_row;
            if (bytes == 0) {
                continue;
            }
            unsigned char* h = host + static_cast<size_t>(r) * host_pitch;
            unsigned char* d = dev + static_cast<size_t>(r) * chunk;
            if (!(to_device ? cuda_ok(cudaMemcpyAsync(d, h, bytes, cudaMemcpyHostToDevice, s), "copy of C")
                            : cuda_ok(cudaMemcpyAsync(h, d, bytes, cudaMemcpyDeviceToHost, s), "copy of the result"))) {
                return false;
            }
        }
        return true;
    };

    cudaStream_t s_in = comm->s_in, s_run = comm->s_run, s_out = comm->s_out, s_coll = comm->s_coll;
    // Upload order: B, then panel by panel this rank's rows of A (the panel's all-gather starts
    // as soon as they have landed) and the panel's C_in.  Panel j can then be multiplied and
    // sent back while the later panels are still on their way up: on the boxes measured the
    // way back is the slower direction when every GPU transfers at once (8 GPUs: 94 GB/s in
    // total against 190 GB/s up), so it has to start early to hide behind the uploads.
    if (kk * nn > 0) {
        cuda_ok(cudaMemcpyAsync(comm->dev_b.ptr, b_shard_host, kk * nn * 2, cudaMemcpyHostToDevice, s_in), "copy of B");
    }
    cuda_ok(cudaEventRecord(comm->ev_b, s_in), "event record");
    for (int j = 0; j < plan.panels && rc == CKL_OK; ++j) {
        unsigned char* slot = dev_a + (static_cast<size_t>(j) * world + static_cast<size_t>(comm->rank)) * pr * a_row;
        const size_t bytes = static_cast<size_t>(rows_of(comm->rank, j)) * a_row;
        if (bytes > 0) {
            cuda_ok(cudaMemcpyAsync(slot, host_a + static_cast<size_t>(j) * pr * a_row, bytes, cudaMemcpyHostToDevice, s_in),
                    "copy of A");
        }
        cuda_ok(cudaEventRecord(comm->ev_a[j], s_in), "event record");
        cuda_ok(cudaStreamWaitEvent(s_coll, comm->ev_a[j], 0), "stream wait");
        if (rc == CKL_OK && comm->world > 1 && a_row > 0) {
            unsigned char* block = dev_a + static_cast<size_t>(j) * world * pr * a_row;
            const int res = api->AllGather(slot, block, pr * a_row, kNcclUint8, comm->nccl, s_coll);
            if (res != 0) {
                rc = nccl_fail(api, res, "ncclAllGather of an A row panel");
            }
        }
        cuda_ok(cudaEventRecord(comm->ev_g[j], s_coll), "event record");
        if (beta != 0.0f) {
            move_c_panel(j, true, s_in);
        }
        cuda_ok(cudaEventRecord(comm->ev_c[j], s_in), "event record");
    }
    for (int j = 0; j < plan.panels && rc == CKL_OK && nn > 0; ++j) {
        if (j == 0) {
            cuda_ok(cudaStreamWaitEvent(s_run, comm->ev_b, 0), "stream wait");
        }
        cuda_ok(cudaStreamWaitEvent(s_run, comm->ev_g[j], 0), "stream wait");
        cuda_ok(cudaStreamWaitEvent(s_run, comm->ev_c[j], 0), "stream wait");
        if (rc != CKL_OK) {
            break;
        }
        const size_t block_rows = world * pr;
        rc = ckl_gemm_ex(ab_dtype, dev_a + static_cast<size_t>(j) * block_rows * a_row, comm->dev_b.ptr,
                         dev_c + static_cast<size_t>(j) * block_rows * c_row, c_dtype, static_cast<int>(block_rows),
                         n_shard, k, k, n_shard, n_shard, alpha, beta, CKL_ALGO_AUTO, s_run);
        if (rc != CKL_OK) {
            break;
        }
        cuda_ok(cudaEventRecord(comm->ev_done[j], s_run), "event record");
        cuda_ok(cudaStreamWaitEvent(s_out, comm->ev_done[j], 0), "stream wait");
        if (rc == CKL_OK) {
            move_c_panel(j, false, s_out);
        }
    }
    return sync_all(comm, rc);
}

}  // extern "C"
