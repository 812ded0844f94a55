// ckl_gemm_streamk_noalloc: the stream-K tensor-core GEMM for callers that must
// not allocate device memory.
//
// Who needs it.  Some hosts hand every byte of device memory to an arena of
// their own at start-up (inference servers, simulation codes with a fixed
// memory plan), so a cudaMalloc made inside a library either fails or eats
// into a budget the host has already promised elsewhere.  Others run the GEMM
// inside a latency-critical loop and cannot accept that cudaMalloc and
// cudaFree synchronise the whole device.  The regular entry points allocate a
// per-device status word on first use and, when the stream-K split is chosen,
// a per-stream workspace for partial tiles.  This entry point allocates
// nothing, ever: its partial-tile workspace and its status word are
// file-scope __device__ arrays that live in the library's own image.
//
// What that costs.  Every GPU that loads the library carries the array
// (kScratchBytes, 37 MiB) until the process exits, whether or not this entry
// point is called.  The CUDA runtime backs the array with device memory when it
// loads this library's device code on a GPU, which with lazy module loading
// happens at the first call made from this file on that GPU: a host that is
// about to hand all device memory to its own arena must make that first call
// BEFORE it does so, or the load itself runs out of memory.  The array is sized for a schedule of at most
// kMaxUnits = 148 CTAs (a B200); a device whose schedule would need more is
// refused with CKL_ERR_TOO_LARGE rather than run with a smaller grid.
//
// Sharing.  All calls on a device use the same array.  Nothing in it has to
// start at zero: a partial slot is always written in full by the GEMM kernel
// before the fix-up pass of the same call reads it, and slots a call does not
// write are not read, so contents left by an earlier call are harmless.  For
// the same reason two calls that overlap on the GPU (different streams, or
// several host threads) would overwrite each other's partial tiles: keep
// calls to this entry point on one stream per device, or order them with
// events.
//
// Set-up.  The first call on each device, made with that device current,
// looks up the device addresses of the arrays (in host code the array's name
// is only a handle for the runtime, not an address a kernel could use), raises
// the kernels' dynamic shared-memory limit and fetches the driver's
// tensor-map encoder.  None of this allocates, but it is one-time work that
// talks to the driver: make the first call on a device during start-up, before
// any stream capture begins.

#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <mutex>

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "ckl_gemm.h"
#include "gemm_umma.cuh"
#include "tile_sched.h"

namespace {

using namespace ckl;

constexpr int kMaxUnits = 148;
constexpr size_t kSlotBytes = UmmaConfig<kModeSingle>::kSlotFloats * sizeof(float);  // 128 KB
constexpr size_t kScratchBytes = 2 * static_cast<size_t>(kMaxUnits) * kSlotBytes;  // 38,797,312

// The scratch itself.  Device code could name these directly; host code below
// must go through cudaGetSymbolAddress.
static __device__ __align__(256) unsigned char g_scratch[kScratchBytes];
static __device__ __align__(16) unsigned int g_status_words[4];

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                   const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                   const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

struct DeviceState {
    bool ready = false;
    int sm_count = 0;
    float* scratch = nullptr;         // device address of g_scratch on this device
    unsigned int* status = nullptr;   // device address of g_status_words on this device
    EncodeTiledFn encode = nullptr;
};

constexpr int kMaxDevices = 64;
DeviceState g_state[kMaxDevices];
std::mutex g_mu;
thread_local char g_message[512];

int fail(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_message, sizeof g_message, fmt, ap);
    va_end(ap);
    return code;
}

#define NOALLOC_TRY(expr)                                                                     \
    do {                                                                                      \
        const cudaError_t err__ = (expr);                                                     \
        if (err__ != cudaSuccess) {                                                           \
            return fail(CKL_ERR_CUDA, "%s failed: %s (%s)", #expr, cudaGetErrorName(err__),   \
                        cudaGetErrorString(err__));                                           \
        }                                                                                     \
    } while (0)

template <typename OutT>
cudaError_t raise_smem_limit() {
    return cudaFuncSetAttribute(umma_gemm_kernel<kModeSingle, OutT>,
                                cudaFuncAttributeMaxDynamicSharedMemorySize,
                                static_cast<int>(UmmaConfig<kModeSingle>::kSmemBytes));
}

// One-time, per device, with that device current.  Allocates nothing.
int set_up(DeviceState** out) {
    int dev = 0;
    NOALLOC_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= kMaxDevices) {
        return fail(CKL_ERR_UNSUPPORTED, "device index %d is outside the supported range", dev);
    }
    std::lock_guard<std::mutex> lock(g_mu);
    DeviceState& st = g_state[dev];
    if (!st.ready) {
        int major = 0, sms = 0;
        NOALLOC_TRY(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev));
        NOALLOC_TRY(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
        if (major != 10) {
            return fail(CKL_ERR_UNSUPPORTED, "device %d is not sm_100", dev);
        }
        void* scratch = nullptr;
        void* status = nullptr;
        NOALLOC_TRY(cudaGetSymbolAddress(&scratch, g_scratch));
        NOALLOC_TRY(cudaGetSymbolAddress(&status, g_status_words));
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult qres;
        NOALLOC_TRY(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres));
        if (fn == nullptr || qres != cudaDriverEntryPointSuccess) {
            return fail(CKL_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
        }
        NOALLOC_TRY(raise_smem_limit<float>());
        NOALLOC_TRY(raise_smem_limit<__half>());
        NOALLOC_TRY(raise_smem_limit<__nv_bfloat16>());
        st.sm_count = sms;
        st.scratch = static_cast<float*>(scratch);
        st.status = static_cast<unsigned int*>(status);
        st.encode = reinterpret_cast<EncodeTiledFn>(fn);
        st.ready = true;
    }
    *out = &st;
    return CKL_OK;
}

int encode(const DeviceState& st, CUtensorMap* map, int dtype, const void* base, uint64_t inner,
           uint64_t outer, uint64_t pitch_elems, uint32_t box_inner, uint32_t box_outer) {
    const size_t esz = dtype == CKL_F32 ? 4 : 2;
    const cuuint64_t dims[2] = {inner, outer};
    const cuuint64_t strides[1] = {pitch_elems * esz};
    const cuuint32_t box[2] = {box_inner, box_outer};
    const cuuint32_t ones[2] = {1, 1};
    const CUtensorMapDataType dt = dtype == CKL_F16    ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16
                                   : dtype == CKL_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                                       : CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
    const CUresult r = st.encode(map, dt, 2, const_cast<void*>(base), dims, strides, box, ones,
                                 CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                 CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                 CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        return fail(CKL_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", static_cast<int>(r));
    }
    return CKL_OK;
}

template <typename OutT>
int launch(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc, const GemmParams& p,
           int grid, cudaStream_t stream) {
    umma_gemm_kernel<kModeSingle, OutT>
        <<<grid, UmmaConfig<kModeSingle>::kThreads, UmmaConfig<kModeSingle>::kSmemBytes, stream>>>(ta, tb, tc, p);
    NOALLOC_TRY(cudaGetLastError());
    if (p.sched.sk_tiles > 0) {
        streamk_fixup_kernel<UmmaConfig<kModeSingle>::kTileM, UmmaConfig<kModeSingle>::kTileN, OutT><<<dim3(static_cast<unsigned>(p.sched.sk_tiles), UmmaConfig<kModeSingle>::kTileM / 32), 256, 0, stream>>>(p);
        NOALLOC_TRY(cudaGetLastError());
    }
    return CKL_OK;
}

}  // namespace

extern "C" {

int ckl_gemm_streamk_noalloc(int ab_dtype, const void* a, const void* b, void* c, int c_dtype, int m,
                             int n, int k, int lda, int ldb, int ldc, float alpha, float beta,
                             ckl_stream_t stream) {
    if ((ab_dtype != CKL_F16 && ab_dtype != CKL_BF16) ||
        (c_dtype != CKL_F32 && c_dtype != CKL_F16 && c_dtype != CKL_BF16)) {
        return fail(CKL_ERR_INVALID_ARG, "bad dtype (A/B %d, C %d)", ab_dtype, c_dtype);
    }
    if (m <= 0 || n <= 0) {
        return CKL_OK;
    }
    if (a == nullptr || b == nullptr || c == nullptr) {
        return fail(CKL_ERR_INVALID_ARG, "A, B or C is null");
    }
    if (k <= 0) {
        return fail(CKL_ERR_UNSUPPORTED,
                    "this entry point only runs the tensor-core kernel, which needs k > 0 (use "
                    "ckl_gemm_ex for C = beta*C)");
    }
    if (lda < k || ldb < n || ldc < n) {
        return fail(CKL_ERR_INVALID_ARG, "need lda >= k, ldb >= n, ldc >= n");
    }
    if (reinterpret_cast<uintptr_t>(a) % 16 != 0 || reinterpret_cast<uintptr_t>(b) % 16 != 0 ||
        lda % 8 != 0 || ldb % 8 != 0) {
        return fail(CKL_ERR_UNSUPPORTED,
                    "this entry point only runs the tensor-core kernel: A and B must be 16-byte "
                    "aligned with lda and ldb multiples of 8 (use ckl_gemm_ex otherwise)");
    }
    DeviceState* st = nullptr;
    if (const int rc = set_up(&st); rc != CKL_OK) {
        return rc;
    }
    // Same planner as every other entry point (pure host arithmetic), split forced on.
    ckl_plan plan;
    if (const int rc = ckl_plan_gemm(m, n, k, lda, ldb, ldc, 16, 16, CKL_ALGO_UMMA_SK, st->sm_count,
                                     &plan);
        rc != CKL_OK) {
        return fail(rc, "planning failed: %s", ckl_last_error());
    }
    if (plan.units > kMaxUnits || plan.workspace_bytes > kScratchBytes) {
        return fail(CKL_ERR_TOO_LARGE,
                    "the schedule for this device needs %zu bytes of partial-tile scratch for %d "
                    "units; the built-in scratch holds %zu bytes (%d units)",
                    plan.workspace_bytes, plan.units, kScratchBytes, kMaxUnits);
    }
    CUtensorMap ta, tb, tc;
    std::memset(&tc, 0, sizeof tc);
    if (int rc = encode(*st, &ta, ab_dtype, a, static_cast<uint64_t>(k), static_cast<uint64_t>(m),
                        static_cast<uint64_t>(lda), 64, 128);
        rc != CKL_OK) {
        return rc;
    }
    if (int rc = encode(*st, &tb, ab_dtype, b, static_cast<uint64_t>(n), static_cast<uint64_t>(k),
                        static_cast<uint64_t>(ldb), 64, 64);
        rc != CKL_OK) {
        return rc;
    }
    GemmParams p = {};
    p.c = c;
    p.bias = nullptr;
    p.workspace = st->scratch;
    p.status = st->status;
    p.m = m;
    p.n = n;
    p.k = k;
    p.ldc = ldc;
    p.alpha = alpha;
    p.beta = beta;
    const size_t csz = c_dtype == CKL_F32 ? 4 : 2;
    p.c_vec = (reinterpret_cast<uintptr_t>(c) % 16 == 0 && (static_cast<size_t>(ldc) * csz) % 16 == 0)
                  ? 1
                  : 0;
    p.c_tma = p.c_vec;
    if (p.c_tma) {
        if (int rc = encode(*st, &tc, c_dtype, c, static_cast<uint64_t>(n), static_cast<uint64_t>(m),
                            static_cast<uint64_t>(ldc), static_cast<uint32_t>(128 / csz), 32);
            rc != CKL_OK) {
            return rc;
        }
    }
    p.epi_mode = kEpiLinear;
    p.idesc = ptx::make_idesc_f16(ab_dtype == CKL_F16 ? 0u : 1u, 0u, 1u, 128u, 256u);
    p.sched.tiles_m = plan.tiles_m;
    p.sched.tiles_n = plan.tiles_n;
    p.sched.k_blocks = plan.k_blocks;
    p.sched.units = plan.units;
    p.sched.dp_tiles = plan.dp_tiles;
    p.sched.sk_tiles = plan.sk_tiles;
    p.sched.group_m = plan.group_m;
    p.sched.sk_iters = plan.sk_iters;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    switch (c_dtype) {
        case CKL_F32: return launch<float>(ta, tb, tc, p, plan.grid, s);
        case CKL_F16: return launch<__half>(ta, tb, tc, p, plan.grid, s);
        default: return launch<__nv_bfloat16>(ta, tb, tc, p, plan.grid, s);
    }
}

int ckl_noalloc_device_status(unsigned int* info) {
    DeviceState* st = nullptr;
    if (const int rc = set_up(&st); rc != CKL_OK) {
        return rc;
    }
    NOALLOC_TRY(cudaDeviceSynchronize());
    unsigned int words[4] = {0, 0, 0, 0};
    NOALLOC_TRY(cudaMemcpy(words, st->status, sizeof words, cudaMemcpyDeviceToHost));
    if (info != nullptr) {
        std::memcpy(info, words, sizeof words);
    }
    if (words[0] != 0) {
        NOALLOC_TRY(cudaMemset(st->status, 0, sizeof words));
        return fail(CKL_ERR_DEVICE,
                    "a kernel of ckl_gemm_streamk_noalloc gave up a bounded wait: code=%u block=%u "
                    "role=%u detail=0x%x; C of that call is incomplete",
                    words[0], words[1], words[2], words[3]);
    }
    return CKL_OK;
}

const char* ckl_noalloc_last_error(void) { return g_message; }

size_t ckl_noalloc_scratch_bytes(void) { return kScratchBytes; }

}  // extern "C"
