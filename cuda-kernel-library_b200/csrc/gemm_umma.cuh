// Tensor-core GEMM for sm_100a: TMA-fed shared-memory ring, tcgen05.mma
// accumulating in tensor memory, warp-specialised persistent CTAs.
//
// Replaces the reference's whole FP16/BF16 ladder (wmma_gemm_kernel,
// include/ckl/detail/wmma_gemm.cuh:49-119; gemm_mma_ptx_kernel,
// src/gemm/gemm_mma_ptx.cu:50-136; gemm_mma_ldmatrix_kernel,
// src/gemm/gemm_mma_ldmatrix.cu:60-133; gemm_mma_opt_kernel,
// src/gemm/gemm_mma_opt.cu:87-195).  It shares nothing with them: there is no
// mma.sync, ldmatrix or cp.async here.
//
// One kernel template, three shapes of worker ("unit"; KernelMode below):
//
//   kPair = false   one CTA per unit, output tile 128 x 256, UMMA 128x256x16,
//                   4-stage ring of (A 128x64, B 64x256) = 48 KB per stage.  With
//                   GemmParams::tile_n = 128 the same kernel runs 128 x 128 tiles
//                   (half of the B boxes, UMMA 128x128x16) for small problems.
//   kPair = true    a cluster of two CTAs per unit, output tile 256 x 256,
//                   UMMA 256x256x16 issued by the leader CTA for both SMs
//                   (cta_group::2).  Each CTA loads only its own 128 rows of A
//                   and its own 128 columns of B (no multicast); a stage holds
//                   128 k elements (64 KB per CTA), 3 stages.
//
// Data layout.  A is row-major m x k, so a 128 x 64 box lands in shared memory
// K-major: 128 rows of 128 bytes under the 128-byte swizzle.  B is row-major
// k x n, i.e. N-major; a stage holds 64-column boxes of 64 k-rows x 128 bytes,
// also 128-byte swizzled, and the MMA reads them through an MN-major
// descriptor (leading offset = one box, stride offset = 8 k-rows), so B is
// never transposed in memory.  TMA zero-fills whatever lies outside the
// matrix, which is what makes ragged m, n and k work: zero rows of A and zero
// k-rows contribute nothing and the epilogue predicates its stores.
//
// Warp roles (192 threads): warp 0 = TMA producer (one lane), warp 1 = MMA
// issuer (one lane) and TMEM owner, warps 2-5 = epilogue (each reads the TMEM
// lane quarter its warp id selects).  The 512 TMEM columns hold two 256-column
// accumulators so the epilogue of one tile overlaps the main loop of the next.
//
// Every wait on an mbarrier is bounded: after kWaitLimitNs the waiter records
// a code in the status word, raises the CTA's abort flag (and the peer's), and
// every role falls through to the common exit, which drains in-flight copies
// and MMAs, frees TMEM and returns.  Nothing traps or spins without limit.
#pragma once

#include <cstdint>

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "ptx.cuh"
#include "tile_sched.h"

namespace ckl {

enum EpilogueMode : int { kEpiLinear = 0, kEpiBiasRelu = 1 };

struct GemmParams {
    void* c;              // output, OutT, row-major, leading dimension ldc
    const float* bias;    // n floats (kEpiBiasRelu) or nullptr
    float* workspace;     // partial-tile slots (stream-K) or nullptr
    unsigned int* sk_flags;  // fused stream-K: one word per (slot, 32-row group, half), or nullptr
    unsigned int sk_epoch;   // value a flag takes when its part of a partial is complete
    unsigned int* status; // 4 words: code, block, role, detail
    int m, n, k;
    int ldc;
    float alpha, beta;
    int c_vec;            // 16-byte vector access to C is legal
    int c_tma;            // C can be described by a TMA tensor map (tmap_c is valid)
    int epi_mode;
    uint32_t idesc;
    Schedule sched;
    // Columns of an output tile.  0 means the kernel shape's own width (256, or 512 for the
    // wide pair tile); the single-CTA kernel also runs 128-column tiles (two of its four B
    // boxes per stage, UMMA 128x128x16), which doubles the tile count of small problems.
    int tile_n;
    // Limit of every bounded wait in nanoseconds; 0 means kWaitLimitNs.
    unsigned long long wait_limit_ns;
    // Test hooks, both 0 in every ordinary launch.  sk_flag_skew is added to the flag value the
    // owner of a split tile waits for, so a non-zero skew makes that wait run out;
    // overstate_first_stage makes unit 0's producer announce 16 bytes more than it loads for
    // its first stage, so that stage never completes and the MMA warp's wait runs out.
    unsigned int sk_flag_skew;
    int overstate_first_stage;
};

// Depth of the shared-memory ring (48 KB per stage for one CTA, 64 KB per CTA of a pair).
#ifndef CKL_STAGES_1CTA
#define CKL_STAGES_1CTA 4
#endif
#ifndef CKL_STAGES_2CTA
#define CKL_STAGES_2CTA 3
#endif
#ifndef CKL_STAGES_WIDE
#define CKL_STAGES_WIDE 3
#endif

// L2 eviction priority of the operand loads (ptx::kL2EvictNormal / First / Last).
#ifndef CKL_HINT_A
#define CKL_HINT_A ptx::kL2EvictNormal
#endif
#ifndef CKL_HINT_B
#define CKL_HINT_B ptx::kL2EvictNormal
#endif

constexpr unsigned long long kWaitLimitNs = 2000000000ull;  // 2 s

enum StatusCode : unsigned int {
    kStatusOk = 0,
    kStatusWaitTimeout = 1,
};
enum Role : unsigned int { kRoleProducer = 1, kRoleMma = 2, kRoleEpilogue = 3, kRoleDrain = 4 };

// Kernel shapes.  kModeSingle: one CTA per 128x256 tile.  kModePair: a CTA pair per
// 256x256 tile, two accumulators in TMEM (epilogue fully overlapped).  kModePairWide: a CTA
// pair per 256x512 tile; the accumulator fills all 512 TMEM columns, so each loaded row of
// A feeds twice as many columns (a quarter less L2-to-SM traffic, the dominant data-movement
// cost under the power cap) at the price of draining TMEM between tiles, which eight
// epilogue warps keep short.
enum KernelMode : int { kModeSingle = 0, kModePair = 1, kModePairWide = 2 };

template <int kMode>
struct UmmaConfig {
    static constexpr bool kPair = kMode != kModeSingle;
    static constexpr bool kWide = kMode == kModePairWide;
    static constexpr int kStages =
        kWide ? CKL_STAGES_WIDE : (kPair ? CKL_STAGES_2CTA : CKL_STAGES_1CTA);
    static constexpr int kNHalves = kWide ? 2 : 1;  // 256-column accumulator halves per tile
    // 64-column boxes of B this CTA loads per 64 k rows
    static constexpr int kBBoxes = kMode == kModePair ? 2 : 4;
    // A stage holds kKSub sub-blocks of 64 k elements.  Freeing a stage costs the pair a
    // cross-SM tcgen05.commit round trip, so a pair stage always carries eight MMAs:
    // 128 k of one 256-column accumulator, or 64 k of two.
    static constexpr int kKSub = kMode == kModePair ? 2 : 1;
    static constexpr uint32_t kASubBytes = 128 * 64 * 2;
    static constexpr uint32_t kBoxBytes = 64 * 64 * 2;
    static constexpr uint32_t kBSubBytes = kBBoxes * kBoxBytes;
    static constexpr uint32_t kABytes = kKSub * kASubBytes;
    static constexpr uint32_t kBBytes = kKSub * kBSubBytes;
    static constexpr uint32_t kStageBytes = kABytes + kBBytes;
    static constexpr uint32_t kTxBytes = kStageBytes * (kPair ? 2 : 1);
    static constexpr int kTileM = kPair ? 256 : 128;
    static constexpr int kTileN = 256 * kNHalves;
    static constexpr int kTileK = 64 * kKSub;
    static constexpr int kAccStages = kWide ? 1 : 2;
    static constexpr int kEpiWarps = kWide ? 8 : 4;
    static constexpr int kThreads = 64 + 32 * kEpiWarps;
    // Epilogue staging: per epilogue warp two buffers of 32 rows x 128 B.
    static constexpr uint32_t kStagingBytes = kEpiWarps * 2 * 4096;
    static constexpr int kNumBarriers = 2 * kStages + 5 + 2 * kEpiWarps;
    // ring + staging + barriers + TMEM slot + abort flag, plus slack to 1024-align the ring
    static constexpr uint32_t kSmemBytes =
        kStages * kStageBytes + kStagingBytes + kNumBarriers * 8 + 16 + 1024;
    static constexpr size_t kSlotFloats = static_cast<size_t>(kTileM) * kTileN;
};

namespace detail {

struct Control {
    volatile int* abort_flag;   // this CTA's flag (generic pointer into shared memory)
    uint32_t abort_flag_smem;   // same, as a shared-window address
    unsigned int* status;
    bool pair;
    uint32_t peer_rank;
    unsigned long long limit_ns;  // every bounded wait gives up after this long
};

__device__ __forceinline__ void raise_abort(const Control& ctl, unsigned int role,
                                            unsigned int detail_word) {
    *ctl.abort_flag = 1;
    if (ctl.pair) {
        const uint32_t remote = ptx::map_to_cta(ctl.abort_flag_smem, ctl.peer_rank);
        asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(remote), "r"(1u) : "memory");
    }
    if (atomicCAS(ctl.status, 0u, static_cast<unsigned int>(kStatusWaitTimeout)) == 0u) {
        ctl.status[1] = blockIdx.x;
        ctl.status[2] = role;
        ctl.status[3] = detail_word;
        __threadfence();
    }
}

// Bounded wait.  Returns false when the limit ran out here or another role
// already aborted; the caller must then leave its loop.
__device__ __forceinline__ bool wait_barrier(uint32_t bar, uint32_t parity, const Control& ctl,
                                             unsigned int role, unsigned int detail_word) {
    if (ptx::mbar_try_wait(bar, parity)) {
        return true;
    }
    unsigned long long t0 = 0;
    unsigned int spins = 0;
    while (true) {
        if (ptx::mbar_try_wait_parked(bar, parity, 4000u)) {
            return true;
        }
        if ((++spins & 15u) == 0u) {
            if (*ctl.abort_flag != 0) {
                return false;
            }
            const unsigned long long now = ptx::global_timer_ns();
            if (t0 == 0) {
                t0 = now;
            } else if (now - t0 > ctl.limit_ns) {
                raise_abort(ctl, role, detail_word);
                return false;
            }
        }
    }
}

// Bounded wait for a flag word another CTA of the same launch publishes (fused stream-K).
// The writer never waits for the reader, so the wait ends as soon as the writer has run;
// the limit only guards against a writer that gave up.
__device__ __forceinline__ bool wait_flag(const unsigned int* flag, unsigned int value,
                                          const Control& ctl, unsigned int role,
                                          unsigned int detail_word) {
    unsigned long long t0 = 0;
    unsigned int spins = 0;
    while (ptx::ld_acquire_gpu(flag) != value) {
        __nanosleep(200);
        if ((++spins & 63u) == 0u) {
            if (*ctl.abort_flag != 0) {
                return false;
            }
            const unsigned long long now = ptx::global_timer_ns();
            if (t0 == 0) {
                t0 = now;
            } else if (now - t0 > ctl.limit_ns) {
                raise_abort(ctl, role, detail_word);
                return false;
            }
        }
    }
    return true;
}

// Short bounded wait used only while draining on the way out: never raises.
__device__ __forceinline__ void drain_wait(uint32_t bar, uint32_t parity) {
    const unsigned long long t0 = ptx::global_timer_ns();
    for (unsigned int i = 0;; ++i) {
        if (ptx::mbar_try_wait(bar, parity)) {
            return;
        }
        if ((i & 63u) == 63u && ptx::global_timer_ns() - t0 > 20000000ull) {  // 20 ms
            return;
        }
    }
}

template <typename OutT>
struct OutTraits;
template <>
struct OutTraits<float> {
    static constexpr int kVec = 4;
    static __device__ __forceinline__ float load(const float* p) { return *p; }
    static __device__ __forceinline__ void store(float* p, float v) { *p = v; }
    static __device__ __forceinline__ void load_vec(const float* p, float (&v)[4]) {
        const float4 t = *reinterpret_cast<const float4*>(p);
        v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
    }
    static __device__ __forceinline__ void store_vec(float* p, const float* v) {
        *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
    }
    static __device__ __forceinline__ void unpack(const uint4& t, float (&v)[4]) {
        v[0] = __uint_as_float(t.x); v[1] = __uint_as_float(t.y);
        v[2] = __uint_as_float(t.z); v[3] = __uint_as_float(t.w);
    }
    // Element e (a compile-time constant after unrolling) of a 16-byte unit.
    static __device__ __forceinline__ float element(const uint4& t, int e) {
        return __uint_as_float(e == 0 ? t.x : e == 1 ? t.y : e == 2 ? t.z : t.w);
    }
};
template <>
struct OutTraits<__half> {
    static constexpr int kVec = 8;
    static __device__ __forceinline__ float load(const __half* p) { return __half2float(*p); }
    static __device__ __forceinline__ void store(__half* p, float v) { *p = __float2half_rn(v); }
    static __device__ __forceinline__ void load_vec(const __half* p, float (&v)[8]) {
        const uint4 t = *reinterpret_cast<const uint4*>(p);
        const __half2* h = reinterpret_cast<const __half2*>(&t);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 f = __half22float2(h[i]);
            v[2 * i] = f.x;
            v[2 * i + 1] = f.y;
        }
    }
    static __device__ __forceinline__ void unpack(const uint4& t, float (&v)[8]) {
        const __half2* h = reinterpret_cast<const __half2*>(&t);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 f = __half22float2(h[i]);
            v[2 * i] = f.x;
            v[2 * i + 1] = f.y;
        }
    }
    static __device__ __forceinline__ float element(const uint4& t, int e) {
        const uint32_t w = (e >> 1) == 0 ? t.x : (e >> 1) == 1 ? t.y : (e >> 1) == 2 ? t.z : t.w;
        const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w));
        return (e & 1) ? f.y : f.x;
    }
    static __device__ __forceinline__ void store_vec(__half* p, const float* v) {
        uint4 t;
        __half2* h = reinterpret_cast<__half2*>(&t);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            h[i] = __floats2half2_rn(v[2 * i], v[2 * i + 1]);
        }
        *reinterpret_cast<uint4*>(p) = t;
    }
};
template <>
struct OutTraits<__nv_bfloat16> {
    static constexpr int kVec = 8;
    static __device__ __forceinline__ float load(const __nv_bfloat16* p) {
        return __bfloat162float(*p);
    }
    static __device__ __forceinline__ void store(__nv_bfloat16* p, float v) {
        *p = __float2bfloat16_rn(v);
    }
    static __device__ __forceinline__ void load_vec(const __nv_bfloat16* p, float (&v)[8]) {
        const uint4 t = *reinterpret_cast<const uint4*>(p);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&t);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 f = __bfloat1622float2(h[i]);
            v[2 * i] = f.x;
            v[2 * i + 1] = f.y;
        }
    }
    static __device__ __forceinline__ void unpack(const uint4& t, float (&v)[8]) {
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&t);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 f = __bfloat1622float2(h[i]);
            v[2 * i] = f.x;
            v[2 * i + 1] = f.y;
        }
    }
    static __device__ __forceinline__ float element(const uint4& t, int e) {
        // BF16 is the upper half of an FP32 word
        const uint32_t w = (e >> 1) == 0 ? t.x : (e >> 1) == 1 ? t.y : (e >> 1) == 2 ? t.z : t.w;
        return __uint_as_float((e & 1) ? (w & 0xffff0000u) : (w << 16));
    }
    static __device__ __forceinline__ void store_vec(__nv_bfloat16* p, const float* v) {
        uint4 t;
        __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&t);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
        }
        *reinterpret_cast<uint4*>(p) = t;
    }
};

// The epilogue arithmetic on 32 consecutive columns of one output row:
// acc (FP32 accumulators) -> alpha / beta / bias / relu -> OutT, stores
// predicated on n.  `row_ptr` points at column 0 of the row in C.
template <typename OutT>
__device__ __forceinline__ void finish_row_chunk(float (&acc)[32], OutT* row_ptr, int col0, int n,
                                                 float alpha, float beta, const float* bias,
                                                 int epi_mode, bool vec_ok) {
    using T = OutTraits<OutT>;
    constexpr int V = T::kVec;
    if (col0 >= n) {
        return;
    }
#pragma unroll
    for (int g = 0; g < 32 / V; ++g) {
        const int col = col0 + g * V;
        if (col >= n) {
            break;
        }
        const bool full = vec_ok && (col + V <= n);
        float out[V];
        if (epi_mode == kEpiBiasRelu) {
#pragma unroll
            for (int e = 0; e < V; ++e) {
                const float bv = (col + e < n) ? __ldg(bias + col + e) : 0.0f;
                out[e] = fmaxf(alpha * acc[g * V + e] + bv, 0.0f);
            }
        } else if (beta != 0.0f) {
            float cin[V];
            if (full) {
                T::load_vec(row_ptr + col, cin);
            } else {
#pragma unroll
                for (int e = 0; e < V; ++e) {
                    cin[e] = (col + e < n) ? T::load(row_ptr + col + e) : 0.0f;
                }
            }
#pragma unroll
            for (int e = 0; e < V; ++e) {
                out[e] = alpha * acc[g * V + e] + beta * cin[e];
            }
        } else {
#pragma unroll
            for (int e = 0; e < V; ++e) {
                out[e] = alpha * acc[g * V + e];
            }
        }
        if (full) {
            T::store_vec(row_ptr + col, out);
        } else {
#pragma unroll
            for (int e = 0; e < V; ++e) {
                if (col + e < n) {
                    T::store(row_ptr + col + e, out[e]);
                }
            }
        }
    }
}

}  // namespace detail

template <int kMode, typename OutT>
__global__ void __launch_bounds__(UmmaConfig<kMode>::kThreads, 1)
umma_gemm_kernel(const __grid_constant__ CUtensorMap tmap_a,
                 const __grid_constant__ CUtensorMap tmap_b,
                 const __grid_constant__ CUtensorMap tmap_c, const GemmParams p) {
    using Cfg = UmmaConfig<kMode>;
    constexpr bool kPair = Cfg::kPair;
    constexpr bool kWide = Cfg::kWide;
    constexpr int kStages = Cfg::kStages;

    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw_addr = ptx::smem_u32(smem_raw);
    const uint32_t ring = (raw_addr + 1023u) & ~1023u;
    uint8_t* ring_ptr = smem_raw + (ring - raw_addr);
    const uint32_t staging = ring + kStages * Cfg::kStageBytes;
    uint8_t* staging_ptr = ring_ptr + kStages * Cfg::kStageBytes;
    const uint32_t bars = staging + Cfg::kStagingBytes;
    uint8_t* bars_ptr = staging_ptr + Cfg::kStagingBytes;

    auto full_bar = [&](int s) { return bars + 8u * static_cast<uint32_t>(s); };
    auto empty_bar = [&](int s) { return bars + 8u * static_cast<uint32_t>(kStages + s); };
    auto acc_full_bar = [&](int a) { return bars + 8u * static_cast<uint32_t>(2 * kStages + a); };
    auto acc_empty_bar = [&](int a) {
        return bars + 8u * static_cast<uint32_t>(2 * kStages + 2 + a);
    };
    const uint32_t drain_bar = bars + 8u * static_cast<uint32_t>(2 * kStages + 4);
    // C_in staging barriers: two per epilogue warp
    auto cin_bar = [&](int w, int b) {
        return bars + 8u * static_cast<uint32_t>(2 * kStages + 5 + 2 * w + b);
    };
    const uint32_t tmem_slot = bars + 8u * static_cast<uint32_t>(Cfg::kNumBarriers);
    volatile uint32_t* tmem_slot_ptr =
        reinterpret_cast<volatile uint32_t*>(bars_ptr + 8 * Cfg::kNumBarriers);

    detail::Control ctl;
    ctl.abort_flag = reinterpret_cast<volatile int*>(bars_ptr + 8 * Cfg::kNumBarriers + 4);
    ctl.abort_flag_smem = tmem_slot + 4u;
    ctl.status = p.status;
    ctl.pair = kPair;
    ctl.limit_ns = p.wait_limit_ns != 0 ? p.wait_limit_ns : kWaitLimitNs;

    const int warp = static_cast<int>(threadIdx.x >> 5);
    const uint32_t lane = ptx::lane_id();
    const uint32_t rank = kPair ? ptx::cluster_cta_rank() : 0u;
    ctl.peer_rank = rank ^ 1u;
    const int unit = kPair ? static_cast<int>(blockIdx.x >> 1) : static_cast<int>(blockIdx.x);
    const bool leader = (rank == 0u);

    // ---- set-up ---------------------------------------------------------------
    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            ptx::mbar_init(full_bar(s), 1);
            ptx::mbar_init(empty_bar(s), 1);
        }
        for (int a = 0; a < 2; ++a) {
            ptx::mbar_init(acc_full_bar(a), 1);
            ptx::mbar_init(acc_empty_bar(a), kPair ? 8 : 4);
        }
        ptx::mbar_init(drain_bar, 1);
        for (int w = 0; w < Cfg::kEpiWarps; ++w) {
            ptx::mbar_init(cin_bar(w, 0), 1);
            ptx::mbar_init(cin_bar(w, 1), 1);
        }
        *ctl.abort_flag = 0;
        ptx::fence_barrier_init();
        ptx::prefetch_tensormap(&tmap_a);
        ptx::prefetch_tensormap(&tmap_b);
        if (p.c_tma) {
            ptx::prefetch_tensormap(&tmap_c);
        }
    }
    if (warp == 1) {
        if constexpr (kPair) {
            ptx::tmem_alloc_pair(tmem_slot, 512);
            ptx::tmem_relinquish_pair();
        } else {
            ptx::tmem_alloc(tmem_slot, 512);
            ptx::tmem_relinquish();
        }
    }
    ptx::tc_fence_before_sync();
    if constexpr (kPair) {
        ptx::cluster_arrive_release();
        ptx::cluster_wait_acquire();
    } else {
        __syncthreads();
    }
    ptx::tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot_ptr;

    // Back-to-back launches: everything above touched only this CTA's shared and tensor
    // memory, so it may run while the previous kernel of the stream is still finishing (the
    // host launches this kernel as a programmatic dependent).  From here on global memory is
    // read and written: wait for the previous kernel.  The kernel after this one gets the same
    // head start: it needs an SM of its own anyway, so it can be let in right away.
    ptx::grid_dependency_wait();
    ptx::launch_dependents();

    const Schedule& sched = p.sched;
    // Tile width: only the single-CTA shape has a narrow form.
    const int tile_n = (kMode == kModeSingle && p.tile_n == 128) ? 128 : Cfg::kTileN;

    // ---- roles ----------------------------------------------------------------
    if (warp == 0) {
        if (ptx::elect_one_sync()) {
            // TMA producer.
            SegmentCursor cur = make_cursor(sched, unit);
            Segment seg;
            constexpr uint64_t hint_a = CKL_HINT_A, hint_b = CKL_HINT_B;
            uint32_t it = 0;       // k blocks issued so far
            int stage = 0;         // it % kStages
            uint32_t phase = 0;    // (it / kStages) & 1
            bool ok = true;
            while (ok && next_segment(sched, &cur, &seg)) {
                int tm, tn;
                tile_coords(sched, seg.tile, &tm, &tn);
                const int a_row = tm * Cfg::kTileM + (kPair ? static_cast<int>(rank) * 128 : 0);
                const int b_col = tn * tile_n + (kPair ? static_cast<int>(rank) * 128 : 0);
                const int b_boxes = kMode == kModeSingle ? tile_n / 64 : Cfg::kBBoxes;
                for (int kb = seg.kb_begin; kb < seg.kb_end; ++kb) {
                    {
                        const bool got = detail::wait_barrier(empty_bar(stage), phase ^ 1u, ctl,
                                                              kRoleProducer, it);
                        if (!got) {
                            ok = false;
                            break;
                        }
                    }
                    const uint32_t a_dst = ring + static_cast<uint32_t>(stage) * Cfg::kStageBytes;
                    const uint32_t b_dst = a_dst + Cfg::kABytes;
                    {
                        uint32_t bar = full_bar(stage);
                        // (test hook: unit 0 may overstate its first stage, see GemmParams)
                        const uint32_t tx = Cfg::kTxBytes -
                                            static_cast<uint32_t>(Cfg::kBBoxes - b_boxes) * Cfg::kKSub * Cfg::kBoxBytes +
                                            ((p.overstate_first_stage != 0 && it == 0 && unit == 0) ? 16u : 0u);
                        if constexpr (kPair) {
                            if (leader) {
                                ptx::mbar_arrive_expect_tx(bar, tx);
                            }
                            bar = ptx::map_to_cta(bar, 0);  // both CTAs credit the leader's barrier
                        } else {
                            ptx::mbar_arrive_expect_tx(bar, tx);
                        }
#pragma unroll
                        for (int sub = 0; sub < Cfg::kKSub; ++sub) {
                            const int k0 = kb * Cfg::kTileK + sub * 64;
                            const uint32_t a_sub = a_dst + sub * Cfg::kASubBytes;
                            const uint32_t b_sub = b_dst + sub * Cfg::kBSubBytes;
                            if constexpr (kPair) {
                                ptx::tma_load_2d_pair_hint(a_sub, &tmap_a, bar, k0, a_row, hint_a);
                            } else {
                                ptx::tma_load_2d_hint(a_sub, &tmap_a, bar, k0, a_row, hint_a);
                            }
#pragma unroll
                            for (int j = 0; j < Cfg::kBBoxes; ++j) {
                                if (j >= b_boxes) {
                                    break;  // narrow tile: columns 128-255 of the stage stay unused
                                }
                                // wide tile: boxes 0,1 belong to columns 0-255 of the tile,
                                // boxes 2,3 to columns 256-511 (this CTA's 128 of each)
                                const int box_col =
                                    kWide ? b_col + (j >> 1) * 256 + (j & 1) * 64 : b_col + j * 64;
                                if constexpr (kPair) {
                                    ptx::tma_load_2d_pair_hint(b_sub + j * Cfg::kBoxBytes, &tmap_b, bar,
                                                               box_col, k0, hint_b);
                                } else {
                                    ptx::tma_load_2d_hint(b_sub + j * Cfg::kBoxBytes, &tmap_b, bar,
                                                          box_col, k0, hint_b);
                                }
                            }
                        }
                    }
                    if constexpr (kWide) {
                        // Wide tile: the epilogue sits between two tiles, so its C_in must
                        // not come from DRAM.  While the last k blocks of the tile stream
                        // in, pull this CTA's 128 x 512 block of C into L2, four boxes
                        // (32 rows x 128 B each) per k block.
                        constexpr int kBoxCols = 128 / static_cast<int>(sizeof(OutT));
                        constexpr int kBoxesPerRowGroup = Cfg::kTileN / kBoxCols;
                        constexpr int kBoxes = 4 * kBoxesPerRowGroup;
                        constexpr int kLead = kBoxes / 4 + 4;  // k blocks before the end
                        const int left = seg.kb_end - kb;
                        if (p.c_tma && p.beta != 0.0f && p.epi_mode == kEpiLinear && seg.slot < 0 &&
                            left <= kLead && left > 4) {
                            const int first = (kLead - left) * 4;
#pragma unroll
                            for (int q = 0; q < 4; ++q) {
                                const int box = first + q;
                                const int r0 = a_row + (box / kBoxesPerRowGroup) * 32;
                                const int c0 = tn * Cfg::kTileN + (box % kBoxesPerRowGroup) * kBoxCols;
                                if (r0 < p.m && c0 < p.n) {
                                    ptx::tma_prefetch_l2_2d(&tmap_c, c0, r0);
                                }
                            }
                        }
                    }
                    ++it;
                    if (++stage == kStages) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
            }
            // Tail: do not leave while the consumer may still signal this CTA's
            // empty barriers or copies into this CTA's ring are in flight.
            const uint32_t first = it > static_cast<uint32_t>(kStages) ? it - kStages : 0u;
            for (uint32_t i = first; i < it; ++i) {
                const int s = static_cast<int>(i % kStages);
                const uint32_t use = i / kStages;
                if (ok) {
                    if (!detail::wait_barrier(empty_bar(s), use & 1u, ctl, kRoleDrain, i)) {
                        ok = false;
                    }
                }
                if (!ok) {
                    // Aborting: only make sure our own copies have landed.
                    if (!kPair || leader) {
                        detail::drain_wait(full_bar(s), use & 1u);
                    } else {
                        __nanosleep(20000);
                    }
                }
            }
        }
    } else if (warp == 1) {
        if (leader && ptx::elect_one_sync()) {
            // MMA issuer.
            SegmentCursor cur = make_cursor(sched, unit);
            Segment seg;
            uint32_t it = 0;
            int stage = 0;
            uint32_t phase = 0;
            uint32_t seg_count = 0;
            bool ok = true;
            while (ok && next_segment(sched, &cur, &seg)) {
                // Two accumulators, used alternately (kAccStages == 2), or one accumulator
                // of two 256-column halves that the epilogue hands back one by one.
                const uint32_t acc = kWide ? 0u : (seg_count & 1u);
                const uint32_t acc_parity = kWide ? (seg_count & 1u) : ((seg_count >> 1) & 1u);
                {
                    bool got = detail::wait_barrier(acc_empty_bar(static_cast<int>(acc)),
                                                    acc_parity ^ 1u, ctl, kRoleMma,
                                                    0x80000000u | seg_count);
                    if (kWide && got) {
                        got = detail::wait_barrier(acc_empty_bar(1), acc_parity ^ 1u, ctl, kRoleMma,
                                                   0x90000000u | seg_count);
                    }
                    if (!got) {
                        ok = false;
                        break;
                    }
                }
                ptx::tc_fence_after_sync();
                const uint32_t d_tmem = tmem_base + acc * 256u;
                // The barrier of the NEXT stage is probed between the MMAs of the current
                // one, so that its latency hides behind tensor-core work and the next
                // k block can be issued back to back.
                bool ready = false;
                for (int kb = seg.kb_begin; kb < seg.kb_end; ++kb) {
                    if (!ready) {
                        const bool got = detail::wait_barrier(full_bar(stage), phase, ctl, kRoleMma, it);
                        if (!got) {
                            ok = false;
                            break;
                        }
                    }
                    const uint32_t a_src = ring + static_cast<uint32_t>(stage) * Cfg::kStageBytes;
                    const uint32_t b_src = a_src + Cfg::kABytes;
                    // A: K-major, 8-row groups 1024 B apart.  B: N-major, 64-column
                    // boxes 8192 B apart (leading), 8-k-row groups 1024 B apart (stride).
                    const uint64_t a_desc = ptx::make_smem_desc_sw128(a_src, 16, 1024);
                    const uint64_t b_desc = ptx::make_smem_desc_sw128(b_src, Cfg::kBoxBytes, 1024);
                    int next_stage = stage + 1;
                    uint32_t next_phase = phase;
                    if (next_stage == kStages) {
                        next_stage = 0;
                        next_phase ^= 1u;
                    }
                    ready = false;
#pragma unroll
                    for (int j = 0; j < 4 * Cfg::kKSub; ++j) {
                        // 16 k elements per instruction: +32 B along a K-major row of A,
                        // +16 k-rows (2048 B) of B; descriptor addresses count 16 B.  Every
                        // fourth instruction moves on to the next 64-k sub-block of the stage.
                        const uint64_t a_off = static_cast<uint64_t>(
                            ((j >> 2) * Cfg::kASubBytes + (j & 3) * 32) >> 4);
                        const uint32_t accumulate = (kb > seg.kb_begin || j > 0) ? 1u : 0u;
#pragma unroll
                        for (int h = 0; h < Cfg::kNHalves; ++h) {
                            // wide tile: the same A rows against the two 256-column halves of B
                            const uint64_t b_off = static_cast<uint64_t>(
                                ((j >> 2) * Cfg::kBSubBytes + h * 2 * Cfg::kBoxBytes + (j & 3) * 2048) >> 4);
                            if constexpr (kPair) {
                                ptx::umma_f16_pair(d_tmem + h * 256u, a_desc + a_off, b_desc + b_off,
                                                   p.idesc, accumulate);
                            } else {
                                ptx::umma_f16(d_tmem + h * 256u, a_desc + a_off, b_desc + b_off,
                                              p.idesc, accumulate);
                            }
                        }
                        if (j == 0 && kb + 1 < seg.kb_end) {
                            ready = ptx::mbar_try_wait(full_bar(next_stage), next_phase);
                        }
                    }
                    if constexpr (kPair) {
                        ptx::umma_commit_pair(empty_bar(stage));
                        ptx::umma_commit_pair(ptx::map_to_cta(empty_bar(stage), 1));
                    } else {
                        ptx::umma_commit(empty_bar(stage));
                    }
                    ++it;
                    stage = next_stage;
                    phase = next_phase;
                }
                if (ok) {
                    if constexpr (kPair) {
                        ptx::umma_commit_pair(acc_full_bar(acc));
                        ptx::umma_commit_pair(ptx::map_to_cta(acc_full_bar(acc), 1));
                    } else {
                        ptx::umma_commit(acc_full_bar(acc));
                    }
                    ++seg_count;
                }
            }
            if (ok) {
                // Tail: the epilogue (of both CTAs) must have drained the last
                // accumulators before TMEM can go.
                if constexpr (kWide) {
                    if (seg_count > 0) {
                        const uint32_t i = seg_count - 1u;
                        ok = detail::wait_barrier(acc_empty_bar(0), i & 1u, ctl, kRoleDrain,
                                                  0x80000000u | i) &&
                             detail::wait_barrier(acc_empty_bar(1), i & 1u, ctl, kRoleDrain,
                                                  0x90000000u | i);
                    }
                } else {
                    const uint32_t first = seg_count > 2u ? seg_count - 2u : 0u;
                    for (uint32_t i = first; i < seg_count && ok; ++i) {
                        ok = detail::wait_barrier(acc_empty_bar(i & 1u), (i >> 1) & 1u, ctl,
                                                  kRoleDrain, 0x80000000u | i);
                    }
                }
            } else {
                // Aborting: wait (bounded) until the MMAs already issued have retired.
                if constexpr (kPair) {
                    ptx::umma_commit_pair(drain_bar);
                } else {
                    ptx::umma_commit(drain_bar);
                }
                detail::drain_wait(drain_bar, 0);
            }
        }
    } else {
        // Epilogue warps 2..; TMEM lane quarter = warp id mod 4.  With the wide tile, warps
        // 2-5 drain columns 0-255 of the accumulator and warps 6-9 columns 256-511.
        const uint32_t quad = static_cast<uint32_t>(warp) & 3u;
        const int ew = warp - 2;  // staging slice of this warp
        const uint32_t half = kWide ? static_cast<uint32_t>(ew >> 2) : 0u;
        SegmentCursor cur = make_cursor(sched, unit);
        Segment seg;
        uint32_t seg_count = 0;
        OutT* c_base = static_cast<OutT*>(p.c);
        const bool vec_ok = p.c_vec != 0;
        // TMA epilogue state: two 4 KB staging buffers (32 rows x 128 B, 128-byte
        // swizzle), one C_in barrier each; bit b of cin_parity = next phase to wait for.
        constexpr int kChunkCols = 128 / static_cast<int>(sizeof(OutT));
        constexpr int kChunks = 256 / kChunkCols;  // a warp always drains 256 columns
        constexpr int kUnitElems = 16 / static_cast<int>(sizeof(OutT));
        const uint32_t stg = staging + static_cast<uint32_t>(ew) * 8192u;
        uint8_t* stg_ptr = staging_ptr + ew * 8192;
        uint32_t cin_parity = 0;
        uint32_t cin_pending = 0;  // lane 0: loads issued and not yet waited for
        const bool reads_c = (p.epi_mode == kEpiLinear) && (p.beta != 0.0f);
        const bool unit_alpha = p.alpha == 1.0f;
        bool alive = true;
        while (alive && next_segment(sched, &cur, &seg)) {
            const uint32_t acc = kWide ? 0u : (seg_count & 1u);
            const uint32_t acc_parity = kWide ? (seg_count & 1u) : ((seg_count >> 1) & 1u);
            const uint32_t acc_cols = kWide ? half * 256u : acc * 256u;  // TMEM column offset
            int tm, tn;
            tile_coords(sched, seg.tile, &tm, &tn);
            const int row_in_tile = (kPair ? static_cast<int>(rank) * 128 : 0) +
                                    static_cast<int>(quad) * 32 + static_cast<int>(lane);
            const int row = tm * Cfg::kTileM + row_in_tile;
            const int row0 = row - static_cast<int>(lane);  // first row of this warp
            const int col_base = tn * tile_n + static_cast<int>(half) * 256;
            const uint32_t t_row = tmem_base + ((quad * 32u) << 16) + acc_cols;
            // A split tile is finished either by the separate fix-up pass (every unit parks its
            // partial) or, fused, by the unit that holds the tile's first k blocks: that unit
            // runs them last, so the others' partials are already in the workspace.
            const bool fused = p.sk_flags != nullptr;
            const bool owner = fused && seg.slot >= 0 && seg.kb_begin == 0;
            const bool parks = seg.slot >= 0 && !owner;
            const bool tma_path = (p.c_tma != 0) && !parks;
            const bool warp_has_rows = row0 < p.m;
            const int group = row_in_tile >> 5;  // 32-row group of the tile this warp drains
            const size_t slot_part = static_cast<size_t>(group * Cfg::kNHalves + static_cast<int>(half)) * 8192u +
                                     lane * 4u;  // this lane's offset inside any slot
            // The other holders of an owned tile are the next units, each with its first slot.
            int peers = 0;
            if (owner) {
                const long long tile_end =
                    static_cast<long long>(seg.tile - sched.dp_tiles + 1) * sched.k_blocks;
                while (unit + 1 + peers < sched.units &&
                       sk_range_begin(sched, unit + 1 + peers) < tile_end) {
                    ++peers;
                }
            }
            // Adds the peers' partials of one 32-column chunk, in ascending unit order.
            auto add_partials = [&](int chunk32, uint32_t* r) {
                for (int v = 0; v < peers; ++v) {
                    const float* src = p.workspace +
                                       static_cast<size_t>(2 * (unit + 1 + v)) * Cfg::kSlotFloats +
                                       slot_part + chunk32 * 1024;
#pragma unroll
                    for (int q = 0; q < 8; ++q) {
                        const float4 t = __ldcg(reinterpret_cast<const float4*>(src + q * 128));
                        r[4 * q + 0] = __float_as_uint(__uint_as_float(r[4 * q + 0]) + t.x);
                        r[4 * q + 1] = __float_as_uint(__uint_as_float(r[4 * q + 1]) + t.y);
                        r[4 * q + 2] = __float_as_uint(__uint_as_float(r[4 * q + 2]) + t.z);
                        r[4 * q + 3] = __float_as_uint(__uint_as_float(r[4 * q + 3]) + t.w);
                    }
                }
            };

            // Hands the accumulator back to the MMA warp, once per tile: called as soon as
            // the last TMEM load of the tile has completed.
            bool released = false;
            auto release_acc = [&]() {
                if (released) {
                    return;
                }
                released = true;
                ptx::tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) {
                    const int release = static_cast<int>(kWide ? half : acc);
                    if constexpr (kPair) {
                        ptx::mbar_arrive_cluster(ptx::map_to_cta(acc_empty_bar(release), 0));
                    } else {
                        ptx::mbar_arrive(acc_empty_bar(release));
                    }
                }
            };

            // Chunks of kChunkCols columns this warp writes through the TMA path.
            const int cols_left = min(p.n - col_base, tile_n);  // columns of this tile this warp drains
            const int n_chunks =
                !tma_path || !warp_has_rows || cols_left <= 0
                    ? 0
                    : (cols_left >= 256 ? kChunks : (cols_left + kChunkCols - 1) / kChunkCols);
            // C_in of the first two chunks is fetched before the accumulator is ready: both
            // staging buffers are idle until then.
            if (reads_c && lane == 0) {
                for (int c = 0; c < 2 && c < n_chunks; ++c) {
                    ptx::mbar_arrive_expect_tx(cin_bar(ew, c), 4096);
                    ptx::tma_load_2d(stg + static_cast<uint32_t>(c) * 4096u, &tmap_c, cin_bar(ew, c),
                                     col_base + c * kChunkCols, row0);
                    cin_pending |= 1u << c;
                }
            }

            int ok = 1;
            if (lane == 0) {
                ok = detail::wait_barrier(acc_full_bar(static_cast<int>(acc)), acc_parity, ctl,
                                          kRoleEpilogue, seg_count)
                         ? 1
                         : 0;
            }
            ok = __shfl_sync(0xFFFFFFFFu, ok, 0);
            if (!ok) {
                break;
            }
            // Every lane observes the completed phase itself (acquire); it cannot
            // advance again before this warp releases the accumulator below.
            for (int i = 0;
                 i < 1024 && !ptx::mbar_try_wait(acc_full_bar(static_cast<int>(acc)), acc_parity); ++i) {
            }
            ptx::tc_fence_after_sync();

            if (peers > 0) {
                // Wait (bounded) until every peer's warp of the same rows and columns has parked
                // its partial.  Each lane then reads the flags itself, so that its loads of the
                // partials are ordered after the writers' release.
                int got = 1;
                if (lane == 0) {
                    for (int v = 0; v < peers && got; ++v) {
                        const unsigned int* flag =
                            p.sk_flags + static_cast<size_t>(2 * (unit + 1 + v)) * 16 + group * 2 + half;
                        got = detail::wait_flag(flag, p.sk_epoch + p.sk_flag_skew, ctl, kRoleEpilogue,
                                                0x50000000u | static_cast<unsigned int>(unit + 1 + v))
                                  ? 1
                                  : 0;
                    }
                }
                got = __shfl_sync(0xFFFFFFFFu, got, 0);
                if (!got) {
                    break;
                }
                for (int v = 0; v < peers; ++v) {
                    const unsigned int* flag =
                        p.sk_flags + static_cast<size_t>(2 * (unit + 1 + v)) * 16 + group * 2 + half;
                    for (int i = 0; i < 1024 && ptx::ld_acquire_gpu(flag) != p.sk_epoch + p.sk_flag_skew; ++i) {
                    }
                }
            }

            if (parks) {
                // Partial accumulator -> FP32 workspace slot, whole tile, no predication.  The
                // slot is not row-major: it is the image of the registers, laid out as
                // [32-row group][256-column half][32-column chunk][4-column unit][lane][4],
                // so every store (and every load of the fix-up pass, which uses the same
                // lane = row mapping) moves 512 contiguous bytes per warp.
                float* dst = p.workspace + static_cast<size_t>(seg.slot) * Cfg::kSlotFloats + slot_part;
                const int park_chunks = min(256, tile_n) / 32;  // a narrow tile has 4 chunks, not 8
#pragma unroll 1
                for (int c = 0; c < park_chunks; ++c) {
                    uint32_t r[32];
                    ptx::tmem_ld_32x32(t_row + static_cast<uint32_t>(c * 32), r);
                    ptx::tmem_ld_wait();
#pragma unroll
                    for (int q = 0; q < 8; ++q) {
                        *reinterpret_cast<uint4*>(dst + c * 1024 + q * 128) =
                            make_uint4(r[4 * q], r[4 * q + 1], r[4 * q + 2], r[4 * q + 3]);
                    }
                }
                if (fused) {
                    // publish: this warp's part of the slot is complete
                    __threadfence();
                    __syncwarp();
                    if (lane == 0) {
                        ptx::st_release_gpu(
                            p.sk_flags + static_cast<size_t>(seg.slot) * 16 + group * 2 + half, p.sk_epoch);
                    }
                }
            } else if (tma_path) {
                // Coalesced path: registers -> swizzled staging -> TMA store; C_in arrives by
                // TMA load into the same buffer.  The accumulator goes back to the MMA warp as
                // soon as its last columns are in registers.
                auto load_acc = [&](int c, uint32_t (&dst)[kChunkCols]) {
#pragma unroll
                    for (int h = 0; h < kChunkCols / 32; ++h) {
                        ptx::tmem_ld_32x32(t_row + static_cast<uint32_t>(c * kChunkCols + h * 32),
                                           *reinterpret_cast<uint32_t(*)[32]>(dst + h * 32));
                    }
                };
                // One chunk: `r` holds its accumulator columns (already waited for).
                auto finish_chunk = [&](int c, uint32_t (&r)[kChunkCols]) -> bool {
                    const int col = col_base + c * kChunkCols;
                    const uint32_t b = static_cast<uint32_t>(c) & 1u;
                    if (!reads_c) {
                        // buffer b was the source of the store two chunks ago
                        if (lane == 0) {
                            ptx::bulk_wait_group_read<1>();
                        }
                        __syncwarp();
                    } else {
                        int got = 1;
                        if (lane == 0) {
                            got = detail::wait_barrier(cin_bar(ew, b), (cin_parity >> b) & 1u, ctl,
                                                       kRoleEpilogue, 0x40000000u | seg_count)
                                      ? 1
                                      : 0;
                            cin_pending &= ~(1u << b);
                        }
                        got = __shfl_sync(0xFFFFFFFFu, got, 0);
                        if (!got) {
                            return false;
                        }
                        for (int i = 0;
                             i < 1024 && !ptx::mbar_try_wait(cin_bar(ew, b), (cin_parity >> b) & 1u); ++i) {
                        }
                        cin_parity ^= 1u << b;
                    }
                    if (reads_c && c >= 1 && c + 1 < n_chunks && lane == 0) {
                        // Buffer b^1 was the source of the previous chunk's store; once that
                        // store has read it, the C_in of the next chunk can land there.
                        ptx::bulk_wait_group_read<0>();
                        ptx::mbar_arrive_expect_tx(cin_bar(ew, b ^ 1u), 4096);
                        ptx::tma_load_2d(stg + (b ^ 1u) * 4096u, &tmap_c, cin_bar(ew, b ^ 1u),
                                         col + kChunkCols, row0);
                        cin_pending |= 1u << (b ^ 1u);
                    }
                    uint8_t* row_smem = stg_ptr + b * 4096u + lane * 128u;
                    // All eight 16-byte units of C_in are read before any result is written
                    // back: reads and writes share the buffer, and interleaving them would
                    // chain every unit behind the previous unit's store.
                    uint4 cin_u[8];
                    if (reads_c) {
#pragma unroll
                        for (int j = 0; j < 8; ++j) {
                            cin_u[j] = *reinterpret_cast<const uint4*>(
                                row_smem + ((static_cast<uint32_t>(j) ^ (lane & 7u)) << 4));
                        }
                    }
                    // One straight-line loop per epilogue flavour: a flavour test inside the
                    // loop would cut it into eight blocks the compiler cannot overlap.
                    auto emit = [&](auto&& value_of) {
#pragma unroll
                        for (int j = 0; j < 8; ++j) {
                            float out[kUnitElems];
#pragma unroll
                            for (int e = 0; e < kUnitElems; ++e) {
                                out[e] = value_of(j, e);
                            }
                            detail::OutTraits<OutT>::store_vec(
                                reinterpret_cast<OutT*>(
                                    row_smem + ((static_cast<uint32_t>(j) ^ (lane & 7u)) << 4)),
                                out);
                        }
                    };
                    auto acc_of = [&](int j, int e) { return __uint_as_float(r[j * kUnitElems + e]); };
                    auto cin = [&](int j, int e) {
                        return detail::OutTraits<OutT>::element(cin_u[j], e);
                    };
                    if (p.epi_mode == kEpiBiasRelu) {
                        emit([&](int j, int e) {
                            const int gc = col + j * kUnitElems + e;
                            const float bv = gc < p.n ? __ldg(p.bias + gc) : 0.0f;
                            return fmaxf(p.alpha * acc_of(j, e) + bv, 0.0f);
                        });
                    } else if (reads_c) {
                        if (unit_alpha) {
                            // alpha == 1 (the common case) needs no multiply; the product
                            // alpha*acc is exact then, so the results are the same
                            emit([&](int j, int e) { return fmaf(p.beta, cin(j, e), acc_of(j, e)); });
                        } else {
                            emit([&](int j, int e) {
                                return fmaf(p.beta, cin(j, e), p.alpha * acc_of(j, e));
                            });
                        }
                    } else if (unit_alpha) {
                        emit([&](int j, int e) { return acc_of(j, e); });
                    } else {
                        emit([&](int j, int e) { return p.alpha * acc_of(j, e); });
                    }
                    ptx::fence_proxy_async_smem();
                    __syncwarp();
                    if (lane == 0) {
                        ptx::tma_store_2d(&tmap_c, stg + b * 4096u, col, row0);
                        ptx::bulk_commit_group();
                    }
                    return true;
                };
#pragma unroll 1
                for (int c = 0; c < n_chunks && alive; ++c) {
                    uint32_t r[kChunkCols];
                    load_acc(c, r);
                    ptx::tmem_ld_wait();
                    if (c + 1 == n_chunks) {
                        release_acc();  // the last columns are in registers
                    }
                    if (peers > 0) {
#pragma unroll
                        for (int h = 0; h < kChunkCols / 32; ++h) {
                            add_partials(c * (kChunkCols / 32) + h, r + h * 32);
                        }
                    }
                    alive = finish_chunk(c, r);
                }
                if (!alive) {
                    break;
                }
            } else {
                OutT* row_ptr = c_base + static_cast<size_t>(row) * static_cast<size_t>(p.ldc);
                const bool row_ok = row < p.m;
#pragma unroll 1
                for (int c = 0; c < 256 / 32; ++c) {
                    if (col_base + c * 32 >= p.n || c * 32 >= tile_n) {
                        break;  // uniform across the warp
                    }
                    uint32_t r[32];
                    ptx::tmem_ld_32x32(t_row + static_cast<uint32_t>(c * 32), r);
                    ptx::tmem_ld_wait();
                    if (peers > 0) {
                        add_partials(c, r);
                    }
                    if (row_ok) {
                        float acc_f[32];
#pragma unroll
                        for (int e = 0; e < 32; ++e) {
                            acc_f[e] = __uint_as_float(r[e]);
                        }
                        detail::finish_row_chunk<OutT>(acc_f, row_ptr, col_base + c * 32, p.n,
                                                       p.alpha, p.beta, p.bias, p.epi_mode, vec_ok);
                    }
                }
            }
            // All TMEM reads of this accumulator are done: hand it back to the MMA warp.
            release_acc();
            if (lane == 0 && tma_path) {
                ptx::bulk_wait_group_read<0>();  // staging is reusable by the next tile
            }
            __syncwarp();
            ++seg_count;
        }
        if (lane == 0) {
            // Leaving: no store may still read staging, no C_in copy may still write it.
            ptx::bulk_wait_group_read<0>();
            for (uint32_t b = 0; b < 2; ++b) {
                if (cin_pending & (1u << b)) {
                    detail::drain_wait(cin_bar(ew, static_cast<int>(b)), (cin_parity >> b) & 1u);
                }
            }
        }
    }

    // ---- common exit ----------------------------------------------------------
    ptx::tc_fence_before_sync();
    if constexpr (kPair) {
        __syncthreads();
        ptx::cluster_arrive_release();
        ptx::cluster_wait_acquire();
    } else {
        __syncthreads();
    }
    if (warp == 1) {
        ptx::tc_fence_after_sync();
        if constexpr (kPair) {
            ptx::tmem_dealloc_pair(tmem_base, 512);
        } else {
            ptx::tmem_dealloc(tmem_base, 512);
        }
    }
}

// Fix-up pass of the stream-K split.  Block (t, g) finishes 32 rows x 256 columns of split
// tile t (g = row group * halves + half): it adds the FP32 partial tiles in ascending unit
// order (so the result does not depend on timing) and applies the epilogue.  Tiles that a
// single unit covered whole were already written by the GEMM kernel and are skipped.  The
// partial slots hold the register image written by the GEMM epilogue: warp w of the block
// takes 32-column chunk w, lane = row, and every load is 512 contiguous bytes per warp.
template <int kTileM, int kTileN, typename OutT>
__global__ void __launch_bounds__(256)
streamk_fixup_kernel(const GemmParams p) {
    constexpr size_t kSlotFloats = static_cast<size_t>(kTileM) * kTileN;
    constexpr int kNHalves = kTileN / 256;
    const Schedule& s = p.sched;
    const int sk_tile = static_cast<int>(blockIdx.x);
    const int gh = static_cast<int>(blockIdx.y);  // group * kNHalves + half

    __shared__ int slots[kMaxFixupSlots];
    __shared__ int n_slots;
    if (threadIdx.x == 0) {
        n_slots = fixup_slots(s, sk_tile, slots, kMaxFixupSlots);
    }
    __syncthreads();
    const int count = n_slots;
    if (count == 0) {
        return;
    }
    int tm, tn;
    tile_coords(s, s.dp_tiles + sk_tile, &tm, &tn);
    const int lane = static_cast<int>(threadIdx.x) & 31;
    const int chunk = static_cast<int>(threadIdx.x) >> 5;  // 8 warps = 8 chunks of 32 columns
    const int row = tm * kTileM + (gh / kNHalves) * 32 + lane;
    const int tile_n = (kTileM == 128 && kTileN == 256 && p.tile_n == 128) ? 128 : kTileN;  // narrow single-CTA tile
    const int col0 = tn * tile_n + (gh % kNHalves) * 256 + chunk * 32;
    if (col0 >= p.n || chunk * 32 >= tile_n) {
        return;  // uniform per warp
    }
    const float* base = p.workspace + static_cast<size_t>(gh) * 8192u + chunk * 1024 + lane * 4;
    float acc[32];
#pragma unroll
    for (int e = 0; e < 32; ++e) {
        acc[e] = 0.0f;
    }
    for (int i = 0; i < count; ++i) {
        const float* src = base + static_cast<size_t>(slots[i]) * kSlotFloats;
        float4 v[8];
#pragma unroll
        for (int q = 0; q < 8; ++q) {
            v[q] = __ldcg(reinterpret_cast<const float4*>(src + q * 128));
        }
#pragma unroll
        for (int q = 0; q < 8; ++q) {
            acc[4 * q] += v[q].x;
            acc[4 * q + 1] += v[q].y;
            acc[4 * q + 2] += v[q].z;
            acc[4 * q + 3] += v[q].w;
        }
    }
    if (row < p.m) {
        OutT* row_ptr = static_cast<OutT*>(p.c) + static_cast<size_t>(row) * static_cast<size_t>(p.ldc);
        detail::finish_row_chunk<OutT>(acc, row_ptr, col0, p.n, p.alpha, p.beta, p.bias, p.epi_mode,
                                       p.c_vec != 0);
    }
}

}  // namespace ckl
