// Inline-PTX wrappers for the sm_100a features the GEMM kernels use: mbarrier,
// TMA bulk-tensor loads, tensor memory (TMEM) management, tcgen05.mma and
// tcgen05.ld.  Everything here is a thin, single-instruction wrapper; the
// protocol (who waits on what) lives in gemm_umma.cuh.
#pragma once

#include <cstdint>

#include <cuda.h>
#include <cuda_runtime.h>

namespace ckl::ptx {

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ uint32_t lane_id() {
    uint32_t v;
    asm volatile("mov.u32 %0, %%laneid;" : "=r"(v));
    return v;
}

__device__ __forceinline__ uint64_t global_timer_ns() {
    uint64_t v;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(v));
    return v;
}

__device__ __forceinline__ uint32_t cluster_cta_rank() {
    uint32_t v;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(v));
    return v;
}

// ---- mbarrier ---------------------------------------------------------------

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}

// Makes barrier initialisation visible to the async proxy (TMA, tcgen05) and,
// in a cluster, to the peer CTA.
__device__ __forceinline__ void fence_barrier_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

// Programmatic dependent launch.  launch_dependents: the next kernel of the stream, if it was
// launched as a programmatic dependent, may be scheduled once every CTA of this grid has said
// so (or exited).  grid_dependency_wait: returns when the kernels this one depends on have
// completed and their memory is visible; a no-op for an ordinary launch.
__device__ __forceinline__ void launch_dependents() {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
__device__ __forceinline__ void grid_dependency_wait() {
    asm volatile("griddepcontrol.wait;" ::: "memory");
}

// Flag words in global memory that one CTA publishes and another polls.
__device__ __forceinline__ unsigned int ld_acquire_gpu(const unsigned int* p) {
    unsigned int v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_gpu(unsigned int* p, unsigned int v) {
    asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

__device__ __forceinline__ void fence_proxy_async_smem() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

// Arrive on a barrier that may live in the peer CTA of the cluster (address in
// the shared::cluster window, from mapa).
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_bar) {
#if defined(CKL_ARRIVE_CLUSTER_RELEASE)
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_bar)
                 : "memory");
#else
    // Default semantics (release at CTA scope).  The arrivals made with this publish no
    // ordinary memory: a drained accumulator is ordered by tcgen05.fence, so the far more
    // expensive cluster-scope release is not needed.
    asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_bar) : "memory");
#endif
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
                 : "memory");
}

// One bounded-time probe of a barrier phase; true once the phase with the
// given parity has completed.
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t done;
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t"
        "}"
        : "=r"(done)
        : "r"(bar), "r"(parity)
        : "memory");
    return done != 0;
}

// Same probe, but the hardware may park the thread for up to `hint_ns` while
// the phase is incomplete (it resumes at once when the phase completes), so a
// long wait costs a handful of instructions instead of a busy spin.
__device__ __forceinline__ bool mbar_try_wait_parked(uint32_t bar, uint32_t parity,
                                                     uint32_t hint_ns) {
    uint32_t done;
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t"
        "}"
        : "=r"(done)
        : "r"(bar), "r"(parity), "r"(hint_ns)
        : "memory");
    return done != 0;
}

// One lane of a fully converged warp (all 32 lanes must execute this).  Unlike a test of the
// lane index, this tells the compiler that exactly one thread follows; the role loops behind
// it (TMA, tcgen05.mma, commits) then execute 13-19 % fewer warp instructions per launch on
// the CTA-pair kernels (measured at 8192^3), at unchanged speed.
__device__ __forceinline__ bool elect_one_sync() {
    uint32_t chosen;
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "elect.sync _|p, 0xFFFFFFFF;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t"
        "}"
        : "=r"(chosen)
        :
        : "memory");
    return chosen != 0;
}

// Address of the same shared-memory offset in another CTA of the cluster.
__device__ __forceinline__ uint32_t map_to_cta(uint32_t smem_addr, uint32_t cta_rank) {
    uint32_t out;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(out) : "r"(smem_addr), "r"(cta_rank));
    return out;
}

__device__ __forceinline__ void cluster_arrive_release() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
}
__device__ __forceinline__ void cluster_wait_acquire() {
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// ---- TMA --------------------------------------------------------------------

__device__ __forceinline__ void prefetch_tensormap(const CUtensorMap* map) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}

// 2-D tiled load, global -> this CTA's shared memory; completion is counted in
// bytes on `bar`.  x is the innermost (contiguous) coordinate and must be a
// multiple of 8 elements for 16-bit types (16-byte rule); callers only pass
// multiples of 64.
__device__ __forceinline__ void tma_load_2d(uint32_t smem_dst, const CUtensorMap* map, uint32_t bar,
                                            int32_t x, int32_t y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%3, %4}], [%2];"
        :
        : "r"(smem_dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(x), "r"(y)
        : "memory");
}

// L2 eviction-priority hints for TMA loads (the 64-bit policy words that
// createpolicy.fractional.L2::evict_{first,last} with fraction 1.0 produce).
constexpr uint64_t kL2EvictNormal = 0x1000000000000000ull;
constexpr uint64_t kL2EvictFirst = 0x12F0000000000000ull;
constexpr uint64_t kL2EvictLast = 0x14F0000000000000ull;

__device__ __forceinline__ void tma_load_2d_hint(uint32_t smem_dst, const CUtensorMap* map,
                                                 uint32_t bar, int32_t x, int32_t y, uint64_t hint) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint"
        " [%0], [%1, {%3, %4}], [%2], %5;"
        :
        : "r"(smem_dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(x), "r"(y), "l"(hint)
        : "memory");
}
__device__ __forceinline__ void tma_load_2d_pair_hint(uint32_t smem_dst, const CUtensorMap* map,
                                                      uint32_t cluster_bar, int32_t x, int32_t y,
                                                      uint64_t hint) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
        ".L2::cache_hint [%0], [%1, {%3, %4}], [%2], %5;"
        :
        : "r"(smem_dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(cluster_bar), "r"(x), "r"(y),
          "l"(hint)
        : "memory");
}

// Same load issued from either CTA of a pair, with the completion bytes
// credited to a barrier that may live in the pair's leader CTA (`bar` is a
// shared::cluster address).  Unicast: each CTA fetches only its own tile.
__device__ __forceinline__ void tma_load_2d_pair(uint32_t smem_dst, const CUtensorMap* map,
                                                 uint32_t cluster_bar, int32_t x, int32_t y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%3, %4}], [%2];"
        :
        : "r"(smem_dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(cluster_bar), "r"(x), "r"(y)
        : "memory");
}

// 2-D tiled store, this CTA's shared memory -> global, tracked by the thread's
// bulk async-group (commit, then wait_group.read before reusing the source).
// Coordinates outside the tensor are clipped; x obeys the same 16-byte rule.
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, uint32_t smem_src, int32_t x,
                                             int32_t y) {
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
                 :
                 : "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_src), "r"(x), "r"(y)
                 : "memory");
}
// Pulls one box of a tensor into L2 only (no shared-memory destination, no completion
// to wait for); x obeys the 16-byte rule.
__device__ __forceinline__ void tma_prefetch_l2_2d(const CUtensorMap* map, int32_t x, int32_t y) {
    asm volatile("cp.async.bulk.prefetch.tensor.2d.L2.global.tile [%0, {%1, %2}];"
                 :
                 : "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y)
                 : "memory");
}
__device__ __forceinline__ void bulk_commit_group() {
    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
// Waits until at most N of this thread's committed bulk groups still READ their
// shared-memory source (the global writes may still be in flight).
template <int N>
__device__ __forceinline__ void bulk_wait_group_read() {
    asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}

// ---- tensor memory ----------------------------------------------------------

// Whole-warp: allocate `cols` (power of two >= 32) TMEM columns; the base
// address is written to shared memory at `smem_dst`.
__device__ __forceinline__ void tmem_alloc(uint32_t smem_dst, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst),
                 "r"(cols)
                 : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols)
                 : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t smem_dst, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst),
                 "r"(cols)
                 : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols)
                 : "memory");
}

__device__ __forceinline__ void tc_fence_before_sync() {
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after_sync() {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// ---- tcgen05.mma ------------------------------------------------------------

// D[tmem] (+)= A[smem] * B[smem], kind::f16 (FP16 or BF16 inputs, FP32
// accumulate).  Issued by ONE thread.  accumulate == 0 overwrites D.
__device__ __forceinline__ void umma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                         uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
        "}"
        :
        : "r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// CTA-pair form: one instruction drives the tensor cores of both SMs of the
// pair (M = 256 split as 128 rows per CTA, each CTA supplying half of B's N).
__device__ __forceinline__ void umma_f16_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                              uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t"
        "}"
        :
        : "r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// Arrive on `bar` once every tcgen05.mma this thread issued so far has
// completed (implies tcgen05.fence::before_thread_sync).
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                     bar)
                 : "memory");
}
// Pair form; `cluster_bar` may address a barrier in either CTA of the pair.
__device__ __forceinline__ void umma_commit_pair(uint32_t cluster_bar) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                     cluster_bar)
                 : "memory");
}


// ---- tcgen05.ld -------------------------------------------------------------

// Warp-collective: each lane reads 32 consecutive 32-bit columns of its own
// TMEM lane (lane = 32 * (warp_id % 4) + lane_id).
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
          "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
          "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]),
          "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]),
          "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() {
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// ---- descriptors ------------------------------------------------------------

// Shared-memory matrix descriptor (64 bit), 128-byte swizzle, sm_100 version.
//   bits  0-13  start address  >> 4
//   bits 16-29  leading-dimension byte offset >> 4
//   bits 32-45  stride-dimension  byte offset >> 4
//   bits 46-47  descriptor version (1 on sm_100)
//   bits 61-63  layout: 2 = SWIZZLE_128B
__device__ __forceinline__ uint64_t make_smem_desc_sw128(uint32_t smem_addr, uint32_t lbo_bytes,
                                                         uint32_t sbo_bytes) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4);
    d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3FFFu) << 16;
    d |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3FFFu) << 32;
    d |= static_cast<uint64_t>(1) << 46;
    d |= static_cast<uint64_t>(2) << 61;
    return d;
}

// Instruction descriptor for kind::f16 with FP32 accumulation.
//   bits  4-5   D format (1 = F32)
//   bits  7-9   A format (0 = F16, 1 = BF16);  bits 10-12 B format
//   bit  15     A major (0 = K-major);         bit 16  B major (1 = MN-major)
//   bits 17-22  N >> 3;                        bits 24-28  M >> 4
__host__ __device__ constexpr uint32_t make_idesc_f16(uint32_t fmt_ab, uint32_t a_mn_major,
                                                      uint32_t b_mn_major, uint32_t m, uint32_t n) {
    return (1u << 4) | (fmt_ab << 7) | (fmt_ab << 10) | (a_mn_major << 15) | (b_mn_major << 16) |
           ((n >> 3) << 17) | ((m >> 4) << 24);
}

}  // namespace ckl::ptx
