#pragma once
// ckl::gemm_* C++ entry points of the B200 build.
//
// Drop-in for the reference library's include/ckl/gemm.hpp: the tensor-core
// launchers keep their names and signatures (reference lines 68-100) so the
// reference's tests/test_gemm_tensor.cpp and benchmarks/bench_gemm_tensor.cpp
// compile and link against this library without edits.  All of them are thin
// inline shims over the C ABI in ckl_gemm.h and throw std::runtime_error when
// it reports a failure, which is how the reference's checked paths fail
// (include/ckl/cuda_check.hpp:23-30 there).
//
// Storage convention (unchanged): row-major, A m x k (ld k), B k x n (ld n),
// C m x n (ld n), C = alpha * A*B + beta * C, device pointers, work enqueued
// on `stream`.
//
// On this hardware every FP16 "rung" of the reference ladder is the same
// TMA + tcgen05 kernel and every FP32 rung the same CUDA-core kernel; the
// distinct names survive only for source compatibility.  Additions over the reference are grouped at the end:
// 16-bit C, explicit leading dimensions, kernel selection, and the N-sharded forms for several
// GPUs of one box (the reference is single-GPU).

#include <cstddef>
#include <stdexcept>
#include <string>

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "../ckl_gemm.h"

namespace ckl {

enum class GemmVariant {
    kNaive,
    kTiled,
    kRegister,
    kCpAsync,
    kWmmaFp16,
    kWmmaBf16,
    kMmaPtx,
    kCutlass,
    kCublas,
};

// Short lower-case label of a ladder rung (reference: src/gemm/gemm_naive.cu:42-64).
inline const char* gemm_variant_name(GemmVariant v) {
    switch (v) {
        case GemmVariant::kNaive: return "naive";
        case GemmVariant::kTiled: return "tiled";
        case GemmVariant::kRegister: return "register";
        case GemmVariant::kCpAsync: return "cp_async";
        case GemmVariant::kWmmaFp16: return "wmma_fp16";
        case GemmVariant::kWmmaBf16: return "wmma_bf16";
        case GemmVariant::kMmaPtx: return "mma_ptx";
        case GemmVariant::kCutlass: return "cutlass";
        case GemmVariant::kCublas: return "cublas";
    }
    return "unknown";
}

namespace detail {
inline void throw_on_error(int status, const char* who) {
    if (status != CKL_OK) {
        throw std::runtime_error(std::string(who) + ": ckl status " + std::to_string(status) +
                                 ": " + ckl_last_error());
    }
}
}  // namespace detail

// ---- reference signatures: FP32 ladder ------------------------------------------
// The four FP32 rungs (reference lines 40-58) differ only in how the reference stages
// data; here they are one CUDA-core kernel with true FP32 arithmetic (ckl_sgemm), which
// is what their 1e-4 agreement with SGEMM requires.

#define CKL_FP32_RUNG(name)                                                                   \
    inline void name(const float* a, const float* b, float* c, int m, int n, int k, float alpha, \
                     float beta, cudaStream_t stream = nullptr) {                              \
        detail::throw_on_error(ckl_sgemm(a, b, c, m, n, k, k, n, n, alpha, beta, stream), #name); \
    }
CKL_FP32_RUNG(gemm_naive)
CKL_FP32_RUNG(gemm_tiled)
CKL_FP32_RUNG(gemm_register)
CKL_FP32_RUNG(gemm_cp_async)
#undef CKL_FP32_RUNG

// ---- reference signatures: FP16 / BF16 in, FP32 C out ---------------------------

inline void gemm_wmma_fp16(const __half* a, const __half* b, float* c, int m, int n, int k,
                           float alpha, float beta, cudaStream_t stream = nullptr) {
    detail::throw_on_error(ckl_gemm_f16(a, b, c, CKL_F32, m, n, k, k, n, n, alpha, beta, stream),
                           "gemm_wmma_fp16");
}

inline void gemm_wmma_bf16(const __nv_bfloat16* a, const __nv_bfloat16* b, float* c, int m, int n,
                           int k, float alpha, float beta, cudaStream_t stream = nullptr) {
    detail::throw_on_error(ckl_gemm_bf16(a, b, c, CKL_F32, m, n, k, k, n, n, alpha, beta, stream),
                           "gemm_wmma_bf16");
}

inline void gemm_mma_ptx(const __half* a, const __half* b, float* c, int m, int n, int k,
                         float alpha, float beta, cudaStream_t stream = nullptr) {
    detail::throw_on_error(ckl_gemm_f16(a, b, c, CKL_F32, m, n, k, k, n, n, alpha, beta, stream),
                           "gemm_mma_ptx");
}

inline void gemm_mma_ldm(const __half* a, const __half* b, float* c, int m, int n, int k,
                         float alpha, float beta, cudaStream_t stream = nullptr) {
    detail::throw_on_error(ckl_gemm_f16(a, b, c, CKL_F32, m, n, k, k, n, n, alpha, beta, stream),
                           "gemm_mma_ldm");
}

inline void gemm_mma_opt(const __half* a, const __half* b, float* c, int m, int n, int k,
                         float alpha, float beta, cudaStream_t stream = nullptr) {
    detail::throw_on_error(ckl_gemm_f16(a, b, c, CKL_F32, m, n, k, k, n, n, alpha, beta, stream),
                           "gemm_mma_opt");
}

// C = relu(alpha * A*B + bias[col]) in one kernel, and the separate pass
// C = relu(C + bias[col]) it is compared with (reference lines 91-93).  Unlike
// the reference's fused launcher, which silently does nothing for shapes that
// are not multiples of its tile (src/gemm/gemm_mma_opt.cu:230-232), this one
// computes every shape.
inline void gemm_mma_opt_bias(const __half* a, const __half* b, float* c, const float* bias, int m,
                              int n, int k, float alpha, cudaStream_t stream = nullptr) {
    detail::throw_on_error(ckl_gemm_bias_relu_ex(CKL_F16, a, b, c, CKL_F32, bias, m, n, k, k, n, n,
                                                 alpha, CKL_ALGO_AUTO, stream),
                           "gemm_mma_opt_bias");
}

inline void gemm_bias_relu(float* c, const float* bias, int m, int n,
                           cudaStream_t stream = nullptr) {
    detail::throw_on_error(ckl_bias_relu_f32(c, bias, m, n, n, stream), "gemm_bias_relu");
}

// cuBLAS comparators (SGEMM; cublasGemmEx with FP32 C).  Test and benchmark code
// only: they are defined in separate translation units that the shipped library
// does not contain (reference: src/gemm/cublas_gemm.cpp, src/gemm/cublas_gemm_ex.cpp:56-66).
void gemm_cublas(const float* a, const float* b, float* c, int m, int n, int k, float alpha,
                 float beta, cudaStream_t stream = nullptr);
void gemm_cublas_fp16(const __half* a, const __half* b, float* c, int m, int n, int k, float alpha,
                      float beta, cudaStream_t stream = nullptr);
void gemm_cublas_bf16(const __nv_bfloat16* a, const __nv_bfloat16* b, float* c, int m, int n, int k,
                      float alpha, float beta, cudaStream_t stream = nullptr);

// ---- additions ---------------------------------------------------------------------

namespace detail {
inline int dtype_of(const float*) { return CKL_F32; }
inline int dtype_of(const __half*) { return CKL_F16; }
inline int dtype_of(const __nv_bfloat16*) { return CKL_BF16; }
}  // namespace detail

// Any supported combination of 16-bit inputs and FP32 / FP16 / BF16 output,
// explicit leading dimensions (for column blocks of a wider matrix) and an
// optional pinned kernel.
template <typename InT, typename OutT>
inline void gemm_tensor(const InT* a, const InT* b, OutT* c, int m, int n, int k, int lda, int ldb,
                        int ldc, float alpha, float beta, cudaStream_t stream = nullptr,
                        int algo = CKL_ALGO_AUTO) {
    detail::throw_on_error(ckl_gemm_ex(detail::dtype_of(a), a, b, c, detail::dtype_of(c), m, n, k,
                                       lda, ldb, ldc, alpha, beta, algo, stream),
                           "gemm_tensor");
}

template <typename InT, typename OutT>
inline void gemm_tensor(const InT* a, const InT* b, OutT* c, int m, int n, int k, float alpha,
                        float beta, cudaStream_t stream = nullptr) {
    gemm_tensor(a, b, c, m, n, k, k, n, n, alpha, beta, stream, CKL_ALGO_AUTO);
}

// ---- several GPUs of one box: one rank (process or thread) per GPU ----------------
// Rank r of `world` owns the column block ckl_column_shard(n, world, r, 8, ...) of B and C;
// A is replicated.  The communicator is made once per rank with its device current:
// rank 0 calls ckl_comm_get_unique_id and hands the 128 bytes to the others, then every rank
// constructs a ShardedComm.  See ckl_gemm.h for the contracts of the calls wrapped here.

class ShardedComm {
public:
    ShardedComm(int world, int rank, const void* unique_id) {
        detail::throw_on_error(ckl_comm_init(&comm_, world, rank, unique_id), "ShardedComm");
    }
    ~ShardedComm() { ckl_comm_destroy(comm_); }
    ShardedComm(const ShardedComm&) = delete;
    ShardedComm& operator=(const ShardedComm&) = delete;
    ckl_comm* get() const { return comm_; }
    int world() const { return ckl_comm_world(comm_); }
    int rank() const { return ckl_comm_rank(comm_); }

    // A buffer that exists on every rank with every copy mapped everywhere (collective).
    void* alloc_shared(std::size_t bytes) {
        void* p = nullptr;
        detail::throw_on_error(ckl_comm_alloc_shared(comm_, bytes, &p), "alloc_shared");
        return p;
    }
    void free_shared(void* p) { detail::throw_on_error(ckl_comm_free_shared(comm_, p), "free_shared"); }

private:
    ckl_comm* comm_ = nullptr;
};

// Host buffers in, host buffers out: a_rows holds the rows of A that
// ckl_plan_host_sharded(m, world, rank) assigns to this rank, b_shard and c_shard its packed
// column blocks.  Collective.
template <typename InT, typename OutT>
inline void gemm_tensor_host_sharded(ShardedComm& comm, const InT* a_rows, const InT* b_shard,
                                     OutT* c_shard, int m, int n_shard, int k, float alpha,
                                     float beta) {
    detail::throw_on_error(
        ckl_gemm_host_sharded(comm.get(), detail::dtype_of(a_rows), a_rows, b_shard, c_shard,
                              detail::dtype_of(c_shard), m, n_shard, k, alpha, beta),
        "gemm_tensor_host_sharded");
}

// Device buffers; every rank ends with the whole row-major m x n matrix in c_full (a buffer
// from ShardedComm::alloc_shared).  c_shard is the rank's packed m x width block.  Collective
// and stream-ordered.
template <typename InT, typename OutT>
inline void gemm_tensor_gathered(ShardedComm& comm, const InT* a, const InT* b_shard, OutT* c_shard,
                                 OutT* c_full, int m, int n, int k, int lda, int ldb, float alpha,
                                 float beta, cudaStream_t stream = nullptr) {
    detail::throw_on_error(
        ckl_gemm_gathered(comm.get(), detail::dtype_of(a), a, b_shard, c_shard, c_full,
                          detail::dtype_of(c_shard), m, n, k, lda, ldb, alpha, beta, stream),
        "gemm_tensor_gathered");
}

}  // namespace ckl
