#pragma once
// ckl::trsm_* C++ entry points of the B200 build: drop-in for the reference library's
// include/ckl/trsm.hpp (lines 19-28 there).  Solves L X = alpha B for X, L an m x m lower
// triangular matrix with a non-unit diagonal, B (overwritten by X) m x n, row-major FP32.
//
// Both hand-written rungs of the reference are the same blocked solve here: 64-row diagonal
// blocks solved directly, the rows below each block updated by the library's FP32 GEMM
// (ckl_strsm_lower in ckl_gemm.h).  Failures throw std::runtime_error, like the
// reference's checked calls.

#include <cuda_runtime.h>

#include "../ckl_gemm.h"
#include "gemm.hpp"

namespace ckl {

inline void trsm_blocked(const float* a, float* b, int m, int n, float alpha,
                         cudaStream_t stream = nullptr) {
    detail::throw_on_error(ckl_strsm_lower(a, b, m, n, m, n, alpha, stream), "trsm_blocked");
}

inline void trsm_naive(const float* a, float* b, int m, int n, float alpha,
                       cudaStream_t stream = nullptr) {
    detail::throw_on_error(ckl_strsm_lower(a, b, m, n, m, n, alpha, stream), "trsm_naive");
}

// cuBLAS STRSM comparator.  Test and benchmark code only: defined in a separate translation
// unit that the shipped library does not contain (reference: src/trsm/cublas_trsm.cpp).
void trsm_cublas(const float* a, float* b, int m, int n, float alpha, cudaStream_t stream = nullptr);

}  // namespace ckl
