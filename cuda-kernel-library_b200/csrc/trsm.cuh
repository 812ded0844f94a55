// Diagonal-block kernel of the blocked triangular solve L X = alpha B (L lower triangular,
// non-unit diagonal, row-major; X overwrites B).  The solve splits the rows in two halves
// recursively: solve the upper half, subtract its contribution from the lower half with one FP32
// GEMM (B_low -= L_low,up * X_up), solve the lower half.  Halves of at most kTrsmBlock rows are
// solved by this kernel against their own triangle; the GEMMs are where the flops are.  The
// reference walks down the diagonal in 32-row blocks and updates the rows below each with a
// one-thread-per-element loop in place of a GEMM (src/trsm/trsm_blocked.cu:46-62,77-90 there).
#pragma once

#include <cstddef>

#include <cuda_runtime.h>

namespace ckl {

constexpr int kTrsmBlock = 64;       // rows per diagonal block
constexpr int kTrsmThreads = 128;    // right-hand-side columns per CTA

// One thread per right-hand-side column.  The block's triangle sits in shared memory (every
// lane reads the same element: broadcast), the thread's kb solved values in registers.  Row i
// of the block needs the i values above it, so the rows are sequential; each row's dot product
// runs on four independent partial sums to shorten the dependent chain.
__global__ void __launch_bounds__(kTrsmThreads)
trsm_diag_block_kernel(const float* __restrict__ l, float* b, int n, int lda, int ldb, int k0, int kb) {
    __shared__ float tri[kTrsmBlock][kTrsmBlock + 1];
    for (int idx = static_cast<int>(threadIdx.x); idx < kTrsmBlock * kTrsmBlock; idx += kTrsmThreads) {
        const int i = idx / kTrsmBlock;
        const int j = idx % kTrsmBlock;
        float v = 0.0f;
        if (i < kb && j <= i) {
            v = l[static_cast<size_t>(k0 + i) * lda + (k0 + j)];
        }
        tri[i][j] = v;
    }
    __syncthreads();
    const int col = static_cast<int>(blockIdx.x) * kTrsmThreads + static_cast<int>(threadIdx.x);
    if (col >= n) {
        return;
    }
    // All right-hand-side values of the block are fetched before the first row is solved and
    // written back after the last: loads and stores go through the same pointer, so interleaved
    // they would have to stay in program order and every row would wait a global-memory round trip.
    float x[kTrsmBlock];
    float* bcol = b + static_cast<size_t>(k0) * ldb + col;
#pragma unroll
    for (int i = 0; i < kTrsmBlock; ++i) {
        x[i] = i < kb ? bcol[static_cast<size_t>(i) * ldb] : 0.0f;
    }
#pragma unroll
    for (int i = 0; i < kTrsmBlock; ++i) {
        float s0 = x[i], s1 = 0.0f, s2 = 0.0f, s3 = 0.0f;
#pragma unroll
        for (int j = 0; j < i; ++j) {
            const float t = tri[i][j] * x[j];
            if ((j & 3) == 0) s0 -= t;
            if ((j & 3) == 1) s1 -= t;
            if ((j & 3) == 2) s2 -= t;
            if ((j & 3) == 3) s3 -= t;
        }
        // rows past kb have a zero triangle row and a zero right-hand side; keep them at zero
        x[i] = i < kb ? ((s0 + s1) + (s2 + s3)) / tri[i][i] : 0.0f;
    }
#pragma unroll
    for (int i = 0; i < kTrsmBlock; ++i) {
        if (i < kb) {
            bcol[static_cast<size_t>(i) * ldb] = x[i];
        }
    }
}

}  // namespace ckl
