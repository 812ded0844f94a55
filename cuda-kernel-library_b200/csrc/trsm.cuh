// Diagonal-block kernel of the blocked triangular solve L X = alpha B (L lower triangular,
// non-unit diagonal, row-major; X overwrites B).  The solve walks down the diagonal in blocks
// of kTrsmBlock rows: this kernel solves one block row against the block's own triangle, and
// everything below it is updated by one FP32 GEMM (B_below -= L_below,block * X_block), which is
// where the flops are.  The reference does the same split but with a one-thread-per-element
// update loop in place of a GEMM (src/trsm/trsm_blocked.cu:46-62,77-90 there).
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
    float x[kTrsmBlock];
    float* bcol = b + static_cast<size_t>(k0) * ldb + col;
#pragma unroll
    for (int i = 0; i < kTrsmBlock; ++i) {
        if (i < kb) {
            float s0 = bcol[static_cast<size_t>(i) * ldb];
            float s1 = 0.0f, s2 = 0.0f, s3 = 0.0f;
#pragma unroll
            for (int j = 0; j < i; ++j) {
                const float t = tri[i][j] * x[j];
                if ((j & 3) == 0) s0 -= t;
                if ((j & 3) == 1) s1 -= t;
                if ((j & 3) == 2) s2 -= t;
                if ((j & 3) == 3) s3 -= t;
            }
            x[i] = ((s0 + s1) + (s2 + s3)) / tri[i][i];
            bcol[static_cast<size_t>(i) * ldb] = x[i];
        } else {
            x[i] = 0.0f;
        }
    }
}

}  // namespace ckl
