// Single-precision GEMM on the CUDA cores: C = alpha * A * B + beta * C with FP32 inputs,
// FP32 multiply-add and FP32 output, row-major, explicit leading dimensions, any shape.
//
// One kernel stands behind the four FP32 rungs of the reference ladder (gemm_naive,
// gemm_tiled, gemm_register, gemm_cp_async: include/ckl/gemm.hpp:40-58 of the reference),
// whose results must agree with SGEMM to 1e-4 relative Frobenius error
// (tests/test_gemm.cpp:50,98-101 there), which rules out TF32 tensor-core arithmetic.
//
// 128 x 128 output tile per CTA of 256 threads, 16-deep k slab, 8 x 8 outputs per thread as
// four 4 x 4 blocks (rows ty*4 and 64+ty*4, columns tx*4 and 64+tx*4, so every shared-memory
// read is a conflict-free or broadcast 16-byte load).  A 64 x 64 tile (one 4 x 4 block per
// thread) takes the problems that would leave most SMs without a 128 x 128 tile.  The next
// slab travels while the current one is multiplied (A through registers, B with asynchronous
// copies in the large tile when the operands are aligned) into the other shared buffer: one __syncthreads per slab.  A is stored transposed
// (sa[k][row]) so that the inner loop reads four consecutive rows with one load.
#pragma once

#include <cstddef>
#include <cstdint>

#include <cuda_runtime.h>

namespace ckl {

namespace fp32 {
constexpr int kTileLarge = 128;
constexpr int kTileSmall = 64;
constexpr int kTileK = 16;
constexpr int kThreads = 256;
}  // namespace fp32

// kVec: A, B, C base pointers are 16-byte aligned and lda, ldb, ldc are multiples of 4, so
// every in-range group of four consecutive elements can move as one float4.
// kTile: edge of the square output tile, 128 or 64.
template <bool kVec, int kTile>
__global__ void __launch_bounds__(fp32::kThreads, 2)
sgemm_kernel(const float* __restrict__ a, const float* __restrict__ b, float* c, int m, int n, int k,
             int lda, int ldb, int ldc, float alpha, float beta) {
    using namespace fp32;
    constexpr int kTileM = kTile, kTileN = kTile;
    constexpr int kPitch = kTile + 4;      // floats; keeps rows 16-byte aligned, spreads banks
    constexpr int kR = kTile / 16;         // outputs per thread along each axis: 8 or 4
    constexpr int kLoads = kTile / 64;     // float4 of A (and of B) per thread and slab
    constexpr int kBRowQuads = kTile / 4;  // float4 per k row of the B slab
    __shared__ __align__(16) float sa[2][kTileK][kPitch];
    __shared__ __align__(16) float sb[2][kTileK][kPitch];

    const int tid = static_cast<int>(threadIdx.x);
    const int tx = tid & 15;
    const int ty = tid >> 4;
    const int m0 = static_cast<int>(blockIdx.y) * kTileM;
    const int n0 = static_cast<int>(blockIdx.x) * kTileN;

    // Staging of one slab.  A travels global memory -> registers -> shared memory, because it
    // is stored transposed.  B keeps its layout, so in the large tile with aligned operands it
    // goes straight into the other shared buffer with 16-byte asynchronous copies (zero-filled
    // past the edges of the matrix), which frees eight staging registers; otherwise through
    // registers like A (the small tile is faster that way: its problems are short and
    // latency-bound).
    constexpr bool kAsyncB = kVec && kTile == 128;
    float4 ra[kLoads];
    float4 rb[kAsyncB ? 1 : kLoads];
    auto fetch = [&](int k0, int buf) {
#pragma unroll
        for (int i = 0; i < kLoads; ++i) {
            const int idx = tid + i * kThreads;
            {
                // A: kTile rows x 16 k, four consecutive k of one row
                const int row = m0 + (idx >> 2);
                const int kk = k0 + (idx & 3) * 4;
                float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
                if (row < m) {
                    const float* src = a + static_cast<size_t>(row) * lda + kk;
                    if (kVec && kk + 3 < k) {
                        v = *reinterpret_cast<const float4*>(src);
                    } else {
                        if (kk < k) v.x = src[0];
                        if (kk + 1 < k) v.y = src[1];
                        if (kk + 2 < k) v.z = src[2];
                        if (kk + 3 < k) v.w = src[3];
                    }
                }
                ra[i] = v;
            }
            {
                // B: 16 k x kTile columns, four consecutive columns of one k row
                const int kr = k0 + idx / kBRowQuads;
                const int col = n0 + (idx % kBRowQuads) * 4;
                if constexpr (kAsyncB) {
                    const bool inside = kr < k && col < n;
                    const int bytes = inside ? min(16, (n - col) * 4) : 0;
                    const float* src = inside ? b + static_cast<size_t>(kr) * ldb + col : b;
                    const uint32_t dst = static_cast<uint32_t>(__cvta_generic_to_shared(
                        &sb[buf][idx / kBRowQuads][(idx % kBRowQuads) * 4]));
                    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(bytes)
                                 : "memory");
                } else {
                    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
                    if (kr < k) {
                        const float* src = b + static_cast<size_t>(kr) * ldb + col;
                        if (kVec && col + 3 < n) {
                            v = *reinterpret_cast<const float4*>(src);
                        } else {
                            if (col < n) v.x = src[0];
                            if (col + 1 < n) v.y = src[1];
                            if (col + 2 < n) v.z = src[2];
                            if (col + 3 < n) v.w = src[3];
                        }
                    }
                    rb[i] = v;
                }
            }
        }
    };
    auto stash = [&](int buf) {
#pragma unroll
        for (int i = 0; i < kLoads; ++i) {
            const int idx = tid + i * kThreads;
            const int r = idx >> 2;
            const int kq = (idx & 3) * 4;
            sa[buf][kq + 0][r] = ra[i].x;
            sa[buf][kq + 1][r] = ra[i].y;
            sa[buf][kq + 2][r] = ra[i].z;
            sa[buf][kq + 3][r] = ra[i].w;
            if constexpr (!kAsyncB) {
                *reinterpret_cast<float4*>(&sb[buf][idx / kBRowQuads][(idx % kBRowQuads) * 4]) = rb[i];
            }
        }
        if constexpr (kAsyncB) {
            asm volatile("cp.async.wait_all;" ::: "memory");
        }
    };

    // Accumulators as column pairs: the packed FP32 multiply-add of sm_100 (two independent
    // IEEE round-to-nearest FMAs per instruction, bit-identical to fmaf on each half) takes half
    // the issue slots of scalar FMAs, which is what this kernel was short of.
    float2 acc[kR][kR / 2];
#pragma unroll
    for (int i = 0; i < kR; ++i) {
#pragma unroll
        for (int j = 0; j < kR / 2; ++j) {
            acc[i][j] = make_float2(0.0f, 0.0f);
        }
    }

    const int slabs = (k + kTileK - 1) / kTileK;
    if (slabs > 0) {
        fetch(0, 0);
        stash(0);
    }
    __syncthreads();
    for (int s = 0; s < slabs; ++s) {
        const int cur = s & 1;
        if (s + 1 < slabs) {
            fetch((s + 1) * kTileK, cur ^ 1);  // that buffer was last read one slab ago
        }
#pragma unroll
        for (int kk = 0; kk < kTileK; ++kk) {
            float av[kR];
            float2 bv[kR / 2];
#pragma unroll
            for (int h = 0; h < kR / 4; ++h) {
                const float4 av4 = *reinterpret_cast<const float4*>(&sa[cur][kk][h * 64 + ty * 4]);
                const float4 bv4 = *reinterpret_cast<const float4*>(&sb[cur][kk][h * 64 + tx * 4]);
                av[h * 4 + 0] = av4.x; av[h * 4 + 1] = av4.y; av[h * 4 + 2] = av4.z; av[h * 4 + 3] = av4.w;
                bv[h * 2 + 0] = make_float2(bv4.x, bv4.y);
                bv[h * 2 + 1] = make_float2(bv4.z, bv4.w);
            }
#pragma unroll
            for (int i = 0; i < kR; ++i) {
                const float2 a2 = make_float2(av[i], av[i]);
#pragma unroll
                for (int j = 0; j < kR / 2; ++j) {
                    acc[i][j] = __ffma2_rn(a2, bv[j], acc[i][j]);
                }
            }
        }
        if (s + 1 < slabs) {
            stash(cur ^ 1);  // last read one slab ago; every thread has passed that barrier
        }
        __syncthreads();
    }

    // C = alpha * acc + beta * C; C is not read when beta == 0 (BLAS convention).
#pragma unroll
    for (int i = 0; i < kR; ++i) {
        const int row = m0 + (i >> 2) * 64 + ty * 4 + (i & 3);
        if (row >= m) {
            continue;
        }
        float* crow = c + static_cast<size_t>(row) * ldc;
#pragma unroll
        for (int h = 0; h < kR / 4; ++h) {
            const int col = n0 + h * 64 + tx * 4;
            float* dst = crow + col;
            if (kVec && col + 3 < n) {
                float4 out;
                if (beta != 0.0f) {
                    const float4 old = *reinterpret_cast<const float4*>(dst);
                    out.x = fmaf(beta, old.x, alpha * acc[i][h * 2 + 0].x);
                    out.y = fmaf(beta, old.y, alpha * acc[i][h * 2 + 0].y);
                    out.z = fmaf(beta, old.z, alpha * acc[i][h * 2 + 1].x);
                    out.w = fmaf(beta, old.w, alpha * acc[i][h * 2 + 1].y);
                } else {
                    out.x = alpha * acc[i][h * 2 + 0].x;
                    out.y = alpha * acc[i][h * 2 + 0].y;
                    out.z = alpha * acc[i][h * 2 + 1].x;
                    out.w = alpha * acc[i][h * 2 + 1].y;
                }
                *reinterpret_cast<float4*>(dst) = out;
            } else {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    if (col + e < n) {
                        const float2 pair = acc[i][h * 2 + (e >> 1)];
                        const float v = alpha * ((e & 1) ? pair.y : pair.x);
                        dst[e] = beta != 0.0f ? fmaf(beta, dst[e], v) : v;
                    }
                }
            }
        }
    }
}

}  // namespace ckl
