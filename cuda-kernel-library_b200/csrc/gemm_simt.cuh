// General-shape GEMM on the CUDA cores: any m, n, k, any leading dimension and
// any pointer alignment, FP16/BF16 inputs, FP32 accumulation.  It takes the
// shapes TMA cannot describe (row pitch not a multiple of 16 bytes, unaligned
// base), the role the scalar half_naive_kernel plays in the reference
// (include/ckl/detail/wmma_gemm.cuh:124-140), but tiled through shared memory:
// 64 x 64 output tile, 16-deep k slab, 4 x 4 outputs per thread.
//
// Also here: C = beta * C for an empty contraction (k <= 0), the unfused
// bias + ReLU pass, and the stream-copy bandwidth probe.
#pragma once

#include <cstdint>

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "gemm_umma.cuh"

namespace ckl {

namespace detail {
__device__ __forceinline__ float in_to_float(__half v) { return __half2float(v); }
__device__ __forceinline__ float in_to_float(__nv_bfloat16 v) { return __bfloat162float(v); }
}  // namespace detail

template <typename InT, typename OutT>
__global__ void __launch_bounds__(256)
simt_gemm_kernel(const InT* __restrict__ a, const InT* __restrict__ b, OutT* c,
                 const float* __restrict__ bias, int m, int n, int k, int lda, int ldb, int ldc,
                 float alpha, float beta, int epi_mode) {
    constexpr int BM = 64, BN = 64, BK = 16;
    __shared__ float sa[BK][BM + 4];  // transposed: sa[kk][row]
    __shared__ float sb[BK][BN + 4];

    const int tid = static_cast<int>(threadIdx.x);
    const int tx = tid % 16;  // column group
    const int ty = tid / 16;  // row group
    const int row0 = static_cast<int>(blockIdx.y) * BM;
    const int col0 = static_cast<int>(blockIdx.x) * BN;

    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            acc[i][j] = 0.0f;
        }
    }

    for (int k0 = 0; k0 < k; k0 += BK) {
        // A slab: 64 rows x 16 k; thread loads 4 elements (consecutive k of one row).
        {
            const int r = tid / 4;
            const int kk = (tid % 4) * 4;
            const int gr = row0 + r;
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int gk = k0 + kk + e;
                float v = 0.0f;
                if (gr < m && gk < k) {
                    v = detail::in_to_float(a[static_cast<size_t>(gr) * lda + gk]);
                }
                sa[kk + e][r] = v;
            }
        }
        // B slab: 16 k x 64 columns; thread loads 4 consecutive columns of one k row.
        {
            const int kk = tid / 16;
            const int cc = (tid % 16) * 4;
            const int gk = k0 + kk;
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int gc = col0 + cc + e;
                float v = 0.0f;
                if (gk < k && gc < n) {
                    v = detail::in_to_float(b[static_cast<size_t>(gk) * ldb + gc]);
                }
                sb[kk][cc + e] = v;
            }
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < BK; ++kk) {
            float av[4], bv[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                av[i] = sa[kk][ty * 4 + i];
                bv[i] = sb[kk][tx * 4 + i];
            }
#pragma unroll
            for (int i = 0; i < 4; ++i) {
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
                }
            }
        }
        __syncthreads();
    }

    using T = detail::OutTraits<OutT>;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int gr = row0 + ty * 4 + i;
        if (gr >= m) {
            continue;
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int gc = col0 + tx * 4 + j;
            if (gc >= n) {
                continue;
            }
            OutT* dst = c + static_cast<size_t>(gr) * ldc + gc;
            float v;
            if (epi_mode == kEpiBiasRelu) {
                v = fmaxf(alpha * acc[i][j] + bias[gc], 0.0f);
            } else if (beta != 0.0f) {
                v = alpha * acc[i][j] + beta * T::load(dst);
            } else {
                v = alpha * acc[i][j];
            }
            T::store(dst, v);
        }
    }
}

// k <= 0: C = beta * C (C = 0 when beta == 0, without reading C), as the
// reference's kernels and oracle do (include/ckl/detail/wmma_gemm.cuh:133-139,
// src/gemm/cublas_gemm_ex.cpp:46-50).  With the bias epilogue the empty
// product gives relu(bias).
template <typename OutT>
__global__ void scale_c_kernel(OutT* c, const float* bias, int m, int n, int ldc, float beta,
                               int epi_mode) {
    using T = detail::OutTraits<OutT>;
    const long long total = static_cast<long long>(m) * n;
    for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
        const int r = static_cast<int>(i / n);
        const int col = static_cast<int>(i % n);
        OutT* dst = c + static_cast<size_t>(r) * ldc + col;
        float v;
        if (epi_mode == kEpiBiasRelu) {
            v = fmaxf(bias[col], 0.0f);
        } else {
            v = beta != 0.0f ? beta * T::load(dst) : 0.0f;
        }
        T::store(dst, v);
    }
}

// Unfused second pass C = relu(C + bias[col]) over FP32 C; replaces
// bias_relu_kernel (src/gemm/gemm_mma_opt.cu:199-206).
__global__ void bias_relu_kernel(float* c, const float* __restrict__ bias, int m, int n, int ldc) {
    const long long total = static_cast<long long>(m) * n;
    for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
        const int r = static_cast<int>(i / n);
        const int col = static_cast<int>(i % n);
        float* dst = c + static_cast<size_t>(r) * ldc + col;
        *dst = fmaxf(*dst + bias[col], 0.0f);
    }
}

// The same pass four columns at a time, for n and ldc multiples of 4 and 16-byte aligned
// pointers: one 16-byte load and store per thread instead of four 4-byte ones.
__global__ void __launch_bounds__(256)
bias_relu_vec4_kernel(float4* c, const float4* __restrict__ bias, int m, int n4, int ldc4) {
    const long long total = static_cast<long long>(m) * n4;
    for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
        const long long r = i / n4;
        const int col = static_cast<int>(i - r * n4);
        float4* dst = c + r * ldc4 + col;
        float4 v = *dst;
        const float4 bv = __ldg(bias + col);
        v.x = fmaxf(v.x + bv.x, 0.0f);
        v.y = fmaxf(v.y + bv.y, 0.0f);
        v.z = fmaxf(v.z + bv.z, 0.0f);
        v.w = fmaxf(v.w + bv.w, 0.0f);
        *dst = v;
    }
}

// Copies a rows x cols matrix of 2- or 4-byte elements between a buffer of any address and
// pitch and one whose base and pitch are 16-byte aligned (so that TMA can describe it).  One
// thread moves one 16-byte group of the aligned side: kDstAligned packs scalar loads into one
// 16-byte store (padding elements of the last group of a row are written as zero), otherwise
// one 16-byte load is scattered with scalar stores (elements past `cols` are dropped).  Pure
// copy, HBM-bound.
template <typename T, bool kDstAligned>
__global__ void __launch_bounds__(256)
copy_rows_kernel(T* __restrict__ dst, const T* __restrict__ src, int rows, int cols, size_t src_pitch,
                 size_t dst_pitch) {
    constexpr int kPer = 16 / static_cast<int>(sizeof(T));
    const size_t groups_per_row = (static_cast<size_t>(cols) + kPer - 1) / kPer;
    const size_t total = groups_per_row * static_cast<size_t>(rows);
    const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
    for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
        const size_t r = i / groups_per_row;
        const int c0 = static_cast<int>(i - r * groups_per_row) * kPer;
        const T* s = src + r * src_pitch + c0;
        T* d = dst + r * dst_pitch + c0;
        union {
            uint4 vec;
            T elem[kPer];
        } v;
        if constexpr (kDstAligned) {
#pragma unroll
            for (int e = 0; e < kPer; ++e) {
                v.elem[e] = (c0 + e < cols) ? s[e] : static_cast<T>(0);
            }
            *reinterpret_cast<uint4*>(d) = v.vec;
        } else {
            v.vec = *reinterpret_cast<const uint4*>(s);
#pragma unroll
            for (int e = 0; e < kPer; ++e) {
                if (c0 + e < cols) {
                    d[e] = v.elem[e];
                }
            }
        }
    }
}

// [parts][m][per_row] -> [m][parts * per_row], in units of T (16-byte vectors
// when the shard row pitch allows).  Follows the all-gather of the N-sharded
// GEMM; pure copy, bound by HBM bandwidth (reads and writes every byte once).
template <typename T>
__global__ void assemble_column_blocks_kernel(T* __restrict__ dst, const T* __restrict__ src,
                                              size_t per_row, int m, int parts) {
    const size_t total = per_row * static_cast<size_t>(m) * static_cast<size_t>(parts);
    const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
    for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
         i += stride) {
        // i indexes dst: row r, part p, offset c inside the part's row segment
        const size_t row_len = per_row * static_cast<size_t>(parts);
        const size_t r = i / row_len;
        const size_t in_row = i - r * row_len;
        const size_t p = in_row / per_row;
        const size_t c = in_row - p * per_row;
        dst[i] = src[(p * static_cast<size_t>(m) + r) * per_row + c];
    }
}

// Bandwidth probe: each thread moves eight 16-byte words per trip, all eight loads issued
// before the first store, with streaming (evict-first) hints on both sides.  HBM3e needs far
// more bytes in flight per SM than the reference's one-load-per-iteration loop provides
// (src/tools/device_probe.cu:25-31 there).
__global__ void __launch_bounds__(1024)
stream_copy_kernel(uint4* __restrict__ dst, const uint4* __restrict__ src, size_t count) {
    // A block copies contiguous 128 KB pieces (8 x 1024 x 16 B), pieces dealt round-robin to
    // blocks: consecutive lines of a DRAM page are touched together.
    constexpr int kUnroll = 8;
    const size_t piece = static_cast<size_t>(kUnroll) * blockDim.x;
    const size_t pieces = count / piece;
    for (size_t t = blockIdx.x; t < pieces; t += gridDim.x) {
        const size_t base = t * piece + threadIdx.x;
        uint4 v[kUnroll];
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            v[u] = __ldcs(src + base + static_cast<size_t>(u) * blockDim.x);
        }
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            __stcs(dst + base + static_cast<size_t>(u) * blockDim.x, v[u]);
        }
    }
    for (size_t i = pieces * piece + static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
         i < count; i += static_cast<size_t>(gridDim.x) * blockDim.x) {
        dst[i] = src[i];
    }
}

}  // namespace ckl
