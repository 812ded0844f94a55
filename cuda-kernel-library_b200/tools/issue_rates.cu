// issue_rates: how many cycles one warp instruction of each kind the GEMM epilogue uses costs,
// per SM sub-partition, with 1, 2 and 4 warps resident on each sub-partition (the epilogue of
// the tensor-core kernels runs 1 or 2).  Every kind is a chain of 16 independent dependent
// sequences, 64 instructions per loop trip, timed with clock64 on one SM.  The shared-memory
// rows use the epilogue's staging pattern (32 rows x 128 B, 16-byte units XOR-swizzled by row).
// Usage: issue_rates   (prints a table; no arguments)
#include <cstdio>
#include <cstdint>
#include <cuda_runtime.h>
#define ITERS 128
#define U 4
template <int KIND>
__global__ void k(uint32_t* out, long long* cyc, int seed) {
    __shared__ __align__(16) uint4 sm[32 * 8 * 8];
    uint32_t r[16];
    for (int i = 0; i < 16; ++i) { r[i] = __float_as_uint((float)(seed + i + threadIdx.x) * 1.001f); }
    const uint32_t sbase = (uint32_t)__cvta_generic_to_shared(sm) + ((threadIdx.x >> 5) & 7) * 4096 + (threadIdx.x & 31) * 128;
    const uint32_t lane = threadIdx.x & 31;
    const uint32_t cst = __float_as_uint(1.0001f) + seed;
    __syncthreads();
    long long t0 = clock64();
#pragma unroll 1
    for (int it = 0; it < ITERS; ++it) {
#pragma unroll
        for (int u = 0; u < U; ++u) {
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                if (KIND == 0) asm volatile("cvt.rn.bf16x2.f32 %0, %0, %1;" : "+r"(r[i]) : "r"(cst));
                if (KIND == 1) asm volatile("cvt.rn.f16x2.f32 %0, %0, %1;" : "+r"(r[i]) : "r"(cst));
                if (KIND == 2) asm volatile("fma.rn.f32 %0, %0, %1, %1;" : "+r"(r[i]) : "r"(cst));
                if (KIND == 3) asm volatile("prmt.b32 %0, %0, %1, 0x7632;" : "+r"(r[i]) : "r"(cst));
                if (KIND == 4) asm volatile("shl.b32 %0, %0, 1;" : "+r"(r[i]));
                if (KIND == 5) asm volatile("lop3.b32 %0, %0, %1, %1, 0x96;" : "+r"(r[i]) : "r"(cst));
                if (KIND == 8) asm volatile("add.u32 %0, %0, %1;" : "+r"(r[i]) : "r"(cst));
            }
            if (KIND == 6) {
#pragma unroll
                for (int j = 0; j < 4; ++j)
                    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(sbase + (((j + 4 * (u & 1)) ^ (lane & 7)) << 4)), "r"(r[4 * j]), "r"(r[4 * j + 1]), "r"(r[4 * j + 2]), "r"(r[4 * j + 3]) : "memory");
            }
            if (KIND == 7) {
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    uint32_t a, b, c, d;
                    asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(a), "=r"(b), "=r"(c), "=r"(d) : "r"(sbase + (((j + 4 * (u & 1)) ^ (lane & 7)) << 4)) : "memory");
                    r[4 * j] ^= a; r[4 * j + 1] ^= b; r[4 * j + 2] ^= c; r[4 * j + 3] ^= d;
                }
            }
            if (KIND == 9) {
#pragma unroll
                for (int i = 0; i < 16; i += 2) {
                    unsigned long long v = (static_cast<unsigned long long>(r[i + 1]) << 32) | r[i];
                    unsigned long long cc = (static_cast<unsigned long long>(cst) << 32) | cst;
                    asm volatile("fma.rn.f32x2 %0, %0, %1, %1;" : "+l"(v) : "l"(cc));
                    r[i] = static_cast<uint32_t>(v); r[i + 1] = static_cast<uint32_t>(v >> 32);
                }
            }
        }
    }
    long long t1 = clock64();
    uint32_t acc = 0;
    for (int i = 0; i < 16; ++i) acc += r[i];
    out[blockIdx.x * blockDim.x + threadIdx.x] = acc;
    if (threadIdx.x == 0 && blockIdx.x == 0) *cyc = t1 - t0;
}
template <int KIND>
void run(const char* name, uint32_t* out, long long* cyc, int per_iter) {
    for (int warps : {4, 8, 16}) {
        k<KIND><<<148, warps * 32>>>(out, cyc, 3);
        cudaDeviceSynchronize();
        k<KIND><<<148, warps * 32>>>(out, cyc, 3);
        cudaDeviceSynchronize();
        long long c;
        cudaMemcpy(&c, cyc, 8, cudaMemcpyDeviceToHost);
        printf("%-24s warps/SMSP %d  cycles per warp instr per SMSP %.2f   (per warp: %.2f)\n", name, warps / 4,
               (double)c / (ITERS * (double)per_iter) / (warps / 4), (double)c / (ITERS * (double)per_iter));
    }
}
int main() {
    uint32_t* out; long long* cyc;
    cudaMalloc(&out, 148 * 1024 * 4); cudaMalloc(&cyc, 8);
    run<0>("cvt.rn.bf16x2.f32", out, cyc, 16 * U);
    run<1>("cvt.rn.f16x2.f32", out, cyc, 16 * U);
    run<2>("fma.rn.f32", out, cyc, 16 * U);
    run<9>("fma.rn.f32x2", out, cyc, 8 * U);
    run<3>("prmt", out, cyc, 16 * U);
    run<4>("shl", out, cyc, 16 * U);
    run<5>("lop3", out, cyc, 16 * U);
    run<8>("add.u32", out, cyc, 16 * U);
    run<6>("st.shared.v4 swizzled", out, cyc, 4 * U);
    run<7>("ld.shared.v4 swizzled", out, cyc, 4 * U);
    printf("%s\n", cudaGetErrorString(cudaGetLastError()));
    return 0;
}
