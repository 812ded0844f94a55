// device_probe: what the machine is, measured rather than quoted.
//
// B200 counterpart of the reference's src/tools/device_probe.cu:74-158 (same
// role, same --json switch).  What changed for this part: the stream-copy probe
// is the library's ckl_stream_copy (four independent 16-byte loads in flight per
// thread, 1 GiB buffers; the reference's one-load loop over 512 MiB cannot fill
// HBM3e); the "peak FP32 = cores x 2 x clock" guess is replaced by the dense
// 16-bit tensor estimate SMs x 8192 FLOP/clk x boost clock, which is what bounds
// the GEMM path; and NVLink peers are counted.

#include <algorithm>
#include <cstdio>
#include <string>
#include <vector>

#include <cuda_runtime.h>

#include "ckl/cuda_check.hpp"
#include "ckl_gemm.h"

namespace {

double median(std::vector<double> v) {
    std::sort(v.begin(), v.end());
    return v[v.size() / 2];
}

// GB/s of a device-to-device copy, read + write bytes counted, median of `reps`.
template <typename Launch>
double copy_bandwidth_gbps(size_t bytes, int reps, Launch launch) {
    cudaEvent_t t0, t1;
    CKL_CUDA_CHECK(cudaEventCreate(&t0));
    CKL_CUDA_CHECK(cudaEventCreate(&t1));
    for (int i = 0; i < 3; ++i) {
        launch();
    }
    CKL_CUDA_CHECK(cudaDeviceSynchronize());
    std::vector<double> gbps;
    for (int i = 0; i < reps; ++i) {
        CKL_CUDA_CHECK(cudaEventRecord(t0));
        launch();
        CKL_CUDA_CHECK(cudaEventRecord(t1));
        CKL_CUDA_CHECK(cudaEventSynchronize(t1));
        float ms = 0.0f;
        CKL_CUDA_CHECK(cudaEventElapsedTime(&ms, t0, t1));
        gbps.push_back(2.0 * static_cast<double>(bytes) / (ms * 1.0e-3) / 1.0e9);
    }
    cudaEventDestroy(t0);
    cudaEventDestroy(t1);
    return median(gbps);
}

}  // namespace

int main(int argc, char** argv) {
    const bool json = argc > 1 && std::string(argv[1]) == "--json";
    int device = 0;
    CKL_CUDA_CHECK(cudaGetDevice(&device));
    cudaDeviceProp p{};
    CKL_CUDA_CHECK(cudaGetDeviceProperties(&p, device));
    int runtime_version = 0, driver_version = 0, mem_khz = 0, core_khz = 0, devices = 0;
    CKL_CUDA_CHECK(cudaRuntimeGetVersion(&runtime_version));
    CKL_CUDA_CHECK(cudaDriverGetVersion(&driver_version));
    CKL_CUDA_CHECK(cudaDeviceGetAttribute(&mem_khz, cudaDevAttrMemoryClockRate, device));
    CKL_CUDA_CHECK(cudaDeviceGetAttribute(&core_khz, cudaDevAttrClockRate, device));
    CKL_CUDA_CHECK(cudaGetDeviceCount(&devices));
    int peers = 0;
    for (int d = 0; d < devices; ++d) {
        int can = 0;
        if (d != device && cudaDeviceCanAccessPeer(&can, device, d) == cudaSuccess && can) {
            ++peers;
        }
    }

    const size_t bytes = size_t(1) << 30;
    void* src = nullptr;
    void* dst = nullptr;
    CKL_CUDA_CHECK(cudaMalloc(&src, bytes));
    CKL_CUDA_CHECK(cudaMalloc(&dst, bytes));
    CKL_CUDA_CHECK(cudaMemset(src, 1, bytes));
    const double kernel_bw = copy_bandwidth_gbps(bytes, 20, [&] {
        if (ckl_stream_copy(dst, src, bytes, nullptr) != CKL_OK) {
            std::fprintf(stderr, "ckl_stream_copy: %s\n", ckl_last_error());
        }
    });
    const double memcpy_bw = copy_bandwidth_gbps(bytes, 20, [&] {
        cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToDevice, nullptr);
    });
    cudaFree(src);
    cudaFree(dst);

    // HBM moves data on both clock edges; bus width is in bits.
    const double theo_bw = static_cast<double>(mem_khz) * 1.0e3 * (p.memoryBusWidth / 8.0) * 2.0 / 1.0e9;
    const double tensor_peak =
        static_cast<double>(p.multiProcessorCount) * 8192.0 * static_cast<double>(core_khz) * 1.0e3 / 1.0e12;

    if (json) {
        std::printf("{\"name\": \"%s\", \"compute_capability\": \"%d.%d\", \"sm_count\": %d, "
                    "\"global_mem_mib\": %.0f, \"mem_bus_width_bits\": %d, \"mem_clock_khz\": %d, "
                    "\"core_clock_khz\": %d, \"l2_cache_kib\": %d, \"shared_mem_per_block_optin_kib\": %zu, "
                    "\"shared_mem_per_sm_kib\": %zu, \"regs_per_sm\": %d, \"max_threads_per_sm\": %d, "
                    "\"tensor_memory_kib_per_sm\": 256, \"nvlink_peers\": %d, "
                    "\"theoretical_bw_gbps\": %.1f, \"measured_bw_gbps\": %.1f, "
                    "\"measured_memcpy_d2d_gbps\": %.1f, \"dense_16bit_tensor_tflops_estimate\": %.1f, "
                    "\"runtime_version\": %d, \"driver_version\": %d}\n",
                    p.name, p.major, p.minor, p.multiProcessorCount,
                    static_cast<double>(p.totalGlobalMem) / (1024.0 * 1024.0), p.memoryBusWidth, mem_khz,
                    core_khz, p.l2CacheSize / 1024, p.sharedMemPerBlockOptin / 1024,
                    p.sharedMemPerMultiprocessor / 1024, p.regsPerMultiprocessor,
                    p.maxThreadsPerMultiProcessor, peers, theo_bw, kernel_bw, memcpy_bw, tensor_peak,
                    runtime_version, driver_version);
        return 0;
    }
    std::printf("ckl device probe (sm_100a build)\n");
    std::printf("Device                   : %s\n", p.name);
    std::printf("Compute capability       : %d.%d\n", p.major, p.minor);
    std::printf("SM count                 : %d\n", p.multiProcessorCount);
    std::printf("Global memory            : %.0f MiB\n", static_cast<double>(p.totalGlobalMem) / (1024.0 * 1024.0));
    std::printf("Memory bus / clock       : %d bits, %.0f MHz\n", p.memoryBusWidth, mem_khz / 1000.0);
    std::printf("Boost clock              : %.0f MHz\n", core_khz / 1000.0);
    std::printf("L2 cache                 : %d KiB\n", p.l2CacheSize / 1024);
    std::printf("Shared memory per CTA/SM : %zu / %zu KiB\n", p.sharedMemPerBlockOptin / 1024,
                p.sharedMemPerMultiprocessor / 1024);
    std::printf("Tensor memory per SM     : 256 KiB (512 columns x 128 lanes x 4 B)\n");
    std::printf("NVLink/P2P peers         : %d of %d other devices\n", peers, devices - 1);
    std::printf("Theoretical HBM BW       : %.1f GB/s (clock x bus x 2)\n", theo_bw);
    std::printf("Measured stream-copy BW  : %.1f GB/s (ckl_stream_copy, 1 GiB, read+write)\n", kernel_bw);
    std::printf("Measured memcpy D2D BW   : %.1f GB/s\n", memcpy_bw);
    std::printf("Dense 16-bit tensor est. : %.1f TFLOP/s (SMs x 8192 FLOP/clk x boost clock)\n", tensor_peak);
    std::printf("CUDA runtime / driver    : %d / %d\n", runtime_version, driver_version);
    return 0;
}
