// roofline: measure this GPU's ceilings and place the GEMM kernels under them.
//
// B200 counterpart of the reference's src/profiler/roofline.cpp:25-38,115-197.
// Bandwidth ceiling: device-to-device cudaMemcpyAsync of 256 MiB, read + write
// bytes (the reference's definition) and the library's stream-copy kernel.
// Tensor ceiling: the reference defines it as "cuBLAS FP16 at 8192^3"; that is
// kept when the reference's cuBLAS wrapper is available (oracle/_ref), and the
// datasheet dense figure and the clock-derived figure are printed beside it.
// Points: every tensor-core kernel of this library at 4096^3 and 8192^3 (BF16).
// Writes <out_dir>/roofline_ceilings.csv and <out_dir>/roofline.csv in the
// column layout the reference's plotting script reads.

#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <string>
#include <thread>
#include <vector>

#include "ckl/device_buffer.hpp"
#include "ckl/event_timer.hpp"
#include "ckl/gemm.hpp"
#include "ckl/roofline.hpp"
#include "harness.hpp"

namespace {

double measure_memcpy_bw(size_t bytes) {
    ckl::DeviceBuffer<char> a(bytes), b(bytes);
    a.zero();
    const ckl::TimingStats t = ckl::time_stream([&](cudaStream_t s) {
        cudaMemcpyAsync(b.data(), a.data(), bytes, cudaMemcpyDeviceToDevice, s);
    });
    return 2.0 * static_cast<double>(bytes) / (t.median_ms * 1.0e-3);
}

double measure_kernel_bw(size_t bytes) {
    ckl::DeviceBuffer<char> a(bytes), b(bytes);
    a.zero();
    const ckl::TimingStats t =
        ckl::time_stream([&](cudaStream_t s) { ckl_stream_copy(b.data(), a.data(), bytes, s); });
    return 2.0 * static_cast<double>(bytes) / (t.median_ms * 1.0e-3);
}

}  // namespace

int main(int argc, char** argv) {
    const std::string out_dir = argc > 1 ? argv[1] : ".";
    const char* root_env = std::getenv("CKL_REPO_ROOT");
    const std::string root = root_env ? root_env : ".";
    cudaDeviceProp prop{};
    CKL_CUDA_CHECK(cudaGetDeviceProperties(&prop, 0));
    int core_khz = 0;
    cudaDeviceGetAttribute(&core_khz, cudaDevAttrClockRate, 0);

    const double bw_memcpy = measure_memcpy_bw(size_t(256) << 20);
    const double bw_kernel = measure_kernel_bw(size_t(1) << 30);
    const double bw = bw_memcpy > bw_kernel ? bw_memcpy : bw_kernel;

    std::vector<ckl::RooflinePoint> points;
    double cublas_peak = 0.0;
    for (int size : {4096, 8192}) {
        const auto ha = ckl_tools::narrowed_matrix<__nv_bfloat16>(size, size, 11, 0.02f);
        const auto hb = ckl_tools::narrowed_matrix<__nv_bfloat16>(size, size, 22, 0.02f);
        ckl::DeviceBuffer<__nv_bfloat16> da(ha.size()), db(hb.size()), dc(ha.size());
        da.copy_from_host(ha);
        db.copy_from_host(hb);
        dc.zero();
        for (int algo : {CKL_ALGO_AUTO, CKL_ALGO_UMMA_1CTA, CKL_ALGO_UMMA_2CTA, CKL_ALGO_UMMA_2CTA_WIDE}) {
            // each variant starts from an idle GPU: back to back, the later ones would be
            // measured at the lower clock the power limit imposes after ~50 launches
            cudaDeviceSynchronize();
            std::this_thread::sleep_for(std::chrono::milliseconds(700));
            const ckl::TimingStats t = ckl::time_stream([&](cudaStream_t s) {
                ckl_gemm_ex(CKL_BF16, da.data(), db.data(), dc.data(), CKL_BF16, size, size, size, size,
                            size, size, 1.0f, 0.0f, algo, s);
            });
            ckl::RooflinePoint pt;
            pt.label = std::string(ckl_algo_name(algo)) + "_bf16_" + std::to_string(size);
            pt.flops = ckl::gemm_flops(size, size, size);
            pt.bytes = ckl::gemm_bytes_ex(size, size, size, 2, 2, false);
            pt.achieved_flops_per_s = pt.flops / (t.median_ms * 1.0e-3);
            pt.tensor = true;
            points.push_back(pt);
        }
        if (size == 8192) {
            if (auto cublas = ckl_tools::find_cublas_comparator(root, true)) {
                ckl::DeviceBuffer<float> ref(static_cast<size_t>(size) * size);
                const ckl::TimingStats t = ckl::time_stream([&](cudaStream_t s) {
                    cublas(da.data(), db.data(), ref.data(), size, size, size, 1.0f, 0.0f, s);
                });
                cublas_peak = ckl::gemm_flops(size, size, size) / (t.median_ms * 1.0e-3);
            }
        }
    }
    // FP32 (CUDA-core) rung and roof: ckl_sgemm at 4096^3; the roof is SGEMM through the
    // reference's cuBLAS wrapper when that build is present, as in the reference's profiler
    // (src/profiler/roofline.cpp:40-53), else 2 FLOP x 128 lanes x SMs x boost clock.
    double fp32_peak = prop.multiProcessorCount * 256.0 * core_khz * 1.0e3;
    bool fp32_measured = false;
    {
        const int size = 4096;
        const auto ha = ckl::random_matrix(size, size, 3);
        const auto hb = ckl::random_matrix(size, size, 4);
        ckl::DeviceBuffer<float> da(ha.size()), db(hb.size()), dc(ha.size());
        da.copy_from_host(ha);
        db.copy_from_host(hb);
        dc.zero();
        const ckl::TimingStats t = ckl::time_stream([&](cudaStream_t s) {
            ckl_sgemm(da.data(), db.data(), dc.data(), size, size, size, size, size, size, 1.0f, 0.0f, s);
        });
        ckl::RooflinePoint pt;
        pt.label = "gemm_cp_async";  // the top FP32 rung's name in the reference's figure
        pt.flops = ckl::gemm_flops(size, size, size);
        pt.bytes = ckl::gemm_bytes(size, size, size, sizeof(float));
        pt.achieved_flops_per_s = pt.flops / (t.median_ms * 1.0e-3);
        pt.tensor = false;
        points.push_back(pt);
        if (auto sgemm = ckl_tools::find_sgemm_comparator(root)) {
            const ckl::TimingStats tc = ckl::time_stream([&](cudaStream_t s) {
                sgemm(da.data(), db.data(), dc.data(), size, size, size, 1.0f, 0.0f, s);
            });
            fp32_peak = ckl::gemm_flops(size, size, size) / (tc.median_ms * 1.0e-3);
            fp32_measured = true;
        }
    }
    if (ckl_device_status(nullptr) != CKL_OK) {
        std::fprintf(stderr, "ckl error: %s\n", ckl_last_error());
        return 1;
    }
    const double datasheet = 2.25e15;
    const double clock_derived = prop.multiProcessorCount * 8192.0 * core_khz * 1.0e3;
    const double tensor_peak = cublas_peak > 0.0 ? cublas_peak : datasheet;
    const double ridge = ckl::ridge_intensity(tensor_peak, bw);

    std::printf("Roofline (ceilings measured on %s)\n", prop.name);
    std::printf("  bandwidth, memcpy D2D 256 MiB : %.1f GB/s\n", bw_memcpy / 1.0e9);
    std::printf("  bandwidth, stream-copy kernel : %.1f GB/s\n", bw_kernel / 1.0e9);
    std::printf("  tensor roof used              : %.1f TFLOP/s (%s)\n", tensor_peak / 1.0e12,
                cublas_peak > 0.0 ? "cuBLAS BF16 8192^3, the reference's definition" : "datasheet");
    std::printf("  datasheet dense 16-bit        : %.1f TFLOP/s\n", datasheet / 1.0e12);
    std::printf("  SMs x 8192 x boost clock      : %.1f TFLOP/s\n", clock_derived / 1.0e12);
    std::printf("  FP32 roof                     : %.1f TFLOP/s (%s)\n", fp32_peak / 1.0e12,
                fp32_measured ? "cuBLAS SGEMM 4096^3, the reference's definition" : "lanes x clock");
    std::printf("  ridge                         : %.1f FLOP/byte\n", ridge);

    const std::string ceilings = out_dir + "/roofline_ceilings.csv";
    if (std::FILE* f = std::fopen(ceilings.c_str(), "w")) {
        std::fprintf(f, "quantity,value\nbandwidth_gbps,%.3f\nfp32_gflops,%.3f\ntensor_gflops,%.3f\n",
                     bw / 1.0e9, fp32_peak / 1.0e9, tensor_peak / 1.0e9);
        std::fprintf(f, "ridge_fp32,%.3f\n", ckl::ridge_intensity(fp32_peak, bw));
        std::fprintf(f, "tensor_gflops_datasheet,%.3f\ntensor_gflops_clock_derived,%.3f\nridge_tensor,%.3f\n",
                     datasheet / 1.0e9, clock_derived / 1.0e9, ridge);
        std::fclose(f);
    }
    const std::string csv_path = out_dir + "/roofline.csv";
    std::FILE* csv = std::fopen(csv_path.c_str(), "w");
    if (csv != nullptr) {
        std::fprintf(csv, "label,intensity_flop_per_byte,achieved_gflops,roof_gflops,ceiling,bound\n");
    }
    std::printf("%-36s %10s %12s %12s %9s %s\n", "variant", "intensity", "gflops", "roof_gflops",
                "pct_roof", "bound");
    for (const auto& p : points) {
        const double peak = p.tensor ? tensor_peak : fp32_peak;
        const double roof = ckl::roofline_flops(p.intensity(), peak, bw) / 1.0e9;
        const char* bound = p.intensity() < ckl::ridge_intensity(peak, bw) ? "memory" : "compute";
        std::printf("%-36s %10.1f %12.1f %12.1f %8.1f%% %s\n", p.label.c_str(), p.intensity(),
                    p.achieved_gflops(), roof, 100.0 * p.achieved_gflops() / roof, bound);
        if (csv != nullptr) {
            std::fprintf(csv, "%s,%.4f,%.1f,%.1f,%s,%s\n", p.label.c_str(), p.intensity(),
                         p.achieved_gflops(), roof, p.tensor ? "tensor" : "fp32", bound);
        }
    }
    if (csv != nullptr) {
        std::fclose(csv);
        std::printf("wrote %s and %s\n", csv_path.c_str(), ceilings.c_str());
    }
    return 0;
}
