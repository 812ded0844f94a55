// bench_all: one configuration in, one JSON row out.
//
// GEMM family of the reference's benchmarks/bench_all.cpp:70-130,248-303 (the
// other families are outside this library).  Same command line
//     bench_all gemm <variant> <dtype> <m> <n> <k> [commit]
// and the same keys in the row, plus tflops, percent of the datasheet dense
// 16-bit peak, the C dtype and the GPU count, which the sweep's resume key uses.
//   variant: auto | simt | umma_1cta | umma_1cta_streamk | umma_2cta |
//            umma_2cta_streamk | umma_2cta_wide | umma_2cta_wide_streamk |
//            umma_1cta_n128 | umma_1cta_n128_streamk
//   dtype  : fp16 | bf16 (FP32 C, as the reference measures) or fp16_c16 | bf16_c16;
//            fp32 with variant sgemm = the CUDA-core kernel behind the reference's FP32 rungs
//     bench_all trsm blocked fp32 <m> <n> 0 [commit]   (the reference's trsm family, line 132-170)
//     bench_all cpu reference fp32 <m> <n> <k> [commit]   the CPU GEMM of ckl/reference.hpp
//            (the reference's include/ckl/reference.hpp:29-46: one thread, double accumulate)
//            timed once on the host: the CPU baseline column of the sweep; no GPU is touched
// Protocol: seeds 11 and 22, alpha 1, beta 0, 5 warm-ups, 20 timed launches, median.
// The baseline column is the reference's cuBLAS wrapper when oracle/_ref holds its build.

#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <string>

#include "ckl/device_buffer.hpp"
#include "ckl/event_timer.hpp"
#include "ckl/gemm.hpp"
#include "ckl/reference.hpp"
#include "harness.hpp"

namespace {

int algo_from_name(const std::string& name) {
    for (int a = 0; a <= CKL_ALGO_UMMA_1CTA_N128_SK; ++a) {
        if (name == ckl_algo_name(a)) {
            return a;
        }
    }
    return -1;
}

struct Result {
    bool ok = false;
    double median_ms = 0, iqr_ms = 0, gflops = 0, baseline_gflops = 0;
};

template <typename T>
Result run(int algo, bool c16, bool bf16, int m, int n, int k, const std::string& root) {
    Result r;
    const auto ha = ckl_tools::narrowed_matrix<T>(m, k, 11);
    const auto hb = ckl_tools::narrowed_matrix<T>(k, n, 22);
    ckl::DeviceBuffer<T> da(ha.size()), db(hb.size());
    da.copy_from_host(ha);
    db.copy_from_host(hb);
    ckl::DeviceBuffer<float> dc32(c16 ? 0 : static_cast<size_t>(m) * n);
    ckl::DeviceBuffer<T> dc16(c16 ? static_cast<size_t>(m) * n : 0);
    dc32.zero();
    dc16.zero();
    const int ab = bf16 ? CKL_BF16 : CKL_F16;
    const int cd = c16 ? ab : CKL_F32;
    void* c = c16 ? static_cast<void*>(dc16.data()) : static_cast<void*>(dc32.data());
    int status = CKL_OK;
    const ckl::TimingStats ks = ckl::time_stream([&](cudaStream_t s) {
        const int rc = ckl_gemm_ex(ab, da.data(), db.data(), c, cd, m, n, k, k, n, n, 1.0f, 0.0f, algo, s);
        if (rc != CKL_OK) {
            status = rc;
        }
    });
    if (status != CKL_OK || ckl_device_status(nullptr) != CKL_OK) {
        std::fprintf(stderr, "ckl error: %s\n", ckl_last_error());
        return r;
    }
    r.ok = true;
    r.median_ms = ks.median_ms;
    r.iqr_ms = ks.iqr_ms;
    r.gflops = ckl::gemm_gflops(m, n, k, ks.median_ms);
    if (auto cublas = ckl_tools::find_cublas_comparator(root, bf16)) {
        ckl::DeviceBuffer<float> ref(static_cast<size_t>(m) * n);
        const ckl::TimingStats os = ckl::time_stream(
            [&](cudaStream_t s) { cublas(da.data(), db.data(), ref.data(), m, n, k, 1.0f, 0.0f, s); });
        r.baseline_gflops = ckl::gemm_gflops(m, n, k, os.median_ms);
    }
    return r;
}

Result run_fp32(int m, int n, int k, const std::string& root) {
    Result r;
    const auto ha = ckl::random_matrix(m, k, 11);
    const auto hb = ckl::random_matrix(k, n, 22);
    ckl::DeviceBuffer<float> da(ha.size()), db(hb.size()), dc(static_cast<size_t>(m) * n);
    da.copy_from_host(ha);
    db.copy_from_host(hb);
    dc.zero();
    int status = CKL_OK;
    const ckl::TimingStats ks = ckl::time_stream([&](cudaStream_t s) {
        const int rc = ckl_sgemm(da.data(), db.data(), dc.data(), m, n, k, k, n, n, 1.0f, 0.0f, s);
        if (rc != CKL_OK) {
            status = rc;
        }
    });
    if (status != CKL_OK) {
        std::fprintf(stderr, "ckl error: %s\n", ckl_last_error());
        return r;
    }
    r.ok = true;
    r.median_ms = ks.median_ms;
    r.iqr_ms = ks.iqr_ms;
    r.gflops = ckl::gemm_gflops(m, n, k, ks.median_ms);
    if (auto sgemm = ckl_tools::find_sgemm_comparator(root)) {
        const ckl::TimingStats os = ckl::time_stream(
            [&](cudaStream_t s) { sgemm(da.data(), db.data(), dc.data(), m, n, k, 1.0f, 0.0f, s); });
        r.baseline_gflops = ckl::gemm_gflops(m, n, k, os.median_ms);
    }
    return r;
}

// L X = alpha B with the diagonally dominant L of the reference's TRSM test
// (tests/test_trsm.cpp:20-31); m*m*n flops.  B is restored before every timed solve by a
// device copy inside the timed lambda (the solve is in place), as the reference's row does.
Result run_trsm(int m, int n, const std::string& root) {
    Result r;
    auto hl = ckl::random_matrix(m, m, 11);
    for (int i = 0; i < m; ++i) {
        for (int j = i + 1; j < m; ++j) {
            hl[static_cast<size_t>(i) * m + j] = 0.0f;
        }
        hl[static_cast<size_t>(i) * m + i] = static_cast<float>(m + 1);
    }
    const auto hb = ckl::random_matrix(m, n, 22);
    ckl::DeviceBuffer<float> dl(hl.size()), db0(hb.size()), db(hb.size());
    dl.copy_from_host(hl);
    db0.copy_from_host(hb);
    int status = CKL_OK;
    const ckl::TimingStats ks = ckl::time_stream([&](cudaStream_t s) {
        cudaMemcpyAsync(db.data(), db0.data(), hb.size() * sizeof(float), cudaMemcpyDeviceToDevice, s);
        const int rc = ckl_strsm_lower(dl.data(), db.data(), m, n, m, n, 1.0f, s);
        if (rc != CKL_OK) {
            status = rc;
        }
    });
    if (status != CKL_OK) {
        std::fprintf(stderr, "ckl error: %s\n", ckl_last_error());
        return r;
    }
    r.ok = true;
    r.median_ms = ks.median_ms;
    r.iqr_ms = ks.iqr_ms;
    r.gflops = static_cast<double>(m) * m * n / (ks.median_ms * 1.0e6);
    if (auto strsm = ckl_tools::find_trsm_comparator(root)) {
        const ckl::TimingStats os = ckl::time_stream([&](cudaStream_t s) {
            cudaMemcpyAsync(db.data(), db0.data(), hb.size() * sizeof(float), cudaMemcpyDeviceToDevice, s);
            strsm(dl.data(), db.data(), m, n, 1.0f, s);
        });
        r.baseline_gflops = static_cast<double>(m) * m * n / (os.median_ms * 1.0e6);
    }
    return r;
}

}  // namespace

int main(int argc, char** argv) {
    const std::string family = argc > 1 ? argv[1] : "";
    if (argc < 7 || (family != "gemm" && family != "trsm" && family != "cpu")) {
        std::fprintf(stderr, "usage: %s gemm|trsm|cpu <variant> <dtype> <m> <n> <k> [commit]\n", argv[0]);
        return 2;
    }
    const std::string variant = argv[2], dtype = argv[3];
    const int m = std::atoi(argv[4]), n = std::atoi(argv[5]), k = std::atoi(argv[6]);
    const std::string commit = argc > 7 ? argv[7] : "unknown";
    if (family == "cpu") {
        if (variant != "reference" || dtype != "fp32" || m <= 0 || n <= 0 || k <= 0) {
            std::fprintf(stderr, "cpu family: bench_all cpu reference fp32 <m> <n> <k>\n");
            return 3;
        }
        const auto ha = ckl::random_matrix(m, k, 11);
        const auto hb = ckl::random_matrix(k, n, 22);
        const std::vector<float> hc(static_cast<size_t>(m) * n, 0.0f);
        const auto t0 = std::chrono::steady_clock::now();
        const auto ref = ckl::gemm_reference(ha, hb, hc, m, n, k, 1.0f, 0.0f);
        const double ms = std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - t0).count();
        std::printf("{\"family\":\"cpu\",\"variant\":\"reference\",\"dtype\":\"fp32\",\"m\":%d,\"n\":%d,"
                    "\"k\":%d,\"gpus\":0,\"median_ms\":%.6f,\"gflops\":%.4f,\"cpu_cores\":1,"
                    "\"checksum\":%.6e,\"commit\":\"%s\"}\n",
                    m, n, k, ms, ckl::gemm_gflops(m, n, k, ms), ref[0] + ref[ref.size() - 1],
                    commit.c_str());
        return 0;
    }
    const char* root_env = std::getenv("CKL_REPO_ROOT");
    const std::string root = root_env ? root_env : ".";
    const bool fp32 = dtype == "fp32";
    const int algo = fp32 ? 0 : algo_from_name(variant);
    const bool bf16 = dtype.rfind("bf16", 0) == 0;
    const bool c16 = dtype.find("_c16") != std::string::npos;
    if (fp32 ? (family == "gemm" ? variant != "sgemm" : variant != "blocked")
             : (family != "gemm" || algo < 0 || (!bf16 && dtype.rfind("fp16", 0) != 0))) {
        std::fprintf(stderr, "unknown variant %s or dtype %s\n", variant.c_str(), dtype.c_str());
        return 3;
    }
    int device = 0;
    cudaGetDevice(&device);
    ckl_tools::NvmlSampler monitor(device);
    monitor.start();
    Result r;
    try {
        r = family == "trsm" ? run_trsm(m, n, root)
            : fp32           ? run_fp32(m, n, k, root)
            : bf16           ? run<__nv_bfloat16>(algo, c16, true, m, n, k, root)
                             : run<__half>(algo, c16, false, m, n, k, root);
    } catch (const std::exception& e) {
        std::fprintf(stderr, "%s\n", e.what());
    }
    const ckl_tools::NvmlSummary nv = monitor.stop();
    if (!r.ok) {
        return 3;
    }
    int rt = 0, drv = 0;
    cudaRuntimeGetVersion(&rt);
    cudaDriverGetVersion(&drv);
    const double pct = r.baseline_gflops > 0.0 ? 100.0 * r.gflops / r.baseline_gflops : 0.0;
    std::printf(
        "{\"family\":\"%s\",\"variant\":\"%s\",\"dtype\":\"%s\",\"m\":%d,\"n\":%d,\"k\":%d,"
        "\"gpus\":1,\"median_ms\":%.6f,\"iqr_ms\":%.6f,\"gflops\":%.3f,\"tflops\":%.3f,"
        "\"pct_peak_datasheet\":%.2f,\"baseline_gflops\":%.3f,\"pct_baseline\":%.2f,"
        "\"nvml_available\":%s,\"median_sm_clock_mhz\":%.0f,\"max_temp_c\":%u,\"max_power_w\":%.1f,"
        "\"throttled\":%s,\"power_capped\":%s,\"nvml_samples\":%d,\"cuda_runtime\":%d,"
        "\"cuda_driver\":%d,\"commit\":\"%s\"}\n",
        family.c_str(), variant.c_str(), dtype.c_str(), m, n, k, r.median_ms, r.iqr_ms, r.gflops,
        r.gflops / 1000.0,
        100.0 * r.gflops / 2.25e6, r.baseline_gflops, pct, nv.available ? "true" : "false",
        nv.median_sm_clock_mhz, nv.max_temperature_c, nv.max_power_w, nv.throttled ? "true" : "false",
        nv.power_capped ? "true" : "false", nv.samples, rt, drv, commit.c_str());
    return 0;
}
