#pragma once
// Shared pieces of the command-line tools: read-only NVML sampling (loaded at
// run time, so the tools link nothing but the CUDA runtime and libckl_gemm),
// host fill + narrowing, and the optional cuBLAS comparator.
//
// The sampler plays the part of the reference's NvmlMonitor
// (src/telemetry/nvml_monitor.cpp:36-144 there): a background thread reads SM
// clock, power, temperature and the clock-event reasons and the run is flagged
// when a slowdown reason was seen.  It only ever READS device state.

#include <atomic>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <string>
#include <thread>
#include <vector>

#include <dlfcn.h>

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "ckl/reference.hpp"

namespace ckl_tools {

struct NvmlSummary {
    bool available = false;
    double median_sm_clock_mhz = 0.0;
    unsigned max_temperature_c = 0;
    double max_power_w = 0.0;
    bool throttled = false;  // hw slowdown or thermal slowdown seen (power cap alone is not)
    bool power_capped = false;
    int samples = 0;
};

class NvmlSampler {
public:
    explicit NvmlSampler(int device_index, int period_ms = 25) : period_ms_(period_ms) {
        lib_ = dlopen("libnvidia-ml.so.1", RTLD_NOW);
        if (lib_ == nullptr) {
            return;
        }
        auto init = reinterpret_cast<int (*)()>(dlsym(lib_, "nvmlInit_v2"));
        auto handle = reinterpret_cast<int (*)(unsigned, void**)>(
            dlsym(lib_, "nvmlDeviceGetHandleByIndex_v2"));
        clock_ = reinterpret_cast<int (*)(void*, int, unsigned*)>(dlsym(lib_, "nvmlDeviceGetClockInfo"));
        power_ = reinterpret_cast<int (*)(void*, unsigned*)>(dlsym(lib_, "nvmlDeviceGetPowerUsage"));
        temp_ = reinterpret_cast<int (*)(void*, int, unsigned*)>(dlsym(lib_, "nvmlDeviceGetTemperature"));
        reasons_ = reinterpret_cast<int (*)(void*, unsigned long long*)>(
            dlsym(lib_, "nvmlDeviceGetCurrentClocksThrottleReasons"));
        if (init == nullptr || handle == nullptr || clock_ == nullptr || init() != 0 ||
            handle(static_cast<unsigned>(device_index), &dev_) != 0) {
            return;
        }
        ok_ = true;
    }
    ~NvmlSampler() {
        stop();
    }
    void start() {
        if (!ok_) {
            return;
        }
        running_ = true;
        thread_ = std::thread([this] {
            while (running_) {
                unsigned mhz = 0, mw = 0, temp = 0;
                unsigned long long why = 0;
                if (clock_(dev_, 1 /* NVML_CLOCK_SM */, &mhz) == 0) {
                    clocks_.push_back(mhz);
                }
                if (power_ != nullptr && power_(dev_, &mw) == 0 && mw / 1000.0 > max_w_) {
                    max_w_ = mw / 1000.0;
                }
                if (temp_ != nullptr && temp_(dev_, 0, &temp) == 0 && temp > max_t_) {
                    max_t_ = temp;
                }
                if (reasons_ != nullptr && reasons_(dev_, &why) == 0) {
                    mask_ |= why;
                }
                std::this_thread::sleep_for(std::chrono::milliseconds(period_ms_));
            }
        });
    }
    NvmlSummary stop() {
        NvmlSummary s;
        if (thread_.joinable()) {
            running_ = false;
            thread_.join();
        }
        s.available = ok_;
        s.samples = static_cast<int>(clocks_.size());
        if (!clocks_.empty()) {
            std::vector<unsigned> sorted = clocks_;
            std::sort(sorted.begin(), sorted.end());
            s.median_sm_clock_mhz = sorted[sorted.size() / 2];
        }
        s.max_temperature_c = max_t_;
        s.max_power_w = max_w_;
        s.throttled = (mask_ & (0x8ull | 0x20ull | 0x40ull | 0x80ull)) != 0;
        s.power_capped = (mask_ & 0x4ull) != 0;
        return s;
    }

private:
    int period_ms_;
    void* lib_ = nullptr;
    void* dev_ = nullptr;
    bool ok_ = false;
    int (*clock_)(void*, int, unsigned*) = nullptr;
    int (*power_)(void*, unsigned*) = nullptr;
    int (*temp_)(void*, int, unsigned*) = nullptr;
    int (*reasons_)(void*, unsigned long long*) = nullptr;
    std::atomic<bool> running_{false};
    std::thread thread_;
    std::vector<unsigned> clocks_;
    double max_w_ = 0.0;
    unsigned max_t_ = 0;
    unsigned long long mask_ = 0;
};

// Host fill with the reference generator, narrowed to 16 bits (round to nearest even).
template <typename T>
std::vector<T> narrowed_matrix(int rows, int cols, std::uint64_t seed, float scale = 1.0f) {
    const std::vector<float> f = ckl::random_matrix(rows, cols, seed);
    std::vector<T> out(f.size());
    for (std::size_t i = 0; i < f.size(); ++i) {
        if constexpr (sizeof(T) == 2 && std::is_same<T, __half>::value) {
            out[i] = __float2half(scale * f[i]);
        } else {
            out[i] = __float2bfloat16(scale * f[i]);
        }
    }
    return out;
}

// Optional comparator: the reference's cuBLAS wrappers, if its build for this GPU sits in
// oracle/_ref (never linked; looked up at run time so the tools work without it).
using CublasFn16 = void (*)(const void*, const void*, float*, int, int, int, float, float,
                            cudaStream_t);
inline CublasFn16 find_cublas_comparator(const std::string& repo_root, bool bf16) {
    const std::string path = repo_root + "/oracle/_ref/libckl_ref_gemm.so";
    void* lib = dlopen(path.c_str(), RTLD_NOW | RTLD_LOCAL);
    if (lib == nullptr) {
        return nullptr;
    }
    const char* name = bf16 ? "_ZN3ckl16gemm_cublas_bf16EPK13__nv_bfloat16S2_PfiiiffP11CUstream_st"
                            : "_ZN3ckl16gemm_cublas_fp16EPK6__halfS2_PfiiiffP11CUstream_st";
    return reinterpret_cast<CublasFn16>(dlsym(lib, name));
}

// The reference's SGEMM wrapper (ckl::gemm_cublas, src/gemm/cublas_gemm.cpp), same lookup.
using CublasFn32 = void (*)(const float*, const float*, float*, int, int, int, float, float,
                            cudaStream_t);
inline CublasFn32 find_sgemm_comparator(const std::string& repo_root) {
    const std::string path = repo_root + "/oracle/_ref/libckl_ref_gemm.so";
    void* lib = dlopen(path.c_str(), RTLD_NOW | RTLD_LOCAL);
    if (lib == nullptr) {
        return nullptr;
    }
    return reinterpret_cast<CublasFn32>(dlsym(lib, "_ZN3ckl11gemm_cublasEPKfS1_PfiiiffP11CUstream_st"));
}

// The reference's STRSM wrapper (ckl::trsm_cublas, src/trsm/cublas_trsm.cpp), same lookup.
using CublasTrsmFn = void (*)(const float*, float*, int, int, float, cudaStream_t);
inline CublasTrsmFn find_trsm_comparator(const std::string& repo_root) {
    const std::string path = repo_root + "/oracle/_ref/libckl_ref_gemm.so";
    void* lib = dlopen(path.c_str(), RTLD_NOW | RTLD_LOCAL);
    if (lib == nullptr) {
        return nullptr;
    }
    return reinterpret_cast<CublasTrsmFn>(dlsym(lib, "_ZN3ckl11trsm_cublasEPKfPfiifP11CUstream_st"));
}

}  // namespace ckl_tools
