#pragma once
// CUDA-event timing with the reference's protocol (include/ckl/event_timer.hpp:28-78):
// warm-up launches, then `reps` individually timed launches; report the
// median, the interquartile range and the minimum, in milliseconds.

#include <algorithm>
#include <functional>
#include <vector>

#include <cuda_runtime.h>

#include "cuda_check.hpp"

namespace ckl {

struct TimingStats {
    double median_ms = 0.0;
    double iqr_ms = 0.0;
    double min_ms = 0.0;
    int reps = 0;
};

namespace detail {
// Linear-interpolated quantile of an ascending sample.
inline double quantile(const std::vector<double>& sorted, double frac) {
    if (sorted.empty()) {
        return 0.0;
    }
    const double pos = frac * static_cast<double>(sorted.size() - 1);
    const std::size_t lo = static_cast<std::size_t>(pos);
    const std::size_t hi = std::min(lo + 1, sorted.size() - 1);
    const double w = pos - static_cast<double>(lo);
    return sorted[lo] * (1.0 - w) + sorted[hi] * w;
}
}  // namespace detail

inline TimingStats time_stream(const std::function<void(cudaStream_t)>& launch,
                               cudaStream_t stream = nullptr, int warmups = 5, int reps = 20) {
    cudaEvent_t t0, t1;
    CKL_CUDA_CHECK(cudaEventCreate(&t0));
    CKL_CUDA_CHECK(cudaEventCreate(&t1));
    for (int w = 0; w < warmups; ++w) {
        launch(stream);
    }
    CKL_CUDA_CHECK(cudaStreamSynchronize(stream));
    std::vector<double> ms(static_cast<std::size_t>(reps), 0.0);
    for (auto& sample : ms) {
        CKL_CUDA_CHECK(cudaEventRecord(t0, stream));
        launch(stream);
        CKL_CUDA_CHECK(cudaEventRecord(t1, stream));
        CKL_CUDA_CHECK(cudaEventSynchronize(t1));
        float elapsed = 0.0f;
        CKL_CUDA_CHECK(cudaEventElapsedTime(&elapsed, t0, t1));
        sample = elapsed;
    }
    CKL_CUDA_CHECK(cudaEventDestroy(t0));
    CKL_CUDA_CHECK(cudaEventDestroy(t1));
    std::sort(ms.begin(), ms.end());
    TimingStats out;
    out.reps = reps;
    out.min_ms = ms.empty() ? 0.0 : ms.front();
    out.median_ms = detail::quantile(ms, 0.5);
    out.iqr_ms = detail::quantile(ms, 0.75) - detail::quantile(ms, 0.25);
    return out;
}

// 2*m*n*k floating-point operations over `ms` milliseconds, in GFLOP/s.
inline double gemm_gflops(int m, int n, int k, double ms) {
    return 2.0 * double(m) * double(n) * double(k) / (ms * 1.0e-3) * 1.0e-9;
}

}  // namespace ckl
