#pragma once
// time_stream(): the reference's timing protocol (include/ckl/event_timer.hpp:28-78 there),
// warm-ups, then `reps` launches each bracketed by its own CUDA event pair, summarised as
// median, interquartile range and minimum in milliseconds.  Each launch is waited for before
// the next one starts, as in the reference.

#include <algorithm>
#include <cstddef>
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

class EventPair {
    cudaEvent_t begin_{}, end_{};

public:
    EventPair() {
        CKL_CUDA_CHECK(cudaEventCreate(&begin_));
        CKL_CUDA_CHECK(cudaEventCreate(&end_));
    }
    EventPair(const EventPair&) = delete;
    EventPair& operator=(const EventPair&) = delete;
    ~EventPair() {
        cudaEventDestroy(begin_);
        cudaEventDestroy(end_);
    }
    template <typename F>
    double time_ms(F&& work, cudaStream_t stream) {
        CKL_CUDA_CHECK(cudaEventRecord(begin_, stream));
        work(stream);
        CKL_CUDA_CHECK(cudaEventRecord(end_, stream));
        CKL_CUDA_CHECK(cudaEventSynchronize(end_));
        float ms = 0.0f;
        CKL_CUDA_CHECK(cudaEventElapsedTime(&ms, begin_, end_));
        return ms;
    }
};

// Quantile of an ascending sample with linear interpolation between neighbours.
inline double quantile(const std::vector<double>& sorted, double frac) {
    if (sorted.empty()) return 0.0;
    const double at = frac * static_cast<double>(sorted.size() - 1);
    const std::size_t below = static_cast<std::size_t>(at);
    const std::size_t above = std::min(below + 1, sorted.size() - 1);
    return sorted[below] + (sorted[above] - sorted[below]) * (at - static_cast<double>(below));
}

}  // namespace detail

inline TimingStats time_stream(const std::function<void(cudaStream_t)>& launch,
                               cudaStream_t stream = nullptr, int warmups = 5, int reps = 20) {
    for (int i = 0; i < warmups; ++i) launch(stream);
    CKL_CUDA_CHECK(cudaStreamSynchronize(stream));

    detail::EventPair events;
    std::vector<double> ms;
    ms.reserve(static_cast<std::size_t>(reps > 0 ? reps : 0));
    while (static_cast<int>(ms.size()) < reps) ms.push_back(events.time_ms(launch, stream));
    std::sort(ms.begin(), ms.end());

    TimingStats out;
    out.reps = reps;
    if (!ms.empty()) {
        out.min_ms = ms.front();
        out.median_ms = detail::quantile(ms, 0.5);
        out.iqr_ms = detail::quantile(ms, 0.75) - detail::quantile(ms, 0.25);
    }
    return out;
}

// GFLOP/s of an m x n x k GEMM (2 FLOP per multiply-add) that took `ms` milliseconds.
inline double gemm_gflops(int m, int n, int k, double ms) {
    const double flop = 2.0 * double(m) * double(n) * double(k);
    return flop / ms * 1.0e-6;
}

}  // namespace ckl
