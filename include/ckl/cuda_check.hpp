#pragma once
// CKL_CUDA_CHECK / CKL_CUDA_LAST_ERROR for harness code (tests, benchmarks, tools).
// Names and behaviour follow the reference's include/ckl/cuda_check.hpp:35-47: a failing
// runtime call becomes a std::runtime_error that names the call and where it was made.

#include <sstream>
#include <stdexcept>

#include <cuda_runtime.h>

namespace ckl {

[[noreturn]] inline void fail(const char* what, const char* expr, const char* file, int line) {
    std::ostringstream os;
    os << what << " failed: " << expr << " at " << file << ':' << line;
    throw std::runtime_error(os.str());
}

inline void check_cuda(cudaError_t status, const char* expr, const char* file, int line) {
    if (status != cudaSuccess) {
        std::ostringstream os;
        os << "CUDA error " << cudaGetErrorName(status) << " (" << cudaGetErrorString(status)
           << "): " << expr << " at " << file << ':' << line;
        throw std::runtime_error(os.str());
    }
}

inline void check_last_error(bool also_sync, const char* file, int line) {
    check_cuda(cudaGetLastError(), "kernel launch", file, line);
    if (also_sync) check_cuda(cudaDeviceSynchronize(), "cudaDeviceSynchronize", file, line);
}

}  // namespace ckl

#define CKL_CUDA_CHECK(expr) ::ckl::check_cuda((expr), #expr, __FILE__, __LINE__)
#define CKL_CUDA_LAST_ERROR(sync) ::ckl::check_last_error((sync), __FILE__, __LINE__)
