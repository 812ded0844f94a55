#pragma once
// Error checking for CUDA runtime calls made by tests, benchmarks and tools.
// Same macro names and the same behaviour (throw std::runtime_error naming
// the failing expression and its location) as the reference's
// include/ckl/cuda_check.hpp:35-47, so harness code written against it
// compiles here unchanged.

#include <stdexcept>
#include <string>

#include <cuda_runtime.h>

namespace ckl {

inline void check_cuda(cudaError_t status, const char* expr, const char* file, int line) {
    if (status == cudaSuccess) {
        return;
    }
    std::string text = "CUDA error ";
    text += cudaGetErrorName(status);
    text += " (";
    text += cudaGetErrorString(status);
    text += "): ";
    text += expr;
    text += " at ";
    text += file;
    text += ":";
    text += std::to_string(line);
    throw std::runtime_error(text);
}

[[noreturn]] inline void fail(const char* what, const char* expr, const char* file, int line) {
    throw std::runtime_error(std::string(what) + " failed: " + expr + " at " + file + ":" +
                             std::to_string(line));
}

}  // namespace ckl

#define CKL_CUDA_CHECK(expr) ::ckl::check_cuda((expr), #expr, __FILE__, __LINE__)

#define CKL_CUDA_LAST_ERROR(sync)                                                          \
    do {                                                                                   \
        ::ckl::check_cuda(cudaGetLastError(), "kernel launch", __FILE__, __LINE__);        \
        if (sync) {                                                                        \
            ::ckl::check_cuda(cudaDeviceSynchronize(), "cudaDeviceSynchronize", __FILE__,  \
                              __LINE__);                                                   \
        }                                                                                  \
    } while (0)
