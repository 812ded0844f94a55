#pragma once
// DeviceBuffer<T>: test/benchmark helper that owns `size()` elements of device memory.
// Interface of the reference's include/ckl/device_buffer.hpp:18-88 so its drivers compile
// unchanged; built here on std::unique_ptr with a cudaFree deleter.  All copies block.

#include <cstddef>
#include <memory>
#include <vector>

#include <cuda_runtime.h>

#include "cuda_check.hpp"

namespace ckl {

namespace detail {
struct CudaFreeDeleter {
    void operator()(void* p) const noexcept {
        if (p) cudaFree(p);
    }
};
inline std::unique_ptr<void, CudaFreeDeleter> device_alloc(std::size_t nbytes) {
    void* raw = nullptr;
    if (nbytes) CKL_CUDA_CHECK(cudaMalloc(&raw, nbytes));
    return std::unique_ptr<void, CudaFreeDeleter>(raw);
}
}  // namespace detail

template <typename T>
class DeviceBuffer {
    std::unique_ptr<void, detail::CudaFreeDeleter> mem_;
    std::size_t elems_ = 0;

public:
    DeviceBuffer() = default;
    explicit DeviceBuffer(std::size_t count)
        : mem_(detail::device_alloc(count * sizeof(T))), elems_(count) {}
    DeviceBuffer(DeviceBuffer&& other) noexcept
        : mem_(std::move(other.mem_)), elems_(other.elems_) {
        other.elems_ = 0;
    }
    DeviceBuffer& operator=(DeviceBuffer&& other) noexcept {
        mem_ = std::move(other.mem_);
        elems_ = other.elems_;
        other.elems_ = 0;
        return *this;
    }

    std::size_t size() const { return elems_; }
    std::size_t bytes() const { return sizeof(T) * elems_; }
    T* data() { return static_cast<T*>(mem_.get()); }
    const T* data() const { return static_cast<const T*>(mem_.get()); }

    void zero() {
        if (elems_) CKL_CUDA_CHECK(cudaMemset(mem_.get(), 0, bytes()));
    }
    void copy_from_host(const T* src, std::size_t count) {
        CKL_CUDA_CHECK(cudaMemcpy(mem_.get(), src, sizeof(T) * count, cudaMemcpyHostToDevice));
    }
    void copy_from_host(const std::vector<T>& src) { copy_from_host(src.data(), src.size()); }
    void copy_to_host(T* dst, std::size_t count) const {
        CKL_CUDA_CHECK(cudaMemcpy(dst, mem_.get(), sizeof(T) * count, cudaMemcpyDeviceToHost));
    }
    std::vector<T> to_host() const {
        std::vector<T> host(elems_);
        if (elems_) copy_to_host(host.data(), elems_);
        return host;
    }
};

}  // namespace ckl
