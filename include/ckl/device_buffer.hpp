#pragma once
// Move-only owner of a device allocation, for tests and benchmarks.  Interface
// of the reference's include/ckl/device_buffer.hpp:18-88 (data, size, bytes,
// copy_from_host, copy_to_host, to_host, zero); copies are synchronous.

#include <cstddef>
#include <utility>
#include <vector>

#include <cuda_runtime.h>

#include "cuda_check.hpp"

namespace ckl {

template <typename T>
class DeviceBuffer {
public:
    DeviceBuffer() = default;
    explicit DeviceBuffer(std::size_t count) : n_(count) {
        if (n_ != 0) {
            CKL_CUDA_CHECK(cudaMalloc(reinterpret_cast<void**>(&p_), n_ * sizeof(T)));
        }
    }
    DeviceBuffer(const DeviceBuffer&) = delete;
    DeviceBuffer& operator=(const DeviceBuffer&) = delete;
    DeviceBuffer(DeviceBuffer&& o) noexcept { swap(o); }
    DeviceBuffer& operator=(DeviceBuffer&& o) noexcept {
        if (this != &o) {
            release();
            swap(o);
        }
        return *this;
    }
    ~DeviceBuffer() { release(); }

    T* data() { return p_; }
    const T* data() const { return p_; }
    std::size_t size() const { return n_; }
    std::size_t bytes() const { return n_ * sizeof(T); }

    void copy_from_host(const T* host, std::size_t count) {
        CKL_CUDA_CHECK(cudaMemcpy(p_, host, count * sizeof(T), cudaMemcpyHostToDevice));
    }
    void copy_from_host(const std::vector<T>& host) { copy_from_host(host.data(), host.size()); }
    void copy_to_host(T* host, std::size_t count) const {
        CKL_CUDA_CHECK(cudaMemcpy(host, p_, count * sizeof(T), cudaMemcpyDeviceToHost));
    }
    std::vector<T> to_host() const {
        std::vector<T> out(n_);
        copy_to_host(out.data(), n_);
        return out;
    }
    void zero() {
        if (n_ != 0) {
            CKL_CUDA_CHECK(cudaMemset(p_, 0, bytes()));
        }
    }

private:
    void swap(DeviceBuffer& o) noexcept {
        std::swap(p_, o.p_);
        std::swap(n_, o.n_);
    }
    void release() noexcept {
        if (p_ != nullptr) {
            cudaFree(p_);
        }
        p_ = nullptr;
        n_ = 0;
    }
    T* p_ = nullptr;
    std::size_t n_ = 0;
};

}  // namespace ckl
