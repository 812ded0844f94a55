#pragma once
// Roofline arithmetic for the GEMM path: work and minimum-traffic counts, the
// attainable rate under a (bandwidth, compute) pair, and where the two roofs
// meet.  Same names as the reference's include/ckl/roofline.hpp:17-57 for the
// GEMM parts; the byte model is extended with distinct input/output element
// sizes and the read of C that a non-zero beta costs, which the reference's
// single-element-size model leaves out.

#include <cstddef>
#include <string>

namespace ckl {

// Ceilings measured on the machine at hand (bytes/s and FLOP/s), never datasheet values.
struct MachineCeilings {
    double bandwidth_bytes_per_s;
    double fp32_flops_per_s;
    double tensor_flops_per_s;
};

struct RooflinePoint {
    std::string label;
    double flops;
    double bytes;
    double achieved_flops_per_s;
    bool tensor;

    double intensity() const { return bytes > 0.0 ? flops / bytes : 0.0; }
    double achieved_gflops() const { return achieved_flops_per_s * 1.0e-9; }
};

inline double ridge_intensity(double flops_per_s, double bandwidth_bytes_per_s) {
    return bandwidth_bytes_per_s > 0.0 ? flops_per_s / bandwidth_bytes_per_s : 0.0;
}

inline double roofline_flops(double intensity, double flops_per_s, double bandwidth_bytes_per_s) {
    const double memory_roof = intensity * bandwidth_bytes_per_s;
    return memory_roof < flops_per_s ? memory_roof : flops_per_s;
}

inline double gemm_flops(int m, int n, int k) { return 2.0 * double(m) * double(n) * double(k); }

// One element size for everything (the reference's model).
inline double gemm_bytes(int m, int n, int k, std::size_t element_size) {
    return (double(m) * k + double(k) * n + double(m) * n) * double(element_size);
}

// Algorithmic bytes of C = alpha*A*B + beta*C: A and B read once, C written
// once and also read once when beta != 0.
inline double gemm_bytes_ex(int m, int n, int k, std::size_t in_size, std::size_t out_size,
                            bool reads_c) {
    const double in = (double(m) * k + double(k) * n) * double(in_size);
    const double out = double(m) * n * double(out_size) * (reads_c ? 2.0 : 1.0);
    return in + out;
}

}  // namespace ckl
