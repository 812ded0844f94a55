#pragma once
// Harness-side ground truth: seeded fill, a GEMM summed in double, and the relative Frobenius
// distance.  These reproduce, value for value, ckl::random_matrix, ckl::gemm_reference and
// ckl::relative_frobenius_error of the reference (include/ckl/reference.hpp:16-63 there); the
// test-suite pins them against vectors generated from that header.  Never used by the library
// itself, which does not compute on the host.

#include <algorithm>
#include <cmath>
#include <cstddef>
#include <cstdint>
#include <numeric>
#include <random>
#include <vector>

namespace ckl {

namespace detail {
inline std::size_t count_of(int rows, int cols) {
    return static_cast<std::size_t>(rows) * static_cast<std::size_t>(cols);
}
}  // namespace detail

// U[-1, 1) from mt19937_64(seed), row-major, one engine draw per element.
inline std::vector<float> random_matrix(int rows, int cols, std::uint64_t seed) {
    std::vector<float> m(detail::count_of(rows, cols));
    std::mt19937_64 gen{seed};
    std::uniform_real_distribution<float> unit{-1.0f, 1.0f};
    std::generate(m.begin(), m.end(), [&] { return unit(gen); });
    return m;
}

// scale * N(0, 1): the transformer-shaped workloads (the reference only draws uniforms).
inline std::vector<float> random_normal_matrix(int rows, int cols, std::uint64_t seed, float scale) {
    std::vector<float> m(detail::count_of(rows, cols));
    std::mt19937_64 gen{seed};
    std::normal_distribution<float> gauss{0.0f, 1.0f};
    std::generate(m.begin(), m.end(), [&] { return scale * gauss(gen); });
    return m;
}

// alpha * A*B + beta * C_in, every dot product accumulated in double with k ascending.
inline std::vector<double> gemm_reference(const std::vector<float>& a, const std::vector<float>& b,
                                          const std::vector<float>& c_in, int m, int n, int k,
                                          float alpha, float beta) {
    const std::size_t ncols = static_cast<std::size_t>(n), depth = static_cast<std::size_t>(k);
    std::vector<double> out(detail::count_of(m, n));
    for (std::size_t at = 0; at < out.size(); ++at) {
        const float* lhs = a.data() + (at / ncols) * depth;  // row of A
        const float* rhs = b.data() + (at % ncols);          // column of B, stride n
        double dot = 0.0;
        for (std::size_t p = 0; p < depth; ++p, rhs += ncols) {
            dot += static_cast<double>(lhs[p]) * static_cast<double>(*rhs);
        }
        out[at] = static_cast<double>(alpha) * dot +
                  static_cast<double>(beta) * static_cast<double>(c_in[at]);
    }
    return out;
}

// ||actual - ref||_F / ||ref||_F, or the numerator alone when ||ref||_F <= 1e-30.
inline double relative_frobenius_error(const std::vector<float>& actual,
                                       const std::vector<double>& ref) {
    double diff_sq = 0.0, ref_sq = 0.0;
    for (std::size_t i = 0; i < ref.size(); ++i) {
        const double delta = static_cast<double>(actual[i]) - ref[i];
        diff_sq += delta * delta;
        ref_sq += ref[i] * ref[i];
    }
    const double diff = std::sqrt(diff_sq), scale = std::sqrt(ref_sq);
    return scale > 1e-30 ? diff / scale : diff;
}

}  // namespace ckl
