#pragma once
// Host-side helpers for the C++ harness: seeded fill, the double-accumulate
// GEMM used as ground truth, and the relative Frobenius error.  Same
// functions and results as the reference's include/ckl/reference.hpp:16-63
// (the tests pin them against vectors generated from that header), written
// over raw loops with hoisted row pointers.  HARNESS ONLY: the library never
// computes on the host.

#include <cmath>
#include <cstddef>
#include <cstdint>
#include <random>
#include <vector>

namespace ckl {

// rows*cols floats, uniform in [-1, 1), from std::mt19937_64(seed), one draw
// per element in row-major order.
inline std::vector<float> random_matrix(int rows, int cols, std::uint64_t seed) {
    const std::size_t count = static_cast<std::size_t>(rows) * static_cast<std::size_t>(cols);
    std::vector<float> out;
    out.reserve(count);
    std::mt19937_64 engine(seed);
    std::uniform_real_distribution<float> uniform(-1.0f, 1.0f);
    for (std::size_t i = 0; i < count; ++i) {
        out.push_back(uniform(engine));
    }
    return out;
}

// Gaussian fill for the transformer-shaped workloads (no counterpart in the
// reference, which only draws uniform values): scale * N(0, 1).
inline std::vector<float> random_normal_matrix(int rows, int cols, std::uint64_t seed, float scale) {
    const std::size_t count = static_cast<std::size_t>(rows) * static_cast<std::size_t>(cols);
    std::vector<float> out(count);
    std::mt19937_64 engine(seed);
    std::normal_distribution<float> normal(0.0f, 1.0f);
    for (auto& v : out) {
        v = scale * normal(engine);
    }
    return out;
}

// C = alpha * A*B + beta * C_in in double, row-major, k summed in ascending order.
inline std::vector<double> gemm_reference(const std::vector<float>& a, const std::vector<float>& b,
                                          const std::vector<float>& c_in, int m, int n, int k,
                                          float alpha, float beta) {
    const std::size_t sn = static_cast<std::size_t>(n);
    const std::size_t sk = static_cast<std::size_t>(k);
    std::vector<double> c(static_cast<std::size_t>(m) * sn);
    const double da = alpha;
    const double db = beta;
    for (int i = 0; i < m; ++i) {
        const float* a_row = a.data() + static_cast<std::size_t>(i) * sk;
        for (int j = 0; j < n; ++j) {
            const float* b_col = b.data() + j;
            double sum = 0.0;
            for (std::size_t p = 0; p < sk; ++p) {
                sum += static_cast<double>(a_row[p]) * static_cast<double>(b_col[p * sn]);
            }
            const std::size_t at = static_cast<std::size_t>(i) * sn + static_cast<std::size_t>(j);
            c[at] = da * sum + db * static_cast<double>(c_in[at]);
        }
    }
    return c;
}

// ||actual - ref||_F / ||ref||_F; the plain error norm when ||ref||_F <= 1e-30.
inline double relative_frobenius_error(const std::vector<float>& actual,
                                       const std::vector<double>& ref) {
    double err2 = 0.0;
    double ref2 = 0.0;
    for (std::size_t i = 0; i < ref.size(); ++i) {
        const double d = static_cast<double>(actual[i]) - ref[i];
        err2 += d * d;
        ref2 += ref[i] * ref[i];
    }
    const double err = std::sqrt(err2);
    const double norm = std::sqrt(ref2);
    return norm > 1e-30 ? err / norm : err;
}

}  // namespace ckl
