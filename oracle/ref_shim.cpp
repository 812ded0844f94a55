// C-linkage shim around the REFERENCE library's own host header.  TEST
// INFRASTRUCTURE ONLY: nothing in the shipped library links this.
//
// It is compiled against the reference source tree where it lies (the header
// is found through -I<reference>/include; no reference source is copied into
// this repository) and produces oracle/_ref/libckl_ref.so.  The functions
// below forward to ckl::random_matrix, ckl::gemm_reference and
// ckl::relative_frobenius_error (include/ckl/reference.hpp:16-63 of the
// reference) so that the plain-C restatement in ckl_oracle.c can be checked
// against the real thing, and so the benchmark can time the reference's own
// CPU GEMM.

#include <cstddef>
#include <cstdint>
#include <cstring>
#include <vector>

#include "ckl/reference.hpp"

extern "C" {

void ckl_ref_random_matrix(int rows, int cols, std::uint64_t seed, float* out) {
    const std::vector<float> v = ckl::random_matrix(rows, cols, seed);
    if (!v.empty()) {
        std::memcpy(out, v.data(), v.size() * sizeof(float));
    }
}

void ckl_ref_gemm_reference(const float* a, const float* b, const float* c_in, int m, int n, int k,
                            float alpha, float beta, double* c_out) {
    const std::size_t sm = static_cast<std::size_t>(m);
    const std::size_t sn = static_cast<std::size_t>(n);
    const std::size_t sk = static_cast<std::size_t>(k);
    const std::vector<float> va(a, a + sm * sk);
    const std::vector<float> vb(b, b + sk * sn);
    const std::vector<float> vc(c_in, c_in + sm * sn);
    const std::vector<double> out = ckl::gemm_reference(va, vb, vc, m, n, k, alpha, beta);
    if (!out.empty()) {
        std::memcpy(c_out, out.data(), out.size() * sizeof(double));
    }
}

double ckl_ref_relative_frobenius_error(const float* actual, const double* ref, std::size_t count) {
    const std::vector<float> va(actual, actual + count);
    const std::vector<double> vr(ref, ref + count);
    return ckl::relative_frobenius_error(va, vr);
}

// Timing helper: B is converted to the std::vector the reference function takes ONCE, so a
// timed call measures ckl::gemm_reference itself and not a 256 MB copy.  Several threads
// may run on one handle at the same time, each on its own block of rows (B is read-only).
struct RefBench {
    std::vector<float> b;
    int n;
    int k;
};

void* ckl_ref_bench_create(const float* b, int k, int n) {
    auto* h = new RefBench;
    h->b.assign(b, b + static_cast<std::size_t>(k) * static_cast<std::size_t>(n));
    h->n = n;
    h->k = k;
    return h;
}

void ckl_ref_bench_run(void* handle, const float* a_rows, const float* c_rows, int rows, float alpha,
                       float beta, double* c_out) {
    const auto* h = static_cast<const RefBench*>(handle);
    const std::vector<float> va(a_rows, a_rows + static_cast<std::size_t>(rows) * h->k);
    const std::vector<float> vc(c_rows, c_rows + static_cast<std::size_t>(rows) * h->n);
    const std::vector<double> out = ckl::gemm_reference(va, h->b, vc, rows, h->n, h->k, alpha, beta);
    std::memcpy(c_out, out.data(), out.size() * sizeof(double));
}

void ckl_ref_bench_destroy(void* handle) { delete static_cast<RefBench*>(handle); }

}  // extern "C"
