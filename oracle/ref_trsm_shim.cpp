// C-linkage shim around the helpers of the REFERENCE library's triangular-solve test.  TEST
// INFRASTRUCTURE ONLY: nothing in the shipped library links this.
//
// make_lower, trsm_reference and residual live in an unnamed namespace of the reference's
// tests/test_trsm.cpp (lines 20-69), so this file includes that source where it lies (its
// main() renamed by the build line, -Dmain=...) and forwards to them from the same translation
// unit.  The device entry points that file names (ckl::trsm_naive, trsm_blocked, trsm_cublas)
// are only referenced by its main(); they are given empty bodies here and never called.
// Output: oracle/_ref/libckl_ref_trsm.so, used to pin ckl_oracle_trsm_* bit for bit.

#include <cstddef>
#include <cstdint>
#include <cstring>
#include <vector>

#include "tests/test_trsm.cpp"

namespace ckl {
void trsm_naive(const float*, float*, int, int, float, cudaStream_t) {}
void trsm_blocked(const float*, float*, int, int, float, cudaStream_t) {}
void trsm_cublas(const float*, float*, int, int, float, cudaStream_t) {}
}  // namespace ckl

extern "C" {

void ckl_ref_make_lower(int m, std::uint64_t seed, float* out) {
    const std::vector<float> v = make_lower(m, seed);
    if (!v.empty()) {
        std::memcpy(out, v.data(), v.size() * sizeof(float));
    }
}

void ckl_ref_trsm_reference(const float* a, const float* b, int m, int n, float alpha, double* x) {
    const std::vector<float> va(a, a + static_cast<std::size_t>(m) * m);
    const std::vector<float> vb(b, b + static_cast<std::size_t>(m) * n);
    const std::vector<double> out = trsm_reference(va, vb, m, n, alpha);
    if (!out.empty()) {
        std::memcpy(x, out.data(), out.size() * sizeof(double));
    }
}

double ckl_ref_trsm_residual(const float* a, const float* x, const float* b, int m, int n, float alpha) {
    const std::vector<float> va(a, a + static_cast<std::size_t>(m) * m);
    const std::vector<float> vx(x, x + static_cast<std::size_t>(m) * n);
    const std::vector<float> vb(b, b + static_cast<std::size_t>(m) * n);
    return residual(va, vx, vb, m, n, alpha);
}

}  // extern "C"
