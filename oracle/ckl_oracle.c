/*
 * CPU oracle for the FP16/BF16 tensor-core GEMM path.  TEST INFRASTRUCTURE ONLY.
 *
 * This file is a checker: it may be called from tests/, from the smoke check
 * and from the benchmark's CPU-baseline leg, and from nowhere else.  The
 * shipped library (libckl_gemm.so) never links or calls it.
 *
 * It restates, in plain C, the host-side helpers the reference library uses
 * to judge its tensor GEMM kernels:
 *
 *   - ckl::random_matrix              include/ckl/reference.hpp:16-24
 *   - ckl::gemm_reference             include/ckl/reference.hpp:29-46
 *   - ckl::relative_frobenius_error   include/ckl/reference.hpp:51-63
 *   - the host float -> FP16 / BF16 narrowing the reference tests apply to
 *     the random floats before upload (tests/test_gemm_tensor.cpp:40-56,
 *     round to nearest even)
 *   - the helpers of the reference's triangular-solve test: make_lower,
 *     trsm_reference and residual (tests/test_trsm.cpp:20-69)
 *
 * random_matrix in the reference is std::mt19937_64 driving
 * std::uniform_real_distribution<float>(-1, 1) as implemented by libstdc++
 * (one 64-bit draw per element).  Both are restated here from their published
 * definitions: MT19937-64 (Matsumoto and Nishimura, 2004) and the libstdc++
 * generate_canonical<float, 24> arithmetic.
 *
 * Parity pinning: the known-answer values in tests/golden/oracle_kat.json were
 * produced by compiling the reference header itself (oracle/ref_shim.cpp ->
 * oracle/_ref/libckl_ref.so) and tests/test_oracle.py checks this restatement
 * against them bit for bit.
 */

#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

/* ------------------------------------------------------------------------ */
/* MT19937-64                                                                */
/* ------------------------------------------------------------------------ */

#define MT_NN 312
#define MT_MM 156
#define MT_MATRIX_A 0xB5026F5AA96619E9ULL
#define MT_UPPER 0xFFFFFFFF80000000ULL
#define MT_LOWER 0x000000007FFFFFFFULL

typedef struct {
    uint64_t state[MT_NN];
    int index;
} mt64_t;

static void mt64_seed(mt64_t* g, uint64_t seed) {
    g->state[0] = seed;
    for (int i = 1; i < MT_NN; ++i) {
        g->state[i] =
            6364136223846793005ULL * (g->state[i - 1] ^ (g->state[i - 1] >> 62)) + (uint64_t)i;
    }
    g->index = MT_NN;
}

static void mt64_refill(mt64_t* g) {
    uint64_t* s = g->state;
    for (int i = 0; i < MT_NN; ++i) {
        const uint64_t x = (s[i] & MT_UPPER) | (s[(i + 1) % MT_NN] & MT_LOWER);
        uint64_t y = x >> 1;
        if (x & 1ULL) {
            y ^= MT_MATRIX_A;
        }
        s[i] = s[(i + MT_MM) % MT_NN] ^ y;
    }
    g->index = 0;
}

static uint64_t mt64_next(mt64_t* g) {
    if (g->index >= MT_NN) {
        mt64_refill(g);
    }
    uint64_t x = g->state[g->index++];
    x ^= (x >> 29) & 0x5555555555555555ULL;
    x ^= (x << 17) & 0x71D67FFFEDA60000ULL;
    x ^= (x << 37) & 0xFFF7EEE000000000ULL;
    x ^= (x >> 43);
    return x;
}

/* One raw 64-bit draw, exposed so the tests can pin the engine separately
 * from the distribution (10000th output of a default-seeded mt19937_64 is a
 * value the C++ standard itself fixes). */
uint64_t ckl_oracle_mt64_nth(uint64_t seed, uint64_t n) {
    mt64_t g;
    mt64_seed(&g, seed);
    uint64_t v = 0;
    for (uint64_t i = 0; i < n; ++i) {
        v = mt64_next(&g);
    }
    return v;
}

/* libstdc++ generate_canonical<float, 24>(mt19937_64): the engine range is
 * 2^64 so a single draw is used; it is converted to float (round to nearest),
 * divided by 2^64, and a result that rounds up to 1.0 is pulled back to the
 * largest float below one. */
static float canonical_float(mt64_t* g) {
    const float range = 18446744073709551616.0f; /* 2^64 */
    float r = (float)mt64_next(g) / range;
    if (r >= 1.0f) {
        r = nextafterf(1.0f, 0.0f);
    }
    return r;
}

/* Follows ckl::random_matrix (include/ckl/reference.hpp:16-24): row-major
 * rows*cols floats, uniform on [-1, 1), one engine draw per element. */
void ckl_oracle_random_matrix(int rows, int cols, uint64_t seed, float* out) {
    mt64_t g;
    mt64_seed(&g, seed);
    const size_t count = (size_t)rows * (size_t)cols;
    for (size_t i = 0; i < count; ++i) {
        out[i] = canonical_float(&g) * (1.0f - -1.0f) + -1.0f;
    }
}

/* ------------------------------------------------------------------------ */
/* GEMM reference (double accumulate)                                        */
/* ------------------------------------------------------------------------ */

static double ref_element(const float* a, const float* b, const float* c_in, int n, int k,
                          float alpha, float beta, int i, int j) {
    double acc = 0.0;
    for (int p = 0; p < k; ++p) {
        acc += (double)a[(size_t)i * k + p] * (double)b[(size_t)p * n + j];
    }
    const size_t idx = (size_t)i * n + j;
    return (double)alpha * acc + (double)beta * (double)c_in[idx];
}

/* Follows ckl::gemm_reference (include/ckl/reference.hpp:29-46) statement for
 * statement: row-major, float inputs, one double accumulator per output
 * element, k walked in increasing order, single thread. */
void ckl_oracle_gemm_reference(const float* a, const float* b, const float* c_in, int m, int n,
                               int k, float alpha, float beta, double* c_out) {
    for (int i = 0; i < m; ++i) {
        for (int j = 0; j < n; ++j) {
            c_out[(size_t)i * n + j] = ref_element(a, b, c_in, n, k, alpha, beta, i, j);
        }
    }
}

/* The same per-element loop with the rows shared among host threads.  Each
 * element's summation order is unchanged, so the result is bit-identical to
 * the single-thread function above (tests assert that).  threads <= 0 means
 * "all the cores OpenMP sees".  Returns the number of threads used. */
int ckl_oracle_gemm_reference_mt(const float* a, const float* b, const float* c_in, int m, int n,
                                 int k, float alpha, float beta, double* c_out, int threads) {
    int used = 1;
#ifdef _OPENMP
    if (threads <= 0) {
        threads = omp_get_max_threads();
    }
    used = threads;
#pragma omp parallel for schedule(dynamic, 4) num_threads(threads)
#endif
    for (int i = 0; i < m; ++i) {
        for (int j = 0; j < n; ++j) {
            c_out[(size_t)i * n + j] = ref_element(a, b, c_in, n, k, alpha, beta, i, j);
        }
    }
    return used;
}

/* Sampled oracle for shapes whose full O(mnk) reference is unaffordable: the
 * listed rows (full rows of C) and the listed columns (full columns of C),
 * every element by the same sequential double loop.  rows_out is
 * [n_rows][n]; cols_out is [n_cols][m]. */
void ckl_oracle_gemm_sampled(const float* a, const float* b, const float* c_in, int m, int n,
                             int k, float alpha, float beta, const int* rows, int n_rows,
                             const int* cols, int n_cols, double* rows_out, double* cols_out) {
#ifdef _OPENMP
#pragma omp parallel for schedule(dynamic, 1)
#endif
    for (int r = 0; r < n_rows; ++r) {
        for (int j = 0; j < n; ++j) {
            rows_out[(size_t)r * n + j] = ref_element(a, b, c_in, n, k, alpha, beta, rows[r], j);
        }
    }
#ifdef _OPENMP
#pragma omp parallel for schedule(dynamic, 1)
#endif
    for (int c = 0; c < n_cols; ++c) {
        for (int i = 0; i < m; ++i) {
            cols_out[(size_t)c * m + i] = ref_element(a, b, c_in, n, k, alpha, beta, i, cols[c]);
        }
    }
}

/* Follows ckl::relative_frobenius_error (include/ckl/reference.hpp:51-63):
 * ||actual - ref||_F / ||ref||_F, absolute error when ||ref||_F <= 1e-30. */
double ckl_oracle_relative_frobenius_error(const float* actual, const double* ref, size_t count) {
    double num = 0.0;
    double den = 0.0;
    for (size_t i = 0; i < count; ++i) {
        const double diff = (double)actual[i] - ref[i];
        num += diff * diff;
        den += ref[i] * ref[i];
    }
    const double rn = sqrt(num);
    const double rd = sqrt(den);
    return rd > 1e-30 ? rn / rd : rn;
}

/* ------------------------------------------------------------------------ */
/* float -> 16-bit storage, round to nearest even, and back                  */
/* ------------------------------------------------------------------------ */

static uint32_t f32_bits(float f) {
    uint32_t u;
    memcpy(&u, &f, sizeof u);
    return u;
}

static float bits_f32(uint32_t u) {
    float f;
    memcpy(&f, &u, sizeof f);
    return f;
}

/* Same result as the host __float2bfloat16 the reference tests call
 * (tests/test_gemm_tensor.cpp:49-56): round to nearest even on the upper 16
 * bits; NaN stays a quiet NaN. */
uint16_t ckl_oracle_f32_to_bf16(float f) {
    const uint32_t u = f32_bits(f);
    if ((u & 0x7FFFFFFFu) > 0x7F800000u) {
        return 0x7FFF;
    }
    const uint32_t bias = 0x7FFFu + ((u >> 16) & 1u);
    return (uint16_t)((u + bias) >> 16);
}

float ckl_oracle_bf16_to_f32(uint16_t h) { return bits_f32((uint32_t)h << 16); }

/* Same result as the host __float2half (tests/test_gemm_tensor.cpp:40-47):
 * IEEE binary16, round to nearest even, gradual underflow, overflow to inf. */
uint16_t ckl_oracle_f32_to_f16(float f) {
    const uint32_t u = f32_bits(f);
    const uint32_t sign = (u >> 16) & 0x8000u;
    const uint32_t mag = u & 0x7FFFFFFFu;
    if (mag > 0x7F800000u) {
        return (uint16_t)(sign | 0x7FFFu);
    }
    if (mag >= 0x477FF000u) { /* rounds to >= 2^16: infinity */
        return (uint16_t)(sign | 0x7C00u);
    }
    if (mag < 0x33000001u) { /* <= 2^-25: rounds to zero (tie goes to even = 0) */
        return (uint16_t)sign;
    }
    const int exp = (int)(mag >> 23) - 127;
    uint32_t mant = (mag & 0x007FFFFFu) | 0x00800000u; /* 24-bit significand */
    int shift;
    uint32_t base;
    if (exp < -14) { /* subnormal half: value = mant * 2^(exp-23), unit 2^-24 */
        shift = -exp - 1; /* = 13 + (-14 - exp) */
        base = 0;
    } else {
        shift = 13;
        base = (uint32_t)(exp + 15) << 10;
        mant &= 0x007FFFFFu;
    }
    const uint32_t kept = mant >> shift;
    const uint32_t rem = mant & ((1u << shift) - 1u);
    const uint32_t half = 1u << (shift - 1);
    uint32_t out = base + kept;
    if (rem > half || (rem == half && (kept & 1u))) {
        out += 1u; /* carries into the exponent correctly */
    }
    return (uint16_t)(sign | out);
}

float ckl_oracle_f16_to_f32(uint16_t h) {
    const uint32_t sign = ((uint32_t)h & 0x8000u) << 16;
    const uint32_t exp = (h >> 10) & 0x1Fu;
    const uint32_t mant = h & 0x3FFu;
    if (exp == 0x1Fu) {
        return bits_f32(sign | 0x7F800000u | (mant << 13));
    }
    if (exp == 0) {
        const float v = (float)mant * 5.9604644775390625e-08f; /* 2^-24 */
        return sign ? -v : v;
    }
    return bits_f32(sign | ((exp + 112u) << 23) | (mant << 13));
}

/* dtype: 1 = FP16, 2 = BF16 (the C ABI's ckl_dtype numbering). */
void ckl_oracle_narrow(const float* src, uint16_t* dst, size_t count, int dtype) {
    for (size_t i = 0; i < count; ++i) {
        dst[i] = dtype == 1 ? ckl_oracle_f32_to_f16(src[i]) : ckl_oracle_f32_to_bf16(src[i]);
    }
}

void ckl_oracle_widen(const uint16_t* src, float* dst, size_t count, int dtype) {
    for (size_t i = 0; i < count; ++i) {
        dst[i] = dtype == 1 ? ckl_oracle_f16_to_f32(src[i]) : ckl_oracle_bf16_to_f32(src[i]);
    }
}

int ckl_oracle_max_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/* ------------------------------------------------------------------------ */
/* Triangular solve helpers of the reference's TRSM test                     */
/* ------------------------------------------------------------------------ */

/* tests/test_trsm.cpp:20-31 of the reference: random_matrix(m, m, seed) with the upper
 * part zeroed and the diagonal set to m + 1 (diagonally dominant, well conditioned). */
void ckl_oracle_make_lower(int m, uint64_t seed, float* out) {
    ckl_oracle_random_matrix(m, m, seed, out);
    for (int i = 0; i < m; ++i) {
        for (int j = i + 1; j < m; ++j) {
            out[(size_t)i * m + j] = 0.0f;
        }
        out[(size_t)i * m + i] = (float)(m + 1);
    }
}

/* tests/test_trsm.cpp:33-47: forward substitution in double, column by column,
 * x[i] = (alpha * b[i] - sum_{j<i} a[i][j] * x[j]) / a[i][i], the sum taken in order of j. */
void ckl_oracle_trsm_reference(const float* a, const float* b, int m, int n, float alpha, double* x) {
#ifdef _OPENMP
#pragma omp parallel for schedule(static)
#endif
    for (int c = 0; c < n; ++c) {
        for (int i = 0; i < m; ++i) {
            double s = (double)alpha * b[(size_t)i * n + c];
            for (int j = 0; j < i; ++j) {
                s -= (double)a[(size_t)i * m + j] * x[(size_t)j * n + c];
            }
            x[(size_t)i * n + c] = s / a[(size_t)i * m + i];
        }
    }
}

/* tests/test_trsm.cpp:50-69: ||L X - alpha B||_F / ||alpha B||_F in double. */
double ckl_oracle_trsm_residual(const float* a, const float* x, const float* b, int m, int n,
                                float alpha) {
    double num = 0.0;
    double den = 0.0;
    for (int i = 0; i < m; ++i) {
        for (int c = 0; c < n; ++c) {
            double lx = 0.0;
            for (int j = 0; j <= i; ++j) {
                lx += (double)a[(size_t)i * m + j] * (double)x[(size_t)j * n + c];
            }
            const double target = (double)alpha * (double)b[(size_t)i * n + c];
            num += (lx - target) * (lx - target);
            den += target * target;
        }
    }
    return sqrt(num) / sqrt(den);
}
