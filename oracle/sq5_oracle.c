/*
 * TEST INFRASTRUCTURE -- NOT PART OF THE PRODUCT.
 *
 * CPU restatement of the randumb pseudorandom-weight path, used only as the
 * checker in tests/, in the smoke test and as the timed CPU baseline of the
 * benchmark.  Nothing under randumb_b200/ may link, load or call this file.
 *
 * Parity pin: the hash below is checked bit-for-bit (as float32 bit patterns)
 * against outputs of the reference's own Triton kernels executed under the
 * Triton interpreter (tests/golden/make_golden.py -> tests/golden/ref_vectors.npz).
 *
 * What it follows in the reference (paths inside the reference project):
 *   hash steps and constants   src/rten_cpp/RandumbTensor.py:130-164
 *                              src/rten_cpp/csrc/cuda/rten.cu:13-48
 *   1-D hash (no row mixing)   src/rten_cpp/RandumbTensor.py:204-232
 *   noise matrix orientation   src/rten_cpp/RandumbTensor.py:78-99 (row = 1st index)
 *   materialise fwd (coef 1-D) src/rten_cpp/RandumbTensor.py:235-290, rten.cu:74-110
 *   materialise bwd            src/rten_cpp/RandumbTensor.py:304-359
 *   "explicit S then matmul"   benchmark.py:144-148, 379-383 (the reference's
 *                              own cross-check pattern; the matrix-coef layer
 *                              W = S*C is built from it)
 *
 * Build:  make -C oracle      (gcc -O2 -fopenmp -shared -fPIC)
 */
#include <stdint.h>
#include <stddef.h>
#include <string.h>
#include <stdlib.h>

#define SQ5_N1 0xd2a80a3fu
#define SQ5_N2 0xa884f197u
#define SQ5_N3 0x6C736F4Bu
#define SQ5_N4 0xB79F3ABBu
#define SQ5_N5 0x1b56c4f5u
#define SQ5_PRIME 198491317u

/* The eleven mixing steps applied to an already-formed 32-bit position. */
static inline uint32_t sq5_mix(uint32_t pos, uint32_t seed)
{
    uint32_t b = pos;
    b *= SQ5_N1;
    b += seed;
    b ^= b >> 9;
    b += SQ5_N2;
    b ^= b >> 11;
    b *= SQ5_N3;
    b ^= b >> 13;
    b += SQ5_N4;
    b ^= b >> 15;
    b *= SQ5_N5;
    b ^= b >> 17;
    return b;
}

/* 2-D position: PRIME*row + col, everything modulo 2^32. */
static inline uint32_t sq5_bits_2d(uint32_t row, uint32_t col, uint32_t seed)
{
    return sq5_mix(SQ5_PRIME * row + col, seed);
}

/* float32(int32(bits)) * float32(1/0x7FFFFFFF); the float32 constant is exactly 2^-31. */
static inline float sq5_to_float(uint32_t bits)
{
    const float scale = 1.0f / (float)0x7FFFFFFF;
    return scale * (float)(int32_t)bits;
}

uint32_t orc_sq5_bits(uint32_t row, uint32_t col, uint32_t seed) { return sq5_bits_2d(row, col, seed); }
uint32_t orc_sq5_bits_1d(uint32_t idx, uint32_t seed) { return sq5_mix(idx, seed); }
float orc_sq5_float(uint32_t row, uint32_t col, uint32_t seed) { return sq5_to_float(sq5_bits_2d(row, col, seed)); }

/* S[rows x cols] as raw hash words, row-major with leading dimension ld. */
void orc_noise_bits(uint32_t *out, int64_t rows, int64_t cols, int64_t ld,
                    int64_t row0, int64_t col0, uint32_t seed)
{
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < rows; ++r)
        for (int64_t c = 0; c < cols; ++c)
            out[r * ld + c] = sq5_bits_2d((uint32_t)(row0 + r), (uint32_t)(col0 + c), seed);
}

/* S[rows x cols] as float32 in [-1, 1]. */
void orc_noise_f32(float *out, int64_t rows, int64_t cols, int64_t ld,
                   int64_t row0, int64_t col0, uint32_t seed)
{
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < rows; ++r)
        for (int64_t c = 0; c < cols; ++c)
            out[r * ld + c] = sq5_to_float(sq5_bits_2d((uint32_t)(row0 + r), (uint32_t)(col0 + c), seed));
}

/* 1-D noise (fused random bias generator of the reference). */
void orc_noise_1d_f32(float *out, int64_t n, int64_t idx0, uint32_t seed)
{
    for (int64_t i = 0; i < n; ++i)
        out[i] = sq5_to_float(sq5_mix((uint32_t)(idx0 + i), seed));
}

/*
 * Reference materialise-forward with a 1-D coefficient vector:
 *   out[n] = sum_m S[sq(n), m] * coef[m],  sq(n) = (n % Q)*stride_Q + (n / Q)*stride_P
 * float32 fused multiply-add in index order, like the CUDA twin of the reference.
 */
void orc_materialize_fwd(float *out, const float *coef, int64_t M, int64_t P, int64_t Q,
                         int64_t stride_P, int64_t stride_Q, uint32_t seed)
{
    for (int64_t n = 0; n < P * Q; ++n) {
        int64_t sq = (n % Q) * stride_Q + (n / Q) * stride_P;
        double acc = 0.0;
        for (int64_t m = 0; m < M; ++m)
            acc += (double)sq5_to_float(sq5_bits_2d((uint32_t)sq, (uint32_t)m, seed)) * (double)coef[m];
        out[n] = (float)acc;
    }
}

/* Reference materialise-backward:  dcoef[m] = sum_n S[n, m] * dout[n]. */
void orc_materialize_bwd(float *dcoef, const float *dout, int64_t Nel, int64_t M, uint32_t seed)
{
    for (int64_t m = 0; m < M; ++m) {
        double acc = 0.0;
        for (int64_t n = 0; n < Nel; ++n)
            acc += (double)sq5_to_float(sq5_bits_2d((uint32_t)n, (uint32_t)m, seed)) * (double)dout[n];
        dcoef[m] = (float)acc;
    }
}

/*
 * Matrix-coefficient layer, plain loops, double accumulation (small cases only).
 *   W[o,i] = sum_k S[row0+o, k] * C[k,i]      S: [N x R], C: [R x K]
 *   y[t,o] = sum_i x[t,i] * W[o,i]
 */
void orc_linear_fwd(double *y, const float *x, const float *C, int64_t T, int64_t K, int64_t N,
                    int64_t R, int64_t row0, uint32_t seed)
{
    double *W = (double *)malloc((size_t)N * K * sizeof(double));
#pragma omp parallel for schedule(static)
    for (int64_t o = 0; o < N; ++o)
        for (int64_t i = 0; i < K; ++i) {
            double acc = 0.0;
            for (int64_t k = 0; k < R; ++k)
                acc += (double)sq5_to_float(sq5_bits_2d((uint32_t)(row0 + o), (uint32_t)k, seed)) * (double)C[k * K + i];
            W[o * K + i] = acc;
        }
#pragma omp parallel for schedule(static)
    for (int64_t t = 0; t < T; ++t)
        for (int64_t o = 0; o < N; ++o) {
            double acc = 0.0;
            for (int64_t i = 0; i < K; ++i) acc += (double)x[t * K + i] * W[o * K + i];
            y[t * N + o] = acc;
        }
    free(W);
}

/*
 *   dX[t,i] = sum_o dY[t,o] * W[o,i]
 *   dC[k,i] = sum_o S[row0+o,k] * (sum_t dY[t,o] * x[t,i])
 */
void orc_linear_bwd(double *dX, double *dC, const float *dY, const float *x, const float *C,
                    int64_t T, int64_t K, int64_t N, int64_t R, int64_t row0, uint32_t seed)
{
    double *W = (double *)malloc((size_t)N * K * sizeof(double));
    double *dW = (double *)malloc((size_t)N * K * sizeof(double));
#pragma omp parallel for schedule(static)
    for (int64_t o = 0; o < N; ++o)
        for (int64_t i = 0; i < K; ++i) {
            double acc = 0.0, accw = 0.0;
            for (int64_t k = 0; k < R; ++k)
                acc += (double)sq5_to_float(sq5_bits_2d((uint32_t)(row0 + o), (uint32_t)k, seed)) * (double)C[k * K + i];
            for (int64_t t = 0; t < T; ++t) accw += (double)dY[t * N + o] * (double)x[t * K + i];
            W[o * K + i] = acc;
            dW[o * K + i] = accw;
        }
#pragma omp parallel for schedule(static)
    for (int64_t t = 0; t < T; ++t)
        for (int64_t i = 0; i < K; ++i) {
            double acc = 0.0;
            for (int64_t o = 0; o < N; ++o) acc += (double)dY[t * N + o] * W[o * K + i];
            dX[t * K + i] = acc;
        }
#pragma omp parallel for schedule(static)
    for (int64_t k = 0; k < R; ++k)
        for (int64_t i = 0; i < K; ++i) {
            double acc = 0.0;
            for (int64_t o = 0; o < N; ++o)
                acc += (double)sq5_to_float(sq5_bits_2d((uint32_t)(row0 + o), (uint32_t)k, seed)) * dW[o * K + i];
            dC[k * K + i] = acc;
        }
    free(W);
    free(dW);
}
