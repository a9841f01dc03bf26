/*
 * CPU oracle, C edition: a plain-C (OpenMP) restatement of the aie4ml AIE kernels' integer
 * arithmetic.  TEST INFRASTRUCTURE ONLY: it is the timed CPU baseline of the benchmark and a
 * second checker beside the NumPy oracle; nothing in the shipped library links or calls it.
 *
 * Each function follows one reference kernel (file:line cited, paths relative to the aie4ml
 * project root).  The reference kernels themselves include AMD's adf.h / aie_api (Vitis 2025.2),
 * which cannot be compiled outside Vitis, so the reference's own code cannot be built here.
 *
 * Pinning: this file is checked against the NumPy oracle on seeded inputs; see that module's
 * header for what is pinned against the reference itself and what is "parity unpinned"
 * (kernel arithmetic has no golden vectors in the reference; LayerNorm's float reciprocal
 * square root is defined here as 1.0f / sqrtf((float)var) in IEEE binary32).
 *
 * Codes shared with the CUDA library's C ABI:
 *   rounding: 0 floor, 1 ceil, 2 positive_inf, 3 negative_inf, 4 symmetric_inf,
 *             5 symmetric_zero, 6 conv_even, 7 conv_odd
 *   dtype:    0 int8, 1 uint8, 2 int16
 */
#include <math.h>
#ifdef _OPENMP
#include <omp.h>
#endif
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define ORC_API __attribute__((visibility("default")))

static inline int64_t round_shift64(int64_t v, int shift, int tok) {
    if (shift <= 0) return v;
    const int64_t q = v >> shift;
    const int64_t r = v & (((int64_t)1 << shift) - 1);
    const int64_t half = (int64_t)1 << (shift - 1);
    int inc;
    switch (tok) {
        case 0: inc = 0; break;
        case 1: inc = r != 0; break;
        case 2: inc = r >= half; break;
        case 3: inc = r > half; break;
        case 4: inc = v >= 0 ? (r >= half) : (r > half); break;
        case 5: inc = v >= 0 ? (r > half) : (r >= half); break;
        case 6: inc = (r > half) || (r == half && (q & 1)); break;
        default: inc = (r > half) || (r == half && !(q & 1)); break;
    }
    return q + inc;
}

static inline int64_t saturate(int64_t v, int dtype) {
    int64_t lo, hi;
    if (dtype == 0) { lo = -128; hi = 127; }
    else if (dtype == 1) { lo = 0; hi = 255; }
    else { lo = -32768; hi = 32767; }
    return v < lo ? lo : (v > hi ? hi : v);
}

static inline void store_out(void* base, int64_t idx, int64_t v, int dtype) {
    if (dtype == 2) ((int16_t*)base)[idx] = (int16_t)v;
    else if (dtype == 1) ((uint8_t*)base)[idx] = (uint8_t)v;
    else ((int8_t*)base)[idx] = (int8_t)v;
}

static inline int64_t srs_out(int64_t v, int shift, int tok, int dtype) {
    return saturate(round_shift64(v, shift, tok), dtype);
}

/* Dense: relu?(srs(A.W + bias)).  dense_single::run,
 * templates/nnet_utils/dense_bias_relu/dense_bias_relu.cpp:67-166 (bias as accumulator init
 * :114-124, acc32 MACs :132-151, ReLU after saturation :153-157).
 * A [M,K] row-major (pitch lda), W [K,N] row-major, bias [N] or NULL, Y [M,N] (pitch ldy). */
ORC_API int orc_dense_i8(const void* A, int64_t lda, const int8_t* W, const int32_t* bias, void* Y, int64_t ldy,
                         int64_t M, int K, int N, int shift, int rounding, int relu, int out_dtype, int a_unsigned) {
    if (M < 0 || K <= 0 || N <= 0 || shift < 0 || shift > 62) return -1;
#pragma omp parallel
    {
        int32_t* acc = (int32_t*)malloc(sizeof(int32_t) * (size_t)N);
#pragma omp for schedule(static)
        for (int64_t m = 0; m < M; ++m) {
            for (int n = 0; n < N; ++n) acc[n] = bias ? bias[n] : 0;
            const int8_t* as = (const int8_t*)A + m * lda;
            const uint8_t* au = (const uint8_t*)A + m * lda;
            for (int k = 0; k < K; ++k) {
                const int32_t a = a_unsigned ? (int32_t)au[k] : (int32_t)as[k];
                const int8_t* w = W + (int64_t)k * N;
                /* unsigned arithmetic: acc32 lanes wrap */
                for (int n = 0; n < N; ++n) acc[n] = (int32_t)((uint32_t)acc[n] + (uint32_t)(a * (int32_t)w[n]));
            }
            for (int n = 0; n < N; ++n) {
                int64_t y = srs_out(acc[n], shift, rounding, out_dtype);
                if (relu && y < 0) y = 0;
                store_out(Y, m * ldy + n, y, out_dtype);
            }
        }
        free(acc);
    }
    return 0;
}

/* Batched dynamic MatMul: C_b = srs(op(A_b).op(B_b)).  matmul_single::run,
 * templates/nnet_utils/matmul/matmul.cpp:32-118; TRANSPOSE_A/B (:60-77) read the stored operand
 * with its two axes swapped.  Stored A_b is [M,K] (or [K,M] when trans_a) with pitch lda;
 * stored B_b is [K,N] (or [N,K] when trans_b) with pitch ldb. */
ORC_API int orc_bmm_i8(const void* A, int64_t lda, int64_t stride_a, const int8_t* B, int64_t ldb, int64_t stride_b,
                       void* C, int64_t ldc, int64_t stride_c, int64_t batch, int M, int K, int N, int trans_a,
                       int trans_b, int shift, int rounding, int out_dtype, int a_unsigned) {
    if (batch < 0 || M <= 0 || K <= 0 || N <= 0 || shift < 0 || shift > 62) return -1;
#pragma omp parallel for schedule(static)
    for (int64_t b = 0; b < batch; ++b) {
        const int8_t* as = (const int8_t*)A + b * stride_a;
        const uint8_t* au = (const uint8_t*)A + b * stride_a;
        const int8_t* bs = B + b * stride_b;
        for (int m = 0; m < M; ++m) {
            for (int n = 0; n < N; ++n) {
                uint32_t acc = 0;
                for (int k = 0; k < K; ++k) {
                    const int64_t ai = trans_a ? (int64_t)k * lda + m : (int64_t)m * lda + k;
                    const int64_t bi = trans_b ? (int64_t)n * ldb + k : (int64_t)k * ldb + n;
                    const int32_t a = a_unsigned ? (int32_t)au[ai] : (int32_t)as[ai];
                    acc += (uint32_t)(a * (int32_t)bs[bi]);
                }
                const int64_t y = srs_out((int32_t)acc, shift, rounding, out_dtype);
                store_out(C, b * stride_c + (int64_t)m * ldc + n, y, out_dtype);
            }
        }
    }
    return 0;
}

/* Elementwise srs(a + b): elementwise_add_kernel::run,
 * templates/nnet_utils/elementwise_add/elementwise_add.cpp:12-37. */
ORC_API int orc_add_sat(const void* a, int64_t lda, const void* b, int64_t ldb, void* out, int64_t ldo,
                        int64_t rows, int64_t cols, int shift, int rounding, int dtype) {
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < rows; ++r)
        for (int64_t c = 0; c < cols; ++c) {
            int64_t va, vb;
            if (dtype == 2) { va = ((const int16_t*)a)[r * lda + c]; vb = ((const int16_t*)b)[r * ldb + c]; }
            else if (dtype == 1) { va = ((const uint8_t*)a)[r * lda + c]; vb = ((const uint8_t*)b)[r * ldb + c]; }
            else { va = ((const int8_t*)a)[r * lda + c]; vb = ((const int8_t*)b)[r * ldb + c]; }
            store_out(out, r * ldo + c, srs_out(va + vb, shift, rounding, dtype), dtype);
        }
    return 0;
}

static inline int32_t round_float_tok(float f, int tok) {
    const float fl = floorf(f);
    const float frac = f - fl;
    const int32_t q = (int32_t)fl;
    switch (tok) {
        case 0: return q;
        case 1: return q + (frac > 0.0f);
        case 2: case 4: return q + (frac >= 0.5f);
        case 3: case 5: return q + (frac > 0.5f);
        case 6: return q + ((frac > 0.5f) || (frac == 0.5f && (q & 1)));
        default: return q + ((frac > 0.5f) || (frac == 0.5f && !(q & 1)));
    }
}

/* Integer LayerNorm over rows of `cols` (power of two) int8 values.
 * layernorm_i8::run + row_statistics, templates/nnet_utils/layer_norm/layer_norm.cpp:15-121.
 * gamma int16 Q7, beta int16 Q15.  addend (may be NULL) fuses a following saturating Add. */
ORC_API int orc_layernorm_i8(const int8_t* x, int64_t ldx, const int16_t* gamma, const int16_t* beta, int8_t* out,
                             int64_t ldo, int64_t rows, int cols, int eps_q0, int out_shift, int rounding) {
    int log2c = 0;
    while ((1 << log2c) < cols) ++log2c;
    if ((1 << log2c) != cols || out_shift < 0 || out_shift > 15) return -1;
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < rows; ++r) {
        const int8_t* xr = x + r * ldx;
        int32_t sum_x = 0, sum_sq = 0;
        for (int c = 0; c < cols; ++c) { sum_x += xr[c]; sum_sq += (int32_t)xr[c] * xr[c]; }
        const int32_t mu = (sum_x + (cols >> 1)) >> log2c;
        const int32_t centered = (int32_t)((uint32_t)sum_sq - 2u * (uint32_t)mu * (uint32_t)sum_x +
                                           (uint32_t)cols * (uint32_t)mu * (uint32_t)mu);
        int32_t var = centered >> log2c;
        if (var < 0) var = 0;
        var += eps_q0;
        const float inv_f = 1.0f / sqrtf((float)var);
        int32_t inv_std = round_float_tok(inv_f * 32768.0f, rounding);
        inv_std = inv_std > 32767 ? 32767 : (inv_std < 0 ? 0 : inv_std);
        for (int c = 0; c < cols; ++c) {
            const int32_t vd = (int32_t)xr[c] - mu;
            const int64_t fscale = saturate(round_shift64((int64_t)inv_std * gamma[c], 7, rounding), 2);
            const int32_t acc = (int32_t)((uint32_t)(vd * (int32_t)fscale) + (uint32_t)(int32_t)beta[c]);
            out[r * ldo + c] = (int8_t)srs_out(acc, 15 - out_shift, rounding, 0);
        }
    }
    return 0;
}

/* 2^(-d*KQ/256) in Q14: exp_score16, templates/nnet_utils/softmax/softmax.cpp:252-273. */
static inline int32_t exp_score16(int32_t d, int32_t kq) {
    int32_t z = d * kq;
    z = z > 32767 ? 32767 : z;
    const int32_t zint = z >> 8, zfrac = z & 255;
    const int32_t t = (zfrac * 2811) >> 8;
    const int32_t inner = t - 11004;
    const int32_t t2 = (inner * zfrac) >> 8;
    int32_t e = t2 + 16384;
    for (int b = 0; b < 4; ++b)
        if (zint & (1 << b)) e >>= (1 << b);
    if (zint >= 16) e = 0;
    return e;
}

/* Quantized softmax over rows of int8.  mode 0 = HCCS surrogate (softmax_i8::softmax_row,
 * templates/nnet_utils/softmax/softmax.cpp:20-88), mode 1 = accurate integer exp
 * (softmax_exp_i8::run, :333-384).  out_dtype 1 = uint8, 2 = int16. */
ORC_API int orc_softmax_i8(const int8_t* x, int64_t ldx, void* out, int64_t ldo, int64_t rows, int cols, int mode,
                           int B, int S, int Dmax, int inv_shift, int use_clb, int exp_kq, int out_dtype) {
    if (out_dtype != 1 && out_dtype != 2) return -1;
    const int64_t numer = out_dtype == 2 ? 32767 : ((int64_t)255 << inv_shift);
    const int out_shift = out_dtype == 2 ? 0 : inv_shift;
#pragma omp parallel
    {
        int32_t* score = (int32_t*)malloc(sizeof(int32_t) * (size_t)cols);
#pragma omp for schedule(static)
        for (int64_t r = 0; r < rows; ++r) {
            const int8_t* xr = x + r * ldx;
            int32_t m = -128;
            for (int c = 0; c < cols; ++c) m = xr[c] > m ? xr[c] : m;
            int64_t sum = 0;
            for (int c = 0; c < cols; ++c) {
                int32_t d = m - xr[c];
                int32_t s;
                if (mode == 0) {
                    d = d < Dmax ? d : Dmax;
                    s = B - S * d;
                    s = s > 32767 ? 32767 : (s < -32768 ? -32768 : s);
                } else {
                    s = exp_score16(d, exp_kq);
                }
                score[c] = s;
                sum += s;
            }
            if (sum <= 0) sum = 1;
            int64_t inv;
            if (use_clb && mode == 0) {
                int k = 0;
                while (((int64_t)1 << (k + 1)) <= sum) ++k;
                if (out_dtype == 2) inv = 32767 >> k;
                else inv = inv_shift - k >= 0 ? ((int64_t)255 << (inv_shift - k)) : ((int64_t)255 >> (k - inv_shift));
            } else {
                inv = numer / sum;
            }
            inv = inv > 32767 ? 32767 : (inv < 0 ? 0 : inv);
            for (int c = 0; c < cols; ++c)
                store_out(out, r * ldo + c, srs_out((int64_t)score[c] * inv, out_shift, 0, out_dtype), out_dtype);
        }
        free(score);
    }
    return 0;
}

/* Override the OpenMP thread count (launchers such as torchrun export OMP_NUM_THREADS=1). */
ORC_API void orc_set_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

ORC_API int orc_num_threads(void) {
    int n = 1;
#ifdef _OPENMP
#pragma omp parallel
    {
#pragma omp master
        n = omp_get_num_threads();
    }
#endif
    return n;
}
