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

/* ---- integer GEMM core ---------------------------------------------------------------------
 * Both matrix products below are blocked over rows and columns with the K loop innermost on 32-bit
 * accumulators that wrap (the AIE acc32 lanes do: every partial sum is taken modulo 2^32, so any
 * order of accumulation gives the same bits).  Two code paths compute the same sums:
 *   - AVX-512 VNNI (when the compiler targets it): vpdpbusd multiplies unsigned bytes by signed
 *     bytes, so a signed A is offset by +128 (a ^ 0x80) and 128 * (column sum of W) is taken back
 *     out of the accumulator's initial value; the non-saturating form wraps like the plain sum.
 *   - portable C: operands widened to int16, dot products the compiler turns into multiply-add
 *     instructions of whatever width the target has.
 */
#if defined(__AVX512VNNI__) && defined(__AVX512BW__) && defined(__AVX512F__)
#include <immintrin.h>
#define ORC_VNNI 1
#else
#define ORC_VNNI 0
#endif

ORC_API int orc_gemm_path(void) { return ORC_VNNI; }   /* 1 = AVX-512 VNNI, 0 = portable C */

#if ORC_VNNI
enum { VN_NR = 64, VN_MR = 6 };

/* W [K,N] (row pitch ldw, element (k,n) at W[k*w_ks + n*w_ns]) -> panels [N/64][K4][64 n][4 k], zero padded;
 * colsum[n] = sum_k W[k,n]. */
static int8_t* vn_pack_w(const int8_t* W, int64_t w_ks, int64_t w_ns, int K, int N, int32_t* colsum) {
    const int K4 = (K + 3) / 4, NP = (N + VN_NR - 1) / VN_NR;
    int8_t* P = (int8_t*)aligned_alloc(64, (size_t)NP * K4 * VN_NR * 4);
    if (!P) return NULL;
#pragma omp parallel for schedule(static)
    for (int np = 0; np < NP; ++np) {
        int8_t* dst = P + (size_t)np * K4 * VN_NR * 4;
        int32_t cs[VN_NR] = {0};
        const int nb = N - np * VN_NR < VN_NR ? N - np * VN_NR : VN_NR;
        for (int k4 = 0; k4 < K4; ++k4)
            for (int kk = 0; kk < 4; ++kk) {
                const int k = k4 * 4 + kk;
                int8_t* d = dst + (size_t)k4 * VN_NR * 4 + kk;
                if (k < K) {
                    const int8_t* src = W + (int64_t)k * w_ks + (int64_t)np * VN_NR * w_ns;   /* 64 columns of row k */
                    for (int j = 0; j < nb; ++j) { const int8_t v = src[(int64_t)j * w_ns]; d[j * 4] = v; cs[j] += v; }
                    for (int j = nb; j < VN_NR; ++j) d[j * 4] = 0;
                } else {
                    for (int j = 0; j < VN_NR; ++j) d[j * 4] = 0;
                }
            }
        for (int j = 0; j < nb; ++j) colsum[np * VN_NR + j] = cs[j];
    }
    return P;
}

/* acc[i][n] (i < mr <= 6, 64 columns) = init[n] + sum_k Au[i][k] * Wp[k][n] over K4 groups of four k.
 * Au: mr rows of unsigned bytes, row pitch a_ld (a multiple of 4, zero or anything in the K padding:
 * the packed W is zero there). */
static void vn_micro(const uint8_t* Au, int64_t a_ld, int mr, const int8_t* Wp, int K4, const int32_t* init,
                     int32_t* out /* [mr][64] */) {
    __m512i acc[VN_MR][4];
    for (int i = 0; i < VN_MR; ++i)
        for (int c = 0; c < 4; ++c) acc[i][c] = _mm512_loadu_si512((const void*)(init + 16 * c));
    const uint8_t* rows[VN_MR];
    for (int i = 0; i < VN_MR; ++i) rows[i] = Au + (int64_t)(i < mr ? i : 0) * a_ld;
    for (int k4 = 0; k4 < K4; ++k4) {
        const __m512i w0 = _mm512_load_si512((const void*)(Wp + (size_t)k4 * 256));
        const __m512i w1 = _mm512_load_si512((const void*)(Wp + (size_t)k4 * 256 + 64));
        const __m512i w2 = _mm512_load_si512((const void*)(Wp + (size_t)k4 * 256 + 128));
        const __m512i w3 = _mm512_load_si512((const void*)(Wp + (size_t)k4 * 256 + 192));
#pragma GCC unroll 6
        for (int i = 0; i < VN_MR; ++i) {
            int32_t a4;
            memcpy(&a4, rows[i] + (size_t)k4 * 4, 4);
            const __m512i a = _mm512_set1_epi32(a4);
            acc[i][0] = _mm512_dpbusd_epi32(acc[i][0], a, w0);
            acc[i][1] = _mm512_dpbusd_epi32(acc[i][1], a, w1);
            acc[i][2] = _mm512_dpbusd_epi32(acc[i][2], a, w2);
            acc[i][3] = _mm512_dpbusd_epi32(acc[i][3], a, w3);
        }
    }
    for (int i = 0; i < mr; ++i)
        for (int c = 0; c < 4; ++c) _mm512_storeu_si512((void*)(out + i * 64 + 16 * c), acc[i][c]);
}
#endif

/* One [M,K] x [K,N] product with the shared epilogue.  A element (m,k) at A[m*a_rs + k*a_cs] (bytes),
 * W element (k,n) at W[k*w_ks + n*w_ns].  `parallel` = split the rows over OpenMP threads (the batched
 * caller parallelises over the batch instead). */
static int gemm_i8(const void* A, int64_t a_rs, int64_t a_cs, int a_unsigned, const int8_t* W, int64_t w_ks, int64_t w_ns,
                   const int32_t* bias, void* Y, int64_t ldy, int64_t M, int K, int N, int shift, int rounding, int relu,
                   int out_dtype, int parallel) {
#if ORC_VNNI
    const int K4 = (K + 3) / 4, Kp = K4 * 4, NP = (N + VN_NR - 1) / VN_NR;
    int32_t* colsum = (int32_t*)calloc((size_t)NP * VN_NR, sizeof(int32_t));
    int32_t* init = (int32_t*)calloc((size_t)NP * VN_NR, sizeof(int32_t));
    int8_t* Wp = colsum && init ? vn_pack_w(W, w_ks, w_ns, K, N, colsum) : NULL;
    if (!Wp) { free(colsum); free(init); return -2; }
    for (int n = 0; n < N; ++n)
        init[n] = (int32_t)((uint32_t)(bias ? bias[n] : 0) - (a_unsigned ? 0u : 128u * (uint32_t)colsum[n]));
    enum { MBLK = 48 };   /* rows converted at a time: 8 micro-kernel row groups share each streamed W panel */
    int fail = 0;
#pragma omp parallel if (parallel)
    {
        uint8_t* Au = (uint8_t*)aligned_alloc(64, ((size_t)MBLK * Kp + 63) / 64 * 64);
        int32_t tile[VN_MR * 64];
        if (!Au) {
#pragma omp atomic write
            fail = 1;
        }
#pragma omp for schedule(dynamic, 1)
        for (int64_t m0 = 0; m0 < M; m0 += MBLK) {
            if (!Au) continue;
            const int mb = (int)(M - m0 < MBLK ? M - m0 : MBLK);
            for (int i = 0; i < mb; ++i) {
                const uint8_t* src = (const uint8_t*)A + (m0 + i) * a_rs;
                uint8_t* dst = Au + (size_t)i * Kp;
                const uint8_t flip = a_unsigned ? 0 : 0x80;
                for (int k = 0; k < K; ++k) dst[k] = src[(int64_t)k * a_cs] ^ flip;
                for (int k = K; k < Kp; ++k) dst[k] = 0;
            }
            for (int np = 0; np < NP; ++np) {
                const int8_t* wp = Wp + (size_t)np * K4 * 256;
                const int nb = N - np * 64 < 64 ? N - np * 64 : 64;
                for (int i0 = 0; i0 < mb; i0 += VN_MR) {
                    const int mr = mb - i0 < VN_MR ? mb - i0 : VN_MR;
                    vn_micro(Au + (size_t)i0 * Kp, Kp, mr, wp, K4, init + np * 64, tile);
                    for (int i = 0; i < mr; ++i)
                        for (int j = 0; j < nb; ++j) {
                            int64_t y = srs_out(tile[i * 64 + j], shift, rounding, out_dtype);
                            if (relu && y < 0) y = 0;
                            store_out(Y, (m0 + i0 + i) * ldy + np * 64 + j, y, out_dtype);
                        }
                }
            }
        }
        free(Au);
    }
    free(Wp); free(colsum); free(init);
    return fail ? -2 : 0;
#else
    /* portable: W^T and a block of A rows widened to int16 with K contiguous; 4 x 4 register tiles of dot products */
    const int Kp = (K + 31) / 32 * 32;
    int16_t* Wt = (int16_t*)aligned_alloc(64, (size_t)N * Kp * sizeof(int16_t));
    if (!Wt) return -2;
#pragma omp parallel for schedule(static) if (parallel)
    for (int n = 0; n < N; ++n) {
        int16_t* dst = Wt + (size_t)n * Kp;
        for (int k = 0; k < K; ++k) dst[k] = W[(int64_t)k * w_ks + (int64_t)n * w_ns];
        for (int k = K; k < Kp; ++k) dst[k] = 0;
    }
    enum { MBLK = 32 };
    int fail = 0;
#pragma omp parallel if (parallel)
    {
        int16_t* Ab = (int16_t*)aligned_alloc(64, (size_t)MBLK * Kp * sizeof(int16_t));
        if (!Ab) {
#pragma omp atomic write
            fail = 1;
        }
#pragma omp for schedule(dynamic, 1)
        for (int64_t m0 = 0; m0 < M; m0 += MBLK) {
            if (!Ab) continue;
            const int mb = (int)(M - m0 < MBLK ? M - m0 : MBLK);
            for (int i = 0; i < mb; ++i) {
                const uint8_t* su = (const uint8_t*)A + (m0 + i) * a_rs;
                const int8_t* ss = (const int8_t*)su;
                int16_t* dst = Ab + (size_t)i * Kp;
                for (int k = 0; k < K; ++k) dst[k] = a_unsigned ? (int16_t)su[(int64_t)k * a_cs] : (int16_t)ss[(int64_t)k * a_cs];
                for (int k = K; k < Kp; ++k) dst[k] = 0;
            }
            for (int n0 = 0; n0 < N; n0 += 4)
                for (int i0 = 0; i0 < mb; i0 += 4) {
                    int32_t acc[4][4] = {{0}};
                    const int16_t* a[4];
                    const int16_t* w[4];
                    for (int t = 0; t < 4; ++t) {
                        a[t] = Ab + (size_t)(i0 + t < mb ? i0 + t : i0) * Kp;
                        w[t] = Wt + (size_t)(n0 + t < N ? n0 + t : n0) * Kp;
                    }
                    for (int k = 0; k < Kp; ++k)   /* signed wrap is defined here: the file is built with -fwrapv */
                        for (int i = 0; i < 4; ++i)
                            for (int j = 0; j < 4; ++j) acc[i][j] += (int32_t)a[i][k] * (int32_t)w[j][k];
                    for (int i = 0; i < 4 && i0 + i < mb; ++i)
                        for (int j = 0; j < 4 && n0 + j < N; ++j) {
                            const int32_t v = (int32_t)((uint32_t)acc[i][j] + (uint32_t)(bias ? bias[n0 + j] : 0));
                            int64_t y = srs_out(v, shift, rounding, out_dtype);
                            if (relu && y < 0) y = 0;
                            store_out(Y, (m0 + i0 + i) * ldy + n0 + j, y, out_dtype);
                        }
                }
        }
        free(Ab);
    }
    free(Wt);
    return fail ? -2 : 0;
#endif
}

/* Dense: relu?(srs(A.W + bias)).  dense_single::run,
 * templates/nnet_utils/dense_bias_relu/dense_bias_relu.cpp:67-166 (bias as accumulator init
 * :114-124, acc32 MACs :132-151, ReLU after saturation :153-157).
 * A [M,K] row-major (pitch lda), W [K,N] row-major, bias [N] or NULL, Y [M,N] (pitch ldy). */
ORC_API int orc_dense_i8(const void* A, int64_t lda, const int8_t* W, const int32_t* bias, void* Y, int64_t ldy,
                         int64_t M, int K, int N, int shift, int rounding, int relu, int out_dtype, int a_unsigned) {
    if (M < 0 || K <= 0 || N <= 0 || shift < 0 || shift > 62) return -1;
    if (M == 0) return 0;
    return gemm_i8(A, lda, 1, a_unsigned, W, N, 1, bias, Y, ldy, M, K, N, shift, rounding, relu, out_dtype, 1);
}

/* Batched dynamic MatMul: C_b = srs(op(A_b).op(B_b)).  matmul_single::run,
 * templates/nnet_utils/matmul/matmul.cpp:32-118; TRANSPOSE_A/B (:60-77) read the stored operand
 * with its two axes swapped.  Stored A_b is [M,K] (or [K,M] when trans_a) with pitch lda;
 * stored B_b is [K,N] (or [N,K] when trans_b) with pitch ldb. */
ORC_API int orc_bmm_i8(const void* A, int64_t lda, int64_t stride_a, const int8_t* B, int64_t ldb, int64_t stride_b,
                       void* C, int64_t ldc, int64_t stride_c, int64_t batch, int M, int K, int N, int trans_a,
                       int trans_b, int shift, int rounding, int out_dtype, int a_unsigned) {
    if (batch < 0 || M <= 0 || K <= 0 || N <= 0 || shift < 0 || shift > 62) return -1;
    const int esz = out_dtype == 2 ? 2 : 1;
    int fail = 0;
#pragma omp parallel for schedule(static)
    for (int64_t b = 0; b < batch; ++b) {
        const int rc = gemm_i8((const uint8_t*)A + b * stride_a, trans_a ? 1 : lda, trans_a ? lda : 1, a_unsigned,
                               B + b * stride_b, trans_b ? 1 : ldb, trans_b ? ldb : 1, NULL,
                               (uint8_t*)C + b * stride_c * esz, ldc, M, K, N, shift, rounding, 0, out_dtype, 0);
        if (rc != 0) {
#pragma omp atomic write
            fail = rc;
        }
    }
    return fail;
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
