/*
 * aie4ml_b200 -- C ABI of the sm_100a kernels that execute aie4ml's lowered, quantized operators.
 *
 * This is the drop-in boundary under the Python runtime.  The reference project (aie4ml) has no FFI
 * for this path: it generates a Vitis C++ project and runs it through `make`
 * (src/aie4ml/model.py:82-147, src/aie4ml/simulation.py:337-341).  Each entry point below therefore
 * cites the reference KERNEL whose arithmetic it replaces and the reference parameter block that
 * defines its arguments.
 *
 * Conventions
 *   - every pointer is DEVICE memory owned by the caller (except where a name ends in _host);
 *   - pitches (ld*) and strides are in ELEMENTS of the tensor they describe;
 *   - calls are asynchronous on `stream` (a cudaStream_t passed as void*; NULL = default stream);
 *   - the return value is 0 or a negative A4C_ERR_* code; invalid shapes / alignment are rejected
 *     on the host before anything is launched; nothing here calls exit() or traps;
 *   - rounding codes: 0 floor, 1 ceil, 2 positive_inf (round half up), 3 negative_inf,
 *     4 symmetric_inf (half away from zero), 5 symmetric_zero (half toward zero), 6 conv_even,
 *     7 conv_odd -- the AIE-API rounding tokens the reference's resolver emits
 *     (src/aie4ml/op_impls/utils/precision.py:13-21) plus the ones it does not;
 *   - dtype codes: 0 int8, 1 uint8, 2 int16;
 *   - saturation is always on, as in every reference kernel
 *     (templates/firmware/variants/dense_bias_relu/parameters.h.jinja:26-29).
 */
#ifndef AIE4ML_B200_H
#define AIE4ML_B200_H

#include <stdint.h>

#if defined(__GNUC__)
#define A4C_API __attribute__((visibility("default")))
#else
#define A4C_API
#endif

#ifdef __cplusplus
extern "C" {
#endif

#define A4C_OK 0
#define A4C_ERR_INVALID_ARG (-1)
#define A4C_ERR_ALIGNMENT (-2)
#define A4C_ERR_UNSUPPORTED (-3)
#define A4C_ERR_CUDA (-4)
#define A4C_ERR_TOO_LARGE (-5)
#define A4C_ERR_DEVICE_TIMEOUT (-6)

/* GEMM kernel selection for a4c_dense_i8 */
#define A4C_ALGO_AUTO 0
#define A4C_ALGO_SIMT 1      /* dp4a tiles, any shape / stride */
#define A4C_ALGO_TCGEN05 2   /* tcgen05 + TMA + TMEM, one CTA per 128x256 tile */
#define A4C_ALGO_TCGEN05_PAIR 3 /* tcgen05 cta_group::2, a CTA pair per 256x256 tile */

/* Options for a4c_set_option */
#define A4C_OPT_ROWOP_PATH 0 /* 0 = auto (bandwidth-oriented row kernels when they apply), 1 = generic kernels only */
#define A4C_OPT_BMM_PATH 1   /* 0 = auto (tcgen05 batched MatMul when its alignment rules hold), 1 = dp4a kernel only */
#define A4C_OPT_DENSE_RESIDENT_W 5 /* tcgen05 Dense, K <= 512: a CTA keeps its weight tile in shared memory and streams A only.  0 = off, 1 = in the general kernel (eight epilogue warps), 2 (default) = 1 plus, when N is a multiple of 128, the short-reduction kernel (same tiles, twelve epilogue warps on half tiles) */
#define A4C_OPT_DENSE_PANEL_MIB 8 /* tcgen05 Dense, streaming tile order: MiB of weights per column panel (default 32; 0 = one panel, column tile fastest over the whole width) */
#define A4C_OPT_WIDE_DENSE_PATH 9 /* a4c_dense_i16 with int8 weights: 0 = auto (tcgen05, the activation's two byte digits in turn), 1 = SIMT kernel only */
#define A4C_OPT_DENSE_LN_PATH 10 /* a4c_dense_add_layernorm_i8 / _supported: 0 = the single kernel where it applies (default), 1 = never (the plan keeps Dense and Add + LayerNorm as two launches) */
#define A4C_OPT_FLOAT_DENSE_PATH 7 /* a4c_dense_f, bfloat16 / fp8: 0 = auto (tcgen05 kernel when its alignment rules hold), 1 = tiled SIMT kernel only */
#define A4C_OPT_MLP_PATH 4   /* a4c_mlp_i8: 0 = auto, 1 = one Dense launch per layer, 2 = the single-kernel narrow chain only */
/* Tuning of the bandwidth-oriented row kernels (results do not depend on either): */
#define A4C_OPT_ROWOP_CHUNKS_PER_LANE 2 /* 0 = automatic (default), else 1, 2 or 4: 16-element chunks of one row per lane */
#define A4C_OPT_ROWOP_MIN_STAGES 3      /* 0 = automatic (default), else 2..4: least depth of the per-warp copy ring */
#define A4C_OPT_ROWOP_CONTIG_COPY 6     /* rows adjacent in memory and several rows per warp item: 1 = one bulk copy per item, 0 = one per row */

/* Library version (major*10000 + minor*100 + patch). */
A4C_API int a4c_version(void);

/* Human-readable text for an A4C_ERR_* code (static storage). */
A4C_API const char* a4c_error_string(int code);

/* Text of the last CUDA runtime error seen by this library on the calling thread (static storage). */
A4C_API const char* a4c_last_cuda_error(void);

/* Process-wide tuning / debugging switch; returns A4C_ERR_INVALID_ARG for an unknown option or value. */
A4C_API int a4c_set_option(int option, int value);

/*
 * Reads (and clears) the current device's kernel status word after synchronising `stream`.
 * 0 = every bounded device-side wait completed; otherwise the code of the first wait that gave up
 * (101 producer/empty slot, 102 MMA/accumulator free, 103 MMA/operands landed, 104 epilogue/accumulator
 * ready, 201 / 202 row of a LayerNorm / Softmax input landed).  Returns A4C_OK, or A4C_ERR_DEVICE_TIMEOUT when *status != 0, or A4C_ERR_CUDA.
 */
A4C_API int a4c_device_status(int* status, void* stream);

/*
 * Dense: Y = relu?( saturate( round_shift( A . W + bias, shift ) ) ), int8 x int8 -> int32 accumulate.
 * Replaces dense_single/first/middle/last::run
 * (src/aie4ml/templates/nnet_utils/dense_bias_relu/dense_bias_relu.cpp:67-430); arguments are the
 * fields of its parameter block (templates/firmware/variants/dense_bias_relu/parameters.h.jinja:1-31:
 * SHIFT, ROUNDING, USE_BIAS, USE_RELU, data_t/result_t).
 *   A   [M, K]  int8 (or uint8 when a_unsigned), K contiguous, row pitch lda
 *   Wt  [N, K]  int8, the weight matrix TRANSPOSED so K is contiguous, row pitch ldw
 *   bias[N]     int32 at the accumulator's fixed point, or NULL
 *   Y   [M, N]  out_dtype, row pitch ldy
 * algo: A4C_ALGO_AUTO picks tcgen05 when its alignment rules hold (lda, ldw, ldy*elt multiples of 16
 * bytes, 16-byte aligned bases, N multiple of 16, 8-bit output), else the SIMT kernel.
 */
A4C_API int a4c_dense_i8(const void* A, int64_t lda, const int8_t* Wt, int64_t ldw, const int32_t* bias, void* Y,
                 int64_t ldy, int64_t M, int K, int N, int shift, int rounding, int relu, int out_dtype,
                 int a_unsigned, int algo, void* stream);

/*
 * Batched dynamic MatMul: C_b = saturate( round_shift( op(A_b) . op(B_b), shift ) ), b = 0..batch-1.
 * Replaces matmul_single/first/middle/last::run
 * (src/aie4ml/templates/nnet_utils/matmul/matmul.cpp:32-390; TRANSPOSE_A/B :60-77) applied once per
 * leading index -- the rank-2 contract of op_impls/families/matmul/resolver.py:440-463, batched.
 *   stored A_b: [M, K] (or [K, M] when trans_a), pitch lda, batch stride stride_a; uint8 when a_unsigned
 *   stored B_b: [K, N] (or [N, K] when trans_b), pitch ldb, batch stride stride_b; always int8
 *   C_b: [M, N] out_dtype, pitch ldc, batch stride stride_c
 * The tcgen05 kernel is used when the stored A is not transposed, pitches / strides / bases are multiples of
 * 16 bytes, N is a multiple of 16 and the output is 8-bit; otherwise the dp4a kernel.
 */
A4C_API int a4c_bmm_i8(const void* A, int64_t lda, int64_t stride_a, const int8_t* B, int64_t ldb, int64_t stride_b,
               void* C, int64_t ldc, int64_t stride_c, int64_t batch, int M, int K, int N, int trans_a,
               int trans_b, int shift, int rounding, int out_dtype, int a_unsigned, void* stream);

/*
 * Integer LayerNorm over rows of `cols` (a power of two) int8 values, int8 out.
 * Replaces layernorm_i8::run / layernorm_i8_tiled::run
 * (src/aie4ml/templates/nnet_utils/layer_norm/layer_norm.cpp:15-231); arguments follow
 * templates/firmware/variants/layer_norm/parameters.h.jinja:1-24 (EPS_Q0, OUT_SHIFT, ROUNDING;
 * GAMMA_SHIFT is the constant 7).  gamma is int16 Q7, beta int16 Q15, both [cols].
 * addend (or NULL): an int8 tensor shaped like the output; when given, the kernel stores
 * saturate(layernorm(x) + addend) -- the exact-type Add of elementwise_add.cpp:12-37 fused in.
 * gamma_absmax: an upper bound of |gamma[c]| known to the caller (the packer has it), or 0 when unknown.
 * It only selects between kernels (a bound <= 16383 admits the bandwidth-oriented one); results do not
 * depend on it as long as it is a true bound.
 */
A4C_API int a4c_layernorm_i8(const int8_t* x, int64_t ldx, const int16_t* gamma, const int16_t* beta,
                     const int8_t* addend, int64_t ldadd, int8_t* out, int64_t ldo, int64_t rows, int cols,
                     int eps_q0, int out_shift, int rounding, int gamma_absmax, void* stream);

/*
 * out = layernorm( saturate_i8(x + residual) ): the exact-type residual Add of elementwise_add.cpp:12-37
 * (SHIFT = 0) followed by the LayerNorm above, in one pass over the rows -- the sum is never written.
 * The reference runs these as two kernels; the result is the same bytes as a4c_add_sat then a4c_layernorm_i8.
 */
A4C_API int a4c_add_layernorm_i8(const int8_t* x, int64_t ldx, const int8_t* residual, int64_t ldr,
                         const int16_t* gamma, const int16_t* beta, int8_t* out, int64_t ldo, int64_t rows,
                         int cols, int eps_q0, int out_shift, int rounding, int gamma_absmax, void* stream);

/*
 * out = layernorm( saturate_i8( dense(A) + residual ) ) in ONE kernel: the Dense of dense_bias_relu.cpp:67-166
 * (int8 output, bias / shift / rounding / relu as a4c_dense_i8), the exact-type residual Add of
 * elementwise_add.cpp:12-37 (SHIFT = 0) and the LayerNorm of layer_norm.cpp:15-121 over the Dense's N columns.
 * The reference connects the three kernels by streams ("direct" transport, passes/transport/classify.py:25-49), so
 * neither intermediate touches memory there either; as separate launches here each would make a round trip through HBM.
 * One accumulator tile must hold whole rows: N = 256, all pitches multiples of 16 bytes, bases 16-byte aligned, and
 * the LayerNorm within the bandwidth-oriented row kernel's envelope (tokens other than symmetric_* / conv_odd,
 * gamma_absmax in [1, 16383], eps_q0 in [1, 2^20], out_shift <= 13).  a4c_dense_add_layernorm_supported returns A4C_OK when
 * the request is inside that envelope and A4C_ERR_UNSUPPORTED otherwise (then run a4c_dense_i8 and
 * a4c_add_layernorm_i8); the launch entry returns the same codes.  The result is the same bytes as those two calls.
 *   A: [M, K] int8 (a_unsigned = 1: uint8), pitch lda;  Wt: [N, K] int8, pitch ldw;  bias: int32 [N] or NULL
 *   residual: [M, N] int8, pitch ldr;  gamma int16 Q7 [N], beta int16 Q15 [N];  out: [M, N] int8, pitch ldo
 */
A4C_API int a4c_dense_add_layernorm_supported(int64_t M, int K, int N, int64_t lda, int64_t ldw, int64_t ldr, int64_t ldo,
                                      int shift, int rounding, int out_shift, int eps_q0, int gamma_absmax);
A4C_API int a4c_dense_add_layernorm_i8(const void* A, int64_t lda, int a_unsigned, const int8_t* Wt, int64_t ldw,
                               const int32_t* bias, int shift, int relu, const int8_t* residual, int64_t ldr,
                               const int16_t* gamma, const int16_t* beta, int8_t* out, int64_t ldo, int64_t M, int K,
                               int N, int eps_q0, int out_shift, int rounding, int gamma_absmax, void* stream);

/*
 * Quantized Softmax over rows of int8, output uint8 (dtype 1) or int16 (dtype 2).
 * mode 0 = HCCS clipped-linear surrogate: replaces softmax_i8::softmax_row / softmax_i8_tiled::run
 *          (src/aie4ml/templates/nnet_utils/softmax/softmax.cpp:20-88, 159-239); B, S, Dmax, inv_shift,
 *          use_clb as in templates/firmware/variants/softmax/parameters.h.jinja:1-44.
 * mode 1 = accurate integer exp: replaces softmax_exp_i8::run / softmax_exp_i8_tiled::run + exp_score16
 *          (softmax.cpp:252-384); exp_kq = EXP_KQ in [1, 128].
 * addend (or NULL): tensor of the OUTPUT dtype; when given the kernel stores saturate(softmax(x) + addend).
 */
A4C_API int a4c_softmax_i8(const int8_t* x, int64_t ldx, const void* addend, int64_t ldadd, void* out, int64_t ldo,
                   int64_t rows, int cols, int mode, int B, int S, int Dmax, int inv_shift, int use_clb,
                   int exp_kq, int out_dtype, void* stream);

/*
 * The 16-bit operand combinations of the same two operators (reference width table
 * src/aie4ml/op_impls/families/matmul/common.py:52: int16 x int8 and int16 x int16; accumulator choice
 * src/aie4ml/op_impls/utils/precision.py:116-127): A is int16; W / B is int8 (w_dtype 0: 32-bit accumulator that
 * wraps) or int16 (w_dtype 2: 64-bit accumulator).  Otherwise the contracts of a4c_dense_i8 / a4c_bmm_i8
 * (dense_bias_relu.cpp:67-166, matmul.cpp:32-118): bias int32, SRS, saturation, ReLU after it; shift <= 31
 * (acc32) or <= 62 (acc64).  Pitches and strides in ELEMENTS of the respective tensor.
 * a4c_dense_i16 with int8 weights runs on the tensor cores when A and W^T start on 16 bytes with 16-byte row pitches
 * and K >= 16: the activations are split into a signed high-byte plane and an unsigned low-byte plane (in a fixed
 * 64 MiB workspace the library allocates per device on first use; rows are processed in chunks that fit it), each
 * plane meets the weights in tcgen05.mma kind::i8, and (high << 8) + low + bias is formed in wrapping 32-bit
 * arithmetic, which is bit for bit the reference's wrapping accumulation.  Everything else (int16 weights, other
 * pitches, a4c_bmm_i16) runs on a tiled SIMT kernel.
 */
A4C_API int a4c_dense_i16(const int16_t* A, int64_t lda, const void* Wt, int w_dtype, int64_t ldw, const int32_t* bias,
                  void* Y, int64_t ldy, int64_t M, int K, int N, int shift, int rounding, int relu, int out_dtype,
                  void* stream);
A4C_API int a4c_bmm_i16(const int16_t* A, int64_t lda, int64_t stride_a, const void* B, int b_dtype, int64_t ldb,
                int64_t stride_b, void* C, int64_t ldc, int64_t stride_c, int64_t batch, int M, int K, int N,
                int trans_a, int trans_b, int shift, int rounding, int out_dtype, void* stream);

/*
 * Dense whose input arrives through a view that swaps the last two axes: the reference's TRANSPOSE_INPUT flag
 * (src/aie4ml/templates/firmware/variants/dense_bias_relu/parameters.h.jinja:12, read by
 * dense_bias_relu.cpp:99,135; set from the input's io_view in op_impls/families/matmul/dense.py:130).
 *   stored A_b: [K, M] a_dtype (int8 / uint8 / int16), pitch lda, batch stride stride_a   (logical input: A_b^T)
 *   W^T [N, K] w_dtype (int8, or int16 with an int16 input), pitch ldw; bias int32 or NULL
 *   Y_b: [M, N] out_dtype, pitch ldy, batch stride stride_y
 * Arithmetic, accumulator width and SRS exactly as a4c_dense_i8 / a4c_dense_i16.  Pitches and strides in
 * ELEMENTS.  8-bit inputs with int8 weights run on the tensor cores when lda, ldw, ldy, the batch strides and N are
 * multiples of 16, the pointers start on 16 bytes and the output is int8 / uint8: the stored [K, M] tile is an
 * MN-major A operand of tcgen05.mma (128-byte-swizzled rows of m).  Other cases run on the any-stride dp4a / wide
 * kernels.
 */
A4C_API int a4c_dense_ta(const void* A, int a_dtype, int64_t lda, int64_t stride_a, const void* Wt, int w_dtype,
                 int64_t ldw, const int32_t* bias, void* Y, int64_t ldy, int64_t stride_y, int64_t batch, int M, int K,
                 int N, int shift, int rounding, int relu, int out_dtype, void* stream);

/*
 * Float-simulation path (reference AIEConfig.ComputeDtype = 'bfloat16' | 'float32',
 * src/aie4ml/passes/force_float_mode.py:22-46; float contract of the matmul family
 * src/aie4ml/op_impls/families/matmul/resolver.py:110-127): the same Dense / MatMul / Add operators computed in
 * floating point.  fdtype 0 = bfloat16 (tensors hold the 16 bits), 1 = float32, 2 = fp8 E4M3 (finite-only
 * variant, the reference's 'fp8_e4m3' of src/aie4ml/aie_types.py:38, tensors hold the 8 bits; results beyond
 * +-448 saturate); accumulation in float32, bias float32, optional ReLU, results rounded to nearest-even into the
 * storage type.  Pitches / strides in elements.
 * a4c_dense_f with bfloat16 or fp8 operands runs on the tensor cores (tcgen05.mma kind::f16 / kind::f8f6f4, float32
 * accumulators in TMEM) when A, W^T and Y start on 16 bytes, their pitches are multiples of 16 bytes and K spans at
 * least 32 bytes; otherwise, and for float32, on a tiled SIMT kernel (any shape and stride).
 * Held to the reference's tolerances (tests/test_float_sim.py:87-93), not to bit equality.
 */
A4C_API int a4c_dense_f(const void* A, int fdtype, int64_t lda, const void* Wt, int64_t ldw, const float* bias, void* Y,
                int64_t ldy, int64_t M, int K, int N, int relu, void* stream);
A4C_API int a4c_bmm_f(const void* A, int fdtype, int64_t lda, int64_t stride_a, const void* B, int64_t ldb,
              int64_t stride_b, void* C, int64_t ldc, int64_t stride_c, int64_t batch, int M, int K, int N, int trans_a,
              int trans_b, void* stream);
A4C_API int a4c_add_f(const void* a, int64_t lda, const void* b, int64_t ldb, void* out, int64_t ldo, int64_t rows,
              int64_t cols, int fdtype, void* stream);

/*
 * One attention head, fused:  out_b = srs( softmax_u8( srs(Q_b . K_b^T, qk_shift) ) . V_b, pv_shift )  for every
 * batch entry b.  The reference has no single kernel for this: it is the chain of its three kernels
 *   matmul_single::run with TRANSPOSE_B (src/aie4ml/templates/nnet_utils/matmul/matmul.cpp:32-118)
 *   -> softmax (softmax.cpp:20-88 HCCS / :252-384 exp, uint8 output)
 *   -> matmul_single::run (uint8 x int8),
 * with the int8 scores and uint8 probabilities kept on chip, and it produces exactly the bytes the three
 * calls a4c_bmm_i8 / a4c_softmax_i8 / a4c_bmm_i8 produce.
 *   q [batch][sq][dh], k [batch][sk][dh], v [batch][sk][dh], out [batch][sq][dh], all int8, row pitches ld*
 *   and batch strides stride_* in bytes (a head is a column slice of a wider tensor: pitch > dh).
 *   qk_shift / pv_shift / rounding: the SRS parameters of the two MatMuls (one rounding token for both).
 *   sm_mode, B, S, Dmax, inv_shift, use_clb, exp_kq: as a4c_softmax_i8.
 * Supported: sk == 128, dh == 64, 16-byte aligned pointers / pitches / strides, inv_shift <= 22, non-negative
 * HCCS scores, shifts both zero or both non-zero.  a4c_attention_i8_supported answers A4C_OK or the error
 * code a4c_attention_i8 would return for the same arguments, without launching anything; callers fall back to
 * the three separate calls.
 */
A4C_API int a4c_attention_i8_supported(const int8_t* q, int64_t ldq, int64_t stride_q, const int8_t* k, int64_t ldk,
                               int64_t stride_k, const int8_t* v, int64_t ldv, int64_t stride_v, const int8_t* out,
                               int64_t ldo, int64_t stride_o, int64_t batch, int sq, int sk, int dh, int qk_shift,
                               int pv_shift, int sm_mode, int B, int S, int Dmax, int inv_shift);
A4C_API int a4c_attention_i8(const int8_t* q, int64_t ldq, int64_t stride_q, const int8_t* k, int64_t ldk,
                     int64_t stride_k, const int8_t* v, int64_t ldv, int64_t stride_v, int8_t* out, int64_t ldo,
                     int64_t stride_o, int64_t batch, int sq, int sk, int dh, int qk_shift, int pv_shift,
                     int rounding, int sm_mode, int B, int S, int Dmax, int inv_shift, int use_clb, int exp_kq,
                     void* stream);

/*
 * The same for `heads` heads per batch entry in one launch: head h of batch entry b starts at
 * base + b * stride_* + h * hstride_* (bytes, multiples of 16) in each of q, k, v and out.  For the usual layout,
 * heads as 64-byte column slices of [rows, heads * 64] tensors (what the reference's Split / Concat placeholders
 * around the per-head MatMuls describe, src/aie4ml/passes/fold_views.py), hstride = 64 and the heads of one row share
 * their memory lines, which then leave HBM once instead of once per head.  Results are those of `heads` calls of
 * a4c_attention_i8.
 */
A4C_API int a4c_attention_heads_i8_supported(const int8_t* q, int64_t ldq, int64_t stride_q, int64_t hstride_q,
                                     const int8_t* k, int64_t ldk, int64_t stride_k, int64_t hstride_k, const int8_t* v,
                                     int64_t ldv, int64_t stride_v, int64_t hstride_v, const int8_t* out, int64_t ldo,
                                     int64_t stride_o, int64_t hstride_o, int64_t batch, int heads, int sq, int sk, int dh,
                                     int qk_shift, int pv_shift, int sm_mode, int B, int S, int Dmax, int inv_shift);
A4C_API int a4c_attention_heads_i8(const int8_t* q, int64_t ldq, int64_t stride_q, int64_t hstride_q, const int8_t* k,
                           int64_t ldk, int64_t stride_k, int64_t hstride_k, const int8_t* v, int64_t ldv, int64_t stride_v,
                           int64_t hstride_v, int8_t* out, int64_t ldo, int64_t stride_o, int64_t hstride_o, int64_t batch,
                           int heads, int sq, int sk, int dh, int qk_shift, int pv_shift, int rounding, int sm_mode, int B,
                           int S, int Dmax, int inv_shift, int use_clb, int exp_kq, void* stream);

/*
 * Elementwise out = saturate( round_shift( a + b, shift ) ) over [rows, cols] tensors of one dtype.
 * Replaces elementwise_add_kernel::run
 * (src/aie4ml/templates/nnet_utils/elementwise_add/elementwise_add.cpp:12-37; SHIFT, ROUNDING from
 * templates/firmware/variants/elementwise_add/parameters.h.jinja:1-20).
 */
A4C_API int a4c_add_sat(const void* a, int64_t lda, const void* b, int64_t ldb, void* out, int64_t ldo, int64_t rows,
                int64_t cols, int shift, int rounding, int dtype, void* stream);

/*
 * A chain of Dense layers in one call: X -> Dense_0 -> ... -> Dense_{L-1} -> Y, each with the contract of
 * a4c_dense_i8 and int8 activations between layers.  Replaces consecutive dense_bias_relu kernels wired buffer to
 * buffer by the reference's top graph (src/aie4ml/templates/firmware/top_graph.h.jinja; per-layer arithmetic
 * src/aie4ml/templates/nnet_utils/dense_bias_relu/dense_bias_relu.cpp:67-166).
 *   dims[L+1]   feature counts: dims[0] = inputs of layer 0, dims[L] = outputs of the last layer
 *   Wt[l]       [dims[l+1], ldw[l]] int8, K contiguous;  bias[l] int32[dims[l+1]] or NULL (bias itself may be NULL)
 *   shift[l], relu[l] per layer; one rounding code for the chain; out_dtype applies to the last layer
 * The activations between layers are written to scratch memory the library allocates on first use, grows on
 * demand and keeps per device.  Two calls that overlap in time on one device would share that scratch: issue
 * them on one stream.
 */
A4C_API int a4c_mlp_i8(const void* X, int64_t ldx, int x_unsigned, int n_layers, const int* dims,
                       const int8_t* const* Wt, const int64_t* ldw, const int32_t* const* bias, const int* shift,
                       const int* relu, int rounding, void* Y, int64_t ldy, int out_dtype, int64_t M, void* stream);

/*
 * 1 when a4c_mlp_i8 would run this chain as ONE kernel that keeps every weight and the activations between
 * layers in shared memory (automatic choice: no layer wider than 64, M <= 65536, int8 / uint8 output; with
 * A4C_OPT_MLP_PATH = 2: any chain of up to 8 layers no wider than 256 whose constants fit in shared memory), in
 * which case it uses no scratch memory at all; 0 otherwise.
 */
A4C_API int a4c_mlp_i8_single_kernel(int n_layers, const int* dims, int out_dtype, int64_t M);

/*
 * a4c_mlp_i8 for callers that must not allocate.  (This entry point has no counterpart in the reference: it
 * exists because of how some hosts embed this library, not because of anything aie4ml does.)
 *
 * Who needs it: code that runs a model from a place where cudaMalloc is off limits -- inside another runtime's
 * stream-ordered callback or captured region, in a process whose device memory is owned by its own pool, or in
 * a loop that may never take the CUDA allocator's lock.  Same arguments and results as a4c_mlp_i8, but the
 * activations between layers (and the kernels' status word) live in a fixed array inside the library image
 * instead of allocated scratch.  The function calls no cudaMalloc, cudaFree or allocating library routine.
 *
 * Limit: M * round_up(widest hidden layer, 16) must not exceed A4C_MLP_STATIC_BYTES (4 MiB); beyond that the
 * call returns A4C_ERR_TOO_LARGE and launches nothing.  The array (two such buffers + 256 bytes) is resident on
 * every GPU that loads the library until the process exits.
 *
 * The first call on a device looks up the array's device address and clears its status word; make that first
 * call outside any stream capture.  Every call uses the same array and finds the previous call's activations
 * in it (harmless: each layer overwrites what the next one reads); two calls that overlap in time on one GPU
 * race on it, so keep calls on one stream or order them yourself.
 *
 * status_out (host pointer, or NULL): when given, the call waits for `stream`, stores the kernels' status word
 * there (0 = every bounded device-side wait completed) and returns A4C_ERR_DEVICE_TIMEOUT if it is not 0;
 * with NULL the call stays asynchronous, and a later a4c_device_status() on the same device (which waits for
 * its stream, allocates its own status word on first use, and is therefore for the set-up or shut-down side of
 * such a caller) reports and clears a timeout that a NULL-status call left behind.
 */
#define A4C_MLP_STATIC_BYTES (4u << 20)
A4C_API int a4c_mlp_i8_static(const void* X, int64_t ldx, int x_unsigned, int n_layers, const int* dims,
                              const int8_t* const* Wt, const int64_t* ldw, const int32_t* const* bias,
                              const int* shift, const int* relu, int rounding, void* Y, int64_t ldy, int out_dtype,
                              int64_t M, int* status_out, void* stream);

#ifdef __cplusplus
}
#endif

#endif /* AIE4ML_B200_H */
