// Internal launcher prototypes shared between the .cu files and the C-ABI layer.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

// Generic strided / batched int8 GEMM on dp4a.  Strides in elements.
int a4c_launch_gemm_simt(const void* A, long long a_rs, long long a_cs, long long a_bs, const void* B,
                         long long b_ks, long long b_ns, long long b_bs, const int32_t* bias, void* C,
                         long long ldc, long long c_bs, long long batch, long long M, int K, int N, int shift,
                         int rounding, int relu, int out_dtype, int a_unsigned, cudaStream_t stream);

// 16-bit operand combinations (gemm_wide.cu): A int8/int16, B int8/int16, 32-bit wrapping or 64-bit accumulator.
// Strides in elements.
int a4c_launch_gemm_wide(const void* A, int a_bytes, long long a_rs, long long a_cs, long long a_bs, const void* B,
                         int b_bytes, long long b_ks, long long b_ns, long long b_bs, const int32_t* bias, void* C,
                         long long ldc, long long c_bs, long long batch, long long M, int K, int N, int shift,
                         int rounding, int relu, int out_dtype, int acc_bits, cudaStream_t stream);

// Float-simulation path (float_ops.cu): kind 0 bfloat16, 1 float32, 2 fp8 E4M3 storage; float32 accumulation.
int a4c_launch_gemm_float(const void* A, long long a_rs, long long a_cs, long long a_bs, const void* B, long long b_ks,
                          long long b_ns, long long b_bs, const float* bias, void* C, long long ldc, long long c_bs,
                          long long batch, long long M, int K, int N, int relu, int kind, cudaStream_t stream);
int a4c_launch_add_float(const void* a, long long lda, const void* b, long long ldb, void* out, long long ldo,
                         long long rows, long long cols, int kind, cudaStream_t stream);

// tcgen05 / TMA / TMEM int8 GEMM: A [M,K] K-contiguous, Wt [N,K] K-contiguous.
// cta_pair = 0: one CTA per 128x256 tile; 1: a CTA pair (cta_group::2) per 256x256 tile.
int a4c_launch_dense_tc(const void* A, long long lda, const void* Wt, long long ldw, const int32_t* bias,
                        void* Y, long long ldy, long long M, int K, int N, int shift, int rounding, int relu,
                        int out_dtype, int a_unsigned, int cta_pair, int* status_word, cudaStream_t stream);
void a4c_dense_tc_set_resident_w(int on);
void a4c_dense_tc_set_panel_mib(int mib);
long long a4c_dense_tc_panel_bytes();   // weights per column panel of the tile order; 0 = one panel
// 0 if the tensor-core path can take this problem, else an A4C_ERR_* code saying why not.
int a4c_dense_tc_supported(const void* A, long long lda, const void* Wt, long long ldw, const void* Y,
                           long long ldy, long long M, int K, int N, int out_dtype);

// pre_add != 0: the addend is added (saturating) to the input before the statistics; otherwise to the result.
int a4c_launch_layernorm(const int8_t* x, long long ldx, const int16_t* gamma, const int16_t* beta,
                         const int8_t* addend, long long ldadd, int pre_add, int8_t* out, long long ldo, long long rows,
                         int cols, int eps_q0, int out_shift, int rounding, cudaStream_t stream);

int a4c_launch_softmax(const int8_t* x, long long ldx, const void* addend, long long ldadd, void* out,
                       long long ldo, long long rows, int cols, int mode, int B, int S, int Dmax, int inv_shift,
                       int use_clb, int exp_kq, int out_dtype, cudaStream_t stream);

int a4c_launch_add(const void* a, long long lda, const void* b, long long ldb, void* out, long long ldo,
                   long long rows, long long cols, int shift, int rounding, int dtype, cudaStream_t stream);

// Bandwidth-oriented variants of the two row ops (rowops_fast.cu).  They return A4C_ERR_UNSUPPORTED when a
// request lies outside what they prove exact; the caller then uses the generic kernels above.
int a4c_launch_layernorm_fast(const int8_t* x, long long ldx, const int16_t* gamma, const int16_t* beta,
                              const int8_t* addend, long long ldadd, int pre_add, int8_t* out, long long ldo,
                              long long rows, int cols, int eps_q0, int out_shift, int rounding, int gamma_absmax,
                              int* status, cudaStream_t stream);
int a4c_launch_softmax_fast(const int8_t* x, long long ldx, const void* addend, long long ldadd, void* out,
                            long long ldo, long long rows, int cols, int mode, int B, int S, int Dmax, int inv_shift,
                            int use_clb, int exp_kq, int out_dtype, int* status, cudaStream_t stream);

// Tuning overrides of rowops_fast.cu (0 = automatic, negative leaves a value unchanged).
void a4c_rowops_fast_tuning(int chunks_per_lane, int min_stages);
void a4c_rowops_fast_contig(int on);

// tcgen05 batched MatMul (bmm_tc.cu).  B stored [N,K] when trans_b (K-major operand) or [K,N] (MN-major operand).
int a4c_bmm_tc_supported(const void* A, long long lda, long long stride_a, const void* B, long long ldb,
                         long long stride_b, const void* C, long long ldc, long long stride_c, long long batch, int M,
                         int K, int N, int trans_a, int trans_b, int out_dtype);
int a4c_launch_bmm_tc(const void* A, long long lda, long long stride_a, const void* B, long long ldb, long long stride_b,
                      void* C, long long ldc, long long stride_c, long long batch, int M, int K, int N, int trans_a,
                      int trans_b, int shift, int rounding, int out_dtype, int a_unsigned, int* status_word,
                      cudaStream_t stream);
// Dense over a transposed input view on the same kernel: A_b stored [K, M] (an MN-major A operand), W^T [N, K] shared
// by every batch entry, int32 bias or NULL, ReLU clamp.
int a4c_dense_ta_tc_supported(const void* A, long long lda, long long stride_a, const void* Wt, long long ldw, const void* Y,
                              long long ldy, long long stride_y, long long batch, int M, int K, int N, int out_dtype);
int a4c_launch_dense_ta_tc(const void* A, long long lda, long long stride_a, const void* Wt, long long ldw,
                           const int32_t* bias, void* Y, long long ldy, long long stride_y, long long batch, int M, int K,
                           int N, int shift, int rounding, int relu, int out_dtype, int a_unsigned, int* status_word,
                           cudaStream_t stream);

// A chain of narrow Dense layers as one kernel (mlp_small.cu), and the choice a4c_mlp_i8 makes (mlp_chain.cu).
int a4c_mlp_small_supported(int n_layers, const int* dims, int out_dtype);
int a4c_launch_mlp_small(const void* X, long long ldx, int x_unsigned, int n_layers, const int* dims,
                         const int8_t* const* Wt, const long long* ldw, const int32_t* const* bias, const int* shift,
                         const int* relu, int rounding, void* Y, long long ldy, int out_dtype, long long M,
                         cudaStream_t stream);
void a4c_mlp_set_path(int path);

// Fused attention heads (attention_tc.cu): scores, softmax and the value product in one kernel; `heads` heads per
// batch entry, hstride_* bytes apart (ignored for heads == 1).
int a4c_attention_tc_supported(const void* q, long long ldq, long long stride_q, const void* k, long long ldk,
                               long long stride_k, const void* v, long long ldv, long long stride_v, const void* out,
                               long long ldo, long long stride_o, long long batch, int sq, int sk, int dh, int qk_shift,
                               int pv_shift, int sm_mode, int B, int S, int Dmax, int inv_shift, int heads,
                               long long hstride_q, long long hstride_k, long long hstride_v, long long hstride_o);
int a4c_launch_attention_tc(const void* q, long long ldq, long long stride_q, const void* k, long long ldk,
                            long long stride_k, const void* v, long long ldv, long long stride_v, void* out,
                            long long ldo, long long stride_o, long long batch, int sq, int sk, int dh, int qk_shift,
                            int pv_shift, int rounding, int sm_mode, int B, int S, int Dmax, int inv_shift, int use_clb,
                            int exp_kq, int heads, long long hstride_q, long long hstride_k, long long hstride_v,
                            long long hstride_o, int* status_word, cudaStream_t stream);

// CTA-pair (cta_group::2) Dense: one 256 x 256 tile per two SMs (dense_tc2.cu); same argument rules as
// a4c_launch_dense_tc.
int a4c_launch_dense_tc2(const void* A, long long lda, const void* Wt, long long ldw, const int32_t* bias,
                         void* Y, long long ldy, long long M, int K, int N, int shift, int rounding, int relu,
                         int out_dtype, int a_unsigned, int* status_word, cudaStream_t stream);

// Records a failed CUDA call for a4c_last_cuda_error() (thread-local, capi.cu); returns true when e is cudaSuccess.
bool a4c_note_cuda(cudaError_t e);

// The status word inside the fixed scratch array of a4c_mlp_i8_static (mlp_chain.cu): copies it to *out and
// clears it when non-zero.  *out = 0 and A4C_OK when the array has not been set up on the current device.  The
// caller has synchronised whatever work could still write the word.  Allocates nothing.
int a4c_mlp_static_status_take(int* out);

// tcgen05 floating-point Dense (dense_tcf.cu): kind 0 = bfloat16 (kind::f16), 2 = fp8 E4M3 (kind::f8f6f4), float32
// accumulation.  Pitches in elements.  _supported returns 0 or the A4C_ERR_* code that says why not.
int a4c_dense_tcf_supported(const void* A, long long lda, const void* Wt, long long ldw, const void* Y, long long ldy,
                            long long M, int K, int N, int kind);
int a4c_launch_dense_tcf(const void* A, long long lda, const void* Wt, long long ldw, const float* bias, void* Y,
                         long long ldy, long long M, int K, int N, int relu, int kind, int* status_word,
                         cudaStream_t stream);

// tcgen05 int16 x int8 Dense (dense_tc16.cu): the activation's two byte digits against the int8 weights, combined in
// wrapping 32-bit arithmetic.  Uses a fixed per-device workspace (64 MiB, allocated on first use).  Pitches in elements.
int a4c_dense_tc16_supported(const void* A, long long lda, const void* Wt, long long ldw, const void* Y, long long ldy,
                             long long M, int K, int N, int out_dtype);
int a4c_launch_dense_tc16(const int16_t* A, long long lda, const int8_t* Wt, long long ldw, const int32_t* bias, void* Y,
                          long long ldy, long long M, int K, int N, int shift, int rounding, int relu, int out_dtype,
                          int* status_word, cudaStream_t stream);

// tcgen05 int8 Dense for K <= 512 and N a multiple of 128 (dense_tcs.cu): the general kernel's 128 x 256 tiles and
// resident weight tile, twelve epilogue warps in three groups that take half tiles in rotation.  The caller has checked
// the alignment rules of a4c_dense_tc_supported.
int a4c_dense_tcs_supported(long long M, int K, int N, int out_dtype, int sms);
int a4c_launch_dense_tcs(const void* A, long long lda, const void* Wt, long long ldw, const int32_t* bias, void* Y,
                         long long ldy, long long M, int K, int N, int shift, int rounding, int relu, int out_dtype,
                         int a_unsigned, int* status_word, cudaStream_t stream);

// Dense -> residual Add -> LayerNorm in one kernel for layers 256 features wide (dense_ln.cu).
int a4c_dense_ln_supported(long long M, int K, int N, long long lda, long long ldw, long long ldr, long long ldo,
                           int shift, int rounding, int out_shift, int eps_q0, int gamma_absmax);
int a4c_launch_dense_ln(const void* A, long long lda, int a_unsigned, const void* Wt, long long ldw, const int32_t* bias,
                        int shift, int relu, const int8_t* residual, long long ldr, const int16_t* gamma,
                        const int16_t* beta, int8_t* out, long long ldo, long long M, int K, int N, int eps_q0,
                        int out_shift, int rounding, int gamma_absmax, int* status_word, cudaStream_t stream);
void a4c_dense_ln_set_enabled(int on);
