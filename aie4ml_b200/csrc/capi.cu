// extern "C" entry points declared in include/aie4ml_b200.h: argument validation on the host,
// kernel selection, and the per-device status word the tensor-core kernels report into.
#include <mutex>

#include "../../include/aie4ml_b200.h"
#include "a4c_common.cuh"
#include "a4c_kernels.h"

namespace {

constexpr int kMaxDevices = 64;
std::mutex g_mutex;
int* g_status[kMaxDevices] = {nullptr};
thread_local const char* t_last_cuda_error = "no error";
int g_rowop_path = 0;  // 0 auto (fast kernels when they apply), 1 generic kernels only
int g_bmm_path = 0;    // 0 auto (tcgen05 when its rules hold), 1 dp4a kernel only
int g_wide_path = 0;   // 0 auto (tcgen05 digit kernel for int16 x int8 when its rules hold), 1 SIMT kernel only
int g_float_path = 0;  // 0 auto (tcgen05 Dense for bfloat16 / fp8 when its rules hold), 1 tiled SIMT kernel only

bool note(cudaError_t e) {
    if (e != cudaSuccess) {
        t_last_cuda_error = cudaGetErrorString(e);
        return false;
    }
    return true;
}

// The status word of the current device, allocated (and zeroed) on first use.
int* status_word() {
    int dev = 0;
    if (!note(cudaGetDevice(&dev)) || dev < 0 || dev >= kMaxDevices) return nullptr;
    std::lock_guard<std::mutex> lock(g_mutex);
    if (g_status[dev] == nullptr) {
        int* p = nullptr;
        if (!note(cudaMalloc(&p, sizeof(int)))) return nullptr;
        if (!note(cudaMemset(p, 0, sizeof(int)))) { cudaFree(p); return nullptr; }
        g_status[dev] = p;
    }
    return g_status[dev];
}

inline bool valid_round(int r) { return r >= 0 && r < A4C_RND_COUNT; }
inline bool valid_dtype(int d) { return d >= 0 && d <= 2; }

int finish() {
    const cudaError_t e = cudaPeekAtLastError();
    return note(e) ? A4C_OK : A4C_ERR_CUDA;
}

}  // namespace

bool a4c_note_cuda(cudaError_t e) { return note(e); }

extern "C" {

int a4c_version(void) { return 100; }

const char* a4c_error_string(int code) {
    switch (code) {
        case A4C_OK: return "ok";
        case A4C_ERR_INVALID_ARG: return "invalid argument (shape, shift or enum value)";
        case A4C_ERR_ALIGNMENT: return "pointer or pitch alignment not supported by the selected kernel";
        case A4C_ERR_UNSUPPORTED: return "no kernel for this request";
        case A4C_ERR_CUDA: return "a CUDA call failed (see a4c_last_cuda_error)";
        case A4C_ERR_TOO_LARGE: return "problem exceeds a stated maximum";
        case A4C_ERR_DEVICE_TIMEOUT: return "a bounded device-side wait gave up";
        default: return "unknown error code";
    }
}

const char* a4c_last_cuda_error(void) { return t_last_cuda_error; }

int a4c_device_status(int* status, void* stream) {
    if (status == nullptr) return A4C_ERR_INVALID_ARG;
    int* word = status_word();
    if (word == nullptr) return A4C_ERR_CUDA;
    cudaStream_t s = (cudaStream_t)stream;
    if (!note(cudaStreamSynchronize(s))) return A4C_ERR_CUDA;
    if (!note(cudaMemcpy(status, word, sizeof(int), cudaMemcpyDeviceToHost))) return A4C_ERR_CUDA;
    if (*status != 0) {
        cudaMemset(word, 0, sizeof(int));
        return A4C_ERR_DEVICE_TIMEOUT;
    }
    // a4c_mlp_i8_static reports into a word of its own (inside its fixed array): a caller that passed no
    // status_out there learns of a timeout here
    const int src = a4c_mlp_static_status_take(status);
    if (src != A4C_OK) return src;
    return *status != 0 ? A4C_ERR_DEVICE_TIMEOUT : A4C_OK;
}

int a4c_dense_i8(const void* A, int64_t lda, const int8_t* Wt, int64_t ldw, const int32_t* bias, void* Y,
                 int64_t ldy, int64_t M, int K, int N, int shift, int rounding, int relu, int out_dtype,
                 int a_unsigned, int algo, void* stream) {
    if (A == nullptr || Wt == nullptr || Y == nullptr) return A4C_ERR_INVALID_ARG;
    if (M < 0 || K <= 0 || N <= 0 || lda < K || ldw < K || ldy < N) return A4C_ERR_INVALID_ARG;
    if (shift < 0 || shift > 31 || !valid_round(rounding) || !valid_dtype(out_dtype)) return A4C_ERR_INVALID_ARG;
    cudaStream_t s = (cudaStream_t)stream;
    int use = algo;
    if (algo == A4C_ALGO_AUTO)
        use = a4c_dense_tc_supported(A, lda, Wt, ldw, Y, ldy, M, K, N, out_dtype) == A4C_OK ? A4C_ALGO_TCGEN05
                                                                                          : A4C_ALGO_SIMT;
    int rc;
    if (use == A4C_ALGO_TCGEN05) {
        int* word = status_word();
        if (word == nullptr) return A4C_ERR_CUDA;
        rc = a4c_launch_dense_tc(A, lda, Wt, ldw, bias, Y, ldy, M, K, N, shift, rounding, relu, out_dtype,
                                 a_unsigned, 0, word, s);
    } else if (use == A4C_ALGO_TCGEN05_PAIR) {
        int* word = status_word();
        if (word == nullptr) return A4C_ERR_CUDA;
        rc = a4c_launch_dense_tc2(A, lda, Wt, ldw, bias, Y, ldy, M, K, N, shift, rounding, relu, out_dtype, a_unsigned,
                                  word, s);
    } else if (use == A4C_ALGO_SIMT) {
        rc = a4c_launch_gemm_simt(A, lda, 1, 0, Wt, 1, ldw, 0, bias, Y, ldy, 0, 1, M, K, N, shift, rounding, relu,
                                  out_dtype, a_unsigned, s);
    } else {
        return A4C_ERR_INVALID_ARG;
    }
    if (rc != A4C_OK) { if (rc == A4C_ERR_CUDA) note(cudaGetLastError()); return rc; }
    return finish();
}

int a4c_bmm_i8(const void* A, int64_t lda, int64_t stride_a, const int8_t* B, int64_t ldb, int64_t stride_b,
               void* C, int64_t ldc, int64_t stride_c, int64_t batch, int M, int K, int N, int trans_a,
               int trans_b, int shift, int rounding, int out_dtype, int a_unsigned, void* stream) {
    if (A == nullptr || B == nullptr || C == nullptr) return A4C_ERR_INVALID_ARG;
    if (batch < 0 || M <= 0 || K <= 0 || N <= 0 || ldc < N) return A4C_ERR_INVALID_ARG;
    if (lda < (trans_a ? M : K) || ldb < (trans_b ? K : N)) return A4C_ERR_INVALID_ARG;
    if (shift < 0 || shift > 31 || !valid_round(rounding) || !valid_dtype(out_dtype)) return A4C_ERR_INVALID_ARG;
    if (g_bmm_path == 0 && a4c_bmm_tc_supported(A, lda, stride_a, B, ldb, stride_b, C, ldc, stride_c, batch, M, K, N,
                                                trans_a, trans_b, out_dtype) == A4C_OK) {
        int* word = status_word();
        if (word == nullptr) return A4C_ERR_CUDA;
        const int trc = a4c_launch_bmm_tc(A, lda, stride_a, B, ldb, stride_b, C, ldc, stride_c, batch, M, K, N, trans_a,
                                          trans_b, shift, rounding, out_dtype, a_unsigned, word, (cudaStream_t)stream);
        if (trc != A4C_OK) { if (trc == A4C_ERR_CUDA) note(cudaGetLastError()); return trc; }
        return finish();
    }
    // A(m,k): row stride lda / column stride 1, swapped when the stored operand is transposed
    const long long a_rs = trans_a ? 1 : lda, a_cs = trans_a ? lda : 1;
    // B(k,n): stored [K,N] -> k stride ldb, n stride 1; stored [N,K] -> k stride 1, n stride ldb
    const long long b_ks = trans_b ? 1 : ldb, b_ns = trans_b ? ldb : 1;
    const int rc = a4c_launch_gemm_simt(A, a_rs, a_cs, stride_a, B, b_ks, b_ns, stride_b, nullptr, C, ldc, stride_c,
                                        batch, M, K, N, shift, rounding, 0, out_dtype, a_unsigned,
                                        (cudaStream_t)stream);
    if (rc != A4C_OK) return rc;
    return finish();
}

int a4c_dense_i16(const int16_t* A, int64_t lda, const void* Wt, int w_dtype, int64_t ldw, const int32_t* bias,
                  void* Y, int64_t ldy, int64_t M, int K, int N, int shift, int rounding, int relu, int out_dtype,
                  void* stream) {
    if (A == nullptr || Wt == nullptr || Y == nullptr) return A4C_ERR_INVALID_ARG;
    if (M < 0 || K <= 0 || N <= 0 || lda < K || ldw < K || ldy < N) return A4C_ERR_INVALID_ARG;
    if ((w_dtype != A4C_I8 && w_dtype != A4C_I16) || !valid_round(rounding) || !valid_dtype(out_dtype))
        return A4C_ERR_INVALID_ARG;
    const int wide = w_dtype == A4C_I16;
    if (shift < 0 || shift > (wide ? 62 : 31)) return A4C_ERR_INVALID_ARG;
    // int16 x int8 whose pitches meet the TMA rules: the tensor cores, one digit of the activation at a time
    if (!wide && g_wide_path == 0 && a4c_dense_tc16_supported(A, lda, Wt, ldw, Y, ldy, M, K, N, out_dtype) == A4C_OK) {
        int* word = status_word();
        if (word == nullptr) return A4C_ERR_CUDA;
        const int trc = a4c_launch_dense_tc16(A, lda, (const int8_t*)Wt, ldw, bias, Y, ldy, M, K, N, shift, rounding, relu,
                                              out_dtype, word, (cudaStream_t)stream);
        if (trc != A4C_OK) { if (trc == A4C_ERR_CUDA) note(cudaGetLastError()); return trc; }
        return finish();
    }
    // W^T [N, ldw]: k stride 1, n stride ldw.  int16 x int8 accumulates in 32 bits, int16 x int16 in 64.
    const int rc = a4c_launch_gemm_wide(A, 2, lda, 1, 0, Wt, wide ? 2 : 1, 1, ldw, 0, bias, Y, ldy, 0, 1, M, K, N, shift,
                                        rounding, relu, out_dtype, wide ? 64 : 32, (cudaStream_t)stream);
    if (rc != A4C_OK) { if (rc == A4C_ERR_CUDA) note(cudaGetLastError()); return rc; }
    return finish();
}

int a4c_dense_ta(const void* A, int a_dtype, int64_t lda, int64_t stride_a, const void* Wt, int w_dtype, int64_t ldw,
                 const int32_t* bias, void* Y, int64_t ldy, int64_t stride_y, int64_t batch, int M, int K, int N,
                 int shift, int rounding, int relu, int out_dtype, void* stream) {
    if (A == nullptr || Wt == nullptr || Y == nullptr) return A4C_ERR_INVALID_ARG;
    if (batch < 0 || M <= 0 || K <= 0 || N <= 0 || lda < M || ldw < K || ldy < N) return A4C_ERR_INVALID_ARG;
    if (!valid_round(rounding) || !valid_dtype(out_dtype) || shift < 0) return A4C_ERR_INVALID_ARG;
    const bool a16 = a_dtype == A4C_I16, w16 = w_dtype == A4C_I16;
    if (!(a_dtype == A4C_I8 || a_dtype == A4C_U8 || a16) || !(w_dtype == A4C_I8 || w16) || (w16 && !a16))
        return A4C_ERR_INVALID_ARG;
    if (shift > (w16 ? 62 : 31)) return A4C_ERR_INVALID_ARG;
    int rc;
    // 8-bit operands whose pitches and pointers meet the TMA rules: the tensor-core kernel with an MN-major A operand
    if (!a16 && !w16 && g_bmm_path == 0 &&
        a4c_dense_ta_tc_supported(A, lda, stride_a, Wt, ldw, Y, ldy, stride_y, batch, M, K, N, out_dtype) == A4C_OK) {
        int* word = status_word();
        if (word == nullptr) return A4C_ERR_CUDA;
        rc = a4c_launch_dense_ta_tc(A, lda, stride_a, Wt, ldw, bias, Y, ldy, stride_y, batch, M, K, N, shift, rounding, relu,
                                    out_dtype, a_dtype == A4C_U8, word, (cudaStream_t)stream);
        if (rc != A4C_OK) { if (rc == A4C_ERR_CUDA) note(cudaGetLastError()); return rc; }
        return finish();
    }
    // stored [K, M]: the row (m) stride is 1 element, the k stride is the pitch
    if (a16)
        rc = a4c_launch_gemm_wide(A, 2, 1, lda, stride_a, Wt, w16 ? 2 : 1, 1, ldw, 0, bias, Y, ldy, stride_y, batch, M, K, N,
                                  shift, rounding, relu, out_dtype, w16 ? 64 : 32, (cudaStream_t)stream);
    else
        rc = a4c_launch_gemm_simt(A, 1, lda, stride_a, Wt, 1, ldw, 0, bias, Y, ldy, stride_y, batch, M, K, N, shift,
                                  rounding, relu, out_dtype, a_dtype == A4C_U8, (cudaStream_t)stream);
    if (rc != A4C_OK) { if (rc == A4C_ERR_CUDA) note(cudaGetLastError()); return rc; }
    return finish();
}

int a4c_bmm_i16(const int16_t* A, int64_t lda, int64_t stride_a, const void* B, int b_dtype, int64_t ldb,
                int64_t stride_b, void* C, int64_t ldc, int64_t stride_c, int64_t batch, int M, int K, int N,
                int trans_a, int trans_b, int shift, int rounding, int out_dtype, void* stream) {
    if (A == nullptr || B == nullptr || C == nullptr) return A4C_ERR_INVALID_ARG;
    if (batch < 0 || M <= 0 || K <= 0 || N <= 0 || ldc < N) return A4C_ERR_INVALID_ARG;
    if (lda < (trans_a ? M : K) || ldb < (trans_b ? K : N)) return A4C_ERR_INVALID_ARG;
    if ((b_dtype != A4C_I8 && b_dtype != A4C_I16) || !valid_round(rounding) || !valid_dtype(out_dtype))
        return A4C_ERR_INVALID_ARG;
    const int wide = b_dtype == A4C_I16;
    const long long a_rs = trans_a ? 1 : lda, a_cs = trans_a ? lda : 1;
    const long long b_ks = trans_b ? 1 : ldb, b_ns = trans_b ? ldb : 1;
    const int rc = a4c_launch_gemm_wide(A, 2, a_rs, a_cs, stride_a, B, wide ? 2 : 1, b_ks, b_ns, stride_b, nullptr, C, ldc,
                                        stride_c, batch, M, K, N, shift, rounding, 0, out_dtype, wide ? 64 : 32,
                                        (cudaStream_t)stream);
    if (rc != A4C_OK) { if (rc == A4C_ERR_CUDA) note(cudaGetLastError()); return rc; }
    return finish();
}

int a4c_dense_f(const void* A, int fdtype, int64_t lda, const void* Wt, int64_t ldw, const float* bias, void* Y,
                int64_t ldy, int64_t M, int K, int N, int relu, void* stream) {
    if (A == nullptr || Wt == nullptr || Y == nullptr) return A4C_ERR_INVALID_ARG;
    if (M < 0 || K <= 0 || N <= 0 || lda < K || ldw < K || ldy < N || (fdtype < 0 || fdtype > 2)) return A4C_ERR_INVALID_ARG;
    if (g_float_path == 0 && a4c_dense_tcf_supported(A, lda, Wt, ldw, Y, ldy, M, K, N, fdtype) == A4C_OK) {
        int* word = status_word();
        if (word == nullptr) return A4C_ERR_CUDA;
        const int trc = a4c_launch_dense_tcf(A, lda, Wt, ldw, bias, Y, ldy, M, K, N, relu, fdtype, word, (cudaStream_t)stream);
        if (trc != A4C_OK) { if (trc == A4C_ERR_CUDA) note(cudaGetLastError()); return trc; }
        return finish();
    }
    const int rc = a4c_launch_gemm_float(A, lda, 1, 0, Wt, 1, ldw, 0, bias, Y, ldy, 0, 1, M, K, N, relu, fdtype,
                                         (cudaStream_t)stream);
    if (rc != A4C_OK) { if (rc == A4C_ERR_CUDA) note(cudaGetLastError()); return rc; }
    return finish();
}

int a4c_bmm_f(const void* A, int fdtype, int64_t lda, int64_t stride_a, const void* B, int64_t ldb, int64_t stride_b,
              void* C, int64_t ldc, int64_t stride_c, int64_t batch, int M, int K, int N, int trans_a, int trans_b,
              void* stream) {
    if (A == nullptr || B == nullptr || C == nullptr) return A4C_ERR_INVALID_ARG;
    if (batch < 0 || M <= 0 || K <= 0 || N <= 0 || ldc < N || (fdtype < 0 || fdtype > 2)) return A4C_ERR_INVALID_ARG;
    if (lda < (trans_a ? M : K) || ldb < (trans_b ? K : N)) return A4C_ERR_INVALID_ARG;
    const long long a_rs = trans_a ? 1 : lda, a_cs = trans_a ? lda : 1;
    const long long b_ks = trans_b ? 1 : ldb, b_ns = trans_b ? ldb : 1;
    const int rc = a4c_launch_gemm_float(A, a_rs, a_cs, stride_a, B, b_ks, b_ns, stride_b, nullptr, C, ldc, stride_c, batch,
                                         M, K, N, 0, fdtype, (cudaStream_t)stream);
    if (rc != A4C_OK) { if (rc == A4C_ERR_CUDA) note(cudaGetLastError()); return rc; }
    return finish();
}

int a4c_add_f(const void* a, int64_t lda, const void* b, int64_t ldb, void* out, int64_t ldo, int64_t rows, int64_t cols,
              int fdtype, void* stream) {
    if (a == nullptr || b == nullptr || out == nullptr || rows < 0 || cols < 0 || (fdtype < 0 || fdtype > 2))
        return A4C_ERR_INVALID_ARG;
    if (lda < cols || ldb < cols || ldo < cols) return A4C_ERR_INVALID_ARG;
    const int rc = a4c_launch_add_float(a, lda, b, ldb, out, ldo, rows, cols, fdtype, (cudaStream_t)stream);
    if (rc != A4C_OK) { if (rc == A4C_ERR_CUDA) note(cudaGetLastError()); return rc; }
    return finish();
}

int a4c_attention_heads_i8_supported(const int8_t* q, int64_t ldq, int64_t stride_q, int64_t hstride_q, const int8_t* k,
                                     int64_t ldk, int64_t stride_k, int64_t hstride_k, const int8_t* v, int64_t ldv,
                                     int64_t stride_v, int64_t hstride_v, const int8_t* out, int64_t ldo, int64_t stride_o,
                                     int64_t hstride_o, int64_t batch, int heads, int sq, int sk, int dh, int qk_shift,
                                     int pv_shift, int sm_mode, int B, int S, int Dmax, int inv_shift) {
    if (q == nullptr || k == nullptr || v == nullptr || out == nullptr) return A4C_ERR_INVALID_ARG;
    return a4c_attention_tc_supported(q, ldq, stride_q, k, ldk, stride_k, v, ldv, stride_v, out, ldo, stride_o, batch,
                                      sq, sk, dh, qk_shift, pv_shift, sm_mode, B, S, Dmax, inv_shift, heads, hstride_q,
                                      hstride_k, hstride_v, hstride_o);
}

int a4c_attention_heads_i8(const int8_t* q, int64_t ldq, int64_t stride_q, int64_t hstride_q, const int8_t* k, int64_t ldk,
                           int64_t stride_k, int64_t hstride_k, const int8_t* v, int64_t ldv, int64_t stride_v,
                           int64_t hstride_v, int8_t* out, int64_t ldo, int64_t stride_o, int64_t hstride_o, int64_t batch,
                           int heads, int sq, int sk, int dh, int qk_shift, int pv_shift, int rounding, int sm_mode, int B,
                           int S, int Dmax, int inv_shift, int use_clb, int exp_kq, void* stream) {
    if (q == nullptr || k == nullptr || v == nullptr || out == nullptr) return A4C_ERR_INVALID_ARG;
    if (!valid_round(rounding)) return A4C_ERR_INVALID_ARG;
    int* word = status_word();
    if (word == nullptr) return A4C_ERR_CUDA;
    const int rc = a4c_launch_attention_tc(q, ldq, stride_q, k, ldk, stride_k, v, ldv, stride_v, out, ldo, stride_o,
                                           batch, sq, sk, dh, qk_shift, pv_shift, rounding, sm_mode, B, S, Dmax,
                                           inv_shift, use_clb, exp_kq, heads, hstride_q, hstride_k, hstride_v, hstride_o,
                                           word, (cudaStream_t)stream);
    if (rc != A4C_OK) { if (rc == A4C_ERR_CUDA) note(cudaGetLastError()); return rc; }
    return finish();
}

int a4c_attention_i8_supported(const int8_t* q, int64_t ldq, int64_t stride_q, const int8_t* k, int64_t ldk,
                               int64_t stride_k, const int8_t* v, int64_t ldv, int64_t stride_v, const int8_t* out,
                               int64_t ldo, int64_t stride_o, int64_t batch, int sq, int sk, int dh, int qk_shift,
                               int pv_shift, int sm_mode, int B, int S, int Dmax, int inv_shift) {
    return a4c_attention_heads_i8_supported(q, ldq, stride_q, 0, k, ldk, stride_k, 0, v, ldv, stride_v, 0, out, ldo,
                                            stride_o, 0, batch, 1, sq, sk, dh, qk_shift, pv_shift, sm_mode, B, S, Dmax,
                                            inv_shift);
}

int a4c_attention_i8(const int8_t* q, int64_t ldq, int64_t stride_q, const int8_t* k, int64_t ldk, int64_t stride_k,
                     const int8_t* v, int64_t ldv, int64_t stride_v, int8_t* out, int64_t ldo, int64_t stride_o,
                     int64_t batch, int sq, int sk, int dh, int qk_shift, int pv_shift, int rounding, int sm_mode, int B,
                     int S, int Dmax, int inv_shift, int use_clb, int exp_kq, void* stream) {
    return a4c_attention_heads_i8(q, ldq, stride_q, 0, k, ldk, stride_k, 0, v, ldv, stride_v, 0, out, ldo, stride_o, 0,
                                  batch, 1, sq, sk, dh, qk_shift, pv_shift, rounding, sm_mode, B, S, Dmax, inv_shift,
                                  use_clb, exp_kq, stream);
}

int a4c_set_option(int option, int value) {
    if (option == A4C_OPT_ROWOP_PATH && (value == 0 || value == 1)) {
        g_rowop_path = value;
        return A4C_OK;
    }
    if (option == A4C_OPT_BMM_PATH && (value == 0 || value == 1)) {
        g_bmm_path = value;
        return A4C_OK;
    }
    if (option == A4C_OPT_DENSE_PANEL_MIB && value >= 0 && value <= 1024) {
        a4c_dense_tc_set_panel_mib(value);
        return A4C_OK;
    }
    if (option == A4C_OPT_WIDE_DENSE_PATH && (value == 0 || value == 1)) {
        g_wide_path = value;
        return A4C_OK;
    }
    if (option == A4C_OPT_DENSE_LN_PATH && (value == 0 || value == 1)) {
        a4c_dense_ln_set_enabled(value == 0);
        return A4C_OK;
    }
    if (option == A4C_OPT_FLOAT_DENSE_PATH && (value == 0 || value == 1)) {
        g_float_path = value;
        return A4C_OK;
    }
    if (option == A4C_OPT_DENSE_RESIDENT_W && value >= 0 && value <= 2) {
        a4c_dense_tc_set_resident_w(value);
        return A4C_OK;
    }
    if (option == A4C_OPT_MLP_PATH && value >= 0 && value <= 2) {
        a4c_mlp_set_path(value);
        return A4C_OK;
    }
    if (option == A4C_OPT_ROWOP_CHUNKS_PER_LANE && (value == 0 || value == 1 || value == 2 || value == 4)) {
        a4c_rowops_fast_tuning(value, -1);
        return A4C_OK;
    }
    if (option == A4C_OPT_ROWOP_MIN_STAGES && (value == 0 || (value >= 2 && value <= 4))) {
        a4c_rowops_fast_tuning(-1, value);
        return A4C_OK;
    }
    if (option == A4C_OPT_ROWOP_CONTIG_COPY && (value == 0 || value == 1)) {
        a4c_rowops_fast_contig(value);
        return A4C_OK;
    }
    return A4C_ERR_INVALID_ARG;
}

static int layernorm_any(const int8_t* x, int64_t ldx, const int16_t* gamma, const int16_t* beta,
                         const int8_t* addend, int64_t ldadd, int pre_add, int8_t* out, int64_t ldo, int64_t rows,
                         int cols, int eps_q0, int out_shift, int rounding, int gamma_absmax, void* stream) {
    if (x == nullptr || gamma == nullptr || beta == nullptr || out == nullptr) return A4C_ERR_INVALID_ARG;
    if (ldx < cols || ldo < cols || (addend && ldadd < cols)) return A4C_ERR_INVALID_ARG;
    if (g_rowop_path == 0 && rows > 0 && cols >= 16 && (cols & (cols - 1)) == 0 && out_shift >= 0 && out_shift <= 15 &&
        eps_q0 >= 1 && valid_round(rounding) && cols % 16 == 0 && ldx % 16 == 0 && ldo % 16 == 0 &&
        (((uintptr_t)x | (uintptr_t)out | (uintptr_t)gamma | (uintptr_t)beta) & 15u) == 0 &&
        (!addend || (ldadd % 16 == 0 && ((uintptr_t)addend & 15u) == 0))) {
        const int frc = a4c_launch_layernorm_fast(x, ldx, gamma, beta, addend, ldadd, pre_add, out, ldo, rows, cols,
                                                  eps_q0, out_shift, rounding, gamma_absmax, status_word(),
                                                  (cudaStream_t)stream);
        if (frc == A4C_OK) return finish();
        if (frc != A4C_ERR_UNSUPPORTED) return frc;
    }
    const int rc = a4c_launch_layernorm(x, ldx, gamma, beta, addend, ldadd, pre_add, out, ldo, rows, cols, eps_q0,
                                        out_shift, rounding, (cudaStream_t)stream);
    if (rc != A4C_OK) return rc;
    return finish();
}

int a4c_layernorm_i8(const int8_t* x, int64_t ldx, const int16_t* gamma, const int16_t* beta,
                     const int8_t* addend, int64_t ldadd, int8_t* out, int64_t ldo, int64_t rows, int cols,
                     int eps_q0, int out_shift, int rounding, int gamma_absmax, void* stream) {
    return layernorm_any(x, ldx, gamma, beta, addend, ldadd, 0, out, ldo, rows, cols, eps_q0, out_shift, rounding,
                         gamma_absmax, stream);
}

int a4c_add_layernorm_i8(const int8_t* x, int64_t ldx, const int8_t* residual, int64_t ldr, const int16_t* gamma,
                         const int16_t* beta, int8_t* out, int64_t ldo, int64_t rows, int cols, int eps_q0,
                         int out_shift, int rounding, int gamma_absmax, void* stream) {
    if (residual == nullptr) return A4C_ERR_INVALID_ARG;
    return layernorm_any(x, ldx, gamma, beta, residual, ldr, 1, out, ldo, rows, cols, eps_q0, out_shift, rounding,
                         gamma_absmax, stream);
}

int a4c_dense_add_layernorm_supported(int64_t M, int K, int N, int64_t lda, int64_t ldw, int64_t ldr, int64_t ldo, int shift,
                                      int rounding, int out_shift, int eps_q0, int gamma_absmax) {
    return a4c_dense_ln_supported(M, K, N, lda, ldw, ldr, ldo, shift, rounding, out_shift, eps_q0, gamma_absmax);
}

int a4c_dense_add_layernorm_i8(const void* A, int64_t lda, int a_unsigned, const int8_t* Wt, int64_t ldw,
                               const int32_t* bias, int shift, int relu, const int8_t* residual, int64_t ldr,
                               const int16_t* gamma, const int16_t* beta, int8_t* out, int64_t ldo, int64_t M, int K,
                               int N, int eps_q0, int out_shift, int rounding, int gamma_absmax, void* stream) {
    if (A == nullptr || Wt == nullptr || residual == nullptr || gamma == nullptr || beta == nullptr || out == nullptr)
        return A4C_ERR_INVALID_ARG;
    if (M < 0 || K <= 0 || N <= 0 || !valid_round(rounding)) return A4C_ERR_INVALID_ARG;
    if (M == 0) return A4C_OK;
    int* status = status_word();
    if (status == nullptr) return A4C_ERR_CUDA;
    const int rc = a4c_launch_dense_ln(A, lda, a_unsigned, Wt, ldw, bias, shift, relu, residual, ldr, gamma, beta, out, ldo, M,
                                       K, N, eps_q0, out_shift, rounding, gamma_absmax, status, (cudaStream_t)stream);
    if (rc != A4C_OK) return rc;
    return finish();
}

int a4c_softmax_i8(const int8_t* x, int64_t ldx, const void* addend, int64_t ldadd, void* out, int64_t ldo,
                   int64_t rows, int cols, int mode, int B, int S, int Dmax, int inv_shift, int use_clb,
                   int exp_kq, int out_dtype, void* stream) {
    if (x == nullptr || out == nullptr) return A4C_ERR_INVALID_ARG;
    if (ldx < cols || ldo < cols || (addend && ldadd < cols)) return A4C_ERR_INVALID_ARG;
    if (g_rowop_path == 0 && rows > 0 && cols >= 16 && cols % 16 == 0 && (mode == 0 || mode == 1) && out_dtype == A4C_U8 &&
        inv_shift >= 1 && ldx % 16 == 0 && ldo % 16 == 0 && (((uintptr_t)x | (uintptr_t)out) & 15u) == 0 &&
        (!addend || (ldadd % 16 == 0 && ((uintptr_t)addend & 15u) == 0)) &&
        (mode == 1 ? (exp_kq >= 1 && exp_kq <= 128)
                   : (B >= 0 && B <= 32767 && S >= 0 && S <= 127 && Dmax >= 0 && Dmax <= 255))) {
        const int frc = a4c_launch_softmax_fast(x, ldx, addend, ldadd, out, ldo, rows, cols, mode, B, S, Dmax, inv_shift,
                                                use_clb, exp_kq, out_dtype, status_word(), (cudaStream_t)stream);
        if (frc == A4C_OK) return finish();
        if (frc != A4C_ERR_UNSUPPORTED) return frc;
    }
    const int rc = a4c_launch_softmax(x, ldx, addend, ldadd, out, ldo, rows, cols, mode, B, S, Dmax, inv_shift,
                                      use_clb, exp_kq, out_dtype, (cudaStream_t)stream);
    if (rc != A4C_OK) return rc;
    return finish();
}

int a4c_add_sat(const void* a, int64_t lda, const void* b, int64_t ldb, void* out, int64_t ldo, int64_t rows,
                int64_t cols, int shift, int rounding, int dtype, void* stream) {
    if (a == nullptr || b == nullptr || out == nullptr) return A4C_ERR_INVALID_ARG;
    if (lda < cols || ldb < cols || ldo < cols) return A4C_ERR_INVALID_ARG;
    const int rc = a4c_launch_add(a, lda, b, ldb, out, ldo, rows, cols, shift, rounding, dtype, (cudaStream_t)stream);
    if (rc != A4C_OK) return rc;
    return finish();
}

}  // extern "C"
