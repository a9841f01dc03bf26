// A chain of Dense layers behind one C-ABI call.  Each layer is a4c_dense_i8 (tcgen05 where its rules hold,
// dp4a otherwise); the int8 activations between layers live in scratch memory owned by the library.
#include <mutex>

#include "../../include/aie4ml_b200.h"
#include "a4c_common.cuh"

namespace {

constexpr int kMaxDevices = 64;
constexpr int kMaxLayers = 64;
std::mutex g_ws_mutex;
void* g_ws[kMaxDevices] = {nullptr};
size_t g_ws_bytes[kMaxDevices] = {0};

inline long long pitch16(long long n) { return (n + 15) / 16 * 16; }

// Validates the chain and returns the bytes ONE intermediate buffer needs (0 when there is a single layer).
int check_chain(const void* X, int64_t ldx, int n_layers, const int* dims, const int8_t* const* Wt, const int64_t* ldw,
                const int* shift, const int* relu, int rounding, const void* Y, int64_t ldy, int out_dtype, int64_t M,
                size_t* inter_bytes) {
    if (X == nullptr || Y == nullptr || dims == nullptr || Wt == nullptr || ldw == nullptr || shift == nullptr ||
        relu == nullptr)
        return A4C_ERR_INVALID_ARG;
    if (n_layers < 1 || n_layers > kMaxLayers || M < 0 || rounding < 0 || rounding >= A4C_RND_COUNT || out_dtype < 0 ||
        out_dtype > 2)
        return A4C_ERR_INVALID_ARG;
    long long widest = 0;
    for (int l = 0; l <= n_layers; ++l) {
        if (dims[l] <= 0) return A4C_ERR_INVALID_ARG;
        if (l > 0 && l < n_layers && dims[l] > widest) widest = dims[l];
    }
    for (int l = 0; l < n_layers; ++l)
        if (Wt[l] == nullptr || ldw[l] < dims[l] || shift[l] < 0 || shift[l] > 31) return A4C_ERR_INVALID_ARG;
    if (ldx < dims[0] || ldy < dims[n_layers]) return A4C_ERR_INVALID_ARG;
    *inter_bytes = (size_t)(M * pitch16(widest));
    return A4C_OK;
}

// Runs the layers with the two given intermediate buffers (each at least inter_bytes).
int run_chain(const void* X, int64_t ldx, int x_unsigned, int n_layers, const int* dims, const int8_t* const* Wt,
              const int64_t* ldw, const int32_t* const* bias, const int* shift, const int* relu, int rounding, void* Y,
              int64_t ldy, int out_dtype, int64_t M, void* buf0, void* buf1, void* stream) {
    const void* in = X;
    long long ld_in = ldx;
    int in_unsigned = x_unsigned;
    for (int l = 0; l < n_layers; ++l) {
        const bool last = l == n_layers - 1;
        void* out = last ? Y : ((l & 1) ? buf1 : buf0);
        const long long ld_out = last ? ldy : pitch16(dims[l + 1]);
        const int rc = a4c_dense_i8(in, ld_in, Wt[l], ldw[l], bias ? bias[l] : nullptr, out, ld_out, M, dims[l],
                                    dims[l + 1], shift[l], rounding, relu[l], last ? out_dtype : A4C_I8, in_unsigned,
                                    A4C_ALGO_AUTO, stream);
        if (rc != A4C_OK) return rc;
        in = out;
        ld_in = ld_out;
        in_unsigned = 0;
    }
    return A4C_OK;
}

}  // namespace

extern "C" int a4c_mlp_i8(const void* X, int64_t ldx, int x_unsigned, int n_layers, const int* dims,
                          const int8_t* const* Wt, const int64_t* ldw, const int32_t* const* bias, const int* shift,
                          const int* relu, int rounding, void* Y, int64_t ldy, int out_dtype, int64_t M, void* stream) {
    size_t inter = 0;
    const int chk = check_chain(X, ldx, n_layers, dims, Wt, ldw, shift, relu, rounding, Y, ldy, out_dtype, M, &inter);
    if (chk != A4C_OK) return chk;
    if (M == 0) return A4C_OK;
    void* buf0 = nullptr;
    void* buf1 = nullptr;
    if (n_layers > 1) {
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return A4C_ERR_CUDA;
        std::lock_guard<std::mutex> lock(g_ws_mutex);
        const size_t need = 2 * ((inter + 255) / 256 * 256);
        if (g_ws_bytes[dev] < need) {
            // grow: nothing of an earlier call may still be using the old buffer
            if (cudaDeviceSynchronize() != cudaSuccess) return A4C_ERR_CUDA;
            if (g_ws[dev]) cudaFree(g_ws[dev]);
            g_ws[dev] = nullptr;
            g_ws_bytes[dev] = 0;
            if (cudaMalloc(&g_ws[dev], need) != cudaSuccess) return A4C_ERR_CUDA;
            g_ws_bytes[dev] = need;
        }
        buf0 = g_ws[dev];
        buf1 = (char*)g_ws[dev] + need / 2;
    }
    return run_chain(X, ldx, x_unsigned, n_layers, dims, Wt, ldw, bias, shift, relu, rounding, Y, ldy, out_dtype, M,
                     buf0, buf1, stream);
}
