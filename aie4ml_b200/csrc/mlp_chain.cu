// A chain of Dense layers behind one C-ABI call.  Each layer is a4c_dense_i8 (tcgen05 where its rules hold,
// dp4a otherwise); the int8 activations between layers live in scratch memory owned by the library.
#include <mutex>

#include "../../include/aie4ml_b200.h"
#include "a4c_common.cuh"
#include "a4c_kernels.h"

namespace {

constexpr int kMaxDevices = 64;
constexpr int kMaxLayers = 64;
std::mutex g_ws_mutex;
void* g_ws[kMaxDevices] = {nullptr};
size_t g_ws_bytes[kMaxDevices] = {0};
int g_mlp_path = 0;   // 0 automatic, 1 layer by layer, 2 the fused narrow-chain kernel only

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

// The automatic choice between the single-kernel narrow chain and one launch per layer (given that the single
// kernel supports the chain).  Measured on B200: the single kernel wins while no layer is wider than 64 and the
// batch is at most 65536 rows (10 us against 19 us for 16-64-32-32-5 at 1024 rows); beyond either limit the
// tensor-core kernels, one launch per layer, are faster.
bool single_kernel_choice(int n_layers, const int* dims, int64_t M) {
    if (g_mlp_path == 2) return true;
    int widest = 0;
    for (int l = 0; l <= n_layers; ++l) widest = dims[l] > widest ? dims[l] : widest;
    return widest <= 64 && M <= 65536;
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
    // Narrow chains run as one kernel with the activations in shared memory.
    if (g_mlp_path != 1) {
        const bool can = a4c_mlp_small_supported(n_layers, dims, out_dtype) == A4C_OK;
        if (g_mlp_path == 2 && !can) return A4C_ERR_UNSUPPORTED;
        if (can && single_kernel_choice(n_layers, dims, M)) {
            static_assert(sizeof(long long) == sizeof(int64_t), "pitch type");
            const int rc = a4c_launch_mlp_small(X, ldx, x_unsigned, n_layers, dims, Wt, (const long long*)ldw, bias, shift,
                                                relu, rounding, Y, ldy, out_dtype, M, (cudaStream_t)stream);
            if (rc != A4C_OK) return rc;
            return cudaPeekAtLastError() == cudaSuccess ? A4C_OK : A4C_ERR_CUDA;
        }
    }
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

void a4c_mlp_set_path(int path) { g_mlp_path = path; }

extern "C" int a4c_mlp_i8_single_kernel(int n_layers, const int* dims, int out_dtype, int64_t M) {
    if (dims == nullptr || n_layers < 1 || n_layers > kMaxLayers || g_mlp_path == 1) return 0;
    for (int l = 0; l <= n_layers; ++l)
        if (dims[l] <= 0) return 0;
    return a4c_mlp_small_supported(n_layers, dims, out_dtype) == A4C_OK && single_kernel_choice(n_layers, dims, M) ? 1 : 0;
}

// ------------------------------------------------------------------------------------------------------
// The same chain for callers that must not allocate.
//
// Some hosts of this library cannot call cudaMalloc at the point where they run a model: a plug-in that
// executes inside another runtime's stream callback or captured region, a process whose device memory is
// handed out entirely by its own pool, or a latency-critical loop that forbids any call that can take the
// allocator's lock.  For them the scratch of the chain is a fixed array that is part of the library image:
// it exists on every GPU that loads the library, from load until exit, and nothing is ever allocated or freed.
//
// Layout of the array: bytes [0, 256) hold the status word that the tensor-core kernels report bounded-wait
// failures into (it must start at zero: it is cleared once at set-up and again whenever it is read back);
// then two activation buffers of A4C_MLP_STATIC_BYTES each.  The activation buffers need no clearing: every
// layer overwrites all bytes the next layer reads.
// ------------------------------------------------------------------------------------------------------
namespace {

constexpr size_t kStaticBuf = (size_t)A4C_MLP_STATIC_BYTES;
static __device__ __align__(256) unsigned char g_mlp_static_scratch[256 + 2 * kStaticBuf];

std::mutex g_static_mutex;
unsigned char* g_static_ptr[kMaxDevices] = {nullptr};

// The array's NAME is only a host-side handle; the device address comes from cudaGetSymbolAddress, asked once
// per device with that device current.
int static_scratch(cudaStream_t stream, unsigned char** out) {
    int dev = 0;
    if (!a4c_note_cuda(cudaGetDevice(&dev)) || dev < 0 || dev >= kMaxDevices) return A4C_ERR_CUDA;
    std::lock_guard<std::mutex> lock(g_static_mutex);
    if (g_static_ptr[dev] == nullptr) {
        unsigned char* p = nullptr;
        if (!a4c_note_cuda(cudaGetSymbolAddress((void**)&p, g_mlp_static_scratch)) || p == nullptr) return A4C_ERR_CUDA;
        if (!a4c_note_cuda(cudaMemsetAsync(p, 0, 256, stream))) return A4C_ERR_CUDA;
        g_static_ptr[dev] = p;
    }
    *out = g_static_ptr[dev];
    return A4C_OK;
}

// One Dense layer through the internal launchers (a4c_dense_i8 itself would allocate its status word).
int dense_no_alloc(const void* A, long long lda, const int8_t* Wt, long long ldw, const int32_t* bias, void* Y,
                   long long ldy, long long M, int K, int N, int shift, int rounding, int relu, int out_dtype,
                   int a_unsigned, int* status, cudaStream_t stream) {
    if (a4c_dense_tc_supported(A, lda, Wt, ldw, Y, ldy, M, K, N, out_dtype) == A4C_OK)
        return a4c_launch_dense_tc(A, lda, Wt, ldw, bias, Y, ldy, M, K, N, shift, rounding, relu, out_dtype, a_unsigned, 0,
                                   status, stream);
    return a4c_launch_gemm_simt(A, lda, 1, 0, Wt, 1, ldw, 0, bias, Y, ldy, 0, 1, M, K, N, shift, rounding, relu, out_dtype,
                                a_unsigned, stream);
}

}  // namespace

int a4c_mlp_static_status_take(int* out) {
    *out = 0;
    int dev = 0;
    if (!a4c_note_cuda(cudaGetDevice(&dev)) || dev < 0 || dev >= kMaxDevices) return A4C_ERR_CUDA;
    unsigned char* base;
    {
        std::lock_guard<std::mutex> lock(g_static_mutex);
        base = g_static_ptr[dev];
    }
    if (base == nullptr) return A4C_OK;   // never set up on this device: nothing can have reported into it
    if (!a4c_note_cuda(cudaMemcpy(out, base, sizeof(int), cudaMemcpyDeviceToHost))) return A4C_ERR_CUDA;
    if (*out != 0 && !a4c_note_cuda(cudaMemset(base, 0, sizeof(int)))) return A4C_ERR_CUDA;
    return A4C_OK;
}

extern "C" int a4c_mlp_i8_static(const void* X, int64_t ldx, int x_unsigned, int n_layers, const int* dims,
                                 const int8_t* const* Wt, const int64_t* ldw, const int32_t* const* bias,
                                 const int* shift, const int* relu, int rounding, void* Y, int64_t ldy, int out_dtype,
                                 int64_t M, int* status_out, void* stream) {
    size_t inter = 0;
    const int chk = check_chain(X, ldx, n_layers, dims, Wt, ldw, shift, relu, rounding, Y, ldy, out_dtype, M, &inter);
    if (chk != A4C_OK) return chk;
    if (n_layers > 1 && inter > kStaticBuf) return A4C_ERR_TOO_LARGE;  // M * pitch16(widest hidden layer) > 4 MiB
    cudaStream_t s = (cudaStream_t)stream;
    unsigned char* base = nullptr;
    const int rc0 = static_scratch(s, &base);
    if (rc0 != A4C_OK) return rc0;
    int* status = reinterpret_cast<int*>(base);
    void* buf[2] = {base + 256, base + 256 + kStaticBuf};
    if (M > 0) {
        const void* in = X;
        long long ld_in = ldx;
        int in_unsigned = x_unsigned;
        for (int l = 0; l < n_layers; ++l) {
            const bool last = l == n_layers - 1;
            void* out = last ? Y : buf[l & 1];
            const long long ld_out = last ? ldy : pitch16(dims[l + 1]);
            const int rc = dense_no_alloc(in, ld_in, Wt[l], ldw[l], bias ? bias[l] : nullptr, out, ld_out, M, dims[l],
                                          dims[l + 1], shift[l], rounding, relu[l], last ? out_dtype : A4C_I8, in_unsigned,
                                          status, s);
            if (rc != A4C_OK) {
                if (rc == A4C_ERR_CUDA) a4c_note_cuda(cudaGetLastError());
                return rc;
            }
            in = out;
            ld_in = ld_out;
            in_unsigned = 0;
        }
        if (!a4c_note_cuda(cudaPeekAtLastError())) return A4C_ERR_CUDA;
    }
    if (status_out != nullptr) {
        if (!a4c_note_cuda(cudaMemcpyAsync(status_out, status, sizeof(int), cudaMemcpyDeviceToHost, s))) return A4C_ERR_CUDA;
        if (!a4c_note_cuda(cudaStreamSynchronize(s))) return A4C_ERR_CUDA;
        if (*status_out != 0) {
            cudaMemsetAsync(status, 0, sizeof(int), s);
            return A4C_ERR_DEVICE_TIMEOUT;
        }
    }
    return A4C_OK;
}
