// Floating-point Dense / batched MatMul / Add: the float-simulation path of aie4ml (AIEConfig.ComputeDtype =
// bfloat16 | float32, passes/force_float_mode.py:22-46) and its fp8_e4m3 tensors (ONNX FLOAT8E4M3FN,
// frontends/onnx/context.py:19-24; op_impls/families/matmul/common.py:39).  Operands are stored in the compute type
// (bfloat16 as its 16 bits, fp8 E4M3 finite-only as its 8), products are accumulated in float32 on top of the
// float32 bias, ReLU follows, and the result is rounded to nearest-even into the storage type (fp8: values beyond
// +-448 saturate to it).  The reference checks this path against a float model with
// rtol 1e-2 / atol 5e-2 (bfloat16) and 1e-3 / 1e-3 (float32) (tests/test_float_sim.py:87-93): the order of the
// float32 additions is not part of its contract.
//
// One generic tiled kernel (64 x 64 outputs per 256-thread block, 4 x 4 per thread, any element strides); this
// path exists for checking a model against its float original, not for throughput.
#include <cuda_bf16.h>
#include <cuda_fp8.h>

#include "a4c_common.cuh"
#include "a4c_kernels.h"

namespace {

constexpr int TM = 64, TN = 64, TK = 16;

struct FloatGemmArgs {
    const void* A; long long a_rs, a_cs, a_bs;
    const void* B; long long b_ks, b_ns, b_bs;
    const float* bias;
    void* C; long long ldc, c_bs;
    long long M; int K, N;
    int relu;
};

// storage kinds (the fdtype argument of the entry points)
constexpr int KIND_BF16 = 0, KIND_F32 = 1, KIND_FP8 = 2;

template <int KIND>
__device__ __forceinline__ float load_f(const void* p, long long idx) {
    if (KIND == KIND_BF16) return __uint_as_float((uint32_t)reinterpret_cast<const uint16_t*>(p)[idx] << 16);
    if (KIND == KIND_FP8) {
        const __half_raw h = __nv_cvt_fp8_to_halfraw(reinterpret_cast<const __nv_fp8_storage_t*>(p)[idx], __NV_E4M3);
        return __half2float(__half(h));
    }
    return reinterpret_cast<const float*>(p)[idx];
}
template <int KIND>
__device__ __forceinline__ void store_f(void* p, long long idx, float v) {
    if (KIND == KIND_BF16) reinterpret_cast<__nv_bfloat16*>(p)[idx] = __float2bfloat16_rn(v);
    else if (KIND == KIND_FP8) reinterpret_cast<__nv_fp8_storage_t*>(p)[idx] = __nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E4M3);
    else reinterpret_cast<float*>(p)[idx] = v;
}

template <int KIND>
__global__ void __launch_bounds__(256) gemm_float_kernel(FloatGemmArgs g) {
    __shared__ float As[TK][TM + 1];
    __shared__ float Bs[TK][TN + 1];
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    const long long m0 = (long long)blockIdx.y * TM;
    const int n0 = blockIdx.x * TN;
    const long long b = blockIdx.z;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.0f;
    for (int k0 = 0; k0 < g.K; k0 += TK) {
        for (int i = threadIdx.x; i < TK * TM; i += 256) {
            const int kk = i / TM, mm = i - kk * TM;
            const long long m = m0 + mm;
            const int k = k0 + kk;
            As[kk][mm] = (m < g.M && k < g.K) ? load_f<KIND>(g.A, b * g.a_bs + m * g.a_rs + (long long)k * g.a_cs) : 0.0f;
        }
        for (int i = threadIdx.x; i < TK * TN; i += 256) {
            const int kk = i / TN, nn = i - kk * TN;
            const int n = n0 + nn, k = k0 + kk;
            Bs[kk][nn] = (n < g.N && k < g.K) ? load_f<KIND>(g.B, b * g.b_bs + (long long)k * g.b_ks + (long long)n * g.b_ns) : 0.0f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < TK; ++kk) {
            float av[4], bv[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) { av[i] = As[kk][ty * 4 + i]; bv[i] = Bs[kk][tx * 4 + i]; }
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const long long m = m0 + ty * 4 + i;
        if (m >= g.M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tx * 4 + j;
            if (n >= g.N) continue;
            float v = acc[i][j] + (g.bias ? g.bias[n] : 0.0f);
            if (g.relu) v = fmaxf(v, 0.0f);
            store_f<KIND>(g.C, b * g.c_bs + m * g.ldc + n, v);
        }
    }
}

template <int KIND>
__global__ void __launch_bounds__(256) add_float_kernel(const void* a, long long lda, const void* b, long long ldb, void* out,
                                                        long long ldo, long long rows, long long cols) {
    const long long total = rows * cols;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const long long r = i / cols, c = i - r * cols;
        store_f<KIND>(out, r * ldo + c, load_f<KIND>(a, r * lda + c) + load_f<KIND>(b, r * ldb + c));
    }
}

}  // namespace

int a4c_launch_gemm_float(const void* A, long long a_rs, long long a_cs, long long a_bs, const void* B, long long b_ks,
                          long long b_ns, long long b_bs, const float* bias, void* C, long long ldc, long long c_bs,
                          long long batch, long long M, int K, int N, int relu, int kind, cudaStream_t stream) {
    if (M == 0 || batch == 0) return A4C_OK;
    const long long grid_y = (M + TM - 1) / TM;
    if (grid_y > 65535 || batch > 65535) return A4C_ERR_TOO_LARGE;
    FloatGemmArgs g;
    g.A = A; g.a_rs = a_rs; g.a_cs = a_cs; g.a_bs = a_bs; g.B = B; g.b_ks = b_ks; g.b_ns = b_ns; g.b_bs = b_bs;
    g.bias = bias; g.C = C; g.ldc = ldc; g.c_bs = c_bs; g.M = M; g.K = K; g.N = N; g.relu = relu;
    const dim3 grid((unsigned)((N + TN - 1) / TN), (unsigned)grid_y, (unsigned)batch);
    if (kind == KIND_BF16) gemm_float_kernel<KIND_BF16><<<grid, 256, 0, stream>>>(g);
    else if (kind == KIND_FP8) gemm_float_kernel<KIND_FP8><<<grid, 256, 0, stream>>>(g);
    else gemm_float_kernel<KIND_F32><<<grid, 256, 0, stream>>>(g);
    return cudaGetLastError() == cudaSuccess ? A4C_OK : A4C_ERR_CUDA;
}

int a4c_launch_add_float(const void* a, long long lda, const void* b, long long ldb, void* out, long long ldo,
                         long long rows, long long cols, int kind, cudaStream_t stream) {
    if (rows == 0 || cols == 0) return A4C_OK;
    const long long total = rows * cols;
    long long blocks = (total + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    if (kind == KIND_BF16) add_float_kernel<KIND_BF16><<<(unsigned)blocks, 256, 0, stream>>>(a, lda, b, ldb, out, ldo, rows, cols);
    else if (kind == KIND_FP8) add_float_kernel<KIND_FP8><<<(unsigned)blocks, 256, 0, stream>>>(a, lda, b, ldb, out, ldo, rows, cols);
    else add_float_kernel<KIND_F32><<<(unsigned)blocks, 256, 0, stream>>>(a, lda, b, ldb, out, ldo, rows, cols);
    return cudaGetLastError() == cudaSuccess ? A4C_OK : A4C_ERR_CUDA;
}
