// Dense / batched MatMul for the 16-bit operand combinations of aie4ml: int16 x int8 (32-bit accumulator) and
// int16 x int16 (64-bit accumulator), the remaining entries of the reference's width table
// (op_impls/families/matmul/common.py:52: {(8,8), (16,8), (16,16)}; accumulator choice
// op_impls/utils/precision.py:116-127).  Arithmetic per output element as dense_single::run /
// matmul_single::run (dense_bias_relu.cpp:67-166, matmul.cpp:32-118): products accumulate on top of the int32
// bias in the accumulator type (wrapping at 32 bits for acc32, exact in 64 bits for acc64), SRS with the
// rounding token, saturation to the output type, ReLU after the saturation.
//
// These shapes are rare next to int8 (no tensor-core instruction takes 16-bit integers), so one generic tiled
// kernel serves them: 64 x 64 output tile per 256-thread block, 4 x 4 outputs per thread, operands staged in
// shared memory as sign-extended 32-bit values, any element strides (transposed views, batches).
#include "a4c_common.cuh"
#include "a4c_kernels.h"

namespace {

constexpr int TM = 64, TN = 64, TK = 16;

struct WideArgs {
    const void* A; long long a_rs, a_cs, a_bs;   // element strides: row, column, batch
    const void* B; long long b_ks, b_ns, b_bs;
    const int32_t* bias;
    void* C; long long ldc, c_bs;
    long long M; int K, N;
    int shift, rounding, relu, out_dtype;
    int a_bytes, b_bytes;   // 1 or 2
};

__device__ __forceinline__ int load_elem(const void* p, long long idx, int bytes) {
    return bytes == 2 ? (int)reinterpret_cast<const int16_t*>(p)[idx] : (int)reinterpret_cast<const int8_t*>(p)[idx];
}

template <bool ACC64>
__global__ void __launch_bounds__(256) gemm_wide_kernel(WideArgs g) {
    __shared__ int As[TK][TM + 1];
    __shared__ int Bs[TK][TN + 1];
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    const long long m0 = (long long)blockIdx.y * TM;
    const int n0 = blockIdx.x * TN;
    const long long b = blockIdx.z;
    const long long a_base = b * g.a_bs, b_base = b * g.b_bs;
    long long acc64[4][4];
    uint32_t acc32[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) { acc64[i][j] = 0; acc32[i][j] = 0u; }

    for (int k0 = 0; k0 < g.K; k0 += TK) {
        for (int i = threadIdx.x; i < TK * TM; i += 256) {
            const int kk = i / TM, mm = i - kk * TM;   // consecutive threads walk m: rows of A are strided anyway
            const long long m = m0 + mm;
            const int k = k0 + kk;
            As[kk][mm] = (m < g.M && k < g.K) ? load_elem(g.A, a_base + m * g.a_rs + (long long)k * g.a_cs, g.a_bytes) : 0;
        }
        for (int i = threadIdx.x; i < TK * TN; i += 256) {
            const int kk = i / TN, nn = i - kk * TN;
            const int n = n0 + nn, k = k0 + kk;
            Bs[kk][nn] = (n < g.N && k < g.K) ? load_elem(g.B, b_base + (long long)k * g.b_ks + (long long)n * g.b_ns, g.b_bytes) : 0;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < TK; ++kk) {
            int av[4], bv[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) { av[i] = As[kk][ty * 4 + i]; bv[i] = Bs[kk][tx * 4 + i]; }
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    if (ACC64) acc64[i][j] += (long long)av[i] * (long long)bv[j];
                    else acc32[i][j] += (uint32_t)(av[i] * bv[j]);   // two's-complement wrap, as a 32-bit accumulator
                }
        }
        __syncthreads();
    }

    int lo, hi;
    dtype_range(g.out_dtype, lo, hi);
    if (g.relu && lo < 0) lo = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const long long m = m0 + ty * 4 + i;
        if (m >= g.M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tx * 4 + j;
            if (n >= g.N) continue;
            const int bias = g.bias ? g.bias[n] : 0;
            long long v;
            if (ACC64) {
                v = round_shift_i64(acc64[i][j] + (long long)bias, g.shift, g.rounding);
            } else {
                const int x = (int)(acc32[i][j] + (uint32_t)bias);
                RoundParams rp = make_round_params(g.shift, g.rounding);
                v = round_shift_i32(x, rp);
            }
            const int y = (int)(v < lo ? lo : (v > hi ? hi : v));
            const long long off = b * g.c_bs + m * g.ldc + n;
            if (g.out_dtype == A4C_I16) reinterpret_cast<int16_t*>(g.C)[off] = (int16_t)y;
            else reinterpret_cast<uint8_t*>(g.C)[off] = (uint8_t)y;
        }
    }
}

}  // namespace

int a4c_launch_gemm_wide(const void* A, int a_bytes, long long a_rs, long long a_cs, long long a_bs, const void* B,
                         int b_bytes, long long b_ks, long long b_ns, long long b_bs, const int32_t* bias, void* C,
                         long long ldc, long long c_bs, long long batch, long long M, int K, int N, int shift,
                         int rounding, int relu, int out_dtype, int acc_bits, cudaStream_t stream) {
    if ((a_bytes != 1 && a_bytes != 2) || (b_bytes != 1 && b_bytes != 2) || (acc_bits != 32 && acc_bits != 64))
        return A4C_ERR_INVALID_ARG;
    if (shift < 0 || shift > (acc_bits == 32 ? 31 : 62)) return A4C_ERR_INVALID_ARG;
    if (M == 0 || batch == 0) return A4C_OK;
    const long long grid_y = (M + TM - 1) / TM;
    if (grid_y > 65535 || batch > 65535) return A4C_ERR_TOO_LARGE;
    WideArgs g;
    g.A = A; g.a_rs = a_rs; g.a_cs = a_cs; g.a_bs = a_bs; g.B = B; g.b_ks = b_ks; g.b_ns = b_ns; g.b_bs = b_bs;
    g.bias = bias; g.C = C; g.ldc = ldc; g.c_bs = c_bs; g.M = M; g.K = K; g.N = N;
    g.shift = shift; g.rounding = rounding; g.relu = relu; g.out_dtype = out_dtype; g.a_bytes = a_bytes; g.b_bytes = b_bytes;
    const dim3 grid((unsigned)((N + TN - 1) / TN), (unsigned)grid_y, (unsigned)batch);
    if (acc_bits == 64) gemm_wide_kernel<true><<<grid, 256, 0, stream>>>(g);
    else gemm_wide_kernel<false><<<grid, 256, 0, stream>>>(g);
    return cudaGetLastError() == cudaSuccess ? A4C_OK : A4C_ERR_CUDA;
}
