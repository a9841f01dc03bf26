// Generic int8 GEMM on the integer dot-product units (dp4a).  It takes arbitrary element strides
// for both operands, so it serves every shape the tensor-core kernels do not: K or N that break
// TMA's 16-byte rules (e.g. N = 5 or 10), transposed / strided views, tiny problems.
//
// Arithmetic contract (aie4ml dense_bias_relu.cpp:67-166 and matmul.cpp:32-118):
//   C = clamp(round_shift(A.B + bias, shift), lo, hi), ReLU folded into lo = max(lo, 0)
// (ReLU after saturation == clamping at max(lo, 0) because saturation is monotonic).
#include "a4c_common.cuh"
#include "a4c_kernels.h"

namespace {

constexpr int TM = 64, TN = 64, TK = 32;  // block tile; TK bytes of K per step
constexpr int PITCH_W = TK / 4 + 1;       // smem row pitch in 32-bit words (+1: bank spread)

template <bool A_UNSIGNED>
__device__ __forceinline__ int dot4(uint32_t a, uint32_t b, int c) {
    int d;
    if (A_UNSIGNED)
        asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    else
        asm("dp4a.s32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}

struct SimtArgs {
    const uint8_t* A; long long a_rs, a_cs, a_bs;  // A(m,k) = A[b*a_bs + m*a_rs + k*a_cs]
    const uint8_t* B; long long b_ks, b_ns, b_bs;  // B(k,n) = B[b*b_bs + k*b_ks + n*b_ns]
    const int32_t* bias;
    uint8_t* C; long long ldc, c_bs;               // element pitch / batch stride of C
    long long M; int N, K; long long batch;
    RoundParams rp; int lo, hi, out_dtype;
};

// Fill one smem tile [ROWS][TK] (K contiguous, zero padded) from a strided operand.
// WORDS: the operand is K-contiguous and 4-byte aligned, so whole words can be loaded.
template <bool WORDS>
__device__ __forceinline__ void load_tile(uint32_t (*dst)[PITCH_W], const uint8_t* src, long long row0,
                                          long long rows, long long rs, long long cs, int k0, int K, int tid) {
    if (WORDS) {
        // 64 rows x 8 words = 512 words, 256 threads -> 2 each
        for (int i = tid; i < TM * (TK / 4); i += 256) {
            const int r = i / (TK / 4), w = i % (TK / 4);
            const long long row = row0 + r;
            const int k = k0 + w * 4;
            uint32_t v = 0;
            if (row < rows && k < K) {
                const uint8_t* p = src + row * rs + k;
                if (k + 4 <= K) {
                    v = *reinterpret_cast<const uint32_t*>(p);
                } else {
                    for (int j = 0; j < K - k; ++j) v |= (uint32_t)p[j] << (8 * j);
                }
            }
            dst[r][w] = v;
        }
    } else {
        for (int i = tid; i < TM * (TK / 4); i += 256) {
            // consecutive threads walk rows first: for an operand whose rows are the contiguous
            // axis (cs large, rs == 1) that keeps the byte loads coalesced
            const int r = i % TM, w = i / TM;
            const long long row = row0 + r;
            uint32_t v = 0;
            if (row < rows) {
                for (int j = 0; j < 4; ++j) {
                    const int k = k0 + w * 4 + j;
                    if (k < K) v |= (uint32_t)src[row * rs + (long long)k * cs] << (8 * j);
                }
            }
            dst[r][w] = v;
        }
    }
}

template <bool A_UNSIGNED, bool A_WORDS, bool B_WORDS>
__global__ void __launch_bounds__(256) gemm_simt_kernel(SimtArgs g) {
    __shared__ uint32_t As[TM][PITCH_W];
    __shared__ uint32_t Bs[TN][PITCH_W];
    const int tid = threadIdx.x;
    const int tx = tid % 16, ty = tid / 16;
    const long long m0 = (long long)blockIdx.x * TM;
    const int n0 = blockIdx.y * TN;

    for (long long b = blockIdx.z; b < g.batch; b += gridDim.z) {
        const uint8_t* A = g.A + b * g.a_bs;
        const uint8_t* B = g.B + b * g.b_bs;
        int acc[4][4];
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) acc[i][j] = 0;

        for (int k0 = 0; k0 < g.K; k0 += TK) {
            load_tile<A_WORDS>(As, A, m0, g.M, g.a_rs, g.a_cs, k0, g.K, tid);
            load_tile<B_WORDS>(Bs, B, n0, g.N, g.b_ns, g.b_ks, k0, g.K, tid);
            __syncthreads();
#pragma unroll
            for (int w = 0; w < TK / 4; ++w) {
                uint32_t a[4], bb[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) a[i] = As[ty * 4 + i][w];
#pragma unroll
                for (int j = 0; j < 4; ++j) bb[j] = Bs[tx * 4 + j][w];
#pragma unroll
                for (int i = 0; i < 4; ++i)
#pragma unroll
                    for (int j = 0; j < 4; ++j) acc[i][j] = dot4<A_UNSIGNED>(a[i], bb[j], acc[i][j]);
            }
            __syncthreads();
        }

        uint8_t* C = g.C + b * g.c_bs * (g.out_dtype == A4C_I16 ? 2 : 1);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const long long m = m0 + ty * 4 + i;
            if (m >= g.M) continue;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int n = n0 + tx * 4 + j;
                if (n >= g.N) continue;
                int v = acc[i][j];
                if (g.bias) v = (int)((uint32_t)v + (uint32_t)g.bias[n]);
                v = clampi(round_shift_i32(v, g.rp), g.lo, g.hi);
                const long long idx = m * g.ldc + n;
                if (g.out_dtype == A4C_I16) reinterpret_cast<int16_t*>(C)[idx] = (int16_t)v;
                else C[idx] = (uint8_t)v;
            }
        }
    }
}

template <bool U>
void launch_simt(const SimtArgs& g, bool a_words, bool b_words, dim3 grid, cudaStream_t s) {
    if (a_words && b_words) gemm_simt_kernel<U, true, true><<<grid, 256, 0, s>>>(g);
    else if (a_words) gemm_simt_kernel<U, true, false><<<grid, 256, 0, s>>>(g);
    else if (b_words) gemm_simt_kernel<U, false, true><<<grid, 256, 0, s>>>(g);
    else gemm_simt_kernel<U, false, false><<<grid, 256, 0, s>>>(g);
}

}  // namespace

int a4c_launch_gemm_simt(const void* A, long long a_rs, long long a_cs, long long a_bs, const void* B,
                         long long b_ks, long long b_ns, long long b_bs, const int32_t* bias, void* C,
                         long long ldc, long long c_bs, long long batch, long long M, int K, int N, int shift,
                         int rounding, int relu, int out_dtype, int a_unsigned, cudaStream_t stream) {
    if (M == 0 || batch == 0) return A4C_OK;
    SimtArgs g;
    g.A = (const uint8_t*)A; g.a_rs = a_rs; g.a_cs = a_cs; g.a_bs = a_bs;
    g.B = (const uint8_t*)B; g.b_ks = b_ks; g.b_ns = b_ns; g.b_bs = b_bs;
    g.bias = bias; g.C = (uint8_t*)C; g.ldc = ldc; g.c_bs = c_bs;
    g.M = M; g.N = N; g.K = K; g.batch = batch;
    g.rp = make_round_params(shift, rounding);
    dtype_range(out_dtype, g.lo, g.hi);
    if (relu && g.lo < 0) g.lo = 0;
    g.out_dtype = out_dtype;
    const bool a_words = a_cs == 1 && (a_rs % 4 == 0) && (a_bs % 4 == 0) && ((uintptr_t)A % 4 == 0);
    const bool b_words = b_ks == 1 && (b_ns % 4 == 0) && (b_bs % 4 == 0) && ((uintptr_t)B % 4 == 0);
    const long long mt = (M + TM - 1) / TM;
    if (mt > 2147483647LL) return A4C_ERR_TOO_LARGE;
    dim3 grid((unsigned)mt, (unsigned)((N + TN - 1) / TN), (unsigned)(batch < 32768 ? batch : 32768));
    if (a_unsigned) launch_simt<true>(g, a_words, b_words, grid, stream);
    else launch_simt<false>(g, a_words, b_words, grid, stream);
    return cudaGetLastError() == cudaSuccess ? A4C_OK : A4C_ERR_CUDA;
}
