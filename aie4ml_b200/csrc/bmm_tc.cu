// Batched dynamic int8 MatMul on the sm_100a tensor cores:  C_b = clamp(round_shift(A_b . op(B_b), shift)).
//
// This is matmul_single::run of aie4ml (matmul.cpp:32-118) applied once per leading index: no bias, no ReLU,
// SRS with the op's rounding token, the A operand possibly uint8 (a softmax output), the B operand stored
// either [N, K] (a folded Transpose: TRANSPOSE_B, matmul.cpp:68-72) or [K, N].
//
// Same main loop as the Dense kernel (TMA producer / MMA issuer, a 4-stage shared-memory ring, two TMEM
// accumulators) with a simpler epilogue (four warps, lane = row, 16-byte global stores), and three differences:
//   * operands come through 3-D tensor maps {inner, rows, batch}, so a tile never reads rows of the next
//     batch entry: rows past the matrix edge are zero-filled by TMA;
//   * B stored [N, K] is a K-major operand exactly like Dense weights; B stored [K, N] is an MN-major operand:
//     the TMA box is [128 k-rows x 64 bytes of n] with 64-byte swizzle, the shared-memory descriptor uses the
//     64-byte-swizzle MN-major canonical layout (k-rows 64 B apart, 8-row groups 512 B apart) and the
//     instruction descriptor marks B as MN-major; the N tile is 64 in that case;
//   * the N tile is a template parameter (64 / 128 / 256);
//   * A stored [K, M] (a folded Transpose on the left operand: TRANSPOSE_A, matmul.cpp:60-67; the transposed input view
//     of a Dense: TRANSPOSE_INPUT, dense_bias_relu.cpp:99,135) is an MN-major A operand: the TMA box is
//     [128 k-rows x 128 bytes of m] with 128-byte swizzle, the same shared-memory descriptor as a K-major tile
//     (rows of 128 bytes, 8-row groups 1024 bytes apart) with the instruction descriptor marking A as MN-major, and
//     one MMA advances 32 k-rows.  With a bias vector, a ReLU clamp and a B operand shared by all batch entries this
//     is the Dense over a transposed input view (a4c_dense_ta).
#include <cuda.h>

#include <mutex>

#include "a4c_common.cuh"
#include "a4c_kernels.h"
#include "tc_common.cuh"

using namespace tc;

namespace {

constexpr int BM = 128;
constexpr int BK = 128;
constexpr int UMMA_K = 32;
constexpr int STAGES = 4;
constexpr int ACC_STAGES = 2;
constexpr int NUM_THREADS = 192;
constexpr int EPI_THREADS = 128;

template <int BN>
struct Cfg {
    static constexpr int A_BYTES = BM * BK;
    static constexpr int B_BYTES = BN * BK;   // K-major: BN rows x 128 B; MN-major (BN = 64): 128 rows x 64 B
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    static constexpr int TMEM_COLS = ACC_STAGES * BN < 32 ? 32 : ACC_STAGES * BN;
};

struct Tail {
    uint64_t full[STAGES];
    uint64_t empty[STAGES];
    uint64_t tmem_full[ACC_STAGES];
    uint64_t tmem_empty[ACC_STAGES];
    uint32_t tmem_base;
    volatile int abort_flag;
};

struct BmmArgs {
    const int32_t* bias;          // per output column, or NULL (Dense over a transposed input view only)
    int b_shared;                 // every batch entry multiplies by the same B (batch coordinate 0)
    uint8_t* C; long long ldc, stride_c;
    long long batch; int M, K, N;
    int m_tiles, n_tiles;
    int shift, lo, hi;
    uint32_t mask, c0, idesc;
    int* status;
};

__device__ __forceinline__ void tma_load_3d(void* dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1, int c2) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
        :: "r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2) : "memory");
}

// MN-major operand, 64-byte swizzle: rows (k) of 64 bytes, 8-row groups 512 bytes apart.
__device__ __forceinline__ uint64_t make_smem_desc_mn64(uint32_t saddr) {
    uint64_t d = 0;
    d |= (uint64_t)((saddr & 0x3FFFFu) >> 4);
    d |= (uint64_t)1 << 16;              // leading byte offset: unused (one 64-byte atom along N)
    d |= (uint64_t)(512 >> 4) << 32;     // stride byte offset between 8-row groups along K
    d |= (uint64_t)1 << 46;              // descriptor version
    d |= (uint64_t)4 << 61;              // SWIZZLE_64B
    return d;
}

template <int MODE>
__device__ __forceinline__ int requant(int acc, const BmmArgs& g) {
    int v = acc;
    if (MODE >= 0) v = round_shift_i32_t<MODE>(acc, g.shift, g.mask, g.c0);
    return min(max(v, g.lo), g.hi);
}

template <int BN, bool B_MN, bool A_MN, int MODE>
__global__ void __launch_bounds__(NUM_THREADS, 1)
bmm_tc_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b, BmmArgs g) {
    using C = Cfg<BN>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    Tail* tail = reinterpret_cast<Tail*>(smem + (size_t)STAGES * C::STAGE_BYTES);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const long long tiles_per_batch = (long long)g.m_tiles * g.n_tiles;
    const long long num_tiles = g.batch * tiles_per_batch;
    const int num_kb = (g.K + BK - 1) / BK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(&tail->full[s], 1); mbar_init(&tail->empty[s], 1); }
        for (int s = 0; s < ACC_STAGES; ++s) { mbar_init(&tail->tmem_full[s], 1); mbar_init(&tail->tmem_empty[s], EPI_THREADS); }
        tail->abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     :: "r"(smem_u32(&tail->tmem_base)), "r"((uint32_t)C::TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tail->tmem_base;
    volatile int* abort_flag = &tail->abort_flag;

    if (warp == 0) {
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (long long tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x) {
                const int b = (int)(tile / tiles_per_batch);
                const int t = (int)(tile % tiles_per_batch);
                const int m0 = (t / g.n_tiles) * BM;
                const int n0 = (t % g.n_tiles) * BN;
                for (int kb = 0; kb < num_kb; ++kb) {
                    ok = mbar_wait(&tail->empty[stage], phase ^ 1u, abort_flag, g.status, 111);
                    if (!ok) break;
                    uint8_t* sa = smem + (size_t)stage * C::STAGE_BYTES;
                    mbar_arrive_expect_tx(&tail->full[stage], C::STAGE_BYTES);
                    const int bb = g.b_shared ? 0 : b;
                    if (A_MN) tma_load_3d(sa, &tmap_a, &tail->full[stage], m0, kb * BK, b);
                    else tma_load_3d(sa, &tmap_a, &tail->full[stage], kb * BK, m0, b);
                    if (B_MN) tma_load_3d(sa + C::A_BYTES, &tmap_b, &tail->full[stage], n0, kb * BK, bb);
                    else tma_load_3d(sa + C::A_BYTES, &tmap_b, &tail->full[stage], kb * BK, n0, bb);
                    if (++stage == STAGES) { stage = 0; phase ^= 1u; }
                }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        if (lane == 0) {
            int stage = 0, acc = 0;
            uint32_t phase = 0, acc_phase = 0;
            bool ok = true;
            for (long long tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x) {
                ok = mbar_wait(&tail->tmem_empty[acc], acc_phase ^ 1u, abort_flag, g.status, 112);
                if (!ok) break;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + (uint32_t)(acc * BN);
                for (int kb = 0; kb < num_kb; ++kb) {
                    ok = mbar_wait(&tail->full[stage], phase, abort_flag, g.status, 113);
                    if (!ok) break;
                    tc_fence_after();
                    const uint32_t sa = smem_u32(smem + (size_t)stage * C::STAGE_BYTES);
                    const uint64_t adesc = make_smem_desc(sa);
                    const uint64_t bdesc = B_MN ? make_smem_desc_mn64(sa + C::A_BYTES) : make_smem_desc(sa + C::A_BYTES);
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k) {
                        // K step: a K-major operand advances 32 bytes inside the swizzle row; an MN-major B advances
                        // 32 k-rows of 64 bytes, an MN-major A 32 k-rows of 128 bytes
                        const uint64_t a_k = adesc + (uint64_t)(A_MN ? k * ((UMMA_K * 128) >> 4) : k * (UMMA_K >> 4));
                        const uint64_t b_k = bdesc + (uint64_t)(B_MN ? k * ((UMMA_K * 64) >> 4) : k * (UMMA_K >> 4));
                        umma_i8(d_tmem, a_k, b_k, g.idesc, (uint32_t)((kb | k) != 0));
                    }
                    umma_commit(&tail->empty[stage]);
                    if (++stage == STAGES) { stage = 0; phase ^= 1u; }
                }
                if (!ok) break;
                umma_commit(&tail->tmem_full[acc]);
                if (++acc == ACC_STAGES) { acc = 0; acc_phase ^= 1u; }
            }
        }
        __syncwarp();
    } else {
        const int quad = warp & 3;
        int acc = 0;
        uint32_t acc_phase = 0;
        bool ok = true;
        for (long long tile = blockIdx.x; tile < num_tiles; tile += gridDim.x) {
            const long long b = tile / tiles_per_batch;
            const int t = (int)(tile % tiles_per_batch);
            const int m0 = (t / g.n_tiles) * BM;
            const int n0 = (t % g.n_tiles) * BN;
            if (ok) ok = mbar_wait(&tail->tmem_full[acc], acc_phase, abort_flag, g.status, 114);
            if (ok) {
                tc_fence_after();
                const int row = m0 + quad * 32 + lane;
                uint8_t* crow = g.C + b * g.stride_c + (long long)row * g.ldc + n0;
                const uint32_t taddr = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(acc * BN);
#pragma unroll 1
                for (int c = 0; c < BN / 32; ++c) {
                    if (n0 + c * 32 >= g.N) break;
                    uint32_t r[32];
                    tmem_ld32(taddr + (uint32_t)(c * 32), r);
                    uint32_t w[8];
#pragma unroll
                    for (int q = 0; q < 8; ++q) {
                        int o[4];
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const int n = n0 + c * 32 + q * 4 + e;
                            // acc32 wraps when the bias is added (it is the accumulator's initial value in the reference)
                            const uint32_t bv = (g.bias != nullptr && n < g.N) ? (uint32_t)__ldg(g.bias + n) : 0u;
                            o[e] = requant<MODE>((int)(r[q * 4 + e] + bv), g);
                        }
                        w[q] = (uint32_t)(o[0] & 0xFF) | ((uint32_t)(o[1] & 0xFF) << 8) |
                               ((uint32_t)(o[2] & 0xFF) << 16) | ((uint32_t)o[3] << 24);
                    }
                    if (row < g.M) {
                        const int col0 = n0 + c * 32;
                        if (col0 < g.N) *reinterpret_cast<uint4*>(crow + c * 32) = make_uint4(w[0], w[1], w[2], w[3]);
                        if (col0 + 16 < g.N)
                            *reinterpret_cast<uint4*>(crow + c * 32 + 16) = make_uint4(w[4], w[5], w[6], w[7]);
                    }
                }
                tc_fence_before();
                mbar_arrive(&tail->tmem_empty[acc]);
            }
            if (++acc == ACC_STAGES) { acc = 0; acc_phase ^= 1u; }
        }
    }

    __syncthreads();
    if (*abort_flag) {
        const uint64_t t0 = a4c_globaltimer();
        while (a4c_globaltimer() - t0 < 2000000ull) __nanosleep(1000);
        __syncthreads();
    }
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;"
                     :: "r"(tmem_base), "r"((uint32_t)C::TMEM_COLS) : "memory");
    }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    });
    return fn;
}

// 3-D uint8 map {inner, rows, batch}; box {box_inner, box_rows, 1}
bool make_map3(CUtensorMap* map, const void* base, long long inner, long long rows, long long batch, long long ld,
               long long stride, int box_inner, int box_rows, CUtensorMapSwizzle swz) {
    EncodeTiledFn fn = get_encode_fn();
    if (!fn) return false;
    if (batch <= 1) stride = (rows > 0 ? rows : 1) * ld;  // a single entry: any legal stride
    cuuint64_t dims[3] = {(cuuint64_t)inner, (cuuint64_t)rows, (cuuint64_t)(batch > 0 ? batch : 1)};
    cuuint64_t strides[2] = {(cuuint64_t)ld, (cuuint64_t)stride};
    cuuint32_t box[3] = {(cuuint32_t)box_inner, (cuuint32_t)box_rows, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<void*>(base), dims, strides, box, estr,
              CU_TENSOR_MAP_INTERLEAVE_NONE, swz, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int BN, bool B_MN, bool A_MN, int MODE>
cudaError_t launch_one(const CUtensorMap& ma, const CUtensorMap& mb, const BmmArgs& g, int grid, cudaStream_t s) {
    constexpr size_t smem = 1024 + (size_t)STAGES * Cfg<BN>::STAGE_BYTES + sizeof(Tail);
    static tc::SmemOptIn opt_in;
    const cudaError_t attr_err = opt_in.ensure(bmm_tc_kernel<BN, B_MN, A_MN, MODE>, smem);
    if (attr_err != cudaSuccess) return attr_err;
    bmm_tc_kernel<BN, B_MN, A_MN, MODE><<<grid, NUM_THREADS, smem, s>>>(ma, mb, g);
    return cudaGetLastError();
}

template <int BN, bool B_MN, bool A_MN = false>
cudaError_t launch_mode(int shift, int rounding, const CUtensorMap& ma, const CUtensorMap& mb, const BmmArgs& g, int grid,
                        cudaStream_t s) {
    if (shift == 0) return launch_one<BN, B_MN, A_MN, -1>(ma, mb, g, grid, s);
    switch (rounding) {
        case A4C_RND_FLOOR: return launch_one<BN, B_MN, A_MN, A4C_RND_FLOOR>(ma, mb, g, grid, s);
        case A4C_RND_CEIL: return launch_one<BN, B_MN, A_MN, A4C_RND_CEIL>(ma, mb, g, grid, s);
        case A4C_RND_POSITIVE_INF: return launch_one<BN, B_MN, A_MN, A4C_RND_POSITIVE_INF>(ma, mb, g, grid, s);
        case A4C_RND_NEGATIVE_INF: return launch_one<BN, B_MN, A_MN, A4C_RND_NEGATIVE_INF>(ma, mb, g, grid, s);
        case A4C_RND_SYMMETRIC_INF: return launch_one<BN, B_MN, A_MN, A4C_RND_SYMMETRIC_INF>(ma, mb, g, grid, s);
        case A4C_RND_SYMMETRIC_ZERO: return launch_one<BN, B_MN, A_MN, A4C_RND_SYMMETRIC_ZERO>(ma, mb, g, grid, s);
        case A4C_RND_CONV_EVEN: return launch_one<BN, B_MN, A_MN, A4C_RND_CONV_EVEN>(ma, mb, g, grid, s);
        default: return launch_one<BN, B_MN, A_MN, A4C_RND_CONV_ODD>(ma, mb, g, grid, s);
    }
}

}  // namespace

int a4c_bmm_tc_supported(const void* A, long long lda, long long stride_a, const void* B, long long ldb,
                         long long stride_b, const void* C, long long ldc, long long stride_c, long long batch, int M,
                         int K, int N, int trans_a, int trans_b, int out_dtype) {
    if (trans_a && !trans_b) return A4C_ERR_UNSUPPORTED;   // both operands MN-major: left to the any-stride kernel
    if (out_dtype != A4C_I8 && out_dtype != A4C_U8) return A4C_ERR_UNSUPPORTED;
    if (N % 16 != 0 || K < 16) return A4C_ERR_UNSUPPORTED;
    if (lda % 16 || ldb % 16 || ldc % 16) return A4C_ERR_ALIGNMENT;
    if (batch > 1 && (stride_a % 16 || stride_b % 16 || stride_c % 16)) return A4C_ERR_ALIGNMENT;
    if (((uintptr_t)A | (uintptr_t)B | (uintptr_t)C) & 15u) return A4C_ERR_ALIGNMENT;
    if (batch > 2147483647LL) return A4C_ERR_TOO_LARGE;
    return A4C_OK;
}

namespace {

// trans_a: A_b stored [K, M] (MN-major operand).  bias / relu / b_shared: the Dense over a transposed input view.
int launch_any(const void* A, long long lda, long long stride_a, const void* B, long long ldb, long long stride_b,
               const int32_t* bias, int relu, int b_shared, void* C, long long ldc, long long stride_c, long long batch, int M,
               int K, int N, int trans_a, int trans_b, int shift, int rounding, int out_dtype, int a_unsigned, int* status_word,
               cudaStream_t stream) {
    if (batch == 0) return A4C_OK;
    const bool b_mn = !trans_b;
    const bool a_mn = trans_a != 0;
    if (a_mn && b_mn) return A4C_ERR_UNSUPPORTED;
    const int BN = b_mn ? 64 : (N <= 64 ? 64 : (N <= 128 ? 128 : 256));
    CUtensorMap ma, mb;
    if (a_mn) {
        if (!make_map3(&ma, A, M, K, batch, lda, stride_a, 128, BK, CU_TENSOR_MAP_SWIZZLE_128B)) return A4C_ERR_CUDA;
    } else {
        if (!make_map3(&ma, A, K, M, batch, lda, stride_a, BK, BM, CU_TENSOR_MAP_SWIZZLE_128B)) return A4C_ERR_CUDA;
    }
    const long long b_batch = b_shared ? 1 : batch;
    if (b_mn) {
        if (!make_map3(&mb, B, N, K, b_batch, ldb, stride_b, 64, BK, CU_TENSOR_MAP_SWIZZLE_64B)) return A4C_ERR_CUDA;
    } else {
        if (!make_map3(&mb, B, K, N, b_batch, ldb, stride_b, BK, BN, CU_TENSOR_MAP_SWIZZLE_128B)) return A4C_ERR_CUDA;
    }
    BmmArgs g;
    g.bias = bias; g.b_shared = b_shared ? 1 : 0;
    g.C = (uint8_t*)C; g.ldc = ldc; g.stride_c = stride_c; g.batch = batch; g.M = M; g.K = K; g.N = N;
    g.m_tiles = (M + BM - 1) / BM;
    g.n_tiles = (N + BN - 1) / BN;
    g.shift = shift;
    dtype_range(out_dtype, g.lo, g.hi);
    if (relu && g.lo < 0) g.lo = 0;
    const RoundParams rp = make_round_params(shift, rounding);
    g.mask = rp.mask; g.c0 = rp.c0;
    g.idesc = make_idesc(BM, BN, a_unsigned != 0) | (b_mn ? (1u << 16) : 0u) | (a_mn ? (1u << 15) : 0u);
    g.status = status_word;
    int dev = 0, sms = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const long long tiles = batch * g.m_tiles * g.n_tiles;
    const int grid = (int)(tiles < sms ? tiles : sms);
    cudaError_t err;
    if (a_mn) {
        if (BN == 64) err = launch_mode<64, false, true>(shift, rounding, ma, mb, g, grid, stream);
        else if (BN == 128) err = launch_mode<128, false, true>(shift, rounding, ma, mb, g, grid, stream);
        else err = launch_mode<256, false, true>(shift, rounding, ma, mb, g, grid, stream);
    }
    else if (b_mn) err = launch_mode<64, true>(shift, rounding, ma, mb, g, grid, stream);
    else if (BN == 64) err = launch_mode<64, false>(shift, rounding, ma, mb, g, grid, stream);
    else if (BN == 128) err = launch_mode<128, false>(shift, rounding, ma, mb, g, grid, stream);
    else err = launch_mode<256, false>(shift, rounding, ma, mb, g, grid, stream);
    return err == cudaSuccess ? A4C_OK : A4C_ERR_CUDA;
}

}  // namespace

int a4c_launch_bmm_tc(const void* A, long long lda, long long stride_a, const void* B, long long ldb, long long stride_b,
                      void* C, long long ldc, long long stride_c, long long batch, int M, int K, int N, int trans_a,
                      int trans_b, int shift, int rounding, int out_dtype, int a_unsigned, int* status_word,
                      cudaStream_t stream) {
    return launch_any(A, lda, stride_a, B, ldb, stride_b, nullptr, 0, 0, C, ldc, stride_c, batch, M, K, N, trans_a, trans_b,
                      shift, rounding, out_dtype, a_unsigned, status_word, stream);
}

int a4c_dense_ta_tc_supported(const void* A, long long lda, long long stride_a, const void* Wt, long long ldw, const void* Y,
                              long long ldy, long long stride_y, long long batch, int M, int K, int N, int out_dtype) {
    // stored A_b [K, M]: the m axis is the contiguous one
    return a4c_bmm_tc_supported(A, lda, stride_a, Wt, ldw, 0, Y, ldy, stride_y, batch, M, K, N, 1, 1, out_dtype);
}

int a4c_launch_dense_ta_tc(const void* A, long long lda, long long stride_a, const void* Wt, long long ldw,
                           const int32_t* bias, void* Y, long long ldy, long long stride_y, long long batch, int M, int K,
                           int N, int shift, int rounding, int relu, int out_dtype, int a_unsigned, int* status_word,
                           cudaStream_t stream) {
    return launch_any(A, lda, stride_a, Wt, ldw, 0, bias, relu, 1, Y, ldy, stride_y, batch, M, K, N, 1, 1, shift, rounding,
                      out_dtype, a_unsigned, status_word, stream);
}
