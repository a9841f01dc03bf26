// Floating-point Dense on the sm_100a tensor cores: bfloat16 operands (tcgen05.mma.kind::f16) and fp8 E4M3
// operands (kind::f8f6f4), float32 accumulation in TMEM.
//
//   Y[m,n] = round_to_storage(relu?(sum_k A[m,k] * W[k,n] + bias[n]))
//
// The float-simulation path of aie4ml (AIEConfig.ComputeDtype = bfloat16, passes/force_float_mode.py:22-46) and its
// fp8_e4m3 tensors (op_impls/families/matmul/common.py:39): operands stored in the compute type, products
// accumulated in float32 on top of nothing, the float32 bias added after, ReLU, and the result rounded to
// nearest-even into the storage type (fp8 saturates at +-448).  The order of the float32 additions is not part of
// that contract (the reference holds the path to rtol 1e-2 / atol 5e-2, tests/test_float_sim.py:87-93), so the
// tensor core's own summation order is as good as any.
//
// Structure: the streaming form of the int8 kernel (dense_tc.cu) -- one persistent CTA per SM, warp 0 TMA producer
// (A tile [128 rows x 128 bytes] and W^T tile [<= 256 rows x 128 bytes] per stage, 128-byte swizzle, 4 stages),
// warp 1 issues four MMAs of 32 bytes of K per stage into one of two 256-column TMEM accumulators, warps 2-9
// convert (two groups of four on alternate tiles): tcgen05.ld of 32 columns, bias, ReLU, rounding, and each lane
// stores its own row's pieces.  Tensor maps describe the operands as bytes, so one map shape serves both types;
// bytes outside the tensors read as zero, which is +0.0 in either format.  Every wait is bounded.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp8.h>

#include <mutex>

#include "a4c_common.cuh"
#include "a4c_kernels.h"
#include "tc_common.cuh"

namespace {

using namespace tc;

constexpr int BM = 128;
constexpr int BN = 256;
constexpr int BKB = 128;         // K BYTES per stage = one 128-byte swizzle row
constexpr int UMMA_KB = 32;      // K bytes per tcgen05.mma (16 bfloat16 or 32 fp8 values)
constexpr int STAGES = 4;
constexpr int A_BYTES = BM * BKB;
constexpr int B_BYTES = BN * BKB;
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int ACC_STAGES = 2;
constexpr int TMEM_COLS = ACC_STAGES * BN;
constexpr int EPI_WARPS = 8;
constexpr int EPI_GROUP_THREADS = 128;
constexpr int NUM_THREADS = 64 + EPI_WARPS * 32;

constexpr int KIND_BF16 = 0, KIND_FP8 = 2;   // the fdtype codes of the C ABI

struct Tail {
    uint64_t full[STAGES];
    uint64_t empty[STAGES];
    uint64_t tmem_full[ACC_STAGES];
    uint64_t tmem_empty[ACC_STAGES];
    uint32_t tmem_base;
    volatile int abort_flag;
};
constexpr size_t SMEM_BYTES = 1024 + (size_t)STAGES * STAGE_BYTES + sizeof(Tail);

struct FArgs {
    const float* bias;
    uint8_t* Y;
    long long ldy_bytes;
    long long M;
    int k_bytes, N;
    int num_m_tiles, num_n_tiles;
    int b_box_rows;
    int relu;
    uint32_t idesc;
    int* status;
};

// Instruction descriptor: [4,6) accumulator format 1 = f32, [7,10) A format, [10,13) B format (kind::f16: 1 = bf16;
// kind::f8f6f4: 0 = e4m3), both operands K-major, [17,23) N >> 3, [24,29) M >> 4.
constexpr uint32_t make_idesc_f(int m, int n, int kind) {
    const uint32_t fmt = kind == KIND_BF16 ? 1u : 0u;
    return (1u << 4) | (fmt << 7) | (fmt << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

template <int KIND>
__device__ __forceinline__ void umma_f(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    if (KIND == KIND_BF16)
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "setp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
            :: "r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
    else
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "setp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}"
            :: "r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}

// 16 float32 results -> storage type, as one or two 16-byte pieces
template <int KIND>
__device__ __forceinline__ void store_piece16(uint8_t* dst, const float* v, int valid) {
    if (KIND == KIND_BF16) {
        uint32_t w[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const __nv_bfloat162 p = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
            w[i] = *reinterpret_cast<const uint32_t*>(&p);
        }
        if (valid >= 16) {
            reinterpret_cast<uint4*>(dst)[0] = make_uint4(w[0], w[1], w[2], w[3]);
            reinterpret_cast<uint4*>(dst)[1] = make_uint4(w[4], w[5], w[6], w[7]);
        } else {
            for (int i = 0; i < valid; ++i)
                reinterpret_cast<uint16_t*>(dst)[i] = (uint16_t)(w[i >> 1] >> (16 * (i & 1)));
        }
    } else {
        uint32_t w[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            uint32_t word = 0;
#pragma unroll
            for (int b = 0; b < 4; ++b)
                word |= (uint32_t)__nv_cvt_float_to_fp8(v[4 * i + b], __NV_SATFINITE, __NV_E4M3) << (8 * b);
            w[i] = word;
        }
        if (valid >= 16) {
            *reinterpret_cast<uint4*>(dst) = make_uint4(w[0], w[1], w[2], w[3]);
        } else {
            for (int i = 0; i < valid; ++i) dst[i] = (uint8_t)(w[i >> 2] >> (8 * (i & 3)));
        }
    }
}

template <int KIND>
__global__ void __launch_bounds__(NUM_THREADS, 1)
dense_tcf_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b, FArgs g) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    Tail* tail = reinterpret_cast<Tail*>(smem + (size_t)STAGES * STAGE_BYTES);
    constexpr int ESZ = KIND == KIND_BF16 ? 2 : 1;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int num_tiles = g.num_m_tiles * g.num_n_tiles;
    const int num_kb = (g.k_bytes + BKB - 1) / BKB;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(&tail->full[s], 1); mbar_init(&tail->empty[s], 1); }
        for (int s = 0; s < ACC_STAGES; ++s) { mbar_init(&tail->tmem_full[s], 1); mbar_init(&tail->tmem_empty[s], EPI_GROUP_THREADS); }
        tail->abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     :: "r"(smem_u32(&tail->tmem_base)), "r"((uint32_t)TMEM_COLS) : "memory");
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
            for (int tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x) {
                const int m0 = (tile / g.num_n_tiles) * BM;
                const int n0 = (tile % g.num_n_tiles) * BN;
                for (int kb = 0; kb < num_kb; ++kb) {
                    ok = mbar_wait(&tail->empty[stage], phase ^ 1u, abort_flag, g.status, 141);
                    if (!ok) break;
                    uint8_t* sa = smem + (size_t)stage * STAGE_BYTES;
                    mbar_arrive_expect_tx(&tail->full[stage], (uint32_t)(A_BYTES + g.b_box_rows * BKB));
                    tma_load_2d(sa, &tmap_a, &tail->full[stage], kb * BKB, m0);
                    tma_load_2d(sa + A_BYTES, &tmap_b, &tail->full[stage], kb * BKB, n0);
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
            for (int tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x) {
                ok = mbar_wait_spin(&tail->tmem_empty[acc], acc_phase ^ 1u, abort_flag, g.status, 142);
                if (!ok) break;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + (uint32_t)(acc * BN);
                for (int kb = 0; kb < num_kb; ++kb) {
                    ok = mbar_wait(&tail->full[stage], phase, abort_flag, g.status, 143);
                    if (!ok) break;
                    tc_fence_after();
                    const uint32_t sa = smem_u32(smem) + (uint32_t)stage * STAGE_BYTES;
                    const uint64_t adesc = make_smem_desc(sa), bdesc = make_smem_desc(sa + A_BYTES);
#pragma unroll
                    for (int k = 0; k < BKB / UMMA_KB; ++k)
                        umma_f<KIND>(d_tmem, adesc + (uint64_t)(k * (UMMA_KB >> 4)), bdesc + (uint64_t)(k * (UMMA_KB >> 4)),
                                     g.idesc, (uint32_t)((kb | k) != 0));
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
        // two groups of four warps on alternate tiles; group g owns accumulator g
        const int quad = warp & 3;
        const int grp = (warp - 2) >> 2;
        uint32_t acc_phase = 0;
        bool ok = true;
        const uint32_t taddr = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(grp * BN);
        for (int tile = (int)blockIdx.x + grp * (int)gridDim.x; tile < num_tiles; tile += 2 * (int)gridDim.x) {
            const int m0 = (tile / g.num_n_tiles) * BM, n0 = (tile % g.num_n_tiles) * BN;
            if (ok) ok = mbar_wait(&tail->tmem_full[grp], acc_phase, abort_flag, g.status, 144);
            acc_phase ^= 1u;
            if (!ok) continue;
            tc_fence_after();
            const long long row = (long long)m0 + quad * 32 + lane;
            uint8_t* yrow = g.Y + row * g.ldy_bytes + (long long)n0 * ESZ;
#pragma unroll 1
            for (int c = 0; c < BN / 32; ++c) {
                const int col0 = n0 + c * 32;
                if (col0 < g.N) {       // warp-uniform
                    uint32_t r[32];
                    tmem_ld32(taddr + (uint32_t)(c * 32), r);
                    if (c == BN / 32 - 1 || col0 + 32 >= g.N) {   // last columns of the tile are in registers
                        tc_fence_before();
                        mbar_arrive(&tail->tmem_empty[grp]);
                    }
                    float v[32];
#pragma unroll
                    for (int i = 0; i < 32; ++i) {
                        const int n = col0 + i;
                        float x = __uint_as_float(r[i]) + ((g.bias != nullptr && n < g.N) ? __ldg(g.bias + n) : 0.0f);
                        v[i] = g.relu ? fmaxf(x, 0.0f) : x;
                    }
                    if (row < g.M) {
                        const int valid = g.N - col0;
                        store_piece16<KIND>(yrow + (long long)(c * 32) * ESZ, v, valid);
                        if (valid > 16) store_piece16<KIND>(yrow + (long long)(c * 32 + 16) * ESZ, v + 16, valid - 16);
                    }
                }
            }
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
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" :: "r"(tmem_base), "r"((uint32_t)TMEM_COLS) : "memory");
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

// byte view of a row-major [rows, row_bytes] operand with pitch ld_bytes; box = [box_rows, 128 bytes]
bool make_map(CUtensorMap* map, const void* base, long long rows, long long row_bytes, long long ld_bytes, int box_rows) {
    EncodeTiledFn fn = get_encode_fn();
    if (!fn) return false;
    cuuint64_t dims[2] = {(cuuint64_t)row_bytes, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld_bytes};
    cuuint32_t box[2] = {(cuuint32_t)BKB, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int KIND>
cudaError_t launch_kind(const CUtensorMap& ma, const CUtensorMap& mb, const FArgs& g, int grid, cudaStream_t s) {
    static tc::SmemOptIn opt_in;
    const cudaError_t e = opt_in.ensure(dense_tcf_kernel<KIND>, SMEM_BYTES);
    if (e != cudaSuccess) return e;
    dense_tcf_kernel<KIND><<<grid, NUM_THREADS, SMEM_BYTES, s>>>(ma, mb, g);
    return cudaGetLastError();
}

}  // namespace

int a4c_dense_tcf_supported(const void* A, long long lda, const void* Wt, long long ldw, const void* Y, long long ldy,
                            long long M, int K, int N, int kind) {
    if (kind != KIND_BF16 && kind != KIND_FP8) return A4C_ERR_UNSUPPORTED;
    const int esz = kind == KIND_BF16 ? 2 : 1;
    if ((long long)K * esz < 32) return A4C_ERR_UNSUPPORTED;           // less than one MMA of K
    if ((lda * esz) % 16 || (ldw * esz) % 16 || (ldy * esz) % 16) return A4C_ERR_ALIGNMENT;
    if (((uintptr_t)A | (uintptr_t)Wt | (uintptr_t)Y) & 15u) return A4C_ERR_ALIGNMENT;
    if (M > 2147483647LL - BM || lda < K || ldw < K || ldy < N) return A4C_ERR_INVALID_ARG;
    if (((M + BM - 1) / BM) * ((N + BN - 1) / BN) > 2147483647LL) return A4C_ERR_TOO_LARGE;
    return A4C_OK;
}

int a4c_launch_dense_tcf(const void* A, long long lda, const void* Wt, long long ldw, const float* bias, void* Y,
                         long long ldy, long long M, int K, int N, int relu, int kind, int* status_word,
                         cudaStream_t stream) {
    const int sup = a4c_dense_tcf_supported(A, lda, Wt, ldw, Y, ldy, M, K, N, kind);
    if (sup != A4C_OK) return sup;
    if (M == 0) return A4C_OK;
    const int esz = kind == KIND_BF16 ? 2 : 1;
    FArgs g;
    g.bias = bias; g.Y = (uint8_t*)Y; g.ldy_bytes = ldy * esz; g.M = M; g.k_bytes = K * esz; g.N = N;
    g.num_m_tiles = (int)((M + BM - 1) / BM);
    g.num_n_tiles = (N + BN - 1) / BN;
    const int umma_n = g.num_n_tiles == 1 ? ((N + 15) / 16) * 16 : BN;
    g.b_box_rows = umma_n;
    g.idesc = make_idesc_f(BM, umma_n, kind);
    g.relu = relu;
    g.status = status_word;
    CUtensorMap ma, mb;
    if (!make_map(&ma, A, M, (long long)K * esz, lda * esz, BM) || !make_map(&mb, Wt, N, (long long)K * esz, ldw * esz, umma_n))
        return A4C_ERR_CUDA;
    int dev = 0, sms = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const long long tiles = (long long)g.num_m_tiles * g.num_n_tiles;
    const int grid = (int)(tiles < sms ? tiles : sms);
    const cudaError_t err = kind == KIND_BF16 ? launch_kind<KIND_BF16>(ma, mb, g, grid, stream)
                                              : launch_kind<KIND_FP8>(ma, mb, g, grid, stream);
    return err == cudaSuccess ? A4C_OK : A4C_ERR_CUDA;
}
