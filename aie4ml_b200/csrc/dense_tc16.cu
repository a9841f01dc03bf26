// int16 x int8 Dense on the sm_100a tensor cores, exact under the reference's 32-bit wrapping accumulator.
//
//   Y[m,n] = clamp(round_shift(wrap32(sum_k A[m,k] * W[k,n] + bias[n]), shift), lo, hi)     (lo = max(lo, 0) with ReLU)
//
// dense_single::run of aie4ml (dense_bias_relu.cpp:67-166) for 16-bit activations against 8-bit weights, which the
// reference accumulates in acc32 lanes (op_impls/utils/precision.py:116-127).  The tensor cores multiply 8-bit
// operands only, so every activation is split into two digits, x = 256 * hi + lo with hi = x >> 8 a signed byte and
// lo = x & 255 an unsigned byte, and
//     sum_k x_k w_k = 256 * sum_k hi_k w_k + sum_k lo_k w_k        (mod 2^32: the ring the accumulator lives in)
// Both digit sums fit 32 bits exactly for any K the kernel accepts, so combining them with wrapping arithmetic in the
// epilogue gives the bits a wrapping accumulation of the 16-bit products gives.
//
// Two kernels per chunk of rows:
//   split_planes_kernel   int16 rows -> a signed high-byte plane and an unsigned low-byte plane (K-contiguous, 16-byte
//                         pitch), in a fixed per-device workspace; rows are processed in chunks that fit it
//   dense_tc16_kernel     persistent, warp-specialised like the int8 kernel: warp 0 loads per stage one [128 x 128 B]
//                         tile of each plane and one [128 x 128 B] tile of W^T (TMA, 128-byte swizzle, 4 stages); warp
//                         1 issues per 32 bytes of K one s8 x s8 MMA into the tile's high accumulator and one u8 x s8 MMA
//                         into its low accumulator (M128 N128 K32; two tiles' accumulator pairs fill the 512 TMEM
//                         columns); warps 2-5 combine, add the bias, requantise and store.
// Every wait is bounded.
#include <cuda.h>

#include <mutex>

#include "a4c_common.cuh"
#include "a4c_kernels.h"
#include "tc_common.cuh"

namespace {

using namespace tc;

constexpr int BM = 128;
constexpr int BN = 128;
constexpr int BK = 128;
constexpr int UMMA_K = 32;
constexpr int STAGES = 4;
constexpr int TILE_BYTES = 128 * BK;                 // every operand tile: 128 rows x 128 bytes
constexpr int STAGE_BYTES = 3 * TILE_BYTES;          // high plane, low plane, weights
constexpr int ACC_STAGES = 2;
constexpr int TMEM_COLS = ACC_STAGES * 2 * BN;       // 512
constexpr int NUM_THREADS = 192;
constexpr int EPI_THREADS = 128;

constexpr long long WORKSPACE_BYTES = 64ll << 20;    // both planes of one chunk of rows
constexpr int kMaxDevices = 64;

struct Tail {
    uint64_t full[STAGES];
    uint64_t empty[STAGES];
    uint64_t tmem_full[ACC_STAGES];
    uint64_t tmem_empty[ACC_STAGES];
    uint32_t tmem_base;
    volatile int abort_flag;
};
constexpr size_t SMEM_BYTES = 1024 + (size_t)STAGES * STAGE_BYTES + sizeof(Tail);

struct Args16 {
    const int32_t* bias;
    uint8_t* Y;
    long long ldy;       // elements
    long long M;
    int K, N;
    int num_m_tiles, num_n_tiles;
    int out_dtype, lo, hi;
    RoundParams rp;
    int* status;
};

// int16 [rows, lda] -> hi int8 [rows, kp], lo uint8 [rows, kp]; columns K..kp-1 are zero.  Eight elements per thread.
__global__ void __launch_bounds__(256) split_planes_kernel(const int16_t* __restrict__ A, long long lda, int8_t* __restrict__ hi,
                                                           uint8_t* __restrict__ lo, long long rows, int K, int kp) {
    const int groups = kp >> 3;
    const long long total = rows * groups;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const long long r = i / groups;
        const int c0 = (int)(i - r * groups) << 3;
        uint32_t w[4] = {0, 0, 0, 0};
        if (c0 + 8 <= K) {
            const uint4 v = *reinterpret_cast<const uint4*>(A + r * lda + c0);
            w[0] = v.x; w[1] = v.y; w[2] = v.z; w[3] = v.w;
        } else {
            for (int e = 0; e < 8 && c0 + e < K; ++e)
                w[e >> 1] |= (uint32_t)(uint16_t)A[r * lda + c0 + e] << (16 * (e & 1));
        }
        // word j holds elements 2j (low half) and 2j + 1: low bytes are bytes 0 and 2, high bytes 1 and 3
        uint32_t lo01, lo23, hi01, hi23;
        asm("prmt.b32 %0, %1, %2, 0x6420;" : "=r"(lo01) : "r"(w[0]), "r"(w[1]));
        asm("prmt.b32 %0, %1, %2, 0x6420;" : "=r"(lo23) : "r"(w[2]), "r"(w[3]));
        asm("prmt.b32 %0, %1, %2, 0x7531;" : "=r"(hi01) : "r"(w[0]), "r"(w[1]));
        asm("prmt.b32 %0, %1, %2, 0x7531;" : "=r"(hi23) : "r"(w[2]), "r"(w[3]));
        *reinterpret_cast<uint2*>(lo + r * kp + c0) = make_uint2(lo01, lo23);
        *reinterpret_cast<uint2*>(hi + r * kp + c0) = make_uint2(hi01, hi23);
    }
}

__global__ void __launch_bounds__(NUM_THREADS, 1)
dense_tc16_kernel(const __grid_constant__ CUtensorMap tmap_hi, const __grid_constant__ CUtensorMap tmap_lo,
                  const __grid_constant__ CUtensorMap tmap_w, Args16 g) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    Tail* tail = reinterpret_cast<Tail*>(smem + (size_t)STAGES * STAGE_BYTES);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int num_tiles = g.num_m_tiles * g.num_n_tiles;
    const int num_kb = (g.K + BK - 1) / BK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(&tail->full[s], 1); mbar_init(&tail->empty[s], 1); }
        for (int s = 0; s < ACC_STAGES; ++s) { mbar_init(&tail->tmem_full[s], 1); mbar_init(&tail->tmem_empty[s], EPI_THREADS); }
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
                const int m0 = (tile / g.num_n_tiles) * BM, n0 = (tile % g.num_n_tiles) * BN;
                for (int kb = 0; kb < num_kb; ++kb) {
                    ok = mbar_wait(&tail->empty[stage], phase ^ 1u, abort_flag, g.status, 151);
                    if (!ok) break;
                    uint8_t* st = smem + (size_t)stage * STAGE_BYTES;
                    mbar_arrive_expect_tx(&tail->full[stage], (uint32_t)STAGE_BYTES);
                    tma_load_2d(st, &tmap_hi, &tail->full[stage], kb * BK, m0);
                    tma_load_2d(st + TILE_BYTES, &tmap_lo, &tail->full[stage], kb * BK, m0);
                    tma_load_2d(st + 2 * TILE_BYTES, &tmap_w, &tail->full[stage], kb * BK, n0);
                    if (++stage == STAGES) { stage = 0; phase ^= 1u; }
                }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        if (lane == 0) {
            const uint32_t idesc_hi = make_idesc(BM, BN, false);   // signed high digit
            const uint32_t idesc_lo = make_idesc(BM, BN, true);    // unsigned low digit
            int stage = 0, acc = 0;
            uint32_t phase = 0, acc_phase = 0;
            bool ok = true;
            for (int tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x) {
                ok = mbar_wait_spin(&tail->tmem_empty[acc], acc_phase ^ 1u, abort_flag, g.status, 152);
                if (!ok) break;
                tc_fence_after();
                const uint32_t d_hi = tmem_base + (uint32_t)(acc * 2 * BN), d_lo = d_hi + (uint32_t)BN;
                for (int kb = 0; kb < num_kb; ++kb) {
                    ok = mbar_wait(&tail->full[stage], phase, abort_flag, g.status, 153);
                    if (!ok) break;
                    tc_fence_after();
                    const uint32_t st = smem_u32(smem) + (uint32_t)stage * STAGE_BYTES;
                    const uint64_t hdesc = make_smem_desc(st), ldesc = make_smem_desc(st + TILE_BYTES);
                    const uint64_t wdesc = make_smem_desc(st + 2 * TILE_BYTES);
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k) {
                        const uint64_t adv = (uint64_t)(k * (UMMA_K >> 4));
                        umma_i8(d_hi, hdesc + adv, wdesc + adv, idesc_hi, (uint32_t)((kb | k) != 0));
                        umma_i8(d_lo, ldesc + adv, wdesc + adv, idesc_lo, (uint32_t)((kb | k) != 0));
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
        const int esz = g.out_dtype == A4C_I16 ? 2 : 1;
        int acc = 0;
        uint32_t acc_phase = 0;
        bool ok = true;
        for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x) {
            const int m0 = (tile / g.num_n_tiles) * BM, n0 = (tile % g.num_n_tiles) * BN;
            if (ok) ok = mbar_wait(&tail->tmem_full[acc], acc_phase, abort_flag, g.status, 154);
            if (ok) {
                tc_fence_after();
                const long long row = (long long)m0 + quad * 32 + lane;
                uint8_t* yrow = g.Y + (row * g.ldy + n0) * esz;
                const uint32_t taddr = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(acc * 2 * BN);
#pragma unroll 1
                for (int c = 0; c < BN / 32; ++c) {
                    const int col0 = n0 + c * 32;
                    if (col0 >= g.N) break;
                    uint32_t rh[32], rl[32];
                    tmem_ld32_async(taddr + (uint32_t)(c * 32), rh);
                    tmem_ld32_async(taddr + (uint32_t)(BN + c * 32), rl);
                    tmem_ld_wait32(rh);
                    tmem_ld_wait32(rl);
                    int o[32];
#pragma unroll
                    for (int i = 0; i < 32; ++i) {
                        const int n = col0 + i;
                        const uint32_t bv = (g.bias != nullptr && n < g.N) ? (uint32_t)__ldg(g.bias + n) : 0u;
                        const int v = (int)((rh[i] << 8) + rl[i] + bv);        // wraps like the 32-bit accumulator
                        o[i] = min(max(round_shift_i32(v, g.rp), g.lo), g.hi);
                    }
                    if (row < g.M) {
                        const int valid = min(32, g.N - col0);
                        if (esz == 1) {
#pragma unroll
                            for (int p = 0; p < 2; ++p) {
                                uint8_t* dst = yrow + c * 32 + p * 16;
                                if (valid >= (p + 1) * 16 && (((uintptr_t)dst) & 15u) == 0) {
                                    uint32_t w[4];
#pragma unroll
                                    for (int q = 0; q < 4; ++q) w[q] = pack4_i8(o[p * 16 + q * 4], o[p * 16 + q * 4 + 1],
                                                                                 o[p * 16 + q * 4 + 2], o[p * 16 + q * 4 + 3]);
                                    *reinterpret_cast<uint4*>(dst) = make_uint4(w[0], w[1], w[2], w[3]);
                                } else {
                                    for (int e = p * 16; e < (p + 1) * 16 && e < valid; ++e) yrow[c * 32 + e] = (uint8_t)o[e];
                                }
                            }
                        } else {
#pragma unroll
                            for (int p = 0; p < 4; ++p) {
                                uint8_t* dst = yrow + (c * 32 + p * 8) * 2;
                                if (valid >= (p + 1) * 8 && (((uintptr_t)dst) & 15u) == 0) {
                                    uint32_t w[4];
#pragma unroll
                                    for (int q = 0; q < 4; ++q)
                                        w[q] = ((uint32_t)o[p * 8 + 2 * q] & 0xFFFFu) | ((uint32_t)o[p * 8 + 2 * q + 1] << 16);
                                    *reinterpret_cast<uint4*>(dst) = make_uint4(w[0], w[1], w[2], w[3]);
                                } else {
                                    for (int e = p * 8; e < (p + 1) * 8 && e < valid; ++e)
                                        reinterpret_cast<int16_t*>(yrow)[c * 32 + e] = (int16_t)o[e];
                                }
                            }
                        }
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

bool make_map(CUtensorMap* map, const void* base, long long rows, long long cols, long long ld) {
    EncodeTiledFn fn = get_encode_fn();
    if (!fn) return false;
    cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld};
    cuuint32_t box[2] = {(cuuint32_t)BK, 128u};
    cuuint32_t estr[2] = {1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

std::mutex g_ws_mutex;
uint8_t* g_ws[kMaxDevices] = {nullptr};

// The digit-plane workspace of the current device (allocated on first use, kept until exit).
uint8_t* workspace() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return nullptr;
    std::lock_guard<std::mutex> lock(g_ws_mutex);
    if (g_ws[dev] == nullptr) {
        void* p = nullptr;
        if (cudaMalloc(&p, (size_t)WORKSPACE_BYTES) != cudaSuccess) return nullptr;
        g_ws[dev] = (uint8_t*)p;
    }
    return g_ws[dev];
}

}  // namespace

int a4c_dense_tc16_supported(const void* A, long long lda, const void* Wt, long long ldw, const void* Y, long long ldy,
                             long long M, int K, int N, int out_dtype) {
    if (out_dtype != A4C_I8 && out_dtype != A4C_U8 && out_dtype != A4C_I16) return A4C_ERR_UNSUPPORTED;
    if (K < 16) return A4C_ERR_UNSUPPORTED;
    if (lda % 8 || ldw % 16) return A4C_ERR_ALIGNMENT;                 // 16-byte row pitches of A (int16) and W^T (int8)
    if (((uintptr_t)A | (uintptr_t)Wt) & 15u) return A4C_ERR_ALIGNMENT;
    if (((uintptr_t)Y) & (out_dtype == A4C_I16 ? 1u : 0u)) return A4C_ERR_ALIGNMENT;
    const long long kp = ((long long)K + 15) / 16 * 16;
    if (2 * kp * BM > WORKSPACE_BYTES) return A4C_ERR_TOO_LARGE;        // one row tile of both planes must fit
    if (M > 2147483647LL - BM || lda < K || ldw < K || ldy < N) return A4C_ERR_INVALID_ARG;
    // both digit sums must fit 32 bits: K * 255 * 128 < 2^31
    if ((long long)K * 255 * 128 >= (1ll << 31)) return A4C_ERR_TOO_LARGE;
    return A4C_OK;
}

int a4c_launch_dense_tc16(const int16_t* A, long long lda, const int8_t* Wt, long long ldw, const int32_t* bias, void* Y,
                          long long ldy, long long M, int K, int N, int shift, int rounding, int relu, int out_dtype,
                          int* status_word, cudaStream_t stream) {
    const int sup = a4c_dense_tc16_supported(A, lda, Wt, ldw, Y, ldy, M, K, N, out_dtype);
    if (sup != A4C_OK) return sup;
    if (M == 0) return A4C_OK;
    uint8_t* ws = workspace();
    if (ws == nullptr) return A4C_ERR_CUDA;
    static tc::SmemOptIn opt_in;
    if (opt_in.ensure(dense_tc16_kernel, SMEM_BYTES) != cudaSuccess) return A4C_ERR_CUDA;
    const int kp = (K + 15) / 16 * 16;
    long long chunk = (WORKSPACE_BYTES / 2 / kp) / BM * BM;             // rows per chunk, whole row tiles
    if (chunk > M) chunk = (M + BM - 1) / BM * BM;
    int8_t* hi = reinterpret_cast<int8_t*>(ws);
    uint8_t* lo = ws + chunk * kp;
    CUtensorMap mw;
    if (!make_map(&mw, Wt, N, K, ldw)) return A4C_ERR_CUDA;
    int dev = 0, sms = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const int esz = out_dtype == A4C_I16 ? 2 : 1;
    for (long long r0 = 0; r0 < M; r0 += chunk) {
        const long long rows = M - r0 < chunk ? M - r0 : chunk;
        const long long groups = rows * (kp / 8);
        long long blocks = (groups + 255) / 256;
        if (blocks > (long long)sms * 8) blocks = (long long)sms * 8;
        split_planes_kernel<<<(unsigned)blocks, 256, 0, stream>>>(A + r0 * lda, lda, hi, lo, rows, K, kp);
        CUtensorMap mh, ml;
        if (!make_map(&mh, hi, rows, K, kp) || !make_map(&ml, lo, rows, K, kp)) return A4C_ERR_CUDA;
        Args16 g;
        g.bias = bias; g.Y = (uint8_t*)Y + r0 * ldy * esz; g.ldy = ldy; g.M = rows; g.K = K; g.N = N;
        g.num_m_tiles = (int)((rows + BM - 1) / BM);
        g.num_n_tiles = (N + BN - 1) / BN;
        g.out_dtype = out_dtype;
        dtype_range(out_dtype, g.lo, g.hi);
        if (relu && g.lo < 0) g.lo = 0;
        g.rp = make_round_params(shift, rounding);
        g.status = status_word;
        const long long tiles = (long long)g.num_m_tiles * g.num_n_tiles;
        const int grid = (int)(tiles < sms ? tiles : sms);
        dense_tc16_kernel<<<grid, NUM_THREADS, SMEM_BYTES, stream>>>(mh, ml, mw, g);
        if (cudaGetLastError() != cudaSuccess) return A4C_ERR_CUDA;
    }
    return A4C_OK;
}
