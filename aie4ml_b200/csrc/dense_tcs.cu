// int8 Dense for SHORT reductions (K <= 512) on the sm_100a tensor cores: the epilogue-bound regime.
//
// Same arithmetic as dense_tc.cu (dense_single::run of aie4ml, dense_bias_relu.cpp:67-166).  With K = 256 a
// 128 x 256 output tile costs the tensor pipe ~1000 cycles and the eight epilogue warps of the general kernel
// ~3000 (each warp converts its rows strictly in sequence: TMEM load, requantise, pack, stage, TMA store), so the
// layer runs at the speed of its epilogue.  This kernel keeps the general kernel's tiles and operand traffic
// (128 x 256 tiles, two 256-column accumulators, the CTA's weight tile resident in shared memory, A streamed through
// a deep ring, CTAs c .. c + n_tiles - 1 on the same row tiles) and gives the epilogue half as many warps again:
//   * twelve epilogue warps in three groups of four (one warp per TMEM lane quadrant);
//   * the unit of epilogue work is a HALF tile (128 rows x 128 columns); half tile h = 2 * tile + {0, 1} goes to group
//     h mod 3, so three half tiles are converted at once and consecutive tiles rotate through the groups;
//   * an accumulator returns to the MMA issuer when both groups that share it have its columns in registers; its
//     completion is signalled on barriers of exactly those groups (one set of "accumulator full" barriers per group),
//     because a waiter that skipped a phase of a shared barrier could not tell tile i from tile i + 4 by parity;
//   * 14 warps = at most four per scheduler, so the register ceiling is 128 (sixteen epilogue warps would force 96
//     and spill: measured slower on the general kernel).
// N must be a multiple of 128 here; other widths stay with the general kernel.  Every wait is bounded.
#include <cuda.h>

#include <mutex>

#include "a4c_common.cuh"
#include "a4c_kernels.h"
#include "tc_common.cuh"

namespace {

using namespace tc;

constexpr int BM = 128;
constexpr int BN = 256;
constexpr int HALF_N = 128;                        // columns of one unit of epilogue work
constexpr int BK = 128;
constexpr int UMMA_K = 32;
constexpr int MAX_KB = 4;                          // K <= 512
constexpr int A_BYTES = BM * BK;                   // 16 KB per ring slot
constexpr int W_KB_BYTES = BN * BK;                // 32 KB per k-block of the resident weight tile
constexpr int ACC_STAGES = 2;
constexpr int TMEM_COLS = ACC_STAGES * BN;         // 512
constexpr int EPI_GROUPS = 3;
constexpr int EPI_WARPS = EPI_GROUPS * 4;
constexpr int EPI_GROUP_THREADS = 128;
constexpr int NUM_THREADS = 64 + EPI_WARPS * 32;   // 448
constexpr int MAX_RING = 8;
constexpr int EPI_STAGE_BYTES = 32 * 64;
constexpr int MODE_HALF_UP_CLAMP = 100;            // see dense_tc.cu
constexpr int MODE_HALF_UP_FLOAT = 102;
constexpr int MAGIC_BITS = 0x4B400000;

struct Tail {
    int32_t bias[BN];
    uint64_t full[MAX_RING];
    uint64_t empty[MAX_RING];
    uint64_t w_full;
    uint64_t tmem_full[EPI_GROUPS][ACC_STAGES];   // per group: it sees one phase per tile it has a half of
    uint64_t tmem_empty[ACC_STAGES];
    uint32_t tmem_base;
    volatile int abort_flag;
};
constexpr size_t SMEM_MAX = 227 * 1024;
constexpr size_t FIXED_BYTES = 1024 + (size_t)EPI_WARPS * EPI_STAGE_BYTES + sizeof(Tail);

struct SArgs {
    const int32_t* bias;
    long long M;
    int K, N;
    int num_m_tiles, num_n_tiles, a_stages;
    int shift, lo, hi;
    uint32_t mask, c0;
    int half, xhi, xlo;
    float fmul, fadd;
    uint32_t idesc;
    int* status;
};

template <int MODE>
__device__ __forceinline__ int requant(int acc, int bias, const SArgs& g) {
    if (MODE == MODE_HALF_UP_FLOAT) {
        const int t = __viaddmin_s32(acc, bias, g.xhi);
        const int u = __viaddmax_s32(t, g.half + MAGIC_BITS, g.xlo + MAGIC_BITS);
        return __float_as_int(__fmaf_rd(__int_as_float(u), g.fmul, g.fadd));        // only the low byte is used
    }
    if (MODE == MODE_HALF_UP_CLAMP) {
        const int t = __viaddmin_s32(acc, bias, g.xhi);
        return __viaddmax_s32(t, g.half, g.xlo) >> g.shift;
    }
    int v = acc + bias;
    if (MODE == A4C_RND_FLOOR) v = v >> g.shift;
    else if (MODE >= 0) v = round_shift_i32_t<MODE>(v, g.shift, g.mask, g.c0);
    return min(max(v, g.lo), g.hi);
}

__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, int c0, int c1, const void* src) {
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%1, %2}], [%3];"
                 :: "l"(map), "r"(c0), "r"(c1), "r"(smem_u32(src)) : "memory");
    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}

// 32 rows x 64 accumulator columns (`r`) -> int8 in the warp's staging patch -> TMA store (clips rows >= M and
// columns >= N).
template <int MODE, bool HAS_BIAS>
__device__ __forceinline__ void convert64(const uint32_t* r, const int32_t* bias64, uint8_t* my_stage, int lane, const SArgs& g,
                                          const CUtensorMap* tmap_y, int row0, int col0) {
    if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");   // the previous store has read the patch
    __syncwarp();
    const int sw_w = (lane >> 1) & 3;   // 64-byte swizzle: 16-byte piece p of row l sits at piece p ^ ((l >> 1) & 3)
#pragma unroll
    for (int piece = 0; piece < 4; ++piece) {
        int4 b[4];
#pragma unroll
        for (int q = 0; q < 4; ++q)
            b[q] = HAS_BIAS ? *reinterpret_cast<const int4*>(bias64 + piece * 16 + q * 4) : make_int4(0, 0, 0, 0);
        uint32_t w[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const uint32_t* a = r + piece * 16 + q * 4;
            w[q] = pack4_i8(requant<MODE>((int)a[0], b[q].x, g), requant<MODE>((int)a[1], b[q].y, g),
                            requant<MODE>((int)a[2], b[q].z, g), requant<MODE>((int)a[3], b[q].w, g));
        }
        *reinterpret_cast<uint4*>(my_stage + lane * 64 + ((piece ^ sw_w) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    __syncwarp();
    if (lane == 0) tma_store_2d(tmap_y, col0, row0, my_stage);
}

template <int MODE, bool HAS_BIAS>
__global__ void __maxnreg__(128)      // 14 warps: four share one scheduler's 16384 registers
dense_tcs_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                 const __grid_constant__ CUtensorMap tmap_y, SArgs g) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    const int num_kb = (g.K + BK - 1) / BK;
    uint8_t* a_ring = smem + (size_t)num_kb * W_KB_BYTES;                       // after the resident weight tile
    uint8_t* epi_stage = a_ring + (size_t)g.a_stages * A_BYTES;                 // 1024-byte aligned
    Tail* tail = reinterpret_cast<Tail*>(epi_stage + (size_t)EPI_WARPS * EPI_STAGE_BYTES);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int nnt = g.num_n_tiles, per = (int)gridDim.x / nnt;
    const int nt = (int)blockIdx.x % nnt, mt0 = (int)blockIdx.x / nnt;
    const int my_tiles = mt0 < g.num_m_tiles ? (g.num_m_tiles - mt0 + per - 1) / per : 0;
    // columns this CTA's tile really has (the last column tile of an odd multiple of 128 has one half)
    const int my_cols = min(BN, g.N - nt * BN);
    const int my_halves = my_cols / HALF_N;

    if (threadIdx.x == 0) {
        for (int s = 0; s < MAX_RING; ++s) { mbar_init(&tail->full[s], 1); mbar_init(&tail->empty[s], 1); }
        mbar_init(&tail->w_full, 1);
        for (int s = 0; s < ACC_STAGES; ++s) {
            for (int e = 0; e < EPI_GROUPS; ++e) mbar_init(&tail->tmem_full[e][s], 1);
            mbar_init(&tail->tmem_empty[s], (uint32_t)(my_halves * EPI_GROUP_THREADS));
        }
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
        // ---------------- TMA producer ----------------
        if (lane == 0 && my_tiles > 0) {
            mbar_arrive_expect_tx(&tail->w_full, (uint32_t)(num_kb * my_cols * BK));
            for (int kb = 0; kb < num_kb; ++kb) {
                // the weight box is 128 rows: one or two loads per k-block (the second half 16 KB further)
                for (int h = 0; h < my_halves; ++h)
                    tma_load_2d(smem + (size_t)kb * W_KB_BYTES + (size_t)h * (HALF_N * BK), &tmap_b, &tail->w_full, kb * BK,
                                nt * BN + h * HALF_N);
            }
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int i = 0; ok && i < my_tiles; ++i) {
                const int m0 = (mt0 + i * per) * BM;
                for (int kb = 0; kb < num_kb; ++kb) {
                    ok = mbar_wait(&tail->empty[stage], phase ^ 1u, abort_flag, g.status, 161);
                    if (!ok) break;
                    mbar_arrive_expect_tx(&tail->full[stage], (uint32_t)A_BYTES);
                    tma_load_2d(a_ring + (size_t)stage * A_BYTES, &tmap_a, &tail->full[stage], kb * BK, m0);
                    if (++stage == g.a_stages) { stage = 0; phase ^= 1u; }
                }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0 && my_tiles > 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = mbar_wait(&tail->w_full, 0u, abort_flag, g.status, 165);
            tc_fence_after();
            const uint32_t w_base = smem_u32(smem), ring_base = smem_u32(a_ring);
            const uint32_t idesc = my_halves == 2 ? g.idesc : make_idesc(BM, HALF_N, (g.idesc & (1u << 7)) == 0);
            for (int i = 0; ok && i < my_tiles; ++i) {
                const int acc = i & 1;
                // epilogue-bound kernel: the issuer mostly waits here, so it sleeps in the barrier instead of polling (a
                // polling issuer takes issue slots from the epilogue warps of its scheduler)
                ok = mbar_wait(&tail->tmem_empty[acc], ((uint32_t)(i >> 1) & 1u) ^ 1u, abort_flag, g.status, 162);
                if (!ok) break;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + (uint32_t)(acc * BN);
                for (int kb = 0; kb < num_kb; ++kb) {
                    ok = mbar_wait_fast(&tail->full[stage], phase, abort_flag, g.status, 163);
                    if (!ok) break;
                    tc_fence_after();
                    const uint64_t adesc = make_smem_desc(ring_base + (uint32_t)stage * A_BYTES);
                    const uint64_t bdesc = make_smem_desc(w_base + (uint32_t)(kb * W_KB_BYTES));
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k)
                        umma_i8(d_tmem, adesc + (uint64_t)(k * (UMMA_K >> 4)), bdesc + (uint64_t)(k * (UMMA_K >> 4)), idesc,
                                (uint32_t)((kb | k) != 0));
                    umma_commit(&tail->empty[stage]);
                    if (++stage == g.a_stages) { stage = 0; phase ^= 1u; }
                }
                if (!ok) break;
                // accumulator complete: tell the group of each of its half tiles
                for (int half = 0; half < my_halves; ++half)
                    umma_commit(&tail->tmem_full[(i * my_halves + half) % EPI_GROUPS][acc]);
            }
        }
        __syncwarp();
    } else {
        // ---------------- epilogue: three groups of four warps; half tile h = my_halves * tile + half -> group h % 3 ----------
        const int quad = warp & 3;
        const int grp = (warp - 2) >> 2;
        uint8_t* my_stage = epi_stage + (size_t)(warp - 2) * EPI_STAGE_BYTES;
        bool ok = true;
        if (HAS_BIAS) {
            // this CTA's bias values once (its column tile never changes)
            for (int i = threadIdx.x - 64; i < BN; i += EPI_WARPS * 32) {
                const int n = nt * BN + i;
                tail->bias[i] = n < g.N ? __ldg(g.bias + n) : 0;
            }
            asm volatile("bar.sync 1, %0;" :: "n"(EPI_WARPS * 32) : "memory");
        }
        const int total_halves = my_tiles * my_halves;
        uint32_t full_phases = 0u;   // bit a: parity of this group's next phase on its barrier of accumulator a
        for (int h = grp; h < total_halves; h += EPI_GROUPS) {
            const int i = h / my_halves, half = h - i * my_halves;
            const int acc = i & 1;
            if (ok) ok = mbar_wait(&tail->tmem_full[grp][acc], (full_phases >> acc) & 1u, abort_flag, g.status, 164);
            full_phases ^= 1u << acc;
            if (!ok) continue;
            tc_fence_after();
            const int row_base = (mt0 + i * per) * BM + quad * 32;
            const uint32_t taddr = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(acc * BN + half * HALF_N);
            uint32_t ra[64];
#pragma unroll 1
            for (int c = 0; c < HALF_N / 64; ++c) {
                tmem_ld32_async(taddr + (uint32_t)(c * 64), ra);
                tmem_ld32_async(taddr + (uint32_t)(c * 64 + 32), ra + 32);
                tmem_ld_wait32(ra);
                tmem_ld_wait32(ra + 32);
                if (c == HALF_N / 64 - 1) {     // this half's last columns are in registers
                    tc_fence_before();
                    mbar_arrive(&tail->tmem_empty[acc]);
                }
                convert64<MODE, HAS_BIAS>(ra, tail->bias + half * HALF_N + c * 64, my_stage, lane, g, &tmap_y, row_base,
                                          nt * BN + half * HALF_N + c * 64);
            }
        }
        if (lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");   // stores complete before the CTA retires
        __syncwarp();
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

bool make_map(CUtensorMap* map, const void* base, long long rows, long long cols, long long ld, int box_cols, int box_rows,
              CUtensorMapSwizzle swz, CUtensorMapL2promotion promo) {
    EncodeTiledFn fn = get_encode_fn();
    if (!fn) return false;
    cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld};
    cuuint32_t box[2] = {(cuuint32_t)box_cols, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr,
              CU_TENSOR_MAP_INTERLEAVE_NONE, swz, promo, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int MODE>
cudaError_t launch_mode(const CUtensorMap& ma, const CUtensorMap& mb, const CUtensorMap& my, const SArgs& g, int grid,
                        size_t smem, cudaStream_t s) {
    static tc::SmemOptIn opt_in[2];
    if (g.bias != nullptr) {
        const cudaError_t e = opt_in[1].ensure(dense_tcs_kernel<MODE, true>, SMEM_MAX);
        if (e != cudaSuccess) return e;
        dense_tcs_kernel<MODE, true><<<grid, NUM_THREADS, smem, s>>>(ma, mb, my, g);
    } else {
        const cudaError_t e = opt_in[0].ensure(dense_tcs_kernel<MODE, false>, SMEM_MAX);
        if (e != cudaSuccess) return e;
        dense_tcs_kernel<MODE, false><<<grid, NUM_THREADS, smem, s>>>(ma, mb, my, g);
    }
    return cudaGetLastError();
}

}  // namespace

// 0 when this kernel takes the problem (the caller has already checked the general kernel's alignment rules).
int a4c_dense_tcs_supported(long long M, int K, int N, int out_dtype, int sms) {
    if (out_dtype != A4C_I8 && out_dtype != A4C_U8) return A4C_ERR_UNSUPPORTED;
    if (K < 16 || K > MAX_KB * BK || N % HALF_N != 0) return A4C_ERR_UNSUPPORTED;
    const int nnt = (N + BN - 1) / BN;
    const int per = sms / nnt;
    const long long m_tiles = (M + BM - 1) / BM;
    if (nnt > 16 || per < 1 || m_tiles < 4LL * per) return A4C_ERR_UNSUPPORTED;   // every CTA gets several row tiles
    return A4C_OK;
}

int a4c_launch_dense_tcs(const void* A, long long lda, const void* Wt, long long ldw, const int32_t* bias, void* Y,
                         long long ldy, long long M, int K, int N, int shift, int rounding, int relu, int out_dtype,
                         int a_unsigned, int* status_word, cudaStream_t stream) {
    int dev = 0, sms = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const int sup = a4c_dense_tcs_supported(M, K, N, out_dtype, sms);
    if (sup != A4C_OK) return sup;
    CUtensorMap ma, mb, my;
    if (!make_map(&ma, A, M, K, lda, BK, BM, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B) ||
        !make_map(&mb, Wt, N, K, ldw, BK, HALF_N, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B) ||
        !make_map(&my, Y, M, N, ldy, 64, 32, CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_NONE))
        return A4C_ERR_CUDA;
    SArgs g;
    g.bias = bias; g.M = M; g.K = K; g.N = N;
    g.num_m_tiles = (int)((M + BM - 1) / BM);
    g.num_n_tiles = (N + BN - 1) / BN;
    g.shift = shift;
    dtype_range(out_dtype, g.lo, g.hi);
    if (relu && g.lo < 0) g.lo = 0;
    const RoundParams rp = make_round_params(shift, rounding);
    g.mask = rp.mask; g.c0 = rp.c0;
    const bool pre_clamp = shift >= 1 && shift <= 22;
    g.half = pre_clamp ? (1 << (shift - 1)) : 0;
    g.xhi = pre_clamp ? g.hi * (1 << shift) : 0;
    g.xlo = pre_clamp ? g.lo * (1 << shift) + g.half : 0;
    g.fmul = pre_clamp ? 1.0f / (float)(1 << shift) : 0.0f;
    g.fadd = 12582912.0f - 12582912.0f * g.fmul;
    g.idesc = make_idesc(BM, BN, a_unsigned != 0);
    g.status = status_word;
    const int num_kb = (K + BK - 1) / BK;
    const int slots = (int)((SMEM_MAX - FIXED_BYTES - (size_t)num_kb * W_KB_BYTES) / A_BYTES);
    g.a_stages = slots < MAX_RING ? slots : MAX_RING;
    if (g.a_stages < 2) return A4C_ERR_UNSUPPORTED;
    const size_t smem = FIXED_BYTES + (size_t)num_kb * W_KB_BYTES + (size_t)g.a_stages * A_BYTES;
    const int grid = (sms / g.num_n_tiles) * g.num_n_tiles;
    cudaError_t err;
    if (shift == 0) err = launch_mode<-1>(ma, mb, my, g, grid, smem, stream);
    else switch (rounding) {
        case A4C_RND_FLOOR: err = launch_mode<A4C_RND_FLOOR>(ma, mb, my, g, grid, smem, stream); break;
        case A4C_RND_CEIL: err = launch_mode<A4C_RND_CEIL>(ma, mb, my, g, grid, smem, stream); break;
        case A4C_RND_POSITIVE_INF:
            err = !pre_clamp ? launch_mode<A4C_RND_POSITIVE_INF>(ma, mb, my, g, grid, smem, stream)
                  : shift <= 13 ? launch_mode<MODE_HALF_UP_FLOAT>(ma, mb, my, g, grid, smem, stream)
                                : launch_mode<MODE_HALF_UP_CLAMP>(ma, mb, my, g, grid, smem, stream);
            break;
        case A4C_RND_NEGATIVE_INF: err = launch_mode<A4C_RND_NEGATIVE_INF>(ma, mb, my, g, grid, smem, stream); break;
        case A4C_RND_SYMMETRIC_INF: err = launch_mode<A4C_RND_SYMMETRIC_INF>(ma, mb, my, g, grid, smem, stream); break;
        case A4C_RND_SYMMETRIC_ZERO: err = launch_mode<A4C_RND_SYMMETRIC_ZERO>(ma, mb, my, g, grid, smem, stream); break;
        case A4C_RND_CONV_EVEN: err = launch_mode<A4C_RND_CONV_EVEN>(ma, mb, my, g, grid, smem, stream); break;
        case A4C_RND_CONV_ODD: err = launch_mode<A4C_RND_CONV_ODD>(ma, mb, my, g, grid, smem, stream); break;
        default: return A4C_ERR_INVALID_ARG;
    }
    return err == cudaSuccess ? A4C_OK : A4C_ERR_CUDA;
}
