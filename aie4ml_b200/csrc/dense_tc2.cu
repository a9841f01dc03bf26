// int8 Dense on a CTA PAIR (tcgen05 cta_group::2): one 256 x 256 output tile per two SMs.
//
// Same arithmetic as dense_tc.cu (dense_single::run of aie4ml, dense_bias_relu.cpp:67-166).  What changes is
// operand delivery: with one CTA per 128 x 256 tile each SM has to stage 48 KB per 512 tensor-core cycles
// (96 B/clk), more than the SM takes in.  Here the pair shares the W^T tile: CTA r stages its own 128 rows of A
// and HALF of the W^T tile (rows n0 + 128 r .. +128), 32 KB per stage, and the leader's single
// tcgen05.mma.cta_group::2 (M = 256, N = 256, K = 32) reads both halves from both CTAs' shared memory and
// writes 128 accumulator rows into each CTA's TMEM.
//
// Synchronisation (all mbarriers; no multicast anywhere):
//   full[s]        lives in the leader; both CTAs' TMA loads complete_tx on it (the peer through a
//                  shared::cluster address with the cta_group::2 form of the copy); the leader's MMA thread waits
//   empty[s]       one per CTA; the leader commits the stage's MMAs to its own and to the peer's barrier
//   tmem_full[a]   one per CTA, committed the same way when an accumulator is complete
//   tmem_empty[a]  lives in the leader, 256 arrivals: every epilogue thread of both CTAs (the peer's remotely)
// Every wait is bounded as in dense_tc.cu; the two CTAs meet on a cluster barrier before freeing TMEM.
#include <cuda.h>

#include <mutex>

#include "a4c_common.cuh"
#include "a4c_kernels.h"
#include "tc_common.cuh"

using namespace tc;

namespace {

constexpr int BM_CTA = 128;      // rows per CTA
constexpr int BM = 256;          // rows per pair tile
constexpr int BN = 256;
constexpr int BN_CTA = 128;      // W^T rows staged per CTA
constexpr int BK = 128;
constexpr int UMMA_K = 32;
constexpr int STAGES = 6;
constexpr int A_BYTES = BM_CTA * BK;             // 16 KB
constexpr int B_BYTES = BN_CTA * BK;             // 16 KB
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;   // 32 KB per CTA
constexpr int ACC_STAGES = 2;
constexpr int TMEM_COLS = ACC_STAGES * BN;       // 512
constexpr int NUM_THREADS = 192;
constexpr int EPI_THREADS = 128;

struct SmemTail {
    int32_t bias[ACC_STAGES][BN];
    uint64_t full[STAGES];
    uint64_t empty[STAGES];
    uint64_t tmem_full[ACC_STAGES];
    uint64_t tmem_empty[ACC_STAGES];
    uint32_t tmem_base;
    volatile int abort_flag;
};
constexpr size_t SMEM_BYTES = 1024 + (size_t)STAGES * STAGE_BYTES + sizeof(SmemTail);

struct Tc2Args {
    const int32_t* bias;
    uint8_t* Y;
    long long ldy;
    long long M;
    int K, N;
    int num_m_tiles, num_n_tiles;   // in 256 x 256 tiles
    int panel;                      // column tiles per panel of the tile order (>= num_n_tiles: one panel)
    int shift, lo, hi;
    uint32_t mask, c0;
    uint32_t idesc;
    int* status;
};

__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// shared::cluster address of `local` (a shared::cta address) in CTA `rank` of this cluster
__device__ __forceinline__ uint32_t map_to_cta(uint32_t local, uint32_t rank) {
    uint32_t a;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(a) : "r"(local), "r"(rank));
    return a;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" :: "r"(cluster_addr) : "memory");
}
// TMA tile load whose completion may be signalled on the peer CTA's barrier (cta_group::2 form, no multicast)
__device__ __forceinline__ void tma_load_2d_pair(void* dst, const CUtensorMap* map, uint32_t bar_cluster_addr, int c0,
                                                 int c1) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        :: "r"(smem_u32(dst)), "l"(map), "r"(bar_cluster_addr), "r"(c0), "r"(c1) : "memory");
}
__device__ __forceinline__ void umma_i8_pair(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                             uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::i8 [%0], %1, %2, %3, p;\n\t}"
        :: "r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit_pair(uint32_t bar_cluster_addr) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];"
                 :: "r"(bar_cluster_addr) : "memory");
}

// Tile order as in dense_tc.cu: panels of g.panel column tiles (at most 32 MiB of weights, which stay in the L2 while
// the row tiles stream past); inside a panel the column tile runs fastest.
__device__ __forceinline__ void tile_coords(int tile, const Tc2Args& g, int& mt, int& nt) {
    const int nnt = g.num_n_tiles;
    if (g.panel >= nnt) { mt = tile / nnt; nt = tile - mt * nnt; return; }
    const int per_panel = g.num_m_tiles * g.panel;
    const int full = nnt / g.panel;
    int pz = tile / per_panel, rem = tile - pz * per_panel, width = g.panel;
    if (pz >= full) { pz = full; rem = tile - full * per_panel; width = nnt - full * g.panel; }
    mt = rem / width;
    nt = pz * g.panel + (rem - mt * width);
}

template <int MODE>
__device__ __forceinline__ int requant(int acc, const Tc2Args& g) {
    int v = acc;
    if (MODE >= 0) v = round_shift_i32_t<MODE>(acc, g.shift, g.mask, g.c0);
    return min(max(v, g.lo), g.hi);
}

template <int MODE>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(NUM_THREADS, 1)
dense_tc2_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b, Tc2Args g) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    SmemTail* tail = reinterpret_cast<SmemTail*>(smem + (size_t)STAGES * STAGE_BYTES);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();
    const bool leader = rank == 0;
    const int num_tiles = g.num_m_tiles * g.num_n_tiles;
    const int num_kb = (g.K + BK - 1) / BK;
    const int pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(&tail->full[s], 1); mbar_init(&tail->empty[s], 1); }
        for (int s = 0; s < ACC_STAGES; ++s) { mbar_init(&tail->tmem_full[s], 1); mbar_init(&tail->tmem_empty[s], 2 * EPI_THREADS); }
        tail->abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {  // one warp of EACH CTA of the pair performs the paired allocation
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;"
                     :: "r"(smem_u32(&tail->tmem_base)), "r"((uint32_t)TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();   // both CTAs' barriers exist before anything remote touches them
    tc_fence_after();
    const uint32_t tmem_base = tail->tmem_base;
    volatile int* abort_flag = &tail->abort_flag;

    if (warp == 0) {
        // ---------------- TMA producer (both CTAs) ----------------
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int tile = pair; ok && tile < num_tiles; tile += num_pairs) {
                int mt, nt;
                tile_coords(tile, g, mt, nt);
                const int m0 = mt * BM + (int)rank * BM_CTA;
                const int n0 = nt * BN + (int)rank * BN_CTA;
                for (int kb = 0; kb < num_kb; ++kb) {
                    ok = mbar_wait(&tail->empty[stage], phase ^ 1u, abort_flag, g.status, 121);
                    if (!ok) break;
                    uint8_t* sa = smem + (size_t)stage * STAGE_BYTES;
                    const uint32_t full_leader = map_to_cta(smem_u32(&tail->full[stage]), 0);
                    if (leader) mbar_arrive_expect_tx(&tail->full[stage], 2 * STAGE_BYTES);
                    tma_load_2d_pair(sa, &tmap_a, full_leader, kb * BK, m0);
                    tma_load_2d_pair(sa + A_BYTES, &tmap_b, full_leader, kb * BK, n0);
                    if (++stage == STAGES) { stage = 0; phase ^= 1u; }
                }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ---------------- MMA issuer (leader CTA only) ----------------
        if (leader && lane == 0) {
            int stage = 0, acc = 0;
            uint32_t phase = 0, acc_phase = 0;
            bool ok = true;
            for (int tile = pair; ok && tile < num_tiles; tile += num_pairs) {
                ok = mbar_wait(&tail->tmem_empty[acc], acc_phase ^ 1u, abort_flag, g.status, 122);
                if (!ok) break;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + (uint32_t)(acc * BN);
                for (int kb = 0; kb < num_kb; ++kb) {
                    ok = mbar_wait(&tail->full[stage], phase, abort_flag, g.status, 123);
                    if (!ok) break;
                    tc_fence_after();
                    const uint32_t sa = smem_u32(smem + (size_t)stage * STAGE_BYTES);
                    const uint64_t adesc = make_smem_desc(sa);
                    const uint64_t bdesc = make_smem_desc(sa + A_BYTES);
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k)
                        umma_i8_pair(d_tmem, adesc + (uint64_t)(k * (UMMA_K >> 4)), bdesc + (uint64_t)(k * (UMMA_K >> 4)),
                                     g.idesc, (uint32_t)((kb | k) != 0));
                    // release the stage in both CTAs once these MMAs have read it
                    umma_commit_pair(smem_u32(&tail->empty[stage]));
                    umma_commit_pair(map_to_cta(smem_u32(&tail->empty[stage]), 1));
                    if (++stage == STAGES) { stage = 0; phase ^= 1u; }
                }
                if (!ok) break;
                umma_commit_pair(smem_u32(&tail->tmem_full[acc]));
                umma_commit_pair(map_to_cta(smem_u32(&tail->tmem_full[acc]), 1));
                if (++acc == ACC_STAGES) { acc = 0; acc_phase ^= 1u; }
            }
        }
        __syncwarp();
    } else {
        // ---------------- epilogue (warps 2..5 of both CTAs) ----------------
        const int quad = warp & 3;
        const int et = threadIdx.x - 64;
        int acc = 0;
        uint32_t acc_phase = 0;
        bool ok = true;
        for (int tile = pair; tile < num_tiles; tile += num_pairs) {
            int mt, nt;
            tile_coords(tile, g, mt, nt);
            const int m0 = mt * BM + (int)rank * BM_CTA;
            const int n0 = nt * BN;
            for (int i = et; i < BN; i += EPI_THREADS) {
                const int n = n0 + i;
                tail->bias[acc][i] = (g.bias != nullptr && n < g.N) ? __ldg(g.bias + n) : 0;
            }
            asm volatile("bar.sync 1, 128;" ::: "memory");
            if (ok) ok = mbar_wait(&tail->tmem_full[acc], acc_phase, abort_flag, g.status, 124);
            if (ok) {
                tc_fence_after();
                const long long row = (long long)m0 + quad * 32 + lane;
                uint8_t* yrow = g.Y + row * g.ldy + n0;
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
                            const int col = c * 32 + q * 4 + e;
                            o[e] = requant<MODE>((int)(r[q * 4 + e] + (uint32_t)tail->bias[acc][col]), g);
                        }
                        w[q] = (uint32_t)(o[0] & 0xFF) | ((uint32_t)(o[1] & 0xFF) << 8) |
                               ((uint32_t)(o[2] & 0xFF) << 16) | ((uint32_t)o[3] << 24);
                    }
                    if (row < g.M) {
                        const int col0 = n0 + c * 32;
                        if (col0 < g.N) *reinterpret_cast<uint4*>(yrow + c * 32) = make_uint4(w[0], w[1], w[2], w[3]);
                        if (col0 + 16 < g.N)
                            *reinterpret_cast<uint4*>(yrow + c * 32 + 16) = make_uint4(w[4], w[5], w[6], w[7]);
                    }
                }
                tc_fence_before();
                mbar_arrive_cluster(map_to_cta(smem_u32(&tail->tmem_empty[acc]), 0));
            }
            if (++acc == ACC_STAGES) { acc = 0; acc_phase ^= 1u; }
        }
    }

    // ---------------- teardown ----------------
    __syncthreads();
    if (*abort_flag) {
        const uint64_t t0 = a4c_globaltimer();
        while (a4c_globaltimer() - t0 < 2000000ull) __nanosleep(1000);
        __syncthreads();
    }
    tc_fence_before();
    cluster_sync_all();   // neither CTA frees TMEM or leaves while the other may still read its memory
    tc_fence_after();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" :: "r"(tmem_base), "r"((uint32_t)TMEM_COLS) : "memory");
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

bool make_map(CUtensorMap* map, const void* base, long long rows, long long cols, long long ld, int box_rows) {
    EncodeTiledFn fn = get_encode_fn();
    if (!fn) return false;
    cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld};
    cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int MODE>
cudaError_t launch_mode(const CUtensorMap& ma, const CUtensorMap& mb, const Tc2Args& g, int grid, cudaStream_t s) {
    static tc::SmemOptIn opt_in;
    const cudaError_t attr_err = opt_in.ensure(dense_tc2_kernel<MODE>, SMEM_BYTES);
    if (attr_err != cudaSuccess) return attr_err;
    dense_tc2_kernel<MODE><<<grid, NUM_THREADS, SMEM_BYTES, s>>>(ma, mb, g);
    return cudaGetLastError();
}

}  // namespace

int a4c_launch_dense_tc2(const void* A, long long lda, const void* Wt, long long ldw, const int32_t* bias,
                         void* Y, long long ldy, long long M, int K, int N, int shift, int rounding, int relu,
                         int out_dtype, int a_unsigned, int* status_word, cudaStream_t stream) {
    const int sup = a4c_dense_tc_supported(A, lda, Wt, ldw, Y, ldy, M, K, N, out_dtype);
    if (sup != A4C_OK) return sup;
    if (N % 16 != 0) return A4C_ERR_UNSUPPORTED;   // this kernel stores 16-byte pieces of a row directly
    if (M == 0) return A4C_OK;
    CUtensorMap ma, mb;
    if (!make_map(&ma, A, M, K, lda, BM_CTA) || !make_map(&mb, Wt, N, K, ldw, BN_CTA)) return A4C_ERR_CUDA;
    Tc2Args g;
    g.bias = bias; g.Y = (uint8_t*)Y; g.ldy = ldy; g.M = M; g.K = K; g.N = N;
    g.num_m_tiles = (int)((M + BM - 1) / BM);
    g.num_n_tiles = (N + BN - 1) / BN;
    g.shift = shift;
    dtype_range(out_dtype, g.lo, g.hi);
    if (relu && g.lo < 0) g.lo = 0;
    const RoundParams rp = make_round_params(shift, rounding);
    g.mask = rp.mask; g.c0 = rp.c0;
    g.idesc = make_idesc(BM, BN, a_unsigned != 0);
    g.status = status_word;
    {
        const long long tile_bytes = (long long)BN * (((long long)K + BK - 1) / BK * BK);
        const long long panel_bytes = a4c_dense_tc_panel_bytes();   // A4C_OPT_DENSE_PANEL_MIB, default 32 MiB
        long long per = panel_bytes / tile_bytes;
        if (per < 1) per = 1;
        g.panel = panel_bytes <= 0 || per >= g.num_n_tiles ? g.num_n_tiles : (int)per;
    }
    int dev = 0, sms = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const long long tiles = (long long)g.num_m_tiles * g.num_n_tiles;
    long long pairs = sms / 2;
    if (tiles < pairs) pairs = tiles;
    const int grid = (int)pairs * 2;
    cudaError_t err;
    if (shift == 0) err = launch_mode<-1>(ma, mb, g, grid, stream);
    else switch (rounding) {
        case A4C_RND_FLOOR: err = launch_mode<A4C_RND_FLOOR>(ma, mb, g, grid, stream); break;
        case A4C_RND_CEIL: err = launch_mode<A4C_RND_CEIL>(ma, mb, g, grid, stream); break;
        case A4C_RND_POSITIVE_INF: err = launch_mode<A4C_RND_POSITIVE_INF>(ma, mb, g, grid, stream); break;
        case A4C_RND_NEGATIVE_INF: err = launch_mode<A4C_RND_NEGATIVE_INF>(ma, mb, g, grid, stream); break;
        case A4C_RND_SYMMETRIC_INF: err = launch_mode<A4C_RND_SYMMETRIC_INF>(ma, mb, g, grid, stream); break;
        case A4C_RND_SYMMETRIC_ZERO: err = launch_mode<A4C_RND_SYMMETRIC_ZERO>(ma, mb, g, grid, stream); break;
        case A4C_RND_CONV_EVEN: err = launch_mode<A4C_RND_CONV_EVEN>(ma, mb, g, grid, stream); break;
        case A4C_RND_CONV_ODD: err = launch_mode<A4C_RND_CONV_ODD>(ma, mb, g, grid, stream); break;
        default: return A4C_ERR_INVALID_ARG;
    }
    return err == cudaSuccess ? A4C_OK : A4C_ERR_CUDA;
}
