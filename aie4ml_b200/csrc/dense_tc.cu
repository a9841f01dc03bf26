// int8 x int8 -> int32 Dense on the sm_100a tensor cores.
//
//   Y[m,n] = clamp(round_shift(sum_k A[m,k]*W[k,n] + bias[n], shift), lo, hi)      (lo = max(lo,0) with ReLU)
//
// which is dense_single::run of aie4ml (dense_bias_relu.cpp:67-166): int32 accumulation, bias as
// the accumulator's initial value, SRS (rounding shift + saturation), ReLU after the saturation.
//
// Structure (one persistent CTA per SM, 320 threads, warp-specialised):
//   warp 0     TMA producer: A tile [128 x 128B] and W^T tile [up to 256 x 128B] per stage, 128-byte swizzle,
//              4-stage shared-memory ring, mbarrier expect-tx completion
//   warp 1     MMA issuer: one elected lane issues tcgen05.mma.kind::i8 (M=128, N<=256, K=32), four per
//              stage; tcgen05.commit releases the stage; accumulators live in TMEM, two of them
//              (2 x 256 columns) so the epilogue of tile i overlaps the main loop of tile i+1
//   warps 2-9  epilogue, two groups of four warps on alternate tiles (group g owns accumulator g): tcgen05.ld
//              of 64 columns at a time (lane = row), bias from a resident shared-memory copy, requantise, pack
//              four int8 per word into the warp's swizzled 32 x 64-byte staging patch, TMA store; the accumulator
//              goes back to the issuer once its last 64 columns are in registers
// Tile order: normally CTA c takes global tiles c, c + grid, ... (column tile fastest) and every stage carries an
// A tile and a W tile.  When the weights are larger than what the L2 keeps (a B200 L2 holds about 60 MB of data that
// every SM reads: 64 MiB of weights at K = N = 8192 were fetched from HBM some 80 times per launch, 6.4 GB of reads for
// 1.1 GB of operands), the column tiles are walked in PANELS of at most 32 MiB of weights: all row tiles of one
// panel, then the next panel.  A panel stays in the L2 while the rows stream past it; A is then read once per panel.  For K <= 512 with enough row tiles, a CTA instead keeps the whole K extent of ONE weight
// tile resident in shared memory (loaded once) and the ring holds A tiles only, up to eight of them, so several
// row tiles are in flight from HBM while one is multiplied; CTAs c .. c + n_tiles - 1 walk the same row tiles, so
// A reaches HBM once and L2 serves the other column tiles (4-10 % faster than the streaming order at K <= 512).
// Every wait is bounded: when a wait gives up, the CTA records a code in the status word, stops
// issuing work, lets what is in flight land, frees its TMEM and returns.
#include <cuda.h>

#include <mutex>

#include "a4c_common.cuh"
#include "a4c_kernels.h"
#include "tc_common.cuh"

namespace {

constexpr int BM = 128;          // rows of A per CTA tile
constexpr int BN = 256;          // output features per tile (UMMA N)
constexpr int BK = 128;          // K bytes per stage = one 128-byte swizzle row
constexpr int UMMA_K = 32;       // K per tcgen05.mma for 8-bit operands
constexpr int STAGES = 4;
constexpr int A_BYTES = BM * BK;                 // 16 KB
constexpr int B_BYTES = BN * BK;                 // 32 KB
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;   // 48 KB
constexpr int ACC_STAGES = 2;
constexpr int TMEM_COLS = ACC_STAGES * BN;       // 512
constexpr int EPI_WARPS = 8;           // two warps per TMEM lane quadrant, each takes half of the tile's columns
constexpr int EPI_THREADS = EPI_WARPS * 32;
constexpr int EPI_GROUP_THREADS = EPI_THREADS / 2;   // one group per accumulator
constexpr int NUM_THREADS = 64 + EPI_THREADS;
// positive_inf with 1 <= shift <= 22: saturate BEFORE the shift (rounding is monotonic, and lo*2^s / hi*2^s
// round to lo / hi exactly), which makes the rounding add overflow-free and folds bias add, both clamps
// and the rounding add into two add-min/max instructions plus the shift.
constexpr int MODE_HALF_UP_CLAMP = 100;
// The same for shift <= 13, with the shift moved off the integer pipe (which bounds this epilogue: it retires
// half a warp per clock): the clamped value n = x + 2^(s-1), |n| < 2^22, is produced directly as the bit pattern
// of the float 1.5*2^23 + n, and one round-down FMA by 2^-s leaves floor(n / 2^s) in the low mantissa bits.
constexpr int MODE_HALF_UP_FLOAT = 102;
constexpr int MAGIC_BITS = 0x4B400000;   // 1.5 * 2^23

constexpr int BIAS_CACHE = 2048;   // whole bias vector resident in shared memory when N fits

constexpr int MAX_RING = 8;        // ring slots: 4 of (A + W) normally, up to 8 of A alone when W stays resident

struct SmemTail {
    int32_t bias[BIAS_CACHE];       // N <= BIAS_CACHE: bias[n]; else two per-tile slices of BN at [0] and [BN]
    uint64_t full[MAX_RING];
    uint64_t empty[MAX_RING];
    uint64_t w_full;                // resident-W mode: the CTA's weight tile has landed
    uint64_t tmem_full[ACC_STAGES];
    uint64_t tmem_empty[ACC_STAGES];
    uint32_t tmem_base;
    volatile int abort_flag;
};
// Output staging: each epilogue warp owns a 32-row x 64-byte patch (64-byte swizzle) that a TMA store
// moves to global memory, so the warps that convert accumulators never wait on the store path.
constexpr int EPI_STAGE_BYTES = 32 * 64;
constexpr size_t SMEM_BYTES = 1024 /*alignment slack*/ + (size_t)STAGES * STAGE_BYTES +
                              (size_t)EPI_WARPS * EPI_STAGE_BYTES + sizeof(SmemTail);

using namespace tc;

int g_dense_resident_w = 2;   // A4C_OPT_DENSE_RESIDENT_W: 0 off, 1 resident weight tile in this kernel, 2 = 1 plus the
                              // short-reduction kernel (dense_tcs.cu, twelve epilogue warps) where it applies
long long g_dense_panel_bytes = 32ll << 20;   // weights per panel of the streaming order; 0 = one panel (A4C_OPT_DENSE_PANEL_MIB)

struct TcArgs {
    const int32_t* bias;
    uint8_t* Y;
    long long ldy;
    long long M;
    int K, N;
    int n_full;          // N rounded down to whole 16-byte pieces of an output row
    int b_box_rows;      // weight rows one TMA box brings in: 256, or N rounded up to 16 for a single narrow tile
    // Resident-W mode (small K): a CTA keeps the whole K extent of ONE weight tile in shared memory and streams
    // only A tiles through a deeper ring, so the HBM latency of an A tile is covered by several tiles of work.
    // CTA c then owns output-column tile c % num_n_tiles and row tiles c / num_n_tiles + i * (grid / num_n_tiles).
    int w_resident, a_stages;
    int num_m_tiles, num_n_tiles;
    int panel;           // column tiles per panel of the streaming tile order (>= num_n_tiles: a single panel)
    int shift, lo, hi;
    uint32_t mask, c0;   // rounding constants (see round_shift_i32_t)
    int half, xhi, xlo;  // MODE_HALF_UP_CLAMP / _FLOAT: 2^(s-1), hi * 2^s, lo * 2^s + 2^(s-1)
    float fmul, fadd;    // MODE_HALF_UP_FLOAT: 2^-s and 1.5*2^23 * (1 - 2^-s)
    uint32_t idesc;
    int* status;
};

template <int MODE>
__device__ __forceinline__ int requant(int acc, int bias, const TcArgs& g) {
    if (MODE == MODE_HALF_UP_FLOAT) {
        const int t = __viaddmin_s32(acc, bias, g.xhi);
        const int u = __viaddmax_s32(t, g.half + MAGIC_BITS, g.xlo + MAGIC_BITS);   // bits of 1.5*2^23 + x + 2^(s-1)
        return __float_as_int(__fmaf_rd(__int_as_float(u), g.fmul, g.fadd));        // only the low byte is used
    }
    if (MODE == MODE_HALF_UP_CLAMP) {
        const int t = __viaddmin_s32(acc, bias, g.xhi);          // min(wrap32(acc + bias), hi * 2^s)
        return __viaddmax_s32(t, g.half, g.xlo) >> g.shift;      // max(t + 2^(s-1), lo * 2^s + 2^(s-1)) >> s
    }
    int v = acc + bias;
    if (MODE == A4C_RND_FLOOR) v = v >> g.shift;
    else if (MODE >= 0) v = round_shift_i32_t<MODE>(v, g.shift, g.mask, g.c0);
    return min(max(v, g.lo), g.hi);
}

// Streaming tile order: global tile index -> (row tile, column tile).  Panels of g.panel column tiles (the last one
// may be narrower); inside a panel the column tile runs fastest.
__device__ __forceinline__ void tile_coords(int tile, const TcArgs& g, int& mt, int& nt) {
    const int nnt = g.num_n_tiles;
    if (g.panel >= nnt) { mt = tile / nnt; nt = tile - mt * nnt; return; }
    const int per_panel = g.num_m_tiles * g.panel;
    const int full = nnt / g.panel;
    int pz = tile / per_panel, rem = tile - pz * per_panel, width = g.panel;
    if (pz >= full) { pz = full; rem = tile - full * per_panel; width = nnt - full * g.panel; }
    mt = rem / width;
    nt = pz * g.panel + (rem - mt * width);
}

__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, int c0, int c1, const void* src) {
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%1, %2}], [%3];"
                 :: "l"(map), "r"(c0), "r"(c1), "r"(smem_u32(src)) : "memory");
    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}

// One epilogue warp turns 32 rows x 64 accumulator columns (two TMEM loads, `r`) into int8 in its shared-memory
// patch and hands the patch to a TMA store (which clips rows >= M and columns >= N).
template <int MODE, bool HAS_BIAS>
__device__ __forceinline__ void epilogue_pair(const uint32_t* r, const int32_t* bias64, uint8_t* my_stage, int lane,
                                              const TcArgs& g, const CUtensorMap* tmap_y, int row0, int col0) {
    // the previous store out of this patch must have read it before it is overwritten
    if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
    __syncwarp();
    const int sw_w = (lane >> 1) & 3;   // 64-byte swizzle: 16-byte piece p of row l sits at piece p ^ ((l >> 1) & 3)
    // the 64 bias values are the same for every lane (a lane is a row): broadcast loads, issued one 16-column
    // piece ahead of their use so that their latency hides under the previous piece's arithmetic.  A layer without
    // a bias (HAS_BIAS false) issues none of them: shared-memory reads queue behind the operand fetch of the MMAs,
    // and with the tensor pipe busy these loads alone doubled the time of a group.
    int4 bnext[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) bnext[q] = HAS_BIAS ? *reinterpret_cast<const int4*>(bias64 + q * 4) : make_int4(0, 0, 0, 0);
#pragma unroll
    for (int piece = 0; piece < 4; ++piece) {
        int4 b[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) b[q] = bnext[q];
        if (HAS_BIAS && piece < 3) {
#pragma unroll
            for (int q = 0; q < 4; ++q) bnext[q] = *reinterpret_cast<const int4*>(bias64 + (piece + 1) * 16 + q * 4);
        }
        uint32_t w[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const uint32_t* a = r + piece * 16 + q * 4;
            w[q] = pack4_i8(requant<MODE>((int)a[0], b[q].x, g), requant<MODE>((int)a[1], b[q].y, g),
                            requant<MODE>((int)a[2], b[q].z, g), requant<MODE>((int)a[3], b[q].w, g));
        }
        *reinterpret_cast<uint4*>(my_stage + lane * 64 + ((piece ^ sw_w) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // generic-proxy writes -> TMA read
    __syncwarp();
    // The tensor map ends at the last whole 16-byte piece of a row (n_full columns): a TMA store writes whole
    // pieces, and the bytes between N and the row pitch may belong to a neighbouring view.
    if (lane == 0 && col0 < g.n_full) tma_store_2d(tmap_y, col0, row0, my_stage);
    if (g.N > g.n_full && col0 <= g.n_full && g.n_full < col0 + 64) {
        // the ragged last piece: each lane copies the valid bytes of its own row
        const int piece = (g.n_full - col0) >> 4;
        const uint4 v = *reinterpret_cast<const uint4*>(my_stage + lane * 64 + ((piece ^ sw_w) << 4));
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
        const long long row = (long long)row0 + lane;
        if (row < g.M) {
            uint8_t* dst = g.Y + row * g.ldy + g.n_full;
            for (int b = 0; b < g.N - g.n_full; ++b) dst[b] = (uint8_t)(w[b >> 2] >> (8 * (b & 3)));
        }
    }
}

// MODE = rounding token, or -1 when shift == 0 (no rounding step).  HAS_BIAS = the layer has a bias vector.
template <int MODE, bool HAS_BIAS>
__global__ void __launch_bounds__(NUM_THREADS, 1)
dense_tc_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                const __grid_constant__ CUtensorMap tmap_y, TcArgs g) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* epi_stage = smem + (size_t)STAGES * STAGE_BYTES;   // 1024-byte aligned: whole swizzle atoms
    SmemTail* tail = reinterpret_cast<SmemTail*>(epi_stage + (size_t)EPI_WARPS * EPI_STAGE_BYTES);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int num_tiles = g.num_m_tiles * g.num_n_tiles;
    const int num_kb = (g.K + BK - 1) / BK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < MAX_RING; ++s) { mbar_init(&tail->full[s], 1); mbar_init(&tail->empty[s], 1); }
        mbar_init(&tail->w_full, 1);
        for (int s = 0; s < ACC_STAGES; ++s) { mbar_init(&tail->tmem_full[s], 1); mbar_init(&tail->tmem_empty[s], EPI_GROUP_THREADS); }
        tail->abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {  // whole warp: allocate all 512 TMEM columns, publish the base address
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
        if (lane == 0 && g.w_resident) {
            const int nnt = g.num_n_tiles, per = (int)gridDim.x / nnt;
            const int n0 = ((int)blockIdx.x % nnt) * BN;
            uint8_t* a_ring = smem + (size_t)num_kb * B_BYTES;
            mbar_arrive_expect_tx(&tail->w_full, (uint32_t)(num_kb * g.b_box_rows * BK));
            for (int kb = 0; kb < num_kb; ++kb) tma_load_2d(smem + (size_t)kb * B_BYTES, &tmap_b, &tail->w_full, kb * BK, n0);
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int mt = (int)blockIdx.x / nnt; ok && mt < g.num_m_tiles; mt += per) {
                for (int kb = 0; kb < num_kb; ++kb) {
                    ok = mbar_wait(&tail->empty[stage], phase ^ 1u, abort_flag, g.status, 101);
                    if (!ok) break;
                    mbar_arrive_expect_tx(&tail->full[stage], (uint32_t)A_BYTES);
                    tma_load_2d(a_ring + (size_t)stage * A_BYTES, &tmap_a, &tail->full[stage], kb * BK, mt * BM);
                    if (++stage == g.a_stages) { stage = 0; phase ^= 1u; }
                }
            }
        } else if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x) {
                int mt, nt;
                tile_coords(tile, g, mt, nt);
                const int m0 = mt * BM, n0 = nt * BN;
                for (int kb = 0; kb < num_kb; ++kb) {
                    ok = mbar_wait(&tail->empty[stage], phase ^ 1u, abort_flag, g.status, 101);
                    if (!ok) break;
                    uint8_t* sa = smem + (size_t)stage * STAGE_BYTES;
                    mbar_arrive_expect_tx(&tail->full[stage], (uint32_t)(A_BYTES + g.b_box_rows * BK));
                    tma_load_2d(sa, &tmap_a, &tail->full[stage], kb * BK, m0);
                    tma_load_2d(sa + A_BYTES, &tmap_b, &tail->full[stage], kb * BK, n0);
                    if (++stage == STAGES) { stage = 0; phase ^= 1u; }
                }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            int stage = 0, acc = 0;
            uint32_t phase = 0, acc_phase = 0;
            bool ok = true;
            const int ring = g.w_resident ? g.a_stages : STAGES;
            const uint32_t a_ring = smem_u32(smem) + (g.w_resident ? (uint32_t)(num_kb * B_BYTES) : 0u);
            const uint32_t slot_bytes = g.w_resident ? (uint32_t)A_BYTES : (uint32_t)STAGE_BYTES;
            // local tile count of this CTA under either tile order
            const int nnt = g.num_n_tiles, per = g.w_resident ? (int)gridDim.x / nnt : 1;
            const int my_tiles = g.w_resident
                                     ? ((int)blockIdx.x / nnt < g.num_m_tiles ? (g.num_m_tiles - (int)blockIdx.x / nnt + per - 1) / per : 0)
                                     : ((int)blockIdx.x < num_tiles ? (num_tiles - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x : 0);
            if (g.w_resident && my_tiles > 0) {
                ok = mbar_wait(&tail->w_full, 0u, abort_flag, g.status, 105);
                tc_fence_after();
            }
            for (int i = 0; ok && i < my_tiles; ++i) {
                ok = mbar_wait_spin(&tail->tmem_empty[acc], acc_phase ^ 1u, abort_flag, g.status, 102);
                if (!ok) break;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + (uint32_t)(acc * BN);
                for (int kb = 0; kb < num_kb; ++kb) {
                    ok = mbar_wait(&tail->full[stage], phase, abort_flag, g.status, 103);
                    if (!ok) break;
                    tc_fence_after();
                    const uint32_t sa = a_ring + (uint32_t)stage * slot_bytes;
                    const uint64_t adesc = make_smem_desc(sa);
                    const uint64_t bdesc = make_smem_desc(g.w_resident ? smem_u32(smem) + (uint32_t)(kb * B_BYTES) : sa + A_BYTES);
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k) {
                        // advancing K inside the swizzle row: +32 bytes = +2 in the (address >> 4) field
                        umma_i8(d_tmem, adesc + (uint64_t)(k * (UMMA_K >> 4)), bdesc + (uint64_t)(k * (UMMA_K >> 4)),
                                g.idesc, (uint32_t)((kb | k) != 0));
                    }
                    umma_commit(&tail->empty[stage]);  // slot reusable once these MMAs have read it
                    if (++stage == ring) { stage = 0; phase ^= 1u; }
                }
                if (!ok) break;
                umma_commit(&tail->tmem_full[acc]);  // accumulator complete
                if (++acc == ACC_STAGES) { acc = 0; acc_phase ^= 1u; }
            }
        }
        __syncwarp();
    } else {
        // ---------------- epilogue: two groups of four warps on alternate tiles ----------------
        // Group 0 (warps 2-5) converts even tiles out of accumulator 0, group 1 (warps 6-9) odd tiles out of
        // accumulator 1.  The two warps that share an SM sub-partition are therefore in different phases:
        // one waits for its accumulator or for a TMEM load while the other keeps the integer pipe busy.
        const int quad = warp & 3;           // TMEM lane quadrant this warp may read
        const int grp = (warp - 2) >> 2;     // which accumulator / which tiles
        const int gt = threadIdx.x - 64 - grp * EPI_GROUP_THREADS;   // 0..127 inside the group
        uint8_t* my_stage = epi_stage + (size_t)(warp - 2) * EPI_STAGE_BYTES;
        uint32_t acc_phase = 0;
        bool ok = true;
        const bool bias_resident = HAS_BIAS && g.num_n_tiles * BN <= BIAS_CACHE;
        if (bias_resident) {
            // the whole (zero-padded) bias vector once: no global load on any tile's critical path
            for (int i = threadIdx.x - 64; i < g.num_n_tiles * BN; i += EPI_THREADS)
                tail->bias[i] = (g.bias != nullptr && i < g.N) ? __ldg(g.bias + i) : 0;
            asm volatile("bar.sync 1, 256;" ::: "memory");
        }
        // This group's tiles are the CTA's local tiles grp, grp + 2, ...
        // Streaming order: local tile i is global tile blockIdx.x + i * gridDim.x (see tile_coords).
        // Resident-W order: column tile fixed, row tile blockIdx.x / nnt + i * (gridDim.x / nnt).
        const int nnt = g.num_n_tiles;
        const int step = g.w_resident ? 2 * ((int)gridDim.x / nnt) : 2 * (int)gridDim.x;
        int cursor = g.w_resident ? (int)blockIdx.x / nnt + grp * ((int)gridDim.x / nnt) : (int)blockIdx.x + grp * (int)gridDim.x;
        const int limit = g.w_resident ? g.num_m_tiles : num_tiles;
        const uint32_t taddr = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(grp * BN);
        for (; cursor < limit; cursor += step) {
            int mt, nt;
            if (g.w_resident) { mt = cursor; nt = (int)blockIdx.x % nnt; }
            else tile_coords(cursor, g, mt, nt);
            const int m0 = mt * BM, n0 = nt * BN;
            const int32_t* tile_bias = tail->bias + (bias_resident ? n0 : grp * BN);
            if (HAS_BIAS && !bias_resident) {
                // stage this tile's bias slice (zero where there is none); the group's previous tile is done with it
                asm volatile("bar.sync %0, 128;" :: "r"(2 + grp) : "memory");
                for (int i = gt; i < BN; i += EPI_GROUP_THREADS) {
                    const int n = n0 + i;
                    tail->bias[grp * BN + i] = (g.bias != nullptr && n < g.N) ? __ldg(g.bias + n) : 0;
                }
                asm volatile("bar.sync %0, 128;" :: "r"(2 + grp) : "memory");
            }
            if (ok) ok = mbar_wait(&tail->tmem_full[grp], acc_phase, abort_flag, g.status, 104);
            acc_phase ^= 1u;
            if (!ok) continue;
            tc_fence_after();
            const int row_base = m0 + quad * 32;
            // Four 64-column groups per warp through ONE register buffer.  Loading the next group while this one is
            // converted (a second buffer of 64 registers) measured 2-6 % slower: at the kernel's register ceiling the
            // conversion code schedules better with the registers than the TMEM load latency costs.  The accumulator
            // goes back to the MMA issuer as soon as its last columns are in registers, before they are converted.
            uint32_t ra[64];
#pragma unroll 1
            for (int c = 0; c < 4; ++c) {
                const bool have = n0 + c * 64 < g.N;   // warp-uniform
                if (have) {
                    tmem_ld32_async(taddr + (uint32_t)(c * 64), ra);
                    tmem_ld32_async(taddr + (uint32_t)(c * 64 + 32), ra + 32);
                    tmem_ld_wait32(ra);
                    tmem_ld_wait32(ra + 32);
                }
                if (c == 3) {
                    tc_fence_before();
                    mbar_arrive(&tail->tmem_empty[grp]);
                }
                if (have) epilogue_pair<MODE, HAS_BIAS>(ra, tile_bias + c * 64, my_stage, lane, g, &tmap_y, row_base, n0 + c * 64);
            }
        }
        // the stores this warp issued must be complete (not merely read) before the CTA retires
        if (lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
        __syncwarp();
    }

    // ---------------- teardown ----------------
    __syncthreads();
    if (*abort_flag) {
        // let TMA copies and MMAs that were already issued land before the CTA gives up its
        // shared memory and TMEM
        const uint64_t t0 = a4c_globaltimer();
        while (a4c_globaltimer() - t0 < 2000000ull) __nanosleep(1000);
        __syncthreads();
    }
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" :: "r"(tmem_base), "r"((uint32_t)TMEM_COLS) : "memory");
    }
}

// ---- host side -----------------------------------------------------------------------------------
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

// 2-D uint8 tensor map over a row-major [rows, cols] matrix with row pitch `ld` bytes,
// box = [box_rows, 128 bytes], 128-byte swizzle, out-of-range elements read as zero.
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

// 2-D uint8 map over the row-major [rows, cols] output, box = [32 rows, 64 bytes], 64-byte swizzle: the
// shape of one epilogue warp's staging patch.
bool make_out_map(CUtensorMap* map, void* base, long long rows, long long cols, long long ld) {
    EncodeTiledFn fn = get_encode_fn();
    if (!fn) return false;
    cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld};
    cuuint32_t box[2] = {64u, 32u};
    cuuint32_t estr[2] = {1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, base, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
              CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) ==
           CUDA_SUCCESS;
}

template <int MODE>
cudaError_t launch_mode(const CUtensorMap& ma, const CUtensorMap& mb, const CUtensorMap& my, const TcArgs& g, int grid,
                        cudaStream_t s) {
    static tc::SmemOptIn opt_in[2];
    if (g.bias != nullptr) {
        const cudaError_t attr_err = opt_in[1].ensure(dense_tc_kernel<MODE, true>, SMEM_BYTES);
        if (attr_err != cudaSuccess) return attr_err;
        dense_tc_kernel<MODE, true><<<grid, NUM_THREADS, SMEM_BYTES, s>>>(ma, mb, my, g);
    } else {
        const cudaError_t attr_err = opt_in[0].ensure(dense_tc_kernel<MODE, false>, SMEM_BYTES);
        if (attr_err != cudaSuccess) return attr_err;
        dense_tc_kernel<MODE, false><<<grid, NUM_THREADS, SMEM_BYTES, s>>>(ma, mb, my, g);
    }
    return cudaGetLastError();
}

}  // namespace

void a4c_dense_tc_set_resident_w(int mode) { g_dense_resident_w = mode < 0 ? 0 : (mode > 2 ? 2 : mode); }
void a4c_dense_tc_set_panel_mib(int mib) { g_dense_panel_bytes = (long long)mib << 20; }
long long a4c_dense_tc_panel_bytes() { return g_dense_panel_bytes; }

int a4c_dense_tc_supported(const void* A, long long lda, const void* Wt, long long ldw, const void* Y,
                           long long ldy, long long M, int K, int N, int out_dtype) {
    if (out_dtype != A4C_I8 && out_dtype != A4C_U8) return A4C_ERR_UNSUPPORTED;
    if (K < 16) return A4C_ERR_UNSUPPORTED;   // any N: TMA zero-fills absent weight rows and clips stored columns
    if (lda % 16 || ldw % 16 || ldy % 16) return A4C_ERR_ALIGNMENT;
    if (((uintptr_t)A | (uintptr_t)Wt | (uintptr_t)Y) & 15u) return A4C_ERR_ALIGNMENT;
    if (M > 2147483647LL - BM || lda < K || ldw < K) return A4C_ERR_INVALID_ARG;
    const long long tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
    if (tiles > 2147483647LL) return A4C_ERR_TOO_LARGE;
    return A4C_OK;
}

int a4c_launch_dense_tc(const void* A, long long lda, const void* Wt, long long ldw, const int32_t* bias,
                        void* Y, long long ldy, long long M, int K, int N, int shift, int rounding, int relu,
                        int out_dtype, int a_unsigned, int cta_pair, int* status_word, cudaStream_t stream) {
    if (cta_pair) return A4C_ERR_UNSUPPORTED;
    const int sup = a4c_dense_tc_supported(A, lda, Wt, ldw, Y, ldy, M, K, N, out_dtype);
    if (sup != A4C_OK) return sup;
    if (M == 0) return A4C_OK;
    {
        // short reductions with enough row tiles: the kernel with more epilogue warps in flight
        int dev0 = 0, sms0 = 148;
        cudaGetDevice(&dev0);
        cudaDeviceGetAttribute(&sms0, cudaDevAttrMultiProcessorCount, dev0);
        if (g_dense_resident_w == 2 && a4c_dense_tcs_supported(M, K, N, out_dtype, sms0) == A4C_OK)
            return a4c_launch_dense_tcs(A, lda, Wt, ldw, bias, Y, ldy, M, K, N, shift, rounding, relu, out_dtype, a_unsigned,
                                        status_word, stream);
    }
    CUtensorMap ma, mb, my;
    const int w_box_rows = (N + BN - 1) / BN == 1 ? ((N + 15) / 16) * 16 : BN;
    if (!make_map(&ma, A, M, K, lda, BM) || !make_map(&mb, Wt, N, K, ldw, w_box_rows) ||
        !make_out_map(&my, Y, M, N >= 16 ? (N / 16) * 16 : 16, ldy))
        return A4C_ERR_CUDA;
    TcArgs g;
    g.bias = bias; g.Y = (uint8_t*)Y; g.ldy = ldy; g.M = M; g.K = K; g.N = N;
    g.n_full = (N / 16) * 16;
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
    // a single narrow N tile (N <= 256) issues MMAs only as wide as the layer, rounded up to 16 columns, and its
    // weight box is that many rows instead of 256 (absent rows would be zero-filled into shared memory for nothing)
    const int umma_n = g.num_n_tiles == 1 ? ((N + 15) / 16) * 16 : BN;
    g.b_box_rows = umma_n;
    g.idesc = make_idesc(BM, umma_n, a_unsigned != 0);
    g.status = status_word;
    int dev = 0, sms = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const long long tiles = (long long)g.num_m_tiles * g.num_n_tiles;
    int grid = (int)(tiles < sms ? tiles : sms);
    // Resident-W mode: the K extent of one weight tile fits beside at least four A slots (K <= 512), every
    // column tile gets the same number of CTAs, and each CTA has several row tiles to stream.
    const int num_kb = (K + BK - 1) / BK;
    const int per = sms / g.num_n_tiles;
    g.w_resident = 0; g.a_stages = STAGES;
    // panels of at most 32 MiB of weights (whole column tiles); one panel when the weights are smaller than that
    {
        const long long tile_bytes = (long long)BN * (((long long)K + BK - 1) / BK * BK);
        long long per = g_dense_panel_bytes / tile_bytes;
        if (per < 1) per = 1;
        g.panel = g_dense_panel_bytes <= 0 || per >= g.num_n_tiles ? g.num_n_tiles : (int)per;
    }
    if (g_dense_resident_w && num_kb <= 4 && g.num_n_tiles <= 16 && per >= 1 && g.num_m_tiles >= 4 * per) {
        g.w_resident = 1;
        const int slots = (STAGES * STAGE_BYTES - num_kb * B_BYTES) / A_BYTES;
        g.a_stages = slots < MAX_RING ? slots : MAX_RING;
        grid = per * g.num_n_tiles;
    }
    cudaError_t err;
    if (shift == 0) err = launch_mode<-1>(ma, mb, my, g, grid, stream);
    else switch (rounding) {
        case A4C_RND_FLOOR: err = launch_mode<A4C_RND_FLOOR>(ma, mb, my, g, grid, stream); break;
        case A4C_RND_CEIL: err = launch_mode<A4C_RND_CEIL>(ma, mb, my, g, grid, stream); break;
        case A4C_RND_POSITIVE_INF:
            err = !pre_clamp ? launch_mode<A4C_RND_POSITIVE_INF>(ma, mb, my, g, grid, stream)
                  : shift <= 13 ? launch_mode<MODE_HALF_UP_FLOAT>(ma, mb, my, g, grid, stream)
                                : launch_mode<MODE_HALF_UP_CLAMP>(ma, mb, my, g, grid, stream);
            break;
        case A4C_RND_NEGATIVE_INF: err = launch_mode<A4C_RND_NEGATIVE_INF>(ma, mb, my, g, grid, stream); break;
        case A4C_RND_SYMMETRIC_INF: err = launch_mode<A4C_RND_SYMMETRIC_INF>(ma, mb, my, g, grid, stream); break;
        case A4C_RND_SYMMETRIC_ZERO: err = launch_mode<A4C_RND_SYMMETRIC_ZERO>(ma, mb, my, g, grid, stream); break;
        case A4C_RND_CONV_EVEN: err = launch_mode<A4C_RND_CONV_EVEN>(ma, mb, my, g, grid, stream); break;
        case A4C_RND_CONV_ODD: err = launch_mode<A4C_RND_CONV_ODD>(ma, mb, my, g, grid, stream); break;
        default: return A4C_ERR_INVALID_ARG;
    }
    return err == cudaSuccess ? A4C_OK : A4C_ERR_CUDA;
}
