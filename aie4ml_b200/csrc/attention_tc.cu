// Attention heads, fused:  O_bh = srs( softmax_u8( srs(Q_bh . K_bh^T) ) . V_bh )  for every batch entry b and head
// h in one launch, with the scores and probabilities never leaving the SM.
//
// This is the chain  matmul_single::run (matmul.cpp:32-118, TRANSPOSE_B) -> softmax (softmax.cpp:20-88 HCCS,
// :252-384 exp) -> matmul_single::run  of aie4ml, with every intermediate rounding and saturation kept:
//   scores  s[m,n] = sat_i8(round_shift(sum_d Q[m,d] K[n,d], qk_shift))
//   probs   p[m,n] = min((score(max_n s - s[m,n]) * inv) >> inv_shift, 255),  inv from the row's score sum
//   out     o[m,d] = sat_i8(round_shift(sum_n p[m,n] V[n,d], pv_shift))
// The three kernels it replaces move the [rows, keys] score and probability matrices through HBM four times;
// here HBM sees Q, K, V once and O once.
//
// Shape of the kernel (one CTA per SM, persistent over (batch entry, 128-query tile, head) items, head fastest:
// heads that are 64-byte column slices of one tensor share the 256-byte lines the TMA unit promotes to, so a line
// is fetched from HBM once instead of once per head):
//   warp 0      TMA producer: Q tile [128 x 64], K [128 keys x 64], V [128 keys x 64] per item, 64-byte swizzle,
//               4-stage ring
//   warp 1      MMA issuer: S = Q K^T (M128 N128 K64, both operands K-major) into one of two TMEM score
//               buffers; later O = P V (M128 N64 K128, P K-major from shared memory, V MN-major) into one of
//               two TMEM output buffers.  The next item's S is issued before this item's O, so the tensor
//               pipe works on scores while the softmax warps are busy.
//   warps 2-17  softmax: group 0 (even items) and group 1 (odd items) of eight warps each.  TWO threads share a
//               query row (a TMEM lane): each takes 64 of the 128 score columns -- tcgen05.ld of 64 accumulators,
//               requantise, maximum, score table lookup (per-lane replicated table in shared memory: no bank
//               conflicts), sum -- and the two exchange the row maximum and the row sum through shared memory
//               (a 64-thread named barrier per warp pair).  Each then normalises its half and writes it as uint8
//               into the 128-byte-swizzled K-major tile the second MMA reads, and later converts and stores 32 of
//               the row's 64 output columns.  Sixteen such warps give every scheduler four of them to interleave
//               (with eight, one thread per row, the integer pipe sat 58 % busy behind load latencies); the
//               register budget is 96 per thread (five of the eighteen warps share one scheduler's 16 K registers).
// Every wait is bounded (tc::mbar_wait): on a timeout the CTA sets the status word and drains.
#include <cuda.h>

#include <mutex>

#include "a4c_common.cuh"
#include "a4c_kernels.h"
#include "tc_common.cuh"

using namespace tc;

namespace {

constexpr int BM = 128;        // query rows per item
constexpr int SK = 128;        // keys per batch entry (exactly)
constexpr int DH = 64;         // head width
constexpr int UMMA_K = 32;
constexpr int STAGES = 4;
constexpr int TILE_BYTES = 128 * DH;              // 8 KB: Q, K and V tiles alike
constexpr int STAGE_BYTES = 3 * TILE_BYTES;
constexpr int P_BYTES = BM * SK;                  // 16 KB per softmax group
constexpr int LUT_BYTES = 256 * 32 * 4;
constexpr int GROUPS = 2;
constexpr int HALVES = 2;                         // threads per query row
constexpr int HALF_COLS = SK / HALVES;            // score columns per thread
constexpr int GROUP_THREADS = 128 * HALVES;
constexpr int NUM_THREADS = 64 + GROUPS * GROUP_THREADS;
constexpr int MAX_REGS = 96;                      // 18 warps: five share one scheduler's 16384 registers
constexpr int TMEM_COLS = 512;                    // scores at columns g*128, outputs at 256 + g*64
constexpr int MODE_HALF_UP_CLAMP = 100;           // positive_inf, both shifts in [1, 22]: saturate before the shift
// The same with both shifts <= 13 and the shift itself moved to the multiply-add pipe: the clamped value n, |n| < 2^22,
// is produced as the bit pattern of the float 1.5*2^23 + n, and one round-down FMA by 2^-s leaves
// 1.5*2^23 + floor(n / 2^s), whose low byte is the result.
constexpr int MODE_HALF_UP_FLOAT = 102;
constexpr int MAGIC_BITS = 0x4B400000;            // 1.5 * 2^23

constexpr float TWO_M64 = 5.421010862427522e-20f;  // 2^-64
constexpr float TWO_P64 = 18446744073709551616.0f; // 2^64

struct Tail {
    uint64_t qkv_full[STAGES];
    uint64_t qkv_empty[STAGES];
    uint64_t s_full[GROUPS];
    uint64_t p_full[GROUPS];
    uint64_t o_full[GROUPS];
    uint64_t pair[GROUPS][4];     // the two warps that share a group's 32 query rows meet here (one arrival per warp)
    uint32_t tmem_base;
    volatile int abort_flag;
    // row maximum (slot 0) and row sum (slot 1) of each half row, read by the thread that holds the other half
    uint32_t xch[GROUPS][2][HALVES][BM];
};

constexpr size_t SMEM_BYTES = 1024 + (size_t)STAGES * STAGE_BYTES + (size_t)GROUPS * P_BYTES + LUT_BYTES + sizeof(Tail);

struct AttnArgs {
    uint8_t* out; long long ldo, stride_o, hstride_o;
    long long batch; int sq, m_tiles, heads;
    int head_inner;   // tensor-map dimension order {64, heads, rows, batch} (heads are column slices) or {64, rows, heads, batch}
    // requantisation of the scores (1) and of the outputs (2)
    int shift1, shift2;
    uint32_t mask1, c01, mask2, c02;          // generic rounding constants
    int xhi1, addb1, xlob1;                   // MODE_HALF_UP_CLAMP / _FLOAT, biased by +128: see score_code
    int xhi2, half2, xlo2;
    float fmul1, fadd1, fmul2, fadd2;         // MODE_HALF_UP_FLOAT: 2^-s and 1.5*2^23 * (1 - 2^-s) per step
    // softmax
    int mode, B, S, Dmax, inv_shift, use_clb, exp_kq;
    int* status;
};

__device__ __forceinline__ void tma_load_4d(void* dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1, int c2,
                                            int c3) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
        :: "r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2), "r"(c3) : "memory");
}

// K-major operand whose K extent is one 64-byte swizzle row: rows of 64 bytes, 8-row groups 512 bytes apart.
__device__ __forceinline__ uint64_t make_smem_desc_k64(uint32_t saddr) {
    uint64_t d = 0;
    d |= (uint64_t)((saddr & 0x3FFFFu) >> 4);
    d |= (uint64_t)1 << 16;
    d |= (uint64_t)(512 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)4 << 61;              // SWIZZLE_64B
    return d;
}
// MN-major operand, 64-byte swizzle: k-rows of 64 bytes, 8-row groups 512 bytes apart.
__device__ __forceinline__ uint64_t make_smem_desc_mn64(uint32_t saddr) { return make_smem_desc_k64(saddr); }

__device__ __forceinline__ float lds32f(uint32_t a) {
    float v;
    asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(a));
    return v;
}
__device__ __forceinline__ uint32_t lds32(uint32_t a) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(a) : "memory");
    return v;
}
__device__ __forceinline__ void sts32(uint32_t a, uint32_t v) {
    asm volatile("st.shared.u32 [%0], %1;" :: "r"(a), "r"(v) : "memory");
}
__device__ __forceinline__ void sts128(uint32_t a, uint32_t x, uint32_t y, uint32_t z, uint32_t w) {
    asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" :: "r"(a), "r"(x), "r"(y), "r"(z), "r"(w) : "memory");
}

// exp_score16, softmax.cpp:252-273
__device__ __forceinline__ int exp_score16(int d, int kq) {
    const int z = min(d * kq, 32767);
    const int zint = z >> 8, zfrac = z & 255;
    const int t = (zfrac * 2811) >> 8;
    const int inner = t - 11004;
    const int t2 = (inner * zfrac) >> 8;
    const int e = t2 + 16384;
    return zint >= 16 ? 0 : (e >> (zint & 15));
}

// Score accumulator -> int8 score + 128 (an unsigned byte whose order is the signed order), plus the constant
// code_bias<MODE>() in the upper bits: differences and maxima of two codes are those of the scores.
template <int MODE>
__device__ __forceinline__ int score_code(int acc, const AttnArgs& g) {
    if (MODE == MODE_HALF_UP_FLOAT) {
        const int u = __viaddmax_s32(min(acc, g.xhi1), g.addb1 + MAGIC_BITS, g.xlob1 + MAGIC_BITS);
        return __float_as_int(__fmaf_rd(__int_as_float(u), g.fmul1, g.fadd1));
    }
    if (MODE == MODE_HALF_UP_CLAMP) {
        // min(acc, 127 * 2^s), then + 2^(s-1) + 128 * 2^s with the lower clamp folded in, then the shift
        return __viaddmax_s32(min(acc, g.xhi1), g.addb1, g.xlob1) >> g.shift1;
    }
    int v = acc;
    if (MODE == A4C_RND_FLOOR) v = acc >> g.shift1;
    else if (MODE >= 0) v = round_shift_i32_t<MODE>(acc, g.shift1, g.mask1, g.c01);
    return min(max(v, -128), 127) + 128;
}

// Output accumulator -> a word whose low byte is the int8 result.
template <int MODE>
__device__ __forceinline__ int requant_out(int acc, const AttnArgs& g) {
    if (MODE == MODE_HALF_UP_FLOAT) {
        const int u = __viaddmax_s32(min(acc, g.xhi2), g.half2 + MAGIC_BITS, g.xlo2 + MAGIC_BITS);
        return __float_as_int(__fmaf_rd(__int_as_float(u), g.fmul2, g.fadd2));
    }
    if (MODE == MODE_HALF_UP_CLAMP) return __viaddmax_s32(min(acc, g.xhi2), g.half2, g.xlo2) >> g.shift2;
    int v = acc;
    if (MODE == A4C_RND_FLOOR) v = acc >> g.shift2;
    else if (MODE >= 0) v = round_shift_i32_t<MODE>(acc, g.shift2, g.mask2, g.c02);
    return min(max(v, -128), 127);
}

template <int MODE>
__global__ void __maxnreg__(MAX_REGS)
attention_tc_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                    const __grid_constant__ CUtensorMap tmap_v, AttnArgs g) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* p_smem = smem + (size_t)STAGES * STAGE_BYTES;
    float* lut = reinterpret_cast<float*>(p_smem + (size_t)GROUPS * P_BYTES);
    Tail* tail = reinterpret_cast<Tail*>(reinterpret_cast<uint8_t*>(lut) + LUT_BYTES);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    // item = ((batch entry * query tiles) + query tile) * heads + head: the heads of one batch entry, which share
    // their 256-byte-promoted L2 lines when they are column slices of one tensor, run at the same time
    const long long num_items = g.batch * g.m_tiles * g.heads;
    // items of this CTA: blockIdx.x, + gridDim.x, ...; n is the CTA-local index
    const long long first = blockIdx.x;
    const int n_local = first < num_items ? (int)((num_items - first + gridDim.x - 1) / gridDim.x) : 0;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(&tail->qkv_full[s], 1); mbar_init(&tail->qkv_empty[s], 1); }
        for (int s = 0; s < GROUPS; ++s) {
            mbar_init(&tail->s_full[s], 1);
            mbar_init(&tail->p_full[s], GROUP_THREADS);
            mbar_init(&tail->o_full[s], 1);
            for (int q = 0; q < 4; ++q) mbar_init(&tail->pair[s][q], HALVES);
        }
        tail->abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     :: "r"(smem_u32(&tail->tmem_base)), "r"((uint32_t)TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    {
        // score table: entry d (= row maximum - score, 0..255) replicated across 32 lanes, scaled by 2^-64 so
        // that the normalising multiply lands in a subnormal whose bit pattern is the integer result
        float* stage_sc = reinterpret_cast<float*>(p_smem);
        if (threadIdx.x < 256) {
            const int d = threadIdx.x;
            int s;
            if (g.mode == 0) s = clampi(g.B - g.S * min(d, g.Dmax), -32768, 32767);
            else s = exp_score16(d, g.exp_kq);
            stage_sc[d] = (float)s * TWO_M64;
        }
        __syncthreads();
        for (int i = threadIdx.x; i < 256 * 32; i += NUM_THREADS) lut[i] = stage_sc[i >> 5];
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tail->tmem_base;
    volatile int* abort_flag = &tail->abort_flag;

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (lane == 0) {
            bool ok = true;
            for (int n = 0; ok && n < n_local; ++n) {
                const long long item = first + (long long)n * gridDim.x;
                const int h = (int)(item % g.heads);
                const long long t = item / g.heads;
                const int b = (int)(t / g.m_tiles);
                const int m0 = (int)(t % g.m_tiles) * BM;
                const int stage = n % STAGES;
                const uint32_t ph = (uint32_t)(n / STAGES) & 1u;
                ok = mbar_wait(&tail->qkv_empty[stage], ph ^ 1u, abort_flag, g.status, 121);
                if (!ok) break;
                uint8_t* st = smem + (size_t)stage * STAGE_BYTES;
                mbar_arrive_expect_tx(&tail->qkv_full[stage], STAGE_BYTES);
                if (g.head_inner) {
                    tma_load_4d(st, &tmap_q, &tail->qkv_full[stage], 0, h, m0, b);
                    tma_load_4d(st + TILE_BYTES, &tmap_k, &tail->qkv_full[stage], 0, h, 0, b);
                    tma_load_4d(st + 2 * TILE_BYTES, &tmap_v, &tail->qkv_full[stage], 0, h, 0, b);
                } else {
                    tma_load_4d(st, &tmap_q, &tail->qkv_full[stage], 0, m0, h, b);
                    tma_load_4d(st + TILE_BYTES, &tmap_k, &tail->qkv_full[stage], 0, 0, h, b);
                    tma_load_4d(st + 2 * TILE_BYTES, &tmap_v, &tail->qkv_full[stage], 0, 0, h, b);
                }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            const uint32_t idesc_s = make_idesc(BM, SK, false);
            const uint32_t idesc_o = make_idesc(BM, DH, true) | (1u << 16);   // P is uint8, V is MN-major
            bool ok = true;
            auto issue_scores = [&](int n) -> bool {
                const int stage = n % STAGES;
                if (!mbar_wait_fast(&tail->qkv_full[stage], (uint32_t)(n / STAGES) & 1u, abort_flag, g.status, 122)) return false;
                tc_fence_after();
                const uint32_t st = smem_u32(smem + (size_t)stage * STAGE_BYTES);
                const uint64_t qd = make_smem_desc_k64(st), kd = make_smem_desc_k64(st + TILE_BYTES);
                const uint32_t d_tmem = tmem_base + (uint32_t)((n & 1) * SK);
#pragma unroll
                for (int k = 0; k < DH / UMMA_K; ++k)
                    umma_i8(d_tmem, qd + (uint64_t)(k * (UMMA_K >> 4)), kd + (uint64_t)(k * (UMMA_K >> 4)), idesc_s,
                            (uint32_t)(k != 0));
                umma_commit(&tail->s_full[n & 1]);
                return true;
            };
            if (n_local > 0) ok = issue_scores(0);
            for (int n = 0; ok && n < n_local; ++n) {
                // the score buffer of item n+1 was last read for item n-1, whose probabilities this thread has
                // already waited for
                if (n + 1 < n_local) { ok = issue_scores(n + 1); if (!ok) break; }
                const int grp = n & 1, stage = n % STAGES;
                ok = mbar_wait_fast(&tail->p_full[grp], (uint32_t)(n >> 1) & 1u, abort_flag, g.status, 123);
                if (!ok) break;
                tc_fence_after();
                const uint64_t pd = make_smem_desc(smem_u32(p_smem + (size_t)grp * P_BYTES));
                const uint64_t vd = make_smem_desc_mn64(smem_u32(smem + (size_t)stage * STAGE_BYTES + 2 * TILE_BYTES));
                const uint32_t d_tmem = tmem_base + (uint32_t)(2 * SK + grp * DH);
#pragma unroll
                for (int k = 0; k < SK / UMMA_K; ++k)
                    umma_i8(d_tmem, pd + (uint64_t)(k * (UMMA_K >> 4)), vd + (uint64_t)(k * ((UMMA_K * DH) >> 4)), idesc_o,
                            (uint32_t)(k != 0));
                umma_commit(&tail->o_full[grp]);
                umma_commit(&tail->qkv_empty[stage]);
            }
        }
        __syncwarp();
    } else {
        // ---------------- softmax + output (two groups of eight warps, two threads per query row) ----------------
        const int quad = warp & 3;                   // TMEM lane quadrant of this warp
        const int grp = (warp - 2) >> 3;             // warps 2-9: even items, warps 10-17: odd items
        const int hf = ((warp - 2) >> 2) & 1;        // which 64 score columns (and which 32 output columns)
        const int r = quad * 32 + lane;              // query row inside the tile
        uint64_t* pair_bar = &tail->pair[grp][quad];   // where the two warps that share these rows meet (bounded wait)
        uint32_t pair_phase = 0;
        // Both warps have written their shared-memory words; returns once the other warp's are readable.
        auto pair_sync = [&]() -> bool {
            __syncwarp();
            if (lane == 0) mbar_arrive(pair_bar);
            const bool met = mbar_wait_fast(pair_bar, pair_phase, abort_flag, g.status, 126);
            pair_phase ^= 1u;
            return met;
        };
        const uint32_t lut_lane = smem_u32(lut) + (uint32_t)lane * 4u;
        const uint32_t p_row = smem_u32(p_smem + (size_t)grp * P_BYTES) + (uint32_t)r * 128u;
        const uint32_t sw = (uint32_t)(r & 7);
        const uint32_t taddr_s = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(grp * SK + hf * HALF_COLS);
        const uint32_t taddr_o = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(2 * SK + grp * DH + hf * (DH / HALVES));
        // exchange words as shared-space addresses: slot 0 (maximum) here, slot 1 (sum) XCH_SLOT bytes further
        const uint32_t xch_mine = smem_u32(&tail->xch[grp][0][hf][r]);
        const uint32_t xch_other = smem_u32(&tail->xch[grp][0][hf ^ 1][r]);
        constexpr uint32_t XCH_SLOT = HALVES * BM * 4;
        const int numer = 255 << g.inv_shift;
        const float numer_f = (float)numer;
        const float out_mul = __int_as_float((127 - (g.inv_shift + 85)) << 23);  // 2^-(inv_shift + 85)
        const bool clb = g.use_clb && g.mode == 0;
        bool ok = true;
        for (int n = grp; ok && n < n_local; n += GROUPS) {
            const long long item = first + (long long)n * gridDim.x;
            const int h = (int)(item % g.heads);
            const long long t = item / g.heads;
            const long long b = t / g.m_tiles;
            const int row = (int)(t % g.m_tiles) * BM + r;
            const uint32_t par = (uint32_t)(n >> 1) & 1u;
            ok = mbar_wait_fast(&tail->s_full[grp], par, abort_flag, g.status, 124);
            if (!ok) break;
            tc_fence_after();

            // this thread's 64 scores: accumulators -> codes (score + 128, plus a constant in the upper bits)
            uint32_t v[HALF_COLS];
            static_assert(HALF_COLS == 64, "two 32-column TMEM loads per thread");
            tmem_ld32_async(taddr_s, v);
            tmem_ld32_async(taddr_s + 32u, v + 32);
            tmem_ld_wait32(v);
            tmem_ld_wait32(v + 32);
            int m = (int)0x80000000;
#pragma unroll
            for (int i = 0; i < HALF_COLS; i += 2) {
                const int c0 = score_code<MODE>((int)v[i], g), c1 = score_code<MODE>((int)v[i + 1], g);
                v[i] = (uint32_t)c0;
                v[i + 1] = (uint32_t)c1;
                m = __vimax3_s32(m, c0, c1);
            }
            sts32(xch_mine, (uint32_t)m);
            ok = pair_sync();
            if (!ok) break;
            m = max(m, (int)lds32(xch_other));
            // table address of score code c: lut_lane + (m - c) * 128, as one multiply-add
            const uint32_t row_base = lut_lane + (uint32_t)m * 128u;
            float fs0 = 0.0f, fs1 = 0.0f;
#pragma unroll
            for (int i = 0; i < HALF_COLS; i += 2) {   // each code is replaced by (the bits of) its table entry
                const float e0 = lds32f(row_base - v[i] * 128u), e1 = lds32f(row_base - v[i + 1] * 128u);
                v[i] = __float_as_uint(e0);
                v[i + 1] = __float_as_uint(e1);
                fs0 += e0;
                fs1 += e1;
            }
            // exact: at most 128 scores <= 32767 (scaled by 2^-64), whatever the order of the additions
            const float fs = fs0 + fs1;
            sts32(xch_mine + XCH_SLOT, __float_as_uint(fs));
            ok = pair_sync();
            if (!ok) break;
            const int sum = __float2int_rn((fs + __uint_as_float(lds32(xch_other + XCH_SLOT))) * TWO_P64);
            const int s = sum > 0 ? sum : 1;
            int inv;
            if (clb) {
                const int k = 31 - __clz(s);
                inv = g.inv_shift - k >= 0 ? (255 << (g.inv_shift - k)) : (255 >> (k - g.inv_shift));
            } else {
                // exact floor(numer / s) wherever it is below 2^15 (larger quotients saturate to 32767 anyway)
                float rcp;
                asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(rcp) : "f"((float)s));
                int q = __float2int_rz(numer_f * rcp);
                const int rem = numer - q * s;
                q += (rem >= s) - (rem < 0);
                inv = q;
            }
            inv = min(max(inv, 0), 32767);
            const float invs = (float)inv * out_mul;
#pragma unroll
            for (int c = 0; c < HALF_COLS / 16; ++c) {
                uint32_t w[4];
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const int i = c * 16 + q * 4;
                    // floor(score * inv / 2^shift) in the low bits of a subnormal (scores are non-negative)
                    // with inv = floor(255 * 2^shift / sum) a score <= sum cannot exceed 255; only the power-of-two
                    // reciprocal (use_clb) needs the saturation
                    int o0 = __float_as_int(__fmaf_rd(__uint_as_float(v[i + 0]), invs, 0.0f));
                    int o1 = __float_as_int(__fmaf_rd(__uint_as_float(v[i + 1]), invs, 0.0f));
                    int o2 = __float_as_int(__fmaf_rd(__uint_as_float(v[i + 2]), invs, 0.0f));
                    int o3 = __float_as_int(__fmaf_rd(__uint_as_float(v[i + 3]), invs, 0.0f));
                    if (clb) { o0 = min(o0, 255); o1 = min(o1, 255); o2 = min(o2, 255); o3 = min(o3, 255); }
                    w[q] = pack4_i8(o0, o1, o2, o3);
                }
                // K-major, 128-byte swizzle: 16-byte piece p of row r sits at piece p ^ (r & 7)
                sts128(p_row + ((((uint32_t)(hf * (HALF_COLS / 16) + c)) ^ sw) << 4), w[0], w[1], w[2], w[3]);
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // generic-proxy stores -> tensor-core reads
            tc_fence_before();
            mbar_arrive(&tail->p_full[grp]);

            // this thread's 32 columns of the output row
            ok = mbar_wait_fast(&tail->o_full[grp], par, abort_flag, g.status, 125);
            if (!ok) break;
            tc_fence_after();
            uint32_t oa[DH / HALVES];
            static_assert(DH / HALVES == 32, "one 32-column TMEM load per thread");
            tmem_ld32(taddr_o, oa);
            tc_fence_before();
            if (row < g.sq) {
                uint8_t* orow = g.out + b * g.stride_o + h * g.hstride_o + (long long)row * g.ldo + hf * (DH / HALVES);
#pragma unroll
                for (int c = 0; c < DH / HALVES / 16; ++c) {
                    uint32_t w[4];
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        const int i = c * 16 + q * 4;
                        w[q] = pack4_i8(requant_out<MODE>((int)oa[i + 0], g), requant_out<MODE>((int)oa[i + 1], g),
                                        requant_out<MODE>((int)oa[i + 2], g), requant_out<MODE>((int)oa[i + 3], g));
                    }
                    *reinterpret_cast<uint4*>(orow + c * 16) = make_uint4(w[0], w[1], w[2], w[3]);
                }
            }
        }
    }

    // ---------------- teardown ----------------
    __syncthreads();
    if (*abort_flag) {
        // let TMA copies and MMAs that were already issued land before the CTA gives up its shared memory and TMEM
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

// 4-D uint8 map over the heads of a tensor, 64-byte swizzle, one box = 128 rows x 64 bytes of one head of one batch
// entry; rows past the end read as zero.  Dimension order keeps the strides ascending: {64, heads, rows, batch} when
// the heads are column slices of a row (head_inner), else {64, rows, heads, batch}.  Extents of one get a stride that
// is merely valid.
bool make_head_map(CUtensorMap* map, const void* base, long long rows, int heads, long long batch, long long ld,
                   long long hstride, long long stride, bool head_inner) {
    EncodeTiledFn fn = get_encode_fn();
    if (!fn) return false;
    if (heads <= 1) hstride = head_inner ? 64 : (rows > 0 ? rows : 1) * ld;
    if (batch <= 1) stride = (rows > 0 ? rows : 1) * ld * (head_inner || heads <= 1 ? 1 : heads);
    const cuuint64_t nh = (cuuint64_t)(heads > 0 ? heads : 1), nb = (cuuint64_t)(batch > 0 ? batch : 1);
    cuuint64_t dims[4] = {(cuuint64_t)DH, head_inner ? nh : (cuuint64_t)rows, head_inner ? (cuuint64_t)rows : nh, nb};
    cuuint64_t strides[3] = {(cuuint64_t)(head_inner ? hstride : ld), (cuuint64_t)(head_inner ? ld : hstride),
                             (cuuint64_t)stride};
    cuuint32_t box[4] = {(cuuint32_t)DH, head_inner ? 1u : 128u, head_inner ? 128u : 1u, 1u};
    cuuint32_t estr[4] = {1, 1, 1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, const_cast<void*>(base), dims, strides, box, estr,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int MODE>
cudaError_t launch_mode(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, const AttnArgs& g, int grid,
                        cudaStream_t s) {
    static tc::SmemOptIn opt_in;
    const cudaError_t attr_err = opt_in.ensure(attention_tc_kernel<MODE>, SMEM_BYTES);
    if (attr_err != cudaSuccess) return attr_err;
    attention_tc_kernel<MODE><<<grid, NUM_THREADS, SMEM_BYTES, s>>>(mq, mk, mv, g);
    return cudaGetLastError();
}

}  // namespace

int a4c_attention_tc_supported(const void* q, long long ldq, long long stride_q, const void* k, long long ldk,
                               long long stride_k, const void* v, long long ldv, long long stride_v, const void* out,
                               long long ldo, long long stride_o, long long batch, int sq, int sk, int dh, int qk_shift,
                               int pv_shift, int sm_mode, int B, int S, int Dmax, int inv_shift, int heads,
                               long long hstride_q, long long hstride_k, long long hstride_v, long long hstride_o) {
    if (sk != SK || dh != DH || sq < 1 || batch < 0 || heads < 1) return A4C_ERR_UNSUPPORTED;
    if (heads > 1 && (hstride_q % 16 || hstride_k % 16 || hstride_v % 16 || hstride_o % 16)) return A4C_ERR_ALIGNMENT;
    if (heads > 1 && (hstride_q < 1 || hstride_k < 1 || hstride_v < 1 || hstride_o < 1)) return A4C_ERR_INVALID_ARG;
    if ((qk_shift == 0) != (pv_shift == 0)) return A4C_ERR_UNSUPPORTED;   // one rounding template serves both steps
    if (qk_shift < 0 || qk_shift > 31 || pv_shift < 0 || pv_shift > 31) return A4C_ERR_INVALID_ARG;
    if (sm_mode != 0 && sm_mode != 1) return A4C_ERR_INVALID_ARG;
    if (inv_shift < 0 || inv_shift > 22) return A4C_ERR_UNSUPPORTED;
    // HCCS: every score must lie in [0, 32767] (the kernel normalises through the bit pattern of a non-negative
    // value); these are the reference resolver's bounds (softmax/common.py:59-89), anything else goes to the
    // separate kernels
    if (sm_mode == 0 && (S < 0 || Dmax < 0 || B < 0 || B > 32767 || B - S * (Dmax < 255 ? Dmax : 255) < 0))
        return A4C_ERR_UNSUPPORTED;
    if (ldq % 16 || ldk % 16 || ldv % 16 || ldo % 16) return A4C_ERR_ALIGNMENT;
    if (batch > 1 && (stride_q % 16 || stride_k % 16 || stride_v % 16 || stride_o % 16)) return A4C_ERR_ALIGNMENT;
    if (((uintptr_t)q | (uintptr_t)k | (uintptr_t)v | (uintptr_t)out) & 15u) return A4C_ERR_ALIGNMENT;
    if (ldq < DH || ldk < DH || ldv < DH || ldo < DH) return A4C_ERR_INVALID_ARG;
    const long long items = batch * ((sq + BM - 1) / BM) * heads;
    if (batch > 2147483647LL || heads > 65535 || items > 2147483647LL) return A4C_ERR_TOO_LARGE;
    return A4C_OK;
}

int a4c_launch_attention_tc(const void* q, long long ldq, long long stride_q, const void* k, long long ldk,
                            long long stride_k, const void* v, long long ldv, long long stride_v, void* out,
                            long long ldo, long long stride_o, long long batch, int sq, int sk, int dh, int qk_shift,
                            int pv_shift, int rounding, int sm_mode, int B, int S, int Dmax, int inv_shift, int use_clb,
                            int exp_kq, int heads, long long hstride_q, long long hstride_k, long long hstride_v,
                            long long hstride_o, int* status_word, cudaStream_t stream) {
    const int sup = a4c_attention_tc_supported(q, ldq, stride_q, k, ldk, stride_k, v, ldv, stride_v, out, ldo, stride_o,
                                               batch, sq, sk, dh, qk_shift, pv_shift, sm_mode, B, S, Dmax, inv_shift,
                                               heads, hstride_q, hstride_k, hstride_v, hstride_o);
    if (sup != A4C_OK) return sup;
    if (rounding < 0 || rounding >= A4C_RND_COUNT) return A4C_ERR_INVALID_ARG;
    if (batch == 0) return A4C_OK;
    CUtensorMap mq, mk, mv;
    // one dimension order for the three maps: heads innermost when every operand's heads are column slices of a row
    const bool head_inner = heads > 1 && hstride_q < ldq && hstride_k < ldk && hstride_v < ldv;
    if (!make_head_map(&mq, q, sq, heads, batch, ldq, hstride_q, stride_q, head_inner) ||
        !make_head_map(&mk, k, sk, heads, batch, ldk, hstride_k, stride_k, head_inner) ||
        !make_head_map(&mv, v, sk, heads, batch, ldv, hstride_v, stride_v, head_inner))
        return A4C_ERR_CUDA;
    AttnArgs g;
    g.out = (uint8_t*)out; g.ldo = ldo; g.stride_o = stride_o; g.hstride_o = heads > 1 ? hstride_o : 0; g.batch = batch;
    g.sq = sq; g.heads = heads; g.head_inner = head_inner ? 1 : 0;
    g.m_tiles = (sq + BM - 1) / BM;
    g.shift1 = qk_shift; g.shift2 = pv_shift;
    const RoundParams r1 = make_round_params(qk_shift, rounding), r2 = make_round_params(pv_shift, rounding);
    g.mask1 = r1.mask; g.c01 = r1.c0; g.mask2 = r2.mask; g.c02 = r2.c0;
    const bool pre_clamp = rounding == A4C_RND_POSITIVE_INF && qk_shift >= 1 && qk_shift <= 22 && pv_shift >= 1 &&
                           pv_shift <= 22;
    g.xhi1 = g.addb1 = g.xlob1 = g.xhi2 = g.half2 = g.xlo2 = 0;
    g.fmul1 = g.fadd1 = g.fmul2 = g.fadd2 = 0.0f;
    const bool float_shift = pre_clamp && qk_shift <= 13 && pv_shift <= 13;
    if (float_shift) {
        g.fmul1 = 1.0f / (float)(1 << qk_shift);
        g.fadd1 = 12582912.0f - 12582912.0f * g.fmul1;
        g.fmul2 = 1.0f / (float)(1 << pv_shift);
        g.fadd2 = 12582912.0f - 12582912.0f * g.fmul2;
    }
    if (pre_clamp) {
        g.xhi1 = 127 * (1 << qk_shift);
        g.addb1 = (1 << (qk_shift - 1)) + 128 * (1 << qk_shift);
        g.xlob1 = -128 * (1 << qk_shift) + g.addb1;
        g.xhi2 = 127 * (1 << pv_shift);
        g.half2 = 1 << (pv_shift - 1);
        g.xlo2 = -128 * (1 << pv_shift) + g.half2;
    }
    g.mode = sm_mode; g.B = B; g.S = S; g.Dmax = Dmax; g.inv_shift = inv_shift; g.use_clb = use_clb; g.exp_kq = exp_kq;
    g.status = status_word;
    int dev = 0, sms = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const long long items = batch * g.m_tiles * heads;
    const int grid = (int)(items < sms ? items : sms);
    cudaError_t err;
    if (qk_shift == 0) err = launch_mode<-1>(mq, mk, mv, g, grid, stream);
    else if (float_shift) err = launch_mode<MODE_HALF_UP_FLOAT>(mq, mk, mv, g, grid, stream);
    else if (pre_clamp) err = launch_mode<MODE_HALF_UP_CLAMP>(mq, mk, mv, g, grid, stream);
    else switch (rounding) {
        case A4C_RND_FLOOR: err = launch_mode<A4C_RND_FLOOR>(mq, mk, mv, g, grid, stream); break;
        case A4C_RND_CEIL: err = launch_mode<A4C_RND_CEIL>(mq, mk, mv, g, grid, stream); break;
        case A4C_RND_POSITIVE_INF: err = launch_mode<A4C_RND_POSITIVE_INF>(mq, mk, mv, g, grid, stream); break;
        case A4C_RND_NEGATIVE_INF: err = launch_mode<A4C_RND_NEGATIVE_INF>(mq, mk, mv, g, grid, stream); break;
        case A4C_RND_SYMMETRIC_INF: err = launch_mode<A4C_RND_SYMMETRIC_INF>(mq, mk, mv, g, grid, stream); break;
        case A4C_RND_SYMMETRIC_ZERO: err = launch_mode<A4C_RND_SYMMETRIC_ZERO>(mq, mk, mv, g, grid, stream); break;
        case A4C_RND_CONV_EVEN: err = launch_mode<A4C_RND_CONV_EVEN>(mq, mk, mv, g, grid, stream); break;
        default: err = launch_mode<A4C_RND_CONV_ODD>(mq, mk, mv, g, grid, stream); break;
    }
    return err == cudaSuccess ? A4C_OK : A4C_ERR_CUDA;
}
