// int8 Dense whose epilogue adds a residual and normalises the row: one kernel for
//
//   d[m,n]   = clamp(round_shift(sum_k A[m,k]*W[k,n] + bias[n], shift), lo, 127)     dense_bias_relu.cpp:67-166
//   x[m,n]   = saturate_i8(d[m,n] + R[m,n])                                          elementwise_add.cpp:12-37 (SHIFT = 0)
//   out[m,:] = layer_norm(x[m,:]; gamma, beta)                                       layer_norm.cpp:15-121
//
// for layers exactly 256 features wide, the case where one 128 x 256 accumulator tile holds whole rows: a row's sum
// and sum of squares are then local to the two threads that read its TMEM lane, and neither d nor x is ever stored.
// The reference runs the three steps as three kernels over stream connections; as separate launches here the Dense
// output and the sum each make a round trip through HBM.
//
// Structure (one persistent CTA per SM, 19 warps):
//   warp 0      TMA producer of the operands: an A tile and a W tile per 128-byte k-block through a 3-slot ring, or,
//               when K <= 256, the whole weight matrix once and only A tiles through a deeper ring
//   warp 1      MMA issuer: tcgen05.mma.kind::i8, M = 128, N = 256, two 256-column accumulators in TMEM
//   warp 2      TMA producer of the residual tile (128 rows x 256 bytes as two 128-byte-swizzled boxes), one buffer per
//               epilogue group; it is a role of its own so that waiting for a buffer never holds back operand loads
//   warps 3-18  epilogue, two groups of eight warps on alternate tiles; the two warps of a TMEM lane quadrant split a
//               row's 256 columns in halves.  Pass 1: TMEM load 32 columns at a time, requantise, add the residual,
//               keep the 128 sums as packed bytes (biased by +128) in 32 registers, accumulate sum and sum of squares
//               with dp4a; the accumulator returns to the issuer and the residual buffer to warp 2 (so the next
//               residual tile of the group loads while this one is normalised); the two halves of a row exchange
//               their partial sums through shared memory (a bounded mbarrier meeting).  Pass 2: normalise out of the
//               registers on the FP32 pipe (the recipe of the row kernel, ln_math.cuh); every thread stores the 128
//               bytes of its half row (one 128-byte line) straight to global memory.
// The integer pipe bounds pass 1, so the common rounding tokens requantise off it: (acc + c) >> s is the upper word of
// one 64-bit multiply-add by 2^(32-s) (FMA pipe), and the saturation to 16 bits happens inside the instruction that
// packs two values (cvt.pack.sat); the +128 bias rides in the addend.
// Every wait is bounded: a wait that gives up records a code in the status word, the CTA stops issuing work, lets
// what is in flight land, frees its TMEM and returns.
#include <cuda.h>

#include <mutex>

#include "a4c_common.cuh"
#include "a4c_kernels.h"
#include "ln_math.cuh"
#include "tc_common.cuh"

namespace {

using namespace tc;

constexpr int BM = 128;
constexpr int BN = 256;                            // = the layer width
constexpr int BK = 128;
constexpr int UMMA_K = 32;
constexpr int STAGES = 3;                          // streaming ring (A + W per slot)
constexpr int A_BYTES = BM * BK;                   // 16 KB
constexpr int B_BYTES = BN * BK;                   // 32 KB
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;     // 48 KB
constexpr int OPERAND_BYTES = STAGES * STAGE_BYTES;   // 144 KB, shared by both operand layouts
constexpr int MAX_RING = 8;
constexpr int RES_BYTES = BM * BN;                 // 32 KB: residual in, normalised bytes out
constexpr int ACC_STAGES = 2;
constexpr int TMEM_COLS = ACC_STAGES * BN;         // 512
constexpr int GROUPS = 2;
constexpr int GROUP_WARPS = 8;
constexpr int GROUP_THREADS = GROUP_WARPS * 32;
constexpr int EPI_WARPS = GROUPS * GROUP_WARPS;
constexpr int FIRST_EPI_WARP = 3;
constexpr int NUM_THREADS = (FIRST_EPI_WARP + EPI_WARPS) * 32;   // 608
constexpr int HALF_COLS = BN / 2;
constexpr int DMODE_WIDE = 1;                      // floor / ceil / half-up / half-down, shift 2..31: multiply-add + packing saturation
constexpr int DMODE_WIDE_RELU = 2;                 // the same with ReLU
constexpr int DMODE_GENERIC = -2;                  // any token, any shift: run-time rounding parameters

struct Tail {
    int32_t bias[BN];
    uint32_t gam[BN];                              // FS 0: gamma / 128 (float); FS 1: gamma (float); FS 2: gamma (int)
    float bet[BN];                                 // (beta + rounding constant + output bias) * 2^-64
    int2 xch[GROUPS][2][2][BM];                    // [group][use parity][column half][row]: (sum, sum of squares)
    uint64_t full[MAX_RING];
    uint64_t empty[MAX_RING];
    uint64_t w_full;
    uint64_t tmem_full[ACC_STAGES];
    uint64_t tmem_empty[ACC_STAGES];
    uint64_t res_full[GROUPS];
    uint64_t res_empty[GROUPS];
    uint64_t pair[GROUPS][4];
    uint32_t tmem_base;
    volatile int abort_flag;
};
constexpr size_t SMEM_BYTES = 1024 + (size_t)OPERAND_BYTES + (size_t)GROUPS * RES_BYTES + sizeof(Tail);
static_assert(SMEM_BYTES <= 227 * 1024, "shared memory budget");

struct LArgs {
    const int32_t* bias;
    const int16_t* gamma;
    const int16_t* beta;
    long long M;
    int K;
    int num_m_tiles;
    int w_resident, a_stages;
    // Dense requantisation
    int lo;                      // -128, or 0 with ReLU
    RoundParams rp;
    int wide_mul;                // DMODE_WIDE: 2^(32 - shift)
    long long wide_add;          // (rounding constant + (128 << shift)) * 2^(32 - shift)
    uint32_t idesc;
    int8_t* out; long long ldo;
    // LayerNorm
    int eps_q0, rounding, s_out, c0_gamma, gamma_absmax;
    float c0_out;
    int* status;
};

// DMODE_WIDE: round_shift(t, s) + 128 for the floor-type tokens = upper word of t * 2^(32-s) + (c + (128 << s)) * 2^(32-s),
// exact for every int32 t (the 64-bit sum cannot overflow); t = acc + bias wraps like the reference's 32-bit accumulator.
__device__ __forceinline__ int requant_wide(int t, const LArgs& g) {
    long long d;
    asm("mad.wide.s32 %0, %1, %2, %3;" : "=l"(d) : "r"(t), "r"(g.wide_mul), "l"(g.wide_add));
    return (int)(d >> 32);
}
__device__ __forceinline__ int dp4a_uu(uint32_t a, uint32_t b, int c) {
    int d;
    asm("dp4a.u32.u32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}

// Four accumulators -> four bytes of saturate_i8(dense + residual) + 128.  `rw` holds the four residual bytes.
template <int DMODE>
__device__ __forceinline__ uint32_t dense_plus_residual(const uint32_t* a, int4 b, uint32_t rw, const LArgs& g) {
    using namespace lnm;
    uint32_t d01, d23;   // Dense outputs + 128 as 16-bit lanes in [0, 255]
    if (DMODE == DMODE_GENERIC) {
        const uint32_t d = pack4_i8(min(max(round_shift_i32((int)a[0] + b.x, g.rp), g.lo), 127),
                                    min(max(round_shift_i32((int)a[1] + b.y, g.rp), g.lo), 127),
                                    min(max(round_shift_i32((int)a[2] + b.z, g.rp), g.lo), 127),
                                    min(max(round_shift_i32((int)a[3] + b.w, g.rp), g.lo), 127)) ^ 0x80808080u;
        d01 = prmt(d, 0, 0x4140);
        d23 = prmt(d, 0, 0x4342);
    } else {
        d01 = __vimin_s16x2_relu(pack_sat_s16x2(requant_wide((int)a[1] + b.y, g), requant_wide((int)a[0] + b.x, g)), 0x00FF00FFu);
        d23 = __vimin_s16x2_relu(pack_sat_s16x2(requant_wide((int)a[3] + b.w, g), requant_wide((int)a[2] + b.z, g)), 0x00FF00FFu);
        if (DMODE == DMODE_WIDE_RELU) {
            d01 = __vimax3_s16x2(d01, 0x00800080u, 0x00800080u);
            d23 = __vimax3_s16x2(d23, 0x00800080u, 0x00800080u);
        }
    }
    // saturating Add in the biased domain (elementwise_add.cpp:30-33, SHIFT = 0): clamp(d + 128 + r, 0, 255) per lane
    const uint32_t x01 = __viaddmin_s16x2_relu(d01, prmt(rw, 0, 0x9180), 0x00FF00FFu);
    const uint32_t x23 = __viaddmin_s16x2_relu(d23, prmt(rw, 0, 0xB3A2), 0x00FF00FFu);
    return prmt(x01, x23, 0x6420);
}

__device__ __forceinline__ uint4 lds128(uint32_t a) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a));
    return v;
}

// Pass 1 of the epilogue for one thread: its 128 accumulator columns -> requantise -> + residual (saturating) ->
// packed bytes (biased by +128) in xw; partial sums of the biased bytes and of their squares in sx / sq.  The
// accumulator is released once its last columns are in registers.
template <int DMODE, bool HAS_BIAS>
__device__ __forceinline__ void pass_one(uint32_t taddr, uint32_t my_res, uint32_t sw, const int32_t* my_bias, const LArgs& g,
                                         uint64_t* acc_empty, uint32_t (&xw)[HALF_COLS / 4], int& sx, int& sq) {
    int sx0 = 0, sx1 = 0, sq0 = 0, sq1 = 0;
#pragma unroll
    for (int c = 0; c < HALF_COLS / 32; ++c) {
        uint32_t ra[32];
        tmem_ld32_async(taddr + (uint32_t)(c * 32), ra);
        tmem_ld_wait32(ra);
        if (c == HALF_COLS / 32 - 1) {
            tc_fence_before();
            mbar_arrive(acc_empty);
        }
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            const int piece = c * 2 + j;
            const uint4 rv = lds128(my_res + (((uint32_t)piece ^ sw) << 4));
            const uint32_t rw[4] = {rv.x, rv.y, rv.z, rv.w};
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const int4 b = HAS_BIAS ? *reinterpret_cast<const int4*>(my_bias + piece * 16 + q * 4) : make_int4(0, 0, 0, 0);
                const uint32_t x = dense_plus_residual<DMODE>(ra + j * 16 + q * 4, b, rw[q], g);
                xw[piece * 4 + q] = x;
                if (q & 1) { sx1 = dp4a_uu(x, 0x01010101u, sx1); sq1 = dp4a_uu(x, x, sq1); }
                else { sx0 = dp4a_uu(x, 0x01010101u, sx0); sq0 = dp4a_uu(x, x, sq0); }
            }
        }
    }
    sx = sx0 + sx1;
    sq = sq0 + sq1;
}

// Pass 2: normalise the packed (biased) bytes of xw (layer_norm.cpp:44-121 on the FP32 pipe, as the row kernel does) and
// store them: `orow` is this thread's 128-byte half row in global memory, or null for a row past the end.  CLAMP: fscale may leave int16 (inv_std * max|gamma| / 128 > 32767), a
// warp-uniform rarity that gets its own copy of the loop so that the common one carries no min / max per value.
template <int FS, bool CLAMP>
__device__ __forceinline__ void pass_two(const uint32_t (&xw)[HALF_COLS / 4], uint8_t* orow, uint32_t s_gam, uint32_t s_bet,
                                         int inv_std, float vdc, float c0g, float out_mul, int c0_gamma) {
    using namespace lnm;
    constexpr bool RN = FS == 0;
    const float inv_f = (float)inv_std;
#pragma unroll
    for (int piece = 0; piece < HALF_COLS / 16; ++piece) {
        uint32_t ow[4];
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            const uint32_t poff = (uint32_t)((piece * 16 + w * 4) * 4);
            float4 bq;
            asm volatile("ld.shared.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(bq.x), "=f"(bq.y), "=f"(bq.z), "=f"(bq.w) : "r"(s_bet + poff));
            const float bet[4] = {bq.x, bq.y, bq.z, bq.w};
            const uint4 gq = lds128(s_gam + poff);
            float F[4];
            if (FS == 0) {
                F[0] = __fmaf_rn(inv_f, __uint_as_float(gq.x), MAGIC); F[1] = __fmaf_rn(inv_f, __uint_as_float(gq.y), MAGIC);
                F[2] = __fmaf_rn(inv_f, __uint_as_float(gq.z), MAGIC); F[3] = __fmaf_rn(inv_f, __uint_as_float(gq.w), MAGIC);
            } else if (FS == 1) {
                // inv_std * gamma + c0 < 2^24 is exact; floor(. / 128) by a round-down FMA
                F[0] = __fmaf_rd(__fmaf_rn(inv_f, __uint_as_float(gq.x), c0g), 0.0078125f, MAGIC);
                F[1] = __fmaf_rd(__fmaf_rn(inv_f, __uint_as_float(gq.y), c0g), 0.0078125f, MAGIC);
                F[2] = __fmaf_rd(__fmaf_rn(inv_f, __uint_as_float(gq.z), c0g), 0.0078125f, MAGIC);
                F[3] = __fmaf_rd(__fmaf_rn(inv_f, __uint_as_float(gq.w), c0g), 0.0078125f, MAGIC);
            } else {
                F[0] = __uint_as_float((uint32_t)((inv_std * (int)gq.x + c0_gamma) >> 7) + MAGIC_BITS);
                F[1] = __uint_as_float((uint32_t)((inv_std * (int)gq.y + c0_gamma) >> 7) + MAGIC_BITS);
                F[2] = __uint_as_float((uint32_t)((inv_std * (int)gq.z + c0_gamma) >> 7) + MAGIC_BITS);
                F[3] = __uint_as_float((uint32_t)((inv_std * (int)gq.w + c0_gamma) >> 7) + MAGIC_BITS);
            }
            if (CLAMP) {
#pragma unroll
                for (int k = 0; k < 4; ++k) F[k] = fminf(fmaxf(F[k], MAGIC - 32768.0f), MAGIC + 32767.0f);
            }
            const uint32_t xb = xw[piece * 4 + w];
            const float xf[4] = {byte_to_f23<0>(xb), byte_to_f23<1>(xb), byte_to_f23<2>(xb), byte_to_f23<3>(xb)};
            int o[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const float vd = xf[k] - vdc;                                      // x - mu, exact
                const float fs = __fmaf_rn(F[k], TWO_M64, -MAGIC * TWO_M64);       // fscale * 2^-64, exact
                const float acc = __fmaf_rn(vd, fs, bet[k]);                       // (vd*fscale + beta + c) * 2^-64
                const float r = RN ? __fmaf_rn(acc, out_mul, 0.0f) : __fmaf_rd(acc, out_mul, 0.0f);
                o[k] = __float_as_int(r);                                          // round(.) + 128 as a (signed) integer
            }
            ow[w] = pack_sat_u8x4(o[0], o[1], o[2], o[3]) ^ 0x80808080u;   // clamp(., 0, 255), pack, un-bias
        }
        if (orow != nullptr) *reinterpret_cast<uint4*>(orow + piece * 16) = make_uint4(ow[0], ow[1], ow[2], ow[3]);
    }
}

// FS as in the row kernel: 0 = conv_even; 1 = floor-type tokens with |gamma| <= 511; 2 = floor-type tokens, any gamma.
template <int DMODE, int FS>
__global__ void __launch_bounds__(NUM_THREADS, 1)
dense_ln_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                const __grid_constant__ CUtensorMap tmap_r, LArgs g) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* res = smem + OPERAND_BYTES;                         // 1024-byte aligned: whole swizzle atoms
    Tail* tail = reinterpret_cast<Tail*>(res + (size_t)GROUPS * RES_BYTES);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int num_kb = (g.K + BK - 1) / BK;
    const int my_tiles = (int)blockIdx.x < g.num_m_tiles ? (g.num_m_tiles - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x : 0;

    if (threadIdx.x == 0) {
        for (int s = 0; s < MAX_RING; ++s) { mbar_init(&tail->full[s], 1); mbar_init(&tail->empty[s], 1); }
        mbar_init(&tail->w_full, 1);
        for (int s = 0; s < ACC_STAGES; ++s) { mbar_init(&tail->tmem_full[s], 1); mbar_init(&tail->tmem_empty[s], GROUP_THREADS); }
        for (int s = 0; s < GROUPS; ++s) {
            mbar_init(&tail->res_full[s], 1);
            mbar_init(&tail->res_empty[s], GROUP_WARPS);
            for (int q = 0; q < 4; ++q) mbar_init(&tail->pair[s][q], 2);
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
        // ---------------- operand producer ----------------
        if (lane == 0 && my_tiles > 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            if (g.w_resident) {
                uint8_t* a_ring = smem + (size_t)num_kb * B_BYTES;
                mbar_arrive_expect_tx(&tail->w_full, (uint32_t)(num_kb * B_BYTES));
                for (int kb = 0; kb < num_kb; ++kb) tma_load_2d(smem + (size_t)kb * B_BYTES, &tmap_b, &tail->w_full, kb * BK, 0);
                for (int i = 0; ok && i < my_tiles; ++i) {
                    const int m0 = ((int)blockIdx.x + i * (int)gridDim.x) * BM;
                    for (int kb = 0; kb < num_kb; ++kb) {
                        ok = mbar_wait(&tail->empty[stage], phase ^ 1u, abort_flag, g.status, 171);
                        if (!ok) break;
                        mbar_arrive_expect_tx(&tail->full[stage], (uint32_t)A_BYTES);
                        tma_load_2d(a_ring + (size_t)stage * A_BYTES, &tmap_a, &tail->full[stage], kb * BK, m0);
                        if (++stage == g.a_stages) { stage = 0; phase ^= 1u; }
                    }
                }
            } else {
                for (int i = 0; ok && i < my_tiles; ++i) {
                    const int m0 = ((int)blockIdx.x + i * (int)gridDim.x) * BM;
                    for (int kb = 0; kb < num_kb; ++kb) {
                        ok = mbar_wait(&tail->empty[stage], phase ^ 1u, abort_flag, g.status, 171);
                        if (!ok) break;
                        uint8_t* sa = smem + (size_t)stage * STAGE_BYTES;
                        mbar_arrive_expect_tx(&tail->full[stage], (uint32_t)STAGE_BYTES);
                        tma_load_2d(sa, &tmap_a, &tail->full[stage], kb * BK, m0);
                        tma_load_2d(sa + A_BYTES, &tmap_b, &tail->full[stage], kb * BK, 0);
                        if (++stage == STAGES) { stage = 0; phase ^= 1u; }
                    }
                }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0 && my_tiles > 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            const int ring = g.w_resident ? g.a_stages : STAGES;
            const uint32_t a_ring = smem_u32(smem) + (g.w_resident ? (uint32_t)(num_kb * B_BYTES) : 0u);
            const uint32_t slot_bytes = g.w_resident ? (uint32_t)A_BYTES : (uint32_t)STAGE_BYTES;
            if (g.w_resident) {
                ok = mbar_wait(&tail->w_full, 0u, abort_flag, g.status, 175);
                tc_fence_after();
            }
            for (int i = 0; ok && i < my_tiles; ++i) {
                const int acc = i & 1;
                // this kernel runs at the speed of its epilogue: the issuer mostly waits here, and a polling wait took a
                // third of all issued instructions from the epilogue warps of its scheduler; it sleeps in the barrier instead
                ok = mbar_wait(&tail->tmem_empty[acc], ((uint32_t)(i >> 1) & 1u) ^ 1u, abort_flag, g.status, 172);
                if (!ok) break;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + (uint32_t)(acc * BN);
                for (int kb = 0; kb < num_kb; ++kb) {
                    ok = mbar_wait_fast(&tail->full[stage], phase, abort_flag, g.status, 173);
                    if (!ok) break;
                    tc_fence_after();
                    const uint32_t sa = a_ring + (uint32_t)stage * slot_bytes;
                    const uint64_t adesc = make_smem_desc(sa);
                    const uint64_t bdesc = make_smem_desc(g.w_resident ? smem_u32(smem) + (uint32_t)(kb * B_BYTES) : sa + A_BYTES);
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k)
                        umma_i8(d_tmem, adesc + (uint64_t)(k * (UMMA_K >> 4)), bdesc + (uint64_t)(k * (UMMA_K >> 4)), g.idesc,
                                (uint32_t)((kb | k) != 0));
                    umma_commit(&tail->empty[stage]);
                    if (++stage == ring) { stage = 0; phase ^= 1u; }
                }
                if (!ok) break;
                umma_commit(&tail->tmem_full[acc]);
            }
        }
        __syncwarp();
    } else if (warp == 2) {
        // ---------------- residual producer: local tile i into the buffer of group i & 1 ----------------
        if (lane == 0) {
            for (int i = 0; i < my_tiles; ++i) {
                const int buf = i & 1;
                if (!mbar_wait(&tail->res_empty[buf], ((uint32_t)(i >> 1) & 1u) ^ 1u, abort_flag, g.status, 176)) break;
                const int m0 = ((int)blockIdx.x + i * (int)gridDim.x) * BM;
                uint8_t* dst = res + (size_t)buf * RES_BYTES;
                mbar_arrive_expect_tx(&tail->res_full[buf], (uint32_t)RES_BYTES);
                tma_load_2d(dst, &tmap_r, &tail->res_full[buf], 0, m0);
                tma_load_2d(dst + RES_BYTES / 2, &tmap_r, &tail->res_full[buf], HALF_COLS, m0);
            }
        }
        __syncwarp();
    } else {
        // ---------------- epilogue ----------------
        using namespace lnm;
        const int e = warp - FIRST_EPI_WARP;
        const int grp = e >> 3;              // which accumulator, residual buffer and tiles
        const int hf = (e >> 2) & 1;         // which 128 columns of the row
        const int quad = warp & 3;           // TMEM lane quadrant this warp may read
        const int r_in_tile = quad * 32 + lane;
        // parameters once per CTA
        for (int c = threadIdx.x - FIRST_EPI_WARP * 32; c < BN; c += EPI_WARPS * 32) {
            tail->bias[c] = g.bias != nullptr ? __ldg(g.bias + c) : 0;
            const int gv = g.gamma[c];
            if (FS == 0) tail->gam[c] = __float_as_uint((float)gv * 0.0078125f);
            else if (FS == 1) tail->gam[c] = __float_as_uint((float)gv);
            else tail->gam[c] = (uint32_t)gv;
            tail->bet[c] = ((float)g.beta[c] + g.c0_out) * TWO_M64;
        }
        asm volatile("bar.sync 1, %0;" :: "n"(EPI_WARPS * 32) : "memory");

        const bool has_bias = g.bias != nullptr;
        const float out_mul = __int_as_float((127 - (g.s_out + 85)) << 23);   // 2^-(s_out + 85)
        const float c0g = (float)g.c0_gamma;
        const int clamp_threshold = (32767 * 128) / g.gamma_absmax;           // inv_std above this may overflow int16
        const bool nearest = g.rounding == A4C_RND_CONV_EVEN || g.rounding == A4C_RND_POSITIVE_INF ||
                             g.rounding == A4C_RND_NEGATIVE_INF;
        const uint32_t my_res = smem_u32(res) + (uint32_t)(grp * RES_BYTES + hf * (RES_BYTES / 2) + r_in_tile * 128);
        const uint32_t sw = (uint32_t)(lane & 7);   // 128-byte swizzle: 16-byte piece p of row r sits at piece p ^ (r & 7)
        const uint32_t taddr = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(grp * BN + hf * HALF_COLS);
        const uint32_t s_gam = smem_u32(tail->gam) + (uint32_t)(hf * HALF_COLS * 4);
        const uint32_t s_bet = smem_u32(tail->bet) + (uint32_t)(hf * HALF_COLS * 4);
        const int32_t* my_bias = tail->bias + hf * HALF_COLS;
        uint64_t* pair_bar = &tail->pair[grp][quad];

        for (int i = grp; i < my_tiles; i += GROUPS) {
            const uint32_t ph = (uint32_t)(i >> 1) & 1u;
            if (!mbar_wait(&tail->tmem_full[grp], ph, abort_flag, g.status, 174)) break;
            if (!mbar_wait(&tail->res_full[grp], ph, abort_flag, g.status, 177)) break;
            tc_fence_after();

            // ---- pass 1: x = saturate(requant(acc) + residual) as packed bytes, row statistics ----
            uint32_t xw[HALF_COLS / 4];
            int sx, sq;
            if (has_bias) pass_one<DMODE, true>(taddr, my_res, sw, my_bias, g, &tail->tmem_empty[grp], xw, sx, sq);
            else pass_one<DMODE, false>(taddr, my_res, sw, my_bias, g, &tail->tmem_empty[grp], xw, sx, sq);
            // the residual bytes are consumed: the buffer goes back to warp 2, which loads the group's next tile into it
            // while this one is normalised
            __syncwarp();
            if (lane == 0) mbar_arrive(&tail->res_empty[grp]);   // one of the group's eight warps
            // ---- the two halves of a row meet ----
            tail->xch[grp][ph][hf][r_in_tile] = make_int2(sx, sq);
            __syncwarp();
            if (lane == 0) mbar_arrive(pair_bar);
            if (!mbar_wait_fast(pair_bar, ph, abort_flag, g.status, 178)) break;
            const int2 other = tail->xch[grp][ph][hf ^ 1][r_in_tile];
            // sums of the biased bytes b = x + 128 over the 256 columns -> sums of x
            const int sum_b = sx + other.x;
            const int sum_x = sum_b - 128 * BN;
            const int sum_sq = sq + other.y - 256 * sum_b + 128 * 128 * BN;
            // layer_norm.cpp:23-31 with 256 columns
            const int mu = (sum_x + (BN >> 1)) >> 8;
            const int centered = (int)((uint32_t)sum_sq - 2u * (uint32_t)mu * (uint32_t)sum_x + (uint32_t)BN * (uint32_t)mu * (uint32_t)mu);
            int var = centered >> 8;
            var = max(var, 0) + g.eps_q0;
            const int inv_std = inv_std_q15(var, g.rounding, nearest);
            const bool need_clamp = __any_sync(0xffffffffu, inv_std > clamp_threshold);
            const float vdc = 8388608.0f + 128.0f + (float)mu;   // (2^23 + b) - vdc = x - mu

            // ---- pass 2: normalise out of the registers, one 128-byte line per thread straight to global memory ----
            const long long row = (long long)((int)blockIdx.x + i * (int)gridDim.x) * BM + r_in_tile;
            uint8_t* orow = row < g.M ? reinterpret_cast<uint8_t*>(g.out) + row * g.ldo + hf * HALF_COLS : nullptr;
            if (need_clamp) pass_two<FS, true>(xw, orow, s_gam, s_bet, inv_std, vdc, c0g, out_mul, g.c0_gamma);
            else pass_two<FS, false>(xw, orow, s_gam, s_bet, inv_std, vdc, c0g, out_mul, g.c0_gamma);
        }
    }

    // ---------------- teardown ----------------
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

// 2-D uint8 map over a row-major [rows, cols] matrix of pitch `ld`, box = [box_rows, 128 bytes], 128-byte swizzle
bool make_map(CUtensorMap* map, const void* base, long long rows, long long cols, long long ld, int box_rows,
              CUtensorMapL2promotion promo) {
    EncodeTiledFn fn = get_encode_fn();
    if (!fn) return false;
    cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld};
    cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, promo, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int DMODE, int FS>
cudaError_t launch_one(const CUtensorMap& ma, const CUtensorMap& mb, const CUtensorMap& mr, const LArgs& g, int grid,
                       cudaStream_t s) {
    static tc::SmemOptIn opt_in;
    const cudaError_t e = opt_in.ensure(dense_ln_kernel<DMODE, FS>, SMEM_BYTES);
    if (e != cudaSuccess) return e;
    dense_ln_kernel<DMODE, FS><<<grid, NUM_THREADS, SMEM_BYTES, s>>>(ma, mb, mr, g);
    return cudaGetLastError();
}

int g_dense_ln_enabled = 1;

}  // namespace

void a4c_dense_ln_set_enabled(int on) { g_dense_ln_enabled = on ? 1 : 0; }

// 0 when the single kernel takes the problem; A4C_ERR_UNSUPPORTED sends the caller to the three separate steps.
int a4c_dense_ln_supported(long long M, int K, int N, long long lda, long long ldw, long long ldr, long long ldo,
                           int shift, int rounding, int out_shift, int eps_q0, int gamma_absmax) {
    if (!g_dense_ln_enabled) return A4C_ERR_UNSUPPORTED;
    if (N != BN || K < 16 || M < 1 || M > 2147483647LL - BM) return A4C_ERR_UNSUPPORTED;
    if (lda % 16 || ldw % 16 || ldr % 16 || ldo % 16 || lda < K || ldw < K || ldr < N || ldo < N) return A4C_ERR_UNSUPPORTED;
    if (shift < 0 || shift > 31) return A4C_ERR_UNSUPPORTED;
    // the normalisation on the FP32 pipe has the row kernel's proofs (rowops_fast.cu)
    const int s_out = 15 - out_shift;
    if (s_out < 2 || s_out > 30 || gamma_absmax <= 0 || gamma_absmax > 16383 || eps_q0 < 1 || eps_q0 > (1 << 20))
        return A4C_ERR_UNSUPPORTED;
    if (rounding < 0 || rounding == A4C_RND_SYMMETRIC_INF || rounding == A4C_RND_SYMMETRIC_ZERO || rounding >= A4C_RND_CONV_ODD)
        return A4C_ERR_UNSUPPORTED;
    return A4C_OK;
}

int a4c_launch_dense_ln(const void* A, long long lda, int a_unsigned, const void* Wt, long long ldw, const int32_t* bias,
                        int shift, int relu, const int8_t* residual, long long ldr, const int16_t* gamma,
                        const int16_t* beta, int8_t* out, long long ldo, long long M, int K, int N, int eps_q0,
                        int out_shift, int rounding, int gamma_absmax, int* status_word, cudaStream_t stream) {
    const int sup = a4c_dense_ln_supported(M, K, N, lda, ldw, ldr, ldo, shift, rounding, out_shift, eps_q0, gamma_absmax);
    if (sup != A4C_OK) return sup;
    if ((((uintptr_t)A | (uintptr_t)Wt | (uintptr_t)residual | (uintptr_t)out) & 15u) != 0) return A4C_ERR_ALIGNMENT;
    if (status_word == nullptr || gamma == nullptr || beta == nullptr) return A4C_ERR_INVALID_ARG;
    CUtensorMap ma, mb, mr;
    if (!make_map(&ma, A, M, K, lda, BM, CU_TENSOR_MAP_L2_PROMOTION_L2_256B) ||
        !make_map(&mb, Wt, N, K, ldw, BN, CU_TENSOR_MAP_L2_PROMOTION_L2_256B) ||
        !make_map(&mr, residual, M, N, ldr, BM, CU_TENSOR_MAP_L2_PROMOTION_L2_256B))
        return A4C_ERR_CUDA;
    LArgs g;
    g.bias = bias; g.gamma = gamma; g.beta = beta; g.M = M; g.K = K;
    g.num_m_tiles = (int)((M + BM - 1) / BM);
    g.lo = relu ? 0 : -128;
    g.rp = make_round_params(shift, rounding);
    // floor-type tokens with a shift of 2..31: (t + c) >> s as the upper word of a 64-bit multiply-add
    const bool wide = shift >= 2 && (rounding == A4C_RND_FLOOR || rounding == A4C_RND_CEIL ||
                                     rounding == A4C_RND_POSITIVE_INF || rounding == A4C_RND_NEGATIVE_INF);
    g.wide_mul = wide ? (int)(1u << (32 - shift)) : 0;
    g.wide_add = wide ? ((long long)g.rp.c0 + (128ll << shift)) << (32 - shift) : 0;
    g.out = out; g.ldo = ldo;
    g.idesc = make_idesc(BM, BN, a_unsigned != 0);
    g.eps_q0 = eps_q0; g.rounding = rounding; g.s_out = 15 - out_shift; g.gamma_absmax = gamma_absmax;
    g.c0_gamma = 0; g.c0_out = 0.0f;
    switch (rounding) {
        case A4C_RND_CEIL: g.c0_gamma = 127; g.c0_out = (float)((1 << g.s_out) - 1); break;
        case A4C_RND_POSITIVE_INF: g.c0_gamma = 64; g.c0_out = (float)(1 << (g.s_out - 1)); break;
        case A4C_RND_NEGATIVE_INF: g.c0_gamma = 63; g.c0_out = (float)((1 << (g.s_out - 1)) - 1); break;
        default: break;
    }
    g.c0_out += (float)(128 << g.s_out);   // outputs are produced biased by +128
    g.status = status_word;
    const int num_kb = (K + BK - 1) / BK;
    g.w_resident = num_kb <= 2 ? 1 : 0;   // the whole weight matrix beside at least five A slots
    g.a_stages = STAGES;
    if (g.w_resident) {
        const int slots = (OPERAND_BYTES - num_kb * B_BYTES) / A_BYTES;
        g.a_stages = slots < MAX_RING ? slots : MAX_RING;
    }
    int dev = 0, sms = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const int grid = g.num_m_tiles < sms ? g.num_m_tiles : sms;
    const int fs = rounding == A4C_RND_CONV_EVEN ? 0 : (gamma_absmax <= 511 ? 1 : 2);
    cudaError_t err;
    if (fs == 0) err = launch_one<DMODE_GENERIC, 0>(ma, mb, mr, g, grid, stream);
    else if (wide && !relu) err = fs == 1 ? launch_one<DMODE_WIDE, 1>(ma, mb, mr, g, grid, stream)
                                          : launch_one<DMODE_WIDE, 2>(ma, mb, mr, g, grid, stream);
    else if (wide) err = fs == 1 ? launch_one<DMODE_WIDE_RELU, 1>(ma, mb, mr, g, grid, stream)
                                 : launch_one<DMODE_WIDE_RELU, 2>(ma, mb, mr, g, grid, stream);
    else err = fs == 1 ? launch_one<DMODE_GENERIC, 1>(ma, mb, mr, g, grid, stream)
                       : launch_one<DMODE_GENERIC, 2>(ma, mb, mr, g, grid, stream);
    return err == cudaSuccess ? A4C_OK : A4C_ERR_CUDA;
}
