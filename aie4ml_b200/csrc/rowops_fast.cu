// Bandwidth-oriented LayerNorm and Softmax row kernels (the common cases of rowops.cu).
//
// Data movement: every warp owns a ring of slots in shared memory that is filled by bulk asynchronous
// copies (cp.async.bulk, completion on an mbarrier): the input rows and, when a saturating Add is fused,
// the addend rows.  Many rows per SM are in flight without holding registers, nothing in the row loop waits
// on a global load, and results leave through 128-bit global stores.
//
// Arithmetic: the integer recipes of the aie4ml kernels (layer_norm.cpp:15-121, softmax.cpp:20-88 and
// :252-384) are evaluated on the FP32 pipe where that is provably exact:
//   * an integer n with |n| < 2^22 is carried as the float MAGIC + n (MAGIC = 1.5 * 2^23), whose low
//     mantissa bits are n in two's complement;
//   * round(v / 2^s) for floor / ceil / half-up / half-down / half-even is ONE fused multiply-add with the
//     matching IEEE rounding direction (constants of the floor-type modes folded into an addend): the FMA
//     forms the exact product and rounds once;
//   * the final rounding writes into a SUBNORMAL: fma(v * 2^-64, 2^-(s+85), 0) has the bit pattern
//     sign | round(v / 2^s), so the integer result needs no conversion, and min.s32.relu clamps it to
//     [0, 255] in one instruction (outputs are produced biased by +128 and un-biased with one XOR per word);
//   * products such as (x - mu) * fscale + beta stay below 2^24 in magnitude, so they are exact.
// Modes or parameters outside those proofs (symmetric rounding, conv_odd, |gamma| > 16383, shifts < 2,
// int16 softmax output, negative HCCS scores, inv_shift > 22, rows longer than 2048 / 1024) take the generic
// integer kernels of rowops.cu.
#include <type_traits>

#include "a4c_common.cuh"
#include "a4c_kernels.h"
#include "ln_math.cuh"

namespace {

using namespace lnm;

constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;
// ---- shared-memory / barrier primitives on 32-bit shared addresses ----------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ uint4 lds128(uint32_t a) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a));
    return v;
}
__device__ __forceinline__ float4 lds128f(uint32_t a) {
    float4 v;
    asm volatile("ld.shared.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(a));
    return v;
}
__device__ __forceinline__ float lds32f(uint32_t a) {
    float v;
    asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(a));
    return v;
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" :: "r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" :: "r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.b32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
// Bounded wait; on timeout records `code` in the status word and returns false.
__device__ __noinline__ bool mbar_wait_slow(uint32_t bar, uint32_t parity, int* status, int code) {
    const uint64_t t0 = a4c_globaltimer();
    for (uint32_t it = 1;; ++it) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((it & 255u) == 0 && a4c_globaltimer() - t0 > A4C_SPIN_LIMIT_NS) {
            atomicCAS(status, 0, code);
            return false;
        }
    }
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, int* status, int code) {
    if (mbar_try_wait(bar, parity)) return true;
    return mbar_wait_slow(bar, parity, status, code);
}
__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 :: "r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
__device__ __forceinline__ void stg16(void* p, uint4 v) {
    asm volatile("st.global.v4.u32 [%0], {%1,%2,%3,%4};" :: "l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
// Sum / maximum over the G = 2^k adjacent lanes that share a row.  A whole warp (G = 32) uses the warp-wide reduce
// instruction.  Given several member masks in one warp that instruction is replayed once per mask (eight times for
// G = 4: 1.3x the run time of a whole LayerNorm at 256 columns), so smaller groups use an xor butterfly, which costs
// log2(G) shuffles for every group at once.
__device__ __forceinline__ int group_sum(int v, int G) {
    if (G == 32) return __reduce_add_sync(0xffffffffu, v);
    for (int d = G >> 1; d > 0; d >>= 1) v += __shfl_xor_sync(0xffffffffu, v, d);
    return v;
}
__device__ __forceinline__ int group_max(int v, int G) {
    if (G == 32) return (int)__reduce_max_sync(0xffffffffu, v);
    for (int d = G >> 1; d > 0; d >>= 1) v = max(v, __shfl_xor_sync(0xffffffffu, v, d));
    return v;
}
// A row of `cols` bytes is nchunks 16-byte chunks.  G lanes share a row (lane gl takes chunks gl, gl + G, ...),
// a warp works on R = 32 / G rows at once.  Rows sit `pitch` bytes apart in a ring slot: when fewer than
// eight lanes share a row, a quarter-warp's 128-bit loads touch several rows, and the pad of G * 16 bytes
// puts those rows on different banks.
struct RowGeom {
    int nchunks, G, R, pitch;
    int contig;   // the R rows of an item are adjacent in memory and in the slot: one copy brings all of them
};

// One warp's ring.  A slot holds R input rows and, with a fused Add, R addend rows behind them.
struct Ring {
    uint32_t slots;   // shared address of slot 0
    uint32_t bars;    // shared address of barrier 0
    uint32_t slot_bytes;
    uint32_t add_off; // offset of the addend rows inside a slot
    const uint8_t* x; long long ldx;
    const uint8_t* addend; long long ldadd;  // byte pitch
    long long rows;
    uint32_t row_bytes;   // bytes copied per row
    uint32_t pitch;       // distance between rows inside a slot (row_bytes + bank-spreading pad)
    int R;
    int contig;           // rows are adjacent in global memory and pitch == row_bytes: one copy per item and operand
};

// Whole warp: lane 0 arms the barrier, lane r (and r + 32, ...) issues the copies of row r, so the R rows of
// an item are requested in parallel instead of one after another.  A copy may complete before the barrier
// has been armed: the phase cannot finish until lane 0's arrival.
__device__ __forceinline__ void ring_issue(const Ring& c, long long item, int stage, int lane) {
    const long long row0 = item * c.R;
    long long nrows = c.rows - row0;
    if (nrows > c.R) nrows = c.R;
    const uint32_t bar = c.bars + stage * 8;
    const uint32_t dst = c.slots + stage * c.slot_bytes;
    if (c.contig) {
        if (lane == 0) {
            const uint32_t bytes = (uint32_t)nrows * c.row_bytes;
            mbar_expect_tx(bar, bytes * (c.addend ? 2u : 1u));
            bulk_load(dst, c.x + row0 * c.ldx, bytes, bar);
            if (c.addend) bulk_load(dst + c.add_off, c.addend + row0 * c.ldadd, bytes, bar);
        }
        return;
    }
    if (lane == 0) mbar_expect_tx(bar, (uint32_t)nrows * c.row_bytes * (c.addend ? 2u : 1u));
    if (lane < (int)nrows) {
        bulk_load(dst + lane * c.pitch, c.x + (row0 + lane) * c.ldx, c.row_bytes, bar);
        if (c.addend) bulk_load(dst + c.add_off + lane * c.pitch, c.addend + (row0 + lane) * c.ldadd, c.row_bytes, bar);
    }
}

// ------------------------------------------------------------------------------------------------
// LayerNorm
// ------------------------------------------------------------------------------------------------
struct LnFastArgs {
    const int8_t* x; long long ldx;
    const int16_t* gamma; const int16_t* beta;
    const int8_t* addend; long long ldadd;
    int8_t* out; long long ldo;
    long long rows; int cols, log2c, eps_q0, rounding;
    int s_out;          // 15 - out_shift (>= 2)
    int c0_gamma;       // rounding constant of the (>> 7) step for the floor-type modes
    float c0_out;       // rounding constant + output bias (128 << s_out), folded into beta
    int gamma_absmax;
    int stages;
    RowGeom geom;
    int* status;
};

// FS = 0: conv_even, fscale = rne(inv_std * gamma / 128) in one nearest-even FMA
// FS = 1: floor-type modes with |gamma| <= 511: inv_std * gamma + c0 is exact in FP32, then one round-down FMA
// FS = 2: floor-type modes with larger gamma: integer multiply-add and shift
template <int NCH, int FS, int ADD>
__global__ void __launch_bounds__(kThreads) layernorm_fast_kernel(LnFastArgs a) {
    constexpr bool HAS_ADD = ADD == 1;   // saturating Add of the result (after the normalisation)
    constexpr bool PRE_ADD = ADD == 2;   // saturating Add of the input (before the statistics)
    constexpr bool RING_ADD = ADD != 0;  // a second row travels through the ring
    extern __shared__ __align__(128) uint8_t smem[];
    // layout: gamma[NCH*4*32*4] | beta[same] | barriers | ring.  Parameters are stored lane-major: position
    // ((j*4 + w)*32 + lane)*4 + k holds column (j*G + lane)*16 + w*4 + k, so for fixed (j, w) a row group reads
    // consecutive 16-byte quads (conflict-free) at an offset that is a compile-time constant.
    constexpr int kParamFloats = NCH * 4 * 32 * 4;
    const uint32_t s_base = smem_u32(smem);
    const uint32_t s_gam = s_base, s_bet = s_base + kParamFloats * 4, s_bar = s_base + kParamFloats * 8;
    const int cols = a.cols;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int G = a.geom.G, R = a.geom.R;
    const int sub = lane / G, gl = lane % G;
    constexpr bool RN = FS == 0;

    for (int c = threadIdx.x; c < cols; c += kThreads) {
        const int chunk = c >> 4, w = (c >> 2) & 3, k = c & 3;
        const int pos = (((chunk / G) * 4 + w) * 32 + (chunk % G)) * 4 + k;
        const int g = a.gamma[c];
        if (FS == 0) reinterpret_cast<float*>(smem)[pos] = (float)g * 0.0078125f;
        else if (FS == 1) reinterpret_cast<float*>(smem)[pos] = (float)g;
        else reinterpret_cast<int*>(smem)[pos] = g;
        reinterpret_cast<float*>(smem)[kParamFloats + pos] = ((float)a.beta[c] + a.c0_out) * TWO_M64;
    }
    Ring rc;
    rc.R = R; rc.contig = a.geom.contig;
    rc.row_bytes = (uint32_t)cols; rc.pitch = (uint32_t)a.geom.pitch;
    rc.add_off = (uint32_t)(R * a.geom.pitch);
    rc.slot_bytes = (uint32_t)(R * a.geom.pitch) * (RING_ADD ? 2u : 1u);
    rc.bars = s_bar + warp * a.stages * 8;
    const uint32_t ring0 = (s_bar + kWarps * a.stages * 8 + 127u) & ~127u;
    rc.slots = ring0 + warp * a.stages * rc.slot_bytes;
    rc.x = reinterpret_cast<const uint8_t*>(a.x); rc.ldx = a.ldx;
    rc.addend = RING_ADD ? reinterpret_cast<const uint8_t*>(a.addend) : nullptr; rc.ldadd = a.ldadd;
    rc.rows = a.rows;
    if (lane == 0)
        for (int s = 0; s < a.stages; ++s) mbar_init(rc.bars + s * 8, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    __syncthreads();

    const long long n_items = (a.rows + R - 1) / R;
    const long long warp_global = (long long)blockIdx.x * kWarps + warp;
    const long long total_warps = (long long)gridDim.x * kWarps;
    for (int s = 0; s < a.stages; ++s) {
        const long long it = warp_global + (long long)s * total_warps;
        if (it < n_items) ring_issue(rc, it, s, lane);
    }

    const float out_mul = __int_as_float((127 - (a.s_out + 85)) << 23);  // 2^-(s_out + 85)
    const float c0g = (float)a.c0_gamma;
    const int clamp_threshold = (32767 * 128) / a.gamma_absmax;  // inv_std above this may overflow int16
    const bool nearest = a.rounding == A4C_RND_CONV_EVEN || a.rounding == A4C_RND_POSITIVE_INF ||
                         a.rounding == A4C_RND_NEGATIVE_INF;
    const uint32_t lane_in_slot = (uint32_t)(sub * a.geom.pitch + gl * 16);
    const uint32_t lane_param = (uint32_t)gl * 16u;
    const long long step_rows = total_warps * R;
    long long row = warp_global * R + sub;
    int stage = 0;
    uint32_t parity = 0;
    for (long long item = warp_global; item < n_items; item += total_warps, row += step_rows) {
        if (!mbar_wait(rc.bars + stage * 8, parity, a.status, 201)) break;
        const bool row_ok = row < a.rows;
        uint4 xv[NCH], av[NCH];
        const uint32_t slot = rc.slots + stage * rc.slot_bytes + lane_in_slot;
#pragma unroll
        for (int j = 0; j < NCH; ++j) {
            const bool ok = row_ok && (j * G + gl) < a.geom.nchunks;
            xv[j] = ok ? lds128(slot + j * G * 16) : make_uint4(0, 0, 0, 0);
            if (RING_ADD) av[j] = ok ? lds128(slot + rc.add_off + j * G * 16) : make_uint4(0, 0, 0, 0);
            if (PRE_ADD) {
                // x <- saturate_i8(x + addend) (elementwise_add.cpp:30-33, SHIFT = 0)
                const uint32_t xs[4] = {sat_add_i8x4(xv[j].x, av[j].x), sat_add_i8x4(xv[j].y, av[j].y),
                                        sat_add_i8x4(xv[j].z, av[j].z), sat_add_i8x4(xv[j].w, av[j].w)};
                xv[j] = make_uint4(xs[0], xs[1], xs[2], xs[3]);
            }
        }
        __syncwarp();
        {
            const long long nxt = item + (long long)a.stages * total_warps;
            if (nxt < n_items && lane < R) {
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                ring_issue(rc, nxt, stage, lane);
            }
        }
        if (++stage == a.stages) { stage = 0; parity ^= 1u; }

        int sx0 = 0, sx1 = 0, sq0 = 0, sq1 = 0;  // two accumulator chains each
#pragma unroll
        for (int j = 0; j < NCH; ++j) {
            sx0 = dp4a_ss(xv[j].x, 0x01010101u, sx0); sq0 = dp4a_ss(xv[j].x, xv[j].x, sq0);
            sx1 = dp4a_ss(xv[j].y, 0x01010101u, sx1); sq1 = dp4a_ss(xv[j].y, xv[j].y, sq1);
            sx0 = dp4a_ss(xv[j].z, 0x01010101u, sx0); sq0 = dp4a_ss(xv[j].z, xv[j].z, sq0);
            sx1 = dp4a_ss(xv[j].w, 0x01010101u, sx1); sq1 = dp4a_ss(xv[j].w, xv[j].w, sq1);
        }
        const int sum_x = group_sum(sx0 + sx1, G);
        const int sum_sq = group_sum(sq0 + sq1, G);
        // layer_norm.cpp:23-31
        const int mu = (sum_x + (cols >> 1)) >> a.log2c;
        const int centered = (int)((uint32_t)sum_sq - 2u * (uint32_t)mu * (uint32_t)sum_x +
                                   (uint32_t)cols * (uint32_t)mu * (uint32_t)mu);
        int var = centered >> a.log2c;
        var = max(var, 0) + a.eps_q0;
        const int inv_std = inv_std_q15(var, a.rounding, nearest);
        const float inv_f = (float)inv_std;
        // fscale can leave int16 only when inv_std * max|gamma| / 128 exceeds 32767
        const bool need_clamp = __any_sync(0xffffffffu, inv_std > clamp_threshold);
        const float vdc = 8388608.0f + 128.0f + (float)mu;  // (2^23 + (x ^ 0x80)) - vdc = x - mu
        uint8_t* orow = reinterpret_cast<uint8_t*>(a.out) + row * a.ldo + gl * 16;

        // fscale can leave int16 only for a rare inv_std (warp-uniform test above): the loop exists twice, and the common
        // copy carries no min / max per value (as a run-time condition the compiler predicates them: two more
        // instructions per value on the integer pipe)
        auto normalise = [&](auto clamp_tag) {
            constexpr bool CLAMP = decltype(clamp_tag)::value;
#pragma unroll
            for (int j = 0; j < NCH; ++j) {
                if (!(row_ok && (j * G + gl) < a.geom.nchunks)) continue;
                const uint32_t xw[4] = {xv[j].x ^ 0x80808080u, xv[j].y ^ 0x80808080u, xv[j].z ^ 0x80808080u,
                                        xv[j].w ^ 0x80808080u};
                uint32_t aw[4] = {0, 0, 0, 0};
                if (HAS_ADD) { aw[0] = av[j].x; aw[1] = av[j].y; aw[2] = av[j].z; aw[3] = av[j].w; }
                uint32_t ow[4];
#pragma unroll
                for (int w = 0; w < 4; ++w) {
                    const uint32_t poff = lane_param + (uint32_t)((j * 4 + w) * 32 * 16);
                    const float4 bq = lds128f(s_bet + poff);
                    const float bet[4] = {bq.x, bq.y, bq.z, bq.w};
                    float F[4];
                    if (FS == 0) {
                        const float4 gq = lds128f(s_gam + poff);
                        F[0] = __fmaf_rn(inv_f, gq.x, MAGIC); F[1] = __fmaf_rn(inv_f, gq.y, MAGIC);
                        F[2] = __fmaf_rn(inv_f, gq.z, MAGIC); F[3] = __fmaf_rn(inv_f, gq.w, MAGIC);
                    } else if (FS == 1) {
                        const float4 gq = lds128f(s_gam + poff);
                        // inv_std * gamma + c0 < 2^24 is exact; floor(. / 128) by a round-down FMA
                        F[0] = __fmaf_rd(__fmaf_rn(inv_f, gq.x, c0g), 0.0078125f, MAGIC);
                        F[1] = __fmaf_rd(__fmaf_rn(inv_f, gq.y, c0g), 0.0078125f, MAGIC);
                        F[2] = __fmaf_rd(__fmaf_rn(inv_f, gq.z, c0g), 0.0078125f, MAGIC);
                        F[3] = __fmaf_rd(__fmaf_rn(inv_f, gq.w, c0g), 0.0078125f, MAGIC);
                    } else {
                        const uint4 gq = lds128(s_gam + poff);
                        F[0] = __uint_as_float((uint32_t)((inv_std * (int)gq.x + a.c0_gamma) >> 7) + MAGIC_BITS);
                        F[1] = __uint_as_float((uint32_t)((inv_std * (int)gq.y + a.c0_gamma) >> 7) + MAGIC_BITS);
                        F[2] = __uint_as_float((uint32_t)((inv_std * (int)gq.z + a.c0_gamma) >> 7) + MAGIC_BITS);
                        F[3] = __uint_as_float((uint32_t)((inv_std * (int)gq.w + a.c0_gamma) >> 7) + MAGIC_BITS);
                    }
                    if (CLAMP) {
#pragma unroll
                        for (int k = 0; k < 4; ++k) F[k] = fminf(fmaxf(F[k], MAGIC - 32768.0f), MAGIC + 32767.0f);
                    }
                    const float xf[4] = {byte_to_f23<0>(xw[w]), byte_to_f23<1>(xw[w]), byte_to_f23<2>(xw[w]),
                                         byte_to_f23<3>(xw[w])};
                    int o[4];
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        const float vd = xf[k] - vdc;                                      // x - mu, exact
                        const float fs = __fmaf_rn(F[k], TWO_M64, -MAGIC * TWO_M64);       // fscale * 2^-64, exact
                        const float acc = __fmaf_rn(vd, fs, bet[k]);                       // (vd*fscale + beta + c) * 2^-64
                        const float r = RN ? __fmaf_rn(acc, out_mul, 0.0f) : __fmaf_rd(acc, out_mul, 0.0f);
                        o[k] = __float_as_int(r);                                          // round(.) + 128 as a signed integer
                    }
                    if (HAS_ADD) {
                        // clamp(., 0, 255) on two outputs per register (16-bit lanes: the packing saturates to 16 bits, one
                        // min + relu finishes the clamp), then the fused saturating Add (elementwise_add.cpp:30-33,
                        // SHIFT = 0): sign-extended addend pairs, packed add + min(., 255) + relu
                        uint32_t p01 = __vimin_s16x2_relu(pack_sat_s16x2(o[1], o[0]), 0x00FF00FFu);
                        uint32_t p23 = __vimin_s16x2_relu(pack_sat_s16x2(o[3], o[2]), 0x00FF00FFu);
                        p01 = __viaddmin_s16x2_relu(p01, prmt(aw[w], 0, 0x9180), 0x00FF00FFu);
                        p23 = __viaddmin_s16x2_relu(p23, prmt(aw[w], 0, 0xB3A2), 0x00FF00FFu);
                        ow[w] = prmt(p01, p23, 0x6420) ^ 0x80808080u;  // low bytes of the four lanes, un-biased
                    } else {
                        ow[w] = pack_sat_u8x4(o[0], o[1], o[2], o[3]) ^ 0x80808080u;   // clamp(., 0, 255), pack, un-bias
                    }
                }
                stg16(orow + j * G * 16, make_uint4(ow[0], ow[1], ow[2], ow[3]));
            }
        };
        if (need_clamp) normalise(std::true_type{});
        else normalise(std::false_type{});
    }
}

// ------------------------------------------------------------------------------------------------
// Softmax (uint8 output)
// ------------------------------------------------------------------------------------------------
struct SmFastArgs {
    const int8_t* x; long long ldx;
    const uint8_t* addend; long long ldadd;
    uint8_t* out; long long ldo;
    long long rows; int cols;
    int mode, B, S, Dmax, inv_shift, use_clb, exp_kq;
    int stages;
    uint32_t lut_row_pitch;   // 128: bytes per row of the score table
    uint32_t two16, two8;     // 65536 and 256 as run-time values (multipliers of the lane-forming multiply-adds)
    RowGeom geom;
    int* status;
};

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

// score(d) * 2^-64 from the per-lane table: byte K of dw selects the table row (128 bytes per row, one float
// per lane -> no bank conflicts).  lut_lane = table base + lane * 4 (shared address).  One byte permute extracts the
// index and one integer multiply-add forms the address: the multiply-add runs on the FMA pipe, which has room, while
// shift + mask + add were three instructions on the integer pipe, the busiest unit of this kernel.  `row_pitch` is the
// table's row pitch (128) passed as a run-time value so that the multiply is not strength-reduced back to the integer pipe.
template <int K>
__device__ __forceinline__ float lut_at(uint32_t lut_lane, uint32_t dw, uint32_t row_pitch) {
    const uint32_t idx = prmt(dw, 0, 0x4440 + K);   // byte K, zero-extended
    uint32_t addr;
    asm("mad.lo.u32 %0, %1, %2, %3;" : "=r"(addr) : "r"(idx), "r"(row_pitch), "r"(lut_lane));
    return lds32f(addr);
}

template <int NCH, bool HAS_ADD, bool CLB>
__global__ void __launch_bounds__(kThreads) softmax_fast_kernel(SmFastArgs a) {
    extern __shared__ __align__(128) uint8_t smem[];
    // layout: score table [256][32] floats (32 KB) | barriers | ring
    const uint32_t s_base = smem_u32(smem);
    const uint32_t s_bar = s_base + 256 * 32 * 4;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int G = a.geom.G, R = a.geom.R, cols = a.cols;
    const int sub = lane / G, gl = lane % G;
    const uint32_t ring0 = (s_bar + kWarps * a.stages * 8 + 127u) & ~127u;
    {
        // one score per thread (kThreads == 256 == table rows), staged in the ring area, then replicated
        // across the 32 lanes of each table row with conflict-free stores
        float* lut = reinterpret_cast<float*>(smem);
        float* stage_sc = reinterpret_cast<float*>(smem + (ring0 - s_base));
        const int d = threadIdx.x;
        int s;
        if (a.mode == 0) s = clampi(a.B - a.S * min(d, a.Dmax), -32768, 32767);
        else s = exp_score16(d, a.exp_kq);
        stage_sc[d] = (float)s * TWO_M64;
        __syncthreads();
        for (int i = threadIdx.x; i < 256 * 32; i += kThreads) lut[i] = stage_sc[i >> 5];
        __syncthreads();
    }
    Ring rc;
    rc.R = R; rc.contig = a.geom.contig;
    rc.row_bytes = (uint32_t)cols; rc.pitch = (uint32_t)a.geom.pitch;
    rc.add_off = (uint32_t)(R * a.geom.pitch);
    rc.slot_bytes = (uint32_t)(R * a.geom.pitch) * (HAS_ADD ? 2u : 1u);
    rc.bars = s_bar + warp * a.stages * 8;
    rc.slots = ring0 + warp * a.stages * rc.slot_bytes;
    rc.x = reinterpret_cast<const uint8_t*>(a.x); rc.ldx = a.ldx;
    rc.addend = HAS_ADD ? a.addend : nullptr; rc.ldadd = a.ldadd;
    rc.rows = a.rows;
    if (lane == 0)
        for (int s = 0; s < a.stages; ++s) mbar_init(rc.bars + s * 8, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    __syncthreads();

    const long long n_items = (a.rows + R - 1) / R;
    const long long warp_global = (long long)blockIdx.x * kWarps + warp;
    const long long total_warps = (long long)gridDim.x * kWarps;
    for (int s = 0; s < a.stages; ++s) {
        const long long it = warp_global + (long long)s * total_warps;
        if (it < n_items) ring_issue(rc, it, s, lane);
    }
    const uint32_t lut_lane = s_base + (uint32_t)lane * 4u;
    const int numer = 255 << a.inv_shift;  // inv_shift <= 22 on this path
    const float numer_f = (float)numer;     // exact: 255 * 2^k
    const float out_mul = __int_as_float((127 - (a.inv_shift + 85)) << 23);  // 2^-(inv_shift + 85)
    const uint32_t lane_in_slot = (uint32_t)(sub * a.geom.pitch + gl * 16);
    const long long step_rows = total_warps * R;
    long long row = warp_global * R + sub;

    int stage = 0;
    uint32_t parity = 0;
    for (long long item = warp_global; item < n_items; item += total_warps, row += step_rows) {
        if (!mbar_wait(rc.bars + stage * 8, parity, a.status, 202)) break;
        const bool row_ok = row < a.rows;
        uint4 xv[NCH], av[NCH];
        const uint32_t slot = rc.slots + stage * rc.slot_bytes + lane_in_slot;
#pragma unroll
        for (int j = 0; j < NCH; ++j) {
            const bool ok = row_ok && (j * G + gl) < a.geom.nchunks;
            // biased bytes (x ^ 0x80): unsigned order == signed order; padding = 0 (the minimum)
            xv[j] = make_uint4(0, 0, 0, 0);
            if (ok) {
                const uint4 v = lds128(slot + j * G * 16);
                xv[j] = make_uint4(v.x ^ 0x80808080u, v.y ^ 0x80808080u, v.z ^ 0x80808080u, v.w ^ 0x80808080u);
            }
            if (HAS_ADD) av[j] = ok ? lds128(slot + rc.add_off + j * G * 16) : make_uint4(0, 0, 0, 0);
        }
        __syncwarp();
        {
            const long long nxt = item + (long long)a.stages * total_warps;
            if (nxt < n_items && lane < R) {
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                ring_issue(rc, nxt, stage, lane);
            }
        }
        if (++stage == a.stages) { stage = 0; parity ^= 1u; }

        // row maximum: even / odd bytes widened to u16x2 lanes, three-input packed maximum
        uint32_t mx = 0;
#pragma unroll
        for (int j = 0; j < NCH; ++j) {
            const uint32_t w4[4] = {xv[j].x, xv[j].y, xv[j].z, xv[j].w};
#pragma unroll
            for (int w = 0; w < 4; ++w) mx = __vimax3_u16x2(mx, prmt(w4[w], 0, 0x4240), prmt(w4[w], 0, 0x4341));
        }
        const int m = group_max((int)max(mx & 0xFFFFu, mx >> 16), G);
        const uint32_t m4 = (uint32_t)m * 0x01010101u;

        // scores (kept in registers for the normalisation pass) and their sum
        float e[NCH][16];
        float fs0 = 0.0f, fs1 = 0.0f;
#pragma unroll
        for (int j = 0; j < NCH; ++j) {
            const uint32_t w4[4] = {xv[j].x, xv[j].y, xv[j].z, xv[j].w};
#pragma unroll
            for (int w = 0; w < 4; ++w) {
                const uint32_t dw = m4 - w4[w];  // per byte: max - x, no borrows
                e[j][w * 4 + 0] = lut_at<0>(lut_lane, dw, a.lut_row_pitch);
                e[j][w * 4 + 1] = lut_at<1>(lut_lane, dw, a.lut_row_pitch);
                e[j][w * 4 + 2] = lut_at<2>(lut_lane, dw, a.lut_row_pitch);
                e[j][w * 4 + 3] = lut_at<3>(lut_lane, dw, a.lut_row_pitch);
            }
            if (row_ok && (j * G + gl) < a.geom.nchunks) {
#pragma unroll
                for (int i = 0; i < 16; i += 2) { fs0 += e[j][i]; fs1 += e[j][i + 1]; }
            }
        }
        // exact: a lane adds at most 32 scores <= 32767 (scaled by 2^-64)
        const int sum = group_sum(__float2int_rn((fs0 + fs1) * TWO_P64), G);
        const int s = sum > 0 ? sum : 1;
        int inv;
        if (CLB) {
            const int k = 31 - __clz(s);
            inv = a.inv_shift - k >= 0 ? (255 << (a.inv_shift - k)) : (255 >> (k - a.inv_shift));
        } else {
            // exact floor(numer / s) when it is below 2^15 (larger quotients saturate to 32767 anyway):
            // reciprocal estimate (relative error < 2^-22), then at most one step either way
            float rcp;
            asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(rcp) : "f"((float)s));
            int q = __float2int_rz(numer_f * rcp);
            const int rem = numer - q * s;
            q += (rem >= s) - (rem < 0);
            inv = q;
        }
        inv = min(max(inv, 0), 32767);
        const float invs = (float)inv * out_mul;  // inv * 2^-(shift + 85), exact
        uint8_t* orow = a.out + row * a.ldo + gl * 16;

#pragma unroll
        for (int j = 0; j < NCH; ++j) {
            if (!(row_ok && (j * G + gl) < a.geom.nchunks)) continue;
            uint32_t aw[4] = {0, 0, 0, 0};
            if (HAS_ADD) { aw[0] = av[j].x; aw[1] = av[j].y; aw[2] = av[j].z; aw[3] = av[j].w; }
            uint32_t ow[4];
#pragma unroll
            for (int w = 0; w < 4; ++w) {
                // floor(score * inv / 2^shift) lands in the low bits of a subnormal (scores are non-negative)
                // With inv = floor(255 * 2^shift / sum) (or its clamp to 32767) a score <= sum gives a result <= 255 by
                // itself; only the power-of-two reciprocal (use_clb) can exceed it and needs the saturation.
                int o0 = __float_as_int(__fmaf_rd(e[j][w * 4 + 0], invs, 0.0f));
                int o1 = __float_as_int(__fmaf_rd(e[j][w * 4 + 1], invs, 0.0f));
                int o2 = __float_as_int(__fmaf_rd(e[j][w * 4 + 2], invs, 0.0f));
                int o3 = __float_as_int(__fmaf_rd(e[j][w * 4 + 3], invs, 0.0f));
                if (CLB) { o0 = min(o0, 255); o1 = min(o1, 255); o2 = min(o2, 255); o3 = min(o3, 255); }
                if (HAS_ADD) {
                    // fused saturating uint8 Add on 16-bit lanes, values 0 / 2 and 1 / 3 paired: the lanes are formed and
                    // merged by integer multiply-adds (FMA pipe; the multipliers 2^16 and 2^8 come in as run-time values
                    // so that they stay multiplies), the addend bytes by one mask and one permute, then packed add + min(., 255)
                    uint32_t p02, p13;
                    asm("mad.lo.u32 %0, %1, %2, %3;" : "=r"(p02) : "r"((uint32_t)o2), "r"(a.two16), "r"((uint32_t)o0));
                    asm("mad.lo.u32 %0, %1, %2, %3;" : "=r"(p13) : "r"((uint32_t)o3), "r"(a.two16), "r"((uint32_t)o1));
                    p02 = __viaddmin_u16x2(p02, aw[w] & 0x00FF00FFu, 0x00FF00FFu);
                    p13 = __viaddmin_u16x2(p13, prmt(aw[w], 0, 0x4341), 0x00FF00FFu);
                    asm("mad.lo.u32 %0, %1, %2, %3;" : "=r"(ow[w]) : "r"(p13), "r"(a.two8), "r"(p02));
                } else {
                    ow[w] = prmt(prmt((uint32_t)o0, (uint32_t)o1, 0x5410), prmt((uint32_t)o2, (uint32_t)o3, 0x5410), 0x6420);
                }
            }
            stg16(orow + j * G * 16, make_uint4(ow[0], ow[1], ow[2], ow[3]));
        }
    }
}

// Tuning overrides (0 = the launcher's own choice).  Chunks per lane: how many 16-element chunks of a row one
// lane works on; the per-row scalar work is amortised over them, at the price of registers and ring bytes.
int g_min_stages = 0;
int g_chunks_per_lane = 0;

int g_contig = 1;   // A4C_OPT_ROWOP_CONTIG_COPY

RowGeom make_geom(int cols, int preferred_nch, bool rows_adjacent) {
    RowGeom g;
    g.nchunks = cols / 16;
    const int target = g_chunks_per_lane > 0 ? g_chunks_per_lane : preferred_nch;
    int G = 1;
    while (G * target < g.nchunks && G < 32) G <<= 1;
    g.G = G;
    g.R = 32 / G;
    g.contig = (g_contig && rows_adjacent && g.R > 1) ? 1 : 0;
    g.pitch = cols + ((!g.contig && G < 8 && cols % 128 == 0) ? G * 16 : 0);
    return g;
}

int sm_count() {
    int dev = 0, sms = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    return sms;
}

// ring depth, shared-memory size and grid size for a kernel with `fixed` bytes of tables and `slot` bytes
// per ring slot
void plan_launch(size_t fixed, size_t slot, long long n_items, int* stages, size_t* smem, int* grid) {
    int st = 4;
    size_t bytes = fixed + kWarps * st * 8 + 128 + (size_t)kWarps * st * slot;
    const int min_st = g_min_stages > 0 ? g_min_stages : 2;
    while (bytes > 72 * 1024 && st > min_st) {  // prefer three blocks per SM over a deeper ring
        --st;
        bytes = fixed + kWarps * st * 8 + 128 + (size_t)kWarps * st * slot;
    }
    int per_sm = (int)((220 * 1024) / bytes);
    if (per_sm < 1) per_sm = 1;
    if (per_sm > 4) per_sm = 4;
    long long blocks = (n_items + kWarps - 1) / kWarps;
    const long long cap = (long long)sm_count() * per_sm;
    if (blocks > cap) blocks = cap;
    *stages = st; *smem = bytes; *grid = (int)blocks;
}

}  // namespace

void a4c_rowops_fast_contig(int on) { g_contig = on ? 1 : 0; }

void a4c_rowops_fast_tuning(int chunks_per_lane, int min_stages) {
    if (chunks_per_lane >= 0) g_chunks_per_lane = chunks_per_lane;
    if (min_stages >= 0) g_min_stages = min_stages;
}

// Returns A4C_ERR_UNSUPPORTED when the request is outside the fast path's proofs (caller falls back
// to the generic kernel).
int a4c_launch_layernorm_fast(const int8_t* x, long long ldx, const int16_t* gamma, const int16_t* beta,
                              const int8_t* addend, long long ldadd, int pre_add, int8_t* out, long long ldo,
                              long long rows, int cols, int eps_q0, int out_shift, int rounding, int gamma_absmax,
                              int* status, cudaStream_t stream) {
    const int s_out = 15 - out_shift;
    if (s_out < 2 || gamma_absmax <= 0 || gamma_absmax > 16383) return A4C_ERR_UNSUPPORTED;
    if (rounding == A4C_RND_SYMMETRIC_INF || rounding == A4C_RND_SYMMETRIC_ZERO || rounding == A4C_RND_CONV_ODD)
        return A4C_ERR_UNSUPPORTED;
    if (cols > 2048 || status == nullptr || eps_q0 > (1 << 20)) return A4C_ERR_UNSUPPORTED;
    LnFastArgs a;
    a.x = x; a.ldx = ldx; a.gamma = gamma; a.beta = beta; a.addend = addend; a.ldadd = ldadd; a.out = out; a.ldo = ldo;
    a.rows = rows; a.cols = cols; a.eps_q0 = eps_q0; a.rounding = rounding; a.s_out = s_out;
    a.gamma_absmax = gamma_absmax; a.status = status;
    a.log2c = 0;
    while ((1 << a.log2c) < cols) ++a.log2c;
    a.c0_gamma = 0; a.c0_out = 0.0f;
    switch (rounding) {
        case A4C_RND_CEIL: a.c0_gamma = 127; a.c0_out = (float)((1 << s_out) - 1); break;
        case A4C_RND_POSITIVE_INF: a.c0_gamma = 64; a.c0_out = (float)(1 << (s_out - 1)); break;
        case A4C_RND_NEGATIVE_INF: a.c0_gamma = 63; a.c0_out = (float)((1 << (s_out - 1)) - 1); break;
        default: break;
    }
    a.c0_out += (float)(128 << s_out);  // outputs are produced biased by +128
    a.geom = make_geom(cols, 4, ldx == cols && (!addend || ldadd == cols));   // 4: measured best from 128 to 2048 columns
    const int nch = (a.geom.nchunks + a.geom.G - 1) / a.geom.G;
    if (nch != 1 && nch != 2 && nch != 4) return A4C_ERR_UNSUPPORTED;
    const size_t fixed = (size_t)nch * 4 * 32 * 4 * 4 * 2;
    const size_t slot = (size_t)a.geom.R * a.geom.pitch * (addend ? 2 : 1);
    const long long n_items = (rows + a.geom.R - 1) / a.geom.R;
    size_t smem; int grid;
    plan_launch(fixed, slot, n_items, &a.stages, &smem, &grid);
    const int fs = rounding == A4C_RND_CONV_EVEN ? 0 : (gamma_absmax <= 511 ? 1 : 2);
#define LN_LAUNCH(NCH_, FS_, ADD_)                                                                                \
    do {                                                                                                           \
        cudaFuncSetAttribute(layernorm_fast_kernel<NCH_, FS_, ADD_>, cudaFuncAttributeMaxDynamicSharedMemorySize,  \
                             (int)smem);                                                                           \
        layernorm_fast_kernel<NCH_, FS_, ADD_><<<grid, kThreads, smem, stream>>>(a);                               \
    } while (0)
#define LN_PICK_FS(NCH_, ADD_)                                                                                     \
    do {                                                                                                           \
        if (fs == 0) LN_LAUNCH(NCH_, 0, ADD_); else if (fs == 1) LN_LAUNCH(NCH_, 1, ADD_); else LN_LAUNCH(NCH_, 2, ADD_); \
    } while (0)
#define LN_PICK(NCH_)                                                                                              \
    do {                                                                                                           \
        if (!addend) LN_PICK_FS(NCH_, 0); else if (pre_add) LN_PICK_FS(NCH_, 2); else LN_PICK_FS(NCH_, 1);         \
    } while (0)
    if (nch == 1) LN_PICK(1);
    else if (nch == 2) LN_PICK(2);
    else LN_PICK(4);
#undef LN_PICK
#undef LN_PICK_FS
#undef LN_LAUNCH
    return cudaGetLastError() == cudaSuccess ? A4C_OK : A4C_ERR_CUDA;
}

int a4c_launch_softmax_fast(const int8_t* x, long long ldx, const void* addend, long long ldadd, void* out,
                            long long ldo, long long rows, int cols, int mode, int B, int S, int Dmax, int inv_shift,
                            int use_clb, int exp_kq, int out_dtype, int* status, cudaStream_t stream) {
    if (out_dtype != A4C_U8 || inv_shift > 22 || cols > 1024 || status == nullptr) return A4C_ERR_UNSUPPORTED;
    if (mode == 0 && B - S * (Dmax < 255 ? Dmax : 255) < 0) return A4C_ERR_UNSUPPORTED;  // negative scores
    SmFastArgs a;
    a.x = x; a.ldx = ldx; a.addend = (const uint8_t*)addend; a.ldadd = ldadd; a.out = (uint8_t*)out; a.ldo = ldo;
    a.rows = rows; a.cols = cols; a.mode = mode; a.B = B; a.S = S; a.Dmax = Dmax; a.inv_shift = inv_shift;
    a.use_clb = use_clb; a.exp_kq = exp_kq; a.status = status;
    a.lut_row_pitch = 128u; a.two16 = 65536u; a.two8 = 256u;
    // four chunks per lane keep 64 scores in registers: worth it only with the fused Add on long rows
    a.geom = make_geom(cols, (addend && cols >= 512) ? 4 : 2, ldx == cols && (!addend || ldadd == cols));
    const int nch = (a.geom.nchunks + a.geom.G - 1) / a.geom.G;
    if (nch != 1 && nch != 2 && nch != 4) return A4C_ERR_UNSUPPORTED;
    const size_t slot = (size_t)a.geom.R * a.geom.pitch * (addend ? 2 : 1);
    const long long n_items = (rows + a.geom.R - 1) / a.geom.R;
    size_t smem; int grid;
    plan_launch(256 * 32 * 4, slot, n_items, &a.stages, &smem, &grid);
#define SM_LAUNCH(NCH_, ADD_)                                                                                      \
    do {                                                                                                           \
        if (clb) {                                                                                                 \
            cudaFuncSetAttribute(softmax_fast_kernel<NCH_, ADD_, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                                 (int)smem);                                                                       \
            softmax_fast_kernel<NCH_, ADD_, true><<<grid, kThreads, smem, stream>>>(a);                            \
        } else {                                                                                                   \
            cudaFuncSetAttribute(softmax_fast_kernel<NCH_, ADD_, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                                 (int)smem);                                                                       \
            softmax_fast_kernel<NCH_, ADD_, false><<<grid, kThreads, smem, stream>>>(a);                           \
        }                                                                                                          \
    } while (0)
    const bool clb = use_clb && mode == 0;   // the power-of-two reciprocal of the HCCS kernel
    if (nch == 1) { if (addend) SM_LAUNCH(1, true); else SM_LAUNCH(1, false); }
    else if (nch == 2) { if (addend) SM_LAUNCH(2, true); else SM_LAUNCH(2, false); }
    else { if (addend) SM_LAUNCH(4, true); else SM_LAUNCH(4, false); }
#undef SM_LAUNCH
    return cudaGetLastError() == cudaSuccess ? A4C_OK : A4C_ERR_CUDA;
}
