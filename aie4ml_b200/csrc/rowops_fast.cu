// Bandwidth-oriented LayerNorm and Softmax row kernels (the common cases of rowops.cu).
//
// Data movement: every warp owns a ring of row slots in shared memory that is filled by bulk
// asynchronous copies (cp.async.bulk, completion on an mbarrier), so many rows per SM are in flight
// without holding registers; results leave through 128-bit global stores.
//
// Arithmetic: the integer recipes of the aie4ml kernels (layer_norm.cpp:15-121, softmax.cpp:20-88 and
// :252-384) are evaluated on the FP32 pipe where that is provably exact:
//   * an integer n with |n| < 2^22 is carried as the float MAGIC + n (MAGIC = 1.5 * 2^23), whose low
//     mantissa bits are n in two's complement;
//   * round(v / 2^s) for the rounding modes floor / ceil / half-up / half-down / half-even is ONE fused
//     multiply-add fma(v, 2^-s, MAGIC [+ folded constant]) with the matching IEEE rounding direction:
//     the FMA forms v * 2^-s + MAGIC exactly and rounds once, to an integer because ulp(2^23..2^24) = 1;
//   * products such as (x - mu) * fscale + beta stay below 2^24 in magnitude, so they are exact.
// Modes or parameters outside those proofs (symmetric rounding, conv_odd, |gamma| > 16383, shifts < 2,
// int16 softmax output, negative HCCS scores, inv_shift > 22) take the generic integer kernels.
#include <mutex>

#include "a4c_common.cuh"
#include "a4c_kernels.h"

namespace {

constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;
constexpr int kStages = 4;
constexpr float MAGIC = 12582912.0f;          // 1.5 * 2^23
constexpr uint32_t MAGIC_BITS = 0x4B400000u;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" :: "r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" :: "r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.b32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return ok != 0;
}
// Bounded wait; on timeout records `code` in the status word and returns false.
__device__ __noinline__ bool mbar_wait_slow(uint64_t* bar, uint32_t parity, int* status, int code) {
    const uint64_t t0 = a4c_globaltimer();
    for (uint32_t it = 1;; ++it) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((it & 255u) == 0 && a4c_globaltimer() - t0 > A4C_SPIN_LIMIT_NS) {
            atomicCAS(status, 0, code);
            return false;
        }
    }
}
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, int* status, int code) {
    if (mbar_try_wait(bar, parity)) return true;
    return mbar_wait_slow(bar, parity, status, code);
}
__device__ __forceinline__ void bulk_load(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 :: "r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void stg16(void* p, uint4 v) {
    asm volatile("st.global.v4.u32 [%0], {%1,%2,%3,%4};" :: "l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
__device__ __forceinline__ uint4 ldg16(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ int dp4a_ss(uint32_t a, uint32_t b, int c) {
    int d;
    asm("dp4a.s32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
// prmt.b32 in its default mode: selector nibble n picks byte (n & 7) of {b:a}; bit 3 of the nibble
// replicates that byte's sign bit instead
__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t d;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(sel));
    return d;
}
// float 2^23 + byte k of w (bytes taken as unsigned)
template <int K>
__device__ __forceinline__ float byte_to_f23(uint32_t w) {
    // result bytes: [w.bK, 0x00, 0x00, 0x4B]; second operand 0x4B000000 supplies bytes 4..7
    return __uint_as_float(prmt(w, 0x4B000000u, 0x7540 + K));
}
// pack the low bytes of four MAGIC-offset floats
__device__ __forceinline__ uint32_t pack_low_bytes(float a, float b, float c, float d) {
    const uint32_t ab = prmt(__float_as_uint(a), __float_as_uint(b), 0x0040);  // [a0, b0, a0, a0]
    const uint32_t cd = prmt(__float_as_uint(c), __float_as_uint(d), 0x0040);
    return prmt(ab, cd, 0x5410);                                              // [a0, b0, c0, d0]
}

struct RowGeom {
    int nchunks, G, R;
};

// A warp's view of the row ring: items of R rows each, loaded ahead by kStages.
struct RingCtx {
    uint8_t* slots;      // this warp's kStages slots
    uint64_t* bars;      // this warp's kStages barriers
    int slot_bytes;      // R * cols
    const uint8_t* src;  // global base of the input
    long long ld;        // input row pitch (bytes, int8 elements)
    long long rows;
    int cols, R;
};

__device__ __forceinline__ void ring_issue(const RingCtx& c, long long item, int stage) {
    // lane 0 only
    const long long row0 = item * c.R;
    long long nrows = c.rows - row0;
    if (nrows > c.R) nrows = c.R;
    if (nrows <= 0) return;
    mbar_expect_tx(&c.bars[stage], (uint32_t)(nrows * c.cols));
    for (int r = 0; r < (int)nrows; ++r)
        bulk_load(c.slots + (size_t)stage * c.slot_bytes + (size_t)r * c.cols, c.src + (row0 + r) * c.ld,
                  (uint32_t)c.cols, &c.bars[stage]);
}

// ------------------------------------------------------------------------------------------------
// LayerNorm
// ------------------------------------------------------------------------------------------------
// Further exactness facts used below:
//   * a float whose exponent field is zero (a subnormal) has the bit pattern sign | n with value
//     n * 2^-149, so fma(v * 2^-64, 2^-(s+85), 0) with a directed or nearest-even rounding mode leaves
//     round(v / 2^s) directly in the low bits, sign-magnitude; min.s32.relu then clamps it to [0, 255] in one
//     instruction.  Outputs are produced biased by +128 (folded into beta) and un-biased with one XOR per word.
constexpr float TWO_M64 = 5.421010862427522e-20f;   // 2^-64

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
    RowGeom geom;
    int* status;
};

// Q15 reciprocal standard deviation for every variance the int8 kernel can see (var <= 128^2 + eps), one table
// per rounding token, filled on the device by the defining expression
//   clamp(round_tok(2^15 * (1.0f / sqrtf((float)var))), 0, 32767)        (layer_norm.cpp:33-39)
// so the row loop replaces a correctly rounded sqrt + divide + rounding by one cached load.
constexpr int kInvStdMaxEps = 1024;
constexpr int kInvStdEntries = 16384 + kInvStdMaxEps + 1;
__device__ int16_t g_inv_std_table[A4C_RND_COUNT][kInvStdEntries];

__device__ __forceinline__ int round_float_tok(float f, int tok) {
    const float fl = floorf(f);
    const float frac = f - fl;
    const int q = (int)fl;
    switch (tok) {
        case A4C_RND_FLOOR: return q;
        case A4C_RND_CEIL: return q + (frac > 0.0f);
        case A4C_RND_POSITIVE_INF:
        case A4C_RND_SYMMETRIC_INF: return q + (frac >= 0.5f);
        case A4C_RND_NEGATIVE_INF:
        case A4C_RND_SYMMETRIC_ZERO: return q + (frac > 0.5f);
        case A4C_RND_CONV_EVEN: return q + ((frac > 0.5f) || (frac == 0.5f && (q & 1)));
        default: return q + ((frac > 0.5f) || (frac == 0.5f && !(q & 1)));
    }
}

__global__ void build_inv_std_table_kernel(int tok) {
    const int var = blockIdx.x * blockDim.x + threadIdx.x;
    if (var >= kInvStdEntries) return;
    int q = 32767;
    if (var > 0) {
        const float inv_f32 = __fdiv_rn(1.0f, __fsqrt_rn(__int2float_rn(var)));
        q = clampi(round_float_tok(__fmul_rn(inv_f32, 32768.0f), tok), 0, 32767);
    }
    g_inv_std_table[tok][var] = (int16_t)q;
}

// position of column c in the lane-major parameter arrays: lanes of a row group read consecutive 16-byte
// quads for a fixed (chunk index j, word w), so the 128-bit shared loads are conflict-free
__device__ __forceinline__ int param_pos(int c, int G) {
    const int chunk = c >> 4, w = (c >> 2) & 3, k = c & 3;
    const int j = chunk / G, gl = chunk % G;
    return (((j * 4 + w) * G + gl) << 2) + k;
}

// FS = 0: conv_even, fscale = rne(inv_std * gamma / 128) in one nearest-even FMA
// FS = 1: floor-type modes with |gamma| <= 511: inv_std * gamma + c0 is exact in FP32, then one round-down FMA
// FS = 2: floor-type modes with larger gamma: integer multiply-add and shift
template <int NCH, int FS>
__global__ void __launch_bounds__(kThreads) layernorm_fast_kernel(LnFastArgs a) {
    extern __shared__ __align__(128) uint8_t smem[];
    const int cols = a.cols;
    float* gam_f = reinterpret_cast<float*>(smem);                      // FS 0: gamma/128, FS 1: gamma
    int* gam_i = reinterpret_cast<int*>(smem);                          // FS 2: gamma
    float* bet_f = reinterpret_cast<float*>(smem + (size_t)cols * 4);   // (beta + constants) * 2^-64
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + (size_t)cols * 8);
    uint8_t* ring = smem + (size_t)cols * 8 + kWarps * kStages * 8;
    ring = reinterpret_cast<uint8_t*>(((uintptr_t)ring + 127) & ~(uintptr_t)127);

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int G = a.geom.G, R = a.geom.R;
    const int sub = lane / G, gl = lane % G;
    constexpr bool RN = FS == 0;

    for (int c = threadIdx.x; c < cols; c += kThreads) {
        const int g = a.gamma[c];
        const int pos = param_pos(c, G);
        if (FS == 0) gam_f[pos] = (float)g * 0.0078125f;
        else if (FS == 1) gam_f[pos] = (float)g;
        else gam_i[pos] = g;
        bet_f[pos] = ((float)a.beta[c] + a.c0_out) * TWO_M64;
    }
    RingCtx rc;
    rc.slot_bytes = R * cols;
    rc.slots = ring + (size_t)warp * kStages * rc.slot_bytes;
    rc.bars = bars + warp * kStages;
    rc.src = reinterpret_cast<const uint8_t*>(a.x);
    rc.ld = a.ldx; rc.rows = a.rows; rc.cols = cols; rc.R = R;
    if (lane == 0)
        for (int s = 0; s < kStages; ++s) mbar_init(&rc.bars[s], 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    __syncthreads();

    const long long n_items = (a.rows + R - 1) / R;
    const long long warp_global = (long long)blockIdx.x * kWarps + warp;
    const long long total_warps = (long long)gridDim.x * kWarps;
    if (lane == 0)
        for (int s = 0; s < kStages; ++s) {
            const long long it = warp_global + (long long)s * total_warps;
            if (it < n_items) ring_issue(rc, it, s);
        }

    const float out_mul = __int_as_float((127 - (a.s_out + 85)) << 23);  // 2^-(s_out + 85)
    const float c0g = (float)a.c0_gamma;
    const uint32_t group_mask = G == 32 ? 0xffffffffu : (((1u << G) - 1u) << (sub * G));
    const int16_t* inv_table = g_inv_std_table[a.rounding];
    const int clamp_threshold = (32767 * 128) / a.gamma_absmax;  // inv_std above this may overflow int16
    const bool has_add = a.addend != nullptr;
    int stage = 0;
    uint32_t parity = 0;
    for (long long item = warp_global; item < n_items; item += total_warps) {
        if (!__all_sync(0xffffffffu, mbar_wait(&rc.bars[stage], parity, a.status, 201))) break;
        const long long row = item * R + sub;
        const bool row_ok = row < a.rows;
        uint4 xv[NCH];
        const uint8_t* slot = rc.slots + (size_t)stage * rc.slot_bytes + (size_t)sub * cols;
#pragma unroll
        for (int j = 0; j < NCH; ++j) {
            const int chunk = j * G + gl;
            xv[j] = (row_ok && chunk < a.geom.nchunks) ? *reinterpret_cast<const uint4*>(slot + chunk * 16)
                                                        : make_uint4(0, 0, 0, 0);
        }
        __syncwarp();
        if (lane == 0) {
            const long long nxt = item + (long long)kStages * total_warps;
            if (nxt < n_items) {
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                ring_issue(rc, nxt, stage);
            }
        }
        if (++stage == kStages) { stage = 0; parity ^= 1u; }

        int sum_x = 0, sum_sq = 0;
#pragma unroll
        for (int j = 0; j < NCH; ++j) {
            sum_x = dp4a_ss(xv[j].x, 0x01010101u, sum_x); sum_sq = dp4a_ss(xv[j].x, xv[j].x, sum_sq);
            sum_x = dp4a_ss(xv[j].y, 0x01010101u, sum_x); sum_sq = dp4a_ss(xv[j].y, xv[j].y, sum_sq);
            sum_x = dp4a_ss(xv[j].z, 0x01010101u, sum_x); sum_sq = dp4a_ss(xv[j].z, xv[j].z, sum_sq);
            sum_x = dp4a_ss(xv[j].w, 0x01010101u, sum_x); sum_sq = dp4a_ss(xv[j].w, xv[j].w, sum_sq);
        }
        sum_x = __reduce_add_sync(group_mask, sum_x);
        sum_sq = __reduce_add_sync(group_mask, sum_sq);
        const int mu = (sum_x + (cols >> 1)) >> a.log2c;
        const int centered = (int)((uint32_t)sum_sq - 2u * (uint32_t)mu * (uint32_t)sum_x +
                                   (uint32_t)cols * (uint32_t)mu * (uint32_t)mu);
        int var = centered >> a.log2c;
        var = max(var, 0) + a.eps_q0;             // <= 16384 + eps_q0 for int8 rows
        const int inv_std = inv_table[min(var, kInvStdEntries - 1)];
        const float inv_f = (float)inv_std;
        // fscale can leave int16 only when inv_std * max|gamma| / 128 exceeds 32767
        const bool need_clamp = __any_sync(0xffffffffu, inv_std > clamp_threshold);
        const float vdc = 8388608.0f + 128.0f + (float)mu;  // (2^23 + (x ^ 0x80)) - vdc = x - mu

#pragma unroll
        for (int j = 0; j < NCH; ++j) {
            const int chunk = j * G + gl;
            if (!(row_ok && chunk < a.geom.nchunks)) continue;
            const uint32_t xw[4] = {xv[j].x ^ 0x80808080u, xv[j].y ^ 0x80808080u, xv[j].z ^ 0x80808080u,
                                    xv[j].w ^ 0x80808080u};
            uint32_t aw[4] = {0, 0, 0, 0};
            if (has_add) {
                const uint4 av = ldg16(a.addend + row * a.ldadd + (long long)chunk * 16);
                aw[0] = av.x; aw[1] = av.y; aw[2] = av.z; aw[3] = av.w;
            }
            uint32_t ow[4];
#pragma unroll
            for (int w = 0; w < 4; ++w) {
                const int pos = ((j * 4 + w) * G + gl) << 2;
                const float4 bq = *reinterpret_cast<const float4*>(bet_f + pos);
                const float bet[4] = {bq.x, bq.y, bq.z, bq.w};
                float F[4];
                if (FS == 0) {
                    const float4 gq = *reinterpret_cast<const float4*>(gam_f + pos);
                    F[0] = __fmaf_rn(inv_f, gq.x, MAGIC); F[1] = __fmaf_rn(inv_f, gq.y, MAGIC);
                    F[2] = __fmaf_rn(inv_f, gq.z, MAGIC); F[3] = __fmaf_rn(inv_f, gq.w, MAGIC);
                } else if (FS == 1) {
                    const float4 gq = *reinterpret_cast<const float4*>(gam_f + pos);
                    // inv_std * gamma + c0 < 2^24 is exact; floor(. / 128) by a round-down FMA
                    F[0] = __fmaf_rd(__fmaf_rn(inv_f, gq.x, c0g), 0.0078125f, MAGIC);
                    F[1] = __fmaf_rd(__fmaf_rn(inv_f, gq.y, c0g), 0.0078125f, MAGIC);
                    F[2] = __fmaf_rd(__fmaf_rn(inv_f, gq.z, c0g), 0.0078125f, MAGIC);
                    F[3] = __fmaf_rd(__fmaf_rn(inv_f, gq.w, c0g), 0.0078125f, MAGIC);
                } else {
                    const int4 gq = *reinterpret_cast<const int4*>(gam_i + pos);
                    F[0] = __uint_as_float((uint32_t)((inv_std * gq.x + a.c0_gamma) >> 7) + MAGIC_BITS);
                    F[1] = __uint_as_float((uint32_t)((inv_std * gq.y + a.c0_gamma) >> 7) + MAGIC_BITS);
                    F[2] = __uint_as_float((uint32_t)((inv_std * gq.z + a.c0_gamma) >> 7) + MAGIC_BITS);
                    F[3] = __uint_as_float((uint32_t)((inv_std * gq.w + a.c0_gamma) >> 7) + MAGIC_BITS);
                }
                if (need_clamp) {
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
                    const float acc = __fmaf_rn(vd, fs, bet[k]);                       // (vd*fscale + beta + c) * 2^-64, exact
                    const float r = RN ? __fmaf_rn(acc, out_mul, 0.0f) : __fmaf_rd(acc, out_mul, 0.0f);
                    o[k] = __vimin_s32_relu(__float_as_int(r), 255);                   // clamp(round(.) + 128, 0, 255)
                }
                // two biased outputs per register as s16x2 lanes
                uint32_t p01 = prmt((uint32_t)o[0], (uint32_t)o[1], 0x5410);
                uint32_t p23 = prmt((uint32_t)o[2], (uint32_t)o[3], 0x5410);
                if (has_add) {
                    // fused saturating Add (elementwise_add.cpp:30-33, SHIFT = 0): sign-extended addend pairs,
                    // packed add + min(., 255) + relu, two elements per instruction
                    p01 = __viaddmin_s16x2_relu(p01, prmt(aw[w], 0, 0x9180), 0x00FF00FFu);
                    p23 = __viaddmin_s16x2_relu(p23, prmt(aw[w], 0, 0xB3A2), 0x00FF00FFu);
                }
                ow[w] = prmt(p01, p23, 0x6420) ^ 0x80808080u;  // low bytes of the four lanes, un-biased
            }
            stg16(a.out + row * a.ldo + (long long)chunk * 16, make_uint4(ow[0], ow[1], ow[2], ow[3]));
        }
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
    RowGeom geom;
    int* status;
};

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
// per lane -> no bank conflicts); byte offset = (d << 7) | (lane * 4), added to the (warp-uniform) table base
template <int K>
__device__ __forceinline__ float lut_at(const float* lut, uint32_t lane4, uint32_t dw) {
    uint32_t sh;
    if (K == 0) sh = dw << 7;
    else if (K == 1) sh = dw >> 1;
    else if (K == 2) sh = dw >> 9;
    else sh = dw >> 17;
    const uint32_t off = (sh & 0x7F80u) | lane4;
    return *reinterpret_cast<const float*>(reinterpret_cast<const uint8_t*>(lut) + off);
}

template <int NCH>
__global__ void __launch_bounds__(kThreads) softmax_fast_kernel(SmFastArgs a) {
    extern __shared__ __align__(128) uint8_t smem[];
    float* lut = reinterpret_cast<float*>(smem);  // [256][32] = 32 KB
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + 256 * 32 * 4);
    uint8_t* ring = smem + 256 * 32 * 4 + kWarps * kStages * 8;
    ring = reinterpret_cast<uint8_t*>(((uintptr_t)ring + 127) & ~(uintptr_t)127);

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int G = a.geom.G, R = a.geom.R, cols = a.cols;
    const int sub = lane / G, gl = lane % G;
    {
        // one score per thread (kThreads == 256 == table rows), staged in the ring area, then replicated
        // across the 32 lanes of each table row with conflict-free stores
        float* stage_sc = reinterpret_cast<float*>(ring);
        const int d = threadIdx.x;
        int s;
        if (a.mode == 0) s = clampi(a.B - a.S * min(d, a.Dmax), -32768, 32767);
        else s = exp_score16(d, a.exp_kq);
        stage_sc[d] = (float)s * TWO_M64;
        __syncthreads();
        for (int i = threadIdx.x; i < 256 * 32; i += kThreads) lut[i] = stage_sc[i >> 5];
        __syncthreads();
    }
    RingCtx rc;
    rc.slot_bytes = R * cols;
    rc.slots = ring + (size_t)warp * kStages * rc.slot_bytes;
    rc.bars = bars + warp * kStages;
    rc.src = reinterpret_cast<const uint8_t*>(a.x);
    rc.ld = a.ldx; rc.rows = a.rows; rc.cols = cols; rc.R = R;
    if (lane == 0)
        for (int s = 0; s < kStages; ++s) mbar_init(&rc.bars[s], 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    __syncthreads();

    const long long n_items = (a.rows + R - 1) / R;
    const long long warp_global = (long long)blockIdx.x * kWarps + warp;
    const long long total_warps = (long long)gridDim.x * kWarps;
    if (lane == 0)
        for (int s = 0; s < kStages; ++s) {
            const long long it = warp_global + (long long)s * total_warps;
            if (it < n_items) ring_issue(rc, it, s);
        }
    const uint32_t lane4 = (uint32_t)lane * 4u;
    const int numer = 255 << a.inv_shift;  // inv_shift <= 22 on this path
    const float numer_f = (float)numer;     // exact: 255 * 2^k
    const uint32_t group_mask = G == 32 ? 0xffffffffu : (((1u << G) - 1u) << (sub * G));
    const float out_mul = __int_as_float((127 - (a.inv_shift + 85)) << 23);  // 2^-(inv_shift + 85)
    const bool has_add = a.addend != nullptr;

    int stage = 0;
    uint32_t parity = 0;
    for (long long item = warp_global; item < n_items; item += total_warps) {
        if (!__all_sync(0xffffffffu, mbar_wait(&rc.bars[stage], parity, a.status, 202))) break;
        const long long row = item * R + sub;
        const bool row_ok = row < a.rows;
        uint4 xv[NCH];
        const uint8_t* slot = rc.slots + (size_t)stage * rc.slot_bytes + (size_t)sub * cols;
#pragma unroll
        for (int j = 0; j < NCH; ++j) {
            const int chunk = j * G + gl;
            // biased bytes (x ^ 0x80): unsigned order == signed order; padding = 0 (the minimum)
            xv[j] = make_uint4(0, 0, 0, 0);
            if (row_ok && chunk < a.geom.nchunks) {
                const uint4 v = *reinterpret_cast<const uint4*>(slot + chunk * 16);
                xv[j] = make_uint4(v.x ^ 0x80808080u, v.y ^ 0x80808080u, v.z ^ 0x80808080u, v.w ^ 0x80808080u);
            }
        }
        __syncwarp();
        if (lane == 0) {
            const long long nxt = item + (long long)kStages * total_warps;
            if (nxt < n_items) {
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                ring_issue(rc, nxt, stage);
            }
        }
        if (++stage == kStages) { stage = 0; parity ^= 1u; }

        // row maximum: even / odd bytes widened to u16x2 lanes, three-input packed maximum
        uint32_t mx = 0;
#pragma unroll
        for (int j = 0; j < NCH; ++j) {
            const uint32_t w4[4] = {xv[j].x, xv[j].y, xv[j].z, xv[j].w};
#pragma unroll
            for (int w = 0; w < 4; ++w) mx = __vimax3_u16x2(mx, prmt(w4[w], 0, 0x4240), prmt(w4[w], 0, 0x4341));
        }
        const int m = (int)__reduce_max_sync(group_mask, max(mx & 0xFFFFu, mx >> 16));
        const uint32_t m4 = (uint32_t)m * 0x01010101u;

        // scores (kept in registers for the normalisation pass) and their sum
        float e[NCH][16];
        float fsum = 0.0f;
#pragma unroll
        for (int j = 0; j < NCH; ++j) {
            const uint32_t w4[4] = {xv[j].x, xv[j].y, xv[j].z, xv[j].w};
#pragma unroll
            for (int w = 0; w < 4; ++w) {
                const uint32_t dw = m4 - w4[w];  // per byte: max - x, no borrows
                e[j][w * 4 + 0] = lut_at<0>(lut, lane4, dw);
                e[j][w * 4 + 1] = lut_at<1>(lut, lane4, dw);
                e[j][w * 4 + 2] = lut_at<2>(lut, lane4, dw);
                e[j][w * 4 + 3] = lut_at<3>(lut, lane4, dw);
            }
            const int chunk = j * G + gl;
            if (row_ok && chunk < a.geom.nchunks) {
#pragma unroll
                for (int i = 0; i < 16; ++i) fsum += e[j][i];
            }
        }
        // exact: a lane adds at most 64 scores <= 32767 (scaled by 2^-64)
        const int sum = __reduce_add_sync(group_mask, __float2int_rn(fsum * 18446744073709551616.0f));
        const int s = sum > 0 ? sum : 1;
        int inv;
        if (a.use_clb && a.mode == 0) {
            const int k = 31 - __clz(s);
            inv = a.inv_shift - k >= 0 ? (255 << (a.inv_shift - k)) : (255 >> (k - a.inv_shift));
        } else {
            // exact floor(numer / s): reciprocal estimate, then at most one step either way
            // (numer < 2^30 and s >= 1, so the estimate is within 1 of the quotient)
            int q = __float2int_rz(__fmul_rz(numer_f, __frcp_rn((float)s)));
            int rem = numer - q * s;
            if (rem < 0) { --q; rem += s; }
            if (rem < 0) { --q; rem += s; }
            if (rem >= s) { ++q; rem -= s; }
            if (rem >= s) { ++q; }
            inv = q;
        }
        inv = min(max(inv, 0), 32767);
        const float invs = (float)inv * out_mul;  // inv * 2^-(shift + 85), exact

#pragma unroll
        for (int j = 0; j < NCH; ++j) {
            const int chunk = j * G + gl;
            if (!(row_ok && chunk < a.geom.nchunks)) continue;
            uint32_t aw[4] = {0, 0, 0, 0};
            if (has_add) {
                const uint4 av = ldg16(a.addend + row * a.ldadd + (long long)chunk * 16);
                aw[0] = av.x; aw[1] = av.y; aw[2] = av.z; aw[3] = av.w;
            }
            uint32_t ow[4];
#pragma unroll
            for (int w = 0; w < 4; ++w) {
                // floor(score * inv / 2^shift) lands in the low bits of a subnormal (scores are non-negative)
                int o0 = __float_as_int(__fmaf_rd(e[j][w * 4 + 0], invs, 0.0f));
                int o1 = __float_as_int(__fmaf_rd(e[j][w * 4 + 1], invs, 0.0f));
                int o2 = __float_as_int(__fmaf_rd(e[j][w * 4 + 2], invs, 0.0f));
                int o3 = __float_as_int(__fmaf_rd(e[j][w * 4 + 3], invs, 0.0f));
                if (has_add) {
                    o0 = min(o0, 255); o1 = min(o1, 255); o2 = min(o2, 255); o3 = min(o3, 255);
                    o0 = __viaddmin_s32(o0, (int)prmt(aw[w], 0, 0x4440), 255);
                    o1 = __viaddmin_s32(o1, (int)prmt(aw[w], 0, 0x4441), 255);
                    o2 = __viaddmin_s32(o2, (int)prmt(aw[w], 0, 0x4442), 255);
                    o3 = __viaddmin_s32(o3, (int)prmt(aw[w], 0, 0x4443), 255);
                } else {
                    o0 = min(o0, 255); o1 = min(o1, 255); o2 = min(o2, 255); o3 = min(o3, 255);
                }
                const uint32_t lo2 = prmt((uint32_t)o0, (uint32_t)o1, 0x0040);
                const uint32_t hi2 = prmt((uint32_t)o2, (uint32_t)o3, 0x0040);
                ow[w] = prmt(lo2, hi2, 0x5410);
            }
            stg16(a.out + row * a.ldo + (long long)chunk * 16, make_uint4(ow[0], ow[1], ow[2], ow[3]));
        }
    }
}

RowGeom make_geom(int cols) {
    RowGeom g;
    g.nchunks = cols / 16;
    int G = 1;
    while (G < g.nchunks && G < 32) G <<= 1;
    g.G = G;
    g.R = 32 / G;
    return g;
}

// Fill the reciprocal-std table of one rounding token once per device (stream-ordered, then waited for so
// that later launches on any stream see it).  Returns false while `stream` is being captured into a graph and
// the table does not exist yet: the caller then uses the generic kernel for that call.
bool ensure_inv_std_table(int tok, cudaStream_t stream) {
    static std::mutex mu;
    static bool built[64][A4C_RND_COUNT] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return false;
    std::lock_guard<std::mutex> lock(mu);
    if (built[dev][tok]) return true;
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(stream, &cap) != cudaSuccess || cap != cudaStreamCaptureStatusNone) return false;
    build_inv_std_table_kernel<<<(kInvStdEntries + 255) / 256, 256, 0, stream>>>(tok);
    if (cudaGetLastError() != cudaSuccess || cudaStreamSynchronize(stream) != cudaSuccess) return false;
    built[dev][tok] = true;
    return true;
}

int sm_count() {
    int dev = 0, sms = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    return sms;
}

}  // namespace

// Returns A4C_ERR_UNSUPPORTED when the request is outside the fast path's proofs (caller falls back
// to the generic kernel).
int a4c_launch_layernorm_fast(const int8_t* x, long long ldx, const int16_t* gamma, const int16_t* beta,
                              const int8_t* addend, long long ldadd, int8_t* out, long long ldo, long long rows,
                              int cols, int eps_q0, int out_shift, int rounding, int gamma_absmax, int* status,
                              cudaStream_t stream) {
    const int s_out = 15 - out_shift;
    if (s_out < 2 || gamma_absmax <= 0 || gamma_absmax > 16383) return A4C_ERR_UNSUPPORTED;
    if (rounding == A4C_RND_SYMMETRIC_INF || rounding == A4C_RND_SYMMETRIC_ZERO || rounding == A4C_RND_CONV_ODD)
        return A4C_ERR_UNSUPPORTED;
    if (cols > 2048 || status == nullptr || eps_q0 > kInvStdMaxEps) return A4C_ERR_UNSUPPORTED;
    if (!ensure_inv_std_table(rounding, stream)) return A4C_ERR_UNSUPPORTED;
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
    a.geom = make_geom(cols);
    const int nch = (a.geom.nchunks + a.geom.G - 1) / a.geom.G;
    const size_t smem = (size_t)cols * 8 + kWarps * kStages * 8 + 128 + (size_t)kWarps * kStages * a.geom.R * cols;
    const long long n_items = (rows + a.geom.R - 1) / a.geom.R;
    long long blocks = (n_items + kWarps - 1) / kWarps;
    const int per_sm = (int)(200 * 1024 / smem) < 1 ? 1 : (int)(200 * 1024 / smem);
    const long long cap = (long long)sm_count() * (per_sm > 4 ? 4 : per_sm);
    if (blocks > cap) blocks = cap;
    const int fs = rounding == A4C_RND_CONV_EVEN ? 0 : (gamma_absmax <= 511 ? 1 : 2);
#define LN_LAUNCH(NCH_, FS_)                                                                                  \
    do {                                                                                                       \
        cudaFuncSetAttribute(layernorm_fast_kernel<NCH_, FS_>, cudaFuncAttributeMaxDynamicSharedMemorySize,    \
                             (int)smem);                                                                       \
        layernorm_fast_kernel<NCH_, FS_><<<(int)blocks, kThreads, smem, stream>>>(a);                          \
    } while (0)
#define LN_PICK(NCH_)                                                                                          \
    do {                                                                                                       \
        if (fs == 0) LN_LAUNCH(NCH_, 0); else if (fs == 1) LN_LAUNCH(NCH_, 1); else LN_LAUNCH(NCH_, 2);        \
    } while (0)
    if (nch == 1) LN_PICK(1);
    else if (nch == 2) LN_PICK(2);
    else if (nch == 4) LN_PICK(4);
    else return A4C_ERR_UNSUPPORTED;
#undef LN_PICK
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
    a.geom = make_geom(cols);
    const int nch = (a.geom.nchunks + a.geom.G - 1) / a.geom.G;
    const size_t smem = 256 * 32 * 4 + kWarps * kStages * 8 + 128 + (size_t)kWarps * kStages * a.geom.R * cols;
    const long long n_items = (rows + a.geom.R - 1) / a.geom.R;
    long long blocks = (n_items + kWarps - 1) / kWarps;
    const int per_sm = (int)(200 * 1024 / smem) < 1 ? 1 : (int)(200 * 1024 / smem);
    const long long cap = (long long)sm_count() * (per_sm > 4 ? 4 : per_sm);
    if (blocks > cap) blocks = cap;
#define SM_LAUNCH(NCH_)                                                                                        \
    do {                                                                                                       \
        cudaFuncSetAttribute(softmax_fast_kernel<NCH_>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        softmax_fast_kernel<NCH_><<<(int)blocks, kThreads, smem, stream>>>(a);                                 \
    } while (0)
    if (nch == 1) SM_LAUNCH(1);
    else if (nch == 2) SM_LAUNCH(2);
    else return A4C_ERR_UNSUPPORTED;
#undef SM_LAUNCH
    return cudaGetLastError() == cudaSuccess ? A4C_OK : A4C_ERR_CUDA;
}
