// Integer LayerNorm arithmetic shared by the row kernel (rowops_fast.cu) and the Dense kernel that ends in a
// residual Add and a LayerNorm (dense_ln.cu): the exact recipes of layer_norm.cpp:15-121 and
// elementwise_add.cpp:12-37 evaluated on the FP32 and packed-integer pipes.
#pragma once

#include "a4c_common.cuh"

namespace lnm {

constexpr float MAGIC = 12582912.0f;               // 1.5 * 2^23
constexpr uint32_t MAGIC_BITS = 0x4B400000u;
constexpr float TWO_M64 = 5.421010862427522e-20f;  // 2^-64
constexpr float TWO_P64 = 18446744073709551616.0f; // 2^64

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
// float 2^23 + byte K of w (bytes taken as unsigned)
template <int K>
__device__ __forceinline__ float byte_to_f23(uint32_t w) {
    return __uint_as_float(prmt(w, 0x4B000000u, 0x7540 + K));
}

// Round a non-negative binary32 value to an integer with an AIE rounding token.
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

// The defining expression of the Q15 reciprocal standard deviation (layer_norm.cpp:33-39):
// clamp(round_tok(2^15 * (1.0f / sqrtf((float)var))), 0, 32767) with correctly rounded sqrt and divide.
static __device__ __noinline__ int inv_std_exact(int var, int tok) {
    const float inv_f32 = __fdiv_rn(1.0f, __fsqrt_rn(__int2float_rn(var)));
    return clampi(round_float_tok(__fmul_rn(inv_f32, 32768.0f), tok), 0, 32767);
}

// Same value, usually in a handful of instructions: y ~= 2^15 * rsqrt(var) from the approximate unit is within
// 0.02 of the exactly rounded product (both relative errors are below 2^-21.4 and y <= 32768); unless y sits
// that close to a rounding boundary of the mode, rounding y gives the defined result.  The rare boundary cases
// (and var < 4, where the clamp is near) take the exact path.
__device__ __forceinline__ int inv_std_q15(int var, int tok, bool nearest) {
    float y;
    asm("rsqrt.approx.f32 %0, %1;" : "=f"(y) : "f"(__int2float_rn(var)));
    y *= 32768.0f;
    const float fl = floorf(y);
    const float frac = y - fl;
    const float dist = nearest ? fabsf(frac - 0.5f) : fminf(frac, 1.0f - frac);
    if (dist < 0.02f || var < 4) return inv_std_exact(var, tok);
    int q = (int)fl;
    if (nearest) q += frac > 0.5f;
    else if (tok == A4C_RND_CEIL) q += 1;
    return q;
}


// saturate_i8(x + addend) on four packed bytes (elementwise_add.cpp:30-33, SHIFT = 0): sign-extended byte pairs,
// packed add + min(., 127), packed max(., -128), low bytes back into one word
__device__ __forceinline__ uint32_t sat_add_i8x4(uint32_t x, uint32_t a) {
    uint32_t lo = __viaddmin_s16x2(prmt(x, 0, 0x9180), prmt(a, 0, 0x9180), 0x007F007Fu);
    uint32_t hi = __viaddmin_s16x2(prmt(x, 0, 0xB3A2), prmt(a, 0, 0xB3A2), 0x007F007Fu);
    lo = __vimax3_s16x2(lo, 0xFF80FF80u, 0xFF80FF80u);
    hi = __vimax3_s16x2(hi, 0xFF80FF80u, 0xFF80FF80u);
    return prmt(lo, hi, 0x6420);
}

// two 32-bit values -> one register of two 16-bit lanes (a above b), each saturated to [-32768, 32767]
__device__ __forceinline__ uint32_t pack_sat_s16x2(int a, int b) {
    uint32_t d;
    asm("cvt.pack.sat.s16.s32 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
    return d;
}
// four 32-bit values -> four bytes (o0 lowest), each saturated to [0, 255]: clamp and pack in two instructions
__device__ __forceinline__ uint32_t pack_sat_u8x4(int o0, int o1, int o2, int o3) {
    uint32_t hi, w;
    asm("cvt.pack.sat.u8.s32.b32 %0, %1, %2, %3;" : "=r"(hi) : "r"(o3), "r"(o2), "r"(0));
    asm("cvt.pack.sat.u8.s32.b32 %0, %1, %2, %3;" : "=r"(w) : "r"(o1), "r"(o0), "r"(hi));
    return w;
}

}  // namespace lnm
