// Shared device helpers: the "SRS" step (rounding right shift + saturation) that every aie4ml
// kernel ends with, plus error codes of the C ABI.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

// ---- C-ABI return codes ---------------------------------------------------------------------
#define A4C_OK 0
#define A4C_ERR_INVALID_ARG (-1)     // bad shape, shift, enum value
#define A4C_ERR_ALIGNMENT (-2)       // pointer / pitch alignment the chosen kernel needs
#define A4C_ERR_UNSUPPORTED (-3)     // valid request, no kernel for it
#define A4C_ERR_CUDA (-4)            // a CUDA runtime / driver call failed
#define A4C_ERR_TOO_LARGE (-5)       // exceeds a stated maximum
#define A4C_ERR_DEVICE_TIMEOUT (-6)  // a bounded device-side wait gave up (read via a4c_device_status)

// ---- enums shared with the host side -----------------------------------------------------------
enum A4cRounding : int {
    A4C_RND_FLOOR = 0,
    A4C_RND_CEIL = 1,
    A4C_RND_POSITIVE_INF = 2,  // nearest, ties toward +inf ("round half up")
    A4C_RND_NEGATIVE_INF = 3,  // nearest, ties toward -inf
    A4C_RND_SYMMETRIC_INF = 4,   // nearest, ties away from zero
    A4C_RND_SYMMETRIC_ZERO = 5,  // nearest, ties toward zero
    A4C_RND_CONV_EVEN = 6,       // nearest, ties to even
    A4C_RND_CONV_ODD = 7,        // nearest, ties to odd
    A4C_RND_COUNT = 8
};

enum A4cDtype : int { A4C_I8 = 0, A4C_U8 = 1, A4C_I16 = 2 };

// Rounding right shift, exact for every int32 input (no intermediate overflow): split into
// quotient q = v >> s and remainder r in [0, 2^s), then decide the +1 from r alone.
//   inc = (r + c0 + sgn*(v<0) + (par & (q ^ par_flip) & 1)) >> s
// with per-mode constants (half = 2^(s-1), full = 2^s - 1):
//   floor          c0 = 0
//   ceil           c0 = full
//   positive_inf   c0 = half
//   negative_inf   c0 = half - 1
//   symmetric_inf  c0 = half,     minus 1 when v < 0
//   symmetric_zero c0 = half - 1, plus 1 when v < 0
//   conv_even      c0 = half - 1, plus 1 when q is odd
//   conv_odd       c0 = half - 1, plus 1 when q is even
struct RoundParams {
    int shift;         // 0..31
    uint32_t mask;     // 2^shift - 1
    uint32_t c0;       // additive constant
    int neg_term;      // added when v < 0: -1, 0 or +1
    uint32_t par_use;  // 1 if the quotient's parity participates
    uint32_t par_flip; // 0: add when q odd; 1: add when q even
};

__host__ __device__ inline RoundParams make_round_params(int shift, int mode) {
    RoundParams p;
    p.shift = shift;
    p.mask = shift > 0 ? ((shift >= 32 ? 0u : (1u << shift)) - 1u) : 0u;
    const uint32_t half = shift > 0 ? (1u << (shift - 1)) : 0u;
    p.c0 = 0;
    p.neg_term = 0;
    p.par_use = 0;
    p.par_flip = 0;
    if (shift <= 0) return p;
    switch (mode) {
        case A4C_RND_FLOOR: break;
        case A4C_RND_CEIL: p.c0 = p.mask; break;
        case A4C_RND_POSITIVE_INF: p.c0 = half; break;
        case A4C_RND_NEGATIVE_INF: p.c0 = half - 1; break;
        case A4C_RND_SYMMETRIC_INF: p.c0 = half; p.neg_term = -1; break;
        case A4C_RND_SYMMETRIC_ZERO: p.c0 = half - 1; p.neg_term = 1; break;
        case A4C_RND_CONV_EVEN: p.c0 = half - 1; p.par_use = 1; break;
        default: p.c0 = half - 1; p.par_use = 1; p.par_flip = 1; break;
    }
    return p;
}

// Generic rounding shift of a 32-bit value (any mode, runtime parameters).
__device__ __forceinline__ int round_shift_i32(int v, const RoundParams& p) {
    if (p.shift == 0) return v;
    const int q = v >> p.shift;
    const uint32_t r = (uint32_t)v & p.mask;
    uint32_t t = r + p.c0;
    t += (uint32_t)(p.neg_term & (v >> 31));  // neg_term * (v < 0): (v>>31) is all ones when negative
    // neg_term = -1: (-1 & -1) = -1 -> subtract 1; neg_term = +1: (1 & -1) = 1 -> add 1
    t += p.par_use & ((uint32_t)q ^ p.par_flip) & 1u;
    return q + (int)(t >> p.shift);
}

// Compile-time-mode variant: the common modes cost 4-5 instructions.
template <int MODE>
__device__ __forceinline__ int round_shift_i32_t(int v, int shift, uint32_t mask, uint32_t c0) {
    // shift > 0 is guaranteed by the caller
    const int q = v >> shift;
    const uint32_t r = (uint32_t)v & mask;
    uint32_t t = r + c0;
    if (MODE == A4C_RND_SYMMETRIC_INF) t -= (uint32_t)v >> 31;
    if (MODE == A4C_RND_SYMMETRIC_ZERO) t += (uint32_t)v >> 31;
    if (MODE == A4C_RND_CONV_EVEN) t += (uint32_t)q & 1u;
    if (MODE == A4C_RND_CONV_ODD) t += ~(uint32_t)q & 1u;
    return q + (int)(t >> shift);
}

// 64-bit variant for products that exceed int32 (LayerNorm's inv_std * gamma stays in int32;
// this is for completeness of the add kernel on int16).
__device__ __forceinline__ long long round_shift_i64(long long v, int shift, int mode) {
    if (shift <= 0) return v;
    const long long q = v >> shift;
    const unsigned long long r = (unsigned long long)v & ((1ull << shift) - 1ull);
    const unsigned long long half = 1ull << (shift - 1);
    bool inc;
    switch (mode) {
        case A4C_RND_FLOOR: inc = false; break;
        case A4C_RND_CEIL: inc = r != 0; break;
        case A4C_RND_POSITIVE_INF: inc = r >= half; break;
        case A4C_RND_NEGATIVE_INF: inc = r > half; break;
        case A4C_RND_SYMMETRIC_INF: inc = v >= 0 ? r >= half : r > half; break;
        case A4C_RND_SYMMETRIC_ZERO: inc = v >= 0 ? r > half : r >= half; break;
        case A4C_RND_CONV_EVEN: inc = r > half || (r == half && (q & 1)); break;
        default: inc = r > half || (r == half && !(q & 1)); break;
    }
    return q + (inc ? 1 : 0);
}

__host__ __device__ inline void dtype_range(int dtype, int& lo, int& hi) {
    if (dtype == A4C_I8) { lo = -128; hi = 127; }
    else if (dtype == A4C_U8) { lo = 0; hi = 255; }
    else { lo = -32768; hi = 32767; }
}

__device__ __forceinline__ int clampi(int v, int lo, int hi) { return min(max(v, lo), hi); }

// Bounded spin support: a device-global status word per library instance.  Non-zero means a wait
// gave up; the value encodes where.
#define A4C_SPIN_LIMIT_NS 2000000000ull  // 2 s

__device__ __forceinline__ uint64_t a4c_globaltimer() {
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
