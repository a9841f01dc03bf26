// Row kernels: quantized LayerNorm, quantized Softmax (HCCS surrogate / accurate integer exp) and
// saturating elementwise Add.  All are HBM-bound: one 128-bit load and one 128-bit store per 16
// int8 elements, a row stays in registers between its reduction and normalisation passes, and a
// following saturating Add can be fused so the intermediate never touches HBM.
//
// Arithmetic follows the aie4ml AIE kernels:
//   layer_norm.cpp:15-121   (statistics, Q15 reciprocal std, Q7 gamma, Q15 beta, two SRS steps)
//   softmax.cpp:20-88       (HCCS: score = B - S*min(max-x, Dmax))
//   softmax.cpp:252-273     (exp_score16: 2nd-order integer exp) and :333-384
//   elementwise_add.cpp:12-37
#include "a4c_common.cuh"
#include "a4c_kernels.h"

namespace {

constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;

__device__ __forceinline__ uint4 ldg16(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ void stg16(void* p, uint4 v) {
    asm volatile("st.global.v4.u32 [%0], {%1,%2,%3,%4};" :: "l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
__device__ __forceinline__ int sbyte(uint32_t w, int k) { return (int)(w << (24 - 8 * k)) >> 24; }
__device__ __forceinline__ int ubyte(uint32_t w, int k) { return (int)((w >> (8 * k)) & 0xFFu); }
__device__ __forceinline__ int dp4a_ss(uint32_t a, uint32_t b, int c) {
    int d;
    asm("dp4a.s32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
__device__ __forceinline__ uint32_t pack4(int a, int b, int c, int d) {
    return (uint32_t)(a & 0xFF) | ((uint32_t)(b & 0xFF) << 8) | ((uint32_t)(c & 0xFF) << 16) | ((uint32_t)d << 24);
}

// Round a non-negative binary32 value to an integer with an AIE rounding token.
__device__ __forceinline__ int round_float_tok(float f, int tok) {
    const float fl = floorf(f);
    const float frac = f - fl;  // exact
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

// Geometry of a row of `cols` bytes split into 16-byte chunks over a group of G lanes.
struct RowGeom {
    int nchunks;  // cols / 16
    int G;        // lanes per row (power of two, <= 32)
    int R;        // rows per warp = 32 / G
};

__host__ inline RowGeom make_geom(int cols) {
    RowGeom g;
    g.nchunks = cols / 16;
    int G = 1;
    while (G < g.nchunks && G < 32) G <<= 1;
    g.G = G;
    g.R = 32 / G;
    return g;
}

// ------------------------------------------------------------------------------------------------
// LayerNorm
// ------------------------------------------------------------------------------------------------
struct LnArgs {
    const int8_t* x; long long ldx;
    const int16_t* gamma; const int16_t* beta;
    const int8_t* addend; long long ldadd;
    int pre_add;  // the addend joins the INPUT (saturating, before the statistics) instead of the result
    int8_t* out; long long ldo;
    long long rows; int cols, log2c, eps_q0, rounding;
    RoundParams rp_gamma;  // shift 7
    RoundParams rp_out;    // shift 15 - out_shift
    RowGeom geom;
};

template <int NCH>
__global__ void __launch_bounds__(kThreads) layernorm_kernel(LnArgs a) {
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const int G = a.geom.G, R = a.geom.R;
    const int sub = lane / G, gl = lane % G;
    const long long warp_global = (long long)blockIdx.x * kWarps + warp;
    const long long stride = (long long)gridDim.x * kWarps * R;

    for (long long row_base = warp_global * R; row_base < a.rows; row_base += stride) {
        const long long row = row_base + sub;
        const bool row_ok = row < a.rows;
        uint4 xv[NCH];
        int sum_x = 0, sum_sq = 0;
#pragma unroll
        for (int j = 0; j < NCH; ++j) {
            const int chunk = j * G + gl;
            xv[j] = make_uint4(0, 0, 0, 0);
            if (row_ok && chunk < a.geom.nchunks) {
                xv[j] = ldg16(a.x + row * a.ldx + (long long)chunk * 16);
                if (a.pre_add) {  // x <- saturate(x + addend) (elementwise_add.cpp:30-33 with SHIFT = 0)
                    const uint4 av = ldg16(a.addend + row * a.ldadd + (long long)chunk * 16);
                    uint32_t xw[4] = {xv[j].x, xv[j].y, xv[j].z, xv[j].w};
                    const uint32_t aw[4] = {av.x, av.y, av.z, av.w};
#pragma unroll
                    for (int w = 0; w < 4; ++w)
                        xw[w] = pack4(clampi(sbyte(xw[w], 0) + sbyte(aw[w], 0), -128, 127),
                                      clampi(sbyte(xw[w], 1) + sbyte(aw[w], 1), -128, 127),
                                      clampi(sbyte(xw[w], 2) + sbyte(aw[w], 2), -128, 127),
                                      clampi(sbyte(xw[w], 3) + sbyte(aw[w], 3), -128, 127));
                    xv[j] = make_uint4(xw[0], xw[1], xw[2], xw[3]);
                }
            }
            sum_x = dp4a_ss(xv[j].x, 0x01010101u, sum_x); sum_sq = dp4a_ss(xv[j].x, xv[j].x, sum_sq);
            sum_x = dp4a_ss(xv[j].y, 0x01010101u, sum_x); sum_sq = dp4a_ss(xv[j].y, xv[j].y, sum_sq);
            sum_x = dp4a_ss(xv[j].z, 0x01010101u, sum_x); sum_sq = dp4a_ss(xv[j].z, xv[j].z, sum_sq);
            sum_x = dp4a_ss(xv[j].w, 0x01010101u, sum_x); sum_sq = dp4a_ss(xv[j].w, xv[j].w, sum_sq);
        }
        for (int off = 1; off < G; off <<= 1) {
            sum_x += __shfl_xor_sync(0xffffffffu, sum_x, off);
            sum_sq += __shfl_xor_sync(0xffffffffu, sum_sq, off);
        }
        // layer_norm.cpp:23-31
        const int mu = (sum_x + (a.cols >> 1)) >> a.log2c;
        const int centered = (int)((uint32_t)sum_sq - 2u * (uint32_t)mu * (uint32_t)sum_x +
                                   (uint32_t)a.cols * (uint32_t)mu * (uint32_t)mu);
        int var = centered >> a.log2c;
        var = max(var, 0) + a.eps_q0;
        // layer_norm.cpp:33-39; 1/sqrt in correctly rounded binary32
        const float inv_f = __fdiv_rn(1.0f, __fsqrt_rn(__int2float_rn(var)));
        const int inv_std = clampi(round_float_tok(__fmul_rn(inv_f, 32768.0f), a.rounding), 0, 32767);

#pragma unroll
        for (int j = 0; j < NCH; ++j) {
            const int chunk = j * G + gl;
            if (!(row_ok && chunk < a.geom.nchunks)) continue;
            const uint4* gp = reinterpret_cast<const uint4*>(a.gamma + chunk * 16);
            const uint4* bp = reinterpret_cast<const uint4*>(a.beta + chunk * 16);
            const uint4 g0 = __ldg(gp), g1 = __ldg(gp + 1), b0 = __ldg(bp), b1 = __ldg(bp + 1);
            const uint32_t gw[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
            const uint32_t bw[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
            const uint32_t xw[4] = {xv[j].x, xv[j].y, xv[j].z, xv[j].w};
            uint32_t ow[4];
#pragma unroll
            for (int w = 0; w < 4; ++w) {
                int o[4];
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const int e = w * 4 + k;
                    const int gam = (int)(int16_t)(gw[e >> 1] >> (16 * (e & 1)));
                    const int bet = (int)(int16_t)(bw[e >> 1] >> (16 * (e & 1)));
                    const int vd = sbyte(xw[w], k) - mu;  // fits int16 (layer_norm.cpp:105-106)
                    const int fscale = clampi(round_shift_i32(inv_std * gam, a.rp_gamma), -32768, 32767);
                    const int acc = (int)((uint32_t)(vd * fscale) + (uint32_t)bet);
                    o[k] = clampi(round_shift_i32(acc, a.rp_out), -128, 127);
                }
                ow[w] = pack4(o[0], o[1], o[2], o[3]);
            }
            if (a.addend && !a.pre_add) {  // fused saturating Add (elementwise_add.cpp:30-33 with SHIFT = 0)
                const uint4 av = ldg16(a.addend + row * a.ldadd + (long long)chunk * 16);
                const uint32_t aw[4] = {av.x, av.y, av.z, av.w};
#pragma unroll
                for (int w = 0; w < 4; ++w)
                    ow[w] = pack4(clampi(sbyte(ow[w], 0) + sbyte(aw[w], 0), -128, 127),
                                  clampi(sbyte(ow[w], 1) + sbyte(aw[w], 1), -128, 127),
                                  clampi(sbyte(ow[w], 2) + sbyte(aw[w], 2), -128, 127),
                                  clampi(sbyte(ow[w], 3) + sbyte(aw[w], 3), -128, 127));
            }
            stg16(a.out + row * a.ldo + (long long)chunk * 16, make_uint4(ow[0], ow[1], ow[2], ow[3]));
        }
    }
}

// ------------------------------------------------------------------------------------------------
// Softmax
// ------------------------------------------------------------------------------------------------
struct SmArgs {
    const int8_t* x; long long ldx;
    const uint8_t* addend; long long ldadd;  // same dtype as the output, or null
    uint8_t* out; long long ldo;             // pitches in elements
    long long rows; int cols;
    int mode, B, S, Dmax, inv_shift, use_clb, exp_kq, out_dtype;
    RowGeom geom;
};

// exp_score16, softmax.cpp:252-273
__device__ __forceinline__ int exp_score16(int d, int kq) {
    int z = min(d * kq, 32767);
    const int zint = z >> 8, zfrac = z & 255;
    const int t = (zfrac * 2811) >> 8;
    const int inner = t - 11004;
    const int t2 = (inner * zfrac) >> 8;
    int e = t2 + 16384;
    e = zint >= 16 ? 0 : (e >> (zint & 15));  // the four conditional halvings compose to one shift
    return e;
}

template <int NCH>
__global__ void __launch_bounds__(kThreads) softmax_kernel(SmArgs a) {
    __shared__ int lut[256];  // score as a function of d = max - x
    {
        const int d = threadIdx.x;
        if (d < 256) {
            int s;
            if (a.mode == 0) s = clampi(a.B - a.S * min(d, a.Dmax), -32768, 32767);
            else s = exp_score16(d, a.exp_kq);
            lut[d] = s;
        }
    }
    __syncthreads();

    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const int G = a.geom.G, R = a.geom.R;
    const int sub = lane / G, gl = lane % G;
    const long long warp_global = (long long)blockIdx.x * kWarps + warp;
    const long long stride = (long long)gridDim.x * kWarps * R;
    const bool out16 = a.out_dtype == A4C_I16;
    const long long numer = out16 ? 32767ll : (255ll << a.inv_shift);
    const int out_shift = out16 ? 0 : a.inv_shift;
    const int lo = out16 ? -32768 : 0, hi = out16 ? 32767 : 255;

    for (long long row_base = warp_global * R; row_base < a.rows; row_base += stride) {
        const long long row = row_base + sub;
        const bool row_ok = row < a.rows;
        uint4 xv[NCH];
        uint32_t vmax = 0x80808080u;  // four int8 -128
#pragma unroll
        for (int j = 0; j < NCH; ++j) {
            const int chunk = j * G + gl;
            xv[j] = make_uint4(0x80808080u, 0x80808080u, 0x80808080u, 0x80808080u);
            if (row_ok && chunk < a.geom.nchunks) xv[j] = ldg16(a.x + row * a.ldx + (long long)chunk * 16);
            vmax = __vmaxs4(vmax, __vmaxs4(__vmaxs4(xv[j].x, xv[j].y), __vmaxs4(xv[j].z, xv[j].w)));
        }
        int m = max(max(sbyte(vmax, 0), sbyte(vmax, 1)), max(sbyte(vmax, 2), sbyte(vmax, 3)));
        for (int off = 1; off < G; off <<= 1) m = max(m, __shfl_xor_sync(0xffffffffu, m, off));

        int sum = 0;
#pragma unroll
        for (int j = 0; j < NCH; ++j) {
            const int chunk = j * G + gl;
            if (!(row_ok && chunk < a.geom.nchunks)) continue;
            const uint32_t xw[4] = {xv[j].x, xv[j].y, xv[j].z, xv[j].w};
#pragma unroll
            for (int w = 0; w < 4; ++w)
#pragma unroll
                for (int k = 0; k < 4; ++k) sum += lut[m - sbyte(xw[w], k)];
        }
        for (int off = 1; off < G; off <<= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off);

        // softmax.cpp:61-76 / batched_reciprocal :108-127: exact floor(NUMER / sum)
        const int s = sum > 0 ? sum : 1;
        long long inv;
        if (a.use_clb && a.mode == 0) {
            const int k = 31 - __clz(s);
            if (out16) inv = 32767 >> k;
            else inv = a.inv_shift - k >= 0 ? (255ll << (a.inv_shift - k)) : (255ll >> (k - a.inv_shift));
        } else {
            inv = numer / s;
        }
        const int inv_q = (int)min(max(inv, 0ll), 32767ll);

#pragma unroll
        for (int j = 0; j < NCH; ++j) {
            const int chunk = j * G + gl;
            if (!(row_ok && chunk < a.geom.nchunks)) continue;
            const uint32_t xw[4] = {xv[j].x, xv[j].y, xv[j].z, xv[j].w};
            int o[16];
#pragma unroll
            for (int w = 0; w < 4; ++w)
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const int sc = lut[m - sbyte(xw[w], k)];
                    o[w * 4 + k] = clampi((sc * inv_q) >> out_shift, lo, hi);  // floor shift, saturate
                }
            if (!out16) {
                if (a.addend) {
                    const uint4 av = ldg16(a.addend + row * a.ldadd + (long long)chunk * 16);
                    const uint32_t aw[4] = {av.x, av.y, av.z, av.w};
#pragma unroll
                    for (int e = 0; e < 16; ++e) o[e] = min(o[e] + ubyte(aw[e >> 2], e & 3), 255);
                }
                stg16(a.out + row * a.ldo + (long long)chunk * 16,
                      make_uint4(pack4(o[0], o[1], o[2], o[3]), pack4(o[4], o[5], o[6], o[7]),
                                 pack4(o[8], o[9], o[10], o[11]), pack4(o[12], o[13], o[14], o[15])));
            } else {
                uint8_t* op = a.out + (row * a.ldo + (long long)chunk * 16) * 2;
                if (a.addend) {
                    const uint8_t* ap = a.addend + (row * a.ldadd + (long long)chunk * 16) * 2;
                    const uint4 a0 = ldg16(ap), a1 = ldg16(ap + 16);
                    const uint32_t aw[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
#pragma unroll
                    for (int e = 0; e < 16; ++e)
                        o[e] = clampi(o[e] + (int)(int16_t)(aw[e >> 1] >> (16 * (e & 1))), -32768, 32767);
                }
                uint32_t h[8];
#pragma unroll
                for (int e = 0; e < 8; ++e) h[e] = ((uint32_t)o[2 * e] & 0xFFFFu) | ((uint32_t)o[2 * e + 1] << 16);
                stg16(op, make_uint4(h[0], h[1], h[2], h[3]));
                stg16(op + 16, make_uint4(h[4], h[5], h[6], h[7]));
            }
        }
    }
}

// ------------------------------------------------------------------------------------------------
// Elementwise Add
// ------------------------------------------------------------------------------------------------
struct AddArgs {
    const uint8_t* a; long long lda;
    const uint8_t* b; long long ldb;
    uint8_t* out; long long ldo;  // pitches in elements
    long long rows, chunks_per_row;  // 16-byte chunks
    int dtype, rounding;
    RoundParams rp;
};

__global__ void __launch_bounds__(kThreads) add_kernel(AddArgs g) {
    const long long total = g.rows * g.chunks_per_row;
    const int esz = g.dtype == A4C_I16 ? 2 : 1;
    int lo, hi;
    dtype_range(g.dtype, lo, hi);
    for (long long i = (long long)blockIdx.x * kThreads + threadIdx.x; i < total;
         i += (long long)gridDim.x * kThreads) {
        const long long r = i / g.chunks_per_row, c = i % g.chunks_per_row;
        const uint4 av = ldg16(g.a + r * g.lda * esz + c * 16);
        const uint4 bv = ldg16(g.b + r * g.ldb * esz + c * 16);
        const uint32_t aw[4] = {av.x, av.y, av.z, av.w}, bw[4] = {bv.x, bv.y, bv.z, bv.w};
        uint32_t ow[4];
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            if (g.dtype == A4C_I16) {
                int o[2];
#pragma unroll
                for (int k = 0; k < 2; ++k) {
                    const int s = (int)(int16_t)(aw[w] >> (16 * k)) + (int)(int16_t)(bw[w] >> (16 * k));
                    o[k] = clampi(round_shift_i32(s, g.rp), lo, hi);
                }
                ow[w] = ((uint32_t)o[0] & 0xFFFFu) | ((uint32_t)o[1] << 16);
            } else {
                int o[4];
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const int s = g.dtype == A4C_U8 ? ubyte(aw[w], k) + ubyte(bw[w], k) : sbyte(aw[w], k) + sbyte(bw[w], k);
                    o[k] = clampi(round_shift_i32(s, g.rp), lo, hi);
                }
                ow[w] = pack4(o[0], o[1], o[2], o[3]);
            }
        }
        stg16(g.out + r * g.ldo * esz + c * 16, make_uint4(ow[0], ow[1], ow[2], ow[3]));
    }
}

inline bool aligned16(const void* p) { return ((uintptr_t)p & 15u) == 0; }

int grid_for(long long work_items, int per_block) {
    int dev = 0, sms = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    long long blocks = (work_items + per_block - 1) / per_block;
    const long long cap = (long long)sms * 8;  // multiple of the SM count; 8 resident blocks of 256 threads
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    return (int)blocks;
}

}  // namespace

int a4c_launch_layernorm(const int8_t* x, long long ldx, const int16_t* gamma, const int16_t* beta,
                         const int8_t* addend, long long ldadd, int pre_add, int8_t* out, long long ldo, long long rows,
                         int cols, int eps_q0, int out_shift, int rounding, cudaStream_t stream) {
    if (rows < 0 || cols <= 0 || (cols & (cols - 1)) != 0 || out_shift < 0 || out_shift > 15 || eps_q0 < 1 ||
        rounding < 0 || rounding >= A4C_RND_COUNT)
        return A4C_ERR_INVALID_ARG;
    if (rows == 0) return A4C_OK;
    if (cols % 16 != 0 || cols > 8 * 32 * 16) return A4C_ERR_UNSUPPORTED;
    if (!aligned16(x) || !aligned16(out) || !aligned16(gamma) || !aligned16(beta) || ldx % 16 || ldo % 16 ||
        (addend && (!aligned16(addend) || ldadd % 16)))
        return A4C_ERR_ALIGNMENT;
    LnArgs a;
    a.x = x; a.ldx = ldx; a.gamma = gamma; a.beta = beta; a.addend = addend; a.ldadd = ldadd;
    a.pre_add = (addend && pre_add) ? 1 : 0;
    a.out = out; a.ldo = ldo; a.rows = rows; a.cols = cols; a.eps_q0 = eps_q0; a.rounding = rounding;
    a.log2c = 0;
    while ((1 << a.log2c) < cols) ++a.log2c;
    a.rp_gamma = make_round_params(7, rounding);
    a.rp_out = make_round_params(15 - out_shift, rounding);
    a.geom = make_geom(cols);
    const int nch = (a.geom.nchunks + a.geom.G - 1) / a.geom.G;
    const int grid = grid_for((rows + a.geom.R - 1) / a.geom.R, kWarps);
    switch (nch) {
        case 1: layernorm_kernel<1><<<grid, kThreads, 0, stream>>>(a); break;
        case 2: layernorm_kernel<2><<<grid, kThreads, 0, stream>>>(a); break;
        case 4: layernorm_kernel<4><<<grid, kThreads, 0, stream>>>(a); break;
        case 8: layernorm_kernel<8><<<grid, kThreads, 0, stream>>>(a); break;
        default: return A4C_ERR_UNSUPPORTED;
    }
    return cudaGetLastError() == cudaSuccess ? A4C_OK : A4C_ERR_CUDA;
}

int a4c_launch_softmax(const int8_t* x, long long ldx, const void* addend, long long ldadd, void* out,
                       long long ldo, long long rows, int cols, int mode, int B, int S, int Dmax, int inv_shift,
                       int use_clb, int exp_kq, int out_dtype, cudaStream_t stream) {
    if (rows < 0 || cols <= 0 || (mode != 0 && mode != 1) || (out_dtype != A4C_U8 && out_dtype != A4C_I16) ||
        inv_shift < 1 || inv_shift > 30)
        return A4C_ERR_INVALID_ARG;
    if (mode == 0 && (B < 0 || B > 32767 || S < 0 || S > 127 || Dmax < 0 || Dmax > 255)) return A4C_ERR_INVALID_ARG;
    if (mode == 1 && (exp_kq < 1 || exp_kq > 128)) return A4C_ERR_INVALID_ARG;
    if (rows == 0) return A4C_OK;
    if (cols % 16 != 0 || cols > 8 * 32 * 16) return A4C_ERR_UNSUPPORTED;
    const int esz = out_dtype == A4C_I16 ? 2 : 1;
    if (!aligned16(x) || !aligned16(out) || ldx % 16 || (ldo * esz) % 16 ||
        (addend && (!aligned16(addend) || (ldadd * esz) % 16)))
        return A4C_ERR_ALIGNMENT;
    SmArgs a;
    a.x = x; a.ldx = ldx; a.addend = (const uint8_t*)addend; a.ldadd = ldadd; a.out = (uint8_t*)out; a.ldo = ldo;
    a.rows = rows; a.cols = cols; a.mode = mode; a.B = B; a.S = S; a.Dmax = Dmax; a.inv_shift = inv_shift;
    a.use_clb = use_clb; a.exp_kq = exp_kq; a.out_dtype = out_dtype;
    a.geom = make_geom(cols);
    const int nch = (a.geom.nchunks + a.geom.G - 1) / a.geom.G;
    const int grid = grid_for((rows + a.geom.R - 1) / a.geom.R, kWarps);
    switch (nch) {
        case 1: softmax_kernel<1><<<grid, kThreads, 0, stream>>>(a); break;
        case 2: softmax_kernel<2><<<grid, kThreads, 0, stream>>>(a); break;
        case 3: case 4: softmax_kernel<4><<<grid, kThreads, 0, stream>>>(a); break;
        case 5: case 6: case 7: case 8: softmax_kernel<8><<<grid, kThreads, 0, stream>>>(a); break;
        default: return A4C_ERR_UNSUPPORTED;
    }
    return cudaGetLastError() == cudaSuccess ? A4C_OK : A4C_ERR_CUDA;
}

int a4c_launch_add(const void* a, long long lda, const void* b, long long ldb, void* out, long long ldo,
                   long long rows, long long cols, int shift, int rounding, int dtype, cudaStream_t stream) {
    if (rows < 0 || cols <= 0 || shift < 0 || shift > 16 || rounding < 0 || rounding >= A4C_RND_COUNT ||
        dtype < 0 || dtype > 2)
        return A4C_ERR_INVALID_ARG;
    if (rows == 0) return A4C_OK;
    const int esz = dtype == A4C_I16 ? 2 : 1;
    if ((cols * esz) % 16 != 0) return A4C_ERR_UNSUPPORTED;
    if (!aligned16(a) || !aligned16(b) || !aligned16(out) || (lda * esz) % 16 || (ldb * esz) % 16 || (ldo * esz) % 16)
        return A4C_ERR_ALIGNMENT;
    AddArgs g;
    g.a = (const uint8_t*)a; g.lda = lda; g.b = (const uint8_t*)b; g.ldb = ldb; g.out = (uint8_t*)out; g.ldo = ldo;
    g.rows = rows; g.chunks_per_row = cols * esz / 16; g.dtype = dtype; g.rounding = rounding;
    g.rp = make_round_params(shift, rounding);
    if (lda == cols && ldb == cols && ldo == cols) {  // contiguous: one long row
        g.chunks_per_row *= rows;
        g.rows = 1;
    }
    const int grid = grid_for(g.rows * g.chunks_per_row, kThreads);
    add_kernel<<<grid, kThreads, 0, stream>>>(g);
    return cudaGetLastError() == cudaSuccess ? A4C_OK : A4C_ERR_CUDA;
}
