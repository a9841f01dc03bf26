// A whole chain of narrow Dense layers in ONE kernel: every weight matrix and bias vector of the chain sits in
// shared memory for the life of the block, a block walks over tiles of up to 32 input rows, and the int8 activations
// between layers never leave shared memory.
//
// Each layer is dense_single::run of aie4ml (dense_bias_relu.cpp:67-166): int8 x int8 products accumulated in
// int32 on top of the bias, SRS with the chain's rounding token, saturation, ReLU after the saturation.  The
// reference wires such layers buffer to buffer in its top graph (top_graph.h.jinja); here they are wired through
// shared memory.  Small multi-layer perceptrons (a 16-64-32-32-5 network at batch 1024, say) are bound by launch
// latency when run layer by layer; this kernel is one launch and reads each input row and writes each output row
// exactly once.
//
// Work split inside a tile: one (row, output neuron) pair per thread per step, pairs enumerated neuron-fastest, so
// a warp reads one activation row (a broadcast) against 32 weight rows.  Weight rows are padded to an odd
// number of 16-byte pieces, which spreads the 128-bit loads of a quarter-warp over all banks.
#include "a4c_common.cuh"
#include "a4c_kernels.h"

namespace {

constexpr int kThreads = 256;
constexpr int kTileRows = 32;   // most rows a block takes at a time (small batches use 16 or 8 to reach more SMs)
constexpr int kMaxLayers = 8;
constexpr int kMaxDim = 256;
constexpr size_t kMaxSmem = 200 * 1024;

struct SmallMlpArgs {
    const uint8_t* X; long long ldx; int x_unsigned;
    uint8_t* Y; long long ldy;
    long long M;
    int n_layers;
    int dims[kMaxLayers + 1];
    const int8_t* W[kMaxLayers]; long long ldw[kMaxLayers];
    const int32_t* bias[kMaxLayers];
    int w_off[kMaxLayers], b_off[kMaxLayers];   // byte offsets in shared memory
    int kp[kMaxLayers];                          // padded K (bytes per weight row)
    RoundParams rp[kMaxLayers];
    int relu[kMaxLayers];
    int lo_last, hi_last;
    int act_pitch, act_off0, act_off1;
    int tile_rows;
    int x_vec;                 // input rows can be read in 16-byte pieces
    int w_vec[kMaxLayers];     // the same for a layer's weight rows
};

// round_up(n, 16), plus 16 when that is an even number of 16-byte pieces
__host__ __device__ inline int odd_pitch(int n) {
    int p = (n + 15) / 16 * 16;
    if (((p / 16) & 1) == 0) p += 16;
    return p;
}

__device__ __forceinline__ int dp4a_ss(uint32_t a, uint32_t b, int c) {
    int d;
    asm("dp4a.s32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
__device__ __forceinline__ int dp4a_us(uint32_t a, uint32_t b, int c) {
    int d;
    asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}

__global__ void __launch_bounds__(kThreads) mlp_small_kernel(SmallMlpArgs a) {
    extern __shared__ __align__(16) uint8_t smem[];
    const int t = threadIdx.x;

    // constants of every layer, once per block; padding bytes of the weight rows are zero
    for (int l = 0; l < a.n_layers; ++l) {
        const int K = a.dims[l], N = a.dims[l + 1], kp = a.kp[l];
        uint8_t* w = smem + a.w_off[l];
        if (a.w_vec[l]) {
            // 16 bytes per thread; bytes at and beyond K (the caller's row padding, contents unknown) are cleared
            const int vpr = kp / 16;
            for (int i = t; i < N * vpr; i += kThreads) {
                const int n = i / vpr, j = i - n * vpr;
                uint4 v = make_uint4(0, 0, 0, 0);
                if (j * 16 < K) {
                    v = __ldg(reinterpret_cast<const uint4*>(a.W[l] + (long long)n * a.ldw[l] + j * 16));
                    const int valid = K - j * 16;   // > 0
                    if (valid < 16) {
                        uint32_t* p = &v.x;
#pragma unroll
                        for (int q = 0; q < 4; ++q) {
                            const int vb = valid - q * 4;
                            p[q] = vb >= 4 ? p[q] : (vb <= 0 ? 0u : (p[q] & ((1u << (8 * vb)) - 1u)));
                        }
                    }
                }
                *reinterpret_cast<uint4*>(w + n * kp + j * 16) = v;
            }
        } else {
            for (int i = t; i < N * kp; i += kThreads) {
                const int n = i / kp, k = i - n * kp;
                w[i] = k < K ? (uint8_t)a.W[l][(long long)n * a.ldw[l] + k] : 0;
            }
        }
        int32_t* b = reinterpret_cast<int32_t*>(smem + a.b_off[l]);
        for (int i = t; i < N; i += kThreads) b[i] = a.bias[l] ? __ldg(a.bias[l] + i) : 0;
    }
    // activation buffers start zeroed so that the padding of a row multiplies as zero from the first tile on
    for (int i = t; i < 2 * kTileRows * a.act_pitch / 16; i += kThreads)
        reinterpret_cast<uint4*>(smem + a.act_off0)[i] = make_uint4(0, 0, 0, 0);
    __syncthreads();

    const int TR = a.tile_rows;
    const long long n_tiles = (a.M + TR - 1) / TR;
    for (long long tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) {
        const long long row0 = tile * TR;
        const int rows = (int)((a.M - row0) < TR ? (a.M - row0) : TR);
        uint8_t* cur = smem + a.act_off0;
        uint8_t* nxt = smem + a.act_off1;
        if (a.x_vec) {
            // whole 16-byte pieces of each input row (what lies beyond K0 meets zero weights)
            const int vpr = (a.dims[0] + 15) / 16;
            for (int i = t; i < rows * vpr; i += kThreads) {
                const int r = i / vpr, j = i - r * vpr;
                *reinterpret_cast<uint4*>(cur + r * a.act_pitch + j * 16) =
                    __ldg(reinterpret_cast<const uint4*>(a.X + (row0 + r) * a.ldx + j * 16));
            }
        } else {
            const int K0 = a.dims[0];
            for (int i = t; i < rows * K0; i += kThreads) {
                const int r = i / K0, k = i - r * K0;
                cur[r * a.act_pitch + k] = a.X[(row0 + r) * a.ldx + k];
            }
        }
        __syncthreads();
        for (int l = 0; l < a.n_layers; ++l) {
            const int N = a.dims[l + 1], kp = a.kp[l];
            const int steps = (a.dims[l] + 15) / 16;
            const uint8_t* w = smem + a.w_off[l];
            const int32_t* b = reinterpret_cast<const int32_t*>(smem + a.b_off[l]);
            const bool last = l == a.n_layers - 1;
            const bool in_unsigned = l == 0 && a.x_unsigned;
            const int lo = last ? a.lo_last : (a.relu[l] ? 0 : -128), hi = last ? a.hi_last : 127;
            for (int idx = t; idx < rows * N; idx += kThreads) {
                const int r = idx / N, n = idx - r * N;
                const uint4* ap = reinterpret_cast<const uint4*>(cur + r * a.act_pitch);
                const uint4* wp = reinterpret_cast<const uint4*>(w + n * kp);
                int acc = b[n];
                if (in_unsigned) {
                    for (int s = 0; s < steps; ++s) {
                        const uint4 av = ap[s], wv = wp[s];
                        acc = dp4a_us(av.x, wv.x, acc); acc = dp4a_us(av.y, wv.y, acc);
                        acc = dp4a_us(av.z, wv.z, acc); acc = dp4a_us(av.w, wv.w, acc);
                    }
                } else {
                    for (int s = 0; s < steps; ++s) {
                        const uint4 av = ap[s], wv = wp[s];
                        acc = dp4a_ss(av.x, wv.x, acc); acc = dp4a_ss(av.y, wv.y, acc);
                        acc = dp4a_ss(av.z, wv.z, acc); acc = dp4a_ss(av.w, wv.w, acc);
                    }
                }
                const int v = clampi(round_shift_i32(acc, a.rp[l]), lo, hi);
                nxt[r * a.act_pitch + n] = (uint8_t)v;
            }
            __syncthreads();
            uint8_t* sw = cur; cur = nxt; nxt = sw;
        }
        {
            const int NL = a.dims[a.n_layers];
            for (int i = t; i < rows * NL; i += kThreads) {
                const int r = i / NL, n = i - r * NL;
                a.Y[(row0 + r) * a.ldy + n] = cur[r * a.act_pitch + n];
            }
        }
        __syncthreads();
    }
}

}  // namespace

// A4C_OK when the fused kernel can run this chain, A4C_ERR_UNSUPPORTED otherwise (the caller then runs the chain
// layer by layer).
int a4c_mlp_small_supported(int n_layers, const int* dims, int out_dtype) {
    if (n_layers < 1 || n_layers > kMaxLayers) return A4C_ERR_UNSUPPORTED;
    if (out_dtype != A4C_I8 && out_dtype != A4C_U8) return A4C_ERR_UNSUPPORTED;
    size_t bytes = 0;
    int widest = 0;
    for (int l = 0; l <= n_layers; ++l) {
        if (dims[l] > kMaxDim) return A4C_ERR_UNSUPPORTED;
        if (dims[l] > widest) widest = dims[l];
    }
    for (int l = 0; l < n_layers; ++l) bytes += (size_t)dims[l + 1] * odd_pitch(dims[l]) + (size_t)dims[l + 1] * 4 + 32;
    bytes += 2 * (size_t)kTileRows * odd_pitch(widest);
    return bytes <= kMaxSmem ? A4C_OK : A4C_ERR_UNSUPPORTED;
}

int a4c_launch_mlp_small(const void* X, long long ldx, int x_unsigned, int n_layers, const int* dims,
                         const int8_t* const* Wt, const long long* ldw, const int32_t* const* bias, const int* shift,
                         const int* relu, int rounding, void* Y, long long ldy, int out_dtype, long long M,
                         cudaStream_t stream) {
    const int sup = a4c_mlp_small_supported(n_layers, dims, out_dtype);
    if (sup != A4C_OK) return sup;
    if (M == 0) return A4C_OK;
    SmallMlpArgs a;
    a.X = (const uint8_t*)X; a.ldx = ldx; a.x_unsigned = x_unsigned; a.Y = (uint8_t*)Y; a.ldy = ldy; a.M = M;
    a.n_layers = n_layers;
    int off = 0, widest = 0;
    for (int l = 0; l <= n_layers; ++l) {
        a.dims[l] = dims[l];
        if (dims[l] > widest) widest = dims[l];
    }
    for (int l = 0; l < n_layers; ++l) {
        a.W[l] = Wt[l]; a.ldw[l] = ldw[l]; a.bias[l] = bias ? bias[l] : nullptr;
        a.kp[l] = odd_pitch(dims[l]);
        a.w_off[l] = off; off += dims[l + 1] * a.kp[l];
        off = (off + 15) / 16 * 16;
        a.b_off[l] = off; off += dims[l + 1] * 4;
        off = (off + 15) / 16 * 16;
        a.rp[l] = make_round_params(shift[l], rounding);
        a.relu[l] = relu[l];
        a.w_vec[l] = ((uintptr_t)Wt[l] % 16 == 0 && ldw[l] % 16 == 0 && ldw[l] >= (dims[l] + 15) / 16 * 16) ? 1 : 0;
    }
    a.x_vec = ((uintptr_t)X % 16 == 0 && ldx % 16 == 0 && ldx >= (dims[0] + 15) / 16 * 16) ? 1 : 0;
    dtype_range(out_dtype, a.lo_last, a.hi_last);
    if (relu[n_layers - 1] && a.lo_last < 0) a.lo_last = 0;
    a.act_pitch = odd_pitch(widest);
    a.act_off0 = off; off += kTileRows * a.act_pitch;
    a.act_off1 = off; off += kTileRows * a.act_pitch;
    const size_t smem = (size_t)off;
    int dev = 0, sms = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    a.tile_rows = M >= 32LL * 2 * sms ? 32 : (M >= 16LL * 2 * sms ? 16 : 8);
    const long long tiles = (M + a.tile_rows - 1) / a.tile_rows;
    int per_sm = (int)((220 * 1024) / (smem + 1024));
    if (per_sm < 1) per_sm = 1;
    if (per_sm > 4) per_sm = 4;
    const long long cap = (long long)sms * per_sm;
    const int grid = (int)(tiles < cap ? tiles : cap);
    if (smem > 48 * 1024 &&
        cudaFuncSetAttribute(mlp_small_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
        return A4C_ERR_CUDA;
    mlp_small_kernel<<<grid, kThreads, smem, stream>>>(a);
    return cudaGetLastError() == cudaSuccess ? A4C_OK : A4C_ERR_CUDA;
}
