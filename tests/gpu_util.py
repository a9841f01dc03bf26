"""Helpers for the GPU parity tests: device buffers from NumPy arrays and C-ABI calls."""

import ctypes

import numpy as np
import torch

from aie4ml_b200 import lib as a4c
from aie4ml_b200.op_impls.precision import DTYPE_CODE, ROUNDING_CODE

NP = {'int8': np.int8, 'uint8': np.uint8, 'int16': np.int16}
TD = {'int8': torch.int8, 'uint8': torch.uint8, 'int16': torch.int16}


def dev(arr):
    return torch.from_numpy(np.ascontiguousarray(arr)).cuda()


def stream():
    return torch.cuda.current_stream().cuda_stream


def padded(arr, pitch, fill=0x5A):
    """Copy a 2-D array into a wider row-major buffer (row pitch `pitch`), poison in the padding."""
    rows, cols = arr.shape
    buf = np.full((rows, pitch), fill, dtype=arr.dtype)
    buf[:, :cols] = arr
    return buf


def pack_wt(w_kn):
    """[K, N] int8 weights -> [N, Kp] K-contiguous with the pitch padded to 16."""
    K, N = w_kn.shape
    kp = (K + 15) // 16 * 16
    out = np.zeros((N, kp), dtype=np.int8)
    out[:, :K] = w_kn.T
    return out


def dense(a, w_kn, bias, *, shift, tok, relu, out_dtype='int8', algo=0, lda=None, ldy=None):
    L = a4c.load()
    M, K = a.shape
    N = w_kn.shape[1]
    lda = lda or (K + 15) // 16 * 16
    esz = np.dtype(NP[out_dtype]).itemsize
    ldy = ldy or (N * esz + 15) // 16 * 16 // esz
    a_d = dev(padded(a, lda))
    wt = dev(pack_wt(w_kn))
    b_d = dev(bias.astype(np.int32)) if bias is not None else None
    y_d = torch.full((M, ldy), 0x5A if esz == 1 else 0x5A5A, dtype=TD[out_dtype], device='cuda')
    rc = L.a4c_dense_i8(a_d.data_ptr(), lda, wt.data_ptr(), wt.shape[1], b_d.data_ptr() if b_d is not None else None,
                        y_d.data_ptr(), ldy, M, K, N, shift, ROUNDING_CODE[tok], int(relu), DTYPE_CODE[out_dtype],
                        int(a.dtype == np.uint8), algo, stream())
    a4c.check(rc, 'a4c_dense_i8')
    a4c.device_status(stream())
    y = y_d.cpu().numpy()
    pad = y[:, N:]
    assert (pad == (0x5A if esz == 1 else 0x5A5A)).all(), 'kernel wrote into the row padding'
    return y[:, :N]


def bmm(a, b, *, shift, tok, trans_a=False, trans_b=False, out_dtype='int8'):
    L = a4c.load()
    batch = a.shape[0]
    M = a.shape[2] if trans_a else a.shape[1]
    K = a.shape[1] if trans_a else a.shape[2]
    N = b.shape[1] if trans_b else b.shape[2]
    a_d, b_d = dev(a), dev(b)
    c_d = torch.zeros((batch, M, N), dtype=TD[out_dtype], device='cuda')
    rc = L.a4c_bmm_i8(a_d.data_ptr(), a.shape[2], a.shape[1] * a.shape[2], b_d.data_ptr(), b.shape[2],
                      b.shape[1] * b.shape[2], c_d.data_ptr(), N, M * N, batch, M, K, N, int(trans_a), int(trans_b), shift,
                      ROUNDING_CODE[tok], DTYPE_CODE[out_dtype], int(a.dtype == np.uint8), stream())
    a4c.check(rc, 'a4c_bmm_i8')
    return c_d.cpu().numpy()


def add_layer_norm(x, residual, gamma, beta, *, eps_q0, out_shift, tok):
    L = a4c.load()
    rows, cols = x.shape
    x_d, r_d = dev(x), dev(residual)
    g_d, b_d = dev(gamma.astype(np.int16)), dev(beta.astype(np.int16))
    o_d = torch.zeros((rows, cols), dtype=torch.int8, device='cuda')
    rc = L.a4c_add_layernorm_i8(x_d.data_ptr(), cols, r_d.data_ptr(), cols, g_d.data_ptr(), b_d.data_ptr(),
                                o_d.data_ptr(), cols, rows, cols, eps_q0, out_shift, ROUNDING_CODE[tok],
                                int(np.abs(gamma).max()), stream())
    a4c.check(rc, 'a4c_add_layernorm_i8')
    a4c.device_status(stream())
    return o_d.cpu().numpy()


def dense_add_layer_norm(a, w_kn, bias, residual, gamma, beta, *, shift, tok, relu, eps_q0, out_shift, ldr=None, ldo=None):
    """The single kernel through the C ABI; None when the library says the request is outside its envelope."""
    L = a4c.load()
    M, K = a.shape
    N = w_kn.shape[1]
    lda = (K + 15) // 16 * 16
    ldr, ldo = ldr or N, ldo or N
    wt = dev(pack_wt(w_kn))
    gmax = int(np.abs(gamma.astype(np.int64)).max())
    if L.a4c_dense_add_layernorm_supported(M, K, N, lda, wt.shape[1], ldr, ldo, shift, ROUNDING_CODE[tok], out_shift, eps_q0,
                                           gmax) != 0:
        return None
    a_d, r_d = dev(padded(a, lda)), dev(padded(residual, ldr))
    b_d = dev(bias.astype(np.int32)) if bias is not None else None
    g_d, be_d = dev(gamma.astype(np.int16)), dev(beta.astype(np.int16))
    o_d = torch.full((M, ldo), 0x5A, dtype=torch.int8, device='cuda')
    rc = L.a4c_dense_add_layernorm_i8(a_d.data_ptr(), lda, int(a.dtype == np.uint8), wt.data_ptr(), wt.shape[1],
                                      b_d.data_ptr() if b_d is not None else None, shift, int(relu), r_d.data_ptr(), ldr,
                                      g_d.data_ptr(), be_d.data_ptr(), o_d.data_ptr(), ldo, M, K, N, eps_q0, out_shift,
                                      ROUNDING_CODE[tok], gmax, stream())
    a4c.check(rc, 'a4c_dense_add_layernorm_i8')
    a4c.device_status(stream())
    y = o_d.cpu().numpy()
    assert (y[:, N:] == 0x5A).all(), 'kernel wrote into the row padding'
    return y[:, :N]


def layer_norm(x, gamma, beta, *, eps_q0, out_shift, tok, addend=None):
    L = a4c.load()
    rows, cols = x.shape
    x_d, g_d, b_d = dev(x), dev(gamma.astype(np.int16)), dev(beta.astype(np.int16))
    a_d = dev(addend) if addend is not None else None
    o_d = torch.zeros((rows, cols), dtype=torch.int8, device='cuda')
    rc = L.a4c_layernorm_i8(x_d.data_ptr(), cols, g_d.data_ptr(), b_d.data_ptr(), a_d.data_ptr() if a_d is not None else None,
                            cols, o_d.data_ptr(), cols, rows, cols, eps_q0, out_shift, ROUNDING_CODE[tok],
                            int(np.abs(gamma.astype(np.int64)).max()), stream())
    a4c.check(rc, 'a4c_layernorm_i8')
    return o_d.cpu().numpy()


def softmax(x, *, mode, B=0, S=0, Dmax=0, inv_shift=15, use_clb=False, exp_kq=0, out_dtype='uint8', addend=None):
    L = a4c.load()
    rows, cols = x.shape
    x_d = dev(x)
    a_d = dev(addend) if addend is not None else None
    o_d = torch.zeros((rows, cols), dtype=TD[out_dtype], device='cuda')
    rc = L.a4c_softmax_i8(x_d.data_ptr(), cols, a_d.data_ptr() if a_d is not None else None, cols, o_d.data_ptr(), cols,
                          rows, cols, 0 if mode == 'hccs' else 1, B, S, Dmax, inv_shift, int(use_clb), exp_kq,
                          DTYPE_CODE[out_dtype], stream())
    a4c.check(rc, 'a4c_softmax_i8')
    return o_d.cpu().numpy()


def add(a, b, *, shift, tok, dtype):
    L = a4c.load()
    rows, cols = a.shape
    a_d, b_d = dev(a), dev(b)
    o_d = torch.zeros((rows, cols), dtype=TD[dtype], device='cuda')
    rc = L.a4c_add_sat(a_d.data_ptr(), cols, b_d.data_ptr(), cols, o_d.data_ptr(), cols, rows, cols, shift,
                       ROUNDING_CODE[tok], DTYPE_CODE[dtype], stream())
    a4c.check(rc, 'a4c_add_sat')
    return o_d.cpu().numpy()


def mlp_chain(x, layers, *, tok, out_dtype='int8', fn_name='a4c_mlp_i8'):
    """layers: list of (w_kn int8, bias int32 or None, shift, relu).  Calls the chain entry point `fn_name`."""
    L = a4c.load()
    fn = getattr(L, fn_name)
    M, K0 = x.shape
    n = len(layers)
    dims = (ctypes.c_int * (n + 1))(K0, *[w.shape[1] for w, _, _, _ in layers])
    wts = [dev(pack_wt(w)) for w, _, _, _ in layers]
    biases = [dev(b.astype(np.int32)) if b is not None else None for _, b, _, _ in layers]
    wt_ptrs = (ctypes.c_void_p * n)(*[t.data_ptr() for t in wts])
    ldw = (ctypes.c_int64 * n)(*[t.shape[1] for t in wts])
    b_ptrs = (ctypes.c_void_p * n)(*[b.data_ptr() if b is not None else None for b in biases])
    shifts = (ctypes.c_int * n)(*[s for _, _, s, _ in layers])
    relus = (ctypes.c_int * n)(*[int(r) for _, _, _, r in layers])
    lda = (K0 + 15) // 16 * 16
    x_d = dev(padded(x, lda))
    N = layers[-1][0].shape[1]
    esz = np.dtype(NP[out_dtype]).itemsize
    ldy = (N * esz + 15) // 16 * 16 // esz
    y_d = torch.zeros((M, ldy), dtype=TD[out_dtype], device='cuda')
    args = [x_d.data_ptr(), lda, int(x.dtype == np.uint8), n, ctypes.cast(dims, ctypes.c_void_p),
            ctypes.cast(wt_ptrs, ctypes.c_void_p), ctypes.cast(ldw, ctypes.c_void_p), ctypes.cast(b_ptrs, ctypes.c_void_p),
            ctypes.cast(shifts, ctypes.c_void_p), ctypes.cast(relus, ctypes.c_void_p), ROUNDING_CODE[tok], y_d.data_ptr(),
            ldy, DTYPE_CODE[out_dtype], M]
    if fn_name == 'a4c_mlp_i8_static':
        args.append(None)    # status_out: stay asynchronous, a4c_device_status below reads the word
    rc = fn(*args, stream())
    a4c.check(rc, fn_name)
    a4c.device_status(stream())
    return y_d.cpu().numpy()[:, :N]


def attention(qkv, heads_at, *, qk_shift, pv_shift, tok, mode, B=0, S=0, Dmax=0, inv_shift=15, use_clb=False, exp_kq=0,
              out_width=None):
    """One fused attention head over a packed [batch, seq, width] int8 tensor: q, k, v are the 64-column
    slices starting at heads_at = (q0, k0, v0); the result lands in columns [o0, o0 + 64) of a
    [batch, seq_q, out_width] tensor pre-filled with 0x5A (o0 = q0).  Returns that whole tensor."""
    L = a4c.load()
    batch, seq, width = qkv.shape
    q0, k0, v0 = heads_at
    d = dev(qkv)
    ow = out_width or width
    out = torch.full((batch, seq, ow), 0x5A, dtype=torch.int8, device='cuda')
    base = d.data_ptr()
    args = (base + q0, width, seq * width, base + k0, width, seq * width, base + v0, width, seq * width,
            out.data_ptr() + q0, ow, seq * ow, batch, seq, seq, 64, qk_shift, pv_shift)
    sm = (0 if mode == 'hccs' else 1, B, S, Dmax, inv_shift)
    a4c.check(L.a4c_attention_i8_supported(*args, *sm), 'a4c_attention_i8_supported')
    rc = L.a4c_attention_i8(*args, ROUNDING_CODE[tok], *sm, int(use_clb), exp_kq, stream())
    a4c.check(rc, 'a4c_attention_i8')
    a4c.device_status(stream())
    return out.cpu().numpy()


def attention_heads(q, k, v, heads, *, qk_shift, pv_shift, tok, mode, B=0, S=0, Dmax=0, inv_shift=15, use_clb=False,
                    exp_kq=0, layout='cols'):
    """All heads of a layer in one launch: q [batch, sq, heads*64], k and v [batch, 128, heads*64] int8, head h in
    columns [64h, 64h + 64).  Returns the [batch, sq, heads*64] output.  layout 'cols' hands the tensors over as they
    are (heads = column slices, 64 bytes apart); 'blocks' stores every head as its own [rows, 64] matrix
    ([batch, heads, rows, 64]) and converts the result back."""
    L = a4c.load()
    batch, sq, width = q.shape
    sk = k.shape[1]
    if layout == 'blocks':
        blocks = lambda t: np.ascontiguousarray(t.reshape(batch, t.shape[1], heads, 64).transpose(0, 2, 1, 3))
        qd, kd, vd = dev(blocks(q)), dev(blocks(k)), dev(blocks(v))
        out = torch.full((batch, heads, sq, 64), 0x5A, dtype=torch.int8, device='cuda')
        geo = lambda rows: (64, heads * rows * 64, rows * 64)
    else:
        qd, kd, vd = dev(q), dev(k), dev(v)
        out = torch.full((batch, sq, width), 0x5A, dtype=torch.int8, device='cuda')
        geo = lambda rows: (width, rows * width, 64)
    args = (qd.data_ptr(), *geo(sq), kd.data_ptr(), *geo(sk), vd.data_ptr(), *geo(sk), out.data_ptr(), *geo(sq), batch, heads,
            sq, sk, 64, qk_shift, pv_shift)
    sm = (0 if mode == 'hccs' else 1, B, S, Dmax, inv_shift)
    a4c.check(L.a4c_attention_heads_i8_supported(*args, *sm), 'a4c_attention_heads_i8_supported')
    a4c.check(L.a4c_attention_heads_i8(*args, ROUNDING_CODE[tok], *sm, int(use_clb), exp_kq, stream()), 'a4c_attention_heads_i8')
    a4c.device_status(stream())
    res = out.cpu().numpy()
    return res.transpose(0, 2, 1, 3).reshape(batch, sq, width) if layout == 'blocks' else res


def dense16(a, w_kn, bias, *, shift, tok, relu, out_dtype='int8'):
    """int16 activations against int8 (32-bit wrapping accumulator) or int16 (64-bit accumulator) weights."""
    L = a4c.load()
    M, K = a.shape
    N = w_kn.shape[1]
    wide = w_kn.dtype == np.int16
    esz = np.dtype(NP[out_dtype]).itemsize
    ldy = (N * esz + 15) // 16 * 16 // esz
    a_d = dev(np.ascontiguousarray(a.astype(np.int16)))
    wt = dev(np.ascontiguousarray(w_kn.T))
    b_d = dev(bias.astype(np.int32)) if bias is not None else None
    y_d = torch.full((M, ldy), 0x5A if esz == 1 else 0x5A5A, dtype=TD[out_dtype], device='cuda')
    rc = L.a4c_dense_i16(a_d.data_ptr(), K, wt.data_ptr(), 2 if wide else 0, K, b_d.data_ptr() if b_d is not None else None,
                         y_d.data_ptr(), ldy, M, K, N, shift, ROUNDING_CODE[tok], int(relu), DTYPE_CODE[out_dtype], stream())
    a4c.check(rc, 'a4c_dense_i16')
    y = y_d.cpu().numpy()
    assert (y[:, N:] == (0x5A if esz == 1 else 0x5A5A)).all(), 'kernel wrote into the row padding'
    return y[:, :N]


def dense_ta(a_t, w_kn, bias, *, shift, tok, relu, out_dtype='int8'):
    """Dense over a stack of stored [K, M] inputs (int8 / uint8 / int16); returns the stack of [M, N] outputs."""
    L = a4c.load()
    batch, K, M = a_t.shape
    N = w_kn.shape[1]
    a_code = {'int8': 0, 'uint8': 1, 'int16': 2}[a_t.dtype.name]
    w_code = {'int8': 0, 'int16': 2}[w_kn.dtype.name]
    a_d, wt = dev(np.ascontiguousarray(a_t)), dev(np.ascontiguousarray(w_kn.T))
    b_d = dev(bias.astype(np.int32)) if bias is not None else None
    y_d = torch.zeros((batch, M, N), dtype=TD[out_dtype], device='cuda')
    rc = L.a4c_dense_ta(a_d.data_ptr(), a_code, M, K * M, wt.data_ptr(), w_code, K,
                        b_d.data_ptr() if b_d is not None else None, y_d.data_ptr(), N, M * N, batch, M, K, N, shift,
                        ROUNDING_CODE[tok], int(relu), DTYPE_CODE[out_dtype], stream())
    a4c.check(rc, 'a4c_dense_ta')
    return y_d.cpu().numpy()


def bmm16(a, b, *, shift, tok, trans_a=False, trans_b=False, out_dtype='int16'):
    L = a4c.load()
    batch = a.shape[0]
    M = a.shape[2] if trans_a else a.shape[1]
    K = a.shape[1] if trans_a else a.shape[2]
    N = b.shape[1] if trans_b else b.shape[2]
    wide = b.dtype == np.int16
    a_d, b_d = dev(np.ascontiguousarray(a.astype(np.int16))), dev(np.ascontiguousarray(b))
    c_d = torch.zeros((batch, M, N), dtype=TD[out_dtype], device='cuda')
    rc = L.a4c_bmm_i16(a_d.data_ptr(), a.shape[2], a.shape[1] * a.shape[2], b_d.data_ptr(), 2 if wide else 0, b.shape[2],
                       b.shape[1] * b.shape[2], c_d.data_ptr(), N, M * N, batch, M, K, N, int(trans_a), int(trans_b), shift,
                       ROUNDING_CODE[tok], DTYPE_CODE[out_dtype], stream())
    a4c.check(rc, 'a4c_bmm_i16')
    return c_d.cpu().numpy()


def dense_float(a, w_kn, bias, *, relu, fmt, simt=False):
    """Floating-point Dense through a4c_dense_f.  a [M, K] and w_kn [K, N] are float arrays; they are rounded to the
    storage type `fmt` ('bfloat16' / 'fp8_e4m3' / 'float32') first.  Returns (float32 result, stored a, stored w) so the
    caller can evaluate its reference on exactly what the kernel saw.  simt=True forces the tiled SIMT kernel."""
    from aie4ml_b200 import quant_utils as Q

    L = a4c.load()
    M, K = a.shape
    N = w_kn.shape[1]
    esz = {'bfloat16': 2, 'fp8_e4m3': 1, 'float32': 4}[fmt]
    code = {'bfloat16': 0, 'float32': 1, 'fp8_e4m3': 2}[fmt]
    pad = lambda n: (n * esz + 15) // 16 * 16 // esz
    a_bits, a_val = Q.to_storage_float(a, fmt)
    w_bits, w_val = Q.to_storage_float(np.ascontiguousarray(w_kn.T), fmt)
    lda, ldw, ldy = pad(K), pad(K), pad(N)
    a_buf = np.zeros((M, lda), dtype=a_bits.dtype); a_buf[:, :K] = a_bits
    w_buf = np.zeros((N, ldw), dtype=w_bits.dtype); w_buf[:, :K] = w_bits
    a_d, w_d = dev(a_buf), dev(w_buf)
    b_d = dev(bias.astype(np.float32)) if bias is not None else None
    y_d = torch.zeros((M, ldy), dtype={2: torch.int16, 1: torch.uint8, 4: torch.float32}[esz], device='cuda')
    L.a4c_set_option(a4c.OPT_FLOAT_DENSE_PATH, 1 if simt else 0)
    try:
        rc = L.a4c_dense_f(a_d.data_ptr(), code, lda, w_d.data_ptr(), ldw, b_d.data_ptr() if b_d is not None else None,
                           y_d.data_ptr(), ldy, M, K, N, int(relu), stream())
        a4c.check(rc, 'a4c_dense_f')
        a4c.device_status(stream())
    finally:
        L.a4c_set_option(a4c.OPT_FLOAT_DENSE_PATH, 0)
    y = y_d.cpu().numpy()
    assert (y[:, N:] == 0).all(), 'kernel wrote into the row padding'
    bits = y[:, :N]
    if fmt == 'bfloat16':
        bits = bits.view(np.uint16) if bits.dtype != np.uint16 else bits
    return Q.from_storage_float(np.ascontiguousarray(bits), fmt), a_val, w_val.T
