"""ctypes binding of the C edition of the oracle (test infrastructure: tests, the benchmark's checker and CPU arm)."""

import ctypes
from ctypes import c_int, c_int64, c_void_p

import numpy as np

ROUND = {'floor': 0, 'ceil': 1, 'positive_inf': 2, 'negative_inf': 3, 'symmetric_inf': 4, 'symmetric_zero': 5,
         'conv_even': 6, 'conv_odd': 7}
DT = {'int8': 0, 'uint8': 1, 'int16': 2}
NP = {'int8': np.int8, 'uint8': np.uint8, 'int16': np.int16}


def _p(a):
    return c_void_p(a.ctypes.data) if a is not None else None


def dense(lib, a, w_kn, bias, *, shift, tok, relu, out_dtype='int8'):
    a = np.ascontiguousarray(a)
    w = np.ascontiguousarray(w_kn.astype(np.int8))
    b = None if bias is None else np.ascontiguousarray(bias.astype(np.int32))
    M, K = a.shape
    N = w.shape[1]
    y = np.zeros((M, N), dtype=NP[out_dtype])
    rc = lib.orc_dense_i8(_p(a), c_int64(K), _p(w), _p(b), _p(y), c_int64(N), c_int64(M), c_int(K), c_int(N), c_int(shift),
                          c_int(ROUND[tok]), c_int(int(relu)), c_int(DT[out_dtype]), c_int(int(a.dtype == np.uint8)))
    assert rc == 0
    return y


def bmm(lib, a, b, *, shift, tok, trans_a=False, trans_b=False, out_dtype='int8'):
    a = np.ascontiguousarray(a)
    b = np.ascontiguousarray(b.astype(np.int8))
    batch = a.shape[0]
    M = a.shape[2] if trans_a else a.shape[1]
    K = a.shape[1] if trans_a else a.shape[2]
    N = b.shape[1] if trans_b else b.shape[2]
    c = np.zeros((batch, M, N), dtype=NP[out_dtype])
    rc = lib.orc_bmm_i8(_p(a), c_int64(a.shape[2]), c_int64(a.shape[1] * a.shape[2]), _p(b), c_int64(b.shape[2]),
                        c_int64(b.shape[1] * b.shape[2]), _p(c), c_int64(N), c_int64(M * N), c_int64(batch), c_int(M),
                        c_int(K), c_int(N), c_int(int(trans_a)), c_int(int(trans_b)), c_int(shift), c_int(ROUND[tok]),
                        c_int(DT[out_dtype]), c_int(int(a.dtype == np.uint8)))
    assert rc == 0
    return c


def add(lib, a, b, *, shift, tok, dtype):
    a = np.ascontiguousarray(a)
    b = np.ascontiguousarray(b)
    out = np.zeros_like(a)
    rows, cols = a.shape
    rc = lib.orc_add_sat(_p(a), c_int64(cols), _p(b), c_int64(cols), _p(out), c_int64(cols), c_int64(rows), c_int64(cols),
                         c_int(shift), c_int(ROUND[tok]), c_int(DT[dtype]))
    assert rc == 0
    return out


def layer_norm(lib, x, gamma, beta, *, eps_q0, out_shift, tok):
    x = np.ascontiguousarray(x.astype(np.int8))
    g = np.ascontiguousarray(gamma.astype(np.int16))
    b = np.ascontiguousarray(beta.astype(np.int16))
    out = np.zeros_like(x)
    rows, cols = x.shape
    rc = lib.orc_layernorm_i8(_p(x), c_int64(cols), _p(g), _p(b), _p(out), c_int64(cols), c_int64(rows), c_int(cols),
                              c_int(eps_q0), c_int(out_shift), c_int(ROUND[tok]))
    assert rc == 0
    return out


def softmax(lib, x, *, mode, B=0, S=0, Dmax=0, inv_shift=15, use_clb=False, exp_kq=0, out_dtype='uint8'):
    x = np.ascontiguousarray(x.astype(np.int8))
    rows, cols = x.shape
    out = np.zeros((rows, cols), dtype=NP[out_dtype])
    rc = lib.orc_softmax_i8(_p(x), c_int64(cols), _p(out), c_int64(cols), c_int64(rows), c_int(cols),
                            c_int(0 if mode == 'hccs' else 1), c_int(B), c_int(S), c_int(Dmax), c_int(inv_shift),
                            c_int(int(use_clb)), c_int(exp_kq), c_int(DT[out_dtype]))
    assert rc == 0
    return out
