"""The oracle itself: hand-checkable rounding / saturation tables, the identities its integer
recipes must satisfy, float sanity bounds, and agreement between its NumPy and C editions."""

import numpy as np
import pytest

from oracle import c_api as C
from oracle import oracle

TOKENS = oracle.ROUNDING_TOKENS


def test_round_shift_hand_table():
    # value / 4 for v = -6..6: exact -1.5, -1.25, -1, -0.75, -0.5, -0.25, 0, 0.25, 0.5, 0.75, 1, 1.25, 1.5
    v = np.arange(-6, 7)
    want = {
        'floor':          [-2, -2, -1, -1, -1, -1, 0, 0, 0, 0, 1, 1, 1],
        'ceil':           [-1, -1, -1, 0, 0, 0, 0, 1, 1, 1, 1, 2, 2],
        'positive_inf':   [-1, -1, -1, -1, 0, 0, 0, 0, 1, 1, 1, 1, 2],
        'negative_inf':   [-2, -1, -1, -1, -1, 0, 0, 0, 0, 1, 1, 1, 1],
        'symmetric_inf':  [-2, -1, -1, -1, -1, 0, 0, 0, 1, 1, 1, 1, 2],
        'symmetric_zero': [-1, -1, -1, -1, 0, 0, 0, 0, 0, 1, 1, 1, 1],
        'conv_even':      [-2, -1, -1, -1, 0, 0, 0, 0, 0, 1, 1, 1, 2],
        'conv_odd':       [-1, -1, -1, -1, -1, 0, 0, 0, 1, 1, 1, 1, 1],
    }
    for tok in TOKENS:
        np.testing.assert_array_equal(oracle.round_shift(v, 2, tok), want[tok], err_msg=tok)


def test_round_shift_against_float_reference():
    rng = np.random.default_rng(0)
    v = rng.integers(-(1 << 30), 1 << 30, 4000)
    for shift in (1, 3, 7, 10, 20):
        x = v.astype(np.float64) / (1 << shift)
        np.testing.assert_array_equal(oracle.round_shift(v, shift, 'floor'), np.floor(x))
        np.testing.assert_array_equal(oracle.round_shift(v, shift, 'ceil'), np.ceil(x))
        np.testing.assert_array_equal(oracle.round_shift(v, shift, 'positive_inf'), np.floor(x + 0.5))
        np.testing.assert_array_equal(oracle.round_shift(v, shift, 'conv_even'), np.round(x))
        away = np.where(x >= 0, np.floor(x + 0.5), np.ceil(x - 0.5))
        np.testing.assert_array_equal(oracle.round_shift(v, shift, 'symmetric_inf'), away)
    np.testing.assert_array_equal(oracle.round_shift(v, 0, 'conv_even'), v)


def test_srs_saturates_every_dtype():
    v = np.array([-70000, -32769, -32768, -129, -128, -1, 0, 127, 128, 255, 256, 32767, 32768, 70000])
    np.testing.assert_array_equal(oracle.srs(v, 0, 'floor', 'int8'), np.clip(v, -128, 127))
    np.testing.assert_array_equal(oracle.srs(v, 0, 'floor', 'uint8'), np.clip(v, 0, 255))
    np.testing.assert_array_equal(oracle.srs(v, 0, 'floor', 'int16'), np.clip(v, -32768, 32767))


def test_dense_relu_after_saturation_and_bias():
    a = np.array([[127, 127], [-128, -128], [1, -1]], dtype=np.int8)
    w = np.array([[127, -128], [127, -128]], dtype=np.int8)
    bias = np.array([5, -5], dtype=np.int32)
    y = oracle.dense(a, w, bias, shift=4, tok='positive_inf', relu=False)
    acc = a.astype(np.int64) @ w.astype(np.int64) + bias
    np.testing.assert_array_equal(y, np.clip(np.floor(acc / 16 + 0.5), -128, 127))
    yr = oracle.dense(a, w, bias, shift=4, tok='positive_inf', relu=True)
    np.testing.assert_array_equal(yr, np.maximum(y, 0))


def test_dense_within_one_lsb_of_float_evaluation():
    # mirrors the reference's own check (scripts/check_onnx_bit_exact.py:37-46,170-179): requantised
    # float evaluation vs integer kernel, at most 1 LSB apart
    rng = np.random.default_rng(1)
    a = rng.integers(-128, 128, (64, 96)).astype(np.int8)
    w = rng.integers(-127, 128, (96, 48)).astype(np.int8)
    bias = rng.integers(-4096, 4096, 48).astype(np.int32)
    y = oracle.dense(a, w, bias, shift=9, tok='conv_even', relu=False)
    f = (a.astype(np.float64) @ w.astype(np.float64) + bias) / 512.0
    assert np.abs(y - np.clip(np.rint(f), -128, 127)).max() <= 1


def test_matmul_transposes():
    rng = np.random.default_rng(2)
    a = rng.integers(-128, 128, (3, 8, 16)).astype(np.int8)
    b = rng.integers(-128, 128, (3, 16, 12)).astype(np.int8)
    ref = oracle.matmul(a, b, shift=5, tok='floor')
    np.testing.assert_array_equal(oracle.matmul(np.swapaxes(a, 1, 2).copy(), b, shift=5, tok='floor', transpose_a=True), ref)
    np.testing.assert_array_equal(oracle.matmul(a, np.swapaxes(b, 1, 2).copy(), shift=5, tok='floor', transpose_b=True), ref)
    u = rng.integers(0, 256, (3, 8, 16)).astype(np.uint8)
    np.testing.assert_array_equal(oracle.matmul(u, b, shift=8, tok='positive_inf'),
                                  np.clip(np.floor(np.matmul(u.astype(np.int64), b.astype(np.int64)) / 256 + 0.5), -128, 127))


def test_exp_score_tracks_real_exponential():
    d = np.arange(256)
    for kq in (1, 23, 46, 128):
        e = oracle.exp_score16(d, kq)
        real = 16384.0 * np.exp2(-(d * kq) / 256.0)
        assert e[0] == 16384
        assert np.all(np.diff(e) <= 0)
        assert np.abs(e - real).max() <= 16384 * 0.004 + 1


def test_softmax_reciprocal_identity_and_range():
    rng = np.random.default_rng(3)
    x = np.clip(np.rint(rng.normal(0, 32, (64, 1024))), -128, 127).astype(np.int8)
    for out_dtype in ('uint8', 'int16'):
        out = oracle.softmax_exp(x, exp_kq=23, out_dtype=out_dtype)
        assert out.dtype == np.dtype(out_dtype)
        assert out.min() >= 0
        m = x.astype(np.int64).max(axis=1, keepdims=True)
        e = oracle.exp_score16(m - x, 23)
        s = e.sum(axis=1)
        numer = oracle.softmax_numer(out_dtype, 15)
        q = numer // s
        assert np.all(q * s <= numer) and np.all((q + 1) * s > numer)
    h = oracle.softmax_hccs(x, B=31, S=1, Dmax=30)
    assert h.max() <= 255 and h.min() >= 0
    # rows sum to about 255 (floor losses only)
    assert np.all(h.astype(np.int64).sum(axis=1) <= 255 * 1.01) and np.all(h.astype(np.int64).sum(axis=1) >= 255 - 1024)


def test_softmax_exp_close_to_float_softmax():
    rng = np.random.default_rng(4)
    x = np.clip(np.rint(rng.normal(0, 24, (32, 128))), -128, 127).astype(np.int8)
    frac = 4
    out = oracle.softmax_exp(x, exp_kq=oracle.exp_kq(frac)).astype(np.float64) / 256.0
    xf = x.astype(np.float64) / (1 << frac)
    p = np.exp(xf - xf.max(axis=1, keepdims=True))
    p /= p.sum(axis=1, keepdims=True)
    assert np.abs(out - p).max() <= 3.0 / 256.0


def test_softmax_clb_matches_definition():
    x = np.arange(-64, 64, dtype=np.int8)[None, :].repeat(4, axis=0)
    got = oracle.softmax_hccs(x, B=200, S=3, Dmax=66, inv_shift=14, use_clb=True)
    d = np.minimum(63 - x.astype(np.int64), 66)
    score = 200 - 3 * d
    k = int(np.floor(np.log2(score[0].sum())))
    inv = 255 << (14 - k)
    np.testing.assert_array_equal(got, np.clip((score * inv) >> 14, 0, 255))


def test_layer_norm_close_to_float_and_inv_std_definition():
    rng = np.random.default_rng(5)
    x = np.clip(np.rint(rng.normal(3, 30, (48, 256))), -128, 127).astype(np.int8)
    gamma = rng.integers(-256, 257, 256)
    beta = rng.integers(-256, 257, 256)
    out_shift = 4
    y = oracle.layer_norm(x, gamma, beta, eps_q0=1, out_shift=out_shift, tok='conv_even').astype(np.float64) / (1 << out_shift)
    xf = x.astype(np.float64)
    norm = (xf - xf.mean(axis=1, keepdims=True)) / np.sqrt(xf.var(axis=1, keepdims=True) + 1.0)
    ref = norm * (gamma / 128.0) + beta / 32768.0
    assert np.abs(y - np.clip(ref, -8, 127 / 16)).max() <= 3.0 / 16.0
    # reciprocal std: exact powers of four hit exact Q15 values; var = 1 clamps to 32767
    np.testing.assert_array_equal(oracle.inv_std_q15(np.array([1, 4, 16, 64, 16384]), 'floor'),
                                  [32767, 16384, 8192, 4096, 256])
    v = np.arange(1, 16386)
    q = oracle.inv_std_q15(v, 'conv_even')
    assert np.all(np.diff(q) <= 0)
    assert np.abs(q - np.minimum(32768.0 / np.sqrt(v), 32767)).max() <= 0.51


def test_layer_norm_fscale_saturates():
    # var small and |gamma| large: inv_std * gamma >> 7 exceeds int16 and must clamp (layer_norm.cpp:108-109)
    x = np.zeros((1, 32), dtype=np.int8)
    x[0, 0] = 1
    gamma = np.full(32, 32767)
    beta = np.zeros(32)
    y = oracle.layer_norm(x, gamma, beta, eps_q0=1, out_shift=0, tok='floor')
    assert y[0, 0] == np.clip((1 * 32767) >> 15, -128, 127)


@pytest.mark.parametrize('tok', TOKENS)
def test_c_edition_matches_numpy_dense_and_add(oracle_c, tok):
    rng = np.random.default_rng(6)
    a = rng.integers(-128, 128, (37, 50)).astype(np.int8)
    w = rng.integers(-128, 128, (50, 21)).astype(np.int8)
    bias = rng.integers(-(1 << 16), 1 << 16, 21).astype(np.int32)
    for shift, relu, od in ((0, False, 'int16'), (7, True, 'int8'), (10, False, 'uint8'), (3, False, 'int8')):
        np.testing.assert_array_equal(C.dense(oracle_c, a, w, bias, shift=shift, tok=tok, relu=relu, out_dtype=od),
                                      oracle.dense(a, w, bias, shift=shift, tok=tok, relu=relu, out_dtype=od))
    u = rng.integers(0, 256, (37, 50)).astype(np.uint8)
    np.testing.assert_array_equal(C.dense(oracle_c, u, w, None, shift=8, tok=tok, relu=False),
                                  oracle.dense(u, w, None, shift=8, tok=tok, relu=False))
    for dt, lo, hi in (('int8', -128, 128), ('uint8', 0, 256), ('int16', -32768, 32768)):
        p = rng.integers(lo, hi, (9, 64)).astype(C.NP[dt])
        q = rng.integers(lo, hi, (9, 64)).astype(C.NP[dt])
        for shift in (0, 1):
            np.testing.assert_array_equal(C.add(oracle_c, p, q, shift=shift, tok=tok, dtype=dt),
                                          oracle.add(p, q, shift=shift, tok=tok, out_dtype=dt))


def test_c_edition_matches_numpy_bmm(oracle_c):
    rng = np.random.default_rng(7)
    a = rng.integers(-128, 128, (5, 12, 20)).astype(np.int8)
    b = rng.integers(-128, 128, (5, 20, 9)).astype(np.int8)
    np.testing.assert_array_equal(C.bmm(oracle_c, a, b, shift=6, tok='conv_even'), oracle.matmul(a, b, shift=6, tok='conv_even'))
    bt = np.swapaxes(b, 1, 2).copy()
    np.testing.assert_array_equal(C.bmm(oracle_c, a, bt, shift=6, tok='floor', trans_b=True),
                                  oracle.matmul(a, bt, shift=6, tok='floor', transpose_b=True))
    at = np.swapaxes(a, 1, 2).copy()
    np.testing.assert_array_equal(C.bmm(oracle_c, at, b, shift=2, tok='ceil', trans_a=True, out_dtype='int16'),
                                  oracle.matmul(at, b, shift=2, tok='ceil', transpose_a=True, out_dtype='int16'))


@pytest.mark.parametrize('tok', ['floor', 'positive_inf', 'conv_even', 'symmetric_inf'])
def test_c_edition_matches_numpy_rowops(oracle_c, tok):
    rng = np.random.default_rng(8)
    x = np.clip(np.rint(rng.normal(0, 32, (33, 256))), -128, 127).astype(np.int8)
    x[0] = 5          # zero variance
    x[1, :] = -128    # extreme mean
    x[2, ::2], x[2, 1::2] = 127, -128
    gamma = rng.integers(-32768, 32768, 256)
    beta = rng.integers(-32768, 32768, 256)
    for out_shift in (0, 4, 15):
        np.testing.assert_array_equal(C.layer_norm(oracle_c, x, gamma, beta, eps_q0=1, out_shift=out_shift, tok=tok),
                                      oracle.layer_norm(x, gamma, beta, eps_q0=1, out_shift=out_shift, tok=tok))
    for od in ('uint8', 'int16'):
        np.testing.assert_array_equal(C.softmax(oracle_c, x, mode='exp', exp_kq=23, out_dtype=od),
                                      oracle.softmax_exp(x, exp_kq=23, out_dtype=od))
        np.testing.assert_array_equal(C.softmax(oracle_c, x, mode='hccs', B=120, S=2, Dmax=59, out_dtype=od),
                                      oracle.softmax_hccs(x, B=120, S=2, Dmax=59, out_dtype=od))
    np.testing.assert_array_equal(C.softmax(oracle_c, x, mode='hccs', B=120, S=2, Dmax=59, inv_shift=14, use_clb=True),
                                  oracle.softmax_hccs(x, B=120, S=2, Dmax=59, inv_shift=14, use_clb=True))


@pytest.mark.parametrize('build', ['portable', 'native'])
def test_c_edition_blocked_products_wrap_like_the_numpy_oracle(oracle_c, oracle_c_native, build):
    """The blocked matrix products of the C edition (portable int16 dot products; AVX-512 VNNI with the +128 offset and
    column-sum correction when the host CPU has it) against the NumPy oracle: ragged shapes around the block sizes,
    unsigned A, full-range biases that make the 32-bit accumulator wrap, strided and transposed MatMul operands."""
    lib = oracle_c if build == 'portable' else oracle_c_native
    rng = np.random.default_rng(60)
    for M, K, N in ((1, 1, 1), (7, 5, 3), (49, 130, 65), (97, 1031, 129), (6, 4100, 64)):
        for unsigned in (False, True):
            a = rng.integers(0 if unsigned else -128, 256 if unsigned else 128, (M, K)).astype(np.uint8 if unsigned else np.int8)
            w = rng.integers(-128, 128, (K, N)).astype(np.int8)
            bias = rng.integers(-(1 << 31), 1 << 31, N).astype(np.int32)
            for tok, shift, od in (('positive_inf', 10, 'int8'), ('conv_even', 3, 'int16'), ('floor', 0, 'uint8')):
                np.testing.assert_array_equal(C.dense(lib, a, w, bias, shift=shift, tok=tok, relu=True, out_dtype=od),
                                              oracle.dense(a, w, bias, shift=shift, tok=tok, relu=True, out_dtype=od))
    # extreme operands: every product at its largest magnitude
    a = np.full((3, 8192), -128, dtype=np.int8)
    w = np.full((8192, 5), -128, dtype=np.int8)
    np.testing.assert_array_equal(C.dense(lib, a, w, None, shift=20, tok='floor', relu=False, out_dtype='int16'),
                                  oracle.dense(a, w, None, shift=20, tok='floor', relu=False, out_dtype='int16'))
    q = rng.integers(-128, 128, (4, 128, 64)).astype(np.int8)
    k = rng.integers(-128, 128, (4, 128, 64)).astype(np.int8)
    p_u8 = rng.integers(0, 256, (4, 128, 128)).astype(np.uint8)
    np.testing.assert_array_equal(C.bmm(lib, q, k, shift=9, tok='positive_inf', trans_b=True),
                                  oracle.matmul(q, k, shift=9, tok='positive_inf', transpose_b=True))
    np.testing.assert_array_equal(C.bmm(lib, p_u8, k, shift=8, tok='conv_even', out_dtype='int16'),
                                  oracle.matmul(p_u8, k, shift=8, tok='conv_even', out_dtype='int16'))
    qt = np.ascontiguousarray(q.transpose(0, 2, 1))
    np.testing.assert_array_equal(C.bmm(lib, qt, k, shift=9, tok='symmetric_inf', trans_a=True, trans_b=True),
                                  oracle.matmul(qt, k, shift=9, tok='symmetric_inf', transpose_a=True, transpose_b=True))


# ---- float cross-checks: dequantised oracle output against a float64 evaluation of the same layer ------------------
# (what the reference's own checker does with ONNX Runtime, scripts/check_onnx_bit_exact.py:37-46,170-179)

@pytest.mark.parametrize('seed', [0, 1, 2])
def test_matmul_and_add_within_one_lsb_of_float_evaluation(seed):
    rng = np.random.default_rng(100 + seed)
    for (bsz, m, k, n), shift in (((3, 16, 64, 24), 9), ((2, 128, 64, 128), 9), ((1, 33, 130, 7), 6)):
        a = rng.integers(-128, 128, (bsz, m, k)).astype(np.int8)
        b = rng.integers(-128, 128, (bsz, k, n)).astype(np.int8)
        f = np.matmul(a.astype(np.float64), b.astype(np.float64)) / float(1 << shift)
        # an int32 sum of int8 products is exact in float64, so rint of it IS convergent rounding: 0 LSB there,
        # at most 1 LSB for the other nearest modes (they differ from it on exact ties only) and for floor / ceil
        np.testing.assert_array_equal(oracle.matmul(a, b, shift=shift, tok='conv_even'), np.clip(np.rint(f), -128, 127))
        for tok in ('positive_inf', 'symmetric_inf', 'symmetric_zero', 'floor', 'ceil'):
            assert np.abs(oracle.matmul(a, b, shift=shift, tok=tok) - np.clip(np.rint(f), -128, 127)).max() <= 1, tok
        bt = np.ascontiguousarray(np.swapaxes(b, 1, 2))
        np.testing.assert_array_equal(oracle.matmul(a, bt, shift=shift, tok='conv_even', transpose_b=True),
                                      np.clip(np.rint(f), -128, 127))
        p = rng.integers(0, 256, (bsz, m, k)).astype(np.uint8)     # probabilities times values: unsigned left operand
        fp = np.matmul(p.astype(np.float64), b.astype(np.float64)) / 256.0
        np.testing.assert_array_equal(oracle.matmul(p, b, shift=8, tok='conv_even'), np.clip(np.rint(fp), -128, 127))
    for dt, lo, hi in (('int8', -128, 127), ('uint8', 0, 255), ('int16', -32768, 32767)):
        x = rng.integers(lo, hi + 1, (40, 96)).astype(C.NP[dt])
        y = rng.integers(lo, hi + 1, (40, 96)).astype(x.dtype)
        # same type on both sides and on the result: shift 0, the float sum clipped to the type IS the result (0 LSB)
        np.testing.assert_array_equal(oracle.add(x, y, shift=0, tok='conv_even', out_dtype=dt),
                                      np.clip(x.astype(np.float64) + y.astype(np.float64), lo, hi))
        for tok in ('conv_even', 'positive_inf', 'floor'):
            f = (x.astype(np.float64) + y.astype(np.float64)) / 2.0
            assert np.abs(oracle.add(x, y, shift=1, tok=tok, out_dtype=dt) - np.clip(np.rint(f), lo, hi)).max() <= 1


@pytest.mark.parametrize('cols,bound', [(32, 1.5), (128, 1.5), (256, 1.5), (1024, 2.25)])
def test_softmax_exp_lsb_bound_against_float_softmax_over_widths_and_seeds(cols, bound):
    """Against a float softmax at the temperature the integer kernel actually uses (2^(-d * EXP_KQ / 256): EXP_KQ is
    a rounded contract parameter, its rounding is not the kernel's error), in uint8 output steps.  Measured worst
    cases over these inputs: 1.36 / 1.35 / 1.38 / 2.06 steps at 32 / 128 / 256 / 1024 columns."""
    worst = 0.0
    for seed in range(8):
        for sigma, frac in ((24, 4), (32, 4), (16, 3), (40, 5), (32, 2)):
            rng = np.random.default_rng(seed)
            x = np.clip(np.rint(rng.normal(0, sigma, (64, cols))), -128, 127).astype(np.int8)
            kq = oracle.exp_kq(frac)
            out = oracle.softmax_exp(x, exp_kq=kq).astype(np.float64)
            d = x.astype(np.int64).max(axis=1, keepdims=True) - x
            p = np.exp2(-d * kq / 256.0)
            p /= p.sum(axis=1, keepdims=True)
            worst = max(worst, float(np.abs(out - 255.0 * p).max()))
    assert worst <= bound, worst


@pytest.mark.parametrize('cols,params', [(32, (1000, 10, 90)), (128, (200, 3, 66)), (1024, (31, 1, 30))])
def test_softmax_hccs_lsb_bound_against_its_real_valued_definition(cols, params):
    """The surrogate normalised in real arithmetic, score / sum(score) * 255: the integer kernel loses at most the
    two floors (reciprocal, product): 1.03 uint8 steps measured, bound 1.25."""
    B, S, Dmax = params
    for seed in range(6):
        rng = np.random.default_rng(seed)
        x = np.clip(np.rint(rng.normal(0, 32, (64, cols))), -128, 127).astype(np.int8)
        out = oracle.softmax_hccs(x, B=B, S=S, Dmax=Dmax).astype(np.float64)
        d = np.minimum(x.astype(np.int64).max(axis=1, keepdims=True) - x, Dmax)
        score = (B - S * d).astype(np.float64)
        assert np.abs(out - 255.0 * score / score.sum(axis=1, keepdims=True)).max() <= 1.25


@pytest.mark.parametrize('cols', [64, 256, 1024])
@pytest.mark.parametrize('tok,bound', [('conv_even', 1.9), ('positive_inf', 1.9), ('floor', 2.4)])
def test_layer_norm_lsb_bound_against_float_layer_norm_over_widths_and_seeds(cols, tok, bound):
    """int8 output steps against float64 LayerNorm with the same gamma (Q7), beta (Q15) and epsilon.  Measured worst
    cases: 1.66 steps with the nearest modes, 2.15 with floor (Q15 reciprocal std, Q7 scale and the mean's rounding
    each contribute a fraction of a step)."""
    worst = 0.0
    for seed in range(6):
        rng = np.random.default_rng(seed)
        x = np.clip(np.rint(rng.normal(3, 30, (64, cols))), -128, 127).astype(np.int8)
        gamma, beta = rng.integers(-256, 257, cols), rng.integers(-256, 257, cols)
        for out_shift in (4, 5):
            y = oracle.layer_norm(x, gamma, beta, eps_q0=1, out_shift=out_shift, tok=tok).astype(np.float64)
            xf = x.astype(np.float64)
            norm = (xf - xf.mean(axis=1, keepdims=True)) / np.sqrt(xf.var(axis=1, keepdims=True) + 1.0)
            ref = (norm * (gamma / 128.0) + beta / 32768.0) * (1 << out_shift)
            worst = max(worst, float(np.abs(y - np.clip(ref, -128, 127)).max()))
    assert worst <= bound, worst
