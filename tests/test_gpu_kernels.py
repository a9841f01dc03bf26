"""Kernel-level parity: every C-ABI entry point against the CPU oracle, bit-exact, on seeded inputs."""

import numpy as np
import pytest

from oracle import oracle

pytestmark = pytest.mark.gpu

TOKENS = oracle.ROUNDING_TOKENS
SIMT, TC, TC2 = 1, 2, 3


def _rand_dense(seed, M, K, N, unsigned=False, big_bias=True):
    rng = np.random.default_rng(seed)
    a = rng.integers(0, 256, (M, K)).astype(np.uint8) if unsigned else rng.integers(-128, 128, (M, K)).astype(np.int8)
    w = rng.integers(-128, 128, (K, N)).astype(np.int8)
    bias = rng.integers(-(1 << 16), 1 << 16, N).astype(np.int32) if big_bias else None
    return a, w, bias


@pytest.mark.parametrize('shape', [(1, 16, 5), (7, 16, 64), (33, 50, 21), (64, 64, 32), (130, 100, 10), (257, 33, 65)])
@pytest.mark.parametrize('tok', ['positive_inf', 'conv_even'])
def test_dense_simt_odd_shapes(shape, tok):
    import gpu_util as G

    M, K, N = shape
    a, w, bias = _rand_dense(hash(shape) % 1000, M, K, N)
    for shift, relu in ((7, True), (0, False), (10, False)):
        got = G.dense(a, w, bias, shift=shift, tok=tok, relu=relu, algo=SIMT)
        np.testing.assert_array_equal(got, oracle.dense(a, w, bias, shift=shift, tok=tok, relu=relu))


@pytest.mark.parametrize('tok', TOKENS)
def test_dense_simt_every_rounding_mode_and_dtype(tok):
    import gpu_util as G

    a, w, bias = _rand_dense(11, 96, 72, 48)
    for shift, od in ((1, 'int16'), (9, 'int8'), (9, 'uint8'), (31, 'int8')):
        got = G.dense(a, w, bias, shift=shift, tok=tok, relu=False, out_dtype=od, algo=SIMT)
        np.testing.assert_array_equal(got, oracle.dense(a, w, bias, shift=shift, tok=tok, relu=False, out_dtype=od))
    u, w2, _ = _rand_dense(12, 40, 64, 32, unsigned=True)
    np.testing.assert_array_equal(G.dense(u, w2, None, shift=8, tok=tok, relu=False, algo=SIMT),
                                  oracle.dense(u, w2, None, shift=8, tok=tok, relu=False))


@pytest.mark.parametrize('shape', [(128, 128, 256), (128, 256, 16), (100, 16, 48), (300, 1024, 272), (1000, 200, 512),
                                   (4096, 512, 1024), (129, 4096, 256)])
@pytest.mark.parametrize('algo', [TC, TC2])
def test_dense_tcgen05_shapes(shape, algo):
    import gpu_util as G

    M, K, N = shape
    a, w, bias = _rand_dense(sum(shape), M, K, N)
    got = G.dense(a, w, bias, shift=10, tok='positive_inf', relu=True, algo=algo)
    np.testing.assert_array_equal(got, oracle.dense(a, w, bias, shift=10, tok='positive_inf', relu=True))


@pytest.mark.parametrize('shape', [(300, 1024, 10), (1000, 64, 5), (260, 128, 200), (129, 48, 270)])
def test_dense_tcgen05_output_widths_that_are_not_multiples_of_16(shape):
    """Classifier heads (N = 10, 5) and ragged widths: absent weight rows read as zero, stored columns are clipped,
    bytes between N and the row pitch stay untouched."""
    import gpu_util as G

    M, K, N = shape
    a, w, bias = _rand_dense(sum(shape), M, K, N)
    for relu, od in ((True, 'int8'), (False, 'uint8')):
        got = G.dense(a, w, bias, shift=9, tok='positive_inf', relu=relu, out_dtype=od, algo=TC)
        np.testing.assert_array_equal(got, oracle.dense(a, w, bias, shift=9, tok='positive_inf', relu=relu, out_dtype=od))
    got = G.dense(a, w, None, shift=6, tok='conv_even', relu=False, algo=TC)
    np.testing.assert_array_equal(got, oracle.dense(a, w, None, shift=6, tok='conv_even', relu=False))


@pytest.mark.parametrize('shape', [(76000, 256, 256), (19100, 128, 1024), (25300, 384, 700), (77000, 512, 40),
                                   (76100, 256, 768), (30001, 200, 384), (40000, 512, 128), (33000, 512, 640)])
@pytest.mark.parametrize('resident', [2, 1, 0])
def test_dense_tcgen05_small_k_with_and_without_a_resident_weight_tile(shape, resident):
    """Shapes large enough for the resident-W tile order (one weight tile per CTA kept in shared memory, A streamed
    through a deeper ring): one, three and four column tiles, ragged last row tile, a narrow classifier head.  Mode 2
    (the default) sends widths that are multiples of 128 to the short-reduction kernel (twelve epilogue warps on half
    tiles): one to four column tiles there, widths whose last column tile is a single half (128, 384, 640), a K tail
    shorter than a stage, K = 512 (four ring slots)."""
    import gpu_util as G
    from aie4ml_b200 import lib as a4c

    L = a4c.load()
    assert L.a4c_set_option(a4c.OPT_DENSE_RESIDENT_W, resident) == 0
    try:
        M, K, N = shape
        a, w, bias = _rand_dense(sum(shape), M, K, N)
        got = G.dense(a, w, bias, shift=9, tok='positive_inf', relu=True, algo=TC)
        np.testing.assert_array_equal(got, oracle.dense(a, w, bias, shift=9, tok='positive_inf', relu=True))
        got = G.dense(a, w, None, shift=8, tok='conv_even', relu=False, algo=TC)
        np.testing.assert_array_equal(got, oracle.dense(a, w, None, shift=8, tok='conv_even', relu=False))
        u = np.random.default_rng(5).integers(0, 256, (M, K)).astype(np.uint8)
        got = G.dense(u, w, bias, shift=10, tok='symmetric_inf', relu=False, out_dtype='uint8', algo=TC)
        np.testing.assert_array_equal(got, oracle.dense(u, w, bias, shift=10, tok='symmetric_inf', relu=False, out_dtype='uint8'))
    finally:
        assert L.a4c_set_option(a4c.OPT_DENSE_RESIDENT_W, 2) == 0


@pytest.mark.parametrize('tok', TOKENS)
@pytest.mark.parametrize('algo', [TC, TC2])
def test_dense_tcgen05_every_rounding_mode(tok, algo):
    import gpu_util as G

    a, w, bias = _rand_dense(21, 384, 384, 320)
    for shift, relu, od in ((9, False, 'int8'), (3, True, 'int8'), (12, False, 'uint8'), (0, False, 'int8')):
        got = G.dense(a, w, bias, shift=shift, tok=tok, relu=relu, out_dtype=od, algo=algo)
        np.testing.assert_array_equal(got, oracle.dense(a, w, bias, shift=shift, tok=tok, relu=relu, out_dtype=od))


@pytest.mark.parametrize('algo', [TC, TC2])
def test_dense_tcgen05_extreme_bias_wraps_like_the_accumulator(algo):
    """Biases across the whole int32 range: acc + bias wraps at 32 bits before the rounding shift,
    on either side of the shift at which the kernel changes its rounding sequence, for both
    signed and unsigned outputs, with and without ReLU."""
    import gpu_util as G

    rng = np.random.default_rng(77)
    a, w, _ = _rand_dense(78, 260, 192, 272)
    bias = rng.integers(-2 ** 31, 2 ** 31, size=272, dtype=np.int64).astype(np.int32)
    bias[:8] = [2 ** 31 - 1, -2 ** 31, 2 ** 31 - 2 ** 20, -2 ** 31 + 2 ** 20, 0, 1, -1, 2 ** 30]
    for shift in (1, 2, 21, 22, 23, 24, 31):
        for relu, od in ((False, 'int8'), (True, 'int8'), (False, 'uint8')):
            got = G.dense(a, w, bias, shift=shift, tok='positive_inf', relu=relu, out_dtype=od, algo=algo)
            np.testing.assert_array_equal(
                got, oracle.dense(a, w, bias, shift=shift, tok='positive_inf', relu=relu, out_dtype=od))


def test_dense_tcgen05_wide_output_streams_the_bias_per_tile():
    """N above the resident-bias limit: the kernel stages one bias slice per tile instead."""
    import gpu_util as G

    a, w, bias = _rand_dense(79, 300, 64, 2304)
    got = G.dense(a, w, bias, shift=7, tok='positive_inf', relu=True, algo=TC)
    np.testing.assert_array_equal(got, oracle.dense(a, w, bias, shift=7, tok='positive_inf', relu=True))


@pytest.mark.parametrize('TC', [TC, TC2])
def test_dense_tcgen05_unsigned_lhs_no_bias_and_many_tiles(TC):
    import gpu_util as G

    u, w, _ = _rand_dense(31, 640, 256, 768, unsigned=True)
    np.testing.assert_array_equal(G.dense(u, w, None, shift=11, tok='conv_even', relu=False, algo=TC),
                                  oracle.dense(u, w, None, shift=11, tok='conv_even', relu=False))
    # more tiles than SMs: the persistent loop and both accumulator stages get reused
    a, w, bias = _rand_dense(32, 128 * 40, 128, 1024)
    np.testing.assert_array_equal(G.dense(a, w, bias, shift=8, tok='floor', relu=True, algo=TC),
                                  oracle.dense(a, w, bias, shift=8, tok='floor', relu=True))


def test_dense_auto_picks_a_working_kernel_and_rejects_bad_arguments():
    import gpu_util as G
    from aie4ml_b200 import lib as a4c

    a, w, bias = _rand_dense(41, 256, 256, 256)
    np.testing.assert_array_equal(G.dense(a, w, bias, shift=10, tok='positive_inf', relu=True, algo=0),
                                  oracle.dense(a, w, bias, shift=10, tok='positive_inf', relu=True))
    a2, w2, b2 = _rand_dense(42, 9, 8, 5)  # K = 8: the tensor-core path cannot take it, auto must still work
    np.testing.assert_array_equal(G.dense(a2, w2, b2, shift=7, tok='positive_inf', relu=False, algo=0),
                                  oracle.dense(a2, w2, b2, shift=7, tok='positive_inf', relu=False))
    with pytest.raises(a4c.A4cError):
        G.dense(a2, w2, b2, shift=7, tok='positive_inf', relu=False, algo=TC)
    a3, w3, b3 = _rand_dense(43, 300, 64, 40)
    with pytest.raises(a4c.A4cError):   # the CTA-pair kernel stores whole 16-byte pieces: N must be a multiple of 16
        G.dense(a3, w3, b3, shift=7, tok='positive_inf', relu=False, algo=TC2)
    with pytest.raises(a4c.A4cError):
        G.dense(a, w, bias, shift=40, tok='positive_inf', relu=False)


@pytest.fixture(params=['auto', 'dp4a'])
def bmm_path(request):
    from aie4ml_b200 import lib as a4c

    L = a4c.load()
    assert L.a4c_set_option(a4c.OPT_BMM_PATH, 0 if request.param == 'auto' else 1) == 0
    yield request.param
    assert L.a4c_set_option(a4c.OPT_BMM_PATH, 0) == 0


def test_bmm_attention_shapes(bmm_path):
    import gpu_util as G

    rng = np.random.default_rng(51)
    q = rng.integers(-128, 128, (6, 128, 64)).astype(np.int8)
    k = rng.integers(-128, 128, (6, 128, 64)).astype(np.int8)
    v = rng.integers(-128, 128, (6, 128, 64)).astype(np.int8)
    p = rng.integers(0, 256, (6, 128, 128)).astype(np.uint8)
    np.testing.assert_array_equal(G.bmm(q, k, shift=9, tok='positive_inf', trans_b=True),
                                  oracle.matmul(q, k, shift=9, tok='positive_inf', transpose_b=True))
    np.testing.assert_array_equal(G.bmm(p, v, shift=8, tok='conv_even'), oracle.matmul(p, v, shift=8, tok='conv_even'))
    for tok in TOKENS:
        np.testing.assert_array_equal(G.bmm(q, k, shift=9, tok=tok, trans_b=True),
                                      oracle.matmul(q, k, shift=9, tok=tok, transpose_b=True), err_msg=tok)
    # ragged: M and K not multiples of the tile, several N tiles, more batches than SMs
    a2 = rng.integers(-128, 128, (200, 72, 80)).astype(np.int8)
    b2 = rng.integers(-128, 128, (200, 80, 144)).astype(np.int8)
    np.testing.assert_array_equal(G.bmm(a2, b2, shift=7, tok='positive_inf', out_dtype='uint8'),
                                  oracle.matmul(a2, b2, shift=7, tok='positive_inf', out_dtype='uint8'))
    b2t = np.ascontiguousarray(np.swapaxes(b2, 1, 2))
    np.testing.assert_array_equal(G.bmm(a2, b2t, shift=7, tok='conv_even', trans_b=True),
                                  oracle.matmul(a2, b2t, shift=7, tok='conv_even', transpose_b=True))
    big_k = rng.integers(-128, 128, (5, 130, 400)).astype(np.int8)
    big_b = rng.integers(-128, 128, (5, 400, 272)).astype(np.int8)
    np.testing.assert_array_equal(G.bmm(big_k, big_b, shift=0, tok='floor', out_dtype='int8'),
                                  oracle.matmul(big_k, big_b, shift=0, tok='floor', out_dtype='int8'))
    a = rng.integers(-128, 128, (3, 20, 37)).astype(np.int8)   # stored [K, M]
    b = rng.integers(-128, 128, (3, 20, 11)).astype(np.int8)
    np.testing.assert_array_equal(G.bmm(a, b, shift=4, tok='floor', trans_a=True, out_dtype='int16'),
                                  oracle.matmul(a, b, shift=4, tok='floor', transpose_a=True, out_dtype='int16'))


@pytest.fixture(params=['auto', 'generic', 'chunks1', 'chunks2', 'chunks4', 'row_copies'])
def rowop_path(request):
    """Runs a row-op test with automatic kernel selection (bandwidth-oriented kernels where they
    apply), with the generic integer kernels forced, with every work split of the
    bandwidth-oriented kernels forced (16-element chunks per lane; shortest copy ring), and with one
    bulk copy per row instead of one per group of adjacent rows."""
    from aie4ml_b200 import lib as a4c

    L = a4c.load()
    assert L.a4c_set_option(a4c.OPT_ROWOP_PATH, 1 if request.param == 'generic' else 0) == 0
    if request.param.startswith('chunks'):
        assert L.a4c_set_option(a4c.OPT_ROWOP_CHUNKS_PER_LANE, int(request.param[-1])) == 0
        assert L.a4c_set_option(a4c.OPT_ROWOP_MIN_STAGES, 2) == 0
    if request.param == 'row_copies':
        assert L.a4c_set_option(a4c.OPT_ROWOP_CONTIG_COPY, 0) == 0
    yield request.param
    assert L.a4c_set_option(a4c.OPT_ROWOP_CONTIG_COPY, 1) == 0
    assert L.a4c_set_option(a4c.OPT_ROWOP_PATH, 0) == 0
    assert L.a4c_set_option(a4c.OPT_ROWOP_CHUNKS_PER_LANE, 0) == 0
    assert L.a4c_set_option(a4c.OPT_ROWOP_MIN_STAGES, 0) == 0


def _ln_inputs(seed, rows, cols):
    rng = np.random.default_rng(seed)
    x = np.clip(np.rint(rng.normal(2, 32, (rows, cols))), -128, 127).astype(np.int8)
    x[0] = 7
    x[1] = -128
    x[2, ::2], x[2, 1::2] = 127, -128
    x[3] = 0
    x[3, 0] = 1
    return x, rng


@pytest.mark.parametrize('cols', [32, 64, 256, 1024, 4096])
@pytest.mark.parametrize('tok', ['positive_inf', 'conv_even', 'floor', 'ceil', 'negative_inf', 'symmetric_inf'])
def test_layer_norm(cols, tok, rowop_path):
    import gpu_util as G

    x, rng = _ln_inputs(cols, 77, cols)
    gamma = rng.integers(-256, 257, cols)
    beta = rng.integers(-256, 257, cols)
    for out_shift in (4, 0, 13, 15):
        np.testing.assert_array_equal(G.layer_norm(x, gamma, beta, eps_q0=1, out_shift=out_shift, tok=tok),
                                      oracle.layer_norm(x, gamma, beta, eps_q0=1, out_shift=out_shift, tok=tok))
    big_g = rng.integers(-32768, 32768, cols)
    big_b = rng.integers(-32768, 32768, cols)
    np.testing.assert_array_equal(G.layer_norm(x, big_g, big_b, eps_q0=3, out_shift=6, tok=tok),
                                  oracle.layer_norm(x, big_g, big_b, eps_q0=3, out_shift=6, tok=tok))
    mid_g = rng.integers(-16383, 16384, cols)   # largest gamma the bandwidth-oriented kernel admits
    np.testing.assert_array_equal(G.layer_norm(x, mid_g, big_b, eps_q0=1, out_shift=2, tok=tok),
                                  oracle.layer_norm(x, mid_g, big_b, eps_q0=1, out_shift=2, tok=tok))
    addend = rng.integers(-128, 128, x.shape).astype(np.int8)
    fused = G.layer_norm(x, gamma, beta, eps_q0=1, out_shift=4, tok=tok, addend=addend)
    want = oracle.add(oracle.layer_norm(x, gamma, beta, eps_q0=1, out_shift=4, tok=tok), addend, out_dtype='int8')
    np.testing.assert_array_equal(fused, want)


@pytest.mark.parametrize('cols', [64, 256, 1024, 4096])
@pytest.mark.parametrize('tok', ['positive_inf', 'conv_even', 'symmetric_inf'])
def test_add_then_layer_norm_in_one_pass(cols, tok, rowop_path):
    """layernorm(saturate(x + residual)) against the oracle's two steps; the sums saturate on both sides."""
    import gpu_util as G

    x, rng = _ln_inputs(cols + 3, 77, cols)
    residual = rng.integers(-128, 128, x.shape).astype(np.int8)
    residual[0] = 127
    residual[1] = -128
    gamma = rng.integers(-256, 257, cols)
    beta = rng.integers(-256, 257, cols)
    for out_shift in (4, 13):
        got = G.add_layer_norm(x, residual, gamma, beta, eps_q0=1, out_shift=out_shift, tok=tok)
        want = oracle.layer_norm(oracle.add(x, residual, out_dtype='int8'), gamma, beta, eps_q0=1, out_shift=out_shift,
                                 tok=tok)
        np.testing.assert_array_equal(got, want)


@pytest.mark.parametrize('M,K', [(1, 16), (129, 256), (300, 96), (257, 100), (5000, 256), (2049, 1024), (777, 1100), (40000, 384)])
@pytest.mark.parametrize('tok', ['positive_inf', 'conv_even', 'floor', 'ceil', 'negative_inf'])
def test_dense_add_layer_norm_single_kernel(M, K, tok):
    """Dense -> residual Add -> LayerNorm in one kernel (256 features) against the oracle's three steps: both operand
    layouts (weights resident for K <= 256, streamed above), ragged last row tile, sums that saturate on both sides,
    with and without bias / ReLU, uint8 activations, large gamma (integer fscale path), padded residual / output rows."""
    import gpu_util as G

    N = 256
    rng = np.random.default_rng(M * 131 + K)
    w = rng.integers(-128, 128, (K, N)).astype(np.int8)
    residual = rng.integers(-128, 128, (M, N)).astype(np.int8)
    residual[0] = 127
    residual[-1] = -128
    shift = max(1, int(np.ceil(np.log2(K))) + 2)
    cases = [dict(relu=False, bias=True, unsigned=False, gmax=256, out_shift=4, ld=N),
             dict(relu=True, bias=False, unsigned=True, gmax=16383, out_shift=13, ld=N + 16)]
    for c in cases:
        a = (rng.integers(0, 256, (M, K)).astype(np.uint8) if c['unsigned'] else rng.integers(-128, 128, (M, K)).astype(np.int8))
        bias = rng.integers(-(1 << 12), 1 << 12, N) if c['bias'] else None
        gamma = rng.integers(-c['gmax'], c['gmax'] + 1, N)
        gamma[0] = c['gmax']
        beta = rng.integers(-20000, 20000, N)
        sh = shift + (1 if c['unsigned'] else 0)
        got = G.dense_add_layer_norm(a, w, bias, residual, gamma, beta, shift=sh, tok=tok, relu=c['relu'], eps_q0=1,
                                     out_shift=c['out_shift'], ldr=c['ld'], ldo=c['ld'])
        assert got is not None, 'the library refused a request inside the documented envelope'
        d = oracle.dense(a, w, bias, shift=sh, tok=tok, relu=c['relu'], out_dtype='int8')
        want = oracle.layer_norm(oracle.add(d, residual, out_dtype='int8'), gamma, beta, eps_q0=1, out_shift=c['out_shift'],
                                 tok=tok)
        np.testing.assert_array_equal(got, want, err_msg=str(c))


def test_dense_add_layer_norm_envelope():
    """Outside the single kernel's envelope the query says so (the plan then keeps two launches); the option turns it off."""
    from aie4ml_b200 import lib as a4c

    L = a4c.load()
    ok = dict(M=1000, K=256, N=256, lda=256, ldw=256, ldr=256, ldo=256, shift=9, rounding=2, out_shift=4, eps_q0=1, gmax=300)

    def q(**kw):
        v = dict(ok, **kw)
        return L.a4c_dense_add_layernorm_supported(v['M'], v['K'], v['N'], v['lda'], v['ldw'], v['ldr'], v['ldo'], v['shift'],
                                                   v['rounding'], v['out_shift'], v['eps_q0'], v['gmax'])

    assert q() == 0
    for bad in (dict(N=128), dict(N=512), dict(K=8), dict(lda=264), dict(ldr=250), dict(rounding=4), dict(rounding=7),
                dict(out_shift=14), dict(gmax=0), dict(gmax=20000), dict(eps_q0=(1 << 20) + 1)):
        assert q(**bad) == -3, bad
    a4c.check(L.a4c_set_option(a4c.OPT_DENSE_LN_PATH, 1), 'set_option')
    try:
        assert q() == -3
    finally:
        a4c.check(L.a4c_set_option(a4c.OPT_DENSE_LN_PATH, 0), 'set_option')


def test_layer_norm_every_rounding_mode(rowop_path):
    import gpu_util as G

    x, rng = _ln_inputs(5, 40, 256)
    gamma = rng.integers(-2000, 2000, 256)
    beta = rng.integers(-20000, 20000, 256)
    for tok in TOKENS:
        np.testing.assert_array_equal(G.layer_norm(x, gamma, beta, eps_q0=1, out_shift=5, tok=tok),
                                      oracle.layer_norm(x, gamma, beta, eps_q0=1, out_shift=5, tok=tok), err_msg=tok)


@pytest.mark.parametrize('cols', [32, 96, 128, 1024, 2048])
@pytest.mark.parametrize('out_dtype', ['uint8', 'int16'])
def test_softmax_both_modes(cols, out_dtype, rowop_path):
    import gpu_util as G

    x, rng = _ln_inputs(cols + 1, 61, cols)
    np.testing.assert_array_equal(G.softmax(x, mode='exp', exp_kq=23, out_dtype=out_dtype),
                                  oracle.softmax_exp(x, exp_kq=23, out_dtype=out_dtype))
    np.testing.assert_array_equal(G.softmax(x, mode='exp', exp_kq=128, out_dtype=out_dtype),
                                  oracle.softmax_exp(x, exp_kq=128, out_dtype=out_dtype))
    B = min(255, 32767 // cols)
    S = 1 if B < 100 else 3
    Dmax = (B - max(1, -(-256 // cols))) // S
    np.testing.assert_array_equal(G.softmax(x, mode='hccs', B=B, S=S, Dmax=Dmax, out_dtype=out_dtype),
                                  oracle.softmax_hccs(x, B=B, S=S, Dmax=Dmax, out_dtype=out_dtype))
    np.testing.assert_array_equal(G.softmax(x, mode='hccs', B=B, S=S, Dmax=Dmax, inv_shift=14, use_clb=True, out_dtype=out_dtype),
                                  oracle.softmax_hccs(x, B=B, S=S, Dmax=Dmax, inv_shift=14, use_clb=True, out_dtype=out_dtype))
    lo, hi = (0, 256) if out_dtype == 'uint8' else (-32768, 32768)
    addend = rng.integers(lo, hi, x.shape).astype(G.NP[out_dtype])
    fused = G.softmax(x, mode='exp', exp_kq=46, out_dtype=out_dtype, addend=addend)
    want = oracle.add(oracle.softmax_exp(x, exp_kq=46, out_dtype=out_dtype), addend, out_dtype=out_dtype)
    np.testing.assert_array_equal(fused, want)


@pytest.mark.parametrize('dtype', ['int8', 'uint8', 'int16'])
def test_add_saturating(dtype):
    import gpu_util as G

    rng = np.random.default_rng(71)
    lo, hi = {'int8': (-128, 128), 'uint8': (0, 256), 'int16': (-32768, 32768)}[dtype]
    a = rng.integers(lo, hi, (37, 256)).astype(G.NP[dtype])
    b = rng.integers(lo, hi, (37, 256)).astype(G.NP[dtype])
    np.testing.assert_array_equal(G.add(a, b, shift=0, tok='conv_even', dtype=dtype),
                                  oracle.add(a, b, shift=0, tok='conv_even', out_dtype=dtype))
    for tok in TOKENS:
        np.testing.assert_array_equal(G.add(a, b, shift=1, tok=tok, dtype=dtype),
                                      oracle.add(a, b, shift=1, tok=tok, out_dtype=dtype), err_msg=tok)


def _chain_layers(seed, dims, bias=True):
    rng = np.random.default_rng(seed)
    layers = []
    for i in range(len(dims) - 1):
        w = rng.integers(-127, 128, (dims[i], dims[i + 1])).astype(np.int8)
        b = rng.integers(-(1 << 12), 1 << 12, dims[i + 1]).astype(np.int32) if bias else None
        layers.append((w, b, 7 if dims[i] <= 64 else 9, i < len(dims) - 2))
    return layers


def _chain_oracle(x, layers, tok, out_dtype='int8'):
    cur = x
    for i, (w, b, shift, relu) in enumerate(layers):
        last = i == len(layers) - 1
        cur = oracle.dense(cur, w, b, shift=shift, tok=tok, relu=relu, out_dtype=out_dtype if last else 'int8')
    return cur


@pytest.fixture(params=['auto', 'per_layer', 'single_kernel'])
def mlp_path(request):
    """a4c_mlp_i8 with its automatic choice, forced to one Dense launch per layer, and forced to the
    single-kernel narrow chain (which answers 'unsupported' for chains it cannot hold)."""
    from aie4ml_b200 import lib as a4c

    L = a4c.load()
    assert L.a4c_set_option(a4c.OPT_MLP_PATH, ['auto', 'per_layer', 'single_kernel'].index(request.param)) == 0
    yield request.param
    assert L.a4c_set_option(a4c.OPT_MLP_PATH, 0) == 0


@pytest.mark.parametrize('dims', [(16, 64, 32, 32, 5), (512, 1024, 1024, 10), (64, 48), (100, 72, 40, 24),
                                  (256, 256, 200, 16)])
def test_mlp_chain_matches_layer_by_layer_oracle(dims, mlp_path):
    import gpu_util as G
    from aie4ml_b200 import lib as a4c

    if mlp_path == 'single_kernel' and max(dims) > 256:
        x = np.zeros((4, dims[0]), np.int8)
        with pytest.raises(a4c.A4cError, match='no kernel'):
            G.mlp_chain(x, _chain_layers(1, dims), tok='floor')
        return
    if mlp_path == 'single_kernel':
        u = np.random.default_rng(1).integers(0, 256, (45, dims[0])).astype(np.uint8)   # unsigned first operand
        layers = _chain_layers(2, dims)
        np.testing.assert_array_equal(G.mlp_chain(u, layers, tok='symmetric_inf', out_dtype='uint8'),
                                      _chain_oracle(u, layers, 'symmetric_inf', out_dtype='uint8'))

    rng = np.random.default_rng(sum(dims))
    for M in (1, 300, 2048):
        x = rng.integers(-128, 128, (M, dims[0])).astype(np.int8)
        layers = _chain_layers(len(dims), dims)
        for tok in ('positive_inf', 'conv_even'):
            np.testing.assert_array_equal(G.mlp_chain(x, layers, tok=tok), _chain_oracle(x, layers, tok))
    layers = _chain_layers(3, dims, bias=False)
    x = rng.integers(-128, 128, (77, dims[0])).astype(np.int8)
    od = 'int8' if mlp_path == 'single_kernel' else 'int16'   # the single kernel writes 8-bit outputs only
    np.testing.assert_array_equal(G.mlp_chain(x, layers, tok='floor', out_dtype=od),
                                  _chain_oracle(x, layers, 'floor', out_dtype=od))


def test_empty_inputs_are_no_ops():
    import gpu_util as G
    import torch
    from aie4ml_b200 import lib as a4c

    L = a4c.load()
    buf = torch.zeros(4096, dtype=torch.int8, device='cuda')
    p = buf.data_ptr()
    assert L.a4c_dense_i8(p, 64, p, 64, None, p, 64, 0, 64, 64, 7, 2, 0, 0, 0, 0, G.stream()) == 0
    assert L.a4c_add_sat(p, 64, p, 64, p, 64, 0, 64, 0, 6, 0, G.stream()) == 0
    assert L.a4c_layernorm_i8(p, 64, p, p, None, 0, p, 64, 0, 64, 1, 4, 6, 0, G.stream()) == 0
    assert L.a4c_softmax_i8(p, 64, None, 0, p, 64, 0, 64, 1, 0, 0, 0, 15, 0, 23, 1, G.stream()) == 0


def _attention_oracle(q, k, v, *, qk_shift, pv_shift, tok, mode, **sm):
    s = oracle.matmul(q, k, shift=qk_shift, tok=tok, transpose_b=True, out_dtype='int8')
    if mode == 'exp':
        p = oracle.softmax_exp(s, exp_kq=sm['exp_kq'], inv_shift=sm.get('inv_shift', 15), out_dtype='uint8')
    else:
        p = oracle.softmax_hccs(s, B=sm['B'], S=sm['S'], Dmax=sm['Dmax'], inv_shift=sm.get('inv_shift', 15),
                                use_clb=sm.get('use_clb', False), out_dtype='uint8')
    return oracle.matmul(p, v, shift=pv_shift, tok=tok, out_dtype='int8')


@pytest.mark.parametrize('tok', ['positive_inf', 'conv_even', 'floor', 'symmetric_inf'])
@pytest.mark.parametrize('mode', ['exp', 'hccs'])
def test_fused_attention_head_equals_matmul_softmax_matmul(tok, mode):
    """The fused kernel against the oracle's three-step chain, on head slices of a packed tensor (pitch 256,
    head offsets 64 / 128 / 192), more items than SMs so every ring stage and both softmax groups wrap."""
    import gpu_util as G

    rng = np.random.default_rng(11)
    batch, seq, width = 333, 128, 256
    qkv = np.clip(np.rint(rng.normal(0, 40, (batch, seq, width))), -128, 127).astype(np.int8)
    qkv[0, :, :64] = 127          # saturating scores
    qkv[1, :, 64:128] = -128
    qkv[2] = 0                    # all scores equal
    sm = dict(exp_kq=23) if mode == 'exp' else dict(B=200, S=3, Dmax=66)
    q0, k0, v0 = 64, 128, 192
    got = G.attention(qkv, (q0, k0, v0), qk_shift=9, pv_shift=8, tok=tok, mode=mode, **sm)
    want = _attention_oracle(qkv[..., q0:q0 + 64], qkv[..., k0:k0 + 64], qkv[..., v0:v0 + 64], qk_shift=9, pv_shift=8,
                             tok=tok, mode=mode, **sm)
    np.testing.assert_array_equal(got[..., q0:q0 + 64], want)
    untouched = np.delete(got, np.s_[q0:q0 + 64], axis=2)
    assert (untouched == 0x5A).all()


@pytest.mark.parametrize('heads,sq,layout', [(4, 128, 'cols'), (3, 200, 'cols'), (1, 77, 'cols'), (4, 128, 'blocks'),
                                             (2, 150, 'blocks')])
@pytest.mark.parametrize('mode', ['exp', 'hccs'])
def test_fused_attention_all_heads_of_a_layer_in_one_launch(heads, sq, layout, mode):
    """(batch entry, head) items with the head index fastest; query counts that are not a multiple of the 128-row tile;
    every head against the oracle's three-step chain; unused width stays untouched."""
    import gpu_util as G

    rng = np.random.default_rng(40 + heads)
    batch, width = 150, heads * 64
    q = np.clip(np.rint(rng.normal(0, 45, (batch, sq, width))), -128, 127).astype(np.int8)
    k = np.clip(np.rint(rng.normal(0, 45, (batch, 128, width))), -128, 127).astype(np.int8)
    v = rng.integers(-128, 128, (batch, 128, width)).astype(np.int8)
    sm = dict(exp_kq=23) if mode == 'exp' else dict(B=200, S=3, Dmax=66)
    got = G.attention_heads(q, k, v, heads, qk_shift=9, pv_shift=8, tok='positive_inf', mode=mode, layout=layout, **sm)
    for h in range(heads):
        cols = slice(64 * h, 64 * h + 64)
        want = _attention_oracle(q[..., cols], k[..., cols], v[..., cols], qk_shift=9, pv_shift=8, tok='positive_inf',
                                 mode=mode, **sm)
        np.testing.assert_array_equal(got[..., cols], want, err_msg=f'head {h}')


def test_fused_attention_other_softmax_parameters_and_rejections():
    import gpu_util as G
    from aie4ml_b200 import lib as a4c

    rng = np.random.default_rng(12)
    qkv = rng.integers(-128, 128, (5, 128, 192)).astype(np.int8)
    for sm in (dict(mode='hccs', B=255, S=1, Dmax=200, inv_shift=14, use_clb=True),
               dict(mode='exp', exp_kq=128, inv_shift=12), dict(mode='exp', exp_kq=1, inv_shift=22)):
        got = G.attention(qkv, (0, 64, 128), qk_shift=11, pv_shift=7, tok='positive_inf', **sm)
        mode = sm.pop('mode')
        want = _attention_oracle(qkv[..., :64], qkv[..., 64:128], qkv[..., 128:], qk_shift=11, pv_shift=7,
                                 tok='positive_inf', mode=mode, **sm)
        np.testing.assert_array_equal(got[..., :64], want)
    L = a4c.load()
    p = G.dev(qkv).data_ptr()
    ok = (p, 192, 128 * 192, p + 64, 192, 128 * 192, p + 128, 192, 128 * 192, p, 192, 128 * 192, 5, 128, 128, 64, 9, 8,
          1, 0, 0, 0, 15)
    assert L.a4c_attention_i8_supported(*ok) == 0
    bad_keys = list(ok); bad_keys[14] = 64
    assert L.a4c_attention_i8_supported(*bad_keys) == a4c.A4C_ERR_UNSUPPORTED
    misaligned = list(ok); misaligned[0] = p + 8
    assert L.a4c_attention_i8_supported(*misaligned) == a4c.A4C_ERR_ALIGNMENT
    one_zero_shift = list(ok); one_zero_shift[16] = 0
    assert L.a4c_attention_i8_supported(*one_zero_shift) == a4c.A4C_ERR_UNSUPPORTED
    # surrogate parameters outside the reference's bounds (softmax/common.py:59-89) are left to the separate kernels:
    # a negative slope makes scores grow past 32767, where the fused kernel's normalisation is not defined
    for B, S, Dmax in ((200, -3, 60), (40000, 1, 10), (-1, 0, 0), (10, 1, 20), (10, 1, -1)):
        bad = list(ok); bad[18:22] = [0, B, S, Dmax]
        assert L.a4c_attention_i8_supported(*bad) == a4c.A4C_ERR_UNSUPPORTED, (B, S, Dmax)
    fine = list(ok); fine[18:22] = [0, 200, 3, 66]
    assert L.a4c_attention_i8_supported(*fine) == 0


@pytest.mark.parametrize('wide', [False, True])
@pytest.mark.parametrize('tok', ['positive_inf', 'conv_even', 'floor', 'symmetric_zero'])
def test_dense_16_bit_operands(wide, tok):
    """int16 x int8 accumulates in 32 bits and wraps (large K and full-range codes make it wrap), int16 x int16 in 64
    bits exactly; bias, ReLU and every output type as for int8."""
    import gpu_util as G

    rng = np.random.default_rng(90 + wide)
    M, K, N = 77, 300, 45
    a = rng.integers(-32768, 32768, (M, K)).astype(np.int16)
    w = (rng.integers(-32768, 32768, (K, N)).astype(np.int16) if wide else rng.integers(-128, 128, (K, N)).astype(np.int8))
    bias = rng.integers(-(1 << 20), 1 << 20, N).astype(np.int32)
    acc_bits = 64 if wide else 32
    for shift, relu, od in ((17 if wide else 9, False, 'int16'), (24 if wide else 16, True, 'int8'), (0, False, 'int16'),
                            (22 if wide else 14, False, 'uint8')):
        got = G.dense16(a, w, bias, shift=shift, tok=tok, relu=relu, out_dtype=od)
        want = oracle.dense(a, w, bias, shift=shift, tok=tok, relu=relu, out_dtype=od, acc_bits=acc_bits)
        np.testing.assert_array_equal(got, want)
    got = G.dense16(a, w, None, shift=40 if wide else 12, tok=tok, relu=False, out_dtype='int16')
    np.testing.assert_array_equal(got, oracle.dense(a, w, None, shift=40 if wide else 12, tok=tok, relu=False,
                                                    out_dtype='int16', acc_bits=acc_bits))


@pytest.mark.parametrize('kind', ['int8', 'uint8', 'int16xint8', 'int16xint16'])
def test_dense_over_a_transposed_stored_input(kind):
    """TRANSPOSE_INPUT of the reference's Dense: the stored tensor is a stack of [K, M] matrices."""
    import gpu_util as G

    rng = np.random.default_rng(120)
    batch, K, M, N = 3, 52, 37, 29
    if kind == 'int8':
        a_t, w = rng.integers(-128, 128, (batch, K, M)).astype(np.int8), rng.integers(-128, 128, (K, N)).astype(np.int8)
    elif kind == 'uint8':
        a_t, w = rng.integers(0, 256, (batch, K, M)).astype(np.uint8), rng.integers(-128, 128, (K, N)).astype(np.int8)
    elif kind == 'int16xint8':
        a_t, w = rng.integers(-32768, 32768, (batch, K, M)).astype(np.int16), rng.integers(-128, 128, (K, N)).astype(np.int8)
    else:
        a_t = rng.integers(-32768, 32768, (batch, K, M)).astype(np.int16)
        w = rng.integers(-32768, 32768, (K, N)).astype(np.int16)
    acc_bits = 64 if kind == 'int16xint16' else 32
    base = {'int8': 7, 'uint8': 8, 'int16xint8': 15, 'int16xint16': 23}[kind]
    bias = rng.integers(-(1 << 16), 1 << 16, N).astype(np.int32)
    a = np.swapaxes(a_t, 1, 2)
    for tok, relu, od, b in (('conv_even', True, 'int8', bias), ('positive_inf', False, 'uint8', bias), ('floor', False, 'int16', None)):
        got = G.dense_ta(a_t, w, b, shift=base, tok=tok, relu=relu, out_dtype=od)
        want = oracle.dense(a, w, b, shift=base, tok=tok, relu=relu, out_dtype=od, acc_bits=acc_bits)
        np.testing.assert_array_equal(got, want)


def test_bmm_16_bit_operands_with_transposes():
    import gpu_util as G

    rng = np.random.default_rng(95)
    a = rng.integers(-3000, 3000, (4, 33, 70)).astype(np.int16)
    b16 = rng.integers(-3000, 3000, (4, 70, 20)).astype(np.int16)
    np.testing.assert_array_equal(G.bmm16(a, b16, shift=14, tok='conv_even'),
                                  oracle.matmul(a, b16, shift=14, tok='conv_even', out_dtype='int16', acc_bits=64))
    bt8 = rng.integers(-128, 128, (4, 20, 70)).astype(np.int8)          # stored [N, K]
    np.testing.assert_array_equal(G.bmm16(a, bt8, shift=9, tok='positive_inf', trans_b=True, out_dtype='int8'),
                                  oracle.matmul(a, bt8, shift=9, tok='positive_inf', transpose_b=True, out_dtype='int8',
                                                acc_bits=32))
    at = rng.integers(-32768, 32768, (2, 70, 33)).astype(np.int16)      # stored [K, M]
    np.testing.assert_array_equal(G.bmm16(at, b16[:2], shift=20, tok='floor', trans_a=True),
                                  oracle.matmul(at, b16[:2], shift=20, tok='floor', transpose_a=True, out_dtype='int16',
                                                acc_bits=64))


@pytest.mark.parametrize('fmt', ['bfloat16', 'fp8_e4m3'])
@pytest.mark.parametrize('shape', [(300, 520, 200), (128, 64, 256), (1000, 2048, 1030), (5, 48, 16)])
def test_float_dense_on_the_tensor_cores(fmt, shape):
    """bfloat16 (kind::f16) and fp8 E4M3 (kind::f8f6f4) Dense with float32 accumulation: against a float64 evaluation
    on the stored operands rounded to the storage type, within one step of that type (the order of the float32
    additions is not part of the contract), and against the tiled SIMT kernel of the same entry point.  Shapes cover
    a K tail shorter than a stage, a ragged last column tile, several row and column tiles, and a single narrow tile."""
    import gpu_util as G

    M, K, N = shape
    rng = np.random.default_rng(M + K + N)
    a = rng.normal(0, 1, (M, K))
    w = rng.normal(0, 0.5 / np.sqrt(K), (K, N)) * (4.0 if fmt == 'fp8_e4m3' else 1.0)
    bias = rng.normal(0, 0.5, N)
    for relu, use_bias in ((True, True), (False, False)):
        got, a_st, w_st = G.dense_float(a, w, bias if use_bias else None, relu=relu, fmt=fmt)
        ref = a_st.astype(np.float64) @ w_st.astype(np.float64) + (bias.astype(np.float32).astype(np.float64) if use_bias else 0.0)
        if relu:
            ref = np.maximum(ref, 0.0)
        want = oracle.round_float(ref, fmt)
        np.testing.assert_array_equal(got, oracle.round_float(got, fmt))      # every result is a value of the type
        step = 2.0 ** -3 if fmt == 'fp8_e4m3' else 2.0 ** -7
        np.testing.assert_allclose(got, want, rtol=step * 1.01, atol=2.0 ** -8)
        assert (got == want).mean() > 0.95
        simt, _, _ = G.dense_float(a, w, bias if use_bias else None, relu=relu, fmt=fmt, simt=True)
        np.testing.assert_allclose(got, simt, rtol=step * 1.01, atol=2.0 ** -8)


@pytest.mark.parametrize('shape', [(3, 200, 160, 48), (2, 64, 128, 256), (1, 1024, 400, 80), (5, 48, 16, 16)])
@pytest.mark.parametrize('unsigned', [False, True])
def test_dense_over_a_transposed_input_on_the_tensor_cores(shape, unsigned):
    """Stored [K, M] inputs whose pitches meet the TMA rules run on the tcgen05 kernel with an MN-major A operand
    (128-byte-swizzled [k, m] tiles): K tails shorter than a stage, M tails shorter than a tile, several column tiles,
    bias that wraps the accumulator, ReLU, both 8-bit input types; and the dp4a kernel on the same arguments."""
    import gpu_util as G
    from aie4ml_b200 import lib as a4c

    batch, K, M, N = shape
    rng = np.random.default_rng(sum(shape) + unsigned)
    a_t = (rng.integers(0, 256, (batch, K, M)).astype(np.uint8) if unsigned
           else rng.integers(-128, 128, (batch, K, M)).astype(np.int8))
    w = rng.integers(-128, 128, (K, N)).astype(np.int8)
    bias = rng.integers(-(1 << 31), 1 << 31, N).astype(np.int32)
    a = np.swapaxes(a_t, 1, 2)
    L = a4c.load()
    for tok, relu, od, b, shift in (('positive_inf', True, 'int8', bias, 9), ('conv_even', False, 'uint8', None, 8),
                                    ('floor', False, 'int8', bias, 0)):
        want = oracle.dense(a, w, b, shift=shift, tok=tok, relu=relu, out_dtype=od)
        got = G.dense_ta(a_t, w, b, shift=shift, tok=tok, relu=relu, out_dtype=od)
        np.testing.assert_array_equal(got, want)
        assert L.a4c_set_option(a4c.OPT_BMM_PATH, 1) == 0          # the any-stride kernel on the same call
        try:
            np.testing.assert_array_equal(G.dense_ta(a_t, w, b, shift=shift, tok=tok, relu=relu, out_dtype=od), want)
        finally:
            assert L.a4c_set_option(a4c.OPT_BMM_PATH, 0) == 0
    a4c.device_status(G.stream())


def test_bmm_with_a_transposed_left_operand_on_the_tensor_cores():
    """TRANSPOSE_A with a K-major right operand (both stored transposed): A_b [K, M] is an MN-major operand."""
    import gpu_util as G
    from aie4ml_b200 import lib as a4c

    rng = np.random.default_rng(321)
    for batch, M, K, N in ((7, 128, 64, 128), (3, 80, 200, 48), (2, 272, 32, 16)):
        at = rng.integers(-128, 128, (batch, K, M)).astype(np.int8)
        bt = rng.integers(-128, 128, (batch, N, K)).astype(np.int8)
        want = oracle.matmul(at, bt, shift=7, tok='positive_inf', transpose_a=True, transpose_b=True)
        np.testing.assert_array_equal(G.bmm(at, bt, shift=7, tok='positive_inf', trans_a=True, trans_b=True), want)
        ut = rng.integers(0, 256, (batch, K, M)).astype(np.uint8)
        np.testing.assert_array_equal(G.bmm(ut, bt, shift=9, tok='conv_even', trans_a=True, trans_b=True, out_dtype='uint8'),
                                      oracle.matmul(ut, bt, shift=9, tok='conv_even', transpose_a=True, transpose_b=True,
                                                    out_dtype='uint8'))
    a4c.device_status(G.stream())


@pytest.mark.parametrize('panel_mib', [1, 2, 0])
def test_dense_tcgen05_column_panels(panel_mib):
    """The streaming tile order walks the column tiles in panels when the weights exceed the panel size: forced here
    with 1 and 2 MiB panels on a 2.25 MiB weight matrix (nine column tiles: panels of 4 + 4 + 1 and 8 + 1), and the
    single-panel order (0), all against the oracle, with more tiles than SMs and ragged last row tile."""
    import gpu_util as G
    from aie4ml_b200 import lib as a4c

    L = a4c.load()
    assert L.a4c_set_option(a4c.OPT_DENSE_PANEL_MIB, panel_mib) == 0
    try:
        a, w, bias = _rand_dense(500 + panel_mib, 3000, 1024, 2304)
        want = oracle.dense(a, w, bias, shift=10, tok='positive_inf', relu=True)
        got = G.dense(a, w, bias, shift=10, tok='positive_inf', relu=True, algo=TC)
        np.testing.assert_array_equal(got, want)
        # the CTA-pair kernel walks its 256 x 256 tiles in the same panels
        np.testing.assert_array_equal(G.dense(a, w, bias, shift=10, tok='positive_inf', relu=True, algo=TC2), want)
        a, w, _ = _rand_dense(600 + panel_mib, 700, 2048, 1300)
        got = G.dense(a, w, None, shift=11, tok='conv_even', relu=False, algo=TC)
        np.testing.assert_array_equal(got, oracle.dense(a, w, None, shift=11, tok='conv_even', relu=False))
    finally:
        assert L.a4c_set_option(a4c.OPT_DENSE_PANEL_MIB, 32) == 0


@pytest.mark.parametrize('shape', [(77, 304, 45), (300, 1024, 272), (1000, 64, 128), (130, 4096, 16), (5, 16, 200)])
@pytest.mark.parametrize('tok', ['positive_inf', 'conv_even', 'floor'])
def test_dense_int16_by_int8_on_the_tensor_cores(shape, tok):
    """int16 activations against int8 weights as two byte digits on tcgen05 (signed high plane, unsigned low plane,
    combined as (high << 8) + low in wrapping 32-bit arithmetic): full-range codes and long K make the 32-bit
    accumulator wrap, which the digit form must reproduce bit for bit; every output type, bias, ReLU, ragged widths;
    and the SIMT kernel on the same arguments."""
    import gpu_util as G
    from aie4ml_b200 import lib as a4c

    M, K, N = shape
    rng = np.random.default_rng(sum(shape))
    a = rng.integers(-32768, 32768, (M, K)).astype(np.int16)
    a[0, :] = 32767
    a[-1, :] = -32768
    w = rng.integers(-128, 128, (K, N)).astype(np.int8)
    w[:, 0] = 127
    bias = rng.integers(-(1 << 31), 1 << 31, N).astype(np.int32)
    L = a4c.load()
    for shift, relu, od, b in ((15, False, 'int8', bias), (12, True, 'int16', bias), (17, False, 'uint8', None), (0, False, 'int16', None)):
        want = oracle.dense(a, w, b, shift=shift, tok=tok, relu=relu, out_dtype=od, acc_bits=32)
        np.testing.assert_array_equal(G.dense16(a, w, b, shift=shift, tok=tok, relu=relu, out_dtype=od), want)
    assert L.a4c_set_option(a4c.OPT_WIDE_DENSE_PATH, 1) == 0
    try:
        np.testing.assert_array_equal(G.dense16(a, w, bias, shift=15, tok=tok, relu=False, out_dtype='int8'),
                                      oracle.dense(a, w, bias, shift=15, tok=tok, relu=False, out_dtype='int8', acc_bits=32))
    finally:
        assert L.a4c_set_option(a4c.OPT_WIDE_DENSE_PATH, 0) == 0
    a4c.device_status(G.stream())
