"""Small lowered-graph cases shared by the fixture generator and the tests that read the fixtures.

Every case fits the reference's AIE tile-memory limits (a 16 KiB bank per operand tile), so the
reference's own Resolve + Pack passes accept it and its numeric decisions can be recorded.
Only rounding modes that exist in the reference's enum are used here.
"""

from __future__ import annotations

import numpy as np

from aie4ml_b200.frontends.graph import GraphBuilder, intent


def _rng(seed):
    return np.random.default_rng(seed)


def case_mlp_onnx_style():
    """16 -> 64 -> 32 MLP, Gemm-style bias (dense + add), ReLU after the first layer, RND_CONV everywhere."""
    r = _rng(10)
    b = GraphBuilder({'Part': 'cuda_b200'}, name='mlp')
    x = b.input('x', (8, 16), intent(8, 4))
    h = b.dense('fc0', x, r.uniform(-1, 1, (16, 64)), intent(8, 6), intent(8, 3), bias=r.uniform(-1, 1, 64),
                bias_precision=intent(32, 10), relu=True)
    y = b.dense('fc1', h, r.uniform(-0.5, 0.5, (64, 32)), intent(8, 7), intent(8, 2), bias=r.uniform(-2, 2, 32),
                bias_precision=intent(32, 10))
    b.output(y)
    return b


def case_dense_modes(out_rounding: str, w_rounding: str, w_sat: str):
    """One dense whose tensors carry hls4ml-style rounding / saturation modes."""
    r = _rng(11)
    b = GraphBuilder({'Part': 'cuda_b200'}, name='dense_modes')
    x = b.input('x', (8, 32), intent(8, 5, rounding='TRN'))
    y = b.dense('fc', x, r.uniform(-2.5, 2.5, (32, 16)), intent(8, 6, rounding=w_rounding, saturation=w_sat),
                intent(8, 4, rounding=out_rounding), bias=r.uniform(-3, 3, 16),
                bias_precision=intent(16, 8, rounding=w_rounding, saturation=w_sat))
    b.output(y)
    return b


def case_attention_piece(softmax: str):
    """q @ k^T (Transpose folded into the matmul), 1/8 scale, softmax, @ v -- one attention head."""
    directives = {}
    if softmax == 'hccs':
        directives = {'sm': {'approximation': 'hccs', 'hccs': {'B': 200, 'S': 3, 'Dmax': 66, 'inv_shift': 14}}}
    b = GraphBuilder({'Part': 'cuda_b200', 'LayerDirectives': directives}, name=f'attn_{softmax}')
    q = b.input('q', (16, 64), intent(8, 5))
    k = b.input('k', (128, 64), intent(8, 5))
    v = b.input('v', (128, 32), intent(8, 5))
    kt = b.transpose('kt', k, [1, 0])
    s = b.matmul('qk', q, kt, intent(8, 1))
    if softmax == 'exp':
        s = b.scale('scale', s, 0.125)
    p = b.softmax('sm', s, intent(8, 8, signed=False))
    o = b.matmul('av', p, v, intent(8, 5))
    b.output(o)
    return b


def case_matmul_output_scale():
    """A constant Mul after a matmul whose consumer cannot absorb it: folds into the matmul's shift."""
    b = GraphBuilder({'Part': 'cuda_b200'}, name='mm_scale')
    a = b.input('a', (16, 64), intent(8, 4))
    c = b.input('c', (64, 32), intent(8, 4))
    m = b.matmul('mm', a, c, intent(8, 2))
    s = b.scale('half', m, 0.25)
    b.output(s)
    return b


def case_layer_norm():
    r = _rng(12)
    b = GraphBuilder({'Part': 'cuda_b200'}, name='ln')
    x = b.input('x', (8, 256), intent(8, 3))
    y = b.layer_norm('ln', x, r.uniform(-2, 2, 256), r.uniform(-0.9, 0.9, 256), intent(8, 5), epsilon=0.015625 * 2)
    b.output(y)
    return b


def case_residual_add():
    r = _rng(13)
    b = GraphBuilder({'Part': 'cuda_b200'}, name='res')
    x = b.input('x', (8, 64), intent(8, 4))
    h = b.dense('fc', x, r.uniform(-1, 1, (64, 64)), intent(8, 6), intent(8, 4))
    y = b.add('res', x, h, intent(8, 4))
    b.output(y)
    return b


def case_dense_16_bit(w_width: int):
    """int16 activations against int8 weights (32-bit accumulator) or int16 weights (64-bit accumulator)."""
    r = _rng(14 + w_width)
    b = GraphBuilder({'Part': 'cuda_b200'}, name=f'dense16x{w_width}')
    x = b.input('x', (8, 32), intent(16, 9))
    w_frac = 6 if w_width == 8 else 12
    y = b.dense('fc', x, r.uniform(-1.5, 1.5, (32, 16)), intent(w_width, w_frac), intent(16 if w_width == 8 else 8, 5),
                bias=r.uniform(-2, 2, 16), bias_precision=intent(32, 9 + w_frac), relu=(w_width == 16))
    b.output(y)
    return b


CASES = {
    'dense_int16_x_int8': lambda: case_dense_16_bit(8),
    'dense_int16_x_int16': lambda: case_dense_16_bit(16),
    'mlp_onnx_style': case_mlp_onnx_style,
    'dense_rnd_trn': lambda: case_dense_modes('RND', 'TRN', 'WRAP'),
    'dense_trnzero_rndzero': lambda: case_dense_modes('TRN_ZERO', 'RND_ZERO', 'SAT_SYM'),
    'dense_rndinf_rndmininf': lambda: case_dense_modes('RND_INF', 'RND_MIN_INF', 'SAT_ZERO'),
    'dense_trn_rndconv': lambda: case_dense_modes('TRN', 'RND_CONV', 'SAT'),
    'attention_exp': lambda: case_attention_piece('exp'),
    'attention_hccs': lambda: case_attention_piece('hccs'),
    'matmul_output_scale': case_matmul_output_scale,
    'layer_norm': case_layer_norm,
    'residual_add': case_residual_add,
}
