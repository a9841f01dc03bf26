"""The ONNX Q/DQ importer on hand-built graph descriptions (no `onnx` package needed): the lowered plan must
equal the plan of the same network built with the programmatic GraphBuilder."""

import numpy as np
import pytest

from aie4ml_b200 import from_graph, intent
from aie4ml_b200.frontends.graph import GraphBuilder
from aie4ml_b200.frontends.onnx_import import OnnxGraph, OnnxNode, from_onnx, lower_onnx_graph, require_onnx


def _qdq(nodes, inits, src, name, frac, dtype=np.int8):
    """x -> QuantizeLinear -> DequantizeLinear; returns the DQ output name."""
    inits[f'{name}_s'] = np.array(2.0 ** -frac, dtype=np.float32)
    inits[f'{name}_z'] = np.array(0, dtype=dtype)
    nodes.append(OnnxNode('QuantizeLinear', f'{name}_q', [src, f'{name}_s', f'{name}_z'], [f'{name}_qo']))
    nodes.append(OnnxNode('DequantizeLinear', f'{name}_dq', [f'{name}_qo', f'{name}_s', f'{name}_z'], [f'{name}_dqo']))
    return f'{name}_dqo'


def _const_dq(nodes, inits, name, codes, frac):
    """An integer initializer -> DequantizeLinear; returns the DQ output name."""
    inits[name] = codes
    inits[f'{name}_s'] = np.array(2.0 ** -frac, dtype=np.float32)
    inits[f'{name}_z'] = np.array(0, dtype=codes.dtype)
    nodes.append(OnnxNode('DequantizeLinear', f'{name}_dq', [name, f'{name}_s', f'{name}_z'], [f'{name}_f']))
    return f'{name}_f'


def _mlp_onnx(rng):
    nodes, inits = [], {}
    w1 = rng.integers(-127, 128, (16, 32)).astype(np.int8)
    b1 = rng.integers(-2000, 2000, 32).astype(np.int32)
    w2 = rng.integers(-127, 128, (8, 32)).astype(np.int8)          # stored [N, K]: Gemm transB = 1
    x = _qdq(nodes, inits, 'x', 'xin', 4)
    nodes.append(OnnxNode('Gemm', 'fc1', [x, _const_dq(nodes, inits, 'w1', w1, 6), _const_dq(nodes, inits, 'b1', b1, 10)],
                          ['fc1_o']))
    nodes.append(OnnxNode('Relu', 'act1', ['fc1_o'], ['act1_o']))
    h = _qdq(nodes, inits, 'act1_o', 'h', 3, np.uint8)
    nodes.append(OnnxNode('Gemm', 'fc2', [h, _const_dq(nodes, inits, 'w2', w2, 7)], ['fc2_o'], {'transB': 1}))
    y = _qdq(nodes, inits, 'fc2_o', 'yq', 2)
    g = OnnxGraph(nodes, inits, {'x': ((5, 16), np.float32)}, [y], 'mlp')
    return g, (w1, b1, w2)


def _mlp_builder(w1, b1, w2):
    b = GraphBuilder({'Part': 'cuda_b200'}, name='mlp')
    x = b.input('x', (5, 16), intent(8, 4))
    h = b.dense('fc1', x, w1.astype(np.float64) / 64.0, intent(8, 6), intent(8, 3), bias=b1.astype(np.float64) / 1024.0,
                bias_precision=intent(32, 10), relu=True, relu_precision=intent(8, 3, signed=False))
    y = b.dense('fc2', h, w2.T.astype(np.float64) / 128.0, intent(8, 7), intent(8, 2))
    b.output(y)
    return b


def test_qdq_mlp_lowers_like_the_programmatic_graph():
    rng = np.random.default_rng(0)
    g, consts = _mlp_onnx(rng)
    got = from_onnx(g, {'Part': 'cuda_b200'}).export_plan()
    want = from_graph(_mlp_builder(*consts)).export_plan()
    assert [op['kind'] for op in got['ops']] == ['dense', 'dense']
    for a, b in zip(got['ops'], want['ops']):
        for key in ('K', 'N', 'shift', 'rounding', 'relu', 'out_dtype', 'lhs_dtype'):
            assert a[key] == b[key], (a['name'], key)
        np.testing.assert_array_equal(got['params'][a['weight']], want['params'][b['weight']])
        assert bool(a['bias']) == bool(b['bias'])
        if a['bias']:
            np.testing.assert_array_equal(got['params'][a['bias']], want['params'][b['bias']])
    assert got['ops'][0]['rounding'] == 'conv_even' and got['ops'][0]['shift'] == 4 + 6 - 3   # ONNX Q/DQ is always RND_CONV
    assert got['outputs'] == ['yq_dqo'] and got['inputs'] == ['x']


def test_attention_pieces_and_view_ops_import():
    rng = np.random.default_rng(1)
    nodes, inits = [], {}
    x = _qdq(nodes, inits, 'x', 'xin', 5)
    inits['split_sizes'] = np.array([32, 32], dtype=np.int64)
    nodes.append(OnnxNode('Split', 'sp', [x, 'split_sizes'], ['a', 'b'], {'axis': -1}))
    nodes.append(OnnxNode('Transpose', 'tr', ['b'], ['bt'], {'perm': [0, 2, 1]}))
    nodes.append(OnnxNode('MatMul', 'qk', ['a', 'bt'], ['s']))
    s = _qdq(nodes, inits, 's', 'sq', 1)
    inits['temp'] = np.array(8.0, dtype=np.float32)
    nodes.append(OnnxNode('Div', 'scale', [s, 'temp'], ['s2']))
    nodes.append(OnnxNode('Softmax', 'sm', ['s2'], ['p'], {'axis': -1}))
    p = _qdq(nodes, inits, 'p', 'pq', 8, np.uint8)
    nodes.append(OnnxNode('MatMul', 'av', [p, 'a'], ['o']))
    o = _qdq(nodes, inits, 'o', 'oq', 5)
    inits['gamma'] = rng.uniform(0.5, 1.5, 32).astype(np.float32)
    inits['beta'] = rng.uniform(-0.1, 0.1, 32).astype(np.float32)
    nodes.append(OnnxNode('LayerNormalization', 'ln', [o, 'gamma', 'beta'], ['n'], {'axis': -1, 'epsilon': 2.0 ** -10}))
    n = _qdq(nodes, inits, 'n', 'nq', 4)
    plan = from_onnx(OnnxGraph(nodes, inits, {'x': ((3, 32, 64), np.float32)}, [n]), {'Part': 'cuda_b200'}).export_plan()
    kinds = [op['kind'] for op in plan['ops']]
    assert kinds == ['slice', 'matmul', 'softmax', 'matmul', 'layer_norm']
    qk, sm, av, ln = (op for op in plan['ops'] if op['kind'] != 'slice')
    assert qk['transpose_rhs'] and qk['shift'] == 5 + 5 - 1 and av['lhs_dtype'] == 'uint8' and av['shift'] == 8 + 5 - 5
    assert sm['approximation'] == 'exp' and sm['exp_kq'] >= 1 and ln['rounding'] == 'conv_even'


def test_importer_rejections_name_the_node():
    inits = {'s': np.array(0.3, dtype=np.float32), 'z': np.array(0, dtype=np.int8)}
    g = OnnxGraph([OnnxNode('QuantizeLinear', 'q0', ['x', 's', 'z'], ['xq'])], inits, {'x': ((2, 16), np.float32)}, ['xq'])
    with pytest.raises(ValueError, match='q0: scale .* is not a power of two'):
        lower_onnx_graph(g, {'Part': 'cuda_b200'})
    inits = {'s': np.array(0.5, dtype=np.float32), 'z': np.array(3, dtype=np.int8)}
    g = OnnxGraph([OnnxNode('QuantizeLinear', 'q0', ['x', 's', 'z'], ['xq'])], inits, {'x': ((2, 16), np.float32)}, ['xq'])
    with pytest.raises(ValueError, match='q0: zero_point must be 0'):
        lower_onnx_graph(g, {'Part': 'cuda_b200'})
    g = OnnxGraph([OnnxNode('Gelu', 'g0', ['x'], ['y'])], {}, {'x': ((2, 16), np.float32)}, ['y'])
    with pytest.raises(NotImplementedError, match='g0: ONNX operator Gelu has no handler'):
        lower_onnx_graph(g, {'Part': 'cuda_b200'})
    g = OnnxGraph([OnnxNode('Relu', 'r0', ['x'], ['y'])], {}, {'w': ((2, 16), np.float32)}, ['y'])
    with pytest.raises(ValueError, match='r0: input x is not a lowered tensor'):
        lower_onnx_graph(g, {'Part': 'cuda_b200'})


def test_from_onnx_without_the_onnx_package_says_what_to_do():
    try:
        require_onnx()
    except ImportError as exc:
        assert 'from_graph' in str(exc)
        with pytest.raises(ImportError, match='onnx'):
            from_onnx('/nonexistent/model.onnx', {'Part': 'cuda_b200'})
    else:
        pytest.skip('onnx is installed here')
