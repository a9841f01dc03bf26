"""The float-simulation path (AIEConfig.ComputeDtype): lowering on CPU, execution on the GPU within the
tolerances the reference states for this path (reference tests/test_float_sim.py:87-93:
bfloat16 rtol 1e-2 / atol 5e-2, float32 rtol 1e-3 / atol 1e-3, against a float model of the same network)."""

import numpy as np
import pytest

from aie4ml_b200 import from_graph
from aie4ml_b200.frontends.graph import GraphBuilder, intent
from aie4ml_b200.quant_utils import from_bf16_bits, from_fp8_bits, to_bf16_bits, to_fp8_bits
from oracle import oracle

TOL = {'bfloat16': dict(rtol=1e-2, atol=5e-2), 'float32': dict(rtol=1e-3, atol=1e-3), 'float': dict(rtol=1e-3, atol=1e-3)}


def _mlp(compute_dtype, batch=4, n_in=32, n_h=32, n_out=16, seed=0):
    """The network of the reference's float test: Dense + ReLU + Dense, 16-bit quantisers, small normal weights."""
    rng = np.random.default_rng(seed)
    w0, b0 = rng.normal(0, 0.05, (n_in, n_h)), rng.normal(0, 0.05, n_h)
    w1, b1 = rng.normal(0, 0.05, (n_h, n_out)), rng.normal(0, 0.05, n_out)
    b = GraphBuilder({'Part': 'cuda_b200', 'AIEConfig': {'ComputeDtype': compute_dtype}}, name=f'mlp_{compute_dtype}')
    x = b.input('x', (batch, n_in), intent(16, 13))
    h = b.dense('dense0', x, w0, intent(16, 13), intent(16, 13), bias=b0, bias_precision=intent(16, 13), relu=True)
    y = b.dense('dense1', h, w1, intent(16, 13), intent(16, 13), bias=b1, bias_precision=intent(16, 13))
    b.output(y)
    return b, (w0, b0, w1, b1)


def _float_model(x, w0, b0, w1, b1):
    return np.maximum(x @ w0 + b0, 0.0) @ w1 + b1


@pytest.mark.parametrize('compute_dtype', ['bfloat16', 'float32', 'float'])
def test_force_float_mode_relabels_every_tensor_and_selects_the_float_variants(compute_dtype):
    b, _ = _mlp(compute_dtype)
    plan = from_graph(b).export_plan()
    fmt = 'bfloat16' if compute_dtype == 'bfloat16' else 'float32'
    assert [(op['kind'], op['dtype'], op['relu']) for op in plan['ops']] == [('dense_f', fmt, True), ('dense_f', fmt, False)]
    assert set(plan['formats'].values()) == {fmt}
    assert all(v.dtype == np.float32 for v in plan['params'].values())


def test_unknown_compute_dtype_is_rejected_and_integer_graphs_are_untouched():
    b, _ = _mlp('float16')
    with pytest.raises(ValueError, match="ComputeDtype='float16' is not recognised"):
        from_graph(b).export_plan()
    b2 = GraphBuilder({'Part': 'cuda_b200'}, name='int')
    x = b2.input('x', (4, 16), intent(8, 4))
    b2.output(b2.dense('fc', x, np.ones((16, 16)) / 8.0, intent(8, 6), intent(8, 3)))
    assert from_graph(b2).export_plan()['ops'][0]['kind'] == 'dense'


def test_bfloat16_bits_round_to_nearest_even():
    f = np.array([1.0, 1.00390625, 1.01171875, -2.5, 0.1, 3.0e38, 0.0], dtype=np.float32)   # 1 + 2^-8 is a tie
    bits = to_bf16_bits(f)
    back = from_bf16_bits(bits)
    assert back[0] == 1.0 and back[1] == 1.0 and back[2] == 1.015625 and back[3] == -2.5
    np.testing.assert_allclose(back, f, rtol=2 ** -8)
    np.testing.assert_array_equal(oracle.round_float(f, 'bfloat16'), back)


def test_fp8_e4m3_bits_round_to_nearest_even_and_saturate():
    """Activations enter and leave fp8 tensors by round-to-nearest-even with saturation at 448 (what the device's
    conversion does); checked against torch's float8_e4m3fn cast inside the finite range and against the oracle's
    independent nearest-value search everywhere."""
    import torch

    rng = np.random.default_rng(0)
    x = np.concatenate([rng.normal(0, 60, 50000), rng.normal(0, 0.01, 20000), np.linspace(-447.9, 447.9, 20001),
                        np.ldexp(np.arange(0, 33) / 2.0, -9), [0.0, -0.0, 448.0, 1.0625, 1.1875]]).astype(np.float32)
    bits = to_fp8_bits(x)
    np.testing.assert_array_equal(bits, torch.from_numpy(x).to(torch.float8_e4m3fn).view(torch.uint8).numpy())
    np.testing.assert_array_equal(from_fp8_bits(np.arange(256, dtype=np.uint8))[:0x7F],
                                  torch.arange(0x7F, dtype=torch.uint8).view(torch.float8_e4m3fn).float().numpy())
    beyond = np.array([449.0, 464.0, 480.0, 1e6, np.inf, -1e6, -np.inf], dtype=np.float32)
    np.testing.assert_array_equal(to_fp8_bits(beyond), [0x7E, 0x7E, 0x7E, 0x7E, 0x7E, 0xFE, 0xFE])
    assert to_fp8_bits(np.array([np.nan], dtype=np.float32))[0] & 0x7F == 0x7F
    wide = np.concatenate([x, beyond[np.isfinite(beyond)], rng.uniform(-600, 600, 5000).astype(np.float32)])
    np.testing.assert_array_equal(from_fp8_bits(to_fp8_bits(wide)), oracle.round_float(wide, 'fp8_e4m3'))
    assert from_fp8_bits(to_fp8_bits(np.float32(1.0625))) == 1.0 and from_fp8_bits(to_fp8_bits(np.float32(1.1875))) == 1.25


def _float_onnx_graph(tag, rng, batch=20):
    """Gemm + Relu -> MatMul -> Add(second input) with no Q/DQ nodes: a floating-point graph of element type `tag`."""
    from aie4ml_b200.frontends.onnx_import import OnnxGraph, OnnxNode

    consts = {'W0': rng.uniform(-0.5, 0.5, (32, 48)).astype(np.float32), 'b0': rng.uniform(-1, 1, 48).astype(np.float32),
              'W1': rng.uniform(-0.5, 0.5, (48, 16)).astype(np.float32)}
    g = OnnxGraph(
        nodes=[OnnxNode('Gemm', 'fc0', ['x', 'W0', 'b0'], ['h0']), OnnxNode('Relu', 'r0', ['h0'], ['h1']),
               OnnxNode('MatMul', 'fc1', ['h1', 'W1'], ['h2']), OnnxNode('Add', 'res', ['h2', 'z'], ['y'])],
        initializers=consts, inputs={'x': ((batch, 32), tag), 'z': ((batch, 16), tag)}, outputs=['y'], name='fnet',
        initializer_formats={} if tag is np.float32 else {k: tag for k in consts})
    return g, consts


@pytest.mark.parametrize('tag,fmt', [('float8_e4m3fn', 'fp8_e4m3'), ('bfloat16', 'bfloat16'), (np.float32, 'float32')])
def test_onnx_graph_without_qdq_lowers_to_the_float_kernels(tag, fmt):
    from aie4ml_b200 import from_onnx

    g, consts = _float_onnx_graph(tag, np.random.default_rng(5))
    model = from_onnx(g, {'Part': 'cuda_b200'})
    plan = model.export_plan()
    assert [(op['kind'], op['dtype']) for op in plan['ops']] == [('dense_f', fmt), ('dense_f', fmt), ('add_f', fmt)]
    assert plan['ops'][0]['relu'] and plan['ops'][0]['bias'] and not plan['ops'][1]['bias']
    assert set(plan['formats'].values()) == {fmt}
    prep = model.prepare_inputs({'x': np.ones((20, 32)), 'z': np.ones((20, 16))})
    assert prep['x'].dtype == {'fp8_e4m3': np.uint8, 'bfloat16': np.uint16, 'float32': np.float32}[fmt]
    # the plan's weights are the values the packed storage holds: fp8 keeps 3 mantissa bits
    w0 = plan['params']['fc0/weights']
    step = {'fp8_e4m3': 2.0 ** -3, 'bfloat16': 2.0 ** -7, 'float32': 1e-7}[fmt]
    np.testing.assert_allclose(w0, consts['W0'], rtol=step, atol=2.0 ** -10)
    if fmt == 'fp8_e4m3':
        assert np.array_equal(from_fp8_bits(to_fp8_bits(w0)), w0)


def test_onnx_integer_graph_input_without_qdq_is_rejected():
    from aie4ml_b200 import from_onnx
    from aie4ml_b200.frontends.onnx_import import OnnxGraph, OnnxNode

    g = OnnxGraph(nodes=[OnnxNode('MatMul', 'fc', ['x', 'W'], ['y'])], initializers={'W': np.ones((8, 8), np.float32)},
                  inputs={'x': ((4, 8), np.int8)}, outputs=['y'])
    with pytest.raises(ValueError, match='Use QDQ wrapping for integer inputs'):
        from_onnx(g, {'Part': 'cuda_b200'}).export_plan()


@pytest.mark.gpu
@pytest.mark.parametrize('tag,fmt', [('float8_e4m3fn', 'fp8_e4m3'), ('bfloat16', 'bfloat16')])
def test_onnx_float_graph_runs_within_one_step_of_the_storage_type(tag, fmt):
    """fp8_e4m3 / bfloat16 graphs from the ONNX front door against the oracle on the exported plan.  The accumulation
    order is not part of the contract, so a result may land on the neighbouring value of the storage type."""
    from aie4ml_b200 import from_onnx

    rng = np.random.default_rng(11)
    g, _ = _float_onnx_graph(tag, rng, batch=200)
    model = from_onnx(g, {'Part': 'cuda_b200'})
    model.compile()
    x, z = rng.normal(0, 1, (200, 32)).astype(np.float32), rng.normal(0, 2, (200, 16)).astype(np.float32)
    got = np.asarray(model.predict({'x': x, 'z': z}))
    assert got.dtype == np.float32 and got.shape == (200, 16)
    np.testing.assert_array_equal(got, oracle.round_float(got, fmt))          # every result is a value of the type
    stored = {'x': oracle.round_float(x, fmt), 'z': oracle.round_float(z, fmt)}
    (_, want), = oracle.run_plan(model.export_plan(), stored).items()
    step = 2.0 ** -3 if fmt == 'fp8_e4m3' else 2.0 ** -7
    np.testing.assert_allclose(got, want, rtol=step * 1.01, atol=2.0 ** -9)
    assert (got == want).mean() > 0.97


@pytest.mark.gpu
@pytest.mark.parametrize('compute_dtype', ['bfloat16', 'float32'])
def test_float_mlp_matches_the_float_model_within_the_reference_tolerances(compute_dtype):
    b, consts = _mlp(compute_dtype)
    model = from_graph(b)
    model.compile()
    x = np.random.default_rng(42).uniform(-2.0, 2.0, (4, 32)).astype(np.float32)
    got = np.asarray(model.predict(x))
    assert got.dtype == np.float32 and got.shape == (4, 16)
    np.testing.assert_allclose(got, _float_model(x.astype(np.float64), *consts), **TOL[compute_dtype])
    # and against the oracle evaluating the exported plan with each tensor's storage rounding
    (_, want), = oracle.run_plan(model.export_plan(), {'x': oracle.round_float(x, model.plan.fmt['x'])}).items()
    np.testing.assert_allclose(got, want, **TOL[compute_dtype])


@pytest.mark.gpu
@pytest.mark.parametrize('compute_dtype', ['bfloat16', 'float32'])
def test_float_matmul_add_and_larger_shapes(compute_dtype):
    rng = np.random.default_rng(7)
    b = GraphBuilder({'Part': 'cuda_b200', 'ComputeDtype': compute_dtype}, name='f2')
    q = b.input('q', (3, 70, 48), intent(16, 12))
    k = b.input('k', (3, 90, 48), intent(16, 12))
    kt = b.transpose('kt', k, [0, 2, 1])
    s = b.matmul('qk', q, kt, intent(16, 10))
    w = rng.normal(0, 0.1, (90, 40))
    d = b.dense('proj', s, w, intent(16, 12), intent(16, 10))
    d2 = b.dense('proj2', s, w * 0.5, intent(16, 12), intent(16, 10), relu=True)
    b.output(b.add('sum', d, d2, intent(16, 10)))
    model = from_graph(b)
    model.context.aie_config['Iterations'] = 2          # the streaming path with floating-point buffers
    model.compile()
    qa = rng.uniform(-1, 1, (2, 3, 70, 48)).astype(np.float32)
    ka = rng.uniform(-1, 1, (2, 3, 90, 48)).astype(np.float32)
    got = np.asarray(model.predict({'q': qa, 'k': ka}))
    s_ref = qa.astype(np.float64) @ np.swapaxes(ka.astype(np.float64), -1, -2)
    want = (s_ref @ w + np.maximum(s_ref @ (w * 0.5), 0.0)).reshape(got.shape)
    tol = dict(rtol=2e-2, atol=2e-1) if compute_dtype == 'bfloat16' else TOL['float32']   # three bf16 roundings in a row
    np.testing.assert_allclose(got, want, **tol)


@pytest.mark.gpu
def test_onnx_fp8_dynamic_matmul_with_a_transposed_operand():
    """Two fp8_e4m3 graph inputs, Transpose -> MatMul (a dynamic, batched product with a transposed right operand)
    followed by an Add with a third input; against the oracle on the exported plan, within one fp8 step."""
    from aie4ml_b200 import from_onnx
    from aie4ml_b200.frontends.onnx_import import OnnxGraph, OnnxNode

    rng = np.random.default_rng(31)
    g = OnnxGraph(
        nodes=[OnnxNode('Transpose', 'kt', ['k'], ['k_t'], {'perm': [0, 2, 1]}), OnnxNode('MatMul', 'qk', ['q', 'k_t'], ['s']),
               OnnxNode('Add', 'res', ['s', 'z'], ['y'])],
        initializers={}, inputs={'q': ((3, 40, 32), 'float8_e4m3fn'), 'k': ((3, 24, 32), 'float8_e4m3fn'),
                                 'z': ((3, 40, 24), 'float8_e4m3fn')}, outputs=['y'], name='f8mm')
    model = from_onnx(g, {'Part': 'cuda_b200'})
    model.compile()
    plan = model.export_plan()
    assert [(op['kind'], op['dtype']) for op in plan['ops']] == [('matmul_f', 'fp8_e4m3'), ('add_f', 'fp8_e4m3')]
    assert plan['ops'][0]['transpose_rhs'] and not plan['ops'][0]['transpose_lhs']
    x = {'q': rng.normal(0, 1, (3, 40, 32)).astype(np.float32), 'k': rng.normal(0, 1, (3, 24, 32)).astype(np.float32),
         'z': rng.normal(0, 4, (3, 40, 24)).astype(np.float32)}
    got = np.asarray(model.predict(x))
    stored = {n: oracle.round_float(v, 'fp8_e4m3') for n, v in x.items()}
    (_, want), = oracle.run_plan(plan, stored).items()
    np.testing.assert_array_equal(got, oracle.round_float(got, 'fp8_e4m3'))
    np.testing.assert_allclose(got, want.reshape(got.shape), rtol=2.0 ** -3 * 1.01, atol=2.0 ** -9)
    assert (got == want.reshape(got.shape)).mean() > 0.97
