"""Whole lowered graphs through the model API (front door -> passes -> plan -> C ABI) against the
oracle evaluating the exported plan, bit-exact, plus size-independent properties at larger sizes."""

import numpy as np
import pytest

from aie4ml_b200 import from_graph
from aie4ml_b200 import workloads as W
from oracle import oracle

pytestmark = pytest.mark.gpu


def _check(builder, inputs, **cfg):
    model = from_graph(builder)
    model.context.aie_config.update(cfg)
    model.compile()
    got = model.predict(inputs, quantize_in=False, dequantize_out=False)
    want = oracle.run_plan(model.export_plan(), inputs)
    (name, ref), = want.items()
    np.testing.assert_array_equal(np.asarray(got), ref.astype(np.int64))
    return model


@pytest.mark.parametrize('rounding', ['half_up', 'conv_even'])
def test_cfg1_mlp(rounding):
    model = _check(*W.mlp_cfg1(1024, rounding=rounding))
    # the four narrow layers run as one kernel; the three intermediates have no buffer
    assert [op['kind'] for op in model.plan.ops] == ['mlp'] and len(model.plan.buffers) == 2
    unfused = _check(*W.mlp_cfg1(1000, rounding=rounding), FusionPolicy={'dense_chain': False})
    assert [op['kind'] for op in unfused.plan.ops] == ['dense'] * 4


@pytest.mark.parametrize('shape', [(1024, 1024, 1024), (512, 4096, 1024), (256, 1024, 4096)])
def test_cfg2_dense(shape):
    _check(*W.dense_cfg2(*shape))


@pytest.mark.parametrize('softmax', ['exp', 'hccs'])
@pytest.mark.parametrize('rounding', ['half_up', 'conv_even'])
def test_cfg3_encoder_block(softmax, rounding):
    model = _check(*W.encoder_cfg3(3, softmax=softmax, rounding=rounding))
    kinds = [op['kind'] for op in model.plan.ops]
    # every head's QK^T -> softmax -> AV chain is fused and the four heads share one launch; scores and
    # probabilities have no buffer
    assert kinds.count('attention') == 1 and kinds.count('matmul') == 0 and kinds.count('softmax') == 0
    att = next(op for op in model.plan.ops if op['kind'] == 'attention')
    assert att['heads'] == 4 and att['head_strides'] == (64, 64, 64, 64)
    # the Q / K / V projections read the same tensor with the same requantisation: one Dense over 768 outputs
    assert model.plan.ops[0]['kind'] == 'dense' and model.plan.ops[0]['N'] == 768
    # wo and ffn2 are 256 wide and feed residual Add -> LayerNorm: each of the two chains is one kernel, and neither the
    # Dense output nor the sum has a buffer
    assert kinds == ['dense', 'attention', 'dense_add_ln', 'dense', 'dense_add_ln']
    assert not any(n.startswith(('qk', 'sm')) for n in model.plan.buffers)
    for op in model.plan.ops:
        if op['kind'] == 'dense_add_ln':
            assert op['dense']['out'] not in model.plan.buffers and op['dense']['N'] == 256
    two_step = _check(*W.encoder_cfg3(3, softmax=softmax, rounding=rounding), FusionPolicy={'dense_ln': False})
    kinds2 = [op['kind'] for op in two_step.plan.ops]
    # both residual Adds then ride inside their LayerNorm launches
    assert len(kinds2) == 7 and kinds2.count('layer_norm') == 2 and kinds2.count('add') == 0
    assert sum(1 for op in two_step.plan.ops if op.get('pre_addend')) == 2
    separate = _check(*W.encoder_cfg3(3, softmax=softmax, rounding=rounding), FusionPolicy={'parallel_dense': False})
    assert len(separate.plan.ops) == 7 and separate.plan.ops[0]['N'] == 256
    unfused = _check(*W.encoder_cfg3(3, softmax=softmax, rounding=rounding), FusionPolicy={'attention': False})
    kinds = [op['kind'] for op in unfused.plan.ops]
    assert kinds.count('matmul') == 8 and kinds.count('softmax') == 4 and kinds.count('attention') == 0


@pytest.mark.parametrize('op', ['layer_norm', 'softmax_exp', 'softmax_hccs'])
def test_cfg4_rowop_plus_add_fused_and_unfused(op):
    b, inp = W.rowops_cfg4(513, 1024, op)
    fused = _check(b, inp)
    assert len(fused.plan.launches) == 1 and fused.plan.fused
    b2, inp2 = W.rowops_cfg4(513, 1024, op)
    unfused = _check(b2, inp2, FusionPolicy={'rowop_add': False})
    assert len(unfused.plan.launches) == 2


def test_cfg5_wide_mlp_with_fanout_and_concat():
    model = _check(*W.wide_mlp_cfg5(300))
    # both branch tails write straight into the concat buffer: no copy kernel; the two first layers read the same
    # input and run as one Dense over 2048 outputs: 9 dense launches
    assert len(model.plan.launches) == 9 and model.plan.ops[0]['N'] == 2048
    assert len(_check(*W.wide_mlp_cfg5(300), FusionPolicy={'parallel_dense': False}).plan.launches) == 10
    assert model.plan.views['b0_fc3_out'].root == model.plan.views['b1_fc3_out'].root == 'cat_out'


def test_cuda_graph_replay_matches_eager():
    b, inp = W.encoder_cfg3(2, softmax='exp')
    model = from_graph(b)
    model.compile()
    eager = model.predict(inp, quantize_in=False, dequantize_out=False)
    model.plan.capture()
    replay = model.predict(inp, quantize_in=False, dequantize_out=False)
    np.testing.assert_array_equal(eager, replay)


def test_float_boundary_quantise_dequantise():
    b, inp = W.mlp_cfg1(64)
    model = from_graph(b)
    model.compile()
    xf = inp['x'].astype(np.float64) / 16.0
    yf = model.predict(xf)
    yi = model.predict(inp, quantize_in=False, dequantize_out=False)
    np.testing.assert_array_equal(yf, yi / 16.0)


def test_dense_linearity_property_at_scale():
    """With shift 0 and int16-free ranges the kernel is linear: Y(a1) + Y(a2) == Y(a1 + a2) when nothing
    saturates -- checked on a problem too large for the oracle to evaluate quickly."""
    import gpu_util as G

    rng = np.random.default_rng(5)
    M, K, N = 8192, 1024, 2048
    a1 = rng.integers(-3, 4, (M, K)).astype(np.int8)
    a2 = rng.integers(-3, 4, (M, K)).astype(np.int8)
    w = rng.integers(-1, 2, (K, N)).astype(np.int8)
    y1 = G.dense(a1, w, None, shift=0, tok='floor', relu=False, out_dtype='int8', algo=2).astype(np.int64)
    y2 = G.dense(a2, w, None, shift=0, tok='floor', relu=False, out_dtype='int8', algo=2).astype(np.int64)
    y12 = G.dense((a1 + a2).astype(np.int8), w, None, shift=0, tok='floor', relu=False, out_dtype='int8', algo=2).astype(np.int64)
    ok = (np.abs(y1 + y2) < 127) & (np.abs(y1) < 127) & (np.abs(y2) < 127) & (np.abs(y12) < 127)
    assert ok.mean() > 0.5
    np.testing.assert_array_equal((y1 + y2)[ok], y12[ok])
    # and the two GEMM kernels agree with each other everywhere
    ys = G.dense(a1, w, None, shift=0, tok='floor', relu=False, out_dtype='int8', algo=1)
    np.testing.assert_array_equal(ys, y1)


@pytest.mark.parametrize('depth', [1, 3])
def test_host_pipeline_streams_a_ragged_batch_bit_exact(depth):
    """A host batch of 3.4 chunks through the three-stream pipeline equals the oracle on the same
    rows, for a multi-launch graph (encoder block) and every slot/graph-replay combination."""
    import torch

    b, inp = W.encoder_cfg3(2, softmax='hccs')
    model = from_graph(b)
    model.compile()
    pipe = model.pipeline(depth)
    (in_name, x), = inp.items()
    rows = 2 * 3 + 1                                      # 3 full chunks of 2 + one half-filled chunk
    rng = np.random.default_rng(5)
    big = rng.integers(-128, 128, size=(rows, *x.shape[1:]), dtype=np.int64).astype(x.dtype)
    host_in = {in_name: torch.from_numpy(big).pin_memory()}
    out_name = pipe.out_names[0]
    t = model.plan.tensor_of(out_name)
    host_out = {out_name: torch.zeros((rows, *t.shape[1:]), dtype=t.dtype).pin_memory()}
    assert pipe.run_and_wait(host_in, host_out) == 4
    plan = model.export_plan()
    for c in range(4):
        chunk = np.zeros_like(x)
        n = min(2, rows - 2 * c)
        chunk[:n] = big[2 * c: 2 * c + n]
        (_, want), = oracle.run_plan(plan, {in_name: chunk}).items()
        np.testing.assert_array_equal(host_out[out_name][2 * c: 2 * c + n].numpy(), want[:n])
    # a second run over the same buffers (events and slots reused) gives the same bytes
    first = host_out[out_name].clone()
    host_out[out_name].zero_()
    pipe.run_and_wait(host_in, host_out)
    assert torch.equal(first, host_out[out_name])


def test_predict_with_iterations_uses_the_pipeline_and_matches_single_runs():
    b, inp = W.mlp_cfg1(256)
    model = from_graph(b)
    model.context.aie_config['Iterations'] = 5
    model.compile()
    rng = np.random.default_rng(9)
    x = rng.integers(-128, 128, size=(5, *inp['x'].shape), dtype=np.int64).astype(inp['x'].dtype)
    got = model.predict(x, quantize_in=False, dequantize_out=False)
    plan = model.export_plan()
    want = np.concatenate([next(iter(oracle.run_plan(plan, {'x': x[i]}).values())) for i in range(5)], axis=0)
    np.testing.assert_array_equal(np.asarray(got), want.astype(np.int64))
    assert model._pipeline is not None


def test_report_times_every_launch_and_names_the_bound():
    from aie4ml_b200.report import format_rows, profile_plan

    b, _ = W.encoder_cfg3(8, softmax='exp')
    model = from_graph(b)
    model.compile()
    rows = profile_plan(model.plan, iters=3)
    assert len(rows) == len(model.plan.launches) and all(r['ms'] > 0 and r['bytes'] > 0 for r in rows)
    kinds = {r['kind'] for r in rows}
    assert {'dense', 'attention', 'dense_add_ln'} <= kinds
    assert all(r['bound'] == 'hbm' for r in rows if r['kind'] == 'dense_add_ln')
    text = format_rows(rows)
    assert 'sum of launches' in text and 'attention' in text
    model.context.aie_config['FusionPolicy'] = {'dense_ln': False}
    model.plan = None
    model.compile()
    rows = profile_plan(model.plan, iters=3)
    assert len(rows) == 7 and all(r['bound'] == 'hbm' for r in rows if r['kind'] == 'layer_norm')


def test_model_with_a_dense_over_a_transposed_input_view():
    """Transpose -> Dense: the transpose folds into the Dense's input view (TRANSPOSE_INPUT in the reference) and
    the kernel reads the stored [K, M] matrices; a second ordinary Dense follows."""
    from aie4ml_b200.frontends.graph import GraphBuilder, intent

    rng = np.random.default_rng(17)
    b = GraphBuilder({'Part': 'cuda_b200'}, name='dense_ta')
    x = b.input('x', (6, 48, 20), intent(8, 4))
    xt = b.transpose('xt', x, [0, 2, 1])
    h = b.dense('fc0', xt, rng.uniform(-1, 1, (48, 24)), intent(8, 6), intent(8, 3), bias=rng.uniform(-1, 1, 24),
                bias_precision=intent(16, 8), relu=True)
    y = b.dense('fc1', h, rng.uniform(-1, 1, (24, 16)), intent(8, 6), intent(8, 3))
    b.output(y)
    model = _check(b, {'x': rng.integers(-128, 128, (6, 48, 20)).astype(np.int8)})
    assert model.plan.ops[0]['transpose_lhs'] and not model.plan.ops[1]['transpose_lhs']


def test_parallel_dense_merge_with_and_without_bias_and_unequal_widths():
    """Three Dense layers read the same tensor with the same requantisation (one has no bias, widths 32 / 48 / 16):
    they run as one Dense over 96 outputs whose column slices are the three results; a fourth with a ReLU
    and a fifth whose width is not a multiple of 16 stay separate.  Every consumer reads its slice."""
    from aie4ml_b200.frontends.graph import GraphBuilder, intent

    rng = np.random.default_rng(23)
    b = GraphBuilder({'Part': 'cuda_b200'}, name='fanout')
    x = b.input('x', (70, 64), intent(8, 4))
    a0 = b.dense('a0', x, rng.uniform(-1, 1, (64, 32)), intent(8, 6), intent(8, 3), bias=rng.uniform(-1, 1, 32),
                 bias_precision=intent(16, 8))
    a1 = b.dense('a1', x, rng.uniform(-1, 1, (64, 48)), intent(8, 6), intent(8, 3))
    a2 = b.dense('a2', x, rng.uniform(-1, 1, (64, 16)), intent(8, 6), intent(8, 3), bias=rng.uniform(-1, 1, 16),
                 bias_precision=intent(16, 8))
    other = b.dense('other', x, rng.uniform(-1, 1, (64, 32)), intent(8, 6), intent(8, 3), relu=True)   # another epilogue
    odd = b.dense('odd', x, rng.uniform(-1, 1, (64, 24)), intent(8, 6), intent(8, 3))          # 24 is not 16-aligned
    s0 = b.add('s0', a0, other, intent(8, 3))
    y0 = b.dense('y0', s0, rng.uniform(-1, 1, (32, 16)), intent(8, 6), intent(8, 3))
    y1 = b.dense('y1', a1, rng.uniform(-1, 1, (48, 16)), intent(8, 6), intent(8, 3))
    y2 = b.dense('y2', odd, rng.uniform(-1, 1, (24, 16)), intent(8, 6), intent(8, 3))
    t = b.add('t0', y0, y1, intent(8, 3))
    t = b.add('t1', t, y2, intent(8, 3))
    b.output(b.add('t2', t, a2, intent(8, 3)))
    model = _check(b, {'x': rng.integers(-128, 128, (70, 64)).astype(np.int8)})
    merged = [op for op in model.plan.ops if op['kind'] == 'dense' and op['N'] == 96]
    assert len(merged) == 1 and merged[0]['name'] == 'a0|a1|a2' and merged[0]['bias']
    assert model.plan.views['a1_out'].root == model.plan.views['a0_out'].root == model.plan.views['a2_out'].root
    assert model.plan.views['a1_out'].offset == 32 and model.plan.views['a2_out'].offset == 80
    assert {op['name'] for op in model.plan.ops if op['kind'] == 'dense'} >= {'other', 'odd', 'y0', 'y1', 'y2'}


def test_model_with_16_bit_activations_and_weights():
    """A three-layer network whose first two layers keep 16-bit activations: int16 x int8 (acc32) into int16,
    int16 x int16 (acc64) into int8, then an ordinary int8 layer; against the oracle on the exported plan."""
    from aie4ml_b200.frontends.graph import GraphBuilder, intent

    rng = np.random.default_rng(3)
    b = GraphBuilder({'Part': 'cuda_b200'}, name='wide')
    x = b.input('x', (50, 48), intent(16, 8))
    h1 = b.dense('fc0', x, rng.uniform(-1, 1, (48, 40)), intent(8, 6), intent(16, 9), bias=rng.uniform(-1, 1, 40),
                 bias_precision=intent(32, 14), relu=True)
    h2 = b.dense('fc1', h1, rng.uniform(-1, 1, (40, 32)), intent(16, 13), intent(8, 4))
    y = b.dense('fc2', h2, rng.uniform(-1, 1, (32, 10)), intent(8, 6), intent(8, 3))
    b.output(y)
    xin = rng.integers(-32768, 32768, (50, 48)).astype(np.int16)
    model = _check(b, {'x': xin})
    ops = model.plan.ops
    assert [op['kind'] for op in ops] == ['dense', 'dense', 'dense']
    assert (ops[0]['lhs_dtype'], ops[0]['rhs_dtype'], ops[0]['acc_bits'], ops[0]['out_dtype']) == ('int16', 'int8', 32, 'int16')
    assert (ops[1]['lhs_dtype'], ops[1]['rhs_dtype'], ops[1]['acc_bits']) == ('int16', 'int16', 64)
