"""Host logic: passes, variant selection, error behaviour, view planning, sharding."""

import numpy as np
import pytest

from aie4ml_b200 import CudaModel, GraphBuilder, from_graph, intent
from aie4ml_b200 import workloads as W
from aie4ml_b200.frontends.graph import lower_graph_dict
from aie4ml_b200.op_impls import get_family_resolver_registry, get_op_impl_registry
from aie4ml_b200.runtime import View, collapse_2d, collapse_batched, contiguous_strides, padded_pitch
from aie4ml_b200.sharding import shard_rows


def lowered(builder):
    return CudaModel.from_context(builder.finalize()).run_pipeline()


def test_registries_hold_the_cuda_variants_under_reference_op_types():
    reg = get_op_impl_registry()
    for op_type, vid in (('dense', 'dense.b.r.cuda.v1'), ('matmul', 'matmul.cuda.v1'), ('add', 'add.cuda.v1'),
                         ('layer_norm', 'layer_norm.i8.cuda.v1'), ('softmax', 'softmax.i8.cuda.v1')):
        ids = [v.variant_id for v in reg.candidates(op_type)]
        assert vid in ids
        # the float-simulation variants rank first (they match only floating-point tensors)
        assert ids == [vid] or ids == [vid.replace('cuda.v1', 'float.cuda.v1'), vid], ids
        get_family_resolver_registry().get(op_type)
    with pytest.raises(NotImplementedError):
        get_family_resolver_registry().get('conv2d')


def test_bias_and_relu_fold_into_dense():
    m = lowered(W.mlp_cfg1(8)[0])
    g = m.context.ir.logical
    assert [n.op_type for n in g.nodes] == ['dense'] * 4
    cfg = m.context.ir.execution.get('fc0').config
    assert cfg.flags.use_bias and cfg.flags.use_relu and cfg.shift == 7 and cfg.rounding_mode == 'positive_inf'
    assert not m.context.ir.execution.get('fc3').config.flags.use_relu


def test_scale_folds_into_softmax_temperature_or_matmul_shift():
    m = lowered(W.encoder_cfg3(1, 'exp')[0])
    ex = m.context.ir.execution
    assert ex.get('sm0').config.exp_kq == 23 and ex.get('qk0').config.shift == 9
    assert ex.get('qk0').config.flags.transpose_rhs and not ex.get('av0').config.flags.transpose_rhs
    assert ex.get('av0').config.precision['lhs'].format == 'uint8'
    with pytest.raises(ValueError, match='cannot apply a runtime input_scale'):
        b = GraphBuilder({'LayerDirectives': {'sm': {'approximation': 'hccs', 'hccs': {'B': 200, 'S': 3, 'Dmax': 66}}}})
        x = b.input('x', (4, 128), intent(8, 1))
        b.output(b.softmax('sm', b.scale('sc', x, 0.125), intent(8, 8, signed=False)))
        lowered(b)


def test_error_messages_name_the_node():
    b = GraphBuilder()
    x = b.input('x', (4, 100), intent(8, 4))
    b.output(b.softmax('soft', x, intent(8, 8, signed=False)))
    with pytest.raises(ValueError, match='soft: softmax axis length 100'):
        lowered(b)
    b = GraphBuilder()
    x = b.input('x', (4, 96), intent(8, 4))
    b.output(b.layer_norm('norm', x, np.ones(96), np.zeros(96), intent(8, 4), eps_q0=1))
    with pytest.raises(ValueError, match='norm: cols=96 must be a power of two'):
        lowered(b)
    b = GraphBuilder()
    x = b.input('x', (4, 64), intent(8, 4))
    y = b.input('y', (4, 64), intent(8, 5))
    b.output(b.add('plus', x, y, intent(8, 4)))
    with pytest.raises(ValueError, match='plus: elementwise Add requires lhs/rhs/output to use the same storage type'):
        lowered(b)
    b = GraphBuilder()
    x = b.input('x', (4, 64), intent(8, 4))
    b.output(b.scale('lonely', x, 0.5))
    with pytest.raises(NotImplementedError, match='lonely: no adjacent op absorbs this scale'):
        lowered(b)
    b = GraphBuilder()
    x = b.input('x', (4, 32), intent(8, 1))
    b.output(b.softmax('s', x, intent(8, 8, signed=False)))
    with pytest.raises(ValueError, match='s: exp Softmax needs 1 <= EXP_KQ <= 128'):
        lowered(b)
    b = GraphBuilder({'LayerDirectives': {'s': {'approximation': 'hccs', 'hccs': {'B': 300, 'S': 1, 'Dmax': 10}}}})
    x = b.input('x', (4, 128), intent(8, 4))
    b.output(b.softmax('s', x, intent(8, 8, signed=False)))
    with pytest.raises(ValueError, match='cols \\* B <= 32767'):
        lowered(b)


def test_unknown_directive_targets_and_parts_are_errors():
    b = GraphBuilder({'LayerDirectives': {'ghost': {'layout': 'tiled'}}})
    x = b.input('x', (4, 64), intent(8, 4))
    b.output(b.dense('fc', x, np.ones((64, 16)) / 64, intent(8, 6), intent(8, 4)))
    with pytest.raises(ValueError, match='ghost'):
        b.finalize()
    with pytest.raises(KeyError):
        GraphBuilder({'Part': 'xilinx_vek280_base_202520_1'})
    with pytest.raises(ValueError, match="use 'cuda'"):
        GraphBuilder({'AIEConfig': {'Target': 'hardware'}})
    # AIE-only directives are accepted and ignored
    b = GraphBuilder({'LayerDirectives': {'fc': {'parallelism': {'cas_num': 4, 'cas_length': 2}, 'layout': 'tiled'}}})
    x = b.input('x', (4, 64), intent(8, 4))
    b.output(b.dense('fc', x, np.ones((64, 16)) / 64, intent(8, 6), intent(8, 4)))
    assert lowered(b).context.ir.execution.get('fc').config.shift == 6


def test_dict_front_door_equals_builder():
    rng = np.random.default_rng(0)
    Wm = rng.integers(-127, 128, (16, 8)) / 128.0
    spec = {
        'name': 'tiny',
        'inputs': [{'name': 'x', 'shape': [4, 16], 'precision': {'width': 8, 'frac': 4}}],
        'params': {'w': {'data': Wm.tolist(), 'precision': {'width': 8, 'frac': 7}},
                   'b': {'data': [0.5] * 8, 'precision': {'width': 32, 'frac': 11}}},
        'nodes': [
            {'name': 'fc', 'op': 'dense', 'inputs': ['x', 'w'], 'roles': ['lhs', 'rhs'],
             'metadata': {'n_in': 16, 'n_out': 8, 'use_bias': False},
             'outputs': [{'name': 'pre', 'shape': [4, 8], 'precision': {'width': 8, 'frac': 4}}]},
            {'name': 'fc_bias', 'op': 'add', 'inputs': ['pre', 'b'], 'roles': ['lhs', 'rhs'],
             'outputs': [{'name': 'biased', 'shape': [4, 8], 'precision': {'width': 8, 'frac': 4}}]},
            {'name': 'act', 'op': 'activation', 'inputs': ['biased'], 'roles': ['lhs'], 'metadata': {'activation': 'relu'},
             'outputs': [{'name': 'y', 'shape': [4, 8], 'precision': {'width': 8, 'frac': 4}}]},
        ],
        'outputs': ['y'],
    }
    m = CudaModel.from_context(lower_graph_dict(spec, {'Part': 'cuda_b200'})).run_pipeline()
    cfg = m.context.ir.execution.get('fc').config
    assert cfg.shift == 7 and cfg.flags.use_bias and cfg.flags.use_relu and cfg.rounding_mode == 'conv_even'
    plan = m.export_plan()
    np.testing.assert_array_equal(plan['params']['fc/weights'], np.rint(Wm * 128))
    np.testing.assert_array_equal(plan['params']['fc/bias'], np.full(8, 1024))


def test_prepare_inputs_shapes_iterations_and_quantisation():
    b, inp = W.mlp_cfg1(4)
    m = from_graph(b)
    m.context.aie_config['Iterations'] = 3
    x = inp['x']
    assert m.prepare_inputs(x, iterations=3)['x'].shape == (3, 4, 16)
    assert m.prepare_inputs(x[None], iterations=3)['x'].shape == (3, 4, 16)
    with pytest.raises(ValueError, match='expected shape'):
        m.prepare_inputs(x[:2], iterations=3)
    with pytest.raises(ValueError, match='quantize=False requires integer inputs'):
        m.prepare_inputs(x.astype(np.float32), iterations=1, quantize=False)
    q = m.prepare_inputs(np.full((4, 16), 100.0), iterations=1)['x']
    assert q.dtype == np.int8 and (q == 127).all()          # 100 * 16 saturates
    q = m.prepare_inputs(np.full((4, 16), 0.09375), iterations=1)['x']
    assert (q == 2).all()                                     # 1.5 rounds half up to 2


def test_views_pitches_and_collapse():
    assert padded_pitch(5, 1) == 16 and padded_pitch(10, 1) == 16 and padded_pitch(1024, 1) == 1024
    assert padded_pitch(5, 2) == 8
    assert contiguous_strides((4, 128, 10), 1) == (128 * 16, 16, 1)
    head = View('qkv', 64, (7, 128, 64), (128 * 256, 256, 1), 'int8')
    assert collapse_2d(head, 't') == (64, 7 * 128, 64, 256)
    assert collapse_batched(head, 't') == (64, 7, 128, 64, 256, 128 * 256)
    with pytest.raises(NotImplementedError):
        collapse_2d(View('x', 0, (4, 8, 16), (300, 16, 1), 'int8'), 't')
    with pytest.raises(NotImplementedError):
        collapse_2d(View('x', 0, (4, 16), (1, 4), 'int8'), 't')


def test_shard_rows_partitions_exactly():
    for total, world in ((262144, 8), (10, 3), (5, 8), (0, 2)):
        spans = [shard_rows(total, r, world) for r in range(world)]
        assert spans[0][0] == 0 and spans[-1][1] == total
        assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
        sizes = [e - s for s, e in spans]
        assert max(sizes) - min(sizes) <= 1


def test_plan_dump_reads_back_and_the_oracle_runs_it(tmp_path):
    from aie4ml_b200.report import load_plan
    from oracle import oracle

    b, inp = W.mlp_cfg1(8)
    m = from_graph(b)
    m.dump(tmp_path)
    plan = load_plan(tmp_path)
    live = m.export_plan()
    assert [op['name'] for op in plan['ops']] == [op['name'] for op in live['ops']]
    for k, v in live['params'].items():
        np.testing.assert_array_equal(plan['params'][k], v)
    (name, want), = oracle.run_plan(live, inp).items()
    np.testing.assert_array_equal(oracle.run_plan(plan, inp)[name], want)
