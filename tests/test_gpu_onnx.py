"""int8 Q/DQ graphs through the ONNX front door on the GPU: ``from_onnx`` -> passes -> plan -> C ABI ->
``predict(dequantize_out=False)`` against the oracle evaluating the exported plan, bit for bit; and the
bit-exactness checker script with the reference script's arguments and seeded inputs."""

import numpy as np
import pytest

import onnx_graphs as OG
from aie4ml_b200 import from_onnx
from oracle import oracle

pytestmark = pytest.mark.gpu


def _run(graph, inputs, config, quantize_in=False):
    model = from_onnx(graph, config)
    model.compile()
    got = model.predict(inputs, quantize_in=quantize_in, dequantize_out=False)
    codes = {n: v[0] for n, v in model.prepare_inputs(inputs, iterations=1, quantize=quantize_in).items()}
    want = oracle.run_plan(model.export_plan(), codes)
    (name, ref), = want.items()
    np.testing.assert_array_equal(np.asarray(got), ref.astype(np.int64))
    return model


def test_cfg1_mlp_as_a_qdq_graph_integer_and_float_inputs():
    graph, inputs = OG.mlp_cfg1_onnx(1024)
    model = _run(graph, inputs, {'Part': 'cuda_b200'})
    # the ONNX path quantises with convergent rounding; the four Gemm + bias + ReLU layers still run as one kernel
    assert [op['kind'] for op in model.plan.ops] == ['mlp']
    assert all(l['rounding'] == 'conv_even' and l['shift'] == 7 and l['bias'] for l in model.plan.ops[0]['layers'])
    graph_f, inputs_f = OG.mlp_cfg1_onnx(1000, seed=5, float_input=True)
    _run(graph_f, inputs_f, {'Part': 'cuda_b200'}, quantize_in=True)


@pytest.mark.parametrize('softmax', ['exp', 'hccs'])
def test_cfg3_encoder_block_as_a_qdq_graph(softmax):
    graph, inputs, config = OG.encoder_cfg3_onnx(5, softmax)
    model = _run(graph, inputs, config)
    kinds = [op['kind'] for op in model.plan.ops]
    # same lowering as the programmatic graph: Q / K / V merged, the four heads fused into one attention launch,
    # wo / ffn2 with their residual Add and LayerNorm in one kernel each
    assert kinds.count('attention') == 1 and kinds.count('matmul') == 0 and kinds.count('softmax') == 0
    att = next(op for op in model.plan.ops if op['kind'] == 'attention')
    assert att['heads'] == 4 and att['rounding'] == 'conv_even'
    assert (att['sm_mode'] == 1 and att['exp_kq'] == 23) if softmax == 'exp' else (att['sm_mode'] == 0 and att['B'] == 200)
    assert model.plan.ops[0]['N'] == 768 and kinds.count('add') == 0 and kinds.count('dense_add_ln') == 2


def test_layer_directives_must_name_nodes_of_the_graph():
    graph, _inputs, config = OG.encoder_cfg3_onnx(2, 'exp')
    config = dict(config, LayerDirectives={'no_such_node': {'approximation': 'hccs'}})
    with pytest.raises(ValueError, match='no_such_node'):
        from_onnx(graph, config).run_pipeline()


@pytest.mark.parametrize('spec,batch', [('builtin:mlp_cfg1', 64), ('builtin:mlp_cfg1_float', 33),
                                        ('builtin:encoder_exp', 3), ('builtin:encoder_hccs', 2)])
def test_bit_exact_checker_script(spec, batch, capsys):
    import check_bit_exact

    assert check_bit_exact.main([spec, '--batch', str(batch), '--seed', '17', '--atol', '0']) == 0
    out = capsys.readouterr().out
    assert 'bit_exact' in out and 'MISMATCH' not in out
