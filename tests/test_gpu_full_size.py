"""Parity at the sizes the benchmark times.

The device computes the WHOLE batch of each benchmark configuration at its full size (Dense M up to 131072 with
K = N up to 8192: 64 k-blocks per tile and ~220 tiles per CTA; 4096 sequences of the encoder block; 2^20 rows of the
row ops; 262144 rows of the wide MLP), and a few hundred sampled units -- first, last, both sides of tile boundaries,
spread over the batch -- are compared bit for bit with the CPU oracle evaluating the exported plan on the same
inputs (every operator is independent along the leading axis, so the oracle's result on a subset equals the subset
of its result).  Both rounding modes the configurations are quoted in: round-half-up and the reference ONNX path's
convergent rounding.
"""

import numpy as np
import pytest

from aie4ml_b200 import from_graph
from aie4ml_b200 import workloads as W
from oracle import checker

pytestmark = pytest.mark.gpu


@pytest.fixture(scope='module')
def c_oracle():
    lib, _ = checker.load_c(native=True)
    return lib


def _sampled_parity(builder, inputs, n_units, lib, expect_launches=None):
    import torch

    model = from_graph(builder)
    model.compile()
    plan = model.plan
    graph = model.context.ir.logical
    for n in graph.input_tensor_names:
        plan.tensor_of(n).copy_(torch.from_numpy(np.ascontiguousarray(inputs[n])).to(plan.device))
    plan.run()
    plan.check_status()
    total = int(next(iter(inputs.values())).shape[0])
    units = checker.sample_units(total, n_units, tile=128, seed=total % 9973)
    idx = torch.from_numpy(units).to(plan.device)
    got = {n: plan.tensor_of(n).index_select(0, idx).cpu().numpy() for n in graph.output_tensor_names}
    res = checker.check_sample(model.export_plan(), inputs, got, units, lib=lib)
    assert res['rows_checked'] >= min(total, n_units) and res['values_checked'] > 0
    assert res['mismatches'] == 0, res
    if expect_launches is not None:
        assert len(plan.launches) == expect_launches
    # something other than zeros came out
    assert any(np.abs(v.astype(np.int64)).max() > 0 for v in got.values())
    del plan, model
    torch.cuda.empty_cache()


@pytest.mark.parametrize('rounding', ['half_up', 'conv_even'])
@pytest.mark.parametrize('kn', [1024, 4096, 8192])
@pytest.mark.parametrize('m', [1024, 16384, 131072])
def test_dense_sweep_every_point_at_full_size(m, kn, rounding, c_oracle):
    _sampled_parity(*W.dense_cfg2(m, kn, kn, rounding=rounding), 256, c_oracle, expect_launches=1)


@pytest.mark.parametrize('rounding', ['half_up', 'conv_even'])
@pytest.mark.parametrize('softmax', ['exp', 'hccs'])
def test_encoder_block_4096_sequences(softmax, rounding, c_oracle):
    _sampled_parity(*W.encoder_cfg3(4096, softmax=softmax, rounding=rounding), 6, c_oracle)


@pytest.mark.parametrize('rounding', ['half_up', 'conv_even'])
@pytest.mark.parametrize('op', ['layer_norm', 'softmax_exp', 'softmax_hccs'])
def test_row_ops_2_pow_20_rows(op, rounding):
    _sampled_parity(*W.rowops_cfg4(1 << 20, 1024, op, rounding=rounding), 512, None, expect_launches=1)


@pytest.mark.parametrize('rounding', ['half_up', 'conv_even'])
def test_wide_mlp_262144_rows(rounding, c_oracle):
    _sampled_parity(*W.wide_mlp_cfg5(262144, rounding=rounding), 256, c_oracle, expect_launches=9)
