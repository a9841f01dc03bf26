"""The package's lowering must make the same numeric decisions as the reference's own Python code.

``tests/golden/reference_contracts.json`` was produced by importing the reference and running its
passes on the cases of ``tests/golden/cases.py`` (see ``make_golden.py``)."""

import json
from pathlib import Path

import numpy as np
import pytest

from aie4ml_b200.model import CudaModel
from aie4ml_b200.op_impls.precision import ROUNDING_TOKEN_MAP
from aie4ml_b200.qtypes import RoundingMode, SaturationMode
from aie4ml_b200.quant_utils import quantize_to_int
from cases import CASES
from oracle import oracle

FIXTURE = json.loads((Path(__file__).parent / 'golden' / 'reference_contracts.json').read_text())


def test_rounding_token_map_matches_reference():
    ref = FIXTURE['rounding_token_map']
    mine = {k.name: v for k, v in ROUNDING_TOKEN_MAP.items() if k.name in ref}
    assert mine == ref
    assert set(ref) == {m.name for m in RoundingMode if m is not RoundingMode.RND_HALF_UP}


@pytest.mark.parametrize('case', sorted(CASES))
def test_lowering_matches_reference(case):
    ref = FIXTURE['cases'][case]
    model = CudaModel.from_context(CASES[case]().finalize()).run_pipeline()
    ctx = model.context
    graph = ctx.ir.logical
    assert [n.name for n in graph.nodes] == ref['node_order']
    assert [n.name for n in graph.nodes if n.is_placeholder] == ref['placeholders']
    assert sorted(graph.tensors) == ref['tensors']
    for name, want in ref['nodes'].items():
        inst = ctx.ir.execution.get(name)
        assert inst is not None, name
        cfg = inst.config
        assert inst.op_type == want['op_type']
        for key in ('shift', 'rounding_mode', 'accumulator_tag', 'exp_kq', 'inv_shift', 'use_clb', 'approximation',
                    'eps_q0', 'out_shift', 'gamma_shift', 'param_sets'):
            if key in want:
                assert getattr(cfg, key) == want[key], (name, key)
        if 'flags' in want:
            for f, v in want['flags'].items():
                assert bool(getattr(cfg.flags, f)) == v, (name, f)
        for role, d in want['precision'].items():
            if role in ('B', 'S', 'Dmax'):
                continue
            got = cfg.precision[role]
            assert got.format == d['format'] and got.frac == d['frac'], (name, role)
            if role != 'acc':
                assert got.rounding.name == d['rounding'] and got.saturation.name == d['saturation'], (name, role)
        if want['op_type'] == 'dense':
            np.testing.assert_array_equal(inst.artifacts['weights_kn'], np.array(want['weights']))
            packed = inst.artifacts['packed_weights']
            K, N = inst.artifacts['weights_kn'].shape
            np.testing.assert_array_equal(packed[:, :K].T, np.array(want['weights']))
            assert not packed[:, K:].any()
            if want['bias'] is None:
                assert inst.artifacts['packed_bias'] is None
            else:
                np.testing.assert_array_equal(inst.artifacts['packed_bias'], np.array(want['bias']))
        if want['op_type'] == 'layer_norm':
            np.testing.assert_array_equal(inst.artifacts['packed_gamma'], np.array(want['gamma']))
            np.testing.assert_array_equal(inst.artifacts['packed_beta'], np.array(want['beta']))
        if 'hccs' in want:
            op = inst.variant.plan_op(inst)
            assert {k: op[k] for k in ('B', 'S', 'Dmax')} == want['hccs']


def test_host_quantizer_matches_reference():
    q = FIXTURE['quantizer']
    values = np.array(q['values'])
    assert len(q['cases']) == 7 * 4 * 3
    for c in q['cases']:
        mine = quantize_to_int(values, c['frac'], c['width'], signed=c['signed'],
                               rounding_mode=RoundingMode[c['rounding']], saturation_mode=SaturationMode[c['saturation']])
        np.testing.assert_array_equal(mine.astype(np.int64), np.array(c['codes']), err_msg=str(c)[:80])
        orc = oracle.quantize(values, frac=c['frac'], width=c['width'], signed=c['signed'], rounding=c['rounding'],
                              saturation=c['saturation'])
        np.testing.assert_array_equal(orc, np.array(c['codes']), err_msg='oracle ' + str(c)[:80])


def test_float_constant_packer_matches_reference():
    """Weights of the floating-point Dense are packed by the reference's own rule (truncation for bfloat16, its
    half-up-on-magnitude scheme for fp8_e4m3), pinned on 590 recorded float32 bit patterns."""
    from aie4ml_b200.quant_utils import pack_constant_float

    rec = FIXTURE['float_packer']
    vals = np.array(rec['bits'], dtype=np.uint32).view(np.float32)
    assert len(vals) > 500
    for fmt in ('fp8_e4m3', 'bfloat16'):
        np.testing.assert_array_equal(pack_constant_float(vals, fmt).astype(np.int64), np.array(rec[fmt]), err_msg=fmt)
