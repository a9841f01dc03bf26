"""Generates ``reference_contracts.json``: numeric decisions of the REFERENCE's own Python code.

Run in a container where the reference checkout is present:

    PYTHONPATH=<reference>/src python tests/golden/make_golden.py <reference>/src

It imports the reference (numpy + jinja2 only), rebuilds each case of ``cases.py`` in the reference's
IR classes, runs the reference's FoldBias / FoldScale / FuseActivationCasts / FoldViewOps / Resolve /
PackKernelArtifacts passes, and records per node: shift, rounding token, accumulator tag, flags,
resolved dtypes, softmax / layernorm constants, and the quantised integer constants.  It also records
the reference's host quantiser (apply_rounding + handle_overflow) on seeded float vectors for every
rounding x saturation mode.  The fixture is committed; the tests never import the reference.
"""

from __future__ import annotations

import json
import sys
import tempfile
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent.parent))
if len(sys.argv) > 1:
    sys.path.insert(0, sys.argv[1])

from aie4ml.aie_types import QuantIntent as RefIntent  # noqa: E402
from aie4ml.aie_types import RoundingMode as RefRounding  # noqa: E402
from aie4ml.aie_types import SaturationMode as RefSaturation  # noqa: E402
from aie4ml.frontends.onnx.utils import create_context  # noqa: E402
from aie4ml.ir.graph import OpNode as RefNode  # noqa: E402
from aie4ml.ir.graph import TensorVar as RefTensor  # noqa: E402
from aie4ml.op_impls.families.matmul.common import quantize_to_int as ref_quantize_to_int  # noqa: E402
from aie4ml.passes import (  # noqa: E402
    FoldBias,
    FoldScale,
    FoldViewOps,
    FuseActivationCasts,
    PackKernelArtifacts,
    Resolve,
)
from aie4ml.passes.base import run_aie_passes  # noqa: E402

from cases import CASES  # noqa: E402


def to_ref_intent(p):
    if p is None:
        return None
    return RefIntent(width=p.width, frac=p.frac, signed=p.signed, rounding=RefRounding[p.rounding.name],
                     saturation=RefSaturation[p.saturation.name])


def rebuild_in_reference(ctx_mine):
    """Copy a pre-lowering logical IR of this package into the reference's IR classes."""
    ctx = create_context({'Part': 'xilinx_vek280_base_202520_1', 'AIEConfig': {'BatchSize': 8, 'Iterations': 1}},
                         tempfile.mkdtemp(), 'golden', None, None)
    g = ctx.ir.logical
    mine = ctx_mine.ir.logical
    tensors = {}
    for name, t in mine.tensors.items():
        prec = to_ref_intent(t.precision)
        if t.is_parameter and prec is None:
            # LayerNorm scale / bias arrive as float32 initializers in the ONNX path
            from aie4ml.aie_types import FloatFormat, FloatIntent
            prec = FloatIntent(width=32, format=FloatFormat.FP32)
        rt = RefTensor(name=name, shape=tuple(t.shape), precision=prec,
                       data=None if t.data is None else np.array(t.data, dtype=np.float64))
        tensors[name] = rt
        g.add_tensor(rt)
    for node in mine.nodes:
        rn = RefNode(name=node.name, op_type=node.op_type, dialect=ctx.device.dialect)
        rn.metadata.update(node.metadata)
        rn.directives.update(node.directives)
        rn.roles = dict(node.roles)
        for t in node.inputs:
            rn.inputs.append(tensors[t.name])
            tensors[t.name].consumers.append(rn)
        for t in node.outputs:
            rn.outputs.append(tensors[t.name])
            tensors[t.name].producer = rn
        g.add_node(rn)
    for n in mine.input_tensor_names:
        g.mark_graph_input(n)
    for n in mine.output_tensor_names:
        g.mark_graph_output(n)
    return ctx


def dtype_dict(d):
    return {'format': d.format, 'frac': int(d.frac), 'rounding': d.rounding.name, 'saturation': d.saturation.name}


def record_case(name):
    builder = CASES[name]()
    ctx = rebuild_in_reference(builder.finalize())
    run_aie_passes(ctx, [FoldBias(), FoldScale(), FuseActivationCasts(), FoldViewOps(), Resolve(), PackKernelArtifacts()])
    nodes = {}
    for inst in ctx.ir.execution:
        cfg = inst.config
        rec = {'op_type': inst.op_type, 'variant_id': inst.variant.variant_id,
               'precision': {k: dtype_dict(v) for k, v in cfg.precision.items() if hasattr(v, 'format')}}
        for key in ('shift', 'rounding_mode', 'accumulator_tag', 'exp_kq', 'inv_shift', 'use_clb', 'approximation',
                    'eps_q0', 'out_shift', 'gamma_shift', 'param_sets'):
            if hasattr(cfg, key):
                rec[key] = getattr(cfg, key)
        if hasattr(cfg, 'flags'):
            rec['flags'] = {f: bool(getattr(cfg.flags, f)) for f in cfg.flags.__dataclass_fields__}
        if inst.op_type == 'dense':
            W, b, _, _ = inst.variant._quantize_weight_bias(inst)
            rec['weights'] = np.asarray(W).astype(int).tolist()
            rec['bias'] = None if b is None else np.asarray(b).astype(int).tolist()
        if inst.op_type == 'layer_norm':
            rec['gamma'] = np.asarray(inst.artifacts['packed_gamma'])[0].astype(int).tolist()
            rec['beta'] = np.asarray(inst.artifacts['packed_beta'])[0].astype(int).tolist()
        if inst.op_type == 'softmax' and cfg.approximation == 'hccs':
            rec['hccs'] = {k: int(np.asarray(cfg.hccs[k]).reshape(-1)[0]) for k in ('B', 'S', 'Dmax')}
        nodes[inst.name] = rec
    g = ctx.ir.logical
    return {'nodes': nodes, 'node_order': [n.name for n in g.nodes],
            'placeholders': [n.name for n in g.nodes if n.is_placeholder],
            'tensors': sorted(g.tensors)}


def record_quantizer():
    rng = np.random.default_rng(99)
    values = np.concatenate([rng.uniform(-3.0, 3.0, 48), np.array([-2.5, -1.5, -0.5, 0.5, 1.5, 2.5, 0.0, 1.984375,
                                                                  -2.0, 1.9921875, 300.0, -300.0])])
    out = {'values': values.tolist(), 'cases': []}
    for rounding in RefRounding:
        for sat in RefSaturation:
            for width, frac, signed in ((8, 6, True), (8, 5, False), (16, 9, True)):
                q = ref_quantize_to_int(values, frac, width, signed=signed, rounding_mode=rounding, saturation_mode=sat)
                out['cases'].append({'rounding': rounding.name, 'saturation': sat.name, 'width': width, 'frac': frac,
                                     'signed': signed, 'codes': np.asarray(q).astype(int).tolist()})
    return out


def record_float_packer():
    """The reference's constant packer for floating-point weights (pack_as_float) on float32 bit patterns that cover
    every fp8 exponent, ties, the subnormal range, the saturation threshold and non-finite inputs."""
    from aie4ml.aie_types import FloatFormat
    from aie4ml.op_impls.families.matmul.common import pack_as_float

    rng = np.random.default_rng(7)
    vals = np.concatenate([
        rng.normal(0, 1, 160), rng.normal(0, 60, 160), rng.normal(0, 0.004, 160),
        np.ldexp(1.0 + np.arange(0, 16) / 16.0, -8), np.ldexp(1.0 + np.arange(0, 16) / 16.0, 3),
        np.ldexp(np.arange(0, 33) / 2.0, -9),                       # every subnormal step and its midpoints
        np.array([0.0, -0.0, 448.0, 463.9, 464.0, 480.0, 511.9, 512.0, 600.0, -600.0, 1e9, np.inf, -np.inf,
                  2.0 ** -10, 2.0 ** -11, 3 * 2.0 ** -11, 1.0 + 2.0 ** -4, 1.0 + 3 * 2.0 ** -4])]).astype(np.float32)
    return {'bits': vals.view(np.uint32).astype(int).tolist(),
            'fp8_e4m3': np.asarray(pack_as_float(vals, FloatFormat.FP8_E4M3)).astype(int).tolist(),
            'bfloat16': np.asarray(pack_as_float(vals, FloatFormat.BF16)).astype(int).tolist()}


def main():
    from aie4ml.op_impls.utils.precision import ROUNDING_TOKEN_MAP

    fixture = {
        'rounding_token_map': {k.name: v for k, v in ROUNDING_TOKEN_MAP.items()},
        'cases': {name: record_case(name) for name in CASES},
        'quantizer': record_quantizer(),
        'float_packer': record_float_packer(),
    }
    path = HERE / 'reference_contracts.json'
    path.write_text(json.dumps(fixture, separators=(',', ':')))
    print(f'wrote {path} ({path.stat().st_size} bytes)')


if __name__ == '__main__':
    main()
