#!/usr/bin/env python
"""Bit-exactness check of an ONNX Q/DQ model on the CUDA target against the CPU oracle.

The counterpart of the reference's ``scripts/check_onnx_bit_exact.py:114-181``, with the same arguments and the
same seeded inputs (integers uniform in [-96, 96] clipped to the input type, floats uniform in [-1, 1), seed 17):
``from_onnx`` -> ``compile`` -> ``predict(..., dequantize_out=False)``, compared per graph output as integer
codes.  Where the reference's golden is ONNX Runtime evaluating the float Q/DQ graph (hence its default ``--atol 1``
for the float32 rounding of that path), the golden here is the integer oracle evaluating the exported lowered
plan, so the default tolerance is 0.

    python tests/check_bit_exact.py MODEL [--batch N] [--seed 17] [--atol 0] [--config cfg.json]
                                          [--quantize-in | --no-quantize-in]

MODEL is a path to an ``.onnx`` file (needs the ``onnx`` package), or ``builtin:NAME`` for one of the graph
descriptions in ``tests/onnx_graphs.py`` (mlp_cfg1, mlp_cfg1_float, encoder_exp, encoder_hccs), which need no
``onnx`` package.  Lives under ``tests/`` because it runs the oracle, which the shipped package never imports.
"""

from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent.parent
for p in (str(ROOT), str(ROOT / 'tests')):
    if p not in sys.path:
        sys.path.insert(0, p)


def seeded_feeds(graph_inputs, batch: int, seed: int):
    """name -> array, drawn as the reference script draws them (``check_onnx_bit_exact.py:71-85``)."""
    rng = np.random.default_rng(seed)
    feeds = {}
    for name, (shape, dtype) in graph_inputs.items():
        shape = [batch if (d is None or int(d) <= 0) else int(d) for d in shape]
        dt = np.dtype(dtype)
        if np.issubdtype(dt, np.floating):
            value = (rng.random(shape, dtype=np.float32) * 2.0) - 1.0
        else:
            info = np.iinfo(dt)
            value = rng.integers(max(info.min, -96), min(info.max, 96) + 1, size=shape, dtype=dt)
        feeds[name] = np.asarray(value, dtype=dt)
    return feeds


def load_model(spec: str, batch: int, seed: int, config_path):
    """-> (graph description or path, config dict, graph inputs {name: (shape, dtype)})"""
    from aie4ml_b200.frontends import onnx_import as OI

    config = {} if config_path is None else json.loads(Path(config_path).read_text())
    if spec.startswith('builtin:'):
        import onnx_graphs as OG

        name = spec.split(':', 1)[1]
        if name not in OG.BUILTIN:
            raise SystemExit(f'unknown builtin graph {name!r}; choose from {sorted(OG.BUILTIN)}')
        graph, _inputs, cfg = OG.BUILTIN[name](batch, seed)
        cfg = dict(cfg)
        cfg.update(config)
        return graph, cfg, graph.inputs
    OI.require_onnx()
    import onnx

    proto = onnx.load(spec)
    for vi in list(proto.graph.input) + list(proto.graph.output) + list(proto.graph.value_info):
        for axis, dim in enumerate(vi.type.tensor_type.shape.dim):
            if dim.dim_param or not dim.HasField('dim_value'):
                if axis != 0:
                    raise ValueError(f'{vi.name}: only a dynamic batch dimension is supported; axis {axis} is dynamic.')
                dim.ClearField('dim_param')
                dim.dim_value = int(batch)
    graph = OI.graph_from_proto(proto)
    config.setdefault('Part', 'cuda_b200')
    return graph, config, graph.inputs


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description='Compare CUDA-target outputs of an ONNX Q/DQ model with the CPU oracle.')
    ap.add_argument('model', help="path to the ONNX model, or builtin:NAME")
    ap.add_argument('--part', default='cuda_b200')
    ap.add_argument('--batch', type=int, default=1)
    ap.add_argument('--seed', type=int, default=17)
    ap.add_argument('--config', type=Path, help='JSON compiler config, including optional LayerDirectives')
    ap.add_argument('--quantize-in', action=argparse.BooleanOptionalAction, default=None,
                    help='override input quantization; default: true for float inputs, false for integer inputs')
    ap.add_argument('--atol', type=int, default=0, help='accepted integer tolerance (default 0: bit-exact)')
    args = ap.parse_args(argv)

    from aie4ml_b200 import from_onnx
    from aie4ml_b200 import quant_utils as Q
    from oracle import oracle

    graph, config, graph_inputs = load_model(args.model, args.batch, args.seed, args.config)
    config['Part'] = args.part
    aie = dict(config.get('AIEConfig', {}))
    aie.update({'BatchSize': int(args.batch), 'Iterations': 1})
    config['AIEConfig'] = aie
    model = from_onnx(graph, config)
    model.compile()
    feeds = seeded_feeds(graph_inputs, args.batch, args.seed)
    floats = [n for n, v in feeds.items() if np.issubdtype(v.dtype, np.floating)]
    if args.quantize_in is None:
        if floats and len(floats) != len(feeds):
            raise ValueError('mixed float/integer graph inputs require explicit --quantize-in or --no-quantize-in.')
        quantize_in = bool(floats)
    else:
        quantize_in = bool(args.quantize_in)
    got = model.predict(feeds, simulator='cuda', quantize_in=quantize_in, dequantize_out=False)
    out_names = list(model.context.ir.logical.output_tensor_names)
    if not isinstance(got, dict):
        got = {out_names[0]: got}
    # the golden: the integer oracle on the exported plan, fed the same integer codes the device was fed
    codes = {n: np.asarray(v)[0] for n, v in model.prepare_inputs(feeds, iterations=1, quantize=quantize_in).items()}
    want = oracle.run_plan(model.export_plan(), codes)
    failed = False
    for index, name in enumerate(out_names):
        ref, dev = np.asarray(want[name]).astype(np.int64), np.asarray(got[name]).astype(np.int64)
        if ref.shape != dev.shape:
            raise RuntimeError(f'output[{index}] shape mismatch: oracle {ref.shape} vs device {dev.shape}')
        diff = np.abs(ref - dev)
        max_diff = int(diff.max()) if diff.size else 0
        mean_diff = float(diff.mean()) if diff.size else 0.0
        ok = max_diff <= args.atol
        status = 'bit_exact' if max_diff == 0 else (f'within_atol={args.atol}' if ok else 'MISMATCH')
        print(f'output[{index}] {name}  max|dq|={max_diff}  mean|dq|={mean_diff:.6g}  {status}')
        failed |= not ok
    return 1 if failed else 0


if __name__ == '__main__':
    raise SystemExit(main())
