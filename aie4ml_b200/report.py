"""Per-launch report of a compiled plan: device time, algorithmic bytes and operations, achieved GB/s and
TOP/s, and the fraction of the bound that applies (measured HBM copy bandwidth or int8 tensor peak).

The counterpart of the reference's ``aie4ml-report`` (``src/aie4ml/report.py:662-677``), which parses Vitis
simulator logs into per-kernel cycle counts; here every launch of the plan is timed on the GPU with CUDA
events (each launch replayed ``iters`` times back to back after a warm-up), and the plan dump
(``cuda_pipeline.json`` + ``params.npz``, ``CudaModel.dump``) can be read back with ``load_plan``.

    python -m aie4ml_b200.report --workload cfg3_exp [--batch N] [--iters 20] [--json] [--no-dense-ln]
"""

from __future__ import annotations

import argparse
import json
from pathlib import Path
from typing import Any, Dict, List

import numpy as np

ESZ = {'int8': 1, 'uint8': 1, 'int16': 2}


def load_plan(directory) -> Dict[str, Any]:
    """Reads back what ``CudaModel.dump`` wrote: the op list with its resolved numerics plus the integer
    constants, in the form ``oracle.run_plan`` and ``CudaModel.export_plan`` use."""
    d = Path(directory)
    plan = json.loads((d / 'cuda_pipeline.json').read_text())
    with np.load(d / 'params.npz') as z:
        plan['params'] = {k.replace('__', '/'): z[k] for k in z.files}
    return plan


def _numel(plan, name: str) -> int:
    return int(np.prod(plan.views[name].shape, dtype=np.int64))


def op_cost(plan, op: Dict[str, Any]) -> Dict[str, float]:
    """Algorithmic bytes (each operand and result once, constants once) and integer operations of one launch."""
    kind = op['kind']
    esz = lambda n: ESZ[plan.fmt[n]]
    if kind == 'dense':
        M = _numel(plan, op['lhs']) // op['K']
        return {'bytes': M * op['K'] * esz(op['lhs']) + op['K'] * op['N'] + 4 * op['N'] + M * op['N'] * esz(op['out']),
                'ops': 2.0 * M * op['K'] * op['N']}
    if kind == 'dense_add_ln':
        d = op['dense']
        M = _numel(plan, op['lhs']) // d['K']
        return {'bytes': M * d['K'] + d['K'] * d['N'] + 8 * d['N'] + 2 * M * d['N'], 'ops': 2.0 * M * d['K'] * d['N']}
    if kind == 'mlp':
        dims = op['dims']
        M = _numel(plan, op['lhs']) // dims[0]
        w = sum(dims[i] * dims[i + 1] + 4 * dims[i + 1] for i in range(len(dims) - 1))
        return {'bytes': M * (dims[0] + dims[-1]) + w, 'ops': 2.0 * M * sum(dims[i] * dims[i + 1] for i in range(len(dims) - 1))}
    if kind == 'matmul':
        a, b, c = (plan.views[op[k]] for k in ('lhs', 'rhs', 'out'))
        K = a.shape[-2] if op['transpose_lhs'] else a.shape[-1]
        return {'bytes': _numel(plan, op['lhs']) * a.esz + _numel(plan, op['rhs']) * b.esz + _numel(plan, op['out']) * c.esz,
                'ops': 2.0 * _numel(plan, op['out']) * K}
    if kind == 'attention':
        q, k = plan.views[op['q']], plan.views[op['k']]
        heads = int(op.get('heads', 1))
        nq, nk = heads * _numel(plan, op['q']), heads * _numel(plan, op['k'])
        sk, dh = k.shape[-2], k.shape[-1]
        return {'bytes': 2 * nq + 2 * nk, 'ops': 2.0 * (nq // dh) * sk * dh * 2}
    if kind in ('layer_norm', 'softmax', 'add'):
        n = _numel(plan, op['lhs'])
        b = n * esz(op['lhs']) + _numel(plan, op['out']) * esz(op['out'])
        other = op.get('addend') or op.get('pre_addend') or (op.get('rhs') if kind == 'add' else None)
        if other:
            b += _numel(plan, other) * esz(other)
        return {'bytes': b, 'ops': 0.0}
    return {'bytes': 0.0, 'ops': 0.0}


def profile_plan(plan, iters: int = 20, hbm_gbs: float = 6552.6, int8_tops: float = 3241.8) -> List[Dict[str, Any]]:
    """Times every launch of ``plan`` on its device.  ``hbm_gbs`` / ``int8_tops`` are the roofline denominators."""
    import torch

    from . import lib as _lib

    rows = []
    stream = torch.cuda.current_stream(plan.device).cuda_stream
    for (fn, args), op in zip(plan.launches, plan.ops):
        for _ in range(3):
            _lib.check(fn(*args, stream), op['name'])
        torch.cuda.synchronize(plan.device)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(iters):
            fn(*args, stream)
        e1.record()
        torch.cuda.synchronize(plan.device)
        ms = e0.elapsed_time(e1) / iters
        cost = op_cost(plan, op)
        gbs = cost['bytes'] / (ms * 1e-3) / 1e9
        tops = cost['ops'] / (ms * 1e-3) / 1e12
        t_hbm, t_tc = cost['bytes'] / (hbm_gbs * 1e9), cost['ops'] / (int8_tops * 1e12)
        bound = 'tensor' if t_tc > t_hbm else 'hbm'
        rows.append({'name': op['name'], 'kind': op['kind'], 'ms': ms, 'bytes': cost['bytes'], 'ops': cost['ops'],
                     'GB/s': gbs, 'TOP/s': tops, 'bound': bound,
                     'roofline_frac': max(t_hbm, t_tc) / (ms * 1e-3) if ms > 0 else 0.0})
    plan.check_status()
    return rows


def format_rows(rows: List[Dict[str, Any]]) -> str:
    total = sum(r['ms'] for r in rows) or 1.0
    out = [f"{'launch':40s} {'kind':10s} {'ms':>9s} {'share':>6s} {'GB/s':>8s} {'TOP/s':>8s} {'bound':>6s} {'of roof':>8s}"]
    for r in rows:
        out.append(f"{r['name'][:40]:40s} {r['kind']:10s} {r['ms']:9.4f} {100 * r['ms'] / total:5.1f}% {r['GB/s']:8.0f} "
                   f"{r['TOP/s']:8.1f} {r['bound']:>6s} {r['roofline_frac']:8.2f}")
    out.append(f"{'sum of launches':40s} {'':10s} {total:9.4f}")
    return '\n'.join(out)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split('\n')[0])
    ap.add_argument('--workload', default='cfg3_exp',
                    help='cfg1, cfg3_exp, cfg3_hccs, cfg4_ln, cfg4_sm_exp, cfg4_sm_hccs, cfg5 or dense')
    ap.add_argument('--batch', type=int, default=0)
    ap.add_argument('--m', type=int, default=16384)
    ap.add_argument('--k', type=int, default=4096)
    ap.add_argument('--n', type=int, default=4096)
    ap.add_argument('--iters', type=int, default=20)
    ap.add_argument('--json', action='store_true')
    ap.add_argument('--no-dense-ln', action='store_true',
                    help='keep Dense and Add + LayerNorm as two launches (the single kernel for 256-wide layers is the default)')
    a = ap.parse_args(argv)
    from . import from_graph
    from . import lib as _lib
    from . import workloads as W

    if a.no_dense_ln:
        _lib.check(_lib.load().a4c_set_option(_lib.OPT_DENSE_LN_PATH, 1), 'a4c_set_option')

    name = a.workload
    if name == 'dense':
        b, inputs = W.dense_cfg2(a.m, a.k, a.n)
    elif name == 'cfg1':
        b, inputs = W.mlp_cfg1(a.batch or 1024)
    elif name in ('cfg3_exp', 'cfg3_hccs'):
        b, inputs = W.encoder_cfg3(a.batch or 4096, softmax=name.split('_')[1])
    elif name in ('cfg4_ln', 'cfg4_sm_exp', 'cfg4_sm_hccs'):
        b, inputs = W.rowops_cfg4(a.batch or (1 << 20), 1024, {'cfg4_ln': 'layer_norm', 'cfg4_sm_exp': 'softmax_exp',
                                                           'cfg4_sm_hccs': 'softmax_hccs'}[name])
    elif name == 'cfg5':
        b, inputs = W.wide_mlp_cfg5(a.batch or 262144)
    else:
        ap.error(f'unknown workload {name!r}')
    model = from_graph(b)
    model.compile()
    # the workload's seeded inputs, then one whole step: every launch is then timed on the data it sees in a real run
    # (on zero-filled buffers every LayerNorm row has zero variance and takes the kernel's rare exact-reciprocal path)
    import torch

    for n in model.plan.graph.input_tensor_names:
        model.plan.tensor_of(n).copy_(torch.from_numpy(np.ascontiguousarray(inputs[n])).to(model.plan.device))
    model.plan.run(use_graph=False)
    rows = profile_plan(model.plan, a.iters)
    print(json.dumps(rows) if a.json else format_rows(rows))
    return 0


if __name__ == '__main__':
    raise SystemExit(main())
