"""Dict / JSON graph front door and a programmatic builder.

Both produce the same pre-lowering logical IR the reference's ONNX importer emits
(``src/aie4ml/frontends/onnx/handlers/*.py``): ``dense`` without bias followed by ``add`` with a
constant (re-fused by FoldBias, handlers/matmul.py:116-137), ``activation`` nodes for ReLU,
``scale`` for constant Mul/Div (handlers/elementwise.py:15-50), ``transpose`` / ``slice`` /
``split`` / ``concat`` view ops (handlers/tensor.py:16-163), ``softmax`` and ``layer_norm``
(handlers/norm.py:17-76), ``matmul`` for a runtime RHS (handlers/matmul.py:52-67).  Tensor
precisions are ``QuantIntent``s: what a Q/DQ pair states in ONNX (power-of-two scale ->
``frac``, zero point 0).  Constants carry float values and are quantised at pack time.
"""

from __future__ import annotations

import json
from typing import Any, Dict, List, Optional, Sequence, Tuple

import numpy as np

from ..ir import BackendContext, DEVICE_CATALOG, LogicalIR, OpNode, TensorVar, set_input_roles
from ..qtypes import QuantIntent, RoundingMode, SaturationMode

_KNOWN_DIRECTIVES = ('placement', 'microtiling', 'parallelism', 'io_route', 'layout', 'approximation', 'hccs')


def normalize_directives(name: str, raw: Any) -> Dict[str, Any]:
    """Validate one ``LayerDirectives`` entry.  AIE-only knobs are accepted (and later ignored by
    the CUDA variants); ``approximation`` and ``hccs`` are honoured."""
    if raw is None:
        return {}
    if not isinstance(raw, dict):
        raise TypeError(f'{name}: layer directives must be a dict.')
    out: Dict[str, Any] = {}
    for key, value in raw.items():
        if key not in _KNOWN_DIRECTIVES:
            raise ValueError(f'{name}: unknown layer directive {key!r}.')
        if key in ('placement', 'microtiling', 'parallelism', 'io_route', 'hccs'):
            if not isinstance(value, dict):
                raise TypeError(f'{name}: {key} override must be a dict.')
            out[key] = dict(value)
        elif key == 'layout':
            if str(value) not in ('linear', 'tiled'):
                raise ValueError(f"{name}: unknown layout {value!r}; expected one of ['linear', 'tiled'].")
            out[key] = str(value)
        else:
            out[key] = str(value)
    return out


def create_context(config: Optional[Dict[str, Any]], project_name: str = 'model',
                   output_dir: Optional[str] = None) -> BackendContext:
    """Build the backend context from the user's config dict.

    ``Part`` (or ``AIEConfig.Part``) selects the device; ``cuda_b200`` is the only entry, and
    ``AIEConfig.Target`` must be ``cuda`` when given.  An AIE part name is an error here: this
    backend has no AIE code generator."""
    config = dict(config or {})
    aie_cfg = dict(config.get('AIEConfig', {}) or {})
    part = aie_cfg.get('Part') or config.get('Part') or aie_cfg.get('Device') or 'cuda_b200'
    device = DEVICE_CATALOG.get(str(part)) or DEVICE_CATALOG.get(str(part).lower())
    if device is None:
        raise KeyError(f'Unknown Part {part!r}; this backend executes on {sorted(DEVICE_CATALOG)}.')
    target = str(aie_cfg.get('Target', 'cuda')).lower()
    if target != 'cuda':
        raise ValueError(f"AIEConfig.Target={target!r} is not available in this backend; use 'cuda'.")
    aie_cfg.setdefault('Iterations', 1)
    if config.get('ComputeDtype'):   # float-simulation switch, accepted at the top level too
        aie_cfg.setdefault('ComputeDtype', config['ComputeDtype'])
    aie_cfg['Part'] = device.part
    aie_cfg['Target'] = 'cuda'
    return BackendContext(device=device, aie_config=aie_cfg, project_name=project_name, output_dir=output_dir)


def intent(width: int = 8, frac: int = 0, signed: bool = True, rounding: str = 'RND_CONV',
           saturation: str = 'SAT') -> QuantIntent:
    return QuantIntent(width=int(width), frac=int(frac), signed=bool(signed), rounding=RoundingMode[rounding],
                       saturation=SaturationMode[saturation])


class GraphBuilder:
    """Builds a logical IR node by node.  Every method returns the output tensor name(s)."""

    def __init__(self, config: Optional[Dict[str, Any]] = None, name: str = 'model'):
        self.config = dict(config or {})
        self.ctx = create_context(self.config, project_name=name)
        self.graph: LogicalIR = self.ctx.ir.logical
        self._directives = {str(k): normalize_directives(str(k), v)
                            for k, v in (self.config.get('LayerDirectives', {}) or {}).items()}
        self._used_directives: set = set()

    # -- tensors ---------------------------------------------------------------------------
    def input(self, name: str, shape: Sequence[int], precision: QuantIntent) -> str:
        self.graph.add_tensor(TensorVar(name=name, shape=tuple(int(s) for s in shape), precision=precision))
        self.graph.mark_graph_input(name)
        return name

    def param(self, name: str, data, precision: Optional[QuantIntent]) -> str:
        arr = np.asarray(data, dtype=np.float64)
        self.graph.add_tensor(TensorVar(name=name, shape=tuple(arr.shape), precision=precision, data=arr))
        return name

    def output(self, name: str) -> None:
        self.graph.mark_graph_output(name)

    def _t(self, name: str) -> TensorVar:
        try:
            return self.graph.tensors[name]
        except KeyError:
            raise ValueError(f'unknown tensor {name!r}') from None

    def emit(self, op_type: str, node_name: str, inputs: Sequence[str],
             outputs: Sequence[Tuple[str, Sequence[int], Optional[QuantIntent]]], *,
             roles: Optional[Sequence[str]] = None, metadata: Optional[Dict[str, Any]] = None) -> OpNode:
        node = OpNode(name=node_name, op_type=op_type, dialect=self.ctx.device.dialect)
        node.metadata.update(metadata or {})
        if node_name in self._directives:
            node.directives.update(self._directives[node_name])
            self._used_directives.add(node_name)
        ins = [self._t(n) for n in inputs]
        for t in ins:
            t.consumers.append(node)
        node.inputs.extend(ins)
        if roles is not None:
            node.metadata['input_roles'] = list(roles)
            set_input_roles(node, ins, roles)
        for out_name, out_shape, out_prec in outputs:
            t = TensorVar(name=out_name, shape=tuple(int(s) for s in out_shape), precision=out_prec, producer=node)
            self.graph.add_tensor(t)
            node.outputs.append(t)
        self.graph.add_node(node)
        return node

    # -- ops -------------------------------------------------------------------------------
    def dense(self, name: str, x: str, weight, w_precision: QuantIntent, out_precision: QuantIntent, *,
              bias=None, bias_precision: Optional[QuantIntent] = None, relu: bool = False,
              relu_precision: Optional[QuantIntent] = None, out_name: Optional[str] = None) -> str:
        """``y = relu?(x @ W + b)``; W is ``[K, N]`` float (code / 2**frac)."""
        W = np.asarray(weight, dtype=np.float64)
        xs = self._t(x).shape
        if W.ndim != 2 or int(xs[-1]) != W.shape[0]:
            raise ValueError(f'{name}: weight shape {W.shape} does not match input features {xs[-1]}.')
        out_shape = tuple(xs[:-1]) + (W.shape[1],)
        final = out_name or f'{name}_out'
        stages = ['mm'] + (['bias'] if bias is not None else []) + (['relu'] if relu else [])
        names = [f'{name}_{s}' for s in stages[:-1]] + [final]
        self.param(f'{name}_weight', W, w_precision)
        self.emit('dense', name, [x, f'{name}_weight'], [(names[0], out_shape, out_precision)],
                  roles=['lhs', 'rhs'],
                  metadata={'n_in': int(W.shape[0]), 'n_out': int(W.shape[1]), 'use_bias': False,
                            'layer_class': 'Dense', 'source_layer': name})
        cur = 0
        if bias is not None:
            if bias_precision is None:
                raise ValueError(f'{name}: bias needs a precision.')
            b = np.asarray(bias, dtype=np.float64).reshape(-1)
            self.param(f'{name}_biasv', b, bias_precision)
            self.emit('add', f'{name}_bias', [names[cur], f'{name}_biasv'],
                      [(names[cur + 1], out_shape, out_precision)], roles=['lhs', 'rhs'],
                      metadata={'layer_class': 'Add', 'source_class': 'Gemm', 'source_layer': name})
            cur += 1
        if relu:
            self.emit('activation', f'{name}_relu', [names[cur]],
                      [(names[cur + 1], out_shape, relu_precision or out_precision)], roles=['lhs'],
                      metadata={'activation': 'relu', 'layer_class': 'Activation', 'source_layer': name})
        return final

    def matmul(self, name: str, a: str, b: str, out_precision: QuantIntent, out_name: Optional[str] = None) -> str:
        sa, sb = self._t(a).shape, self._t(b).shape
        out_shape = tuple(sa[:-1]) + (sb[-1],)
        out = out_name or f'{name}_out'
        self.emit('matmul', name, [a, b], [(out, out_shape, out_precision)], roles=['lhs', 'rhs'],
                  metadata={'n_in': int(sb[-2]), 'n_out': int(sb[-1]), 'use_bias': False, 'layer_class': 'MatMul',
                            'source_layer': name})
        return out

    def add(self, name: str, a: str, b: str, out_precision: QuantIntent, out_name: Optional[str] = None) -> str:
        out = out_name or f'{name}_out'
        self.emit('add', name, [a, b], [(out, self._t(a).shape, out_precision)], roles=['lhs', 'rhs'],
                  metadata={'layer_class': 'Add', 'source_class': 'Add', 'source_layer': name})
        return out

    def scale(self, name: str, x: str, scale: float, out_name: Optional[str] = None) -> str:
        out = out_name or f'{name}_out'
        t = self._t(x)
        self.emit('scale', name, [x], [(out, t.shape, t.precision)], roles=['lhs'],
                  metadata={'scale': float(scale), 'layer_class': 'Mul', 'source_layer': name})
        return out

    def softmax(self, name: str, x: str, out_precision: QuantIntent, axis: int = -1,
                out_name: Optional[str] = None) -> str:
        out = out_name or f'{name}_out'
        t = self._t(x)
        axis = axis + len(t.shape) if axis < 0 else axis
        self.emit('softmax', name, [x], [(out, t.shape, out_precision)], roles=['lhs'],
                  metadata={'axis': axis, 'layer_class': 'Softmax', 'source_layer': name})
        return out

    def layer_norm(self, name: str, x: str, gamma, beta, out_precision: QuantIntent, *, epsilon=None,
                   eps_q0: Optional[int] = None, out_name: Optional[str] = None) -> str:
        out = out_name or f'{name}_out'
        t = self._t(x)
        self.param(f'{name}_gamma', gamma, None)
        self.param(f'{name}_beta', beta, None)
        meta: Dict[str, Any] = {'axis': len(t.shape) - 1, 'layer_class': 'LayerNormalization', 'source_layer': name}
        if epsilon is not None:
            meta['epsilon'] = float(epsilon)
        if eps_q0 is not None:
            meta['eps_q0'] = int(eps_q0)
        self.emit('layer_norm', name, [x, f'{name}_gamma', f'{name}_beta'], [(out, t.shape, out_precision)],
                  roles=['lhs', 'gamma', 'beta'], metadata=meta)
        return out

    def transpose(self, name: str, x: str, perm: Sequence[int], out_name: Optional[str] = None) -> str:
        out = out_name or f'{name}_out'
        t = self._t(x)
        perm = [int(p) for p in perm]
        self.emit('transpose', name, [x], [(out, tuple(t.shape[p] for p in perm), t.precision)], roles=['lhs'],
                  metadata={'perm': perm, 'data_format': 'channels_last', 'layer_class': 'Transpose',
                            'source_layer': name})
        return out

    def split(self, name: str, x: str, sizes: Sequence[int], axis: int = -1,
              out_names: Optional[Sequence[str]] = None) -> List[str]:
        t = self._t(x)
        rank = len(t.shape)
        axis = axis + rank if axis < 0 else axis
        sizes = [int(s) for s in sizes]
        if sum(sizes) != int(t.shape[axis]) or any(s <= 0 for s in sizes):
            raise ValueError(f'{name}: Split sizes must be positive and cover axis {axis} exactly.')
        names = list(out_names) if out_names else [f'{name}_out{i}' for i in range(len(sizes))]
        ranges, cursor = [], 0
        for s in sizes:
            ranges.append({'start': cursor, 'extent': s})
            cursor += s
        outs = [(n, tuple(t.shape[:axis]) + (s,) + tuple(t.shape[axis + 1:]), t.precision)
                for n, s in zip(names, sizes)]
        self.emit('split', name, [x], outs, roles=['lhs'],
                  metadata={'axis': axis, 'slices': ranges, 'layer_class': 'Split', 'source_layer': name})
        return names

    def slice(self, name: str, x: str, start: int, end: int, axis: int = -1, out_name: Optional[str] = None) -> str:
        t = self._t(x)
        rank = len(t.shape)
        axis = axis + rank if axis < 0 else axis
        start = max(0, min(int(t.shape[axis]), int(start)))
        end = max(start, min(int(t.shape[axis]), int(end)))
        out = out_name or f'{name}_out'
        shape = tuple(t.shape[:axis]) + (end - start,) + tuple(t.shape[axis + 1:])
        self.emit('slice', name, [x], [(out, shape, t.precision)], roles=['lhs'],
                  metadata={'axis': axis, 'slices': [{'start': start, 'extent': end - start}],
                            'layer_class': 'Slice', 'source_layer': name})
        return out

    def concat(self, name: str, xs: Sequence[str], axis: int = -1, out_name: Optional[str] = None) -> str:
        ts = [self._t(x) for x in xs]
        rank = len(ts[0].shape)
        axis = axis + rank if axis < 0 else axis
        for t in ts[1:]:
            if t.precision != ts[0].precision:
                raise ValueError(f'{name}: Concat inputs must use identical precision contracts.')
            if len(t.shape) != rank or t.shape[:axis] != ts[0].shape[:axis] or t.shape[axis + 1:] != ts[0].shape[axis + 1:]:
                raise ValueError(f'{name}: Concat input shapes disagree outside axis {axis}.')
        total = sum(int(t.shape[axis]) for t in ts)
        shape = tuple(ts[0].shape[:axis]) + (total,) + tuple(ts[0].shape[axis + 1:])
        out = out_name or f'{name}_out'
        self.emit('concat', name, list(xs), [(out, shape, ts[0].precision)],
                  metadata={'axis': axis, 'layer_class': 'Concat', 'source_layer': name})
        return out

    # -- finish ----------------------------------------------------------------------------
    def finalize(self) -> BackendContext:
        unused = sorted(set(self._directives) - self._used_directives)
        if unused:
            raise ValueError(f'LayerDirectives references unknown ONNX node names: {unused}.')
        for t in self.graph.tensors.values():
            if not t.is_parameter and t.precision is None:
                raise ValueError(f'activation tensor {t.name!r} has no quantisation intent.')
        if not self.graph.output_tensor_names:
            raise ValueError('graph has no outputs')
        self.graph.verify()
        return self.ctx


# ---------------------------------------------------------------------------------------------
# dict / JSON form
# ---------------------------------------------------------------------------------------------

def _prec(d) -> Optional[QuantIntent]:
    if d is None:
        return None
    if isinstance(d, QuantIntent):
        return d
    return QuantIntent.from_dict(d)


def lower_graph_dict(spec: Dict[str, Any], config: Optional[Dict[str, Any]] = None) -> BackendContext:
    """Lower ``{'name', 'inputs': [...], 'params': {...}, 'nodes': [...], 'outputs': [...]}``.

    Each node is ``{'name', 'op', 'inputs': [tensor names], 'outputs': [{'name','shape','precision'}],
    'roles': [...], 'metadata': {...}}`` with ``op`` one of dense, matmul, add, activation, scale,
    softmax, layer_norm, transpose, slice, split, concat -- the op vocabulary of the logical IR."""
    b = GraphBuilder(config, name=str(spec.get('name', 'model')))
    for item in spec.get('inputs', []):
        b.input(item['name'], item['shape'], _prec(item['precision']))
    for pname, item in (spec.get('params', {}) or {}).items():
        b.param(pname, np.asarray(item['data'], dtype=np.float64), _prec(item.get('precision')))
    for node in spec.get('nodes', []):
        outs = [(o['name'], o['shape'], _prec(o.get('precision'))) for o in node['outputs']]
        b.emit(str(node['op']), str(node['name']), list(node['inputs']), outs, roles=node.get('roles'),
               metadata=dict(node.get('metadata', {}) or {}))
    for name in spec.get('outputs', []):
        b.output(name)
    return b.finalize()


def load_graph_json(path: str, config: Optional[Dict[str, Any]] = None) -> BackendContext:
    with open(path) as fh:
        return lower_graph_dict(json.load(fh), config)
