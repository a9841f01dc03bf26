"""ONNX (Q/DQ) front door: QuantizeLinear / DequantizeLinear pairs become quantisation intents on tensors,
compute nodes become the same pre-lowering IR the programmatic ``GraphBuilder`` emits.

Mirrors the reference importer (``src/aie4ml/frontends/onnx/importer.py:30-130``, ``quantize.py:35-135``,
``handlers/matmul.py:16-159``, ``handlers/elementwise.py:15-81``, ``handlers/norm.py:17-76``,
``handlers/tensor.py:16-163``):

* a Q/DQ pair with a power-of-two scale and zero point 0 labels a tensor ``QuantIntent(width, frac = -log2(scale),
  signed, RND_CONV, SAT)`` (``utils.py:186-214``); a Quantize that follows a Relu / scalar Mul / Add also pins the
  still-unlabelled tensor in front of that node, as the reference does;
* ``MatMul`` / ``Gemm`` with a constant right-hand side is ``dense`` (Gemm's bias becomes ``dense -> add``, which
  ``FoldBias`` re-fuses), with two activations it is a dynamic ``matmul``; ``Add``, ``Relu``, scalar ``Mul`` /
  ``Div`` (-> ``scale``), ``Softmax``, ``LayerNormalization``, ``Transpose``, ``Split``, ``Slice``, ``Concat``
  map one to one.

A graph without Q/DQ nodes is a floating-point graph: a bare graph input of element type FLOAT / BFLOAT16 /
FLOAT8E4M3FN and a float initializer used directly carry a ``FloatIntent`` (``context.py:19-24,127-144``,
``utils.py:229-241``), and MatMul / Gemm / Add / LayerNormalization outputs inherit their left input's float intent
(``handlers/matmul.py:51``, ``elementwise.py:61``), which selects the floating-point Dense / MatMul / Add kernels.

The importer itself works on a small neutral description (``OnnxGraph``: nodes, initializers as NumPy arrays, input
shapes), so it is testable without the ``onnx`` package; ``from_onnx`` needs ``onnx`` only to read a ``ModelProto``
(or a path) into that description.  Output shapes are derived from the operators, not from ONNX shape inference.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from pathlib import Path
from typing import Any, Dict, List, Optional, Sequence, Tuple

import numpy as np

from ..ir import BackendContext, TensorVar
from ..qtypes import FloatFormat, FloatIntent, QuantIntent, RoundingMode, SaturationMode
from .graph import GraphBuilder


@dataclass
class OnnxNode:
    op_type: str
    name: str
    inputs: List[str]
    outputs: List[str]
    attrs: Dict[str, Any] = field(default_factory=dict)


@dataclass
class OnnxGraph:
    nodes: List[OnnxNode]
    initializers: Dict[str, np.ndarray]
    inputs: Dict[str, Tuple[Tuple[int, ...], Any]]   # name -> (shape, numpy dtype of the declared element type, or
                                                     #          'bfloat16' / 'float8_e4m3fn', which NumPy lacks)
    outputs: List[str]
    name: str = 'model'
    # initializers stored as bfloat16 / float8_e4m3fn in the file: name -> that type's name (the array holds the values)
    initializer_formats: Dict[str, str] = field(default_factory=dict)


def require_onnx():
    try:
        import onnx
        from onnx import helper, numpy_helper
    except ImportError as exc:  # same wording as the reference (frontends/onnx/utils.py)
        raise ImportError('The `onnx` package is required for aie4ml_b200.from_onnx(); it is not installed. '
                          'Build the model with aie4ml_b200.from_graph (GraphBuilder, dict or JSON) instead, '
                          'or describe it as an aie4ml_b200.frontends.onnx_import.OnnxGraph.') from exc
    return onnx, helper, numpy_helper


_ONNX_ELEM_TO_NP = {1: np.float32, 2: np.uint8, 3: np.int8, 4: np.uint16, 5: np.int16, 6: np.int32, 7: np.int64,
                    11: np.float64, 16: 'bfloat16', 17: 'float8_e4m3fn'}


def float_intent_of(tag) -> Optional[FloatIntent]:
    """Element type (NumPy dtype or type name) -> FloatIntent, None when it is not one of the three float types."""
    name = tag if isinstance(tag, str) else np.dtype(tag).name
    if name == 'float32':
        return FloatIntent(width=32, format=FloatFormat.FP32)
    if name == 'bfloat16':
        return FloatIntent(width=16, format=FloatFormat.BF16)
    if name in ('float8_e4m3fn', 'fp8_e4m3'):
        return FloatIntent(width=8, format=FloatFormat.FP8_E4M3)
    return None


def graph_from_proto(model_proto) -> OnnxGraph:
    """ModelProto -> OnnxGraph (needs the ``onnx`` package)."""
    _onnx, helper, numpy_helper = require_onnx()
    g = model_proto.graph
    inits, init_formats = {}, {}
    for t in g.initializer:
        arr = np.asarray(numpy_helper.to_array(t))
        if int(t.data_type) in (16, 17):
            init_formats[t.name] = _ONNX_ELEM_TO_NP[int(t.data_type)]
            arr = arr.astype(np.float32)
        inits[t.name] = arr
    inputs: Dict[str, Tuple[Tuple[int, ...], Any]] = {}
    for vi in g.input:
        if vi.name in inits:
            continue
        tt = vi.type.tensor_type
        shape = tuple(int(d.dim_value) for d in tt.shape.dim)
        inputs[vi.name] = (shape, _ONNX_ELEM_TO_NP.get(int(tt.elem_type), np.float32))
    nodes = []
    for i, n in enumerate(g.node):
        attrs = {a.name: helper.get_attribute_value(a) for a in n.attribute}
        nodes.append(OnnxNode(n.op_type, n.name or f'{n.op_type}_{i}', list(n.input), list(n.output), attrs))
    return OnnxGraph(nodes, inits, inputs, [o.name for o in g.output], g.name or 'model', init_formats)


def intent_from_qparams(inits: Dict[str, np.ndarray], scale_name: str, zero_name: str, qdtype, where: str) -> QuantIntent:
    """Symmetric power-of-two Q/DQ parameters -> intent (reference ``frontends/onnx/utils.py:186-214``)."""
    for n in (scale_name, zero_name):
        if n not in inits or np.asarray(inits[n]).size != 1:
            raise ValueError(f'{where}: scale and zero_point must be scalar constant initializers.')
    scale = float(np.asarray(inits[scale_name]).reshape(-1)[0])
    zero = int(np.asarray(inits[zero_name]).reshape(-1)[0])
    if zero != 0:
        raise ValueError(f'{where}: zero_point must be 0 for symmetric quantization.')
    dtype = np.dtype(qdtype)
    if not np.issubdtype(dtype, np.integer):
        raise ValueError(f'{where}: only integer quantization is supported; got {dtype}.')
    if scale <= 0.0:
        raise ValueError(f'{where}: quantization scale must be positive.')
    log2_scale = float(np.log2(scale))
    rounded = round(log2_scale)
    if not np.isclose(log2_scale, rounded, atol=1e-7):
        raise ValueError(f'{where}: scale {scale} is not a power of two.')
    return QuantIntent(width=int(dtype.itemsize * 8), frac=int(-rounded), signed=bool(np.issubdtype(dtype, np.signedinteger)),
                       rounding=RoundingMode.RND_CONV, saturation=SaturationMode.SAT)


class _Importer:
    def __init__(self, g: OnnxGraph, config: Optional[Dict[str, Any]]):
        self.g = g
        self.b = GraphBuilder(config, name=g.name)
        self.graph = self.b.graph
        self.value: Dict[str, TensorVar] = {}          # ONNX value name -> lowered tensor
        self.q_alias: Dict[str, Tuple[str, Any, QuantIntent, Tuple[int, ...]]] = {}
        self.mirrors: List[Tuple[str, str]] = []

    # ---- tensor plumbing ----------------------------------------------------------------------
    def bind(self, onnx_name: str, tensor: TensorVar) -> None:
        self.value[onnx_name] = tensor

    def param(self, name: str, data, precision) -> TensorVar:
        if name in self.graph.tensors:
            return self.graph.tensors[name]
        self.b.param(name, data, precision)
        return self.graph.tensors[name]

    def graph_input(self, name: str, shape, intent: QuantIntent) -> TensorVar:
        if name in self.graph.tensors:
            t = self.graph.tensors[name]
            if t.precision is not None and t.precision != intent:
                raise ValueError(f'{name}: graph input quantized with two different intents.')
            t.precision = intent
            return t
        if not shape:
            raise ValueError(f'{name}: scalar inputs are not supported.')
        self.b.input(name, shape, intent)
        return self.graph.tensors[name]

    def source(self, onnx_name: str, where: str) -> TensorVar:
        if onnx_name in self.value:
            return self.value[onnx_name]
        if onnx_name in self.g.inputs:
            # a bare graph input (no Q/DQ in front): only the three float element types can be computed on as they are
            shape, dt = self.g.inputs[onnx_name]
            intent = float_intent_of(dt)
            if intent is None:
                raise ValueError(f'{where}: graph input "{onnx_name}" has unsupported element type {dt}. '
                                 'Use QDQ wrapping for integer inputs.')
            t = self.graph_input(onnx_name, shape, intent)
            self.bind(onnx_name, t)
            return t
        raise ValueError(f'{where}: input {onnx_name} is not a lowered tensor (a float graph input or initializer must '
                         'pass through QuantizeLinear / DequantizeLinear first).')

    def param_source(self, onnx_name: str, where: str, like=None) -> TensorVar:
        """A constant operand.  ``like``: precision of the activation it meets; next to a floating-point activation a
        float initializer carries the float intent of its own stored type."""
        if onnx_name in self.value:
            return self.value[onnx_name]
        if onnx_name in self.g.initializers:
            arr = np.asarray(self.g.initializers[onnx_name])
            if not np.issubdtype(arr.dtype, np.floating):
                raise ValueError(f'{where}: constant {onnx_name} must be float or pass through DequantizeLinear.')
            intent = None
            if isinstance(like, FloatIntent):
                intent = float_intent_of(self.g.initializer_formats.get(onnx_name, arr.dtype))
                if intent is None:
                    raise ValueError(f'{where}: direct initializer inputs must be float32/bfloat16/fp8_e4m3, or quantized '
                                     f'via DequantizeLinear; got {arr.dtype}.')
            return self.param(onnx_name, arr.astype(np.float64), intent)
        raise ValueError(f'{where}: constant input {onnx_name} not found.')

    def emit(self, op_type, name, inputs: Sequence[TensorVar], outputs, roles, metadata) -> None:
        node = self.b.emit(op_type, name, [t.name for t in inputs], outputs, roles=roles, metadata=metadata)
        for t in node.outputs:
            self.value[t.name] = t

    # ---- Q / DQ -------------------------------------------------------------------------------
    @staticmethod
    def _pin(tensor: Optional[TensorVar], intent: QuantIntent, force_signed: bool) -> None:
        if tensor is None or tensor.is_parameter or tensor.precision is not None:
            return
        tensor.precision = (QuantIntent(width=intent.width, frac=intent.frac, signed=True, rounding=intent.rounding,
                                        saturation=intent.saturation) if force_signed else intent)

    def quantize_linear(self, n: OnnxNode) -> None:
        if len(n.inputs) != 3:
            raise ValueError(f'{n.name}: QuantizeLinear must have exactly 3 inputs.')
        src, scale, zero = n.inputs
        if zero not in self.g.initializers:
            raise ValueError(f'{n.name}: zero_point must be a constant initializer.')
        intent = intent_from_qparams(self.g.initializers, scale, zero, np.asarray(self.g.initializers[zero]).dtype, n.name)
        out = n.outputs[0]
        if src in self.value:
            t = self.value[src]
            prod = t.producer
            relu = prod is not None and prod.op_type == 'activation' and prod.metadata.get('activation') == 'relu'
            scale_p = prod is not None and prod.op_type == 'scale'
            add_p = prod is not None and prod.op_type == 'add'
            if t.precision is None:
                if relu:
                    self._pin(prod.inputs[0], intent, True)
                elif scale_p:
                    self._pin(prod.inputs[0], intent, False)
                elif add_p:
                    for inp in prod.inputs:
                        self._pin(inp, intent, False)
                t.precision = intent
            elif t.precision != intent:
                if relu:
                    self._pin(prod.inputs[0], intent, True)
                    t.precision = intent
                else:
                    raise ValueError(f'{n.name}: QuantizeLinear intent does not match source tensor precision.')
            self.q_alias[out] = ('tensor', t, intent, tuple(t.shape))
        elif src in self.g.inputs:
            self.q_alias[out] = ('input', src, intent, tuple(self.g.inputs[src][0]))
        elif src in self.g.initializers:
            self.q_alias[out] = ('initializer', src, intent, tuple(np.asarray(self.g.initializers[src]).shape))
        else:
            raise ValueError(f'{n.name}: QuantizeLinear input {src} is unsupported.')

    def dequantize_linear(self, n: OnnxNode) -> None:
        if len(n.inputs) != 3:
            raise ValueError(f'{n.name}: DequantizeLinear must have exactly 3 inputs.')
        src, scale, zero = n.inputs
        out = n.outputs[0]
        inits = self.g.initializers

        def dequant(data) -> np.ndarray:
            s = float(np.asarray(inits[scale]).reshape(-1)[0])
            z = int(np.asarray(inits[zero]).reshape(-1)[0])
            return (np.asarray(data, dtype=np.float64) - float(z)) * s

        if src in self.q_alias:
            kind, ref, q_intent, shape = self.q_alias[src]
            intent = intent_from_qparams(inits, scale, zero, np.asarray(inits[zero]).dtype, n.name)
            if intent != q_intent:
                raise ValueError(f'{n.name}: QuantizeLinear/DequantizeLinear parameters do not match.')
            if kind == 'tensor':
                t = ref
            elif kind == 'input':
                t = self.graph_input(ref, shape, intent)
            else:
                # a float initializer quantized inside the graph: the constant packer applies the same rounding
                # (half to even) and saturation when it turns the value into the intent's integer code
                t = self.param(ref, np.asarray(inits[ref], dtype=np.float64), intent)
            self.bind(out, t)
            return
        if src in inits:
            intent = intent_from_qparams(inits, scale, zero, np.asarray(inits[src]).dtype, n.name)
            self.bind(out, self.param(src, dequant(inits[src]), intent))
            return
        if src in self.g.inputs:
            shape, dt = self.g.inputs[src]
            if not np.issubdtype(np.dtype(dt), np.integer):
                raise ValueError(f'{n.name}: direct DequantizeLinear on a graph input requires an integer input type.')
            intent = intent_from_qparams(inits, scale, zero, dt, n.name)
            self.bind(out, self.graph_input(src, shape, intent))
            return
        raise ValueError(f'{n.name}: DequantizeLinear input {src} is unsupported.')

    # ---- compute nodes ------------------------------------------------------------------------
    def matmul_gemm(self, n: OnnxNode) -> None:
        gemm = n.op_type == 'Gemm'
        if gemm:
            if len(n.inputs) not in (2, 3):
                raise ValueError(f'{n.name}: Gemm must have 2 or 3 inputs.')
            if float(n.attrs.get('alpha', 1.0)) != 1.0 or float(n.attrs.get('beta', 1.0)) != 1.0:
                raise ValueError(f'{n.name}: Gemm alpha and beta must be 1.')
            if int(n.attrs.get('transA', 0)) != 0:
                raise ValueError(f'{n.name}: Gemm transA is not supported.')
        elif len(n.inputs) != 2:
            raise ValueError(f'{n.name}: MatMul must have exactly 2 inputs.')
        lhs_name, rhs_name = n.inputs[:2]
        bias_name = n.inputs[2] if gemm and len(n.inputs) == 3 else None
        trans_b = gemm and int(n.attrs.get('transB', 0)) == 1
        lhs = self.source(lhs_name, n.name)
        if lhs.is_parameter:
            raise ValueError(f'{n.name}: activation input cannot be constant.')
        rhs_const = gemm or rhs_name in self.g.initializers or (rhs_name in self.value and self.value[rhs_name].is_parameter)
        out = n.outputs[0]
        out_p = lhs.precision if isinstance(lhs.precision, FloatIntent) else None
        if not rhs_const:
            rhs = self.source(rhs_name, n.name)
            shape = tuple(lhs.shape[:-1]) + (int(rhs.shape[-1]),)
            if int(lhs.shape[-1]) != int(rhs.shape[-2]):
                raise ValueError(f'{n.name}: MatMul operands do not contract ({lhs.shape} x {rhs.shape}).')
            self.emit('matmul', n.name, [lhs, rhs], [(out, shape, out_p)], ['lhs', 'rhs'],
                      {'n_in': int(rhs.shape[-2]), 'n_out': int(rhs.shape[-1]), 'use_bias': False, 'layer_class': 'MatMul',
                       'source_class': 'MatMul', 'source_layer': n.name})
            return
        rhs_t = self.param_source(rhs_name, n.name, like=lhs.precision)
        if not rhs_t.is_parameter:
            raise ValueError(f'{n.name}: weight input must be a constant initializer.')
        W = np.asarray(rhs_t.data, dtype=np.float64)
        if trans_b:
            W = W.T
        if W.ndim != 2:
            raise NotImplementedError(f'{n.name}: a constant right-hand side of rank {W.ndim} has no kernel; express it as Dense.')
        if int(lhs.shape[-1]) != W.shape[0]:
            raise ValueError(f'{n.name}: weight shape {W.shape} does not match input features {lhs.shape[-1]}.')
        n_in, n_out = int(W.shape[0]), int(W.shape[1])
        shape = tuple(lhs.shape[:-1]) + (n_out,)
        w_param = self.param(f'{n.name}_weight', W, rhs_t.precision)
        meta = {'n_in': n_in, 'n_out': n_out, 'use_bias': False, 'layer_class': 'Dense', 'source_class': n.op_type,
                'source_layer': n.name}
        if bias_name is None:
            self.emit('dense', n.name, [lhs, w_param], [(out, shape, out_p)], ['lhs', 'rhs'], meta)
            return
        pre = f'{n.name}_prebias'
        self.mirrors.append((pre, out))
        self.emit('dense', n.name, [lhs, w_param], [(pre, shape, out_p)], ['lhs', 'rhs'], meta)
        bias_t = self.param_source(bias_name, n.name, like=lhs.precision)
        if not bias_t.is_parameter:
            raise ValueError(f'{n.name}: Gemm bias must be constant.')
        bias = np.asarray(bias_t.data, dtype=np.float64).reshape(-1)
        if bias.size != n_out:
            raise ValueError(f'{n.name}: Gemm bias must contain exactly {n_out} elements.')
        b_param = self.param(f'{n.name}_bias', bias, bias_t.precision)
        self.emit('add', f'{n.name}_bias', [self.value[pre], b_param], [(out, shape, out_p)], ['lhs', 'rhs'],
                  {'layer_class': 'Add', 'source_class': 'Gemm', 'source_layer': n.name})

    def add(self, n: OnnxNode) -> None:
        if len(n.inputs) != 2:
            raise ValueError(f'{n.name}: Add must have exactly 2 inputs.')
        acts = [self.source(name, n.name) for name in n.inputs if name in self.value or name in self.g.inputs]
        like = acts[0].precision if acts else None
        ts = []
        for name in n.inputs:
            ts.append(self.value[name] if name in self.value else self.param_source(name, n.name, like=like))
        lhs, rhs = ts
        if lhs.is_parameter and not rhs.is_parameter:
            lhs, rhs = rhs, lhs
        if lhs.is_parameter == rhs.is_parameter and tuple(lhs.shape) != tuple(rhs.shape):
            raise ValueError(f'{n.name}: generic Add only supports exact-shape elementwise inputs; got {lhs.shape} and {rhs.shape}.')
        out_p = lhs.precision if isinstance(lhs.precision, FloatIntent) else None
        self.emit('add', n.name, [lhs, rhs], [(n.outputs[0], tuple(lhs.shape), out_p)], ['lhs', 'rhs'],
                  {'layer_class': 'Add', 'source_class': 'Add', 'source_layer': n.name})

    def relu(self, n: OnnxNode) -> None:
        if len(n.inputs) != 1:
            raise ValueError(f'{n.name}: Relu must have exactly 1 input.')
        src = self.source(n.inputs[0], n.name)
        out_p = src.precision if isinstance(src.precision, FloatIntent) else None
        self.emit('activation', n.name, [src], [(n.outputs[0], tuple(src.shape), out_p)], ['lhs'],
                  {'activation': 'relu', 'layer_class': 'Activation', 'source_class': 'Relu', 'source_layer': n.name})

    def mul_div(self, n: OnnxNode) -> None:
        if len(n.inputs) != 2:
            raise ValueError(f'{n.name}: {n.op_type} must have exactly 2 inputs.')
        inits = self.g.initializers
        if n.op_type == 'Mul':
            consts = [x for x in n.inputs if x in inits]
            if len(consts) != 1:
                raise NotImplementedError(f'{n.name}: Mul currently requires exactly one constant input.')
            const = consts[0]
            src_name = n.inputs[1] if n.inputs[0] == const else n.inputs[0]
            scale = float(np.asarray(inits[const]).reshape(-1)[0])
        else:
            src_name, const = n.inputs
            if const not in inits:
                raise NotImplementedError(f'{n.name}: Div currently requires a constant divisor.')
            div = float(np.asarray(inits[const]).reshape(-1)[0])
            if div == 0.0:
                raise ValueError(f'{n.name}: Div constant divisor must be nonzero.')
            scale = 1.0 / div
        if np.asarray(inits[const]).size != 1:
            raise NotImplementedError(f'{n.name}: {n.op_type} currently requires a scalar constant.')
        src = self.source(src_name, n.name)
        self.emit('scale', n.name, [src], [(n.outputs[0], tuple(src.shape), src.precision)], ['lhs'],
                  {'scale': scale, 'layer_class': n.op_type, 'source_class': n.op_type, 'source_layer': n.name})

    def softmax(self, n: OnnxNode) -> None:
        src = self.source(n.inputs[0], n.name)
        rank = len(src.shape)
        axis = int(n.attrs.get('axis', -1))
        axis = axis + rank if axis < 0 else axis
        if not 0 <= axis < rank:
            raise ValueError(f'{n.name}: Softmax axis {axis} out of range for rank {rank}.')
        self.emit('softmax', n.name, [src], [(n.outputs[0], tuple(src.shape), None)], ['lhs'],
                  {'axis': axis, 'layer_class': 'Softmax', 'source_class': 'Softmax', 'source_layer': n.name})

    def layer_norm(self, n: OnnxNode) -> None:
        if len(n.inputs) not in (2, 3):
            raise ValueError(f'{n.name}: LayerNormalization must have 2 or 3 inputs.')
        x = self.source(n.inputs[0], n.name)
        rank = len(x.shape)
        axis = int(n.attrs.get('axis', -1))
        axis = axis + rank if axis < 0 else axis
        gamma = self.param_source(n.inputs[1], n.name)
        if not gamma.is_parameter:
            raise ValueError(f'{n.name}: LayerNormalization Scale must be a constant initializer.')
        if len(n.inputs) == 3:
            beta = self.param_source(n.inputs[2], n.name)
            if not beta.is_parameter:
                raise ValueError(f'{n.name}: LayerNormalization Bias must be a constant initializer.')
        else:
            beta = self.param(f'{n.name}_beta_zero', np.zeros(tuple(x.shape[axis:]), dtype=np.float64), gamma.precision)
        self.emit('layer_norm', n.name, [x, gamma, beta], [(n.outputs[0], tuple(x.shape), None)], ['lhs', 'gamma', 'beta'],
                  {'layer_class': 'LayerNormalization', 'source_class': 'LayerNormalization', 'source_layer': n.name,
                   'epsilon': float(n.attrs.get('epsilon', 1e-5)), 'axis': axis})

    def transpose(self, n: OnnxNode) -> None:
        src = self.source(n.inputs[0], n.name)
        perm = [int(p) for p in n.attrs.get('perm', list(range(len(src.shape)))[::-1])]
        self.emit('transpose', n.name, [src], [(n.outputs[0], tuple(src.shape[p] for p in perm), src.precision)], ['lhs'],
                  {'perm': perm, 'data_format': 'channels_last', 'layer_class': 'Transpose', 'source_class': 'Transpose',
                   'source_layer': n.name})

    def _const_ints(self, name: str, where: str) -> List[int]:
        if name not in self.g.initializers:
            raise NotImplementedError(f'{where}: {name} must be a constant initializer.')
        return [int(v) for v in np.asarray(self.g.initializers[name]).reshape(-1)]

    def split(self, n: OnnxNode) -> None:
        src = self.source(n.inputs[0], n.name)
        rank = len(src.shape)
        axis = int(n.attrs.get('axis', 0))
        axis = axis + rank if axis < 0 else axis
        if len(n.inputs) > 1 and n.inputs[1]:
            sizes = self._const_ints(n.inputs[1], n.name)
        elif 'split' in n.attrs:
            sizes = [int(v) for v in n.attrs['split']]
        else:
            parts = len(n.outputs)
            if int(src.shape[axis]) % parts:
                raise ValueError(f'{n.name}: Split axis {axis} of extent {src.shape[axis]} does not divide into {parts}.')
            sizes = [int(src.shape[axis]) // parts] * parts
        if len(sizes) != len(n.outputs) or sum(sizes) != int(src.shape[axis]) or any(s <= 0 for s in sizes):
            raise ValueError(f'{n.name}: Split sizes must be positive and cover axis {axis} exactly.')
        ranges, cursor, outs = [], 0, []
        for name, s in zip(n.outputs, sizes):
            ranges.append({'start': cursor, 'extent': s})
            cursor += s
            outs.append((name, tuple(src.shape[:axis]) + (s,) + tuple(src.shape[axis + 1:]), src.precision))
        self.emit('split', n.name, [src], outs, ['lhs'],
                  {'axis': axis, 'slices': ranges, 'layer_class': 'Split', 'source_class': 'Split', 'source_layer': n.name})

    def slice(self, n: OnnxNode) -> None:
        src = self.source(n.inputs[0], n.name)
        rank = len(src.shape)
        if len(n.inputs) < 3:
            raise NotImplementedError(f'{n.name}: Slice needs constant starts and ends inputs (opset 10 or later).')
        starts, ends = self._const_ints(n.inputs[1], n.name), self._const_ints(n.inputs[2], n.name)
        axes = self._const_ints(n.inputs[3], n.name) if len(n.inputs) > 3 and n.inputs[3] else list(range(len(starts)))
        steps = self._const_ints(n.inputs[4], n.name) if len(n.inputs) > 4 and n.inputs[4] else [1] * len(starts)
        if len(starts) != 1 or len(ends) != 1 or len(axes) != 1 or steps != [1]:
            raise NotImplementedError(f'{n.name}: Slice supports one axis with step 1.')
        axis = axes[0] + rank if axes[0] < 0 else axes[0]
        extent = int(src.shape[axis])
        start = starts[0] + extent if starts[0] < 0 else starts[0]
        end = ends[0] + extent if ends[0] < 0 else ends[0]
        start = max(0, min(extent, start))
        end = max(start, min(extent, end))
        shape = tuple(src.shape[:axis]) + (end - start,) + tuple(src.shape[axis + 1:])
        self.emit('slice', n.name, [src], [(n.outputs[0], shape, src.precision)], ['lhs'],
                  {'axis': axis, 'slices': [{'start': start, 'extent': end - start}], 'layer_class': 'Slice',
                   'source_class': 'Slice', 'source_layer': n.name})

    def concat(self, n: OnnxNode) -> None:
        if not n.inputs:
            raise ValueError(f'{n.name}: Concat must have at least one input.')
        ts = [self.source(x, n.name) for x in n.inputs]
        rank = len(ts[0].shape)
        axis = int(n.attrs.get('axis', 0))
        axis = axis + rank if axis < 0 else axis
        for t in ts[1:]:
            if t.precision != ts[0].precision:
                raise ValueError(f'{n.name}: Concat inputs must use identical precision contracts.')
            if len(t.shape) != rank or t.shape[:axis] != ts[0].shape[:axis] or t.shape[axis + 1:] != ts[0].shape[axis + 1:]:
                raise ValueError(f'{n.name}: Concat input shapes disagree outside axis {axis}.')
        total = sum(int(t.shape[axis]) for t in ts)
        shape = tuple(ts[0].shape[:axis]) + (total,) + tuple(ts[0].shape[axis + 1:])
        self.emit('concat', n.name, ts, [(n.outputs[0], shape, ts[0].precision)], None,
                  {'axis': axis, 'layer_class': 'Concat', 'source_class': 'Concat', 'source_layer': n.name})

    HANDLERS = {'QuantizeLinear': quantize_linear, 'DequantizeLinear': dequantize_linear, 'MatMul': matmul_gemm,
                'Gemm': matmul_gemm, 'Add': add, 'Relu': relu, 'Mul': mul_div, 'Div': mul_div, 'Softmax': softmax,
                'LayerNormalization': layer_norm, 'Transpose': transpose, 'Split': split, 'Slice': slice,
                'Concat': concat}

    # ---- driver -------------------------------------------------------------------------------
    def run(self) -> BackendContext:
        for n in self.g.nodes:
            h = self.HANDLERS.get(n.op_type)
            if h is None:
                raise NotImplementedError(f'{n.name}: ONNX operator {n.op_type} has no handler '
                                          f'(supported: {", ".join(sorted(self.HANDLERS))}).')
            h(self, n)
        graph = self.graph
        for out in self.g.outputs:
            if out not in self.value:
                raise ValueError(f'Graph output {out}: expected a lowered semantic tensor.')
            t = self.value[out]
            if out not in graph.tensors:
                graph.tensors.pop(t.name, None)
                t.name = out
                graph.tensors[out] = t
            self.b.output(out)
        for target, source in self.mirrors:
            t, o = graph.tensors.get(target), graph.tensors.get(source)
            if t is not None and t.precision is None and o is not None:
                t.precision = o.precision
        for t in graph.tensors.values():
            if not t.is_parameter and t.precision is None:
                raise ValueError(f'{t.name}: missing quantization intent after ONNX QDQ lowering.')
        return self.b.finalize()


def lower_onnx_graph(g: OnnxGraph, config: Optional[Dict[str, Any]] = None) -> BackendContext:
    """OnnxGraph -> backend context holding the pre-lowering logical IR (run the pass pipeline next)."""
    return _Importer(g, config).run()


def lower_onnx_model(model_or_path, config: Optional[Dict[str, Any]] = None, **_ignored) -> BackendContext:
    """ModelProto or path -> backend context (reference ``lower_onnx_model``, ``importer.py:30-77``); ``output_dir``,
    ``project_name``, ``stamp`` and ``custom_sources`` belong to the Vitis project writer and are accepted and ignored."""
    onnx, _h, _n = require_onnx()
    proto = onnx.load(str(model_or_path)) if isinstance(model_or_path, (str, Path)) else model_or_path
    return lower_onnx_graph(graph_from_proto(proto), config)


def from_onnx(model_or_path, config: Optional[Dict[str, Any]] = None, *, output_dir=None, project_name: Optional[str] = None,
              **kwargs):
    """ONNX model (path, ModelProto or OnnxGraph) -> ``CudaModel`` (reference ``from_onnx``, ``importer.py:113-130``)."""
    from ..model import CudaModel

    if isinstance(model_or_path, OnnxGraph):
        ctx = lower_onnx_graph(model_or_path, config)
    else:
        ctx = lower_onnx_model(model_or_path, config)
    if output_dir is not None:
        ctx.output_dir = str(output_dir)
    return CudaModel.from_context(ctx, source_model=model_or_path)
