"""Floating-point variants of Dense, MatMul and Add: the reference's float-simulation path.

With ``AIEConfig.ComputeDtype`` = ``'bfloat16'`` or ``'float32'`` the ``ForceFloatMode`` pass relabels every
tensor as floating point (reference ``passes/force_float_mode.py:22-46``); the matmul family then resolves to
its float contract (``op_impls/families/matmul/resolver.py:110-127``: lhs / rhs / output share one float
precision, accumulator ``accfloat``, no shift, no rounding token) and Add to a plain float add.  Storage is the
compute type (bfloat16 values are kept as their 16 bits), accumulation is float32, results are rounded to
nearest-even when stored.  The reference holds this path to rtol 1e-2 / atol 5e-2 (bfloat16) and 1e-3 / 1e-3
(float32) against a float model (``tests/test_float_sim.py:87-93``); the tests here use the same tolerances.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict

import numpy as np

from ..ir import ExecutionEntry, OpNode, input_tensor_for_role, optional_tensor_for_role
from ..qtypes import FLOAT_FORMATS, AIEDataType, FloatIntent
from ..quant_utils import from_storage_float, pack_constant_float
from .base import CUDA_GENERATIONS, OpImplVariant, register_variant
from .matmul import _transposed
from .precision import resolve_exact_storage_dtype
from .views import view_shape


def is_float_node(node: OpNode) -> bool:
    return isinstance(input_tensor_for_role(node, 'lhs').precision, FloatIntent)


def _float_precision(node: OpNode, roles) -> Dict[str, AIEDataType]:
    out = {'output': resolve_exact_storage_dtype(node.outputs[0].precision, namespace='output', layer_name=node.name)}
    for role in roles:
        t = input_tensor_for_role(node, role)
        out[role] = resolve_exact_storage_dtype(t.precision, namespace=role, layer_name=node.name)
    fmts = {p.format for p in out.values()}
    if len(fmts) != 1 or not fmts <= set(FLOAT_FORMATS):
        raise ValueError(f'{node.name}: float {node.op_type} requires lhs/rhs/output to share float precision.')
    out['acc'] = AIEDataType(format='float32', frac=0)
    return out


@dataclass(frozen=True)
class FloatMatmulConfig:
    precision: Dict[str, AIEDataType]
    use_relu: bool
    use_bias: bool
    transpose_lhs: bool
    transpose_rhs: bool
    n_in: int
    n_out: int
    shift: int = 0
    accumulator_tag: str = 'accfloat'
    rounding_mode: str = 'conv_even'


@register_variant
class CudaFloatDenseVariant(OpImplVariant):
    variant_id = 'dense.b.r.float.cuda.v1'
    op_type = 'dense'
    plevel = 30

    def matches(self, node: OpNode, device) -> bool:
        return device.generation in CUDA_GENERATIONS and is_float_node(node)

    def resolve(self, node: OpNode, device, directives=None) -> FloatMatmulConfig:
        if node.traits.get('output_scale') is not None:
            raise NotImplementedError(f'{node.name}: fused output scaling is not implemented for float MatMul-family ops.')
        fused = node.traits.get('fused_activation')
        lhs = input_tensor_for_role(node, 'lhs')
        return FloatMatmulConfig(
            precision=_float_precision(node, ('lhs', 'rhs')),
            use_relu=((fused.data.get('activation') if fused else '') or '').lower() == 'relu',
            use_bias=bool(node.metadata.get('use_bias')), transpose_lhs=_transposed(node, lhs), transpose_rhs=False,
            n_in=int(node.metadata['n_in']), n_out=int(node.metadata['n_out']))

    def validate_config(self, node: OpNode, config: FloatMatmulConfig, _device) -> None:
        if config.transpose_lhs:
            raise NotImplementedError(f'{node.name}: float dense over a transposed input view has no kernel.')

    def pack(self, inst: ExecutionEntry) -> Dict[str, Any]:
        node, cfg = inst.node, inst.config
        fmt = cfg.precision['output'].format
        W = np.asarray(input_tensor_for_role(node, 'rhs').data, dtype=np.float64)
        W = W.reshape(-1, W.shape[-2], W.shape[-1])[-1]
        K, N = int(W.shape[0]), int(W.shape[1])
        kp = (K + 15) // 16 * 16
        stored = pack_constant_float(W.T, fmt)               # [N, K] in storage form, by the reference's packer
        values = from_storage_float(stored, fmt)             # ... and the float32 values that storage holds
        packed = np.zeros((N, kp), dtype=stored.dtype)
        packed[:, :K] = stored
        bias = optional_tensor_for_role(node, 'bias')
        b = None if bias is None else np.asarray(bias.data, dtype=np.float32).reshape(-1)
        return {'weights_kn': np.ascontiguousarray(values.T.astype(np.float32)), 'packed_weights': packed, 'packed_bias': b}

    def plan_op(self, inst: ExecutionEntry) -> Dict[str, Any]:
        node, cfg = inst.node, inst.config
        return {'kind': 'dense_f', 'name': node.name, 'lhs': input_tensor_for_role(node, 'lhs').name,
                'out': node.outputs[0].name, 'weight': f'{node.name}/weights',
                'bias': f'{node.name}/bias' if cfg.use_bias else None, 'K': cfg.n_in, 'N': cfg.n_out,
                'relu': bool(cfg.use_relu), 'dtype': cfg.precision['output'].format}


@register_variant
class CudaFloatMatmulVariant(OpImplVariant):
    variant_id = 'matmul.float.cuda.v1'
    op_type = 'matmul'
    plevel = 30

    def matches(self, node: OpNode, device) -> bool:
        return device.generation in CUDA_GENERATIONS and is_float_node(node)

    def resolve(self, node: OpNode, device, directives=None) -> FloatMatmulConfig:
        if node.traits.get('output_scale') is not None:
            raise NotImplementedError(f'{node.name}: fused output scaling is not implemented for float MatMul-family ops.')
        lhs, rhs = input_tensor_for_role(node, 'lhs'), input_tensor_for_role(node, 'rhs')
        return FloatMatmulConfig(
            precision=_float_precision(node, ('lhs', 'rhs')), use_relu=False, use_bias=False,
            transpose_lhs=_transposed(node, lhs), transpose_rhs=_transposed(node, rhs),
            n_in=int(node.metadata.get('n_in', view_shape(node, rhs, 'inputs')[-2])),
            n_out=int(node.metadata.get('n_out', view_shape(node, rhs, 'inputs')[-1])))

    def plan_op(self, inst: ExecutionEntry) -> Dict[str, Any]:
        node, cfg = inst.node, inst.config
        return {'kind': 'matmul_f', 'name': node.name, 'lhs': input_tensor_for_role(node, 'lhs').name,
                'rhs': input_tensor_for_role(node, 'rhs').name, 'out': node.outputs[0].name,
                'transpose_lhs': bool(cfg.transpose_lhs), 'transpose_rhs': bool(cfg.transpose_rhs),
                'dtype': cfg.precision['output'].format}


@dataclass(frozen=True)
class FloatAddConfig:
    precision: Dict[str, AIEDataType]
    shift: int = 0
    accumulator_tag: str = 'accfloat'
    rounding_mode: str = 'conv_even'


@register_variant
class CudaFloatAddVariant(OpImplVariant):
    variant_id = 'add.float.cuda.v1'
    op_type = 'add'
    plevel = 30

    def matches(self, node: OpNode, device) -> bool:
        return device.generation in CUDA_GENERATIONS and is_float_node(node)

    def resolve(self, node: OpNode, device, directives=None) -> FloatAddConfig:
        return FloatAddConfig(precision=_float_precision(node, ('lhs', 'rhs')))

    def plan_op(self, inst: ExecutionEntry) -> Dict[str, Any]:
        node, cfg = inst.node, inst.config
        return {'kind': 'add_f', 'name': node.name, 'lhs': input_tensor_for_role(node, 'lhs').name,
                'rhs': input_tensor_for_role(node, 'rhs').name, 'out': node.outputs[0].name,
                'dtype': cfg.precision['output'].format}
