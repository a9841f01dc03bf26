"""Quantized Softmax contracts (HCCS surrogate and accurate integer exp) for the CUDA target.

Reference: ``src/aie4ml/op_impls/families/softmax/softmax.py`` -- approximation default :34-39,
shared resolve :92-158, output dtype rule :160-163, HCCS parameters :258-285, EXP_KQ :304-349;
HCCS validation ``softmax/common.py:59-89``; last-axis-only rule ``softmax/resolver.py:20-25``.
``layout`` (linear / tiled) selects between numerically identical AIE kernels and is a no-op here.
"""

from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Any, Dict

import numpy as np

from ..ir import ExecutionEntry, OpNode, input_tensor_for_role
from ..qtypes import AIEDataType
from .base import CUDA_GENERATIONS, FamilyResolver, OpImplVariant, family_resolver, register_variant
from .precision import resolve_exact_storage_dtype
from .views import view_shape

DEFAULT_INV_SHIFT = 15
SOFTMAX_I8_VEC_SIZE = 32
EXP_ZF = 8
EXP_KQ_MAX = 32767 // 255


@dataclass(frozen=True)
class SoftmaxConfig:
    precision: Dict[str, AIEDataType]
    approximation: str
    rows: int
    cols: int
    inv_shift: int
    use_clb: bool
    param_sets: int
    exp_kq: int
    hccs: Dict[str, Any] = field(default_factory=dict, hash=False, compare=False)


def _requested_approximation(node: OpNode) -> str:
    approx = (node.directives or {}).get('approximation')
    return 'exp' if approx is None else str(approx).lower()


def _scalar_params(values, *, name: str, lo: int, hi: int) -> np.ndarray:
    arr = np.asarray(values, dtype=np.int64).reshape(-1)
    if arr.size == 0:
        raise ValueError(f'HCCS Softmax parameter {name!r} must not be empty.')
    if np.any((arr < lo) | (arr > hi)):
        raise ValueError(f'HCCS Softmax parameter {name!r} must be in [{lo}, {hi}].')
    return arr


def infer_hccs_param_sets(hccs: Dict[str, Any]) -> int:
    sizes = [int(np.asarray(hccs[k]).size) for k in ('B', 'S', 'Dmax')]
    multi = [s for s in sizes if s > 1]
    if any(s < 1 for s in sizes):
        raise ValueError('HCCS Softmax parameters must not be empty.')
    if multi and any(s != multi[0] for s in multi):
        raise ValueError(f'HCCS Softmax non-scalar parameter lengths must match, got {multi}.')
    inferred = multi[0] if multi else 1
    explicit = hccs.get('param_sets')
    sets = int(explicit) if explicit is not None else inferred
    if sets < 1:
        raise ValueError(f'HCCS Softmax param_sets must be positive, got {sets}.')
    if inferred > 1 and sets != inferred:
        raise ValueError(f'HCCS Softmax param_sets={sets} must match non-scalar parameter length {inferred}.')
    return sets


def validate_hccs_params(hccs: Dict[str, Any], *, cols: int, param_sets: int) -> None:
    """Kernel ABI constraints on B / S / Dmax (reference ``softmax/common.py:59-89``)."""
    if int(param_sets) != 1:
        raise ValueError(f'HCCS Softmax compile-time scalar parameter packing requires param_sets=1, got {param_sets}.')
    b = _scalar_params(hccs['B'], name='B', lo=0, hi=32767)
    s = _scalar_params(hccs['S'], name='S', lo=0, hi=127)
    dmax = _scalar_params(hccs['Dmax'], name='Dmax', lo=0, hi=127)
    if b.size != 1 or s.size != 1 or dmax.size != 1:
        raise ValueError('HCCS Softmax parameters must be scalars when param_sets=1.')
    floor_score = int(b[0] - s[0] * dmax[0])
    if floor_score < 0:
        raise ValueError(f'HCCS Softmax requires B - S*Dmax >= 0 for every row; got {floor_score}.')
    if floor_score * int(cols) < 256:
        raise ValueError('HCCS Softmax requires cols * (B - S*Dmax) >= 256 for reciprocal range; '
                         f'got {floor_score * int(cols)}.')
    if int(b[0]) * int(cols) > 32767:
        raise ValueError('HCCS Softmax requires cols * B <= 32767 so score sum fits int16 range.')


def exp_kq_for(input_scale: float) -> int:
    """log2(e) * input_scale in Q8: the per-unit-gap step of the integer exp."""
    return int(round(math.log2(math.e) * float(input_scale) * (1 << EXP_ZF)))


@family_resolver('softmax')
class SoftmaxFamilyResolver(FamilyResolver):
    op_type = 'softmax'

    def validate_structure(self, node, _device) -> None:
        lhs = input_tensor_for_role(node, 'lhs')
        shape = view_shape(node, lhs, 'inputs')
        if len(shape) < 2:
            raise ValueError(f'{node.name}: Softmax requires rank>=2, got {len(shape)}.')
        axis = int(node.metadata.get('axis', len(shape) - 1))
        if axis < 0:
            axis += len(shape)
        if axis != len(shape) - 1:
            raise ValueError(f'{node.name}: Softmax is implemented over the last axis only, got axis={axis}.')
        approx = _requested_approximation(node)
        if approx not in ('exp', 'hccs'):
            raise ValueError(f'{node.name}: unknown softmax approximation {approx!r}; expected exp or hccs.')


@register_variant
class CudaSoftmaxVariant(OpImplVariant):
    """int8 in -> uint8 / int16 out row softmax; one kernel, two score functions."""

    variant_id = 'softmax.i8.cuda.v1'
    op_type = 'softmax'

    def matches(self, node: OpNode, device) -> bool:
        if device.generation not in CUDA_GENERATIONS:
            return False
        lhs = input_tensor_for_role(node, 'lhs')
        if lhs.precision is None:
            return False
        return resolve_exact_storage_dtype(lhs.precision, namespace='lhs', layer_name=node.name).format == 'int8'

    def resolve(self, node: OpNode, device, directives=None) -> SoftmaxConfig:
        directives = directives if directives is not None else (node.directives or {})
        lhs = input_tensor_for_role(node, 'lhs')
        precision = {
            'lhs': resolve_exact_storage_dtype(lhs.precision, namespace='lhs', layer_name=node.name),
            'output': resolve_exact_storage_dtype(node.outputs[0].precision, namespace='output', layer_name=node.name),
        }
        shape = view_shape(node, lhs, 'inputs')
        cols = int(shape[-1])
        rows = int(np.prod(shape[:-1], dtype=np.int64))
        if cols % SOFTMAX_I8_VEC_SIZE != 0:
            raise ValueError(f'{node.name}: softmax axis length {cols} must be a multiple of '
                             f'vec_size={SOFTMAX_I8_VEC_SIZE}; pad the softmax dimension before lowering.')
        approx = _requested_approximation(node)
        temperature = float(node.trait_data('input_scale').get('scale', 1.0))
        if approx == 'hccs':
            hccs = dict(directives.get('hccs', {}) or {})
            missing = [k for k in ('B', 'S', 'Dmax') if k not in hccs]
            if missing:
                raise ValueError(f'{node.name}: HCCS Softmax directives missing {", ".join(missing)}.')
            if abs(temperature - 1.0) > 1e-9:
                raise ValueError(
                    f'{node.name}: {self.variant_id} cannot apply a runtime input_scale={temperature}; bake the '
                    'softmax temperature into the HCCS B/S/Dmax calibration, or drop the approximation directive '
                    'to use the accurate exp Softmax, which applies input_scale directly.')
            return SoftmaxConfig(precision=precision, approximation='hccs', rows=rows, cols=cols,
                                 inv_shift=int(hccs.get('inv_shift', DEFAULT_INV_SHIFT)),
                                 use_clb=bool(hccs.get('use_clb', False)),
                                 param_sets=infer_hccs_param_sets(hccs), exp_kq=0, hccs=hccs)
        input_scale = (2.0 ** -int(precision['lhs'].frac)) * temperature
        return SoftmaxConfig(precision=precision, approximation='exp', rows=rows, cols=cols,
                             inv_shift=DEFAULT_INV_SHIFT, use_clb=False, param_sets=1,
                             exp_kq=exp_kq_for(input_scale), hccs={})

    def validate_config(self, node: OpNode, config: SoftmaxConfig, _device) -> None:
        out_format = config.precision['output'].format
        if out_format not in ('uint8', 'int16'):
            raise ValueError(f'{node.name}: {self.variant_id} requires uint8 or int16 output, got {out_format!r}.')
        if config.approximation == 'hccs':
            if config.param_sets != 1:
                raise ValueError(f'{node.name}: {self.variant_id} does not support multi-head '
                                 f'param_sets={config.param_sets}; lower attention to one Softmax op per head.')
            if not 1 <= int(config.inv_shift) <= 30:
                raise ValueError(f'{node.name}: HCCS Softmax inv_shift must be in [1, 30], got {config.inv_shift}.')
            try:
                validate_hccs_params(config.hccs, cols=config.cols, param_sets=config.param_sets)
            except ValueError as exc:
                raise ValueError(f'{node.name}: {exc}') from None
        else:
            if not 1 <= int(config.exp_kq) <= EXP_KQ_MAX:
                raise ValueError(
                    f'{node.name}: exp Softmax needs 1 <= EXP_KQ <= {EXP_KQ_MAX}, got {config.exp_kq}. The input '
                    'fixed-point scale is out of range (roughly frac in [2, 9]): too fine and every logit gap '
                    'rounds to zero; too coarse and (max-x)*KQ overflows int16. Requantise the softmax input.')

    def plan_op(self, inst: ExecutionEntry) -> Dict[str, Any]:
        node, cfg = inst.node, inst.config
        op = {
            'kind': 'softmax', 'name': node.name, 'lhs': input_tensor_for_role(node, 'lhs').name,
            'out': node.outputs[0].name, 'approximation': cfg.approximation, 'cols': cfg.cols,
            'inv_shift': int(cfg.inv_shift), 'use_clb': bool(cfg.use_clb), 'exp_kq': int(cfg.exp_kq),
            'B': 0, 'S': 0, 'Dmax': 0, 'out_dtype': cfg.precision['output'].format,
        }
        if cfg.approximation == 'hccs':
            for key in ('B', 'S', 'Dmax'):
                op[key] = int(np.asarray(cfg.hccs[key]).reshape(-1)[0])
        return op
