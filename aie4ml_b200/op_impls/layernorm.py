"""Integer LayerNorm contract for the CUDA target.

Reference: ``src/aie4ml/op_impls/families/layernorm/layer_norm.py`` -- EPS_Q0 :40-61, dtype gate
:78-88, resolve :94-167, validate :169-175; parameter quantisation
``layernorm/common.py:36-93`` (gamma int16 Q7, beta int16 Q15, ``np.rint``, range-checked).
"""

from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Any, Dict

import numpy as np

from ..ir import ExecutionEntry, OpNode, input_tensor_for_role
from ..qtypes import AIEDataType
from .base import CUDA_GENERATIONS, FamilyResolver, OpImplVariant, family_resolver, register_variant
from .precision import aie_rounding_token, resolve_exact_storage_dtype, to_quant_intent
from .views import view_shape

GAMMA_FRAC_BITS = 7
BETA_FRAC_BITS = 15
LAYERNORM_VEC_SIZE = 32


@dataclass(frozen=True)
class LayerNormConfig:
    precision: Dict[str, AIEDataType]
    rows: int
    cols: int
    gamma_shift: int
    out_shift: int
    eps_q0: int
    rounding_mode: str


def _resolve_eps_q0(node_name: str, metadata: dict, input_frac: int) -> int:
    if 'epsilon' in metadata:
        epsilon = float(metadata['epsilon'])
        if epsilon < 0.0:
            raise ValueError(f'{node_name}: LayerNormalization epsilon must be non-negative, got {epsilon}.')
        exact = epsilon * float(1 << (2 * int(input_frac)))
        eps_q0 = int(round(exact))
        if not math.isclose(exact, float(eps_q0), rel_tol=0.0, abs_tol=1e-6):
            raise ValueError(f'{node_name}: epsilon={epsilon} is not exactly representable as integer EPS_Q0 '
                             f'for input frac={input_frac} (epsilon / input_scale^2 = {exact}).')
        if eps_q0 < 1:
            raise ValueError(f'{node_name}: epsilon={epsilon} maps to EPS_Q0={eps_q0}; '
                             'integer LayerNorm requires a positive variance floor.')
        return eps_q0
    eps_q0 = int(metadata.get('eps_q0', 1))
    if eps_q0 < 1:
        raise ValueError(f'{node_name}: eps_q0 must be positive, got {eps_q0}.')
    return eps_q0


def pack_layernorm_param(values, *, name: str, full_inner: int, frac: int) -> np.ndarray:
    """Quantise gamma (Q7) or beta (Q15) to int16 with round-half-even; out-of-range is an error."""
    arr = np.asarray(values, dtype=np.float64).reshape(-1)
    if arr.shape[0] != int(full_inner):
        raise ValueError(f'LayerNorm parameter {name!r} length {arr.shape[0]} does not match '
                         f'full_inner={int(full_inner)}.')
    if not np.all(np.isfinite(arr)):
        raise ValueError(f'LayerNorm parameter {name!r} contains non-finite values.')
    scale = float(1 << int(frac)) if frac > 0 else 1.0
    codes = np.rint(arr * scale).astype(np.int64)
    if np.any((codes < -32768) | (codes > 32767)):
        raise ValueError(f'LayerNorm parameter {name!r} cannot be represented as signed int16 Q{int(frac)}: '
                         f'value range [{float(arr.min())}, {float(arr.max())}], representable range '
                         f'[{-32768 / scale}, {32767 / scale}].')
    return codes.astype(np.int16)


@family_resolver('layer_norm')
class LayerNormFamilyResolver(FamilyResolver):
    op_type = 'layer_norm'

    def validate_structure(self, node, _device) -> None:
        lhs = input_tensor_for_role(node, 'lhs')
        shape = view_shape(node, lhs, 'inputs')
        if len(shape) < 2:
            raise ValueError(f'{node.name}: LayerNorm requires rank>=2, got {len(shape)}.')
        axis = int(node.metadata.get('axis', len(shape) - 1))
        if axis < 0:
            axis += len(shape)
        if axis != len(shape) - 1:
            raise ValueError(f'{node.name}: LayerNorm is implemented over the last axis only, got axis={axis}.')
        input_tensor_for_role(node, 'gamma')
        input_tensor_for_role(node, 'beta')


@register_variant
class CudaLayerNormVariant(OpImplVariant):
    """int8 -> int8 integer LayerNorm over a power-of-two last axis."""

    variant_id = 'layer_norm.i8.cuda.v1'
    op_type = 'layer_norm'

    def matches(self, node: OpNode, device) -> bool:
        if device.generation not in CUDA_GENERATIONS:
            return False
        lhs = input_tensor_for_role(node, 'lhs')
        if lhs.precision is None or node.outputs[0].precision is None:
            return False
        i = resolve_exact_storage_dtype(lhs.precision, namespace='lhs', layer_name=node.name)
        o = resolve_exact_storage_dtype(node.outputs[0].precision, namespace='output', layer_name=node.name)
        return i.format == 'int8' and o.format == 'int8'

    def resolve(self, node: OpNode, device, directives=None) -> LayerNormConfig:
        lhs = input_tensor_for_role(node, 'lhs')
        out = node.outputs[0]
        precision = {
            'lhs': resolve_exact_storage_dtype(lhs.precision, namespace='lhs', layer_name=node.name),
            'output': resolve_exact_storage_dtype(out.precision, namespace='output', layer_name=node.name),
            'gamma': AIEDataType(format='int16', frac=GAMMA_FRAC_BITS),
            'beta': AIEDataType(format='int16', frac=BETA_FRAC_BITS),
        }
        shape = view_shape(node, lhs, 'inputs')
        cols = int(shape[-1])
        if cols % LAYERNORM_VEC_SIZE != 0:
            raise ValueError(f'{node.name}: full_inner={cols} must be a multiple of vec_size={LAYERNORM_VEC_SIZE}; '
                             'pad the inner dimension before LayerNorm.')
        return LayerNormConfig(
            precision=precision,
            rows=int(np.prod(shape[:-1], dtype=np.int64)),
            cols=cols,
            gamma_shift=GAMMA_FRAC_BITS,
            out_shift=int(to_quant_intent(out.precision).frac),
            eps_q0=_resolve_eps_q0(node.name, node.metadata, int(precision['lhs'].frac)),
            rounding_mode=aie_rounding_token(precision['output']),
        )

    def validate_config(self, node: OpNode, config: LayerNormConfig, _device) -> None:
        if config.cols <= 0 or (config.cols & (config.cols - 1)) != 0:
            raise ValueError(f'{node.name}: cols={config.cols} must be a power of two.')
        if not 0 <= config.out_shift <= 15:
            raise ValueError(f'{node.name}: out_shift={config.out_shift} must be in [0, 15]; '
                             'integer LayerNorm cannot left-shift or exceed NORM_SHIFT=15.')

    def pack(self, inst: ExecutionEntry) -> Dict[str, Any]:
        cfg = inst.config
        gamma = input_tensor_for_role(inst.node, 'gamma')
        beta = input_tensor_for_role(inst.node, 'beta')
        return {
            'packed_gamma': pack_layernorm_param(gamma.data, name='gamma', full_inner=cfg.cols, frac=GAMMA_FRAC_BITS),
            'packed_beta': pack_layernorm_param(beta.data, name='beta', full_inner=cfg.cols, frac=BETA_FRAC_BITS),
        }

    def plan_op(self, inst: ExecutionEntry) -> Dict[str, Any]:
        node, cfg = inst.node, inst.config
        return {
            'kind': 'layer_norm', 'name': node.name, 'lhs': input_tensor_for_role(node, 'lhs').name,
            'out': node.outputs[0].name, 'gamma': f'{node.name}/gamma', 'beta': f'{node.name}/beta',
            'cols': cfg.cols, 'eps_q0': int(cfg.eps_q0), 'out_shift': int(cfg.out_shift),
            'rounding': cfg.rounding_mode, 'out_dtype': cfg.precision['output'].format,
        }
