"""Dense and dynamic-MatMul contracts for the CUDA target.

Numeric rules follow the reference's matmul family: dtype resolution and accumulator tag
(``src/aie4ml/op_impls/families/matmul/resolver.py:110-144``), bias dtype (:147-157), folded
power-of-two output scale (:160-175), the rank contract (:440-463), DenseConfig / MatmulConfig
fields (``config.py:36-58``), shift and flags (``dense.py:94-133``, ``matmul.py:47-98``), weight and
bias quantisation (``dense.py:135-171``).  The AIE tiling / cascade / staging search
(resolver.py:178-362) is replaced by the CUDA kernels' own tiling and is absent.

Packing lays constants out for the kernels: weights as int8 ``[N, Kp]`` (K contiguous, row
pitch padded to 16 bytes so a TMA descriptor can address it), bias as int32 ``[N]``.
"""

from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Any, Dict, Optional

import numpy as np

from ..ir import ExecutionEntry, OpNode, input_tensor_for_role, optional_tensor_for_role
from ..qtypes import FLOAT_FORMATS, AIEDataType
from ..quant_utils import quantize_to_int
from .base import CUDA_GENERATIONS, FamilyResolver, OpImplVariant, family_resolver, register_variant
from .precision import (
    aie_rounding_token,
    infer_accumulator_tag,
    resolve_accumulator_output_shift,
    resolve_exact_storage_dtype,
    to_quant_intent,
)
from .views import is_identity, is_last_two_swap, view_perm, view_shape


@dataclass(frozen=True)
class DenseFlags:
    use_relu: bool
    transpose_lhs: bool
    use_bias: bool


@dataclass(frozen=True)
class MatmulFlags:
    transpose_lhs: bool
    transpose_rhs: bool


@dataclass(frozen=True)
class DenseConfig:
    precision: Dict[str, AIEDataType]
    shift: int
    accumulator_tag: str
    rounding_mode: str
    flags: DenseFlags
    n_in: int
    n_out: int


@dataclass(frozen=True)
class MatmulConfig:
    precision: Dict[str, AIEDataType]
    shift: int
    accumulator_tag: str
    rounding_mode: str
    flags: MatmulFlags
    n_in: int
    n_out: int


def _resolve_numeric(node: OpNode) -> Dict[str, AIEDataType]:
    lhs = input_tensor_for_role(node, 'lhs')
    rhs = input_tensor_for_role(node, 'rhs')
    out = node.outputs[0]
    if any(t.precision is None for t in (lhs, rhs, out)):
        raise ValueError(f'{node.name}: missing precision metadata for {node.op_type}.')
    resolved = {
        'lhs': resolve_exact_storage_dtype(lhs.precision, namespace='lhs', layer_name=node.name),
        'rhs': resolve_exact_storage_dtype(rhs.precision, namespace='rhs', layer_name=node.name),
        'output': resolve_exact_storage_dtype(out.precision, namespace='output', layer_name=node.name),
    }
    if resolved['lhs'].width <= 8 and resolved['rhs'].width > 8:
        raise RuntimeError(f'{node.name}: unsupported int8 x int16 precision mix; no implementation variant available.')
    tag = infer_accumulator_tag(resolved['lhs'], resolved['rhs'])
    resolved['acc'] = AIEDataType(format='int32' if tag == 'acc32' else 'int64',
                                  frac=int(resolved['lhs'].frac + resolved['rhs'].frac))
    return resolved


def _resolve_bias_dtype(node: OpNode, precision: Dict[str, AIEDataType]) -> AIEDataType:
    frac = int(precision['lhs'].frac) + int(precision['rhs'].frac)
    bias = optional_tensor_for_role(node, 'bias')
    if bias is not None and bias.precision is not None:
        intent = to_quant_intent(bias.precision)
        return AIEDataType(format='int32', frac=frac, rounding=intent.rounding, saturation=intent.saturation)
    return AIEDataType(format='int32', frac=frac)


def _resolve_output_scale_shift(node: OpNode) -> int:
    trait = node.traits.get('output_scale')
    if trait is None:
        return 0
    scale = float(trait.data['scale'])
    if scale <= 0.0 or scale > 1.0:
        raise ValueError(f'{node.name}: fused output scale must be in the range (0, 1], got {scale}.')
    shift = int(round(-math.log2(scale)))
    if not math.isclose(scale, math.ldexp(1.0, -shift), rel_tol=0.0, abs_tol=1e-12):
        raise NotImplementedError(f'{node.name}: fused output scale {scale} is not a power of two; '
                                  'fixed-point multiplier scaling is not implemented.')
    return shift


def _validate_rank_contract(node: OpNode, *, allow_batched_rhs: bool) -> None:
    lhs = input_tensor_for_role(node, 'lhs')
    rhs = input_tensor_for_role(node, 'rhs')
    lhs_shape = tuple(view_shape(node, lhs, 'inputs'))
    rhs_shape = tuple(view_shape(node, rhs, 'inputs'))
    if len(lhs_shape) < 2:
        raise ValueError(f'{node.name}: {node.op_type}.v1 requires rank>=2 LHS tensors, got {lhs_shape}.')
    if len(rhs_shape) < 2:
        raise ValueError(f'{node.name}: {node.op_type}.v1 requires rank>=2 RHS tensors, got {rhs_shape}.')
    if lhs_shape[-1] != rhs_shape[-2]:
        raise ValueError(f'{node.name}: contraction mismatch, lhs {lhs_shape} vs rhs {rhs_shape}.')
    rhs_batch = rhs_shape[:-2]
    if rhs_batch and any(d != 1 for d in rhs_batch):
        # The reference rejects this outright (one KxN matrix per op).  The CUDA matmul kernel is
        # batched: it applies the same rank-2 contract to every leading index, so a batched RHS is
        # accepted when its leading axes equal the LHS's.
        if not allow_batched_rhs or tuple(rhs_batch) != tuple(lhs_shape[:-2]):
            raise ValueError(f'{node.name}: {node.op_type}.v1 does not support batched RHS with leading axes '
                             f'{rhs_batch} against lhs shape {lhs_shape}.')


@family_resolver('dense')
class DenseFamilyResolver(FamilyResolver):
    op_type = 'dense'

    def validate_structure(self, node, _device) -> None:
        _validate_rank_contract(node, allow_batched_rhs=False)


@family_resolver('matmul')
class MatmulFamilyResolver(FamilyResolver):
    op_type = 'matmul'

    def validate_structure(self, node, _device) -> None:
        _validate_rank_contract(node, allow_batched_rhs=True)
        rhs = input_tensor_for_role(node, 'rhs')
        if rhs.is_parameter and len(rhs.shape) == 2:
            raise ValueError(f'{node.name}: a constant rank-2 RHS lowers to dense, not matmul.')


def _bitwidths_supported(node: OpNode) -> bool:
    try:
        p = _resolve_numeric(node)
    except (ValueError, RuntimeError):
        return False
    if p['lhs'].format in FLOAT_FORMATS or p['rhs'].format in FLOAT_FORMATS:
        return False   # the float-simulation variants take those
    # the reference's width table (families/matmul/common.py:52); 16-bit operands are signed
    if (p['lhs'].width, p['rhs'].width) not in ((8, 8), (16, 8), (16, 16)) or not p['rhs'].signed:
        return False
    return p['lhs'].width == 8 or p['lhs'].signed


def _shift_for(node: OpNode) -> int:
    lhs = input_tensor_for_role(node, 'lhs')
    rhs = input_tensor_for_role(node, 'rhs')
    shift = resolve_accumulator_output_shift(lhs.precision, node.outputs[0].precision, rhs.precision)
    return shift + _resolve_output_scale_shift(node)


def _transposed(node: OpNode, tensor) -> bool:
    perm = view_perm(node, tensor, 'inputs')
    if is_identity(perm):
        return False
    if is_last_two_swap(perm):
        return True
    raise ValueError(f'{node.name}: only a swap of the last two axes is executable, got io_view perm {perm} '
                     f'on {tensor.name!r}.')


@register_variant
class CudaDenseVariant(OpImplVariant):
    """int8 x int8 -> int32 Dense with fused bias, requantise (rounding shift + saturate) and ReLU."""

    variant_id = 'dense.b.r.cuda.v1'
    op_type = 'dense'

    def matches(self, node: OpNode, device) -> bool:
        return device.generation in CUDA_GENERATIONS and _bitwidths_supported(node)

    def resolve(self, node: OpNode, device, directives=None) -> DenseConfig:
        precision = _resolve_numeric(node)
        precision['bias'] = _resolve_bias_dtype(node, precision)
        fused = node.traits.get('fused_activation')
        use_relu = ((fused.data.get('activation') if fused else '') or '').lower() == 'relu'
        lhs = input_tensor_for_role(node, 'lhs')
        return DenseConfig(
            precision=precision,
            shift=_shift_for(node),
            accumulator_tag=infer_accumulator_tag(precision['lhs'], precision['rhs']),
            rounding_mode=aie_rounding_token(precision['output']),
            flags=DenseFlags(use_relu=use_relu, transpose_lhs=_transposed(node, lhs),
                             use_bias=bool(node.metadata.get('use_bias'))),
            n_in=int(node.metadata['n_in']),
            n_out=int(node.metadata['n_out']),
        )

    def validate_config(self, node: OpNode, config: DenseConfig, _device) -> None:
        if config.shift < 0:
            raise ValueError(f'{node.name}: dense accumulator output shift must be non-negative, got {config.shift}.')
        limit = 62 if config.accumulator_tag == 'acc64' else 31
        if config.shift > limit:
            raise ValueError(f'{node.name}: dense accumulator output shift {config.shift} exceeds the '
                             f'{limit + 1}-bit accumulator.')
        if config.precision['output'].format not in ('int8', 'uint8', 'int16'):
            raise ValueError(f'{node.name}: dense output must be int8, uint8 or int16, got '
                             f'{config.precision["output"].format!r}.')

    def _quantize_weight_bias(self, inst: ExecutionEntry):
        node = inst.node
        lhs = input_tensor_for_role(node, 'lhs')
        weight = input_tensor_for_role(node, 'rhs')
        bias = optional_tensor_for_role(node, 'bias')
        wi = to_quant_intent(weight.precision)
        W = quantize_to_int(weight.data, wi.frac, wi.width, signed=wi.signed, rounding_mode=wi.rounding,
                            saturation_mode=wi.saturation)
        b = None
        if bias is not None:
            bi = to_quant_intent(bias.precision)
            accum_frac = to_quant_intent(lhs.precision).frac + wi.frac
            b = quantize_to_int(bias.data, accum_frac, 32, signed=bi.signed, rounding_mode=bi.rounding,
                                saturation_mode=bi.saturation)
        W = np.asarray(W)
        if W.ndim < 2:
            raise ValueError(f'{inst.name}: weight matrix must have at least 2 dimensions, got {W.ndim}.')
        return W.reshape(-1, W.shape[-2], W.shape[-1])[-1], b

    def pack(self, inst: ExecutionEntry) -> Dict[str, Any]:
        W, b = self._quantize_weight_bias(inst)
        K, N = int(W.shape[0]), int(W.shape[1])
        kp = (K + 15) // 16 * 16
        wdt = np.int16 if inst.config.precision['rhs'].width > 8 else np.int8
        packed = np.zeros((N, kp), dtype=wdt)
        packed[:, :K] = W.T.astype(wdt)
        out = {'weights_kn': W.astype(wdt), 'packed_weights': packed}
        out['packed_bias'] = None if b is None else np.asarray(b, dtype=np.int32).reshape(-1)
        return out

    def plan_op(self, inst: ExecutionEntry) -> Dict[str, Any]:
        node, cfg = inst.node, inst.config
        return {
            'kind': 'dense', 'name': node.name,
            'lhs': input_tensor_for_role(node, 'lhs').name, 'out': node.outputs[0].name,
            'weight': f'{node.name}/weights', 'bias': f'{node.name}/bias' if cfg.flags.use_bias else None,
            'K': cfg.n_in, 'N': cfg.n_out, 'shift': int(cfg.shift), 'rounding': cfg.rounding_mode,
            'relu': bool(cfg.flags.use_relu), 'transpose_lhs': bool(cfg.flags.transpose_lhs),
            'lhs_dtype': cfg.precision['lhs'].format, 'rhs_dtype': cfg.precision['rhs'].format,
            'out_dtype': cfg.precision['output'].format, 'acc_bits': 64 if cfg.accumulator_tag == 'acc64' else 32,
        }


@register_variant
class CudaMatmulVariant(OpImplVariant):
    """Dynamic (both operands runtime tensors) batched int8 MatMul with requantise."""

    variant_id = 'matmul.cuda.v1'
    op_type = 'matmul'

    def matches(self, node: OpNode, device) -> bool:
        return device.generation in CUDA_GENERATIONS and _bitwidths_supported(node)

    def resolve(self, node: OpNode, device, directives=None) -> MatmulConfig:
        precision = _resolve_numeric(node)
        lhs = input_tensor_for_role(node, 'lhs')
        rhs = input_tensor_for_role(node, 'rhs')
        return MatmulConfig(
            precision=precision,
            shift=_shift_for(node),
            accumulator_tag=infer_accumulator_tag(precision['lhs'], precision['rhs']),
            rounding_mode=aie_rounding_token(precision['output']),
            flags=MatmulFlags(transpose_lhs=_transposed(node, lhs), transpose_rhs=_transposed(node, rhs)),
            n_in=int(node.metadata.get('n_in', view_shape(node, rhs, 'inputs')[-2])),
            n_out=int(node.metadata.get('n_out', view_shape(node, rhs, 'inputs')[-1])),
        )

    def validate_config(self, node: OpNode, config: MatmulConfig, _device) -> None:
        if not config.precision['rhs'].signed:
            raise ValueError(f'{node.name}: matmul RHS must use a signed integer precision.')
        if not 0 <= config.shift <= 31:
            raise ValueError(f'{node.name}: matmul output shift must be in [0, 31], got {config.shift}.')
        if config.precision['output'].format not in ('int8', 'uint8', 'int16'):
            raise ValueError(f'{node.name}: matmul output must be int8, uint8 or int16.')

    def plan_op(self, inst: ExecutionEntry) -> Dict[str, Any]:
        node, cfg = inst.node, inst.config
        return {
            'kind': 'matmul', 'name': node.name,
            'lhs': input_tensor_for_role(node, 'lhs').name, 'rhs': input_tensor_for_role(node, 'rhs').name,
            'out': node.outputs[0].name, 'shift': int(cfg.shift), 'rounding': cfg.rounding_mode,
            'transpose_lhs': bool(cfg.flags.transpose_lhs), 'transpose_rhs': bool(cfg.flags.transpose_rhs),
            'lhs_dtype': cfg.precision['lhs'].format, 'rhs_dtype': cfg.precision['rhs'].format,
            'out_dtype': cfg.precision['output'].format, 'acc_bits': 64 if cfg.accumulator_tag == 'acc64' else 32,
        }
