"""Exact-shape elementwise Add contract for the CUDA target.

Reference: ``src/aie4ml/op_impls/families/elementwise/resolver.py:14-33`` (lhs, rhs and output must
share one storage type and shape; rank >= 2; no broadcast) and ``elementwise/add.py:57-164``
(shift :150, rounding token :152).  With equal types the shift is 0: a saturating add.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict

from ..ir import ExecutionEntry, OpNode, input_tensor_for_role
from ..qtypes import AIEDataType
from .base import CUDA_GENERATIONS, FamilyResolver, OpImplVariant, family_resolver, register_variant
from .precision import aie_rounding_token, resolve_accumulator_output_shift, resolve_exact_storage_dtype
from .views import view_shape


@dataclass(frozen=True)
class AddConfig:
    precision: Dict[str, AIEDataType]
    shift: int
    accumulator_tag: str
    rounding_mode: str


@family_resolver('add')
class AddFamilyResolver(FamilyResolver):
    op_type = 'add'

    def validate_structure(self, node, _device) -> None:
        lhs = input_tensor_for_role(node, 'lhs')
        rhs = input_tensor_for_role(node, 'rhs')
        if lhs.is_parameter or rhs.is_parameter:
            raise NotImplementedError(f'{node.name}: a constant addend is only supported as a dense bias '
                                      '(there is no standalone constant-add kernel).')
        lhs_shape = tuple(view_shape(node, lhs, 'inputs'))
        rhs_shape = tuple(view_shape(node, rhs, 'inputs'))
        if len(lhs_shape) < 2:
            raise ValueError(f'{node.name}: elementwise Add requires rank>=2, got {len(lhs_shape)}.')
        if lhs_shape != rhs_shape:
            raise ValueError(f'{node.name}: elementwise Add requires exact-shape inputs, got {lhs_shape} and '
                             f'{rhs_shape}.')
        types = [resolve_exact_storage_dtype(t.precision, namespace=ns, layer_name=node.name)
                 for t, ns in ((lhs, 'lhs'), (rhs, 'rhs'), (node.outputs[0], 'output'))]
        if types[0] != types[1] or types[0] != types[2]:
            raise ValueError(f'{node.name}: elementwise Add requires lhs/rhs/output to use the same storage type.')


@register_variant
class CudaAddVariant(OpImplVariant):
    variant_id = 'add.cuda.v1'
    op_type = 'add'

    def matches(self, node: OpNode, device) -> bool:
        from ..qtypes import FloatIntent

        return (device.generation in CUDA_GENERATIONS
                and not isinstance(input_tensor_for_role(node, 'lhs').precision, FloatIntent))

    def resolve(self, node: OpNode, device, directives=None) -> AddConfig:
        lhs = input_tensor_for_role(node, 'lhs')
        rhs = input_tensor_for_role(node, 'rhs')
        precision = {
            'lhs': resolve_exact_storage_dtype(lhs.precision, namespace='lhs', layer_name=node.name),
            'rhs': resolve_exact_storage_dtype(rhs.precision, namespace='rhs', layer_name=node.name),
            'output': resolve_exact_storage_dtype(node.outputs[0].precision, namespace='output', layer_name=node.name),
        }
        return AddConfig(precision=precision,
                         shift=resolve_accumulator_output_shift(lhs.precision, node.outputs[0].precision),
                         accumulator_tag='acc32', rounding_mode=aie_rounding_token(precision['output']))

    def validate_config(self, node: OpNode, config: AddConfig, _device) -> None:
        if config.precision['output'].format not in ('int8', 'uint8', 'int16'):
            raise ValueError(f'{node.name}: Add supports int8, uint8 and int16 tensors, got '
                             f'{config.precision["output"].format!r}.')

    def plan_op(self, inst: ExecutionEntry) -> Dict[str, Any]:
        node, cfg = inst.node, inst.config
        return {
            'kind': 'add', 'name': node.name, 'lhs': input_tensor_for_role(node, 'lhs').name,
            'rhs': input_tensor_for_role(node, 'rhs').name, 'out': node.outputs[0].name,
            'shift': int(cfg.shift), 'rounding': cfg.rounding_mode, 'out_dtype': cfg.precision['output'].format,
        }
