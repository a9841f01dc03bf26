"""Numeric resolution rules shared by every op family.

Reference: ``src/aie4ml/op_impls/utils/precision.py`` -- ROUNDING_TOKEN_MAP :13-21,
resolve_exact_storage_dtype :64-71, infer_accumulator_tag :74-127,
resolve_accumulator_output_shift :138-150.
"""

from __future__ import annotations

from typing import Any, Dict, Optional

from ..qtypes import AIEDataType, FloatIntent, QuantIntent, RoundingMode

ROUNDING_TOKEN_MAP: Dict[RoundingMode, str] = {
    RoundingMode.TRN: 'floor',
    RoundingMode.RND_MIN_INF: 'floor',
    RoundingMode.RND_INF: 'ceil',
    RoundingMode.RND: 'symmetric_inf',
    RoundingMode.TRN_ZERO: 'symmetric_zero',
    RoundingMode.RND_ZERO: 'symmetric_zero',
    RoundingMode.RND_CONV: 'conv_even',
    RoundingMode.RND_HALF_UP: 'positive_inf',
}

# Codes the C ABI takes for a rounding token.
ROUNDING_CODE = {'floor': 0, 'ceil': 1, 'positive_inf': 2, 'negative_inf': 3, 'symmetric_inf': 4,
                 'symmetric_zero': 5, 'conv_even': 6, 'conv_odd': 7}
# Codes the C ABI takes for an element type.
DTYPE_CODE = {'int8': 0, 'uint8': 1, 'int16': 2}
# Codes the floating-point entry points take.
FLOAT_CODE = {'bfloat16': 0, 'float32': 1, 'fp8_e4m3': 2}


def to_quant_intent(precision: Any) -> QuantIntent:
    if isinstance(precision, QuantIntent):
        return precision
    if isinstance(precision, AIEDataType):
        return QuantIntent(width=precision.width, frac=precision.frac, signed=precision.signed,
                           rounding=precision.rounding, saturation=precision.saturation)
    raise TypeError(f'Unsupported precision representation {type(precision)}')


def resolve_exact_storage_dtype(precision: Any, *, namespace: str, layer_name: str) -> AIEDataType:
    """Narrowest of 8/16/32-bit storage that holds the intent's width, keeping frac/rounding/saturation."""
    if precision is None:
        raise ValueError(f'{layer_name}: missing precision metadata for {namespace}.')
    if isinstance(precision, FloatIntent):
        return AIEDataType(format=precision.format.value, frac=0)
    intent = to_quant_intent(precision)
    width = int(intent.width)
    if width <= 0:
        raise ValueError(f'{layer_name}: invalid {namespace} width {width}.')
    for bits in (8, 16, 32):
        if width <= bits:
            return AIEDataType(format=f'{"int" if intent.signed else "uint"}{bits}', frac=int(intent.frac),
                               rounding=intent.rounding, saturation=intent.saturation)
    raise ValueError(f'{layer_name}: {namespace} width {width} exceeds supported widths (8, 16, 32).')


def infer_accumulator_tag(lhs: Optional[AIEDataType], rhs: Optional[AIEDataType]) -> str:
    """acc32 for 8x8 and 16x8, acc64 otherwise (the AIE-ML table of the reference, :116-127)."""
    lw, rw = int(lhs.width), int(rhs.width)
    if max(lw, rw) <= 8 or {lw, rw} == {8, 16}:
        return 'acc32'
    if max(lw, rw) <= 32:
        return 'acc64'
    raise ValueError(f'No accumulator tag for lhs {lw}-bit and rhs {rw}-bit precisions.')


def aie_rounding_token(source: Any) -> str:
    mode = getattr(source, 'rounding', None) or RoundingMode.TRN
    try:
        return ROUNDING_TOKEN_MAP[mode]
    except KeyError:
        raise ValueError(f'Unsupported rounding mode {mode} for a kernel.') from None


def resolve_accumulator_output_shift(lhs_precision: Any, output_precision: Any, rhs_precision: Any = None) -> int:
    """Right shift from accumulator fixed point to output fixed point:
    ``max(0, lhs.frac + rhs.frac - out.frac)`` (rhs.frac = 0 for elementwise add)."""
    lhs_frac = to_quant_intent(lhs_precision).frac
    out_frac = to_quant_intent(output_precision).frac
    rhs_frac = to_quant_intent(rhs_precision).frac if rhs_precision is not None else 0
    return max(0, int(lhs_frac + rhs_frac - out_frac))
