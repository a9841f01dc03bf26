"""Host-side fixed-point helpers used at graph boundaries and when constants are packed.

Behaviour matches the reference's ``src/aie4ml/quant_utils.py`` (apply_rounding :48-61,
handle_overflow :64-89, dtype_for_precision :15-35) and ``quantize_to_int``
(``op_impls/families/matmul/common.py:287-304``).
"""

from __future__ import annotations

import numpy as np

from .qtypes import RoundingMode, SaturationMode

_SIGNED = ((8, np.int8), (16, np.int16), (32, np.int32), (64, np.int64))
_UNSIGNED = ((8, np.uint8), (16, np.uint16), (32, np.uint32), (64, np.uint64))


def dtype_for_precision(width, signed: bool):
    """Smallest NumPy integer dtype holding ``width`` bits (int32 when width is unknown)."""
    if width is None:
        return np.int32
    for bits, dt in (_SIGNED if signed else _UNSIGNED):
        if int(width) <= bits:
            return dt
    return np.int64 if signed else np.uint64


def apply_rounding(values, mode: RoundingMode):
    values = np.asarray(values, dtype=np.float64)
    if mode in (RoundingMode.TRN, RoundingMode.RND_MIN_INF):
        return np.floor(values)
    if mode in (RoundingMode.TRN_ZERO, RoundingMode.RND_ZERO):
        return np.trunc(values)
    if mode is RoundingMode.RND_INF:
        return np.ceil(values)
    if mode is RoundingMode.RND_CONV:
        return np.round(values)
    if mode is RoundingMode.RND:
        away = np.ceil(values - 0.5)
        return np.where(values >= 0, np.floor(values + 0.5), away)
    if mode is RoundingMode.RND_HALF_UP:
        return np.floor(values + 0.5)
    raise ValueError(f'Unsupported rounding mode {mode}')


def handle_overflow(values, width: int, signed: bool, mode: SaturationMode):
    values = np.asarray(values)
    hi = (1 << (width - 1)) - 1 if signed else (1 << width) - 1
    lo = -(1 << (width - 1)) if signed else 0
    if mode is SaturationMode.WRAP:
        out = np.mod(values, 1 << width)
        return np.where(out > hi, out - (1 << width), out) if signed else out
    if mode is SaturationMode.SAT:
        return np.clip(values, lo, hi)
    if mode is SaturationMode.SAT_ZERO:
        return np.where(values < 0, 0, np.minimum(values, hi))
    if mode is SaturationMode.SAT_SYM:
        return np.clip(values, -hi if signed else 0, hi)
    raise ValueError(f'Unsupported saturation mode {mode}')


def quantize_to_int(array, frac_bits: int, target_bits: int, signed: bool = True,
                    rounding_mode: RoundingMode = RoundingMode.RND_CONV,
                    saturation_mode: SaturationMode = SaturationMode.SAT):
    """float -> integer codes at ``2**frac_bits`` with the tensor's own rounding / overflow."""
    if array is None:
        return None
    scale = float(1 << frac_bits) if frac_bits > 0 else 1.0
    codes = apply_rounding(np.asarray(array, dtype=np.float64) * scale, rounding_mode).astype(np.int64)
    codes = handle_overflow(codes, int(target_bits), bool(signed), saturation_mode)
    return codes.astype(dtype_for_precision(target_bits, signed), copy=False)


def dequantize(codes, frac: int):
    """integer codes -> float64 (reference: ``src/aie4ml/simulation.py:248-257``)."""
    frac = max(0, int(frac))
    return np.asarray(codes, dtype=np.float64) / float(1 << frac)


# ---- floating-point storage (the float-simulation path) ---------------------------------------
def to_bf16_bits(values) -> np.ndarray:
    """float -> bfloat16 bit patterns (uint16), round to nearest even (NaN payloads are not preserved)."""
    f = np.ascontiguousarray(np.asarray(values, dtype=np.float32))
    u = f.view(np.uint32).astype(np.uint64)
    rounded = (u + 0x7FFF + ((u >> 16) & 1)) >> 16
    return rounded.astype(np.uint16).reshape(f.shape)


def from_bf16_bits(bits) -> np.ndarray:
    b = np.ascontiguousarray(np.asarray(bits, dtype=np.uint16))
    return (b.astype(np.uint32) << 16).view(np.float32).reshape(b.shape)


def to_storage_float(values, fmt: str):
    """-> (array in storage form, float32 values that storage holds) for 'bfloat16' or 'float32'."""
    if fmt == 'bfloat16':
        bits = to_bf16_bits(values)
        return bits, from_bf16_bits(bits)
    if fmt == 'float32':
        f = np.ascontiguousarray(np.asarray(values, dtype=np.float32))
        return f, f
    raise ValueError(f'not a floating-point storage format: {fmt!r}')


def from_storage_float(stored, fmt: str) -> np.ndarray:
    return from_bf16_bits(stored) if fmt == 'bfloat16' else np.asarray(stored, dtype=np.float32)
