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


def to_fp8_bits(values) -> np.ndarray:
    """float -> FP8 E4M3 (finite-only "fn" variant: bias 7, largest finite 448, 0x7F = NaN) bit patterns, round to
    nearest even, values beyond the largest finite saturate to it.  This is what the device's conversion does and
    what activations entering or leaving the graph go through."""
    f = np.ascontiguousarray(np.asarray(values, dtype=np.float32))
    u = f.view(np.uint32)
    sign = ((u >> 24) & 0x80).astype(np.uint8)
    mag = u & 0x7FFFFFFF
    a = mag.view(np.float32)
    # normal range: keep 3 mantissa bits, ties to even; exponent field moves from bias 127 to bias 7
    r = ((mag.astype(np.uint64) + 0x7FFFF + ((mag >> 20) & 1)) >> 20).astype(np.int64) - (120 << 3)
    code = np.clip(r, 0, 0x7E)
    # below 2^-6 the spacing is 2^-9: the rounded count is the encoding itself (8 = 2^-6 = the first normal)
    with np.errstate(invalid='ignore'):
        small = a < np.float32(2.0 ** -6)
        code = np.where(small, np.rint(a.astype(np.float64) * 512.0).astype(np.int64), code)
    code = np.where(np.isnan(a), 0x7F, code)
    return (code.astype(np.uint8) | sign).reshape(f.shape)


_FP8_VALUES = None


def from_fp8_bits(bits) -> np.ndarray:
    global _FP8_VALUES
    if _FP8_VALUES is None:
        c = np.arange(256)
        e, m = (c >> 3) & 15, (c & 7).astype(np.float64)
        mag = np.where(e == 0, m * 2.0 ** -9, (1.0 + m / 8.0) * np.exp2(e.astype(np.float64) - 7.0))
        mag = np.where((c & 0x7F) == 0x7F, np.nan, mag)
        _FP8_VALUES = np.where(c & 0x80, -mag, mag).astype(np.float32)
    return _FP8_VALUES[np.asarray(bits, dtype=np.uint8)]


def pack_constant_float(values, fmt: str) -> np.ndarray:
    """Weights of a floating-point Dense in storage form, by the reference's constant packer
    (``src/aie4ml/op_impls/families/matmul/common.py:253-284``): bfloat16 keeps the upper 16 bits of the float32
    (truncation, not rounding); fp8_e4m3 adds half of the kept mantissa's last place to the float32 bit pattern and
    truncates (ties away from zero), encodes magnitudes of 2^9 and above as 0x7F, and below 2^-10 as zero."""
    f = np.ascontiguousarray(np.asarray(values, dtype=np.float32))
    if fmt == 'float32':
        return f
    u = f.view(np.uint32)
    if fmt == 'bfloat16':
        return (u >> 16).astype(np.uint16).reshape(f.shape)
    if fmt != 'fp8_e4m3':
        raise ValueError(f'not a floating-point storage format: {fmt!r}')
    h = (u.astype(np.uint64) + 0x80000) & 0xFFFFFFFF
    e = ((h >> 23) & 0xFF).astype(np.int64)
    m = (h & 0x7FFFFF).astype(np.int64)
    sign = ((h >> 24) & 0x80).astype(np.int64)
    normal = (((e - 120) << 3) & 0x78) | (m >> 20)
    sub_shift = np.clip(140 - e, 0, 63)
    subnormal = (((0x780000 + m) >> sub_shift) + 1) >> 1
    mag = np.where(e > 135, 0x7F, np.where(e > 120, normal, np.where(e > 116, subnormal, 0)))
    return ((sign | mag) & 0xFF).astype(np.uint8).reshape(f.shape)


def to_storage_float(values, fmt: str):
    """-> (array in storage form, float32 values that storage holds) for 'bfloat16', 'float32' or 'fp8_e4m3'."""
    if fmt == 'bfloat16':
        bits = to_bf16_bits(values)
        return bits, from_bf16_bits(bits)
    if fmt == 'float32':
        f = np.ascontiguousarray(np.asarray(values, dtype=np.float32))
        return f, f
    if fmt == 'fp8_e4m3':
        bits = to_fp8_bits(values)
        return bits, from_fp8_bits(bits)
    raise ValueError(f'not a floating-point storage format: {fmt!r}')


def from_storage_float(stored, fmt: str) -> np.ndarray:
    if fmt == 'bfloat16':
        return from_bf16_bits(stored)
    if fmt == 'fp8_e4m3':
        return from_fp8_bits(stored)
    return np.asarray(stored, dtype=np.float32)
