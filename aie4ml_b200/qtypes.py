"""Quantisation vocabulary of the lowered operator graph.

Same public names and meaning as the reference's ``src/aie4ml/aie_types.py`` (RoundingMode
:9-16, SaturationMode :19-23, QuantIntent :26-32, AIEDataType :132-178), restricted to the
integer formats the CUDA kernels execute.
"""

from __future__ import annotations

from dataclasses import dataclass
from enum import Enum

import numpy as np


class RoundingMode(Enum):
    TRN = 'TRN'
    RND_MIN_INF = 'RND_MIN_INF'
    TRN_ZERO = 'TRN_ZERO'
    RND_ZERO = 'RND_ZERO'
    RND_INF = 'RND_INF'
    RND_CONV = 'RND_CONV'
    RND = 'RND'
    # Extension (not in the reference enum): nearest, ties toward +inf ("round half up"); the
    # AIE API calls it positive_inf.  The benchmark configurations name this mode.
    RND_HALF_UP = 'RND_HALF_UP'


class SaturationMode(Enum):
    WRAP = 'WRAP'
    SAT = 'SAT'
    SAT_ZERO = 'SAT_ZERO'
    SAT_SYM = 'SAT_SYM'


@dataclass(frozen=True)
class QuantIntent:
    """What a tensor's producer promised: ``value = code / 2**frac`` with ``width`` bits."""

    width: int
    frac: int
    signed: bool = True
    rounding: RoundingMode = RoundingMode.RND_CONV
    saturation: SaturationMode = SaturationMode.SAT

    def to_dict(self) -> dict:
        return {'width': int(self.width), 'frac': int(self.frac), 'signed': bool(self.signed),
                'rounding': self.rounding.name, 'saturation': self.saturation.name}

    @classmethod
    def from_dict(cls, d: dict) -> 'QuantIntent':
        return cls(width=int(d['width']), frac=int(d.get('frac', 0)), signed=bool(d.get('signed', True)),
                   rounding=RoundingMode[str(d.get('rounding', 'RND_CONV'))],
                   saturation=SaturationMode[str(d.get('saturation', 'SAT'))])


class FloatFormat(Enum):
    BF16 = 'bfloat16'
    FP32 = 'float32'
    FP8_E4M3 = 'fp8_e4m3'


@dataclass(frozen=True)
class FloatIntent:
    """A tensor computed in floating point (the reference's float-simulation path,
    ``src/aie4ml/aie_types.py:95-98``; set by ``ForceFloatMode`` from ``AIEConfig.ComputeDtype``)."""

    width: int
    format: FloatFormat


FLOAT_FORMATS = ('bfloat16', 'float32', 'fp8_e4m3')

# format -> (bits, signed, numpy dtype, C type); bfloat16 is stored as its 16 bits, fp8 (E4M3, finite-only) as its 8
_FORMATS = {
    'bfloat16': (16, True, np.uint16, 'uint16_t'),
    'float32': (32, True, np.float32, 'float'),
    'fp8_e4m3': (8, True, np.uint8, 'uint8_t'),
    'int8': (8, True, np.int8, 'int8_t'),
    'uint8': (8, False, np.uint8, 'uint8_t'),
    'int16': (16, True, np.int16, 'int16_t'),
    'uint16': (16, False, np.uint16, 'uint16_t'),
    'int32': (32, True, np.int32, 'int32_t'),
    'uint32': (32, False, np.uint32, 'uint32_t'),
    'int64': (64, True, np.int64, 'int64_t'),
}


@dataclass(frozen=True)
class AIEDataType:
    """Resolved storage type of a tensor: an integer format plus its binary point."""

    format: str
    frac: int = 0
    rounding: RoundingMode = RoundingMode.RND
    saturation: SaturationMode = SaturationMode.SAT

    def __post_init__(self) -> None:
        if self.format not in _FORMATS:
            raise ValueError(f'Unknown AIEDataType format: {self.format!r}')

    @property
    def width(self) -> int:
        return _FORMATS[self.format][0]

    @property
    def signed(self) -> bool:
        return _FORMATS[self.format][1]

    @property
    def np_dtype(self):
        return _FORMATS[self.format][2]

    @property
    def c_type(self) -> str:
        return _FORMATS[self.format][3]

    def to_dict(self) -> dict:
        return {'format': self.format, 'frac': int(self.frac), 'rounding': self.rounding.name,
                'saturation': self.saturation.name}

    @classmethod
    def from_dict(cls, data: dict) -> 'AIEDataType':
        return cls(format=str(data['format']), frac=int(data['frac']), rounding=RoundingMode[str(data['rounding'])],
                   saturation=SaturationMode[str(data['saturation'])])
